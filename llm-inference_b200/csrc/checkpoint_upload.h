// Checkpoint tensor -> device memory, shared by the model families that load config.json + model.safetensors: the
// tensor's shape is checked against what the configuration needs, and its values are converted to the serving dtype
// (bfloat16 kept as stored) or to fp32 (norm weights, router weights and the like). Rows of several tensors are stacked
// into one device matrix by passing destinations inside it.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <string>
#include <vector>

#include "b200_llama.h"
#include "safetensors.h"

namespace b200 {

inline int upload_tensor(const SafeTensorsFile& st, const std::string& name, const std::vector<long long>& shape, bool as_f32,
                         int serving_dtype, void* dst, std::string& err) {
    const SafeTensor* t = st.find(name);
    if (!t) { err = "tensor " + name + " is missing"; return B200_EINVAL; }
    if (t->shape != shape) {
        std::string got, want;
        for (long long d : t->shape) got += std::to_string(d) + ",";
        for (long long d : shape) want += std::to_string(d) + ",";
        err = "tensor " + name + " has shape [" + got + "], the configuration needs [" + want + "]";
        return B200_EINVAL;
    }
    if (t->dtype != "BF16" && t->dtype != "F32") { err = "tensor " + name + ": dtype " + t->dtype + " not supported here"; return B200_EINVAL; }
    const size_t n = t->elems();
    cudaError_t e;
    if (!as_f32 && serving_dtype == B200_BF16 && t->dtype == "BF16") {
        e = cudaMemcpy(dst, t->data, n * 2, cudaMemcpyHostToDevice);
    } else if (!as_f32 && serving_dtype == B200_BF16) {
        std::vector<__nv_bfloat16> tmp(n);
        for (size_t i = 0; i < n; ++i) tmp[i] = __float2bfloat16_rn(st_value(*t, i));
        e = cudaMemcpy(dst, tmp.data(), n * 2, cudaMemcpyHostToDevice);
    } else {
        std::vector<float> tmp(n);
        for (size_t i = 0; i < n; ++i) tmp[i] = st_value(*t, i);
        e = cudaMemcpy(dst, tmp.data(), n * 4, cudaMemcpyHostToDevice);
    }
    if (e != cudaSuccess) { err = "upload of " + name + ": " + cudaGetErrorString(e); return (int)e; }
    return B200_OK;
}

}  // namespace b200
