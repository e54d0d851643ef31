// Embedding with learned positions and layer norm (weight + bias), beside norm.cu's RMS norms.
// The residual stream these kernels read and write is fp32; their outputs feed GEMMs and take the serving dtype.
#include "b200_serve.h"
#include "common.cuh"
#include "launch_count.h"

namespace b200 {

template <typename T>
__global__ void embed_positions_kernel(const int* __restrict__ ids, const int* __restrict__ pos, const T* __restrict__ table,
                                       const T* __restrict__ pos_table, float* __restrict__ out, int width) {
    const int t = blockIdx.x;
    const T* e = table + (size_t)ids[t] * width;
    const T* p = pos_table + (size_t)pos[t] * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x) out[(size_t)t * width + i] = DT<T>::to_f(e[i]) + DT<T>::to_f(p[i]);
}

__device__ __forceinline__ float ln_block_sum(float v, float* red) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32, nw = blockDim.x / 32;
    __syncthreads();   // red may still be read from the previous call
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float s = 0.f;
    for (int i = 0; i < nw; ++i) s += red[i];   // same order in every thread: one value per block
    return s;
}

// one CTA per row; the row is kept in shared memory between the passes (mean, then squared deviations, then output)
template <typename T>
__global__ void __launch_bounds__(256) layernorm_pair_kernel(const float* __restrict__ x, const int* __restrict__ rows,
                                                             int width, float eps, const float* __restrict__ w1,
                                                             const float* __restrict__ b1, T* __restrict__ out1,
                                                             const float* __restrict__ w2, const float* __restrict__ b2,
                                                             T* __restrict__ out2) {
    extern __shared__ float row[];
    __shared__ float red[8];
    const int i = blockIdx.x;
    const float* src = x + (size_t)(rows ? rows[i] : i) * width;
    float s = 0.f;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        const float v = src[c];
        row[c] = v;
        s += v;
    }
    const float mean = ln_block_sum(s, red) / (float)width;
    float q = 0.f;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        const float d = row[c] - mean;
        q += d * d;
    }
    const float rstd = 1.0f / sqrtf(ln_block_sum(q, red) / (float)width + eps);
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        const float n = (row[c] - mean) * rstd;
        out1[(size_t)i * width + c] = DT<T>::from_f(n * w1[c] + b1[c]);
        if (out2) out2[(size_t)i * width + c] = DT<T>::from_f(n * w2[c] + b2[c]);
    }
}

}  // namespace b200

using namespace b200;

extern "C" int b200_embed_positions(const int* ids, const int* pos, const void* table, const void* pos_table, float* out,
                                    int n_tokens, int width, int dtype, void* stream) {
    if (!ids || !pos || !table || !pos_table || !out || n_tokens < 0 || width < 1) return B200_EINVAL;
    if (n_tokens == 0) return B200_OK;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == B200_BF16)
        embed_positions_kernel<__nv_bfloat16><<<n_tokens, 128, 0, s>>>(ids, pos, (const __nv_bfloat16*)table,
                                                                      (const __nv_bfloat16*)pos_table, out, width);
    else if (dtype == B200_F32)
        embed_positions_kernel<float><<<n_tokens, 128, 0, s>>>(ids, pos, (const float*)table, (const float*)pos_table, out, width);
    else
        return B200_EINVAL;
    count_launch();
    return (int)cudaGetLastError();
}

extern "C" int b200_layernorm_pair(const float* x, const int* rows, int n_rows, int width, float eps, const float* w1,
                                   const float* b1, void* out1, const float* w2, const float* b2, void* out2, int out_dtype,
                                   void* stream) {
    if (!x || !w1 || !b1 || !out1 || n_rows < 0 || width < 1) return B200_EINVAL;
    if (out2 && (!w2 || !b2)) return B200_EINVAL;
    if (n_rows == 0) return B200_OK;
    const size_t smem = (size_t)width * sizeof(float);
    if (smem > 200 * 1024) return B200_EUNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    if (out_dtype == B200_BF16) {
        static unsigned long long done = 0;
        if (smem > 48 * 1024) ensure_max_dynamic_smem((const void*)layernorm_pair_kernel<__nv_bfloat16>, (int)smem, done);
        layernorm_pair_kernel<__nv_bfloat16><<<n_rows, 256, smem, s>>>(x, rows, width, eps, w1, b1, (__nv_bfloat16*)out1, w2, b2,
                                                                      (__nv_bfloat16*)out2);
    } else if (out_dtype == B200_F32) {
        static unsigned long long done = 0;
        if (smem > 48 * 1024) ensure_max_dynamic_smem((const void*)layernorm_pair_kernel<float>, (int)smem, done);
        layernorm_pair_kernel<float><<<n_rows, 256, smem, s>>>(x, rows, width, eps, w1, b1, (float*)out1, w2, b2, (float*)out2);
    } else
        return B200_EINVAL;
    count_launch();
    return (int)cudaGetLastError();
}
