// Latent attention: the cache holds ONE normed low-rank row c_j per token and layer (no per-head keys or values).
// With k_j = W_uk c_j and v_j = W_uv c_j the key up-projection is folded into the query (qa = W_uk,h^T q_h) and the
// value up-projection is applied after the weighted sum, so attention runs on the cached rows themselves:
//   s_j = scale <qa_h, c_j>,  out_h = sum_j p_j c_j,  p = softmax over {s_j} and one sink logit per head that has no
//   row and no value (it only enlarges the denominator).
// Rows live in a page pool [n_pages, page_rows, rank] addressed through per-sequence page lists (page_pool.h), the
// same lists for every layer. Scores, softmax and the weighted sum are fp32 whatever the cache dtype.
//
// Kernels:
//   latent_store_kernel        RMS norm (eps inside the root) of the down-projected row, times weight -> its page slot
//   latent_attn_kernel         one CTA per (token, head): the warps walk the visible rows round-robin, each row read
//                              coalesced by one warp; per-warp online softmax, merged with the sink at the end
//   latent_attn_tile_kernel    bf16 tensor-core form (mma.sync): one CTA per 16 consecutive tokens x 4 heads of an entry;
//                              rows staged in shared memory once per CTA and used for both the score and the weighted sum
#include "b200_serve.h"
#include "common.cuh"
#include "launch_count.h"

namespace b200 {

constexpr int kMaxRankPerLane = 16;   // rank <= 512

template <typename T>
__global__ void __launch_bounds__(128) latent_store_kernel(const float* __restrict__ raw, long long ld_raw,
                                                           const float* __restrict__ w, float eps, T* __restrict__ pool,
                                                           const int* __restrict__ pages, int max_pages, int page_rows,
                                                           const int* __restrict__ slot, const int* __restrict__ pos,
                                                           int rank) {
    __shared__ float red[4];
    const int t = blockIdx.x;
    const float* src = raw + (size_t)t * ld_raw;
    float q = 0.f;
    for (int i = threadIdx.x; i < rank; i += blockDim.x) q += src[i] * src[i];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) q += __shfl_xor_sync(0xffffffffu, q, o);
    if (threadIdx.x % 32 == 0) red[threadIdx.x / 32] = q;
    __syncthreads();
    const float tot = red[0] + red[1] + red[2] + red[3];
    const float r = 1.0f / sqrtf(tot / (float)rank + eps);
    const int p = pos[t];
    const size_t row = (size_t)pages[(size_t)slot[t] * max_pages + p / page_rows] * page_rows + p % page_rows;
    T* dst = pool + row * rank;
    for (int i = threadIdx.x; i < rank; i += blockDim.x) dst[i] = DT<T>::from_f(src[i] * r * w[i]);
}

template <typename T>
__global__ void __launch_bounds__(128) latent_attn_kernel(const float* __restrict__ qa, float* __restrict__ out,
                                                          const T* __restrict__ pool, const int* __restrict__ pages,
                                                          int max_pages, int page_rows, const int* __restrict__ slot,
                                                          const int* __restrict__ pos, const float* __restrict__ sink,
                                                          float scale, int heads, int rank) {
    extern __shared__ float sm[];          // q[rank] | o[4][rank] | m[4] | l[4]
    float* q = sm;
    float* so = sm + rank;
    float* sml = so + 4 * rank;
    const int t = blockIdx.x, h = blockIdx.y;
    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const float* qsrc = qa + ((size_t)t * heads + h) * rank;
    for (int i = threadIdx.x; i < rank; i += blockDim.x) q[i] = qsrc[i];
    __syncthreads();
    float qr[kMaxRankPerLane], o[kMaxRankPerLane];
#pragma unroll
    for (int i = 0; i < kMaxRankPerLane; ++i) {
        const int r = i * 32 + lane;
        qr[i] = r < rank ? q[r] : 0.f;
        o[i] = 0.f;
    }
    const int n_keys = pos[t] + 1;
    const int* list = pages + (size_t)slot[t] * max_pages;
    float m = -INFINITY, l = 0.f;
    for (int j = warp; j < n_keys; j += 4) {
        const T* c = pool + ((size_t)list[j / page_rows] * page_rows + j % page_rows) * rank;
        float cr[kMaxRankPerLane];
        float d = 0.f;
#pragma unroll
        for (int i = 0; i < kMaxRankPerLane; ++i) {
            const int r = i * 32 + lane;
            cr[i] = (i * 32 < rank && r < rank) ? DT<T>::to_f(c[r]) : 0.f;
            d = fmaf(qr[i], cr[i], d);
        }
#pragma unroll
        for (int s = 16; s > 0; s >>= 1) d += __shfl_xor_sync(0xffffffffu, d, s);
        const float sc = d * scale;
        const float mn = fmaxf(m, sc);
        const float alpha = expf(m - mn), p = expf(sc - mn);
        l = l * alpha + p;
#pragma unroll
        for (int i = 0; i < kMaxRankPerLane; ++i) o[i] = o[i] * alpha + p * cr[i];
        m = mn;
    }
#pragma unroll
    for (int i = 0; i < kMaxRankPerLane; ++i) {
        const int r = i * 32 + lane;
        if (r < rank) so[warp * rank + r] = o[i];
    }
    if (lane == 0) { sml[warp] = m; sml[4 + warp] = l; }
    __syncthreads();
    const float sk = sink[h];
    float M = sk;
#pragma unroll
    for (int w = 0; w < 4; ++w) M = fmaxf(M, sml[w]);
    float f[4], den = expf(sk - M);
#pragma unroll
    for (int w = 0; w < 4; ++w) {
        f[w] = expf(sml[w] - M);     // a warp without rows: exp(-inf) = 0
        den += sml[4 + w] * f[w];
    }
    const float inv = 1.0f / den;
    float* dst = out + ((size_t)t * heads + h) * rank;
    for (int r = threadIdx.x; r < rank; r += blockDim.x)
        dst[r] = (so[r] * f[0] + so[rank + r] * f[1] + so[2 * rank + r] * f[2] + so[3 * rank + r] * f[3]) * inv;
}

}  // namespace b200

using namespace b200;

extern "C" int b200_latent_store(const float* raw, long long ld_raw, const float* w, float eps, void* pool, const int* pages,
                                 int max_pages, int page_rows, const int* slot, const int* pos, int n_tokens, int rank,
                                 int dtype, void* stream) {
    if (!raw || !w || !pool || !pages || !slot || !pos || n_tokens < 0 || rank < 1 || page_rows < 1) return B200_EINVAL;
    if (n_tokens == 0) return B200_OK;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == B200_BF16)
        latent_store_kernel<__nv_bfloat16><<<n_tokens, 128, 0, s>>>(raw, ld_raw, w, eps, (__nv_bfloat16*)pool, pages, max_pages,
                                                                   page_rows, slot, pos, rank);
    else if (dtype == B200_F32)
        latent_store_kernel<float><<<n_tokens, 128, 0, s>>>(raw, ld_raw, w, eps, (float*)pool, pages, max_pages, page_rows, slot,
                                                           pos, rank);
    else
        return B200_EINVAL;
    count_launch();
    return (int)cudaGetLastError();
}

extern "C" int b200_latent_attention(const float* qa, float* out, const void* pool, const int* pages, int max_pages,
                                     int page_rows, const int* slot, const int* pos, const float* sink, float scale,
                                     int n_tokens, int heads, int rank, int dtype, void* stream) {
    if (!qa || !out || !pool || !pages || !slot || !pos || !sink || n_tokens < 0 || heads < 1 || rank < 1) return B200_EINVAL;
    if (rank > 32 * kMaxRankPerLane || heads > 65535) return B200_EUNSUPPORTED;
    if (n_tokens == 0) return B200_OK;
    cudaStream_t s = (cudaStream_t)stream;
    const size_t smem = ((size_t)5 * rank + 8) * sizeof(float);
    dim3 grid(n_tokens, heads);
    if (dtype == B200_BF16)
        latent_attn_kernel<__nv_bfloat16><<<grid, 128, smem, s>>>(qa, out, (const __nv_bfloat16*)pool, pages, max_pages, page_rows,
                                                                 slot, pos, sink, scale, heads, rank);
    else if (dtype == B200_F32)
        latent_attn_kernel<float><<<grid, 128, smem, s>>>(qa, out, (const float*)pool, pages, max_pages, page_rows, slot, pos,
                                                         sink, scale, heads, rank);
    else
        return B200_EINVAL;
    count_launch();
    return (int)cudaGetLastError();
}
