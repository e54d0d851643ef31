// b200_paged_attention: causal attention over paged per-head keys and values with grouped query heads, a tanh cap on
// the scores and a constant added to the softmax denominator (a sink of score 0 that owns no value). Prompt portions,
// single decoded tokens and mixed batches run through the same launch: every token carries its sequence slot and
// position, and only sees its own sequence's pages.
//
//   paged_attn_row_kernel   one CTA per (token, query head), fp32 arithmetic on caches of either dtype: each warp
//                           takes blocks of 32 keys (a lane scores one key; the weighted value sum runs with a lane per
//                           output column), keeps its own running maximum / denominator / output and the warps merge at
//                           the end. The sink is the initial state of warp 0 (m = 0, l = denom_bias).
//   paged_attn_tile_kernel  bfloat16 prompt portions on mma.sync tiles (further down).
#include <cuda_bf16.h>
#include <math.h>

#include "b200_serve.h"
#include "common.cuh"
#include "launch_count.h"

namespace b200 {

struct PA {
    const void* q; void* out; const void* k_pool; const void* v_pool;
    const int* pages; int max_pages, page_rows;
    const int* slot; const int* pos;
    int n_tokens, heads, kv_heads, dim, vdim;
    float scale, softcap, denom_bias;
};

constexpr int kRowWarps = 4;
constexpr int kMaxVPerLane = 8;   // vdim <= 256

template <typename T>
__device__ __forceinline__ float dot_row(const float* q, const T* k, int dim) {
    float acc = 0.f;
    if ((dim % DT<T>::kPer16B) == 0 && (reinterpret_cast<uintptr_t>(k) & 15u) == 0) {
        for (int i = 0; i < dim; i += DT<T>::kPer16B) {
            float f[DT<T>::kPer16B];
            const Pack16 pk = ld16(k + i);
            if constexpr (sizeof(T) == 4) {
#pragma unroll
                for (int e = 0; e < 4; ++e) f[e] = __uint_as_float(pk.w[e]);
            } else {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float2 v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&pk.w[e]));
                    f[2 * e] = v.x;
                    f[2 * e + 1] = v.y;
                }
            }
#pragma unroll
            for (int e = 0; e < DT<T>::kPer16B; ++e) acc = fmaf(q[i + e], f[e], acc);
        }
    } else {
        for (int i = 0; i < dim; ++i) acc = fmaf(q[i], DT<T>::to_f(k[i]), acc);
    }
    return acc;
}

template <typename T>
__global__ void __launch_bounds__(kRowWarps * 32) paged_attn_row_kernel(const PA a) {
    extern __shared__ float sm[];
    float* qs = sm;                                   // [dim]
    float* om = sm + a.dim;                           // [kRowWarps][vdim]
    __shared__ float ms[kRowWarps], ls[kRowWarps];
    const int t = blockIdx.x, h = blockIdx.y, warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const int g = h / (a.heads / a.kv_heads), p = a.pos[t];
    const int* plist = a.pages + (size_t)a.slot[t] * a.max_pages;
    const T* q = reinterpret_cast<const T*>(a.q) + ((size_t)t * a.heads + h) * a.dim;
    for (int i = threadIdx.x; i < a.dim; i += blockDim.x) qs[i] = DT<T>::to_f(q[i]);
    __syncthreads();
    const T* K = reinterpret_cast<const T*>(a.k_pool);
    const T* V = reinterpret_cast<const T*>(a.v_pool);
    float m = -INFINITY, l = 0.f, o[kMaxVPerLane];
#pragma unroll
    for (int c = 0; c < kMaxVPerLane; ++c) o[c] = 0.f;
    if (warp == 0 && a.denom_bias > 0.f) { m = 0.f; l = a.denom_bias; }
    for (int j0 = warp * 32; j0 <= p; j0 += kRowWarps * 32) {
        const int j = j0 + lane;
        const bool ok = j <= p;
        size_t row = 0;
        float s = -INFINITY;
        if (ok) {
            row = ((size_t)plist[j / a.page_rows] * a.page_rows + j % a.page_rows) * a.kv_heads + g;
            s = dot_row<T>(qs, K + row * a.dim, a.dim) * a.scale;
            if (a.softcap > 0.f) s = a.softcap * tanhf(s / a.softcap);
        }
        float bm = s;
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, d));
        const float mn = fmaxf(m, bm);
        const float corr = expf(m - mn);   // m = -inf: 0
        const float pj = ok ? expf(s - mn) : 0.f;
        float ps = pj;
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, d);
        l = l * corr + ps;
        m = mn;
#pragma unroll
        for (int c = 0; c < kMaxVPerLane; ++c) o[c] *= corr;
        const int n = min(32, p - j0 + 1);
        for (int kk = 0; kk < n; ++kk) {
            const float pk = __shfl_sync(0xffffffffu, pj, kk);
            const size_t r = __shfl_sync(0xffffffffu, (unsigned long long)row, kk);
            const T* vr = V + r * a.vdim;
#pragma unroll
            for (int c = 0; c < kMaxVPerLane; ++c)
                if (lane + 32 * c < a.vdim) o[c] = fmaf(pk, DT<T>::to_f(vr[lane + 32 * c]), o[c]);
        }
    }
    if (lane == 0) { ms[warp] = m; ls[warp] = l; }
#pragma unroll
    for (int c = 0; c < kMaxVPerLane; ++c)
        if (lane + 32 * c < a.vdim) om[warp * a.vdim + lane + 32 * c] = o[c];
    __syncthreads();
    float M = ms[0];
    for (int w = 1; w < kRowWarps; ++w) M = fmaxf(M, ms[w]);
    float L = 0.f;
    for (int w = 0; w < kRowWarps; ++w) L += ls[w] * expf(ms[w] - M);
    T* dst = reinterpret_cast<T*>(a.out) + ((size_t)t * a.heads + h) * a.vdim;
    for (int c = threadIdx.x; c < a.vdim; c += blockDim.x) {
        float v = 0.f;
        for (int w = 0; w < kRowWarps; ++w) v += om[w * a.vdim + c] * expf(ms[w] - M);
        dst[c] = DT<T>::from_f(v / L);
    }
}

}  // namespace b200

using namespace b200;

extern "C" int b200_paged_attention(const b200_paged_attention_args* p, void* stream) {
    if (!p || !p->q || !p->out || !p->k_pool || !p->v_pool || !p->pages || !p->slot || !p->pos || p->n_tokens < 0 || p->heads < 1 ||
        p->kv_heads < 1 || p->heads % p->kv_heads || p->dim < 1 || p->vdim < 1 || p->page_rows < 1 || p->denom_bias < 0.f)
        return B200_EINVAL;
    if (p->vdim > 32 * kMaxVPerLane) return B200_EUNSUPPORTED;
    if (p->n_tokens == 0) return B200_OK;
    PA a{p->q, p->out, p->k_pool, p->v_pool, p->pages, p->max_pages, p->page_rows, p->slot, p->pos, p->n_tokens, p->heads,
         p->kv_heads, p->dim, p->vdim, p->scale, p->softcap, p->denom_bias};
    cudaStream_t s = (cudaStream_t)stream;
    const dim3 grid(p->n_tokens, p->heads);
    const size_t smem = ((size_t)p->dim + (size_t)kRowWarps * p->vdim) * sizeof(float);
    if (smem > 48 * 1024) return B200_EUNSUPPORTED;
    if (p->dtype == B200_BF16) paged_attn_row_kernel<__nv_bfloat16><<<grid, kRowWarps * 32, smem, s>>>(a);
    else if (p->dtype == B200_F32) paged_attn_row_kernel<float><<<grid, kRowWarps * 32, smem, s>>>(a);
    else return B200_EINVAL;
    count_launch();
    return (int)cudaGetLastError();
}
