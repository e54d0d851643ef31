// Retention (linear attention with a fixed decay per head and a carried state, no softmax) and the unit-RMS output gate.
// Everything here is fp32: the rotated q and k, the state, the decays and the sums.
//
//   retention_walk_kernel   one CTA per (entry, head, group of value columns): a thread owns one column of the state
//                           S[:, c] in registers and walks the entry's tokens in order, S <- decay S + k_t v_t[c],
//                           out[t, c] = <S[:, c], q_t>. Columns are independent, so no thread waits on another inside a
//                           token; q_t and k_t are rotated and staged in shared memory eight tokens at a time.
//                           Decode batches (one token per entry) and prompt portions take the same path.
#include <math.h>

#include "b200_serve.h"
#include "common.cuh"
#include "launch_count.h"
#include "rotary.cuh"

namespace b200 {

struct RT {
    const float* proj; long long ld_proj; int q_off, k_off, v_off;
    const float* cos; const float* sin; int rot_dims, rot_layout;
    const float* decay; float k_scale;
    float* state; float* out;
    const int* ent_row; const int* ent_len; const int* slot; const int* pos;
    int heads, dim, vdim;
};

constexpr int kWalkTokens = 8;   // tokens whose q / k are staged per synchronisation

template <int DIM>
__global__ void __launch_bounds__(128) retention_walk_kernel(const RT a) {
    extern __shared__ float sm[];
    const int dim = a.dim;
    float* raw = sm;                              // [2][dim] un-rotated q, k of the token being staged
    float* rq = sm + 2 * dim;                     // [kWalkTokens][dim]
    float* rk = rq + kWalkTokens * dim;           // [kWalkTokens][dim]
    const int e = blockIdx.x, h = blockIdx.y, c = blockIdx.z * blockDim.x + threadIdx.x;
    const int row0 = a.ent_row[e], n = a.ent_len[e], b = a.slot[row0], p0 = a.pos[row0];
    const bool live = c < a.vdim;
    const float decay = a.decay[h];
    float S[DIM];
    float* sp = a.state + (((size_t)b * a.heads + h) * dim) * a.vdim + c;
#pragma unroll
    for (int d = 0; d < DIM; ++d) S[d] = (live && d < dim && p0 > 0) ? sp[(size_t)d * a.vdim] : 0.f;
    const int nf = a.rot_dims / 2;
    for (int t0 = 0; t0 < n; t0 += kWalkTokens) {
        const int nt = min(kWalkTokens, n - t0);
        for (int k = 0; k < nt; ++k) {
            const size_t r = (size_t)(row0 + t0 + k);
            __syncthreads();   // raw (and, for k = 0, rq / rk of the previous group) are free
            for (int i = threadIdx.x; i < 2 * dim; i += blockDim.x)
                raw[i] = a.proj[r * a.ld_proj + (i < dim ? a.q_off + h * dim + i : a.k_off + h * dim + (i - dim))];
            __syncthreads();
            for (int i = threadIdx.x; i < 2 * dim; i += blockDim.x) {
                const bool is_k = i >= dim;
                const int d = is_k ? i - dim : i;
                const float v = rotary_component(raw + (is_k ? dim : 0), d, a.rot_dims, a.rot_layout, a.cos + r * nf, a.sin + r * nf);
                if (is_k) rk[k * dim + d] = v * a.k_scale;
                else rq[k * dim + d] = v;
            }
        }
        __syncthreads();
        if (live) {
            for (int k = 0; k < nt; ++k) {
                const size_t r = (size_t)(row0 + t0 + k);
                const float v = a.proj[r * a.ld_proj + a.v_off + h * a.vdim + c];
                float acc = 0.f;
#pragma unroll
                for (int d = 0; d < DIM; ++d)
                    if (d < dim) {
                        S[d] = fmaf(decay, S[d], rk[k * dim + d] * v);
                        acc = fmaf(S[d], rq[k * dim + d], acc);
                    }
                a.out[r * ((size_t)a.heads * a.vdim) + h * a.vdim + c] = acc;
            }
        }
    }
    if (live) {
#pragma unroll
        for (int d = 0; d < DIM; ++d)
            if (d < dim) sp[(size_t)d * a.vdim] = S[d];
    }
}

// one warp per (token, head)
template <typename T>
__global__ void unit_rms_gate_kernel(const float* __restrict__ o, const float* __restrict__ gate, long long ld_gate, T* __restrict__ out,
                                     int units, int heads, int vdim, float eps) {
    const int u = blockIdx.x * (blockDim.x / 32) + threadIdx.x / 32, lane = threadIdx.x % 32;
    if (u >= units) return;
    const int t = u / heads, h = u % heads;
    const float* src = o + (size_t)u * vdim;
    float ss = 0.f;
    for (int i = lane; i < vdim; i += 32) ss += src[i] * src[i];
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, d);
    const float rinv = 1.0f / sqrtf(ss / (float)vdim + eps);
    const float* g = gate + (size_t)t * ld_gate + (size_t)h * vdim;
    for (int i = lane; i < vdim; i += 32) {
        const float z = g[i];
        out[(size_t)u * vdim + i] = DT<T>::from_f(src[i] * rinv * (z / (1.f + expf(-z))));
    }
}

}  // namespace b200

using namespace b200;

extern "C" size_t b200_retention_workspace_bytes(int, int, int, int, int) { return 0; }

extern "C" int b200_retention(const b200_retention_args* p, void* stream) {
    if (!p || !p->proj || !p->decay || !p->state || !p->out || !p->ent_row || !p->ent_len || !p->slot || !p->pos || p->n_entries < 0 ||
        p->heads < 1 || p->dim < 1 || p->vdim < 1)
        return B200_EINVAL;
    if (p->rot_dims < 0 || (p->rot_dims & 1) || p->rot_dims > p->dim || (p->rot_dims && (!p->cos || !p->sin))) return B200_EINVAL;
    if (p->rot_layout != B200_ROPE_HALF && p->rot_layout != B200_ROPE_INTERLEAVED) return B200_EINVAL;
    if (p->dim > 256) return B200_EUNSUPPORTED;
    if (p->n_entries == 0) return B200_OK;
    RT a{p->proj, p->ld_proj, p->q_off, p->k_off, p->v_off, p->cos, p->sin, p->rot_dims, p->rot_layout, p->decay, p->k_scale,
         p->state, p->out, p->ent_row, p->ent_len, p->slot, p->pos, p->heads, p->dim, p->vdim};
    const int threads = p->vdim <= 32 ? 32 : p->vdim <= 64 ? 64 : 128;
    const dim3 grid(p->n_entries, p->heads, (p->vdim + threads - 1) / threads);
    if (grid.y > 65535 || grid.z > 65535) return B200_EUNSUPPORTED;
    const size_t smem = (size_t)(2 + 2 * kWalkTokens) * p->dim * sizeof(float);
    cudaStream_t s = (cudaStream_t)stream;
    if (p->dim <= 32) retention_walk_kernel<32><<<grid, threads, smem, s>>>(a);
    else if (p->dim <= 64) retention_walk_kernel<64><<<grid, threads, smem, s>>>(a);
    else if (p->dim <= 128) retention_walk_kernel<128><<<grid, threads, smem, s>>>(a);
    else retention_walk_kernel<256><<<grid, threads, smem, s>>>(a);
    count_launch();
    return (int)cudaGetLastError();
}

extern "C" int b200_unit_rms_gate(const float* o, const float* gate, long long ld_gate, void* out, int n_tokens, int heads, int vdim,
                                  float eps, int out_dtype, void* stream) {
    if (!o || !gate || !out || n_tokens < 0 || heads < 1 || vdim < 1) return B200_EINVAL;
    if (n_tokens == 0) return B200_OK;
    const int units = n_tokens * heads;
    const dim3 grid((units + 3) / 4);
    cudaStream_t s = (cudaStream_t)stream;
    if (out_dtype == B200_BF16) unit_rms_gate_kernel<__nv_bfloat16><<<grid, 128, 0, s>>>(o, gate, ld_gate, (__nv_bfloat16*)out, units, heads, vdim, eps);
    else if (out_dtype == B200_F32) unit_rms_gate_kernel<float><<<grid, 128, 0, s>>>(o, gate, ld_gate, (float*)out, units, heads, vdim, eps);
    else return B200_EINVAL;
    count_launch();
    return (int)cudaGetLastError();
}
