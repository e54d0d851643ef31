// Retention (linear attention with a fixed decay per head and a carried state, no softmax) and the unit-RMS output gate.
// Everything here is fp32: the rotated q and k, the state, the decays and the sums.
//
//   retention_walk_kernel   one CTA per (entry, head, group of value columns): a thread owns one column of the state
//                           S[:, c] in registers and walks the entry's tokens in order, S <- decay S + k_t v_t[c],
//                           out[t, c] = <S[:, c], q_t>. Columns are independent, so no thread waits on another inside a
//                           token; q_t and k_t are rotated and staged in shared memory eight tokens at a time.
//                           Decode batches and short portions take this path.
//   chunk form (entries of 128 tokens and more): the same recurrence regrouped over chunks of 64 tokens, three launches:
//     retention_chunk_state_kernel   U_c = sum_j decay^(L-1-j) k_j v_j^T of every chunk, chunks in parallel;
//     retention_chunk_scan_kernel    S at the start of every chunk, S_(c+1) = decay^L S_c + U_c, element-wise, and the
//                                    state the entry leaves behind;
//     retention_chunk_out_kernel     out_i = decay^(i+1) S_c^T q_i + sum_(j<=i) decay^(i-j) (q_i . k_j) v_j, chunks in parallel.
//   The same sums in another order: results agree with the walk to fp32 rounding.
#include <math.h>
#include <stdlib.h>

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


// ---------------------------------------------------------------------------------------------------------------
// chunk form
// ---------------------------------------------------------------------------------------------------------------
constexpr int kChunk = 64, kColsPerThread = 2, kChunkCols = 64 * kColsPerThread;   // a thread owns columns c, c + 64

struct RC {
    RT a;
    float* chunk_state;   // [chunk slot, head, dim, vdim]; slot of chunk c of entry e = ent_row[e] / kChunk + e + c
    int col_blocks;       // blocks of kChunkCols value columns; blockIdx.x = entry * col_blocks + column block
};

__host__ __device__ __forceinline__ int chunk_row_stride(int dim) { return ((dim + 3) & ~3) + 4; }   // floats; rows stay 16-byte aligned

// rotated q (or k * k_scale * weight[j]) of a chunk into shared memory; the padding columns are zero
__device__ __forceinline__ void stage_rotated(const RT& a, float* dst, int col_off, int h, int row0, int len, float mul, const float* rowmul) {
    const int dim = a.dim, nf = a.rot_dims / 2, rs = chunk_row_stride(dim);
    for (int i = threadIdx.x; i < len * rs; i += blockDim.x) {
        const int j = i / rs, d = i - j * rs;
        const size_t r = (size_t)(row0 + j);
        float v = 0.f;
        if (d < dim)
            v = rotary_component(a.proj + r * a.ld_proj + col_off + h * dim, d, a.rot_dims, a.rot_layout, a.cos + r * nf, a.sin + r * nf) * mul *
                (rowmul ? rowmul[j] : 1.f);
        dst[i] = v;
    }
}

template <int NACC>   // accumulators per thread (a multiple of 4): dim <= 4 * NACC
__global__ void __launch_bounds__(256) retention_chunk_state_kernel(const RC rc) {
    extern __shared__ __align__(16) float sm[];
    const RT& a = rc.a;
    const int e = blockIdx.x / rc.col_blocks, cb = blockIdx.x % rc.col_blocks;
    const int c_in = blockIdx.y, h = blockIdx.z;
    const int row_e = a.ent_row[e], n = a.ent_len[e];
    if (c_in * kChunk >= n) return;
    const int row0 = row_e + c_in * kChunk, len = min(kChunk, n - c_in * kChunk), dim = a.dim, rs = chunk_row_stride(dim);
    float* Kw = sm;                  // [kChunk][rs], row j weighted by decay^(len-1-j)
    float* pw = sm + kChunk * rs;    // [kChunk]
    const float decay = a.decay[h];
    for (int j = threadIdx.x; j < len; j += blockDim.x) pw[j] = powf(decay, (float)(len - 1 - j));
    __syncthreads();
    stage_rotated(a, Kw, a.k_off, h, row0, len, a.k_scale, pw);
    __syncthreads();
    // thread: kColsPerThread value columns, NACC consecutive rows of the state (read from shared memory four at a time)
    const int c = cb * kChunkCols + (threadIdx.x & 63), d0 = (threadIdx.x >> 6) * NACC, dpad = (dim + 3) & ~3;
    float acc[kColsPerThread][NACC];
#pragma unroll
    for (int q = 0; q < kColsPerThread; ++q)
#pragma unroll
        for (int k = 0; k < NACC; ++k) acc[q][k] = 0.f;
    if (c < a.vdim && d0 < dim) {
        const float* vcol = a.proj + (size_t)row0 * a.ld_proj + a.v_off + h * a.vdim + c;
        for (int j = 0; j < len; ++j) {
            float v[kColsPerThread];
#pragma unroll
            for (int q = 0; q < kColsPerThread; ++q) v[q] = c + 64 * q < a.vdim ? vcol[(size_t)j * a.ld_proj + 64 * q] : 0.f;
            const float* kr = Kw + j * rs + d0;
#pragma unroll
            for (int k = 0; k < NACC; k += 4)
                if (d0 + k < dpad) {
                    const float4 k4 = *reinterpret_cast<const float4*>(kr + k);
#pragma unroll
                    for (int q = 0; q < kColsPerThread; ++q) {
                        acc[q][k] = fmaf(k4.x, v[q], acc[q][k]);
                        acc[q][k + 1] = fmaf(k4.y, v[q], acc[q][k + 1]);
                        acc[q][k + 2] = fmaf(k4.z, v[q], acc[q][k + 2]);
                        acc[q][k + 3] = fmaf(k4.w, v[q], acc[q][k + 3]);
                    }
                }
        }
        float* U = rc.chunk_state + (((size_t)(row_e / kChunk + e + c_in) * a.heads + h) * dim) * a.vdim + c;
#pragma unroll
        for (int q = 0; q < kColsPerThread; ++q)
            if (c + 64 * q < a.vdim)
#pragma unroll
                for (int k = 0; k < NACC; ++k)
                    if (d0 + k < dim) U[(size_t)(d0 + k) * a.vdim + 64 * q] = acc[q][k];
    }
}

// element-wise over (dim, vdim): walks the entry's chunks, leaves S at each chunk's start in place of its U
__global__ void __launch_bounds__(256) retention_chunk_scan_kernel(const RC rc) {
    const RT& a = rc.a;
    const int e = blockIdx.x, h = blockIdx.y, i = blockIdx.z * blockDim.x + threadIdx.x;
    const int per = a.dim * a.vdim;
    if (i >= per) return;
    const int row_e = a.ent_row[e], n = a.ent_len[e], b = a.slot[row_e], p0 = a.pos[row_e];
    const float decay = a.decay[h];
    float* sp = a.state + ((size_t)b * a.heads + h) * per + i;
    float S = p0 > 0 ? *sp : 0.f;
    const float full = powf(decay, (float)kChunk);
    const int chunks = (n + kChunk - 1) / kChunk;
    float* U = rc.chunk_state + ((size_t)(row_e / kChunk + e) * a.heads + h) * per + i;
    const size_t step = (size_t)a.heads * per;
    for (int c0 = 0; c0 < chunks; c0 += 8) {   // eight loads in flight, then the dependent chain
        float u[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) u[k] = c0 + k < chunks ? U[(size_t)(c0 + k) * step] : 0.f;
#pragma unroll
        for (int k = 0; k < 8; ++k)
            if (c0 + k < chunks) {
                const int len = min(kChunk, n - (c0 + k) * kChunk);
                U[(size_t)(c0 + k) * step] = S;
                S = fmaf(len == kChunk ? full : powf(decay, (float)len), S, u[k]);
            }
    }
    *sp = S;
}

__global__ void __launch_bounds__(256) retention_chunk_out_kernel(const RC rc) {
    extern __shared__ __align__(16) float sm[];
    const RT& a = rc.a;
    const int e = blockIdx.x / rc.col_blocks, cb = blockIdx.x % rc.col_blocks;
    const int c_in = blockIdx.y, h = blockIdx.z;
    const int row_e = a.ent_row[e], n = a.ent_len[e];
    if (c_in * kChunk >= n) return;
    const int row0 = row_e + c_in * kChunk, len = min(kChunk, n - c_in * kChunk), dim = a.dim, rs = chunk_row_stride(dim);
    constexpr int AS = kChunk + 4;                // row stride of A in floats
    float* Qc = sm;                               // [kChunk][rs]
    float* Kc = Qc + kChunk * rs;                 // [kChunk][rs]
    float* A = Kc + kChunk * rs;                  // [kChunk][AS]
    float* pw = A + kChunk * AS;                  // [kChunk + 1]: decay^k
    const float decay = a.decay[h];
    for (int k = threadIdx.x; k <= kChunk; k += blockDim.x) pw[k] = powf(decay, (float)k);
    stage_rotated(a, Qc, a.q_off, h, row0, len, 1.f, nullptr);
    stage_rotated(a, Kc, a.k_off, h, row0, len, a.k_scale, nullptr);
    __syncthreads();
    const int dpad = (dim + 3) & ~3;
    for (int idx = threadIdx.x; idx < kChunk * kChunk; idx += blockDim.x) {
        const int i = idx / kChunk, j = idx % kChunk;
        float v = 0.f;
        if (j <= i && i < len) {
            const float* q = Qc + i * rs;
            const float* k = Kc + j * rs;
            for (int d = 0; d < dpad; d += 4) {
                const float4 q4 = *reinterpret_cast<const float4*>(q + d), k4 = *reinterpret_cast<const float4*>(k + d);
                v = fmaf(q4.x, k4.x, v); v = fmaf(q4.y, k4.y, v); v = fmaf(q4.z, k4.z, v); v = fmaf(q4.w, k4.w, v);
            }
            v *= pw[i - j];
        }
        A[i * AS + j] = v;
    }
    __syncthreads();
    const int c = cb * kChunkCols + (threadIdx.x & 63), rg = threadIdx.x >> 6;   // thread: columns c, c + 64; rows rg, rg + 4, ...
    if (c >= a.vdim) return;
    constexpr int NR = kChunk / 4, CP = kColsPerThread;
    float acc[CP][NR], cross[CP][NR];
#pragma unroll
    for (int q = 0; q < CP; ++q)
#pragma unroll
        for (int k = 0; k < NR; ++k) acc[q][k] = cross[q][k] = 0.f;
    const float* vcol = a.proj + (size_t)row0 * a.ld_proj + a.v_off + h * a.vdim + c;
    for (int j = 0; j < len; j += 4) {
        float v[CP][4];
#pragma unroll
        for (int q = 0; q < CP; ++q)
#pragma unroll
            for (int x = 0; x < 4; ++x) v[q][x] = (j + x < len && c + 64 * q < a.vdim) ? vcol[(size_t)(j + x) * a.ld_proj + 64 * q] : 0.f;
#pragma unroll
        for (int k = 0; k < NR; ++k) {
            const float4 a4 = *reinterpret_cast<const float4*>(A + (rg + 4 * k) * AS + j);
#pragma unroll
            for (int q = 0; q < CP; ++q) {
                acc[q][k] = fmaf(a4.x, v[q][0], acc[q][k]); acc[q][k] = fmaf(a4.y, v[q][1], acc[q][k]);
                acc[q][k] = fmaf(a4.z, v[q][2], acc[q][k]); acc[q][k] = fmaf(a4.w, v[q][3], acc[q][k]);
            }
        }
    }
    const float* S = rc.chunk_state + (((size_t)(row_e / kChunk + e + c_in) * a.heads + h) * dim) * a.vdim + c;
    for (int d = 0; d < dpad; d += 4) {
        float sv[CP][4];
#pragma unroll
        for (int q = 0; q < CP; ++q)
#pragma unroll
            for (int x = 0; x < 4; ++x) sv[q][x] = (d + x < dim && c + 64 * q < a.vdim) ? S[(size_t)(d + x) * a.vdim + 64 * q] : 0.f;
#pragma unroll
        for (int k = 0; k < NR; ++k) {
            const float4 q4 = *reinterpret_cast<const float4*>(Qc + (rg + 4 * k) * rs + d);
#pragma unroll
            for (int q = 0; q < CP; ++q) {
                cross[q][k] = fmaf(q4.x, sv[q][0], cross[q][k]); cross[q][k] = fmaf(q4.y, sv[q][1], cross[q][k]);
                cross[q][k] = fmaf(q4.z, sv[q][2], cross[q][k]); cross[q][k] = fmaf(q4.w, sv[q][3], cross[q][k]);
            }
        }
    }
#pragma unroll
    for (int q = 0; q < CP; ++q)
#pragma unroll
        for (int k = 0; k < NR; ++k) {
            const int i = rg + 4 * k;
            if (i < len && c + 64 * q < a.vdim)
                a.out[(size_t)(row0 + i) * ((size_t)a.heads * a.vdim) + h * a.vdim + c + 64 * q] = fmaf(pw[i + 1], cross[q][k], acc[q][k]);
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

extern "C" size_t b200_retention_workspace_bytes(int n_tokens, int n_entries, int heads, int dim, int vdim) {
    if (n_tokens < 2 * kChunk || n_entries < 1 || heads < 1 || dim < 1 || vdim < 1) return 0;
    return (size_t)(n_tokens / kChunk + n_entries + 1) * heads * dim * vdim * sizeof(float);
}

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
    cudaStream_t s = (cudaStream_t)stream;
    const char* env = getenv("B200_RETENTION_WALK");   // 1: every entry on the token-by-token kernel (debugging aid)
    const size_t need = b200_retention_workspace_bytes(p->n_tokens, p->n_entries, p->heads, p->dim, p->vdim);
    if (p->longest_entry >= 2 * kChunk && need > 0 && p->workspace && p->workspace_bytes >= need && !(env && env[0] == '1')) {
        RC rc{a, reinterpret_cast<float*>(p->workspace), 1};
        const int col_blocks = (p->vdim + kChunkCols - 1) / kChunkCols, chunks = (p->longest_entry + kChunk - 1) / kChunk;
        if (chunks > 65535 || p->heads > 65535) return B200_EUNSUPPORTED;
        const dim3 grid(p->n_entries * col_blocks, chunks, p->heads);
        const int rs = chunk_row_stride(p->dim);
        const size_t smem1 = ((size_t)kChunk * rs + kChunk) * sizeof(float);
        const size_t smem3 = ((size_t)2 * kChunk * rs + kChunk * (kChunk + 4) + kChunk + 4) * sizeof(float);
        static unsigned long long done1[4] = {0, 0, 0, 0}, done3 = 0;
        // the attribute is set once per kernel: to the most any supported dim (256) needs
        constexpr int kMax1 = (kChunk * 260 + kChunk) * 4, kMax3 = (2 * kChunk * 260 + kChunk * (kChunk + 4) + kChunk + 4) * 4;
        cudaError_t e = ensure_max_dynamic_smem((const void*)retention_chunk_out_kernel, kMax3, done3);
        if (e != cudaSuccess) return (int)e;
        rc.col_blocks = col_blocks;
        if (p->dim <= 32) { ensure_max_dynamic_smem((const void*)retention_chunk_state_kernel<8>, kMax1, done1[0]); retention_chunk_state_kernel<8><<<grid, 256, smem1, s>>>(rc); }
        else if (p->dim <= 64) { ensure_max_dynamic_smem((const void*)retention_chunk_state_kernel<16>, kMax1, done1[1]); retention_chunk_state_kernel<16><<<grid, 256, smem1, s>>>(rc); }
        else if (p->dim <= 128) { ensure_max_dynamic_smem((const void*)retention_chunk_state_kernel<32>, kMax1, done1[2]); retention_chunk_state_kernel<32><<<grid, 256, smem1, s>>>(rc); }
        else { ensure_max_dynamic_smem((const void*)retention_chunk_state_kernel<64>, kMax1, done1[3]); retention_chunk_state_kernel<64><<<grid, 256, smem1, s>>>(rc); }
        const int per = p->dim * p->vdim;
        retention_chunk_scan_kernel<<<dim3(p->n_entries, p->heads, (per + 255) / 256), 256, 0, s>>>(rc);
        retention_chunk_out_kernel<<<grid, 256, smem3, s>>>(rc);
        count_launch(3);
        return (int)cudaGetLastError();
    }
    const int threads = p->vdim <= 32 ? 32 : p->vdim <= 64 ? 64 : 128;
    const dim3 grid(p->n_entries, p->heads, (p->vdim + threads - 1) / threads);
    if (grid.y > 65535 || grid.z > 65535) return B200_EUNSUPPORTED;
    const size_t smem = (size_t)(2 + 2 * kWalkTokens) * p->dim * sizeof(float);
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
