// Rotary positions from a per-token table of cos / sin (b200_rope_angles): the rotated value of ONE component of a head
// whose un-rotated components lie in `vals`. The first `dims` components are rotated, the rest pass unchanged. Pairing:
// B200_ROPE_HALF pairs component i with i + dims/2, B200_ROPE_INTERLEAVED pairs 2i with 2i + 1; the pair (u, v) with
// angle a becomes (u cos a - v sin a, v cos a + u sin a).
#pragma once
#include "b200_serve.h"

namespace b200 {

__device__ __forceinline__ float rotary_component(const float* vals, int i, int dims, int layout, const float* cs, const float* sn) {
    if (i >= dims) return vals[i];
    int f, lo, hi;
    if (layout == B200_ROPE_HALF) {
        const int h = dims / 2;
        f = i < h ? i : i - h;
        lo = f;
        hi = f + h;
    } else {
        f = i / 2;
        lo = 2 * f;
        hi = lo + 1;
    }
    const float u = vals[lo], v = vals[hi], c = cs[f], s = sn[f];
    return i == lo ? u * c - v * s : v * c + u * s;
}

}  // namespace b200
