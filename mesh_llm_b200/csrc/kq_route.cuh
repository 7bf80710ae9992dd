// The router's choice for one token, made by one warp: probs = softmax over all E experts (E <= 256);
// the choice is made on probs + mask (0 for an allowed expert, -inf for a masked one:
// third_party/llama.cpp/patches/0003 lines 82-108), ties to the lower index; the weights are the
// unmasked probs of the k chosen experts (k <= 32), renormalised.  mask: one byte per expert
// (1 = allowed) or null.  lr may be read through any path that sees the logits' latest values.
#pragma once
#include "kq_common.cuh"

__device__ __forceinline__ void kq_route_warp(const float *lr, int E, int k, const uint8_t *mask, int32_t *ids, float *w,
                                              int lane) {
    float v[8];
    float mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const int e = lane + 32 * i;
        v[i] = e < E ? __ldcg(lr + e) : -INFINITY; // L2: another CTA of the same launch may have written them
        mx = fmaxf(mx, v[i]);
    }
    mx = kq_warp_max(mx);
    float den = 0.f;
#pragma unroll
    for (int i = 0; i < 8; i++) {
        v[i] = (lane + 32 * i) < E ? expf(v[i] - mx) : 0.f;
        den += v[i];
    }
    den = kq_warp_sum(den);
    // selection key, larger = preferred: the prob of an allowed expert as its bit pattern (probs are not
    // negative, so the patterns order as the values do) + 4; 3 for a masked expert (all equal, below every
    // allowed one, as -inf is); 2 once taken; 1 outside the table
    uint32_t key[8];
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const int e = lane + 32 * i;
        v[i] = v[i] / den;
        key[i] = e >= E ? 1u : ((mask && !mask[e]) ? 3u : __float_as_uint(v[i]) + 4u);
    }
    float wsum = 0.f, mine = 0.f;
    int myid = 0;
    for (int s = 0; s < k; s++) {
        uint32_t bk = key[0];
        int bi = 0;
#pragma unroll
        for (int i = 1; i < 8; i++)
            if (key[i] > bk) { bk = key[i]; bi = i; } // ties inside a lane: the lower expert
        const uint32_t top = __reduce_max_sync(0xffffffffu, bk);
        const int be = (int)__reduce_min_sync(0xffffffffu, bk == top ? (uint32_t)(lane + 32 * bi) : 0xffffffffu); // ties: the lower expert
        float pv = v[0];
#pragma unroll
        for (int i = 1; i < 8; i++)
            if (i == (be >> 5)) pv = v[i];
        const float bp = __shfl_sync(0xffffffffu, pv, be & 31);
        wsum += bp;
        if (lane == s) { mine = bp; myid = be; }
        if ((be & 31) == lane) {
#pragma unroll
            for (int i = 0; i < 8; i++)
                if (i == (be >> 5)) key[i] = 2u; // taken
        }
    }
    if (lane < k) {
        ids[lane] = myid;
        w[lane] = mine / wsum;
    }
}
