// The router's choice for one token, made by one warp: probs = softmax over all E experts (E <= 256);
// the choice is made on probs + mask (0 for an allowed expert, -inf for a masked one:
// third_party/llama.cpp/patches/0003 lines 82-108), ties to the lower index; the weights are the
// unmasked probs of the k chosen experts (k <= 32), renormalised.  mask: one byte per expert
// (1 = allowed) or null.  lr may be read through any path that sees the logits' latest values.
#pragma once
#include "kq_common.cuh"

__device__ __forceinline__ void kq_route_warp(const float *lr, int E, int k, const uint8_t *mask, int32_t *ids, float *w,
                                              int lane) {
    float v[8], sel[8];
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
    // selection value: the prob of an allowed expert (>= 0), -1 for a masked one (all equal, below every
    // allowed one, as -inf is), -2 once taken, -3 outside the table
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const int e = lane + 32 * i;
        v[i] = v[i] / den;
        sel[i] = e >= E ? -3.f : ((mask && !mask[e]) ? -1.f : v[i]);
    }
    float wsum = 0.f, mine = 0.f;
    int myid = 0;
    for (int s = 0; s < k; s++) {
        float best = -4.f, bp = 0.f;
        int be = 0x7fffffff;
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const int e = lane + 32 * i;
            if (sel[i] > best || (sel[i] == best && e < be)) { best = sel[i]; be = e; bp = v[i]; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oe = __shfl_xor_sync(0xffffffffu, be, o);
            const float op = __shfl_xor_sync(0xffffffffu, bp, o);
            if (ov > best || (ov == best && oe < be)) { best = ov; be = oe; bp = op; }
        }
        wsum += bp;
        if (lane == s) { mine = bp; myid = be; }
        if ((be & 31) == lane) {
#pragma unroll
            for (int i = 0; i < 8; i++)
                if (i == (be >> 5)) sel[i] = -2.f; // taken
        }
    }
    if (lane < k) {
        ids[lane] = myid;
        w[lane] = mine / wsum;
    }
}
