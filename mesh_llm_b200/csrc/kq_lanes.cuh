// Per-lane decoders of the packed weight blocks, shared by the decode kernels.
//
// A warp covers 4 consecutive 256-blocks per step: 8 lanes per block, each lane one 16-byte chunk
// of the block's quant bytes (chunk c = lane & 7).  The integer routines below are the only place
// where quantised weights meet int8 activations; the exact-sum instrumentation calls the same code.
#pragma once
#include "kq_common.cuh"

// ---- Q4_K: one lane's share of one block -----------------------------------------------------
// hdr = first 16 bytes of the block (f16 d, f16 dmin, 12 bytes of 6-bit scales/mins); w = the
// lane's 16 quant bytes (chunk c of 8): low nibbles belong to sub-block 2g, high nibbles to
// sub-block 2g+1, g = c >> 1.
struct Q4Scales {
    int sc0, sc1, m0, m1;
    float d, dmin;
};

static __device__ __forceinline__ Q4Scales q4k_lane_scales(const uint4 &hdr, int c) {
    Q4Scales s;
    const int g = c >> 1;
    const int sh = (g & 1) * 16;
    const uint32_t ty = (hdr.y >> sh) & 0xFFFFu, tz = (hdr.z >> sh) & 0xFFFFu,
                   tw = (hdr.w >> sh) & 0xFFFFu;
    if (g < 2) {
        s.sc0 = ty & 63;
        s.sc1 = (ty >> 8) & 63;
        s.m0 = tz & 63;
        s.m1 = (tz >> 8) & 63;
    } else {
        s.sc0 = (tw & 0xF) | ((ty >> 2) & 0x30);
        s.sc1 = ((tw >> 8) & 0xF) | ((ty >> 10) & 0x30);
        s.m0 = ((tw >> 4) & 0xF) | ((tz >> 2) & 0x30);
        s.m1 = ((tw >> 12) & 0xF) | ((tz >> 10) & 0x30);
    }
    const __half2 dm = *reinterpret_cast<const __half2 *>(&hdr.x);
    const float2 f = __half22float2(dm);
    s.d = f.x;
    s.dmin = f.y;
    return s;
}

static __device__ __forceinline__ void q4k_lane_ints(const uint4 &w, const Q4Scales &s, const int4 &alo,
                                              const int4 &ahi, int bl, int bh, int &isum,
                                              int &msum) {
    int dl = __dp4a((int)(w.x & 0x0F0F0F0Fu), alo.x, 0);
    dl = __dp4a((int)(w.y & 0x0F0F0F0Fu), alo.y, dl);
    dl = __dp4a((int)(w.z & 0x0F0F0F0Fu), alo.z, dl);
    dl = __dp4a((int)(w.w & 0x0F0F0F0Fu), alo.w, dl);
    int dh = __dp4a((int)((w.x >> 4) & 0x0F0F0F0Fu), ahi.x, 0);
    dh = __dp4a((int)((w.y >> 4) & 0x0F0F0F0Fu), ahi.y, dh);
    dh = __dp4a((int)((w.z >> 4) & 0x0F0F0F0Fu), ahi.z, dh);
    dh = __dp4a((int)((w.w >> 4) & 0x0F0F0F0Fu), ahi.w, dh);
    isum = s.sc0 * dl + s.sc1 * dh;
    msum = s.m0 * bl + s.m1 * bh;
}

// ---- Q6_K (device layout): one lane's share of one block ----------------------------------------
// ql = the lane's 16 low-nibble bytes (chunk c of 8, half h = c >> 2, cc = c & 3); qh = the 16
// bytes of 2-bit highs that cover the same 16 positions; the lane's low nibbles are elements
// 128h + 16cc .. +15 and its high nibbles elements 128h + 64 + 16cc .. +15.
// the lane's 32 six-bit codes, assembled once per weight row: vl = four words of the low-nibble elements
// (128h + 16cc .. +15), vh = four words of the high-nibble elements (128h + 64 + 16cc .. +15)
static __device__ __forceinline__ void q6k_lane_codes(const uint4 &ql, const uint4 &qh, int cc, uint32_t (&vl)[4],
                                                      uint32_t (&vh)[4]) {
    const int s_lo = 2 * (cc >> 1), s_hi = 4 + s_lo;
    const uint32_t w[4] = {ql.x, ql.y, ql.z, ql.w}, h[4] = {qh.x, qh.y, qh.z, qh.w};
#pragma unroll
    for (int i = 0; i < 4; i++) {
        vl[i] = (w[i] & 0x0F0F0F0Fu) | (((h[i] >> s_lo) & 0x03030303u) << 4);
        vh[i] = ((w[i] >> 4) & 0x0F0F0F0Fu) | (((h[i] >> s_hi) & 0x03030303u) << 4);
    }
}
// ... against one token's activations (the same integer as q6k_lane_ints)
static __device__ __forceinline__ int q6k_lane_dot(const uint32_t (&vl)[4], const uint32_t (&vh)[4], int sc_lo, int sc_hi,
                                                   const int4 &alo, const int4 &ahi, int bl, int bh) {
    int dl = __dp4a((int)vl[0], alo.x, 0), dh = __dp4a((int)vh[0], ahi.x, 0);
    dl = __dp4a((int)vl[1], alo.y, dl);
    dh = __dp4a((int)vh[1], ahi.y, dh);
    dl = __dp4a((int)vl[2], alo.z, dl);
    dh = __dp4a((int)vh[2], ahi.z, dh);
    dl = __dp4a((int)vl[3], alo.w, dl);
    dh = __dp4a((int)vh[3], ahi.w, dh);
    // codes are stored with +32 bias: sum (q-32) a = sum q a - 32 sum a
    return sc_lo * (dl - 32 * bl) + sc_hi * (dh - 32 * bh);
}

static __device__ __forceinline__ int q6k_lane_ints(const uint4 &ql, const uint4 &qh, int cc, int sc_lo,
                                             int sc_hi, const int4 &alo, const int4 &ahi, int bl,
                                             int bh) {
    const int s_lo = 2 * (cc >> 1), s_hi = 4 + s_lo;
    int dl = 0, dh = 0;
#define KQ_Q6_STEP(W, H, AL, AH)                                                            \
    {                                                                                       \
        uint32_t vl = ((W) & 0x0F0F0F0Fu) | ((((H) >> s_lo) & 0x03030303u) << 4);           \
        uint32_t vh = (((W) >> 4) & 0x0F0F0F0Fu) | ((((H) >> s_hi) & 0x03030303u) << 4);    \
        dl = __dp4a((int)vl, (AL), dl);                                                     \
        dh = __dp4a((int)vh, (AH), dh);                                                     \
    }
    KQ_Q6_STEP(ql.x, qh.x, alo.x, ahi.x)
    KQ_Q6_STEP(ql.y, qh.y, alo.y, ahi.y)
    KQ_Q6_STEP(ql.z, qh.z, alo.z, ahi.z)
    KQ_Q6_STEP(ql.w, qh.w, alo.w, ahi.w)
#undef KQ_Q6_STEP
    // codes are stored with +32 bias: sum (q-32) a = sum q a - 32 sum a
    return sc_lo * (dl - 32 * bl) + sc_hi * (dh - 32 * bh);
}

