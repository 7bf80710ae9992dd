// KV-cache row formats.  mesh-llm starts its servers with --cache-type-k / --cache-type-v chosen
// by model size (mesh-llm/src/inference/launch.rs:568-591): f16 / f16 below 5 GB, q8_0 K with
// q4_0 V from 5 to 50 GB, q4_0 / q4_0 above.  The block arithmetic is ggml's (block of 32 values,
// one f16 scale: q8_0 d = amax / 127, q = round(x / d); q4_0 d = (value of largest magnitude) / -8,
// q = min(15, trunc(x / d + 8.5)), decode (q - 8) * d).
//
// Device layout of one quantised row (one position, one KV head, hd values): the codes of all
// hd / 32 blocks first (q8_0: hd bytes; q4_0: hd / 2 bytes, block b in bytes [16 b, 16 b + 16), value
// j of the block in the low and value j + 16 in the high nibble of byte j), then the hd / 32 f16
// scales, padded to a multiple of 16 bytes so that a row can be the inner extent of a TMA box and
// 16-byte loads of the codes stay aligned.  hd = 128: 144 bytes (q8_0), 80 bytes (q4_0).
#pragma once
#include "kq_common.cuh"

constexpr int KQ_KV_F16 = 1, KQ_KV_Q4_0 = 2, KQ_KV_Q8_0 = 8; // ggml type ids

struct KqKvTypes {
    int k = KQ_KV_F16, v = KQ_KV_F16;
    __host__ __device__ bool quantised() const { return k != KQ_KV_F16 || v != KQ_KV_F16; }
};

__host__ __device__ inline bool kq_kv_type_ok(int type) { return type == KQ_KV_F16 || type == KQ_KV_Q4_0 || type == KQ_KV_Q8_0; }
__host__ __device__ inline int kq_kv_codes_bytes(int type, int hd) {
    return type == KQ_KV_Q8_0 ? hd : type == KQ_KV_Q4_0 ? hd / 2 : hd * 2;
}
__host__ __device__ inline int kq_kv_row_bytes(int type, int hd) {
    if (type == KQ_KV_Q8_0 || type == KQ_KV_Q4_0) return (kq_kv_codes_bytes(type, hd) + hd / 16 + 15) & ~15;
    return hd * 2;
}

#ifdef __CUDACC__
// One warp quantises a block of 32 values (lane = value within the block, x = that value): q is the
// lane's code (q8_0: -127 .. 127; q4_0: 0 .. 15), dh the block's f16 scale; returns the f16 value the
// cache will decode the lane's code to.  Multiplications, the addition and the divisions are the
// individually rounded IEEE operations of the scalar definition (no fused multiply-add).
__device__ __forceinline__ __half kq_kv_block_codes(int type, float x, int &q, __half &dh) {
    const float ax = fabsf(x);
    const float amax = kq_warp_max(ax);
    if (type == KQ_KV_Q8_0) {
        const float d = __fdiv_rn(amax, 127.f);
        const float id = d != 0.f ? __fdiv_rn(1.f, d) : 0.f;
        q = (int)roundf(__fmul_rn(x, id));
        dh = __float2half_rn(d);
        return __float2half_rn(__fmul_rn((float)q, __half2float(dh)));
    }
    // q4_0: the first value of largest magnitude sets the scale, with its sign
    const unsigned who = __ballot_sync(0xffffffffu, ax == amax);
    const float first = __shfl_sync(0xffffffffu, x, __ffs(who) - 1);
    const float mx = amax == 0.f ? 0.f : first;
    const float d = __fdiv_rn(mx, -8.f);
    const float id = d != 0.f ? __fdiv_rn(1.f, d) : 0.f;
    q = (int)__fadd_rn(__fmul_rn(x, id), 8.5f); // truncation, values in [0.5, 16.5]
    q = min(q, 15);
    dh = __float2half_rn(d);
    return __float2half_rn(__fmul_rn((float)(q - 8), __half2float(dh)));
}

// ... and stores it as block `blk` of a row in the device layout (codes of all blocks, then the scales)
__device__ __forceinline__ __half kq_kv_store_block(int type, float x, uint8_t *row, int hd, int blk, int lane) {
    int q;
    __half dh;
    const __half back = kq_kv_block_codes(type, x, q, dh);
    __half *scales = reinterpret_cast<__half *>(row + kq_kv_codes_bytes(type, hd));
    if (type == KQ_KV_Q8_0) {
        row[blk * 32 + lane] = (uint8_t)(int8_t)q;
    } else {
        const int hi = __shfl_down_sync(0xffffffffu, q, 16);
        if (lane < 16) row[blk * 16 + lane] = (uint8_t)(q | (hi << 4));
    }
    if (lane == 0) scales[blk] = dh;
    return back;
}

// ... or as a block of ggml's own layout (block_q8_0: f16 d, int8 qs[32], 34 bytes; block_q4_0: f16 d,
// uint8 qs[16] with value j in the low and value j + 16 in the high nibble of byte j, 18 bytes)
__device__ __forceinline__ void kq_kv_store_ggml_block(int type, float x, uint8_t *block, int lane) {
    int q;
    __half dh;
    kq_kv_block_codes(type, x, q, dh);
    if (type == KQ_KV_Q8_0) {
        block[2 + lane] = (uint8_t)(int8_t)q;
    } else {
        const int hi = __shfl_down_sync(0xffffffffu, q, 16);
        if (lane < 16) block[2 + lane] = (uint8_t)(q | (hi << 4));
    }
    if (lane == 0) *reinterpret_cast<__half *>(block) = dh; // blocks are 2-byte aligned
}

__device__ __forceinline__ uint32_t kq_kv_h2(float a, float b) {
    const __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<const uint32_t *>(&h);
}

// values [16 c, 16 c + 16) of a q8_0 row as f16: out[0] holds the first eight, out[1] the rest
__device__ __forceinline__ void kq_kv_decode16_q8_0(const uint8_t *row, int hd, int c, uint4 (&out)[2]) {
    const uint4 raw = *reinterpret_cast<const uint4 *>(row + c * 16);
    const float d = __half2float(reinterpret_cast<const __half *>(row + hd)[c >> 1]);
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
    uint32_t o[8];
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const float f0 = (float)(int)(int8_t)(w[i] & 0xFF), f1 = (float)(int)(int8_t)((w[i] >> 8) & 0xFF),
                    f2 = (float)(int)(int8_t)((w[i] >> 16) & 0xFF), f3 = (float)(int)(int8_t)(w[i] >> 24);
        o[2 * i] = kq_kv_h2(__fmul_rn(f0, d), __fmul_rn(f1, d));
        o[2 * i + 1] = kq_kv_h2(__fmul_rn(f2, d), __fmul_rn(f3, d));
    }
    out[0] = make_uint4(o[0], o[1], o[2], o[3]);
    out[1] = make_uint4(o[4], o[5], o[6], o[7]);
}

// block b (32 values) of a q4_0 row as f16: out[i] holds values [8 i, 8 i + 8) of the block
__device__ __forceinline__ void kq_kv_decode32_q4_0(const uint8_t *row, int hd, int b, uint4 (&out)[4]) {
    const uint4 raw = *reinterpret_cast<const uint4 *>(row + b * 16);
    const float d = __half2float(reinterpret_cast<const __half *>(row + hd / 2)[b]);
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
    uint32_t lo[8], hi[8];
#pragma unroll
    for (int i = 0; i < 4; i++) {
        float l[4], h[4];
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int byte = (w[i] >> (8 * j)) & 0xFF;
            l[j] = __fmul_rn((float)((byte & 15) - 8), d);
            h[j] = __fmul_rn((float)((byte >> 4) - 8), d);
        }
        lo[2 * i] = kq_kv_h2(l[0], l[1]);
        lo[2 * i + 1] = kq_kv_h2(l[2], l[3]);
        hi[2 * i] = kq_kv_h2(h[0], h[1]);
        hi[2 * i + 1] = kq_kv_h2(h[2], h[3]);
    }
    out[0] = make_uint4(lo[0], lo[1], lo[2], lo[3]);
    out[1] = make_uint4(lo[4], lo[5], lo[6], lo[7]);
    out[2] = make_uint4(hi[0], hi[1], hi[2], hi[3]);
    out[3] = make_uint4(hi[4], hi[5], hi[6], hi[7]);
}
#endif
