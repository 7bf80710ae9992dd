// Causal attention for a batch of new tokens (prefill) over the KV cache (f16, or q8_0 / q4_0 rows
// decoded to f16 while a tile is staged), on the tensor cores.
//
// One CTA serves 16 consecutive query rows of one sequence for the G query heads that share a KV
// head: warp w owns head kh*G + w, so a K / V tile brought into shared memory once is used by all
// G heads.  Tiles of 64 positions are staged with cp.async (double-buffered, rows padded by 16 bytes
// so that ldmatrix reads eight rows from eight different bank groups).  Per tile a warp forms
// S = Q K^T with mma.m16n8k16 (Q in f16 registers, pre-scaled by 1/sqrt(hd) * log2 e; K fragments by
// ldmatrix), applies the causal mask, updates the running row maximum and sum in f32 (online
// softmax, base 2), turns the probabilities into f16 A-fragments in registers and accumulates
// O += P V (V fragments by ldmatrix.trans).  Only tiles up to the diagonal are visited; the query
// tiles with the longest history are scheduled first.
#include "kq_common.cuh"
#include "kq_kvq.cuh"

#include <math.h>

namespace {

constexpr int HD = 128, BQ = 16, BK = 64, PITCH = HD * 2 + 16, TILE_BYTES = BK * PITCH;

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ uint32_t pack_h2(float a, float b) {
    const __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<const uint32_t *>(&h);
}
__device__ __forceinline__ void mma_f16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t &r0, uint32_t &r1, uint32_t &r2, uint32_t &r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t &r0, uint32_t &r1, uint32_t &r2, uint32_t &r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}

template <int G>
__global__ void __launch_bounds__(G * 32) attn_prefill_kernel(const float *q, const __half *kc,
                                                               const __half *vc, int T, const int32_t *pos0_dev,
                                                               int pos0, int n_head, int n_kv, int64_t seq_stride,
                                                               float scale_log2, float *out, KqKvTypes kvt) {
    KQ_PDL_ENTER();
    extern __shared__ __align__(128) uint8_t sm[]; // K tiles [2], then V tiles [2]
    const int qt = (int)gridDim.x - 1 - (int)blockIdx.x, kh = blockIdx.y, seq = blockIdx.z;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
    const int head = kh * G + warp;
    const int p0 = pos0_dev ? *pos0_dev : pos0;
    const int r0 = qt * BQ, ra = r0 + g, rb = r0 + g + 8;
    const bool va = ra < T, vb = rb < T;
    const int kv_end = p0 + min(T, r0 + BQ); // positions [0, kv_end) can be visible to this tile
    const int n_tiles = (kv_end + BK - 1) / BK;
    const __half *kbase = kc + seq * seq_stride + (int64_t)kh * HD;
    const __half *vbase = vc + seq * seq_stride + (int64_t)kh * HD;
    const int64_t pstride = (int64_t)n_kv * HD;

    // a quantised row: decoded by plain loads into the same f16 tile layout (rows past the end as zeros)
    auto decode_tile = [&](uint8_t *dst, const __half *cache, int type, int tile) {
        const int rb = kq_kv_row_bytes(type, HD);
        const uint8_t *base = reinterpret_cast<const uint8_t *>(cache) + (seq * (seq_stride / HD) + kh) * rb;
        const int per_row = type == KQ_KV_Q8_0 ? 8 : 4; // tasks of 16 (q8_0) or 32 (q4_0) values
        for (int i = threadIdx.x; i < BK * per_row; i += G * 32) {
            const int row = i / per_row, c = i % per_row, pos = tile * BK + row;
            uint4 v[4] = {};
            if (pos < kv_end) {
                const uint8_t *src = base + (int64_t)pos * n_kv * rb;
                if (type == KQ_KV_Q8_0) {
                    uint4 t2[2];
                    kq_kv_decode16_q8_0(src, HD, c, t2);
                    v[0] = t2[0];
                    v[1] = t2[1];
                } else {
                    kq_kv_decode32_q4_0(src, HD, c, v);
                }
            }
            uint4 *o = reinterpret_cast<uint4 *>(dst + row * PITCH + c * (type == KQ_KV_Q8_0 ? 32 : 64));
            o[0] = v[0];
            o[1] = v[1];
            if (type != KQ_KV_Q8_0) {
                o[2] = v[2];
                o[3] = v[3];
            }
        }
    };
    auto load_tile = [&](int buf, int tile) {
        const uint32_t ks = smem_u32(sm + buf * TILE_BYTES), vs = smem_u32(sm + (2 + buf) * TILE_BYTES);
        const bool kf = kvt.k == KQ_KV_F16, vf = kvt.v == KQ_KV_F16;
        if (kf || vf)
            for (int i = threadIdx.x; i < BK * 16; i += G * 32) {
                const int row = i >> 4, c = i & 15, pos = tile * BK + row;
                const bool in = pos < kv_end;
                const int64_t off = (int64_t)(in ? pos : 0) * pstride + c * 8;
                const uint32_t bytes = in ? 16u : 0u; // rows past the end arrive as zeros
                if (kf)
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(ks + row * PITCH + c * 16), "l"(kbase + off), "r"(bytes)
                                 : "memory");
                if (vf)
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(vs + row * PITCH + c * 16), "l"(vbase + off), "r"(bytes)
                                 : "memory");
            }
        asm volatile("cp.async.commit_group;" ::: "memory");
        if (!kf) decode_tile(sm + buf * TILE_BYTES, kc, kvt.k, tile);
        if (!vf) decode_tile(sm + (2 + buf) * TILE_BYTES, vc, kvt.v, tile);
    };
    load_tile(0, 0);

    // Q fragments: rows ra / rb of this head, 8 k-steps of 16 dims
    uint32_t qf[8][4];
    {
        const float *qa = q + ((int64_t)(seq * T + (va ? ra : 0)) * n_head + head) * HD;
        const float *qb = q + ((int64_t)(seq * T + (vb ? rb : 0)) * n_head + head) * HD;
#pragma unroll
        for (int kk = 0; kk < 8; kk++) {
            const float2 a0 = *reinterpret_cast<const float2 *>(qa + 16 * kk + 2 * t);
            const float2 a1 = *reinterpret_cast<const float2 *>(qa + 16 * kk + 8 + 2 * t);
            const float2 b0 = *reinterpret_cast<const float2 *>(qb + 16 * kk + 2 * t);
            const float2 b1 = *reinterpret_cast<const float2 *>(qb + 16 * kk + 8 + 2 * t);
            qf[kk][0] = va ? pack_h2(a0.x * scale_log2, a0.y * scale_log2) : 0u;
            qf[kk][1] = vb ? pack_h2(b0.x * scale_log2, b0.y * scale_log2) : 0u;
            qf[kk][2] = va ? pack_h2(a1.x * scale_log2, a1.y * scale_log2) : 0u;
            qf[kk][3] = vb ? pack_h2(b1.x * scale_log2, b1.y * scale_log2) : 0u;
        }
    }
    float o[16][4];
#pragma unroll
    for (int i = 0; i < 16; i++) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.f, l_b = 0.f;
    const int lim_a = p0 + ra, lim_b = p0 + rb; // last visible position of each row

    for (int tile = 0; tile < n_tiles; tile++) {
        const int buf = tile & 1;
        if (tile + 1 < n_tiles) {
            load_tile(buf ^ 1, tile + 1);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();
        const uint32_t ks = smem_u32(sm + buf * TILE_BYTES), vs = smem_u32(sm + (2 + buf) * TILE_BYTES);
        // ---- S = Q K^T for 64 positions
        float s[8][4];
#pragma unroll
        for (int j = 0; j < 8; j++) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
        const int lm = lane >> 3, lr = lane & 7;
#pragma unroll
        for (int kk = 0; kk < 8; kk++) {
#pragma unroll
            for (int j = 0; j < 8; j += 2) {
                uint32_t b0, b1, b2, b3;
                ldsm_x4(ks + (8 * (j + (lm >> 1)) + lr) * PITCH + (16 * kk + 8 * (lm & 1)) * 2, b0, b1, b2, b3);
                mma_f16(s[j], qf[kk], b0, b1);
                mma_f16(s[j + 1], qf[kk], b2, b3);
            }
        }
        // ---- causal mask, running maximum
        const int pbase = tile * BK + 2 * t;
        float tm_a = -INFINITY, tm_b = -INFINITY;
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const int p = pbase + 8 * j;
            if (p > lim_a) s[j][0] = -INFINITY;
            if (p + 1 > lim_a) s[j][1] = -INFINITY;
            if (p > lim_b) s[j][2] = -INFINITY;
            if (p + 1 > lim_b) s[j][3] = -INFINITY;
            tm_a = fmaxf(tm_a, fmaxf(s[j][0], s[j][1]));
            tm_b = fmaxf(tm_b, fmaxf(s[j][2], s[j][3]));
        }
        tm_a = fmaxf(tm_a, __shfl_xor_sync(0xffffffffu, tm_a, 1));
        tm_a = fmaxf(tm_a, __shfl_xor_sync(0xffffffffu, tm_a, 2));
        tm_b = fmaxf(tm_b, __shfl_xor_sync(0xffffffffu, tm_b, 1));
        tm_b = fmaxf(tm_b, __shfl_xor_sync(0xffffffffu, tm_b, 2));
        const float mn_a = fmaxf(m_a, tm_a), mn_b = fmaxf(m_b, tm_b);
        const float al_a = mn_a == -INFINITY ? 1.f : exp2f(m_a - mn_a), al_b = mn_b == -INFINITY ? 1.f : exp2f(m_b - mn_b);
        const float sub_a = mn_a == -INFINITY ? 0.f : mn_a, sub_b = mn_b == -INFINITY ? 0.f : mn_b;
        m_a = mn_a;
        m_b = mn_b;
        l_a *= al_a;
        l_b *= al_b;
#pragma unroll
        for (int i = 0; i < 16; i++) {
            o[i][0] *= al_a; o[i][1] *= al_a; o[i][2] *= al_b; o[i][3] *= al_b;
        }
        // ---- probabilities as f16 A-fragments; O += P V
#pragma unroll
        for (int k2 = 0; k2 < 4; k2++) {
            uint32_t pf[4];
            {
                const float e00 = exp2f(s[2 * k2][0] - sub_a), e01 = exp2f(s[2 * k2][1] - sub_a);
                const float e02 = exp2f(s[2 * k2][2] - sub_b), e03 = exp2f(s[2 * k2][3] - sub_b);
                const float e10 = exp2f(s[2 * k2 + 1][0] - sub_a), e11 = exp2f(s[2 * k2 + 1][1] - sub_a);
                const float e12 = exp2f(s[2 * k2 + 1][2] - sub_b), e13 = exp2f(s[2 * k2 + 1][3] - sub_b);
                l_a += (e00 + e01) + (e10 + e11);
                l_b += (e02 + e03) + (e12 + e13);
                pf[0] = pack_h2(e00, e01);
                pf[1] = pack_h2(e02, e03);
                pf[2] = pack_h2(e10, e11);
                pf[3] = pack_h2(e12, e13);
            }
#pragma unroll
            for (int nt = 0; nt < 16; nt += 2) {
                uint32_t b0, b1, b2, b3;
                ldsm_x4_t(vs + (16 * k2 + 8 * (lm & 1) + lr) * PITCH + (8 * (nt + (lm >> 1))) * 2, b0, b1, b2, b3);
                mma_f16(o[nt], pf, b0, b1);
                mma_f16(o[nt + 1], pf, b2, b3);
            }
        }
        __syncthreads(); // the buffer is refilled two tiles later
    }
    l_a += __shfl_xor_sync(0xffffffffu, l_a, 1);
    l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
    l_b += __shfl_xor_sync(0xffffffffu, l_b, 1);
    l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);
    const float ia = l_a > 0.f ? 1.f / l_a : 0.f, ib = l_b > 0.f ? 1.f / l_b : 0.f;
    float *oa = out + ((int64_t)(seq * T + ra) * n_head + head) * HD;
    float *ob = out + ((int64_t)(seq * T + rb) * n_head + head) * HD;
#pragma unroll
    for (int nt = 0; nt < 16; nt++) {
        if (va) *reinterpret_cast<float2 *>(oa + 8 * nt + 2 * t) = make_float2(o[nt][0] * ia, o[nt][1] * ia);
        if (vb) *reinterpret_cast<float2 *>(ob + 8 * nt + 2 * t) = make_float2(o[nt][2] * ib, o[nt][3] * ib);
    }
}

} // namespace

// q [n_seq * T][n_head][128] f32 (already rotated), caches [seq][pos][n_kv] rows of 128 values; returns
// B200_ERR_UNSUPPORTED when the shape is not one this kernel is built for (the caller then uses the
// per-row kernel).
b200_status kq_attention_prefill_mma(const float *q, const uint16_t *kc, const uint16_t *vc, int n_seq, int T,
                                     const int32_t *pos0_dev, int pos0, int n_head, int n_kv, int hd, int64_t seq_stride,
                                     float *out, KqKvTypes kvt, cudaStream_t st) {
    if (hd != HD || n_kv <= 0 || n_head % n_kv != 0) return B200_ERR_UNSUPPORTED;
    const int G = n_head / n_kv;
    if (((uintptr_t)q & 7) || ((uintptr_t)out & 7) || ((uintptr_t)kc & 15) || ((uintptr_t)vc & 15) || (seq_stride & 7))
        return B200_ERR_UNSUPPORTED;
    const float scale_log2 = 1.4426950408889634f / sqrtf((float)hd);
    const dim3 grid((unsigned)kq_div_up(T, BQ), (unsigned)n_kv, (unsigned)n_seq);
    const int smem = 4 * TILE_BYTES;
#define KQ_APF(GG)                                                                                                         \
    {                                                                                                                      \
        static bool attr[16]; /* the attribute belongs to a (kernel, device) pair */                                      \
        int dev = 0;                                                                                                       \
        KQ_CUDA(cudaGetDevice(&dev));                                                                                      \
        if (dev < 0 || dev >= 16 || !attr[dev]) {                                                                          \
            KQ_CUDA(cudaFuncSetAttribute(attn_prefill_kernel<GG>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));     \
            if (dev >= 0 && dev < 16) attr[dev] = true;                                                                    \
        }                                                                                                                  \
        kq_launch(attn_prefill_kernel<GG>, grid, GG * 32, smem, st, q, (const __half *)kc, (const __half *)vc, T, pos0_dev, \
                  pos0, n_head, n_kv, seq_stride, scale_log2, out, kvt);                                                      \
    }
    switch (G) {
    case 1: KQ_APF(1); break;
    case 2: KQ_APF(2); break;
    case 4: KQ_APF(4); break;
    case 5: KQ_APF(5); break;
    case 8: KQ_APF(8); break;
    default: return B200_ERR_UNSUPPORTED;
    }
#undef KQ_APF
    KQ_COUNT_LAUNCH();
    KQ_LAUNCH_CHECK();
    return B200_OK;
}
