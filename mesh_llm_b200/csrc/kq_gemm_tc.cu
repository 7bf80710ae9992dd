// Prefill contraction on the 5th-generation tensor cores: y[m][n] = sum_k W[n][k] x[m][k] for M > 8
// tokens, W in Q4_K / Q6_K blocks, x in Q8 blocks of 256, computed with tcgen05.mma kind::i8 into
// TMEM accumulators and an exact integer recombination per 256-element super-block.
//
// K-quant scales differ per 32 (Q4_K) or 16 (Q6_K) elements, so int8 products cannot simply be
// accumulated along K.  Instead the integer scale is folded into the weight:  w' = sc_j * q  is
// 10 bits (Q4_K, 0..945) or 13 bits signed (Q6_K, sc_t * (q - 32)), and is split into two int8
// planes, w' = hi * R + lo  (R = 32 / 64).  Two MMAs per 32-element K step accumulate
// sum hi*a and sum lo*a over the whole super-block in int32 (|sum| < 2^26), and the epilogue forms
// R*acc_hi + acc_lo -- bit-for-bit the integer  sum_j sc_j sum_i q_ij a_ij  of the decode kernels --
// and applies the f32 scales d_w[n,b] * d_a[m,b] once per super-block.  The Q4_K min term
// sum_j m_j * bsum_j is one more MMA (kind::f16, K = 16, small integers exact in f16 / f32).
//
// One CTA computes a 128-token x 128-row tile.  Tokens are the M (TMEM lane) dimension, weight rows
// the N (column) dimension.  Per super-block: all warps stage the tile in shared memory in the
// canonical K-major no-swizzle UMMA layout (activations copied, weights unpacked to the two
// planes), one thread issues the MMAs, and after the commit barrier all warps run the epilogue out
// of TMEM; the running f32 result also lives in TMEM (columns 384..511), so registers stay small.
// Every barrier wait is bounded; on a time-out the kernel sets an error word, frees its TMEM and
// returns.
#include "kq_common.cuh"

namespace {

constexpr int TM = 128, TN = 128, NTHREADS = 256;
constexpr int LBO = TM * 16;        // bytes between consecutive 16-byte K chunks of an operand
constexpr int SBO = 128;            // bytes between consecutive groups of 8 rows
constexpr int OP_BYTES = TM * 256;  // one int8 operand slab: 128 rows x 256 K bytes
constexpr int MIN_BYTES = TM * 32;  // one f16 operand slab of the min term: 128 rows x 16 halves
constexpr int SMEM_A = 0, SMEM_BHI = OP_BYTES, SMEM_BLO = 2 * OP_BYTES, SMEM_AMIN = 3 * OP_BYTES,
              SMEM_BMIN = 3 * OP_BYTES + MIN_BYTES, SMEM_SCAL = 3 * OP_BYTES + 2 * MIN_BYTES,
              SMEM_TOTAL = SMEM_SCAL + 3 * TM * 4 + 64;
constexpr uint32_t TMEM_COLS = 512, COL_HI = 0, COL_LO = 128, COL_MIN = 256, COL_Y = 384;
constexpr uint32_t SPIN = 1u << 20;

__device__ int g_gemm_error;

struct GemmParams {
    const uint8_t *W; // device-layout rows
    const int8_t *aq;
    const float *ad;
    const int16_t *abs16;
    float *y;
    const float *bias, *residual;
    int32_t M, N, K, nb;
    uint32_t type;
};

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

// canonical K-major, no swizzle: 16-byte chunk kc of row r
__device__ __forceinline__ uint32_t op_off(int r, int kc) { return kc * LBO + (r >> 3) * SBO + (r & 7) * 16; }

__device__ __forceinline__ uint64_t make_desc(uint32_t saddr) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFF) >> 4);
    d |= (uint64_t)(LBO >> 4) << 16;
    d |= (uint64_t)(SBO >> 4) << 32;
    d |= (uint64_t)1 << 46; // descriptor version of this architecture
    return d;               // layout type 0: no swizzle
}

// kind::i8: D s32, A s8, B s8 or u8, both K-major, M = 128, N = 128
__device__ __forceinline__ uint32_t idesc_i8(bool b_signed) {
    return (2u << 4) | (1u << 7) | ((b_signed ? 1u : 0u) << 10) | ((uint32_t)(TN >> 3) << 17) | ((uint32_t)(TM >> 4) << 24);
}
// kind::f16: D f32, A f16, B f16
__device__ __forceinline__ uint32_t idesc_f16() {
    return (1u << 4) | ((uint32_t)(TN >> 3) << 17) | ((uint32_t)(TM >> 4) << 24);
}

__device__ __forceinline__ void mma_i8(uint32_t d_tmem, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
                 :
                 : "r"(d_tmem), "l"(a), "l"(b), "r"(idesc), "r"(accumulate)
                 : "memory");
}
__device__ __forceinline__ void mma_f16(uint32_t d_tmem, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 :
                 : "r"(d_tmem), "l"(a), "l"(b), "r"(idesc), "r"(accumulate)
                 : "memory");
}

#define TMEM_LD16(taddr, r)                                                                                        \
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];" \
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),     \
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]) \
                 : "r"(taddr)                                                                                      \
                 : "memory")
#define TMEM_ST16(taddr, r)                                                                                        \
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};" \
                 :                                                                                                 \
                 : "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), \
                   "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])     \
                 : "memory")

// two 16-bit lanes per word: (q_a | q_b << 16) * sc, split into the planes and interleaved back to bytes
__device__ __forceinline__ void q4_planes(uint32_t nib4, uint32_t sc, uint32_t &hi, uint32_t &lo) {
    const uint32_t p02 = (nib4 & 0x000F000Fu) * sc;        // bytes 0 and 2
    const uint32_t p13 = ((nib4 >> 8) & 0x000F000Fu) * sc; // bytes 1 and 3
    hi = ((p02 >> 5) & 0x00FF00FFu) | (((p13 >> 5) & 0x00FF00FFu) << 8);
    lo = (p02 & 0x001F001Fu) | ((p13 & 0x001F001Fu) << 8);
}

__global__ void __launch_bounds__(NTHREADS, 1) gemm_tc_kernel(const GemmParams p) {
    KQ_PDL_ENTER();
    extern __shared__ __align__(1024) uint8_t smem[];
    __shared__ uint64_t mbar;
    __shared__ uint32_t s_tmem;
    __shared__ int s_abort;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int m0 = blockIdx.y * TM, n0 = blockIdx.x * TN;
    float *da_s = reinterpret_cast<float *>(smem + SMEM_SCAL);
    float *dw_s = da_s + TM, *dmin_s = dw_s + TM;
    const uint32_t mbar_a = smem_u32(&mbar);

    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem)),
                     "r"(TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    if (tid == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(mbar_a), "r"(1));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        s_abort = 0;
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = s_tmem;
    // this thread's TMEM window: lanes of its warp quarter, columns of its half of the tile
    const int row = (warp & 3) * 32 + lane; // token row of the tile = TMEM lane
    const int chalf = warp >> 2;            // columns [64*chalf, 64*chalf + 64)
    const uint32_t tlane = tmem + ((uint32_t)((warp & 3) * 32) << 16);

    { // running result starts at zero
        uint32_t z[16];
#pragma unroll
        for (int i = 0; i < 16; i++) z[i] = 0u;
#pragma unroll
        for (int c = 0; c < 64; c += 16) TMEM_ST16(tlane + COL_Y + chalf * 64 + c, z);
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
    }

    const uint32_t a_base = smem_u32(smem + SMEM_A), bhi_base = smem_u32(smem + SMEM_BHI),
                   blo_base = smem_u32(smem + SMEM_BLO), amin_base = smem_u32(smem + SMEM_AMIN),
                   bmin_base = smem_u32(smem + SMEM_BMIN);
    const bool q4 = p.type == B200_TYPE_Q4_K;
    const int64_t wstride = kq_device_row_bytes(p.type, p.K);
    uint32_t phase = 0;
    bool failed = false;

    for (int b = 0; b < p.nb && !failed; b++) {
        // ---- stage the tile of super-block b ---------------------------------------------------
        // activations: 128 rows x 16 chunks
        for (int i = tid; i < TM * 16; i += NTHREADS) {
            const int r = i >> 4, kc = i & 15;
            int4 v = make_int4(0, 0, 0, 0);
            if (m0 + r < p.M) v = *reinterpret_cast<const int4 *>(p.aq + (int64_t)(m0 + r) * p.K + b * 256 + kc * 16);
            *reinterpret_cast<int4 *>(smem + SMEM_A + op_off(r, kc)) = v;
        }
        if (tid < TM) {
            const int r = tid;
            da_s[r] = m0 + r < p.M ? p.ad[(int64_t)(m0 + r) * p.nb + b] : 0.f;
            if (q4) { // sums of 16 as f16 (|sum| <= 2032: exact)
                __half h[16];
#pragma unroll
                for (int k = 0; k < 16; k++)
                    h[k] = __int2half_rn(m0 + r < p.M ? (int)p.abs16[((int64_t)(m0 + r) * p.nb + b) * 16 + k] : 0);
                *reinterpret_cast<uint4 *>(smem + SMEM_AMIN + op_off(r, 0)) = *reinterpret_cast<uint4 *>(&h[0]);
                *reinterpret_cast<uint4 *>(smem + SMEM_AMIN + op_off(r, 1)) = *reinterpret_cast<uint4 *>(&h[8]);
            }
        }
        if (q4) {
            // weights: 128 rows x 8 quant chunks; chunk c gives K chunks 4g+h (low nibbles) and 4g+2+h (high)
            for (int i = tid; i < TN * 8; i += NTHREADS) {
                const int r = i >> 3, c = i & 7;
                const int g = c >> 1, h = c & 1;
                uint4 w = make_uint4(0, 0, 0, 0);
                uint32_t sc0 = 0, sc1 = 0;
                if (n0 + r < p.N) {
                    const uint8_t *blk = p.W + (int64_t)(n0 + r) * wstride + (int64_t)b * KQ_Q4K_BYTES;
                    const uint4 hdr = __ldg(reinterpret_cast<const uint4 *>(blk));
                    w = __ldg(reinterpret_cast<const uint4 *>(blk + 16 + 16 * c));
                    const uint32_t sc_lo = hdr.y & 0x3F3F3F3Fu, sc_hi = (hdr.w & 0x0F0F0F0Fu) | ((hdr.y >> 2) & 0x30303030u);
                    const uint32_t scw = g < 2 ? sc_lo : sc_hi;
                    sc0 = (scw >> (8 * ((2 * g) & 3))) & 0xFF;
                    sc1 = (scw >> (8 * ((2 * g + 1) & 3))) & 0xFF;
                    if (c == 0) {
                        const uint32_t m_lo = hdr.z & 0x3F3F3F3Fu, m_hi = ((hdr.w >> 4) & 0x0F0F0F0Fu) | ((hdr.z >> 2) & 0x30303030u);
                        const float2 dd = __half22float2(*reinterpret_cast<const __half2 *>(&hdr.x));
                        dw_s[r] = dd.x;
                        dmin_s[r] = dd.y;
                        __half mh[16]; // m_j against both sums of 16 of sub-block j
#pragma unroll
                        for (int j = 0; j < 8; j++) {
                            const uint32_t mw = j < 4 ? m_lo : m_hi;
                            const __half v = __int2half_rn((int)((mw >> (8 * (j & 3))) & 0xFF));
                            mh[2 * j] = v;
                            mh[2 * j + 1] = v;
                        }
                        *reinterpret_cast<uint4 *>(smem + SMEM_BMIN + op_off(r, 0)) = *reinterpret_cast<uint4 *>(&mh[0]);
                        *reinterpret_cast<uint4 *>(smem + SMEM_BMIN + op_off(r, 1)) = *reinterpret_cast<uint4 *>(&mh[8]);
                    }
                } else if (c == 0) {
                    dw_s[r] = 0.f;
                    dmin_s[r] = 0.f;
                    *reinterpret_cast<uint4 *>(smem + SMEM_BMIN + op_off(r, 0)) = make_uint4(0, 0, 0, 0);
                    *reinterpret_cast<uint4 *>(smem + SMEM_BMIN + op_off(r, 1)) = make_uint4(0, 0, 0, 0);
                }
                uint4 hi_l, lo_l, hi_h, lo_h;
                q4_planes(w.x & 0x0F0F0F0Fu, sc0, hi_l.x, lo_l.x);
                q4_planes(w.y & 0x0F0F0F0Fu, sc0, hi_l.y, lo_l.y);
                q4_planes(w.z & 0x0F0F0F0Fu, sc0, hi_l.z, lo_l.z);
                q4_planes(w.w & 0x0F0F0F0Fu, sc0, hi_l.w, lo_l.w);
                q4_planes((w.x >> 4) & 0x0F0F0F0Fu, sc1, hi_h.x, lo_h.x);
                q4_planes((w.y >> 4) & 0x0F0F0F0Fu, sc1, hi_h.y, lo_h.y);
                q4_planes((w.z >> 4) & 0x0F0F0F0Fu, sc1, hi_h.z, lo_h.z);
                q4_planes((w.w >> 4) & 0x0F0F0F0Fu, sc1, hi_h.w, lo_h.w);
                const uint32_t o_l = op_off(r, 4 * g + h), o_h = op_off(r, 4 * g + 2 + h);
                *reinterpret_cast<uint4 *>(smem + SMEM_BHI + o_l) = hi_l;
                *reinterpret_cast<uint4 *>(smem + SMEM_BLO + o_l) = lo_l;
                *reinterpret_cast<uint4 *>(smem + SMEM_BHI + o_h) = hi_h;
                *reinterpret_cast<uint4 *>(smem + SMEM_BLO + o_h) = lo_h;
            }
        } else {
            // Q6_K: one task per (row, qh chunk j): 4 scale groups of 16 elements, w' = sc * (q - 32)
            // split as hi * 64 + lo with lo in 0..63 (unsigned plane) and hi in -64..64 (signed plane)
            for (int i = tid; i < TN * 4; i += NTHREADS) {
                const int r = i >> 2, j = i & 3;
                const int hh = j >> 1, c1 = j & 1;
                uint32_t hw[4] = {0, 0, 0, 0}, aw[4] = {0, 0, 0, 0}, bw[4] = {0, 0, 0, 0};
                int scg[4] = {0, 0, 0, 0};
                if (n0 + r < p.N) {
                    const uint8_t *rowp = p.W + (int64_t)(n0 + r) * wstride;
                    const KqQ6Addr qa = kq_q6_addr(p.nb, b);
                    const uint4 hv = __ldg(reinterpret_cast<const uint4 *>(rowp + qa.qh + j * qa.cs));
                    const uint4 la = __ldg(reinterpret_cast<const uint4 *>(rowp + qa.ql + (4 * hh + c1) * qa.cs));
                    const uint4 lb = __ldg(reinterpret_cast<const uint4 *>(rowp + qa.ql + (4 * hh + c1 + 2) * qa.cs));
                    hw[0] = hv.x; hw[1] = hv.y; hw[2] = hv.z; hw[3] = hv.w;
                    aw[0] = la.x; aw[1] = la.y; aw[2] = la.z; aw[3] = la.w;
                    bw[0] = lb.x; bw[1] = lb.y; bw[2] = lb.z; bw[3] = lb.w;
                    const int8_t *scp = reinterpret_cast<const int8_t *>(rowp + qa.sc);
#pragma unroll
                    for (int q = 0; q < 4; q++) scg[q] = scp[8 * hh + 2 * q + c1];
                    if (j == 0) {
                        dw_s[r] = kq_h2f(*reinterpret_cast<const uint16_t *>(rowp + qa.d));
                        dmin_s[r] = 0.f;
                    }
                } else if (j == 0) {
                    dw_s[r] = 0.f;
                    dmin_s[r] = 0.f;
                }
#pragma unroll
                for (int q = 0; q < 4; q++) { // bit pair q of the qh bytes: elements 128hh + 32q + 16c1 + i
                    uint32_t hi4[4], lo4[4];
#pragma unroll
                    for (int wd = 0; wd < 4; wd++) {
                        const uint32_t nib = (q & 1) ? bw[wd] : aw[wd];
                        const uint32_t l4 = (q & 2) ? (nib >> 4) & 0x0F0F0F0Fu : nib & 0x0F0F0F0Fu;
                        const uint32_t h2 = (hw[wd] >> (2 * q)) & 0x03030303u;
                        const uint32_t code = l4 | (h2 << 4); // 4 codes 0..63
                        uint32_t hi = 0, lo = 0;
#pragma unroll
                        for (int k = 0; k < 4; k++) {
                            const int wv = scg[q] * ((int)((code >> (8 * k)) & 0xFF) - 32);
                            hi |= (uint32_t)((wv >> 6) & 0xFF) << (8 * k);
                            lo |= (uint32_t)(wv & 63) << (8 * k);
                        }
                        hi4[wd] = hi;
                        lo4[wd] = lo;
                    }
                    const uint32_t o = op_off(r, 8 * hh + 2 * q + c1);
                    *reinterpret_cast<uint4 *>(smem + SMEM_BHI + o) = make_uint4(hi4[0], hi4[1], hi4[2], hi4[3]);
                    *reinterpret_cast<uint4 *>(smem + SMEM_BLO + o) = make_uint4(lo4[0], lo4[1], lo4[2], lo4[3]);
                }
            }
        }
        // shared-memory writes of the generic proxy must be visible to the tensor core's async proxy
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();
        // ---- MMAs ------------------------------------------------------------------------------
        if (warp == 0) {
          // the whole warp stays here while its first lane issues, so that no lane of the issuing
          // warp sits in a blocking barrier wait before the MMAs have been handed to the tensor core
          if (lane == 0) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t id_hi = idesc_i8(true), id_lo = idesc_i8(q4 ? true : false);
#pragma unroll
            for (int s = 0; s < 8; s++) { // K = 32 per instruction: chunks 2s, 2s+1
                const uint64_t ad = make_desc(a_base + 2 * s * LBO);
                mma_i8(tmem + COL_HI, ad, make_desc(bhi_base + 2 * s * LBO), id_hi, s > 0);
                mma_i8(tmem + COL_LO, ad, make_desc(blo_base + 2 * s * LBO), id_lo, s > 0);
            }
            if (q4) mma_f16(tmem + COL_MIN, make_desc(amin_base), make_desc(bmin_base), idesc_f16(), 0);
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(mbar_a)
                         : "memory");
          }
          __syncwarp();
        }
        { // bounded wait for the MMAs of this super-block
            const bool ok = s_abort ? false : kq_mbar_wait(mbar_a, phase, 5 * KQ_WAIT_LIMIT_NS);
            if (!ok) {
                s_abort = 1;
                atomicExch(&g_gemm_error, 1);
            }
            phase ^= 1;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (s_abort) failed = true;
        // ---- epilogue of the super-block: y += d_a * (d_w * (R*hi + lo) - dmin * min) ------------
        if (!failed) {
            const float da = da_s[row];
            const int R = q4 ? 32 : 64;
#pragma unroll 1
            for (int c = 0; c < 64; c += 16) {
                const uint32_t col = chalf * 64 + c;
                uint32_t hi[16], lo[16], mn[16], yy[16];
                TMEM_LD16(tlane + COL_HI + col, hi);
                TMEM_LD16(tlane + COL_LO + col, lo);
                TMEM_LD16(tlane + COL_Y + col, yy);
                if (q4) TMEM_LD16(tlane + COL_MIN + col, mn);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                for (int i = 0; i < 16; i++) {
                    const int main_i = R * (int)hi[i] + (int)lo[i];
                    float t = dw_s[col + i] * (float)main_i;
                    if (q4) t -= dmin_s[col + i] * __uint_as_float(mn[i]);
                    yy[i] = __float_as_uint(fmaf(da, t, __uint_as_float(yy[i])));
                }
                TMEM_ST16(tlane + COL_Y + col, yy);
            }
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads(); // accumulators and the staging buffers are free again
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    }

    // ---- write the tile -------------------------------------------------------------------------
    if (!failed) { // tcgen05.ld is warp-collective: every lane takes part, only the stores are masked
#pragma unroll 1
        for (int c = 0; c < 64; c += 16) {
            const int col = chalf * 64 + c;
            uint32_t yy[16];
            TMEM_LD16(tlane + COL_Y + col, yy);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            const int64_t o = (int64_t)(m0 + row) * p.N + n0 + col;
#pragma unroll
            for (int i = 0; i < 16; i++) {
                if (m0 + row < p.M && n0 + col + i < p.N) {
                    float v = __uint_as_float(yy[i]);
                    if (p.bias) v += p.bias[n0 + col + i];
                    if (p.residual) v += p.residual[o + i];
                    p.y[o + i] = v;
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
}

} // namespace

int kq_gemm_error_fetch() {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_gemm_error, sizeof(int)) != cudaSuccess) return -1;
    if (v) cudaMemcpyToSymbol(g_gemm_error, &zero, sizeof(int));
    return v;
}

b200_status kq_launch_gemm_tc(uint32_t type, const uint8_t *W, const int8_t *q, const float *d, const int16_t *bs,
                              int64_t M, int64_t N, int64_t K, float *y, const float *bias, const float *residual,
                              cudaStream_t st) {
    KQ_REQUIRE(type == B200_TYPE_Q4_K || type == B200_TYPE_Q6_K, "gemm: weight type %u", type);
    KQ_REQUIRE(K % 256 == 0 && M > 0 && N > 0, "gemm: bad shape");
    KQ_REQUIRE(((uintptr_t)W & 15) == 0 && ((uintptr_t)q & 15) == 0, "gemm: operands must be 16-byte aligned");
    GemmParams p = {W, q, d, bs, y, bias, residual, (int32_t)M, (int32_t)N, (int32_t)K, (int32_t)(K / 256), type};
    static bool attr = false;
    // 118 KB of dynamic shared memory also keeps a second CTA off the SM: a CTA holds all 512 TMEM columns
    const int smem = SMEM_TOTAL > 118 * 1024 ? SMEM_TOTAL : 118 * 1024;
    if (!attr) {
        KQ_CUDA(cudaFuncSetAttribute(gemm_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        attr = true;
    }
    dim3 grid((unsigned)kq_div_up(N, TN), (unsigned)kq_div_up(M, TM));
    kq_launch(gemm_tc_kernel, grid, NTHREADS, smem, st, p);
    KQ_COUNT_LAUNCH();
    KQ_LAUNCH_CHECK();
    return B200_OK;
}
