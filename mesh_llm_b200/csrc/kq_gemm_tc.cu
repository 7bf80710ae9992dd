// Prefill contraction on the 5th-generation tensor cores: y[m][n] = sum_k W[n][k] x[m][k] for M > 8
// tokens, W in Q4_K / Q6_K blocks, x in Q8 blocks of 256, computed with tcgen05.mma kind::i8 into
// TMEM accumulators and an exact integer recombination per 256-element super-block.
//
// K-quant scales differ per 32 (Q4_K) or 16 (Q6_K) elements, so int8 products cannot simply be
// accumulated along K.  Instead the integer scale is folded into the weight:  w' = sc_j * q  is
// 10 bits (Q4_K, 0..945) or 13 bits signed (Q6_K, sc_t * (q - 32)), and is split into two int8
// planes, w' = hi * R + lo  (R = 256 / 64; low plane unsigned).  Two MMAs per 32-element K step accumulate
// sum hi*a and sum lo*a over the whole super-block in int32 (|sum| < 2^26), and the epilogue forms
// R*acc_hi + acc_lo -- bit-for-bit the integer  sum_j sc_j sum_i q_ij a_ij  of the decode kernels --
// and applies the f32 scales d_w[n,b] * d_a[m,b] once per super-block.  The Q4_K min term
// sum_j m_j * bsum_j is one more MMA (kind::f16, K = 16, small integers exact in f16 / f32).
//
// One CTA computes a 128-token x 64-row tile, and two CTAs share an SM (256 TMEM columns and under
// half of the shared memory each), so one CTA's unpacking and TMEM draining overlap the other's MMAs
// and copies.  Tokens are the M (TMEM lane) dimension, weight rows the N (column) dimension.  A small
// kernel first re-tiles the Q8 codes so that one super-block of a token tile is a contiguous 32 KB
// run in the canonical K-major no-swizzle UMMA layout.  Per super-block the copy engine brings that
// run and the packed Q4_K blocks of the 64 weight rows (one tiled TMA box out of the row-major
// matrix, requested one super-block ahead); all warps unpack the weights from shared memory to the
// two planes, one thread issues the MMAs, and after the commit barrier all warps run the epilogue
// out of TMEM into the running f32 result in registers.
// Every barrier wait is bounded; on a time-out the kernel sets an error word, frees its TMEM and
// returns.
#include "kq_common.cuh"

#include <algorithm>
#include <mutex>
#include <stdlib.h>

#include <cuda.h> // CUtensorMap and the encode entry point's types; the driver is reached through the runtime
#include <string.h>

namespace {

constexpr int TM = 128, TN = 64, NTHREADS = 256, NCOL = TN / 2; // NCOL: result columns per thread
constexpr int LBO_A = TM * 16;      // bytes between consecutive 16-byte K chunks of the token operand
constexpr int LBO_B = 2 * TN * 16;  // ... of the weight operand: the hi plane's rows, then the lo plane's (one tile of 2 TN rows)
constexpr int LBO_BMIN = TN * 16;   // ... of the f16 min operand
constexpr int SBO = 128;            // bytes between consecutive groups of 8 rows
constexpr int A_BYTES = TM * 256;   // int8 token slab: 128 rows x 256 K bytes
constexpr int B_BYTES = TN * 256;   // one int8 weight plane
constexpr int AMIN_BYTES = TM * 32; // f16 operands of the min term: 16 halves per row
constexpr int BMIN_BYTES = TN * 32;
constexpr int RAW_BYTES = TN * KQ_Q4K_BYTES; // packed Q4_K blocks of one super-block column
constexpr int SMEM_A = 0, SMEM_BHI = A_BYTES, SMEM_BLO = SMEM_BHI + B_BYTES, SMEM_AMIN = SMEM_BLO + B_BYTES,
              SMEM_BMIN = SMEM_AMIN + AMIN_BYTES, SMEM_RAW = SMEM_BMIN + BMIN_BYTES, SMEM_SCAL = SMEM_RAW + 2 * RAW_BYTES,
              SMEM_TOTAL = SMEM_SCAL + (TM + 2 * TN) * 4 + 64;
static_assert(SMEM_RAW % 128 == 0 && RAW_BYTES % 128 == 0, "TMA destinations are 128-byte aligned");
constexpr uint32_t TMEM_COLS = 256, COL_HI = 0, COL_LO = TN, COL_MIN = 2 * TN;
constexpr int KQ_MAX_DEVICES = 16;

__device__ int g_gemm_error;
#ifdef KQ_GEMM_PROF
__device__ long long g_gemm_prof[8];
#define PROF_T(var) const long long var = clock64()
#define PROF_ADD(i, a, b) do { if (blockIdx.x == 0 && blockIdx.y == 0 && tid == 32) g_gemm_prof[i] += (b) - (a); } while (0)
#else
#define PROF_T(var)
#define PROF_ADD(i, a, b)
#endif

struct GemmParams {
    const uint8_t *W; // device-layout rows
    const int8_t *aq;  // activations re-tiled for the tensor core: [M/128][K/16][128 rows][16 bytes]
    const float *ad;
    const int16_t *abs16;
    float *y;
    const float *bias, *residual;
    int32_t M, N, K, nb;
    uint32_t type;
    // grouped (per-expert) mode, MUL_MAT_ID: token tile blockIdx.y belongs to expert tile_expert[y]; its
    // rows are the gathered (token, slot) pairs row_src[y * 128 + r] (-1 = padding), whose activations
    // are those of row row_src / act_div and whose result goes to row row_src of y.  Null: dense mode.
    const int32_t *row_src, *tile_expert, *n_tiles;
    int32_t act_div;
    int64_t expert_stride; // bytes between consecutive expert matrices
};

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

// canonical K-major, no swizzle: 16-byte chunk kc of row r
__device__ __forceinline__ uint32_t op_off_a(int r, int kc) { return kc * LBO_A + (r >> 3) * SBO + (r & 7) * 16; }
// weight operand: rows 0 .. TN-1 of the tile are the hi plane, rows TN .. 2 TN-1 the lo plane
__device__ __forceinline__ uint32_t op_off_b(int r, int kc) { return kc * LBO_B + (r >> 3) * SBO + (r & 7) * 16; }
__device__ __forceinline__ uint32_t op_off_bmin(int r, int kc) { return kc * LBO_BMIN + (r >> 3) * SBO + (r & 7) * 16; }

__device__ __forceinline__ uint64_t make_desc(uint32_t saddr, uint32_t lbo) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFF) >> 4);
    d |= (uint64_t)(lbo >> 4) << 16;
    d |= (uint64_t)(SBO >> 4) << 32;
    d |= (uint64_t)1 << 46; // descriptor version of this architecture
    return d;               // layout type 0: no swizzle
}

// kind::i8: D s32, A s8, B s8 or u8, both K-major, M = 128, N = 2 TN (both planes in one instruction)
__device__ __forceinline__ uint32_t idesc_i8(bool b_signed) {
    return (2u << 4) | (1u << 7) | ((b_signed ? 1u : 0u) << 10) | ((uint32_t)((2 * TN) >> 3) << 17) | ((uint32_t)(TM >> 4) << 24);
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

// Packed f32 pairs: sm_100 issues mul / fma on two floats per instruction (same IEEE results as the
// scalar forms), which halves the floating-point instructions of the epilogue.
__device__ __forceinline__ uint64_t pack2(float a, float b) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
    return r;
}
__device__ __forceinline__ uint64_t pack2u(uint32_t a, uint32_t b) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(a), "r"(b));
    return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float &a, float &b) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v));
}
__device__ __forceinline__ uint64_t mul2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}

// Four 4-bit codes (one per byte of nib4) times the sub-block scale, split into the planes
// hi = (sc*q) >> 8 and lo = (sc*q) & 255.  Two 16-bit lanes per multiply; the products' low and high
// bytes are then already byte-aligned, so one byte permute per plane puts them back in code order.
__device__ __forceinline__ void q4_planes(uint32_t nib4, uint32_t sc, uint32_t &hi, uint32_t &lo) {
    const uint32_t p02 = (nib4 & 0x000F000Fu) * sc;        // codes 0 and 2: bytes [lo0 hi0 lo2 hi2]
    const uint32_t p13 = ((nib4 >> 8) & 0x000F000Fu) * sc; // codes 1 and 3: bytes [lo1 hi1 lo3 hi3]
    lo = __byte_perm(p02, p13, 0x6240);
    hi = __byte_perm(p02, p13, 0x7351);
}

// ---- weights of one super-block -> the two int8 planes (and the f16 min operand, the f32 block scales) ----
// Q4_K, one task per (row r of the tile, 16-byte chunk c of the block's quants): hdr = the block's first 16
// bytes, w = chunk c.  Chunk c gives K chunks 4g+h (low nibbles, sub-block 2g) and 4g+2+h (high, 2g+1).
__device__ __forceinline__ void unpack_q4_task(const uint4 &hdr, const uint4 &w, int r, int c, uint8_t *bhi, float *dw_s,
                                               float *dmin_s, uint8_t *bmin) {
    const int g = c >> 1, h = c & 1;
    const uint32_t sc_lo = hdr.y & 0x3F3F3F3Fu, sc_hi = (hdr.w & 0x0F0F0F0Fu) | ((hdr.y >> 2) & 0x30303030u);
    const uint32_t scw = g < 2 ? sc_lo : sc_hi;
    const uint32_t sc0 = (scw >> (8 * ((2 * g) & 3))) & 0xFF, sc1 = (scw >> (8 * ((2 * g + 1) & 3))) & 0xFF;
    if (c == 0) {
        const uint32_t m_lo = hdr.z & 0x3F3F3F3Fu, m_hi = ((hdr.w >> 4) & 0x0F0F0F0Fu) | ((hdr.z >> 2) & 0x30303030u);
        const float2 dd = __half22float2(*reinterpret_cast<const __half2 *>(&hdr.x));
        dw_s[r] = dd.x;
        dmin_s[r] = -dd.y; // kept negated: the epilogue subtracts the min term with one fused multiply-add
        __half mh[16]; // m_j against both sums of 16 of sub-block j
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const uint32_t mw = j < 4 ? m_lo : m_hi;
            const __half v = __int2half_rn((int)((mw >> (8 * (j & 3))) & 0xFF));
            mh[2 * j] = v;
            mh[2 * j + 1] = v;
        }
        *reinterpret_cast<uint4 *>(bmin + op_off_bmin(r, 0)) = *reinterpret_cast<uint4 *>(&mh[0]);
        *reinterpret_cast<uint4 *>(bmin + op_off_bmin(r, 1)) = *reinterpret_cast<uint4 *>(&mh[8]);
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
    const int kc_l = 4 * g + h, kc_h = 4 * g + 2 + h;
    *reinterpret_cast<uint4 *>(bhi + op_off_b(r, kc_l)) = hi_l;
    *reinterpret_cast<uint4 *>(bhi + op_off_b(TN + r, kc_l)) = lo_l;
    *reinterpret_cast<uint4 *>(bhi + op_off_b(r, kc_h)) = hi_h;
    *reinterpret_cast<uint4 *>(bhi + op_off_b(TN + r, kc_h)) = lo_h;
}

// Q6_K, one task per (row r, qh chunk j): qh4 = the chunk of 2-bit highs, qa4 / qb4 its two chunks of low
// nibbles, sc4 = the four int8 scales of its scale groups, dwv = the block's f32 scale.  4 scale groups of 16
// elements, w' = sc * (q - 32) split as hi * 64 + lo with lo in 0..63 and hi in -64..63 (both planes signed).
__device__ __forceinline__ void unpack_q6_task(const uint4 &qh4, const uint4 &qa4, const uint4 &qb4, uint32_t sc4, float dwv,
                                               int r, int j, uint8_t *bhi, float *dw_s, float *dmin_s) {
    const int hh = j >> 1, c1 = j & 1;
    const uint32_t hw[4] = {qh4.x, qh4.y, qh4.z, qh4.w};
    const uint32_t aw[4] = {qa4.x, qa4.y, qa4.z, qa4.w};
    const uint32_t bw[4] = {qb4.x, qb4.y, qb4.z, qb4.w};
    if (j == 0) {
        dw_s[r] = dwv;
        dmin_s[r] = 0.f;
    }
#pragma unroll
    for (int q = 0; q < 4; q++) { // bit pair q of the qh bytes: elements 128hh + 32q + 16c1 + i
        const int scq = (int)(int8_t)((sc4 >> (8 * q)) & 0xFF);
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
                const int wv = scq * ((int)((code >> (8 * k)) & 0xFF) - 32);
                hi |= (uint32_t)((wv >> 6) & 0xFF) << (8 * k);
                lo |= (uint32_t)(wv & 63) << (8 * k);
            }
            hi4[wd] = hi;
            lo4[wd] = lo;
        }
        const int kc = 8 * hh + 2 * q + c1;
        *reinterpret_cast<uint4 *>(bhi + op_off_b(r, kc)) = make_uint4(hi4[0], hi4[1], hi4[2], hi4[3]);
        *reinterpret_cast<uint4 *>(bhi + op_off_b(TN + r, kc)) = make_uint4(lo4[0], lo4[1], lo4[2], lo4[3]);
    }
}

// Q8 codes [M][K] -> [M/128][K/16][128 rows][16 bytes]: one super-block of a 128-token tile becomes a
// contiguous 32 KB run already in the operand layout; rows past M are zero.
__global__ void __launch_bounds__(256) retile_act_kernel(const int8_t *q, uint4 *out, int M, int K,
                                                         int64_t n_piece) {
    KQ_PDL_ENTER();
    const int kcs = K / 16;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_piece; i += (int64_t)gridDim.x * blockDim.x) {
        const int r = (int)(i % TM);
        const int64_t t = i / TM;
        const int kc = (int)(t % kcs), mt = (int)(t / kcs);
        const int m = mt * TM + r;
        out[i] = m < M ? *reinterpret_cast<const uint4 *>(q + (int64_t)m * K + kc * 16) : make_uint4(0, 0, 0, 0);
    }
}

// The same for gathered rows: tile t, row r takes the codes of activation row row_src[t * 128 + r] / act_div
// (zeros where row_src is negative: padding behind an expert's last pair).  Tiles past *n_tiles are skipped.
__global__ void __launch_bounds__(256) retile_gather_kernel(const int8_t *q, uint4 *out,
                                                            const int32_t *row_src, const int32_t *n_tiles,
                                                            int act_div, int K, int64_t n_piece) {
    KQ_PDL_ENTER();
    const int kcs = K / 16;
    const int64_t live = (int64_t)(*n_tiles) * kcs * TM;
    if (live < n_piece) n_piece = live;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_piece; i += (int64_t)gridDim.x * blockDim.x) {
        const int r = (int)(i % TM);
        const int64_t t = i / TM;
        const int kc = (int)(t % kcs), mt = (int)(t / kcs);
        const int src = row_src[mt * TM + r];
        out[i] = src >= 0 ? *reinterpret_cast<const uint4 *>(q + (int64_t)(src / act_div) * K + kc * 16) : make_uint4(0, 0, 0, 0);
    }
}

__global__ void __launch_bounds__(NTHREADS, 2) gemm_tc_kernel(const GemmParams p, const __grid_constant__ CUtensorMap wmap) {
    KQ_PDL_ENTER();
    extern __shared__ __align__(1024) uint8_t smem[];
    __shared__ uint64_t mbar;      // the MMAs of a super-block have completed
    __shared__ uint64_t full_raw[2]; // packed weight blocks of a stage have landed
    __shared__ uint64_t full_a;      // the token slab has landed
    __shared__ uint32_t s_tmem;
    __shared__ int s_abort;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int m0 = blockIdx.y * TM, n0 = blockIdx.x * TN;
    const bool grouped = p.row_src != nullptr;
    if (grouped && (int)blockIdx.y >= *p.n_tiles) return; // the grid is sized for the worst case
    const int expert = grouped ? p.tile_expert[blockIdx.y] : 0;
    float *da_s = reinterpret_cast<float *>(smem + SMEM_SCAL);
    float *dw_s = da_s + TM, *dmin_s = dw_s + TN;
    const uint32_t mbar_a = smem_u32(&mbar);

    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem)),
                     "r"(TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    if (tid == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(mbar_a), "r"(1));
        asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(&full_raw[0])), "r"(1));
        asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(&full_raw[1])), "r"(1));
        asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(&full_a)), "r"(1));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        s_abort = 0;
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = s_tmem;
    // this thread's TMEM window: lanes of its warp quarter, columns of its half of the tile
    const int row = (warp & 3) * 32 + lane; // token row of the tile = TMEM lane
    const int chalf = warp >> 2;            // columns [NCOL*chalf, NCOL*chalf + NCOL)
    const uint32_t tlane = tmem + ((uint32_t)((warp & 3) * 32) << 16);

    uint64_t yacc[NCOL / 2]; // running f32 result of this thread's token row x its weight columns, as f32 pairs
#pragma unroll
    for (int i = 0; i < NCOL / 2; i++) yacc[i] = 0ull;

    const uint32_t a_base = smem_u32(smem + SMEM_A), bhi_base = smem_u32(smem + SMEM_BHI),
                   amin_base = smem_u32(smem + SMEM_AMIN),
                   bmin_base = smem_u32(smem + SMEM_BMIN);
    const bool q4 = p.type == B200_TYPE_Q4_K;
    const int64_t wstride = kq_device_row_bytes(p.type, p.K);
    uint32_t phase = 0;
    bool failed = false;

    // ---- software pipeline.  Two CTAs share an SM, so while this one unpacks or drains TMEM the
    // tensor core and the copy engine work for the other one.  Inside a CTA the packed weights are
    // requested one super-block ahead (two raw buffers); the token slab is single-buffered and
    // requested as soon as the MMAs that read it have completed.
    constexpr int WT4 = TN * 8 / NTHREADS, WT6 = TN * 4 / NTHREADS; // weight tasks per thread
    uint4 p6_h[WT6], p6_a[WT6], p6_b[WT6]; // Q6_K: qh chunk and its two ql chunks per task
    uint32_t p6_sc[WT6];
    float p6_d[WT6];
    float pf_da = 0.f;
    int4 pf_bs0 = make_int4(0, 0, 0, 0), pf_bs1 = make_int4(0, 0, 0, 0);

    // activation row of this thread's token duty (threads 0 .. TM-1), -1 past the end / for padding
    int src_act = -1;
    if (tid < TM) {
        if (grouped) {
            const int sr = p.row_src[m0 + tid];
            src_act = sr >= 0 ? sr / p.act_div : -1;
        } else if (m0 + tid < p.M) {
            src_act = m0 + tid;
        }
    }
    const uint8_t *const Wb = p.W + (int64_t)expert * p.expert_stride;
    auto issue_raw = [&](int b) { // one tiled TMA box: 64 rows x 144 bytes; rows past N arrive as zeros
        if (q4 && warp == 1 && lane == 0) {
            const uint32_t bar = smem_u32(&full_raw[b & 1]);
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(RAW_BYTES) : "memory");
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
                             smem_u32(smem + SMEM_RAW + (b & 1) * RAW_BYTES)),
                         "l"(&wmap), "r"(b * KQ_Q4K_BYTES), "r"(n0 + expert * p.N), "r"(bar)
                         : "memory");
        }
    };
    auto issue_a = [&](int b) { // the re-tiled activations of a super-block are one contiguous 32 KB run
        if (warp == 1 && lane == 0) {
            const uint32_t bar = smem_u32(&full_a);
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(A_BYTES) : "memory");
            const int8_t *src = p.aq + ((int64_t)blockIdx.y * (p.K / 16) + (int64_t)b * 16) * (TM * 16);
            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                             a_base),
                         "l"(src), "r"(A_BYTES), "r"(bar)
                         : "memory");
        }
    };
    auto prefetch = [&](int b) { // per-token scalars and (Q6_K) the weight pieces, into registers
        if (tid < TM) {
            const bool in = src_act >= 0;
            pf_da = in ? p.ad[(int64_t)src_act * p.nb + b] : 0.f;
            if (q4) {
                const int4 *bsp = reinterpret_cast<const int4 *>(p.abs16 + ((int64_t)src_act * p.nb + b) * 16);
                pf_bs0 = in ? bsp[0] : make_int4(0, 0, 0, 0);
                pf_bs1 = in ? bsp[1] : make_int4(0, 0, 0, 0);
            }
        }
        if (!q4) {
            const KqQ6Addr qa = kq_q6_addr(p.nb, b);
#pragma unroll
            for (int t = 0; t < WT6; t++) {
                const int wt = warp + t * (NTHREADS / 32), r = 8 * wt + (lane & 7), j = lane >> 3;
                const int hh = j >> 1, c1 = j & 1;
                p6_h[t] = p6_a[t] = p6_b[t] = make_uint4(0, 0, 0, 0);
                p6_sc[t] = 0;
                p6_d[t] = 0.f;
                if (n0 + r < p.N) {
                    const uint8_t *rowp = Wb + (int64_t)(n0 + r) * wstride;
                    p6_h[t] = __ldg(reinterpret_cast<const uint4 *>(rowp + qa.qh + j * qa.cs));
                    p6_a[t] = __ldg(reinterpret_cast<const uint4 *>(rowp + qa.ql + (4 * hh + c1) * qa.cs));
                    p6_b[t] = __ldg(reinterpret_cast<const uint4 *>(rowp + qa.ql + (4 * hh + c1 + 2) * qa.cs));
                    const uint8_t *scp = rowp + qa.sc + 8 * hh + c1; // scale groups 8hh + 2q + c1
                    p6_sc[t] = (uint32_t)scp[0] | ((uint32_t)scp[2] << 8) | ((uint32_t)scp[4] << 16) | ((uint32_t)scp[6] << 24);
                    p6_d[t] = kq_h2f(*reinterpret_cast<const uint16_t *>(rowp + qa.d));
                }
            }
        }
    };

    issue_raw(0);
    issue_a(0);
    prefetch(0);
    int last_raw = 0, last_a = 0; // newest super-blocks handed to the copy engine
    for (int b = 0; b < p.nb && !failed; b++) {
        PROF_T(t_0);
        if (q4 && !kq_mbar_wait(smem_u32(&full_raw[b & 1]), (uint32_t)((b >> 1) & 1), 5 * KQ_WAIT_LIMIT_NS)) {
            s_abort = 1;
            atomicExch(&g_gemm_error, 2);
        }
        // ---- unpack the weights of super-block b into the two int8 planes --------------------------
        if (tid < TM) {
            const int r = tid;
            da_s[r] = pf_da;
            if (q4) { // sums of 16 as f16 (|sum| <= 2032: exact)
                const int16_t *s16a = reinterpret_cast<const int16_t *>(&pf_bs0);
                const int16_t *s16b = reinterpret_cast<const int16_t *>(&pf_bs1);
                __half h[16];
#pragma unroll
                for (int k = 0; k < 8; k++) {
                    h[k] = __int2half_rn((int)s16a[k]);
                    h[8 + k] = __int2half_rn((int)s16b[k]);
                }
                *reinterpret_cast<uint4 *>(smem + SMEM_AMIN + op_off_a(r, 0)) = *reinterpret_cast<uint4 *>(&h[0]);
                *reinterpret_cast<uint4 *>(smem + SMEM_AMIN + op_off_a(r, 1)) = *reinterpret_cast<uint4 *>(&h[8]);
            }
        }
        if (q4) {
            // chunk c of a block gives K chunks 4g+h (low nibbles, sub-block 2g) and 4g+2+h (high, 2g+1)
#pragma unroll
            for (int t = 0; t < WT4; t++) {
                const int wt = warp + t * (NTHREADS / 32), r = 8 * (wt >> 1) + (lane & 7), c = 4 * (wt & 1) + (lane >> 3);
                const uint8_t *blk = smem + SMEM_RAW + (b & 1) * RAW_BYTES + r * KQ_Q4K_BYTES;
                const uint4 hdr = *reinterpret_cast<const uint4 *>(blk), w = *reinterpret_cast<const uint4 *>(blk + 16 + 16 * c);
                unpack_q4_task(hdr, w, r, c, smem + SMEM_BHI, dw_s, dmin_s, smem + SMEM_BMIN);
            }
        } else {
            // Q6_K: one task per (row, qh chunk j): 4 scale groups of 16 elements, w' = sc * (q - 32)
            // split as hi * 64 + lo with lo in 0..63 and hi in -64..63 (both planes signed)
#pragma unroll
            for (int t = 0; t < WT6; t++) {
                const int wt = warp + t * (NTHREADS / 32), r = 8 * wt + (lane & 7), j = lane >> 3;
                unpack_q6_task(p6_h[t], p6_a[t], p6_b[t], p6_sc[t], p6_d[t], r, j, smem + SMEM_BHI, dw_s, dmin_s);
            }
        }
        PROF_T(t_1);
        // shared-memory writes of the generic proxy must be visible to the tensor core's async proxy
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();
        PROF_T(t_2);
        // ---- MMAs ------------------------------------------------------------------------------
        if (warp == 0) {
          // the whole warp stays here while its first lane issues, so that no lane of the issuing
          // warp sits in a blocking barrier wait before the MMAs have been handed to the tensor core
          if (lane == 0) {
            // the token slab of this super-block must have landed; on a time-out nothing is issued and
            // the commit below completes at once, so that the other threads find the abort flag
            const bool a_ok = kq_mbar_wait(smem_u32(&full_a), (uint32_t)(b & 1), 5 * KQ_WAIT_LIMIT_NS);
            if (!a_ok) {
                s_abort = 1;
                atomicExch(&g_gemm_error, 3);
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            if (a_ok && !s_abort) {
                // Q4_K planes are unsigned (hi 0..3, lo 0..255), Q6_K planes signed (hi -64..63, lo 0..63)
                const uint32_t id_main = idesc_i8(!q4);
#pragma unroll
                for (int s = 0; s < 8; s++) // K = 32 per instruction: chunks 2s, 2s+1; N = hi rows | lo rows
                    mma_i8(tmem + COL_HI, make_desc(a_base + 2 * s * LBO_A, LBO_A), make_desc(bhi_base + 2 * s * LBO_B, LBO_B),
                           id_main, s > 0);
                if (q4) mma_f16(tmem + COL_MIN, make_desc(amin_base, LBO_A), make_desc(bmin_base, LBO_BMIN), idesc_f16(), 0);
            }
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(mbar_a)
                         : "memory");
          }
          __syncwarp();
        }
        PROF_T(t_3);
        if (b + 1 < p.nb) { // weights and scalars of the next super-block fly during MMA + epilogue
            issue_raw(b + 1);
            prefetch(b + 1);
            last_raw = b + 1;
        }
        PROF_T(t_4);
        { // bounded wait for the MMAs of this super-block
            const bool ok = s_abort ? false : kq_mbar_wait(mbar_a, phase, 5 * KQ_WAIT_LIMIT_NS);
            if (!ok) {
                s_abort = 1;
                atomicExch(&g_gemm_error, 1);
            }
            phase ^= 1;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        PROF_T(t_5);
        if (s_abort) failed = true;
        if (!failed && b + 1 < p.nb) { // the slab is free again
            issue_a(b + 1);
            last_a = b + 1;
        }
        // ---- epilogue of the super-block: y += d_a * (d_w * (R*hi + lo) - dmin * min) ------------
        if (!failed) {
            const float da = da_s[row];
            const uint64_t da2 = pack2(da, da);
            const int R = q4 ? 256 : 64;
#pragma unroll
            for (int c = 0; c < NCOL; c += 16) {
                const uint32_t col = chalf * NCOL + c;
                uint32_t hi[16], lo[16], mn[16];
                TMEM_LD16(tlane + COL_HI + col, hi);
                TMEM_LD16(tlane + COL_LO + col, lo);
                if (q4) TMEM_LD16(tlane + COL_MIN + col, mn);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                for (int i4 = 0; i4 < 16; i4 += 4) {
                    // t = dw * main - dmin * min (one rounding each for the product and the fused subtract),
                    // y = fma(da, t, y): the arithmetic of the scalar form, two columns per instruction
                    const ulonglong2 dw4 = *reinterpret_cast<const ulonglong2 *>(&dw_s[col + i4]);
                    const ulonglong2 dm4 = *reinterpret_cast<const ulonglong2 *>(&dmin_s[col + i4]);
                    const uint64_t dwp[2] = {dw4.x, dw4.y}, dmp[2] = {dm4.x, dm4.y}; // -dmin
#pragma unroll
                    for (int k = 0; k < 2; k++) {
                        const int i = i4 + 2 * k;
                        const float f0 = (float)(R * (int)hi[i] + (int)lo[i]), f1 = (float)(R * (int)hi[i + 1] + (int)lo[i + 1]);
                        uint64_t t = mul2(dwp[k], pack2(f0, f1));
                        if (q4) t = fma2(dmp[k], pack2u(mn[i], mn[i + 1]), t);
                        yacc[(c + i) / 2] = fma2(da2, t, yacc[(c + i) / 2]);
                    }
                }
            }
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads(); // accumulators and the staging buffers are free again
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        PROF_T(t_6);
        PROF_ADD(0, t_0, t_1); PROF_ADD(1, t_1, t_2); PROF_ADD(2, t_2, t_3); PROF_ADD(3, t_3, t_4);
        PROF_ADD(4, t_4, t_5); PROF_ADD(5, t_5, t_6);
    }

    if (failed) { // never leave with bulk copies still writing this CTA's shared memory
        if (q4) {
            kq_mbar_wait(smem_u32(&full_raw[last_raw & 1]), (uint32_t)((last_raw >> 1) & 1), 5 * KQ_WAIT_LIMIT_NS);
            if (last_raw > 0)
                kq_mbar_wait(smem_u32(&full_raw[(last_raw - 1) & 1]), (uint32_t)(((last_raw - 1) >> 1) & 1),
                             5 * KQ_WAIT_LIMIT_NS);
        }
        kq_mbar_wait(smem_u32(&full_a), (uint32_t)(last_a & 1), 5 * KQ_WAIT_LIMIT_NS);
    }
    // ---- write the tile -------------------------------------------------------------------------
    const int out_row = grouped ? p.row_src[m0 + row] : (m0 + row < p.M ? m0 + row : -1);
    if (!failed && out_row >= 0) {
#pragma unroll
        for (int c = 0; c < NCOL; c++) {
            const int col = chalf * NCOL + c;
            if (n0 + col < p.N) {
                const int64_t o = (int64_t)out_row * p.N + n0 + col;
                float v, v_odd;
                unpack2(yacc[c / 2], v, v_odd);
                if (c & 1) v = v_odd;
                if (p.bias) v += p.bias[n0 + col];
                if (p.residual) v += p.residual[o];
                p.y[o] = v;
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
}

// ====================================================================================================
// Pre-unpacked planes: the form for two or more 128-token tiles.
// gemm_tc_kernel unpacks a weight tile once per token tile.  With several token tiles the unpacked operand
// is built once instead -- unpack_planes_kernel writes, for every (64-row tile, super-block), the image the
// tensor core reads: [hi | lo planes 32 KB | f16 min operand 2 KB | d_w 64 f32 | d_min 64 f32] -- and
// gemm_planes_kernel brings an image in with one bulk copy per super-block and does no CUDA-core work before
// its MMAs.  The token side is prepared alike (retile_act_img_kernel: [codes 32 KB | f16 sums-of-16 operand
// 4 KB] per token tile and super-block).  Token tiles of one weight tile are neighbours in the grid, so an
// image is fetched from HBM once and served from L2 to the other token tiles.  The arithmetic, operand
// layouts, MMAs and epilogue are those of gemm_tc_kernel: results are bit-identical.
// ====================================================================================================
constexpr int IMG_BMIN = 2 * B_BYTES;               // offsets inside a weight image
constexpr int IMG_DW = IMG_BMIN + BMIN_BYTES;
constexpr int IMG_DMIN = IMG_DW + TN * 4;
constexpr int IMG_BYTES = IMG_DMIN + TN * 4;        // 35328
constexpr int AIMG_AMIN = A_BYTES;                  // offset of the f16 operand inside a token image
constexpr int AIMG_BYTES = A_BYTES + AMIN_BYTES;    // 36864
constexpr int PL_SMEM_A = 0, PL_SMEM_B = AIMG_BYTES, PL_SMEM_TOTAL = AIMG_BYTES + 2 * IMG_BYTES + 64;
static_assert(IMG_BYTES % 16 == 0 && AIMG_BYTES % 1024 == 0, "bulk copies move multiples of 16 bytes to aligned places");
static_assert(PL_SMEM_TOTAL <= 112 * 1024, "two CTAs per SM");

// grid (super-blocks, weight tiles); one image per CTA, staged in shared memory and written with one bulk store
__global__ void __launch_bounds__(NTHREADS) unpack_planes_kernel(uint32_t type, const uint8_t *W, int N, int nb, uint8_t *img) {
    KQ_PDL_ENTER();
    extern __shared__ __align__(1024) uint8_t smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int b = blockIdx.x, nt = blockIdx.y, n0 = nt * TN;
    float *dw_s = reinterpret_cast<float *>(smem + IMG_DW), *dmin_s = reinterpret_cast<float *>(smem + IMG_DMIN);
    const int64_t wstride = kq_device_row_bytes(type, (int64_t)nb * 256);
    if (type == B200_TYPE_Q4_K) {
        constexpr int WT4 = TN * 8 / NTHREADS;
#pragma unroll
        for (int t = 0; t < WT4; t++) {
            const int wt = warp + t * (NTHREADS / 32), r = 8 * (wt >> 1) + (lane & 7), c = 4 * (wt & 1) + (lane >> 3);
            uint4 hdr = make_uint4(0, 0, 0, 0), w = make_uint4(0, 0, 0, 0); // rows past N: zero blocks
            if (n0 + r < N) {
                const uint8_t *blk = W + (int64_t)(n0 + r) * wstride + (int64_t)b * KQ_Q4K_BYTES;
                hdr = __ldg(reinterpret_cast<const uint4 *>(blk));
                w = __ldg(reinterpret_cast<const uint4 *>(blk + 16 + 16 * c));
            }
            unpack_q4_task(hdr, w, r, c, smem, dw_s, dmin_s, smem + IMG_BMIN);
        }
    } else {
        constexpr int WT6 = TN * 4 / NTHREADS;
        const KqQ6Addr qa = kq_q6_addr(nb, b);
        for (int i = tid; i < BMIN_BYTES / 16; i += NTHREADS) reinterpret_cast<uint4 *>(smem + IMG_BMIN)[i] = make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int t = 0; t < WT6; t++) {
            const int wt = warp + t * (NTHREADS / 32), r = 8 * wt + (lane & 7), j = lane >> 3;
            const int hh = j >> 1, c1 = j & 1;
            uint4 h4 = make_uint4(0, 0, 0, 0), a4 = h4, b4 = h4;
            uint32_t sc = 0;
            float dv = 0.f;
            if (n0 + r < N) {
                const uint8_t *rowp = W + (int64_t)(n0 + r) * wstride;
                h4 = __ldg(reinterpret_cast<const uint4 *>(rowp + qa.qh + j * qa.cs));
                a4 = __ldg(reinterpret_cast<const uint4 *>(rowp + qa.ql + (4 * hh + c1) * qa.cs));
                b4 = __ldg(reinterpret_cast<const uint4 *>(rowp + qa.ql + (4 * hh + c1 + 2) * qa.cs));
                const uint8_t *scp = rowp + qa.sc + 8 * hh + c1; // scale groups 8hh + 2q + c1
                sc = (uint32_t)scp[0] | ((uint32_t)scp[2] << 8) | ((uint32_t)scp[4] << 16) | ((uint32_t)scp[6] << 24);
                dv = kq_h2f(*reinterpret_cast<const uint16_t *>(rowp + qa.d));
            }
            unpack_q6_task(h4, a4, b4, sc, dv, r, j, smem, dw_s, dmin_s);
        }
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncthreads();
    if (tid == 0) {
        uint8_t *dst = img + ((int64_t)nt * nb + b) * IMG_BYTES;
        asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(smem_u32(smem)), "r"(IMG_BYTES)
                     : "memory");
        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); // the store has left shared memory and is complete
    }
}

// Q8 codes and sums of 16 -> token images: (token tile mt, super-block b) at (mt * nb + b) * AIMG_BYTES.
// One thread per 16-byte piece: pieces 0..15 of a row are its code chunks, 16 and 17 its sums as f16.
__global__ void __launch_bounds__(256) retile_act_img_kernel(const int8_t *q, const int16_t *bs, uint8_t *out, int M, int K,
                                                             int64_t n_piece) {
    KQ_PDL_ENTER();
    const int nb = K / 256;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_piece; i += (int64_t)gridDim.x * blockDim.x) {
        const int r = (int)(i % TM);
        int64_t t = i / TM;
        const int j = (int)(t % 18);
        t /= 18;
        const int b = (int)(t % nb), mt = (int)(t / nb);
        const int m = mt * TM + r;
        uint8_t *rec = out + ((int64_t)mt * nb + b) * AIMG_BYTES;
        if (j < 16) {
            const uint4 v = m < M ? *reinterpret_cast<const uint4 *>(q + (int64_t)m * K + b * 256 + j * 16) : make_uint4(0, 0, 0, 0);
            *reinterpret_cast<uint4 *>(rec + op_off_a(r, j)) = v;
        } else { // sums of 16 as f16 (|sum| <= 2032: exact)
            uint4 v = make_uint4(0, 0, 0, 0);
            if (m < M) {
                const int4 s8 = *reinterpret_cast<const int4 *>(bs + ((int64_t)m * nb + b) * 16 + 8 * (j - 16));
                const int16_t *s16 = reinterpret_cast<const int16_t *>(&s8);
                __half h[8];
#pragma unroll
                for (int k = 0; k < 8; k++) h[k] = __int2half_rn((int)s16[k]);
                v = *reinterpret_cast<uint4 *>(&h[0]);
            }
            *reinterpret_cast<uint4 *>(rec + AIMG_AMIN + op_off_a(r, j - 16)) = v;
        }
    }
}

struct PlanesParams {
    const uint8_t *bimg; // weight images, [weight tile][super-block]
    const uint8_t *aimg; // token images, [token tile][super-block]
    const float *ad;     // Q8 block scales [M][nb]
    float *y;
    const float *bias, *residual;
    int32_t M, N, nb;
    uint32_t type;
};

// grid (token tiles, weight tiles): the token tiles of one weight tile run side by side
__global__ void __launch_bounds__(NTHREADS, 2) gemm_planes_kernel(const PlanesParams p) {
    KQ_PDL_ENTER();
    extern __shared__ __align__(1024) uint8_t smem[];
    __shared__ uint64_t mbar;      // the MMAs of a super-block have completed
    __shared__ uint64_t full_b[2]; // a weight image has landed
    __shared__ uint64_t full_a;    // the token image has landed
    __shared__ uint32_t s_tmem;
    __shared__ int s_abort;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int mt = blockIdx.x, nt = blockIdx.y, m0 = mt * TM, n0 = nt * TN;
    const uint32_t mbar_a = smem_u32(&mbar);
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem)), "r"(TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    if (tid == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(mbar_a), "r"(1));
        asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(&full_b[0])), "r"(1));
        asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(&full_b[1])), "r"(1));
        asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(&full_a)), "r"(1));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        s_abort = 0;
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = s_tmem;
    const int row = (warp & 3) * 32 + lane; // token row of the tile = TMEM lane
    const int chalf = warp >> 2;            // columns [NCOL*chalf, NCOL*chalf + NCOL)
    const uint32_t tlane = tmem + ((uint32_t)((warp & 3) * 32) << 16);
    uint64_t yacc[NCOL / 2];
#pragma unroll
    for (int i = 0; i < NCOL / 2; i++) yacc[i] = 0ull;
    const bool q4 = p.type == B200_TYPE_Q4_K;
    const int nb = p.nb;
    const uint8_t *bsrc = p.bimg + (int64_t)nt * nb * IMG_BYTES, *asrc = p.aimg + (int64_t)mt * nb * AIMG_BYTES;
    const uint32_t a_base = smem_u32(smem + PL_SMEM_A), amin_base = a_base + AIMG_AMIN;
    auto issue_b = [&](int b) { // the whole weight image of super-block b: one contiguous run
        if (warp == 1 && lane == 0) {
            const uint32_t bar = smem_u32(&full_b[b & 1]);
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(IMG_BYTES) : "memory");
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                             smem_u32(smem + PL_SMEM_B + (b & 1) * IMG_BYTES)),
                         "l"(bsrc + (int64_t)b * IMG_BYTES), "r"(IMG_BYTES), "r"(bar)
                         : "memory");
        }
    };
    auto issue_a = [&](int b) {
        if (warp == 1 && lane == 0) {
            const uint32_t bar = smem_u32(&full_a);
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(AIMG_BYTES) : "memory");
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(a_base),
                         "l"(asrc + (int64_t)b * AIMG_BYTES), "r"(AIMG_BYTES), "r"(bar)
                         : "memory");
        }
    };
    const bool row_in = m0 + row < p.M;
    const float *ad_row = p.ad + (int64_t)(row_in ? m0 + row : 0) * nb;
    issue_b(0);
    issue_a(0);
    if (nb > 1) issue_b(1);
    float pf_da = row_in ? ad_row[0] : 0.f;
    int last_b = nb > 1 ? 1 : 0, last_a = 0; // newest images handed to the copy engine
    uint32_t phase = 0;
    bool failed = false;
    for (int b = 0; b < nb && !failed; b++) {
        const uint8_t *img = smem + PL_SMEM_B + (b & 1) * IMG_BYTES;
        if (warp == 0) {
            if (lane == 0) {
                bool ok = kq_mbar_wait(smem_u32(&full_a), (uint32_t)(b & 1), 5 * KQ_WAIT_LIMIT_NS);
                ok = ok && kq_mbar_wait(smem_u32(&full_b[b & 1]), (uint32_t)((b >> 1) & 1), 5 * KQ_WAIT_LIMIT_NS);
                if (!ok) {
                    s_abort = 1;
                    atomicExch(&g_gemm_error, 4);
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                if (ok && !s_abort) {
                    const uint32_t id_main = idesc_i8(!q4), bhi_base = smem_u32(img);
#pragma unroll
                    for (int s = 0; s < 8; s++) // K = 32 per instruction: chunks 2s, 2s+1; N = hi rows | lo rows
                        mma_i8(tmem + COL_HI, make_desc(a_base + 2 * s * LBO_A, LBO_A), make_desc(bhi_base + 2 * s * LBO_B, LBO_B),
                               id_main, s > 0);
                    if (q4) mma_f16(tmem + COL_MIN, make_desc(amin_base, LBO_A), make_desc(bhi_base + IMG_BMIN, LBO_BMIN), idesc_f16(), 0);
                }
                asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(mbar_a) : "memory");
            }
            __syncwarp();
        }
        const float da = pf_da;
        if (b + 1 < nb) pf_da = row_in ? ad_row[b + 1] : 0.f;
        {
            const bool ok = s_abort ? false : kq_mbar_wait(mbar_a, phase, 5 * KQ_WAIT_LIMIT_NS);
            if (!ok) {
                s_abort = 1;
                atomicExch(&g_gemm_error, 1);
            }
            phase ^= 1;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        // every thread observes the image's own barrier (complete by now) before it reads the block scales
        if (!s_abort && !kq_mbar_wait(smem_u32(&full_b[b & 1]), (uint32_t)((b >> 1) & 1), 5 * KQ_WAIT_LIMIT_NS)) s_abort = 1;
        if (s_abort) failed = true;
        if (!failed && b + 1 < nb) { // the token image has been read
            issue_a(b + 1);
            last_a = b + 1;
        }
        if (!failed) { // y += d_a * (d_w * (R*hi + lo) - dmin * min), as in gemm_tc_kernel
            const float *dw_s = reinterpret_cast<const float *>(img + IMG_DW), *dmin_s = reinterpret_cast<const float *>(img + IMG_DMIN);
            const uint64_t da2 = pack2(da, da);
            const int R = q4 ? 256 : 64;
#pragma unroll
            for (int c = 0; c < NCOL; c += 16) {
                const uint32_t col = chalf * NCOL + c;
                uint32_t hi[16], lo[16], mn[16];
                TMEM_LD16(tlane + COL_HI + col, hi);
                TMEM_LD16(tlane + COL_LO + col, lo);
                if (q4) TMEM_LD16(tlane + COL_MIN + col, mn);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                for (int i4 = 0; i4 < 16; i4 += 4) {
                    const ulonglong2 dw4 = *reinterpret_cast<const ulonglong2 *>(&dw_s[col + i4]);
                    const ulonglong2 dm4 = *reinterpret_cast<const ulonglong2 *>(&dmin_s[col + i4]);
                    const uint64_t dwp[2] = {dw4.x, dw4.y}, dmp[2] = {dm4.x, dm4.y}; // -dmin
#pragma unroll
                    for (int k = 0; k < 2; k++) {
                        const int i = i4 + 2 * k;
                        const float f0 = (float)(R * (int)hi[i] + (int)lo[i]), f1 = (float)(R * (int)hi[i + 1] + (int)lo[i + 1]);
                        uint64_t t = mul2(dwp[k], pack2(f0, f1));
                        if (q4) t = fma2(dmp[k], pack2u(mn[i], mn[i + 1]), t);
                        yacc[(c + i) / 2] = fma2(da2, t, yacc[(c + i) / 2]);
                    }
                }
            }
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads(); // the accumulators and this image's buffer are free again
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (!s_abort && b + 2 < nb) {
            issue_b(b + 2);
            last_b = b + 2;
        }
    }
    if (failed || s_abort) { // never leave with bulk copies still writing this CTA's shared memory
        kq_mbar_wait(smem_u32(&full_b[last_b & 1]), (uint32_t)((last_b >> 1) & 1), 5 * KQ_WAIT_LIMIT_NS);
        if (last_b > 0) kq_mbar_wait(smem_u32(&full_b[(last_b - 1) & 1]), (uint32_t)(((last_b - 1) >> 1) & 1), 5 * KQ_WAIT_LIMIT_NS);
        kq_mbar_wait(smem_u32(&full_a), (uint32_t)(last_a & 1), 5 * KQ_WAIT_LIMIT_NS);
        failed = true;
    }
    if (!failed && row_in) {
#pragma unroll
        for (int c = 0; c < NCOL; c++) {
            const int col = chalf * NCOL + c;
            if (n0 + col < p.N) {
                const int64_t o = (int64_t)(m0 + row) * p.N + n0 + col;
                float v, v_odd;
                unpack2(yacc[c / 2], v, v_odd);
                if (c & 1) v = v_odd;
                if (p.bias) v += p.bias[n0 + col];
                if (p.residual) v += p.residual[o];
                p.y[o] = v;
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
}

// ---- expert-major order of the (token, slot) pairs of a routed batch (MUL_MAT_ID with many tokens) ----
// A stable counting sort by expert: the pairs of expert e, in pair order, become the rows of that
// expert's token tiles; every expert starts on a tile boundary, the rows behind its last pair are
// padding (-1).  One CTA of 8 warps; warp w walks a contiguous range of the pairs 32 at a time, so the
// order inside an expert is the pair order whatever the timing.  Output: n_tiles, the expert of each
// tile, and for each tile row the pair it holds.
constexpr int SORT_WARPS = 8, SORT_MAX_E = 256;
__global__ void __launch_bounds__(SORT_WARPS * 32) moe_sort_kernel(const int32_t *ids, int n_pairs, int E,
                                                                   int32_t *n_tiles_out, int32_t *tile_expert, int32_t *row_src) {
    KQ_PDL_ENTER();
    __shared__ int cnt[SORT_WARPS][SORT_MAX_E]; // pass 1: pairs of expert e in warp w's range; then the range's offset inside the expert
    __shared__ int tile_start[SORT_MAX_E];
    __shared__ int s_tiles;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int i = threadIdx.x; i < SORT_WARPS * SORT_MAX_E; i += blockDim.x) (&cnt[0][0])[i] = 0;
    __syncthreads();
    const int chunk = ((n_pairs + SORT_WARPS - 1) / SORT_WARPS + 31) & ~31;
    const int begin = min(n_pairs, warp * chunk), end = min(n_pairs, begin + chunk);
    for (int i = begin; i < end; i += 32) {
        const int pr = i + lane;
        int e = pr < end ? ids[pr] : -1;
        if (e < 0 || e >= E) e = -1; // not an expert of this table: the pair is dropped
        const unsigned same = __match_any_sync(0xffffffffu, e);
        if (e >= 0 && lane == __ffs(same) - 1) cnt[warp][e] += __popc(same);
        __syncwarp();
    }
    __syncthreads();
    if ((int)threadIdx.x < E) {
        int run = 0;
        for (int w = 0; w < SORT_WARPS; w++) {
            const int c = cnt[w][threadIdx.x];
            cnt[w][threadIdx.x] = run;
            run += c;
        }
        tile_start[threadIdx.x] = run; // the expert's pair count, for the moment
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int t = 0;
        for (int e = 0; e < E; e++) {
            const int nt = (tile_start[e] + TM - 1) / TM;
            tile_start[e] = t;
            for (int k = 0; k < nt; k++) tile_expert[t + k] = e;
            t += nt;
        }
        s_tiles = t;
        *n_tiles_out = t;
    }
    __syncthreads();
    const int live = s_tiles * TM;
    for (int i = threadIdx.x; i < live; i += blockDim.x) row_src[i] = -1;
    __syncthreads();
    for (int i = begin; i < end; i += 32) {
        const int pr = i + lane;
        int e = pr < end ? ids[pr] : -1;
        if (e < 0 || e >= E) e = -1;
        const unsigned same = __match_any_sync(0xffffffffu, e);
        const int leader = __ffs(same) - 1;
        int base = 0;
        if (e >= 0 && lane == leader) base = cnt[warp][e];
        base = __shfl_sync(0xffffffffu, base, leader);
        if (e >= 0) row_src[tile_start[e] * TM + base + __popc(same & ((1u << lane) - 1u))] = pr;
        __syncwarp();
        if (e >= 0 && lane == leader) cnt[warp][e] = base + __popc(same);
        __syncwarp();
    }
}

} // namespace

#ifdef KQ_GEMM_PROF
extern "C" __attribute__((visibility("default"))) void kq_gemm_prof_fetch(long long *out) {
    cudaMemcpyFromSymbol(out, g_gemm_prof, sizeof(long long) * 8);
    long long z[8] = {0};
    cudaMemcpyToSymbol(g_gemm_prof, z, sizeof(z));
}
#endif
int kq_gemm_error_fetch() {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_gemm_error, sizeof(int)) != cudaSuccess) return -1;
    if (v) cudaMemcpyToSymbol(g_gemm_error, &zero, sizeof(int));
    return v;
}

namespace {
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// bytes of a Q4_K matrix as a 2-D tensor [N rows][row_bytes], box = one super-block column of 128 rows
b200_status make_weight_map(CUtensorMap *map, const uint8_t *W, int64_t N, int64_t row_bytes) {
    static EncodeTiledFn encode = nullptr;
    if (!encode) {
        void *fn = nullptr;
        cudaDriverEntryPointQueryResult qr = cudaDriverEntryPointSymbolNotFound;
        KQ_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qr));
        KQ_REQUIRE(fn && qr == cudaDriverEntryPointSuccess, "gemm: the driver does not export cuTensorMapEncodeTiled");
        encode = (EncodeTiledFn)fn;
    }
    const cuuint64_t dims[2] = {(cuuint64_t)row_bytes, (cuuint64_t)N};
    const cuuint64_t strides[1] = {(cuuint64_t)row_bytes};
    const cuuint32_t box[2] = {(cuuint32_t)KQ_Q4K_BYTES, (cuuint32_t)TN};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult rc = encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint8_t *>(W), dims, strides, box, estr,
                               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    KQ_REQUIRE(rc == CUDA_SUCCESS, "gemm: tensor map encode failed (%d)", (int)rc);
    return B200_OK;
}
} // namespace

// Generic tiled tensor map for other kernels (the type lives in <cuda.h>; callers pass 128 bytes).
// elem_bytes 1, 2 or 8; swizzle128 selects the 128-byte swizzle (inner box extent <= 128 bytes).
b200_status kq_tmap_encode(void *map128, int elem_bytes, int rank, const void *base, const uint64_t *dims,
                           const uint64_t *strides_bytes, const uint32_t *box, int swizzle128) {
    static EncodeTiledFn encode = nullptr;
    if (!encode) {
        void *fn = nullptr;
        cudaDriverEntryPointQueryResult qr = cudaDriverEntryPointSymbolNotFound;
        KQ_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qr));
        KQ_REQUIRE(fn && qr == cudaDriverEntryPointSuccess, "the driver does not export cuTensorMapEncodeTiled");
        encode = (EncodeTiledFn)fn;
    }
    cuuint64_t d[5], sb[4];
    cuuint32_t bx[5], es[5];
    for (int i = 0; i < rank; i++) {
        d[i] = dims[i];
        bx[i] = box[i];
        es[i] = 1;
        if (i + 1 < rank) sb[i] = strides_bytes[i];
    }
    const CUresult rc = encode((CUtensorMap *)map128, elem_bytes == 8 ? CU_TENSOR_MAP_DATA_TYPE_UINT64 : elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_UINT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8,
                               (cuuint32_t)rank, const_cast<void *>(base), d, sb, bx, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                               swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    KQ_REQUIRE(rc == CUDA_SUCCESS, "tensor map encode failed (%d)", (int)rc);
    return B200_OK;
}

// Per-device scratch for the re-tiled activations, grown on demand and kept; launches that share
// it are ordered by using one stream per device at a time, as the stage engine and the backend do.
// Host threads may call for different devices at the same time: the table and its growth are
// guarded, the launches themselves are not serialised.
static b200_status kq_gemm_scratch(int dev, size_t need, cudaStream_t st, uint4 **out) {
    static std::mutex scratch_mu;
    std::lock_guard<std::mutex> scratch_lock(scratch_mu);
    static uint4 *tiled[KQ_MAX_DEVICES];
    static size_t tiled_cap[KQ_MAX_DEVICES];
    static bool attr[KQ_MAX_DEVICES];
    if (need > tiled_cap[dev]) {
        cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
        KQ_CUDA(cudaStreamIsCapturing(st, &cs));
        KQ_REQUIRE(cs == cudaStreamCaptureStatusNone, "gemm: activation scratch cannot grow during stream capture");
        KQ_CUDA(cudaDeviceSynchronize());
        if (tiled[dev]) KQ_CUDA(cudaFree(tiled[dev]));
        tiled[dev] = nullptr;
        tiled_cap[dev] = 0;
        KQ_CUDA(cudaMalloc(&tiled[dev], need));
        tiled_cap[dev] = need;
    }
    if (!attr[dev]) {
        KQ_CUDA(cudaFuncSetAttribute(gemm_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_TOTAL));
        attr[dev] = true;
    }
    *out = tiled[dev];
    return B200_OK;
}

// scratch of the planes form: weight images and token images of one matmul, per device, grown on demand
static b200_status kq_gemm_planes_scratch(int dev, size_t need_b, size_t need_a, cudaStream_t st, uint8_t **bimg, uint8_t **aimg) {
    static std::mutex mu;
    std::lock_guard<std::mutex> lock(mu);
    static uint8_t *buf[KQ_MAX_DEVICES][2];
    static size_t cap[KQ_MAX_DEVICES][2];
    static bool attr[KQ_MAX_DEVICES];
    const size_t need[2] = {need_b, need_a};
    for (int i = 0; i < 2; i++) {
        if (need[i] <= cap[dev][i]) continue;
        cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
        KQ_CUDA(cudaStreamIsCapturing(st, &cs));
        KQ_REQUIRE(cs == cudaStreamCaptureStatusNone, "gemm: operand scratch cannot grow during stream capture");
        KQ_CUDA(cudaDeviceSynchronize());
        if (buf[dev][i]) KQ_CUDA(cudaFree(buf[dev][i]));
        buf[dev][i] = nullptr;
        cap[dev][i] = 0;
        if (cudaMalloc(&buf[dev][i], need[i]) != cudaSuccess) {
            cudaGetLastError();
            return B200_ERR_UNSUPPORTED; // no room for the images: the caller takes the form that needs none
        }
        cap[dev][i] = need[i];
    }
    if (!attr[dev]) {
        KQ_CUDA(cudaFuncSetAttribute(gemm_planes_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PL_SMEM_TOTAL));
        attr[dev] = true;
    }
    *bimg = buf[dev][0];
    *aimg = buf[dev][1];
    return B200_OK;
}

static int planes_min_m() {
    static int v = -1;
    if (v < 0) {
        const char *e = getenv("B200_GEMM_PLANES_MIN_M"); // 0 switches the form off
        v = e ? atoi(e) : 3 * TM; // measured: from three token tiles on the images pay for themselves
        if (v <= 0) v = 1 << 30;
    }
    return v;
}

// the form with pre-unpacked operands; B200_ERR_UNSUPPORTED (nothing launched) when it does not apply
static b200_status launch_gemm_planes(uint32_t type, const uint8_t *W, const int8_t *q, const float *d, const int16_t *bs, int64_t M,
                                      int64_t N, int64_t K, float *y, const float *bias, const float *residual, int dev,
                                      cudaStream_t st) {
    const int64_t m_tiles = kq_div_up(M, TM), n_tiles = kq_div_up(N, TN), nb = K / 256;
    if (M < planes_min_m() || n_tiles > 65535 || m_tiles > 0x7fffffff / 2) return B200_ERR_UNSUPPORTED;
    uint8_t *bimg = nullptr, *aimg = nullptr;
    const b200_status rs = kq_gemm_planes_scratch(dev, (size_t)n_tiles * nb * IMG_BYTES, (size_t)m_tiles * nb * AIMG_BYTES, st, &bimg, &aimg);
    if (rs != B200_OK) return rs;
    KQ_CUDA(kq_launch(unpack_planes_kernel, dim3((unsigned)nb, (unsigned)n_tiles), dim3(NTHREADS), (size_t)IMG_BYTES, st, type, W, (int)N,
                      (int)nb, bimg));
    KQ_COUNT_LAUNCH();
    const int64_t n_piece = m_tiles * nb * 18 * TM;
    KQ_CUDA(kq_launch(retile_act_img_kernel, dim3((unsigned)std::min<int64_t>(kq_div_up(n_piece, 256), 1 << 20)), dim3(256), 0, st, q, bs,
                      aimg, (int)M, (int)K, n_piece));
    KQ_COUNT_LAUNCH();
    PlanesParams p = {bimg, aimg, d, y, bias, residual, (int32_t)M, (int32_t)N, (int32_t)nb, type};
    KQ_CUDA(kq_launch(gemm_planes_kernel, dim3((unsigned)m_tiles, (unsigned)n_tiles), dim3(NTHREADS), (size_t)PL_SMEM_TOTAL, st, p));
    KQ_COUNT_LAUNCH();
    KQ_LAUNCH_CHECK();
    return B200_OK;
}

b200_status kq_launch_gemm_tc(uint32_t type, const uint8_t *W, const int8_t *q, const float *d, const int16_t *bs,
                              int64_t M, int64_t N, int64_t K, float *y, const float *bias, const float *residual,
                              cudaStream_t st) {
    KQ_REQUIRE(type == B200_TYPE_Q4_K || type == B200_TYPE_Q6_K, "gemm: weight type %u", type);
    KQ_REQUIRE(K % 256 == 0 && M > 0 && N > 0, "gemm: bad shape");
    KQ_REQUIRE(((uintptr_t)W & 15) == 0 && ((uintptr_t)q & 15) == 0, "gemm: operands must be 16-byte aligned");
    int dev = 0;
    KQ_CUDA(cudaGetDevice(&dev));
    KQ_REQUIRE(dev >= 0 && dev < KQ_MAX_DEVICES, "gemm: device %d out of range", dev);
    {
        const b200_status rp = launch_gemm_planes(type, W, q, d, bs, M, N, K, y, bias, residual, dev, st);
        if (rp != B200_ERR_UNSUPPORTED) return rp;
    }
    const int64_t m_tiles = kq_div_up(M, TM);
    const size_t need = (size_t)m_tiles * TM * K;
    uint4 *tiled_dev = nullptr;
    {
        const b200_status rc = kq_gemm_scratch(dev, need, st, &tiled_dev);
        if (rc != B200_OK) return rc;
    }
    const int64_t n_piece = (int64_t)need / 16;
    kq_launch(retile_act_kernel, dim3((unsigned)kq_div_up(n_piece, 256)), 256, 0, st, q, tiled_dev, (int)M, (int)K, n_piece);
    KQ_COUNT_LAUNCH();
    GemmParams p = {W, reinterpret_cast<const int8_t *>(tiled_dev), d, bs, y, bias, residual,
                    (int32_t)M, (int32_t)N, (int32_t)K, (int32_t)(K / 256), type, nullptr, nullptr, nullptr, 1, 0};
    // two CTAs per SM: each holds 256 of the 512 TMEM columns and under half of the shared memory
    const int smem = SMEM_TOTAL;
    static_assert(SMEM_TOTAL <= 112 * 1024, "two tiles must fit the shared memory of an SM");
    CUtensorMap wmap;
    memset(&wmap, 0, sizeof(wmap));
    if (type == B200_TYPE_Q4_K) {
        const b200_status rc = make_weight_map(&wmap, W, N, kq_device_row_bytes(type, K));
        if (rc != B200_OK) return rc;
    }
    dim3 grid((unsigned)kq_div_up(N, TN), (unsigned)kq_div_up(M, TM));
    kq_launch(gemm_tc_kernel, grid, NTHREADS, smem, st, p, wmap);
    KQ_COUNT_LAUNCH();
    KQ_LAUNCH_CHECK();
    return B200_OK;
}

// ---- MUL_MAT_ID over many tokens: pairs gathered per expert, one grouped launch of the tensor-core kernel ----
// Scratch of the sort, in int32 words: [0] number of live tiles, [1 .. 1 + max_tiles) expert per tile,
// [1 + max_tiles ..) pair per tile row; max_tiles = ceil(n_pairs / 128) + n_expert bounds sum_e ceil(c_e / 128).
static inline int64_t moe_max_tiles(int64_t n_pairs, int64_t E) { return kq_div_up(n_pairs, TM) + E; }

size_t kq_moe_sort_scratch_bytes(int64_t n_pairs, int64_t E) {
    const int64_t mt = moe_max_tiles(n_pairs, E);
    return (size_t)(1 + mt + mt * TM + 64) * sizeof(int32_t);
}

b200_status kq_moe_sort(const int32_t *ids, int64_t n_pairs, int64_t E, int32_t *scratch, size_t scratch_bytes, cudaStream_t st) {
    KQ_REQUIRE(ids && scratch && n_pairs >= 1 && E >= 1 && E <= SORT_MAX_E, "moe_sort: n_pairs >= 1, 1 <= experts <= %d", SORT_MAX_E);
    KQ_REQUIRE(scratch_bytes >= kq_moe_sort_scratch_bytes(n_pairs, E), "moe_sort: scratch of %zu bytes, %zu needed", scratch_bytes,
               kq_moe_sort_scratch_bytes(n_pairs, E));
    const int64_t mt = moe_max_tiles(n_pairs, E);
    kq_launch(moe_sort_kernel, 1, SORT_WARPS * 32, 0, st, ids, (int)n_pairs, (int)E, scratch, scratch + 1, scratch + 1 + mt);
    KQ_COUNT_LAUNCH();
    KQ_LAUNCH_CHECK();
    return B200_OK;
}

// y[pair][N] = W[expert of the pair] . x[pair / act_div]: q / d / bs are the quantised activations of the
// n_pairs / act_div source rows, sorted = the scratch kq_moe_sort left for these pairs.
b200_status kq_launch_gemm_grouped(uint32_t type, const uint8_t *W, int64_t expert_stride, const int8_t *q, const float *d,
                                   const int16_t *bs, int act_div, int64_t n_pairs, int64_t E, int64_t N, int64_t K, float *y,
                                   const int32_t *sorted, cudaStream_t st) {
    KQ_REQUIRE(type == B200_TYPE_Q4_K || type == B200_TYPE_Q6_K, "grouped gemm: weight type %u", type);
    KQ_REQUIRE(K % 256 == 0 && n_pairs > 0 && N > 0 && act_div >= 1, "grouped gemm: bad shape");
    if (N % TN != 0) return B200_ERR_UNSUPPORTED; // an expert's last row tile would run into the next expert's rows
    KQ_REQUIRE(((uintptr_t)W & 15) == 0 && ((uintptr_t)q & 15) == 0 && expert_stride % 16 == 0, "grouped gemm: operands must be 16-byte aligned");
    int dev = 0;
    KQ_CUDA(cudaGetDevice(&dev));
    KQ_REQUIRE(dev >= 0 && dev < KQ_MAX_DEVICES, "gemm: device %d out of range", dev);
    const int64_t mt = moe_max_tiles(n_pairs, E);
    uint4 *tiled_dev = nullptr;
    b200_status rc = kq_gemm_scratch(dev, (size_t)mt * TM * K, st, &tiled_dev);
    if (rc != B200_OK) return rc;
    const int64_t n_piece = mt * TM * K / 16;
    const int64_t blocks = kq_div_up(n_piece, 256);
    kq_launch(retile_gather_kernel, dim3((unsigned)(blocks > 65535 * 16 ? 65535 * 16 : blocks)), 256, 0, st, q, tiled_dev,
              sorted + 1 + mt, sorted, act_div, (int)K, n_piece);
    KQ_COUNT_LAUNCH();
    GemmParams p = {W, reinterpret_cast<const int8_t *>(tiled_dev), d, bs, y, nullptr, nullptr,
                    (int32_t)(mt * TM), (int32_t)N, (int32_t)K, (int32_t)(K / 256), type,
                    sorted + 1 + mt, sorted + 1, sorted, (int32_t)act_div, expert_stride};
    CUtensorMap wmap;
    memset(&wmap, 0, sizeof(wmap));
    if (type == B200_TYPE_Q4_K) {
        KQ_REQUIRE(expert_stride == kq_device_row_bytes(type, K) * N, "grouped gemm: expert matrices must be contiguous");
        rc = make_weight_map(&wmap, W, N * E, kq_device_row_bytes(type, K));
        if (rc != B200_OK) return rc;
    }
    dim3 grid((unsigned)(N / TN), (unsigned)mt);
    kq_launch(gemm_tc_kernel, grid, NTHREADS, SMEM_TOTAL, st, p, wmap);
    KQ_COUNT_LAUNCH();
    KQ_LAUNCH_CHECK();
    return B200_OK;
}
