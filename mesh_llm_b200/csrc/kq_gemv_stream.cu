// Decode GEMV for M <= 2 tokens, streaming form: y[m][n] = sum_k W[n][k] x[m][k], W in Q4_K or
// Q6_K blocks, x in Q8 blocks of 256.
//
// The weight stream is the whole cost of a decode step, so the kernel is built around two things.
//
// 1. Bytes in flight.  Every warp runs its own ring of shared-memory slots filled by the copy engine
//    -- one tiled copy per slot (cp.async.bulk.tensor: a box of the unit's rows x one K slice out of the
//    matrix seen as [rows][row bytes / 8]), or one cp.async.bulk per row where a box does not fit the
//    slot's alignment -- that complete on mbarriers, and
//    computes out of shared memory while later slices are on their way.  Registers hold only
//    accumulators, so the bytes in flight per SM are set by the ring depth, not by occupancy.
//    The first copies are issued before the kernel waits for its predecessor in the stream
//    (weights never depend on it), which hides the launch and the first DRAM round trip.
//
// 2. Instructions per weight.  A lane owns a whole 256-block: the 6-bit scales and mins of a Q4_K
//    block are unpacked once with a few word-wide logic ops, high nibbles are used in place (x16,
//    shifted out of the integer sum at the end), the min / bias terms are dp2a, and the dp4a of a
//    block run as independent chains: about 0.6 (Q4_K) and 1.4 (Q6_K) lane-instructions per weight
//    against 2.5 for a lane-per-16-byte-chunk mapping, which was instruction-bound.
//
// Work unit: Q4_K 8 rows x 4 blocks (lanes 4r..4r+3 hold row r), Q6_K 4 rows x 8 blocks (lanes
// 8r..8r+7), one contiguous 16-byte aligned run per row.  Shared-memory pitches (144-byte blocks in
// 576-byte rows; Q6_K chunk-major groups; activation blocks padded to 272 bytes) keep the 16-byte
// reads of a quarter-warp on distinct banks.  The (row group, K slice) units of a matrix are laid
// end to end and cut into equal contiguous ranges, one per warp of a persistent grid ("stream-K"),
// so every SM streams the same number of bytes whatever N and K are.  A row group whose K range is
// cut between warps is finished by the warp that holds its first slice: the others publish their
// partial sums (they reach them at the start of their range), the owner adds them in warp order
// at the end of its own -- deterministic, no float atomics.  Every wait (mbarrier or flag) is
// bounded and reports through an error word instead of hanging.
#include "kq_common.cuh"

#include <cuda.h> // CUtensorMap
#include <stdlib.h>
#include <string.h>

b200_status kq_tmap_encode(void *map128, int elem_bytes, int rank, const void *base, const uint64_t *dims,
                           const uint64_t *strides_bytes, const uint32_t *box, int swizzle128);

namespace {

constexpr int MAX_UNITS = 160 * 16;
constexpr uint32_t SPIN_LIMIT = 1u << 16;
constexpr int ACT_BLK = 272; // 256 int8 codes + 16 bytes of padding
// Bytes between the staged activations of consecutive tokens, beyond a multiple of 128: the kernels for 3 to 8
// tokens read one token per group of four lanes, and the offset puts those loads on different banks (8-byte
// loads of the Q4_K form: 32; 16-byte loads of the 8-token Q6_K form: 16).
template <uint32_t TYPE, int M>
constexpr int tok_pad() {
    return M <= 2 ? 0 : (TYPE == B200_TYPE_Q6_K && M > 4 ? 16 : 32);
}

// Cross-warp fix-up scratch, one 128-byte line per warp of the grid.  An entry is a partial sum and
// its ready flag in one 8-byte word (low half: float bits, high half: 1 when valid), written and
// read with single 64-bit accesses, so publishing needs no fence and collecting costs one round
// trip to L2.  The collector clears the entry after reading it.
__device__ unsigned long long g_partials[MAX_UNITS][16];
__device__ unsigned long long g_partials8[MAX_UNITS][64]; // the same for the 8-token kernel: [row][token]
__device__ int g_stream_error; // 0 ok, 1 mbarrier wait gave up, 2 partial-sum wait gave up

#ifndef KQ_GEMV_WARPS
#define KQ_GEMV_WARPS 16
#endif
#ifndef KQ_GEMV_CTAS
#define KQ_GEMV_CTAS 1
#endif
#ifndef KQ_GEMV_PB
#define KQ_GEMV_PB 2 // 256-blocks of the activation row a warp holds in registers while it prepares them (rows up to 8192 in one round)
#endif
#ifndef KQ_GEMV_GRIDMUL
#define KQ_GEMV_GRIDMUL 1
#endif
#ifdef KQ_GEMV_TRACE
// debug build only: per CTA and launch, %globaltimer at the phase boundaries of the kernel
__device__ unsigned long long g_trace[32768][16];
__device__ unsigned long long g_trace_w[32768][16]; // per warp: clock at the end of its work
__device__ unsigned long long g_trace_p[32768][16]; // per warp: cycles in post (bits 0..23), in wait_slot (24..47), units (48..63)
__device__ unsigned int g_trace_n;
#define TRACE_MARK(i) do { if (threadIdx.x == 0 && s_trace < 32768u) g_trace[s_trace][i] = (unsigned long long)clock64(); } while (0)
#else
#define TRACE_MARK(i)
#endif
template <uint32_t TYPE>
struct Fmt;
template <>
struct Fmt<B200_TYPE_Q4_K> {
    static constexpr int ROWS = 8, KB = 4, LPR = 4;          // rows / unit, blocks / slice, lanes / row
    static constexpr int PITCH = KB * KQ_Q4K_BYTES;          // 576: rows land 16 banks apart
    static constexpr int SLOT = ROWS * PITCH;                // 4608 = 36 x 128
    static constexpr int WARPS = KQ_GEMV_WARPS, CTAS_PER_SM = KQ_GEMV_CTAS, SMEM_CAP = 216 * 1024 / KQ_GEMV_CTAS;
};
template <>
struct Fmt<B200_TYPE_Q6_K> {
    static constexpr int ROWS = 4, KB = 8, LPR = 8;
    static constexpr int PITCH = KQ_Q6_GROUP_BYTES;          // one 1680-byte group
    static constexpr int SLOT = (ROWS * PITCH + 127) & ~127; // 6720 -> 6784: slots start on 128-byte boundaries
    static constexpr int WARPS = KQ_GEMV_WARPS, CTAS_PER_SM = KQ_GEMV_CTAS, SMEM_CAP = 216 * 1024 / KQ_GEMV_CTAS;
};

struct StreamParams {
    // One tensor map per weight segment: the matrix as [rows][row bytes / 8] of 8-byte words with a box of
    // one work unit (all of its rows, one K slice), so that a ring slot is requested by one tiled copy instead
    // of one bulk copy per row.  use_tma == 0: the maps are unset and the rows are copied one by one.
    alignas(64) CUtensorMap map[3];
    int32_t use_tma;
    int32_t pf_mode; // L2 prefetch before the dependency wait: 1 norm weights, 2 and the biases
    KqGemvSeg seg[3];
    int32_t rg_end[3];
    int32_t nseg, n_rg, nb, K, nsteps, swiglu;
    int32_t ns; // ring depth per warp
    // a launch that serves two matrix types at once gives each its own range of CTAs [cta0, cta0 + n_cta)
    // (n_cta == 0: the whole grid); the fix-up scratch is indexed by the warp's number in the whole grid
    int32_t cta0, n_cta;
    int32_t m_actual; // tokens really present (the 8-token kernel pads the rest with zeros)
    // A launch may cover a range of K only (rows too long for all tokens' activations to sit in shared memory
    // are done in several launches, each adding to the output of the one before): K, nb, nsteps then describe
    // the range, K_row the whole row (stride of the matrix), ks0 the range's first K slice, and the activation
    // pointers already point at the range while their token strides stay those of the whole row.
    int32_t K_row, ks0, a_ldk, a_ldb;
    // The (row group, K slice) work items are dealt to the warps of the launch part in order: uq items each, and
    // one more for the first ur warps.  The extra items thus fill whole CTAs, whose
    // warps then all end together, instead of leaving a few longer warps in every CTA (measured: 1.5 % of the
    // step; a linear tilt of the CTAs' shares towards the CTAs that start first, tried next, only costs).  Set
    // by the host, which knows the grid: the kernel needs no division before its first copy can go out.
    int32_t uq, ur;
    // fused gate / up only: the Q8 form of the output for the matmul that follows (see KqEmitQ8); e_q null = off
    int8_t *e_q;
    float *e_d;
    int16_t *e_bs;
    int32_t *e_cnt;
    const int8_t *aq;
    const float *ad;
    const int16_t *abs16;
    const float *residual;
    // fused activation preparation: when x is set the kernel quantises the f32 activations itself
    // (after an optional RMSNorm with weight norm_w) instead of reading aq / ad / abs16
    const float *x;
    const float *norm_w;
    float eps;
    int32_t do_norm;
};

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok)
                 : "r"(bar), "r"(parity)
                 : "memory");
    return ok != 0;
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}
__device__ __forceinline__ void tma_box(uint32_t dst, const CUtensorMap *map, int x, int y, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
                 "l"(map), "r"(x), "r"(y), "r"(bar)
                 : "memory");
}
// bounded wait on a ring slot; after a first give-up the CTA stops waiting altogether
__device__ __forceinline__ void wait_slot(uint32_t bar, uint32_t parity, volatile int *abort_flag) {
    if (*abort_flag) return;
    if (kq_mbar_wait(bar, parity, KQ_WAIT_LIMIT_NS)) return;
    *abort_flag = 1;
    atomicExch(&g_stream_error, 1);
}
// unsigned bytes of a times signed bytes of b, accumulated into c
__device__ __forceinline__ int dp4a_us(uint32_t a, int b, int c) {
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
#define KQ_BYTE(w, k) (((w) >> (8 * (k))) & 0xFFu)
#define KQ_SBYTE(w, k) ((int)(int8_t)(((w) >> (8 * (k))) & 0xFFu))

// first work item of warp u of the launch part
__device__ __forceinline__ int unit_first(const StreamParams &p, int u) { return u * p.uq + min(u, p.ur); }

template <uint32_t TYPE>
__device__ __forceinline__ void locate(const StreamParams &p, int rg, int &seg, int &row0) {
    int si = 0, rg0 = 0;
    if (p.nseg > 1 && rg >= p.rg_end[0]) { si = 1; rg0 = p.rg_end[0]; }
    if (p.nseg > 2 && rg >= p.rg_end[1]) { si = 2; rg0 = p.rg_end[1]; }
    seg = si;
    row0 = (rg - rg0) * (p.swiglu ? Fmt<TYPE>::ROWS / 2 : Fmt<TYPE>::ROWS);
}

// row slot rs of a group -> device row; swiglu: first half of the slots from the gate matrix,
// second half the same rows of the up matrix
template <uint32_t TYPE>
__device__ __forceinline__ const uint8_t *row_ptr(const StreamParams &p, int seg, int row0, int rs, int64_t stride) {
    constexpr int H = Fmt<TYPE>::ROWS / 2;
    if (p.swiglu) {
        const KqGemvSeg &sg = p.seg[rs / H];
        return sg.W + (int64_t)min(row0 + rs % H, sg.n_rows - 1) * stride;
    }
    return p.seg[seg].W + (int64_t)min(row0 + rs, p.seg[seg].n_rows - 1) * stride;
}

// Issue side of a warp's ring.  The copies of a unit are posted by ROWS lanes in parallel (lane r
// owns row slot r and keeps that row's address), so handing a slot back costs a few instructions
// instead of a serial loop on one lane.  All lanes keep (rg, ks) in step.
template <uint32_t TYPE>
struct Issuer {
    using F = Fmt<TYPE>;
    int rg, ks;
    const uint8_t *row; // lanes < ROWS: device row of slot `lane` in row group rg
    int64_t stride;

    __device__ __forceinline__ void seek(const StreamParams &p, int lane) {
        if (lane < F::ROWS && rg < p.n_rg) {
            int seg, row0;
            locate<TYPE>(p, rg, seg, row0);
            row = row_ptr<TYPE>(p, seg, row0, lane, stride);
        }
    }
    __device__ __forceinline__ void init(const StreamParams &p, int first, int lane) {
        rg = first / p.nsteps;
        ks = first % p.nsteps;
        stride = kq_device_row_bytes(TYPE, p.K_row);
        row = nullptr;
        if (!p.use_tma) seek(p, lane);
    }
    // post the next unit into the slot at slot_addr.  reuse: the slot has been read by this warp before (the
    // proxy fence orders those reads before the copy engine's writes); a slot that is filled for the first
    // time needs none.
    __device__ __forceinline__ void post(const StreamParams &p, int lane, uint32_t slot_addr, uint32_t bar, bool reuse = true) {
        if (p.use_tma) {
            // one box per unit (two with fused gate / up: half the rows from each matrix).  Rows past the
            // matrix and blocks past the row arrive as zeros; the box always counts its full size.
            if (lane == 0) {
                int seg, row0;
                locate<TYPE>(p, rg, seg, row0);
                const int x = (ks + p.ks0) * (F::PITCH / 8);
                mbar_expect_tx(bar, F::ROWS * F::PITCH);
#ifndef KQ_NO_REPOST_FENCE
                if (reuse) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
#endif
                if (p.swiglu) {
                    tma_box(slot_addr, &p.map[0], x, row0, bar);
                    tma_box(slot_addr + (F::ROWS / 2) * F::PITCH, &p.map[1], x, row0, bar);
                } else {
                    tma_box(slot_addr, &p.map[seg], x, row0, bar);
                }
            }
            if (++ks == p.nsteps) {
                ks = 0;
                rg++;
            }
            return;
        }
        const int kbn = min(F::KB, p.nb - ks * F::KB);
        uint32_t bytes;
        int64_t off;
        if (TYPE == B200_TYPE_Q4_K) {
            bytes = kbn * KQ_Q4K_BYTES;
            off = (int64_t)(ks + p.ks0) * F::KB * KQ_Q4K_BYTES;
        } else {
            bytes = (uint32_t)kq_q6_group_bytes(kbn);
            off = (int64_t)(ks + p.ks0) * KQ_Q6_GROUP_BYTES;
        }
        if (lane == 0) mbar_expect_tx(bar, bytes * F::ROWS);
        __syncwarp();
        if (lane < F::ROWS) {
            if (reuse) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            bulk_g2s(slot_addr + lane * F::PITCH, row + off, bytes, bar);
        }
        if (++ks == p.nsteps) {
            ks = 0;
            rg++;
            seek(p, lane);
        }
    }
};

// ---- one lane, one Q4_K block against M activation rows ----------------------------------------
// b: the 144 bytes of the block in shared memory; act: staged activations of token 0 (tokens are
// act_tok bytes apart): padded codes, then sums of 32 (int16 x 8 per block), then scales.
template <int M>
__device__ __forceinline__ void block_q4k(const uint8_t *b, const uint8_t *act, int act_tok, int act_q, int act_s,
                                          int blk, float (&acc)[M]) {
    const uint4 hdr = *reinterpret_cast<const uint4 *>(b);
    const uint32_t sc_lo = hdr.y & 0x3F3F3F3Fu, m_lo = hdr.z & 0x3F3F3F3Fu;
    const uint32_t sc_hi = (hdr.w & 0x0F0F0F0Fu) | ((hdr.y >> 2) & 0x30303030u);
    const uint32_t m_hi = ((hdr.w >> 4) & 0x0F0F0F0Fu) | ((hdr.z >> 2) & 0x30303030u);
    const float2 dd = __half22float2(*reinterpret_cast<const __half2 *>(&hdr.x));
    uint4 w[8];
#pragma unroll
    for (int i = 0; i < 8; i++) w[i] = *reinterpret_cast<const uint4 *>(b + 16 + 16 * i);
#pragma unroll
    for (int m = 0; m < M; m++) {
        const uint8_t *tq = act + m * act_tok;
        const uint8_t *a = tq + blk * ACT_BLK;
        int s_even = 0, s_odd16 = 0;
#pragma unroll
        for (int g = 0; g < 4; g++) { // 32 quant bytes: sub-block 2g in the low nibbles, 2g+1 in the high
            const int4 a0 = *reinterpret_cast<const int4 *>(a + 64 * g);
            const int4 a1 = *reinterpret_cast<const int4 *>(a + 64 * g + 16);
            const int4 a2 = *reinterpret_cast<const int4 *>(a + 64 * g + 32);
            const int4 a3 = *reinterpret_cast<const int4 *>(a + 64 * g + 48);
            const uint4 w0 = w[2 * g], w1 = w[2 * g + 1];
            int dl = dp4a_us(w0.x & 0x0F0F0F0Fu, a0.x, 0);
            dl = dp4a_us(w0.y & 0x0F0F0F0Fu, a0.y, dl);
            dl = dp4a_us(w0.z & 0x0F0F0F0Fu, a0.z, dl);
            dl = dp4a_us(w0.w & 0x0F0F0F0Fu, a0.w, dl);
            int dl2 = dp4a_us(w1.x & 0x0F0F0F0Fu, a1.x, 0);
            dl2 = dp4a_us(w1.y & 0x0F0F0F0Fu, a1.y, dl2);
            dl2 = dp4a_us(w1.z & 0x0F0F0F0Fu, a1.z, dl2);
            dl2 = dp4a_us(w1.w & 0x0F0F0F0Fu, a1.w, dl2);
            int dh = dp4a_us(w0.x & 0xF0F0F0F0u, a2.x, 0); // 16 x the high-nibble dot
            dh = dp4a_us(w0.y & 0xF0F0F0F0u, a2.y, dh);
            dh = dp4a_us(w0.z & 0xF0F0F0F0u, a2.z, dh);
            dh = dp4a_us(w0.w & 0xF0F0F0F0u, a2.w, dh);
            int dh2 = dp4a_us(w1.x & 0xF0F0F0F0u, a3.x, 0);
            dh2 = dp4a_us(w1.y & 0xF0F0F0F0u, a3.y, dh2);
            dh2 = dp4a_us(w1.z & 0xF0F0F0F0u, a3.z, dh2);
            dh2 = dp4a_us(w1.w & 0xF0F0F0F0u, a3.w, dh2);
            const uint32_t scw = g < 2 ? sc_lo : sc_hi;
            const int k0 = (2 * g) & 3;
            s_even += (int)KQ_BYTE(scw, k0) * (dl + dl2);
            s_odd16 += (int)KQ_BYTE(scw, k0 + 1) * (dh + dh2);
        }
        const int isum = s_even + (s_odd16 >> 4);
        const uint4 bsw = *reinterpret_cast<const uint4 *>(tq + act_q + blk * 16);
        int msum = __dp2a_lo((int)bsw.x, (int)m_lo, 0);
        msum = __dp2a_hi((int)bsw.y, (int)m_lo, msum);
        msum = __dp2a_lo((int)bsw.z, (int)m_hi, msum);
        msum = __dp2a_hi((int)bsw.w, (int)m_hi, msum);
        const float da = reinterpret_cast<const float *>(tq + act_q + act_s)[blk];
        acc[m] = fmaf(dd.x * da, (float)isum, acc[m]);
        acc[m] = fmaf(-(dd.y * da), (float)msum, acc[m]);
    }
}

// ---- one lane, one Q6_K block (block bl of a group of g blocks, chunk-major planes) ----------------
// For Q6_K the staged sums are kept per 16 elements (int16 x 16 per block, 32 bytes).
template <int M>
__device__ __forceinline__ void block_q6k(const uint8_t *grp, int g, int bl, const uint8_t *act, int act_tok,
                                          int act_q, int act_s, int blk, float (&acc)[M]) {
    const uint8_t *ql = grp + bl * 16, *qh = grp + g * 128 + bl * 16;
    const int cs = g * 16; // distance between consecutive chunks of one block
    const uint4 scv = *reinterpret_cast<const uint4 *>(grp + g * 192 + bl * 16);
    const float dw = kq_h2f(*reinterpret_cast<const uint16_t *>(grp + g * 208 + bl * 2));
    const uint32_t scw[4] = {scv.x, scv.y, scv.z, scv.w};
    int isum[M];
#pragma unroll
    for (int m = 0; m < M; m++) isum[m] = 0;
#pragma unroll
    for (int j = 0; j < 4; j++) {
        // qh chunk j = positions 16*c1 .. +15 of half h; its bit pairs q = 0..3 belong to the
        // elements 128h + 32q + 16c1 + i, i.e. scale group 8h + 2q + c1
        const int h = j >> 1, c1 = j & 1;
        const uint4 hv = *reinterpret_cast<const uint4 *>(qh + j * cs);
        const uint4 la = *reinterpret_cast<const uint4 *>(ql + (4 * h + c1) * cs);     // q = 0 (low), 2 (high)
        const uint4 lb = *reinterpret_cast<const uint4 *>(ql + (4 * h + c1 + 2) * cs); // q = 1 (low), 3 (high)
        const uint32_t hw[4] = {hv.x, hv.y, hv.z, hv.w};
        const uint32_t aw[4] = {la.x, la.y, la.z, la.w};
        const uint32_t bw[4] = {lb.x, lb.y, lb.z, lb.w};
        uint32_t v0[4], v1[4], v2[4], v3[4];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            v0[i] = (aw[i] & 0x0F0F0F0Fu) | ((hw[i] << 4) & 0x30303030u);
            v1[i] = (bw[i] & 0x0F0F0F0Fu) | ((hw[i] << 2) & 0x30303030u);
            v2[i] = ((aw[i] >> 4) & 0x0F0F0F0Fu) | (hw[i] & 0x30303030u);
            v3[i] = ((bw[i] >> 4) & 0x0F0F0F0Fu) | ((hw[i] >> 2) & 0x30303030u);
        }
        const int e0 = 128 * h + 16 * c1;
        const int s0 = 8 * h + c1; // scale group of q = 0; q adds 2
#pragma unroll
        for (int m = 0; m < M; m++) {
            const uint8_t *a = act + m * act_tok + blk * ACT_BLK + e0;
            const int4 a0 = *reinterpret_cast<const int4 *>(a);
            const int4 a1 = *reinterpret_cast<const int4 *>(a + 32);
            const int4 a2 = *reinterpret_cast<const int4 *>(a + 64);
            const int4 a3 = *reinterpret_cast<const int4 *>(a + 96);
            int d0 = dp4a_us(v0[0], a0.x, 0), d1 = dp4a_us(v1[0], a1.x, 0), d2 = dp4a_us(v2[0], a2.x, 0),
                d3 = dp4a_us(v3[0], a3.x, 0);
            d0 = dp4a_us(v0[1], a0.y, d0); d1 = dp4a_us(v1[1], a1.y, d1); d2 = dp4a_us(v2[1], a2.y, d2); d3 = dp4a_us(v3[1], a3.y, d3);
            d0 = dp4a_us(v0[2], a0.z, d0); d1 = dp4a_us(v1[2], a1.z, d1); d2 = dp4a_us(v2[2], a2.z, d2); d3 = dp4a_us(v3[2], a3.z, d3);
            d0 = dp4a_us(v0[3], a0.w, d0); d1 = dp4a_us(v1[3], a1.w, d1); d2 = dp4a_us(v2[3], a2.w, d2); d3 = dp4a_us(v3[3], a3.w, d3);
            isum[m] += KQ_SBYTE(scw[(s0) >> 2], (s0) & 3) * d0 + KQ_SBYTE(scw[(s0 + 2) >> 2], (s0 + 2) & 3) * d1 +
                       KQ_SBYTE(scw[(s0 + 4) >> 2], (s0 + 4) & 3) * d2 + KQ_SBYTE(scw[(s0 + 6) >> 2], (s0 + 6) & 3) * d3;
        }
    }
#pragma unroll
    for (int m = 0; m < M; m++) {
        const uint8_t *tq = act + m * act_tok;
        // codes carry a +32 bias: sum (q - 32) a = sum q a - 32 sum a, with sum a per scale group
        const uint4 b0 = *reinterpret_cast<const uint4 *>(tq + act_q + blk * 32);
        const uint4 b1 = *reinterpret_cast<const uint4 *>(tq + act_q + blk * 32 + 16);
        int bias = __dp2a_lo((int)b0.x, (int)scw[0], 0);
        bias = __dp2a_hi((int)b0.y, (int)scw[0], bias);
        bias = __dp2a_lo((int)b0.z, (int)scw[1], bias);
        bias = __dp2a_hi((int)b0.w, (int)scw[1], bias);
        bias = __dp2a_lo((int)b1.x, (int)scw[2], bias);
        bias = __dp2a_hi((int)b1.y, (int)scw[2], bias);
        bias = __dp2a_lo((int)b1.z, (int)scw[3], bias);
        bias = __dp2a_hi((int)b1.w, (int)scw[3], bias);
        const float da = reinterpret_cast<const float *>(tq + act_q + act_s)[blk];
        acc[m] = fmaf(dw * da, (float)(isum[m] - 32 * bias), acc[m]);
    }
}

// ---- 3 to 8 tokens: the integer dot products on the tensor cores --------------------------------
// With several tokens the dp4a work per weight byte grows with the token count and the kernel turns
// issue-bound; mma.m16n8k32 (u8 x s8 -> s32) does the 32-element sub-block products of 8 weight rows
// against 8 tokens in one instruction.  A warp works through the blocks of its unit one at a time:
// lane (r, t) = (lane / 4, lane % 4) holds row r; the nibbles of 8 consecutive bytes of a 32-byte
// group are its A fragments for the two sub-blocks of that group (elements 8t .. 8t+7; the same
// permutation of k is used for the activation fragments, so the sums are unchanged), rows 8..15 of
// the tile are zero.  The accumulators come back as (row r, tokens 2t, 2t+1); the 6-bit scales, the
// min term and the f32 combination are the decode kernel's, so results are identical token by token.
// d = a * b with a zero accumulator: rows 8..15 of the A tile are zero, only d0 / d1 (row lane/4, tokens
// 2 (lane%4), +1) are used
__device__ __forceinline__ void mma_u8s8(int &d0, int &d1, uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
    int d2, d3;
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                 : "=r"(d0), "=r"(d1), "=r"(d2), "=r"(d3)
                 : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1), "r"(0));
}

template <uint32_t TYPE, int M>
__device__ __forceinline__ void mma_units(const StreamParams &p, const uint8_t *smem, int act_tok, int act_q, int act_s,
                                          const uint8_t *ring, uint32_t ring_addr, uint32_t bar_addr, Issuer<TYPE> &iss,
                                          int count, int begin, int unit, int n_units, int total,
                                          volatile int *s_abort) {
    using F = Fmt<TYPE>;
    static_assert(TYPE == B200_TYPE_Q4_K, "the tensor-core batch path is built for Q4_K");
    const int lane = threadIdx.x & 31, r = lane >> 2, t = lane & 3, nb = p.nb;
    const int tokB = lane >> 2;                       // token whose activations this lane feeds to the MMA
    const bool tokB_ok = tokB < M;                     // M = tokens staged in shared memory (4 or 8)
    const uint8_t *actB = smem + (tokB_ok ? tokB : 0) * act_tok;
    const int tok0 = 2 * t, tok1 = 2 * t + 1;         // tokens of this lane's accumulators
    const uint8_t *act0 = smem + (tok0 < M ? tok0 : 0) * act_tok, *act1 = smem + (tok1 < M ? tok1 : 0) * act_tok;
    float acc0 = 0.f, acc1 = 0.f;
    int rg = begin / p.nsteps, ks = begin % p.nsteps;
    for (int j = 0; j < count; j++) {
        const int slot = j % p.ns;
        wait_slot(bar_addr + slot * 8, (uint32_t)((j / p.ns) & 1), s_abort);
        const uint8_t *rowp = ring + (size_t)slot * F::SLOT + r * F::PITCH;
        const int kbn = min(F::KB, nb - ks * F::KB);
        for (int kb = 0; kb < kbn; kb++) {
            const int blk = ks * F::KB + kb;
            const uint8_t *b = rowp + kb * KQ_Q4K_BYTES;
            const uint4 hdr = *reinterpret_cast<const uint4 *>(b);
            const uint32_t sc_lo = hdr.y & 0x3F3F3F3Fu, m_lo = hdr.z & 0x3F3F3F3Fu;
            const uint32_t sc_hi = (hdr.w & 0x0F0F0F0Fu) | ((hdr.y >> 2) & 0x30303030u);
            const uint32_t m_hi = ((hdr.w >> 4) & 0x0F0F0F0Fu) | ((hdr.z >> 2) & 0x30303030u);
            const float2 dd = __half22float2(*reinterpret_cast<const __half2 *>(&hdr.x));
            int ev0 = 0, ev1 = 0, od0 = 0, od1 = 0; // odd sub-blocks carry a factor 16 (high nibbles left in place)
#pragma unroll
            for (int g = 0; g < 4; g++) {
                const uint2 w = *reinterpret_cast<const uint2 *>(b + 16 + 32 * g + 8 * t);
                uint2 x0 = make_uint2(0u, 0u), x1 = make_uint2(0u, 0u);
                if (tokB_ok) {
                    x0 = *reinterpret_cast<const uint2 *>(actB + blk * ACT_BLK + 64 * g + 8 * t);
                    x1 = *reinterpret_cast<const uint2 *>(actB + blk * ACT_BLK + 64 * g + 32 + 8 * t);
                }
                const uint32_t scw = g < 2 ? sc_lo : sc_hi;
                const int k0 = (2 * g) & 3;
                int c0, c1, e0, e1;
                mma_u8s8(c0, c1, w.x & 0x0F0F0F0Fu, w.y & 0x0F0F0F0Fu, x0.x, x0.y); // sub-block 2g
                mma_u8s8(e0, e1, w.x & 0xF0F0F0F0u, w.y & 0xF0F0F0F0u, x1.x, x1.y); // 16 x sub-block 2g + 1
                ev0 += (int)KQ_BYTE(scw, k0) * c0;
                ev1 += (int)KQ_BYTE(scw, k0) * c1;
                od0 += (int)KQ_BYTE(scw, k0 + 1) * e0;
                od1 += (int)KQ_BYTE(scw, k0 + 1) * e1;
            }
            const int is0 = ev0 + (od0 >> 4), is1 = ev1 + (od1 >> 4);
            // min term and f32 combination exactly as the one- and two-token kernel does them
            const uint4 q0 = *reinterpret_cast<const uint4 *>(act0 + act_q + blk * 16);
            const uint4 q1 = *reinterpret_cast<const uint4 *>(act1 + act_q + blk * 16);
            int mn0 = __dp2a_lo((int)q0.x, (int)m_lo, 0), mn1 = __dp2a_lo((int)q1.x, (int)m_lo, 0);
            mn0 = __dp2a_hi((int)q0.y, (int)m_lo, mn0);
            mn1 = __dp2a_hi((int)q1.y, (int)m_lo, mn1);
            mn0 = __dp2a_lo((int)q0.z, (int)m_hi, mn0);
            mn1 = __dp2a_lo((int)q1.z, (int)m_hi, mn1);
            mn0 = __dp2a_hi((int)q0.w, (int)m_hi, mn0);
            mn1 = __dp2a_hi((int)q1.w, (int)m_hi, mn1);
            const float da0 = reinterpret_cast<const float *>(act0 + act_q + act_s)[blk];
            const float da1 = reinterpret_cast<const float *>(act1 + act_q + act_s)[blk];
            acc0 = fmaf(dd.x * da0, (float)is0, acc0);
            acc0 = fmaf(-(dd.y * da0), (float)mn0, acc0);
            acc1 = fmaf(dd.x * da1, (float)is1, acc1);
            acc1 = fmaf(-(dd.y * da1), (float)mn1, acc1);
        }
        __syncwarp();
        if (j + p.ns < count) iss.post(p, lane, ring_addr + slot * F::SLOT, bar_addr + slot * 8);
        const bool last_slice = ks == p.nsteps - 1, last_unit = j == count - 1;
        if (last_slice || last_unit) {
            float v0 = acc0, v1 = acc1;
            acc0 = acc1 = 0.f;
            const int64_t rg_first = (int64_t)rg * p.nsteps;
            if (rg_first < begin) { // the head of this row group belongs to an earlier warp
                *(volatile unsigned long long *)&g_partials8[unit][r * 8 + tok0] = (unsigned long long)__float_as_uint(v0) | (1ull << 32);
                *(volatile unsigned long long *)&g_partials8[unit][r * 8 + tok1] = (unsigned long long)__float_as_uint(v1) | (1ull << 32);
            } else {
                if (!last_slice) { // later warps hold the tail: every lane collects its own two entries, in unit order
                    const int64_t rg_last = rg_first + p.nsteps;
                    for (int u2 = unit + 1; u2 < n_units; u2++) {
                        const int b2 = unit_first(p, u2), e2 = unit_first(p, u2 + 1);
                        if (b2 >= rg_last) break;
                        if (e2 <= b2) continue;
#pragma unroll
                        for (int i = 0; i < 2; i++) {
                            volatile unsigned long long *e = &g_partials8[u2][r * 8 + tok0 + i];
                            unsigned long long wv = 0;
                            bool ok = false;
                            const uint64_t t0 = kq_globaltimer_ns();
                            while (true) {
                                wv = *e;
                                ok = (wv >> 32) != 0;
                                if (ok || *s_abort || kq_globaltimer_ns() - t0 > KQ_WAIT_LIMIT_NS) break;
                                __nanosleep(64);
                            }
                            if (!ok && !*s_abort) {
                                *s_abort = 1;
                                atomicExch(&g_stream_error, 2);
                            }
                            *e = 0ull;
                            (i == 0 ? v0 : v1) += __uint_as_float((uint32_t)wv);
                        }
                    }
                }
                int seg, row0;
                locate<TYPE>(p, rg, seg, row0);
                if (p.swiglu) { // rows 0..3 of the tile are gate rows, rows 4..7 the same rows of the up matrix
                    const float u0 = __shfl_down_sync(0xffffffffu, v0, 16), u1 = __shfl_down_sync(0xffffffffu, v1, 16);
                    const int row = row0 + r;
                    if (r < F::ROWS / 2 && row < p.seg[0].n_rows) {
                        const float bg = p.seg[0].bias ? p.seg[0].bias[row] : 0.f, bu = p.seg[1].bias ? p.seg[1].bias[row] : 0.f;
                        if (tok0 < p.m_actual) {
                            const float gt = v0 + bg;
                            p.seg[0].y[(int64_t)tok0 * p.seg[0].ldy + row] = (gt / (1.0f + expf(-gt))) * (u0 + bu);
                        }
                        if (tok1 < p.m_actual) {
                            const float gt = v1 + bg;
                            p.seg[0].y[(int64_t)tok1 * p.seg[0].ldy + row] = (gt / (1.0f + expf(-gt))) * (u1 + bu);
                        }
                    }
                } else {
                    const KqGemvSeg &sg = p.seg[seg];
                    const int row = row0 + r;
                    if (row < sg.n_rows) {
                        const float bb = sg.bias ? sg.bias[row] : 0.f;
                        if (tok0 < p.m_actual) {
                            float x = v0 + bb;
                            if (p.residual) x += p.residual[(int64_t)tok0 * sg.ldy + row];
                            sg.y[(int64_t)tok0 * sg.ldy + row] = x;
                        }
                        if (tok1 < p.m_actual) {
                            float x = v1 + bb;
                            if (p.residual) x += p.residual[(int64_t)tok1 * sg.ldy + row];
                            sg.y[(int64_t)tok1 * sg.ldy + row] = x;
                        }
                    }
                }
            }
        }
        if (++ks == p.nsteps) {
            ks = 0;
            rg++;
        }
    }
}

// ---- 5 to 8 tokens, Q6_K: the same idea on 4-row units ---------------------------------------------
// A Q6_K unit is four rows by one group of eight blocks, and its scales cover 16 elements, half of the
// k = 32 of one instruction.  So the 8 x 32 A tile holds, for weight row w = (lane / 4) % 4, one scale
// group in k = 0..15 of tile row w (zeros in k = 16..31) and another in k = 16..31 of tile row w + 4 (zeros
// in k = 0..15): one instruction gives the 16-element products of two scale groups of four rows against
// eight tokens, each in its own accumulator.  Lanes 0..15 (h2 = 0) assemble the codes that sit in the low
// nibbles of the block's ql bytes (q = 0, 1), lanes 16..31 (h2 = 1) those in the high nibbles (q = 2, 3);
// both take word lane % 4 of the 16-byte chunks, so the weight loads are conflict free (rows are 1680 bytes
// apart).  The activations are staged for this kernel as [block][lane % 4][scale group][4 codes], which
// makes the B fragments of a block four 16-byte loads per lane.  Integer sums, the -32 offset through
// the staged sums and the f32 combination are those of the dp4a form, block by block.
template <int M>
__device__ __forceinline__ void mma_units_q6(const StreamParams &p, const uint8_t *smem, int act_tok, int act_q, int act_s,
                                             const uint8_t *ring, uint32_t ring_addr, uint32_t bar_addr,
                                             Issuer<B200_TYPE_Q6_K> &iss, int count, int begin, int unit, int n_units,
                                             int total, volatile int *s_abort) {
    using F = Fmt<B200_TYPE_Q6_K>;
    static_assert(M == 8, "eight staged tokens (padding tokens are zeros)");
    const int lane = threadIdx.x & 31, g8 = lane >> 2, t = lane & 3, nb = p.nb;
    const int rw = g8 & 3, h2 = g8 >> 2;               // weight row of the unit; nibble half this lane assembles
    const uint8_t *actB = smem + g8 * act_tok;          // token whose activations this lane feeds to the MMA
    const int tok0 = 2 * t, tok1 = 2 * t + 1;           // tokens of this lane's accumulators
    const uint8_t *act0 = smem + tok0 * act_tok, *act1 = smem + tok1 * act_tok;
    const uint8_t *actS = h2 ? act1 : act0;             // token whose -32 term this lane works out
    const uint32_t m_lo = h2 ? 0u : 0x3F3F3F3Fu, m_hi = h2 ? 0x3F3F3F3Fu : 0u;
    const int sh4 = 4 * h2, r1 = h2 ? 0 : 4, r2 = h2 ? 30 : 2;
    float acc0 = 0.f, acc1 = 0.f;
    int rg = begin / p.nsteps, ks = begin % p.nsteps;
    for (int j = 0; j < count; j++) {
        const int slot = j % p.ns;
        wait_slot(bar_addr + slot * 8, (uint32_t)((j / p.ns) & 1), s_abort);
        const uint8_t *grp = ring + (size_t)slot * F::SLOT + rw * F::PITCH;
        const int gn = min(F::KB, nb - ks * F::KB); // blocks in this group
        const int cs = gn * 16;                      // distance between consecutive chunks of one block
        for (int bl = 0; bl < gn; bl++) {
            const int blk = ks * F::KB + bl;
            const uint8_t *ql = grp + bl * 16 + 4 * t, *qh = grp + gn * 128 + bl * 16 + 4 * t;
            const uint4 scv = *reinterpret_cast<const uint4 *>(grp + gn * 192 + bl * 16);
            const float dw = kq_h2f(*reinterpret_cast<const uint16_t *>(grp + gn * 208 + bl * 2));
            const uint32_t sw[2] = {h2 ? scv.y : scv.x, h2 ? scv.w : scv.z}; // scale groups 8h + 4 h2 .. + 3
            uint32_t xb[16];
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const uint4 v = *reinterpret_cast<const uint4 *>(actB + blk * ACT_BLK + 64 * t + 16 * i);
                xb[4 * i] = v.x; xb[4 * i + 1] = v.y; xb[4 * i + 2] = v.z; xb[4 * i + 3] = v.w;
            }
            int is0 = 0, is1 = 0;
#pragma unroll
            for (int jj = 0; jj < 4; jj++) {
                // qh chunk jj = bytes 16 c1 .. of half h; bit pair q of a byte belongs to element 128 h + 32 q + 16 c1 + i,
                // scale group 8 h + 2 q + c1; its low four bits are in ql chunk 4 h + c1 (q = 0 low, 2 high nibble)
                // or 4 h + c1 + 2 (q = 1, 3)
                const int h = jj >> 1, c1 = jj & 1;
                const uint32_t hv = *reinterpret_cast<const uint32_t *>(qh + jj * cs);
                const uint32_t la = *reinterpret_cast<const uint32_t *>(ql + (4 * h + c1) * cs);
                const uint32_t lb = *reinterpret_cast<const uint32_t *>(ql + (4 * h + c1 + 2) * cs);
                // q = 0 (h2 = 0) in k 0..15, q = 2 (h2 = 1) in k 16..31
                const uint32_t a1 = (((la >> sh4) & 0x0F0F0F0Fu) | (__funnelshift_l(hv, hv, r1) & 0xF0F0F0F0u));
                int c0, c1v;
                mma_u8s8(c0, c1v, a1 & m_lo, a1 & m_hi, xb[8 * h + c1], xb[8 * h + 4 + c1]);
                const int s1 = KQ_SBYTE(sw[h], c1);
                is0 += s1 * c0;
                is1 += s1 * c1v;
                // q = 1 (h2 = 0), q = 3 (h2 = 1)
                const uint32_t a2 = (((lb >> sh4) & 0x0F0F0F0Fu) | (__funnelshift_l(hv, hv, r2) & 0xF0F0F0F0u));
                int e0, e1;
                mma_u8s8(e0, e1, a2 & m_lo, a2 & m_hi, xb[8 * h + 2 + c1], xb[8 * h + 6 + c1]);
                const int s2 = KQ_SBYTE(sw[h], c1 + 2);
                is0 += s2 * e0;
                is1 += s2 * e1;
            }
            // the two nibble halves of a row add up; each half works out the -32 term of one of the two tokens
            is0 += __shfl_xor_sync(0xffffffffu, is0, 16);
            is1 += __shfl_xor_sync(0xffffffffu, is1, 16);
            const uint4 b0 = *reinterpret_cast<const uint4 *>(actS + act_q + blk * 32);
            const uint4 b1 = *reinterpret_cast<const uint4 *>(actS + act_q + blk * 32 + 16);
            int bias = __dp2a_lo((int)b0.x, (int)scv.x, 0);
            bias = __dp2a_hi((int)b0.y, (int)scv.x, bias);
            bias = __dp2a_lo((int)b0.z, (int)scv.y, bias);
            bias = __dp2a_hi((int)b0.w, (int)scv.y, bias);
            bias = __dp2a_lo((int)b1.x, (int)scv.z, bias);
            bias = __dp2a_hi((int)b1.y, (int)scv.z, bias);
            bias = __dp2a_lo((int)b1.z, (int)scv.w, bias);
            bias = __dp2a_hi((int)b1.w, (int)scv.w, bias);
            const int other = __shfl_xor_sync(0xffffffffu, bias, 16);
            const int bias0 = h2 ? other : bias, bias1 = h2 ? bias : other;
            const float da0 = reinterpret_cast<const float *>(act0 + act_q + act_s)[blk];
            const float da1 = reinterpret_cast<const float *>(act1 + act_q + act_s)[blk];
            acc0 = fmaf(dw * da0, (float)(is0 - 32 * bias0), acc0);
            acc1 = fmaf(dw * da1, (float)(is1 - 32 * bias1), acc1);
        }
        __syncwarp();
        if (j + p.ns < count) iss.post(p, lane, ring_addr + slot * F::SLOT, bar_addr + slot * 8);
        const bool last_slice = ks == p.nsteps - 1, last_unit = j == count - 1;
        if (last_slice || last_unit) {
            float v0 = acc0, v1 = acc1;
            acc0 = acc1 = 0.f;
            const int64_t rg_first = (int64_t)rg * p.nsteps;
            if (h2 == 0) { // lanes 16..31 hold the same values
                if (rg_first < begin) { // the head of this row group belongs to an earlier warp
                    *(volatile unsigned long long *)&g_partials8[unit][rw * 8 + tok0] = (unsigned long long)__float_as_uint(v0) | (1ull << 32);
                    *(volatile unsigned long long *)&g_partials8[unit][rw * 8 + tok1] = (unsigned long long)__float_as_uint(v1) | (1ull << 32);
                } else {
                    if (!last_slice) { // later warps hold the tail: every lane collects its own two entries, in unit order
                        const int64_t rg_last = rg_first + p.nsteps;
                        for (int u2 = unit + 1; u2 < n_units; u2++) {
                            const int b2 = unit_first(p, u2), e2 = unit_first(p, u2 + 1);
                            if (b2 >= rg_last) break;
                            if (e2 <= b2) continue;
#pragma unroll
                            for (int i = 0; i < 2; i++) {
                                volatile unsigned long long *e = &g_partials8[u2][rw * 8 + tok0 + i];
                                unsigned long long wv = 0;
                                bool ok = false;
                                const uint64_t t0 = kq_globaltimer_ns();
                                while (true) {
                                    wv = *e;
                                    ok = (wv >> 32) != 0;
                                    if (ok || *s_abort || kq_globaltimer_ns() - t0 > KQ_WAIT_LIMIT_NS) break;
                                    __nanosleep(64);
                                }
                                if (!ok && !*s_abort) {
                                    *s_abort = 1;
                                    atomicExch(&g_stream_error, 2);
                                }
                                *e = 0ull;
                                (i == 0 ? v0 : v1) += __uint_as_float((uint32_t)wv);
                            }
                        }
                    }
                    int seg, row0;
                    locate<B200_TYPE_Q6_K>(p, rg, seg, row0);
                    const KqGemvSeg &sg = p.seg[seg];
                    const int row = row0 + rw;
                    if (row < sg.n_rows) {
                        const float bb = sg.bias ? sg.bias[row] : 0.f;
                        if (tok0 < p.m_actual) {
                            float x = v0 + bb;
                            if (p.residual) x += p.residual[(int64_t)tok0 * sg.ldy + row];
                            sg.y[(int64_t)tok0 * sg.ldy + row] = x;
                        }
                        if (tok1 < p.m_actual) {
                            float x = v1 + bb;
                            if (p.residual) x += p.residual[(int64_t)tok1 * sg.ldy + row];
                            sg.y[(int64_t)tok1 * sg.ldy + row] = x;
                        }
                    }
                }
            }
            __syncwarp();
        }
        if (++ks == p.nsteps) {
            ks = 0;
            rg++;
        }
    }
}

// ---- several dependent matmuls in one launch ------------------------------------------------------
// A decode layer is a chain of matrix-vector products, each needing the whole output of the one
// before.  As separate launches every link costs the tail of one kernel (the last warps finishing,
// the fix-up), the hand-over and the head of the next (its first copies queueing) with HBM idle in
// between.  The fused kernel runs the links as phases of one persistent grid: a warp that has
// finished its share of phase i at once starts the weight stream of its share of phase i + 1 into
// its own ring (weights depend on nothing), and only then joins the grid-wide barrier after which
// the activations of phase i + 1 can be read.  Shared memory has one layout for all phases
// (activation area of the longest row, then a fixed byte range per warp for its ring), so the early
// copies of one warp never touch what another warp still reads.
struct FusedCtx {
    int act_bytes;   // activation area at the start of shared memory (all phases)
    int ring_bytes;  // ring range of one warp
    int phase;       // 0 = first phase (waits for the previous kernel), else waits for the grid
    unsigned target; // arrivals the barrier before this phase has to see
};
__device__ unsigned int g_fused_bar[2]; // arrivals at the phase barriers, CTAs that have left; both return to 0

// All threads of the CTA.  The barrier doubles as the arrival for the phase that ends: everything the CTA
// wrote is made visible before it counts itself in.  Bounded like every other wait of the library.
// The barrier comes in two halves so that the copies of the next phase can be posted between them: the
// fence of the arrival would otherwise have to sit behind those copies.
__device__ __forceinline__ void fused_grid_arrive() {
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        atomicAdd(&g_fused_bar[0], 1u);
    }
}
__device__ __forceinline__ void fused_grid_wait(unsigned target, volatile int *s_abort) {
    if (threadIdx.x == 0) {
        const uint64_t t0 = kq_globaltimer_ns();
        while (true) {
            unsigned v;
            asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(&g_fused_bar[0]) : "memory");
            if (v >= target || *s_abort) break;
            if (kq_globaltimer_ns() - t0 > KQ_WAIT_LIMIT_NS) {
                *s_abort = 1;
                atomicExch(&g_stream_error, 3);
                break;
            }
            __nanosleep(32);
        }
    }
    __syncthreads();
}

// activations written earlier in the same launch by other SMs are read through L2
template <bool FUSED>
__device__ __forceinline__ float4 ld_act4(const float *p) {
    return FUSED ? __ldcg(reinterpret_cast<const float4 *>(p)) : *reinterpret_cast<const float4 *>(p);
}
template <bool FUSED>
__device__ __forceinline__ float ld_act1(const float *p) {
    return FUSED ? __ldcg(p) : *p;
}

template <uint32_t TYPE, int M, bool FUSED>
__device__ __forceinline__ void stream_body(const StreamParams &p, uint8_t *smem, int &s_abort, const FusedCtx &fx,
                                            uint32_t (&uses)[4]) {
    using F = Fmt<TYPE>;
    constexpr int WARPS = F::WARPS;
#ifdef KQ_GEMV_TRACE
    __shared__ unsigned int s_trace;
    if (threadIdx.x == 0) {
        s_trace = atomicAdd(&g_trace_n, 1u);
    }
    __syncthreads();
    TRACE_MARK(0);
    if (threadIdx.x == 0 && s_trace < 32768u) {
        g_trace[s_trace][7] = ((unsigned long long)blockIdx.x << 32) | (unsigned)p.n_rg;
        g_trace[s_trace][8] = kq_globaltimer_ns();
        unsigned smid;
        asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
        g_trace[s_trace][13] = smid;
    }
#endif
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int rs = lane / F::LPR, t = lane % F::LPR;
    const int nb = p.nb;
    // the copy engine's descriptors: fetched now, so that the first copy does not wait for them
    if (p.use_tma && lane == 0 && warp < (p.swiglu ? 2 : p.nseg)) asm volatile("prefetch.tensormap [%0];" ::"l"(&p.map[warp]) : "memory");

    // ---- shared memory: per token [padded int8 codes][int16 sums][f32 scales], then rings, then mbarriers
    constexpr int SUMS = TYPE == B200_TYPE_Q4_K ? 16 : 32; // bytes of sums per block
    const int act_q = (nb * ACT_BLK + 127) & ~127, act_s = (nb * SUMS + 127) & ~127, act_d = (nb * 4 + 127) & ~127;
    // 8-token kernel: tokens 32 bytes apart modulo 128, so that the B-fragment loads of the eight
    // token lanes of a warp fall on different banks
    const int act_tok = act_q + act_s + act_d + tok_pad<TYPE, M>();
    if (FUSED && fx.phase > 0) fused_grid_arrive(); // everything this CTA wrote in the phase before is published
    const int ns = FUSED ? min(4, fx.ring_bytes / F::SLOT) : p.ns; // ring depth
    uint8_t *ring = FUSED ? smem + fx.act_bytes + (size_t)warp * fx.ring_bytes : smem + M * act_tok + (size_t)warp * ns * F::SLOT;
    uint64_t *bars = FUSED ? reinterpret_cast<uint64_t *>(smem + fx.act_bytes + (size_t)WARPS * fx.ring_bytes) + warp * 4
                           : reinterpret_cast<uint64_t *>(smem + M * act_tok + (size_t)WARPS * ns * F::SLOT) + warp * ns;
    if (!FUSED && threadIdx.x == 0) s_abort = 0;
    // the ring and its barriers are private to the warp: set them up and start the weight stream
    // before anything that depends on the previous kernel.  Later phases of a fused launch keep the
    // barriers of the first one (all four, whatever the ring depth of a phase) and continue their
    // parity: uses[s] counts how often barrier s has completed so far.
    if (lane == 0 && !(FUSED && fx.phase > 0))
        for (int s = 0; s < (FUSED ? 4 : ns); s++) mbar_init(smem_u32(&bars[s]), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    __syncwarp();
    TRACE_MARK(14);
    const int unit = ((int)blockIdx.x - p.cta0) * WARPS + warp, n_units = (p.n_cta ? p.n_cta : (int)gridDim.x) * WARPS;
    const int pbase = p.cta0 * WARPS; // this launch part's first line of the fix-up scratch
    const int total = p.n_rg * p.nsteps;
    const int begin = unit_first(p, unit), end = unit_first(p, unit + 1);
    const int count = end - begin;
    const uint32_t ring_addr = smem_u32(ring), bar_addr = smem_u32(bars);
    Issuer<TYPE> iss;
    iss.init(p, begin, lane);
    TRACE_MARK(15);
    // The first slot of the ring goes out at once; the remaining slots are posted only after the loads of
    // the activations have been issued.  Measured both ways: with everything posted before the dependency
    // wait the activation loads queue behind twice the weight traffic and the step is 2 % slower; with
    // nothing posted before it, 1.5 % slower.
    const int pre = min(count, ns);
    if (pre > 0) iss.post(p, lane, ring_addr, bar_addr, FUSED && fx.phase > 0);
    bool rest_posted = false;
    auto post_rest = [&]() {
        if (!rest_posted) {
            for (int j = 1; j < pre; j++) iss.post(p, lane, ring_addr + j * F::SLOT, bar_addr + j * 8, FUSED && fx.phase > 0);
            rest_posted = true;
        }
    };
    // The norm weights are read once per step, so they come from HBM; they do not depend on the kernel before.
    // Each CTA pulls its share of their lines into L2 now (a line or two), so that after the wait all CTAs read
    // them from L2.
    if (!FUSED && p.pf_mode >= 1 && p.x && p.do_norm && p.norm_w && threadIdx.x == 0) {
        const int lines = (p.K * 4 + 127) / 128;
        for (int ln = blockIdx.x; ln < lines; ln += gridDim.x)
            asm volatile("prefetch.global.L2 [%0];" ::"l"(reinterpret_cast<const char *>(p.norm_w) + (size_t)ln * 128));
    }
    // ... and so are the biases, which the last instructions of a row group would otherwise fetch from HBM
    if (!FUSED && p.pf_mode >= 2 && threadIdx.x == 32) {
        const int nsg = p.swiglu ? 2 : p.nseg;
        for (int i = 0; i < nsg; i++) {
            if (!p.seg[i].bias) continue;
            const int lines = (p.seg[i].n_rows * 4 + 127) / 128;
            for (int ln = blockIdx.x; ln < lines; ln += gridDim.x)
                asm volatile("prefetch.global.L2 [%0];" ::"l"(reinterpret_cast<const char *>(p.seg[i].bias) + (size_t)ln * 128));
        }
    }
    TRACE_MARK(1);
    if (FUSED && fx.phase > 0) fused_grid_wait(fx.target, &s_abort); // the phase before this one is complete everywhere
    else KQ_PDL_WAIT(); // activations (and the output buffer) belong to earlier kernels up to here
    if (FUSED && s_abort) {
        // a wait of this CTA gave up: take no further part, but let the copies already posted land first
        for (int j = 0; j < pre; j++) kq_mbar_wait(bar_addr + j * 8, uses[j] & 1, KQ_WAIT_LIMIT_NS);
        for (int j = 0; j < pre; j++) uses[j]++;
        return;
    }
    TRACE_MARK(2);
    if (p.x) {
        // Every CTA prepares the activations for itself: RMSNorm with the sum of squares in double,
        // then the Q8 quantiser, one warp per 256-block, PB blocks per warp in flight.  A row of up
        // to PB * WARPS blocks is read from L2 once and stays in registers for both steps.
        constexpr int PB = KQ_GEMV_PB;
        __shared__ double s_part[WARPS];
        __shared__ float s_scale[2];
        const bool in_regs = nb <= PB * WARPS;
        for (int m = 0; m < M; m++) {
            const float *xr = p.x + (int64_t)m * p.K;
            uint8_t *tq = smem + m * act_tok;
            if (p.do_norm && !in_regs) { // long rows: statistics in a pass of their own
                double ss = 0.0;
                for (int i = threadIdx.x * 4; i < p.K; i += WARPS * 128) {
                    const float4 v = ld_act4<FUSED>(xr + i);
                    ss += (double)v.x * v.x + (double)v.y * v.y + (double)v.z * v.z + (double)v.w * v.w;
                }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
                if (lane == 0) s_part[warp] = ss;
                __syncthreads();
                if (threadIdx.x == 0) {
                    double tsum = 0.0;
                    for (int i = 0; i < WARPS; i++) tsum += s_part[i];
                    s_scale[m] = 1.0f / sqrtf((float)(tsum / (double)p.K) + p.eps);
                }
                __syncthreads();
            }
            for (int base = 0; base < nb; base += PB * WARPS) {
                float4 va[PB], vb[PB], wa[PB], wb[PB];
#pragma unroll
                for (int i = 0; i < PB; i++) {
                    const int b = base + warp + i * WARPS;
                    va[i] = vb[i] = make_float4(0.f, 0.f, 0.f, 0.f);
                    wa[i] = wb[i] = make_float4(1.f, 1.f, 1.f, 1.f);
                    if (b < nb) {
                        const int o = b * 256 + lane * 8;
                        va[i] = ld_act4<FUSED>(xr + o);
                        vb[i] = ld_act4<FUSED>(xr + o + 4);
                        if (p.do_norm && p.norm_w) {
                            wa[i] = *reinterpret_cast<const float4 *>(p.norm_w + o);
                            wb[i] = *reinterpret_cast<const float4 *>(p.norm_w + o + 4);
                        }
                    }
                }
                TRACE_MARK(10);
                post_rest();
                TRACE_MARK(11);
                float scale = 1.0f;
                if (p.do_norm && in_regs) {
                    double ss = 0.0;
#pragma unroll
                    for (int i = 0; i < PB; i++)
                        ss += (double)va[i].x * va[i].x + (double)va[i].y * va[i].y + (double)va[i].z * va[i].z +
                              (double)va[i].w * va[i].w + (double)vb[i].x * vb[i].x + (double)vb[i].y * vb[i].y +
                              (double)vb[i].z * vb[i].z + (double)vb[i].w * vb[i].w;
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
                    if (m > 0) __syncthreads(); // the partials of the previous token have been read
                    if (lane == 0) s_part[warp] = ss;
                    __syncthreads();
                    double tsum = 0.0;
#pragma unroll
                    for (int i = 0; i < WARPS; i++) tsum += s_part[i];
                    scale = 1.0f / sqrtf((float)(tsum / (double)p.K) + p.eps);
                } else if (p.do_norm) {
                    scale = s_scale[m];
                }
                TRACE_MARK(12);
#pragma unroll
                for (int i = 0; i < PB; i++) {
                    const int b = base + warp + i * WARPS;
                    if (b >= nb) continue;
                    float v[8] = {va[i].x, va[i].y, va[i].z, va[i].w, vb[i].x, vb[i].y, vb[i].z, vb[i].w};
                    if (p.do_norm) {
                        const float g[8] = {wa[i].x, wa[i].y, wa[i].z, wa[i].w, wb[i].x, wb[i].y, wb[i].z, wb[i].w};
#pragma unroll
                        for (int k = 0; k < 8; k++) v[k] = v[k] * scale * g[k];
                    }
                    float amax = 0.f;
#pragma unroll
                    for (int k = 0; k < 8; k++) amax = fmaxf(amax, fabsf(v[k]));
                    amax = kq_warp_max(amax);
                    const float dq = kq_act_scale(amax), id = kq_act_inv(dq);
                    int c8[8], sum = 0;
#pragma unroll
                    for (int k = 0; k < 8; k++) {
                        c8[k] = kq_act_code(v[k], id);
                        sum += c8[k];
                    }
                    uint2 pk;
                    pk.x = (uint32_t)(c8[0] & 0xFF) | ((uint32_t)(c8[1] & 0xFF) << 8) | ((uint32_t)(c8[2] & 0xFF) << 16) |
                           ((uint32_t)(c8[3] & 0xFF) << 24);
                    pk.y = (uint32_t)(c8[4] & 0xFF) | ((uint32_t)(c8[5] & 0xFF) << 8) | ((uint32_t)(c8[6] & 0xFF) << 16) |
                           ((uint32_t)(c8[7] & 0xFF) << 24);
                    *reinterpret_cast<uint2 *>(tq + b * ACT_BLK + lane * 8) = pk;
                    sum += __shfl_xor_sync(0xffffffffu, sum, 1); // 16 elements
                    if (TYPE == B200_TYPE_Q4_K) {
                        sum += __shfl_xor_sync(0xffffffffu, sum, 2); // 32 elements
                        if ((lane & 3) == 0) reinterpret_cast<int16_t *>(tq + act_q)[b * 8 + (lane >> 2)] = (int16_t)sum;
                    } else {
                        if ((lane & 1) == 0) reinterpret_cast<int16_t *>(tq + act_q)[b * 16 + (lane >> 1)] = (int16_t)sum;
                    }
                    if (lane == 0) reinterpret_cast<float *>(tq + act_q + act_s)[b] = dq;
                }
            }
        }
    } else {
        for (int m = 0; m < M; m++) {
            uint8_t *tq = smem + m * act_tok;
            if (M > 2 && m >= p.m_actual) { // padding token: all-zero codes, sums and scales
                for (int i = threadIdx.x * 16; i < act_tok - tok_pad<TYPE, M>(); i += WARPS * 32 * 16)
                    *reinterpret_cast<int4 *>(tq + i) = make_int4(0, 0, 0, 0);
                continue;
            }
            const int4 *src = reinterpret_cast<const int4 *>(p.aq + (int64_t)m * p.a_ldk);
            const int16_t *b16 = p.abs16 + (int64_t)m * p.a_ldb * 16;
            const int n16 = nb * 16;
            // first wave of loads (codes, sums, scales) in flight together, behind the posting
            constexpr int NT = WARPS * 32;
            int4 c0 = make_int4(0, 0, 0, 0), c1 = c0, c2 = c0, c3 = c0, s0 = c0;
            float d0 = 0.f;
            const int i0 = threadIdx.x, i1 = threadIdx.x + NT, i2 = threadIdx.x + 2 * NT, i3 = threadIdx.x + 3 * NT;
            if (i0 < n16) c0 = src[i0];
            if (i1 < n16) c1 = src[i1];
            if (i2 < n16) c2 = src[i2]; // rows of up to 32768 codes in one round of loads
            if (i3 < n16) c3 = src[i3];
            if (i0 < nb * 2) s0 = reinterpret_cast<const int4 *>(b16)[i0]; // 8 sums of 16
            if (i0 < nb) d0 = p.ad[m * p.a_ldb + i0];
            post_rest();
            // 16 codes of scale group i % 16 of block i / 16
            auto put = [&](int i, const int4 &c) {
                if constexpr (TYPE == B200_TYPE_Q6_K && M > 4) { // [lane % 4][scale group][4 codes], see mma_units_q6
                    uint32_t *dst = reinterpret_cast<uint32_t *>(tq + (i >> 4) * ACT_BLK) + (i & 15);
                    dst[0] = (uint32_t)c.x;
                    dst[16] = (uint32_t)c.y;
                    dst[32] = (uint32_t)c.z;
                    dst[48] = (uint32_t)c.w;
                } else {
                    *reinterpret_cast<int4 *>(tq + (i >> 4) * ACT_BLK + (i & 15) * 16) = c;
                }
            };
            if (i0 < n16) put(i0, c0);
            if (i1 < n16) put(i1, c1);
            if (i2 < n16) put(i2, c2);
            if (i3 < n16) put(i3, c3);
            for (int i = threadIdx.x + 4 * NT; i < n16; i += NT) put(i, src[i]);
            for (int i = threadIdx.x; i < nb * 2; i += NT) {
                const int4 sv = i == i0 ? s0 : reinterpret_cast<const int4 *>(b16)[i];
                const int16_t *h = reinterpret_cast<const int16_t *>(&sv);
                if (TYPE == B200_TYPE_Q4_K) {
                    int16_t o4[4];
#pragma unroll
                    for (int k = 0; k < 4; k++) o4[k] = (int16_t)(h[2 * k] + h[2 * k + 1]);
                    *reinterpret_cast<uint2 *>(reinterpret_cast<int16_t *>(tq + act_q) + i * 4) = *reinterpret_cast<uint2 *>(o4);
                } else {
                    *reinterpret_cast<int4 *>(reinterpret_cast<int16_t *>(tq + act_q) + i * 8) = sv;
                }
            }
            for (int i = threadIdx.x; i < nb; i += NT)
                reinterpret_cast<float *>(tq + act_q + act_s)[i] = i == i0 ? d0 : p.ad[m * p.a_ldb + i];
        }
    }
    post_rest();
    __syncthreads();
    TRACE_MARK(3);
    if (count <= 0) return;
    if constexpr (M > 2 && TYPE == B200_TYPE_Q4_K) {
        mma_units<TYPE, M>(p, smem, act_tok, act_q, act_s, ring, ring_addr, bar_addr, iss, count, begin, unit, n_units, total,
                           &s_abort);
        return;
    }
    if constexpr (M > 4 && TYPE == B200_TYPE_Q6_K) {
        mma_units_q6<M>(p, smem, act_tok, act_q, act_s, ring, ring_addr, bar_addr, iss, count, begin, unit, n_units, total, &s_abort);
        return;
    }
    // Q6_K with 3 or 4 tokens takes the loop below: one lane per block against all staged tokens, the block
    // decoded once; rows x tokens = 16 partial sums per unit is what a line of the fix-up scratch holds
    static_assert(M <= 2 || TYPE == B200_TYPE_Q4_K || M > 4 || F::ROWS * M <= 16, "a unit's partial sums must fit one line of the fix-up scratch");

    float acc[M];
#pragma unroll
    for (int m = 0; m < M; m++) acc[m] = 0.f;
    int rg = begin / p.nsteps, ks = begin % p.nsteps;
#ifdef KQ_GEMV_TRACE
    unsigned long long tr_post = 0, tr_wait = 0;
#endif
    float pre_bias = 0.f, pre_res[M];
#pragma unroll
    for (int m = 0; m < M; m++) pre_res[m] = 0.f;
    for (int j = 0; j < count; j++) {
        const int slot = j % ns;
#ifdef KQ_GEMV_TRACE
        const long long tw0 = clock64();
#endif
        wait_slot(bar_addr + slot * 8, (uint32_t)(((FUSED ? uses[slot] : 0u) + j / ns) & 1), &s_abort);
#ifdef KQ_GEMV_TRACE
        tr_wait += (unsigned long long)(clock64() - tw0);
#endif
#ifdef KQ_GEMV_TRACE
        if (j == 0) TRACE_MARK(4);
#endif
        if (!p.swiglu && ks == 0 && t == 0) {
            // this warp will write the rows of this row group: fetch their bias and residual now, so that the
            // last instructions of the row group do not wait for a round trip to L2
            int seg, row0;
            locate<TYPE>(p, rg, seg, row0);
            const KqGemvSeg &sg = p.seg[seg];
            const int row = row0 + rs;
            pre_bias = 0.f;
#pragma unroll
            for (int m = 0; m < M; m++) pre_res[m] = 0.f;
            if (row < sg.n_rows) {
                if (sg.bias) pre_bias = sg.bias[row];
                if (p.residual)
#pragma unroll
                    for (int m = 0; m < M; m++)
                        if (M <= 2 || m < p.m_actual) pre_res[m] = ld_act1<FUSED>(p.residual + (int64_t)m * sg.ldy + row);
            }
        }
        const int blk = ks * F::KB + t;
        if (blk < nb) {
            const uint8_t *row = ring + (size_t)slot * F::SLOT + rs * F::PITCH;
            if (TYPE == B200_TYPE_Q4_K)
                block_q4k<M>(row + t * KQ_Q4K_BYTES, smem, act_tok, act_q, act_s, blk, acc);
            else
                block_q6k<M>(row, min(F::KB, nb - ks * F::KB), t, smem, act_tok, act_q, act_s, blk, acc);
        }
        // the slot has been read by every lane: hand it back to the copy engine for unit j + ns
        __syncwarp();
#ifdef KQ_GEMV_TRACE
        const long long tp0 = clock64();
#endif
        if (j + ns < count) iss.post(p, lane, ring_addr + slot * F::SLOT, bar_addr + slot * 8);
#ifdef KQ_GEMV_TRACE
        tr_post += (unsigned long long)(clock64() - tp0);
#endif
        const bool last_slice = ks == p.nsteps - 1, last_unit = j == count - 1;
        if (last_slice || last_unit) {
            // row totals: the LPR lanes of a row add up; afterwards the row's first lane has it
            float v[M];
#pragma unroll
            for (int m = 0; m < M; m++) {
                float x = acc[m];
#pragma unroll
                for (int o = 1; o < F::LPR; o <<= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
                v[m] = x;
                acc[m] = 0.f;
            }
            const int64_t rg_first = (int64_t)rg * p.nsteps;
            if (rg_first < begin) {
                // the head of this row group belongs to an earlier warp: publish the partial sums
                if (t == 0)
#pragma unroll
                    for (int m = 0; m < M; m++)
                        *(volatile unsigned long long *)&g_partials[pbase + unit][rs * M + m] =
                            (unsigned long long)__float_as_uint(v[m]) | (1ull << 32);
            } else {
                if (!last_slice) {
                    // This warp owns the row group but later warps hold its tail.  The LPR lanes of
                    // a row each wait for one of the following warps, then the row's first lane adds
                    // what they fetched in warp order.
                    const int64_t rg_last = rg_first + p.nsteps;
                    for (int base = unit + 1; base < n_units; base += F::LPR) {
                        const int b0 = unit_first(p, base);
                        if (b0 >= rg_last) break;
                        const int u2 = base + t;
                        bool mine = false;
                        if (u2 < n_units) {
                            const int b2 = unit_first(p, u2), e2 = unit_first(p, u2 + 1);
                            mine = b2 < rg_last && e2 > b2;
                        }
                        float got[M];
#pragma unroll
                        for (int m = 0; m < M; m++) {
                            got[m] = 0.f;
                            if (mine) {
                                volatile unsigned long long *e = &g_partials[pbase + u2][rs * M + m];
                                unsigned long long w = 0;
                                bool ok = false;
                                const uint64_t t0 = kq_globaltimer_ns();
                                while (true) {
                                    w = *e;
                                    ok = (w >> 32) != 0;
                                    if (ok || s_abort || kq_globaltimer_ns() - t0 > KQ_WAIT_LIMIT_NS) break;
                                    __nanosleep(64);
                                }
                                if (!ok && !s_abort) {
                                    s_abort = 1;
                                    atomicExch(&g_stream_error, 2);
                                }
                                got[m] = __uint_as_float((uint32_t)w);
                                *e = 0ull;
                            }
                        }
#pragma unroll
                        for (int m = 0; m < M; m++)
#pragma unroll
                            for (int o = 0; o < F::LPR; o++)
                                v[m] += __shfl_sync(0xffffffffu, got[m], rs * F::LPR + o);
                    }
                }
                int seg, row0;
                locate<TYPE>(p, rg, seg, row0);
                if (p.swiglu) {
#pragma unroll
                    for (int m = 0; m < M; m++) {
                        const float up = __shfl_down_sync(0xffffffffu, v[m], 16); // same row of the up matrix
                        const int row = row0 + rs;
                        if (t == 0 && rs < F::ROWS / 2 && row < p.seg[0].n_rows && (M <= 2 || m < p.m_actual)) {
                            float gt = v[m], ut = up;
                            if (p.seg[0].bias) gt += p.seg[0].bias[row];
                            if (p.seg[1].bias) ut += p.seg[1].bias[row];
                            p.seg[0].y[(int64_t)m * p.seg[0].ldy + row] = (gt / (1.0f + expf(-gt))) * ut;
                        }
                    }
                } else if (t == 0) {
                    const KqGemvSeg &sg = p.seg[seg];
                    const int row = row0 + rs;
                    if (row < sg.n_rows) {
#pragma unroll
                        for (int m = 0; m < M; m++) {
                            if (M > 2 && m >= p.m_actual) continue; // a padding token
                            float x = v[m];
                            if (sg.bias) x += pre_bias;
                            if (p.residual) x += pre_res[m];
                            sg.y[(int64_t)m * sg.ldy + row] = x;
                        }
                    }
                }
            }
        }
        if (++ks == p.nsteps) {
            ks = 0;
            rg++;
        }
    }
    if (!FUSED && M <= 2 && p.swiglu && p.e_q) {
        // Q8 of the SwiGLU values for the down projection.  This warp wrote the rows of the row groups whose
        // first K slice it holds; it adds their number to the counter of each 256-element block they lie in,
        // and the warp that completes a block quantises it (the values come back from L2).
        constexpr int RPB = 256 / (F::ROWS / 2); // row groups per block
        __threadfence(); // this lane's stores of y before the counts below
        __syncwarp();
        const int r_lo = (begin + p.nsteps - 1) / p.nsteps, r_hi = (end - 1) / p.nsteps;
        const int nbo = p.seg[0].n_rows / 256; // blocks of an output row
        for (int b = r_lo / RPB; r_lo <= r_hi && b <= r_hi / RPB; b++) {
            const int lo = max(r_lo, b * RPB), hi = min(r_hi, b * RPB + RPB - 1);
            int last = 0;
            if (lane == 0) last = (atomicAdd(&p.e_cnt[b], hi - lo + 1) + (hi - lo + 1) == RPB) ? 1 : 0;
            last = __shfl_sync(0xffffffffu, last, 0);
            if (!last) continue;
            __threadfence();
            if (lane == 0) p.e_cnt[b] = 0; // ready for the next launch
#pragma unroll
            for (int m = 0; m < M; m++) {
                const float *src = p.seg[0].y + (int64_t)m * p.seg[0].ldy + b * 256 + lane * 8;
                const float4 a0 = __ldcg(reinterpret_cast<const float4 *>(src)), a1 = __ldcg(reinterpret_cast<const float4 *>(src) + 1);
                const float v[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
                kq_quantize_block_warp(v, lane, p.e_q + (int64_t)m * p.seg[0].n_rows + b * 256, p.e_d + m * nbo + b,
                                       p.e_bs + ((int64_t)m * nbo + b) * 16);
            }
        }
    }
    if (FUSED)
#pragma unroll
        for (int sl = 0; sl < 4; sl++)
            if (sl < ns && count > sl) uses[sl] += (uint32_t)((count - sl + ns - 1) / ns);
#ifdef KQ_GEMV_TRACE
    TRACE_MARK(5);
    if (lane == 0 && s_trace < 32768u) g_trace_w[s_trace][warp & 15] = (unsigned long long)clock64();
    if (lane == 0 && s_trace < 32768u)
        g_trace_p[s_trace][warp & 15] = (tr_post & 0xFFFFFFull) | ((tr_wait & 0xFFFFFFull) << 24) | ((unsigned long long)count << 48);
    if (lane == 0 && s_trace < 32768u) {
        atomicMax(&g_trace[s_trace][6], (unsigned long long)clock64());
        atomicMax(&g_trace[s_trace][9], kq_globaltimer_ns());
    }
#endif
}

template <uint32_t TYPE, int M>
__global__ void __launch_bounds__(Fmt<TYPE>::WARPS * 32, Fmt<TYPE>::CTAS_PER_SM) gemv_block_kernel(const __grid_constant__ StreamParams p) {
    KQ_PDL_TRIGGER();
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ int s_abort;
    const FusedCtx none = {0, 0, 0, 0u};
    uint32_t uses[4] = {0u, 0u, 0u, 0u};
    stream_body<TYPE, M, false>(p, smem, s_abort, none, uses);
}

// One launch for a projection whose matrices are of both types (Q4_K attn_q / attn_k with a Q6_K attn_v):
// the first p4.n_cta CTAs stream the Q4_K rows, the rest the Q6_K rows, each part dealt over its own CTAs
// in proportion to its bytes, so both finish together and the second launch with its fixed cost is gone.
template <int M>
__global__ void __launch_bounds__(KQ_GEMV_WARPS * 32, 1) gemv_mixed_kernel(const __grid_constant__ StreamParams p4,
                                                                           const __grid_constant__ StreamParams p6) {
    KQ_PDL_TRIGGER();
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ int s_abort;
    const FusedCtx none = {0, 0, 0, 0u};
    uint32_t uses[4] = {0u, 0u, 0u, 0u};
    if ((int)blockIdx.x < p4.n_cta) stream_body<B200_TYPE_Q4_K, M, false>(p4, smem, s_abort, none, uses);
    else stream_body<B200_TYPE_Q6_K, M, false>(p6, smem, s_abort, none, uses);
}

struct FusedParams {
    StreamParams ph[3];
    uint32_t type[3];
    int32_t n_phase, act_bytes, ring_bytes;
};

template <int M>
__global__ void __launch_bounds__(KQ_GEMV_WARPS * 32, 1) gemv_fused_kernel(const __grid_constant__ FusedParams fp) {
    KQ_PDL_TRIGGER();
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ int s_abort;
    if (threadIdx.x == 0) s_abort = 0;
    __syncthreads();
    uint32_t uses[4] = {0u, 0u, 0u, 0u}; // completions of this warp's ring barriers so far
    for (int ph = 0; ph < fp.n_phase; ph++) {
        const FusedCtx fx = {fp.act_bytes, fp.ring_bytes, ph, (unsigned)ph * gridDim.x};
        if (fp.type[ph] == B200_TYPE_Q4_K) stream_body<B200_TYPE_Q4_K, M, true>(fp.ph[ph], smem, s_abort, fx, uses);
        else stream_body<B200_TYPE_Q6_K, M, true>(fp.ph[ph], smem, s_abort, fx, uses);
    }
    // the CTA that leaves last returns the barrier words to zero for the next launch
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned prev = atomicAdd(&g_fused_bar[1], 1u);
        if (prev == gridDim.x - 1) {
            g_fused_bar[0] = 0u;
            __threadfence();
            g_fused_bar[1] = 0u;
        }
    }
}

int env_int2(const char *name, int dflt) {
    const char *v = getenv(name);
    return v ? atoi(v) : dflt;
}

template <uint32_t TYPE>
void fill_params(StreamParams &p, const KqGemvSeg *segs, int nseg, const int8_t *q, const float *d, const int16_t *bs,
                 int64_t K, const float *residual, int swiglu_pairs, const KqActPrep *prep) {
    using F = Fmt<TYPE>;
    p = StreamParams{};
    const int rows_per_rg = swiglu_pairs ? F::ROWS / 2 : F::ROWS;
    int tot = 0;
    for (int i = 0; i < nseg; i++) {
        p.seg[i] = segs[i];
        if (!(swiglu_pairs && i == 1)) tot += (int)kq_div_up(segs[i].n_rows, rows_per_rg);
        p.rg_end[i] = tot;
    }
    p.nseg = swiglu_pairs ? 1 : nseg;
    p.n_rg = tot;
    p.nb = (int)(K / 256);
    p.K = (int)K;
    p.K_row = (int)K;
    p.ks0 = 0;
    p.a_ldk = (int)K;
    p.a_ldb = p.nb;
    p.nsteps = (int)kq_div_up(p.nb, F::KB);
    p.swiglu = swiglu_pairs;
    p.aq = q;
    p.ad = d;
    p.abs16 = bs;
    p.residual = residual;
    if (prep && prep->x) {
        p.x = prep->x;
        p.norm_w = prep->norm_w;
        p.eps = prep->eps;
        p.do_norm = prep->do_norm;
    }
}

// how the work items of a launch part are dealt to its n_units warps (StreamParams::uq, ur)
inline bool set_split(StreamParams &p, int n_units) {
    const int64_t total = (int64_t)p.n_rg * p.nsteps;
    if (total >= (1ll << 30) || n_units < 1) return false;
    p.uq = (int32_t)(total / n_units);
    p.ur = (int32_t)(total % n_units);
    return true;
}

// Tensor maps of the segments for the tiled-copy form of the ring (B200_GEMV_TMA=0 keeps one bulk copy per
// row).  Not used where a box would not start on a 128-byte boundary of the slot (Q6_K with fused gate / up).
template <uint32_t TYPE>
b200_status make_maps(StreamParams &p, int nseg_all) {
    using F = Fmt<TYPE>;
    static int on = -1;
    if (on < 0) on = env_int2("B200_GEMV_TMA", 1);
    static int pf = -1;
    if (pf < 0) pf = env_int2("B200_GEMV_PREFETCH", 2);
    p.pf_mode = pf;
    p.use_tma = 0;
    memset(p.map, 0, sizeof(p.map));
    const int box_rows = p.swiglu ? F::ROWS / 2 : F::ROWS;
    if (!on || (p.swiglu && ((box_rows * F::PITCH) & 127) != 0)) return B200_OK;
    const int64_t row_bytes = kq_device_row_bytes(TYPE, p.K_row);
    if (row_bytes % 16 != 0) return B200_OK;
    for (int i = 0; i < nseg_all; i++) {
        if (p.seg[i].expert_stride != 0 || ((uintptr_t)p.seg[i].W & 15) != 0) return B200_OK;
        const uint64_t dims[2] = {(uint64_t)(row_bytes / 8), (uint64_t)p.seg[i].n_rows};
        const uint64_t strides[1] = {(uint64_t)row_bytes};
        const uint32_t box[2] = {(uint32_t)(F::PITCH / 8), (uint32_t)box_rows};
        const b200_status rc = kq_tmap_encode(&p.map[i], 8, 2, p.seg[i].W, dims, strides, box, 0);
        if (rc != B200_OK) return rc;
    }
    p.use_tma = 1;
    return B200_OK;
}

// bytes of one token's staged activations (codes, sums, scales) for rows of nb blocks
inline int act_tok_bytes(uint32_t type, int nb, int M) {
    const int sums = type == B200_TYPE_Q4_K ? 16 : 32;
    return ((nb * ACT_BLK + 127) & ~127) + ((nb * sums + 127) & ~127) + ((nb * 4 + 127) & ~127) + (M > 2 ? 32 : 0);
}

template <uint32_t TYPE, int M>
b200_status launch_block(const KqGemvSeg *segs, int nseg, const int8_t *q, const float *d, const int16_t *bs,
                         int64_t K, const float *residual, int swiglu_pairs, const KqActPrep *prep, cudaStream_t st,
                         int m_actual = M, int64_t K_row = 0, int blk0 = 0, KqEmitQ8 *emit = nullptr) {
    using F = Fmt<TYPE>;
    StreamParams p;
    fill_params<TYPE>(p, segs, nseg, q, d, bs, K, residual, swiglu_pairs, prep);
    const bool emit_on = emit && emit->q && emit->d && emit->bs && emit->counters && M <= 2 && swiglu_pairs &&
                         segs[0].n_rows % 256 == 0 && segs[0].ldy % 4 == 0 && ((uintptr_t)segs[0].y & 15) == 0;
    if (emit_on) {
        p.e_q = emit->q;
        p.e_d = emit->d;
        p.e_bs = emit->bs;
        p.e_cnt = emit->counters;
    }
    if (K_row) { // a range of K: blocks blk0 .. blk0 + K / 256 of rows of K_row elements; q, d, bs point at the range
        if (blk0 % F::KB != 0 || (prep && prep->x)) return B200_ERR_INVALID;
        p.K_row = (int)K_row;
        p.ks0 = blk0 / F::KB;
        p.a_ldk = (int)K_row;
        p.a_ldb = (int)(K_row / 256);
    }
    {
        const b200_status rm = make_maps<TYPE>(p, nseg);
        if (rm != B200_OK) return rm;
    }
    const int sums = TYPE == B200_TYPE_Q4_K ? 16 : 32;
    const int act_tok = ((p.nb * ACT_BLK + 127) & ~127) + ((p.nb * sums + 127) & ~127) + ((p.nb * 4 + 127) & ~127) + tok_pad<TYPE, M>();
    p.m_actual = m_actual;
    constexpr int WARPS = F::WARPS;
    int cap = F::SMEM_CAP;
    if (M * act_tok + WARPS * F::SLOT + 1024 > cap) cap = 216 * 1024; // long rows: take the whole SM
    int ns = (cap - M * act_tok - WARPS * 8 * 8) / (WARPS * F::SLOT);
    if (ns > 4) ns = 4;
    ns = env_int2("B200_GEMV_NS", ns);
    if (ns < 1) return B200_ERR_UNSUPPORTED;
    p.ns = ns;
    const size_t smem = (size_t)M * act_tok + (size_t)WARPS * ns * F::SLOT + (size_t)WARPS * ns * 8;
    if (smem > 226 * 1024) return B200_ERR_UNSUPPORTED;
    int grid = kq_sm_count() * KQ_GEMV_GRIDMUL;
    if (grid * WARPS > MAX_UNITS) grid = MAX_UNITS / WARPS;
    const int64_t want = kq_div_up((int64_t)p.n_rg * p.nsteps, WARPS);
    if (want < grid) grid = (int)(want < 1 ? 1 : want);
    if (!set_split(p, grid * WARPS)) return B200_ERR_UNSUPPORTED;
    static bool attr_done[16]; // the attribute belongs to a (kernel, device) pair
    int dev = 0;
    KQ_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 16 || !attr_done[dev]) {
        KQ_CUDA(cudaFuncSetAttribute(gemv_block_kernel<TYPE, M>, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024));
        if (dev >= 0 && dev < 16) attr_done[dev] = true;
    }
    kq_launch(gemv_block_kernel<TYPE, M>, grid, WARPS * 32, smem, st, p);
    KQ_COUNT_LAUNCH();
    KQ_LAUNCH_CHECK();
    if (emit_on) emit->done = 1;
    return B200_OK;
}

// MT staged tokens (3 to 8) in one pass over the matrix.  Rows too long for the activations of MT tokens to sit
// in shared memory next to the ring go out as up to four launches over ranges of K, each adding to the output
// of the one before (one segment, no fused gate / up); B200_GEMV_KPARTS=0 refuses those instead.
template <uint32_t TYPE, int MT>
bool batch_fits(int nb) {
    using F = Fmt<TYPE>;
    const int sums = TYPE == B200_TYPE_Q4_K ? 16 : 32;
    const int act_tok = ((nb * ACT_BLK + 127) & ~127) + ((nb * sums + 127) & ~127) + ((nb * 4 + 127) & ~127) + tok_pad<TYPE, MT>();
    return (size_t)MT * act_tok + (size_t)F::WARPS * F::SLOT + (size_t)F::WARPS * 8 * 8 <= 216 * 1024;
}

template <uint32_t TYPE, int MT>
b200_status launch_parts(const KqGemvSeg *segs, int nseg, const int8_t *q, const float *d, const int16_t *bs, int64_t K,
                         const float *residual, int swiglu_pairs, cudaStream_t st, int m_actual) {
    using F = Fmt<TYPE>;
    const int nb = (int)(K / 256);
    if (batch_fits<TYPE, MT>(nb)) return launch_block<TYPE, MT>(segs, nseg, q, d, bs, K, residual, swiglu_pairs, nullptr, st, m_actual);
    if (nseg != 1 || swiglu_pairs || env_int2("B200_GEMV_KPARTS", 1) == 0) return B200_ERR_UNSUPPORTED;
    const int nsteps = (int)kq_div_up(nb, F::KB);
    for (int parts = 2; parts <= 4; parts++) {
        const int per = (int)kq_div_up(nsteps, parts) * F::KB; // blocks per range, whole K slices
        if (!batch_fits<TYPE, MT>(per)) continue;
        for (int b0 = 0, i = 0; b0 < nb; b0 += per, i++) {
            const int nbp = nb - b0 < per ? nb - b0 : per;
            KqGemvSeg sg = segs[0];
            if (i > 0) sg.bias = nullptr;
            const b200_status rc = launch_block<TYPE, MT>(&sg, 1, q + (int64_t)b0 * 256, d + b0, bs + (int64_t)b0 * 16, (int64_t)nbp * 256,
                                                          i == 0 ? residual : sg.y, 0, nullptr, st, m_actual, K, b0);
            if (rc != B200_OK) return i == 0 ? rc : B200_ERR_INVALID; // the output already holds the first ranges
        }
        return B200_OK;
    }
    return B200_ERR_UNSUPPORTED;
}

// ring depth and shared-memory bytes of one launch part; false when the row does not fit
template <uint32_t TYPE, int M>
bool plan_part(StreamParams &p, size_t &smem) {
    using F = Fmt<TYPE>;
    const int sums = TYPE == B200_TYPE_Q4_K ? 16 : 32;
    const int act_tok = ((p.nb * ACT_BLK + 127) & ~127) + ((p.nb * sums + 127) & ~127) + ((p.nb * 4 + 127) & ~127) + tok_pad<TYPE, M>();
    int cap = F::SMEM_CAP;
    if (M * act_tok + F::WARPS * F::SLOT + 1024 > cap) cap = 216 * 1024;
    int ns = (cap - M * act_tok - F::WARPS * 8 * 8) / (F::WARPS * F::SLOT);
    if (ns > 4) ns = 4;
    if (ns < 1) return false;
    p.ns = ns;
    smem = (size_t)M * act_tok + (size_t)F::WARPS * ns * F::SLOT + (size_t)F::WARPS * ns * 8;
    return smem <= 226 * 1024;
}

template <int M>
b200_status launch_mixed(const KqGemvSeg *s4, int n4, const KqGemvSeg *s6, int n6, const int8_t *q, const float *d,
                         const int16_t *bs, int64_t K, const KqActPrep *prep, cudaStream_t st, const float *residual = nullptr,
                         int swiglu_pairs = 0, KqEmitQ8 *emit = nullptr) {
    // n4 == 0 or n6 == 0: a projection of one type through the same kernel (all CTAs on that type)
    if (n4 + n6 < 1 || (swiglu_pairs && !((n4 == 2 && n6 == 0) || (n4 == 0 && n6 == 2)))) return B200_ERR_UNSUPPORTED;
    if (residual && n4 + n6 != 1) return B200_ERR_UNSUPPORTED;
    StreamParams p4 = {}, p6 = {};
    if (n4) fill_params<B200_TYPE_Q4_K>(p4, s4, n4, q, d, bs, K, residual, swiglu_pairs, prep);
    if (n6) fill_params<B200_TYPE_Q6_K>(p6, s6, n6, q, d, bs, K, residual, swiglu_pairs, prep);
    p4.m_actual = p6.m_actual = M;
    {
        b200_status rm = n4 ? make_maps<B200_TYPE_Q4_K>(p4, n4) : B200_OK;
        if (rm == B200_OK && n6) rm = make_maps<B200_TYPE_Q6_K>(p6, n6);
        if (rm != B200_OK) return rm;
    }
    size_t sm4 = 0, sm6 = 0;
    if ((n4 && !plan_part<B200_TYPE_Q4_K, M>(p4, sm4)) || (n6 && !plan_part<B200_TYPE_Q6_K, M>(p6, sm6))) return B200_ERR_UNSUPPORTED;
    int total = kq_sm_count();
    if (total * KQ_GEMV_WARPS > MAX_UNITS) total = MAX_UNITS / KQ_GEMV_WARPS;
    const int64_t want4 = n4 ? kq_div_up((int64_t)p4.n_rg * p4.nsteps, KQ_GEMV_WARPS) : 0;
    const int64_t want6 = n6 ? kq_div_up((int64_t)p6.n_rg * p6.nsteps, KQ_GEMV_WARPS) : 0;
    int c4 = 0, c6 = 0;
    if (n4 && n6) {
        double b4 = 0, b6 = 0;
        for (int i = 0; i < n4; i++) b4 += (double)s4[i].n_rows * kq_device_row_bytes(B200_TYPE_Q4_K, K);
        for (int i = 0; i < n6; i++) b6 += (double)s6[i].n_rows * kq_device_row_bytes(B200_TYPE_Q6_K, K);
        // a Q6_K CTA needs longer for its bytes than a Q4_K CTA (larger units, more arithmetic per weight, and at
        // these sizes a warp holds one or two units): its bytes count more when the CTAs are divided
        static int w6_pct = -1;
        if (w6_pct < 0) w6_pct = env_int2("B200_GEMV_MIX_W6", 225);
        b6 *= w6_pct / 100.0;
        c6 = (int)(total * b6 / (b4 + b6) + 0.5);
        if (c6 < 1) c6 = 1;
        if (c6 > total - 1) c6 = total - 1;
        c4 = total - c6;
    } else if (n4) {
        c4 = total;
    } else {
        c6 = total;
    }
    if (n4 && want4 < c4) c4 = (int)(want4 < 1 ? 1 : want4);
    if (n6 && want6 < c6) c6 = (int)(want6 < 1 ? 1 : want6);
    p4.cta0 = 0;
    p4.n_cta = c4; // 0: no CTA takes the Q4_K branch
    p6.cta0 = c4;
    p6.n_cta = c6;
    if ((n4 && !set_split(p4, c4 * KQ_GEMV_WARPS)) || (n6 && !set_split(p6, c6 * KQ_GEMV_WARPS))) return B200_ERR_UNSUPPORTED;
    StreamParams &pe = n4 ? p4 : p6; // where the fused gate / up lives, if any
    const KqGemvSeg *se = n4 ? s4 : s6;
    const bool emit_on = emit && emit->q && emit->d && emit->bs && emit->counters && swiglu_pairs && se[0].n_rows % 256 == 0 &&
                         se[0].ldy % 4 == 0 && ((uintptr_t)se[0].y & 15) == 0;
    if (emit_on) {
        pe.e_q = emit->q;
        pe.e_d = emit->d;
        pe.e_bs = emit->bs;
        pe.e_cnt = emit->counters;
    }
    const size_t smem = sm4 > sm6 ? sm4 : sm6;
    static bool attr_done[16];
    int dev = 0;
    KQ_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 16 || !attr_done[dev]) {
        KQ_CUDA(cudaFuncSetAttribute(gemv_mixed_kernel<M>, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024));
        if (dev >= 0 && dev < 16) attr_done[dev] = true;
    }
    kq_launch(gemv_mixed_kernel<M>, c4 + c6, KQ_GEMV_WARPS * 32, smem, st, p4, p6);
    KQ_COUNT_LAUNCH();
    KQ_LAUNCH_CHECK();
    if (emit_on) emit->done = 1;
    return B200_OK;
}

template <int M>
b200_status launch_fused(const FusedParams &fp, size_t smem, cudaStream_t st) {
    static bool attr_done[16];
    int dev = 0;
    KQ_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 16 || !attr_done[dev]) {
        KQ_CUDA(cudaFuncSetAttribute(gemv_fused_kernel<M>, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024));
        if (dev >= 0 && dev < 16) attr_done[dev] = true;
    }
    // one CTA per SM, all resident together: the phases meet at grid-wide barriers
    kq_launch(gemv_fused_kernel<M>, kq_sm_count(), KQ_GEMV_WARPS * 32, smem, st, fp);
    KQ_COUNT_LAUNCH();
    KQ_LAUNCH_CHECK();
    return B200_OK;
}

} // namespace

// Up to three dependent matmuls (each with the fused activation preparation) as phases of one
// launch.  Returns B200_ERR_UNSUPPORTED when the shapes do not fit; nothing has been launched then.
b200_status kq_launch_gemv_fused(const KqFusedPhase *ph, int n_phase, int M, cudaStream_t st) {
    if (n_phase < 2 || n_phase > 3 || M < 1 || M > 2) return B200_ERR_UNSUPPORTED;
    if (kq_sm_count() * KQ_GEMV_WARPS > MAX_UNITS) return B200_ERR_UNSUPPORTED;
    FusedParams fp = {};
    fp.n_phase = n_phase;
    int act = 0;
    for (int i = 0; i < n_phase; i++) {
        const KqFusedPhase &f = ph[i];
        if (f.nseg < 1 || f.nseg > 2 || f.K % 256 != 0 || !f.prep.x || ((uintptr_t)f.prep.x & 15) != 0) return B200_ERR_UNSUPPORTED;
        if (f.swiglu && f.nseg != 2) return B200_ERR_UNSUPPORTED;
        const uint32_t type = f.segs[0].type;
        if (type != B200_TYPE_Q4_K && type != B200_TYPE_Q6_K) return B200_ERR_UNSUPPORTED;
        for (int j = 0; j < f.nseg; j++)
            if (f.segs[j].type != type || ((uintptr_t)f.segs[j].W & 15) != 0) return B200_ERR_UNSUPPORTED;
        fp.type[i] = type;
        if (type == B200_TYPE_Q4_K)
            fill_params<B200_TYPE_Q4_K>(fp.ph[i], f.segs, f.nseg, nullptr, nullptr, nullptr, f.K, f.residual, f.swiglu, &f.prep);
        else
            fill_params<B200_TYPE_Q6_K>(fp.ph[i], f.segs, f.nseg, nullptr, nullptr, nullptr, f.K, f.residual, f.swiglu, &f.prep);
        fp.ph[i].m_actual = M;
        if (!set_split(fp.ph[i], kq_sm_count() * KQ_GEMV_WARPS)) return B200_ERR_UNSUPPORTED;
        const int a = M * act_tok_bytes(type, (int)(f.K / 256), M);
        if (a > act) act = a;
    }
    fp.act_bytes = (act + 127) & ~127;
    // every warp gets the same byte range for its ring in all phases: two Q4_K units, which also holds one Q6_K unit
    const int cap = 216 * 1024 - fp.act_bytes - KQ_GEMV_WARPS * 4 * 8;
    int ring = cap / KQ_GEMV_WARPS;
    const int want = 2 * Fmt<B200_TYPE_Q4_K>::SLOT;
    if (ring > want) ring = want;
    ring &= ~127;
    if (ring < Fmt<B200_TYPE_Q6_K>::SLOT) return B200_ERR_UNSUPPORTED;
    fp.ring_bytes = ring;
    const size_t smem = (size_t)fp.act_bytes + (size_t)KQ_GEMV_WARPS * ring + (size_t)KQ_GEMV_WARPS * 4 * 8;
    return M == 1 ? launch_fused<1>(fp, smem, st) : launch_fused<2>(fp, smem, st);
}

#ifdef KQ_GEMV_TRACE
extern "C" __attribute__((visibility("default"))) int kq_gemv_trace_fetch(unsigned long long *out, int max_rec) {
    unsigned int n = 0, zero = 0;
    cudaDeviceSynchronize();
    cudaMemcpyFromSymbol(&n, g_trace_n, sizeof(n));
    if ((int)n > max_rec) n = max_rec;
    if (n > 32768u) n = 32768u;
    if (out && n) cudaMemcpyFromSymbol(out, g_trace, sizeof(unsigned long long) * 16 * n);
    if (out && n) cudaMemcpyFromSymbol(out + 16 * (size_t)max_rec, g_trace_w, sizeof(unsigned long long) * 16 * n);
    if (out && n) cudaMemcpyFromSymbol(out + 32 * (size_t)max_rec, g_trace_p, sizeof(unsigned long long) * 16 * n);
    cudaMemcpyToSymbol(g_trace_n, &zero, sizeof(zero));
    return (int)n;
}
#endif
// Callers synchronise the device first.  After a wait gave up, a producer that was merely late may
// still have left flagged entries in the fix-up scratch (or arrivals at the phase barrier) that the
// next launch would take for its own: everything is returned to zero before the error is reported.
int kq_stream_error_fetch() {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_stream_error, sizeof(int)) != cudaSuccess) return -1;
    if (v) {
        void *p = nullptr;
        if (cudaGetSymbolAddress(&p, g_partials) == cudaSuccess) cudaMemset(p, 0, sizeof(g_partials));
        if (cudaGetSymbolAddress(&p, g_partials8) == cudaSuccess) cudaMemset(p, 0, sizeof(g_partials8));
        if (cudaGetSymbolAddress(&p, g_fused_bar) == cudaSuccess) cudaMemset(p, 0, sizeof(g_fused_bar));
        cudaMemcpyToSymbol(g_stream_error, &zero, sizeof(int));
    }
    return v;
}

// Launches the streaming kernel(s) for M <= 2; returns B200_ERR_UNSUPPORTED when the call does not
// fit (the caller then uses the plain kernel).  Segments of different types go out as one launch
// per type.
b200_status kq_launch_gemv_stream(const KqGemvSeg *segs, int nseg, const int8_t *q, const float *d,
                                  const int16_t *bs, int M, int64_t K, const float *residual, int swiglu_pairs,
                                  const KqActPrep *prep, cudaStream_t st, KqEmitQ8 *emit) {
    if (emit) emit->done = 0;
    if (M < 1 || M > 8 || K % 256 != 0 || env_int2("B200_GEMV_STREAM", 1) == 0) return B200_ERR_UNSUPPORTED;
    if (M > 2) {
        // 3..8 tokens: the tensor-core kernel, Q4_K only, on activations that are already quantised.
        // It stages 8 tokens when they fit in shared memory next to the ring, else 4 at a time (the
        // matrix is then streamed once per group of 4 tokens).
        if ((prep && prep->x) || env_int2("B200_GEMV_MMA", 1) == 0) return B200_ERR_UNSUPPORTED;
        bool all4 = true, all6 = true;
        for (int i = 0; i < nseg; i++) {
            if (((uintptr_t)segs[i].W & 15) != 0) return B200_ERR_UNSUPPORTED;
            all4 = all4 && segs[i].type == B200_TYPE_Q4_K;
            all6 = all6 && segs[i].type == B200_TYPE_Q6_K;
        }
        if ((((uintptr_t)q | (uintptr_t)bs) & 15) != 0 || ((uintptr_t)d & 3) != 0) return B200_ERR_UNSUPPORTED;
        if (all6 && !swiglu_pairs && env_int2("B200_GEMV_Q6_BATCH", 1)) {
            // Q6_K, 5 to 8 tokens: the tensor-core form, one pass over the matrix
            if (M > 4 && env_int2("B200_GEMV_Q6_MMA", 1)) {
                const b200_status rc = launch_parts<B200_TYPE_Q6_K, 8>(segs, nseg, q, d, bs, K, residual, 0, st, M);
                if (rc != B200_ERR_UNSUPPORTED) return rc;
            }
            // else the streaming kernel's dp4a form with four tokens staged, the matrix streamed once per group of four
            const int64_t nb6 = K / 256;
            for (int m0 = 0; m0 < M; m0 += 4) {
                KqGemvSeg sh[3];
                for (int i = 0; i < nseg; i++) {
                    sh[i] = segs[i];
                    sh[i].y = segs[i].y + (int64_t)m0 * segs[i].ldy;
                }
                const int mc = M - m0 < 4 ? M - m0 : 4;
                const b200_status rc = launch_parts<B200_TYPE_Q6_K, 4>(sh, nseg, q + (int64_t)m0 * K, d + m0 * nb6, bs + m0 * nb6 * 16, K,
                                                                       residual ? residual + (int64_t)m0 * segs[0].ldy : nullptr, 0, st, mc);
                if (rc != B200_OK) return m0 == 0 ? rc : B200_ERR_INVALID;
            }
            return B200_OK;
        }
        if (!all4) return B200_ERR_UNSUPPORTED;
        if (M > 4) {
            const b200_status rc = launch_parts<B200_TYPE_Q4_K, 8>(segs, nseg, q, d, bs, K, residual, swiglu_pairs, st, M);
            if (rc != B200_ERR_UNSUPPORTED) return rc;
        }
        const int64_t nb = K / 256;
        for (int m0 = 0; m0 < M; m0 += 4) {
            KqGemvSeg sh[3];
            for (int i = 0; i < nseg; i++) {
                sh[i] = segs[i];
                sh[i].y = segs[i].y + (int64_t)m0 * segs[i].ldy;
            }
            const int mc = M - m0 < 4 ? M - m0 : 4;
            const b200_status rc = launch_block<B200_TYPE_Q4_K, 4>(sh, nseg, q + (int64_t)m0 * K, d + m0 * nb, bs + m0 * nb * 16, K,
                                                                   residual ? residual + (int64_t)m0 * segs[0].ldy : nullptr,
                                                                   swiglu_pairs, nullptr, st, mc);
            if (rc != B200_OK) return m0 == 0 ? rc : B200_ERR_INVALID; // nothing written yet only for the first group
        }
        return B200_OK;
    }
    for (int i = 0; i < nseg; i++) {
        if (segs[i].type != B200_TYPE_Q4_K && segs[i].type != B200_TYPE_Q6_K) return B200_ERR_UNSUPPORTED;
        if (((uintptr_t)segs[i].W & 15) != 0) return B200_ERR_UNSUPPORTED;
    }
    if (!(prep && prep->x) && ((((uintptr_t)q | (uintptr_t)bs) & 15) != 0 || ((uintptr_t)d & 3) != 0)) return B200_ERR_UNSUPPORTED;
    if (prep && prep->x && ((uintptr_t)prep->x & 15) != 0) return B200_ERR_UNSUPPORTED;
    // B200_GEMV_ONE_KERNEL=1: every projection of 1 or 2 tokens through the two-type kernel, so that a decode step
    // alternates between two kernels' code only (this one and the attention) instead of four
    static int one_kernel = -1;
    if (one_kernel < 0) one_kernel = env_int2("B200_GEMV_ONE_KERNEL", 0);
    if (one_kernel) {
        KqGemvSeg s4[3], s6[3];
        int n4 = 0, n6 = 0;
        for (int i = 0; i < nseg; i++) (segs[i].type == B200_TYPE_Q4_K ? s4[n4++] : s6[n6++]) = segs[i];
        const b200_status rc = M == 1 ? launch_mixed<1>(s4, n4, s6, n6, q, d, bs, K, prep, st, residual, swiglu_pairs, emit)
                                      : launch_mixed<2>(s4, n4, s6, n6, q, d, bs, K, prep, st, residual, swiglu_pairs, emit);
        if (rc != B200_ERR_UNSUPPORTED) return rc;
    }
    if (!swiglu_pairs && !residual && env_int2("B200_GEMV_MIXED", 1)) {
        // matrices of both types in one projection: one launch with the CTAs divided between the types
        KqGemvSeg s4[3], s6[3];
        int n4 = 0, n6 = 0;
        for (int i = 0; i < nseg; i++) (segs[i].type == B200_TYPE_Q4_K ? s4[n4++] : s6[n6++]) = segs[i];
        if (n4 > 0 && n6 > 0) {
            const b200_status rc = M == 1 ? launch_mixed<1>(s4, n4, s6, n6, q, d, bs, K, prep, st)
                                          : launch_mixed<2>(s4, n4, s6, n6, q, d, bs, K, prep, st);
            if (rc != B200_ERR_UNSUPPORTED) return rc;
        }
    }
    for (uint32_t type : {(uint32_t)B200_TYPE_Q4_K, (uint32_t)B200_TYPE_Q6_K}) {
        KqGemvSeg sel[3];
        int n = 0;
        for (int i = 0; i < nseg; i++)
            if (segs[i].type == type) sel[n++] = segs[i];
        if (n == 0) continue;
        if (swiglu_pairs && n != 2) return B200_ERR_UNSUPPORTED;
        b200_status rc;
        if (type == B200_TYPE_Q4_K)
            rc = M == 1 ? launch_block<B200_TYPE_Q4_K, 1>(sel, n, q, d, bs, K, residual, swiglu_pairs, prep, st, 1, 0, 0, emit)
                        : launch_block<B200_TYPE_Q4_K, 2>(sel, n, q, d, bs, K, residual, swiglu_pairs, prep, st, 2, 0, 0, emit);
        else
            rc = M == 1 ? launch_block<B200_TYPE_Q6_K, 1>(sel, n, q, d, bs, K, residual, swiglu_pairs, prep, st, 1, 0, 0, emit)
                        : launch_block<B200_TYPE_Q6_K, 2>(sel, n, q, d, bs, K, residual, swiglu_pairs, prep, st, 2, 0, 0, emit);
        if (rc != B200_OK) return rc;
    }
    return B200_OK;
}
