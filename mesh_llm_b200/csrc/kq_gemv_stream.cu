// Decode GEMV for M <= 2 tokens, streaming form.
//
// The weight stream is the whole cost of a decode step, so this kernel is built around keeping
// enough of it in flight: every warp runs its own ring of shared-memory slots that are filled by
// bulk asynchronous copies (cp.async.bulk, the untiled TMA path) completing on mbarriers, and
// computes out of shared memory while later slices are still on their way.  Registers hold only
// the accumulators, so the bytes in flight per SM are set by the ring depth, not by occupancy.
//
// Work unit: 2 weight rows x 8 consecutive 256-blocks (2304 bytes of Q4_K, 3360 of Q6_K): one
// contiguous, 16-byte aligned run per row in both device layouts.  The (row pair, K slice) units
// of a matrix are laid end to end and cut into equal contiguous ranges, one per warp of a
// persistent grid ("stream-K"), so every SM streams the same number of bytes whatever N and K are.
// A row pair whose K range is cut between warps is finished by the warp that holds its first
// slice: the others publish their partial sums (they reach them at the start of their range), the
// owner adds them in warp order at the end of its own -- deterministic, no float atomics.
// Every wait in here (mbarrier or flag) is bounded and reports through an error word instead of
// hanging.
#include "kq_common.cuh"
#include "kq_lanes.cuh"

#include <stdlib.h>

namespace {

constexpr int WARPS = 16;          // warps per CTA, each with a private ring
constexpr int KB = 8;              // blocks per slice
constexpr int ROWS = 2;            // rows per unit
constexpr int MAX_UNITS = 160 * WARPS;
constexpr uint32_t SPIN_LIMIT = 1u << 16;

// cross-warp fix-up scratch: partial sums and ready flags, one line per warp of the grid
__device__ float g_partials[MAX_UNITS][ROWS * 2];
__device__ int g_flags[MAX_UNITS];
__device__ int g_stream_error; // 0 ok, 1 mbarrier wait gave up, 2 partial-sum wait gave up

struct StreamParams {
    KqGemvSeg seg[3];
    int32_t rg_end[3];
    int32_t nseg, n_rg, nb, K, nsteps, swiglu;
    int32_t ns;         // ring depth per warp
    int32_t slot_bytes; // bytes of one ring slot
    int32_t act_smem;   // activations staged in shared memory
    const int8_t *aq;
    const float *ad;
    const int16_t *abs16;
    const float *residual;
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

// bounded wait on a ring slot; after a first give-up the CTA stops waiting altogether
__device__ __forceinline__ void wait_slot(uint32_t bar, uint32_t parity, volatile int *abort_flag) {
    if (*abort_flag) return;
    for (uint32_t i = 0; i < SPIN_LIMIT; i++) {
        if (mbar_try_wait(bar, parity)) return;
        if (i > 64) __nanosleep(64);
    }
    *abort_flag = 1;
    atomicExch(&g_stream_error, 1);
}

struct RowPair {
    const uint8_t *w[ROWS]; // device rows
    int row[ROWS];          // row index inside the segment (for the epilogue)
    int seg;                // segment of row 0
    uint32_t type;
};

__device__ __forceinline__ RowPair locate(const StreamParams &p, int rg) {
    RowPair rp;
    int si = 0, rg0 = 0;
    if (p.nseg > 1 && rg >= p.rg_end[0]) { si = 1; rg0 = p.rg_end[0]; }
    if (p.nseg > 2 && rg >= p.rg_end[1]) { si = 2; rg0 = p.rg_end[1]; }
    rp.seg = si;
    rp.type = p.seg[si].type;
    const int64_t stride = kq_device_row_bytes(rp.type, p.K);
    if (p.swiglu) { // row 0 from the gate matrix, row 1 the same row of the up matrix
        rp.row[0] = rp.row[1] = rg;
        rp.w[0] = p.seg[0].W + (int64_t)rg * stride;
        rp.w[1] = p.seg[1].W + (int64_t)rg * stride;
    } else {
#pragma unroll
        for (int r = 0; r < ROWS; r++) {
            rp.row[r] = (rg - rg0) * ROWS + r;
            rp.w[r] = p.seg[si].W + (int64_t)min(rp.row[r], p.seg[si].n_rows - 1) * stride;
        }
    }
    return rp;
}

// lane 0: post the copies of slice `ks` of row group `rg` into ring slot `slot`
__device__ __forceinline__ void issue(const StreamParams &p, int rg, int ks, uint32_t slot_addr, uint32_t bar) {
    const RowPair rp = locate(p, rg);
    const int kb0 = ks * KB, kbn = min(KB, p.nb - kb0);
    uint32_t bytes;
    int64_t off;
    if (rp.type == B200_TYPE_Q4_K) {
        bytes = kbn * KQ_Q4K_BYTES;
        off = (int64_t)kb0 * KQ_Q4K_BYTES;
    } else {
        bytes = (uint32_t)kq_q6_group_bytes(kbn);
        off = (int64_t)ks * KQ_Q6_GROUP_BYTES;
    }
    mbar_expect_tx(bar, bytes * ROWS);
    const uint32_t pitch = p.slot_bytes / ROWS;
#pragma unroll
    for (int r = 0; r < ROWS; r++) bulk_g2s(slot_addr + r * pitch, rp.w[r] + off, bytes, bar);
}

template <int M>
__global__ void __launch_bounds__(WARPS * 32, 1) gemv_stream_kernel(const StreamParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ int s_abort;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int sub = lane >> 3, c = lane & 7;
    const int nb = p.nb;

    // ---- shared memory carve-up: [activations][rings][mbarriers]
    const int act_q = (M * p.K + 127) & ~127, act_d = (M * nb * 4 + 127) & ~127, act_s = (M * nb * 32 + 127) & ~127;
    const int act_bytes = p.act_smem ? act_q + act_d + act_s : 0;
    uint8_t *ring = smem + act_bytes + (size_t)warp * p.ns * p.slot_bytes;
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + act_bytes + (size_t)WARPS * p.ns * p.slot_bytes) + warp * p.ns;
    if (threadIdx.x == 0) s_abort = 0;
    if (lane == 0)
        for (int s = 0; s < p.ns; s++) mbar_init(smem_u32(&bars[s]), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    const int8_t *aq = p.aq;
    const float *ad = p.ad;
    const int16_t *abs16 = p.abs16;
    if (p.act_smem) {
        const int4 *src = reinterpret_cast<const int4 *>(p.aq);
        int4 *dst = reinterpret_cast<int4 *>(smem);
        for (int i = threadIdx.x; i < M * p.K / 16; i += blockDim.x) dst[i] = src[i];
        float *sd = reinterpret_cast<float *>(smem + act_q);
        for (int i = threadIdx.x; i < M * nb; i += blockDim.x) sd[i] = p.ad[i];
        int4 *ss = reinterpret_cast<int4 *>(smem + act_q + act_d);
        const int4 *sb = reinterpret_cast<const int4 *>(p.abs16);
        for (int i = threadIdx.x; i < M * nb * 2; i += blockDim.x) ss[i] = sb[i];
        aq = reinterpret_cast<const int8_t *>(smem);
        ad = sd;
        abs16 = reinterpret_cast<const int16_t *>(ss);
    }
    __syncthreads();

    // ---- this warp's contiguous range of (row group, slice) units
    const int unit = blockIdx.x * WARPS + warp, n_units = gridDim.x * WARPS;
    const int64_t total = (int64_t)p.n_rg * p.nsteps;
    const int64_t begin = total * unit / n_units, end = total * (unit + 1) / n_units;
    const int count = (int)(end - begin);
    if (count <= 0) return;
    const uint32_t ring_addr = smem_u32(ring), bar_addr = smem_u32(bars);
    const uint32_t pitch = p.slot_bytes / ROWS;

    if (lane == 0) {
        const int pre = min(count, p.ns);
        for (int j = 0; j < pre; j++) {
            const int64_t i = begin + j;
            issue(p, (int)(i / p.nsteps), (int)(i % p.nsteps), ring_addr + j * p.slot_bytes, bar_addr + j * 8);
        }
    }

    float acc[ROWS][M];
#pragma unroll
    for (int r = 0; r < ROWS; r++)
#pragma unroll
        for (int m = 0; m < M; m++) acc[r][m] = 0.f;

    int rg = (int)(begin / p.nsteps), ks = (int)(begin % p.nsteps);
    RowPair rp = locate(p, rg);
    for (int j = 0; j < count; j++) {
        const int slot = j % p.ns;
        wait_slot(bar_addr + slot * 8, (uint32_t)((j / p.ns) & 1), &s_abort);
        const uint8_t *sl = ring + (size_t)slot * p.slot_bytes;
        const int kb0 = ks * KB, kbn = min(KB, nb - kb0);
        if (rp.type == B200_TYPE_Q4_K) {
            const int e_lo = 64 * (c >> 1) + 16 * (c & 1);
#pragma unroll
            for (int half = 0; half < 2; half++) {
                const int bl = half * 4 + sub;
                if (bl < kbn) {
                    const int blk = kb0 + bl;
                    uint4 hdr[ROWS], w[ROWS];
#pragma unroll
                    for (int r = 0; r < ROWS; r++) {
                        const uint8_t *b = sl + r * pitch + bl * KQ_Q4K_BYTES;
                        hdr[r] = *reinterpret_cast<const uint4 *>(b);
                        w[r] = *reinterpret_cast<const uint4 *>(b + 16 + 16 * c);
                    }
                    Q4Scales sc[ROWS];
#pragma unroll
                    for (int r = 0; r < ROWS; r++) sc[r] = q4k_lane_scales(hdr[r], c);
#pragma unroll
                    for (int m = 0; m < M; m++) {
                        const int8_t *a = aq + (int64_t)m * p.K + blk * 256 + e_lo;
                        const int4 alo = *reinterpret_cast<const int4 *>(a);
                        const int4 ahi = *reinterpret_cast<const int4 *>(a + 32);
                        const float da = ad[m * nb + blk];
                        const int16_t *s16 = abs16 + ((int64_t)m * nb + blk) * 16 + (e_lo >> 4);
                        const int bsl = s16[0], bsh = s16[2];
#pragma unroll
                        for (int r = 0; r < ROWS; r++) {
                            int isum, msum;
                            q4k_lane_ints(w[r], sc[r], alo, ahi, bsl, bsh, isum, msum);
                            acc[r][m] = fmaf(sc[r].d * da, (float)isum, acc[r][m]);
                            acc[r][m] = fmaf(-(sc[r].dmin * da), (float)msum, acc[r][m]);
                        }
                    }
                }
            }
        } else {
            const int h = c >> 2, cc = c & 3, e_lo = 128 * h + 16 * cc;
#pragma unroll
            for (int half = 0; half < 2; half++) {
                const int bl = half * 4 + sub;
                if (bl < kbn) {
                    const int blk = kb0 + bl;
                    uint4 ql[ROWS], qh[ROWS];
                    int scl[ROWS], sch[ROWS];
                    float dw[ROWS];
#pragma unroll
                    for (int r = 0; r < ROWS; r++) {
                        const uint8_t *g = sl + r * pitch; // one group of kbn blocks
                        ql[r] = *reinterpret_cast<const uint4 *>(g + bl * 128 + 16 * c);
                        qh[r] = *reinterpret_cast<const uint4 *>(g + kbn * 128 + bl * 64 + 16 * (2 * h + (cc & 1)));
                        const int8_t *scp = reinterpret_cast<const int8_t *>(g + kbn * 192 + bl * 16);
                        scl[r] = scp[8 * h + cc];
                        sch[r] = scp[8 * h + 4 + cc];
                        dw[r] = kq_h2f(*reinterpret_cast<const uint16_t *>(g + kbn * 208 + bl * 2));
                    }
#pragma unroll
                    for (int m = 0; m < M; m++) {
                        const int8_t *a = aq + (int64_t)m * p.K + blk * 256 + e_lo;
                        const int4 alo = *reinterpret_cast<const int4 *>(a);
                        const int4 ahi = *reinterpret_cast<const int4 *>(a + 64);
                        const float da = ad[m * nb + blk];
                        const int16_t *s16 = abs16 + ((int64_t)m * nb + blk) * 16 + (e_lo >> 4);
                        const int bsl = s16[0], bsh = s16[4];
#pragma unroll
                        for (int r = 0; r < ROWS; r++) {
                            const int isum = q6k_lane_ints(ql[r], qh[r], cc, scl[r], sch[r], alo, ahi, bsl, bsh);
                            acc[r][m] = fmaf(dw[r] * da, (float)isum, acc[r][m]);
                        }
                    }
                }
            }
        }
        // the slot has been read by every lane: hand it back to the copy engine for unit j + ns
        __syncwarp();
        if (lane == 0 && j + p.ns < count) {
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            const int64_t i2 = begin + j + p.ns;
            issue(p, (int)(i2 / p.nsteps), (int)(i2 % p.nsteps), ring_addr + slot * p.slot_bytes, bar_addr + slot * 8);
        }

        // ---- end of this warp's share of the row group?
        const bool last_slice = ks == p.nsteps - 1, last_unit = j == count - 1;
        if (last_slice || last_unit) {
            // lane l < ROWS*M ends up holding element (r = l / M, m = l % M)
            float v = 0.f;
#pragma unroll
            for (int r = 0; r < ROWS; r++)
#pragma unroll
                for (int m = 0; m < M; m++) {
                    const float t = kq_warp_sum(acc[r][m]);
                    if (lane == r * M + m) v = t;
                    acc[r][m] = 0.f;
                }
            const int64_t rg_first = (int64_t)rg * p.nsteps;
            const bool has_first = rg_first >= begin;
            if (!has_first) {
                // the head of this row group belongs to an earlier warp: publish the partial sums
                if (lane < ROWS * M) g_partials[unit][lane] = v;
                __threadfence();
                __syncwarp();
                if (lane == 0) atomicExch(&g_flags[unit], 1);
            } else {
                if (!last_slice) {
                    // this warp owns the row group but later warps hold its tail: collect in order
                    const int64_t rg_last = rg_first + p.nsteps;
                    for (int u2 = unit + 1; u2 < n_units; u2++) {
                        const int64_t b2 = total * u2 / n_units, e2 = total * (u2 + 1) / n_units;
                        if (b2 >= rg_last) break;
                        if (e2 <= b2) continue;
                        bool ok = s_abort != 0;
                        for (uint32_t spin = 0; !ok && spin < SPIN_LIMIT; spin++) {
                            ok = *(volatile int *)&g_flags[u2] != 0;
                            if (!ok) __nanosleep(128);
                        }
                        if (!ok) {
                            s_abort = 1;
                            atomicExch(&g_stream_error, 2);
                        }
                        __threadfence();
                        if (lane < ROWS * M) v += *(volatile float *)&g_partials[u2][lane];
                        __syncwarp();
                        if (lane == 0) atomicExch(&g_flags[u2], 0);
                    }
                }
                // epilogue
                const KqGemvSeg &sg = p.seg[rp.seg];
                if (p.swiglu) {
                    const float up = __shfl_sync(0xffffffffu, v, min(lane + M, 31));
                    if (lane < M && rp.row[0] < p.seg[0].n_rows) {
                        float gt = v, ut = up;
                        if (p.seg[0].bias) gt += p.seg[0].bias[rp.row[0]];
                        if (p.seg[1].bias) ut += p.seg[1].bias[rp.row[0]];
                        p.seg[0].y[(int64_t)lane * p.seg[0].ldy + rp.row[0]] = (gt / (1.0f + expf(-gt))) * ut;
                    }
                } else if (lane < ROWS * M) {
                    const int r = lane / M, m = lane % M;
                    const int rw = r == 0 ? rp.row[0] : rp.row[1];
                    if (rw < sg.n_rows) {
                        if (sg.bias) v += sg.bias[rw];
                        if (p.residual) v += p.residual[(int64_t)m * sg.ldy + rw];
                        sg.y[(int64_t)m * sg.ldy + rw] = v;
                    }
                }
            }
        }
        if (++ks == p.nsteps) {
            ks = 0;
            rg++;
            if (j + 1 < count) rp = locate(p, rg);
        }
    }
}

// ================================================================================================
// Q4_K, one lane per 256-block.
//
// The form above spends about 4.5 lane-instructions per weight, most of them on per-chunk scale
// decoding, address arithmetic and nibble shifts, and that -- not memory -- is what limits it.
// Here a lane owns a whole block: the 8 six-bit scales and mins are unpacked once per block with a
// handful of word-wide logic ops, the high nibbles are used in place (x16, shifted out of the
// integer sum at the end), the min term is four dp2a, and the 64 dp4a of a block run as eight
// independent chains.  That is about 0.6 lane-instructions per weight.
//
// A warp takes 8 rows x 4 blocks per unit: lanes 4r..4r+3 hold row r, so a row sum needs two
// shuffles.  Shared-memory pitches are chosen so that neither the weight reads (144-byte blocks,
// 576-byte rows) nor the activation reads (blocks padded to 272 bytes) conflict on banks.
constexpr int Q4_ROWS = 8, Q4_KB = 4, Q4_PITCH = Q4_KB * KQ_Q4K_BYTES, Q4_SLOT = Q4_ROWS * Q4_PITCH;
constexpr int ACT_BLK = 272; // 256 codes + 16 bytes of padding
__device__ float g_partials4[MAX_UNITS][Q4_ROWS * 2];
__device__ int g_flags4[MAX_UNITS];

struct Rows8 {
    const uint8_t *w[Q4_ROWS];
    int row0;   // first row (inside the segment) of the group; swiglu: rows row0..row0+3 of both
    int seg;
};

__device__ __forceinline__ void locate8(const StreamParams &p, int rg, int &seg, int &row0) {
    int si = 0, rg0 = 0;
    if (p.nseg > 1 && rg >= p.rg_end[0]) { si = 1; rg0 = p.rg_end[0]; }
    if (p.nseg > 2 && rg >= p.rg_end[1]) { si = 2; rg0 = p.rg_end[1]; }
    seg = si;
    row0 = (rg - rg0) * (p.swiglu ? Q4_ROWS / 2 : Q4_ROWS);
}

// row slot rs of the group -> (matrix, row)
__device__ __forceinline__ const uint8_t *row_ptr8(const StreamParams &p, int seg, int row0, int rs, int64_t stride,
                                                   int &row) {
    if (p.swiglu) {
        row = row0 + (rs & 3);
        const KqGemvSeg &sg = p.seg[rs >> 2];
        return sg.W + (int64_t)min(row, sg.n_rows - 1) * stride;
    }
    row = row0 + rs;
    return p.seg[seg].W + (int64_t)min(row, p.seg[seg].n_rows - 1) * stride;
}

__device__ __forceinline__ void issue8(const StreamParams &p, int rg, int ks, uint32_t slot_addr, uint32_t bar) {
    int seg, row0;
    locate8(p, rg, seg, row0);
    const int kb0 = ks * Q4_KB, kbn = min(Q4_KB, p.nb - kb0);
    const uint32_t bytes = kbn * KQ_Q4K_BYTES;
    const int64_t stride = (int64_t)p.nb * KQ_Q4K_BYTES, off = (int64_t)kb0 * KQ_Q4K_BYTES;
    mbar_expect_tx(bar, bytes * Q4_ROWS);
#pragma unroll
    for (int rs = 0; rs < Q4_ROWS; rs++) {
        int row;
        const uint8_t *w = row_ptr8(p, seg, row0, rs, stride, row);
        bulk_g2s(slot_addr + rs * Q4_PITCH, w + off, bytes, bar);
    }
}

#define KQ_BYTE(w, k) (((w) >> (8 * (k))) & 0xFFu)

// unsigned bytes of a times signed bytes of b, accumulated into c
__device__ __forceinline__ int dp4a_us(uint32_t a, int b, int c) {
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

template <int M>
__global__ void __launch_bounds__(WARPS * 32, 1) gemv_q4k_block_kernel(const StreamParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ int s_abort;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int rs = lane >> 2, t = lane & 3;
    const int nb = p.nb;

    // ---- shared memory: [padded int8 codes][sums of 32 as int16 x 8][scales][rings][mbarriers]
    const int act_q = (nb * ACT_BLK + 127) & ~127, act_s = (nb * 16 + 127) & ~127, act_d = (nb * 4 + 127) & ~127;
    const int act_tok = act_q + act_s + act_d;
    uint8_t *ring = smem + M * act_tok + (size_t)warp * p.ns * Q4_SLOT;
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + M * act_tok + (size_t)WARPS * p.ns * Q4_SLOT) + warp * p.ns;
    if (threadIdx.x == 0) s_abort = 0;
    if (lane == 0)
        for (int s = 0; s < p.ns; s++) mbar_init(smem_u32(&bars[s]), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    for (int m = 0; m < M; m++) {
        uint8_t *tq = smem + m * act_tok;
        const int4 *src = reinterpret_cast<const int4 *>(p.aq + (int64_t)m * p.K);
        for (int i = threadIdx.x; i < nb * 16; i += blockDim.x)
            *reinterpret_cast<int4 *>(tq + (i >> 4) * ACT_BLK + (i & 15) * 16) = src[i];
        for (int i = threadIdx.x; i < nb * 8; i += blockDim.x) {
            const int16_t *b16 = p.abs16 + ((int64_t)m * nb * 16) + 2 * i;
            reinterpret_cast<int16_t *>(tq + act_q)[i] = (int16_t)(b16[0] + b16[1]);
        }
        for (int i = threadIdx.x; i < nb; i += blockDim.x)
            reinterpret_cast<float *>(tq + act_q + act_s)[i] = p.ad[m * nb + i];
    }
    __syncthreads();

    const int unit = blockIdx.x * WARPS + warp, n_units = gridDim.x * WARPS;
    const int64_t total = (int64_t)p.n_rg * p.nsteps;
    const int64_t begin = total * unit / n_units, end = total * (unit + 1) / n_units;
    const int count = (int)(end - begin);
    if (count <= 0) return;
    const uint32_t ring_addr = smem_u32(ring), bar_addr = smem_u32(bars);
    if (lane == 0) {
        const int pre = min(count, p.ns);
        for (int j = 0; j < pre; j++) {
            const int64_t i = begin + j;
            issue8(p, (int)(i / p.nsteps), (int)(i % p.nsteps), ring_addr + j * Q4_SLOT, bar_addr + j * 8);
        }
    }
    float acc[M];
#pragma unroll
    for (int m = 0; m < M; m++) acc[m] = 0.f;
    int rg = (int)(begin / p.nsteps), ks = (int)(begin % p.nsteps);
    for (int j = 0; j < count; j++) {
        const int slot = j % p.ns;
        wait_slot(bar_addr + slot * 8, (uint32_t)((j / p.ns) & 1), &s_abort);
        const int blk = ks * Q4_KB + t;
        if (blk < nb) {
            const uint8_t *b = ring + (size_t)slot * Q4_SLOT + rs * Q4_PITCH + t * KQ_Q4K_BYTES;
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
                const uint8_t *tq = smem + m * act_tok;
                const uint8_t *a = tq + blk * ACT_BLK;
                int s_even = 0, s_odd16 = 0;
#pragma unroll
                for (int g = 0; g < 4; g++) {
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
        __syncwarp();
        if (lane == 0 && j + p.ns < count) {
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            const int64_t i2 = begin + j + p.ns;
            issue8(p, (int)(i2 / p.nsteps), (int)(i2 % p.nsteps), ring_addr + slot * Q4_SLOT, bar_addr + slot * 8);
        }
        const bool last_slice = ks == p.nsteps - 1, last_unit = j == count - 1;
        if (last_slice || last_unit) {
            // row totals: lanes 4r..4r+3 hold row r; afterwards lane 4r has it
            float v[M];
#pragma unroll
            for (int m = 0; m < M; m++) {
                float x = acc[m];
                x += __shfl_xor_sync(0xffffffffu, x, 1);
                x += __shfl_xor_sync(0xffffffffu, x, 2);
                v[m] = x;
                acc[m] = 0.f;
            }
            const int64_t rg_first = (int64_t)rg * p.nsteps;
            const bool has_first = rg_first >= begin;
            if (!has_first) {
                if (t == 0)
#pragma unroll
                    for (int m = 0; m < M; m++) g_partials4[unit][rs * M + m] = v[m];
                __threadfence();
                __syncwarp();
                if (lane == 0) atomicExch(&g_flags4[unit], 1);
            } else {
                if (!last_slice) {
                    const int64_t rg_last = rg_first + p.nsteps;
                    for (int u2 = unit + 1; u2 < n_units; u2++) {
                        const int64_t b2 = total * u2 / n_units, e2 = total * (u2 + 1) / n_units;
                        if (b2 >= rg_last) break;
                        if (e2 <= b2) continue;
                        bool ok = s_abort != 0;
                        for (uint32_t spin = 0; !ok && spin < SPIN_LIMIT; spin++) {
                            ok = *(volatile int *)&g_flags4[u2] != 0;
                            if (!ok) __nanosleep(128);
                        }
                        if (!ok) {
                            s_abort = 1;
                            atomicExch(&g_stream_error, 2);
                        }
                        __threadfence();
#pragma unroll
                        for (int m = 0; m < M; m++) v[m] += *(volatile float *)&g_partials4[u2][rs * M + m];
                        __syncwarp();
                        if (lane == 0) atomicExch(&g_flags4[u2], 0);
                    }
                }
                int seg, row0;
                locate8(p, rg, seg, row0);
                if (p.swiglu) {
#pragma unroll
                    for (int m = 0; m < M; m++) {
                        const float up = __shfl_down_sync(0xffffffffu, v[m], 16);
                        const int row = row0 + rs;
                        if (t == 0 && rs < 4 && row < p.seg[0].n_rows) {
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
                            float x = v[m];
                            if (sg.bias) x += sg.bias[row];
                            if (p.residual) x += p.residual[(int64_t)m * sg.ldy + row];
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
}

int env_int2(const char *name, int dflt) {
    const char *v = getenv(name);
    return v ? atoi(v) : dflt;
}

} // namespace

int kq_stream_error_fetch() {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_stream_error, sizeof(int)) != cudaSuccess) return -1;
    if (v) cudaMemcpyToSymbol(g_stream_error, &zero, sizeof(int));
    return v;
}

// returns B200_ERR_UNSUPPORTED when the shape does not fit this kernel (caller uses the plain one)
b200_status kq_launch_gemv_stream(const KqGemvSeg *segs, int nseg, const int8_t *q, const float *d,
                                  const int16_t *bs, int M, int64_t K, const float *residual, int swiglu_pairs,
                                  cudaStream_t st) {
    if (M < 1 || M > 2 || env_int2("B200_GEMV_STREAM", 1) == 0) return B200_ERR_UNSUPPORTED;
    {
        bool all_q4 = true;
        for (int i = 0; i < nseg; i++) all_q4 &= segs[i].type == B200_TYPE_Q4_K && ((uintptr_t)segs[i].W & 15) == 0;
        if (all_q4 && env_int2("B200_GEMV_BLOCK", 1)) {
            StreamParams p = {};
            const int rows_per_rg = swiglu_pairs ? Q4_ROWS / 2 : Q4_ROWS;
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
            p.nsteps = (int)kq_div_up(p.nb, Q4_KB);
            p.swiglu = swiglu_pairs;
            p.aq = q;
            p.ad = d;
            p.abs16 = bs;
            p.residual = residual;
            const int act_tok = ((p.nb * ACT_BLK + 127) & ~127) + ((p.nb * 16 + 127) & ~127) + ((p.nb * 4 + 127) & ~127);
            const int cap = 216 * 1024;
            int ns = (cap - M * act_tok - WARPS * 8 * 8) / (WARPS * Q4_SLOT);
            ns = env_int2("B200_GEMV_NS", ns > 4 ? 4 : ns);
            if (ns >= 2) {
                p.ns = ns;
                const size_t smem = (size_t)M * act_tok + (size_t)WARPS * ns * Q4_SLOT + (size_t)WARPS * ns * 8;
                int grid = kq_sm_count();
                if (grid * WARPS > MAX_UNITS) grid = MAX_UNITS / WARPS;
                const int64_t want = kq_div_up((int64_t)p.n_rg * p.nsteps, WARPS);
                if (want < grid) grid = (int)(want < 1 ? 1 : want);
                auto kern = M == 1 ? gemv_q4k_block_kernel<1> : gemv_q4k_block_kernel<2>;
                static bool attr4[2] = {false, false};
                if (!attr4[M - 1]) {
                    KQ_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024));
                    attr4[M - 1] = true;
                }
                kern<<<grid, WARPS * 32, smem, st>>>(p);
                KQ_COUNT_LAUNCH();
                KQ_LAUNCH_CHECK();
                return B200_OK;
            }
        }
    }
    StreamParams p = {};
    int tot = 0;
    bool any_q6 = false;
    for (int i = 0; i < nseg; i++) {
        if (segs[i].type != B200_TYPE_Q4_K && segs[i].type != B200_TYPE_Q6_K) return B200_ERR_UNSUPPORTED;
        if (((uintptr_t)segs[i].W & 15) != 0) return B200_ERR_UNSUPPORTED;
        any_q6 |= segs[i].type == B200_TYPE_Q6_K;
        p.seg[i] = segs[i];
        if (swiglu_pairs) {
            if (i == 0) tot = segs[0].n_rows;
        } else {
            tot += (int)kq_div_up(segs[i].n_rows, ROWS);
        }
        p.rg_end[i] = tot;
    }
    p.nseg = swiglu_pairs ? 1 : nseg;
    p.n_rg = tot;
    p.nb = (int)(K / 256);
    p.K = (int)K;
    p.nsteps = (int)kq_div_up(p.nb, KB);
    p.swiglu = swiglu_pairs;
    p.aq = q;
    p.ad = d;
    p.abs16 = bs;
    p.residual = residual;
    p.slot_bytes = ROWS * (any_q6 ? 1792 : 1152); // per-row pitch: 8 blocks, rounded to 128
    const int smem_cap = 200 * 1024;
    const int act_bytes = ((M * p.K + 127) & ~127) + ((M * p.nb * 4 + 127) & ~127) + ((M * p.nb * 32 + 127) & ~127);
    p.act_smem = act_bytes <= 72 * 1024;
    const int avail = smem_cap - (p.act_smem ? act_bytes : 0) - WARPS * 8 * 8;
    int ns = avail / (WARPS * p.slot_bytes);
    ns = env_int2("B200_GEMV_NS", ns > 6 ? 6 : ns);
    if (ns < 2) return B200_ERR_UNSUPPORTED;
    p.ns = ns;
    const size_t smem = (size_t)(p.act_smem ? act_bytes : 0) + (size_t)WARPS * ns * p.slot_bytes + (size_t)WARPS * ns * 8;
    int grid = kq_sm_count();
    if (grid * WARPS > MAX_UNITS) grid = MAX_UNITS / WARPS;
    const int64_t total = (int64_t)p.n_rg * p.nsteps;
    const int64_t want = kq_div_up(total, WARPS);
    if (want < grid) grid = (int)(want < 1 ? 1 : want);
    auto kern = M == 1 ? gemv_stream_kernel<1> : gemv_stream_kernel<2>;
    static bool attr_done[2] = {false, false};
    if (!attr_done[M - 1]) {
        KQ_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_cap + 8192));
        attr_done[M - 1] = true;
    }
    kern<<<grid, WARPS * 32, smem, st>>>(p);
    KQ_COUNT_LAUNCH();
    KQ_LAUNCH_CHECK();
    return B200_OK;
}
