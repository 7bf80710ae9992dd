// Decode attention (one new token per sequence) as ONE launch per layer: RoPE of q and k, the
// store of the new K / V row into the cache (f16, or q8_0 / q4_0 rows), split-KV attention over the cache, and the combination
// of the splits by whichever CTA finishes last.  At batch 1 this op reads a few MB, so its cost is
// launches, round trips and dependent instruction chains, not bytes; the three kernels it replaces
// (rope + store, attention, combine) each paid a launch and a drain.  The work is cut fine -- one
// warp per (query head, 32 positions) -- because a thousand short warps finish sooner than a few
// hundred long ones.
#include "kq_common.cuh"
#include "kq_kvq.cuh"

#include <cuda.h> // CUtensorMap
#include <math.h>
#include <stdlib.h>
#include <string.h>

#include <map>
#include <tuple>

b200_status kq_tmap_encode(void *map128, int elem_bytes, int rank, const void *base, const uint64_t *dims,
                           const uint64_t *strides_bytes, const uint32_t *box, int swizzle128);

namespace {
#ifdef KQ_ATTN_TRACE
// debug build only: clock64 at the phase boundaries of the decode attention kernel, one record per CTA
// ([10]: block index, [11]: %globaltimer at the start); read with kq_attn_trace_fetch()
__device__ unsigned long long g_atr[8192][12];
__device__ unsigned int g_atr_n;
#define AT_MARK(i) do { if (threadIdx.x == 0 && s_tr < 8192u) g_atr[s_tr][i] = (unsigned long long)clock64(); } while (0)
#else
#define AT_MARK(i)
#endif

struct RopeTab {
    float inv_freq[64];
};

__device__ int g_attn_error; // set if the split counter misbehaves (never expected)

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

// grid (n_kv, n_split, n_seq), 4 * G warps: warp (ti, g) serves query head kh * G + g on rows
// ti*32 .. ti*32+31 of the CTA's current 128-row chunk.  The K and V rows of a chunk are brought
// into shared memory by tiled TMA copies out of the cache viewed as [seq][position][kv head][dim]:
// one box of 128 rows x 64 dims (128 bytes) per instruction, with the 128-byte swizzle, so that the
// per-lane 16-byte reads of K (lane = row) fall on distinct banks; the copies of the first chunk are
// issued before the kernel waits for its predecessor -- rows of earlier positions do not depend on
// it.  The row of the new position is computed here and overwrites its (stale) copy in the chunk.
// A quantised cache is fetched as one box of 128 raw rows per tensor (row bytes x 128, no swizzle)
// and decoded into the same swizzled f16 chunk, so the arithmetic below does not depend on the type.
constexpr int ROWS_PER_CTA = 128;

// byte offset of 16-byte chunk c of row r inside a 128-row x 128-byte box with the 128-byte swizzle
__device__ __forceinline__ int sw_off(int r, int c) { return r * 128 + ((c ^ (r & 7)) << 4); }
constexpr int BOX_BYTES = ROWS_PER_CTA * 128;
// address of the half at (row, dim) of a swizzled chunk made of HD/64 boxes
__device__ __forceinline__ uint8_t *sw_elem(uint8_t *base, int row, int dim) {
    const int byte = dim * 2, box = byte >> 7, off = byte & 127;
    return base + box * BOX_BYTES + sw_off(row, off >> 4) + (off & 15);
}

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
constexpr int QH_PITCH = 128 * 2 + 16; // bytes per row of the f16 copy of q: eight rows fall on eight bank groups

// MMA = false: 4 * G warps, warp (ti, g) serves query head g on rows ti*32 .. ti*32+31 of a chunk with scalar
// FMAs (lane = row).  MMA = true (head_dim 128, G <= 8): eight warps, one per head for everything that is per
// head; the first four compute: warp ti takes the same 32 rows for ALL
// G heads on the tensor cores: S = Q K^T as mma.m16n8k16 with the heads as the 16 rows of the tile (K
// fragments by ldmatrix out of the swizzled chunk), softmax on the accumulator fragments, and the values
// as O^T = V^T P^T, for which the probabilities are already in the B-fragment layout and V comes in by
// ldmatrix.trans -- dims are the rows of that product, so none of its tile is wasted.  q and the probabilities
// enter as hi + lo pairs of f16 (two MMAs each), K and V are f16 as stored, accumulation is f32: the result
// agrees with the f32 scalar form to rounding of the sums.
template <int HD, int G, bool MMA>
__global__ void __launch_bounds__(MMA ? 256 : 128 * G, MMA ? 2 : 1) attn_decode_kernel(const __grid_constant__ CUtensorMap kmap,
                                                              const __grid_constant__ CUtensorMap vmap,
                                                              const float *q, const float *k_new,
                                                              const float *v_new, __half *kc, __half *vc,
                                                              const int32_t *pos_dev, int pos_val, int n_head, int n_kv,
                                                              int64_t seq_stride, int n_split, int unit_chunk, float scale,
                                                              int neox, RopeTab tab, float *out, float *part_o,
                                                              float *part_ml, int *counters, KqKvTypes kvt) {
    KQ_PDL_TRIGGER();
#ifdef KQ_ATTN_TRACE
    __shared__ unsigned int s_tr;
    if (threadIdx.x == 0) {
        s_tr = atomicAdd(&g_atr_n, 1u);
        if (s_tr < 8192u) {
            g_atr[s_tr][10] = ((unsigned long long)blockIdx.x << 40) | ((unsigned long long)blockIdx.y << 20) | blockIdx.z;
            g_atr[s_tr][11] = kq_globaltimer_ns();
        }
    }
    __syncthreads();
#endif
    AT_MARK(0);
    // the copy engine's descriptors: fetched while the position is being read
    if (threadIdx.x == 0) asm volatile("prefetch.tensormap [%0];" ::"l"(&kmap) : "memory");
    if (threadIdx.x == 32) asm volatile("prefetch.tensormap [%0];" ::"l"(&vmap) : "memory");
    constexpr int DPL = HD / 32, HALF = HD / 2, NBOX = HD / 64, NT = MMA ? 256 : 128 * G;
    static_assert(!MMA || (HD == 128 && G <= 8), "the tensor-core form is built for head_dim 128 and up to 8 heads per KV head");
    extern __shared__ __align__(1024) uint8_t dsm_raw[];
    uint8_t *dsm = dsm_raw + ((1024u - (smem_u32(dsm_raw) & 1023u)) & 1023u); // swizzled boxes start on 1 KB
    uint8_t *k_s = dsm, *v_s = dsm + NBOX * BOX_BYTES;
    float (*o_s)[G][HD] = reinterpret_cast<float (*)[G][HD]>(dsm + 2 * NBOX * BOX_BYTES); // [4][G][HD]
    const bool kq = kvt.k != KQ_KV_F16, vq = kvt.v != KQ_KV_F16;
    const int k_row = kq_kv_row_bytes(kvt.k, HD), v_row = kq_kv_row_bytes(kvt.v, HD);
    uint8_t *kraw_s = dsm + 2 * NBOX * BOX_BYTES + 4 * G * HD * (int)sizeof(float); // raw rows of a quantised chunk
    uint8_t *vraw_s = kraw_s + (kq ? ROWS_PER_CTA * k_row : 0);
    __shared__ float q_s[G][HD];
    __shared__ __align__(16) uint8_t qh_s[MMA ? 2 * 16 * QH_PITCH : 16]; // MMA: q as f16 hi + lo parts, 16 rows each (rows >= G zero)
    __shared__ float p_s[4 * G][32];
    __shared__ float ml_s[4][G][2];
    __shared__ float w_s[G][64];
    __shared__ uint64_t bar;
    __shared__ int s_last, s_abort;
    const int kh = blockIdx.x, split = blockIdx.y, seq = blockIdx.z;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = MMA ? 0 : warp % G, ti = MMA ? warp : warp / G;
    __half *kbase = kc + seq * seq_stride + (int64_t)kh * HD;
    __half *vbase = vc + seq * seq_stride + (int64_t)kh * HD;
    const int pos = pos_dev ? *pos_dev : pos_val; // written before this step started; first used after the early copy request
    const int64_t pstride = (int64_t)n_kv * HD;
    const int64_t cache_row0 = seq * (seq_stride / HD) + kh; // row index of (seq, position 0, kh) in a quantised cache
    const uint32_t bar_a = smem_u32(&bar);
    if (threadIdx.x == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar_a), "r"(1));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        s_abort = 0;
    }
    // thread 0: request the 128-row chunk that starts at position cb (whole boxes always: rows past the context
    // arrive as zeros, rows not yet written are never read)
    auto issue_chunk = [&](int cb) {
        const int tx = (kq ? ROWS_PER_CTA * k_row : NBOX * BOX_BYTES) + (vq ? ROWS_PER_CTA * v_row : NBOX * BOX_BYTES);
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar_a), "r"(tx) : "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        if (kq)
            asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];" ::"r"(
                             smem_u32(kraw_s)),
                         "l"(&kmap), "r"(0), "r"(kh), "r"(cb), "r"(seq), "r"(bar_a)
                         : "memory");
        if (vq)
            asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];" ::"r"(
                             smem_u32(vraw_s)),
                         "l"(&vmap), "r"(0), "r"(kh), "r"(cb), "r"(seq), "r"(bar_a)
                         : "memory");
#pragma unroll
        for (int bx = 0; bx < NBOX; bx++) {
            if (!kq)
                asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];" ::"r"(
                                 smem_u32(k_s + bx * BOX_BYTES)),
                             "l"(&kmap), "r"(64 * bx), "r"(kh), "r"(cb), "r"(seq), "r"(bar_a)
                             : "memory");
            if (!vq)
                asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];" ::"r"(
                                 smem_u32(v_s + bx * BOX_BYTES)),
                             "l"(&vmap), "r"(64 * bx), "r"(kh), "r"(cb), "r"(seq), "r"(bar_a)
                             : "memory");
        }
    };
    // unit_chunk: the launcher knows that every slice is one 128-row chunk (one slice per 128 positions), so the
    // chunk's rows are known without the position and their copy goes out while the position is still on its way
    if (unit_chunk && threadIdx.x == 0) issue_chunk(split * ROWS_PER_CTA);
    AT_MARK(1); // chunk copy requested
    const int L = pos + 1;
    int chunk = (L + n_split - 1) / n_split;
    chunk = (chunk + ROWS_PER_CTA - 1) / ROWS_PER_CTA * ROWS_PER_CTA;
    const int p_begin = split * chunk, p_end = min(L, p_begin + chunk);
    __syncthreads();
    AT_MARK(2); // position known, barrier
    uint32_t phase = 0;
    bool early_done = unit_chunk != 0;
    if (early_done && (chunk != ROWS_PER_CTA || p_begin >= p_end)) {
        // not what the launcher promised: let the early copy land, report, and go on without it
        if (threadIdx.x == 0) {
            kq_mbar_wait(bar_a, phase, KQ_WAIT_LIMIT_NS);
            atomicExch(&g_attn_error, 3);
        }
        __syncthreads();
        phase ^= 1;
        early_done = false;
    }

    float m = -INFINITY, l = 0.f, o[DPL]; // MMA: m and l belong to head lane / 4 (all four lanes of a quad hold them)
#pragma unroll
    for (int i = 0; i < DPL; i++) o[i] = 0.f;
    float oacc[MMA ? 8 : 1][4]; // MMA: O^T tiles: rows = dims 16 mt + lane/4 (+8), columns = heads 2 (lane%4), +1
#pragma unroll
    for (int i = 0; i < (MMA ? 8 : 1); i++) oacc[i][0] = oacc[i][1] = oacc[i][2] = oacc[i][3] = 0.f;
    bool first = true;
    // rotation factors of this lane's frequencies (lane, lane + 32, ..): they need the position only, so they are
    // worked out before the dependency wait
    constexpr int NF = HALF / 32;
    float rc[NF], rs[NF];
#pragma unroll
    for (int u = 0; u < NF; u++) {
        const float ang = (float)pos * tab.inv_freq[lane + 32 * u];
        rc[u] = cosf(ang);
        rs[u] = sinf(ang);
    }
    // MMA form, f16 cache: the new position's k and v rows are fetched and rotated next to q (warps KW and VW), parked
    // in shared memory (each lane reads back what it wrote), and put over the stale copy of that row once the
    // chunk has landed
    constexpr int KW = G % 8, VW = (G + 1) % 8;
    __shared__ __half new_s[2][HD];
    bool new_in_regs = false;
    for (int cb = p_begin; cb < p_end || first; cb += ROWS_PER_CTA) {
        const int ccnt = max(0, min(ROWS_PER_CTA, p_end - cb));
        const bool has_new = pos >= cb && pos < cb + ccnt;
        if (ccnt > 0 && threadIdx.x == 0 && !early_done) issue_chunk(cb);
        early_done = false;
        if (first) {
            if (MMA) { // rows of the q tile that no head fills must be zero: cleared while the projection still runs
                for (int i = threadIdx.x; i < 2 * 16 * QH_PITCH / 16; i += NT) reinterpret_cast<uint4 *>(qh_s)[i] = make_uint4(0, 0, 0, 0);
                __syncthreads();
            }
            KQ_PDL_WAIT(); // q, k_new, v_new come from the projection that precedes this kernel
            AT_MARK(3); // dependency wait over
            for (int gg = MMA ? warp : g; gg < (MMA ? G : g + 1); gg += 8) {
                if (!MMA && ti != 0) break;
#pragma unroll
                for (int u = 0; u < NF; u++) { // query head gg, rotated and pre-scaled
                    const int f = lane + 32 * u;
                    const float c = rc[u], sn = rs[u];
                    const int i0 = neox ? f : 2 * f, i1 = neox ? f + HALF : 2 * f + 1;
                    const float *qv = q + ((int64_t)seq * n_head + kh * G + gg) * HD;
                    const float a = qv[i0], b = qv[i1];
                    const float r0 = (a * c - b * sn) * scale, r1 = (a * sn + b * c) * scale;
                    if (MMA) { // q = hi + lo with both parts in f16: the products lose nothing of the f32 value that matters
                        const __half h0 = __float2half_rn(r0), h1 = __float2half_rn(r1);
                        *reinterpret_cast<__half *>(qh_s + gg * QH_PITCH + i0 * 2) = h0;
                        *reinterpret_cast<__half *>(qh_s + gg * QH_PITCH + i1 * 2) = h1;
                        *reinterpret_cast<__half *>(qh_s + (16 + gg) * QH_PITCH + i0 * 2) = __float2half_rn(r0 - __half2float(h0));
                        *reinterpret_cast<__half *>(qh_s + (16 + gg) * QH_PITCH + i1 * 2) = __float2half_rn(r1 - __half2float(h1));
                    } else {
                        q_s[gg][i0] = r0;
                        q_s[gg][i1] = r1;
                    }
                }
            }
            if (MMA && has_new && !kq && !vq) {
                new_in_regs = true;
                if (warp == KW) {
                    const float *kv = k_new + ((int64_t)seq * n_kv + kh) * HD;
#pragma unroll
                    for (int u = 0; u < NF; u++) {
                        const int f = lane + 32 * u;
                        const int i0 = neox ? f : 2 * f, i1 = neox ? f + HALF : 2 * f + 1;
                        const float a = kv[i0], b = kv[i1];
                        const __half r0 = __float2half_rn(a * rc[u] - b * rs[u]), r1 = __float2half_rn(a * rs[u] + b * rc[u]);
                        new_s[0][i0] = r0;
                        new_s[0][i1] = r1;
                        kbase[pos * pstride + i0] = r0;
                        kbase[pos * pstride + i1] = r1;
                    }
                }
                if (warp == VW) {
                    const float *vv = v_new + ((int64_t)seq * n_kv + kh) * HD;
#pragma unroll
                    for (int u = 0; u < HD / 32; u++) {
                        const __half r = __float2half_rn(vv[lane + 32 * u]);
                        new_s[1][lane + 32 * u] = r;
                        vbase[pos * pstride + lane + 32 * u] = r;
                    }
                }
            }
            first = false;
        }
        AT_MARK(4); // q (and the new row) staged
        if (ccnt == 0) break; // CTA-uniform: an empty slice only takes part in the combine below
        { // bounded wait for the chunk
            const bool ok = s_abort ? false : kq_mbar_wait(bar_a, phase, KQ_WAIT_LIMIT_NS);
            if (!ok && !s_abort) {
                s_abort = 1;
                atomicExch(&g_attn_error, 2);
            }
            phase ^= 1;
        }
        AT_MARK(5); // chunk arrived
        // raw rows of a quantised chunk -> the swizzled f16 chunk (the new position's row comes from below)
        if (kq || vq) {
            const int rr_new = has_new ? pos - cb : -1;
            const int kper = kvt.k == KQ_KV_Q8_0 ? HD / 16 : HD / 32, vper = kvt.v == KQ_KV_Q8_0 ? HD / 16 : HD / 32;
            const int kn = kq ? ccnt * kper : 0, vn = vq ? ccnt * vper : 0;
            for (int i = threadIdx.x; i < kn + vn; i += NT) {
                const bool is_k = i < kn;
                const int j = is_k ? i : i - kn, per = is_k ? kper : vper, type = is_k ? kvt.k : kvt.v;
                const int row = j / per, c = j % per;
                if (row == rr_new) continue;
                const uint8_t *src = is_k ? kraw_s + row * k_row : vraw_s + row * v_row;
                uint8_t *dst = is_k ? k_s : v_s;
                if (type == KQ_KV_Q8_0) {
                    uint4 t2[2];
                    kq_kv_decode16_q8_0(src, HD, c, t2);
                    *reinterpret_cast<uint4 *>(sw_elem(dst, row, c * 16)) = t2[0];
                    *reinterpret_cast<uint4 *>(sw_elem(dst, row, c * 16 + 8)) = t2[1];
                } else {
                    uint4 t4[4];
                    kq_kv_decode32_q4_0(src, HD, c, t4);
#pragma unroll
                    for (int u = 0; u < 4; u++) *reinterpret_cast<uint4 *>(sw_elem(dst, row, c * 32 + 8 * u)) = t4[u];
                }
            }
        }
        if (has_new && (kq || vq)) {
            // the new rows of a quantised cache: one warp per block of 32 values
            const float *kv = k_new + ((int64_t)seq * n_kv + kh) * HD;
            const float *vv = v_new + ((int64_t)seq * n_kv + kh) * HD;
            const int rr = pos - cb;
            constexpr int NB = HD / 32;
            for (int u = warp; u < 2 * NB; u += NT / 32) {
                const bool is_k = u < NB;
                const int blk = is_k ? u : u - NB, e = blk * 32 + lane;
                if (is_k ? !kq : !vq) continue;
                float val;
                if (is_k) {
                    const int f = neox ? e % HALF : e / 2;
                    const float ang = (float)pos * tab.inv_freq[f];
                    const float c = cosf(ang), sn = sinf(ang);
                    const float a = kv[neox ? f : 2 * f], b = kv[neox ? f + HALF : 2 * f + 1];
                    const bool first_of_pair = neox ? e < HALF : !(e & 1);
                    val = first_of_pair ? a * c - b * sn : a * sn + b * c;
                } else {
                    val = vv[e];
                }
                const int type = is_k ? kvt.k : kvt.v;
                uint8_t *grow = reinterpret_cast<uint8_t *>(is_k ? kc : vc) +
                                (cache_row0 + (int64_t)pos * n_kv) * (is_k ? k_row : v_row);
                const __half r = kq_kv_store_block(type, val, grow, HD, blk, lane);
                *reinterpret_cast<__half *>(sw_elem(is_k ? k_s : v_s, rr, e)) = r;
            }
        }
        if (has_new && new_in_regs) {
            const int rr = pos - cb;
            if (warp == KW) {
#pragma unroll
                for (int u = 0; u < NF; u++) {
                    const int f = lane + 32 * u;
                    const int i0 = neox ? f : 2 * f, i1 = neox ? f + HALF : 2 * f + 1;
                    *reinterpret_cast<__half *>(sw_elem(k_s, rr, i0)) = new_s[0][i0];
                    *reinterpret_cast<__half *>(sw_elem(k_s, rr, i1)) = new_s[0][i1];
                }
            }
            if (warp == VW) {
#pragma unroll
                for (int u = 0; u < HD / 32; u++) *reinterpret_cast<__half *>(sw_elem(v_s, rr, lane + 32 * u)) = new_s[1][lane + 32 * u];
            }
            new_in_regs = false;
        } else if (has_new) {
            // rotate k, round k and v to f16 as later steps will read them, into the cache and over the
            // stale copy of that row in the chunk
            const float *kv = k_new + ((int64_t)seq * n_kv + kh) * HD;
            const float *vv = v_new + ((int64_t)seq * n_kv + kh) * HD;
            const int rr = pos - cb;
            for (int f = threadIdx.x; f < (kq ? 0 : HALF); f += NT) {
                const float ang = (float)pos * tab.inv_freq[f];
                const float c = cosf(ang), sn = sinf(ang);
                const int i0 = neox ? f : 2 * f, i1 = neox ? f + HALF : 2 * f + 1;
                const float a = kv[i0], b = kv[i1];
                const __half r0 = __float2half_rn(a * c - b * sn), r1 = __float2half_rn(a * sn + b * c);
                *reinterpret_cast<__half *>(sw_elem(k_s, rr, i0)) = r0;
                *reinterpret_cast<__half *>(sw_elem(k_s, rr, i1)) = r1;
                kbase[pos * pstride + i0] = r0;
                kbase[pos * pstride + i1] = r1;
            }
            for (int i = threadIdx.x; i < (vq ? 0 : HD); i += NT) {
                const __half r = __float2half_rn(vv[i]);
                *reinterpret_cast<__half *>(sw_elem(v_s, rr, i)) = r;
                vbase[pos * pstride + i] = r;
            }
        }
        __syncthreads();
        // this warp's tile: rows ti*32 .. +31 of the chunk
        const int cnt = max(0, min(32, ccnt - ti * 32));
        if constexpr (MMA) {
            if (cnt > 0 && warp < 4) {
                const int t4 = lane & 3, kb = ti * 32;
                if (cnt < 32) { // rows of the tile past the context may hold anything: their values must not reach the MMA
                    for (int i = lane; i < (32 - cnt) * 16; i += 32) {
                        const int r = kb + cnt + (i >> 4), c = i & 15;
                        *reinterpret_cast<uint4 *>(v_s + (c >> 3) * BOX_BYTES + r * 128 + ((c & 7) << 4)) = make_uint4(0, 0, 0, 0);
                    }
                    __syncwarp();
                }
                const uint32_t qh = smem_u32(qh_s), ks = smem_u32(k_s), vs = smem_u32(v_s);
                float sacc[4][4];
#pragma unroll
                for (int nt = 0; nt < 4; nt++) sacc[nt][0] = sacc[nt][1] = sacc[nt][2] = sacc[nt][3] = 0.f;
#pragma unroll
                for (int kk = 0; kk < 8; kk++) { // 16 dims per step
                    uint32_t qa[4], ql[4];
                    const uint32_t qoff = ((lane & 7) + ((lane >> 3) & 1) * 8) * QH_PITCH + (16 * kk + (lane >> 4) * 8) * 2;
                    ldsm_x4(qh + qoff, qa[0], qa[1], qa[2], qa[3]);
                    ldsm_x4(qh + 16 * QH_PITCH + qoff, ql[0], ql[1], ql[2], ql[3]);
#pragma unroll
                    for (int np = 0; np < 2; np++) { // two key tiles of 8 per load
                        const int key = kb + 8 * (2 * np + (lane >> 4)) + (lane & 7), c = 2 * kk + ((lane >> 3) & 1);
                        uint32_t r0, r1, r2, r3;
                        ldsm_x4(ks + (c >> 3) * BOX_BYTES + sw_off(key, c & 7), r0, r1, r2, r3);
                        mma_f16(sacc[2 * np], qa, r0, r1);
                        mma_f16(sacc[2 * np + 1], qa, r2, r3);
                        mma_f16(sacc[2 * np], ql, r0, r1);
                        mma_f16(sacc[2 * np + 1], ql, r2, r3);
                    }
                }
                // softmax of head g4 over this tile's keys (this thread: keys 8 nt + 2 t4, +1)
                float mt = -INFINITY;
#pragma unroll
                for (int nt = 0; nt < 4; nt++)
#pragma unroll
                    for (int j = 0; j < 2; j++) {
                        if (8 * nt + 2 * t4 + j >= cnt) sacc[nt][j] = -INFINITY;
                        mt = fmaxf(mt, sacc[nt][j]);
                    }
                mt = fmaxf(mt, __shfl_xor_sync(0xffffffffu, mt, 1));
                mt = fmaxf(mt, __shfl_xor_sync(0xffffffffu, mt, 2));
                const float mn = fmaxf(m, mt); // cnt > 0: at least key 0 is finite
                const float alpha = (m == -INFINITY) ? 0.f : expf(m - mn);
                float rs = 0.f;
                uint32_t pb[4], pl[4]; // probabilities as f16 pairs, hi and lo parts: the B fragments of O^T = V^T P^T
#pragma unroll
                for (int nt = 0; nt < 4; nt++) {
                    const float p0 = expf(sacc[nt][0] - mn), p1 = expf(sacc[nt][1] - mn); // exp(-inf) = 0 for masked keys
                    rs += p0 + p1;
                    const __half2 hi = __floats2half2_rn(p0, p1);
                    const float2 back = __half22float2(hi);
                    pb[nt] = *reinterpret_cast<const uint32_t *>(&hi);
                    pl[nt] = pack_h2(p0 - back.x, p1 - back.y);
                }
                rs += __shfl_xor_sync(0xffffffffu, rs, 1);
                rs += __shfl_xor_sync(0xffffffffu, rs, 2);
                l = l * alpha + rs;
                m = mn;
                // this thread's accumulator columns are heads 2 t4 and 2 t4 + 1: their factors sit in other quads
                const float a0 = __shfl_sync(0xffffffffu, alpha, (2 * t4) * 4), a1 = __shfl_sync(0xffffffffu, alpha, (2 * t4 + 1) * 4);
#pragma unroll
                for (int mt8 = 0; mt8 < 8; mt8++) {
                    oacc[mt8][0] *= a0;
                    oacc[mt8][1] *= a1;
                    oacc[mt8][2] *= a0;
                    oacc[mt8][3] *= a1;
                }
#pragma unroll
                for (int ks2 = 0; ks2 < 2; ks2++) { // 16 keys per step
                    const int key = kb + 16 * ks2 + ((lane >> 4) & 1) * 8 + (lane & 7);
#pragma unroll
                    for (int mt8 = 0; mt8 < 8; mt8++) { // 16 dims per tile
                        const int c = 2 * mt8 + ((lane >> 3) & 1);
                        uint32_t va[4];
                        ldsm_x4_t(vs + (c >> 3) * BOX_BYTES + sw_off(key, c & 7), va[0], va[1], va[2], va[3]);
                        mma_f16(oacc[mt8], va, pb[2 * ks2], pb[2 * ks2 + 1]);
                        mma_f16(oacc[mt8], va, pl[2 * ks2], pl[2 * ks2 + 1]);
                    }
                }
            }
        } else if (cnt > 0) {
            const bool valid = lane < cnt;
            float sc = 0.f;
            if (valid) {
                const int kr_row = ti * 32 + lane;
#pragma unroll
                for (int c8 = 0; c8 < HD / 8; c8++) {
                    const uint4 raw = *reinterpret_cast<const uint4 *>(k_s + (c8 >> 3) * BOX_BYTES + sw_off(kr_row, c8 & 7));
                    const __half2 *h2 = reinterpret_cast<const __half2 *>(&raw);
                    const float2 f0 = __half22float2(h2[0]), f1 = __half22float2(h2[1]), f2 = __half22float2(h2[2]),
                                 f3 = __half22float2(h2[3]);
                    const float4 qa = *reinterpret_cast<const float4 *>(&q_s[g][c8 * 8]);
                    const float4 qb = *reinterpret_cast<const float4 *>(&q_s[g][c8 * 8 + 4]);
                    sc = fmaf(qa.x, f0.x, sc); sc = fmaf(qa.y, f0.y, sc); sc = fmaf(qa.z, f1.x, sc); sc = fmaf(qa.w, f1.y, sc);
                    sc = fmaf(qb.x, f2.x, sc); sc = fmaf(qb.y, f2.y, sc); sc = fmaf(qb.z, f3.x, sc); sc = fmaf(qb.w, f3.y, sc);
                }
            }
            const float sv = valid ? sc : -INFINITY;
            const float mt = kq_warp_max(sv);
            const float mn = fmaxf(m, mt);
            const float alpha = (m == -INFINITY) ? 0.f : expf(m - mn);
            const float pv = valid ? expf(sv - mn) : 0.f;
            l = l * alpha + kq_warp_sum(pv);
            m = mn;
#pragma unroll
            for (int i = 0; i < DPL; i++) o[i] *= alpha;
            p_s[warp][lane] = pv;
            __syncwarp();
            for (int j = 0; j < cnt; j++) {
                const __half *vr = reinterpret_cast<const __half *>(sw_elem(v_s, ti * 32 + j, lane * DPL));
                const float pj = p_s[warp][j];
                if (DPL == 4) {
                    const uint2 raw = *reinterpret_cast<const uint2 *>(vr);
                    const __half2 *h2 = reinterpret_cast<const __half2 *>(&raw);
                    const float2 a = __half22float2(h2[0]), b = __half22float2(h2[1]);
                    o[0] = fmaf(pj, a.x, o[0]); o[1] = fmaf(pj, a.y, o[1]); o[2] = fmaf(pj, b.x, o[2]); o[3] = fmaf(pj, b.y, o[3]);
                } else {
#pragma unroll
                    for (int i = 0; i < DPL; i++) o[i] = fmaf(pj, __half2float(vr[i]), o[i]);
                }
            }
        }
        __syncthreads(); // the chunk may be overwritten by the next one
    }

    AT_MARK(6); // products, softmax, values done
    // combine the 4 tiles of each head inside the CTA (tile order)
    if constexpr (MMA) {
        const int g4 = lane >> 2, t4 = lane & 3;
        if (warp < 4) {
#pragma unroll
        for (int mt8 = 0; mt8 < 8; mt8++)
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const int hh = 2 * t4 + (j & 1), dim = 16 * mt8 + g4 + (j >> 1) * 8;
                if (hh < G) o_s[ti][hh][dim] = oacc[mt8][j];
            }
        if (t4 == 0 && g4 < G) {
            ml_s[ti][g4][0] = m;
            ml_s[ti][g4][1] = l;
        }
        }
    } else {
#pragma unroll
        for (int i = 0; i < DPL; i++) o_s[ti][g][lane * DPL + i] = o[i];
        if (lane == 0) {
            ml_s[ti][g][0] = m;
            ml_s[ti][g][1] = l;
        }
    }
    __syncthreads();
    // one warp per head from here on: warp g of the G * 4 (ti == 0), or the four warps taking heads in turn
    for (int g = MMA ? warp : (ti == 0 ? warp % G : G); g < G; g += MMA ? 8 : G) {
    const int head = kh * G + g;
    {
        float mm = -INFINITY;
        for (int w = 0; w < 4; w++) mm = fmaxf(mm, ml_s[w][g][0]);
        float acc[DPL], ll = 0.f;
#pragma unroll
        for (int i = 0; i < DPL; i++) acc[i] = 0.f;
        for (int w = 0; w < 4; w++) {
            const float mw = ml_s[w][g][0];
            const float wgt = (mw == -INFINITY) ? 0.f : expf(mw - mm);
#pragma unroll
            for (int i = 0; i < DPL; i++) acc[i] += wgt * o_s[w][g][lane * DPL + i];
            ll += wgt * ml_s[w][g][1];
        }
        if (n_split == 1) {
#pragma unroll
            for (int i = 0; i < DPL; i++) out[((int64_t)seq * n_head + head) * HD + lane * DPL + i] = acc[i] / ll;
        } else {
            const int64_t pi = ((int64_t)seq * n_head + head) * n_split + split;
#pragma unroll
            for (int i = 0; i < DPL; i++) part_o[pi * HD + lane * DPL + i] = acc[i];
            if (lane == 0) {
                part_ml[pi * 2] = mm;
                part_ml[pi * 2 + 1] = ll;
            }
        }
    }
    }
    AT_MARK(7); // CTA combine done, partial results written
    if (n_split == 1) return;
    // the CTA that finishes last combines the splits of its G heads (in split order) and re-arms
    // the counter for the next launch
    // the CTA's partial results are ordered before its arrival by the barrier and one thread's fence (fences are
    // cumulative), and the arrival before the last CTA's reads by that thread's second fence and the barrier
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        const int prev = atomicAdd(&counters[seq * n_kv + kh], 1);
        if (prev < 0 || prev >= n_split) atomicExch(&g_attn_error, 1);
        s_last = prev == n_split - 1;
        __threadfence();
    }
    __syncthreads();
    AT_MARK(8); // arrival counted
    if (!s_last) return;
    for (int g = MMA ? warp : (ti == 0 ? warp % G : G); g < G; g += MMA ? 8 : G) {
        const int head = kh * G + g;
        // splits were written by other SMs: read them through L2 (ld.cg).  Lane sp (and sp + 32) holds split sp's
        // maximum and sum; the head's maximum and the weighted sum of sums are warp reductions in a fixed order
        float m_sp[2], l_sp[2], mm = -INFINITY;
#pragma unroll
        for (int u = 0; u < 2; u++) {
            const int sp = lane + 32 * u;
            m_sp[u] = -INFINITY;
            l_sp[u] = 0.f;
            if (sp < n_split) {
                const int64_t e = (((int64_t)seq * n_head + head) * n_split + sp) * 2;
                m_sp[u] = __ldcg(&part_ml[e]);
                l_sp[u] = __ldcg(&part_ml[e + 1]);
            }
        }
        // the first round of the partial outputs goes out before the weights are worked out
        const float *po = part_o + (((int64_t)seq * n_head + head) * n_split) * HD + lane * DPL;
        constexpr int RND = 24; // splits whose loads are in flight together (context up to 3072 in one round)
        float t[RND][DPL];
#pragma unroll
        for (int u = 0; u < RND; u++)
#pragma unroll
            for (int i = 0; i < DPL; i++) t[u][i] = u < n_split ? __ldcg(po + (int64_t)u * HD + i) : 0.f;
        mm = fmaxf(m_sp[0], m_sp[1]);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mm = fmaxf(mm, __shfl_xor_sync(0xffffffffu, mm, o));
        float ll = 0.f;
#pragma unroll
        for (int u = 0; u < 2; u++) {
            const float wgt = (m_sp[u] == -INFINITY) ? 0.f : expf(m_sp[u] - mm);
            const int sp = lane + 32 * u;
            if (sp < n_split) w_s[g][sp] = wgt;
            ll += wgt * l_sp[u];
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ll += __shfl_xor_sync(0xffffffffu, ll, o);
        __syncwarp();
        float acc[DPL];
#pragma unroll
        for (int i = 0; i < DPL; i++) acc[i] = 0.f;
        for (int s0 = 0; s0 < n_split; s0 += RND) {
            if (s0 > 0) {
#pragma unroll
                for (int u = 0; u < RND; u++)
#pragma unroll
                    for (int i = 0; i < DPL; i++) t[u][i] = s0 + u < n_split ? __ldcg(po + (int64_t)(s0 + u) * HD + i) : 0.f;
            }
#pragma unroll
            for (int u = 0; u < RND; u++)
                if (s0 + u < n_split)
#pragma unroll
                    for (int i = 0; i < DPL; i++) acc[i] += w_s[g][s0 + u] * t[u][i];
        }
#pragma unroll
        for (int i = 0; i < DPL; i++) out[((int64_t)seq * n_head + head) * HD + lane * DPL + i] = acc[i] / ll;
    }
    __syncthreads();
    if (threadIdx.x == 0) counters[seq * n_kv + kh] = 0;
    AT_MARK(9); // last CTA: merge of the slices done
}

template <int HD>
b200_status launch_g(int G, dim3 grid, cudaStream_t st, const CUtensorMap &kmap, const CUtensorMap &vmap, const float *q,
                     const float *k, const float *v, __half *kc, __half *vc, const int32_t *pos_dev, int pos, int n_head,
                     int n_kv, int64_t seq_stride, int n_split, int unit_chunk, float scale, int neox, const RopeTab &tab, float *out,
                     float *po, float *pml, int *counters, KqKvTypes kvt) {
    const size_t raw = (kvt.k != KQ_KV_F16 ? ROWS_PER_CTA * kq_kv_row_bytes(kvt.k, HD) : 0) +
                       (kvt.v != KQ_KV_F16 ? ROWS_PER_CTA * kq_kv_row_bytes(kvt.v, HD) : 0);
    const size_t smem = 2 * (HD / 64) * BOX_BYTES + (size_t)4 * G * HD * sizeof(float) + raw + 1024; // + room to align to 1 KB
    // head_dim 128: the tensor-core form (eight warps per CTA); B200_ATTN_DECODE_MMA=0 keeps the scalar one
    static int use_mma = -1;
    if (use_mma < 0) {
        const char *e = getenv("B200_ATTN_DECODE_MMA");
        use_mma = !(e && e[0] == '0');
    }
#define KQ_AD(GG)                                                                                              \
    if constexpr (HD == 128) {                                                                                 \
        if (use_mma) {                                                                                         \
            if (smem > 48 * 1024)                                                                              \
                cudaFuncSetAttribute(attn_decode_kernel<HD, GG, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            kq_launch(attn_decode_kernel<HD, GG, true>, grid, 256, smem, st, kmap, vmap, q, k, v, kc, vc, pos_dev, pos, n_head,  \
                      n_kv, seq_stride, n_split, unit_chunk, scale, neox, tab, out, po, pml, counters, kvt);                 \
            break;                                                                                             \
        }                                                                                                      \
    }                                                                                                          \
    if (smem > 48 * 1024)                                                                                      \
        cudaFuncSetAttribute(attn_decode_kernel<HD, GG, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);    \
    kq_launch(attn_decode_kernel<HD, GG, false>, grid, 128 * GG, smem, st, kmap, vmap, q, k, v, kc, vc, pos_dev, pos, n_head, n_kv, \
              seq_stride, n_split, unit_chunk, scale, neox, tab, out, po, pml, counters, kvt)
    switch (G) {
    case 1: KQ_AD(1); break;
    case 2: KQ_AD(2); break;
    case 4: KQ_AD(4); break;
    case 5: KQ_AD(5); break;
    case 8: KQ_AD(8); break;
    default: kq_set_error("attention: %d query heads per KV head not supported", G); return B200_ERR_UNSUPPORTED;
    }
#undef KQ_AD
    KQ_COUNT_LAUNCH();
    KQ_LAUNCH_CHECK();
    return B200_OK;
}

// tensor maps of a cache, made once per (base, shape, types).  f16: [seq][position][kv head][dim] of
// 2-byte elements, box = 128 positions x 64 dims of one head, 128-byte swizzle.  Quantised:
// [seq][position][kv head][row bytes], box = 128 positions x one whole row, no swizzle.
struct CacheMaps { CUtensorMap k, v; };
b200_status encode_cache_map(CUtensorMap *m, const void *base, int type, int n_seq, int n_kv, int hd, uint64_t n_ctx) {
    if (type == KQ_KV_F16) {
        const uint64_t dims[4] = {(uint64_t)hd, (uint64_t)n_kv, n_ctx, (uint64_t)n_seq};
        const uint64_t strides[3] = {(uint64_t)hd * 2, (uint64_t)n_kv * hd * 2, n_ctx * n_kv * hd * 2};
        const uint32_t box[4] = {64, 1, ROWS_PER_CTA, 1};
        return kq_tmap_encode(m, 2, 4, base, dims, strides, box, 1);
    }
    const uint64_t rb = (uint64_t)kq_kv_row_bytes(type, hd);
    const uint64_t dims[4] = {rb, (uint64_t)n_kv, n_ctx, (uint64_t)n_seq};
    const uint64_t strides[3] = {rb, (uint64_t)n_kv * rb, n_ctx * n_kv * rb};
    const uint32_t box[4] = {(uint32_t)rb, 1, ROWS_PER_CTA, 1};
    return kq_tmap_encode(m, 1, 4, base, dims, strides, box, 0);
}
b200_status cache_maps(const uint16_t *kc, const uint16_t *vc, int n_seq, int n_kv, int hd, int64_t seq_stride, KqKvTypes kvt,
                       const CacheMaps **out) {
    static std::map<std::tuple<const void *, const void *, int, int, int, int64_t, int, int>, CacheMaps> cache;
    const auto key = std::make_tuple((const void *)kc, (const void *)vc, n_seq, n_kv, hd, seq_stride, kvt.k, kvt.v);
    auto it = cache.find(key);
    if (it == cache.end()) {
        KQ_REQUIRE(seq_stride % ((int64_t)n_kv * hd) == 0, "attention: the cache stride is not a whole number of positions");
        const uint64_t n_ctx = (uint64_t)(seq_stride / ((int64_t)n_kv * hd));
        CacheMaps m;
        memset(&m, 0, sizeof(m));
        b200_status rc = encode_cache_map(&m.k, kc, kvt.k, n_seq, n_kv, hd, n_ctx);
        if (rc != B200_OK) return rc;
        rc = encode_cache_map(&m.v, vc, kvt.v, n_seq, n_kv, hd, n_ctx);
        if (rc != B200_OK) return rc;
        if (cache.size() > 4096) cache.clear(); // a bound, not a policy
        it = cache.emplace(key, m).first;
    }
    *out = &it->second;
    return B200_OK;
}

} // namespace

// Number of position slices for a context of L rows: one per 128 rows, at most 64, so that every
// CTA of the launch has rows to work on; with several sequences (pairs = sequences x KV heads) no more
// than fill the GPU once (two CTAs per SM are resident), a CTA then walks through several 128-row chunks
// instead of the launch running in waves (8 sequences at context 2048: 29.6 -> 20.9 us per layer).  A captured decode step is keyed by this number, so a sequence
// re-captures its step once per 128 positions.
int kq_attention_decode_splits(int64_t L, int pairs) {
    int64_t n = (L + ROWS_PER_CTA - 1) / ROWS_PER_CTA;
    static int one_wave = -1;
    if (one_wave < 0) {
        const char *e = getenv("B200_ATTN_DECODE_WAVE");
        one_wave = e ? atoi(e) : 2 * kq_sm_count();
    }
    if (pairs > 8 && one_wave > 0) {
        const int64_t cap = one_wave / pairs;
        if (n > cap) n = cap;
    }
    return (int)(n < 1 ? 1 : (n > 64 ? 64 : n));
}

// q [n_seq][n_head][hd], k / v [n_seq][n_kv][hd] f32 as they come out of the qkv projection (not yet
// rotated); the cache of sequence s starts s * seq_stride elements (seq_stride / hd rows) in.  scratch holds the split
// partials, counters one zero-initialised int per (sequence, kv head).
b200_status kq_attention_decode(const float *q, const float *k, const float *v, uint16_t *kc, uint16_t *vc,
                                int n_seq, const int32_t *pos_dev, int pos, int n_head, int n_kv, int hd,
                                int64_t seq_stride, float theta, int neox, int n_split, float *out, float *scratch,
                                size_t scratch_bytes, int *counters, KqKvTypes kvt, cudaStream_t st) {
    KQ_REQUIRE(hd == 128 || hd == 64, "attention: head_dim %d not supported", hd);
    KQ_REQUIRE(kq_kv_type_ok(kvt.k) && kq_kv_type_ok(kvt.v), "attention: KV cache types %d / %d", kvt.k, kvt.v);
    KQ_REQUIRE(n_kv > 0 && n_head % n_kv == 0, "attention: n_head %% n_kv");
    if (n_split > 64) n_split = 64;
    size_t need = (size_t)n_seq * n_head * n_split * (hd + 2) * sizeof(float);
    while (n_split > 1 && (need > scratch_bytes || !counters)) {
        n_split /= 2;
        need = (size_t)n_seq * n_head * n_split * (hd + 2) * sizeof(float);
    }
    RopeTab tab;
    for (int i = 0; i < hd / 2; i++) tab.inv_freq[i] = (float)pow((double)theta, -2.0 * i / (double)hd);
    float *po = scratch, *pml = scratch ? scratch + (size_t)n_seq * n_head * n_split * hd : nullptr;
    const float scale = 1.0f / sqrtf((float)hd);
    dim3 grid(n_kv, n_split, n_seq);
    // one slice per 128 positions (not capped): a CTA's only chunk starts at slice * 128 whatever the position is
    static int early_env = -1;
    if (early_env < 0) {
        const char *e = getenv("B200_ATTN_DECODE_EARLY");
        early_env = e ? atoi(e) : 1;
    }
    const int unit_chunk = early_env && n_split == (pos + 1 + ROWS_PER_CTA - 1) / ROWS_PER_CTA ? 1 : 0;
    const int G = n_head / n_kv;
    KQ_REQUIRE((((uintptr_t)kc | (uintptr_t)vc) & 15) == 0, "attention: the cache must be 16-byte aligned");
    const CacheMaps *maps = nullptr;
    const b200_status rc = cache_maps(kc, vc, n_seq, n_kv, hd, seq_stride, kvt, &maps);
    if (rc != B200_OK) return rc;
    if (hd == 128)
        return launch_g<128>(G, grid, st, maps->k, maps->v, q, k, v, (__half *)kc, (__half *)vc, pos_dev, pos, n_head, n_kv,
                             seq_stride, n_split, unit_chunk, scale, neox, tab, out, po, pml, counters, kvt);
    return launch_g<64>(G, grid, st, maps->k, maps->v, q, k, v, (__half *)kc, (__half *)vc, pos_dev, pos, n_head, n_kv,
                        seq_stride, n_split, unit_chunk, scale, neox, tab, out, po, pml, counters, kvt);
}

#ifdef KQ_ATTN_TRACE
extern "C" __attribute__((visibility("default"))) int kq_attn_trace_fetch(unsigned long long *out, int max_rec) {
    unsigned int n = 0, zero = 0;
    cudaDeviceSynchronize();
    cudaMemcpyFromSymbol(&n, g_atr_n, sizeof(n));
    if ((int)n > max_rec) n = max_rec;
    if (n > 8192u) n = 8192u;
    if (out && n) cudaMemcpyFromSymbol(out, g_atr, sizeof(unsigned long long) * 12 * n);
    cudaMemcpyToSymbol(g_atr_n, &zero, sizeof(zero));
    return (int)n;
}
#endif
