// Causal attention for a batch of new tokens (prefill) over an f16 KV cache on the 5th-generation
// tensor cores: S = Q K^T and O += P V are tcgen05.mma kind::f16 with the accumulators in TMEM, the K and
// V tiles arrive by tiled TMA copies, the probabilities go back into TMEM and are the A operand of the
// second product.  The reference runs its servers with flash attention always on
// (mesh-llm/src/inference/launch.rs:1352-1353), so this op carries the O(T^2) part of every prefill.
//
// One CTA serves the G query heads that share a KV head for 128 / G consecutive positions: 128 query
// rows (TMEM lanes), row r = (position r / G, head r % G).  Warps 0-7 are the softmax: a row is shared by two
// threads (warps w and w + 4 reach the same TMEM lanes), each taking 64 of the 128 keys of a tile; warp 8
// issues copies and MMAs.
//
// Shared-memory operand layout.  A K or V tile (128 positions x 128 dims, f16) arrives as two TMA boxes of
// 128 positions x 64 dims out of the cache viewed as [seq][position][kv head][dim], each box landing as
// [position][128 bytes] with the 128-byte swizzle.  Read with a K-major descriptor (rows = positions,
// K = dims, 8-row groups 1024 bytes apart, 32 bytes further per K = 16 step, the second box for dims
// 64..127) this is the B operand K^T; read with an MN-major descriptor (N = dims: the two boxes are the
// two 64-dim atoms, 16 KB apart; K = positions: groups of 8 positions 1024 bytes apart) it is the B
// operand V -- so neither tile is transposed or touched by CUDA cores.  Q is converted to f16
// (pre-scaled by log2(e) / sqrt(head_dim)) into the same swizzled K-major layout once per CTA.
//
// Per key tile: S (128 x 128 f32, TMEM columns 0..127) <- 8 MMAs of K = 16; each softmax thread reads
// its half row twice (maximum, exchanged with its partner through shared memory; then exponentials, row
// sum, f16 pairs) and stores its 32 packed words of P over columns of S that both partners have already
// taken into registers; if a row maximum grew, the thread rescales its half of the row of O (columns
// 128..255) first; O += P V is 8 MMAs with A from TMEM.  Online softmax in base 2, f32
// throughout, P and Q rounded to f16 as in the mma.sync kernel this one supersedes for f16 caches.
// A CTA holds 256 TMEM columns and 96 KB of shared memory, so two CTAs share an SM and one's MMAs run
// under the other's softmax.  K of the next tile is requested as soon as S is complete, V as soon as
// P V is.  Every wait is bounded; on a time-out the kernel records an error, lets its copies land,
// frees its TMEM and returns.
#include "kq_common.cuh"
#include "kq_kvq.cuh"

#include <cuda.h>
#include <math.h>
#include <string.h>

#include <map>
#include <tuple>

b200_status kq_tmap_encode(void *map128, int elem_bytes, int rank, const void *base, const uint64_t *dims,
                           const uint64_t *strides_bytes, const uint32_t *box, int swizzle128);

namespace {

constexpr int HD = 128, BK = 128, TILE_BYTES = BK * HD * 2, HALF_BYTES = TILE_BYTES / 2; // K or V tile: two boxes of 16 KB
constexpr int SMEM_Q = 0, SMEM_K = TILE_BYTES, SMEM_V = 2 * TILE_BYTES, SMEM_TOTAL = 3 * TILE_BYTES;
constexpr uint32_t TMEM_COLS = 256, COL_S = 0, COL_O = 128;

__device__ int g_attn_tc_error;
#ifdef KQ_ATTN_PROF
__device__ long long g_attn_prof[8];
#define APROF_T(v) const long long v = clock64()
#define APROF_ADD(i, a, b) do { if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) g_attn_prof[i] += (b) - (a); } while (0)
#else
#define APROF_T(v)
#define APROF_ADD(i, a, b)
#endif

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

// shared-memory matrix descriptor, 128-byte swizzle (layout type 2)
__device__ __forceinline__ uint64_t make_desc(uint32_t saddr, uint32_t lbo, uint32_t sbo) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFF) >> 4);
    d |= (uint64_t)(lbo >> 4) << 16;
    d |= (uint64_t)(sbo >> 4) << 32;
    d |= (uint64_t)1 << 46; // descriptor version of this architecture
    d |= (uint64_t)2 << 61; // SWIZZLE_128B
    return d;
}
// K-major operand (Q, K^T): rows of 128 bytes, 8-row groups 1024 bytes apart; K step s of 16 dims
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t tile, int s) {
    return make_desc(tile + (s >> 2) * HALF_BYTES + (s & 3) * 32, 16, 1024);
}
// MN-major operand (V): 64-dim atoms 16 KB apart, groups of 8 positions 1024 bytes apart; K step s of 16 positions
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t tile, int s) { return make_desc(tile + s * 2048, HALF_BYTES, 1024); }
// kind::f16: D f32, A f16, B f16, M = 128, N = 128; b_mn: B is MN-major (V), else K-major (K^T)
__device__ __forceinline__ uint32_t idesc(bool b_mn) {
    return (1u << 4) | ((b_mn ? 1u : 0u) << 16) | ((uint32_t)(128 >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}
__device__ __forceinline__ void mma_ss(uint32_t d_tmem, uint64_t a, uint64_t b, uint32_t id, uint32_t acc) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 :
                 : "r"(d_tmem), "l"(a), "l"(b), "r"(id), "r"(acc)
                 : "memory");
}
__device__ __forceinline__ void mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b, uint32_t id, uint32_t acc) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
                 :
                 : "r"(d_tmem), "r"(a_tmem), "l"(b), "r"(id), "r"(acc)
                 : "memory");
}
__device__ __forceinline__ void commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

#define TMEM_LD32(taddr, r)                                                                                             \
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"        \
                 "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"                              \
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),      \
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), \
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]),            \
                   "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]),            \
                   "=r"(r[30]), "=r"(r[31])                                                                             \
                 : "r"(taddr)                                                                                           \
                 : "memory")
#define TMEM_ST32(taddr, r)                                                                                             \
    asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"  \
                 "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"                                     \
                 :                                                                                                      \
                 : "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),  \
                   "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),         \
                   "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),       \
                   "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])        \
                 : "memory")
#define TMEM_ST16(taddr, r)                                                                                             \
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};" \
                 :                                                                                                      \
                 : "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),  \
                   "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])          \
                 : "memory")

// 2^x by the special-function unit (x <= 0 here; results below 2^-126 flush to zero, which is what a
// probability that small contributes anyway)
__device__ __forceinline__ float ex2(float x) {
#ifdef KQ_ATTN_SLOW_EXP
    return exp2f(x);
#else
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
#endif
}
__device__ __forceinline__ uint32_t pack_h2(float a, float b) {
    const __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<const uint32_t *>(&h);
}

constexpr uint64_t LIMIT = 5 * KQ_WAIT_LIMIT_NS;

constexpr int NSOFT = 256, NTHREADS = NSOFT + 32; // eight softmax warps and the issuing warp
__device__ __forceinline__ void softmax_barrier() { asm volatile("bar.sync 1, %0;" ::"n"(NSOFT) : "memory"); }

// grid (query tiles, n_kv, n_seq); two CTAs per SM
__global__ void __launch_bounds__(NTHREADS, 2) attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap kmap,
                                                                      const __grid_constant__ CUtensorMap vmap, const float *q,
                                                                      int T, const int32_t *pos0_dev, int pos0_val, int n_head,
                                                                      int G, int PQ, float scale_log2, float *out) {
    KQ_PDL_ENTER();
    extern __shared__ __align__(1024) uint8_t sm[];
    __shared__ uint64_t full_k, full_v; // the K / V tile has landed
    __shared__ uint64_t s_ready;        // S = Q K^T of the current tile is in TMEM
    __shared__ uint64_t p_ready;        // all rows of P are in TMEM
    __shared__ uint64_t pv_done;        // O += P V of the current tile has completed
    __shared__ float red[2][2][128];    // [tile parity][half][row]: the half rows' maxima
    __shared__ float lsum[128];         // second halves' row sums at the end
    __shared__ uint32_t s_tmem;
    __shared__ int s_abort;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    // the query tiles with the longest history first
    const int qt = (int)gridDim.x - 1 - (int)blockIdx.x, kh = blockIdx.y, seq = blockIdx.z;
    const int pos0 = pos0_dev ? *pos0_dev : pos0_val;
    const int p_base = qt * PQ;                   // first position (inside the batch) of this tile
    const int p_last = min(T, p_base + PQ) - 1;   // last one
    const int n_tiles = (pos0 + p_last) / BK + 1; // key tiles up to the diagonal
    const uint32_t bar_k = smem_u32(&full_k), bar_v = smem_u32(&full_v), bar_s = smem_u32(&s_ready), bar_p = smem_u32(&p_ready),
                   bar_pv = smem_u32(&pv_done);

    if (warp == 8) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem)), "r"(TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    if (tid == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar_k), "r"(1));
        asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar_v), "r"(1));
        asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar_s), "r"(1));
        asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar_p), "r"(NSOFT));
        asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar_pv), "r"(1));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        s_abort = 0;
    }
    // ---- rows: thread (row, half) with row = tid % 128 (position p_base + row / G, head kh * G + row % G)
    const int row = tid & 127, half = (tid >> 7) & 1;
    const int p_loc = row / G, g = row % G;
    const bool row_ok = warp < 8 && p_loc < PQ && p_base + p_loc < T;
    const int lim = row_ok ? pos0 + p_base + p_loc : -1; // last visible key of this row
    if (warp < 8) { // Q tile to f16, K-major, swizzled: this thread's 64 dims of its row (box `half`)
        const float *qr = q + ((int64_t)(seq * T + (row_ok ? p_base + p_loc : 0)) * n_head + kh * G + g) * HD + 64 * half;
        uint8_t *dst = sm + SMEM_Q + half * HALF_BYTES + row * 128;
#pragma unroll 4
        for (int c = 0; c < 8; c++) { // chunk c: dims 8c .. 8c+7 of the box; 16-byte slot c ^ (row % 8)
            uint4 v = make_uint4(0, 0, 0, 0);
            if (row_ok) {
                const float4 a = *reinterpret_cast<const float4 *>(qr + 8 * c), b = *reinterpret_cast<const float4 *>(qr + 8 * c + 4);
                v.x = pack_h2(a.x * scale_log2, a.y * scale_log2);
                v.y = pack_h2(a.z * scale_log2, a.w * scale_log2);
                v.z = pack_h2(b.x * scale_log2, b.y * scale_log2);
                v.w = pack_h2(b.z * scale_log2, b.w * scale_log2);
            }
            *reinterpret_cast<uint4 *>(dst + ((c ^ (row & 7)) << 4)) = v;
        }
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = s_tmem;

    if (warp == 8) {
        // ---------------------------------------------------------------- copies and MMAs
        if (lane == 0) {
            auto load = [&](const CUtensorMap *map, int smem_off, uint32_t bar, int tile) { // two boxes of 64 dims x 128 positions
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(TILE_BYTES) : "memory");
#pragma unroll
                for (int hb = 0; hb < 2; hb++)
                    asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];" ::"r"(
                                     smem_u32(sm + smem_off + hb * HALF_BYTES)),
                                 "l"(map), "r"(hb * 64), "r"(kh), "r"(tile * BK), "r"(seq), "r"(bar)
                                 : "memory");
            };
            load(&kmap, SMEM_K, bar_k, 0);
            load(&vmap, SMEM_V, bar_v, 0);
            const uint32_t q_addr = smem_u32(sm + SMEM_Q), k_addr = smem_u32(sm + SMEM_K), v_addr = smem_u32(sm + SMEM_V);
            auto wait = [&](uint32_t bar, uint32_t parity, int code) {
                if (!s_abort && !kq_mbar_wait(bar, parity, LIMIT)) {
                    s_abort = 1;
                    atomicExch(&g_attn_tc_error, code);
                }
            };
            for (int i = 0; i < n_tiles; i++) {
                const uint32_t ph = (uint32_t)(i & 1);
                wait(bar_k, ph, 1);
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                if (!s_abort) {
#pragma unroll
                    for (int s = 0; s < 8; s++) // K = 16 dims per instruction
                        mma_ss(tmem + COL_S, desc_kmajor(q_addr, s), desc_kmajor(k_addr, s), idesc(false), s > 0);
                }
                commit(bar_s);
                wait(bar_s, ph, 2); // K has been read: the next tile's K can come in
                if (!s_abort && i + 1 < n_tiles) load(&kmap, SMEM_K, bar_k, i + 1);
                wait(bar_p, ph, 3);
                wait(bar_v, ph, 4);
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                if (!s_abort) {
#pragma unroll
                    for (int s = 0; s < 8; s++) // K = 16 positions per instruction: eight packed columns of P, which lie at the start of each half's columns of S
                        mma_ts(tmem + COL_O, tmem + COL_S + 64 * (s >> 2) + 8 * (s & 3), desc_mnmajor(v_addr, s), idesc(true), (i > 0 || s > 0) ? 1u : 0u);
                }
                commit(bar_pv);
                wait(bar_pv, ph, 5); // P (over S) and V have been read, O is complete up to this tile
                if (!s_abort && i + 1 < n_tiles) load(&vmap, SMEM_V, bar_v, i + 1);
            }
        }
        __syncwarp();
    } else {
        // ---------------------------------------------------------------- online softmax, half a row per thread
        const uint32_t tl = tmem + ((uint32_t)((warp & 3) * 32) << 16);
        const int c0 = 64 * half; // this thread's key columns of a tile
        float m = -INFINITY, l = 0.f;
        for (int i = 0; i < n_tiles; i++) {
            if (!s_abort && !kq_mbar_wait(bar_s, (uint32_t)(i & 1), LIMIT)) {
                s_abort = 1;
                atomicExch(&g_attn_tc_error, 6);
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int k0 = i * BK + c0;
            const bool diag = i * BK + BK - 1 > pos0 + p_base; // some row of the tile sees only part of these keys
            float t4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int c = 0; c < 2; c++) {
                uint32_t s[32];
                TMEM_LD32(tl + COL_S + c0 + 32 * c, s);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (!diag) {
#pragma unroll
                    for (int j = 0; j < 32; j++) t4[j & 3] = fmaxf(t4[j & 3], __uint_as_float(s[j]));
                } else {
#pragma unroll
                    for (int j = 0; j < 32; j++)
                        if (k0 + 32 * c + j <= lim) t4[j & 3] = fmaxf(t4[j & 3], __uint_as_float(s[j]));
                }
            }
            red[i & 1][half][row] = row_ok ? fmaxf(fmaxf(t4[0], t4[1]), fmaxf(t4[2], t4[3])) : -INFINITY;
            softmax_barrier(); // both halves' maxima are in
            const float m_new = fmaxf(m, fmaxf(red[i & 1][0][row], red[i & 1][1][row]));
            const float alpha = (m_new == -INFINITY || m == m_new) ? 1.f : ex2(m - m_new); // m = -inf: nothing accumulated yet
            const float sub = m_new == -INFINITY ? 0.f : m_new;
            // S was issued after the P V of the tile before had completed, so O is at rest here
            if (i > 0 && !s_abort && __any_sync(0xffffffffu, alpha != 1.f)) {
#pragma unroll
                for (int c = 0; c < 2; c++) {
                    uint32_t o[32];
                    TMEM_LD32(tl + COL_O + c0 + 32 * c, o);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                    for (int j = 0; j < 32; j++) o[j] = __float_as_uint(__uint_as_float(o[j]) * alpha);
                    TMEM_ST32(tl + COL_O + c0 + 32 * c, o);
                }
            }
            l *= alpha;
            m = m_new;
            float l4[4] = {0.f, 0.f, 0.f, 0.f};
            // P of this half row goes over the first 32 of its own 64 columns of S, chunk by chunk behind the reads
#pragma unroll
            for (int c = 0; c < 2; c++) {
                uint32_t s[32], pk[16];
                TMEM_LD32(tl + COL_S + c0 + 32 * c, s);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (!diag) {
#pragma unroll
                    for (int j = 0; j < 32; j += 2) {
                        const float e0 = ex2(__uint_as_float(s[j]) - sub), e1 = ex2(__uint_as_float(s[j + 1]) - sub);
                        l4[(j >> 1) & 3] += e0 + e1;
                        pk[j >> 1] = pack_h2(e0, e1);
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 32; j += 2) {
                        const float e0 = k0 + 32 * c + j <= lim ? ex2(__uint_as_float(s[j]) - sub) : 0.f;
                        const float e1 = k0 + 32 * c + j + 1 <= lim ? ex2(__uint_as_float(s[j + 1]) - sub) : 0.f;
                        l4[(j >> 1) & 3] += e0 + e1;
                        pk[j >> 1] = pack_h2(e0, e1);
                    }
                }
                if (!s_abort) TMEM_ST16(tl + COL_S + c0 + 16 * c, pk);
            }
            if (row_ok) l += (l4[0] + l4[1]) + (l4[2] + l4[3]);
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar_p) : "memory");
        }
        // ---- O / l -> out
        if (half == 1) lsum[row] = l;
        softmax_barrier();
        if (half == 0) l += lsum[row];
        else l += 0.f;
        if (half == 0) lsum[row] = l;
        softmax_barrier();
        l = lsum[row];
        if (!s_abort && !kq_mbar_wait(bar_pv, (uint32_t)((n_tiles - 1) & 1), LIMIT)) {
            s_abort = 1;
            atomicExch(&g_attn_tc_error, 7);
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (!s_abort) {
            const float inv = l > 0.f ? 1.f / l : 0.f;
            float *orow = out + ((int64_t)(seq * T + (row_ok ? p_base + p_loc : 0)) * n_head + kh * G + g) * HD + c0;
#pragma unroll
            for (int c = 0; c < 2; c++) {
                uint32_t o[32];
                TMEM_LD32(tl + COL_O + c0 + 32 * c, o);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (row_ok) {
#pragma unroll
                    for (int j = 0; j < 32; j += 4)
                        *reinterpret_cast<float4 *>(orow + 32 * c + j) =
                            make_float4(__uint_as_float(o[j]) * inv, __uint_as_float(o[j + 1]) * inv,
                                        __uint_as_float(o[j + 2]) * inv, __uint_as_float(o[j + 3]) * inv);
                }
            }
        }
    }
    if (s_abort && warp == 8 && lane == 0) { // copies that were posted must land before the CTA goes away
        kq_mbar_wait(bar_k, 0u, KQ_WAIT_LIMIT_NS);
        kq_mbar_wait(bar_k, 1u, KQ_WAIT_LIMIT_NS);
        kq_mbar_wait(bar_v, 0u, KQ_WAIT_LIMIT_NS);
        kq_mbar_wait(bar_v, 1u, KQ_WAIT_LIMIT_NS);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 8) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
}

struct Maps {
    CUtensorMap k, v;
};

// the cache [seq][position][kv head][128]: boxes of 64 dims x 128 positions with the 128-byte swizzle
b200_status encode_tile_map(CUtensorMap *m, const void *base, int n_seq, int n_kv, uint64_t n_ctx, int64_t seq_stride) {
    const uint64_t dims[4] = {(uint64_t)HD, (uint64_t)n_kv, n_ctx, (uint64_t)n_seq};
    const uint64_t strides[3] = {(uint64_t)HD * 2, (uint64_t)n_kv * HD * 2, (uint64_t)seq_stride * 2};
    const uint32_t box[4] = {64, 1, BK, 1};
    return kq_tmap_encode(m, 2, 4, base, dims, strides, box, 1);
}

} // namespace

#ifdef KQ_ATTN_PROF
extern "C" __attribute__((visibility("default"))) void kq_attn_prof_fetch(long long *out) {
    cudaMemcpyFromSymbol(out, g_attn_prof, sizeof(long long) * 8);
    long long z[8] = {0};
    cudaMemcpyToSymbol(g_attn_prof, z, sizeof(z));
}
#endif
int kq_attn_tc_error_fetch() {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_attn_tc_error, sizeof(int)) != cudaSuccess) return -1;
    if (v) cudaMemcpyToSymbol(g_attn_tc_error, &zero, sizeof(int));
    return v;
}

// q [n_seq * T][n_head][128] f32 (already rotated), f16 caches [seq][pos][n_kv][128]; returns
// B200_ERR_UNSUPPORTED when the shape is not one this kernel is built for (the caller then uses another kernel).
b200_status kq_attention_prefill_tc(const float *q, const uint16_t *kc, const uint16_t *vc, int n_seq, int T,
                                    const int32_t *pos0_dev, int pos0, int n_head, int n_kv, int hd, int64_t seq_stride,
                                    float *out, cudaStream_t st) {
    if (hd != HD || n_kv <= 0 || n_head % n_kv != 0) return B200_ERR_UNSUPPORTED;
    const int G = n_head / n_kv;
    if (G > 128 || seq_stride % ((int64_t)n_kv * HD) != 0) return B200_ERR_UNSUPPORTED;
    // positions the tensor map may touch: the cache's extent per sequence; a caller that passes a single
    // sequence without a stride has vouched for pos0 + T positions only
    if (seq_stride == 0 && (n_seq != 1 || pos0_dev)) return B200_ERR_UNSUPPORTED;
    const uint64_t n_ctx = seq_stride ? (uint64_t)(seq_stride / ((int64_t)n_kv * HD)) : (uint64_t)(pos0 + T);
    if (n_ctx < 1) return B200_ERR_UNSUPPORTED;
    if (((uintptr_t)q & 15) || ((uintptr_t)out & 15) || ((uintptr_t)kc & 15) || ((uintptr_t)vc & 15)) return B200_ERR_UNSUPPORTED;
    static std::map<std::tuple<const void *, const void *, int, int, int64_t, uint64_t>, Maps> cache;
    const auto key = std::make_tuple((const void *)kc, (const void *)vc, n_seq, n_kv, seq_stride, n_ctx);
    auto it = cache.find(key);
    if (it == cache.end()) {
        Maps m;
        memset(&m, 0, sizeof(m));
        const int64_t sstride = seq_stride ? seq_stride : (int64_t)n_ctx * n_kv * HD;
        if (encode_tile_map(&m.k, kc, n_seq, n_kv, n_ctx, sstride) != B200_OK ||
            encode_tile_map(&m.v, vc, n_seq, n_kv, n_ctx, sstride) != B200_OK)
            return B200_ERR_UNSUPPORTED;
        if (cache.size() > 4096) cache.clear();
        it = cache.emplace(key, m).first;
    }
    const int PQ = 128 / G;
    const float scale_log2 = 1.4426950408889634f / sqrtf((float)hd);
    static bool attr[16];
    int dev = 0;
    KQ_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 16 || !attr[dev]) {
        KQ_CUDA(cudaFuncSetAttribute(attn_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_TOTAL));
        if (dev >= 0 && dev < 16) attr[dev] = true;
    }
    const dim3 grid((unsigned)kq_div_up(T, PQ), (unsigned)n_kv, (unsigned)n_seq);
    kq_launch(attn_prefill_tc_kernel, grid, NTHREADS, SMEM_TOTAL, st, it->second.k, it->second.v, q, T, pos0_dev, pos0, n_head, G, PQ,
              scale_log2, out);
    KQ_COUNT_LAUNCH();
    KQ_LAUNCH_CHECK();
    return B200_OK;
}
