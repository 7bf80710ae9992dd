// Decode GEMV: y[m][n] = sum_k W[n][k] x[m][k] for M <= 8 tokens, W in Q4_K / Q6_K blocks, x in
// Q8 blocks of 256.  This is MUL_MAT of the ggml op surface at decode batch sizes; the kernel is
// bound by HBM bandwidth (0.5625 / 0.8203 bytes per weight), so everything here is about
// streaming the packed blocks once with 16-byte loads and enough of them in flight.
//
// Work split: a warp owns R weight rows; its 32 lanes cover 4 consecutive super-blocks per
// step (8 lanes x 16 bytes = the 128 quant bytes of one block).  Each lane keeps f32 partial sums
// for its R rows x M tokens; the activations of a block are loaded once and reused for the R
// rows.  Long rows are additionally split over the 2 or 4 warps of a CTA and combined in shared
// memory in a fixed order, so results are deterministic (no float atomics).
#include "kq_common.cuh"
#include "kq_lanes.cuh"

#include <stdlib.h>

namespace {

struct GemvParams {
    KqGemvSeg seg[3];
    int32_t rg_end[3]; // exclusive prefix of row groups per segment
    int32_t nseg;
    int32_t n_rg;      // total row groups
    int32_t nb;        // blocks per row
    int32_t K;
    int32_t wk;        // warps of a CTA sharing one row group along K (1, 2 or 4)
    int32_t swiglu;    // segments 0/1 are gate/up; a warp takes R/2 rows of each
    const int8_t *aq;
    const float *ad;
    const int16_t *abs16;
    const float *residual; // [M][ldy of segment 0] or null (single segment only)
    // expert-indexed mode (MUL_MAT_ID): blockIdx.y walks (token, slot) pairs; pair p uses the
    // expert matrix ids[p], activation row p / act_div and output row p.  M is 1 in this mode.
    const int32_t *expert_ids;
    int32_t act_div;
};

template <int M, int R>
__global__ void __launch_bounds__(128) gemv_kernel(const GemvParams p) {
    KQ_PDL_ENTER();
    __shared__ float red[4][R * M];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int wk = p.wk, wn = 4 / wk;
    const int kslot = warp % wk, nslot = warp / wk;
    const int sub = lane >> 3, c = lane & 7;
    const int nb = p.nb;
    const int pair = blockIdx.y;
    int64_t expert = 0;
    const int8_t *aq = p.aq;
    const float *ad = p.ad;
    const int16_t *abs16 = p.abs16;
    if (p.expert_ids) {
        expert = p.expert_ids[pair];
        const int arow = pair / p.act_div;
        aq += (int64_t)arow * p.K;
        ad += (int64_t)arow * nb;
        abs16 += (int64_t)arow * nb * 16;
    }

    for (int base = blockIdx.x * wn; base < p.n_rg; base += gridDim.x * wn) {
        const int rg = base + nslot;
        const bool active = rg < p.n_rg;
        int si = 0, rg0 = 0;
        if (active) {
            if (p.nseg > 1 && rg >= p.rg_end[0]) { si = 1; rg0 = p.rg_end[0]; }
            if (p.nseg > 2 && rg >= p.rg_end[1]) { si = 2; rg0 = p.rg_end[1]; }
        }
        const KqGemvSeg &sg = p.seg[si];
        const uint32_t type = sg.type;
        const int64_t stride = kq_device_row_bytes(type, p.K);
        float acc[R][M];
#pragma unroll
        for (int r = 0; r < R; r++)
#pragma unroll
            for (int m = 0; m < M; m++) acc[r][m] = 0.f;

        const uint8_t *rp[R];
        int row[R];
        if (active) {
#pragma unroll
            for (int r = 0; r < R; r++) {
                if (p.swiglu) {
                    row[r] = (rg - rg0) * (R / 2) + (r % (R / 2));
                    const KqGemvSeg &s2 = p.seg[r / (R / 2)];
                    rp[r] = s2.W + expert * s2.expert_stride + (int64_t)min(row[r], s2.n_rows - 1) * stride;
                } else {
                    row[r] = (rg - rg0) * R + r;
                    rp[r] = sg.W + expert * sg.expert_stride + (int64_t)min(row[r], sg.n_rows - 1) * stride;
                }
            }
            if (type == B200_TYPE_Q4_K) {
                const int e_lo = 64 * (c >> 1) + 16 * (c & 1);
                for (int it = kslot; it * 4 < nb; it += wk) {
                    const int blk = it * 4 + sub;
                    if (blk < nb) {
                        uint4 hdr[R], w[R];
#pragma unroll
                        for (int r = 0; r < R; r++) {
                            const uint8_t *b = rp[r] + (int64_t)blk * KQ_Q4K_BYTES;
                            hdr[r] = __ldg(reinterpret_cast<const uint4 *>(b));
                            w[r] = kq_ld_stream(b + 16 + 16 * c);
                        }
                        Q4Scales sc[R];
#pragma unroll
                        for (int r = 0; r < R; r++) sc[r] = q4k_lane_scales(hdr[r], c);
#pragma unroll
                        for (int m = 0; m < M; m++) {
                            const int8_t *a = aq + (int64_t)m * p.K + blk * 256 + e_lo;
                            const int4 alo = *reinterpret_cast<const int4 *>(a);
                            const int4 ahi = *reinterpret_cast<const int4 *>(a + 32);
                            const float da = ad[m * nb + blk];
                            const int16_t *s16 = abs16 + ((int64_t)m * nb + blk) * 16 + (e_lo >> 4);
                            const int bl = s16[0], bh = s16[2];
#pragma unroll
                            for (int r = 0; r < R; r++) {
                                int isum, msum;
                                q4k_lane_ints(w[r], sc[r], alo, ahi, bl, bh, isum, msum);
                                acc[r][m] = fmaf(sc[r].d * da, (float)isum, acc[r][m]);
                                acc[r][m] = fmaf(-(sc[r].dmin * da), (float)msum, acc[r][m]);
                            }
                        }
                    }
                }
            } else { // Q6_K device layout
                const int h = c >> 2, cc = c & 3;
                const int e_lo = 128 * h + 16 * cc;
                for (int it = kslot; it * 4 < nb; it += wk) {
                    const int blk = it * 4 + sub;
                    if (blk < nb) {
                        uint4 ql[R], qh[R];
                        int scl[R], sch[R];
                        float dw[R];
#pragma unroll
                        for (int r = 0; r < R; r++) {
                            const KqQ6Addr qa = kq_q6_addr(nb, blk);
                            ql[r] = kq_ld_stream(rp[r] + qa.ql + qa.cs * c);
                            qh[r] = __ldg(reinterpret_cast<const uint4 *>(rp[r] + qa.qh + qa.cs * (2 * h + (cc & 1))));
                            const int8_t *scp = reinterpret_cast<const int8_t *>(rp[r] + qa.sc);
                            scl[r] = scp[8 * h + cc];
                            sch[r] = scp[8 * h + 4 + cc];
                            dw[r] = kq_h2f(*reinterpret_cast<const uint16_t *>(rp[r] + qa.d));
                        }
                        uint32_t vl[R][4], vh[R][4]; // the six-bit codes, assembled once for all tokens
#pragma unroll
                        for (int r = 0; r < R; r++) q6k_lane_codes(ql[r], qh[r], cc, vl[r], vh[r]);
#pragma unroll
                        for (int m = 0; m < M; m++) {
                            const int8_t *a = aq + (int64_t)m * p.K + blk * 256 + e_lo;
                            const int4 alo = *reinterpret_cast<const int4 *>(a);
                            const int4 ahi = *reinterpret_cast<const int4 *>(a + 64);
                            const float da = ad[m * nb + blk];
                            const int16_t *s16 = abs16 + ((int64_t)m * nb + blk) * 16 + (e_lo >> 4);
                            const int bl = s16[0], bh = s16[4];
#pragma unroll
                            for (int r = 0; r < R; r++) {
                                const int isum = q6k_lane_dot(vl[r], vh[r], scl[r], sch[r], alo, ahi, bl, bh);
                                acc[r][m] = fmaf(dw[r] * da, (float)isum, acc[r][m]);
                            }
                        }
                    }
                }
            }
        }
        // warp reduce, then combine the K-slices of the CTA in a fixed order
#pragma unroll
        for (int r = 0; r < R; r++)
#pragma unroll
            for (int m = 0; m < M; m++) {
                const float v = kq_warp_sum(acc[r][m]);
                if (lane == 0) red[warp][r * M + m] = v;
            }
        __syncthreads();
        if (active && kslot == 0) {
            if (p.swiglu) {
                if (lane < (R / 2) * M) {
                    const int r = lane / M, m = lane % M;
                    float g = 0.f, u = 0.f;
                    for (int k = 0; k < wk; k++) {
                        g += red[warp + k][r * M + m];
                        u += red[warp + k][(r + R / 2) * M + m];
                    }
                    int rw = row[0];
#pragma unroll
                    for (int rr = 1; rr < R / 2; rr++)
                        if (r == rr) rw = row[rr];
                    if (rw < p.seg[0].n_rows) {
                        if (p.seg[0].bias) g += p.seg[0].bias[rw];
                        if (p.seg[1].bias) u += p.seg[1].bias[rw];
                        p.seg[0].y[((int64_t)m + pair) * p.seg[0].ldy + rw] = (g / (1.0f + expf(-g))) * u;
                    }
                }
            } else if (lane < R * M) {
                const int r = lane / M, m = lane % M;
                float v = 0.f;
                for (int k = 0; k < wk; k++) v += red[warp + k][r * M + m];
                // row[] is register-resident per r; select without dynamic indexing
                int rw = row[0];
#pragma unroll
                for (int rr = 1; rr < R; rr++)
                    if (r == rr) rw = row[rr];
                if (rw < sg.n_rows) {
                    if (sg.bias) v += sg.bias[rw];
                    if (p.residual) v += p.residual[((int64_t)m + pair) * sg.ldy + rw];
                    sg.y[((int64_t)m + pair) * sg.ldy + rw] = v;
                }
            }
        }
        __syncthreads();
    }
}

// ---- exact per-block integer sums (parity instrumentation) -----------------------------------
// Uses the same per-lane integer routines as the GEMV; lanes of a block add their shares with
// integer atomics (exact, order-independent) into zero-initialised outputs.
__global__ void __launch_bounds__(128) block_sums_kernel(uint32_t type, const uint8_t *W,
                                                         const int8_t *aq, const int16_t *abs16,
                                                         int M, int N, int K, int32_t *sumi,
                                                         int32_t *summ) {
    KQ_PDL_ENTER();
    const int nb = K / 256;
    const int lane = threadIdx.x & 31, sub = lane >> 3, c = lane & 7;
    const int64_t warp = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
    const int groups = (nb + 3) / 4;
    const int64_t total = (int64_t)M * N * groups;
    if (warp >= total) return;
    const int gi = (int)(warp % groups);
    const int n = (int)((warp / groups) % N);
    const int m = (int)(warp / groups / N);
    const int blk = gi * 4 + sub;
    if (blk >= nb) return;
    const uint8_t *rp = W + (int64_t)n * kq_device_row_bytes(type, K);
    const int64_t o = ((int64_t)m * N + n) * nb + blk;
    if (type == B200_TYPE_Q4_K) {
        const int e_lo = 64 * (c >> 1) + 16 * (c & 1);
        const uint8_t *b = rp + (int64_t)blk * KQ_Q4K_BYTES;
        const uint4 hdr = __ldg(reinterpret_cast<const uint4 *>(b));
        const uint4 w = kq_ld_stream(b + 16 + 16 * c);
        const Q4Scales sc = q4k_lane_scales(hdr, c);
        const int8_t *a = aq + (int64_t)m * K + blk * 256 + e_lo;
        const int4 alo = *reinterpret_cast<const int4 *>(a);
        const int4 ahi = *reinterpret_cast<const int4 *>(a + 32);
        const int16_t *s16 = abs16 + ((int64_t)m * nb + blk) * 16 + (e_lo >> 4);
        int isum, msum;
        q4k_lane_ints(w, sc, alo, ahi, s16[0], s16[2], isum, msum);
        atomicAdd(&sumi[o], isum);
        if (summ) atomicAdd(&summ[o], msum);
    } else {
        const int h = c >> 2, cc = c & 3, e_lo = 128 * h + 16 * cc;
        const KqQ6Addr qa = kq_q6_addr(nb, blk);
        const uint4 ql = kq_ld_stream(rp + qa.ql + qa.cs * c);
        const uint4 qh = __ldg(reinterpret_cast<const uint4 *>(rp + qa.qh + qa.cs * (2 * h + (cc & 1))));
        const int8_t *scp = reinterpret_cast<const int8_t *>(rp + qa.sc);
        const int8_t *a = aq + (int64_t)m * K + blk * 256 + e_lo;
        const int4 alo = *reinterpret_cast<const int4 *>(a);
        const int4 ahi = *reinterpret_cast<const int4 *>(a + 64);
        const int16_t *s16 = abs16 + ((int64_t)m * nb + blk) * 16 + (e_lo >> 4);
        const int isum = q6k_lane_ints(ql, qh, cc, scp[8 * h + cc], scp[8 * h + 4 + cc], alo, ahi,
                                       s16[0], s16[4]);
        atomicAdd(&sumi[o], isum);
    }
}

int env_int(const char *name, int dflt) {
    const char *v = getenv(name);
    return v ? atoi(v) : dflt;
}

template <int M, int R>
b200_status launch_mr(const GemvParams &p, int wn, int n_pairs, cudaStream_t st) {
    static int ctas_per_sm = 0;
    if (!ctas_per_sm) {
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&ctas_per_sm, gemv_kernel<M, R>, 128, 0);
        if (ctas_per_sm < 1) ctas_per_sm = 1;
    }
    int64_t want = kq_div_up(p.n_rg, wn);
    int64_t cap = (int64_t)kq_sm_count() * ctas_per_sm;
    if (n_pairs > 1) cap = kq_div_up(cap, n_pairs);
    int gx = (int)(want < cap ? want : cap);
    if (gx < 1) gx = 1;
    dim3 grid(gx, n_pairs);
    kq_launch(gemv_kernel<M, R>, grid, 128, 0, st, p);
    KQ_COUNT_LAUNCH();
    KQ_LAUNCH_CHECK();
    return B200_OK;
}

} // namespace

b200_status kq_launch_gemv(const KqGemvSeg *segs, int nseg, const int8_t *q, const float *d,
                           const int16_t *bs, int M, int64_t K, const float *residual,
                           int swiglu_pairs, const KqGemvIndirect *ind, cudaStream_t st, const KqActPrep *prep,
                           KqEmitQ8 *emit) {
    if (emit) emit->done = 0;
    KQ_REQUIRE(nseg >= 1 && nseg <= 3, "gemv: 1..3 segments");
    KQ_REQUIRE(M >= 1 && M <= 8, "gemv: M must be 1..8 (got %d)", M);
    KQ_REQUIRE(K > 0 && K % 256 == 0, "gemv: K must be a positive multiple of 256");
    KQ_REQUIRE(!swiglu_pairs || (nseg == 2 && segs[0].type == segs[1].type &&
                                 segs[0].n_rows == segs[1].n_rows),
               "gemv: swiglu needs two equal segments");
    KQ_REQUIRE(!residual || nseg == 1, "gemv: residual only with one segment");
    if (!(ind && ind->expert_ids) && K % 256 == 0) { // M <= 2: streaming kernel; 3..8 tokens of Q4_K: its tensor-core form
        const b200_status rs = kq_launch_gemv_stream(segs, nseg, q, d, bs, M, K, residual, swiglu_pairs, prep, st, emit);
        if (rs != B200_ERR_UNSUPPORTED) return rs;
        if (M > 2 && nseg > 1 && !swiglu_pairs && !(prep && prep->x)) {
            // a fused projection of mixed types: its Q4_K matrices still take the tensor-core form,
            // the others the plain kernel below
            KqGemvSeg a[3], b[3];
            int na = 0, nb_ = 0;
            for (int i = 0; i < nseg; i++) (segs[i].type == B200_TYPE_Q4_K ? a[na++] : b[nb_++]) = segs[i];
            if (na > 0 && nb_ > 0 && kq_launch_gemv_stream(a, na, q, d, bs, M, K, nullptr, 0, nullptr, st) == B200_OK)
                return kq_launch_gemv(b, nb_, q, d, bs, M, K, nullptr, 0, nullptr, st, nullptr);
        }
    }
    if (prep && prep->x) {
        // the plain kernel wants quantised activations: prepare them into the caller's scratch
        KQ_REQUIRE(q && d && bs, "gemv: activation scratch required");
        b200_status rc = prep->do_norm ? kq_rms_norm(prep->x, prep->norm_w, M, K, prep->eps, nullptr, (int8_t *)q, (float *)d,
                                                     (int16_t *)bs, st, 0)
                                       : b200_quantize_act(prep->x, M, K, (int8_t *)q, (float *)d, (int16_t *)bs, st);
        if (rc != B200_OK) return rc;
    }
    GemvParams p = {};
    const int R = M <= 4 ? 4 : 2;
    const int rows_per_rg = swiglu_pairs ? R / 2 : R;
    int tot = 0;
    for (int i = 0; i < nseg; i++) {
        KQ_REQUIRE(segs[i].type == B200_TYPE_Q4_K || segs[i].type == B200_TYPE_Q6_K,
                   "gemv: weight type %u not supported", segs[i].type);
        KQ_REQUIRE(((uintptr_t)segs[i].W & 15) == 0, "gemv: weights must be 16-byte aligned");
        p.seg[i] = segs[i];
        if (!(swiglu_pairs && i == 1)) tot += (int)kq_div_up(segs[i].n_rows, rows_per_rg);
        p.rg_end[i] = tot;
    }
    KQ_REQUIRE(((uintptr_t)q & 15) == 0, "gemv: activations must be 16-byte aligned");
    p.nseg = swiglu_pairs ? 1 : nseg;
    p.n_rg = tot;
    p.nb = (int)(K / 256);
    p.K = (int)K;
    p.swiglu = swiglu_pairs;
    p.aq = q;
    p.ad = d;
    p.abs16 = bs;
    p.residual = residual;
    int n_pairs = 1;
    if (ind && ind->expert_ids) {
        KQ_REQUIRE(M == 1 && ind->n_pairs >= 1 && ind->act_div >= 1, "gemv: expert mode needs M == 1");
        p.expert_ids = ind->expert_ids;
        p.act_div = ind->act_div;
        n_pairs = ind->n_pairs;
    }
    const int its = (p.nb + 3) / 4;
    int wk = its >= 16 ? 4 : (its >= 8 ? 2 : 1);
    wk = env_int("B200_GEMV_WK", wk);
    if (wk != 1 && wk != 2 && wk != 4) wk = 1;
    p.wk = wk;
    const int wn = 4 / wk;
    switch (M) {
    case 1: return launch_mr<1, 4>(p, wn, n_pairs, st);
    case 2: return launch_mr<2, 4>(p, wn, n_pairs, st);
    case 3: return launch_mr<3, 4>(p, wn, n_pairs, st);
    case 4: return launch_mr<4, 4>(p, wn, n_pairs, st);
    case 5: return launch_mr<5, 2>(p, wn, n_pairs, st);
    case 6: return launch_mr<6, 2>(p, wn, n_pairs, st);
    case 7: return launch_mr<7, 2>(p, wn, n_pairs, st);
    default: return launch_mr<8, 2>(p, wn, n_pairs, st);
    }
}

extern "C" b200_status b200_block_sums(uint32_t type, const void *W, const int8_t *q,
                                       const int16_t *bsum16, int64_t M, int64_t N, int64_t K,
                                       int32_t *sumi, int32_t *summ, void *stream) {
    KQ_REQUIRE(type == B200_TYPE_Q4_K || type == B200_TYPE_Q6_K, "block_sums: type %u", type);
    KQ_REQUIRE(K > 0 && K % 256 == 0 && M > 0 && N > 0, "block_sums: bad shape");
    cudaStream_t st = (cudaStream_t)stream;
    const int64_t nb = K / 256, cnt = M * N * nb;
    KQ_CUDA(cudaMemsetAsync(sumi, 0, cnt * 4, st));
    if (summ) KQ_CUDA(cudaMemsetAsync(summ, 0, cnt * 4, st));
    const int64_t warps = M * N * ((nb + 3) / 4);
    kq_launch(block_sums_kernel, (unsigned)kq_div_up(warps, 4), 128, 0, st, 
        type, (const uint8_t *)W, q, bsum16, (int)M, (int)N, (int)K, sumi, summ);
    KQ_COUNT_LAUNCH();
    KQ_LAUNCH_CHECK();
    return B200_OK;
}
