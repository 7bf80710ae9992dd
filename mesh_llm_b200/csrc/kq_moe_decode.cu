// Expert layer of a decode step (1 .. 8 tokens): the work around the two expert matmuls in two launches
// instead of five.
//
//   moe_router_fused_kernel   RMSNorm of the residual row, its Q8 form for the expert matmuls, the router's
//                             f32 logits (ffn_gate_inp) and, in the last CTA of a token to finish, softmax +
//                             masked top-k + renormalised weights: llama.cpp's build_moe_ffn up to
//                             ggml_argsort_top_k (third_party/llama.cpp/patches/0003 lines 82-108)
//   moe_down_combine_kernel   quantises the SwiGLU outputs of a token's (token, slot) pairs in its prologue,
//                             multiplies each by the down matrix of its expert (MUL_MAT_ID) and leaves
//                             x + sum_s w_s y_s directly: no [pairs x n_embd] intermediate, no combine launch
//
// Every arithmetic step is the one of the separate kernels it replaces (rms_norm_kernel, router_logits_kernel,
// moe_route_kernel, quantize_act_kernel, gemv_kernel in expert mode, moe_combine_kernel), in the same order
// (for expert widths of up to 7 blocks of 256, where the separate matmul does not split rows over warps),
// so the stage's results do not depend on which form ran.
#include "kq_common.cuh"
#include "kq_lanes.cuh"
#include "kq_route.cuh"

namespace {

constexpr int ROUTER_CTAS = 16; // CTAs per token: with 128 experts one expert per warp

__global__ void __launch_bounds__(256) moe_router_fused_kernel(const float *x, const float *norm_w, float eps, const float *Wr,
                                                               int E, int h, int k, const uint8_t *mask, float *rl,
                                                               int32_t *ids, float *wts, int8_t *q, float *d, int16_t *bs,
                                                               unsigned int *counters) {
    KQ_PDL_ENTER();
    extern __shared__ __align__(16) float xn[]; // the normalised row
    __shared__ double part[8];
    __shared__ float s_scale;
    __shared__ int s_last;
    const int row = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float *xr = x + (int64_t)row * h;
    double ss = 0.0; // in double, so that the scale does not depend on the order of the reduction
    for (int i = tid * 4; i < h; i += 1024) {
        const float4 v = *reinterpret_cast<const float4 *>(xr + i);
        ss += (double)v.x * v.x + (double)v.y * v.y + (double)v.z * v.z + (double)v.w * v.w;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (lane == 0) part[warp] = ss;
    __syncthreads();
    if (tid == 0) {
        double t = 0.0;
        for (int i = 0; i < 8; i++) t += part[i];
        s_scale = 1.0f / sqrtf((float)(t / (double)h) + eps);
    }
    __syncthreads();
    const float scale = s_scale;
    const int nb = h / 256;
    for (int b = warp; b < nb; b += 8) {
        const int o = b * 256 + lane * 8;
        const float4 a = *reinterpret_cast<const float4 *>(xr + o);
        const float4 c = *reinterpret_cast<const float4 *>(xr + o + 4);
        float v[8] = {a.x, a.y, a.z, a.w, c.x, c.y, c.z, c.w};
#pragma unroll
        for (int i = 0; i < 8; i++) v[i] = v[i] * scale * norm_w[o + i];
        *reinterpret_cast<float4 *>(xn + o) = make_float4(v[0], v[1], v[2], v[3]);
        *reinterpret_cast<float4 *>(xn + o + 4) = make_float4(v[4], v[5], v[6], v[7]);
        if (blockIdx.x == 0) { // one CTA of the token leaves the Q8 form for the expert matmuls
            const int64_t gb = (int64_t)row * nb + b;
            kq_quantize_block_warp(v, lane, q + gb * 256, d + gb, bs + gb * 16);
        }
    }
    __syncthreads();
    for (int e = blockIdx.x * 8 + warp; e < E; e += gridDim.x * 8) { // one warp per expert
        const float4 *wr = reinterpret_cast<const float4 *>(Wr + (int64_t)e * h);
        const float4 *xv = reinterpret_cast<const float4 *>(xn);
        float acc = 0.f;
        for (int i = lane; i < h / 4; i += 32) {
            const float4 a = __ldg(wr + i), b = xv[i];
            acc += a.x * b.x + a.y * b.y + a.z * b.z + a.w * b.w;
        }
        acc = kq_warp_sum(acc);
        if (lane == 0) rl[(int64_t)row * E + e] = acc;
    }
    // the CTA that finishes a token's logits last routes it
    __threadfence();
    __syncthreads();
    if (tid == 0) s_last = atomicAdd(&counters[row], 1u) == gridDim.x - 1;
    __syncthreads();
    if (s_last && warp == 0) {
        __threadfence();
        kq_route_warp(rl + (int64_t)row * E, E, k, mask, ids + (int64_t)row * k, wts + (int64_t)row * k, lane);
        if (lane == 0) counters[row] = 0u; // ready for the next launch
    }
}

constexpr int DOWN_ROWS = 16; // output rows per CTA: two per warp

template <uint32_t TYPE>
__global__ void __launch_bounds__(256) moe_down_combine_kernel(const uint8_t *W, int64_t expert_stride, const float *hp,
                                                               const int32_t *ids, const float *wts, const float *res, int ku,
                                                               int h, int fe, float *out) {
    KQ_PDL_ENTER();
    extern __shared__ __align__(16) uint8_t sm[];
    const int t = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int nb = fe / 256, nblk = ku * nb;
    int8_t *aq = reinterpret_cast<int8_t *>(sm);                                   // [ku][fe]
    float *ad = reinterpret_cast<float *>(sm + (size_t)ku * fe);                   // [ku][nb]
    int16_t *abs16 = reinterpret_cast<int16_t *>(sm + (size_t)ku * fe + (((size_t)nblk * 4 + 15) & ~(size_t)15)); // [ku][nb][16]
    // the token's pairs are consecutive rows of hp: its ku * nb blocks are one run
    const float *hrow = hp + (int64_t)t * ku * fe;
    for (int b = warp; b < nblk; b += 8) {
        const float4 *xp = reinterpret_cast<const float4 *>(hrow + (int64_t)b * 256 + lane * 8);
        const float4 a = xp[0], c4 = xp[1];
        const float v[8] = {a.x, a.y, a.z, a.w, c4.x, c4.y, c4.z, c4.w};
        kq_quantize_block_warp(v, lane, aq + b * 256, ad + b, abs16 + b * 16);
    }
    __syncthreads();
    const int sub = lane >> 3, c = lane & 7;
    const int64_t stride = kq_device_row_bytes(TYPE, fe);
    for (int rr = 0; rr < 2; rr++) {
        const int n = blockIdx.x * DOWN_ROWS + warp * 2 + rr;
        if (n >= h) break; // the whole warp
        float acc[8];
#pragma unroll
        for (int s = 0; s < 8; s++) acc[s] = 0.f;
        for (int it = 0; it * 4 < nb; it++) {
            const int blk = it * 4 + sub;
            const bool on = blk < nb;
#pragma unroll
            for (int s0 = 0; s0 < 8; s0 += 4) { // four slots' weights in flight at a time
                if (s0 >= ku) break;
                if (TYPE == B200_TYPE_Q4_K) {
                    uint4 hdr[4], w[4];
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        hdr[j] = w[j] = make_uint4(0, 0, 0, 0);
                        if (on && s0 + j < ku) {
                            const uint8_t *b = W + (int64_t)ids[(int64_t)t * ku + s0 + j] * expert_stride + (int64_t)n * stride +
                                               (int64_t)blk * KQ_Q4K_BYTES;
                            hdr[j] = __ldg(reinterpret_cast<const uint4 *>(b));
                            w[j] = kq_ld_stream(b + 16 + 16 * c);
                        }
                    }
                    const int e_lo = 64 * (c >> 1) + 16 * (c & 1);
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        if (on && s0 + j < ku) {
                            const int s = s0 + j;
                            const Q4Scales sc = q4k_lane_scales(hdr[j], c);
                            const int8_t *a = aq + s * fe + blk * 256 + e_lo;
                            const int4 alo = *reinterpret_cast<const int4 *>(a);
                            const int4 ahi = *reinterpret_cast<const int4 *>(a + 32);
                            const float da = ad[s * nb + blk];
                            const int16_t *s16 = abs16 + (s * nb + blk) * 16 + (e_lo >> 4);
                            int isum, msum;
                            q4k_lane_ints(w[j], sc, alo, ahi, s16[0], s16[2], isum, msum);
                            acc[s] = fmaf(sc.d * da, (float)isum, acc[s]);
                            acc[s] = fmaf(-(sc.dmin * da), (float)msum, acc[s]);
                        }
                    }
                } else {
                    const int hh = c >> 2, cc = c & 3;
                    const int e_lo = 128 * hh + 16 * cc;
                    uint4 ql[4], qh[4];
                    int scl[4], sch[4];
                    float dw[4];
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        ql[j] = qh[j] = make_uint4(0, 0, 0, 0);
                        scl[j] = sch[j] = 0;
                        dw[j] = 0.f;
                        if (on && s0 + j < ku) {
                            const uint8_t *rp = W + (int64_t)ids[(int64_t)t * ku + s0 + j] * expert_stride + (int64_t)n * stride;
                            const KqQ6Addr qa = kq_q6_addr(nb, blk);
                            ql[j] = kq_ld_stream(rp + qa.ql + qa.cs * c);
                            qh[j] = __ldg(reinterpret_cast<const uint4 *>(rp + qa.qh + qa.cs * (2 * hh + (cc & 1))));
                            const int8_t *scp = reinterpret_cast<const int8_t *>(rp + qa.sc);
                            scl[j] = scp[8 * hh + cc];
                            sch[j] = scp[8 * hh + 4 + cc];
                            dw[j] = kq_h2f(*reinterpret_cast<const uint16_t *>(rp + qa.d));
                        }
                    }
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        if (on && s0 + j < ku) {
                            const int s = s0 + j;
                            const int8_t *a = aq + s * fe + blk * 256 + e_lo;
                            const int4 alo = *reinterpret_cast<const int4 *>(a);
                            const int4 ahi = *reinterpret_cast<const int4 *>(a + 64);
                            const float da = ad[s * nb + blk];
                            const int16_t *s16 = abs16 + (s * nb + blk) * 16 + (e_lo >> 4);
                            const int isum = q6k_lane_ints(ql[j], qh[j], cc, scl[j], sch[j], alo, ahi, s16[0], s16[4]);
                            acc[s] = fmaf(dw[j] * da, (float)isum, acc[s]);
                        }
                    }
                }
            }
        }
        // per slot the full dot product first, then the weighted sum in slot order on top of the residual
        float y = 0.f;
#pragma unroll
        for (int s = 0; s < 8; s++) {
            if (s < ku) {
                const float v = kq_warp_sum(acc[s]);
                y += wts[(int64_t)t * ku + s] * v;
            }
        }
        if (lane == 0) out[(int64_t)t * h + n] = res[(int64_t)t * h + n] + y;
    }
}

} // namespace

// RMSNorm + Q8 + router logits + routing of `rows` tokens.  counters: rows zero-initialised words that
// the kernel leaves at zero.  Returns B200_ERR_UNSUPPORTED (nothing launched) for shapes outside its reach.
b200_status kq_moe_router_fused(const float *x, const float *norm_w, float eps, const float *router_w, int rows, int E, int h,
                                int k, const uint8_t *mask, float *rl, int32_t *ids, float *wts, int8_t *q, float *d,
                                int16_t *bs, unsigned int *counters, cudaStream_t st) {
    if (rows < 1 || h % 256 != 0 || h > 8192 || E < 1 || E > 256 || k < 1 || k > 32 || k > E || !norm_w) return B200_ERR_UNSUPPORTED;
    KQ_CUDA(kq_launch(moe_router_fused_kernel, dim3(ROUTER_CTAS, rows), dim3(256), (size_t)h * 4, st, x, norm_w, eps, router_w, E, h,
                      k, mask, rl, ids, wts, q, d, bs, counters));
    KQ_COUNT_LAUNCH();
    KQ_LAUNCH_CHECK();
    return B200_OK;
}

// out[t] = res[t] + sum_s wts[t][s] * (W[ids[t][s]] . quantised(hp[t * ku + s])) for `rows` tokens
b200_status kq_moe_down_combine(uint32_t type, const uint8_t *W, int64_t expert_stride, const float *hp, const int32_t *ids,
                                const float *wts, const float *res, int rows, int ku, int h, int fe, float *out,
                                cudaStream_t st) {
    if (rows < 1 || ku < 1 || ku > 8 || fe % 256 != 0 || (type != B200_TYPE_Q4_K && type != B200_TYPE_Q6_K)) return B200_ERR_UNSUPPORTED;
    const int nblk = ku * (fe / 256);
    const size_t smem = (size_t)ku * fe + (((size_t)nblk * 4 + 15) & ~(size_t)15) + (size_t)nblk * 32;
    if (smem > 48 * 1024) return B200_ERR_UNSUPPORTED;
    const dim3 grid((unsigned)kq_div_up(h, DOWN_ROWS), rows);
    if (type == B200_TYPE_Q4_K)
        KQ_CUDA(kq_launch(moe_down_combine_kernel<B200_TYPE_Q4_K>, grid, dim3(256), smem, st, W, expert_stride, hp, ids, wts, res, ku, h,
                          fe, out));
    else
        KQ_CUDA(kq_launch(moe_down_combine_kernel<B200_TYPE_Q6_K>, grid, dim3(256), smem, st, W, expert_stride, hp, ids, wts, res, ku, h,
                          fe, out));
    KQ_COUNT_LAUNCH();
    KQ_LAUNCH_CHECK();
    return B200_OK;
}
