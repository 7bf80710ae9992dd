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
    KQ_PDL_TRIGGER();
    extern __shared__ __align__(16) float xn[]; // the normalised row
    __shared__ double part[8];
    __shared__ float s_scale;
    __shared__ int s_last;
    const int row = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    // The router's weights do not depend on the kernel before: the first 2048 of this warp's first expert
    // row are requested before the dependency wait and fly during the norm.
    constexpr int PRE = 16;
    float4 wpre[PRE];
    const int e_first = blockIdx.x * 8 + warp, n4 = h / 4;
    if (e_first < E) {
        const float4 *wr = reinterpret_cast<const float4 *>(Wr + (int64_t)e_first * h);
#pragma unroll
        for (int j = 0; j < PRE; j++)
            if (lane + 32 * j < n4) wpre[j] = __ldg(wr + lane + 32 * j);
    }
    KQ_PDL_WAIT();
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
    for (int e = e_first; e < E; e += gridDim.x * 8) { // one warp per expert
        const float4 *wr = reinterpret_cast<const float4 *>(Wr + (int64_t)e * h);
        const float4 *xv = reinterpret_cast<const float4 *>(xn);
        float acc = 0.f;
        int i0 = lane;
        if (e == e_first) { // the part requested ahead; the sum keeps its order
#pragma unroll
            for (int j = 0; j < PRE; j++)
                if (lane + 32 * j < n4) {
                    const float4 b = xv[lane + 32 * j];
                    acc += wpre[j].x * b.x + wpre[j].y * b.y + wpre[j].z * b.z + wpre[j].w * b.w;
                }
            i0 = lane + 32 * PRE;
        }
        for (; i0 < n4; i0 += 32 * 8) { // eight loads in flight per lane
            float4 a[8];
#pragma unroll
            for (int j = 0; j < 8; j++)
                if (i0 + 32 * j < n4) a[j] = __ldg(wr + i0 + 32 * j);
#pragma unroll
            for (int j = 0; j < 8; j++)
                if (i0 + 32 * j < n4) {
                    const float4 b = xv[i0 + 32 * j];
                    acc += a[j].x * b.x + a[j].y * b.y + a[j].z * b.z + a[j].w * b.w;
                }
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

constexpr int DOWN_ROWS = 8; // output rows per CTA: one per warp

// the lane's share of one block of one (row, slot): requested early, consumed after the prologue
template <uint32_t TYPE>
struct LaneBlock;
template <>
struct LaneBlock<B200_TYPE_Q4_K> {
    uint4 hdr, w;
    __device__ __forceinline__ void load(const uint8_t *rowp, int nb, int blk, int c) {
        const uint8_t *b = rowp + (int64_t)blk * KQ_Q4K_BYTES;
        hdr = __ldg(reinterpret_cast<const uint4 *>(b));
        w = kq_ld_stream(b + 16 + 16 * c);
    }
    __device__ __forceinline__ float dot(const int8_t *aq, float da, const int16_t *s16blk, int c, float acc) const {
        const int e_lo = 64 * (c >> 1) + 16 * (c & 1);
        const Q4Scales sc = q4k_lane_scales(hdr, c);
        const int4 alo = *reinterpret_cast<const int4 *>(aq + e_lo);
        const int4 ahi = *reinterpret_cast<const int4 *>(aq + e_lo + 32);
        const int16_t *s16 = s16blk + (e_lo >> 4);
        int isum, msum;
        q4k_lane_ints(w, sc, alo, ahi, s16[0], s16[2], isum, msum);
        acc = fmaf(sc.d * da, (float)isum, acc);
        return fmaf(-(sc.dmin * da), (float)msum, acc);
    }
};
template <>
struct LaneBlock<B200_TYPE_Q6_K> {
    uint4 ql, qh;
    int scl, sch;
    float dw;
    __device__ __forceinline__ void load(const uint8_t *rowp, int nb, int blk, int c) {
        const int hh = c >> 2, cc = c & 3;
        const KqQ6Addr qa = kq_q6_addr(nb, blk);
        ql = kq_ld_stream(rowp + qa.ql + qa.cs * c);
        qh = __ldg(reinterpret_cast<const uint4 *>(rowp + qa.qh + qa.cs * (2 * hh + (cc & 1))));
        const int8_t *scp = reinterpret_cast<const int8_t *>(rowp + qa.sc);
        scl = scp[8 * hh + cc];
        sch = scp[8 * hh + 4 + cc];
        dw = kq_h2f(*reinterpret_cast<const uint16_t *>(rowp + qa.d));
    }
    __device__ __forceinline__ float dot(const int8_t *aq, float da, const int16_t *s16blk, int c, float acc) const {
        const int hh = c >> 2, cc = c & 3;
        const int e_lo = 128 * hh + 16 * cc;
        const int4 alo = *reinterpret_cast<const int4 *>(aq + e_lo);
        const int4 ahi = *reinterpret_cast<const int4 *>(aq + e_lo + 64);
        const int16_t *s16 = s16blk + (e_lo >> 4);
        const int isum = q6k_lane_ints(ql, qh, cc, scl, sch, alo, ahi, s16[0], s16[4]);
        return fmaf(dw * da, (float)isum, acc);
    }
};

// gate and up rows of the experts chosen for each (token, slot) pair, SwiGLU applied: one warp per output
// element (its gate row and its up row), all of the rows' blocks requested at once.  grid (fe / 4, pairs).
template <uint32_t TYPE>
__global__ void __launch_bounds__(128) moe_gate_up_kernel(const uint8_t *Wg, const uint8_t *Wu, int64_t expert_stride,
                                                          const int8_t *aq, const float *ad, const int16_t *abs16,
                                                          const int32_t *ids, int ku, int K, int fe, float *hp) {
    KQ_PDL_ENTER();
    const int pair = blockIdx.y, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int j = blockIdx.x * 4 + warp;
    if (j >= fe) return; // the whole warp
    const int nb = K / 256, sub = lane >> 3, c = lane & 7;
    const int64_t stride = kq_device_row_bytes(TYPE, K);
    const int64_t off = (int64_t)ids[pair] * expert_stride + (int64_t)j * stride;
    const int arow = pair / ku;
    const int8_t *a_row = aq + (int64_t)arow * K;
    const float *d_row = ad + (int64_t)arow * nb;
    const int16_t *s_row = abs16 + (int64_t)arow * nb * 16;
    float g = 0.f, u = 0.f;
    for (int it0 = 0; it0 * 4 < nb; it0 += 2) { // two steps of four blocks in flight for each of the two rows
        LaneBlock<TYPE> lg[2], lu[2];
#pragma unroll
        for (int i = 0; i < 2; i++) {
            const int blk = (it0 + i) * 4 + sub;
            if (blk < nb) {
                lg[i].load(Wg + off, nb, blk, c);
                lu[i].load(Wu + off, nb, blk, c);
            }
        }
#pragma unroll
        for (int i = 0; i < 2; i++) {
            const int blk = (it0 + i) * 4 + sub;
            if (blk < nb) {
                g = lg[i].dot(a_row + blk * 256, d_row[blk], s_row + blk * 16, c, g);
                u = lu[i].dot(a_row + blk * 256, d_row[blk], s_row + blk * 16, c, u);
            }
        }
    }
    g = kq_warp_sum(g);
    u = kq_warp_sum(u);
    if (lane == 0) hp[(int64_t)pair * fe + j] = (g / (1.0f + expf(-g))) * u;
}

template <uint32_t TYPE>
__global__ void __launch_bounds__(256, 2) moe_down_combine_kernel(const uint8_t *W, int64_t expert_stride, const float *hp,
                                                               const int32_t *ids, const float *wts, const float *res, int ku,
                                                               int h, int fe, float *out) {
    KQ_PDL_ENTER();
    extern __shared__ __align__(16) uint8_t sm[];
    const int t = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int nb = fe / 256, nblk = ku * nb;
    int8_t *aq = reinterpret_cast<int8_t *>(sm);                                   // [ku][fe]
    float *ad = reinterpret_cast<float *>(sm + (size_t)ku * fe);                   // [ku][nb]
    int16_t *abs16 = reinterpret_cast<int16_t *>(sm + (size_t)ku * fe + (((size_t)nblk * 4 + 15) & ~(size_t)15)); // [ku][nb][16]
    const int sub = lane >> 3, c = lane & 7;
    const int64_t stride = kq_device_row_bytes(TYPE, fe);
    const int n = blockIdx.x * DOWN_ROWS + warp; // this warp's output row
    const bool row_on = n < h;
    // the first four blocks of every slot's row are requested before anything else: they fly while the
    // prologue quantises the activations
    const uint8_t *rowp[8];
    LaneBlock<TYPE> lb[8];
#pragma unroll
    for (int s = 0; s < 8; s++) {
        rowp[s] = nullptr;
        if (s < ku && row_on) rowp[s] = W + (int64_t)ids[(int64_t)t * ku + s] * expert_stride + (int64_t)n * stride;
    }
#pragma unroll
    for (int s = 0; s < 8; s++)
        if (s < ku && row_on && sub < nb) lb[s].load(rowp[s], nb, sub, c);
    // the token's pairs are consecutive rows of hp: its ku * nb blocks are one run
    const float *hrow = hp + (int64_t)t * ku * fe;
    for (int b = warp; b < nblk; b += 8) {
        const float4 *xp = reinterpret_cast<const float4 *>(hrow + (int64_t)b * 256 + lane * 8);
        const float4 a = xp[0], c4 = xp[1];
        const float v[8] = {a.x, a.y, a.z, a.w, c4.x, c4.y, c4.z, c4.w};
        kq_quantize_block_warp(v, lane, aq + b * 256, ad + b, abs16 + b * 16);
    }
    __syncthreads();
    if (!row_on) return; // the whole warp
    float acc[8];
#pragma unroll
    for (int s = 0; s < 8; s++) acc[s] = 0.f;
    for (int it = 0; it * 4 < nb; it++) {
        const int blk = it * 4 + sub;
        if (it > 0) {
#pragma unroll
            for (int s = 0; s < 8; s++)
                if (s < ku && blk < nb) lb[s].load(rowp[s], nb, blk, c);
        }
        if (blk < nb) {
#pragma unroll
            for (int s = 0; s < 8; s++)
                if (s < ku) acc[s] = lb[s].dot(aq + s * fe + blk * 256, ad[s * nb + blk], abs16 + (s * nb + blk) * 16, c, acc[s]);
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

// hp[pair] = swiglu(Wg[ids[pair]] . a, Wu[ids[pair]] . a) with a = the Q8 activations of token pair / ku
b200_status kq_moe_gate_up(uint32_t type, const uint8_t *Wg, const uint8_t *Wu, int64_t expert_stride, const int8_t *aq,
                           const float *ad, const int16_t *abs16, const int32_t *ids, int pairs, int ku, int K, int fe, float *hp,
                           cudaStream_t st) {
    if (pairs < 1 || pairs > 65535 || ku < 1 || K % 256 != 0 || (type != B200_TYPE_Q4_K && type != B200_TYPE_Q6_K)) return B200_ERR_UNSUPPORTED;
    const dim3 grid((unsigned)kq_div_up(fe, 4), pairs);
    if (type == B200_TYPE_Q4_K)
        KQ_CUDA(kq_launch(moe_gate_up_kernel<B200_TYPE_Q4_K>, grid, dim3(128), 0, st, Wg, Wu, expert_stride, aq, ad, abs16, ids, ku, K, fe, hp));
    else
        KQ_CUDA(kq_launch(moe_gate_up_kernel<B200_TYPE_Q6_K>, grid, dim3(128), 0, st, Wg, Wu, expert_stride, aq, ad, abs16, ids, ku, K, fe, hp));
    KQ_COUNT_LAUNCH();
    KQ_LAUNCH_CHECK();
    return B200_OK;
}
