// The small ops around the quantised contraction: RoPE, KV-cache write, causal attention over an
// f16 KV cache (split-KV, GQA-aware), SwiGLU, adds, embedding rows, argmax and the MoE router.
// All of them are bandwidth-trivial next to the weight stream; they are written to cost few
// launches and to read the KV cache once per group of query heads.
#include "kq_common.cuh"
#include "kq_route.cuh"
#include "kq_kvq.cuh"

#include <math.h>
#include <stdlib.h>

b200_status kq_attention_prefill_tc(const float *q, const uint16_t *kc, const uint16_t *vc, int n_seq, int T,
                                    const int32_t *pos0_dev, int pos0, int n_head, int n_kv, int hd, int64_t seq_stride,
                                    float *out, cudaStream_t st);
b200_status kq_attention_prefill_mma(const float *q, const uint16_t *kc, const uint16_t *vc, int n_seq, int T,
                                     const int32_t *pos0_dev, int pos0, int n_head, int n_kv, int hd, int64_t seq_stride,
                                     float *out, KqKvTypes kvt, cudaStream_t st);

namespace {

struct RopeTable {
    float inv_freq[128]; // head_dim / 2 entries used
};

// q: [rows][n_head][hd] f32 rotated in place.  k (optional): [rows][n_kv][hd] f32 rotated and
// stored into the cache at the row's position (f16, or q8_0 / q4_0 rows); v likewise without
// rotation.  seq_stride counts cache elements (positions x kv heads x hd) per sequence.
__global__ void rope_store_kernel(float *q, const float *k, const float *v, const int32_t *pos,
                                  const int32_t *pos0_dev, int pos0, int T, int n_head, int n_kv, int hd, int neox,
                                  RopeTable tab, __half *k_cache, __half *v_cache,
                                  int64_t seq_stride, KqKvTypes kvt) {
    KQ_PDL_ENTER();
    const int row = blockIdx.x; // row = seq * T + t
    const int seq = row / T, t = row % T;
    const int p = pos ? pos[row] : (pos0_dev ? *pos0_dev : pos0) + t;
    const int half = hd / 2;
    const bool kq = k && kvt.k != KQ_KV_F16, vq = v && kvt.v != KQ_KV_F16;
    if (kq || vq) {
        // quantised rows: one warp per block of 32 values (lane = value), the rotation recomputed per value
        const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5, nb = hd / 32;
        const int64_t cache_row = seq * (seq_stride / hd) + (int64_t)p * n_kv;
        for (int u = warp; u < (kq ? n_kv * nb : 0); u += nw) {
            const int kh = u / nb, blk = u % nb, e = blk * 32 + lane;
            const float *vv = k + ((int64_t)row * n_kv + kh) * hd;
            const int f = neox ? e % half : e / 2;
            const float ang = (float)p * tab.inv_freq[f];
            const float c = cosf(ang), s = sinf(ang);
            const float a = vv[neox ? f : 2 * f], b = vv[neox ? f + half : 2 * f + 1];
            const bool first = neox ? e < half : !(e & 1);
            const float val = first ? a * c - b * s : a * s + b * c;
            uint8_t *dst = reinterpret_cast<uint8_t *>(k_cache) + (cache_row + kh) * kq_kv_row_bytes(kvt.k, hd);
            kq_kv_store_block(kvt.k, val, dst, hd, blk, lane);
        }
        for (int u = warp; u < (vq ? n_kv * nb : 0); u += nw) {
            const int kh = u / nb, blk = u % nb, e = blk * 32 + lane;
            uint8_t *dst = reinterpret_cast<uint8_t *>(v_cache) + (cache_row + kh) * kq_kv_row_bytes(kvt.v, hd);
            kq_kv_store_block(kvt.v, v[((int64_t)row * n_kv + kh) * hd + e], dst, hd, blk, lane);
        }
    }
    const int n_rot = (n_head + (k && !kq ? n_kv : 0)) * half;
    for (int i = threadIdx.x; i < n_rot; i += blockDim.x) {
        const int hidx = i / half, f = i % half;
        const float ang = (float)p * tab.inv_freq[f];
        const float c = cosf(ang), s = sinf(ang);
        const int i0 = neox ? f : 2 * f, i1 = neox ? f + half : 2 * f + 1;
        if (hidx < n_head) {
            float *vv = q + ((int64_t)row * n_head + hidx) * hd;
            const float a = vv[i0], b = vv[i1];
            vv[i0] = a * c - b * s;
            vv[i1] = a * s + b * c;
        } else {
            const int kh = hidx - n_head;
            const float *vv = k + ((int64_t)row * n_kv + kh) * hd;
            __half *dst = k_cache + seq * seq_stride + ((int64_t)p * n_kv + kh) * hd;
            const float a = vv[i0], b = vv[i1];
            dst[i0] = __float2half_rn(a * c - b * s);
            dst[i1] = __float2half_rn(a * s + b * c);
        }
    }
    if (v && !vq) {
        const int n = n_kv * hd;
        __half *dst = v_cache + seq * seq_stride + (int64_t)p * n;
        for (int i = threadIdx.x; i < n; i += blockDim.x)
            dst[i] = __float2half_rn(v[(int64_t)row * n + i]);
    }
}

// ---- attention ---------------------------------------------------------------------------------
// grid (n_kv, n_split, rows); 128 threads.  A CTA serves the G = n_head / n_kv query heads that
// share one KV head, for one query row, over one slice of the positions.  Inside a warp each lane
// scores one position against all G heads (K row read once), the tile's probabilities go through
// shared memory, and each lane accumulates 4 of the 128 output dims for all G heads.
template <int HD, int G>
__global__ void __launch_bounds__(128) attention_kernel(const float *q,
                                                        const __half *kc,
                                                        const __half *vc, int T,
                                                        const int32_t *pos0_dev, int pos0, int n_head, int n_kv, int64_t seq_stride,
                                                        int n_split, float scale, float *out,
                                                        float *part_o, float *part_ml) {
    KQ_PDL_ENTER();
    constexpr int DPL = HD / 32; // output dims per lane
    __shared__ float q_s[G][HD];
    __shared__ float p_s[4][G][32];
    __shared__ float o_s[4][G][HD];
    __shared__ float ml_s[4][G][2];
    const int kh = blockIdx.x, split = blockIdx.y, row = blockIdx.z;
    const int seq = row / T, t = row % T;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int L = (pos0_dev ? *pos0_dev : pos0) + t + 1;
    int chunk = (L + n_split - 1) / n_split;
    chunk = (chunk + 127) / 128 * 128;
    const int p_begin = split * chunk, p_end = min(L, p_begin + chunk);

    for (int i = threadIdx.x; i < G * HD; i += 128)
        q_s[i / HD][i % HD] = q[((int64_t)row * n_head + kh * G + i / HD) * HD + i % HD] * scale;
    __syncthreads();

    const __half *kbase = kc + seq * seq_stride + (int64_t)kh * HD;
    const __half *vbase = vc + seq * seq_stride + (int64_t)kh * HD;
    const int64_t pstride = (int64_t)n_kv * HD;

    float m[G], l[G], o[G][DPL];
#pragma unroll
    for (int g = 0; g < G; g++) {
        m[g] = -INFINITY;
        l[g] = 0.f;
#pragma unroll
        for (int i = 0; i < DPL; i++) o[g][i] = 0.f;
    }
    for (int tb = p_begin + warp * 32; tb < p_end; tb += 128) {
        const int p = tb + lane;
        const bool valid = p < p_end;
        float s[G];
#pragma unroll
        for (int g = 0; g < G; g++) s[g] = 0.f;
        if (valid) {
            // the whole K row is requested up front (8 loads in flight per lane), q comes from
            // shared memory as float4 broadcasts
            const uint4 *kr = reinterpret_cast<const uint4 *>(kbase + p * pstride);
#pragma unroll
            for (int c0 = 0; c0 < HD / 8; c0 += 8) {
                uint4 raw[8];
#pragma unroll
                for (int u = 0; u < 8; u++) raw[u] = kr[c0 + u];
#pragma unroll
                for (int u = 0; u < 8; u++) {
                    const __half2 *h2 = reinterpret_cast<const __half2 *>(&raw[u]);
                    const float2 f0 = __half22float2(h2[0]), f1 = __half22float2(h2[1]), f2 = __half22float2(h2[2]),
                                 f3 = __half22float2(h2[3]);
#pragma unroll
                    for (int g = 0; g < G; g++) {
                        const float4 qa = *reinterpret_cast<const float4 *>(&q_s[g][(c0 + u) * 8]);
                        const float4 qb = *reinterpret_cast<const float4 *>(&q_s[g][(c0 + u) * 8 + 4]);
                        float t = s[g];
                        t = fmaf(qa.x, f0.x, t); t = fmaf(qa.y, f0.y, t); t = fmaf(qa.z, f1.x, t); t = fmaf(qa.w, f1.y, t);
                        t = fmaf(qb.x, f2.x, t); t = fmaf(qb.y, f2.y, t); t = fmaf(qb.z, f3.x, t); t = fmaf(qb.w, f3.y, t);
                        s[g] = t;
                    }
                }
            }
        }
#pragma unroll
        for (int g = 0; g < G; g++) {
            const float sv = valid ? s[g] : -INFINITY;
            const float mt = kq_warp_max(sv);
            const float mn = fmaxf(m[g], mt);
            const float alpha = (m[g] == -INFINITY) ? 0.f : expf(m[g] - mn);
            const float pv = valid ? expf(sv - mn) : 0.f;
            l[g] = l[g] * alpha + kq_warp_sum(pv);
            m[g] = mn;
#pragma unroll
            for (int i = 0; i < DPL; i++) o[g][i] *= alpha;
            p_s[warp][g][lane] = pv;
        }
        __syncwarp();
        const int cnt = min(32, p_end - tb);
        // V rows in batches of 8: all loads of a batch are issued before the first is used
        for (int j0 = 0; j0 < cnt; j0 += 8) {
            float vf[8][DPL];
#pragma unroll
            for (int u = 0; u < 8; u++) {
                const bool in = j0 + u < cnt;
                const __half *vr = vbase + (tb + (in ? j0 + u : 0)) * pstride + lane * DPL;
                if (DPL == 4) {
                    const uint2 raw = in ? *reinterpret_cast<const uint2 *>(vr) : make_uint2(0u, 0u);
                    const __half2 *h2 = reinterpret_cast<const __half2 *>(&raw);
                    const float2 a = __half22float2(h2[0]), b = __half22float2(h2[1]);
                    vf[u][0] = a.x; vf[u][1] = a.y; vf[u][2] = b.x; vf[u][3] = b.y;
                } else {
#pragma unroll
                    for (int i = 0; i < DPL; i++) vf[u][i] = in ? __half2float(vr[i]) : 0.f;
                }
            }
#pragma unroll
            for (int u = 0; u < 8; u++) {
                if (j0 + u < cnt) {
#pragma unroll
                    for (int g = 0; g < G; g++) {
                        const float pv = p_s[warp][g][j0 + u];
#pragma unroll
                        for (int i = 0; i < DPL; i++) o[g][i] = fmaf(pv, vf[u][i], o[g][i]);
                    }
                }
            }
        }
        __syncwarp();
    }
    // combine the 4 warps of the CTA
#pragma unroll
    for (int g = 0; g < G; g++) {
#pragma unroll
        for (int i = 0; i < DPL; i++) o_s[warp][g][lane * DPL + i] = o[g][i];
        if (lane == 0) {
            ml_s[warp][g][0] = m[g];
            ml_s[warp][g][1] = l[g];
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < G * HD; i += 128) {
        const int g = i / HD, dim = i % HD;
        float mm = -INFINITY;
        for (int w = 0; w < 4; w++) mm = fmaxf(mm, ml_s[w][g][0]);
        float acc = 0.f, ll = 0.f;
        for (int w = 0; w < 4; w++) {
            const float mw = ml_s[w][g][0];
            const float wgt = (mw == -INFINITY) ? 0.f : expf(mw - mm);
            acc += wgt * o_s[w][g][dim];
            ll += wgt * ml_s[w][g][1];
        }
        const int head = kh * G + g;
        if (n_split == 1) {
            out[((int64_t)row * n_head + head) * HD + dim] = acc / ll;
        } else {
            const int64_t pi = ((int64_t)row * n_head + head) * n_split + split;
            part_o[pi * HD + dim] = acc;
            if (dim == 0) {
                part_ml[pi * 2] = mm;
                part_ml[pi * 2 + 1] = ll;
            }
        }
    }
}

template <int HD>
__global__ void attention_combine_kernel(const float *part_o, const float *part_ml, int n_head,
                                         int n_split, float *out) {
    KQ_PDL_ENTER();
    const int head = blockIdx.x, row = blockIdx.y, dim = threadIdx.x;
    const int64_t base = ((int64_t)row * n_head + head) * n_split;
    float mm = -INFINITY;
    for (int s = 0; s < n_split; s++) mm = fmaxf(mm, part_ml[(base + s) * 2]);
    float acc = 0.f, ll = 0.f;
    for (int s = 0; s < n_split; s++) {
        const float ms = part_ml[(base + s) * 2];
        const float wgt = (ms == -INFINITY) ? 0.f : expf(ms - mm);
        acc += wgt * part_o[(base + s) * HD + dim];
        ll += wgt * part_ml[(base + s) * 2 + 1];
    }
    out[((int64_t)row * n_head + head) * HD + dim] = acc / ll;
}

__global__ void swiglu_kernel(const float *g, const float *u, int64_t n, float *y) {
    KQ_PDL_ENTER();
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) {
        const float a = g[i];
        y[i] = (a / (1.0f + expf(-a))) * u[i];
    }
}
__global__ void add_kernel(const float *a, const float *b, int64_t n, float *y) {
    KQ_PDL_ENTER();
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) y[i] = a[i] + b[i];
}
__global__ void add_bias_kernel(float *y, const float *bias, int64_t total, int64_t n) {
    KQ_PDL_ENTER();
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < total) y[i] += bias[i % n];
}
__global__ void cpy_f16_kernel(const float *x, int64_t n, __half *y) {
    KQ_PDL_ENTER();
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) y[i] = __float2half_rn(x[i]);
}

// embedding rows: one thread per element
__global__ void get_rows_kernel(uint32_t type, const uint8_t *W, const int32_t *ids, int64_t T, int K,
                                float *y) {
    KQ_PDL_ENTER();
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= T * K) return;
    const int64_t t = i / K;
    const int e = (int)(i % K), b = e >> 8, j = e & 255;
    const int nb = K >> 8;
    const uint8_t *rp = W + (int64_t)ids[t] * kq_device_row_bytes(type, K);
    float v;
    if (type == B200_TYPE_Q4_K) {
        const uint8_t *blk = rp + (int64_t)b * KQ_Q4K_BYTES;
        const float d = kq_h2f(*reinterpret_cast<const uint16_t *>(blk));
        const float dmin = kq_h2f(*reinterpret_cast<const uint16_t *>(blk + 2));
        const uint8_t *s = blk + 4;
        const int sb = j >> 5;
        int sc, mn;
        if (sb < 4) {
            sc = s[sb] & 63;
            mn = s[sb + 4] & 63;
        } else {
            sc = (s[sb + 4] & 0xF) | ((s[sb - 4] >> 6) << 4);
            mn = (s[sb + 4] >> 4) | ((s[sb] >> 6) << 4);
        }
        const uint8_t qb = blk[16 + 32 * (j >> 6) + (j & 31)];
        const int qv = (j & 32) ? (qb >> 4) : (qb & 0xF);
        v = d * (float)sc * (float)qv - dmin * (float)mn;
    } else if (type == B200_TYPE_Q6_K) {
        const int h = j >> 7, r = j & 127, k = r >> 5, i5 = r & 31;
        const KqQ6Addr qa = kq_q6_addr(nb, b);
        const int nl = 64 * h + 32 * (k & 1) + i5, nh = 32 * h + i5; // byte inside the block's ql / qh
        const uint8_t lb = rp[qa.ql + (nl >> 4) * qa.cs + (nl & 15)];
        const uint8_t hb = rp[qa.qh + (nh >> 4) * qa.cs + (nh & 15)];
        const int lo = (k & 2) ? (lb >> 4) : (lb & 0xF);
        const int qv = (lo | (((hb >> (2 * k)) & 3) << 4)) - 32;
        const int sc = (int8_t)rp[qa.sc + (j >> 4)];
        const float d = kq_h2f(*reinterpret_cast<const uint16_t *>(rp + qa.d));
        v = d * (float)sc * (float)qv;
    } else {
        v = reinterpret_cast<const float *>(rp)[e];
    }
    y[i] = v;
}

__global__ void __launch_bounds__(1024) argmax_kernel(const float *x, int64_t n, int32_t *idx) {
    KQ_PDL_ENTER();
    __shared__ float bv[32];
    __shared__ int bi[32];
    const float *xr = x + (int64_t)blockIdx.x * n;
    float best = -INFINITY;
    int besti = 0x7fffffff;
    for (int64_t i = threadIdx.x; i < n; i += blockDim.x) {
        const float v = xr[i];
        if (v > best || (v == best && (int)i < besti)) { best = v; besti = (int)i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, besti, o);
        if (ov > best || (ov == best && oi < besti)) { best = ov; besti = oi; }
    }
    if ((threadIdx.x & 31) == 0) { bv[threadIdx.x >> 5] = best; bi[threadIdx.x >> 5] = besti; }
    __syncthreads();
    if (threadIdx.x < 32) {
        best = threadIdx.x < (blockDim.x >> 5) ? bv[threadIdx.x] : -INFINITY;
        besti = threadIdx.x < (blockDim.x >> 5) ? bi[threadIdx.x] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, besti, o);
            if (ov > best || (ov == best && oi < besti)) { best = ov; besti = oi; }
        }
        if (threadIdx.x == 0) idx[blockIdx.x] = besti == 0x7fffffff ? 0 : besti;
    }
}

// router: one warp per token; E <= 256, k <= 32.  probs = softmax over all experts; the choice is made
// on probs + mask (0 for an allowed expert, -inf for a masked one: third_party/llama.cpp/patches/0003
// lines 82-108), ties to the lower index; the weights are the unmasked probs of the chosen experts,
// renormalised.  mask: one byte per expert (1 = allowed) or null.
__global__ void __launch_bounds__(128) moe_route_kernel(const float *logits, int64_t T, int E, int k,
                                                        const uint8_t *mask, int32_t *ids, float *w) {
    KQ_PDL_ENTER();
    const int lane = threadIdx.x & 31;
    const int64_t t = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
    if (t >= T) return;
    kq_route_warp(logits + t * E, E, k, mask, ids + t * k, w + t * k, lane);
}

template <int HD>
b200_status launch_attention_g(int G, dim3 grid, const float *q, const __half *kc, const __half *vc,
                               int T, const int32_t *pos0_dev, int pos0, int n_head, int n_kv, int64_t seq_stride, int n_split,
                               float scale, float *out, float *po, float *pml, cudaStream_t st) {
#define KQ_ATT(GG)                                                                                  \
    kq_launch(attention_kernel<HD, GG>, grid, 128, 0, st, q, kc, vc, T, pos0_dev, pos0, n_head, n_kv, seq_stride, \
                                                   n_split, scale, out, po, pml)
    switch (G) {
    case 1: KQ_ATT(1); break;
    case 2: KQ_ATT(2); break;
    case 4: KQ_ATT(4); break;
    case 5: KQ_ATT(5); break;
    case 8: KQ_ATT(8); break;
    default: kq_set_error("attention: %d query heads per KV head not supported", G); return B200_ERR_UNSUPPORTED;
    }
#undef KQ_ATT
    KQ_COUNT_LAUNCH();
    KQ_LAUNCH_CHECK();
    return B200_OK;
}

} // namespace

int kq_attention_splits(int64_t rows, int n_kv, int64_t L) {
    const int64_t ctas = rows * n_kv;
    int64_t want = kq_div_up(2 * (int64_t)kq_sm_count(), ctas);
    // the cap follows the context length in powers of two, so a decode loop that captured its
    // launch configuration keeps it for a long stretch of positions
    int64_t cap = 1;
    while (cap * 128 < L) cap *= 2;
    if (want > cap) want = cap;
    if (want > 64) want = 64;
    return want < 1 ? 1 : (int)want;
}

// rows = n_seq * T query rows; caches of sequence s start at s * seq_stride elements.
b200_status kq_attention(const float *q, const uint16_t *kc, const uint16_t *vc, int n_seq, int T,
                         const int32_t *pos0_dev, int pos0, int n_head, int n_kv, int hd,
                         int64_t seq_stride, float *out, float *scratch, size_t scratch_bytes,
                         int force_splits, KqKvTypes kvt, cudaStream_t st) {
    KQ_REQUIRE(hd == 128 || hd == 64, "attention: head_dim %d not supported", hd);
    KQ_REQUIRE(n_kv > 0 && n_head % n_kv == 0, "attention: n_head %% n_kv");
    const int rows = n_seq * T, G = n_head / n_kv;
    if (kvt.quantised()) {
        // quantised rows are decoded while the tiles of the tensor-core kernel are staged
        const b200_status rc = kq_attention_prefill_mma(q, kc, vc, n_seq, T, pos0_dev, pos0, n_head, n_kv, hd, seq_stride, out, kvt, st);
        if (rc == B200_ERR_UNSUPPORTED) kq_set_error("attention: a quantised KV cache needs head_dim 128 and 1, 2, 4, 5 or 8 query heads per KV head");
        return rc;
    }
    // batches of new tokens go to the tensor-core kernel (B200_ATTN_MMA=0 keeps the per-row kernel)
    static int use_mma = -1;
    if (use_mma < 0) {
        const char *v = getenv("B200_ATTN_MMA");
        use_mma = !(v && v[0] == '0');
    }
    // f16 caches, head_dim 128: the tcgen05 kernel (B200_ATTN_TC=0 keeps the mma.sync kernel)
    static int use_tc = -1;
    if (use_tc < 0) {
        const char *v = getenv("B200_ATTN_TC");
        use_tc = !(v && v[0] == '0');
    }
    if (use_mma && use_tc && T >= 32 && force_splits <= 0) {
        const b200_status rc = kq_attention_prefill_tc(q, kc, vc, n_seq, T, pos0_dev, pos0, n_head, n_kv, hd, seq_stride, out, st);
        if (rc != B200_ERR_UNSUPPORTED) return rc;
    }
    if (use_mma && T >= 32 && force_splits <= 0) {
        const b200_status rc = kq_attention_prefill_mma(q, kc, vc, n_seq, T, pos0_dev, pos0, n_head, n_kv, hd, seq_stride, out, kvt, st);
        if (rc != B200_ERR_UNSUPPORTED) return rc;
    }
    int n_split = force_splits > 0 ? force_splits : kq_attention_splits(rows, n_kv, pos0 + T);
    const size_t need = (size_t)rows * n_head * n_split * (hd + 2) * sizeof(float);
    if (n_split > 1 && need > scratch_bytes) n_split = 1;
    float *po = scratch, *pml = scratch ? scratch + (size_t)rows * n_head * n_split * hd : nullptr;
    const float scale = 1.0f / sqrtf((float)hd);
    dim3 grid(n_kv, n_split, rows);
    b200_status rc;
    if (hd == 128)
        rc = launch_attention_g<128>(G, grid, q, (const __half *)kc, (const __half *)vc, T, pos0_dev, pos0, n_head,
                                     n_kv, seq_stride, n_split, scale, out, po, pml, st);
    else
        rc = launch_attention_g<64>(G, grid, q, (const __half *)kc, (const __half *)vc, T, pos0_dev, pos0, n_head,
                                    n_kv, seq_stride, n_split, scale, out, po, pml, st);
    if (rc != B200_OK) return rc;
    if (n_split > 1) {
        dim3 g2(n_head, rows);
        if (hd == 128) kq_launch(attention_combine_kernel<128>, g2, 128, 0, st, po, pml, n_head, n_split, out);
        else kq_launch(attention_combine_kernel<64>, g2, 64, 0, st, po, pml, n_head, n_split, out);
        KQ_COUNT_LAUNCH();
        KQ_LAUNCH_CHECK();
    }
    return B200_OK;
}

b200_status kq_rope_store(float *q, const float *k, const float *v, const int32_t *pos,
                          const int32_t *pos0_dev, int pos0, int n_seq, int T, int n_head, int n_kv, int hd, float theta, int neox,
                          uint16_t *k_cache, uint16_t *v_cache, int64_t seq_stride, KqKvTypes kvt, cudaStream_t st) {
    KQ_REQUIRE(hd % 2 == 0 && hd <= 256, "rope: head_dim %d", hd);
    KQ_REQUIRE(kq_kv_type_ok(kvt.k) && kq_kv_type_ok(kvt.v), "rope: KV cache types %d / %d", kvt.k, kvt.v);
    KQ_REQUIRE(!kvt.quantised() || hd % 32 == 0, "rope: quantised KV rows need head_dim %% 32 == 0");
    RopeTable tab;
    for (int i = 0; i < hd / 2; i++) tab.inv_freq[i] = (float)pow((double)theta, -2.0 * i / (double)hd);
    kq_launch(rope_store_kernel, n_seq * T, 256, 0, st, q, k, v, pos, pos0_dev, pos0, T, n_head, n_kv, hd, neox, tab,
                                                 (__half *)k_cache, (__half *)v_cache, seq_stride, kvt);
    KQ_COUNT_LAUNCH();
    KQ_LAUNCH_CHECK();
    return B200_OK;
}

extern "C" {

b200_status b200_rope(float *x, const int32_t *pos, int64_t T, int64_t n_head, int64_t hd, float theta,
                      int32_t neox, void *stream) {
    KQ_REQUIRE(T > 0 && pos, "rope: positions required");
    return kq_rope_store(x, nullptr, nullptr, pos, nullptr, 0, 1, (int)T, (int)n_head, 0, (int)hd, theta, neox,
                         nullptr, nullptr, 0, KqKvTypes(), (cudaStream_t)stream);
}

b200_status b200_swiglu(const float *gate, const float *up, int64_t n, float *y, void *stream) {
    kq_launch(swiglu_kernel, (unsigned)kq_div_up(n, 256), 256, 0, (cudaStream_t)stream, gate, up, n, y);
    KQ_COUNT_LAUNCH();
    KQ_LAUNCH_CHECK();
    return B200_OK;
}

b200_status b200_add(const float *a, const float *b, int64_t n, float *y, void *stream) {
    kq_launch(add_kernel, (unsigned)kq_div_up(n, 256), 256, 0, (cudaStream_t)stream, a, b, n, y);
    KQ_COUNT_LAUNCH();
    KQ_LAUNCH_CHECK();
    return B200_OK;
}

b200_status b200_add_bias(float *y, const float *bias, int64_t T, int64_t n, void *stream) {
    kq_launch(add_bias_kernel, (unsigned)kq_div_up(T * n, 256), 256, 0, (cudaStream_t)stream, y, bias, T * n, n);
    KQ_COUNT_LAUNCH();
    KQ_LAUNCH_CHECK();
    return B200_OK;
}

b200_status b200_cpy_f32_f16(const float *x, int64_t n, uint16_t *y, void *stream) {
    kq_launch(cpy_f16_kernel, (unsigned)kq_div_up(n, 256), 256, 0, (cudaStream_t)stream, x, n, (__half *)y);
    KQ_COUNT_LAUNCH();
    KQ_LAUNCH_CHECK();
    return B200_OK;
}

size_t b200_attention_scratch_bytes(int64_t T, int64_t n_head, int64_t hd, int64_t n_ctx) {
    return (size_t)T * n_head * 64 * (hd + 2) * sizeof(float);
}

b200_status b200_attention(const float *q, const uint16_t *k_cache, const uint16_t *v_cache, int64_t T,
                           int64_t pos0, int64_t n_head, int64_t n_kv, int64_t hd, float *out,
                           void *scratch, size_t scratch_bytes, void *stream) {
    KQ_REQUIRE(T > 0 && pos0 >= 0, "attention: bad shape");
    return kq_attention(q, k_cache, v_cache, 1, (int)T, nullptr, (int)pos0, (int)n_head, (int)n_kv, (int)hd,
                        0, out, (float *)scratch, scratch_bytes, 0, KqKvTypes(), (cudaStream_t)stream);
}

size_t b200_kv_row_bytes(uint32_t type, int64_t hd) {
    if (!kq_kv_type_ok((int)type) || hd <= 0 || hd % 32) return 0;
    return (size_t)kq_kv_row_bytes((int)type, (int)hd);
}

b200_status b200_kv_store(const float *k, const float *v, const int32_t *pos, int64_t T, int64_t n_kv, int64_t hd,
                          float theta, int32_t neox, uint32_t k_type, uint32_t v_type, void *k_cache, void *v_cache,
                          void *stream) {
    KQ_REQUIRE(T > 0 && pos && k && v && k_cache && v_cache, "kv_store: positions, rows and caches required");
    KqKvTypes kvt;
    kvt.k = (int)k_type;
    kvt.v = (int)v_type;
    return kq_rope_store(nullptr, k, v, pos, nullptr, 0, 1, (int)T, 0, (int)n_kv, (int)hd, theta, neox,
                         (uint16_t *)k_cache, (uint16_t *)v_cache, 0, kvt, (cudaStream_t)stream);
}

b200_status b200_attention_kv(const float *q, const void *k_cache, const void *v_cache, uint32_t k_type, uint32_t v_type,
                              int64_t T, int64_t pos0, int64_t n_head, int64_t n_kv, int64_t hd, float *out, void *scratch,
                              size_t scratch_bytes, void *stream) {
    KQ_REQUIRE(T > 0 && pos0 >= 0, "attention: bad shape");
    KqKvTypes kvt;
    kvt.k = (int)k_type;
    kvt.v = (int)v_type;
    KQ_REQUIRE(kq_kv_type_ok(kvt.k) && kq_kv_type_ok(kvt.v), "attention: KV cache types %u / %u", k_type, v_type);
    return kq_attention(q, (const uint16_t *)k_cache, (const uint16_t *)v_cache, 1, (int)T, nullptr, (int)pos0, (int)n_head,
                        (int)n_kv, (int)hd, 0, out, (float *)scratch, scratch_bytes, 0, kvt, (cudaStream_t)stream);
}

b200_status b200_get_rows(uint32_t type, const void *W, const int32_t *ids, int64_t T, int64_t K,
                          float *y, void *stream) {
    KQ_REQUIRE(type == B200_TYPE_Q4_K || type == B200_TYPE_Q6_K || type == B200_TYPE_F32,
               "get_rows: type %u", type);
    KQ_REQUIRE(type == B200_TYPE_F32 || K % 256 == 0, "get_rows: K %% 256");
    kq_launch(get_rows_kernel, (unsigned)kq_div_up(T * K, 256), 256, 0, (cudaStream_t)stream, 
        type, (const uint8_t *)W, ids, T, (int)K, y);
    KQ_COUNT_LAUNCH();
    KQ_LAUNCH_CHECK();
    return B200_OK;
}

b200_status b200_argmax(const float *x, int64_t T, int64_t n, int32_t *idx, void *stream) {
    kq_launch(argmax_kernel, (unsigned)T, 1024, 0, (cudaStream_t)stream, x, n, idx);
    KQ_COUNT_LAUNCH();
    KQ_LAUNCH_CHECK();
    return B200_OK;
}

b200_status b200_moe_route_masked(const float *logits, int64_t T, int64_t E, int64_t k, const uint8_t *mask,
                                  int32_t *ids, float *w, void *stream) {
    KQ_REQUIRE(logits && ids && w && T >= 1, "moe_route: null argument");
    KQ_REQUIRE(E >= 1 && E <= 256 && k >= 1 && k <= 32 && k <= E, "moe_route: E <= 256, k <= 32");
    kq_launch(moe_route_kernel, (unsigned)kq_div_up(T, 4), 128, 0, (cudaStream_t)stream, logits, T, (int)E, (int)k,
                                                                                mask, ids, w);
    KQ_COUNT_LAUNCH();
    KQ_LAUNCH_CHECK();
    return B200_OK;
}

b200_status b200_moe_route(const float *logits, int64_t T, int64_t E, int64_t k, int32_t *ids, float *w,
                           void *stream) {
    return b200_moe_route_masked(logits, T, E, k, nullptr, ids, w, stream);
}

} // extern "C"

// ---- small f32 matmul (router gate, F32 weights): one warp per output element --------------------
namespace {
__global__ void __launch_bounds__(128) f32_matmul_kernel(const float *W, const float *x, int64_t M, int64_t N,
                                                         int K, float *out) {
    KQ_PDL_ENTER();
    const int lane = threadIdx.x & 31;
    const int64_t w = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
    if (w >= M * N) return;
    const int64_t m = w / N, n = w % N;
    const float *wr = W + n * K, *xr = x + m * K;
    float acc = 0.f;
    for (int i = lane; i < K; i += 32) acc = fmaf(wr[i], xr[i], acc);
    acc = kq_warp_sum(acc);
    if (lane == 0) out[w] = acc;
}
} // namespace

b200_status kq_f32_matmul(const float *W, const float *x, int64_t M, int64_t N, int64_t K, float *y,
                          cudaStream_t st) {
    KQ_REQUIRE(M > 0 && N > 0 && K > 0, "f32 matmul: bad shape");
    kq_launch(f32_matmul_kernel, (unsigned)kq_div_up(M * N, 4), 128, 0, st, W, x, M, N, (int)K, y);
    KQ_COUNT_LAUNCH();
    KQ_LAUNCH_CHECK();
    return B200_OK;
}
