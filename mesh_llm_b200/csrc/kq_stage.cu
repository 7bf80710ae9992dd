// One serving stage: a contiguous layer range of a Q4_K_M decoder resident on one B200.
//
// This is the unit mesh-llm distributes: a worker holds blk.[a,b) (plus the embeddings on the
// first stage and output_norm + output on the last), loads exactly its own tensors by name, and
// exchanges one [tokens x n_embd] f32 activation with its neighbour per micro-batch.  The forward
// pass below is the graph llama.cpp builds for these architectures, expressed as launches of the
// kernels in this directory; decode steps (T == 1) are captured once into a CUDA graph and
// replayed, since at batch 1 the step is a chain of ~10 short kernels per layer.
#include "kq_common.cuh"
#include "kq_kvq.cuh"

#include <stdlib.h>

#include <map>
#include <string>
#include <vector>

b200_status kq_synth_weights(uint32_t type, void *W, int64_t n_rows, int64_t K, uint64_t key, float mean,
                             float sigma, cudaStream_t st);
b200_status kq_rms_norm(const float *x, const float *w, int64_t T, int64_t h, float eps, float *y,
                        int8_t *q, float *d, int16_t *bs, cudaStream_t st, int64_t x_row_stride = 0);
b200_status kq_moe_router_fused(const float *x, const float *norm_w, float eps, const float *router_w, int rows, int E, int h,
                                int k, const uint8_t *mask, float *rl, int32_t *ids, float *wts, int8_t *q, float *d,
                                int16_t *bs, unsigned int *counters, cudaStream_t st);
b200_status kq_swiglu_quantize(const float *g, const float *u, int64_t M, int64_t K, float *y, int8_t *q, float *d, int16_t *bs,
                               cudaStream_t st);
b200_status kq_moe_gate_up(uint32_t type, const uint8_t *Wg, const uint8_t *Wu, int64_t expert_stride, const int8_t *aq,
                           const float *ad, const int16_t *abs16, const int32_t *ids, int pairs, int ku, int K, int fe, float *hp,
                           cudaStream_t st);
b200_status kq_moe_down_combine(uint32_t type, const uint8_t *W, int64_t expert_stride, const float *hp, const int32_t *ids,
                                const float *wts, const float *res, int rows, int ku, int h, int fe, float *out,
                                cudaStream_t st);
b200_status kq_attention(const float *q, const uint16_t *kc, const uint16_t *vc, int n_seq, int T,
                         const int32_t *pos0_dev, int pos0, int n_head, int n_kv, int hd,
                         int64_t seq_stride, float *out, float *scratch, size_t scratch_bytes,
                         int force_splits, KqKvTypes kvt, cudaStream_t st);
int kq_attention_splits(int64_t rows, int n_kv, int64_t L);
int kq_attention_decode_splits(int64_t L, int pairs);
b200_status kq_attention_decode(const float *q, const float *k, const float *v, uint16_t *kc, uint16_t *vc,
                                int n_seq, const int32_t *pos_dev, int pos, int n_head, int n_kv, int hd,
                                int64_t seq_stride, float theta, int neox, int n_split, float *out, float *scratch,
                                size_t scratch_bytes, int *counters, KqKvTypes kvt, cudaStream_t st);
b200_status kq_rope_store(float *q, const float *k, const float *v, const int32_t *pos,
                          const int32_t *pos0_dev, int pos0, int n_seq, int T, int n_head, int n_kv, int hd,
                          float theta, int neox, uint16_t *k_cache, uint16_t *v_cache, int64_t seq_stride,
                          KqKvTypes kvt, cudaStream_t st);

namespace {

struct StTensor {
    std::string name;
    uint32_t type = 0;
    int64_t ne[3] = {0, 0, 0};
    void *dev = nullptr;
    size_t dev_bytes = 0;
    bool loaded = false;
};

struct LayerW {
    const float *attn_norm = nullptr, *ffn_norm = nullptr, *bq = nullptr, *bk = nullptr, *bv = nullptr,
                *q_norm = nullptr, *k_norm = nullptr, *router = nullptr;
    StTensor *wq = nullptr, *wk = nullptr, *wv = nullptr, *wo = nullptr, *gate = nullptr, *up = nullptr,
             *down = nullptr, *gate_e = nullptr, *up_e = nullptr, *down_e = nullptr;
};

struct GraphKey {
    int n_seq, n_split, seq0, pad_;
    const void *tokens, *hidden_in, *hidden_out, *logits, *next;
    bool operator<(const GraphKey &o) const {
        return memcmp(this, &o, sizeof(GraphKey)) < 0;
    }
};

struct GraphEntry {
    int n_split = 0; // attention slices the instantiated graph was last captured / updated for
    cudaGraphExec_t exec = nullptr;
    long long launches = 0;
};

// f32 matvec for the router: one warp per (token, expert)
__global__ void __launch_bounds__(128) router_logits_kernel(const float *W, const float *x, int T, int E,
                                                            int h, float *out) {
    KQ_PDL_ENTER();
    const int lane = threadIdx.x & 31;
    const int64_t w = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
    if (w >= (int64_t)T * E) return;
    const int t = (int)(w / E), e = (int)(w % E);
    const float4 *wr = reinterpret_cast<const float4 *>(W + (int64_t)e * h);
    const float4 *xr = reinterpret_cast<const float4 *>(x + (int64_t)t * h);
    float acc = 0.f;
    for (int i = lane; i < h / 4; i += 32) {
        const float4 a = wr[i], b = xr[i];
        acc += a.x * b.x + a.y * b.y + a.z * b.z + a.w * b.w;
    }
    acc = kq_warp_sum(acc);
    if (lane == 0) out[w] = acc;
}

// out[t] = res[t] + sum_s w[t][s] * y[t*k+s]   (slot order, deterministic)
__global__ void moe_combine_kernel(const float *y, const float *w, const float *res, int T, int k, int h,
                                   float *out) {
    KQ_PDL_ENTER();
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (int64_t)T * h) return;
    const int t = (int)(i / h), c = (int)(i % h);
    float acc = 0.f;
    for (int s = 0; s < k; s++) acc += w[t * k + s] * y[((int64_t)t * k + s) * h + c];
    out[i] = res[i] + acc;
}

__global__ void gather_rows_kernel(const float *x, int64_t row_stride, int64_t first, int n_rows, int h,
                                   float *y) {
    KQ_PDL_ENTER();
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (int64_t)n_rows * h) return;
    y[i] = x[(first + (i / h) * row_stride) * h + i % h];
}

__global__ void set_pos_kernel(int32_t *p, int v) {
    KQ_PDL_ENTER(); *p = v; }

uint64_t mix64_host(uint64_t z) {
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
uint64_t name_hash(const char *s) {
    uint64_t h = 0xCBF29CE484222325ull;
    for (; *s; s++) h = (h ^ (uint8_t)*s) * 0x100000001B3ull;
    return h;
}

} // namespace

struct b200_stage {
    b200_stage_config c;
    std::vector<StTensor> tensors;
    std::map<std::string, int> index;
    std::vector<LayerW> layers;
    StTensor *tok_embd = nullptr, *out_w = nullptr;
    const float *out_norm = nullptr;
    bool resolved = false;
    // KV cache [layer_local][seq][ctx][n_kv][hd] f16
    uint16_t *kc = nullptr, *vc = nullptr;
    KqKvTypes kvt;
    int k_row = 0, v_row = 0; // bytes of one (position, kv head) row of each cache
    // activations
    int rows_max = 0;
    float *x = nullptr, *xn = nullptr, *q = nullptr, *k = nullptr, *v = nullptr, *att = nullptr, *g = nullptr,
          *u = nullptr, *last = nullptr, *logits_int = nullptr, *att_scratch = nullptr, *rl = nullptr,
          *rw = nullptr, *hp = nullptr, *hp2 = nullptr, *yp = nullptr;
    int32_t *moe_sorted = nullptr; // expert-major order of the routed pairs of a batch
    size_t moe_sorted_bytes = 0;
    uint8_t *expert_mask = nullptr; // one byte per expert, 1 = allowed (all ones when no mask is set)
    int32_t *rid = nullptr, *pos0_dev = nullptr, *rid_scratch = nullptr, *attn_counters = nullptr;
    unsigned int *moe_counters = nullptr; // one word per token row, zero between launches (moe_router_fused_kernel)
    int32_t *emit_counters = nullptr;     // one word per 256 rows of the feed-forward width, zero between launches (KqEmitQ8)
    size_t att_scratch_bytes = 0;
    void *scan_scratch = nullptr; // slices and counters of the vocabulary scan
    size_t scan_scratch_bytes = 0;
    int8_t *aq = nullptr;
    float *ad = nullptr;
    int16_t *abs16 = nullptr;
    int64_t kmax = 0;
    std::map<GraphKey, GraphEntry> graphs;
    cudaStream_t cap_stream = nullptr;
    long long launches = 0;
    bool use_graph = true;
    std::vector<void *> allocs;
};

namespace {

b200_status dev_alloc(b200_stage *st, void **p, size_t bytes) {
    *p = nullptr;
    if (bytes == 0) bytes = 256;
    cudaError_t e = cudaMalloc(p, bytes);
    if (e != cudaSuccess) {
        cudaGetLastError();
        kq_set_error("stage: cudaMalloc(%zu) failed: %s", bytes, cudaGetErrorString(e));
        return B200_ERR_ALLOC;
    }
    st->allocs.push_back(*p);
    return B200_OK;
}

void add_tensor(b200_stage *st, const std::string &name, uint32_t type, int64_t ne0, int64_t ne1,
                int64_t ne2) {
    StTensor t;
    t.name = name;
    t.type = type;
    t.ne[0] = ne0;
    t.ne[1] = ne1;
    t.ne[2] = ne2;
    t.dev_bytes = (size_t)(kq_device_row_bytes(type, ne0) * ne1 * ne2);
    st->index[name] = (int)st->tensors.size();
    st->tensors.push_back(t);
}

StTensor *find(b200_stage *st, const std::string &name) {
    auto it = st->index.find(name);
    return it == st->index.end() ? nullptr : &st->tensors[it->second];
}

StTensor *lt(b200_stage *st, int l, const char *what) {
    char buf[96];
    snprintf(buf, sizeof(buf), "blk.%d.%s", l, what);
    return find(st, buf);
}

#define KQ_TRY(expr)                      \
    do {                                  \
        b200_status rc__ = (expr);        \
        if (rc__ != B200_OK) return rc__; \
    } while (0)

// MUL_MAT on quantised activations already sitting in st->aq/ad/abs16
b200_status mm(b200_stage *st, const StTensor *w, int rows, float *y, const float *bias,
               const float *residual, cudaStream_t s) {
    return b200_mul_mat_q8(w->type, w->dev, st->aq, st->ad, st->abs16, rows, w->ne[1], w->ne[0], y, bias,
                           residual, s);
}

enum { CLS_GEMV = 1, CLS_ATTN = 2, CLS_OTHER = 4, CLS_ALL = 7 };

// `classes` selects which kernel classes are launched; anything but CLS_ALL is timing
// instrumentation (the outputs are then meaningless).
b200_status forward_body(b200_stage *st, const int32_t *tokens, const float *hidden_in, int seq0, int n_seq,
                         int T, int pos0, bool pos_from_dev, int force_splits, float *hidden_out, float *logits,
                         int all_logits, int32_t *next_tokens, cudaStream_t s, unsigned classes = CLS_ALL) {
#define GEMV_(expr) do { if (classes & CLS_GEMV) KQ_TRY(expr); } while (0)
#define ATTN_(expr) do { if (classes & CLS_ATTN) KQ_TRY(expr); } while (0)
#define OTHER_(expr) do { if (classes & CLS_OTHER) KQ_TRY(expr); } while (0)
    const b200_stage_config &c = st->c;
    const int rows = n_seq * T;
    const int h = c.n_embd, hd = c.head_dim, nq = c.n_head * hd, nkv = c.n_head_kv * hd;
    const int64_t seq_stride = (int64_t)c.n_ctx * nkv;
    const int32_t *pos_dev = pos_from_dev ? st->pos0_dev : nullptr;
    const float *xin;
    if (c.has_embd) {
        OTHER_(b200_get_rows(st->tok_embd->type, st->tok_embd->dev, tokens, rows, h, st->x, s));
        xin = st->x;
    } else {
        xin = hidden_in;
    }
    const int n_local = c.layer_end - c.layer_begin;
    for (int ll = 0; ll < n_local; ll++) {
        const LayerW &L = st->layers[ll];
        const bool last_layer = ll == n_local - 1;
        // caches are [layer][sequence][position][kv head] rows of k_row / v_row bytes
        const int64_t seq_rows = (int64_t)c.n_ctx * c.n_head_kv;
        uint16_t *kc = (uint16_t *)((uint8_t *)st->kc + ((int64_t)ll * c.n_seq + seq0) * seq_rows * st->k_row);
        uint16_t *vc = (uint16_t *)((uint8_t *)st->vc + ((int64_t)ll * c.n_seq + seq0) * seq_rows * st->v_row);
        const KqKvTypes kvt = st->kvt;
        // ---- attention block
        const bool fuse = rows <= 2; // the streaming GEMV normalises and quantises its own input
        if (!fuse) OTHER_(kq_rms_norm(xin, L.attn_norm, rows, h, c.rms_eps, nullptr, st->aq, st->ad, st->abs16, s));
        if (rows <= 8) {
            KqGemvSeg segs[3] = {
                {(const uint8_t *)L.wq->dev, L.wq->type, nq, st->q, L.bq, nq, 0},
                {(const uint8_t *)L.wk->dev, L.wk->type, nkv, st->k, L.bk, nkv, 0},
                {(const uint8_t *)L.wv->dev, L.wv->type, nkv, st->v, L.bv, nkv, 0},
            };
            KqActPrep pr = {xin, L.attn_norm, c.rms_eps, 1};
            GEMV_(kq_launch_gemv(segs, 3, st->aq, st->ad, st->abs16, rows, h, nullptr, 0, nullptr, s,
                                 fuse ? &pr : nullptr));
        } else {
            GEMV_(mm(st, L.wq, rows, st->q, L.bq, nullptr, s));
            GEMV_(mm(st, L.wk, rows, st->k, L.bk, nullptr, s));
            GEMV_(mm(st, L.wv, rows, st->v, L.bv, nullptr, s));
        }
        if (c.qk_norm) {
            OTHER_(kq_rms_norm(st->q, L.q_norm, (int64_t)rows * c.n_head, hd, c.rms_eps, st->q, nullptr,
                               nullptr, nullptr, s));
            OTHER_(kq_rms_norm(st->k, L.k_norm, (int64_t)rows * c.n_head_kv, hd, c.rms_eps, st->k, nullptr,
                               nullptr, nullptr, s));
        }
        if (T == 1) {
            // decode: RoPE, KV store, attention and the split combine are one launch
            const int ns = kq_attention_decode_splits(pos0 + 1, n_seq * c.n_head_kv);
            ATTN_(kq_attention_decode(st->q, st->k, st->v, kc, vc, n_seq, pos_dev, pos0, c.n_head, c.n_head_kv, hd,
                                      seq_stride, c.rope_theta, c.rope_neox, ns, st->att, st->att_scratch,
                                      st->att_scratch_bytes, st->attn_counters, kvt, s));
        } else {
            OTHER_(kq_rope_store(st->q, st->k, st->v, nullptr, pos_dev, pos0, n_seq, T, c.n_head, c.n_head_kv, hd,
                                 c.rope_theta, c.rope_neox, kc, vc, seq_stride, kvt, s));
            ATTN_(kq_attention(st->q, kc, vc, n_seq, T, pos_dev, pos0, c.n_head, c.n_head_kv, hd, seq_stride,
                               st->att, st->att_scratch, st->att_scratch_bytes, force_splits, kvt, s));
        }
        float *xout = (last_layer && !c.has_output && hidden_out) ? hidden_out : st->x;
        bool ffn_done = false, wo_done = false; // what has already gone out as part of a fused launch
        if (fuse && c.n_expert == 0 && (classes & CLS_GEMV)) {
            // attention output, gate / up with SwiGLU and down as three phases of one launch
            KqFusedPhase ph[3] = {};
            ph[0].segs[0] = {(const uint8_t *)L.wo->dev, L.wo->type, h, st->x, nullptr, h, 0};
            ph[0].nseg = 1;
            ph[0].K = nq;
            ph[0].residual = xin;
            ph[0].prep = {st->att, nullptr, 0.f, 0};
            ph[1].segs[0] = {(const uint8_t *)L.gate->dev, L.gate->type, c.n_ff, st->g, nullptr, c.n_ff, 0};
            ph[1].segs[1] = {(const uint8_t *)L.up->dev, L.up->type, c.n_ff, st->g, nullptr, c.n_ff, 0};
            ph[1].nseg = 2;
            ph[1].K = h;
            ph[1].swiglu = 1;
            ph[1].prep = {st->x, L.ffn_norm, c.rms_eps, 1};
            ph[2].segs[0] = {(const uint8_t *)L.down->dev, L.down->type, h, xout, nullptr, h, 0};
            ph[2].nseg = 1;
            ph[2].K = c.n_ff;
            ph[2].residual = st->x;
            ph[2].prep = {st->g, nullptr, 0.f, 0};
            static int mode = -1; // B200_GEMV_FUSED: 0 separate launches, 2 gate / up + down in one launch, 3 all three
            if (mode < 0) {
                const char *v = getenv("B200_GEMV_FUSED");
                mode = v ? atoi(v) : 0;
            }
            b200_status frc = B200_ERR_UNSUPPORTED;
            if (mode >= 3) {
                frc = kq_launch_gemv_fused(ph, 3, rows, s);
            } else if (mode == 2) {
                KqGemvSeg so = {(const uint8_t *)L.wo->dev, L.wo->type, h, st->x, nullptr, h, 0};
                KqActPrep pr = {st->att, nullptr, 0.f, 0};
                KQ_TRY(kq_launch_gemv(&so, 1, st->aq, st->ad, st->abs16, rows, nq, xin, 0, nullptr, s, &pr));
                frc = kq_launch_gemv_fused(ph + 1, 2, rows, s);
                if (frc == B200_ERR_UNSUPPORTED) wo_done = true;
            }
            if (frc == B200_OK) ffn_done = true;
            else if (frc != B200_ERR_UNSUPPORTED) return frc;
        }
        if (ffn_done || wo_done) {
        } else if (fuse) {
            KqGemvSeg so = {(const uint8_t *)L.wo->dev, L.wo->type, h, st->x, nullptr, h, 0};
            KqActPrep pr = {st->att, nullptr, 0.f, 0};
            GEMV_(kq_launch_gemv(&so, 1, st->aq, st->ad, st->abs16, rows, nq, xin, 0, nullptr, s, &pr));
        } else {
            OTHER_(b200_quantize_act(st->att, rows, nq, st->aq, st->ad, st->abs16, s));
            GEMV_(mm(st, L.wo, rows, st->x, nullptr, xin, s)); // x = xin + Wo.att
        }
        // ---- feed-forward block
        if (ffn_done) {
        } else if (c.n_expert > 0) {
            const int E = c.n_expert, ku = c.n_expert_used, fe = c.n_ff_exp, pairs = rows * ku;
            // Few tokens (a decode step): norm, Q8, router logits and routing are one launch, and the down
            // matmul quantises its own input and leaves the weighted sum on the residual (kq_moe_decode.cu).
            // B200_MOE_FUSED=0 keeps the separate launches.
            static int moe_fused_on = -1;
            if (moe_fused_on < 0) {
                const char *v = getenv("B200_MOE_FUSED");
                moe_fused_on = !(v && v[0] == '0');
            }
            bool fused_small = moe_fused_on && rows <= 8 && classes == CLS_ALL && ku <= 8 && fe % 256 == 0 && h % 256 == 0;
            if (fused_small) {
                const b200_status rs = kq_moe_router_fused(st->x, L.ffn_norm, c.rms_eps, L.router, (int)rows, (int)E, (int)h, (int)ku,
                                                           st->expert_mask, st->rl, st->rid, st->rw, st->aq, st->ad, st->abs16,
                                                           st->moe_counters, s);
                if (rs == B200_ERR_UNSUPPORTED) fused_small = false;
                else KQ_TRY(rs);
            }
            if (!fused_small) {
            OTHER_(kq_rms_norm(st->x, L.ffn_norm, rows, h, c.rms_eps, st->xn, st->aq, st->ad, st->abs16, s));
            if (classes & CLS_OTHER) {
            kq_launch(router_logits_kernel, (unsigned)kq_div_up((int64_t)rows * E, 4), 128, 0, s, L.router, st->xn,
                                                                                          rows, E, h, st->rl);
            KQ_COUNT_LAUNCH();
            KQ_LAUNCH_CHECK();
            }
            OTHER_(b200_moe_route_masked(st->rl, rows, E, ku, st->expert_mask, st->rid, st->rw, s));
            }
            // gate/up of the selected experts with fused SwiGLU, one (token, slot) pair per grid row
            const int64_t gstride = kq_device_row_bytes(L.gate_e->type, h) * fe;
            const int64_t dstride = kq_device_row_bytes(L.down_e->type, fe) * h;
            KqGemvSeg gu[2] = {
                {(const uint8_t *)L.gate_e->dev, L.gate_e->type, fe, st->hp, nullptr, fe, gstride},
                {(const uint8_t *)L.up_e->dev, L.up_e->type, fe, st->hp, nullptr, fe, gstride},
            };
            // Many tokens: the pairs are gathered per expert and each expert-packed matrix is one grouped
            // launch of the tensor-core GEMM (build_moe_ffn's MUL_MAT_ID); few tokens: one indirect GEMV
            // row per pair.  B200_MOE_GROUPED=0 keeps the second form for every batch size.
            static int grouped_on = -1;
            if (grouped_on < 0) {
                const char *v = getenv("B200_MOE_GROUPED");
                grouped_on = !(v && v[0] == '0');
            }
            bool grouped = grouped_on && rows > 8 && fe % 64 == 0 && h % 64 == 0 && classes == CLS_ALL;
            if (grouped) {
                KQ_TRY(kq_moe_sort(st->rid, pairs, E, st->moe_sorted, st->moe_sorted_bytes, s));
                KQ_TRY(kq_launch_gemm_grouped(L.gate_e->type, (const uint8_t *)L.gate_e->dev, gstride, st->aq, st->ad, st->abs16, ku,
                                              pairs, E, fe, h, st->hp, st->moe_sorted, s));
                KQ_TRY(kq_launch_gemm_grouped(L.up_e->type, (const uint8_t *)L.up_e->dev, gstride, st->aq, st->ad, st->abs16, ku,
                                              pairs, E, fe, h, st->hp2, st->moe_sorted, s));
                KQ_TRY(kq_swiglu_quantize(st->hp, st->hp2, pairs, fe, st->hp, st->aq, st->ad, st->abs16, s));
                KQ_TRY(kq_launch_gemm_grouped(L.down_e->type, (const uint8_t *)L.down_e->dev, dstride, st->aq, st->ad, st->abs16, 1,
                                              pairs, E, h, fe, st->yp, st->moe_sorted, s));
            } else {
            KqGemvIndirect ind = {st->rid, pairs, ku};
            b200_status rg = B200_ERR_UNSUPPORTED;
            if (fused_small && L.gate_e->type == L.up_e->type)
                rg = kq_moe_gate_up(L.gate_e->type, (const uint8_t *)L.gate_e->dev, (const uint8_t *)L.up_e->dev, gstride, st->aq,
                                    st->ad, st->abs16, st->rid, (int)pairs, (int)ku, (int)h, (int)fe, st->hp, s);
            if (rg == B200_ERR_UNSUPPORTED) GEMV_(kq_launch_gemv(gu, 2, st->aq, st->ad, st->abs16, 1, h, nullptr, 1, &ind, s));
            else KQ_TRY(rg);
            if (fused_small) {
                const b200_status rs = kq_moe_down_combine(L.down_e->type, (const uint8_t *)L.down_e->dev, dstride, st->hp, st->rid,
                                                           st->rw, st->x, (int)rows, (int)ku, (int)h, (int)fe, xout, s);
                if (rs == B200_ERR_UNSUPPORTED) fused_small = false;
                else KQ_TRY(rs);
            }
            if (!fused_small) {
            OTHER_(b200_quantize_act(st->hp, pairs, fe, st->aq, st->ad, st->abs16, s));
            KqGemvSeg dn = {(const uint8_t *)L.down_e->dev, L.down_e->type, h, st->yp, nullptr, h, dstride};
            KqGemvIndirect ind2 = {st->rid, pairs, 1};
            GEMV_(kq_launch_gemv(&dn, 1, st->aq, st->ad, st->abs16, 1, fe, nullptr, 0, &ind2, s));
            }
            }
            if (!fused_small && (classes & CLS_OTHER)) {
            kq_launch(moe_combine_kernel, (unsigned)kq_div_up((int64_t)rows * h, 256), 256, 0, s, 
                st->yp, st->rw, st->x, rows, ku, h, xout);
            KQ_COUNT_LAUNCH();
            KQ_LAUNCH_CHECK();
            }
        } else {
            if (!fuse) OTHER_(kq_rms_norm(st->x, L.ffn_norm, rows, h, c.rms_eps, nullptr, st->aq, st->ad, st->abs16, s));
            KqEmitQ8 emit = {st->aq, st->ad, st->abs16, st->emit_counters, 0};
            if (rows <= 8) {
                KqGemvSeg gu[2] = {
                    {(const uint8_t *)L.gate->dev, L.gate->type, c.n_ff, st->g, nullptr, c.n_ff, 0},
                    {(const uint8_t *)L.up->dev, L.up->type, c.n_ff, st->g, nullptr, c.n_ff, 0},
                };
                KqActPrep pr = {st->x, L.ffn_norm, c.rms_eps, 1};
                // the launch also leaves the Q8 form of its output for the down projection (B200_GEMV_EMIT_Q8=0: off)
                const char *ev = getenv("B200_GEMV_EMIT_Q8"); // read when a step is captured
                const bool want = fuse && (ev ? atoi(ev) : 1) && (classes & CLS_GEMV);
                GEMV_(kq_launch_gemv(gu, 2, st->aq, st->ad, st->abs16, rows, h, nullptr, 1, nullptr, s,
                                     fuse ? &pr : nullptr, want ? &emit : nullptr));
            } else {
                GEMV_(mm(st, L.gate, rows, st->g, nullptr, nullptr, s));
                GEMV_(mm(st, L.up, rows, st->u, nullptr, nullptr, s));
                // SwiGLU and the Q8 form the down projection reads, in one pass
                OTHER_(kq_swiglu_quantize(st->g, st->u, rows, c.n_ff, st->g, st->aq, st->ad, st->abs16, s));
            }
            if (fuse && emit.done) {
                GEMV_(mm(st, L.down, rows, xout, nullptr, st->x, s)); // reads the Q8 form the gate / up launch wrote
            } else if (fuse) {
                KqGemvSeg sd = {(const uint8_t *)L.down->dev, L.down->type, h, xout, nullptr, h, 0};
                KqActPrep pr = {st->g, nullptr, 0.f, 0};
                GEMV_(kq_launch_gemv(&sd, 1, st->aq, st->ad, st->abs16, rows, c.n_ff, st->x, 0, nullptr, s, &pr));
            } else {
                if (rows <= 8) OTHER_(b200_quantize_act(st->g, rows, c.n_ff, st->aq, st->ad, st->abs16, s));
                GEMV_(mm(st, L.down, rows, xout, nullptr, st->x, s)); // x = x + Wdown.act
            }
        }
        xin = xout;
    }
    if (n_local == 0 && !c.has_output && hidden_out && xin != hidden_out)
        KQ_CUDA(cudaMemcpyAsync(hidden_out, xin, (size_t)rows * h * 4, cudaMemcpyDeviceToDevice, s));
    if (c.has_output) {
        if (hidden_out && xin != hidden_out)
            KQ_CUDA(cudaMemcpyAsync(hidden_out, xin, (size_t)rows * h * 4, cudaMemcpyDeviceToDevice, s));
        const int out_rows = all_logits ? rows : n_seq;
        float *lg = logits ? logits : st->logits_int;
        if (lg && (logits || next_tokens)) {
            KQ_REQUIRE(logits || out_rows <= c.n_seq, "stage: internal logits hold one row per sequence");
            // last token of each sequence: rows T-1, 2T-1, ...
            const float *src = all_logits ? xin : xin + (int64_t)(T - 1) * h;
            if (out_rows <= 2 && (T == 1 || all_logits)) {
                KqGemvSeg sh = {(const uint8_t *)st->out_w->dev, st->out_w->type, c.n_vocab, lg, nullptr, c.n_vocab, 0};
                KqActPrep pr = {src, st->out_norm, c.rms_eps, 1};
                GEMV_(kq_launch_gemv(&sh, 1, st->aq, st->ad, st->abs16, out_rows, h, nullptr, 0, nullptr, s, &pr));
            } else {
                OTHER_(kq_rms_norm(src, st->out_norm, out_rows, h, c.rms_eps, nullptr, st->aq, st->ad, st->abs16, s,
                                   all_logits ? h : (int64_t)T * h));
                GEMV_(mm(st, st->out_w, out_rows, lg, nullptr, nullptr, s));
            }
            // greedy token: the sliced vocabulary scan (argmax only here; the same launch can also
            // leave entropy / margin / top tokens through b200_logit_signals)
            if (next_tokens)
                OTHER_(b200_logit_signals(lg, out_rows, c.n_vocab, nullptr, nullptr, next_tokens, st->scan_scratch,
                                          st->scan_scratch_bytes, s));
        }
    }
    return B200_OK;
#undef GEMV_
#undef ATTN_
#undef OTHER_
}

b200_status resolve(b200_stage *st) {
    if (st->resolved) return B200_OK;
    for (auto &t : st->tensors)
        if (!t.loaded) {
            kq_set_error("stage: tensor %s has not been loaded", t.name.c_str());
            return B200_ERR_STATE;
        }
    const b200_stage_config &c = st->c;
    st->layers.assign(c.layer_end - c.layer_begin, LayerW());
    for (int l = c.layer_begin; l < c.layer_end; l++) {
        LayerW &L = st->layers[l - c.layer_begin];
        auto f32 = [&](const char *w) -> const float * {
            StTensor *t = lt(st, l, w);
            return t ? (const float *)t->dev : nullptr;
        };
        L.attn_norm = f32("attn_norm.weight");
        L.ffn_norm = f32("ffn_norm.weight");
        L.bq = f32("attn_q.bias");
        L.bk = f32("attn_k.bias");
        L.bv = f32("attn_v.bias");
        L.q_norm = f32("attn_q_norm.weight");
        L.k_norm = f32("attn_k_norm.weight");
        L.router = f32("ffn_gate_inp.weight");
        L.wq = lt(st, l, "attn_q.weight");
        L.wk = lt(st, l, "attn_k.weight");
        L.wv = lt(st, l, "attn_v.weight");
        L.wo = lt(st, l, "attn_output.weight");
        L.gate = lt(st, l, "ffn_gate.weight");
        L.up = lt(st, l, "ffn_up.weight");
        L.down = lt(st, l, "ffn_down.weight");
        L.gate_e = lt(st, l, "ffn_gate_exps.weight");
        L.up_e = lt(st, l, "ffn_up_exps.weight");
        L.down_e = lt(st, l, "ffn_down_exps.weight");
    }
    st->tok_embd = find(st, "token_embd.weight");
    st->out_w = find(st, "output.weight");
    StTensor *on = find(st, "output_norm.weight");
    st->out_norm = on ? (const float *)on->dev : nullptr;
    st->resolved = true;
    return B200_OK;
}

} // namespace

extern "C" {

b200_status b200_stage_create(const b200_stage_config *cfg, b200_stage **out) {
    KQ_REQUIRE(cfg && out, "stage_create: null argument");
    const b200_stage_config &c = *cfg;
    KQ_REQUIRE(c.n_embd > 0 && c.n_embd % 256 == 0, "stage: n_embd must be a multiple of 256");
    KQ_REQUIRE(c.head_dim == 128 || c.head_dim == 64, "stage: head_dim 64 or 128");
    KQ_REQUIRE(c.n_head > 0 && c.n_head_kv > 0 && c.n_head % c.n_head_kv == 0, "stage: head counts");
    KQ_REQUIRE((c.n_head * c.head_dim) % 256 == 0, "stage: n_head*head_dim must be a multiple of 256");
    KQ_REQUIRE(c.layer_begin >= 0 && c.layer_begin <= c.layer_end && c.layer_end <= c.n_layer,
               "stage: bad layer range [%d,%d) of %d", c.layer_begin, c.layer_end, c.n_layer);
    KQ_REQUIRE(c.n_expert > 0 ? (c.n_ff_exp > 0 && c.n_ff_exp % 256 == 0 && c.n_expert_used >= 1 &&
                                 c.n_expert_used <= c.n_expert && c.n_expert <= 256)
                              : (c.n_ff > 0 && c.n_ff % 256 == 0),
               "stage: feed-forward sizes must be multiples of 256");
    KQ_REQUIRE(c.n_ctx > 0 && c.n_seq > 0 && c.n_ubatch > 0, "stage: n_ctx, n_seq, n_ubatch");
    KQ_REQUIRE(!c.has_output || c.n_vocab > 0, "stage: n_vocab");
    KqKvTypes kvt;
    kvt.k = c.kv_type_k ? c.kv_type_k : KQ_KV_F16;
    kvt.v = c.kv_type_v ? c.kv_type_v : KQ_KV_F16;
    KQ_REQUIRE(kq_kv_type_ok(kvt.k) && kq_kv_type_ok(kvt.v), "stage: KV cache types %d / %d (f16 = 1, q4_0 = 2, q8_0 = 8)",
               kvt.k, kvt.v);
    if (kvt.quantised()) {
        const int g = c.n_head_kv > 0 ? c.n_head / c.n_head_kv : 0;
        if (c.head_dim != 128 || !(g == 1 || g == 2 || g == 4 || g == 5 || g == 8)) {
            kq_set_error("stage: a quantised KV cache needs head_dim 128 and 1, 2, 4, 5 or 8 query heads per KV head");
            return B200_ERR_UNSUPPORTED;
        }
    }
    KqDevGuard dev_guard(c.device);
    b200_stage *st = new b200_stage();
    st->c = c;
    st->kvt = kvt;
    st->k_row = kq_kv_row_bytes(kvt.k, c.head_dim);
    st->v_row = kq_kv_row_bytes(kvt.v, c.head_dim);
    const int64_t h = c.n_embd, hd = c.head_dim, nq = (int64_t)c.n_head * hd, nkv = (int64_t)c.n_head_kv * hd;
    if (c.has_embd) add_tensor(st, "token_embd.weight", B200_TYPE_Q4_K, h, c.n_vocab, 1);
    for (int l = c.layer_begin; l < c.layer_end; l++) {
        const uint32_t alt = (l & 1) ? B200_TYPE_Q6_K : B200_TYPE_Q4_K;
        auto add = [&](const char *w, uint32_t ty, int64_t a, int64_t b, int64_t cc) {
            char buf[96];
            snprintf(buf, sizeof(buf), "blk.%d.%s", l, w);
            add_tensor(st, buf, ty, a, b, cc);
        };
        add("attn_norm.weight", B200_TYPE_F32, h, 1, 1);
        add("attn_q.weight", B200_TYPE_Q4_K, h, nq, 1);
        add("attn_k.weight", B200_TYPE_Q4_K, h, nkv, 1);
        add("attn_v.weight", alt, h, nkv, 1);
        add("attn_output.weight", B200_TYPE_Q4_K, nq, h, 1);
        if (c.qkv_bias) {
            add("attn_q.bias", B200_TYPE_F32, nq, 1, 1);
            add("attn_k.bias", B200_TYPE_F32, nkv, 1, 1);
            add("attn_v.bias", B200_TYPE_F32, nkv, 1, 1);
        }
        if (c.qk_norm) {
            add("attn_q_norm.weight", B200_TYPE_F32, hd, 1, 1);
            add("attn_k_norm.weight", B200_TYPE_F32, hd, 1, 1);
        }
        add("ffn_norm.weight", B200_TYPE_F32, h, 1, 1);
        if (c.n_expert > 0) {
            add("ffn_gate_inp.weight", B200_TYPE_F32, h, c.n_expert, 1);
            add("ffn_gate_exps.weight", B200_TYPE_Q4_K, h, c.n_ff_exp, c.n_expert);
            add("ffn_up_exps.weight", B200_TYPE_Q4_K, h, c.n_ff_exp, c.n_expert);
            add("ffn_down_exps.weight", alt, c.n_ff_exp, h, c.n_expert);
        } else {
            add("ffn_gate.weight", B200_TYPE_Q4_K, h, c.n_ff, 1);
            add("ffn_up.weight", B200_TYPE_Q4_K, h, c.n_ff, 1);
            add("ffn_down.weight", alt, c.n_ff, h, 1);
        }
    }
    if (c.has_output) {
        add_tensor(st, "output_norm.weight", B200_TYPE_F32, h, 1, 1);
        add_tensor(st, "output.weight", B200_TYPE_Q6_K, h, c.n_vocab, 1);
    }
    b200_status rc = B200_OK;
    auto A = [&](void **p, size_t bytes) {
        if (rc == B200_OK) rc = dev_alloc(st, p, bytes);
    };
    for (auto &t : st->tensors) A(&t.dev, t.dev_bytes + 16);
    const int64_t n_local = c.layer_end - c.layer_begin;
    const size_t kv_rows = (size_t)(n_local * c.n_seq * c.n_ctx * c.n_head_kv);
    const size_t kv_k = kv_rows * st->k_row, kv_v = kv_rows * st->v_row;
    A((void **)&st->kc, kv_k);
    A((void **)&st->vc, kv_v);
    const int64_t R = st->rows_max = c.n_ubatch;
    const int64_t ff = c.n_expert > 0 ? 0 : c.n_ff;
    const int64_t pairs = c.n_expert > 0 ? R * c.n_expert_used : 0;
    st->kmax = std::max<int64_t>(std::max<int64_t>(h, nq), std::max<int64_t>(ff, (int64_t)c.n_ff_exp));
    const int64_t qrows = std::max<int64_t>(R, pairs);
    A((void **)&st->x, R * h * 4);
    A((void **)&st->xn, R * h * 4);
    A((void **)&st->q, R * nq * 4);
    A((void **)&st->k, R * nkv * 4);
    A((void **)&st->v, R * nkv * 4);
    A((void **)&st->att, R * nq * 4);
    A((void **)&st->g, R * ff * 4);
    A((void **)&st->u, R > 8 ? R * ff * 4 : 0);
    A((void **)&st->aq, qrows * st->kmax);
    A((void **)&st->ad, qrows * (st->kmax / 256) * 4);
    A((void **)&st->abs16, qrows * (st->kmax / 16) * 2);
    st->att_scratch_bytes = (size_t)std::min<int64_t>(R, 64) * c.n_head * 64 * (hd + 2) * 4;
    A((void **)&st->att_scratch, st->att_scratch_bytes);
    A((void **)&st->pos0_dev, 256);
    A((void **)&st->rid_scratch, 1024);
    A((void **)&st->attn_counters, (size_t)c.n_seq * c.n_head_kv * 4 + 256);
    A((void **)&st->emit_counters, (size_t)(c.n_ff / 256 + 1) * 4);
    if (rc == B200_OK && cudaMemset(st->emit_counters, 0, (size_t)(c.n_ff / 256 + 1) * 4) != cudaSuccess) rc = B200_ERR_CUDA;
    if (c.has_output) A((void **)&st->logits_int, (size_t)c.n_seq * c.n_vocab * 4);
    if (c.has_output) {
        st->scan_scratch_bytes = b200_logit_signals_scratch_bytes(std::max<int64_t>(R, c.n_seq));
        A(&st->scan_scratch, st->scan_scratch_bytes);
        if (rc == B200_OK && cudaMemset(st->scan_scratch, 0, st->scan_scratch_bytes) != cudaSuccess) rc = B200_ERR_CUDA;
    }
    if (c.n_expert > 0) {
        A((void **)&st->rl, R * c.n_expert * 4);
        A((void **)&st->rw, pairs * 4);
        A((void **)&st->rid, pairs * 4);
        A((void **)&st->hp, pairs * c.n_ff_exp * 4);
        A((void **)&st->hp2, R > 8 ? pairs * c.n_ff_exp * 4 : 0);
        st->moe_sorted_bytes = kq_moe_sort_scratch_bytes(pairs, c.n_expert);
        A((void **)&st->moe_sorted, st->moe_sorted_bytes);
        A((void **)&st->yp, pairs * h * 4);
        A((void **)&st->expert_mask, 256);
        if (rc == B200_OK && cudaMemset(st->expert_mask, 1, 256) != cudaSuccess) rc = B200_ERR_CUDA;
        A((void **)&st->moe_counters, 256);
        if (rc == B200_OK && cudaMemset(st->moe_counters, 0, 256) != cudaSuccess) rc = B200_ERR_CUDA;
    }
    if (rc == B200_OK && cudaStreamCreateWithFlags(&st->cap_stream, cudaStreamNonBlocking) != cudaSuccess) {
        kq_set_error("stage: cudaStreamCreate failed");
        rc = B200_ERR_CUDA;
    }
    if (rc == B200_OK && cudaMemset(st->attn_counters, 0, (size_t)c.n_seq * c.n_head_kv * 4 + 256) != cudaSuccess) {
        kq_set_error("stage: clearing the attention counters failed");
        rc = B200_ERR_CUDA;
    }
    if (rc == B200_OK && kv_rows) {
        if (cudaMemset(st->kc, 0, kv_k) != cudaSuccess || cudaMemset(st->vc, 0, kv_v) != cudaSuccess) {
            kq_set_error("stage: clearing the KV cache failed");
            rc = B200_ERR_CUDA;
        }
    }
    if (rc != B200_OK) {
        b200_stage_free(st);
        return rc;
    }
    const char *ng = getenv("B200_NO_GRAPH");
    st->use_graph = !(ng && ng[0] == '1');
    *out = st;
    return B200_OK;
}

void b200_stage_free(b200_stage *st) {
    if (!st) return;
    KqDevGuard dev_guard(st->c.device);
    cudaDeviceSynchronize();
    for (auto &g : st->graphs)
        if (g.second.exec) cudaGraphExecDestroy(g.second.exec);
    if (st->cap_stream) cudaStreamDestroy(st->cap_stream);
    for (void *p : st->allocs) cudaFree(p);
    delete st;
}

int64_t b200_stage_tensor_count(b200_stage *st) { return st ? (int64_t)st->tensors.size() : -1; }

b200_status b200_stage_tensor_info(b200_stage *st, int64_t i, char *name, size_t name_cap, uint32_t *type, int64_t ne[3]) {
    KQ_REQUIRE(st && name && name_cap > 0, "stage_tensor_info: null argument");
    KQ_REQUIRE(i >= 0 && i < (int64_t)st->tensors.size(), "stage_tensor_info: index %lld out of range", (long long)i);
    const StTensor &t = st->tensors[(size_t)i];
    KQ_REQUIRE(t.name.size() < name_cap, "stage_tensor_info: name buffer of %zu bytes is too small", name_cap);
    snprintf(name, name_cap, "%s", t.name.c_str());
    if (type) *type = t.type;
    if (ne)
        for (int d = 0; d < 3; d++) ne[d] = t.ne[d];
    return B200_OK;
}

b200_status b200_stage_set_tensor(b200_stage *st, const char *name, uint32_t type, const void *host_data,
                                  size_t nbytes) {
    KQ_REQUIRE(st && name && host_data, "stage_set_tensor: null argument");
    StTensor *t = find(st, name);
    if (!t) {
        kq_set_error("stage_set_tensor: %s is not a tensor of this stage", name);
        return B200_ERR_INVALID;
    }
    const int64_t rows = t->ne[1] * t->ne[2];
    KQ_REQUIRE(type == B200_TYPE_F32 ? t->type == B200_TYPE_F32
                                     : (type == B200_TYPE_Q4_K || type == B200_TYPE_Q6_K) &&
                                           t->type != B200_TYPE_F32,
               "stage_set_tensor: %s cannot take type %u", name, type);
    const size_t want = (size_t)(kq_row_bytes(type, t->ne[0]) * rows);
    if (nbytes != want) {
        kq_set_error("stage_set_tensor: %s expects %zu bytes, got %zu", name, want, nbytes);
        return B200_ERR_BOUNDS;
    }
    KqDevGuard dev_guard(st->c.device);
    if (type != t->type) { // same shape, other K-quant: reallocate the device rows
        void *p = nullptr;
        const size_t nb = (size_t)(kq_device_row_bytes(type, t->ne[0]) * rows);
        KQ_TRY(dev_alloc(st, &p, nb + 16));
        t->dev = p;
        t->dev_bytes = nb;
        t->type = type;
        st->resolved = false;
        for (auto &g : st->graphs)
            if (g.second.exec) cudaGraphExecDestroy(g.second.exec);
        st->graphs.clear();
    }
    if (type == B200_TYPE_Q6_K) {
        void *tmp = nullptr;
        if (cudaMalloc(&tmp, nbytes + 16) != cudaSuccess) {
            cudaGetLastError();
            kq_set_error("stage_set_tensor: staging allocation of %zu bytes failed", nbytes);
            return B200_ERR_ALLOC;
        }
        cudaError_t e = cudaMemcpy(tmp, host_data, nbytes, cudaMemcpyHostToDevice);
        b200_status rc = e == cudaSuccess ? b200_repack_q6k(tmp, t->dev, rows, t->ne[0], nullptr) : B200_ERR_CUDA;
        if (rc == B200_OK && cudaDeviceSynchronize() != cudaSuccess) rc = B200_ERR_CUDA;
        cudaFree(tmp);
        if (rc != B200_OK) {
            kq_set_error("stage_set_tensor: upload of %s failed", name);
            return rc;
        }
    } else {
        KQ_CUDA(cudaMemcpy(t->dev, host_data, nbytes, cudaMemcpyHostToDevice));
    }
    t->loaded = true;
    return B200_OK;
}

b200_status b200_stage_get_tensor(b200_stage *st, const char *name, void *host_data, size_t nbytes) {
    KQ_REQUIRE(st && name && host_data, "stage_get_tensor: null argument");
    StTensor *t = find(st, name);
    if (!t) {
        kq_set_error("stage_get_tensor: %s is not a tensor of this stage", name);
        return B200_ERR_INVALID;
    }
    const int64_t rows = t->ne[1] * t->ne[2];
    const size_t want = (size_t)(kq_row_bytes(t->type, t->ne[0]) * rows);
    if (nbytes != want) {
        kq_set_error("stage_get_tensor: %s holds %zu bytes, asked for %zu", name, want, nbytes);
        return B200_ERR_BOUNDS;
    }
    KqDevGuard dev_guard(st->c.device);
    if (t->type == B200_TYPE_Q6_K) {
        void *tmp = nullptr;
        if (cudaMalloc(&tmp, nbytes + 16) != cudaSuccess) {
            cudaGetLastError();
            return B200_ERR_ALLOC;
        }
        b200_status rc = b200_unpack_q6k(t->dev, tmp, rows, t->ne[0], nullptr);
        if (rc == B200_OK && cudaMemcpy(host_data, tmp, nbytes, cudaMemcpyDeviceToHost) != cudaSuccess)
            rc = B200_ERR_CUDA;
        cudaFree(tmp);
        return rc;
    }
    KQ_CUDA(cudaMemcpy(host_data, t->dev, nbytes, cudaMemcpyDeviceToHost));
    return B200_OK;
}

b200_status b200_stage_generate(b200_stage *st, uint64_t seed) {
    KQ_REQUIRE(st, "stage_generate: null stage");
    KqDevGuard dev_guard(st->c.device);
    for (auto &t : st->tensors) {
        const uint64_t key = mix64_host(seed ^ name_hash(t.name.c_str()));
        const bool is_norm = t.name.find("norm.weight") != std::string::npos;
        KQ_TRY(kq_synth_weights(t.type, t.dev, t.ne[1] * t.ne[2], t.ne[0], key, is_norm ? 1.0f : 0.0f, 0.02f,
                                nullptr));
        t.loaded = true;
    }
    KQ_CUDA(cudaDeviceSynchronize());
    return B200_OK;
}

size_t b200_stage_weight_bytes(b200_stage *st) {
    size_t n = 0;
    if (st)
        for (auto &t : st->tensors) n += (size_t)(kq_row_bytes(t.type, t.ne[0]) * t.ne[1] * t.ne[2]);
    return n;
}

b200_status b200_stage_forward(b200_stage *st, const int32_t *tokens, const float *hidden_in, int32_t seq0,
                               int32_t n_seq, int32_t T, int32_t pos0, float *hidden_out, float *logits,
                               int32_t all_logits, int32_t *next_tokens, void *stream) {
    KQ_REQUIRE(st, "stage_forward: null stage");
    const b200_stage_config &c = st->c;
    KQ_REQUIRE(n_seq >= 1 && seq0 >= 0 && seq0 + n_seq <= c.n_seq && T >= 1,
               "stage_forward: seq0=%d n_seq=%d T=%d (cache holds %d sequences)", seq0, n_seq, T, c.n_seq);
    KQ_REQUIRE((int64_t)n_seq * T <= st->rows_max, "stage_forward: %d rows exceed n_ubatch=%d", n_seq * T,
               st->rows_max);
    KQ_REQUIRE(pos0 >= 0 && pos0 + T <= c.n_ctx, "stage_forward: positions [%d,%d) exceed n_ctx=%d", pos0,
               pos0 + T, c.n_ctx);
    KQ_REQUIRE(c.has_embd ? tokens != nullptr : hidden_in != nullptr, "stage_forward: missing input");
    KQ_REQUIRE(c.has_output || hidden_out, "stage_forward: missing hidden_out");
    KqDevGuard dev_guard(c.device);
    KQ_TRY(resolve(st));
    cudaStream_t s = (cudaStream_t)stream;
    const long long before = g_kq_launches;
    if (T == 1 && st->use_graph) {
        // decode step: positions come from device memory so one captured graph serves every step
        const int n_split = kq_attention_decode_splits(pos0 + 1, n_seq * st->c.n_head_kv);
        GraphKey key;
        memset(&key, 0, sizeof(key));
        key.n_seq = n_seq;
        key.n_split = 0; // the slice count changes every 128 positions: the entry is updated in place, not re-keyed
        key.seq0 = seq0;
        key.tokens = tokens;
        key.hidden_in = hidden_in;
        key.hidden_out = hidden_out;
        key.logits = logits;
        key.next = next_tokens;
        auto it = st->graphs.find(key);
        if (it == st->graphs.end() || it->second.n_split != n_split) {
            cudaGraph_t graph = nullptr;
            KQ_CUDA(cudaStreamBeginCapture(st->cap_stream, cudaStreamCaptureModeThreadLocal));
            b200_status rc = forward_body(st, tokens, hidden_in, seq0, n_seq, 1, pos0, true, n_split, hidden_out,
                                          logits, all_logits, next_tokens, st->cap_stream);
            cudaError_t e = cudaStreamEndCapture(st->cap_stream, &graph);
            if (rc != B200_OK) {
                if (graph) cudaGraphDestroy(graph);
                return rc;
            }
            KQ_CUDA(e);
            const long long n_launch = g_kq_launches - before;
            if (it != st->graphs.end()) {
                // same topology, other attention grids: patch the instantiated graph (about a millisecond)
                // instead of instantiating a new one (tens of milliseconds)
                cudaGraphExecUpdateResultInfo info;
                if (cudaGraphExecUpdate(it->second.exec, graph, &info) != cudaSuccess) {
                    cudaGetLastError();
                    cudaGraphExecDestroy(it->second.exec);
                    it->second.exec = nullptr;
                    e = cudaGraphInstantiate(&it->second.exec, graph, 0);
                }
                cudaGraphDestroy(graph);
                KQ_CUDA(e);
                it->second.n_split = n_split;
                it->second.launches = n_launch;
            } else {
                GraphEntry ge;
                ge.launches = n_launch;
                ge.n_split = n_split;
                e = cudaGraphInstantiate(&ge.exec, graph, 0);
                cudaGraphDestroy(graph);
                KQ_CUDA(e);
                it = st->graphs.emplace(key, ge).first;
            }
        }
        kq_launch(set_pos_kernel, 1, 1, 0, s, st->pos0_dev, pos0);
        KQ_LAUNCH_CHECK();
        KQ_CUDA(cudaGraphLaunch(it->second.exec, s));
        st->launches += it->second.launches + 1;
        g_kq_launches = before + it->second.launches + 1;
        return B200_OK;
    }
    b200_status rc = forward_body(st, tokens, hidden_in, seq0, n_seq, T, pos0, false, 0, hidden_out, logits,
                                  all_logits, next_tokens, s);
    st->launches += g_kq_launches - before;
    return rc;
}

b200_status b200_stage_profile_decode(b200_stage *st, int32_t n_seq, int32_t pos0, uint32_t classes,
                                      int32_t iters, float *ms_per_step, int64_t *launches_per_step) {
    KQ_REQUIRE(st && ms_per_step && iters >= 1, "stage_profile_decode: bad arguments");
    const b200_stage_config &c = st->c;
    KQ_REQUIRE(n_seq >= 1 && n_seq <= c.n_seq && n_seq <= st->rows_max && pos0 >= 0 && pos0 < c.n_ctx,
               "stage_profile_decode: n_seq=%d pos0=%d", n_seq, pos0);
    KQ_REQUIRE((classes & ~CLS_ALL) == 0 && classes != 0, "stage_profile_decode: classes mask");
    KqDevGuard dev_guard(c.device);
    KQ_TRY(resolve(st));
    // inputs of the replayed step live in the stage's own scratch (their values do not matter)
    int32_t *tok = (int32_t *)st->rid_scratch;
    float *hin = st->xn, *hout = st->att;
    cudaStream_t s = st->cap_stream;
    KQ_CUDA(cudaMemsetAsync(tok, 0, 256, s));
    kq_launch(set_pos_kernel, 1, 1, 0, s, st->pos0_dev, pos0);
    KQ_LAUNCH_CHECK();
    const long long before = g_kq_launches;
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
    KQ_CUDA(cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal));
    b200_status rc = forward_body(st, tok, hin, 0, n_seq, 1, pos0, true,
                                  kq_attention_splits(n_seq, c.n_head_kv, pos0 + 1),
                                  c.has_output ? nullptr : hout, nullptr, 0,
                                  c.has_output ? (int32_t *)st->rid_scratch + 32 : nullptr, s, classes);
    cudaError_t e = cudaStreamEndCapture(s, &graph);
    const long long per_step = g_kq_launches - before;
    g_kq_launches = before;
    if (rc != B200_OK) {
        if (graph) cudaGraphDestroy(graph);
        return rc;
    }
    KQ_CUDA(e);
    e = cudaGraphInstantiate(&exec, graph, 0);
    cudaGraphDestroy(graph);
    KQ_CUDA(e);
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0);
    cudaEventCreate(&e1);
    for (int i = 0; i < 2; i++) cudaGraphLaunch(exec, s); // warm-up
    cudaEventRecord(e0, s);
    for (int i = 0; i < iters; i++) cudaGraphLaunch(exec, s);
    cudaEventRecord(e1, s);
    e = cudaStreamSynchronize(s);
    float ms = 0.f;
    cudaEventElapsedTime(&ms, e0, e1);
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    cudaGraphExecDestroy(exec);
    KQ_CUDA(e);
    *ms_per_step = ms / iters;
    if (launches_per_step) *launches_per_step = per_step;
    return B200_OK;
}

b200_status b200_stage_peek(b200_stage *st, const char *which, float *host_out, size_t n_floats) {
    KQ_REQUIRE(st && which && host_out, "stage_peek: null argument");
    const b200_stage_config &c = st->c;
    const size_t R = (size_t)st->rows_max, nq = (size_t)c.n_head * c.head_dim, nkv = (size_t)c.n_head_kv * c.head_dim;
    const float *src = nullptr;
    size_t cap = 0;
    const std::string w(which);
    if (w == "x") { src = st->x; cap = R * c.n_embd; }
    else if (w == "q") { src = st->q; cap = R * nq; }
    else if (w == "k") { src = st->k; cap = R * nkv; }
    else if (w == "v") { src = st->v; cap = R * nkv; }
    else if (w == "att") { src = st->att; cap = R * nq; }
    else if (w == "g") { src = st->g; cap = R * (size_t)(c.n_expert > 0 ? 0 : c.n_ff); }
    else if (w == "hp") { src = st->hp; cap = R * (size_t)c.n_expert_used * c.n_ff_exp; }
    else if (w == "yp") { src = st->yp; cap = R * (size_t)c.n_expert_used * c.n_embd; }
    else if (w == "sorted") { src = (const float *)st->moe_sorted; cap = st->moe_sorted_bytes / 4; }
    else if (w == "rid") { src = (const float *)st->rid; cap = R * (size_t)c.n_expert_used; }
    KQ_REQUIRE(src, "stage_peek: no buffer named %s (x, q, k, v, att, g)", which);
    KQ_REQUIRE(n_floats <= cap, "stage_peek: %s holds %zu floats, asked for %zu", which, cap, n_floats);
    KqDevGuard dev_guard(c.device);
    KQ_CUDA(cudaDeviceSynchronize());
    KQ_CUDA(cudaMemcpy(host_out, src, n_floats * 4, cudaMemcpyDeviceToHost));
    return B200_OK;
}

b200_status b200_stage_set_expert_mask(b200_stage *st, const uint8_t *mask, int32_t n_mask) {
    KQ_REQUIRE(st, "stage_set_expert_mask: null stage");
    KQ_REQUIRE(st->c.n_expert > 0, "stage_set_expert_mask: the stage has no experts");
    KQ_REQUIRE(!mask || n_mask == st->c.n_expert, "stage_set_expert_mask: %d entries for %d experts", n_mask,
               st->c.n_expert);
    KqDevGuard dev_guard(st->c.device);
    // The router always reads the stage's mask array (a captured decode graph holds its address);
    // "no mask" is all ones.  The copy is ordered after everything already queued on the device.
    uint8_t host[256];
    for (int i = 0; i < 256; i++) host[i] = (!mask || i >= n_mask) ? 1 : (mask[i] ? 1 : 0);
    KQ_CUDA(cudaDeviceSynchronize());
    KQ_CUDA(cudaMemcpy(st->expert_mask, host, 256, cudaMemcpyHostToDevice));
    return B200_OK;
}

b200_status b200_stage_synchronize(b200_stage *st) {
    KQ_REQUIRE(st, "stage_synchronize: null stage");
    KqDevGuard dev_guard(st->c.device);
    KQ_CUDA(cudaDeviceSynchronize());
    const int werr = kq_stream_error_fetch() | (kq_gemm_error_fetch() << 4) | (kq_attn_tc_error_fetch() << 8);
    if (werr) {
        kq_set_error("stage_synchronize: a bounded device-side wait gave up (code %d)", werr);
        return B200_ERR_TIMEOUT;
    }
    return B200_OK;
}

int64_t b200_stage_kernel_launches(b200_stage *st) { return st ? st->launches : 0; }

} // extern "C"
