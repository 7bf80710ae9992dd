/*
 * kquant_oracle.h -- CPU oracle for the K-quant forward pass.  TEST INFRASTRUCTURE ONLY.
 *
 * This is a plain-C restatement of the arithmetic that mesh-llm's serving stages execute
 * inside llama.cpp/ggml (the dependency pinned at third_party/llama.cpp/upstream.txt:1,
 * 45155597aa23243c5f6d10064bd9bca3eaddee16, which is NOT vendored in the reference tree).
 * It is the checker for the CUDA path and the timed CPU baseline; nothing in the product
 * library links, imports or calls it.
 *
 * PARITY STATUS: the block formats (Q4_K / Q6_K decode) are pinned against gguf-py's
 * independent decoder via committed golden vectors; the stage hand-off is pinned byte-exact
 * the way patches/0002 test_direct_push pins it.  The quantised contraction, norms, RoPE,
 * attention and MoE routing are "parity unpinned": the reference holds no golden vector for
 * them (its CI only asserts non-empty completions), so this file restates the published
 * algorithm and the activation quantiser below is this repository's own specification.
 *
 * Conventions (ggml's): ne0 is the contiguous K dimension; a weight matrix [N x K] holds
 * N rows of K/256 blocks; activations are [M tokens x K] f32 row-major.
 */
#ifndef KQUANT_ORACLE_H
#define KQUANT_ORACLE_H

#include <stdint.h>
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ORC_QK_K 256
#define ORC_Q4K_BYTES 144 /* f16 d, f16 dmin, 12 B scales/mins, 128 B nibbles */
#define ORC_Q6K_BYTES 210 /* 128 B ql, 64 B qh, 16 x int8 scales, f16 d     */

/* ggml type ids (constants.py GGMLQuantizationType) */
enum { ORC_TYPE_F32 = 0, ORC_TYPE_F16 = 1, ORC_TYPE_Q4_0 = 2, ORC_TYPE_Q8_0 = 8, ORC_TYPE_Q4_K = 12, ORC_TYPE_Q6_K = 14 };

/* ---- block formats ------------------------------------------------------------------- */
void orc_dequant_q4k(const uint8_t *blocks, int64_t nblocks, float *out);
void orc_dequant_q6k(const uint8_t *blocks, int64_t nblocks, float *out);
/* plain (non-search) weight quantisers; any valid block is a valid input to the path */
void orc_quantize_q4k(const float *x, int64_t n, uint8_t *out);
void orc_quantize_q6k(const float *x, int64_t n, uint8_t *out);
int64_t orc_row_bytes(int type, int64_t k);

/* ---- activation quantiser (repository specification) ------------------------------------
 * blocks of 256 along K:  amax = max|x|, d = amax/127, id = d ? 1/d : 0,
 * q = clamp(rint(x*id), -127, 127) (ties to even), bsum16[t] = sum of q over 16 elements.
 * q: [M][K] int8, d: [M][K/256] f32, bsum16: [M][K/16] int16.                              */
void orc_quantize_act(const float *x, int64_t M, int64_t K, int8_t *q, float *d, int16_t *bsum16);

/* ---- quantised contraction -------------------------------------------------------------- */
/* per (m, n, block) integer sums.  Q4_K: sumi = sum_j sc_j * sum_i q_ij a_ij,
 * summ = sum_j m_j * bsum_j.  Q6_K: sumi = sum_t sc_t * sum_i (q-32)_ti a_ti, summ = 0.
 * layout [M][N][K/256] int32.                                                              */
void orc_block_sums(int type, const uint8_t *W, const int8_t *q, const int16_t *bsum16,
                    int64_t M, int64_t N, int64_t K, int32_t *sumi, int32_t *summ);
/* y[M][N] = W[N x K] . x[M][K] with x quantised by orc_quantize_act                        */
void orc_mul_mat(int type, const uint8_t *W, const float *x, int64_t M, int64_t N, int64_t K,
                 float *y);
void orc_mul_mat_q8(int type, const uint8_t *W, const int8_t *q, const float *d,
                    const int16_t *bsum16, int64_t M, int64_t N, int64_t K, float *y);

/* ---- surrounding ops --------------------------------------------------------------------- */
void orc_rms_norm(const float *x, const float *w, int64_t T, int64_t h, float eps, float *y);
/* x: [T][n_head][hd] in place; neox!=0 pairs (i, i+hd/2), else (2i, 2i+1)                   */
void orc_rope(float *x, const int32_t *pos, int64_t T, int64_t n_head, int64_t hd, float theta,
              int neox);
void orc_rope_inv_freq(float theta, int64_t hd, float *inv_freq /* hd/2 */);
void orc_swiglu(const float *gate, const float *up, int64_t n, float *y);
void orc_f32_to_f16(const float *x, int64_t n, uint16_t *y);
void orc_f16_to_f32(const uint16_t *x, int64_t n, float *y);
/* causal attention of T new queries at positions pos0.. against an f16 KV cache that already
 * holds rows [0, pos0+T).  q: [T][n_head][hd]; k/v cache: [n_ctx][n_kv][hd] f16.            */
void orc_attention(const float *q, const uint16_t *kc, const uint16_t *vc, int64_t T,
                   int64_t pos0, int64_t n_head, int64_t n_kv, int64_t hd, float *out);
/* KV-cache row formats (ggml block_q8_0: f16 d + 32 x int8, 34 bytes; block_q4_0: f16 d + 16 bytes
 * of nibbles, element j in the low and element j + 16 in the high nibble of byte j, 18 bytes).
 * Quantisers as published in ggml-quants.c (quantize_row_q8_0_ref: d = amax / 127, q = round(x / d);
 * quantize_row_q4_0_ref: d = (the element of largest magnitude) / -8, q = min(15, (int)(x / d + 8.5)));
 * mesh-llm selects these types by model size (mesh-llm/src/inference/launch.rs:568-591).    */
void orc_quantize_q8_0(const float *x, int64_t n, uint8_t *blocks);
void orc_quantize_q4_0(const float *x, int64_t n, uint8_t *blocks);
void orc_dequant_q8_0(const uint8_t *blocks, int64_t nblocks, float *out);
void orc_dequant_q4_0(const uint8_t *blocks, int64_t nblocks, float *out);
/* what attention reads back from a cache of `type` for the f32 row x: x itself rounded to f16
 * (F16), or quantised, decoded and rounded to f16                                           */
void orc_kv_round_trip(int type, const float *x, int64_t n, uint16_t *y);
void orc_get_rows(int type, const uint8_t *W, const int32_t *ids, int64_t T, int64_t K, float *y);
void orc_argmax(const float *x, int64_t T, int64_t n, int32_t *idx);
/* router: softmax over E logits, top-k (ties -> lower id), weights renormalised to sum 1     */
void orc_moe_route(const float *logits, int64_t T, int64_t E, int64_t k, int32_t *ids, float *w);
/* the same with the reference's expert mask (one byte per expert, 1 = allowed; NULL = none) */
void orc_moe_route_masked(const float *logits, int64_t T, int64_t E, int64_t k, const uint8_t *mask,
                          int32_t *ids, float *w);

/* ---- whole stage ------------------------------------------------------------------------- */
typedef struct {
    int32_t n_layer;      /* layers of the full model                         */
    int32_t layer_begin;  /* this stage holds blk.[layer_begin, layer_end)    */
    int32_t layer_end;
    int32_t n_embd, n_head, n_head_kv, head_dim, n_ff, n_vocab;
    int32_t n_expert, n_expert_used, n_ff_exp; /* 0 = dense                   */
    int32_t n_ctx, n_seq;
    int32_t rope_neox, qkv_bias, qk_norm;
    int32_t has_embd, has_output;              /* first / last stage          */
    float rms_eps, rope_theta;
    int32_t kv_type_k, kv_type_v; /* 0 or ORC_TYPE_F16 = f16; ORC_TYPE_Q8_0; ORC_TYPE_Q4_0      */
} orc_config;

typedef struct orc_model orc_model;

orc_model *orc_model_create(const orc_config *cfg);
void orc_model_free(orc_model *m);
/* seeded N(0, 0.02) f32 weights quantised to the Q4_K_M mix (Q4_K; attn_v / ffn_down on odd
 * layers and output.weight Q6_K; norms 1 + N(0,0.02); router / biases f32 N(0,0.02)).
 * The stream depends on (seed, tensor name) only, so a stage holds the same bytes as the
 * corresponding slice of the full model.                                                    */
void orc_model_generate(orc_model *m, uint64_t seed);
/* tensor access by GGUF name ("blk.3.attn_q.weight"); returns 0 if absent                   */
int orc_model_get_tensor(orc_model *m, const char *name, int32_t *type, const void **data,
                         int64_t *nbytes, int64_t ne[3]);
int orc_model_set_tensor(orc_model *m, const char *name, int32_t type, const void *data,
                         int64_t nbytes);
/* expert mask of a mixture-of-experts model: one byte per expert (1 = allowed), NULL clears;
 * returns -1 when n_mask is not the model's expert count, else 0                            */
int orc_model_set_expert_mask(orc_model *m, const uint8_t *mask, int32_t n_mask);
int orc_model_n_tensors(orc_model *m);
const char *orc_model_tensor_name(orc_model *m, int i);
/* run T tokens of sequence `seq` starting at position pos0.  First stage takes tokens, other
 * stages take hidden_in [T][n_embd].  Last stage writes logits [T][n_vocab] (if logits != 0)
 * else hidden_out [T][n_embd] is the stage-boundary activation.                             */
int orc_model_forward(orc_model *m, int32_t seq, const int32_t *tokens, const float *hidden_in,
                      int64_t T, int64_t pos0, float *hidden_out, float *logits);
void orc_set_threads(int n);
int orc_get_threads(void);

#ifdef __cplusplus
}
#endif
#endif
