/*
 * b200_kquant.h -- C ABI of the B200 (sm_100a) K-quant stage library.
 *
 * This is the drop-in boundary for the one hot path every mesh-llm serving stage executes: the
 * quantised forward pass that llama.cpp's scheduler drives through the ggml backend interface
 * inside `llama-server` / `rpc-server` (spawned by mesh-llm/src/inference/launch.rs:887 and
 * :1250).  The reference reaches that interface through the calls visible in its patch queue;
 * each group below cites the call it replaces.  "patches/000N" means
 * third_party/llama.cpp/patches/000N-*.patch in the reference tree.
 *
 * Rules of the ABI: plain pointers and sizes, opaque handles, no exceptions cross it, every
 * entry point returns a status (or bool where the reference call does) and never aborts.
 * Device pointers are CUDA device addresses; `stream` is a cudaStream_t passed as void*
 * (NULL = the legacy default stream).  There is no CPU fallback anywhere behind this header:
 * an unsupported request returns B200_ERR_UNSUPPORTED.
 */
#ifndef B200_KQUANT_H
#define B200_KQUANT_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200_API __attribute__((visibility("default")))

/* ---- status (ggml_status-like: 0 success, negative failure) -------------------------------- */
typedef int32_t b200_status;
enum {
    B200_OK = 0,
    B200_ERR_INVALID = -1,     /* bad argument / shape / alignment                            */
    B200_ERR_ALLOC = -2,       /* device or host allocation failed (GGML_STATUS_ALLOC_FAILED)  */
    B200_ERR_CUDA = -3,        /* a CUDA runtime call failed; see b200_last_error()            */
    B200_ERR_UNSUPPORTED = -4, /* op / type not on the hot path                               */
    B200_ERR_BOUNDS = -5,      /* access outside the owning buffer                            */
    B200_ERR_TIMEOUT = -6,     /* a bounded device-side wait gave up                          */
    B200_ERR_STATE = -7        /* call made in the wrong state (e.g. weights not loaded)      */
};
B200_API const char *b200_status_string(b200_status s);
B200_API const char *b200_last_error(void); /* thread-local, valid until the next failing call */
/* Synchronises the current device and reports B200_ERR_TIMEOUT if any bounded device-side wait
 * (copy barrier, tensor-core commit, cross-CTA flag) gave up since the last check; the results of
 * the affected launch are then invalid.  Clears the condition.  A stage whose step was affected
 * keeps arrival counters of that step in its own memory: close it and create it again.          */
B200_API b200_status b200_check_device_waits(void);

/* ---- tensor types: ggml type ids (mesh-client/src/models/gguf.rs:19-35) -------------------- */
enum {
    B200_TYPE_F32 = 0,
    B200_TYPE_F16 = 1,
    B200_TYPE_Q4_0 = 2,  /* KV-cache rows only: 32 elements / 18 bytes */
    B200_TYPE_Q8_0 = 8,  /* KV-cache rows only: 32 elements / 34 bytes */
    B200_TYPE_Q4_K = 12, /* 256 elements / 144 bytes */
    B200_TYPE_Q6_K = 14, /* 256 elements / 210 bytes */
    B200_TYPE_I32 = 26
};

/* ---- ops understood by graph_compute (the subset on the hot path) -------------------------- */
enum {
    B200_OP_NONE = 0,
    B200_OP_MUL_MAT,     /* src0 = weights [K, N] (Q4_K/Q6_K/F32), src1 = x [K, M] f32 -> [N, M]  */
    B200_OP_MUL_MAT_ID,  /* src0 = experts [K, N, E], src1 = x [K, n_used|1, T], src2 = ids i32   */
    B200_OP_RMS_NORM,    /* op_params[0] = eps (f32 bits)                                         */
    B200_OP_MUL,         /* broadcast multiply by a row vector (norm weight)                      */
    B200_OP_ADD,         /* elementwise, or broadcast add of a row vector (bias)                  */
    B200_OP_ROPE,        /* src1 = positions i32; op_params: [0]=n_dims [1]=mode(0 norm, 2 neox)
                            [2]=theta (f32 bits)                                                 */
    B200_OP_SWIGLU,      /* silu(src0) * src1                                                     */
    B200_OP_GET_ROWS,    /* src0 = table (Q4_K/Q6_K/F32), src1 = ids i32                          */
    B200_OP_CPY,         /* f32 -> f32 / f16 / q8_0 / q4_0 (KV-cache write; quantised rows in ggml's
                            34 / 18-byte blocks)                                                  */
    B200_OP_ATTN,        /* fused causal attention (FLASH_ATTN_EXT): src0 = q [hd, n_head, T],
                            src1 = K cache [hd, n_kv, n_ctx] of type f16, q8_0 or q4_0 (ggml block
                            layout, read in place; quantised: hd = 128), src2 = V cache likewise;
                            op_params[0] = scale (f32 bits), [1] = pos0                          */
    B200_OP_MOE_ROUTE,   /* softmax + top-k + renormalise: src0 = logits [E, T];
                            op_params[0] = k; output = weights f32 [k, T]; ids written to src1   */
    B200_OP_ARGMAX,
    B200_OP_COUNT
};

/* ---- tensor descriptor: field-for-field the wire form `rpc_tensor`
 *      (patches/0002 lines 1070-1085; 296 bytes packed).  ne[0] is the contiguous dimension,
 *      nb[] are strides in bytes, `data` is a device address inside `buffer`.               */
#pragma pack(push, 1)
typedef struct b200_tensor {
    uint64_t id;
    uint32_t type;
    uint64_t buffer; /* b200_buffer* as integer */
    uint32_t ne[4];
    uint32_t nb[4];
    uint32_t op;
    int32_t op_params[16];
    int32_t flags;
    uint64_t src[10]; /* ids of source tensors, 0 = none */
    uint64_t view_src;
    uint64_t view_offs;
    uint64_t data;
    char name[64];
    char padding[4];
} b200_tensor;
#pragma pack(pop)

typedef struct b200_buffer b200_buffer;
typedef struct b200_backend b200_backend;
typedef struct b200_stage b200_stage;

/* ---- registry and devices: ggml_backend_reg / ggml_backend_dev
 *      (device selection by name, launch.rs:69-82 and :920-925; ggml_backend_dev_memory,
 *      patches/0002 lines 464-467).                                                        */
B200_API const char *b200_reg_name(void); /* "B200" */
B200_API int32_t b200_reg_device_count(void);
B200_API b200_status b200_dev_name(int32_t dev, char *out, size_t cap); /* "B200_<i>" */
B200_API b200_status b200_dev_description(int32_t dev, char *out, size_t cap);
B200_API b200_status b200_dev_memory(int32_t dev, size_t *free_bytes, size_t *total_bytes);
/* 1 if graph_compute can run `node` whose sources have the given types, else 0               */
B200_API int32_t b200_dev_supports_op(uint32_t op, uint32_t type_src0, uint32_t type_src1);

/* ---- buffer type: get_alignment / get_max_size / get_alloc_size
 *      (patches/0001 lines 96-147, patches/0002 lines 352-371).                             */
B200_API size_t b200_buft_alignment(void);
B200_API size_t b200_buft_max_size(int32_t dev);
/* bytes a tensor occupies on the device; Q6_K rows are padded to 16 bytes by the repack      */
B200_API size_t b200_buft_alloc_size(uint32_t type, const uint32_t ne[4]);

/* ---- buffers: alloc / free / get_base / clear / init_tensor / set_tensor / get_tensor /
 *      cpy_tensor (patches/0001 lines 68-91, patches/0002 lines 181-261).  set_tensor repacks
 *      Q6_K into the device layout and get_tensor returns the original bytes; every access is
 *      bounds-checked against the owning buffer (patches/0001 lines 228-239).               */
B200_API b200_status b200_buffer_alloc(int32_t dev, size_t size, b200_buffer **out);
B200_API void b200_buffer_free(b200_buffer *buf);
B200_API void *b200_buffer_get_base(b200_buffer *buf);
B200_API size_t b200_buffer_get_size(b200_buffer *buf);
B200_API int32_t b200_buffer_get_device(b200_buffer *buf);
B200_API b200_status b200_buffer_clear(b200_buffer *buf, uint8_t value);
B200_API b200_status b200_buffer_init_tensor(b200_buffer *buf, b200_tensor *t);
B200_API b200_status b200_buffer_set_tensor(b200_buffer *buf, const b200_tensor *t,
                                            const void *host_data, size_t offset, size_t size);
B200_API b200_status b200_buffer_get_tensor(b200_buffer *buf, const b200_tensor *t,
                                            void *host_data, size_t offset, size_t size);
/* Stage-boundary hand-off.  Replaces ggml_backend_rpc_buffer_cpy_tensor ->
 * RPC_CMD_PUSH_TENSOR_TO_PEER -> RPC_CMD_PEER_TENSOR_DATA (patches/0002 lines 184-259 and
 * 544-622: device -> host vector -> TCP -> host -> device) by one device-to-device copy over
 * NVLink.  Copies `size` bytes starting `offset` bytes into both tensors.  Returns 1 on
 * success and 0 if the copy cannot be done directly, in which case the caller falls back to
 * get_tensor + set_tensor exactly as the reference does (patches/0002 lines 250-254).       */
B200_API int32_t b200_buffer_cpy_tensor(const b200_tensor *src, const b200_tensor *dst,
                                        size_t offset, size_t size);

/* ---- backend: graph_compute / synchronize (patches/0002 lines 443-459).  The graph arrives
 *      the way the RPC server receives it: node ids in execution order plus the table of all
 *      tensors they reference.                                                             */
B200_API b200_status b200_backend_init(int32_t dev, b200_backend **out);
B200_API void b200_backend_free(b200_backend *be);
B200_API b200_status b200_backend_graph_compute(b200_backend *be, const uint64_t *node_ids,
                                                uint32_t n_nodes, const b200_tensor *tensors,
                                                uint32_t n_tensors);
B200_API b200_status b200_backend_synchronize(b200_backend *be);
B200_API void *b200_backend_stream(b200_backend *be);

/* ---- direct kernel entry points (device pointers) -------------------------------------------
 * ORDERING RULE for everything below that launches a matmul (b200_mul_mat, b200_mul_mat_q8,
 * b200_mul_mat_static, b200_stage_forward, b200_backend_graph_compute): per device, such calls must
 * be ordered on the GPU -- issued to one stream, or to streams the caller has ordered with events.
 * The decode kernels combine partial sums through small per-device arrays inside the library (and the
 * prefill GEMM keeps a per-device staging buffer); two matmul launches that overlap on one GPU would
 * read each other's entries and return wrong numbers without any error.  This is the reference's own
 * calling pattern: one decode thread per llama-server, and in rpc-server every backend call behind
 * one mutex (patches/0002 lines 320-337).  Calls may come from different host threads as long as
 * they do not overlap.  Activation pointers (x, q) must be 16-byte aligned.
 *
 * Weight matrices passed to these are in DEVICE layout: Q4_K rows are the GGUF bytes
 * unchanged; Q6_K rows are repacked (b200_repack_q6k) into groups of 8 blocks, each group
 * [ql | qh | scales | d] with chunk-major ql / qh planes, 1680 bytes, so that a row slice is one
 * aligned contiguous run.                                                                    */
B200_API size_t b200_row_bytes(uint32_t type, int64_t k);        /* GGUF bytes of one row     */
B200_API size_t b200_device_row_bytes(uint32_t type, int64_t k); /* device bytes of one row   */
B200_API b200_status b200_repack_q6k(const void *gguf_rows_dev, void *device_rows, int64_t n_rows,
                                     int64_t k, void *stream);
B200_API b200_status b200_unpack_q6k(const void *device_rows, void *gguf_rows_dev, int64_t n_rows,
                                     int64_t k, void *stream);

/* f32 activations -> Q8 blocks of 256: q int8 [M][K], d f32 [M][K/256], bsum16 int16 [M][K/16] */
B200_API b200_status b200_quantize_act(const float *x, int64_t M, int64_t K, int8_t *q, float *d,
                                       int16_t *bsum16, void *stream);
/* bytes of scratch b200_mul_mat needs for M x K activations                                    */
B200_API size_t b200_mul_mat_scratch_bytes(int64_t M, int64_t K);
/* y[M][N] = W[N x K] . x[M][K].  MUL_MAT of the ggml op surface for Q4_K / Q6_K weights:
 * decode GEMV for M <= 8, tiled GEMM above.  `scratch` holds the quantised activations.       */
B200_API b200_status b200_mul_mat(uint32_t type, const void *W, const float *x, int64_t M,
                                  int64_t N, int64_t K, float *y, void *scratch,
                                  size_t scratch_bytes, void *stream);
/* same contraction on already-quantised activations, with optional fused epilogue:
 * y = W.x (+ bias[N]) (+ residual[M][N])                                                       */
B200_API b200_status b200_mul_mat_q8(uint32_t type, const void *W, const int8_t *q, const float *d,
                                     const int16_t *bsum16, int64_t M, int64_t N, int64_t K,
                                     float *y, const float *bias, const float *residual,
                                     void *stream);
/* MUL_MAT_ID of the ggml op surface (build_moe_ffn's expert matmuls, third_party/llama.cpp/patches/0003
 * lines 82-108): W holds E expert matrices [N x K] one after the other (device layout); pair p of the
 * n_pairs (token, slot) pairs uses expert ids[p] (device i32) on activation row p / (n_pairs / n_x_rows)
 * of x [n_x_rows][K] and writes y[p][N].  With more than 8 pairs the pairs are gathered per expert (a
 * stable counting sort on the device) and every expert's rows go through the tensor-core GEMM in one
 * grouped launch; with fewer, one streamed matrix-vector product per pair.  E <= 256.               */
B200_API size_t b200_mul_mat_id_scratch_bytes(int64_t n_x_rows, int64_t n_pairs, int64_t K, int64_t E);
B200_API b200_status b200_mul_mat_id(uint32_t type, const void *W, int64_t E, const float *x, int64_t n_x_rows,
                                     const int32_t *ids, int64_t n_pairs, int64_t N, int64_t K, float *y,
                                     void *scratch, size_t scratch_bytes, void *stream);
/* The same contraction as b200_mul_mat for callers that must not allocate and have no scratch
 * to lend (no counterpart in the reference; an addition of this library).  Meant for a stage whose
 * device memory was budgeted in full before it started, for a decode loop that cannot afford
 * cudaMalloc's device-wide synchronisation, and for hosts that own all device memory through their
 * own allocator.  The quantised activations go to a fixed array that is part of the library image,
 * so every GPU that loads the library holds about 292 KiB for it until the process exits.
 * Limits: M <= 8 tokens and K <= 32768; anything larger returns B200_ERR_INVALID with a message
 * (use b200_mul_mat with caller scratch instead).  The call itself performs no cudaMalloc /
 * cudaFree.  The first call on each device looks the array's address up once
 * (cudaGetSymbolAddress, with that device current); make that first call before starting any
 * stream capture.  All calls on a device share the one array: calls whose kernels can overlap on
 * the GPU (different streams) race on it, so serialise them.  Nothing needs clearing between
 * calls -- each call rewrites every byte it later reads.                                        */
#define B200_MUL_MAT_STATIC_MAX_TOKENS 8
#define B200_MUL_MAT_STATIC_MAX_K 32768
B200_API b200_status b200_mul_mat_static(uint32_t type, const void *W, const float *x, int64_t M,
                                         int64_t N, int64_t K, float *y, void *stream);
/* Measurement aid with no counterpart in the reference: times a bare loop of the prefill GEMM's
 * tensor-core instruction (tcgen05.mma kind::i8, M 128 x N 256 x K 32, operands resting in shared
 * memory, no loads and no epilogue) on every SM of the current device and returns the int8 rate
 * in TOP/s (best of `repeats` launches of `n_mma` instructions per SM) -- the measured ceiling
 * the GEMM's useful rate is reported against.  Synchronises the device.                         */
B200_API b200_status b200_probe_int8_mma(int32_t n_mma, int32_t repeats, double *tops_out, double *ms_out);
/* exact per-block integer sums [M][N][K/256] (parity instrumentation; summ may be NULL)        */
B200_API b200_status b200_block_sums(uint32_t type, const void *W, const int8_t *q,
                                     const int16_t *bsum16, int64_t M, int64_t N, int64_t K,
                                     int32_t *sumi, int32_t *summ, void *stream);

B200_API b200_status b200_rms_norm(const float *x, const float *w, int64_t T, int64_t h, float eps,
                                   float *y, void *stream);
B200_API b200_status b200_rope(float *x, const int32_t *pos, int64_t T, int64_t n_head, int64_t hd,
                               float theta, int32_t neox, void *stream);
B200_API b200_status b200_swiglu(const float *gate, const float *up, int64_t n, float *y,
                                 void *stream);
B200_API b200_status b200_add(const float *a, const float *b, int64_t n, float *y, void *stream);
B200_API b200_status b200_add_bias(float *y, const float *bias, int64_t T, int64_t n, void *stream);
B200_API b200_status b200_cpy_f32_f16(const float *x, int64_t n, uint16_t *y, void *stream);
B200_API b200_status b200_attention(const float *q, const uint16_t *k_cache, const uint16_t *v_cache,
                                    int64_t T, int64_t pos0, int64_t n_head, int64_t n_kv,
                                    int64_t hd, float *out, void *scratch, size_t scratch_bytes,
                                    void *stream);
B200_API size_t b200_attention_scratch_bytes(int64_t T, int64_t n_head, int64_t hd, int64_t n_ctx);
/* Quantised KV cache: the --cache-type-k / --cache-type-v pairs mesh-llm starts its servers with
 * (mesh-llm/src/inference/launch.rs:568-591: f16 / f16 below 5 GB of model, q8_0 K + q4_0 V from 5
 * to 50 GB, q4_0 / q4_0 above).  Block arithmetic is ggml's block_q8_0 / block_q4_0; on the device
 * a row (one position, one KV head) holds the codes of its hd / 32 blocks, then their f16 scales,
 * padded to a multiple of 16 bytes: b200_kv_row_bytes (hd = 128: 144 / 80 bytes; f16: 2 hd).
 * b200_kv_store rotates k by RoPE at pos[t] and writes the K / V rows of T tokens at those
 * positions of one sequence's caches ([position][n_kv] rows); b200_attention_kv is b200_attention
 * over caches of the given types (quantised types need hd = 128).                               */
B200_API size_t b200_kv_row_bytes(uint32_t type, int64_t hd);
/* the pair mesh-llm picks for a model file of this size (thresholds 5e9 and 50e9 bytes)          */
B200_API void b200_kv_types_for_model_bytes(uint64_t model_bytes, uint32_t *k_type, uint32_t *v_type);
B200_API b200_status b200_kv_store(const float *k, const float *v, const int32_t *pos, int64_t T,
                                   int64_t n_kv, int64_t hd, float theta, int32_t neox,
                                   uint32_t k_type, uint32_t v_type, void *k_cache, void *v_cache,
                                   void *stream);
B200_API b200_status b200_attention_kv(const float *q, const void *k_cache, const void *v_cache,
                                       uint32_t k_type, uint32_t v_type, int64_t T, int64_t pos0,
                                       int64_t n_head, int64_t n_kv, int64_t hd, float *out,
                                       void *scratch, size_t scratch_bytes, void *stream);
B200_API b200_status b200_get_rows(uint32_t type, const void *W, const int32_t *ids, int64_t T,
                                   int64_t K, float *y, void *stream);
B200_API b200_status b200_argmax(const float *x, int64_t T, int64_t n, int32_t *idx, void *stream);
/* Router of the expert layer (build_moe_ffn, third_party/llama.cpp/patches/0003 lines 82-108):
 * softmax over the E logits of a token, the k largest selected (ties to the lower index), their
 * probabilities renormalised to sum 1.  The masked form adds the reference's expert mask before the
 * selection: mask (device, one byte per expert, 1 = allowed, NULL = none) gives a masked expert the
 * selection value -inf, the weights still come from the unmasked probabilities.                  */
B200_API b200_status b200_moe_route(const float *logits, int64_t T, int64_t E, int64_t k,
                                    int32_t *ids, float *w, void *stream);
B200_API b200_status b200_moe_route_masked(const float *logits, int64_t T, int64_t E, int64_t k,
                                           const uint8_t *mask, int32_t *ids, float *w, void *stream);
/* Statistics of the output distribution per row of logits [T][n], computed on the device: what the
 * reference's server derives on the CPU from the full-vocabulary softmax after the prefill and
 * after every generated token when its mesh hooks are on (third_party/llama.cpp/patches/0005:
 * mesh_compute_entropy = -sum p log2 p, margin = p[0] - p[1], the top tokens of the hook payload,
 * the probability of the sampled token).  chosen (device, optional): the sampled token per row,
 * default the argmax.  argmax_out (device, optional) receives the greedy token (lowest index on
 * ties).  scratch: b200_logit_signals_scratch_bytes(T) bytes of device memory, zeroed once by the
 * caller before the first use; calls that share it must be ordered on one stream.                */
typedef struct b200_logit_signals_t {
    float entropy;  /* bits                                                                   */
    float margin;   /* p(top 1) - p(top 2); 1 for a single-entry row                           */
    float p_chosen;
    float top_p[5]; /* probabilities of the five most likely tokens, best first                */
    int32_t top_id[5];
} b200_logit_signals_t;
B200_API size_t b200_logit_signals_scratch_bytes(int64_t T);
B200_API b200_status b200_logit_signals(const float *logits, int64_t T, int64_t n, const int32_t *chosen,
                                        b200_logit_signals_t *signals, int32_t *argmax_out,
                                        void *scratch, size_t scratch_bytes, void *stream);

/* ---- stage: one contiguous layer range of a model resident on one GPU ------------------------
 * This is what a mesh-llm worker is: `rpc-server -d DEV --gguf PATH` holding blk.[a,b) and
 * loading exactly its own tensors by name from its local GGUF (patches/0001 lines 179-266);
 * the partition follows election.rs:3095-3114 (contiguous ranges, embeddings on the first
 * stage, output_norm + output on the last).                                                 */
typedef struct b200_stage_config {
    int32_t n_layer, layer_begin, layer_end;
    int32_t n_embd, n_head, n_head_kv, head_dim, n_ff, n_vocab;
    int32_t n_expert, n_expert_used, n_ff_exp; /* 0 = dense                                   */
    int32_t n_ctx, n_seq;                      /* KV cache: n_seq sequences of n_ctx tokens   */
    int32_t rope_neox, qkv_bias, qk_norm;
    int32_t has_embd, has_output;
    float rms_eps, rope_theta;
    int32_t n_ubatch; /* largest number of tokens per forward call                           */
    int32_t device;
    int32_t kv_type_k, kv_type_v; /* KV-cache row types: 0 or B200_TYPE_F16, B200_TYPE_Q8_0, B200_TYPE_Q4_0 */
} b200_stage_config;

B200_API b200_status b200_stage_create(const b200_stage_config *cfg, b200_stage **out);
B200_API void b200_stage_free(b200_stage *st);
/* load one tensor by its GGUF name from host memory in GGUF byte layout                        */
B200_API b200_status b200_stage_set_tensor(b200_stage *st, const char *name, uint32_t type,
                                           const void *host_data, size_t nbytes);
/* read a tensor back in GGUF byte layout (inverse of the device repack)                        */
B200_API b200_status b200_stage_get_tensor(b200_stage *st, const char *name, void *host_data,
                                           size_t nbytes);
/* fill every tensor with seeded N(0, 0.02) weights quantised on the device to the Q4_K_M mix   */
B200_API b200_status b200_stage_generate(b200_stage *st, uint64_t seed);
B200_API size_t b200_stage_weight_bytes(b200_stage *st);
/* Run T tokens per sequence for `n_seq_active` sequences (rows ordered sequence-major; they use
 * KV-cache slots seq0 .. seq0 + n_seq_active - 1) starting at position pos0.  First stage: tokens (device i32); other stages: hidden_in (device f32
 * [rows][n_embd]).  Last stage writes logits for the last token of each sequence (or all rows
 * if all_logits) and the greedy argmax into next_tokens; other stages write hidden_out.        */
B200_API b200_status b200_stage_forward(b200_stage *st, const int32_t *tokens,
                                        const float *hidden_in, int32_t seq0, int32_t n_seq_active,
                                        int32_t T, int32_t pos0, float *hidden_out, float *logits,
                                        int32_t all_logits, int32_t *next_tokens, void *stream);
/* Timing instrumentation: captures one decode step (T = 1, n_seq sequences at position pos0) into
 * a CUDA graph restricted to the kernel classes in `classes` (1 = quantised GEMV, 2 = attention,
 * 4 = everything else, 7 = the whole step), replays it `iters` times and reports the mean device
 * time per step measured with CUDA events.  Outputs of a partial step are meaningless.          */
B200_API b200_status b200_stage_profile_decode(b200_stage *st, int32_t n_seq, int32_t pos0,
                                               uint32_t classes, int32_t iters, float *ms_per_step,
                                               int64_t *launches_per_step);
/* the tensors a stage owns, by GGUF name: what a loader has to supply (ne[0] = row length K,
 * ne[1] = rows, ne[2] = experts or 1); type is the type currently allocated                      */
B200_API int64_t b200_stage_tensor_count(b200_stage *st);
B200_API b200_status b200_stage_tensor_info(b200_stage *st, int64_t i, char *name, size_t name_cap,
                                            uint32_t *type, int64_t ne[3]);
/* Expert mask of a mixture-of-experts stage: llama_model_set_expert_mask (patches/0003 lines 44-48 and
 * 159-181).  mask (host): n_mask bytes, nonzero = expert allowed; NULL clears the mask.  Returns
 * B200_ERR_INVALID when n_mask is not the stage's expert count (the reference returns -1) or the
 * stage is dense.  Takes effect from the next forward call, captured decode graphs included.    */
B200_API b200_status b200_stage_set_expert_mask(b200_stage *st, const uint8_t *mask, int32_t n_mask);
/* Diagnostics: copies the first n_floats of one of the stage's activation buffers, as the last forward
 * call (of the stage's last layer) left it, to host memory.  which: "q", "k", "v" (projections; q and
 * k after RoPE when T > 1), "att" (attention output), "g" (SwiGLU output), "x" (residual stream).     */
B200_API b200_status b200_stage_peek(b200_stage *st, const char *which, float *host_out, size_t n_floats);
B200_API b200_status b200_stage_synchronize(b200_stage *st);
B200_API int64_t b200_stage_kernel_launches(b200_stage *st); /* launches issued so far        */

/* ---- GGUF container: header scan, tensor index, selective load --------------------------------
 * Replaces, for this path, the header scanner mesh-llm uses to plan a deployment
 * (mesh-client/src/models/gguf.rs:319-421 compact metadata, :476-572 resident / expert byte
 * profile, limits :4-9) and the worker-side load of a stage's own tensors by name from its local
 * file (SET_TENSOR_GGUF, third_party/llama.cpp/patches/0001 lines 179-266).  Malformed files are
 * rejected with B200_ERR_INVALID and a message; nothing aborts.                                  */
typedef struct b200_gguf b200_gguf;
typedef struct b200_gguf_meta {
    char architecture[64], tokenizer_model[64];
    uint32_t context_length, vocab_size, embedding_length, head_count, head_count_kv, block_count;
    uint32_t feed_forward_length, key_length, value_length;
    uint32_t expert_count, expert_used_count, expert_feed_forward_length;
    float rope_freq_base, rope_scale, rms_epsilon;
} b200_gguf_meta;
typedef struct b200_gguf_tensor {
    char name[128];
    uint32_t type, n_dims; /* ggml type id                                                    */
    int64_t ne[4];
    uint64_t file_offset;  /* absolute offset of the tensor's bytes in the file               */
    uint64_t nbytes;       /* from type and shape; 0 when the type's block size is not known  */
} b200_gguf_tensor;
typedef struct b200_gguf_byte_profile_t {
    uint32_t expert_count, expert_used_count;
    uint64_t full_model_bytes, base_resident_bytes, expert_tensor_bytes, file_overhead_bytes;
} b200_gguf_byte_profile_t;

B200_API b200_status b200_gguf_open(const char *path, b200_gguf **out);
B200_API void b200_gguf_close(b200_gguf *g);
B200_API b200_status b200_gguf_get_meta(const b200_gguf *g, b200_gguf_meta *out);
B200_API int64_t b200_gguf_tensor_count(const b200_gguf *g);
B200_API b200_status b200_gguf_tensor_info(const b200_gguf *g, int64_t i, b200_gguf_tensor *out);
B200_API int64_t b200_gguf_find_tensor(const b200_gguf *g, const char *name); /* -1: not in the file */
B200_API b200_status b200_gguf_read_tensor(const b200_gguf *g, int64_t i, void *dst, size_t nbytes);
B200_API b200_status b200_gguf_byte_profile(const b200_gguf *g, b200_gguf_byte_profile_t *out);
/* stage configuration for layers [layer_begin, layer_end) of the model in the file (layer_end < 0:
 * to the last layer); embeddings go with layer 0, output_norm + output with the last layer       */
B200_API b200_status b200_gguf_stage_config(const b200_gguf *g, int32_t layer_begin, int32_t layer_end,
                                            int32_t n_ctx, int32_t n_seq, int32_t n_ubatch,
                                            int32_t device, b200_stage_config *cfg);
/* reads every tensor the stage owns, and nothing else, from the file and uploads it               */
B200_API b200_status b200_stage_load_gguf(b200_stage *st, const b200_gguf *g, int64_t *n_loaded,
                                          int64_t *bytes_read);

/* ---- expert shards of a mixture-of-experts model ----------------------------------------------
 * Which experts a node holds (mesh-llm/src/inference/moe.rs:535-636: mode 0 = shared core of the
 * `min_experts` most used experts on every node, the rest round-robin with `overlap` copies each;
 * mode 1 = shared core + snake draft), and the file a node loads: trunk + the listed experts, the
 * router rows gathered, expert_count rewritten and expert_used_count clamped (llama-moe-split,
 * third_party/llama.cpp/patches/0003 lines 945-955, 1040-1113, 1142-1191).                        */
B200_API b200_status b200_moe_assign(const uint32_t *ranking, int32_t n_expert, int32_t n_nodes,
                                     int32_t min_experts, int32_t overlap, int32_t mode, int32_t node,
                                     uint32_t *experts_out, int32_t cap, int32_t *n_out,
                                     int32_t *n_shared, int32_t *n_unique);
B200_API b200_status b200_gguf_write_expert_shard(const b200_gguf *g, const int32_t *expert_ids,
                                                  int32_t n_ids, const char *dst_path,
                                                  uint64_t *bytes_written);

/* ---- stage-boundary hand-off through peer memory -----------------------------------------------
 * Replaces the activation transfer between two stages (third_party/llama.cpp/patches/0002 lines
 * 544-622: device -> host -> TCP -> host -> device; direct push lines 624-735) for stages on GPUs
 * of one box.  The receiver creates an endpoint: a ring of n_slots landing slots in its own HBM.
 * The sender maps it (handoff_open with the 64-byte handle exported by the receiver's process, or
 * handoff_open_local inside one process) and sends payload number seqno = 0, 1, 2, ... : one
 * kernel writes the payload over NVLink and publishes the number.  The receiver's handoff_wait is
 * one kernel that acquires payload seqno and copies it to dst (dst null: *slot is the payload in
 * place; call handoff_release(seqno) after its readers).  Waits are bounded by limit_ns (0 = 5 s):
 * when one runs out, nothing is copied and handoff_status (call it after synchronising the stream)
 * returns 1 on the sender's mapping (no free slot) or 2 on the endpoint (payload not arrived); the
 * calls that follow on that object then give up at once.  Sizes are multiples of 4 bytes.        */
typedef struct b200_handoff b200_handoff;
B200_API b200_status b200_handoff_create(size_t slot_bytes, int32_t n_slots, b200_handoff **out);
B200_API b200_status b200_handoff_export(const b200_handoff *endpoint, void *handle64);
B200_API b200_status b200_handoff_open(const void *handle64, size_t slot_bytes, int32_t n_slots,
                                       b200_handoff **out);
B200_API b200_status b200_handoff_open_local(const b200_handoff *endpoint, b200_handoff **out);
B200_API b200_status b200_handoff_send(b200_handoff *remote, const void *src, size_t bytes,
                                       uint64_t seqno, uint64_t limit_ns, void *stream);
B200_API b200_status b200_handoff_wait(b200_handoff *endpoint, void *dst, size_t bytes, uint64_t seqno,
                                       uint64_t limit_ns, const void **slot, void *stream);
B200_API b200_status b200_handoff_release(b200_handoff *endpoint, uint64_t seqno, void *stream);
B200_API b200_status b200_handoff_status(b200_handoff *h, int32_t *status);
B200_API void b200_handoff_free(b200_handoff *h);

/* ---- worker front end: the ggml RPC wire protocol (version 4.1) served from this backend ------
 * What mesh-llm spawns as `rpc-server -d DEV -p PORT --gguf PATH` (mesh-llm/src/inference/launch.rs:
 * 887-933).  Commands and packed messages as in third_party/llama.cpp/patches/0002 lines 1042-1146
 * and patches/0001 lines 49-63; REGISTER_PEER / PUSH_TENSOR_TO_PEER / PEER_TENSOR_DATA as in
 * patches/0002 lines 544-735 (a push between two devices of one server is a single NVLink copy).
 * port 0 picks a free port.  The server runs on its own threads until it is stopped.              */
typedef struct b200_rpc_server b200_rpc_server;
B200_API b200_status b200_rpc_server_start(const char *host, int32_t port, const char *gguf_path,
                                           b200_rpc_server **out);
B200_API int32_t b200_rpc_server_port(const b200_rpc_server *srv);
B200_API void b200_rpc_server_stop(b200_rpc_server *srv);

#ifdef __cplusplus
}
#endif
#endif /* B200_KQUANT_H */
