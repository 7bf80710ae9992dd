// The ggml-shaped boundary: buffers that own device memory, tensor set/get with the Q6_K repack,
// the device-to-device stage hand-off (cpy_tensor), and graph_compute over the ops of the hot path.
//
// The shape follows what the reference's RPC server does with a backend: alloc_buffer / get_base /
// set_tensor / get_tensor / copy / graph_compute, every access bounds-checked against the owning
// buffer (third_party/llama.cpp/patches/0001 lines 228-239, patches/0002 lines 570-582).
#include "kq_common.cuh"
#include "kq_kvq.cuh"

#include <math.h>
#include <mutex>
#include <string.h>
#include <unordered_map>
#include <vector>

b200_status kq_rms_norm(const float *x, const float *w, int64_t T, int64_t h, float eps, float *y,
                        int8_t *q, float *d, int16_t *bs, cudaStream_t st, int64_t x_row_stride = 0);
b200_status kq_attention(const float *q, const uint16_t *kc, const uint16_t *vc, int n_seq, int T,
                         const int32_t *pos0_dev, int pos0, int n_head, int n_kv, int hd,
                         int64_t seq_stride, float *out, float *scratch, size_t scratch_bytes,
                         int force_splits, KqKvTypes kvt, cudaStream_t st);
b200_status kq_f32_matmul(const float *W, const float *x, int64_t M, int64_t N, int64_t K, float *y,
                          cudaStream_t st);

struct b200_buffer {
    int32_t dev;
    uint8_t *base;
    size_t size;
};

struct b200_backend {
    int32_t dev;
    cudaStream_t stream;
    void *scratch;
    size_t scratch_bytes;
    std::mutex mu; // one graph at a time per device, as the reference serialises its backend calls
};

namespace {

__global__ void mul_rows_kernel(const float *a, const float *b, int64_t total, int64_t n, int64_t nb_elems,
                                float *y) {
    KQ_PDL_ENTER();
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < total) y[i] = a[i] * b[nb_elems == total ? i : i % n];
}
__global__ void add_bcast_kernel(const float *a, const float *b, int64_t total, int64_t n, int64_t nb_elems,
                                 float *y) {
    KQ_PDL_ENTER();
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < total) y[i] = a[i] + b[nb_elems == total ? i : i % n];
}

// CPY f32 -> q8_0 / q4_0: how llama.cpp writes a quantised KV cache.  One warp per block of 32 values,
// ggml's block layout at the destination.
__global__ void cpy_f32_kvq_kernel(const float *x, int64_t n_blocks, int type, uint8_t *dst) {
    KQ_PDL_ENTER();
    const int64_t blk = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (blk >= n_blocks) return; // whole warps leave together
    const int lane = threadIdx.x & 31;
    kq_kv_store_ggml_block(type, x[blk * 32 + lane], dst + blk * (type == KQ_KV_Q8_0 ? 34 : 18), lane);
}

// A quantised cache tensor in ggml's block layout -> this library's row layout (codes of a row's blocks,
// then their scales; 16-byte aligned rows, which the attention kernels fetch as TMA boxes).  Bytes are
// moved, never changed.  One thread per block of a row.
__global__ void kvq_ggml_to_rows_kernel(const uint8_t *src, int64_t n_rows, int hd, int type, uint8_t *dst) {
    KQ_PDL_ENTER();
    const int nb = hd / 32, cb = type == KQ_KV_Q8_0 ? 32 : 16;
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_rows * nb) return;
    const int64_t r = i / nb;
    const int b = (int)(i % nb);
    const uint16_t *in = reinterpret_cast<const uint16_t *>(src + (r * nb + b) * (cb + 2));
    uint8_t *row = dst + r * kq_kv_row_bytes(type, hd);
    reinterpret_cast<uint16_t *>(row + nb * cb)[b] = in[0];
    uint16_t *codes = reinterpret_cast<uint16_t *>(row + b * cb);
    for (int k = 0; k < cb / 2; k++) codes[k] = in[1 + k];
}

inline int64_t nelements(const b200_tensor *t) {
    return (int64_t)t->ne[0] * t->ne[1] * t->ne[2] * t->ne[3];
}
inline int64_t nrows(const b200_tensor *t) { return (int64_t)t->ne[1] * t->ne[2] * t->ne[3]; }
inline size_t gguf_bytes(const b200_tensor *t) {
    if (t->type == B200_TYPE_I32) return (size_t)nelements(t) * 4;
    return (size_t)(kq_row_bytes(t->type, t->ne[0]) * nrows(t));
}
inline size_t device_bytes(const b200_tensor *t) {
    if (t->type == B200_TYPE_I32) return (size_t)nelements(t) * 4;
    return (size_t)(kq_device_row_bytes(t->type, t->ne[0]) * nrows(t));
}

// The four extents arrive as 32-bit words from the wire; their product has to stay far inside int64
// (and inside any buffer this library can allocate) for the byte counts below to mean anything.
inline bool extents_ok(const b200_tensor *t) {
    uint64_t n = 1;
    for (int i = 0; i < 4; i++) {
        if (t->ne[i] == 0) return true; // an empty tensor: every product is 0
        n *= (uint64_t)t->ne[i];
        if (n > (1ull << 46)) return false;
    }
    return true;
}

// tensor [data, data + device_bytes) must lie inside its buffer
b200_status check_tensor(const b200_tensor *t) {
    KQ_REQUIRE(t, "null tensor");
    if (!extents_ok(t)) {
        kq_set_error("tensor %.64s: extents %u x %u x %u x %u overflow", t->name, t->ne[0], t->ne[1], t->ne[2], t->ne[3]);
        return B200_ERR_BOUNDS;
    }
    const b200_buffer *buf = (const b200_buffer *)(uintptr_t)t->buffer;
    KQ_REQUIRE(buf && buf->base, "tensor %.64s has no buffer", t->name);
    const uint64_t lo = (uint64_t)(uintptr_t)buf->base, hi = lo + buf->size;
    const uint64_t need = device_bytes(t);
    if (t->data < lo || t->data > hi || need > hi - t->data) {
        kq_set_error("tensor %.64s: [%llx, +%llu) is outside its buffer [%llx, +%zu)", t->name,
                     (unsigned long long)t->data, (unsigned long long)need, (unsigned long long)lo, buf->size);
        return B200_ERR_BOUNDS;
    }
    if (t->type == B200_TYPE_Q4_K || t->type == B200_TYPE_Q6_K) {
        KQ_REQUIRE(t->ne[0] % 256 == 0, "tensor %.64s: ne[0] must be a multiple of 256", t->name);
        KQ_REQUIRE((t->data & 15) == 0, "tensor %.64s: quantised data must be 16-byte aligned", t->name);
    }
    if (t->type == B200_TYPE_Q4_0 || t->type == B200_TYPE_Q8_0) {
        KQ_REQUIRE(t->ne[0] % 32 == 0, "tensor %.64s: ne[0] must be a multiple of 32", t->name);
        KQ_REQUIRE((t->data & 1) == 0, "tensor %.64s: q4_0 / q8_0 blocks must be 2-byte aligned", t->name);
    }
    return B200_OK;
}

#define KQ_TRY(expr)                      \
    do {                                  \
        b200_status rc__ = (expr);        \
        if (rc__ != B200_OK) return rc__; \
    } while (0)

struct DevGuard {
    int prev = -1;
    explicit DevGuard(int dev) {
        cudaGetDevice(&prev);
        if (prev != dev) cudaSetDevice(dev);
        else prev = -1;
    }
    ~DevGuard() {
        if (prev >= 0) cudaSetDevice(prev);
    }
};

// host <-> Q6_K tensor with an arbitrary byte window: work on whole rows through a staging copy
b200_status q6k_window(b200_buffer *buf, const b200_tensor *t, void *host, size_t offset, size_t size,
                       bool write) {
    const int64_t K = t->ne[0];
    const size_t rb = (size_t)kq_row_bytes(B200_TYPE_Q6_K, K), drb = (size_t)kq_device_row_bytes(B200_TYPE_Q6_K, K);
    const int64_t r0 = (int64_t)(offset / rb), r1 = (int64_t)((offset + size + rb - 1) / rb);
    const int64_t n = r1 - r0;
    uint8_t *dev_rows = (uint8_t *)(uintptr_t)t->data + (size_t)r0 * drb;
    void *tmp = nullptr;
    if (cudaMalloc(&tmp, (size_t)n * rb + 16) != cudaSuccess) {
        cudaGetLastError();
        kq_set_error("q6k staging allocation of %zu bytes failed", (size_t)n * rb);
        return B200_ERR_ALLOC;
    }
    b200_status rc = B200_OK;
    const bool whole = offset % rb == 0 && size % rb == 0;
    const size_t in_off = offset - (size_t)r0 * rb;
    if (write) {
        if (!whole) rc = b200_unpack_q6k(dev_rows, tmp, n, K, nullptr);
        if (rc == B200_OK && cudaMemcpy((uint8_t *)tmp + in_off, host, size, cudaMemcpyHostToDevice) != cudaSuccess)
            rc = B200_ERR_CUDA;
        if (rc == B200_OK) rc = b200_repack_q6k(tmp, dev_rows, n, K, nullptr);
        if (rc == B200_OK && cudaDeviceSynchronize() != cudaSuccess) rc = B200_ERR_CUDA;
    } else {
        rc = b200_unpack_q6k(dev_rows, tmp, n, K, nullptr);
        if (rc == B200_OK && cudaMemcpy(host, (uint8_t *)tmp + in_off, size, cudaMemcpyDeviceToHost) != cudaSuccess)
            rc = B200_ERR_CUDA;
    }
    cudaFree(tmp);
    if (rc == B200_ERR_CUDA) kq_set_error("q6k window transfer failed: %s", cudaGetErrorString(cudaGetLastError()));
    return rc;
}

b200_status window_check(b200_buffer *buf, const b200_tensor *t, const void *host, size_t offset, size_t size) {
    KQ_REQUIRE(buf && t && (host || size == 0), "null argument");
    KQ_REQUIRE((b200_buffer *)(uintptr_t)t->buffer == buf, "tensor %.64s does not belong to this buffer", t->name);
    KQ_TRY(check_tensor(t));
    const size_t total = gguf_bytes(t);
    if (offset > total || size > total - offset) {
        kq_set_error("tensor %.64s: window [%zu, +%zu) exceeds %zu bytes", t->name, offset, size, total);
        return B200_ERR_BOUNDS;
    }
    return B200_OK;
}

// the node's own tensor must have the type the kernel writes and room for every element it writes
b200_status out_holds(const b200_tensor *t, uint32_t type, int64_t n_elems) {
    if (t->type != type) {
        kq_set_error("graph_compute: node %.64s: output type %u, the op writes type %u", t->name, t->type, type);
        return B200_ERR_INVALID;
    }
    if (nelements(t) < n_elems) {
        kq_set_error("graph_compute: node %.64s: output holds %lld elements, the op writes %lld", t->name,
                     (long long)nelements(t), (long long)n_elems);
        return B200_ERR_BOUNDS;
    }
    return B200_OK;
}

float f32_param(const b200_tensor *t, int i) {
    float f;
    memcpy(&f, &t->op_params[i], 4);
    return f;
}

} // namespace

extern "C" {

b200_status b200_buffer_alloc(int32_t dev, size_t size, b200_buffer **out) {
    KQ_REQUIRE(out, "buffer_alloc: null out");
    *out = nullptr;
    KQ_REQUIRE(dev >= 0 && dev < b200_reg_device_count(), "buffer_alloc: no device %d", dev);
    DevGuard g(dev);
    void *p = nullptr;
    cudaError_t e = cudaMalloc(&p, size ? size : 256);
    if (e != cudaSuccess) {
        cudaGetLastError();
        kq_set_error("buffer_alloc: cudaMalloc(%zu) on device %d failed: %s", size, dev, cudaGetErrorString(e));
        return B200_ERR_ALLOC;
    }
    b200_buffer *b = new b200_buffer();
    b->dev = dev;
    b->base = (uint8_t *)p;
    b->size = size;
    *out = b;
    return B200_OK;
}

void b200_buffer_free(b200_buffer *buf) {
    if (!buf) return;
    DevGuard g(buf->dev);
    cudaFree(buf->base);
    delete buf;
}

void *b200_buffer_get_base(b200_buffer *buf) { return buf ? buf->base : nullptr; }
size_t b200_buffer_get_size(b200_buffer *buf) { return buf ? buf->size : 0; }
int32_t b200_buffer_get_device(b200_buffer *buf) { return buf ? buf->dev : -1; }

b200_status b200_buffer_clear(b200_buffer *buf, uint8_t value) {
    KQ_REQUIRE(buf, "buffer_clear: null buffer");
    DevGuard g(buf->dev);
    KQ_CUDA(cudaMemset(buf->base, value, buf->size));
    return B200_OK;
}

b200_status b200_buffer_init_tensor(b200_buffer *buf, b200_tensor *t) {
    KQ_REQUIRE(buf && t, "init_tensor: null argument");
    KQ_REQUIRE((b200_buffer *)(uintptr_t)t->buffer == buf, "init_tensor: tensor %.64s names another buffer", t->name);
    return check_tensor(t);
}

b200_status b200_buffer_set_tensor(b200_buffer *buf, const b200_tensor *t, const void *host_data, size_t offset,
                                   size_t size) {
    KQ_TRY(window_check(buf, t, host_data, offset, size));
    if (size == 0) return B200_OK;
    DevGuard g(buf->dev);
    if (t->type == B200_TYPE_Q6_K) return q6k_window(buf, t, const_cast<void *>(host_data), offset, size, true);
    KQ_CUDA(cudaMemcpy((uint8_t *)(uintptr_t)t->data + offset, host_data, size, cudaMemcpyHostToDevice));
    return B200_OK;
}

b200_status b200_buffer_get_tensor(b200_buffer *buf, const b200_tensor *t, void *host_data, size_t offset,
                                   size_t size) {
    KQ_TRY(window_check(buf, t, host_data, offset, size));
    if (size == 0) return B200_OK;
    DevGuard g(buf->dev);
    if (t->type == B200_TYPE_Q6_K) return q6k_window(buf, t, host_data, offset, size, false);
    KQ_CUDA(cudaMemcpy(host_data, (const uint8_t *)(uintptr_t)t->data + offset, size, cudaMemcpyDeviceToHost));
    return B200_OK;
}

int32_t b200_buffer_cpy_tensor(const b200_tensor *src, const b200_tensor *dst, size_t offset, size_t size) {
    if (!src || !dst) return 0;
    if (check_tensor(src) != B200_OK || check_tensor(dst) != B200_OK) return 0;
    if (src->type != dst->type || src->type == B200_TYPE_Q6_K) return 0; // repacked rows: use set/get
    const size_t ns = gguf_bytes(src), nd = gguf_bytes(dst);
    if (offset > ns || size > ns - offset || offset > nd || size > nd - offset) {
        kq_set_error("cpy_tensor: window [%zu, +%zu) exceeds src %zu / dst %zu bytes", offset, size, ns, nd);
        return 0;
    }
    if (size == 0) return 1;
    const b200_buffer *sb = (const b200_buffer *)(uintptr_t)src->buffer;
    const b200_buffer *db = (const b200_buffer *)(uintptr_t)dst->buffer;
    const void *sp = (const uint8_t *)(uintptr_t)src->data + offset;
    void *dp = (uint8_t *)(uintptr_t)dst->data + offset;
    DevGuard g(sb->dev);
    cudaError_t e;
    if (sb->dev == db->dev) {
        e = cudaMemcpy(dp, sp, size, cudaMemcpyDeviceToDevice);
    } else {
        // the stage boundary: one copy over NVLink, no host bounce
        e = cudaMemcpyPeer(dp, db->dev, sp, sb->dev, size);
    }
    if (e != cudaSuccess) {
        cudaGetLastError();
        kq_set_error("cpy_tensor: %s", cudaGetErrorString(e));
        return 0;
    }
    return 1;
}

b200_status b200_backend_init(int32_t dev, b200_backend **out) {
    KQ_REQUIRE(out, "backend_init: null out");
    *out = nullptr;
    KQ_REQUIRE(dev >= 0 && dev < b200_reg_device_count(), "backend_init: no device %d", dev);
    DevGuard g(dev);
    b200_backend *be = new b200_backend();
    be->dev = dev;
    be->scratch = nullptr;
    be->scratch_bytes = 0;
    if (cudaStreamCreateWithFlags(&be->stream, cudaStreamNonBlocking) != cudaSuccess) {
        kq_set_error("backend_init: stream creation failed");
        delete be;
        return B200_ERR_CUDA;
    }
    *out = be;
    return B200_OK;
}

void b200_backend_free(b200_backend *be) {
    if (!be) return;
    DevGuard g(be->dev);
    cudaStreamSynchronize(be->stream);
    cudaStreamDestroy(be->stream);
    if (be->scratch) cudaFree(be->scratch);
    delete be;
}

void *b200_backend_stream(b200_backend *be) { return be ? (void *)be->stream : nullptr; }

b200_status b200_backend_synchronize(b200_backend *be) {
    KQ_REQUIRE(be, "backend_synchronize: null backend");
    DevGuard g(be->dev);
    KQ_CUDA(cudaStreamSynchronize(be->stream));
    const int werr = kq_stream_error_fetch() | (kq_gemm_error_fetch() << 4) | (kq_attn_tc_error_fetch() << 8);
    if (werr) {
        kq_set_error("backend_synchronize: a bounded device-side wait gave up (code %d)", werr);
        return B200_ERR_TIMEOUT;
    }
    return B200_OK;
}

static b200_status ensure_scratch(b200_backend *be, size_t bytes) {
    if (bytes <= be->scratch_bytes) return B200_OK;
    cudaStreamSynchronize(be->stream);
    if (be->scratch) cudaFree(be->scratch);
    be->scratch = nullptr;
    be->scratch_bytes = 0;
    bytes = (bytes + (1 << 20)) & ~(size_t)((1 << 20) - 1);
    if (cudaMalloc(&be->scratch, bytes) != cudaSuccess) {
        cudaGetLastError();
        kq_set_error("graph_compute: scratch allocation of %zu bytes failed", bytes);
        return B200_ERR_ALLOC;
    }
    be->scratch_bytes = bytes;
    return B200_OK;
}

b200_status b200_backend_graph_compute(b200_backend *be, const uint64_t *node_ids, uint32_t n_nodes,
                                       const b200_tensor *tensors, uint32_t n_tensors) {
    KQ_REQUIRE(be && (node_ids || n_nodes == 0) && (tensors || n_tensors == 0), "graph_compute: null argument");
    std::lock_guard<std::mutex> lock(be->mu);
    DevGuard g(be->dev);
    std::unordered_map<uint64_t, const b200_tensor *> by_id;
    for (uint32_t i = 0; i < n_tensors; i++) by_id[tensors[i].id] = &tensors[i];
    cudaStream_t s = be->stream;
    auto src = [&](const b200_tensor *t, int i) -> const b200_tensor * {
        if (!t->src[i]) return nullptr;
        auto it = by_id.find(t->src[i]);
        return it == by_id.end() ? nullptr : it->second;
    };
    for (uint32_t ni = 0; ni < n_nodes; ni++) {
        auto it = by_id.find(node_ids[ni]);
        KQ_REQUIRE(it != by_id.end(), "graph_compute: node id %llu is not in the tensor table",
                   (unsigned long long)node_ids[ni]);
        const b200_tensor *t = it->second;
        if (t->op == B200_OP_NONE) continue;
        KQ_TRY(check_tensor(t));
        const b200_tensor *a = src(t, 0), *b = src(t, 1), *c = src(t, 2);
        KQ_REQUIRE(a, "graph_compute: node %.64s has no src0", t->name);
        KQ_TRY(check_tensor(a));
        if (b) KQ_TRY(check_tensor(b));
        if (c) KQ_TRY(check_tensor(c));
        if (!b200_dev_supports_op(t->op, a->type, b ? b->type : B200_TYPE_F32)) {
            kq_set_error("graph_compute: node %.64s: op %u with types %u/%u is not on the hot path", t->name,
                         t->op, a->type, b ? b->type : 0);
            return B200_ERR_UNSUPPORTED;
        }
        float *y = (float *)(uintptr_t)t->data;
        const void *pa = (const void *)(uintptr_t)a->data;
        const void *pb = b ? (const void *)(uintptr_t)b->data : nullptr;
        switch (t->op) {
        case B200_OP_MUL_MAT: {
            KQ_REQUIRE(b && a->ne[0] == b->ne[0], "MUL_MAT %.64s: K mismatch", t->name);
            const int64_t K = a->ne[0], N = a->ne[1], M = nrows(b);
            KQ_REQUIRE(t->ne[0] == N && nrows(t) == M && t->type == B200_TYPE_F32, "MUL_MAT %.64s: bad output shape", t->name);
            if (a->type == B200_TYPE_F32) {
                KQ_TRY(kq_f32_matmul((const float *)pa, (const float *)pb, M, N, K, y, s));
            } else {
                const size_t need = b200_mul_mat_scratch_bytes(M, K);
                KQ_TRY(ensure_scratch(be, need));
                KQ_TRY(b200_mul_mat(a->type, pa, (const float *)pb, M, N, K, y, be->scratch, be->scratch_bytes, s));
            }
            break;
        }
        case B200_OP_MUL_MAT_ID: {
            KQ_REQUIRE(b && c && c->type == B200_TYPE_I32, "MUL_MAT_ID %.64s: needs x and i32 ids", t->name);
            const int64_t K = a->ne[0], N = a->ne[1], E = a->ne[2];
            const int64_t n_used = c->ne[0], T = c->ne[1];
            KQ_REQUIRE(b->ne[0] == K && b->ne[2] == T && (b->ne[1] == n_used || b->ne[1] == 1),
                       "MUL_MAT_ID %.64s: x must be [K, n_used|1, T]", t->name);
            KQ_REQUIRE(t->ne[0] == N && t->ne[1] == n_used && t->ne[2] == T && t->type == B200_TYPE_F32,
                       "MUL_MAT_ID %.64s: bad output shape", t->name);
            KQ_REQUIRE(E >= 1 && E <= 256, "MUL_MAT_ID %.64s: at most 256 experts", t->name);
            const int64_t xrows = b->ne[1] * T, pairs = n_used * T;
            const size_t need = b200_mul_mat_id_scratch_bytes(xrows, pairs, K, E);
            KQ_TRY(ensure_scratch(be, need));
            // more than 8 pairs: gathered per expert and run through the tensor-core GEMM in one grouped launch
            KQ_TRY(b200_mul_mat_id(a->type, pa, E, (const float *)pb, xrows, (const int32_t *)(uintptr_t)c->data, pairs, N, K, y,
                                   be->scratch, be->scratch_bytes, s));
            break;
        }
        case B200_OP_RMS_NORM:
            KQ_TRY(out_holds(t, B200_TYPE_F32, nelements(a)));
            KQ_TRY(kq_rms_norm((const float *)pa, nullptr, nrows(a), a->ne[0], f32_param(t, 0), y, nullptr, nullptr,
                               nullptr, s));
            break;
        case B200_OP_MUL:
        case B200_OP_ADD: {
            KQ_REQUIRE(b && b->type == B200_TYPE_F32 && b->ne[0] == a->ne[0], "%.64s: operand shapes", t->name);
            const int64_t total = nelements(a), nbe = nelements(b);
            KQ_REQUIRE(nbe == total || nbe == a->ne[0], "%.64s: src1 must match or be one row", t->name);
            KQ_TRY(out_holds(t, B200_TYPE_F32, total));
            if (t->op == B200_OP_MUL)
                kq_launch(mul_rows_kernel, (unsigned)kq_div_up(total, 256), 256, 0, s, (const float *)pa, (const float *)pb,
                                                                               total, a->ne[0], nbe, y);
            else
                kq_launch(add_bcast_kernel, (unsigned)kq_div_up(total, 256), 256, 0, s, (const float *)pa, (const float *)pb,
                                                                                total, a->ne[0], nbe, y);
            KQ_COUNT_LAUNCH();
            KQ_LAUNCH_CHECK();
            break;
        }
        case B200_OP_ROPE: {
            KQ_REQUIRE(b && b->ne[0] == a->ne[2], "ROPE %.64s: one position per token", t->name);
            KQ_REQUIRE(t->op_params[0] == (int32_t)a->ne[0], "ROPE %.64s: partial rotation is not supported", t->name);
            KQ_TRY(out_holds(t, B200_TYPE_F32, nelements(a)));
            if (t->data != a->data)
                KQ_CUDA(cudaMemcpyAsync(y, pa, (size_t)nelements(a) * 4, cudaMemcpyDeviceToDevice, s));
            KQ_TRY(b200_rope(y, (const int32_t *)pb, a->ne[2], a->ne[1], a->ne[0], f32_param(t, 2),
                             t->op_params[1] == 2, s));
            break;
        }
        case B200_OP_SWIGLU:
            KQ_REQUIRE(b && b->type == B200_TYPE_F32 && nelements(b) == nelements(a), "SWIGLU %.64s: shapes", t->name);
            KQ_TRY(out_holds(t, B200_TYPE_F32, nelements(a)));
            KQ_TRY(b200_swiglu((const float *)pa, (const float *)pb, nelements(a), y, s));
            break;
        case B200_OP_GET_ROWS:
            KQ_REQUIRE(b, "GET_ROWS %.64s: ids", t->name);
            KQ_TRY(out_holds(t, B200_TYPE_F32, nelements(b) * (int64_t)a->ne[0]));
            KQ_TRY(b200_get_rows(a->type, pa, (const int32_t *)pb, nelements(b), a->ne[0], y, s));
            break;
        case B200_OP_CPY:
            if (t->type == B200_TYPE_F16 || t->type == B200_TYPE_F32) KQ_TRY(out_holds(t, t->type, nelements(a)));
            if (t->type == B200_TYPE_F16)
                KQ_TRY(b200_cpy_f32_f16((const float *)pa, nelements(a), (uint16_t *)y, s));
            else if (t->type == B200_TYPE_F32)
                KQ_CUDA(cudaMemcpyAsync(y, pa, (size_t)nelements(a) * 4, cudaMemcpyDeviceToDevice, s));
            else if (t->type == B200_TYPE_Q8_0 || t->type == B200_TYPE_Q4_0) { // a quantised KV cache being written
                KQ_REQUIRE(a->type == B200_TYPE_F32 && a->ne[0] % 32 == 0, "CPY %.64s: f32 rows of whole blocks", t->name);
                KQ_TRY(out_holds(t, t->type, nelements(a)));
                const int64_t n_blocks = nelements(a) / 32;
                if (n_blocks > 0) {
                    KQ_CUDA(kq_launch(cpy_f32_kvq_kernel, dim3((unsigned)kq_div_up(n_blocks, 8)), dim3(256), 0, s, (const float *)pa,
                                     n_blocks, (int)t->type, (uint8_t *)y));
                }
            } else {
                kq_set_error("CPY %.64s: destination type %u", t->name, t->type);
                return B200_ERR_UNSUPPORTED;
            }
            break;
        case B200_OP_ATTN: {
            KQ_REQUIRE(b && c && kq_kv_type_ok((int)b->type) && kq_kv_type_ok((int)c->type),
                       "ATTN %.64s: K and V caches of type f16, q8_0 or q4_0", t->name);
            const int hd = a->ne[0], n_head = a->ne[1], T = a->ne[2], n_kv = b->ne[1];
            const int pos0 = t->op_params[1];
            KQ_REQUIRE(b->ne[0] == a->ne[0] && c->ne[0] == a->ne[0] && c->ne[1] == b->ne[1] && c->ne[2] == b->ne[2],
                       "ATTN %.64s: K and V caches must be [head_dim, n_kv, n_ctx] with q's head_dim", t->name);
            KQ_REQUIRE(n_kv > 0 && n_head % n_kv == 0, "ATTN %.64s: %d query heads over %d KV heads", t->name, n_head, n_kv);
            KQ_TRY(out_holds(t, B200_TYPE_F32, nelements(a)));
            KQ_REQUIRE(pos0 >= 0 && (int64_t)pos0 + T <= (int64_t)b->ne[2], "ATTN %.64s: positions exceed the cache", t->name);
            KqKvTypes kvt;
            kvt.k = (int)b->type;
            kvt.v = (int)c->type;
            KQ_REQUIRE(!kvt.quantised() || hd == 128, "ATTN %.64s: quantised caches need head_dim 128", t->name);
            // A quantised cache arrives in ggml's block layout (34 / 18-byte blocks, 2-byte aligned).  The rows
            // in use are re-laid into the scratch in this library's 16-byte-aligned row layout -- a move of
            // bytes -- and attended to there; the cache tensor itself is only read.
            const int64_t rows = (int64_t)(pos0 + T) * n_kv;
            const size_t kq_bytes = kvt.k != KQ_KV_F16 ? (size_t)rows * kq_kv_row_bytes(kvt.k, hd) : 0;
            const size_t vq_bytes = kvt.v != KQ_KV_F16 ? (size_t)rows * kq_kv_row_bytes(kvt.v, hd) : 0;
            const size_t att = (b200_attention_scratch_bytes(std::min(T, 64), n_head, hd, b->ne[2]) + 255) & ~(size_t)255;
            KQ_TRY(ensure_scratch(be, att + kq_bytes + vq_bytes));
            const uint8_t *kp = (const uint8_t *)pb, *vp = (const uint8_t *)(uintptr_t)c->data;
            uint8_t *stage = (uint8_t *)be->scratch + att;
            if (kq_bytes) {
                KQ_CUDA(kq_launch(kvq_ggml_to_rows_kernel, dim3((unsigned)kq_div_up(rows * (hd / 32), 256)), dim3(256), 0, s, kp,
                                 rows, hd, kvt.k, stage));
                kp = stage;
            }
            if (vq_bytes) {
                KQ_CUDA(kq_launch(kvq_ggml_to_rows_kernel, dim3((unsigned)kq_div_up(rows * (hd / 32), 256)), dim3(256), 0, s, vp,
                                 rows, hd, kvt.v, stage + kq_bytes));
                vp = stage + kq_bytes;
            }
            KQ_TRY(kq_attention((const float *)pa, (const uint16_t *)kp, (const uint16_t *)vp, 1, T, nullptr, pos0, n_head, n_kv,
                                hd, 0, y, (float *)be->scratch, att, 0, kvt, s));
            break;
        }
        case B200_OP_MOE_ROUTE:
            KQ_REQUIRE(b && b->type == B200_TYPE_I32, "MOE_ROUTE %.64s: src1 receives the ids", t->name);
            KQ_REQUIRE(t->op_params[0] >= 1 && (uint32_t)t->op_params[0] <= a->ne[0], "MOE_ROUTE %.64s: k = %d of %u experts",
                       t->name, t->op_params[0], a->ne[0]);
            KQ_TRY(out_holds(t, B200_TYPE_F32, (int64_t)t->op_params[0] * nrows(a)));
            KQ_TRY(out_holds(b, B200_TYPE_I32, (int64_t)t->op_params[0] * nrows(a)));
            KQ_TRY(b200_moe_route((const float *)pa, a->ne[1], a->ne[0], t->op_params[0],
                                  (int32_t *)(uintptr_t)b->data, y, s));
            break;
        case B200_OP_ARGMAX:
            KQ_TRY(out_holds(t, B200_TYPE_I32, nrows(a)));
            KQ_TRY(b200_argmax((const float *)pa, nrows(a), a->ne[0], (int32_t *)y, s));
            break;
        default:
            kq_set_error("graph_compute: node %.64s: op %u is not on the hot path", t->name, t->op);
            return B200_ERR_UNSUPPORTED;
        }
    }
    cudaError_t e = cudaStreamSynchronize(s);
    if (e != cudaSuccess) {
        kq_set_error("graph_compute: %s", cudaGetErrorString(e));
        return B200_ERR_CUDA;
    }
    return B200_OK;
}

} // extern "C"
