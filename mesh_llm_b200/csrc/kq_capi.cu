// C ABI plumbing: error strings, registry / device queries, and the MUL_MAT entry points that pick
// between the decode GEMV (M <= 8) and the prefill GEMM.
#include "kq_common.cuh"

#include <stdarg.h>
#include <stdlib.h>
#include <string.h>

long long g_kq_launches = 0;

static int pdl_default() {
    const char *v = getenv("B200_NO_PDL");
    return !(v && v[0] == '1');
}
int g_kq_pdl = pdl_default();

static thread_local char t_err[512] = "";

void kq_set_error(const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(t_err, sizeof(t_err), fmt, ap);
    va_end(ap);
}

int kq_sm_count() {
    static int n[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (!n[dev]) {
        cudaDeviceProp p;
        n[dev] = (cudaGetDeviceProperties(&p, dev) == cudaSuccess) ? p.multiProcessorCount : 148;
    }
    return n[dev];
}

extern "C" {

const char *b200_last_error(void) { return t_err; }

const char *b200_status_string(b200_status s) {
    switch (s) {
    case B200_OK: return "ok";
    case B200_ERR_INVALID: return "invalid argument";
    case B200_ERR_ALLOC: return "allocation failed";
    case B200_ERR_CUDA: return "CUDA error";
    case B200_ERR_UNSUPPORTED: return "unsupported";
    case B200_ERR_BOUNDS: return "out of bounds";
    case B200_ERR_TIMEOUT: return "device wait timed out";
    case B200_ERR_STATE: return "invalid state";
    default: return "unknown status";
    }
}

b200_status b200_check_device_waits(void) {
    KQ_CUDA(cudaDeviceSynchronize());
    const int werr = kq_stream_error_fetch() | (kq_gemm_error_fetch() << 4) | (kq_attn_tc_error_fetch() << 8);
    if (werr) {
        kq_set_error("a bounded device-side wait gave up (code 0x%x)", werr);
        return B200_ERR_TIMEOUT;
    }
    return B200_OK;
}

const char *b200_reg_name(void) { return "B200"; }

int32_t b200_reg_device_count(void) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return n;
}

b200_status b200_dev_name(int32_t dev, char *out, size_t cap) {
    KQ_REQUIRE(out && cap > 0 && dev >= 0, "dev_name: bad arguments");
    snprintf(out, cap, "B200_%d", dev);
    return B200_OK;
}

b200_status b200_dev_description(int32_t dev, char *out, size_t cap) {
    KQ_REQUIRE(out && cap > 0, "dev_description: bad arguments");
    cudaDeviceProp p;
    KQ_CUDA(cudaGetDeviceProperties(&p, dev));
    snprintf(out, cap, "%s (sm_%d%d, %d SMs)", p.name, p.major, p.minor, p.multiProcessorCount);
    return B200_OK;
}

b200_status b200_dev_memory(int32_t dev, size_t *free_bytes, size_t *total_bytes) {
    int cur = 0;
    KQ_CUDA(cudaGetDevice(&cur));
    KQ_CUDA(cudaSetDevice(dev));
    size_t f = 0, t = 0;
    cudaError_t e = cudaMemGetInfo(&f, &t);
    cudaSetDevice(cur);
    KQ_CUDA(e);
    if (free_bytes) *free_bytes = f;
    if (total_bytes) *total_bytes = t;
    return B200_OK;
}

int32_t b200_dev_supports_op(uint32_t op, uint32_t t0, uint32_t t1) {
    const bool kq = t0 == B200_TYPE_Q4_K || t0 == B200_TYPE_Q6_K;
    switch (op) {
    case B200_OP_MUL_MAT: return (kq || t0 == B200_TYPE_F32) && t1 == B200_TYPE_F32;
    case B200_OP_MUL_MAT_ID: return kq && t1 == B200_TYPE_F32;
    case B200_OP_GET_ROWS: return (kq || t0 == B200_TYPE_F32) && t1 == B200_TYPE_I32;
    case B200_OP_RMS_NORM:
    case B200_OP_MUL:
    case B200_OP_ADD:
    case B200_OP_SWIGLU:
    case B200_OP_MOE_ROUTE:
    case B200_OP_ARGMAX: return t0 == B200_TYPE_F32;
    case B200_OP_ROPE: return t0 == B200_TYPE_F32 && t1 == B200_TYPE_I32;
    case B200_OP_CPY: return t0 == B200_TYPE_F32;
    case B200_OP_ATTN: // K cache (src1; V may differ): f16, or ggml's q8_0 / q4_0 blocks
        return t0 == B200_TYPE_F32 && (t1 == B200_TYPE_F16 || t1 == B200_TYPE_Q8_0 || t1 == B200_TYPE_Q4_0);
    default: return 0;
    }
}

size_t b200_buft_alignment(void) { return 256; }

size_t b200_buft_max_size(int32_t dev) {
    size_t f = 0, t = 0;
    if (b200_dev_memory(dev, &f, &t) != B200_OK) return 0;
    return t;
}

size_t b200_row_bytes(uint32_t type, int64_t k) { return (size_t)kq_row_bytes(type, k); }
size_t b200_device_row_bytes(uint32_t type, int64_t k) { return (size_t)kq_device_row_bytes(type, k); }

size_t b200_buft_alloc_size(uint32_t type, const uint32_t ne[4]) {
    const size_t rows = (size_t)ne[1] * ne[2] * ne[3];
    size_t rb = (type == B200_TYPE_I32) ? (size_t)ne[0] * 4 : (size_t)kq_device_row_bytes(type, ne[0]);
    return (rows * rb + 255) / 256 * 256;
}

size_t b200_mul_mat_scratch_bytes(int64_t M, int64_t K) {
    // q (M*K) + d (M*K/256 f32) + bsum16 (M*K/16 i16), each part 256-byte aligned
    auto up = [](size_t v) { return (v + 255) / 256 * 256; };
    return up((size_t)(M * K)) + up((size_t)(M * K / 256 * 4)) + up((size_t)(M * K / 16 * 2));
}

b200_status b200_mul_mat_q8(uint32_t type, const void *W, const int8_t *q, const float *d,
                            const int16_t *bsum16, int64_t M, int64_t N, int64_t K, float *y,
                            const float *bias, const float *residual, void *stream) {
    KQ_REQUIRE(M > 0 && N > 0 && K > 0 && K % 256 == 0, "mul_mat: bad shape M=%lld N=%lld K=%lld",
               (long long)M, (long long)N, (long long)K);
    KQ_REQUIRE(type == B200_TYPE_Q4_K || type == B200_TYPE_Q6_K, "mul_mat: weight type %u", type);
    cudaStream_t st = (cudaStream_t)stream;
    if (M <= 8) {
        KqGemvSeg sg = {(const uint8_t *)W, type, (int32_t)N, y, bias, (int32_t)N, 0};
        return kq_launch_gemv(&sg, 1, q, d, bsum16, (int)M, K, residual, 0, nullptr, st);
    }
    return kq_launch_gemm(type, (const uint8_t *)W, q, d, bsum16, M, N, K, y, bias, residual, st);
}

b200_status b200_mul_mat(uint32_t type, const void *W, const float *x, int64_t M, int64_t N, int64_t K,
                         float *y, void *scratch, size_t scratch_bytes, void *stream) {
    KQ_REQUIRE(M > 0 && K > 0 && K % 256 == 0, "mul_mat: bad shape");
    KQ_REQUIRE(scratch && scratch_bytes >= b200_mul_mat_scratch_bytes(M, K),
               "mul_mat: scratch too small (%zu < %zu)", scratch_bytes, b200_mul_mat_scratch_bytes(M, K));
    KQ_REQUIRE(((uintptr_t)scratch & 255) == 0, "mul_mat: scratch must be 256-byte aligned");
    auto up = [](size_t v) { return (v + 255) / 256 * 256; };
    int8_t *q = (int8_t *)scratch;
    float *d = (float *)((char *)scratch + up((size_t)(M * K)));
    int16_t *bs = (int16_t *)((char *)d + up((size_t)(M * K / 256 * 4)));
    b200_status rc = b200_quantize_act(x, M, K, q, d, bs, stream);
    if (rc != B200_OK) return rc;
    return b200_mul_mat_q8(type, W, q, d, bs, M, N, K, y, nullptr, nullptr, stream);
}

size_t b200_mul_mat_id_scratch_bytes(int64_t n_x_rows, int64_t n_pairs, int64_t K, int64_t E) {
    return b200_mul_mat_scratch_bytes(n_x_rows, K) + ((kq_moe_sort_scratch_bytes(n_pairs, E) + 255) / 256) * 256;
}

b200_status b200_mul_mat_id(uint32_t type, const void *W, int64_t E, const float *x, int64_t n_x_rows, const int32_t *ids,
                            int64_t n_pairs, int64_t N, int64_t K, float *y, void *scratch, size_t scratch_bytes,
                            void *stream) {
    KQ_REQUIRE(type == B200_TYPE_Q4_K || type == B200_TYPE_Q6_K, "mul_mat_id: weight type %u", type);
    KQ_REQUIRE(W && x && ids && y && scratch, "mul_mat_id: null pointer");
    KQ_REQUIRE(E >= 1 && E <= 256 && N >= 1 && K >= 256 && K % 256 == 0, "mul_mat_id: bad shape E=%lld N=%lld K=%lld",
               (long long)E, (long long)N, (long long)K);
    KQ_REQUIRE(n_x_rows >= 1 && n_pairs >= n_x_rows && n_pairs % n_x_rows == 0,
               "mul_mat_id: %lld pairs over %lld activation rows", (long long)n_pairs, (long long)n_x_rows);
    KQ_REQUIRE(((uintptr_t)scratch & 255) == 0 && scratch_bytes >= b200_mul_mat_id_scratch_bytes(n_x_rows, n_pairs, K, E),
               "mul_mat_id: scratch must be 256-byte aligned and hold %zu bytes", b200_mul_mat_id_scratch_bytes(n_x_rows, n_pairs, K, E));
    cudaStream_t st = (cudaStream_t)stream;
    auto up = [](size_t v) { return (v + 255) / 256 * 256; };
    int8_t *q = (int8_t *)scratch;
    float *d = (float *)((char *)scratch + up((size_t)(n_x_rows * K)));
    int16_t *bs = (int16_t *)((char *)d + up((size_t)(n_x_rows * K / 256 * 4)));
    int32_t *sorted = (int32_t *)((char *)scratch + b200_mul_mat_scratch_bytes(n_x_rows, K));
    b200_status rc = b200_quantize_act(x, n_x_rows, K, q, d, bs, stream);
    if (rc != B200_OK) return rc;
    const int act_div = (int)(n_pairs / n_x_rows);
    const int64_t estride = kq_device_row_bytes(type, K) * N;
    if (n_pairs > 8) { // many pairs: gathered per expert, one grouped launch of the tensor-core kernel
        rc = kq_moe_sort(ids, n_pairs, E, sorted, kq_moe_sort_scratch_bytes(n_pairs, E), st);
        if (rc != B200_OK) return rc;
        rc = kq_launch_gemm_grouped(type, (const uint8_t *)W, estride, q, d, bs, act_div, n_pairs, E, N, K, y, sorted, st);
        if (rc != B200_ERR_UNSUPPORTED) return rc;
    }
    KqGemvSeg sg = {(const uint8_t *)W, type, (int32_t)N, y, nullptr, (int32_t)N, estride};
    KqGemvIndirect ind = {ids, (int32_t)n_pairs, (int32_t)act_div};
    return kq_launch_gemv(&sg, 1, q, d, bs, 1, K, nullptr, 0, &ind, st);
}

} // extern "C"
