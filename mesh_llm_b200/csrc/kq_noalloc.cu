// b200_mul_mat_static: the decode MUL_MAT (f32 activations in, quantised weights, f32 out) for
// callers that must not allocate.
//
// Who that is: a serving stage whose device memory was budgeted to the byte before it started --
// the orchestrator sized weights, KV cache and context from the VRAM it granted the process, and
// a scratch allocation made later, at request time, can fail outright or eat into a neighbour's
// share of the same GPU; a decode loop in which cudaMalloc's implicit device-wide synchronisation
// would stall every stream; or a host program that owns all device memory through its own
// allocator and forbids libraries to take more.  For them the Q8 scratch that b200_mul_mat asks
// its caller to provide lives here instead, in a fixed array inside the library image.
//
// The array is held by every GPU that loads the library, from load until the process exits.
#include "kq_common.cuh"

#include <mutex>

#define KQ_STATIC_MAX_TOKENS 8
#define KQ_STATIC_MAX_K 32768

namespace {

constexpr size_t up256(size_t v) { return (v + 255) / 256 * 256; }
constexpr size_t STATIC_Q_BYTES = up256((size_t)KQ_STATIC_MAX_TOKENS * KQ_STATIC_MAX_K);
constexpr size_t STATIC_D_BYTES = up256((size_t)KQ_STATIC_MAX_TOKENS * KQ_STATIC_MAX_K / 256 * 4);
constexpr size_t STATIC_BS_BYTES = up256((size_t)KQ_STATIC_MAX_TOKENS * KQ_STATIC_MAX_K / 16 * 2);
constexpr size_t STATIC_BYTES = STATIC_Q_BYTES + STATIC_D_BYTES + STATIC_BS_BYTES; // 299,008 bytes

// Quantised activations of the call in flight: int8 codes, then per-block scales, then the sums of
// 16.  In host code this name is only a handle for the runtime, never a device address.
static __device__ __align__(256) unsigned char g_static_scratch[STATIC_BYTES];

std::mutex g_mu;
unsigned char *g_scratch_addr[64] = {nullptr}; // device address of the array, per device ordinal

// One-time set-up for the current device: ask the runtime where this device's copy of the array
// lives.  Nothing is allocated; the array came with the module.
b200_status static_scratch(unsigned char **out) {
    int dev = -1;
    KQ_CUDA(cudaGetDevice(&dev));
    KQ_REQUIRE(dev >= 0 && dev < 64, "mul_mat_static: device ordinal %d out of range", dev);
    std::lock_guard<std::mutex> lock(g_mu);
    if (!g_scratch_addr[dev]) {
        void *p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);
        if (e != cudaSuccess || !p) {
            cudaGetLastError();
            kq_set_error("mul_mat_static: cudaGetSymbolAddress failed on device %d: %s", dev,
                         cudaGetErrorString(e));
            return B200_ERR_CUDA;
        }
        g_scratch_addr[dev] = (unsigned char *)p;
    }
    *out = g_scratch_addr[dev];
    return B200_OK;
}

} // namespace

extern "C" b200_status b200_mul_mat_static(uint32_t type, const void *W, const float *x, int64_t M,
                                           int64_t N, int64_t K, float *y, void *stream) {
    KQ_REQUIRE(type == B200_TYPE_Q4_K || type == B200_TYPE_Q6_K, "mul_mat_static: weight type %u", type);
    KQ_REQUIRE(W && x && y, "mul_mat_static: null pointer");
    KQ_REQUIRE(M >= 1 && N >= 1 && K >= 256 && K % 256 == 0, "mul_mat_static: bad shape M=%lld N=%lld K=%lld",
               (long long)M, (long long)N, (long long)K);
    if (M > KQ_STATIC_MAX_TOKENS || K > KQ_STATIC_MAX_K) {
        kq_set_error("mul_mat_static: M=%lld, K=%lld exceed the built-in scratch (at most %d tokens of at most "
                     "%d elements); use b200_mul_mat with caller-provided scratch for larger calls",
                     (long long)M, (long long)K, KQ_STATIC_MAX_TOKENS, KQ_STATIC_MAX_K);
        return B200_ERR_INVALID;
    }
    unsigned char *base = nullptr;
    b200_status rc = static_scratch(&base);
    if (rc != B200_OK) return rc;
    // Every byte the GEMV reads (M*K codes, M*K/256 scales, M*K/16 sums) is rewritten by the
    // quantiser below before it is read, so nothing left over from the previous call is used and
    // nothing needs to start at zero.
    int8_t *q = (int8_t *)base;
    float *d = (float *)(base + STATIC_Q_BYTES);
    int16_t *bs = (int16_t *)(base + STATIC_Q_BYTES + STATIC_D_BYTES);
    rc = b200_quantize_act(x, M, K, q, d, bs, stream);
    if (rc != B200_OK) return rc;
    return b200_mul_mat_q8(type, W, q, d, bs, M, N, K, y, nullptr, nullptr, stream);
}
