// Shared declarations of the B200 K-quant stage library (sm_100a only).
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/b200_kquant.h"

#define KQ_QK 256
#define KQ_Q4K_BYTES 144
#define KQ_Q6K_BYTES 210

// ---- error plumbing -----------------------------------------------------------------------
void kq_set_error(const char *fmt, ...);

#define KQ_CUDA(call)                                                                          \
    do {                                                                                       \
        cudaError_t e__ = (call);                                                              \
        if (e__ != cudaSuccess) {                                                              \
            kq_set_error("%s:%d %s -> %s", __FILE__, __LINE__, #call, cudaGetErrorString(e__)); \
            return B200_ERR_CUDA;                                                              \
        }                                                                                      \
    } while (0)

#define KQ_REQUIRE(cond, ...)            \
    do {                                 \
        if (!(cond)) {                   \
            kq_set_error(__VA_ARGS__);   \
            return B200_ERR_INVALID;     \
        }                                \
    } while (0)

#define KQ_LAUNCH_CHECK()                                                                   \
    do {                                                                                    \
        cudaError_t e__ = cudaGetLastError();                                               \
        if (e__ != cudaSuccess) {                                                           \
            kq_set_error("%s:%d launch -> %s", __FILE__, __LINE__, cudaGetErrorString(e__)); \
            return B200_ERR_CUDA;                                                           \
        }                                                                                   \
    } while (0)

// every kernel launch of the library goes through this counter (reported by the bench)
extern long long g_kq_launches;
#define KQ_COUNT_LAUNCH() (++g_kq_launches)

static inline int64_t kq_div_up(int64_t a, int64_t b) { return (a + b - 1) / b; }

// Makes `dev` current for the lifetime of the object and gives the caller its own device back
// afterwards: an entry point must not leave the thread's current device changed.
struct KqDevGuard {
    int prev = -1;
    explicit KqDevGuard(int dev) {
        cudaGetDevice(&prev);
        if (prev != dev) cudaSetDevice(dev);
        else prev = -1;
    }
    ~KqDevGuard() {
        if (prev >= 0) cudaSetDevice(prev);
    }
    KqDevGuard(const KqDevGuard &) = delete;
    KqDevGuard &operator=(const KqDevGuard &) = delete;
};
int kq_sm_count();

// ---- device row geometry -------------------------------------------------------------------
static inline __host__ __device__ int64_t kq_row_bytes(uint32_t type, int64_t k) {
    switch (type) {
    case B200_TYPE_F32: return k * 4;
    case B200_TYPE_F16: return k * 2;
    case B200_TYPE_Q4_K: return k / KQ_QK * KQ_Q4K_BYTES;
    case B200_TYPE_Q6_K: return k / KQ_QK * KQ_Q6K_BYTES;
    case B200_TYPE_Q4_0: return k / 32 * 18; // ggml block_q4_0: f16 d, 16 bytes of nibbles
    case B200_TYPE_Q8_0: return k / 32 * 34; // ggml block_q8_0: f16 d, 32 int8
    default: return 0;
    }
}
// Q6_K rows live on the device as groups of up to 8 blocks, each group laid out as planes
// [ql g*128 | qh g*64 | scales g*16 | d g*2 (padded to 16)], g = blocks in the group.  Inside the
// ql and qh planes the 16-byte chunks are stored chunk-major: chunk k of block b sits at
// (k*g + b)*16, so the lanes that hold neighbouring blocks read neighbouring 16-byte words (no
// shared-memory bank conflicts, full sectors from global memory).  A full group is 1680 bytes (a
// multiple of 16 with no padding), so any 8-block slice of a row is one contiguous, 16-byte
// aligned run; only the last, partial group of a row carries padding (< 16 bytes).
#define KQ_Q6_GROUP 8
#define KQ_Q6_GROUP_BYTES 1680
static inline __host__ __device__ int64_t kq_q6_group_bytes(int g) {
    return g == KQ_Q6_GROUP ? KQ_Q6_GROUP_BYTES : (g ? (int64_t)g * 208 + 16 : 0);
}
static inline __host__ __device__ int64_t kq_device_row_bytes(uint32_t type, int64_t k) {
    if (type == B200_TYPE_Q6_K) {
        const int64_t nb = k / KQ_QK;
        return nb / KQ_Q6_GROUP * KQ_Q6_GROUP_BYTES + kq_q6_group_bytes((int)(nb % KQ_Q6_GROUP));
    }
    return kq_row_bytes(type, k);
}
// byte offsets, inside a device row of nb blocks, of the four pieces of block `blk`: ql / qh point
// at chunk 0 of the block, consecutive chunks are `cs` bytes apart
struct KqQ6Addr {
    int64_t ql, qh, sc, d;
    int cs;
};
static inline __host__ __device__ KqQ6Addr kq_q6_addr(int nb, int blk) {
    const int grp = blk / KQ_Q6_GROUP, b8 = blk % KQ_Q6_GROUP;
    const int left = nb - grp * KQ_Q6_GROUP;
    const int g = left < KQ_Q6_GROUP ? left : KQ_Q6_GROUP;
    const int64_t base = (int64_t)grp * KQ_Q6_GROUP_BYTES;
    KqQ6Addr a;
    a.cs = g * 16;
    a.ql = base + b8 * 16;
    a.qh = base + g * 128 + b8 * 16;
    a.sc = base + g * 192 + b8 * 16;
    a.d = base + g * 208 + b8 * 2;
    return a;
}

// ---- launches -------------------------------------------------------------------------------
// Every kernel of the library is launched with programmatic stream serialisation allowed: the
// next kernel of the stream may be scheduled while this one drains, and blocks in
// KQ_PDL_WAIT() until its predecessors have completed and their writes are visible.  A decode
// step is a chain of some 700 short kernels, so taking the launch latency off the critical path
// is worth about as much as a faster kernel.  Kernels may do work that does not depend on earlier
// kernels (prefetching weights) before KQ_PDL_WAIT(); they must not read activations or write
// anything before it.  For the same reason no kernel parameter that points at data another kernel of
// the stream produces is declared `const T *__restrict__`: the compiler may treat loads through such
// a pointer as invariant and move them above the wait (a load placed right behind the wait was seen
// to return the predecessor's stale value).
extern int g_kq_pdl;
#ifdef __CUDACC__
#define KQ_PDL_TRIGGER() asm volatile("griddepcontrol.launch_dependents;" ::: "memory")
#define KQ_PDL_WAIT() asm volatile("griddepcontrol.wait;" ::: "memory")
#define KQ_PDL_ENTER() \
    do {               \
        KQ_PDL_TRIGGER(); \
        KQ_PDL_WAIT();    \
    } while (0)

template <typename... KArgs, typename... Args>
static inline cudaError_t kq_launch(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                                    Args &&...args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = g_kq_pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, KArgs(args)...);
}
#endif

// ---- device helpers ------------------------------------------------------------------------
#ifdef __CUDACC__
__device__ __forceinline__ float kq_warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float kq_warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float kq_h2f(uint16_t h) { return __half2float(__ushort_as_half(h)); }

// 16-byte streaming load of weight bytes: read once, keep out of L1
__device__ __forceinline__ uint4 kq_ld_stream(const void *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

// ---- bounded waits ------------------------------------------------------------------------------
// Every device-side wait of the library is bounded in wall-clock time (not in iterations:
// mbarrier.try_wait may itself suspend the thread for a system-dependent while), after which the
// caller records an error and carries on to its exit path.
__device__ __forceinline__ uint64_t kq_globaltimer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ bool kq_mbar_try(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok)
                 : "r"(bar), "r"(parity)
                 : "memory");
    return ok != 0;
}
// true when the phase completed, false after limit_ns without completion
__device__ __forceinline__ bool kq_mbar_wait(uint32_t bar, uint32_t parity, uint64_t limit_ns) {
    if (kq_mbar_try(bar, parity)) return true;
    const uint64_t t0 = kq_globaltimer_ns();
    while (!kq_mbar_try(bar, parity))
        if (kq_globaltimer_ns() - t0 > limit_ns) return false;
    return true;
}
#define KQ_WAIT_LIMIT_NS 20000000ull /* 20 ms: four orders of magnitude above any healthy wait */

// The activation quantiser of the library (same arithmetic as the CPU oracle, operation for
// operation, so the int8 codes are bit-identical): d = amax / 127, id = 1 / d, q = rint(x * id).
__device__ __forceinline__ float kq_act_scale(float amax) { return __fdiv_rn(amax, 127.0f); }
__device__ __forceinline__ float kq_act_inv(float d) { return d > 0.f ? __fdiv_rn(1.0f, d) : 0.f; }
__device__ __forceinline__ int kq_act_code(float x, float id) {
    int v = __float2int_rn(__fmul_rn(x, id));
    return max(-127, min(127, v));
}

// The quantiser applied to one block by one warp (b200_quantize_act and every fused form of it).
// One warp per 256-element block.  Lane l owns elements 8l .. 8l+7 (values in v[8]).
__device__ __forceinline__ void kq_quantize_block_warp(const float (&v)[8], int lane, int8_t *qb,
                                                    float *d_out, int16_t *bs_out) {
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 8; i++) amax = fmaxf(amax, fabsf(v[i]));
    amax = kq_warp_max(amax);
    const float d = kq_act_scale(amax), id = kq_act_inv(d);
    int c[8], s = 0;
#pragma unroll
    for (int i = 0; i < 8; i++) {
        c[i] = kq_act_code(v[i], id);
        s += c[i];
    }
    uint2 pk;
    pk.x = (uint32_t)(c[0] & 0xFF) | ((uint32_t)(c[1] & 0xFF) << 8) | ((uint32_t)(c[2] & 0xFF) << 16) |
           ((uint32_t)(c[3] & 0xFF) << 24);
    pk.y = (uint32_t)(c[4] & 0xFF) | ((uint32_t)(c[5] & 0xFF) << 8) | ((uint32_t)(c[6] & 0xFF) << 16) |
           ((uint32_t)(c[7] & 0xFF) << 24);
    *reinterpret_cast<uint2 *>(qb + lane * 8) = pk;
    s += __shfl_xor_sync(0xffffffffu, s, 1);
    if ((lane & 1) == 0) bs_out[lane >> 1] = (int16_t)s;
    if (lane == 0) *d_out = d;
}
#endif

// ---- internal launchers shared between translation units -----------------------------------
struct KqGemvSeg {
    const uint8_t *W; // device layout rows
    uint32_t type;
    int32_t n_rows;
    float *y;          // [M][ldy], rows of this segment start at column 0 of y
    const float *bias; // [n_rows] or null
    int32_t ldy;
    int64_t expert_stride; // bytes between consecutive expert matrices (expert-indexed mode)
};

struct KqGemvIndirect {
    const int32_t *expert_ids; // device, one expert id per (token, slot) pair
    int32_t n_pairs;
    int32_t act_div;           // activation row of pair p is p / act_div
};

// f32 activations to be prepared by the GEMV itself: optional RMSNorm (weight may be null = 1),
// then the Q8 quantiser.  q / d / bs passed alongside are scratch for the case that the plain
// kernel has to be used.
struct KqActPrep {
    const float *x;      // [M][K]
    const float *norm_w; // [K] or null
    float eps;
    int32_t do_norm;
};

// The Q8 form of a fused gate / up launch's output (SwiGLU values), written by that launch itself for the
// matmul that follows: whichever warp completes the last row of a 256-element block quantises the block.
// counters: one zero-initialised int per block, returned to zero by the launch.  done is set by the
// launcher when the launch will write q / d / bs (rows a multiple of 256, streaming kernel, 1 or 2 tokens).
struct KqEmitQ8 {
    int8_t *q;
    float *d;
    int16_t *bs;
    int32_t *counters;
    int32_t done;
};

// one phase of a fused chain of decode matmuls: y = W . prep(x) (+ residual / SwiGLU of a gate-up pair)
struct KqFusedPhase {
    KqGemvSeg segs[2];
    int32_t nseg;
    int64_t K;
    const float *residual;
    int32_t swiglu;
    KqActPrep prep;
};
b200_status kq_launch_gemv_fused(const KqFusedPhase *ph, int n_phase, int M, cudaStream_t st);

b200_status kq_launch_gemv(const KqGemvSeg *segs, int nseg, const int8_t *q, const float *d,
                           const int16_t *bs, int M, int64_t K, const float *residual,
                           int swiglu_pairs, const KqGemvIndirect *ind, cudaStream_t st,
                           const KqActPrep *prep = nullptr, KqEmitQ8 *emit = nullptr);
b200_status kq_launch_gemv_stream(const KqGemvSeg *segs, int nseg, const int8_t *q, const float *d,
                                  const int16_t *bs, int M, int64_t K, const float *residual, int swiglu_pairs,
                                  const KqActPrep *prep, cudaStream_t st, KqEmitQ8 *emit = nullptr);
b200_status kq_rms_norm(const float *x, const float *w, int64_t T, int64_t h, float eps, float *y, int8_t *q,
                        float *d, int16_t *bs, cudaStream_t st, int64_t x_row_stride);
// MUL_MAT_ID over many tokens: stable expert-major order of the (token, slot) pairs, then one grouped
// launch of the tensor-core GEMM per expert-packed matrix (y[pair][N] = W[expert(pair)] . x[pair / act_div])
size_t kq_moe_sort_scratch_bytes(int64_t n_pairs, int64_t E);
b200_status kq_moe_sort(const int32_t *ids, int64_t n_pairs, int64_t E, int32_t *scratch, size_t scratch_bytes, cudaStream_t st);
b200_status kq_launch_gemm_grouped(uint32_t type, const uint8_t *W, int64_t expert_stride, const int8_t *q, const float *d,
                                   const int16_t *bs, int act_div, int64_t n_pairs, int64_t E, int64_t N, int64_t K, float *y,
                                   const int32_t *sorted, cudaStream_t st);
int kq_stream_error_fetch(); // 0 ok; nonzero = a bounded device-side wait gave up since the last call
int kq_gemm_error_fetch();
int kq_attn_tc_error_fetch();
b200_status kq_launch_gemm(uint32_t type, const uint8_t *W, const int8_t *q, const float *d,
                           const int16_t *bs, int64_t M, int64_t N, int64_t K, float *y,
                           const float *bias, const float *residual, cudaStream_t st);
