// Measured ceiling of the tensor core for the prefill GEMM's instruction: a bare loop of
// tcgen05.mma.cta_group::1.kind::i8 (M = 128, N = 256, K = 32, operands resting in shared memory,
// accumulators in TMEM), one CTA per SM, no loads, no epilogue.  The prefill GEMM's useful rate is
// reported against the figure this returns (two of its MMAs make one useful product, so its own
// ceiling is half of it).  A measurement aid: it has no counterpart in the reference.
#include "kq_common.cuh"

#include <cuda_runtime.h>

namespace {

constexpr int PM = 128, PN = 256, PK = 32;
constexpr int KCH = 8;                          // 16-byte K chunks staged per operand (K = 128 bytes in all)
constexpr int A_BYTES = PM * 16 * KCH, B_BYTES = PN * 16 * KCH;
constexpr uint32_t TMEM_COLS = 512;             // two accumulators of 256 columns, used alternately

__device__ int g_peak_error;

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

// canonical K-major layout without swizzle: 16-byte chunk kc of row r at kc * rows * 16 + (r / 8) * 128 + (r % 8) * 16
__device__ __forceinline__ uint64_t make_desc(uint32_t saddr, uint32_t lbo) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFF) >> 4);
    d |= (uint64_t)(lbo >> 4) << 16;
    d |= (uint64_t)(128 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    return d;
}

__global__ void __launch_bounds__(128, 1) int8_mma_loop_kernel(int n_mma, int *sink) {
    extern __shared__ __align__(1024) uint8_t sm[];
    __shared__ uint64_t done;
    __shared__ uint32_t s_tmem;
    const int tid = threadIdx.x, warp = tid >> 5;
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem)), "r"(TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    if (tid == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(&done)), "r"(1));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    // operand bytes: a fixed pseudo-random pattern (the data path toggles as it does on real codes)
    for (int i = tid; i < (A_BYTES + B_BYTES) / 4; i += blockDim.x) {
        uint32_t v = (uint32_t)i * 2654435761u + blockIdx.x * 40503u;
        v ^= v >> 15;
        v *= 2246822519u;
        v ^= v >> 13;
        reinterpret_cast<uint32_t *>(sm)[i] = v;
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = s_tmem;
    if (tid == 0) {
        // D s32, A s8, B s8, both K-major
        const uint32_t idesc = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(PN >> 3) << 17) | ((uint32_t)(PM >> 4) << 24);
        const uint32_t a = smem_u32(sm), b = smem_u32(sm + A_BYTES);
        for (int i = 0; i < n_mma; i++) {
            const int kc = 2 * (i & 3); // K = 32: chunks kc, kc + 1
            const uint32_t acc = (i & 4) ? 1u : 0u;
            asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                         "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
                         :
                         : "r"(tmem + acc * 256u), "l"(make_desc(a + kc * PM * 16, PM * 16)), "l"(make_desc(b + kc * PN * 16, PN * 16)),
                           "r"(idesc), "r"(i >= 8 ? 1u : 0u)
                         : "memory");
        }
        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(&done)) : "memory");
        if (!kq_mbar_wait(smem_u32(&done), 0u, 2000000000ull)) atomicExch(&g_peak_error, 1);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    }
    __syncthreads();
    if (warp == 0) { // read one accumulator word so that the products cannot be dropped
        uint32_t v;
        asm volatile("tcgen05.ld.sync.aligned.32x32b.x1.b32 {%0}, [%1];" : "=r"(v) : "r"(tmem) : "memory");
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (v == 0x7fffffffu && sink) *sink = (int)v;
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
}

} // namespace

extern "C" __attribute__((visibility("default"))) b200_status b200_probe_int8_mma(int32_t n_mma, int32_t repeats, double *tops_out,
                                                                                  double *ms_out) {
    KQ_REQUIRE(n_mma >= 16 && n_mma <= (1 << 22) && repeats >= 1 && repeats <= 1000 && tops_out,
               "b200_probe_int8_mma: n_mma in 16 .. 2^22, repeats in 1 .. 1000");
    int dev = 0, sms = 0;
    KQ_CUDA(cudaGetDevice(&dev));
    KQ_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    const int smem = A_BYTES + B_BYTES;
    KQ_CUDA(cudaFuncSetAttribute(int8_mma_loop_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    cudaEvent_t e0, e1;
    KQ_CUDA(cudaEventCreate(&e0));
    KQ_CUDA(cudaEventCreate(&e1));
    int8_mma_loop_kernel<<<sms, 128, smem>>>(n_mma, nullptr); // warm-up
    float best = 1e30f;
    for (int r = 0; r < repeats; r++) {
        cudaEventRecord(e0);
        int8_mma_loop_kernel<<<sms, 128, smem>>>(n_mma, nullptr);
        cudaEventRecord(e1);
        cudaError_t e = cudaEventSynchronize(e1);
        if (e != cudaSuccess) {
            cudaEventDestroy(e0);
            cudaEventDestroy(e1);
            kq_set_error("b200_probe_int8_mma: %s", cudaGetErrorString(e));
            return B200_ERR_CUDA;
        }
        float ms = 0.f;
        cudaEventElapsedTime(&ms, e0, e1);
        best = ms < best ? ms : best;
    }
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    int err = 0;
    KQ_CUDA(cudaMemcpyFromSymbol(&err, g_peak_error, sizeof(err)));
    if (err) {
        const int z = 0;
        cudaMemcpyToSymbol(g_peak_error, &z, sizeof(z));
        kq_set_error("b200_probe_int8_mma: the tensor core's commit did not arrive");
        return B200_ERR_TIMEOUT;
    }
    const double ops = 2.0 * PM * PN * PK * (double)n_mma * sms;
    *tops_out = ops / (best * 1e-3) / 1e12;
    if (ms_out) *ms_out = best;
    return B200_OK;
}
