// Prefill contraction (M > 8 tokens): dispatch between the tensor-core kernel and, as a fall-back
// that can be forced with B200_GEMM_TC=0, a walk over the token batch in slabs of 8 through the
// decode kernel (identical results token for token, but weight-stream bound).
#include "kq_common.cuh"

#include <stdlib.h>

b200_status kq_launch_gemm_tc(uint32_t type, const uint8_t *W, const int8_t *q, const float *d, const int16_t *bs,
                              int64_t M, int64_t N, int64_t K, float *y, const float *bias, const float *residual,
                              cudaStream_t st);

b200_status kq_launch_gemm(uint32_t type, const uint8_t *W, const int8_t *q, const float *d,
                           const int16_t *bs, int64_t M, int64_t N, int64_t K, float *y,
                           const float *bias, const float *residual, cudaStream_t st) {
    static int use_tc = -1;
    if (use_tc < 0) {
        const char *v = getenv("B200_GEMM_TC");
        use_tc = !(v && v[0] == '0');
    }
    if (use_tc) return kq_launch_gemm_tc(type, W, q, d, bs, M, N, K, y, bias, residual, st);
    const int64_t nb = K / 256;
    for (int64_t m0 = 0; m0 < M; m0 += 8) {
        const int mc = (int)(M - m0 < 8 ? M - m0 : 8);
        KqGemvSeg sg = {W, type, (int32_t)N, y + m0 * N, bias, (int32_t)N, 0};
        b200_status rc = kq_launch_gemv(&sg, 1, q + m0 * K, d + m0 * nb, bs + m0 * nb * 16, mc, K,
                                        residual ? residual + m0 * N : nullptr, 0, nullptr, st);
        if (rc != B200_OK) return rc;
    }
    return B200_OK;
}
