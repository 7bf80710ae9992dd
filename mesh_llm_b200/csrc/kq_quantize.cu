// Activation quantiser (f32 -> Q8 blocks of 256), its fused forms (RMSNorm -> Q8), the Q6_K
// device repack, and the on-device generator of synthetic Q4_K_M weights.
#include "kq_common.cuh"

namespace {

__global__ void __launch_bounds__(128) quantize_act_kernel(const float *x, int64_t nblocks,
                                                           int8_t *q, float *d, int16_t *bs) {
    KQ_PDL_ENTER();
    const int lane = threadIdx.x & 31;
    const int64_t blk = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
    if (blk >= nblocks) return;
    const float4 *xp = reinterpret_cast<const float4 *>(x + blk * 256 + lane * 8);
    const float4 a = xp[0], b = xp[1];
    const float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    kq_quantize_block_warp(v, lane, q + blk * 256, d + blk, bs + blk * 16);
}

// SwiGLU and the Q8 quantiser of its result in one pass (the input of the down projection in a prefill): one warp
// per 256-element block, lane l on elements 8l .. 8l+7; y (f32, may alias g) is written when it is not null.
// Same expression and same quantiser as the separate kernels, so codes and values are theirs.
__global__ void __launch_bounds__(128) swiglu_quantize_kernel(const float *g, const float *u, int64_t nblocks, float *y, int8_t *q,
                                                              float *d, int16_t *bs) {
    KQ_PDL_ENTER();
    const int lane = threadIdx.x & 31;
    const int64_t blk = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
    if (blk >= nblocks) return;
    const int64_t o = blk * 256 + lane * 8;
    const float4 g0 = *reinterpret_cast<const float4 *>(g + o), g1 = *reinterpret_cast<const float4 *>(g + o + 4);
    const float4 u0 = *reinterpret_cast<const float4 *>(u + o), u1 = *reinterpret_cast<const float4 *>(u + o + 4);
    const float a[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w}, b[8] = {u0.x, u0.y, u0.z, u0.w, u1.x, u1.y, u1.z, u1.w};
    float v[8];
#pragma unroll
    for (int i = 0; i < 8; i++) v[i] = (a[i] / (1.0f + expf(-a[i]))) * b[i];
    if (y) {
        *reinterpret_cast<float4 *>(y + o) = make_float4(v[0], v[1], v[2], v[3]);
        *reinterpret_cast<float4 *>(y + o + 4) = make_float4(v[4], v[5], v[6], v[7]);
    }
    kq_quantize_block_warp(v, lane, q + blk * 256, d + blk, bs + blk * 16);
}

// RMSNorm (x * rsqrt(mean(x^2) + eps) * w) with optional f32 output and optional Q8 output.
// One CTA of 256 threads per row; h is a multiple of 256 when q != null.
__global__ void __launch_bounds__(256) rms_norm_kernel(const float *x,
                                                       const float *w, int h, float eps,
                                                       float *y, int8_t *q, float *d, int16_t *bs,
                                                       int64_t x_row_stride) {
    KQ_PDL_ENTER();
    __shared__ double part[8];
    __shared__ float s_scale;
    const int row = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float *xr = x + (int64_t)row * x_row_stride;
    // the sum of squares is carried in double so that the scale does not depend on the order of
    // the reduction: the normalised values, and with them the Q8 codes, are then reproducible
    double ss = 0.0;
    for (int i = tid * 4; i < h; i += 1024) {
        const float4 v = *reinterpret_cast<const float4 *>(xr + i);
        ss += (double)v.x * v.x + (double)v.y * v.y + (double)v.z * v.z + (double)v.w * v.w;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (lane == 0) part[warp] = ss;
    __syncthreads();
    if (tid == 0) {
        double t = 0.0;
        for (int i = 0; i < 8; i++) t += part[i];
        s_scale = 1.0f / sqrtf((float)(t / (double)h) + eps);
    }
    __syncthreads();
    const float scale = s_scale;
    if (q) {
        const int nb = h / 256;
        for (int b = warp; b < nb; b += 8) {
            const int o = b * 256 + lane * 8;
            const float4 a = *reinterpret_cast<const float4 *>(xr + o);
            const float4 c = *reinterpret_cast<const float4 *>(xr + o + 4);
            float v[8] = {a.x, a.y, a.z, a.w, c.x, c.y, c.z, c.w};
#pragma unroll
            for (int i = 0; i < 8; i++) v[i] = v[i] * scale * (w ? w[o + i] : 1.0f);
            if (y) {
                float *yo = y + (int64_t)row * h + o;
                *reinterpret_cast<float4 *>(yo) = make_float4(v[0], v[1], v[2], v[3]);
                *reinterpret_cast<float4 *>(yo + 4) = make_float4(v[4], v[5], v[6], v[7]);
            }
            const int64_t gb = (int64_t)row * nb + b;
            kq_quantize_block_warp(v, lane, q + gb * 256, d + gb, bs + gb * 16);
        }
    } else {
        for (int i = tid; i < h; i += 256) y[(int64_t)row * h + i] = xr[i] * scale * (w ? w[i] : 1.0f);
    }
}

// ---- Q6_K repack: GGUF block-interleaved rows <-> device rows [ql | qh | scales | d | pad] ------
__global__ void repack_q6k_kernel(const uint16_t *src, uint16_t *dst,
                                  int64_t n_rows, int nb, int64_t dst_row_u16, int inverse) {
    KQ_PDL_ENTER();
    const int64_t per_row = (int64_t)nb * 105;
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_rows * per_row) return;
    const int64_t row = i / per_row;
    const int r = (int)(i % per_row), b = r / 105, o = r % 105; // u16 index inside the block
    const KqQ6Addr qa = kq_q6_addr(nb, b);
    int64_t dev; // u16 offset inside the device row
    if (o < 64) dev = (qa.ql + ((2 * o) >> 4) * qa.cs + ((2 * o) & 15)) / 2;
    else if (o < 96) dev = (qa.qh + ((2 * (o - 64)) >> 4) * qa.cs + ((2 * (o - 64)) & 15)) / 2;
    else if (o < 104) dev = qa.sc / 2 + (o - 96);
    else dev = qa.d / 2;
    const int64_t g = row * per_row + r, dv = row * dst_row_u16 + dev;
    if (inverse) dst[g] = src[dv];
    else dst[dv] = src[g];
}

// ---- synthetic weights ------------------------------------------------------------------------
__device__ __forceinline__ uint64_t mix64(uint64_t z) {
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
__device__ __forceinline__ float gauss_at(uint64_t key, uint64_t i) {
    const uint64_t r = mix64(key + i * 0xD1342543DE82EF95ull);
    const float u1 = ((float)((uint32_t)(r >> 32) >> 8) + 1.0f) * (1.0f / 16777216.0f);
    const float u2 = (float)((uint32_t)r >> 8) * (1.0f / 16777216.0f);
    return sqrtf(-2.0f * __logf(u1)) * __cosf(6.28318530717958647692f * u2);
}

// One warp per 256-element block; writes the block in device layout.
__global__ void __launch_bounds__(128) synth_kquant_kernel(uint32_t type, uint8_t *W, int64_t n_rows,
                                                           int nb, uint64_t key, float sigma) {
    KQ_PDL_ENTER();
    __shared__ uint8_t codes[4][256];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t gb = (int64_t)blockIdx.x * 4 + warp;
    if (gb >= n_rows * nb) return;
    const int64_t row = gb / nb;
    const int b = (int)(gb % nb);
    float v[8];
#pragma unroll
    for (int i = 0; i < 8; i++) v[i] = sigma * gauss_at(key, (uint64_t)(gb * 256 + lane * 8 + i));
    uint8_t *rp = W + row * kq_device_row_bytes(type, (int64_t)nb * 256);
    uint8_t *cd = codes[warp];
    if (type == B200_TYPE_Q4_K) {
        float lo = 0.f, hi = 0.f;
#pragma unroll
        for (int i = 0; i < 8; i++) { lo = fminf(lo, v[i]); hi = fmaxf(hi, v[i]); }
        lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, 1));
        lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, 2));
        hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, 1));
        hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, 2));
        const float scale = (hi - lo) / 15.0f, mn = -lo;
        const __half dh = __float2half_rn(kq_warp_max(scale) / 63.0f);
        const __half mh = __float2half_rn(kq_warp_max(mn) / 63.0f);
        const float d = __half2float(dh), dmin = __half2float(mh);
        const int sc = d > 0.f ? max(0, min(63, __float2int_rn(scale / d))) : 0;
        const int mc = dmin > 0.f ? max(0, min(63, __float2int_rn(mn / dmin))) : 0;
        const float dl = d * (float)sc, ml = dmin * (float)mc;
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const int qv = dl > 0.f ? __float2int_rn((v[i] + ml) / dl) : 0;
            cd[lane * 8 + i] = (uint8_t)max(0, min(15, qv));
        }
        __syncwarp();
        uint8_t *blk = rp + (int64_t)b * KQ_Q4K_BYTES;
        // 128 quant bytes: lane writes bytes 4l .. 4l+3
        uint32_t pk = 0;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int byte = lane * 4 + i, g = byte >> 5, k = byte & 31;
            pk |= (uint32_t)(cd[64 * g + k] | (cd[64 * g + 32 + k] << 4)) << (8 * i);
        }
        *reinterpret_cast<uint32_t *>(blk + 16 + lane * 4) = pk;
        // header: gather the 8 scale / min codes (sub-block j lives in lanes 4j..4j+3)
        int scj[8], mcj[8];
#pragma unroll
        for (int j = 0; j < 8; j++) {
            scj[j] = __shfl_sync(0xffffffffu, sc, 4 * j);
            mcj[j] = __shfl_sync(0xffffffffu, mc, 4 * j);
        }
        if (lane == 0) {
            uint8_t s[12];
#pragma unroll
            for (int j = 0; j < 4; j++) {
                s[j] = (uint8_t)(scj[j] | ((scj[j + 4] >> 4) << 6));
                s[j + 4] = (uint8_t)(mcj[j] | ((mcj[j + 4] >> 4) << 6));
                s[j + 8] = (uint8_t)((scj[j + 4] & 0xF) | ((mcj[j + 4] & 0xF) << 4));
            }
            uint4 hdr;
            hdr.x = (uint32_t)__half_as_ushort(dh) | ((uint32_t)__half_as_ushort(mh) << 16);
            hdr.y = s[0] | (s[1] << 8) | (s[2] << 16) | ((uint32_t)s[3] << 24);
            hdr.z = s[4] | (s[5] << 8) | (s[6] << 16) | ((uint32_t)s[7] << 24);
            hdr.w = s[8] | (s[9] << 8) | (s[10] << 16) | ((uint32_t)s[11] << 24);
            *reinterpret_cast<uint4 *>(blk) = hdr;
        }
    } else { // Q6_K, symmetric per 16 elements (2 lanes)
        float am = 0.f;
#pragma unroll
        for (int i = 0; i < 8; i++) am = fmaxf(am, fabsf(v[i]));
        am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, 1));
        const float scale = am / 31.0f;
        const __half dh = __float2half_rn(kq_warp_max(scale) / 127.0f);
        const float d = __half2float(dh);
        const int sc = d > 0.f ? max(0, min(127, __float2int_rn(scale / d))) : 0;
        const float dl = d * (float)sc;
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const int qv = dl > 0.f ? __float2int_rn(v[i] / dl) : 0;
            cd[lane * 8 + i] = (uint8_t)(max(-32, min(31, qv)) + 32);
        }
        __syncwarp();
        // ql: 128 bytes, lane writes bytes 4l..4l+3; byte 64h+k = elem 128h+k | elem 128h+64+k << 4
        uint32_t pk = 0;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int byte = lane * 4 + i, h = byte >> 6, k = byte & 63;
            pk |= (uint32_t)((cd[128 * h + k] & 0xF) | ((cd[128 * h + 64 + k] & 0xF) << 4)) << (8 * i);
        }
        const KqQ6Addr qa = kq_q6_addr(nb, b);
        *reinterpret_cast<uint32_t *>(rp + qa.ql + ((lane * 4) >> 4) * qa.cs + ((lane * 4) & 15)) = pk;
        // qh: 64 bytes, lane writes bytes 2l, 2l+1; byte 32h+k = hi2 of elems 128h+k+{0,32,64,96}
        uint16_t ph = 0;
#pragma unroll
        for (int i = 0; i < 2; i++) {
            const int byte = lane * 2 + i, h = byte >> 5, k = byte & 31;
            const uint32_t v8 = (cd[128 * h + k] >> 4) | ((cd[128 * h + 32 + k] >> 4) << 2) |
                                ((cd[128 * h + 64 + k] >> 4) << 4) | ((cd[128 * h + 96 + k] >> 4) << 6);
            ph |= (uint16_t)(v8 << (8 * i));
        }
        *reinterpret_cast<uint16_t *>(rp + qa.qh + ((lane * 2) >> 4) * qa.cs + ((lane * 2) & 15)) = ph;
        if ((lane & 1) == 0) rp[qa.sc + (lane >> 1)] = (uint8_t)(int8_t)sc;
        if (lane == 0) *reinterpret_cast<uint16_t *>(rp + qa.d) = __half_as_ushort(dh);
    }
}

__global__ void synth_f32_kernel(float *w, int64_t n, uint64_t key, float mean, float sigma) {
    KQ_PDL_ENTER();
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) w[i] = mean + sigma * gauss_at(key, (uint64_t)i);
}

} // namespace

b200_status kq_synth_weights(uint32_t type, void *W, int64_t n_rows, int64_t K, uint64_t key,
                             float mean, float sigma, cudaStream_t st) {
    if (type == B200_TYPE_F32) {
        const int64_t n = n_rows * K;
        kq_launch(synth_f32_kernel, (unsigned)kq_div_up(n, 256), 256, 0, st, (float *)W, n, key, mean, sigma);
    } else {
        KQ_REQUIRE(type == B200_TYPE_Q4_K || type == B200_TYPE_Q6_K, "synth: type %u", type);
        KQ_REQUIRE(K % 256 == 0, "synth: K %% 256");
        const int64_t blocks = n_rows * (K / 256);
        kq_launch(synth_kquant_kernel, (unsigned)kq_div_up(blocks, 4), 128, 0, st, type, (uint8_t *)W, n_rows,
                                                                           (int)(K / 256), key, sigma);
    }
    KQ_COUNT_LAUNCH();
    KQ_LAUNCH_CHECK();
    return B200_OK;
}

b200_status kq_rms_norm(const float *x, const float *w, int64_t T, int64_t h, float eps, float *y,
                        int8_t *q, float *d, int16_t *bs, cudaStream_t st, int64_t x_row_stride) {
    KQ_REQUIRE(T > 0 && h > 0 && h % 4 == 0, "rms_norm: bad shape");
    KQ_REQUIRE(!q || h % 256 == 0, "rms_norm: Q8 output needs h %% 256 == 0");
    KQ_REQUIRE(y || q, "rms_norm: no output");
    kq_launch(rms_norm_kernel, (unsigned)T, 256, 0, st, x, w, (int)h, eps, y, q, d, bs, x_row_stride ? x_row_stride : h);
    KQ_COUNT_LAUNCH();
    KQ_LAUNCH_CHECK();
    return B200_OK;
}

// y = silu(g) * u for [M][K] and its Q8 form; K a multiple of 256, pointers 16-byte aligned; y may be null or alias g
b200_status kq_swiglu_quantize(const float *g, const float *u, int64_t M, int64_t K, float *y, int8_t *q, float *d, int16_t *bs,
                               cudaStream_t st) {
    KQ_REQUIRE(M > 0 && K > 0 && K % 256 == 0, "swiglu_quantize: K must be a multiple of 256");
    KQ_REQUIRE((((uintptr_t)g | (uintptr_t)u | (uintptr_t)y | (uintptr_t)q) & 15) == 0, "swiglu_quantize: alignment");
    const int64_t nblocks = M * (K / 256);
    kq_launch(swiglu_quantize_kernel, (unsigned)kq_div_up(nblocks, 4), 128, 0, st, g, u, nblocks, y, q, d, bs);
    KQ_COUNT_LAUNCH();
    KQ_LAUNCH_CHECK();
    return B200_OK;
}

extern "C" b200_status b200_quantize_act(const float *x, int64_t M, int64_t K, int8_t *q, float *d,
                                         int16_t *bsum16, void *stream) {
    KQ_REQUIRE(M > 0 && K > 0 && K % 256 == 0, "quantize_act: K must be a multiple of 256");
    KQ_REQUIRE(((uintptr_t)x & 15) == 0 && ((uintptr_t)q & 15) == 0, "quantize_act: alignment");
    const int64_t nblocks = M * (K / 256);
    kq_launch(quantize_act_kernel, (unsigned)kq_div_up(nblocks, 4), 128, 0, (cudaStream_t)stream, x, nblocks, q, d,
                                                                                        bsum16);
    KQ_COUNT_LAUNCH();
    KQ_LAUNCH_CHECK();
    return B200_OK;
}

extern "C" b200_status b200_rms_norm(const float *x, const float *w, int64_t T, int64_t h, float eps,
                                     float *y, void *stream) {
    return kq_rms_norm(x, w, T, h, eps, y, nullptr, nullptr, nullptr, (cudaStream_t)stream, 0);
}

static b200_status repack(const void *src, void *dst, int64_t n_rows, int64_t k, int inverse,
                          cudaStream_t st) {
    KQ_REQUIRE(n_rows > 0 && k > 0 && k % 256 == 0, "repack_q6k: bad shape");
    const int nb = (int)(k / 256);
    const int64_t total = n_rows * nb * 105;
    kq_launch(repack_q6k_kernel, (unsigned)kq_div_up(total, 256), 256, 0, st, 
        (const uint16_t *)src, (uint16_t *)dst, n_rows, nb, kq_device_row_bytes(B200_TYPE_Q6_K, k) / 2,
        inverse);
    KQ_COUNT_LAUNCH();
    KQ_LAUNCH_CHECK();
    return B200_OK;
}

extern "C" b200_status b200_repack_q6k(const void *gguf_rows_dev, void *device_rows, int64_t n_rows,
                                       int64_t k, void *stream) {
    return repack(gguf_rows_dev, device_rows, n_rows, k, 0, (cudaStream_t)stream);
}
extern "C" b200_status b200_unpack_q6k(const void *device_rows, void *gguf_rows_dev, int64_t n_rows,
                                       int64_t k, void *stream) {
    return repack(device_rows, gguf_rows_dev, n_rows, k, 1, (cudaStream_t)stream);
}
