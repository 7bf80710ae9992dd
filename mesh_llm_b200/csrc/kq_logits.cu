// Per-token statistics of the output distribution, computed where the logits are: greedy argmax,
// Shannon entropy (bits) of the full-vocabulary softmax, the margin between the two most likely
// tokens, the probability of the chosen token and the five most likely tokens.  With its mesh hooks
// on, the reference's server derives exactly these on the CPU after the prefill and after every
// generated token (third_party/llama.cpp/patches/0005: entropy = -sum p log2 p over the sorted
// distribution, margin = p[0] - p[1], top tokens for the hook payload); on a 152 k vocabulary that is
// a 600 KB read per token that belongs next to the LM head.
//
// One row is cut into slices, one CTA each; a slice leaves (max, argmax, Z = sum e^(x - max),
// S = sum e^(x - max) (x - max), its five largest entries) in scratch, and the CTA that arrives last
// at the row's counter merges the slices in slice order, so the result does not depend on timing.
#include "kq_common.cuh"

#include <math.h>

namespace {

constexpr int SLICES_MAX = 64, NT = 256, TOPK = 5;

struct SlicePart {
    float m, z, s;
    int arg;
    float tv[TOPK];
    int ti[TOPK];
};

__device__ __forceinline__ bool better(float v, int i, float bv, int bi) { return v > bv || (v == bv && i < bi); }

// keep (tv, ti) sorted best first
__device__ __forceinline__ void top_insert(float (&tv)[TOPK], int (&ti)[TOPK], float v, int i) {
    if (!better(v, i, tv[TOPK - 1], ti[TOPK - 1])) return;
    tv[TOPK - 1] = v;
    ti[TOPK - 1] = i;
#pragma unroll
    for (int k = TOPK - 1; k > 0; k--)
        if (better(tv[k], ti[k], tv[k - 1], ti[k - 1])) {
            const float fv = tv[k]; tv[k] = tv[k - 1]; tv[k - 1] = fv;
            const int fi = ti[k]; ti[k] = ti[k - 1]; ti[k - 1] = fi;
        }
}

// Every thread holds a sorted candidate list; the TOPK best of the whole CTA end up, in order, in
// out_v / out_i (shared).  A round takes the best head, its owner pops it.
__device__ void block_topk(float (&tv)[TOPK], int (&ti)[TOPK], float *out_v, int *out_i, float *red_v, int *red_i) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    int head = 0;
    for (int r = 0; r < TOPK; r++) {
        float v = head < TOPK ? tv[0] : -INFINITY;
        int i = head < TOPK ? ti[0] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, v, o);
            const int oi = __shfl_xor_sync(0xffffffffu, i, o);
            if (better(ov, oi, v, i)) { v = ov; i = oi; }
        }
        if (lane == 0) { red_v[warp] = v; red_i[warp] = i; }
        __syncthreads();
        if (warp == 0) {
            v = lane < nwarp ? red_v[lane] : -INFINITY;
            i = lane < nwarp ? red_i[lane] : 0x7fffffff;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, v, o);
                const int oi = __shfl_xor_sync(0xffffffffu, i, o);
                if (better(ov, oi, v, i)) { v = ov; i = oi; }
            }
            if (lane == 0) { out_v[r] = v; out_i[r] = i; }
        }
        __syncthreads();
        if (head < TOPK && ti[0] == out_i[r] && tv[0] == out_v[r]) { // the winner's owner pops it
#pragma unroll
            for (int k = 0; k < TOPK - 1; k++) { tv[k] = tv[k + 1]; ti[k] = ti[k + 1]; }
            tv[TOPK - 1] = -INFINITY;
            ti[TOPK - 1] = 0x7fffffff;
            head++;
        }
        __syncthreads();
    }
}

__global__ void __launch_bounds__(NT) logit_scan_kernel(const float *x, int64_t n, int n_slice,
                                                        const int32_t *chosen, SlicePart *parts, int *counters,
                                                        b200_logit_signals_t *sig, int32_t *argmax_out) {
    KQ_PDL_ENTER();
    __shared__ float red_v[32], out_v[TOPK];
    __shared__ int red_i[32], out_i[TOPK];
    __shared__ float red_z[32], red_s[32];
    __shared__ int s_last;
    const int row = blockIdx.y, slice = blockIdx.x;
    const float *xr = x + (int64_t)row * n;
    const int64_t per = (n + n_slice - 1) / n_slice;
    const int64_t i0 = (int64_t)slice * per, i1 = i0 + per < n ? i0 + per : n;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

    float tv[TOPK];
    int ti[TOPK];
#pragma unroll
    for (int k = 0; k < TOPK; k++) { tv[k] = -INFINITY; ti[k] = 0x7fffffff; }
    for (int64_t i = i0 + threadIdx.x; i < i1; i += NT) top_insert(tv, ti, xr[i], (int)i);
    const float my_best = tv[0];
    block_topk(tv, ti, out_v, out_i, red_v, red_i);
    const float m = out_v[0]; // slice maximum (-inf for an empty slice)
    float z = 0.f, s = 0.f;
    if (m > -INFINITY)
        for (int64_t i = i0 + threadIdx.x; i < i1; i += NT) { // second pass: the slice is in L1 / L2
            const float d = xr[i] - m, e = expf(d);
            z += e;
            if (e > 0.f) s += e * d;
        }
    (void)my_best;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        z += __shfl_xor_sync(0xffffffffu, z, o);
        s += __shfl_xor_sync(0xffffffffu, s, o);
    }
    if (lane == 0) { red_z[warp] = z; red_s[warp] = s; }
    __syncthreads();
    SlicePart *mine = parts + (int64_t)row * n_slice + slice;
    if (threadIdx.x == 0) {
        float zz = 0.f, ss = 0.f;
        for (int w = 0; w < NT / 32; w++) { zz += red_z[w]; ss += red_s[w]; }
        mine->m = m;
        mine->z = zz;
        mine->s = ss;
        mine->arg = out_i[0];
#pragma unroll
        for (int k = 0; k < TOPK; k++) { mine->tv[k] = out_v[k]; mine->ti[k] = out_i[k]; }
        __threadfence();
        const int prev = atomicAdd(&counters[row], 1);
        s_last = prev == n_slice - 1;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    // ---- merge of the row's slices by its last CTA (first warp; slices in index order)
    if (warp == 0) {
        const volatile SlicePart *pr = parts + (int64_t)row * n_slice;
        float gm = -INFINITY;
        for (int sl = lane; sl < n_slice; sl += 32) gm = fmaxf(gm, pr[sl].m);
        gm = kq_warp_max(gm);
        float zz = 0.f, ss = 0.f;
        float cv[TOPK];
        int ci[TOPK];
#pragma unroll
        for (int k = 0; k < TOPK; k++) { cv[k] = -INFINITY; ci[k] = 0x7fffffff; }
        for (int sl = lane; sl < n_slice; sl += 32) {
            const float ml = pr[sl].m;
            if (ml > -INFINITY) {
                const float sc = expf(ml - gm), zl = pr[sl].z;
                zz += zl * sc;
                ss += sc * (pr[sl].s + zl * (ml - gm));
            }
#pragma unroll
            for (int k = 0; k < TOPK; k++) top_insert(cv, ci, pr[sl].tv[k], pr[sl].ti[k]);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            zz += __shfl_xor_sync(0xffffffffu, zz, o);
            ss += __shfl_xor_sync(0xffffffffu, ss, o);
        }
        float bv[TOPK];
        int bi[TOPK];
        for (int r = 0; r < TOPK; r++) { // warp-wide: best head, owner pops
            float v = cv[0];
            int i = ci[0];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, v, o);
                const int oi = __shfl_xor_sync(0xffffffffu, i, o);
                if (better(ov, oi, v, i)) { v = ov; i = oi; }
            }
            bv[r] = v;
            bi[r] = i;
            if (ci[0] == i && cv[0] == v) {
#pragma unroll
                for (int k = 0; k < TOPK - 1; k++) { cv[k] = cv[k + 1]; ci[k] = ci[k + 1]; }
                cv[TOPK - 1] = -INFINITY;
                ci[TOPK - 1] = 0x7fffffff;
            }
        }
        if (lane == 0) {
            if (argmax_out) argmax_out[row] = bi[0] == 0x7fffffff ? 0 : bi[0];
            if (sig) {
                b200_logit_signals_t o;
                const float inv = zz > 0.f ? 1.0f / zz : 0.f;
                o.entropy = zz > 0.f ? log2f(zz) - ss * inv * 1.4426950408889634f : 0.f;
                for (int k = 0; k < TOPK; k++) {
                    o.top_id[k] = bi[k] == 0x7fffffff ? -1 : bi[k];
                    o.top_p[k] = bv[k] > -INFINITY ? expf(bv[k] - gm) * inv : 0.f;
                }
                o.margin = o.top_id[1] >= 0 ? o.top_p[0] - o.top_p[1] : 1.0f;
                const int c = chosen ? chosen[row] : bi[0];
                o.p_chosen = (c >= 0 && c < n) ? expf(xr[c] - gm) * inv : 0.f;
                sig[row] = o;
            }
            counters[row] = 0; // armed for the next launch
        }
    }
}

} // namespace

extern "C" {

size_t b200_logit_signals_scratch_bytes(int64_t T) {
    if (T < 1) T = 1;
    return (size_t)T * SLICES_MAX * sizeof(SlicePart) + (size_t)T * sizeof(int) + 256;
}

b200_status b200_logit_signals(const float *logits, int64_t T, int64_t n, const int32_t *chosen,
                               b200_logit_signals_t *signals, int32_t *argmax_out, void *scratch,
                               size_t scratch_bytes, void *stream) {
    KQ_REQUIRE(logits && scratch && T >= 1 && n >= 1, "logit_signals: null or empty argument");
    KQ_REQUIRE(n < 0x7fffffff, "logit_signals: row too long");
    KQ_REQUIRE(scratch_bytes >= b200_logit_signals_scratch_bytes(T), "logit_signals: scratch of %zu bytes, %zu needed",
               scratch_bytes, b200_logit_signals_scratch_bytes(T));
    KQ_REQUIRE(((uintptr_t)scratch & 15) == 0, "logit_signals: scratch must be 16-byte aligned");
    // the counters sit behind the slice records and must start at zero: the caller hands in zeroed
    // scratch once (cudaMemset), every launch leaves them zero again
    int n_slice = (int)kq_div_up(n, 4096);
    if (n_slice > SLICES_MAX) n_slice = SLICES_MAX;
    if (n_slice < 1) n_slice = 1;
    // Layout of the scratch: the per-row counters first, then the slice records.  Where the records
    // start depends on the size of the scratch only, never on this call's T: calls with different row
    // counts that share one scratch (a prefill with all rows, then decode steps with one) must find the
    // counters, which every launch leaves at zero, in the same place.
    const size_t rows_cap = (scratch_bytes - 256) / ((size_t)SLICES_MAX * sizeof(SlicePart) + sizeof(int));
    int *counters = (int *)scratch;
    SlicePart *parts = (SlicePart *)((uint8_t *)scratch + ((rows_cap * sizeof(int) + 255) & ~(size_t)255));
    kq_launch(logit_scan_kernel, dim3((unsigned)n_slice, (unsigned)T), NT, 0, (cudaStream_t)stream, logits, n, n_slice,
              chosen, parts, counters, signals, argmax_out);
    KQ_COUNT_LAUNCH();
    KQ_LAUNCH_CHECK();
    return B200_OK;
}

} // extern "C"
