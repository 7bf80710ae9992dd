// Stage-boundary hand-off through peer memory.
//
// What it replaces: the activation a stage hands to the next one.  In the reference that is a ggml-RPC
// round trip (third_party/llama.cpp/patches/0002 lines 544-622: device -> host -> TCP -> host ->
// device) or, with direct push, PUSH_TENSOR_TO_PEER writing into the receiver's buffer (lines 624-735).
// Here the receiver owns a landing ring in its own HBM; the sender's kernel writes the payload into
// the next free slot through the NVLink peer mapping and then publishes the slot's sequence number
// with a system-scope release store; the receiver's kernel acquires that number, copies the slot to
// where the stage reads its input and publishes how many slots it has consumed.  The payload crosses
// NVLink once, there is no host round trip and no rendezvous: a send never waits for the receive to
// be posted, only (bounded) for a free slot.
//
// Every wait is bounded: when a limit runs out the kernel records a status in the endpoint's error
// word and returns without touching the payload, so the context stays usable and the host reads the
// status.  Sender and receiver are different GPUs (or one GPU with the send ordered before the wait
// on one stream); two kernels that wait on one another are never put on the same GPU.
#include "kq_common.cuh"

#include <algorithm>

#include <string.h>

namespace {

constexpr uint32_t HANDOFF_MAGIC = 0x48444F46u; // "HDOF"
constexpr int CTRL_BYTES = 256;                  // consumed counter and error word, apart from the flags

struct Layout {
    size_t slot_stride, flags_off, ctrl_off, total;
};
Layout layout_of(size_t slot_bytes, int n_slots) {
    Layout l;
    l.slot_stride = (slot_bytes + 255) & ~(size_t)255;
    l.flags_off = l.slot_stride * n_slots;
    l.ctrl_off = l.flags_off + (((size_t)n_slots * 8 + 255) & ~(size_t)255);
    l.total = l.ctrl_off + CTRL_BYTES;
    return l;
}

} // namespace

// A receive endpoint (owned == true: memory of this process) or the mapping of another endpoint that
// this process sends to.
struct b200_handoff {
    uint32_t magic = HANDOFF_MAGIC;
    bool owned = false, ipc = false;
    int device = 0, n_slots = 0;
    size_t slot_bytes = 0;
    Layout lay{};
    uint8_t *base = nullptr;    // ring | flags | control
    uint64_t *known = nullptr;  // sender side: last consumed count seen (device word of this process)
    int *send_err = nullptr;    // sender side: error word of this process
};

namespace {

__device__ __forceinline__ uint64_t ld_acquire_sys(const uint64_t *p) {
    uint64_t v;
    asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(uint64_t *p, uint64_t v) {
    asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}

// One CTA.  ring / flags / consumed belong to the receiver (peer memory when it is another GPU).
__global__ void __launch_bounds__(256) handoff_send_kernel(const uint4 *src, size_t bytes, uint8_t *ring,
                                                            size_t slot_stride, uint64_t *flags, const uint64_t *consumed,
                                                            uint64_t *known, int *err, uint64_t seqno, int n_slots,
                                                            uint64_t limit_ns) {
    KQ_PDL_WAIT(); // src is the output of the kernels before this one
    __shared__ int s_ok;
    if (threadIdx.x == 0) {
        // a slot is free once the receiver has consumed the payload that used it n_slots sends ago;
        // the receiver's counter is read over the link only when the cached value does not suffice
        int ok = *reinterpret_cast<volatile int *>(err) == 0; // after one time-out the following sends give up at once
        if (ok && seqno >= *known + (uint64_t)n_slots) {
            const uint64_t t0 = kq_globaltimer_ns();
            uint64_t c = ld_acquire_sys(consumed);
            while (seqno >= c + (uint64_t)n_slots) {
                if (kq_globaltimer_ns() - t0 > limit_ns) {
                    ok = 0;
                    break;
                }
                __nanosleep(200);
                c = ld_acquire_sys(consumed);
            }
            *known = c;
        }
        if (!ok) atomicCAS(err, 0, 1); // no free slot in time
        s_ok = ok;
    }
    __syncthreads();
    if (!s_ok) return;
    const int slot = (int)(seqno % (uint64_t)n_slots);
    uint4 *dst = reinterpret_cast<uint4 *>(ring + (size_t)slot * slot_stride);
    const size_t n16 = ((uintptr_t)src & 15) ? 0 : bytes / 16; // whole 16-byte words, then the 4-byte rest
    for (size_t i = threadIdx.x; i < n16; i += blockDim.x) dst[i] = src[i];
    for (size_t i = n16 * 4 + threadIdx.x; i < bytes / 4; i += blockDim.x)
        reinterpret_cast<uint32_t *>(dst)[i] = reinterpret_cast<const uint32_t *>(src)[i];
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) st_release_sys(flags + slot, seqno + 1);
}

// Large payloads (a prefill micro-batch: megabytes) go out as three launches on the sender's stream:
// reserve (one thread waits for the slot to be free), copy (a grid of CTAs stores the payload into the
// peer's slot), publish (system-scope fence, then the payload's number).  The copy kernel has finished,
// and with it all its stores, before the publishing kernel starts.
__global__ void handoff_reserve_kernel(const uint64_t *consumed, uint64_t *known, int *err, uint64_t seqno, int n_slots,
                                       uint64_t limit_ns) {
    KQ_PDL_WAIT();
    int ok = *reinterpret_cast<volatile int *>(err) == 0;
    if (ok && seqno >= *known + (uint64_t)n_slots) {
        const uint64_t t0 = kq_globaltimer_ns();
        uint64_t c = ld_acquire_sys(consumed);
        while (seqno >= c + (uint64_t)n_slots) {
            if (kq_globaltimer_ns() - t0 > limit_ns) {
                ok = 0;
                break;
            }
            __nanosleep(200);
            c = ld_acquire_sys(consumed);
        }
        *known = c;
    }
    if (!ok) atomicCAS(err, 0, 1); // no free slot in time
}
__global__ void __launch_bounds__(256) handoff_copy_kernel(const uint4 *src, uint4 *dst, size_t n16, const int *err) {
    KQ_PDL_WAIT(); // src is the output of the kernels before; the reservation precedes this kernel
    if (*reinterpret_cast<const volatile int *>(err) != 0) return;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += (size_t)gridDim.x * blockDim.x) dst[i] = src[i];
}
__global__ void handoff_publish_kernel(uint64_t *flag, const int *err, uint64_t seqno) {
    KQ_PDL_WAIT(); // every store of the copy kernel has been performed
    if (*reinterpret_cast<const volatile int *>(err) != 0) return;
    __threadfence_system();
    st_release_sys(flag, seqno + 1);
}

// One CTA on the receiver.  dst may be null: the caller then reads the slot in place.
__global__ void __launch_bounds__(256) handoff_wait_kernel(uint4 *dst, size_t bytes, const uint8_t *ring,
                                                            size_t slot_stride, const uint64_t *flags, uint64_t *consumed,
                                                            int *err, uint64_t seqno, int n_slots, uint64_t limit_ns) {
    KQ_PDL_WAIT(); // dst may still be read by the kernels before this one
    __shared__ int s_ok;
    const int slot = (int)(seqno % (uint64_t)n_slots);
    if (threadIdx.x == 0) {
        int ok = *reinterpret_cast<volatile int *>(err) == 0; // after one time-out the following waits give up at once
        const uint64_t t0 = kq_globaltimer_ns();
        while (ok && ld_acquire_sys(flags + slot) != seqno + 1) {
            if (kq_globaltimer_ns() - t0 > limit_ns) {
                ok = 0;
                break;
            }
            __nanosleep(100);
        }
        if (!ok) atomicCAS(err, 0, 2); // the payload did not arrive in time
        s_ok = ok;
    }
    __syncthreads();
    if (!s_ok) return;
    if (dst) {
        const uint4 *src = reinterpret_cast<const uint4 *>(ring + (size_t)slot * slot_stride);
        const size_t n16 = ((uintptr_t)dst & 15) ? 0 : bytes / 16;
        for (size_t i = threadIdx.x; i < n16; i += blockDim.x) dst[i] = __ldcg(src + i);
        for (size_t i = n16 * 4 + threadIdx.x; i < bytes / 4; i += blockDim.x)
            reinterpret_cast<uint32_t *>(dst)[i] = __ldcg(reinterpret_cast<const uint32_t *>(src) + i);
        __syncthreads();
    }
    if (threadIdx.x == 0 && dst) st_release_sys(consumed, seqno + 1);
}

__global__ void handoff_release_kernel(uint64_t *consumed, uint64_t seqno) {
    KQ_PDL_WAIT(); // the readers of the slot come before this kernel
    st_release_sys(consumed, seqno + 1);
}

bool valid(const b200_handoff *h) { return h && h->magic == HANDOFF_MAGIC; }

} // namespace

extern "C" {

b200_status b200_handoff_create(size_t slot_bytes, int32_t n_slots, b200_handoff **out) {
    KQ_REQUIRE(out && slot_bytes > 0 && slot_bytes % 4 == 0 && n_slots >= 2 && n_slots <= 4096,
               "handoff_create: slot_bytes must be a positive multiple of 4 and 2 <= n_slots <= 4096");
    b200_handoff *h = new b200_handoff();
    h->owned = true;
    h->n_slots = n_slots;
    h->slot_bytes = slot_bytes;
    h->lay = layout_of(slot_bytes, n_slots);
    if (cudaGetDevice(&h->device) != cudaSuccess || cudaMalloc((void **)&h->base, h->lay.total) != cudaSuccess ||
        cudaMemset(h->base, 0, h->lay.total) != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess) {
        kq_set_error("handoff_create: allocating %zu bytes failed: %s", h->lay.total, cudaGetErrorString(cudaGetLastError()));
        if (h->base) cudaFree(h->base);
        delete h;
        return B200_ERR_CUDA;
    }
    *out = h;
    return B200_OK;
}

b200_status b200_handoff_export(const b200_handoff *h, void *handle64) {
    KQ_REQUIRE(valid(h) && h->owned && handle64, "handoff_export: a local endpoint and a 64-byte buffer are required");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    cudaIpcMemHandle_t ipc;
    KQ_CUDA(cudaIpcGetMemHandle(&ipc, h->base));
    memcpy(handle64, &ipc, 64);
    return B200_OK;
}

static b200_status finish_remote(b200_handoff *r) {
    if (cudaMalloc((void **)&r->known, 256) != cudaSuccess || cudaMemset(r->known, 0, 256) != cudaSuccess ||
        cudaDeviceSynchronize() != cudaSuccess) {
        kq_set_error("handoff: allocating the sender's words failed");
        return B200_ERR_CUDA;
    }
    r->send_err = reinterpret_cast<int *>(r->known + 8);
    return B200_OK;
}

b200_status b200_handoff_open(const void *handle64, size_t slot_bytes, int32_t n_slots, b200_handoff **out) {
    KQ_REQUIRE(out && handle64 && slot_bytes > 0 && slot_bytes % 4 == 0 && n_slots >= 2,
               "handoff_open: handle, slot_bytes and n_slots of the endpoint are required");
    cudaIpcMemHandle_t ipc;
    memcpy(&ipc, handle64, 64);
    b200_handoff *r = new b200_handoff();
    r->ipc = true;
    r->n_slots = n_slots;
    r->slot_bytes = slot_bytes;
    r->lay = layout_of(slot_bytes, n_slots);
    cudaGetDevice(&r->device);
    if (cudaIpcOpenMemHandle((void **)&r->base, ipc, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
        kq_set_error("handoff_open: mapping the peer's landing ring failed: %s", cudaGetErrorString(cudaGetLastError()));
        delete r;
        return B200_ERR_CUDA;
    }
    const b200_status rc = finish_remote(r);
    if (rc != B200_OK) {
        cudaIpcCloseMemHandle(r->base);
        delete r;
        return rc;
    }
    *out = r;
    return B200_OK;
}

b200_status b200_handoff_open_local(const b200_handoff *endpoint, b200_handoff **out) {
    KQ_REQUIRE(valid(endpoint) && endpoint->owned && out, "handoff_open_local: a local endpoint is required");
    int dev = 0;
    KQ_CUDA(cudaGetDevice(&dev));
    if (dev != endpoint->device) {
        int can = 0;
        KQ_CUDA(cudaDeviceCanAccessPeer(&can, dev, endpoint->device));
        KQ_REQUIRE(can, "handoff_open_local: device %d cannot map the memory of device %d", dev, endpoint->device);
        const cudaError_t e = cudaDeviceEnablePeerAccess(endpoint->device, 0);
        if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled) KQ_CUDA(e);
        cudaGetLastError();
    }
    b200_handoff *r = new b200_handoff();
    r->n_slots = endpoint->n_slots;
    r->slot_bytes = endpoint->slot_bytes;
    r->lay = endpoint->lay;
    r->device = dev;
    r->base = endpoint->base;
    const b200_status rc = finish_remote(r);
    if (rc != B200_OK) {
        delete r;
        return rc;
    }
    *out = r;
    return B200_OK;
}

b200_status b200_handoff_send(b200_handoff *remote, const void *src, size_t bytes, uint64_t seqno, uint64_t limit_ns,
                              void *stream) {
    KQ_REQUIRE(valid(remote) && !remote->owned && src, "handoff_send: a mapping made by handoff_open is required");
    KQ_REQUIRE(bytes > 0 && bytes % 4 == 0 && bytes <= remote->slot_bytes && ((uintptr_t)src & 3) == 0,
               "handoff_send: %zu bytes do not fit a slot of %zu (multiples of 4, 4-byte aligned)", bytes, remote->slot_bytes);
    uint8_t *b = remote->base;
    if (bytes >= (256u << 10) && bytes % 16 == 0 && ((uintptr_t)src & 15) == 0) {
        // a micro-batch: reserve, copy with a whole grid, publish
        const uint64_t lim = limit_ns ? limit_ns : 5000000000ull;
        const int slot = (int)(seqno % (uint64_t)remote->n_slots);
        cudaStream_t st = (cudaStream_t)stream;
        kq_launch(handoff_reserve_kernel, 1, 1, 0, st, (const uint64_t *)(b + remote->lay.ctrl_off), remote->known,
                  remote->send_err, seqno, remote->n_slots, lim);
        const size_t n16 = bytes / 16;
        const unsigned grid = (unsigned)std::min<size_t>((n16 + 255) / 256, (size_t)kq_sm_count() * 4);
        kq_launch(handoff_copy_kernel, grid, 256, 0, st, (const uint4 *)src, (uint4 *)(b + (size_t)slot * remote->lay.slot_stride), n16,
                  (const int *)remote->send_err);
        kq_launch(handoff_publish_kernel, 1, 1, 0, st, (uint64_t *)(b + remote->lay.flags_off) + slot, (const int *)remote->send_err, seqno);
        KQ_COUNT_LAUNCH();
        KQ_COUNT_LAUNCH();
        KQ_COUNT_LAUNCH();
        KQ_LAUNCH_CHECK();
        return B200_OK;
    }
    kq_launch(handoff_send_kernel, 1, 256, 0, (cudaStream_t)stream, (const uint4 *)src, bytes, b, remote->lay.slot_stride,
              (uint64_t *)(b + remote->lay.flags_off), (const uint64_t *)(b + remote->lay.ctrl_off), remote->known,
              remote->send_err, seqno, remote->n_slots, limit_ns ? limit_ns : 5000000000ull);
    KQ_COUNT_LAUNCH();
    KQ_LAUNCH_CHECK();
    return B200_OK;
}

b200_status b200_handoff_wait(b200_handoff *h, void *dst, size_t bytes, uint64_t seqno, uint64_t limit_ns,
                              const void **slot, void *stream) {
    KQ_REQUIRE(valid(h) && h->owned, "handoff_wait: a local endpoint is required");
    KQ_REQUIRE(bytes % 4 == 0 && bytes <= h->slot_bytes && ((uintptr_t)dst & 3) == 0, "handoff_wait: bad size or alignment");
    uint8_t *b = h->base;
    kq_launch(handoff_wait_kernel, 1, 256, 0, (cudaStream_t)stream, (uint4 *)dst, bytes, (const uint8_t *)b, h->lay.slot_stride,
              (const uint64_t *)(b + h->lay.flags_off), (uint64_t *)(b + h->lay.ctrl_off), (int *)(b + h->lay.ctrl_off + 64),
              seqno, h->n_slots, limit_ns ? limit_ns : 5000000000ull);
    KQ_COUNT_LAUNCH();
    KQ_LAUNCH_CHECK();
    if (slot) *slot = b + (size_t)(seqno % (uint64_t)h->n_slots) * h->lay.slot_stride;
    return B200_OK;
}

b200_status b200_handoff_release(b200_handoff *h, uint64_t seqno, void *stream) {
    KQ_REQUIRE(valid(h) && h->owned, "handoff_release: a local endpoint is required");
    kq_launch(handoff_release_kernel, 1, 1, 0, (cudaStream_t)stream, (uint64_t *)(h->base + h->lay.ctrl_off), seqno);
    KQ_COUNT_LAUNCH();
    KQ_LAUNCH_CHECK();
    return B200_OK;
}

b200_status b200_handoff_status(b200_handoff *h, int32_t *status) {
    KQ_REQUIRE(valid(h) && status, "handoff_status: null argument");
    int v = 0;
    const int *word = h->owned ? (const int *)(h->base + h->lay.ctrl_off + 64) : h->send_err;
    KQ_CUDA(cudaMemcpy(&v, word, sizeof(int), cudaMemcpyDeviceToHost)); // orders after the default stream's work
    *status = v;
    return B200_OK;
}

void b200_handoff_free(b200_handoff *h) {
    if (!valid(h)) return;
    if (h->owned) {
        if (h->base) cudaFree(h->base);
    } else {
        if (h->ipc && h->base) cudaIpcCloseMemHandle(h->base);
        if (h->known) cudaFree(h->known);
    }
    h->magic = 0;
    delete h;
}

} // extern "C"
