// (batch x head) sharding across the GPUs of one box and the all-gather of O, without taking SMs.
//
// The attention path shards by independent (b, h) slices (src/models/gpt.rs:139-144 is batched over the
// two leading axes), so forward and backward need no exchange.  The one collective is for callers that
// want the whole O on every GPU.  Every rank owns a full-size [B*H, T, D] buffer; its forward writes its
// own slices in place, and the gather PUSHES that byte range into the same range of every peer's buffer
// with plain device-to-device copies over NVLink, ordered after the forward by an event; by default one push
// at a time, in a rotation in which no two ranks send to the same GPU (4 GPUs: a step with the gather beside
// it took 2.76 ms with one push in flight, 3.06 with two, 3.10 with all three), deers_b200_comm_set_lanes
// changes that.  Copies run on the copy engines: unlike a library all-gather they launch no CTAs, so the
// persistent attention kernels of the backward (one CTA per SM) keep every SM while O travels.
// No kernel of this library ever reads a peer's memory.
//
// Two ways to learn the peers' buffers:
//   deers_b200_comm_init_all   one process drives all GPUs (the reference's single global runtime,
//                              src/storage/cuda.rs:455-462, extended by a device ordinal): peer access is
//                              enabled pairwise and the pointers are used directly;
//   deers_b200_comm_export /   one process per GPU: each rank exports a 64-byte handle of its buffer, the
//   deers_b200_comm_init_ipc   host program exchanges the handles (any transport) and every rank maps the
//                              others' buffers.
#include "common.cuh"

#include <new>

constexpr int DEERS_MAX_WORLD = 16;

struct deers_comm {
    deers_ctx* ctx;
    int rank, world;
    size_t bytes;
    char* full[DEERS_MAX_WORLD];            // every rank's buffer as seen from this process
    void* base[DEERS_MAX_WORLD];            // mapping of a peer's whole allocation (full[p] lies inside it)
    bool mapped[DEERS_MAX_WORLD];           // opened from an IPC handle: close on destroy
    cudaStream_t copy_stream[DEERS_MAX_WORLD];
    cudaEvent_t ready;                      // recorded on the compute stream when the range may leave
    cudaEvent_t sent[DEERS_MAX_WORLD];      // last push to that peer
    bool pending;
    int lanes;                              // pushes in flight at once (copy streams used), 1 .. world - 1
};

extern "C" void deers_b200_shard_range(int64_t n_slices, int32_t world, int32_t rank, int64_t* begin, int64_t* end) {
    // contiguous, near-equal ranges: the first (n mod world) ranks hold one slice more
    if (!begin || !end) return;
    if (world < 1 || rank < 0 || rank >= world || n_slices < 0) { *begin = *end = 0; return; }
    const int64_t base = n_slices / world, extra = n_slices % world;
    *begin = rank * base + (rank < extra ? rank : extra);
    *end = *begin + base + (rank < extra ? 1 : 0);
}

namespace {

int comm_new(deers_ctx* ctx, int rank, int world, size_t bytes, deers_comm** out) {
    deers_comm* c = new (std::nothrow) deers_comm();
    if (!c) return DEERS_ERR_CUDA;
    memset(c, 0, sizeof(*c));
    *out = c;                                                 // the caller destroys it even when set-up fails below
    c->ctx = ctx; c->rank = rank; c->world = world; c->bytes = bytes;
    c->lanes = 1;                                             // measured best at 4 GPUs: one push at a time
    DEERS_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    DEERS_CUDA_TRY(ctx, cudaEventCreateWithFlags(&c->ready, cudaEventDisableTiming));
    for (int p = 0; p < world; ++p) {
        if (p == rank) continue;
        DEERS_CUDA_TRY(ctx, cudaStreamCreateWithFlags(&c->copy_stream[p], cudaStreamNonBlocking));
        DEERS_CUDA_TRY(ctx, cudaEventCreateWithFlags(&c->sent[p], cudaEventDisableTiming));
    }
    return DEERS_OK;
}

}  // namespace

extern "C" void deers_b200_comm_destroy(deers_comm* c) {
    if (!c) return;
    cudaSetDevice(c->ctx->device);
    for (int p = 0; p < c->world; ++p) {
        if (c->copy_stream[p]) { cudaStreamSynchronize(c->copy_stream[p]); cudaStreamDestroy(c->copy_stream[p]); }
        if (c->sent[p]) cudaEventDestroy(c->sent[p]);
        if (c->mapped[p] && c->base[p]) cudaIpcCloseMemHandle(c->base[p]);
    }
    if (c->ready) cudaEventDestroy(c->ready);
    delete c;
}

extern "C" int deers_b200_comm_init_all(int32_t n, deers_ctx* const* ctxs, void* const* full_buffers, size_t bytes,
                                        deers_comm** out) {
    if (!ctxs || !full_buffers || !out) return DEERS_ERR_NULL;
    if (n < 1 || n > DEERS_MAX_WORLD) return DEERS_ERR_SHAPE;
    for (int r = 0; r < n; ++r) {
        out[r] = nullptr;
        if (!ctxs[r] || !full_buffers[r]) return DEERS_ERR_NULL;
    }
    for (int r = 0; r < n; ++r) {
        deers_ctx* ctx = ctxs[r];
        DEERS_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
        for (int p = 0; p < n; ++p) {
            if (p == r || ctxs[p]->device == ctx->device) continue;
            int can = 0;
            DEERS_CUDA_TRY(ctx, cudaDeviceCanAccessPeer(&can, ctx->device, ctxs[p]->device));
            if (!can) {
                snprintf(ctx->last_error, sizeof(ctx->last_error), "device %d cannot reach device %d", ctx->device,
                         ctxs[p]->device);
                return DEERS_ERR_DEVICE;
            }
            const cudaError_t e = cudaDeviceEnablePeerAccess(ctxs[p]->device, 0);
            if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled) DEERS_CUDA_TRY(ctx, e);
            cudaGetLastError();
        }
        int rc = comm_new(ctx, r, n, bytes, &out[r]);
        if (rc) return rc;
        for (int p = 0; p < n; ++p) out[r]->full[p] = (char*)full_buffers[p];
    }
    return DEERS_OK;
}

extern "C" int deers_b200_comm_export(deers_ctx* ctx, void* buffer, unsigned char* handle) {
    if (!ctx || !buffer || !handle) return DEERS_ERR_NULL;
    static_assert(sizeof(cudaIpcMemHandle_t) + sizeof(uint64_t) == DEERS_IPC_HANDLE_BYTES, "handle size");
    DEERS_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    // An IPC handle names a whole allocation; a buffer carved out of a larger one (a framework's caching
    // allocator) travels as handle + offset from the allocation's base.
    typedef CUresult (*GetRange)(CUdeviceptr*, size_t*, CUdeviceptr);
    cudaDriverEntryPointQueryResult qres;
    void* fn = nullptr;
    if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &fn, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess || !fn) {
        snprintf(ctx->last_error, sizeof(ctx->last_error), "cuMemGetAddressRange is not available");
        cudaGetLastError();
        return DEERS_ERR_CUDA;
    }
    CUdeviceptr base = 0;
    size_t span = 0;
    if (((GetRange)fn)(&base, &span, (CUdeviceptr)buffer) != CUDA_SUCCESS) {
        snprintf(ctx->last_error, sizeof(ctx->last_error), "comm_export: not a device allocation");
        return DEERS_ERR_CUDA;
    }
    cudaIpcMemHandle_t h;
    DEERS_CUDA_TRY(ctx, cudaIpcGetMemHandle(&h, (void*)base));
    const uint64_t offset = (uint64_t)((CUdeviceptr)buffer - base);
    memcpy(handle, &h, sizeof(h));
    memcpy(handle + sizeof(h), &offset, sizeof(offset));
    return DEERS_OK;
}

extern "C" int deers_b200_comm_init_ipc(deers_ctx* ctx, int32_t rank, int32_t world, void* local_buffer, size_t bytes,
                                        const unsigned char* handles, deers_comm** out) {
    if (!ctx || !local_buffer || !handles || !out) return DEERS_ERR_NULL;
    *out = nullptr;
    if (world < 1 || world > DEERS_MAX_WORLD || rank < 0 || rank >= world) return DEERS_ERR_SHAPE;
    deers_comm* c = nullptr;
    int rc = comm_new(ctx, rank, world, bytes, &c);
    if (rc) { deers_b200_comm_destroy(c); return rc; }
    c->full[rank] = (char*)local_buffer;
    for (int p = 0; p < world; ++p) {
        if (p == rank) { c->full[p] = (char*)local_buffer; continue; }
        cudaIpcMemHandle_t h;
        uint64_t offset = 0;
        memcpy(&h, handles + (size_t)p * DEERS_IPC_HANDLE_BYTES, sizeof(h));
        memcpy(&offset, handles + (size_t)p * DEERS_IPC_HANDLE_BYTES + sizeof(h), sizeof(offset));
        void* ptr = nullptr;
        const cudaError_t e = cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) {
            snprintf(ctx->last_error, sizeof(ctx->last_error), "cudaIpcOpenMemHandle(rank %d): %s", p, cudaGetErrorString(e));
            cudaGetLastError();
            deers_b200_comm_destroy(c);
            return DEERS_ERR_CUDA;
        }
        c->base[p] = ptr;
        c->full[p] = (char*)ptr + offset;
        c->mapped[p] = true;
    }
    *out = c;
    return DEERS_OK;
}

extern "C" int deers_b200_allgather_o(deers_comm* c, size_t offset, size_t bytes) {
    if (!c) return DEERS_ERR_NULL;
    if (offset > c->bytes || bytes > c->bytes - offset) return DEERS_ERR_SHAPE;
    deers_ctx* ctx = c->ctx;
    if (bytes == 0 || c->world == 1) return DEERS_OK;
    DEERS_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    DEERS_CUDA_TRY(ctx, cudaEventRecord(c->ready, ctx->stream));
    // Push i goes to peer rank + i (every rank starts with a different peer, and in step i of a rotation no
    // two ranks send to the same GPU).  The pushes are dealt round-robin onto `lanes` streams: with one lane
    // they leave one after the other, each with the whole link; with world - 1 lanes all at once.
    for (int i = 1; i < c->world; ++i) {
        const int p = (c->rank + i) % c->world;
        const int lane_peer = (c->rank + 1 + (i - 1) % c->lanes) % c->world;      // the stream of the lane's first peer
        cudaStream_t st = c->copy_stream[lane_peer];
        if (i <= c->lanes) DEERS_CUDA_TRY(ctx, cudaStreamWaitEvent(st, c->ready, 0));
        DEERS_CUDA_TRY(ctx, cudaMemcpyAsync(c->full[p] + offset, c->full[c->rank] + offset, bytes, cudaMemcpyDefault, st));
        DEERS_CUDA_TRY(ctx, cudaEventRecord(c->sent[p], st));
    }
    c->pending = true;
    return DEERS_OK;
}

extern "C" int deers_b200_comm_set_lanes(deers_comm* c, int lanes) {
    if (!c) return DEERS_ERR_NULL;
    if (lanes < 1) return DEERS_ERR_SHAPE;
    if (c->world > 1 && lanes > c->world - 1) lanes = c->world - 1;
    if (c->pending) {
        const int rc = deers_b200_allgather_flush(c);             // no push may change streams in mid-flight
        if (rc) return rc;
    }
    c->lanes = c->world > 1 ? lanes : 1;
    return DEERS_OK;
}

extern "C" int deers_b200_allgather_join(deers_comm* c) {
    if (!c) return DEERS_ERR_NULL;
    if (!c->pending) return DEERS_OK;
    deers_ctx* ctx = c->ctx;
    DEERS_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    for (int p = 0; p < c->world; ++p)
        if (p != c->rank) DEERS_CUDA_TRY(ctx, cudaStreamWaitEvent(ctx->stream, c->sent[p], 0));
    c->pending = false;
    return DEERS_OK;
}

extern "C" int deers_b200_allgather_flush(deers_comm* c) {
    if (!c) return DEERS_ERR_NULL;
    deers_ctx* ctx = c->ctx;
    DEERS_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    for (int p = 0; p < c->world; ++p)
        if (p != c->rank && c->copy_stream[p]) DEERS_CUDA_TRY(ctx, cudaStreamSynchronize(c->copy_stream[p]));
    return DEERS_OK;
}
