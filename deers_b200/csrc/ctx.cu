// Context, buffers, copies, status strings and argument validation of the
// deers_b200 C ABI.  The attention entry points validate here and dispatch to the
// f32 (FFMA) or f16 (tcgen05) kernel files; there is no CPU fallback.
#include "common.cuh"

#include <new>
#include <queue>
#include <vector>

static const char* kStatus[] = {
    "ok",
    "null pointer argument",
    "unsupported shape",
    "unsupported dtype",
    "layout not accepted (inner stride must be 1, rows 16-byte aligned): compact and retry",
    "workspace missing or too small",
    "CUDA call failed",
    "kernel gave up on a bounded wait",
    "no kernel for this request",
    "device is not sm_100",
};

extern "C" const char* deers_b200_status_string(int status) {
    if (status < 0 || status > DEERS_ERR_DEVICE) return "unknown status";
    return kStatus[status];
}

extern "C" const char* deers_b200_last_error(deers_ctx* ctx) { return ctx ? ctx->last_error : ""; }

extern "C" uint64_t deers_b200_launch_count(deers_ctx* ctx) { return ctx ? ctx->launches : 0; }

extern "C" void deers_b200_attn_desc_compact(deers_attn_desc* d, int32_t B, int32_t H, int32_t T,
                                             int32_t D, int32_t dtype, int32_t causal, float scale) {
    if (!d) return;
    d->B = B; d->H = H; d->T = T; d->D = D;
    d->dtype = dtype; d->causal = causal; d->scale = scale;
    const int64_t s[4] = {(int64_t)H * T * D, (int64_t)T * D, (int64_t)D, 1};
    int64_t* all[8] = {d->q_strides, d->k_strides, d->v_strides, d->o_strides,
                       d->do_strides, d->dq_strides, d->dk_strides, d->dv_strides};
    for (int t = 0; t < 8; ++t)
        for (int i = 0; i < 4; ++i) all[t][i] = s[i];
}

extern "C" int deers_b200_init(int device_ordinal, void* stream, deers_ctx** out) {
    if (!out) return DEERS_ERR_NULL;
    *out = nullptr;
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || device_ordinal < 0 || device_ordinal >= count)
        return DEERS_ERR_CUDA;
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, device_ordinal) != cudaSuccess) return DEERS_ERR_CUDA;
    if (prop.major != 10) return DEERS_ERR_DEVICE;
    if (cudaSetDevice(device_ordinal) != cudaSuccess) return DEERS_ERR_CUDA;

    deers_ctx* ctx = new (std::nothrow) deers_ctx();
    if (!ctx) return DEERS_ERR_CUDA;
    memset(ctx, 0, sizeof(*ctx));
    ctx->device = device_ordinal;
    ctx->sm_count = prop.multiProcessorCount;
    if (stream) {
        ctx->stream = (cudaStream_t)stream;
        ctx->owns_stream = false;
    } else {
        if (cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking) != cudaSuccess) {
            delete ctx;
            return DEERS_ERR_CUDA;
        }
        ctx->owns_stream = true;
    }
    // The error word lives in device memory (every CTA reads it once at start-up; a
    // host-mapped word would cost each of them a PCIe round trip) with a pinned host
    // mirror that sync() refreshes.
    if (cudaHostAlloc((void**)&ctx->host_err, sizeof(unsigned int), cudaHostAllocDefault) != cudaSuccess ||
        cudaMalloc((void**)&ctx->dev_err, sizeof(unsigned int)) != cudaSuccess ||
        cudaMemset(ctx->dev_err, 0, sizeof(unsigned int)) != cudaSuccess) {
        if (ctx->owns_stream) cudaStreamDestroy(ctx->stream);
        if (ctx->host_err) cudaFreeHost(ctx->host_err);
        delete ctx;
        return DEERS_ERR_CUDA;
    }
    *ctx->host_err = 0;
    for (int e = 0; e < DEERS_SCHED_ENTRIES; ++e) {
        deers_sched_entry* se = &ctx->sched[e];
        se->key[0] = -1;
        if (cudaMalloc((void**)&se->dev, sizeof(int) * DEERS_SCHED_CAP) != cudaSuccess ||
            cudaHostAlloc((void**)&se->host, sizeof(int) * DEERS_SCHED_CAP, cudaHostAllocDefault) != cudaSuccess ||
            cudaEventCreateWithFlags(&se->uploaded, cudaEventDisableTiming) != cudaSuccess) {
            cudaGetLastError();
            if (se->dev) cudaFree(se->dev);
            if (se->host) cudaFreeHost(se->host);
            se->dev = nullptr; se->host = nullptr; se->uploaded = nullptr;   // this slot stays unused
        }
    }
    cudaDriverEntryPointQueryResult qres;
    void* fn = nullptr;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess)
        fn = nullptr;
    ctx->encode_tiled = fn;
    *out = ctx;
    return DEERS_OK;
}

extern "C" void deers_b200_destroy(deers_ctx* ctx) {
    if (!ctx) return;
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    if (ctx->owns_stream) cudaStreamDestroy(ctx->stream);
    if (ctx->host_err) cudaFreeHost(ctx->host_err);
    if (ctx->dev_err) cudaFree(ctx->dev_err);
    for (int e = 0; e < DEERS_SCHED_ENTRIES; ++e) {
        if (ctx->sched[e].dev) cudaFree(ctx->sched[e].dev);
        if (ctx->sched[e].host) cudaFreeHost(ctx->sched[e].host);
        if (ctx->sched[e].uploaded) cudaEventDestroy(ctx->sched[e].uploaded);
    }
    if (ctx->pipe_ready) {
        cudaStreamDestroy(ctx->h2d_stream);
        cudaStreamDestroy(ctx->d2h_stream);
        for (int s2 = 0; s2 < 3; ++s2)
            for (int e = 0; e < 3; ++e) cudaEventDestroy(ctx->pipe_ev[s2][e]);
    }
    for (int k = 0; k < DEERS_K_COUNT; ++k) {
        deers_ktimer* t = &ctx->kt[k];
        if (t->start && t->stop)
            for (int i = 0; i < DEERS_KT_RING; ++i) { cudaEventDestroy(t->start[i]); cudaEventDestroy(t->stop[i]); }
        delete[] t->start;
        delete[] t->stop;
    }
    delete ctx;
}

extern "C" int deers_b200_set_stream(deers_ctx* ctx, void* stream) {
    if (!ctx) return DEERS_ERR_NULL;
    if (ctx->owns_stream) {
        cudaStreamSynchronize(ctx->stream);
        cudaStreamDestroy(ctx->stream);
        ctx->owns_stream = false;
    }
    ctx->stream = (cudaStream_t)stream;
    return DEERS_OK;
}

extern "C" void* deers_b200_stream(deers_ctx* ctx) { return ctx ? (void*)ctx->stream : nullptr; }

extern "C" int deers_b200_alloc(deers_ctx* ctx, size_t bytes, void** dptr) {
    if (!ctx || !dptr) return DEERS_ERR_NULL;
    DEERS_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    DEERS_CUDA_TRY(ctx, cudaMallocAsync(dptr, bytes ? bytes : 1, ctx->stream));
    return DEERS_OK;
}

extern "C" int deers_b200_free(deers_ctx* ctx, void* dptr) {
    if (!ctx) return DEERS_ERR_NULL;
    if (!dptr) return DEERS_OK;
    DEERS_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    DEERS_CUDA_TRY(ctx, cudaFreeAsync(dptr, ctx->stream));
    return DEERS_OK;
}

extern "C" int deers_b200_mem_info(deers_ctx* ctx, size_t* free_bytes, size_t* total_bytes) {
    if (!ctx || !free_bytes || !total_bytes) return DEERS_ERR_NULL;
    DEERS_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    DEERS_CUDA_TRY(ctx, cudaMemGetInfo(free_bytes, total_bytes));
    return DEERS_OK;
}

extern "C" int deers_b200_memcpy_h2d(deers_ctx* ctx, void* dst, const void* src, size_t bytes) {
    if (!ctx || (bytes && (!dst || !src))) return DEERS_ERR_NULL;
    DEERS_CUDA_TRY(ctx, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, ctx->stream));
    return DEERS_OK;
}

extern "C" int deers_b200_memcpy_d2h(deers_ctx* ctx, void* dst, const void* src, size_t bytes) {
    if (!ctx || (bytes && (!dst || !src))) return DEERS_ERR_NULL;
    DEERS_CUDA_TRY(ctx, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, ctx->stream));
    DEERS_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
    return DEERS_OK;
}

extern "C" int deers_b200_memcpy_d2d(deers_ctx* ctx, void* dst, const void* src, size_t bytes) {
    if (!ctx || (bytes && (!dst || !src))) return DEERS_ERR_NULL;
    DEERS_CUDA_TRY(ctx, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, ctx->stream));
    return DEERS_OK;
}

extern "C" int deers_b200_sync(deers_ctx* ctx) {
    if (!ctx) return DEERS_ERR_NULL;
    DEERS_CUDA_TRY(ctx, cudaMemcpyAsync(ctx->host_err, ctx->dev_err, sizeof(unsigned int), cudaMemcpyDeviceToHost,
                                        ctx->stream));
    DEERS_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
    const unsigned int e = *(volatile unsigned int*)ctx->host_err;
    if (e != 0) {
        *(volatile unsigned int*)ctx->host_err = 0;
        DEERS_CUDA_TRY(ctx, cudaMemsetAsync(ctx->dev_err, 0, sizeof(unsigned int), ctx->stream));
        snprintf(ctx->last_error, sizeof(ctx->last_error),
                 "kernel error word 0x%x (kernel family 0x%x, wait id %u)", e, e & 0xf00u, e & 0xffu);
        return DEERS_ERR_KERNEL;
    }
    return DEERS_OK;
}

// ---------------------------------------------------------------------------
// Work schedule of the persistent kernels
// ---------------------------------------------------------------------------
const int4* deers_get_schedule(deers_ctx* ctx, int B, int H, int ntile, int causal, int grid, int* rows) {
    *rows = 0;
    const long long n_items = (long long)B * H * ntile;
    if (grid < 1 || n_items < 1) return nullptr;
    const int key[5] = {B, H, ntile, causal, grid};
    deers_sched_entry* victim = nullptr;
    for (int e = 0; e < DEERS_SCHED_ENTRIES; ++e) {
        deers_sched_entry* se = &ctx->sched[e];
        if (!se->dev) continue;
        if (se->key[0] >= 0 && memcmp(key, se->key, sizeof(key)) == 0) {
            se->last_use = ++ctx->sched_clock;
            *rows = se->rows;
            return se->rows > 0 ? reinterpret_cast<const int4*>(se->dev) : nullptr;
        }
        if (!victim || se->key[0] < 0 || (victim->key[0] >= 0 && se->last_use < victim->last_use)) victim = se;
    }
    if (!victim) return nullptr;
    // A miss while the stream is being captured takes the plain strided assignment: the upload would become a
    // graph node that re-reads the staging copy at every replay.
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(ctx->stream, &cap) != cudaSuccess || cap != cudaStreamCaptureStatusNone) {
        cudaGetLastError();
        return nullptr;
    }
    // Greedy list scheduling in item order: each item goes to the CTA with the least work so far.
    std::vector<std::vector<int>> lists(grid);
    typedef std::pair<long long, int> Load;                            // (work so far, cta)
    std::priority_queue<Load, std::vector<Load>, std::greater<Load>> heap;
    for (int c = 0; c < grid; ++c) heap.push(Load(0, c));
    const int BH = B * H;
    for (long long w = 0; w < n_items; ++w) {
        const int group = (int)(w / (16LL * ntile));
        const int gsize = BH - group * 16 < 16 ? BH - group * 16 : 16;
        const int slot = (int)((w - (long long)group * 16 * ntile) / gsize);
        const long long weight = (causal ? ntile - slot : ntile) + 1;  // +1: per-item start-up and epilogue
        Load l = heap.top();
        heap.pop();
        lists[l.second].push_back((int)w);
        heap.push(Load(l.first + weight, l.second));
    }
    size_t nrows = 0;
    for (auto& v : lists) nrows = v.size() > nrows ? v.size() : nrows;
    memcpy(victim->key, key, sizeof(key));
    victim->last_use = ++ctx->sched_clock;
    victim->rows = 0;
    if (nrows * (size_t)grid * 4 > (size_t)DEERS_SCHED_CAP) return nullptr;   // cached as "no table": strided assignment
    // The staging copy of this slot may still be the source of an earlier upload: wait for that one copy.
    if (cudaEventSynchronize(victim->uploaded) != cudaSuccess) { cudaGetLastError(); victim->key[0] = -1; return nullptr; }
    // Entry = {slot, slice, batch, head}: the kernels' single issuing threads would otherwise spend about a
    // thousand cycles per item on the integer divisions that turn an item index into these.
    int4* table = reinterpret_cast<int4*>(victim->host);
    for (size_t i = 0; i < nrows * grid; ++i) table[i] = make_int4(-1, 0, 0, 0);
    for (int c = 0; c < grid; ++c)
        for (size_t n = 0; n < lists[c].size(); ++n) {
            const long long w = lists[c][n];
            const int group = (int)(w / (16LL * ntile));
            const int gsize = BH - group * 16 < 16 ? BH - group * 16 : 16;
            const int within = (int)(w - (long long)group * 16 * ntile);
            const int bh = group * 16 + within % gsize;
            table[n * grid + c] = make_int4(within / gsize, bh, bh / H, bh % H);
        }
    if (cudaMemcpyAsync(victim->dev, victim->host, nrows * grid * sizeof(int4), cudaMemcpyHostToDevice, ctx->stream) !=
            cudaSuccess ||
        cudaEventRecord(victim->uploaded, ctx->stream) != cudaSuccess) {
        cudaGetLastError();
        victim->key[0] = -1;
        return nullptr;
    }
    victim->rows = (int)nrows;
    *rows = victim->rows;
    return reinterpret_cast<const int4*>(victim->dev);
}

// ---------------------------------------------------------------------------
// Validation shared by forward and backward
// ---------------------------------------------------------------------------
int deers_check_tensor(const deers_attn_desc* d, const void* p, const int64_t* s, size_t esize) {
    if (!p) return DEERS_ERR_NULL;
    if (s[3] != 1) return DEERS_ERR_LAYOUT;
    // f16 (TMA) needs 16-byte aligned bases and row starts; the f32 kernels fall
    // back to scalar loads when a row is not 16-byte aligned, so 4 bytes suffice.
    const uintptr_t mask = (esize == 2) ? 15u : 3u;
    if (((uintptr_t)p & mask) != 0) return DEERS_ERR_LAYOUT;
    for (int i = 0; i < 3; ++i) {
        if (s[i] < 0) return DEERS_ERR_LAYOUT;
        const int64_t extent = (i == 0) ? d->B : (i == 1) ? d->H : d->T;
        if (extent > 1 && ((s[i] * (int64_t)esize) & (int64_t)mask) != 0) return DEERS_ERR_LAYOUT;
    }
    return DEERS_OK;
}

int deers_check_desc(const deers_attn_desc* d) {
    if (!d) return DEERS_ERR_NULL;
    if (d->dtype != DEERS_F16 && d->dtype != DEERS_F32) return DEERS_ERR_DTYPE;
    if (d->B < 1 || d->H < 1 || d->T < 1 || d->D < 1) return DEERS_ERR_SHAPE;
    if ((int64_t)d->B * d->H > 0x7fffffffLL / 64) return DEERS_ERR_SHAPE;
    if (d->T > (1 << 20)) return DEERS_ERR_SHAPE;
    if (d->dtype == DEERS_F32) {
        if (d->D > 128) return DEERS_ERR_SHAPE;
    } else {
        // tcgen05 tile shapes are 64 and 128; other multiples of 8 run zero-padded to the next of the two
        if (d->D > 128 || d->D % 8 != 0) return DEERS_ERR_SHAPE;
    }
    if (!(d->scale == d->scale)) return DEERS_ERR_SHAPE;
    return DEERS_OK;
}

// Everything deers_b200_attn_bwd and deers_b200_attn_bwd_f16_static check before looking at scratch memory.
int deers_check_bwd_args(const deers_attn_desc* d, const void* q, const void* k, const void* v, const void* o,
                         const float* lse, const void* d_o, void* dq, void* dk, void* dv) {
    int rc = deers_check_desc(d);
    if (rc) return rc;
    if (!lse) return DEERS_ERR_NULL;
    const size_t es = d->dtype == DEERS_F16 ? 2 : 4;
    if ((rc = deers_check_tensor(d, q, d->q_strides, es))) return rc;
    if ((rc = deers_check_tensor(d, k, d->k_strides, es))) return rc;
    if ((rc = deers_check_tensor(d, v, d->v_strides, es))) return rc;
    if ((rc = deers_check_tensor(d, o, d->o_strides, es))) return rc;
    if ((rc = deers_check_tensor(d, d_o, d->do_strides, es))) return rc;
    if ((rc = deers_check_tensor(d, dq, d->dq_strides, es))) return rc;
    if ((rc = deers_check_tensor(d, dk, d->dk_strides, es))) return rc;
    if ((rc = deers_check_tensor(d, dv, d->dv_strides, es))) return rc;
    return DEERS_OK;
}

static size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

static size_t delta_bytes(const deers_attn_desc* d) {
    return align_up((size_t)d->B * d->H * d->T * sizeof(float), 256);
}

// ---------------------------------------------------------------------------
// f16 head dims other than 64 / 128 (the reference derives head_dim = n_embd / n_head freely,
// src/models/gpt.rs:86-100): operands are copied into dense [B,H,T,Dp] buffers, Dp = 64 or 128, with zero
// columns behind D (zero columns change neither Q K^T nor P V), the native kernels run on those, and the first D
// columns of the results are copied back.  A compatibility path: it costs one extra pass over every tensor.
// ---------------------------------------------------------------------------
static int padded_dim(const deers_attn_desc* d) { return d->D <= 64 ? 64 : 128; }
static bool needs_pad(const deers_attn_desc* d) { return d->dtype == DEERS_F16 && d->D != 64 && d->D != 128; }
static size_t padded_tensor_bytes(const deers_attn_desc* d) {
    return align_up((size_t)d->B * d->H * d->T * padded_dim(d) * 2, 256);
}
static deers_attn_desc padded_desc(const deers_attn_desc* d) {
    deers_attn_desc p = *d;
    p.D = padded_dim(d);
    const int64_t s[4] = {(int64_t)d->H * d->T * p.D, (int64_t)d->T * p.D, p.D, 1};
    for (int i = 0; i < 4; ++i) {
        p.q_strides[i] = p.k_strides[i] = p.v_strides[i] = p.o_strides[i] = p.do_strides[i] = s[i];
        p.dq_strides[i] = p.dk_strides[i] = p.dv_strides[i] = s[i];
    }
    return p;
}

// One thread per 16-byte piece (8 halves) of a padded row.  TO_PADDED: strided [.., D] -> dense [.., DP] with
// zero fill; otherwise dense [.., DP] -> strided [.., D].
template <bool TO_PADDED>
__global__ void __launch_bounds__(256) pad_rows_f16_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, int H, int T,
                                                           int D8, int DP8, long long sb, long long sh, long long st,
                                                           long long rows) {
    const long long total = rows * DP8;
    for (long long i = (long long)blockIdx.x * 256 + threadIdx.x; i < total; i += (long long)gridDim.x * 256) {
        const long long row = i / DP8;
        const int c = (int)(i % DP8);
        const long long t = row % T, h = (row / T) % H, b = row / ((long long)T * H);
        const long long strided = (b * sb + h * sh + t * st) / 8 + c;         // strides are multiples of 8 halves
        if (TO_PADDED) dst[i] = c < D8 ? src[strided] : make_uint4(0u, 0u, 0u, 0u);
        else if (c < D8) dst[strided] = src[i];
    }
}

static int pad_copy(deers_ctx* ctx, const deers_attn_desc* d, const void* strided, const int64_t* s, void* dense, bool to_padded) {
    const long long rows = (long long)d->B * d->H * d->T;
    const int D8 = d->D / 8, DP8 = padded_dim(d) / 8;
    long long want = (rows * DP8 + 255) / 256;
    const long long cap = 32LL * ctx->sm_count;
    const unsigned grid = (unsigned)(want < cap ? want : cap);
    if (to_padded)
        pad_rows_f16_kernel<true><<<grid, 256, 0, ctx->stream>>>((const uint4*)strided, (uint4*)dense, d->H, d->T, D8, DP8, s[0], s[1], s[2], rows);
    else
        pad_rows_f16_kernel<false><<<grid, 256, 0, ctx->stream>>>((const uint4*)dense, (uint4*)const_cast<void*>(strided), d->H, d->T, D8, DP8, s[0], s[1], s[2], rows);
    ctx->launches += 1;
    DEERS_CUDA_TRY(ctx, cudaGetLastError());
    return DEERS_OK;
}

extern "C" size_t deers_b200_attn_workspace_bytes(const deers_attn_desc* d, int pass) {
    if (deers_check_desc(d) != DEERS_OK) return 0;
    if (needs_pad(d)) {
        // pass 0: Q, K, V, O padded; passes 1, 2: the eight padded tensors of the backward + its own workspace
        const deers_attn_desc p = padded_desc(d);
        if (pass == 0) return 4 * padded_tensor_bytes(d);
        return 8 * padded_tensor_bytes(d) + align_up(attn_bwd_f16_workspace_bytes(&p, pass >= 2), 256);
    }
    if (pass == 0) return 0;
    // pass 1: the least the backward needs; pass 2: what lets the f16 backward keep its dS tiles
    return d->dtype == DEERS_F16 ? attn_bwd_f16_workspace_bytes(d, pass >= 2) : delta_bytes(d);
}

extern "C" int deers_b200_attn_fwd(deers_ctx* ctx, const deers_attn_desc* d, const void* q,
                                   const void* k, const void* v, void* o, float* lse, void* workspace,
                                   size_t workspace_bytes) {
    if (!ctx) return DEERS_ERR_NULL;
    int rc = deers_check_desc(d);
    if (rc) return rc;
    if (!lse) return DEERS_ERR_NULL;
    const size_t es = d->dtype == DEERS_F16 ? 2 : 4;
    if ((rc = deers_check_tensor(d, q, d->q_strides, es))) return rc;
    if ((rc = deers_check_tensor(d, k, d->k_strides, es))) return rc;
    if ((rc = deers_check_tensor(d, v, d->v_strides, es))) return rc;
    if ((rc = deers_check_tensor(d, o, d->o_strides, es))) return rc;
    DEERS_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    if (d->dtype == DEERS_F32)
        return launch_attn_fwd_f32(ctx, d, (const float*)q, (const float*)k, (const float*)v, (float*)o, lse);
    if (needs_pad(d)) {
        const size_t tb = padded_tensor_bytes(d);
        if (!workspace || workspace_bytes < 4 * tb || ((uintptr_t)workspace & 255u) != 0) return DEERS_ERR_WORKSPACE;
        char* w = (char*)workspace;
        const deers_attn_desc p = padded_desc(d);
        if ((rc = pad_copy(ctx, d, q, d->q_strides, w, true))) return rc;
        if ((rc = pad_copy(ctx, d, k, d->k_strides, w + tb, true))) return rc;
        if ((rc = pad_copy(ctx, d, v, d->v_strides, w + 2 * tb, true))) return rc;
        if ((rc = launch_attn_fwd_f16(ctx, &p, w, w + tb, w + 2 * tb, w + 3 * tb, lse))) return rc;
        return pad_copy(ctx, d, o, d->o_strides, w + 3 * tb, false);
    }
    return launch_attn_fwd_f16(ctx, d, q, k, v, o, lse);
}

extern "C" int deers_b200_attn_bwd(deers_ctx* ctx, const deers_attn_desc* d, const void* q,
                                   const void* k, const void* v, const void* o, const float* lse,
                                   const void* d_o, void* dq, void* dk, void* dv, void* workspace,
                                   size_t workspace_bytes) {
    if (!ctx) return DEERS_ERR_NULL;
    int rc = deers_check_bwd_args(d, q, k, v, o, lse, d_o, dq, dk, dv);
    if (rc) return rc;
    const size_t need = deers_b200_attn_workspace_bytes(d, 1);
    if (!workspace || workspace_bytes < need || ((uintptr_t)workspace & 255u) != 0)
        return DEERS_ERR_WORKSPACE;
    DEERS_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    if (d->dtype == DEERS_F32)
        return launch_attn_bwd_f32(ctx, d, (const float*)q, (const float*)k, (const float*)v,
                                   (const float*)o, lse, (const float*)d_o, (float*)dq, (float*)dk,
                                   (float*)dv, (float*)workspace);
    const bool keep_ds = workspace_bytes >= deers_b200_attn_workspace_bytes(d, 2);
    if (needs_pad(d)) {
        const size_t tb = padded_tensor_bytes(d);
        char* w = (char*)workspace;
        const deers_attn_desc p = padded_desc(d);
        const void* in[5] = {q, k, v, o, d_o};
        const int64_t* in_s[5] = {d->q_strides, d->k_strides, d->v_strides, d->o_strides, d->do_strides};
        for (int i = 0; i < 5; ++i)
            if ((rc = pad_copy(ctx, d, in[i], in_s[i], w + i * tb, true))) return rc;
        if ((rc = launch_attn_bwd_f16(ctx, &p, w, w + tb, w + 2 * tb, w + 3 * tb, lse, w + 4 * tb, w + 5 * tb, w + 6 * tb,
                                      w + 7 * tb, w + 8 * tb, keep_ds)))
            return rc;
        void* out[3] = {dq, dk, dv};
        const int64_t* out_s[3] = {d->dq_strides, d->dk_strides, d->dv_strides};
        for (int i = 0; i < 3; ++i)
            if ((rc = pad_copy(ctx, d, out[i], out_s[i], w + (5 + i) * tb, false))) return rc;
        return DEERS_OK;
    }
    return launch_attn_bwd_f16(ctx, d, q, k, v, o, lse, d_o, dq, dk, dv, workspace, keep_ds);
}

static int drain_timer(deers_ctx* ctx, deers_ktimer* t) {
    for (int i = 0; i < t->pending; ++i) {
        float ms = 0.f;
        DEERS_CUDA_TRY(ctx, cudaEventElapsedTime(&ms, t->start[i], t->stop[i]));
        t->total_ms += ms;
        t->launches += 1;
    }
    t->pending = 0;
    return DEERS_OK;
}

extern "C" int deers_b200_kernel_timing(deers_ctx* ctx, int enable) {
    if (!ctx) return DEERS_ERR_NULL;
    DEERS_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    if (enable) {
        for (int k = 0; k < DEERS_K_COUNT; ++k) {
            deers_ktimer* t = &ctx->kt[k];
            if (!t->start) {
                t->start = new (std::nothrow) cudaEvent_t[DEERS_KT_RING];
                t->stop = new (std::nothrow) cudaEvent_t[DEERS_KT_RING];
                if (!t->start || !t->stop) return DEERS_ERR_CUDA;
                for (int i = 0; i < DEERS_KT_RING; ++i) {
                    DEERS_CUDA_TRY(ctx, cudaEventCreate(&t->start[i]));
                    DEERS_CUDA_TRY(ctx, cudaEventCreate(&t->stop[i]));
                }
            }
            t->pending = 0; t->total_ms = 0.0; t->launches = 0;
        }
    }
    ctx->timing = enable != 0;
    return DEERS_OK;
}

extern "C" int deers_b200_kernel_time(deers_ctx* ctx, int kind, int reset, double* total_ms, uint64_t* launches) {
    if (!ctx || !total_ms || !launches) return DEERS_ERR_NULL;
    if (kind < 0 || kind >= DEERS_K_COUNT) return DEERS_ERR_SHAPE;
    DEERS_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
    deers_ktimer* t = &ctx->kt[kind];
    int rc = drain_timer(ctx, t);
    if (rc) return rc;
    *total_ms = t->total_ms;
    *launches = t->launches;
    if (reset) { t->total_ms = 0.0; t->launches = 0; }
    return DEERS_OK;
}

// ---------------------------------------------------------------------------
// Host-tensor pipeline
// ---------------------------------------------------------------------------
namespace {
constexpr int kPipeSets = 3;

struct ChunkLayout {
    size_t tensor_bytes;    // one [chunk, T, D] tensor
    size_t lse_bytes;
    size_t ws_bytes;
    size_t set_bytes;       // 8 tensors + lse + workspace, each 256-byte aligned
};

ChunkLayout chunk_layout(const deers_attn_desc* d, int chunk) {
    ChunkLayout l;
    const size_t es = d->dtype == DEERS_F16 ? 2 : 4;
    l.tensor_bytes = align_up((size_t)chunk * d->T * d->D * es, 256);
    l.lse_bytes = align_up((size_t)chunk * d->T * sizeof(float), 256);
    deers_attn_desc c;
    deers_b200_attn_desc_compact(&c, chunk, 1, d->T, d->D, d->dtype, d->causal, d->scale);
    l.ws_bytes = align_up(deers_b200_attn_workspace_bytes(&c, 1), 256);
    l.set_bytes = 8 * l.tensor_bytes + l.lse_bytes + l.ws_bytes;
    return l;
}
}  // namespace

extern "C" size_t deers_b200_attn_host_scratch_bytes(const deers_attn_desc* d, int chunk_slices) {
    if (deers_check_desc(d) != DEERS_OK || chunk_slices < 1) return 0;
    return kPipeSets * chunk_layout(d, chunk_slices).set_bytes;
}

extern "C" int deers_b200_attn_fwd_bwd_host(deers_ctx* ctx, const deers_attn_desc* d, const void* q_host,
                                            const void* k_host, const void* v_host, const void* do_host, void* o_host,
                                            float* lse_host, void* dq_host, void* dk_host, void* dv_host,
                                            int chunk_slices, void* device_scratch, size_t scratch_bytes) {
    if (!ctx || !q_host || !k_host || !v_host || !do_host || !o_host || !dq_host || !dk_host || !dv_host) return DEERS_ERR_NULL;
    int rc = deers_check_desc(d);
    if (rc) return rc;
    if (needs_pad(d)) return DEERS_ERR_UNSUPPORTED;                   // f16 head dims other than 64 / 128: device calls only
    if (chunk_slices < 1) return DEERS_ERR_SHAPE;
    const size_t need = deers_b200_attn_host_scratch_bytes(d, chunk_slices);
    if (!device_scratch || scratch_bytes < need || ((uintptr_t)device_scratch & 255u) != 0) return DEERS_ERR_WORKSPACE;
    DEERS_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    if (!ctx->pipe_ready) {
        DEERS_CUDA_TRY(ctx, cudaStreamCreateWithFlags(&ctx->h2d_stream, cudaStreamNonBlocking));
        DEERS_CUDA_TRY(ctx, cudaStreamCreateWithFlags(&ctx->d2h_stream, cudaStreamNonBlocking));
        for (int s = 0; s < kPipeSets; ++s)
            for (int e = 0; e < 3; ++e) DEERS_CUDA_TRY(ctx, cudaEventCreateWithFlags(&ctx->pipe_ev[s][e], cudaEventDisableTiming));
        ctx->pipe_ready = true;
    }
    const ChunkLayout l = chunk_layout(d, chunk_slices);
    const size_t es = d->dtype == DEERS_F16 ? 2 : 4;
    const long long n_slices = (long long)d->B * d->H;
    const size_t slice_bytes = (size_t)d->T * d->D * es;
    const void* in_host[4] = {q_host, k_host, v_host, do_host};
    void* out_host[4] = {o_host, dq_host, dk_host, dv_host};

    // Inputs already on the context's stream (e.g. earlier work of the caller) come first.
    cudaEvent_t start = ctx->pipe_ev[0][2];
    DEERS_CUDA_TRY(ctx, cudaEventRecord(start, ctx->stream));
    DEERS_CUDA_TRY(ctx, cudaStreamWaitEvent(ctx->h2d_stream, start, 0));

    int chunk_idx = 0;
    for (long long s0 = 0; s0 < n_slices; s0 += chunk_slices, ++chunk_idx) {
        const int n = (int)((n_slices - s0) < chunk_slices ? (n_slices - s0) : chunk_slices);
        const int set = chunk_idx % kPipeSets;
        char* base = (char*)device_scratch + (size_t)set * l.set_bytes;
        void* dev[8];
        for (int t = 0; t < 8; ++t) dev[t] = base + (size_t)t * l.tensor_bytes;        // q k v do | o dq dk dv
        float* lse_dev = (float*)(base + 8 * l.tensor_bytes);
        void* ws = base + 8 * l.tensor_bytes + l.lse_bytes;
        cudaEvent_t h2d_done = ctx->pipe_ev[set][0], comp_done = ctx->pipe_ev[set][1], d2h_done = ctx->pipe_ev[set][2];

        // This buffer set was last used kPipeSets chunks ago: its results must have left the device.
        if (chunk_idx >= kPipeSets) DEERS_CUDA_TRY(ctx, cudaStreamWaitEvent(ctx->h2d_stream, d2h_done, 0));
        for (int t = 0; t < 4; ++t)
            DEERS_CUDA_TRY(ctx, cudaMemcpyAsync(dev[t], (const char*)in_host[t] + (size_t)s0 * slice_bytes,
                                                (size_t)n * slice_bytes, cudaMemcpyHostToDevice, ctx->h2d_stream));
        DEERS_CUDA_TRY(ctx, cudaEventRecord(h2d_done, ctx->h2d_stream));

        DEERS_CUDA_TRY(ctx, cudaStreamWaitEvent(ctx->stream, h2d_done, 0));
        deers_attn_desc c;
        deers_b200_attn_desc_compact(&c, n, 1, d->T, d->D, d->dtype, d->causal, d->scale);
        if ((rc = deers_b200_attn_fwd(ctx, &c, dev[0], dev[1], dev[2], dev[4], lse_dev, nullptr, 0))) return rc;
        if ((rc = deers_b200_attn_bwd(ctx, &c, dev[0], dev[1], dev[2], dev[4], lse_dev, dev[3], dev[5], dev[6], dev[7], ws,
                                      l.ws_bytes)))
            return rc;
        DEERS_CUDA_TRY(ctx, cudaEventRecord(comp_done, ctx->stream));

        DEERS_CUDA_TRY(ctx, cudaStreamWaitEvent(ctx->d2h_stream, comp_done, 0));
        for (int t = 0; t < 4; ++t)
            DEERS_CUDA_TRY(ctx, cudaMemcpyAsync((char*)out_host[t] + (size_t)s0 * slice_bytes, dev[4 + t],
                                                (size_t)n * slice_bytes, cudaMemcpyDeviceToHost, ctx->d2h_stream));
        if (lse_host)
            DEERS_CUDA_TRY(ctx, cudaMemcpyAsync(lse_host + (size_t)s0 * d->T, lse_dev, (size_t)n * d->T * sizeof(float),
                                                cudaMemcpyDeviceToHost, ctx->d2h_stream));
        DEERS_CUDA_TRY(ctx, cudaEventRecord(d2h_done, ctx->d2h_stream));
    }
    DEERS_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->d2h_stream));
    return deers_b200_sync(ctx);
}

extern "C" int deers_b200_selftest_umma(deers_ctx* ctx, float* max_abs_err) {
    if (!ctx || !max_abs_err) return DEERS_ERR_NULL;
    DEERS_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    return run_selftest_umma(ctx, max_abs_err);
}

extern "C" int deers_b200_selftest_wait(deers_ctx* ctx, uint32_t limit_ms, int32_t* result) {
    if (!ctx || !result) return DEERS_ERR_NULL;
    if (limit_ms < 1 || limit_ms > 1000) return DEERS_ERR_SHAPE;
    DEERS_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    return run_selftest_wait(ctx, limit_ms, result);
}
