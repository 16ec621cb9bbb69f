// Shared internals of the deers_b200 library: the context object, status helpers
// and the launch prototypes each kernel file exports to the C-ABI layer.
#pragma once
#include <cuda_runtime.h>
#include <cuda.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include "../../include/deers_b200.h"

constexpr int DEERS_KT_RING = 512;

struct deers_ktimer {
    cudaEvent_t* start;     // DEERS_KT_RING events each, created when timing is first enabled
    cudaEvent_t* stop;
    int pending;            // recorded pairs not yet folded into total_ms
    double total_ms;
    uint64_t launches;
};

constexpr int DEERS_SCHED_CAP = 1 << 20;                 // ints per schedule table
constexpr int DEERS_SCHED_ENTRIES = 4;
struct deers_sched_entry {
    int key[5];             // key[0] < 0: empty
    int rows;
    int* dev;               // DEERS_SCHED_CAP ints of device memory
    int* host;              // pinned staging of the same size
    cudaEvent_t uploaded;   // recorded after the upload: the staging copy may be rewritten once it has fired
    uint64_t last_use;
};

struct deers_ctx {
    int device;
    cudaStream_t stream;
    bool owns_stream;
    int sm_count;
    // Error word the kernels write when a bounded wait gives up: dev_err in device
    // memory, host_err its pinned host mirror, refreshed by deers_b200_sync().
    unsigned int* host_err;
    unsigned int* dev_err;
    uint64_t launches;
    char last_error[256];
    // cuTensorMapEncodeTiled, fetched through the runtime so that the library
    // does not link against the driver.
    void* encode_tiled;
    bool timing;
    deers_ktimer kt[DEERS_K_COUNT];
    // Balanced work schedules of the persistent f16 kernels: table[n * grid + cta] = n-th work item
    // of that CTA (or -1), built on the host per (B, H, tiles, causal, grid).  A few shapes stay cached
    // (least recently used goes first), each with its own device table and pinned staging copy, so that a
    // caller alternating shapes (training / evaluation, the ragged last chunk of the host pipeline) neither
    // rebuilds nor waits: the upload is an asynchronous copy on the context's stream.
    deers_sched_entry sched[DEERS_SCHED_ENTRIES];
    uint64_t sched_clock;
    // Side streams and events of the host-tensor pipeline (created on first use).
    cudaStream_t h2d_stream, d2h_stream;
    cudaEvent_t pipe_ev[3][3];      // [buffer set][h2d done, compute done, d2h done]
    bool pipe_ready;
};

// Brackets one kernel launch with events when timing is on.  A full ring drops the sample.
struct KernelTimerScope {
    deers_ctx* ctx;
    deers_ktimer* t;
    KernelTimerScope(deers_ctx* c, int kind) : ctx(c), t(nullptr) {
        if (c->timing && c->kt[kind].start && c->kt[kind].pending < DEERS_KT_RING) {
            t = &c->kt[kind];
            cudaEventRecord(t->start[t->pending], c->stream);
        }
    }
    ~KernelTimerScope() {
        if (t) {
            cudaEventRecord(t->stop[t->pending], ctx->stream);
            t->pending += 1;
        }
    }
};

#define DEERS_CUDA_TRY(ctx, expr)                                                            \
    do {                                                                                      \
        cudaError_t _e = (expr);                                                              \
        if (_e != cudaSuccess) {                                                              \
            snprintf((ctx)->last_error, sizeof((ctx)->last_error), "%s: %s", #expr,           \
                     cudaGetErrorString(_e));                                                 \
            return DEERS_ERR_CUDA;                                                            \
        }                                                                                     \
    } while (0)

// Device-side error codes (upper byte: which kernel, lower bits: which wait).
enum {
    DEERS_KERR_FWD_F16 = 0x100,
    DEERS_KERR_BWD_F16 = 0x200,
    DEERS_KERR_SELFTEST = 0x300,
    DEERS_KERR_GEMM = 0x400,
    DEERS_KERR_GPT = 0x500,      // token id / target out of range
};

// Work schedule shared by the persistent f16 kernels (ctx.cu).  Work items are ordered in groups
// of 16 slices, heaviest tiles first inside a group (item -> (slot, slice), slot 0 heaviest, weight
// ntile - slot when causal).  The table hands the items, in that order, to whichever CTA is least
// loaded so far, which balances the causal triangle for any slice count.  Returns nullptr (plain
// strided assignment) when the table would not fit.
const int4* deers_get_schedule(deers_ctx* ctx, int B, int H, int ntile, int causal, int grid, int* rows);

// Argument validation shared by every attention entry point (ctx.cu)
int deers_check_desc(const deers_attn_desc* d);
int deers_check_tensor(const deers_attn_desc* d, const void* p, const int64_t* s, size_t esize);
int deers_check_bwd_args(const deers_attn_desc* d, const void* q, const void* k, const void* v, const void* o,
                         const float* lse, const void* d_o, void* dq, void* dk, void* dv);

// f32 FFMA path (attn_f32.cu)
int launch_attn_fwd_f32(deers_ctx* ctx, const deers_attn_desc* d, const float* q, const float* k,
                        const float* v, float* o, float* lse);
int launch_attn_bwd_f32(deers_ctx* ctx, const deers_attn_desc* d, const float* q, const float* k,
                        const float* v, const float* o, const float* lse, const float* d_o, float* dq,
                        float* dk, float* dv, float* delta);

// f16 tcgen05 path (attn_f16_sm100.cu)
int launch_attn_fwd_f16(deers_ctx* ctx, const deers_attn_desc* d, const void* q, const void* k,
                        const void* v, void* o, float* lse);
int launch_attn_bwd_f16(deers_ctx* ctx, const deers_attn_desc* d, const void* q, const void* k,
                        const void* v, const void* o, const float* lse, const void* d_o, void* dq,
                        void* dk, void* dv, void* workspace, bool keep_ds);
size_t attn_bwd_f16_workspace_bytes(const deers_attn_desc* d, bool keep_ds);
int run_selftest_umma(deers_ctx* ctx, float* max_abs_err);
int run_selftest_wait(deers_ctx* ctx, unsigned int limit_ms, int* result_host);

// f32 GEMM (gemm_f32.cu)
size_t gemm_f32_workspace_bytes(const deers_ctx* ctx, int M, int N, int K);
int launch_gemm_f32(deers_ctx* ctx, int M, int N, int K, const float* a, long long lda, int a_mn, const float* b,
                    long long ldb, int b_mn, float* c, long long ldc, int epi, const float* r, long long ldr, float* aux,
                    void* workspace, size_t ws_bytes, bool counters_zero);
// RMSNorm (rmsnorm.cu)
int launch_rmsnorm_fwd(deers_ctx* ctx, long long rows, int C, double eps, const float* x, float* y, float* inv_norm);
int launch_rmsnorm_bwd(deers_ctx* ctx, long long rows, int C, const float* x, const float* inv_norm, const float* dy,
                       const float* add, float* dx);
// embedding and cross-entropy (gpt_ops.cu)
int launch_embedding_fwd(deers_ctx* ctx, const float* weight, const long long* ids, long long n_ids, int C, long long V,
                         float* out);
int launch_embedding_bwd(deers_ctx* ctx, const float* dout, const long long* ids, long long n_ids, int C, long long V,
                         float* dweight);
int launch_cross_entropy_fwd(deers_ctx* ctx, const float* logits, long long ld, const long long* targets, long long rows,
                             long long V, float* lse, float* picked, float* loss);
int launch_cross_entropy_bwd(deers_ctx* ctx, const float* logits, long long ld, const long long* targets, const float* lse,
                             long long rows, long long V, float upstream, float* dlogits, long long ldd);
// AdamW with the trainer's rule "no update when the gradient norm is not finite" (optim.cu)
int launch_adamw(deers_ctx* ctx, int n_tensors, const deers_optim_tensor* tensors, const deers_adamw_hyper* h,
                 const float* norm_dev, double max_norm, bool skip_nonfinite);
// f32-accurate tensor-core GEMM on split f16 operands (gemm_f16x3_sm100.cu) and the split writers
size_t gemm_f16x3_workspace_bytes(const deers_ctx* ctx, int M, int N, int K);
int launch_split_f16x3(deers_ctx* ctx, long long rows, int cols, const float* src, long long ld_src, float scale,
                       void* hi, void* lo, long long ld_dst);
int launch_gemm_f16x3(deers_ctx* ctx, int M, int N, int K, const void* a_hi, const void* a_lo, long long lda, int a_mn,
                      const void* b_hi, const void* b_lo, long long ldb, int b_mn, float* c, long long ldc, float out_scale,
                      void* workspace, size_t ws_bytes);
int launch_cross_entropy_bwd_split(deers_ctx* ctx, const float* logits, long long ld, const long long* targets,
                                   const float* lse, long long rows, long long V, float upstream, float scale, void* hi,
                                   void* lo, long long ldd);
