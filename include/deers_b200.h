/*
 * deers_b200 — C ABI of the B200 (sm_100a) causal self-attention path for deers.
 *
 * The deers repository has no FFI of its own: its CUDA backend is Rust over
 * cudarc.  These entry points are what `src/storage/cuda.rs` would bind (with
 * `extern "C"` declarations, linked by a `build.rs` that runs nvcc) to replace
 * the matmul -> scale -> mask -> softmax -> matmul chain of
 * `src/models/gpt.rs:139-144` and its autograd backward by one fused op.  Each
 * declaration cites the reference interface it stands in for.
 *
 * Conventions
 *  - Every pointer named q/k/v/o/d_o/dq/dk/dv/lse/workspace is a DEVICE pointer
 *    owned by the caller.  Tensors are [B, H, T, D]; strides are in elements;
 *    the innermost (D) stride must be 1 and every base pointer and every row
 *    start must be 16-byte aligned, otherwise DEERS_ERR_LAYOUT is returned so
 *    that the caller can compact() and retry.  Outputs are written with the
 *    strides given in the descriptor.
 *  - Work is enqueued on the context's stream and the call returns at once; no
 *    allocation and no stream synchronisation happens inside attn_fwd / attn_bwd.
 *    On the f16 path the first call with a new (B, H, T, causal) builds a small
 *    work-schedule table on the host and uploads it asynchronously from pinned
 *    memory; the tables of the last few shapes stay cached.
 *  - Nothing aborts or traps.  Every function returns a status (0 = OK) and
 *    device-side waits are bounded: a kernel that gives up records a code that
 *    deers_b200_sync() reports as DEERS_ERR_KERNEL.
 *  - lse is float32 [B, H, T], the natural-log row sums of exp(scale * scores)
 *    over the unmasked columns: the quantity `CpuStorage::log_sum_exp`
 *    (`src/storage/cpu.rs:755-770`) produces on the scaled, masked scores.
 */
#ifndef DEERS_B200_H
#define DEERS_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#pragma GCC visibility push(default)
#endif

typedef struct deers_ctx deers_ctx;

enum {
    DEERS_OK = 0,
    DEERS_ERR_NULL = 1,        /* a required pointer was NULL                           */
    DEERS_ERR_SHAPE = 2,       /* B,H,T,D out of the supported range                    */
    DEERS_ERR_DTYPE = 3,       /* dtype not DEERS_F16 / DEERS_F32                       */
    DEERS_ERR_LAYOUT = 4,      /* inner stride != 1 or misaligned: compact() and retry  */
    DEERS_ERR_WORKSPACE = 5,   /* workspace missing or too small                        */
    DEERS_ERR_CUDA = 6,        /* a CUDA runtime/driver call failed (see last_error)    */
    DEERS_ERR_KERNEL = 7,      /* a kernel gave up on a bounded wait (see last_error)   */
    DEERS_ERR_UNSUPPORTED = 8, /* valid request this build has no kernel for            */
    DEERS_ERR_DEVICE = 9       /* device is not an sm_100 part                          */
};

enum { DEERS_F16 = 0, DEERS_F32 = 1 };

/*
 * One attention problem.  Mirrors the arguments the reference passes down its
 * storage layer: a Layout (shape + strides in elements, `src/layout.rs:151-202`)
 * per operand, the dtype (`src/dtype.rs:14-21`) and the scale the module
 * computes (`src/models/gpt.rs:139`).
 */
typedef struct {
    int32_t B, H, T, D;
    int32_t dtype;            /* DEERS_F16 (f32 accumulate) or DEERS_F32 (FFMA, no TF32)  */
    int32_t causal;           /* 1: column j > row i is masked (`src/nn/functional.rs:38-51`) */
    float scale;              /* multiplies q.k^T, normally (float)(1/sqrt((double)D))    */
    int64_t q_strides[4];     /* strides of [B,H,T,D] in elements; [3] must be 1          */
    int64_t k_strides[4];
    int64_t v_strides[4];
    int64_t o_strides[4];     /* o in fwd (written) and in bwd (read)                     */
    int64_t do_strides[4];    /* bwd only                                                 */
    int64_t dq_strides[4];    /* bwd only: strides the gradients are written with         */
    int64_t dk_strides[4];
    int64_t dv_strides[4];
} deers_attn_desc;

/* Fills every stride field for compact [B,H,T,D] tensors. */
void deers_b200_attn_desc_compact(deers_attn_desc* desc, int32_t B, int32_t H, int32_t T, int32_t D,
                                  int32_t dtype, int32_t causal, float scale);

/*
 * Context: device, stream, error word.  Stands in for the process-global
 * `CudaRuntime` of `src/storage/cuda.rs:455-521` (context on device 0, default
 * stream, module, cuBLAS), with a device ordinal added so that one process per
 * GPU can shard (batch x head) slices.  `stream` may be NULL (the context then
 * creates its own non-blocking stream) or an existing cudaStream_t to enqueue on
 * (the reference's single default stream, `src/storage/cuda.rs:505`); pass
 * cudaStreamLegacy to name the legacy default stream.
 */
int deers_b200_init(int device_ordinal, void* stream, deers_ctx** out);
void deers_b200_destroy(deers_ctx* ctx);
int deers_b200_set_stream(deers_ctx* ctx, void* stream);
void* deers_b200_stream(deers_ctx* ctx);

/*
 * Buffers and copies: `CudaStorage` allocation, upload and read-back
 * (`src/storage/cuda.rs:637-706`, `:1541-1555`).  alloc/free are stream-ordered;
 * memcpy_d2h synchronises the stream, the other copies are asynchronous.
 */
int deers_b200_alloc(deers_ctx* ctx, size_t bytes, void** dptr);
int deers_b200_free(deers_ctx* ctx, void* dptr);
/* Free and total device memory in bytes (what a caller weighs the larger backward workspace against). */
int deers_b200_mem_info(deers_ctx* ctx, size_t* free_bytes, size_t* total_bytes);
int deers_b200_memcpy_h2d(deers_ctx* ctx, void* dst, const void* src, size_t bytes);
int deers_b200_memcpy_d2h(deers_ctx* ctx, void* dst, const void* src, size_t bytes);
int deers_b200_memcpy_d2d(deers_ctx* ctx, void* dst, const void* src, size_t bytes);

/*
 * `Device::synchronize` (`src/device.rs:66-72` -> `src/storage/cuda.rs:1598-1602`).
 * Also reads the device error word: returns DEERS_ERR_KERNEL if any kernel since
 * the last sync gave up on a bounded wait, and clears the word.
 */
int deers_b200_sync(deers_ctx* ctx);

/*
 * Scratch memory a pass needs (pass 0 = forward, 1 = backward, 2 = fast backward), in bytes.
 * Forward needs none, except for f16 head dims other than 64 and 128: the tensor-core tiles are 64 or 128
 * wide, the reference derives head_dim = n_embd / n_head freely (`src/models/gpt.rs:86-100`), so any
 * multiple of 8 up to 128 is accepted and runs on zero-padded copies kept in the workspace (four tensors of
 * B*H*T*Dp halves forward, eight more bytes-wise for the backward; Dp = 64 or 128).  Backward keeps rowsum(dO * O) per row (and, for f16, the
 * row lse in log2 units), padded to whole tiles.  The reference allocates the equivalent temporaries
 * inside each op (`src/storage/cuda.rs:637-644`; its backward also keeps the whole [B,H,T,T]
 * probability tensor alive from the forward, `src/ops.rs:1162-1175`).
 * Pass 2 (f16; for f32 it equals pass 1) adds room for the dS tiles the mask leaves, 32 KB per
 * (slice, 128-row query tile, 128-row key tile): B*H*nq*(nq+1)/2 tiles causal, nq = ceil(T/128).
 * deers_b200_attn_bwd given at least that much keeps dS between its two main kernels, so dQ is one
 * streaming product instead of a second recomputation of S and dP (7 tile products become 5);
 * given less (but at least the pass-1 size) it recomputes.  Both give the same results up to
 * f16 rounding of the same dS values and both are bitwise reproducible.
 */
size_t deers_b200_attn_workspace_bytes(const deers_attn_desc* desc, int pass);

/*
 * Fused forward: O = softmax(scale * Q K^T + causal mask) V and the per-row lse.
 * Replaces `src/models/gpt.rs:139-144` (MatMul `src/ops.rs:1013-1106`, ScalarMul
 * `:613-648`, causal_mask + Broadcast + EWiseAdd, softmax `src/tensor.rs:408-458`,
 * MatMul) — the storage-level hook is a new `BackendStorage::attention_fwd` added
 * the way `log_softmax_fwd` was (`src/storage.rs:284-302,379-418`).
 * `workspace` (256-byte aligned, deers_b200_attn_workspace_bytes(desc, 0) bytes) may be NULL when that size
 * is 0; DEERS_ERR_WORKSPACE otherwise.
 */
int deers_b200_attn_fwd(deers_ctx* ctx, const deers_attn_desc* desc, const void* q, const void* k,
                        const void* v, void* o, float* lse, void* workspace, size_t workspace_bytes);

/*
 * Fused backward: dQ, dK, dV from dO, recomputing P from lse.  Replaces the
 * chain `MatMul::backward` (`src/ops.rs:1089-1101`), `EWiseExp::backward`
 * (`:422-425`), log-softmax backward (`:210-214,777-799,1162-1175`),
 * `ScalarMul::backward` (`:638-643`), `MatMul::backward`.  dQ, dK and dV are
 * accumulated per tile without atomics (bitwise reproducible).
 */
int deers_b200_attn_bwd(deers_ctx* ctx, const deers_attn_desc* desc, const void* q, const void* k,
                        const void* v, const void* o, const float* lse, const void* d_o, void* dq,
                        void* dk, void* dv, void* workspace, size_t workspace_bytes);

/*
 * Forward + backward on HOST tensors, for callers whose tensors live in host memory (the
 * reference moves data between host and device with `clone_htod` / `clone_dtoh`,
 * `src/storage/cuda.rs:692-706,1541-1555`, one whole tensor at a time).  q, k, v, d_o (inputs) and
 * o, dq, dk, dv (outputs; lse_host may be NULL) are compact [B,H,T,D] host arrays, ideally pinned.
 * The (batch x head) slices are processed in chunks of `chunk_slices`; host->device copies of the
 * next chunk, the kernels of the current one and the device->host copies of the previous one run
 * on three streams, so the PCIe link is used in both directions while the GPU computes.
 * `device_scratch` is caller-owned device memory of at least
 * deers_b200_attn_host_scratch_bytes(desc, chunk_slices) bytes (256-byte aligned); nothing is
 * allocated inside.  The call returns after the last copy has finished.
 */
size_t deers_b200_attn_host_scratch_bytes(const deers_attn_desc* desc, int chunk_slices);
int deers_b200_attn_fwd_bwd_host(deers_ctx* ctx, const deers_attn_desc* desc, const void* q_host, const void* k_host,
                                 const void* v_host, const void* do_host, void* o_host, float* lse_host, void* dq_host,
                                 void* dk_host, void* dv_host, int chunk_slices, void* device_scratch,
                                 size_t scratch_bytes);

/*
 * The f16 backward for callers that cannot provide scratch memory.  No counterpart in the
 * reference (its ops allocate their temporaries freely, `src/storage/cuda.rs:637-644`).
 *
 * Who needs it: code that runs where allocation is off limits - inside an allocator or
 * memory-pool callback, in a host application that freezes its device-memory plan after start-up
 * and forbids plugins to call cudaMalloc, or on a real-time path that may not take the
 * allocator's locks.  Same arguments and results as deers_b200_attn_bwd with dtype DEERS_F16, minus
 * the workspace: the per-row scratch lives in an 8 MiB array inside the library image, which every
 * GPU that loads the library holds until the process exits.
 *
 * Limits and rules:
 *  - B * H * ceil(T/128)*128 must not exceed 1,048,576 rows; larger problems return
 *    DEERS_ERR_WORKSPACE (deers_b200_last_error names the sizes) and must use deers_b200_attn_bwd.
 *  - The call allocates nothing.  The first call on each device looks up the array's device address
 *    (cudaGetSymbolAddress), and the first call with a new (B, H, T, causal) builds a work-schedule table
 *    on the host and uploads it with an asynchronous copy (as deers_b200_attn_bwd does); a few shapes
 *    stay cached.  Make those first calls outside any stream capture: a new shape met while capturing
 *    falls back to an unbalanced work assignment.  The only host-side wait is for an earlier upload from
 *    the same cache slot, which has long finished unless shapes change on every call.
 *  - All calls on a device share the one array, which keeps the previous call's contents.  The
 *    backward's first kernel overwrites everything it later reads, so nothing has to be cleared, but
 *    two calls that overlap on the GPU (different streams or contexts) race on it: serialise them.
 */
int deers_b200_attn_bwd_f16_static(deers_ctx* ctx, const deers_attn_desc* desc, const void* q, const void* k,
                                   const void* v, const void* o, const float* lse, const void* d_o, void* dq,
                                   void* dk, void* dv);

/*
 * Rotary embedding fused with the head-major pack that feeds the attention op, and its inverse for
 * the gradients.  Replaces, for q and for k: `apply_rotary_emb` (`src/models/gpt.rs:49-73`: two
 * narrows, four multiplies, two adds and a `cat` that is built from two transposes,
 * `src/tensor.rs:428-440`), the `permute([0,2,1,3])` that follows it (`gpt.rs:135-136`) and the
 * compaction copy the batched GEMM then needs (`src/ops.rs:913`) — about 14 launches and three
 * tensor-sized copies per layer; the backward of those ops is the same call with `inverse = 1`.
 *
 * One row of D elements is read at src + b*src_strides[0] + t*src_strides[1] + h*src_strides[2],
 * split into halves x1 | x2, rotated with row t of the cos / sin cache ([T, D/2] contiguous, same
 * dtype as the tensor: `precompute_rotary_embeddings`, `gpt.rs:12-46`) and written at the matching
 * dst address:
 *     inverse = 0:  y1 = x1*cos + x2*sin,      y2 = x1*(-sin) + x2*cos
 *     inverse = 1:  x1 = y1*cos + y2*(-sin),   x2 = y1*sin + y2*cos
 * Every multiply and add rounds to the storage type, exactly like the reference's separate ops, so
 * results are bit-identical to its CPU path.  Strides are in elements, in (b, t, h, d) order for BOTH
 * tensors, inner stride 1: the forward call passes the [B,T,H,D] strides of the projection output as
 * src and the strides of a [B,H,T,D] buffer (b: H*T*D, t: D, h: T*D) as dst; the backward call swaps
 * them.  Rows, halves and cache rows on 16-byte boundaries take the 16-byte path, anything else a
 * scalar path.  Enqueued on the context's stream; no allocation, no synchronisation.
 */
typedef struct deers_rope_desc {
    int32_t B, T, H, D;        /* D even */
    int32_t dtype;             /* DEERS_F16 or DEERS_F32: tensor and cache */
    int32_t inverse;           /* 0 rotate, 1 rotate back (gradients) */
    int64_t src_strides[4];    /* (b, t, h, d), elements */
    int64_t dst_strides[4];
} deers_rope_desc;
int deers_b200_rope_pack(deers_ctx* ctx, const deers_rope_desc* desc, const void* src, const void* cos_cache,
                         const void* sin_cache, void* dst);

/*
 * Multi-tensor AdamW step with the global gradient-norm clip folded in, f32.  Replaces
 * `AdamW::step_with_grads` (`src/optim.rs:214-251`: about twelve element-wise ops and ten temporaries per
 * parameter) and `clip_grad_norm` (`src/optim.rs:257-297`: a multiply, a full reduction and an add per
 * parameter, a host read of the norm, and a scalar multiply per gradient when it clips).
 *
 * A parameter is described by device pointers to its weights w, gradient g and moments m, v (n f32
 * elements each, 4-byte aligned; 16-byte alignment of all of them enables the 16-byte path); moments of
 * a parameter seen for the first time must be zero (`param.zeros_like()`, `optim.rs:229,233`).  Up to
 * 256 tensors per call.  Everything is enqueued on the context's stream; nothing allocates or
 * synchronises.
 *
 *   grad_norm   norm_dev[0] = sqrt(sum over all tensors of g*g), f32, summed in a fixed order (the
 *               reference sums each tensor left to right and adds the tensors in turn, so the last
 *               bits can differ).  `scratch` is deers_b200_optim_scratch_bytes() of device memory.
 *   grad_clip   what clip_grad_norm does after it has the norm: nothing if the norm is not finite or
 *               <= max_norm, else every g *= (f32)(max_norm / ((f64)norm + 1e-6)) in place.  The
 *               decision is taken on the device from norm_dev.  max_norm must be > 0
 *               (DEERS_ERR_SHAPE otherwise; the reference asserts).
 *   adamw_step  m = m*b1 + g*(1-b1);  v = v*b2 + (g*g)*(1-b2);  m_hat = m*(1/(1-b1^t));
 *               v_hat = v*(1/(1-b2^t));  w = (wd > 0 ? w*(1-lr*wd) : w) - (m_hat/(sqrt(v_hat)+eps))*lr,
 *               one rounding per operation and each scalar an f64 rounded to f32, exactly as the
 *               reference's scalar ops do (`src/storage.rs:105-123`), so w, m, v are bit-identical to
 *               its CPU path.  `hyper->step` is the step count AFTER the increment of
 *               `optim.rs:215` (t >= 1).  With norm_dev != NULL the clip of grad_clip is applied to
 *               g on the fly, which removes the host round trip of clip_grad_norm from the training
 *               step; with NULL the gradients are used as they are.  NOTE: g itself is left untouched,
 *               whereas the reference's clip_grad_norm replaces the gradients in the GradientStore
 *               (`optim.rs:287-294`): a caller that reads, logs or accumulates gradients after the step
 *               and wants the clipped values calls deers_b200_grad_clip first and passes NULL here.
 */
typedef struct deers_optim_tensor {
    void* w;        /* weights, updated in place (unused by grad_norm / grad_clip) */
    void* g;        /* gradient; grad_clip scales it in place */
    void* m;        /* first moment, updated in place */
    void* v;        /* second moment, updated in place */
    int64_t n;      /* elements */
} deers_optim_tensor;
typedef struct deers_adamw_hyper {
    double lr, beta1, beta2, eps, weight_decay;   /* AdamWConfig defaults: betas (0.9, 0.999), eps 1e-8, wd 0 */
    int64_t step;                                 /* t of the bias correction, >= 1 */
} deers_adamw_hyper;
size_t deers_b200_optim_scratch_bytes(void);
int deers_b200_grad_norm(deers_ctx* ctx, int n_tensors, const deers_optim_tensor* tensors, float* norm_dev,
                         void* scratch, size_t scratch_bytes);
int deers_b200_grad_clip(deers_ctx* ctx, int n_tensors, const deers_optim_tensor* tensors, const float* norm_dev,
                         double max_norm);
int deers_b200_adamw_step(deers_ctx* ctx, int n_tensors, const deers_optim_tensor* tensors,
                          const deers_adamw_hyper* hyper, const float* norm_dev, double max_norm);

/*
 * RMSNorm forward and backward over the last axis of a compact [rows, C] f32 tensor.  Replaces
 * `RMSNorm::forward` (`src/nn.rs:244-251`: x*x, mean over the last axis, + eps, ^-0.5, broadcast
 * multiply — six graph ops) and the autograd backward of those ops (`src/ops.rs:210-214,638-643,675-679,
 * 777-799`).  fwd writes y = x * inv and inv_norm[row] = 1/sqrt(mean(x*x) + eps) (rows floats the caller
 * keeps for the backward, the way the attention op keeps its row lse); bwd writes
 * dx = dy*inv - x * (sum(dy*x) * inv^3 / C).  eps is the module's f64 rounded to f32 (`storage.rs:105-123`).
 * Row sums are f32 shuffle trees, the reference's are left-to-right f32 sums: parity is to rounding
 * (1e-5 of the tensor's max-abs), not to the bit.  Enqueued on the context's stream; no allocation.
 */
int deers_b200_rmsnorm_fwd(deers_ctx* ctx, int64_t rows, int32_t C, double eps, const float* x, float* y,
                           float* inv_norm);
int deers_b200_rmsnorm_bwd(deers_ctx* ctx, int64_t rows, int32_t C, const float* x, const float* inv_norm,
                           const float* dy, float* dx);

/*
 * Decode-time attention with a key / value cache: Tq new query rows (1 when sampling) against Tk = Tq +
 * seqlen_offset cached key and value rows per (batch, head) slice,
 *     O = softmax(scale * Q K^T + mask) V,   key j masked for query i iff causal and j > i + (Tk - Tq),
 * the mask `functional::causal_mask(batch, tgt_len = Tq, seqlen_offset = Tk - Tq)` builds
 * (`src/nn/functional.rs:12-55`).  The reference has no cache: its sampling loop re-runs the whole prefix
 * through `GPT::forward` for every token; with this entry point a step reads K and V once (split over the
 * keys across CTAs, merged by a second launch).  q, o: [B,H,Tq,D]; k_cache, v_cache: [B,H,Tk,D]; strides in
 * elements, inner stride 1 (a cache allocated for more than Tk rows is passed with its own row / slice
 * strides).  f16 or f32 storage, f32 arithmetic; D <= 256, Tq <= 128, B*H <= 65535.  lse (optional, [B,H,Tq]
 * f32, natural log) like deers_b200_attn_fwd.  Workspace: deers_b200_attn_decode_workspace_bytes(desc)
 * of device memory.  Enqueued on the context's stream; no allocation, no synchronisation.
 */
typedef struct deers_decode_desc {
    int32_t B, H, Tq, Tk, D;
    int32_t dtype;            /* DEERS_F16 / DEERS_F32 */
    int32_t causal;
    float scale;
    int64_t q_strides[4], k_strides[4], v_strides[4], o_strides[4];
} deers_decode_desc;
size_t deers_b200_attn_decode_workspace_bytes(const deers_decode_desc* desc);
int deers_b200_attn_decode(deers_ctx* ctx, const deers_decode_desc* desc, const void* q, const void* k_cache,
                           const void* v_cache, void* o, float* lse, void* workspace, size_t workspace_bytes);

/*
 * f16 GEMM with f32 accumulation for the projections around the attention op: C[M,N] = A * B, C row-major
 * with leading dimension ldc.  Replaces the `cublasGemmStridedBatchedEx` call behind `Tensor::matmul`
 * for f16 operands (`src/storage/cuda.rs:1147-1177`) as `Linear::forward` uses it (`src/nn.rs:184-190`,
 * weight stored [in_features, out_features]) and as the matmul backward does (`src/ops.rs:1089-1101`):
 *     a_mn_major = 0: A is stored [M][K] (K contiguous);   1: A is stored [K][M] (M contiguous)
 *     b_mn_major = 0: B is stored [N][K] (K contiguous);   1: B is stored [K][N] (N contiguous)
 *     forward  y  = x  W     : gemm(M=rows, N=out, K=in,  x, 0,  W, 1)
 *     dgrad    dx = dy W^T   : gemm(M=rows, N=in,  K=out, dy, 0, W, 0)      (W read as [N'=in][K'=out])
 *     wgrad    dW = x^T dy   : gemm(M=in,   N=out, K=rows, x, 1, dy, 1)
 * Leading dimensions in elements, multiples of 8 (16-byte rows); N a multiple of 8; pointers 16-byte
 * aligned (DEERS_ERR_LAYOUT otherwise).  Enqueued on the context's stream; no allocation.
 */
int deers_b200_gemm_f16(deers_ctx* ctx, int32_t M, int32_t N, int32_t K, const void* a, int64_t lda, int32_t a_mn_major,
                        const void* b, int64_t ldb, int32_t b_mn_major, void* c, int64_t ldc);

/*
 * f32 GEMM in full f32 arithmetic (FFMA; no TF32) for the projections of the f32 model: C[M,N] = A * B,
 * C row-major with leading dimension ldc.  Replaces the `cublasGemmStridedBatchedEx` call with
 * CUBLAS_COMPUTE_32F behind `Tensor::matmul` for f32 operands (`src/storage/cuda.rs:1098-1128`) as
 * `Linear::forward` uses it (`src/nn.rs:184-190`, weight stored [in_features, out_features]) and as the
 * matmul backward does (`src/ops.rs:1089-1101`); operand orders as for deers_b200_gemm_f16:
 *     a_mn_major = 0: A is stored [M][K] (K contiguous);   1: A is stored [K][M] (M contiguous)
 *     b_mn_major = 0: B is stored [N][K] (K contiguous);   1: B is stored [K][N] (N contiguous)
 *     forward  y  = x  W     : gemm(M=rows, N=out, K=in,  x, 0,  W, 1)
 *     dgrad    dx = dy W^T   : gemm(M=rows, N=in,  K=out, dy, 0, W, 0)
 *     wgrad    dW = x^T dy   : gemm(M=in,   N=out, K=rows, x, 1, dy, 1)
 * Any leading dimension and any 4-byte aligned pointer is accepted (16-byte loads are used when base and
 * leading dimension allow).  An optional epilogue runs on the tile while it is in registers and replaces the
 * element-wise graph ops around the projections:
 *     DEERS_EPI_ADD       C = residual + A*B                 `x + attn(...)`, `x + mlp(...)` (`src/models/gpt.rs:237-239`)
 *     DEERS_EPI_RELU_SQ   r = max(A*B, 0); C = r*r; aux = r  `relu` and `y * y` of the MLP (`gpt.rs:194-196`)
 *     DEERS_EPI_MUL_AUX2  t = (A*B) * aux; C = t + t         their backward (`src/ops.rs:210-214, 560-568`) given aux = r
 * aux has the shape and leading dimension of C.  Shapes with few output tiles and a long K are split along K;
 * the parts are added in a fixed order, so results are bitwise reproducible.  `workspace` must hold
 * deers_b200_gemm_f32_workspace_bytes(ctx, M, N, K) bytes (0 for most shapes; 256-byte aligned).  Enqueued on
 * the context's stream; no allocation, no synchronisation.
 */
enum { DEERS_EPI_NONE = 0, DEERS_EPI_ADD = 1, DEERS_EPI_RELU_SQ = 2, DEERS_EPI_MUL_AUX2 = 3 };
typedef struct deers_gemm_epilogue {
    int32_t kind;             /* DEERS_EPI_* */
    const float* residual;    /* DEERS_EPI_ADD: [M][ld_residual] */
    int64_t ld_residual;
    float* aux;               /* DEERS_EPI_RELU_SQ: written; DEERS_EPI_MUL_AUX2: read; [M][ldc] */
} deers_gemm_epilogue;
size_t deers_b200_gemm_f32_workspace_bytes(deers_ctx* ctx, int32_t M, int32_t N, int32_t K);
int deers_b200_gemm_f32(deers_ctx* ctx, int32_t M, int32_t N, int32_t K, const float* a, int64_t lda, int32_t a_mn_major,
                        const float* b, int64_t ldb, int32_t b_mn_major, float* c, int64_t ldc,
                        const deers_gemm_epilogue* epilogue, void* workspace, size_t workspace_bytes);

/*
 * f32-accurate GEMM on the tensor core: C[M,N] = A * B in f32 where every f32 operand is carried as an f16 pair
 * (x * s = hi + lo * 2^-11) and the product is three tcgen05 f16 products with f32 accumulation (main = hi*hi,
 * correction = hi*lo + lo*hi; the dropped lo*lo term is below 2^-22 of a product).  Same role as
 * deers_b200_gemm_f32 - the reference's f32 matmul (`src/storage/cuda.rs:1098-1128`, CUBLAS_COMPUTE_32F) behind
 * `Linear::forward` and the matmul backward - for the products large enough to be worth the tensor core: the
 * language-model head (`src/models/gpt.rs:351`) and its two backward products, 80 % of a training step's FLOPs.
 *   split_f16x3   hi = f16(src * scale), lo = f16((src * scale - hi) * 2^11) for a [rows, cols] f32 matrix; scale is
 *                 a power of two that brings the values into f16 range (1 for activations and weights; gradients
 *                 of a mean-reduced loss want about rows * 4096).  hi / lo: f16 [rows][ld_dst].
 *   gemm_f16x3    operand orders as deers_b200_gemm_f16 (a_mn_major, b_mn_major); lda, ldb multiples of 8, ldc a
 *                 multiple of 4, pointers 16-byte aligned (DEERS_ERR_LAYOUT otherwise); any M, N, K.
 *                 C = (A*B) * out_scale: pass 1 / (scale_a * scale_b).  Products with few output tiles and a long K
 *                 are split along K and summed in a fixed order (bitwise reproducible); `workspace` then needs
 *                 deers_b200_gemm_f16x3_workspace_bytes(ctx, M, N, K) bytes (0 otherwise).
 * Enqueued on the context's stream; no allocation, no synchronisation.
 */
int deers_b200_split_f16x3(deers_ctx* ctx, int64_t rows, int32_t cols, const float* src, int64_t ld_src, float scale,
                           void* hi, void* lo, int64_t ld_dst);
size_t deers_b200_gemm_f16x3_workspace_bytes(deers_ctx* ctx, int32_t M, int32_t N, int32_t K);
int deers_b200_gemm_f16x3(deers_ctx* ctx, int32_t M, int32_t N, int32_t K, const void* a_hi, const void* a_lo, int64_t lda,
                          int32_t a_mn_major, const void* b_hi, const void* b_lo, int64_t ldb, int32_t b_mn_major, float* c,
                          int64_t ldc, float out_scale, void* workspace, size_t workspace_bytes);

/*
 * RMSNorm backward that also adds the gradient arriving over the residual connection:
 * dx = residual_grad + (dy*inv - x * (sum(dy*x) * inv^3 / C)).  In the block `x + f(norm(x))`
 * (`src/models/gpt.rs:236-240`) the reference's GradientStore adds the two contributions to x with a separate
 * element-wise add (`src/backprop.rs:101-112`).
 */
int deers_b200_rmsnorm_bwd_add(deers_ctx* ctx, int64_t rows, int32_t C, const float* x, const float* inv_norm,
                               const float* dy, const float* residual_grad, float* dx);

/*
 * Embedding lookup and its backward, f32 table [vocab, C], int64 token ids on the device.  Replaces
 * `Embedding::forward` (`src/nn.rs:214-221`: `index_select(0, ids)`, kernel `src/storage/cuda.rs:381-390`) and
 * the index_add of its backward (`src/storage/cuda.rs:392-402`, atomic adds into a zeroed table).  bwd zeroes
 * dweight and adds the rows of dout in token order (the first occurrence of an id owns the row), so repeated
 * tokens give a reproducible sum equal to the CPU backend's.  An id outside [0, vocab) makes the next
 * deers_b200_sync return DEERS_ERR_KERNEL; the row is skipped (forward: written as zeros).
 */
int deers_b200_embedding_fwd(deers_ctx* ctx, const float* weight, const int64_t* ids, int64_t n_ids, int32_t C,
                             int64_t vocab, float* out);
int deers_b200_embedding_bwd(deers_ctx* ctx, const float* dout, const int64_t* ids, int64_t n_ids, int32_t C,
                             int64_t vocab, float* dweight);

/*
 * Cross-entropy over [rows, vocab] f32 logits (row stride ld) with int64 targets on the device.  Replaces
 * `loss::cross_entropy` (`src/loss.rs:21-24`: log_softmax, gather, sum, scalar multiply) and its backward.
 *   fwd  lse[row] = ln(sum exp(x - max)) + max (`src/storage/cpu.rs:755-770`); loss[0] = sum over rows of
 *        (x[target] - lse) * (float)(-1/rows).  The log-probabilities are never written.  `scratch`:
 *        deers_b200_cross_entropy_scratch_bytes(rows) of device memory.
 *   bwd  dlogits = (onehot * g - exp(x - lse) * g) * upstream, g = (float)(-1/rows): gather backward and the
 *        `x - lse` backward (`src/ops.rs:210-214, 777-799, 1162-1175`) in one pass; dlogits may be the logits
 *        buffer itself (in place).  `upstream` is the gradient of the loss (1 for `loss.backward()`).  rows <= 65535.
 */
size_t deers_b200_cross_entropy_scratch_bytes(int64_t rows);
int deers_b200_cross_entropy_fwd(deers_ctx* ctx, int64_t rows, int64_t vocab, const float* logits, int64_t ld,
                                 const int64_t* targets, float* lse, float* loss, void* scratch, size_t scratch_bytes);
int deers_b200_cross_entropy_bwd(deers_ctx* ctx, int64_t rows, int64_t vocab, const float* logits, int64_t ld,
                                 const int64_t* targets, const float* lse, float upstream, float* dlogits,
                                 int64_t ld_dlogits);

/*
 * The GPT of `src/models/gpt.rs` as one device-resident object: parameters, gradients, AdamW moments and
 * activations live in device memory owned by the model; a training step is `GPT::forward` (`gpt.rs:329-355`) ->
 * `loss::cross_entropy` (`src/loss.rs:21-24`) -> `backward()` -> `clip_grad_norm` (`src/optim.rs:257-297`) ->
 * `AdamW::step_with_grads` (`src/optim.rs:214-251`), the loop body of `examples/tinystories_train.rs:188-218`
 * with one micro-batch, enqueued as about 160 kernels of this library and nothing else (no host round trip:
 * the clip decision and the "skip the update when the norm is not finite" rule of the trainer are taken on the
 * device).  After the first step of a (B, T) the forward/backward part is replayed from a CUDA graph.
 *
 * deers_gpt_config mirrors `GPTConfig` (`gpt.rs:259-285`).  Parameters are addressed by index in the order of
 * `GPT::parameters` (`gpt.rs:358-365`): 0 wte.weight [vocab, n_embd]; then per block q_proj, k_proj, v_proj,
 * out_proj [n_embd, n_embd], up_proj [n_embd, mlp], down_proj [mlp, n_embd]; last lm_head.weight [n_embd, vocab];
 * names as the reference's checkpoint keys (`blocks.{i}.attn.q_proj.weight`, ...).  Host arrays passed to
 * param_set / param_get are compact row-major [rows, cols]; internally q, k and v of a block share one
 * [n_embd, 3*n_embd] buffer so the three projections are one GEMM.
 *   create           allocates everything for up to max_batch * sequence_len tokens; weights start at zero.
 *   param_set/get    upload / read back one tensor: what = 0 weight, 1 gradient, 2 first moment, 3 second moment.
 *   forward          logits [B*T, vocab] (compact, device) for ids [B*T] (device); logits may be NULL.
 *   forward_backward forward, loss and every parameter gradient; loss_dev (1 float, device) may be NULL.
 *   train_step       forward_backward, then gradient norm (written to grad_norm_dev if not NULL), clip at
 *                    max_grad_norm (<= 0: no clipping) and the AdamW update; hyper->step is t >= 1.
 *   train_step_host  the same with ids / targets in host memory and the loss read back: copies 16*B*T bytes in,
 *                    4 bytes out and synchronises.
 * Everything is enqueued on the context's stream; only create, param_set, param_get and train_step_host
 * synchronise.  Graph replay needs a capturable stream: a context on the legacy default stream runs every step
 * eagerly (same kernels, more launch overhead); deers_b200_gpt_graph_active tells which.
 */
typedef struct deers_gpt_config {
    int32_t vocab_size, sequence_len, n_layer, n_head, n_embd, mlp_hidden_dim;
    double rms_norm_eps;
    float rope_base;
} deers_gpt_config;
typedef struct deers_gpt deers_gpt;
int deers_b200_gpt_create(deers_ctx* ctx, const deers_gpt_config* config, int32_t max_batch, deers_gpt** out);
void deers_b200_gpt_destroy(deers_gpt* model);
int deers_b200_gpt_num_params(const deers_gpt* model);
int deers_b200_gpt_param_info(const deers_gpt* model, int index, char* name, size_t name_bytes, int64_t* rows,
                              int64_t* cols);
int deers_b200_gpt_param_set(deers_gpt* model, int index, int what, const float* host);
int deers_b200_gpt_param_get(deers_gpt* model, int index, int what, float* host);
int deers_b200_gpt_set_graph(deers_gpt* model, int enable);
int deers_b200_gpt_graph_active(const deers_gpt* model);   /* 1 once a step is being replayed from a captured graph */
int deers_b200_gpt_forward(deers_gpt* model, const int64_t* ids, int32_t B, int32_t T, float* logits);
int deers_b200_gpt_forward_backward(deers_gpt* model, const int64_t* ids, const int64_t* targets, int32_t B, int32_t T,
                                    float* loss_dev);
int deers_b200_gpt_train_step(deers_gpt* model, const int64_t* ids, const int64_t* targets, int32_t B, int32_t T,
                              const deers_adamw_hyper* hyper, double max_grad_norm, float* loss_dev,
                              float* grad_norm_dev);
int deers_b200_gpt_train_step_host(deers_gpt* model, const int64_t* ids_host, const int64_t* targets_host, int32_t B,
                                   int32_t T, const deers_adamw_hyper* hyper, double max_grad_norm, float* loss_host,
                                   float* grad_norm_host);

/*
 * Multi-GPU: (batch x head) shards over the GPUs of one box and the all-gather of O.  No counterpart in the
 * reference, which runs one context on device 0 (`src/storage/cuda.rs:455-462,503`; `Device::Cuda` carries no
 * ordinal, `src/device.rs:15-22`).  The slices of [B,H,T,D] are independent in forward and backward
 * (`src/models/gpt.rs:139-144` is batched over the two leading axes), so a rank runs deers_b200_attn_fwd / _bwd on
 * its own contiguous range of flattened (b*H + h) slices and nothing is exchanged for the gradients.
 *
 *   shard_range     [begin, end) of the slices rank owns: contiguous, the first n mod world ranks one longer.
 *   comm_init_all   one process, one context per GPU: full_buffers[r] is rank r's [n_slices, T, D] gather
 *                   buffer (device memory of ctxs[r]'s GPU, `bytes` long); enables peer access between the GPUs
 *                   and writes one communicator per rank to out[0..n).
 *   comm_export /   one process per GPU: export writes a DEERS_IPC_HANDLE_BYTES handle of this rank's buffer
 *   comm_init_ipc   (memory from cudaMalloc, possibly carved out of a larger allocation by a caching allocator;
 *                   stream-ordered pool memory such as deers_b200_alloc's is NOT exportable); the host program
 *                   passes all ranks' handles, in rank order, to init_ipc on every rank.
 *   allgather_o     pushes bytes [offset, offset + bytes) of this rank's buffer (normally the range its forward
 *                   just wrote its O slices to) into the same range of every peer's buffer: one device-to-device
 *                   copy per peer over NVLink, each on its own stream, ordered after the work already enqueued on
 *                   the context's stream.  The copies run on the copy engines and take no SM from the kernels that
 *                   follow (the persistent backward kernels want one CTA on every SM).  Returns at once.
 *   comm_set_lanes  how many of a call's world - 1 pushes are in flight at once (1 .. world - 1; default 1).  The
 *                   pushes are dealt round-robin onto that many copy streams; with one lane they leave one after the
 *                   other, each with the whole link, in an order in which no two ranks send to the same GPU at a time.
 *   allgather_join  makes the context's stream wait for this rank's pushes (no host wait).
 *   allgather_flush host-side wait for this rank's pushes.  A peer's slices are complete in this rank's buffer once
 *                   THAT peer's pushes have finished: exchange that fact on the host (the transport that carried the
 *                   handles, a barrier) after flush and before reading the gathered O.  A failed copy (a peer that
 *                   went away) surfaces as DEERS_ERR_CUDA from the call that meets it, never as a device-side wait.
 * No kernel of this library reads another GPU's memory.
 */
#define DEERS_IPC_HANDLE_BYTES 72
typedef struct deers_comm deers_comm;
void deers_b200_shard_range(int64_t n_slices, int32_t world, int32_t rank, int64_t* begin, int64_t* end);
int deers_b200_comm_init_all(int32_t n, deers_ctx* const* ctxs, void* const* full_buffers, size_t bytes, deers_comm** out);
int deers_b200_comm_export(deers_ctx* ctx, void* buffer, unsigned char* handle);
int deers_b200_comm_init_ipc(deers_ctx* ctx, int32_t rank, int32_t world, void* local_buffer, size_t bytes,
                             const unsigned char* handles, deers_comm** out);
void deers_b200_comm_destroy(deers_comm* comm);
int deers_b200_comm_set_lanes(deers_comm* comm, int32_t lanes);
int deers_b200_allgather_o(deers_comm* comm, size_t offset, size_t bytes);
int deers_b200_allgather_join(deers_comm* comm);
int deers_b200_allgather_flush(deers_comm* comm);

/*
 * Status text, the way backend failures become `Error::Cuda(String)`
 * (`src/error.rs:40-41`).  last_error adds the detail of the most recent failure
 * on this context (CUDA error string, or which kernel wait gave up).
 */
const char* deers_b200_status_string(int status);
const char* deers_b200_last_error(deers_ctx* ctx);

/*
 * Number of kernel launches this context has enqueued so far (the reference
 * counts launches per op in its profiler, `src/profiler.rs:160-224`).
 */
uint64_t deers_b200_launch_count(deers_ctx* ctx);

/*
 * Per-kernel device timing, the counterpart of the reference's profiler hook that
 * brackets every launch with two CUDA events (`src/storage/cuda.rs:530-561`).
 * While enabled, each launch of the attention path is bracketed by events on the
 * context's stream.  kernel_time() synchronises the stream and returns the total
 * milliseconds and the number of launches of one kernel kind since timing was
 * enabled (or since the last call with reset != 0).
 */
enum { DEERS_K_FWD = 0, DEERS_K_BWD_PREP = 1, DEERS_K_BWD_MAIN = 2, DEERS_K_BWD_DQ = 3, DEERS_K_ROPE = 4, DEERS_K_OPTIM = 5, DEERS_K_NORM = 6, DEERS_K_DECODE = 7, DEERS_K_GEMM = 8, DEERS_K_GPT = 9, DEERS_K_GEMM_X3 = 10, DEERS_K_COUNT = 11 };
int deers_b200_kernel_timing(deers_ctx* ctx, int enable);
int deers_b200_kernel_time(deers_ctx* ctx, int kind, int reset, double* total_ms, uint64_t* launches);

/*
 * Tensor-core self-test: runs one small tcgen05 GEMM per operand layout the f16
 * kernels rely on (K-major and MN-major shared-memory operands, TMA 128-byte
 * swizzle, A operand in tensor memory) and compares with a host product.
 * `max_abs_err` (DEERS_SELFTEST_CASES floats, host memory) receives the error of
 * each case.  No counterpart in the reference,
 * whose GEMMs are cuBLAS calls (`src/storage/cuda.rs:1098-1177`).
 */
enum { DEERS_SELFTEST_CASES = 6 };
int deers_b200_selftest_umma(deers_ctx* ctx, float* max_abs_err);

/*
 * Bounded-wait self-test: runs the give-up path of the device-side waits without a fault or a hang.  One small
 * kernel waits, through the same helper every kernel of the library uses, on a barrier that nothing completes,
 * with a limit of `limit_ms` (1..1000) milliseconds instead of the usual two seconds.  result (4 ints, host):
 * [0] 1 if the first wait gave up, [1] 1 if a second wait in the same CTA returned through the abort flag,
 * [2], [3] the microseconds each of them spent.  The call waits for the kernel but leaves the error word set:
 * the next deers_b200_sync() returns DEERS_ERR_KERNEL and clears it; until then the persistent f16 kernels,
 * which read the word when they start, return without writing their outputs.  No counterpart in the
 * reference (it has no device-side waits).
 */
int deers_b200_selftest_wait(deers_ctx* ctx, uint32_t limit_ms, int32_t* result);

#if defined(__GNUC__)
#pragma GCC visibility pop
#endif

#ifdef __cplusplus
}
#endif
#endif /* DEERS_B200_H */
