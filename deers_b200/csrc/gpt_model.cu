// The f32 GPT of src/models/gpt.rs as a device-resident object and its training step.
//
// Forward (GPT::forward, gpt.rs:329-355), per block (Block::forward, gpt.rs:236-240):
//   n1 = rmsnorm(x); qkv = n1 * [Wq|Wk|Wv] (one GEMM); q, k rotated and packed head-major in one launch
//   (rope over 2H "heads" of the fused buffer), v read in place as a strided view; fused attention writing
//   O token-major; x1 = x + O * Wout (residual in the GEMM epilogue); n2 = rmsnorm(x1);
//   r = relu(n2 * Wup), h = r*r (GEMM epilogue); x2 = x1 + h * Wdown (epilogue).
// Head: xf = rmsnorm(x); logits = xf * Wlm; cross-entropy reads the logits once; the backward overwrites
// them with their gradient in one pass and feeds the two head GEMMs.
// Backward: the exact transposes of the above, with the relu^2 backward in a GEMM epilogue, the residual
// gradient added inside the RMSNorm backward, dQ / dK rotated back straight into the fused [N, 3C]
// gradient buffer next to dV, and one GEMM each for d[Wq|Wk|Wv] and for the sum of the three input
// gradients.  Every launch is one of this library's kernels; there is no host round trip in a step.
// The weight gradients are off the critical path (nothing in the backward reads them): they run on a second
// stream, forked from the main one where their operands are complete and joined before the gradient norm;
// captured, the two streams become two branches of the step's graph.
#include "common.cuh"

#include <math.h>
#include <new>
#include <string>
#include <vector>

namespace {

struct LayerW {              // offsets (in floats) into the parameter-shaped arenas
    size_t qkv, out, up, down;
};

struct LayerAct {
    float *n1, *inv1, *qkv, *qk, *o, *lse, *x1, *inv2, *n2, *r, *h, *x2;
};

size_t align64(size_t n) { return (n + 63) / 64 * 64; }     // floats: 256-byte boundaries

}  // namespace

struct deers_gpt {
    deers_ctx* ctx;
    deers_gpt_config cfg;
    int max_batch;
    long long max_tokens;
    int D, Vld;
    // parameter-shaped arenas: weights, gradients, first and second moments
    size_t arena_floats;
    float* arena[4];
    size_t off_wte, off_lm;
    std::vector<LayerW> lw;
    std::vector<deers_optim_tensor> opt;           // one entry per physical buffer
    // activations
    float* act_base;
    float *x0, *invf, *xf, *logits, *ce_lse, *picked, *cosv, *sinv;
    std::vector<LayerAct> la;
    float *dx_a, *dx_b, *dtmp, *dh, *dqkv, *dqk, *attn_ws;
    size_t attn_ws_bytes;
    void* gemm_ws;
    void* gemm_ws_side;          // split-K workspace of the weight-gradient stream
    size_t gemm_ws_bytes;
    // second stream for the weight gradients; events are markers only (no timing)
    cudaStream_t side;
    cudaEvent_t ev_fork, ev_join, ev_done[4];
    bool done_valid[4];          // ev_done[i] was recorded in the current backward pass
    bool on_side;                // launches currently go to the side stream
    void* optim_scratch;
    float *loss_dev, *norm_dev;
    long long *ids_dev, *tgt_dev;
    // The head on the tensor core (gemm_f16x3_sm100.cu): f16 pairs of xf, of the head weight and of dlogits
    bool tc_head;
    void *xf_hi, *xf_lo, *w_hi, *w_lo, *dl_hi, *dl_lo;
    void* x3_ws;
    void* x3_ws_side;
    size_t x3_ws_bytes;
    // pinned staging for train_step_host
    long long* ids_pin;
    float* out_pin;
    // CUDA graph of forward + loss + backward + gradient norm, for the last (B, T) seen
    bool graph_enabled;
    cudaGraphExec_t graph_exec;
    int graph_B, graph_T;
    int eager_steps_BT;          // eager steps run at (graph_B, graph_T) before capturing
};

namespace {

#define GPT_TRY(expr)              \
    do {                           \
        int _rc = (expr);          \
        if (_rc) return _rc;       \
    } while (0)

int gemm(deers_gpt* m, int M, int N, int K, const float* a, long long lda, int a_mn, const float* b, long long ldb, int b_mn,
         float* c, long long ldc, int epi = DEERS_EPI_NONE, const float* r = nullptr, long long ldr = 0,
         float* aux = nullptr) {
    return launch_gemm_f32(m->ctx, M, N, K, a, lda, a_mn, b, ldb, b_mn, c, ldc, epi, r, ldr, aux,
                           m->on_side ? m->gemm_ws_side : m->gemm_ws, m->gemm_ws_bytes, true);
}

// Launches made while a SideScope lives go to the weight-gradient stream, ordered after everything the main
// stream holds at construction.  done(i) marks the side stream's progress for a later wait_done(i) on the
// main stream (before it overwrites a buffer the side work reads).  With kernel timing on, or without a
// second stream, everything stays on the main stream.
struct SideScope {
    deers_gpt* m;
    cudaStream_t main;
    bool active;
    int rc;
    explicit SideScope(deers_gpt* m_) : m(m_), main(m_->ctx->stream), active(m_->side && !m_->ctx->timing), rc(DEERS_OK) {
        if (!active) return;
        if (cudaEventRecord(m->ev_fork, main) != cudaSuccess || cudaStreamWaitEvent(m->side, m->ev_fork, 0) != cudaSuccess) {
            rc = DEERS_ERR_CUDA;
            active = false;
            return;
        }
        m->ctx->stream = m->side;
        m->on_side = true;
    }
    int done(int i) {
        if (!active) return rc;
        if (cudaEventRecord(m->ev_done[i], m->side) != cudaSuccess) return DEERS_ERR_CUDA;
        m->done_valid[i] = true;
        return DEERS_OK;
    }
    ~SideScope() {
        if (active) { m->ctx->stream = main; m->on_side = false; }
    }
};

int wait_done(deers_gpt* m, int i) {
    if (!m->done_valid[i]) return DEERS_OK;
    return cudaStreamWaitEvent(m->ctx->stream, m->ev_done[i], 0) == cudaSuccess ? DEERS_OK : DEERS_ERR_CUDA;
}

// The main stream waits for all side work enqueued so far.
int join_side(deers_gpt* m) {
    if (!m->side || m->ctx->timing) return DEERS_OK;
    if (cudaEventRecord(m->ev_join, m->side) != cudaSuccess || cudaStreamWaitEvent(m->ctx->stream, m->ev_join, 0) != cudaSuccess)
        return DEERS_ERR_CUDA;
    return DEERS_OK;
}

void attn_desc(const deers_gpt* m, int B, int T, deers_attn_desc* d) {
    const int H = m->cfg.n_head, D = m->D, C = m->cfg.n_embd;
    memset(d, 0, sizeof(*d));
    d->B = B; d->H = H; d->T = T; d->D = D;
    d->dtype = DEERS_F32; d->causal = 1;
    d->scale = (float)(1.0 / sqrt((double)D));                       // gpt.rs:139, storage.rs:115-117
    const int64_t qk[4] = {(int64_t)2 * H * T * D, (int64_t)T * D, D, 1};        // inside the [B, 2H, T, D] pack
    const int64_t v[4] = {(int64_t)T * 3 * C, D, (int64_t)3 * C, 1};             // column slice of [N, 3C]
    const int64_t o[4] = {(int64_t)T * C, D, C, 1};                              // token-major [B, T, H, D]
    for (int i = 0; i < 4; ++i) {
        d->q_strides[i] = qk[i]; d->k_strides[i] = qk[i]; d->dq_strides[i] = qk[i]; d->dk_strides[i] = qk[i];
        d->v_strides[i] = v[i]; d->dv_strides[i] = v[i];
        d->o_strides[i] = o[i]; d->do_strides[i] = o[i];
    }
}

void rope_desc(const deers_gpt* m, int B, int T, int inverse, deers_rope_desc* d) {
    const int H = m->cfg.n_head, D = m->D, C = m->cfg.n_embd;
    memset(d, 0, sizeof(*d));
    d->B = B; d->T = T; d->H = 2 * H; d->D = D;                      // q and k heads side by side
    d->dtype = DEERS_F32; d->inverse = inverse;
    const int64_t tok[4] = {(int64_t)T * 3 * C, (int64_t)3 * C, D, 1};           // (b, t, h, d) in [N, 3C]
    const int64_t head[4] = {(int64_t)2 * H * T * D, D, (int64_t)T * D, 1};      // (b, t, h, d) in [B, 2H, T, D]
    for (int i = 0; i < 4; ++i) {
        d->src_strides[i] = inverse ? head[i] : tok[i];
        d->dst_strides[i] = inverse ? tok[i] : head[i];
    }
}

int forward(deers_gpt* m, const long long* ids, int B, int T) {
    deers_ctx* ctx = m->ctx;
    const deers_gpt_config& c = m->cfg;
    const int C = c.n_embd, Hm = c.mlp_hidden_dim, V = c.vocab_size, H = c.n_head, D = m->D;
    const long long N = (long long)B * T;
    float* W = m->arena[0];
    for (bool& v : m->done_valid) v = false;
    if (m->tc_head) {
        // the head weight's f16 pair (it changes every step) is made beside the blocks, not in front of the head
        SideScope side(m);
        GPT_TRY(side.rc);
        GPT_TRY(launch_split_f16x3(ctx, C, V, W + m->off_lm, m->Vld, 1.0f, m->w_hi, m->w_lo, m->Vld));
        GPT_TRY(side.done(0));
    }
    GPT_TRY(launch_embedding_fwd(ctx, W + m->off_wte, ids, N, C, V, m->x0));                 // gpt.rs:343
    deers_attn_desc ad;
    attn_desc(m, B, T, &ad);
    deers_rope_desc rd;
    rope_desc(m, B, T, 0, &rd);
    const float* x = m->x0;
    for (int l = 0; l < c.n_layer; ++l) {
        const LayerW& w = m->lw[l];
        LayerAct& a = m->la[l];
        GPT_TRY(launch_rmsnorm_fwd(ctx, N, C, c.rms_norm_eps, x, a.n1, a.inv1));             // norm1
        GPT_TRY(gemm(m, (int)N, 3 * C, C, a.n1, C, 0, W + w.qkv, 3 * C, 1, a.qkv, 3 * C));   // q | k | v projections
        GPT_TRY(deers_b200_rope_pack(ctx, &rd, a.qkv, m->cosv, m->sinv, a.qk));              // gpt.rs:135-136
        GPT_TRY(deers_b200_attn_fwd(ctx, &ad, a.qk, a.qk + (size_t)H * T * D, a.qkv + 2 * C, a.o, a.lse, nullptr, 0));
        GPT_TRY(gemm(m, (int)N, C, C, a.o, C, 0, W + w.out, C, 1, a.x1, C, DEERS_EPI_ADD, x, C));       // x + out_proj
        GPT_TRY(launch_rmsnorm_fwd(ctx, N, C, c.rms_norm_eps, a.x1, a.n2, a.inv2));          // norm2
        GPT_TRY(gemm(m, (int)N, Hm, C, a.n2, C, 0, W + w.up, Hm, 1, a.h, Hm, DEERS_EPI_RELU_SQ, nullptr, 0, a.r));
        GPT_TRY(gemm(m, (int)N, C, Hm, a.h, Hm, 0, W + w.down, C, 1, a.x2, C, DEERS_EPI_ADD, a.x1, C)); // x1 + down_proj
        x = a.x2;
    }
    GPT_TRY(launch_rmsnorm_fwd(ctx, N, C, c.rms_norm_eps, x, m->xf, m->invf));               // gpt.rs:347
    if (m->tc_head) {
        // lm_head on the tensor core at f32 accuracy: both operands as f16 pairs (the weight changes every step)
        GPT_TRY(launch_split_f16x3(ctx, N, C, m->xf, C, 1.0f, m->xf_hi, m->xf_lo, C));
        GPT_TRY(wait_done(m, 0));
        GPT_TRY(launch_gemm_f16x3(ctx, (int)N, V, C, m->xf_hi, m->xf_lo, C, 0, m->w_hi, m->w_lo, m->Vld, 1, m->logits, m->Vld,
                                  1.0f, m->x3_ws, m->x3_ws_bytes));
    } else {
        GPT_TRY(gemm(m, (int)N, V, C, m->xf, C, 0, W + m->off_lm, m->Vld, 1, m->logits, m->Vld)); // lm_head
    }
    return DEERS_OK;
}

int loss_and_backward(deers_gpt* m, const long long* ids, const long long* targets, int B, int T) {
    deers_ctx* ctx = m->ctx;
    const deers_gpt_config& c = m->cfg;
    const int C = c.n_embd, Hm = c.mlp_hidden_dim, V = c.vocab_size, H = c.n_head, D = m->D;
    const long long N = (long long)B * T;
    const int Vld = m->Vld;
    float* W = m->arena[0];
    float* G = m->arena[1];
    for (bool& v : m->done_valid) v = false;
    GPT_TRY(launch_cross_entropy_fwd(ctx, m->logits, Vld, targets, N, V, m->ce_lse, m->picked, m->loss_dev));
    const float* x_last = c.n_layer ? m->la[c.n_layer - 1].x2 : m->x0;
    if (m->tc_head) {
        // dlogits leave the cross-entropy backward as f16 pairs scaled by rows * 4096 (|dlogit| <= 1 / rows)
        const float dscale = (float)N * 4096.0f;
        GPT_TRY(launch_cross_entropy_bwd_split(ctx, m->logits, Vld, targets, m->ce_lse, N, V, 1.0f, dscale, m->dl_hi, m->dl_lo, Vld));
        GPT_TRY(launch_gemm_f16x3(ctx, (int)N, C, V, m->dl_hi, m->dl_lo, Vld, 0, m->w_hi, m->w_lo, Vld, 0, m->dtmp, C,
                                  1.0f / dscale, m->x3_ws, m->x3_ws_bytes));                  // d xf = dlogits Wlm^T
        {
            SideScope side(m);
            GPT_TRY(side.rc);
            GPT_TRY(launch_gemm_f16x3(ctx, C, V, (int)N, m->xf_hi, m->xf_lo, C, 1, m->dl_hi, m->dl_lo, Vld, 1, G + m->off_lm, Vld,
                                      1.0f / dscale, m->x3_ws_side, m->x3_ws_bytes));         // d lm_head = xf^T dlogits
        }
    } else {
        GPT_TRY(launch_cross_entropy_bwd(ctx, m->logits, Vld, targets, m->ce_lse, N, V, 1.0f, m->logits, Vld));
        GPT_TRY(gemm(m, (int)N, C, V, m->logits, Vld, 0, W + m->off_lm, Vld, 0, m->dtmp, C));    // d xf = dlogits Wlm^T
        {
            SideScope side(m);
            GPT_TRY(side.rc);
            GPT_TRY(gemm(m, C, V, (int)N, m->xf, C, 1, m->logits, Vld, 1, G + m->off_lm, Vld));  // d lm_head = xf^T dlogits
        }
    }
    GPT_TRY(launch_rmsnorm_bwd(ctx, N, C, x_last, m->invf, m->dtmp, nullptr, m->dx_a));
    deers_attn_desc ad;
    attn_desc(m, B, T, &ad);
    deers_rope_desc rd;
    rope_desc(m, B, T, 1, &rd);
    for (int l = c.n_layer - 1; l >= 0; --l) {
        const LayerW& w = m->lw[l];
        LayerAct& a = m->la[l];
        const float* x_in = l ? m->la[l - 1].x2 : m->x0;
        // MLP branch: x2 = x1 + relu(n2 Wup)^2 Wdown
        {
            SideScope side(m);
            GPT_TRY(side.rc);
            GPT_TRY(gemm(m, Hm, C, (int)N, a.h, Hm, 1, m->dx_a, C, 1, G + w.down, C));       // d Wdown = h^T dx
            GPT_TRY(side.done(0));
        }
        GPT_TRY(wait_done(m, 1));                                                            // the previous d Wup has read dh
        GPT_TRY(gemm(m, (int)N, Hm, C, m->dx_a, C, 0, W + w.down, C, 0, m->dh, Hm, DEERS_EPI_MUL_AUX2, nullptr, 0, a.r));
        {
            SideScope side(m);
            GPT_TRY(side.rc);
            GPT_TRY(gemm(m, C, Hm, (int)N, a.n2, C, 1, m->dh, Hm, 1, G + w.up, Hm));         // d Wup = n2^T du
            GPT_TRY(side.done(1));
        }
        GPT_TRY(gemm(m, (int)N, C, Hm, m->dh, Hm, 0, W + w.up, Hm, 0, m->dtmp, C));          // d n2 = du Wup^T
        GPT_TRY(wait_done(m, 2));                                                            // the previous d Wout has read dx_b
        GPT_TRY(launch_rmsnorm_bwd(ctx, N, C, a.x1, a.inv2, m->dtmp, m->dx_a, m->dx_b));     // d x1
        // attention branch: x1 = x + attn(n1) Wout
        {
            SideScope side(m);
            GPT_TRY(side.rc);
            GPT_TRY(gemm(m, C, C, (int)N, a.o, C, 1, m->dx_b, C, 1, G + w.out, C));          // d Wout = o^T dx1
            GPT_TRY(side.done(2));
        }
        GPT_TRY(gemm(m, (int)N, C, C, m->dx_b, C, 0, W + w.out, C, 0, m->dtmp, C));          // d o (token-major)
        GPT_TRY(wait_done(m, 3));                                                            // the previous d Wqkv has read dqkv
        GPT_TRY(deers_b200_attn_bwd(ctx, &ad, a.qk, a.qk + (size_t)H * T * D, a.qkv + 2 * C, a.o, a.lse, m->dtmp, m->dqk,
                                    m->dqk + (size_t)H * T * D, m->dqkv + 2 * C, m->attn_ws, m->attn_ws_bytes));
        GPT_TRY(deers_b200_rope_pack(ctx, &rd, m->dqk, m->cosv, m->sinv, m->dqkv));          // d q | d k back to [N, 3C]
        {
            SideScope side(m);
            GPT_TRY(side.rc);
            GPT_TRY(gemm(m, C, 3 * C, (int)N, a.n1, C, 1, m->dqkv, 3 * C, 1, G + w.qkv, 3 * C)); // d [Wq|Wk|Wv]
            GPT_TRY(side.done(3));
        }
        GPT_TRY(gemm(m, (int)N, C, 3 * C, m->dqkv, 3 * C, 0, W + w.qkv, 3 * C, 0, m->dtmp, C)); // d n1 (three terms in one)
        GPT_TRY(wait_done(m, 0));                                                            // this layer's d Wdown has read dx_a
        GPT_TRY(launch_rmsnorm_bwd(ctx, N, C, x_in, a.inv1, m->dtmp, m->dx_b, m->dx_a));     // d x
    }
    GPT_TRY(launch_embedding_bwd(ctx, m->dx_a, ids, N, C, V, G + m->off_wte));
    return join_side(m);
}

int grad_norm(deers_gpt* m) {
    return deers_b200_grad_norm(m->ctx, (int)m->opt.size(), m->opt.data(), m->norm_dev, m->optim_scratch,
                                deers_b200_optim_scratch_bytes());
}

int check_bt(const deers_gpt* m, int B, int T) {
    if (B < 1 || T < 1 || B > m->max_batch || T > m->cfg.sequence_len) return DEERS_ERR_SHAPE;   // gpt.rs:335
    return DEERS_OK;
}

// Brings the caller's ids / targets into the model's own buffers, so that a captured graph reads fixed addresses.
int stage_ids(deers_gpt* m, const int64_t* ids, const int64_t* targets, long long N, cudaMemcpyKind kind) {
    deers_ctx* ctx = m->ctx;
    if ((const long long*)ids != m->ids_dev)
        DEERS_CUDA_TRY(ctx, cudaMemcpyAsync(m->ids_dev, ids, (size_t)N * sizeof(long long), kind, ctx->stream));
    if (targets && (const long long*)targets != m->tgt_dev)
        DEERS_CUDA_TRY(ctx, cudaMemcpyAsync(m->tgt_dev, targets, (size_t)N * sizeof(long long), kind, ctx->stream));
    return DEERS_OK;
}

void drop_graph(deers_gpt* m) {
    if (m->graph_exec) cudaGraphExecDestroy(m->graph_exec);
    m->graph_exec = nullptr;
}

// forward + loss + backward + gradient norm on the staged ids, replayed from a graph once a (B, T) repeats
int run_fwd_bwd(deers_gpt* m, int B, int T, bool with_norm) {
    deers_ctx* ctx = m->ctx;
    const bool can_graph = m->graph_enabled && with_norm && !ctx->timing;
    if (can_graph && m->graph_exec && m->graph_B == B && m->graph_T == T) {
        DEERS_CUDA_TRY(ctx, cudaGraphLaunch(m->graph_exec, ctx->stream));
        ctx->launches += 1;
        return DEERS_OK;
    }
    if (can_graph && (m->graph_B != B || m->graph_T != T)) {
        drop_graph(m);
        m->graph_B = B; m->graph_T = T; m->eager_steps_BT = 0;
    }
    if (can_graph && m->eager_steps_BT >= 1) {
        // the shape has run eagerly once (every kernel's attributes are set): capture it
        cudaGraph_t graph = nullptr;
        if (cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal) == cudaSuccess) {
            int rc = forward(m, m->ids_dev, B, T);
            if (!rc) rc = loss_and_backward(m, m->ids_dev, m->tgt_dev, B, T);
            if (!rc) rc = grad_norm(m);
            const cudaError_t ce = cudaStreamEndCapture(ctx->stream, &graph);
            if (!rc && ce == cudaSuccess && graph &&
                cudaGraphInstantiate(&m->graph_exec, graph, 0) == cudaSuccess) {
                cudaGraphDestroy(graph);
                DEERS_CUDA_TRY(ctx, cudaGraphLaunch(m->graph_exec, ctx->stream));
                ctx->launches += 1;
                return DEERS_OK;
            }
            if (graph) cudaGraphDestroy(graph);
            m->graph_exec = nullptr;
            cudaGetLastError();
            m->graph_enabled = false;                                 // stay eager from here on
            if (rc) return rc;
        } else {
            cudaGetLastError();
            m->graph_enabled = false;
        }
    }
    GPT_TRY(forward(m, m->ids_dev, B, T));
    GPT_TRY(loss_and_backward(m, m->ids_dev, m->tgt_dev, B, T));
    if (with_norm) GPT_TRY(grad_norm(m));
    if (can_graph) m->eager_steps_BT += 1;
    return DEERS_OK;
}

const char* kBlockNames[6] = {"attn.q_proj", "attn.k_proj", "attn.v_proj", "attn.out_proj", "mlp.up_proj", "mlp.down_proj"};

// Logical parameter `index` -> device pointer inside arena `what`, shape and row stride.
int locate(const deers_gpt* m, int index, int what, float** ptr, long long* rows, long long* cols, long long* ld) {
    const deers_gpt_config& c = m->cfg;
    const int n = 2 + 6 * c.n_layer;
    if (index < 0 || index >= n || what < 0 || what > 3) return DEERS_ERR_SHAPE;
    float* base = m->arena[what];
    const int C = c.n_embd, Hm = c.mlp_hidden_dim;
    if (index == 0) { *ptr = base + m->off_wte; *rows = c.vocab_size; *cols = C; *ld = C; return DEERS_OK; }
    if (index == n - 1) { *ptr = base + m->off_lm; *rows = C; *cols = c.vocab_size; *ld = m->Vld; return DEERS_OK; }
    const int l = (index - 1) / 6, k = (index - 1) % 6;
    const LayerW& w = m->lw[l];
    switch (k) {
        case 0: case 1: case 2: *ptr = base + w.qkv + (size_t)k * C; *rows = C; *cols = C; *ld = 3 * C; break;
        case 3: *ptr = base + w.out; *rows = C; *cols = C; *ld = C; break;
        case 4: *ptr = base + w.up; *rows = C; *cols = Hm; *ld = Hm; break;
        default: *ptr = base + w.down; *rows = Hm; *cols = C; *ld = C; break;
    }
    return DEERS_OK;
}

}  // namespace

extern "C" int deers_b200_gpt_create(deers_ctx* ctx, const deers_gpt_config* cfg, int32_t max_batch, deers_gpt** out) {
    if (!ctx || !cfg || !out) return DEERS_ERR_NULL;
    *out = nullptr;
    if (cfg->vocab_size < 1 || cfg->sequence_len < 1 || cfg->n_layer < 0 || cfg->n_head < 1 || cfg->n_embd < 1 ||
        cfg->mlp_hidden_dim < 1 || max_batch < 1)
        return DEERS_ERR_SHAPE;
    if (cfg->n_embd % cfg->n_head) return DEERS_ERR_SHAPE;            // "n_embd must be divisible by n_head", gpt.rs:301
    const int D = cfg->n_embd / cfg->n_head;
    if (D % 2 || D > 128) return DEERS_ERR_SHAPE;                     // RoPE needs an even head_dim; f32 attention D <= 128
    if (2 + 4 * cfg->n_layer > 256) return DEERS_ERR_SHAPE;           // optimizer tensors per call
    const long long max_tokens = (long long)max_batch * cfg->sequence_len;
    if (max_tokens > 65535) return DEERS_ERR_SHAPE;                   // rows of the cross-entropy backward grid
    DEERS_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    deers_gpt* m = new (std::nothrow) deers_gpt();
    if (!m) return DEERS_ERR_CUDA;
    m->ctx = ctx; m->cfg = *cfg; m->max_batch = max_batch; m->max_tokens = max_tokens; m->D = D;
    m->Vld = (cfg->vocab_size + 7) / 8 * 8;                           // rows of the head, of the logits and of their f16 pairs start 16-byte aligned
    // Heads that fill the tensor core take the split-f16 products; small ones stay on the FFMA kernel.
    m->tc_head = cfg->vocab_size >= 1024 && cfg->n_embd % 8 == 0 && cfg->n_embd >= 64;
    m->graph_enabled = true; m->graph_exec = nullptr; m->graph_B = m->graph_T = -1; m->eager_steps_BT = 0;
    m->on_side = false;
    {
        // the weight-gradient stream and its markers; without them the step simply runs on one stream
        bool ok = cudaStreamCreateWithFlags(&m->side, cudaStreamNonBlocking) == cudaSuccess;
        if (!ok) m->side = nullptr;
        cudaEvent_t* evs[6] = {&m->ev_fork, &m->ev_join, &m->ev_done[0], &m->ev_done[1], &m->ev_done[2], &m->ev_done[3]};
        for (cudaEvent_t* e : evs)
            if (cudaEventCreateWithFlags(e, cudaEventDisableTiming) != cudaSuccess) { *e = nullptr; ok = false; }
        if (!ok && m->side) { cudaStreamDestroy(m->side); m->side = nullptr; }
        cudaGetLastError();
    }
    const size_t C = cfg->n_embd, Hm = cfg->mlp_hidden_dim, V = cfg->vocab_size, N = (size_t)max_tokens;

    // ---- parameter-shaped arenas
    size_t off = 0;
    auto take = [&off](size_t n) { const size_t o = off; off += align64(n); return o; };
    m->off_wte = take(V * C);
    m->lw.resize(cfg->n_layer);
    for (auto& w : m->lw) { w.qkv = take(C * 3 * C); w.out = take(C * C); w.up = take(C * Hm); w.down = take(Hm * C); }
    m->off_lm = take(C * (size_t)m->Vld);
    m->arena_floats = off;
    int rc = DEERS_OK;
    for (int a = 0; a < 4 && !rc; ++a) {
        if (cudaMalloc((void**)&m->arena[a], off * sizeof(float)) != cudaSuccess ||
            cudaMemsetAsync(m->arena[a], 0, off * sizeof(float), ctx->stream) != cudaSuccess)
            rc = DEERS_ERR_CUDA;
    }
    auto add_opt = [m](size_t o, size_t n) {
        deers_optim_tensor t;
        t.w = m->arena[0] + o; t.g = m->arena[1] + o; t.m = m->arena[2] + o; t.v = m->arena[3] + o; t.n = (int64_t)n;
        m->opt.push_back(t);
    };
    if (!rc) {
        add_opt(m->off_wte, V * C);
        for (auto& w : m->lw) { add_opt(w.qkv, C * 3 * C); add_opt(w.out, C * C); add_opt(w.up, C * Hm); add_opt(w.down, Hm * C); }
        add_opt(m->off_lm, C * (size_t)m->Vld);
    }

    // ---- activations, scratch
    off = 0;
    const size_t HTD = N * C;                                          // B * H * T * D
    struct Slot { float** p; size_t n; };
    std::vector<Slot> slots;
    auto want = [&slots](float** p, size_t n) { slots.push_back({p, n}); };
    want(&m->x0, N * C); want(&m->invf, N); want(&m->xf, N * C); want(&m->logits, N * (size_t)m->Vld);
    want(&m->ce_lse, N); want(&m->picked, N);
    want(&m->cosv, (size_t)cfg->sequence_len * (D / 2)); want(&m->sinv, (size_t)cfg->sequence_len * (D / 2));
    m->la.resize(cfg->n_layer);
    for (auto& a : m->la) {
        want(&a.n1, N * C); want(&a.inv1, N); want(&a.qkv, N * 3 * C); want(&a.qk, 2 * HTD); want(&a.o, N * C);
        want(&a.lse, N * cfg->n_head); want(&a.x1, N * C); want(&a.inv2, N); want(&a.n2, N * C);
        want(&a.r, N * Hm); want(&a.h, N * Hm); want(&a.x2, N * C);
    }
    want(&m->dx_a, N * C); want(&m->dx_b, N * C); want(&m->dtmp, N * C); want(&m->dh, N * Hm);
    want(&m->dqkv, N * 3 * C); want(&m->dqk, 2 * HTD);
    deers_attn_desc ad;
    attn_desc(m, max_batch, cfg->sequence_len, &ad);
    m->attn_ws_bytes = deers_b200_attn_workspace_bytes(&ad, 1);
    want(&m->attn_ws, m->attn_ws_bytes / sizeof(float) + 64);
    want(&m->loss_dev, 64);
    m->norm_dev = nullptr;
    size_t total = 0;
    for (auto& s : slots) total += align64(s.n);
    // split-K workspace: the largest any GEMM of the step asks for (tokens vary: take the maximum over B*T <= N by
    // probing the shapes at full size, which is where the partial tiles are largest)
    size_t gws = 0;
    {
        const int n = (int)N, c = (int)C, h = (int)Hm, v = (int)V;
        const int shapes[][3] = {{n, 3 * c, c}, {n, c, c}, {n, h, c}, {n, c, h}, {n, v, c}, {c, v, n}, {n, c, v},
                                 {h, c, n}, {c, h, n}, {c, c, n}, {c, 3 * c, n}, {n, c, 3 * c}};
        for (auto& s : shapes) {
            for (int frac = 1; frac <= 64; frac *= 2) {               // smaller batches change the split, not the bound by much
                const int tok = n / frac > 0 ? n / frac : 1;
                const int M2 = s[0] == n ? tok : s[0], N2 = s[1] == n ? tok : s[1], K2 = s[2] == n ? tok : s[2];
                const size_t b = gemm_f32_workspace_bytes(ctx, M2, N2, K2);
                gws = b > gws ? b : gws;
            }
        }
    }
    // any token count in between stays below (tiles + 3 * SMs) partial tiles of at most 128 x 128 floats
    const size_t gws_floor = (size_t)5 * ctx->sm_count * 128 * 128 * sizeof(float) + 65536;
    if (gws < gws_floor) gws = gws_floor;
    m->gemm_ws_bytes = gws;
    const size_t opt_bytes = deers_b200_optim_scratch_bytes();
    const size_t id_bytes = ((size_t)N * sizeof(long long) + 255) / 256 * 256;
    auto up256 = [](size_t b) { return (b + 255) / 256 * 256; };
    const size_t xf_h = up256(N * C * 2), w_h = up256(C * (size_t)m->Vld * 2), dl_h = up256(N * (size_t)m->Vld * 2);
    // K-split partial tiles of the head's input gradient: parts * tokens <= 148 * 128 * 128 / C + tokens
    const size_t x3 = m->tc_head ? up256(((size_t)148 * 16384 + N * C) * sizeof(float) * 2) : 0;
    m->x3_ws_bytes = x3;
    const size_t tc_bytes = m->tc_head ? 2 * (xf_h + w_h + dl_h) + 2 * x3 : 0;
    const size_t bytes = total * sizeof(float) + 2 * (gws + 256) + opt_bytes + 256 + 2 * id_bytes + tc_bytes;
    char* base = nullptr;
    if (!rc && cudaMalloc((void**)&base, bytes) != cudaSuccess) rc = DEERS_ERR_CUDA;
    if (!rc && cudaMemsetAsync(base, 0, bytes, ctx->stream) != cudaSuccess) rc = DEERS_ERR_CUDA;   // split-K counters start at zero
    if (!rc) {
        m->act_base = (float*)base;
        float* p = (float*)base;
        for (auto& s : slots) { *s.p = p; p += align64(s.n); }
        m->norm_dev = m->loss_dev + 1;
        char* q = (char*)p;
        m->gemm_ws = gws ? q : nullptr; q += (gws + 255) / 256 * 256;
        m->gemm_ws_side = gws ? q : nullptr; q += (gws + 255) / 256 * 256;
        m->optim_scratch = q; q += (opt_bytes + 255) / 256 * 256;
        m->ids_dev = (long long*)q; q += id_bytes;
        m->tgt_dev = (long long*)q; q += id_bytes;
        if (m->tc_head) {
            m->xf_hi = q; q += xf_h; m->xf_lo = q; q += xf_h;
            m->w_hi = q; q += w_h; m->w_lo = q; q += w_h;
            m->dl_hi = q; q += dl_h; m->dl_lo = q; q += dl_h;
            m->x3_ws = q; q += x3;
            m->x3_ws_side = q; q += x3;
        }
        // rotary cache, f32 arithmetic of gpt.rs:12-46
        const int half = D / 2;
        std::vector<float> hc((size_t)cfg->sequence_len * half), hs(hc.size());
        for (int t = 0; t < cfg->sequence_len; ++t)
            for (int i = 0; i < half; ++i) {
                const float channel = (float)(2 * i);
                const float inv_freq = 1.0f / powf(cfg->rope_base, channel / (float)D);
                const float f = (float)t * inv_freq;
                hc[(size_t)t * half + i] = cosf(f);
                hs[(size_t)t * half + i] = sinf(f);
            }
        if (cudaMemcpyAsync(m->cosv, hc.data(), hc.size() * sizeof(float), cudaMemcpyHostToDevice, ctx->stream) != cudaSuccess ||
            cudaMemcpyAsync(m->sinv, hs.data(), hs.size() * sizeof(float), cudaMemcpyHostToDevice, ctx->stream) != cudaSuccess ||
            cudaStreamSynchronize(ctx->stream) != cudaSuccess)
            rc = DEERS_ERR_CUDA;
    }
    if (!rc && (cudaHostAlloc((void**)&m->ids_pin, 2 * (size_t)N * sizeof(long long), cudaHostAllocDefault) != cudaSuccess ||
                cudaHostAlloc((void**)&m->out_pin, 2 * sizeof(float), cudaHostAllocDefault) != cudaSuccess))
        rc = DEERS_ERR_CUDA;
    if (rc) {
        snprintf(ctx->last_error, sizeof(ctx->last_error), "gpt_create: %s", cudaGetErrorString(cudaGetLastError()));
        deers_b200_gpt_destroy(m);
        return rc;
    }
    *out = m;
    return DEERS_OK;
}

extern "C" void deers_b200_gpt_destroy(deers_gpt* m) {
    if (!m) return;
    cudaSetDevice(m->ctx->device);
    cudaStreamSynchronize(m->ctx->stream);
    drop_graph(m);
    if (m->side) { cudaStreamSynchronize(m->side); cudaStreamDestroy(m->side); }
    {
        cudaEvent_t evs[6] = {m->ev_fork, m->ev_join, m->ev_done[0], m->ev_done[1], m->ev_done[2], m->ev_done[3]};
        for (cudaEvent_t e : evs)
            if (e) cudaEventDestroy(e);
    }
    for (int a = 0; a < 4; ++a)
        if (m->arena[a]) cudaFree(m->arena[a]);
    if (m->act_base) cudaFree(m->act_base);
    if (m->ids_pin) cudaFreeHost(m->ids_pin);
    if (m->out_pin) cudaFreeHost(m->out_pin);
    delete m;
}

extern "C" int deers_b200_gpt_num_params(const deers_gpt* m) { return m ? 2 + 6 * m->cfg.n_layer : 0; }

extern "C" int deers_b200_gpt_param_info(const deers_gpt* m, int index, char* name, size_t name_bytes, int64_t* rows,
                                         int64_t* cols) {
    if (!m) return DEERS_ERR_NULL;
    float* p;
    long long r, c, ld;
    GPT_TRY(locate(m, index, 0, &p, &r, &c, &ld));
    if (rows) *rows = r;
    if (cols) *cols = c;
    if (name && name_bytes) {
        const int n = 2 + 6 * m->cfg.n_layer;
        if (index == 0) snprintf(name, name_bytes, "wte.weight");
        else if (index == n - 1) snprintf(name, name_bytes, "lm_head.weight");
        else snprintf(name, name_bytes, "blocks.%d.%s.weight", (index - 1) / 6, kBlockNames[(index - 1) % 6]);
    }
    return DEERS_OK;
}

extern "C" int deers_b200_gpt_param_set(deers_gpt* m, int index, int what, const float* host) {
    if (!m || !host) return DEERS_ERR_NULL;
    float* p;
    long long r, c, ld;
    GPT_TRY(locate(m, index, what, &p, &r, &c, &ld));
    deers_ctx* ctx = m->ctx;
    DEERS_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    DEERS_CUDA_TRY(ctx, cudaMemcpy2DAsync(p, (size_t)ld * sizeof(float), host, (size_t)c * sizeof(float),
                                          (size_t)c * sizeof(float), (size_t)r, cudaMemcpyHostToDevice, ctx->stream));
    DEERS_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));          // the host array may be pageable and short-lived
    return DEERS_OK;
}

extern "C" int deers_b200_gpt_param_get(deers_gpt* m, int index, int what, float* host) {
    if (!m || !host) return DEERS_ERR_NULL;
    float* p;
    long long r, c, ld;
    GPT_TRY(locate(m, index, what, &p, &r, &c, &ld));
    deers_ctx* ctx = m->ctx;
    DEERS_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    DEERS_CUDA_TRY(ctx, cudaMemcpy2DAsync(host, (size_t)c * sizeof(float), p, (size_t)ld * sizeof(float),
                                          (size_t)c * sizeof(float), (size_t)r, cudaMemcpyDeviceToHost, ctx->stream));
    DEERS_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
    return DEERS_OK;
}

extern "C" int deers_b200_gpt_set_graph(deers_gpt* m, int enable) {
    if (!m) return DEERS_ERR_NULL;
    m->graph_enabled = enable != 0;
    if (!enable) { drop_graph(m); m->graph_B = m->graph_T = -1; }
    return DEERS_OK;
}

extern "C" int deers_b200_gpt_graph_active(const deers_gpt* m) { return (m && m->graph_exec) ? 1 : 0; }

extern "C" int deers_b200_gpt_forward(deers_gpt* m, const int64_t* ids, int32_t B, int32_t T, float* logits) {
    if (!m || !ids) return DEERS_ERR_NULL;
    GPT_TRY(check_bt(m, B, T));
    deers_ctx* ctx = m->ctx;
    DEERS_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    const long long N = (long long)B * T;
    GPT_TRY(stage_ids(m, ids, nullptr, N, cudaMemcpyDeviceToDevice));
    GPT_TRY(forward(m, m->ids_dev, B, T));
    if (logits)
        DEERS_CUDA_TRY(ctx, cudaMemcpy2DAsync(logits, (size_t)m->cfg.vocab_size * sizeof(float), m->logits,
                                              (size_t)m->Vld * sizeof(float), (size_t)m->cfg.vocab_size * sizeof(float),
                                              (size_t)N, cudaMemcpyDeviceToDevice, ctx->stream));
    return DEERS_OK;
}

extern "C" int deers_b200_gpt_forward_backward(deers_gpt* m, const int64_t* ids, const int64_t* targets, int32_t B,
                                               int32_t T, float* loss_dev) {
    if (!m || !ids || !targets) return DEERS_ERR_NULL;
    GPT_TRY(check_bt(m, B, T));
    deers_ctx* ctx = m->ctx;
    DEERS_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    GPT_TRY(stage_ids(m, ids, targets, (long long)B * T, cudaMemcpyDeviceToDevice));
    GPT_TRY(run_fwd_bwd(m, B, T, false));
    if (loss_dev)
        DEERS_CUDA_TRY(ctx, cudaMemcpyAsync(loss_dev, m->loss_dev, sizeof(float), cudaMemcpyDeviceToDevice, ctx->stream));
    return DEERS_OK;
}

static int train_step_common(deers_gpt* m, int B, int T, const deers_adamw_hyper* hyper, double max_grad_norm) {
    GPT_TRY(run_fwd_bwd(m, B, T, true));
    // clip_grad_norm + step_with_grads; "if grad_norm.is_finite() { step }" of tinystories_train.rs:213-216
    return launch_adamw(m->ctx, (int)m->opt.size(), m->opt.data(), hyper, m->norm_dev, max_grad_norm, true);
}

extern "C" int deers_b200_gpt_train_step(deers_gpt* m, const int64_t* ids, const int64_t* targets, int32_t B, int32_t T,
                                         const deers_adamw_hyper* hyper, double max_grad_norm, float* loss_dev,
                                         float* grad_norm_dev) {
    if (!m || !ids || !targets || !hyper) return DEERS_ERR_NULL;
    GPT_TRY(check_bt(m, B, T));
    if (hyper->step < 1) return DEERS_ERR_SHAPE;
    deers_ctx* ctx = m->ctx;
    DEERS_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    GPT_TRY(stage_ids(m, ids, targets, (long long)B * T, cudaMemcpyDeviceToDevice));
    GPT_TRY(train_step_common(m, B, T, hyper, max_grad_norm));
    if (loss_dev)
        DEERS_CUDA_TRY(ctx, cudaMemcpyAsync(loss_dev, m->loss_dev, sizeof(float), cudaMemcpyDeviceToDevice, ctx->stream));
    if (grad_norm_dev)
        DEERS_CUDA_TRY(ctx, cudaMemcpyAsync(grad_norm_dev, m->norm_dev, sizeof(float), cudaMemcpyDeviceToDevice, ctx->stream));
    return DEERS_OK;
}

extern "C" int deers_b200_gpt_train_step_host(deers_gpt* m, const int64_t* ids_host, const int64_t* targets_host, int32_t B,
                                              int32_t T, const deers_adamw_hyper* hyper, double max_grad_norm,
                                              float* loss_host, float* grad_norm_host) {
    if (!m || !ids_host || !targets_host || !hyper) return DEERS_ERR_NULL;
    GPT_TRY(check_bt(m, B, T));
    if (hyper->step < 1) return DEERS_ERR_SHAPE;
    deers_ctx* ctx = m->ctx;
    DEERS_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    const long long N = (long long)B * T;
    memcpy(m->ids_pin, ids_host, (size_t)N * sizeof(long long));
    memcpy(m->ids_pin + m->max_tokens, targets_host, (size_t)N * sizeof(long long));
    GPT_TRY(stage_ids(m, (const int64_t*)m->ids_pin, (const int64_t*)(m->ids_pin + m->max_tokens), N, cudaMemcpyHostToDevice));
    GPT_TRY(train_step_common(m, B, T, hyper, max_grad_norm));
    DEERS_CUDA_TRY(ctx, cudaMemcpyAsync(m->out_pin, m->loss_dev, 2 * sizeof(float), cudaMemcpyDeviceToHost, ctx->stream));
    const int rc = deers_b200_sync(ctx);
    if (loss_host) *loss_host = m->out_pin[0];
    if (grad_norm_host) *grad_norm_host = m->out_pin[1];
    return rc;
}
