/*
 * TEST INFRASTRUCTURE, NOT PRODUCT CODE.
 *
 * CPU restatement (plain C, f32, OpenMP) of one training step of the GPT of
 * vitillo/deers as its CPU backend executes it, op by op: forward, cross-entropy,
 * backward through every op's backward rule.  It is the parity checker for the
 * CUDA step and the timed CPU baseline of that step; nothing in the shipped
 * library links or calls it.
 *
 * Pinned by the literal values the reference's own tests hold: NLL loss and its
 * gradient (src/loss.rs:31-65), cross-entropy rows (src/loss.rs:67-84), RMSNorm of
 * [1,2,3] (tests/nn.rs:172-186), the causal mask (tests/nn.rs:194-232, in
 * attn_ref.c).  The whole-model test of the reference (tests/gpt.rs:272-343)
 * computes its expectation with candle at run time from unseeded weights, so the
 * composition itself is cross-checked against an independent float64 autograd run
 * of the same model at that test's shape (tests/golden/make_golden.py).
 *
 * Reference lines followed (paths inside the deers repository):
 *   src/models/gpt.rs:329-355   GPT::forward: wte -> blocks -> norm -> lm_head
 *   src/models/gpt.rs:236-240   Block::forward: x + attn(norm1(x)); x + mlp(norm2(x))
 *   src/models/gpt.rs:102-148   CausalSelfAttention::forward (projections, RoPE, permutes, core, out_proj)
 *   src/models/gpt.rs:186-200   MLP::forward: up_proj, relu, y*y, down_proj
 *   src/models/gpt.rs:12-46     precompute_rotary_embeddings
 *   src/nn.rs:184-190           Linear::forward = x.matmul(weight), weight [in, out]
 *   src/nn.rs:214-221           Embedding::forward = index_select(0, ids)
 *   src/nn.rs:244-251           RMSNorm::forward
 *   src/loss.rs:11-24           nll_loss, cross_entropy
 *   src/tensor.rs:408-425       log_softmax = x - log_sum_exp(x)
 *   src/storage/cpu.rs:755-770  log_sum_exp: max, left-to-right f32 sum of exp(x-max), ln + max
 *   src/ops.rs:1089-1101        matmul backward: dA = dC @ B^T, dB = A^T @ dC
 *   src/ops.rs:560-568          relu backward: g * (x > 0)
 *   src/ops.rs:210-214          multiply backward: g * other (y*y: both contributions added, backprop.rs:101-112)
 *   src/ops.rs:1162-1175        log_sum_exp backward: g * softmax
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define API __attribute__((visibility("default")))

/* From attn_ref.c (same shared object). */
int ref_attn_fwd(const float* q, const float* k, const float* v, int B, int H, int T, int D, float scale, int causal,
                 float* o, float* lse);
int ref_attn_fwd_bwd(const float* q, const float* k, const float* v, const float* d_o, int B, int H, int T, int D,
                     float scale, int causal, float* o, float* lse, float* dq, float* dk, float* dv);
void ref_rope_pack(const float* x, const float* cosv, const float* sinv, int B, int T, int H, int D, int inverse,
                   float* y);
void ref_rmsnorm(const float* x, long long rows, int C, double eps, const float* dy, float* y, float* dx);

/* C[M,N] = A[M,K] @ B[K,N]; each output is a k-sequential f32 sum (src/storage/cpu.rs:729-747). */
API void ref_matmul_nn(const float* A, const float* B, float* C, long long M, long long N, long long K) {
#pragma omp parallel for schedule(static)
    for (long long m = 0; m < M; ++m) {
        float* c = C + m * N;
        for (long long n = 0; n < N; ++n) c[n] = 0.0f;
        for (long long k = 0; k < K; ++k) {
            const float a = A[m * K + k];
            const float* b = B + k * N;
            for (long long n = 0; n < N; ++n) c[n] += a * b[n];
        }
    }
}

/* C[M,N] = A[M,K] @ B[N,K]^T  (dA = dC @ B^T of the matmul backward) */
API void ref_matmul_nt(const float* A, const float* B, float* C, long long M, long long N, long long K) {
#pragma omp parallel for schedule(static)
    for (long long m = 0; m < M; ++m) {
        const float* a = A + m * K;
        for (long long n = 0; n < N; ++n) {
            const float* b = B + n * K;
            float acc = 0.0f;
            for (long long k = 0; k < K; ++k) acc += a[k] * b[k];
            C[m * N + n] = acc;
        }
    }
}

/* C[M,N] = A[K,M]^T @ B[K,N]  (dB = A^T @ dC of the matmul backward) */
API void ref_matmul_tn(const float* A, const float* B, float* C, long long M, long long N, long long K) {
#pragma omp parallel for schedule(static)
    for (long long m = 0; m < M; ++m) {
        float* c = C + m * N;
        for (long long n = 0; n < N; ++n) c[n] = 0.0f;
        for (long long k = 0; k < K; ++k) {
            const float a = A[k * M + m];
            const float* b = B + k * N;
            for (long long n = 0; n < N; ++n) c[n] += a * b[n];
        }
    }
}

/* src/nn.rs:214-221: out[n, :] = weight[ids[n], :] */
API void ref_embedding_fwd(const float* weight, const long long* ids, long long n_ids, int C, float* out) {
#pragma omp parallel for schedule(static)
    for (long long n = 0; n < n_ids; ++n) memcpy(out + n * C, weight + ids[n] * C, (size_t)C * sizeof(float));
}

/* index_select backward (index_add into zeros): rows added in token order. */
API void ref_embedding_bwd(const float* dout, const long long* ids, long long n_ids, int C, long long vocab,
                           float* dweight) {
    memset(dweight, 0, (size_t)vocab * C * sizeof(float));
    for (long long n = 0; n < n_ids; ++n) {
        float* d = dweight + ids[n] * C;
        const float* s = dout + n * C;
        for (int c = 0; c < C; ++c) d[c] += s[c];
    }
}

/*
 * log_softmax over the last axis and nll_loss (src/tensor.rs:408-425, src/loss.rs:11-24):
 *   lse = ln(sum exp(x - max)) + max;  lsm = x - lse;  loss = sum_n lsm[n, target[n]] * (float)(-1/rows).
 * lsm may be NULL (only the loss is wanted); lse_out may be NULL.
 */
API float ref_cross_entropy_fwd(const float* logits, const long long* targets, long long rows, long long V,
                                float* lsm, float* lse_out) {
    float* picked = (float*)malloc((size_t)rows * sizeof(float));
#pragma omp parallel for schedule(static)
    for (long long n = 0; n < rows; ++n) {
        const float* x = logits + n * V;
        float mx = -INFINITY;
        for (long long j = 0; j < V; ++j) mx = fmaxf(mx, x[j]);
        float s = 0.0f;
        for (long long j = 0; j < V; ++j) s += expf(x[j] - mx);
        const float l = logf(s) + mx;
        if (lse_out) lse_out[n] = l;
        if (lsm) for (long long j = 0; j < V; ++j) lsm[n * V + j] = x[j] - l;
        picked[n] = x[targets[n]] - l;
    }
    float tot = 0.0f;
    for (long long n = 0; n < rows; ++n) tot = n == 0 ? picked[n] : tot + picked[n];
    free(picked);
    return tot * (float)(-1.0 / (double)rows);
}

/* nll_loss alone on given log-probabilities (src/loss.rs:11-15) and its gradient (gather backward: scatter of g). */
API float ref_nll_loss(const float* log_probs, const long long* targets, long long rows, long long V, float* grad) {
    float tot = 0.0f;
    const float g = (float)(-1.0 / (double)rows);
    if (grad) memset(grad, 0, (size_t)rows * V * sizeof(float));
    for (long long n = 0; n < rows; ++n) {
        const float p = log_probs[n * V + targets[n]];
        tot = n == 0 ? p : tot + p;
        if (grad) grad[n * V + targets[n]] += g;
    }
    return tot * g;
}

/*
 * Gradient of cross_entropy w.r.t. the logits, upstream gradient 1:
 *   d lsm = onehot * (float)(-1/rows);  d logits = d lsm - softmax * rowsum(d lsm)   (x - lse backward,
 *   src/ops.rs:210-214, 777-799, 1162-1175), softmax = exp(x - lse).
 */
API void ref_cross_entropy_bwd(const float* logits, const long long* targets, long long rows, long long V,
                               float* dlogits) {
    const float g = (float)(-1.0 / (double)rows);
#pragma omp parallel for schedule(static)
    for (long long n = 0; n < rows; ++n) {
        const float* x = logits + n * V;
        float mx = -INFINITY;
        for (long long j = 0; j < V; ++j) mx = fmaxf(mx, x[j]);
        float s = 0.0f;
        for (long long j = 0; j < V; ++j) s += expf(x[j] - mx);
        const float l = logf(s) + mx;
        float* d = dlogits + n * V;
        for (long long j = 0; j < V; ++j) {
            const float p = expf(x[j] - l);
            const float gj = (j == targets[n]) ? g : 0.0f;
            d[j] = gj - p * g;
        }
    }
}

/* gpt.rs:12-46, f32 arithmetic: inv_freq = 1 / base^(2i/D); angle = t * inv_freq; cos, sin: [T, D/2] */
API void ref_rotary_cache(int T, int D, float base, float* cosv, float* sinv) {
    const int half = D / 2;
    for (int t = 0; t < T; ++t)
        for (int i = 0; i < half; ++i) {
            const float channel = (float)(2 * i);
            const float inv_freq = 1.0f / powf(base, channel / (float)D);
            const float f = (float)t * inv_freq;
            cosv[(size_t)t * half + i] = cosf(f);
            sinv[(size_t)t * half + i] = sinf(f);
        }
}

static void permute_0213(const float* x, int B, int T, int H, int D, float* y) {   /* [B,T,H,D] -> [B,H,T,D] */
#pragma omp parallel for collapse(2) schedule(static)
    for (int b = 0; b < B; ++b)
        for (int t = 0; t < T; ++t)
            for (int h = 0; h < H; ++h)
                memcpy(y + (((size_t)b * H + h) * T + t) * D, x + (((size_t)b * T + t) * H + h) * D,
                       (size_t)D * sizeof(float));
}

typedef struct {
    float *x, *n1, *qh, *kh, *vh, *of, *x1, *n2, *u, *h;
} layer_act;

static float* falloc(size_t n) { return (float*)malloc((n ? n : 1) * sizeof(float)); }

/*
 * One forward (and, with targets and grads, backward) of the model.
 *   cfg = {vocab, n_layer, n_head, n_embd, mlp_hidden};  params / grads: 2 + 6*n_layer arrays in the order of
 *   GPT::parameters (gpt.rs:358-365): wte [V,C]; per block q,k,v,out [C,C], up [C,Hm], down [Hm,C]; lm_head [C,V].
 *   ids, targets: [B*T] token ids.  logits_out ([B*T, V]) and loss_out may be NULL.
 * Returns 0, or 1 when an allocation failed.
 */
API int ref_gpt_step(const int* cfg, double eps, float rope_base, int B, int T, const long long* ids,
                     const long long* targets, const float* const* params, float* logits_out, float* loss_out,
                     float* const* grads) {
    const int V = cfg[0], L = cfg[1], H = cfg[2], C = cfg[3], Hm = cfg[4];
    const int D = C / H;
    const long long N = (long long)B * T;
    const float scale = (float)(1.0 / sqrt((double)D));          /* gpt.rs:139, storage.rs:115-117 */
    const size_t NC = (size_t)N * C;
    int fail = 0;

    float* cosv = falloc((size_t)T * (D / 2));
    float* sinv = falloc((size_t)T * (D / 2));
    layer_act* acts = (layer_act*)calloc((size_t)L, sizeof(layer_act));
    float* x = falloc(NC);
    float* tmp = falloc(NC);
    float* tmp2 = falloc(NC);
    float* tmp3 = falloc(NC);
    float* xf = falloc(NC);
    float* logits = falloc((size_t)N * V);
    float* lse_tmp = falloc((size_t)N * H);
    if (!cosv || !sinv || !acts || !x || !tmp || !tmp2 || !tmp3 || !xf || !logits || !lse_tmp) return 1;
    ref_rotary_cache(T, D, rope_base, cosv, sinv);

    ref_embedding_fwd(params[0], ids, N, C, x);                  /* gpt.rs:343 */
    for (int l = 0; l < L; ++l) {
        const float* const* w = params + 1 + 6 * l;
        layer_act* a = &acts[l];
        a->x = falloc(NC); a->n1 = falloc(NC); a->qh = falloc(NC); a->kh = falloc(NC); a->vh = falloc(NC);
        a->of = falloc(NC); a->x1 = falloc(NC); a->n2 = falloc(NC);
        a->u = falloc((size_t)N * Hm); a->h = falloc((size_t)N * Hm);
        if (!a->x || !a->n1 || !a->qh || !a->kh || !a->vh || !a->of || !a->x1 || !a->n2 || !a->u || !a->h) return 1;
        memcpy(a->x, x, NC * sizeof(float));
        ref_rmsnorm(x, N, C, eps, NULL, a->n1, NULL);            /* gpt.rs:237 norm1 */
        ref_matmul_nn(a->n1, w[0], tmp, N, C, C);                /* gpt.rs:116 q_proj */
        ref_rope_pack(tmp, cosv, sinv, B, T, H, D, 0, a->qh);    /* gpt.rs:135 */
        ref_matmul_nn(a->n1, w[1], tmp, N, C, C);                /* k_proj */
        ref_rope_pack(tmp, cosv, sinv, B, T, H, D, 0, a->kh);
        ref_matmul_nn(a->n1, w[2], tmp, N, C, C);                /* v_proj */
        permute_0213(tmp, B, T, H, D, a->vh);                    /* gpt.rs:137 */
        fail |= ref_attn_fwd(a->qh, a->kh, a->vh, B, H, T, D, scale, 1, tmp, lse_tmp);   /* gpt.rs:139-144 */
        permute_0213(tmp, B, H, T, D, a->of);                    /* [B,H,T,D] -> [B,T,H,D] = [N,C], gpt.rs:144 */
        ref_matmul_nn(a->of, w[3], tmp, N, C, C);                /* out_proj */
        for (size_t i = 0; i < NC; ++i) a->x1[i] = x[i] + tmp[i];                     /* gpt.rs:237 */
        ref_rmsnorm(a->x1, N, C, eps, NULL, a->n2, NULL);        /* norm2 */
        ref_matmul_nn(a->n2, w[4], a->u, N, Hm, C);              /* up_proj */
        for (size_t i = 0; i < (size_t)N * Hm; ++i) {            /* relu, y*y */
            const float r = a->u[i] > 0.0f ? a->u[i] : 0.0f;
            a->h[i] = r * r;
        }
        ref_matmul_nn(a->h, w[5], tmp, N, C, Hm);                /* down_proj */
        for (size_t i = 0; i < NC; ++i) x[i] = a->x1[i] + tmp[i];                     /* gpt.rs:239 */
    }
    ref_rmsnorm(x, N, C, eps, NULL, xf, NULL);                   /* gpt.rs:347 */
    ref_matmul_nn(xf, params[1 + 6 * L], logits, N, V, C);       /* gpt.rs:351 lm_head */
    if (logits_out) memcpy(logits_out, logits, (size_t)N * V * sizeof(float));

    if (targets) {
        const float loss = ref_cross_entropy_fwd(logits, targets, N, V, NULL, NULL);
        if (loss_out) *loss_out = loss;
    }
    if (targets && grads) {
        float* dlogits = falloc((size_t)N * V);
        float* dx = falloc(NC);
        float* dhid = falloc((size_t)N * Hm);
        float* dqkv[3] = {falloc(NC), falloc(NC), falloc(NC)};
        if (!dlogits || !dx || !dhid || !dqkv[0] || !dqkv[1] || !dqkv[2]) return 1;
        ref_cross_entropy_bwd(logits, targets, N, V, dlogits);
        ref_matmul_tn(xf, dlogits, grads[1 + 6 * L], C, V, N);   /* d lm_head = xf^T @ dlogits */
        ref_matmul_nt(dlogits, params[1 + 6 * L], tmp, N, C, V); /* d xf = dlogits @ W^T */
        ref_rmsnorm(x, N, C, eps, tmp, NULL, dx);                /* final norm backward */
        for (int l = L - 1; l >= 0; --l) {
            const float* const* w = params + 1 + 6 * l;
            float* const* g = grads + 1 + 6 * l;
            layer_act* a = &acts[l];
            /* mlp branch */
            ref_matmul_tn(a->h, dx, g[5], Hm, C, N);             /* d down = h^T @ dx */
            ref_matmul_nt(dx, w[5], dhid, N, Hm, C);             /* d h = dx @ Wdown^T */
            for (size_t i = 0; i < (size_t)N * Hm; ++i) {
                const float r = a->u[i] > 0.0f ? a->u[i] : 0.0f;
                const float t = dhid[i] * r;
                const float dr = t + t;                          /* y*y backward, two contributions */
                dhid[i] = dr * (a->u[i] > 0.0f ? 1.0f : 0.0f);   /* relu backward */
            }
            ref_matmul_tn(a->n2, dhid, g[4], C, Hm, N);          /* d up */
            ref_matmul_nt(dhid, w[4], tmp, N, C, Hm);            /* d n2 */
            ref_rmsnorm(a->x1, N, C, eps, tmp, NULL, tmp2);      /* norm2 backward */
            for (size_t i = 0; i < NC; ++i) dx[i] = dx[i] + tmp2[i];                  /* d x1 */
            /* attention branch */
            ref_matmul_tn(a->of, dx, g[3], C, C, N);             /* d out_proj */
            ref_matmul_nt(dx, w[3], tmp, N, C, C);               /* d o_flat [B,T,H,D] */
            permute_0213(tmp, B, T, H, D, tmp2);                 /* -> [B,H,T,D] */
            fail |= ref_attn_fwd_bwd(a->qh, a->kh, a->vh, tmp2, B, H, T, D, scale, 1, NULL, NULL, dqkv[0], dqkv[1], tmp3);
            ref_rope_pack(dqkv[0], cosv, sinv, B, T, H, D, 1, tmp);   /* d q [B,T,H,D] */
            ref_matmul_tn(a->n1, tmp, g[0], C, C, N);
            ref_matmul_nt(tmp, w[0], tmp2, N, C, C);             /* d n1 (from q) */
            ref_rope_pack(dqkv[1], cosv, sinv, B, T, H, D, 1, tmp);   /* d k */
            ref_matmul_tn(a->n1, tmp, g[1], C, C, N);
            ref_matmul_nt(tmp, w[1], dqkv[0], N, C, C);
            for (size_t i = 0; i < NC; ++i) tmp2[i] += dqkv[0][i];
            permute_0213(tmp3, B, H, T, D, tmp);                 /* d v [B,T,H,D] */
            ref_matmul_tn(a->n1, tmp, g[2], C, C, N);
            ref_matmul_nt(tmp, w[2], dqkv[0], N, C, C);
            for (size_t i = 0; i < NC; ++i) tmp2[i] += dqkv[0][i];
            ref_rmsnorm(a->x, N, C, eps, tmp2, NULL, tmp);       /* norm1 backward */
            for (size_t i = 0; i < NC; ++i) dx[i] = dx[i] + tmp[i];
        }
        ref_embedding_bwd(dx, ids, N, C, V, grads[0]);
        free(dlogits); free(dx); free(dhid); free(dqkv[0]); free(dqkv[1]); free(dqkv[2]);
    }
    for (int l = 0; l < L; ++l) {
        layer_act* a = &acts[l];
        free(a->x); free(a->n1); free(a->qh); free(a->kh); free(a->vh); free(a->of); free(a->x1); free(a->n2);
        free(a->u); free(a->h);
    }
    free(acts); free(cosv); free(sinv); free(x); free(tmp); free(tmp2); free(tmp3); free(xf); free(logits); free(lse_tmp);
    return fail;
}
