/*
 * TEST INFRASTRUCTURE, NOT PRODUCT CODE.
 *
 * CPU restatement (plain C, f32, OpenMP over (batch, head) slices) of the causal
 * self-attention path of vitillo/deers as its CPU backend executes it, op by op,
 * materialising every T x T tensor exactly like the reference graph does.  It is
 * the parity checker for the CUDA kernels and the timed CPU baseline; nothing in
 * the shipped library links or calls it.
 *
 * PARITY UNPINNED for attention itself: the reference is Rust (no toolchain in
 * the build image), its GEMM is the un-vendored crate `gemm 0.19.0` and its own
 * tests compute expected values with candle at test time, so no stored golden
 * vector for attention exists.  What IS pinned by stored reference values is
 * the mask (ref_causal_mask, literal vectors in tests/nn.rs:194-232).  The
 * restatement is additionally cross-checked against an independent float64
 * autograd implementation (tests/golden/make_golden.py).
 *
 * Reference lines followed (paths inside the deers repository):
 *   src/models/gpt.rs:139-144      scores = (q @ k^T) * scale; softmax(scores + mask); @ v
 *   src/storage/cpu.rs:688-753     batched matmul, serial over the batch, f32 accumulate
 *   src/storage.rs:105-123         scalar multiply: the f64 scale is cast to f32 first
 *   src/nn/functional.rs:12-55     additive mask: 0 where j <= i, -inf where j > i
 *   src/storage/cpu.rs:755-770     log_sum_exp: max, left-to-right f32 sum of exp(x-max), ln + max
 *   src/tensor.rs:408-425,456-458  softmax = exp(x - lse)
 *   src/ops.rs:1089-1101           matmul backward: dA = dC @ B^T, dB = A^T @ dC
 *   src/ops.rs:422-425             exp backward: g * exp(x)
 *   src/ops.rs:210-214,777-799,1162-1175  x - lse backward: g - softmax * rowsum(g)
 *   src/ops.rs:638-643             scalar multiply backward: g * scale
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define API __attribute__((visibility("default")))

API int ref_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* Sets the OpenMP thread count (launchers may export OMP_NUM_THREADS=1); returns the count in use. */
API int ref_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
    return omp_get_max_threads();
#else
    (void)n;
    return 1;
#endif
}

/* src/nn/functional.rs:12-55 — [batch, 1, tgt_len, tgt_len + offset], 0 or -inf. */
API void ref_causal_mask(int batch, int tgt_len, int offset, float* out) {
    const int total = tgt_len + offset;
    for (int b = 0; b < batch; ++b)
        for (int i = 0; i < tgt_len; ++i)
            for (int j = 0; j < total; ++j)
                out[((size_t)b * tgt_len + i) * total + j] =
                    (j >= offset && j - offset > i) ? -INFINITY : 0.0f;
}

/* C[m,n] = sum_k A[m,k] * B[n,k]   (A @ B^T), f32 accumulate; src/storage/cpu.rs:729-747 */
static void gemm_nt(const float* A, const float* B, float* C, int M, int N, int K) {
    for (int m = 0; m < M; ++m) {
        const float* a = A + (size_t)m * K;
        for (int n = 0; n < N; ++n) {
            const float* b = B + (size_t)n * K;
            float acc = 0.0f;
            for (int k = 0; k < K; ++k) acc += a[k] * b[k];
            C[(size_t)m * N + n] = acc;
        }
    }
}

/* C[m,n] = sum_k A[m,k] * B[k,n]   (A @ B) */
static void gemm_nn(const float* A, const float* B, float* C, int M, int N, int K) {
    for (int m = 0; m < M; ++m) {
        float* c = C + (size_t)m * N;
        for (int n = 0; n < N; ++n) c[n] = 0.0f;
        for (int k = 0; k < K; ++k) {
            const float a = A[(size_t)m * K + k];
            const float* b = B + (size_t)k * N;
            for (int n = 0; n < N; ++n) c[n] += a * b[n];
        }
    }
}

/* C[m,n] = sum_k A[k,m] * B[k,n]   (A^T @ B) */
static void gemm_tn(const float* A, const float* B, float* C, int M, int N, int K) {
    for (size_t i = 0; i < (size_t)M * N; ++i) C[i] = 0.0f;
    for (int k = 0; k < K; ++k) {
        const float* a = A + (size_t)k * M;
        const float* b = B + (size_t)k * N;
        for (int m = 0; m < M; ++m) {
            const float am = a[m];
            float* c = C + (size_t)m * N;
            for (int n = 0; n < N; ++n) c[n] += am * b[n];
        }
    }
}

/* One (batch, head) slice, forward.  P (T x T) is left in `P` for the backward. */
static void slice_fwd(const float* q, const float* k, const float* v, int T, int D, float scale,
                      int causal, float* o, float* lse, float* P) {
    gemm_nt(q, k, P, T, T, D);                               /* gpt.rs:140 */
    for (size_t i = 0; i < (size_t)T * T; ++i) P[i] *= scale; /* gpt.rs:139-140, storage.rs:115-117 */
    if (causal)
        for (int i = 0; i < T; ++i)                           /* functional.rs:38-51, gpt.rs:142 */
            for (int j = i + 1; j < T; ++j) P[(size_t)i * T + j] += -INFINITY;
    for (int i = 0; i < T; ++i) {                             /* cpu.rs:759-770 */
        float* row = P + (size_t)i * T;
        float mx = -INFINITY;
        for (int j = 0; j < T; ++j) mx = fmaxf(mx, row[j]);
        float sum = 0.0f;
        for (int j = 0; j < T; ++j) sum += expf(row[j] - mx);
        const float l = logf(sum) + mx;
        lse[i] = l;
        for (int j = 0; j < T; ++j) row[j] = expf(row[j] - l); /* tensor.rs:419-424,456-458 */
    }
    gemm_nn(P, v, o, T, D, T);                                /* gpt.rs:143-144 */
}

/*
 * Forward over compact [B,H,T,D] f32 tensors.  o: [B,H,T,D], lse: [B,H,T]
 * (natural log of the row sums of exp(scaled, masked scores)).
 */
API int ref_attn_fwd(const float* q, const float* k, const float* v, int B, int H, int T, int D,
                     float scale, int causal, float* o, float* lse) {
    const int BH = B * H;
    const size_t n = (size_t)T * D;
    int fail = 0;
#pragma omp parallel for schedule(dynamic, 1)
    for (int s = 0; s < BH; ++s) {
        float* P = (float*)malloc((size_t)T * T * sizeof(float));
        if (!P) { fail = 1; continue; }
        slice_fwd(q + s * n, k + s * n, v + s * n, T, D, scale, causal, o + s * n, lse + (size_t)s * T, P);
        free(P);
    }
    return fail;
}

/*
 * Forward + backward over compact [B,H,T,D] f32 tensors, the way the reference
 * graph runs it: the forward's P is kept and the backward is the chain of the
 * per-op backward rules.  Any of o/lse may be NULL.
 */
API int ref_attn_fwd_bwd(const float* q, const float* k, const float* v, const float* d_o, int B,
                         int H, int T, int D, float scale, int causal, float* o, float* lse,
                         float* dq, float* dk, float* dv) {
    const int BH = B * H;
    const size_t n = (size_t)T * D;
    int fail = 0;
#pragma omp parallel for schedule(dynamic, 1)
    for (int s = 0; s < BH; ++s) {
        float* P = (float*)malloc((size_t)T * T * sizeof(float));
        float* G = (float*)malloc((size_t)T * T * sizeof(float));
        float* o_s = (float*)malloc(n * sizeof(float));
        float* lse_s = (float*)malloc((size_t)T * sizeof(float));
        if (!P || !G || !o_s || !lse_s) { fail = 1; free(P); free(G); free(o_s); free(lse_s); continue; }
        slice_fwd(q + s * n, k + s * n, v + s * n, T, D, scale, causal, o_s, lse_s, P);
        if (o) memcpy(o + s * n, o_s, n * sizeof(float));
        if (lse) memcpy(lse + (size_t)s * T, lse_s, (size_t)T * sizeof(float));
        const float* go = d_o + s * n;
        gemm_tn(P, go, dv + s * n, T, D, T);          /* dV = P^T @ dO      ops.rs:1089-1101 */
        gemm_nt(go, v + s * n, G, T, T, D);           /* dP = dO @ V^T      ops.rs:1089-1101 */
        for (int i = 0; i < T; ++i) {
            float* g = G + (size_t)i * T;
            const float* p = P + (size_t)i * T;
            float rs = 0.0f;
            for (int j = 0; j < T; ++j) { g[j] *= p[j]; rs += g[j]; }  /* ops.rs:422-425; Broadcast bwd sum ops.rs:777-799 */
            for (int j = 0; j < T; ++j) g[j] = (g[j] - p[j] * rs) * scale; /* ops.rs:210-214,1162-1175; 638-643 */
        }
        gemm_nn(G, k + s * n, dq + s * n, T, D, T);   /* dQ = dS @ K        ops.rs:1089-1101 */
        gemm_tn(G, q + s * n, dk + s * n, T, D, T);   /* dK = dS^T @ Q      ops.rs:1089-1101 */
        free(P); free(G); free(o_s); free(lse_s);
    }
    return fail;
}

/*
 * Rotary embedding + head-major permute, f32, op by op as the reference graph evaluates it
 * (paths inside the deers repository):
 *   src/models/gpt.rs:49-73    apply_rotary_emb on [B,T,H,D]: x1 = x[..., :D/2], x2 = x[..., D/2:],
 *                              y1 = x1*cos + x2*sin, y2 = x1*(sin * -1) + x2*cos, cat([y1, y2], 3)
 *   src/models/gpt.rs:135-136  .permute([0,2,1,3]) -> [B,H,T,D]
 *   src/ops.rs:130-173, 176-254 EWiseAdd / EWiseMul: one rounding per op (no fused multiply-add), and
 *                              their backward (g*other, g) summed by backprop.rs:101-112
 * inverse = 0: x is [B,T,H,D], y is [B,H,T,D].
 * inverse = 1: x is the gradient w.r.t. y laid out [B,H,T,D], y receives the gradient w.r.t. x as
 *              [B,T,H,D]: dx1 = dy1*cos + dy2*(sin * -1), dx2 = dy1*sin + dy2*cos.
 * cos / sin: [T, D/2].  The products must round separately, so contraction into FMA is disabled.
 */
__attribute__((visibility("default"), optimize("fp-contract=off")))
void ref_rope_pack(const float* x, const float* cosv, const float* sinv, int B, int T, int H, int D, int inverse,
                   float* y) {
    const int half = D / 2;
#pragma omp parallel for collapse(2) schedule(static)
    for (int b = 0; b < B; ++b) {
        for (int t = 0; t < T; ++t) {
            for (int h = 0; h < H; ++h) {
                const size_t bthd = (((size_t)b * T + t) * H + h) * D;
                const size_t bhtd = (((size_t)b * H + h) * T + t) * D;
                const float* src = x + (inverse ? bhtd : bthd);
                float* dst = y + (inverse ? bthd : bhtd);
                for (int i = 0; i < half; ++i) {
                    const float c = cosv[(size_t)t * half + i];
                    const float s = inverse ? -sinv[(size_t)t * half + i] : sinv[(size_t)t * half + i];
                    const float a = src[i], bb = src[half + i];
                    const float p1 = a * c, p2 = bb * s;       /* EWiseMul, EWiseMul */
                    const float ns = s * -1.0f;                 /* ScalarMul by -1 (exact) */
                    const float p3 = a * ns, p4 = bb * c;
                    dst[i] = p1 + p2;                           /* EWiseAdd */
                    dst[half + i] = p3 + p4;
                }
            }
        }
    }
}

/*
 * AdamW and clip_grad_norm, f32, op by op as the reference evaluates them on its CPU backend
 * (paths inside the deers repository):
 *   src/optim.rs:214-251   step_with_grads: m = m*b1 + g*(1-b1); v = v*b2 + (g*g)*(1-b2);
 *                          m_hat = m*(1/bc1); v_hat = v*(1/bc2); decayed = w*(1-lr*wd) if wd > 0;
 *                          update = m_hat / (sqrt(v_hat) + eps); w = decayed - update*lr
 *   src/storage.rs:105-123 scalar ops cast their f64 operand to f32 (`self.0 as f32`)
 *   src/optim.rs:257-297   clip_grad_norm: total += sum(g*g) per parameter (left-to-right f32 sum,
 *                          src/storage/cpu.rs:323-345), norm = sqrt(total)
 * Products and sums round separately (contraction into FMA disabled).  Pinned by the literal values of
 * the reference's own test (src/optim.rs:556-570: gradient [3, 4], max_norm 1 -> norm 5, [0.6, 0.8]).
 */
static double ref_powi(double a, int b) {      /* f64::powi: exponentiation by squaring */
    const int recip = b < 0;
    double r = 1.0;
    for (;;) {
        if (b & 1) r *= a;
        b /= 2;
        if (b == 0) break;
        a *= a;
    }
    return recip ? 1.0 / r : r;
}

__attribute__((visibility("default"), optimize("fp-contract=off")))
void ref_adamw_step(float* w, const float* g, float* m, float* v, long long n, double lr, double beta1, double beta2,
                    double eps, double weight_decay, int step) {
    const double bc1 = 1.0 - ref_powi(beta1, step), bc2 = 1.0 - ref_powi(beta2, step);
    const float b1 = (float)beta1, omb1 = (float)(1.0 - beta1), b2 = (float)beta2, omb2 = (float)(1.0 - beta2);
    const float ibc1 = (float)(1.0 / bc1), ibc2 = (float)(1.0 / bc2);
    const float decay = (float)(1.0 - lr * weight_decay), lrf = (float)lr, epsf = (float)eps;
#pragma omp parallel for schedule(static)
    for (long long i = 0; i < n; ++i) {
        const float gi = g[i];
        const float t1 = m[i] * b1, t2 = gi * omb1;
        const float mi = t1 + t2;
        const float gg = gi * gi;
        const float t3 = v[i] * b2, t4 = gg * omb2;
        const float vi = t3 + t4;
        const float m_hat = mi * ibc1, v_hat = vi * ibc2;
        const float decayed = weight_decay > 0.0 ? w[i] * decay : w[i];
        const float denom = sqrtf(v_hat) + epsf;
        const float update = m_hat / denom;
        const float ul = update * lrf;
        m[i] = mi;
        v[i] = vi;
        w[i] = decayed - ul;
    }
}

/* sum over one gradient of g*g: the product tensor first, then a left-to-right f32 sum. */
__attribute__((visibility("default"), optimize("fp-contract=off")))
float ref_grad_sq_sum(const float* g, long long n) {
    float s = 0.0f;
    for (long long i = 0; i < n; ++i) {
        const float p = g[i] * g[i];
        s = (i == 0) ? p : s + p;
    }
    return s;
}

/*
 * RMSNorm forward and backward, f32, op by op as the reference graph evaluates it (paths inside the
 * deers repository):
 *   src/nn.rs:244-251        mean_sq = (x*x).mean([last], keep); inv = (mean_sq + eps)^-0.5; y = x * inv
 *   src/tensor.rs:461-465    mean = sum * (1.0 / n as f64), the scalar cast to f32 (storage.rs:105-123)
 *   src/storage/cpu.rs:323-345  sum: left-to-right f32
 *   src/ops.rs:675-679       scalar power backward: g * e * arg^(e-1)
 *   src/ops.rs:210-214 (multiply backward), 777-799 (broadcast backward: sum over the broadcast axis),
 *   638-643 (scalar multiply backward), src/backprop.rs:101-112 (contributions to x are added as they
 *   arrive; this restatement adds the broadcast-multiply term first, then the two x*x terms)
 * No stored reference vector exists for RMSNorm (tests/nn.rs compares with candle at run time): unpinned,
 * cross-checked against float64 autograd (tests/golden/make_golden.py).
 */
__attribute__((visibility("default"), optimize("fp-contract=off")))
void ref_rmsnorm(const float* x, long long rows, int C, double eps, const float* dy, float* y, float* dx) {
    const float inv_n = (float)(1.0 / (double)C), epsf = (float)eps;
#pragma omp parallel for schedule(static)
    for (long long r = 0; r < rows; ++r) {
        const float* xr = x + r * C;
        float s = 0.0f;
        for (int c = 0; c < C; ++c) { const float p = xr[c] * xr[c]; s = c == 0 ? p : s + p; }
        const float a = s * inv_n + epsf;
        const float inv = powf(a, -0.5f);
        if (y) for (int c = 0; c < C; ++c) y[r * C + c] = xr[c] * inv;
        if (dy && dx) {
            const float* g = dy + r * C;
            float dinv = 0.0f;
            for (int c = 0; c < C; ++c) { const float p = g[c] * xr[c]; dinv = c == 0 ? p : dinv + p; }
            const float da = (dinv * -0.5f) * powf(a, -1.5f);
            const float ds = da * inv_n;
            for (int c = 0; c < C; ++c) {
                const float t1 = g[c] * inv, t2 = ds * xr[c];
                dx[r * C + c] = (t1 + t2) + t2;
            }
        }
    }
}
