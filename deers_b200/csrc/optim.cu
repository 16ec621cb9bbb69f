// Multi-tensor AdamW with the global gradient-norm clip folded in (f32).
//
// The reference composes one optimizer step from about twelve element-wise tensor ops and ten
// temporaries PER PARAMETER (AdamW::step_with_grads, src/optim.rs:214-251) and clips gradients with
// one multiply, one full reduction and one add per parameter plus a host read of the norm
// (clip_grad_norm, src/optim.rs:257-297).  Here all parameters are handled by a handful of launches:
//   grad_sq_sum_kernel    per-block partial sums of g*g over every gradient (fixed grid, fixed
//                         order: the result does not depend on timing)
//   grad_norm_kernel      sums the partials in a fixed order, writes sqrt(total) to device memory
//   adamw_kernel<MODE>    MODE_STEP: reads w, g, m, v once, writes w, m, v once (28 bytes per
//                         element); MODE_CLIP: scales the gradients in place.  Both read the norm
//                         from device memory and decide about clipping there, so the fused path
//                         has no host synchronisation.
// Arithmetic follows the reference op by op: every multiply, add, divide and square root rounds
// to f32 on its own (no FMA contraction) and every scalar is an f64 rounded to f32 at the point
// where the reference's scalar ops do it (src/storage.rs:105-123), so that the update is
// bit-identical to the CPU path whenever the clip scale is (the norm itself is a differently
// ordered f32 sum).
#include "common.cuh"

namespace {

constexpr int OPT_MAXT = 64;            // tensors per launch (kernel parameter space)
constexpr int OPT_CHUNK = 4096;         // elements per block iteration: 256 threads x 4 x float4
constexpr int OPT_MAX_GROUPS = 4;       // launches per call: up to 256 tensors

struct OptTensors {
    float* w[OPT_MAXT];
    float* g[OPT_MAXT];
    float* m[OPT_MAXT];
    float* v[OPT_MAXT];
    long long n[OPT_MAXT];
    int chunk_start[OPT_MAXT + 1];      // prefix sums of ceil(n / OPT_CHUNK)
    int count;
    int vec_ok;                         // every pointer 16-byte aligned
};

struct OptScalars {                     // f64 hyper-parameters rounded to f32 where the reference does
    float beta1, one_minus_beta1, beta2, one_minus_beta2;
    float inv_bc1, inv_bc2;             // 1 / (1 - beta^t)
    float decay;                        // 1 - lr * weight_decay
    float lr, eps;
    int has_decay;
    int use_clip;
    int skip_nonfinite;                 // leave w, m, v untouched when the norm is not finite
    double max_norm;
};

__device__ __forceinline__ int find_tensor(const OptTensors& t, int chunk) {
    int lo = 0, hi = t.count;           // chunk_start[lo] <= chunk < chunk_start[hi]
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (t.chunk_start[mid] <= chunk) lo = mid; else hi = mid;
    }
    return lo;
}

// Partial sums of squares: block b takes chunks b, b + grid, ...; thread-local accumulation in
// element order, then a fixed shuffle / shared-memory tree.
__global__ void __launch_bounds__(256) grad_sq_sum_kernel(const __grid_constant__ OptTensors t, float* __restrict__ partial) {
    const int total_chunks = t.chunk_start[t.count];
    float acc = 0.f;
    for (int chunk = blockIdx.x; chunk < total_chunks; chunk += gridDim.x) {
        const int ti = find_tensor(t, chunk);
        const long long base = (long long)(chunk - t.chunk_start[ti]) * OPT_CHUNK;
        const long long n = t.n[ti];
        const float* __restrict__ g = t.g[ti];
        if (t.vec_ok && base + OPT_CHUNK <= n) {
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                const float4 x = *reinterpret_cast<const float4*>(g + base + (r * 256 + threadIdx.x) * 4);
                acc = __fadd_rn(acc, __fmul_rn(x.x, x.x));
                acc = __fadd_rn(acc, __fmul_rn(x.y, x.y));
                acc = __fadd_rn(acc, __fmul_rn(x.z, x.z));
                acc = __fadd_rn(acc, __fmul_rn(x.w, x.w));
            }
        } else {
            for (long long i = base + threadIdx.x; i < n && i < base + OPT_CHUNK; i += 256) acc = __fadd_rn(acc, __fmul_rn(g[i], g[i]));
        }
    }
    __shared__ float warp_sum[8];
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
    if ((threadIdx.x & 31) == 0) warp_sum[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
        float s = 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w) s += warp_sum[w];
        partial[blockIdx.x] = s;
    }
}

// norm = sqrt(sum of the partials), summed by one block in a fixed order.
__global__ void __launch_bounds__(1024) grad_norm_kernel(const float* __restrict__ partial, int n, float* __restrict__ norm) {
    __shared__ float sh[1024];
    float acc = 0.f;
    for (int i = threadIdx.x; i < n; i += 1024) acc += partial[i];
    sh[threadIdx.x] = acc;
    __syncthreads();
    for (int s = 512; s >= 1; s >>= 1) {
        if ((int)threadIdx.x < s) sh[threadIdx.x] += sh[threadIdx.x + s];
        __syncthreads();
    }
    if (threadIdx.x == 0) *norm = __fsqrt_rn(sh[0]);
}

enum { MODE_STEP = 0, MODE_CLIP = 1 };

// The clip rule of clip_grad_norm (src/optim.rs:281-295): no change when the norm is not finite or
// not above max_norm, else every gradient is multiplied by max_norm / (norm + 1e-6) (f64, rounded
// to f32 by the scalar multiply).
__device__ __forceinline__ bool clip_scale(const OptScalars& s, const float* norm, float& scale) {
    scale = 1.0f;
    if (!s.use_clip) return false;
    const float nv = *norm;
    if (!isfinite(nv) || nv <= (float)s.max_norm) return false;
    scale = (float)(s.max_norm / ((double)nv + 1e-6));
    return true;
}

__device__ __forceinline__ void adamw_element(const OptScalars& s, bool clip, float scale, float& w, float g, float& m,
                                              float& v) {
    if (clip) g = __fmul_rn(g, scale);
    // m = m*beta1 + g*(1-beta1);  v = v*beta2 + (g*g)*(1-beta2)          optim.rs:229-234
    m = __fadd_rn(__fmul_rn(m, s.beta1), __fmul_rn(g, s.one_minus_beta1));
    v = __fadd_rn(__fmul_rn(v, s.beta2), __fmul_rn(__fmul_rn(g, g), s.one_minus_beta2));
    // m_hat = m * (1/bc1);  v_hat = v * (1/bc2)                            optim.rs:237-238
    const float m_hat = __fmul_rn(m, s.inv_bc1), v_hat = __fmul_rn(v, s.inv_bc2);
    // decayed = w * (1 - lr*wd) when wd > 0                                 optim.rs:241-242
    const float decayed = s.has_decay ? __fmul_rn(w, s.decay) : w;
    // update = m_hat / (sqrt(v_hat) + eps);  w = decayed - update*lr        optim.rs:245-246
    const float update = __fdiv_rn(m_hat, __fadd_rn(__fsqrt_rn(v_hat), s.eps));
    w = __fsub_rn(decayed, __fmul_rn(update, s.lr));
}

template <int MODE>
__global__ void __launch_bounds__(256) adamw_kernel(const __grid_constant__ OptTensors t, const __grid_constant__ OptScalars s,
                                                    const float* __restrict__ norm) {
    float scale;
    const bool clip = clip_scale(s, norm, scale);
    if (MODE == MODE_CLIP && !clip) return;
    if (MODE == MODE_STEP && s.skip_nonfinite && !isfinite(*norm)) return;
    const int total_chunks = t.chunk_start[t.count];
    for (int chunk = blockIdx.x; chunk < total_chunks; chunk += gridDim.x) {
        const int ti = find_tensor(t, chunk);
        const long long base = (long long)(chunk - t.chunk_start[ti]) * OPT_CHUNK;
        const long long n = t.n[ti];
        float* __restrict__ w = t.w[ti];
        float* __restrict__ g = t.g[ti];
        float* __restrict__ m = t.m[ti];
        float* __restrict__ v = t.v[ti];
        if (t.vec_ok && base + OPT_CHUNK <= n) {
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                const long long i = base + (r * 256 + threadIdx.x) * 4;
                float4 gv = *reinterpret_cast<const float4*>(g + i);
                if (MODE == MODE_CLIP) {
                    gv.x = __fmul_rn(gv.x, scale); gv.y = __fmul_rn(gv.y, scale);
                    gv.z = __fmul_rn(gv.z, scale); gv.w = __fmul_rn(gv.w, scale);
                    *reinterpret_cast<float4*>(g + i) = gv;
                } else {
                    float4 wv = *reinterpret_cast<const float4*>(w + i);
                    float4 mv = *reinterpret_cast<const float4*>(m + i);
                    float4 vv = *reinterpret_cast<const float4*>(v + i);
                    adamw_element(s, clip, scale, wv.x, gv.x, mv.x, vv.x);
                    adamw_element(s, clip, scale, wv.y, gv.y, mv.y, vv.y);
                    adamw_element(s, clip, scale, wv.z, gv.z, mv.z, vv.z);
                    adamw_element(s, clip, scale, wv.w, gv.w, mv.w, vv.w);
                    *reinterpret_cast<float4*>(w + i) = wv;
                    *reinterpret_cast<float4*>(m + i) = mv;
                    *reinterpret_cast<float4*>(v + i) = vv;
                }
            }
        } else {
            for (long long i = base + threadIdx.x; i < n && i < base + OPT_CHUNK; i += 256) {
                if (MODE == MODE_CLIP) {
                    g[i] = __fmul_rn(g[i], scale);
                } else {
                    float wv = w[i], mv = m[i], vv = v[i];
                    adamw_element(s, clip, scale, wv, g[i], mv, vv);
                    w[i] = wv; m[i] = mv; v[i] = vv;
                }
            }
        }
    }
}

// Fills one launch group; returns the number of tensors taken.
int fill_group(const deers_optim_tensor* ts, int n, int first, bool need_all, OptTensors* out) {
    OptTensors& t = *out;
    t.count = 0;
    t.vec_ok = 1;
    t.chunk_start[0] = 0;
    int i = first;
    for (; i < n && t.count < OPT_MAXT; ++i) {
        if (ts[i].n == 0) continue;
        const int c = t.count;
        t.w[c] = (float*)ts[i].w; t.g[c] = (float*)ts[i].g; t.m[c] = (float*)ts[i].m; t.v[c] = (float*)ts[i].v;
        t.n[c] = ts[i].n;
        const long long chunks = (ts[i].n + OPT_CHUNK - 1) / OPT_CHUNK;
        if ((long long)t.chunk_start[c] + chunks > 0x7fffffffLL) break;
        t.chunk_start[c + 1] = t.chunk_start[c] + (int)chunks;
        uintptr_t bits = (uintptr_t)ts[i].g;
        if (need_all) bits |= (uintptr_t)ts[i].w | (uintptr_t)ts[i].m | (uintptr_t)ts[i].v;
        if (bits & 15u) t.vec_ok = 0;
        t.count = c + 1;
    }
    return i - first;
}

// f64 integer power by squaring, the algorithm behind Rust's f64::powi (optim.rs:218-219).
double powi(double a, int b) {
    const bool recip = b < 0;
    double r = 1.0;
    while (true) {
        if (b & 1) r *= a;
        b /= 2;
        if (b == 0) break;
        a *= a;
    }
    return recip ? 1.0 / r : r;
}

int check_tensors(const deers_optim_tensor* ts, int n, bool need_all) {
    if (!ts || n < 0) return DEERS_ERR_NULL;
    if (n > OPT_MAXT * OPT_MAX_GROUPS) return DEERS_ERR_SHAPE;
    for (int i = 0; i < n; ++i) {
        if (ts[i].n < 0) return DEERS_ERR_SHAPE;
        if (ts[i].n == 0) continue;
        if (!ts[i].g || (need_all && (!ts[i].w || !ts[i].m || !ts[i].v))) return DEERS_ERR_NULL;
        uintptr_t bits = (uintptr_t)ts[i].g;
        if (need_all) bits |= (uintptr_t)ts[i].w | (uintptr_t)ts[i].m | (uintptr_t)ts[i].v;
        if (bits & 3u) return DEERS_ERR_LAYOUT;
    }
    return DEERS_OK;
}

unsigned optim_grid(const deers_ctx* ctx, int chunks) {
    const long long cap = 8LL * ctx->sm_count;
    return (unsigned)(chunks < cap ? (chunks > 0 ? chunks : 1) : cap);
}

}  // namespace

extern "C" size_t deers_b200_optim_scratch_bytes(void) {
    return (size_t)OPT_MAX_GROUPS * 8 * 256 * sizeof(float);   // partial sums: at most 8 blocks per SM, 256 SMs, per group
}

extern "C" int deers_b200_grad_norm(deers_ctx* ctx, int n_tensors, const deers_optim_tensor* tensors, float* norm_dev,
                                    void* scratch, size_t scratch_bytes) {
    if (!ctx || !norm_dev) return DEERS_ERR_NULL;
    int rc = check_tensors(tensors, n_tensors, false);
    if (rc) return rc;
    if (!scratch || scratch_bytes < deers_b200_optim_scratch_bytes() || ((uintptr_t)scratch & 3u)) return DEERS_ERR_WORKSPACE;
    DEERS_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    float* partial = (float*)scratch;
    int n_partial = 0;
    for (int first = 0; first < n_tensors;) {
        OptTensors t;
        const int took = fill_group(tensors, n_tensors, first, false, &t);
        if (took == 0) return DEERS_ERR_SHAPE;
        first += took;
        if (t.count == 0) continue;
        const unsigned grid = optim_grid(ctx, t.chunk_start[t.count]);
        if ((size_t)(n_partial + grid) * sizeof(float) > scratch_bytes) return DEERS_ERR_WORKSPACE;
        {
            KernelTimerScope ts(ctx, DEERS_K_OPTIM);
            grad_sq_sum_kernel<<<grid, 256, 0, ctx->stream>>>(t, partial + n_partial);
        }
        ctx->launches += 1;
        n_partial += (int)grid;
    }
    {
        KernelTimerScope ts(ctx, DEERS_K_OPTIM);
        grad_norm_kernel<<<1, 1024, 0, ctx->stream>>>(partial, n_partial, norm_dev);
    }
    ctx->launches += 1;
    DEERS_CUDA_TRY(ctx, cudaGetLastError());
    return DEERS_OK;
}

static int optim_apply(deers_ctx* ctx, int n_tensors, const deers_optim_tensor* tensors, const OptScalars& s,
                       const float* norm_dev, int mode) {
    for (int first = 0; first < n_tensors;) {
        OptTensors t;
        const int took = fill_group(tensors, n_tensors, first, mode == MODE_STEP, &t);
        if (took == 0) return DEERS_ERR_SHAPE;
        first += took;
        if (t.count == 0) continue;
        const unsigned grid = optim_grid(ctx, t.chunk_start[t.count]);
        {
            KernelTimerScope ts(ctx, DEERS_K_OPTIM);
            if (mode == MODE_STEP) adamw_kernel<MODE_STEP><<<grid, 256, 0, ctx->stream>>>(t, s, norm_dev);
            else adamw_kernel<MODE_CLIP><<<grid, 256, 0, ctx->stream>>>(t, s, norm_dev);
        }
        ctx->launches += 1;
    }
    DEERS_CUDA_TRY(ctx, cudaGetLastError());
    return DEERS_OK;
}

extern "C" int deers_b200_grad_clip(deers_ctx* ctx, int n_tensors, const deers_optim_tensor* tensors, const float* norm_dev,
                                    double max_norm) {
    if (!ctx || !norm_dev) return DEERS_ERR_NULL;
    if (!(max_norm > 0.0)) return DEERS_ERR_SHAPE;                      // "max_norm must be positive", optim.rs:262
    int rc = check_tensors(tensors, n_tensors, false);
    if (rc) return rc;
    DEERS_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    OptScalars s = {};
    s.use_clip = 1;
    s.max_norm = max_norm;
    return optim_apply(ctx, n_tensors, tensors, s, norm_dev, MODE_CLIP);
}

extern "C" int deers_b200_adamw_step(deers_ctx* ctx, int n_tensors, const deers_optim_tensor* tensors,
                                     const deers_adamw_hyper* h, const float* norm_dev, double max_norm) {
    return launch_adamw(ctx, n_tensors, tensors, h, norm_dev, max_norm, false);
}

int launch_adamw(deers_ctx* ctx, int n_tensors, const deers_optim_tensor* tensors, const deers_adamw_hyper* h,
                 const float* norm_dev, double max_norm, bool skip_nonfinite) {
    if (!ctx || !h) return DEERS_ERR_NULL;
    if (h->step < 1) return DEERS_ERR_SHAPE;
    if (norm_dev && !(max_norm > 0.0) && !skip_nonfinite) return DEERS_ERR_SHAPE;
    int rc = check_tensors(tensors, n_tensors, true);
    if (rc) return rc;
    DEERS_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    OptScalars s = {};
    // f64 arithmetic on the host exactly as optim.rs:217-219,230-246 does it, then one rounding to f32
    // where the reference's scalar ops cast (`self.0 as f32`, src/storage.rs:105-123).
    const double bc1 = 1.0 - powi(h->beta1, (int)h->step);
    const double bc2 = 1.0 - powi(h->beta2, (int)h->step);
    s.beta1 = (float)h->beta1; s.one_minus_beta1 = (float)(1.0 - h->beta1);
    s.beta2 = (float)h->beta2; s.one_minus_beta2 = (float)(1.0 - h->beta2);
    s.inv_bc1 = (float)(1.0 / bc1); s.inv_bc2 = (float)(1.0 / bc2);
    s.has_decay = h->weight_decay > 0.0 ? 1 : 0;
    s.decay = (float)(1.0 - h->lr * h->weight_decay);
    s.lr = (float)h->lr; s.eps = (float)h->eps;
    s.use_clip = (norm_dev && max_norm > 0.0) ? 1 : 0;
    s.skip_nonfinite = (skip_nonfinite && norm_dev) ? 1 : 0;
    s.max_norm = max_norm;
    return optim_apply(ctx, n_tensors, tensors, s, norm_dev, MODE_STEP);
}
