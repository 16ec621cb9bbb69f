// RMSNorm forward and backward, f32, one pass each.
//
// The reference evaluates `x * (mean(x*x, last axis) + eps)^-0.5` (RMSNorm::forward,
// src/nn.rs:244-251) as six graph ops (multiply, sum, scalar multiply, scalar add, scalar power,
// broadcast multiply) and its backward as the autograd of those (src/ops.rs:210-214, 638-643,
// 675-679, 777-799): about fifteen launches and ten row- or tensor-sized temporaries per call, twice
// per transformer block plus once before the head.  Here a warp owns a row: it reads the row once,
// reduces x*x with shuffles, and writes y (and the row's inverse norm, kept for the backward like the
// row lse of the attention op); the backward reads x and dy once and writes dx:
//     inv = 1 / sqrt(sum(x*x) / n + eps)            y  = x * inv
//     dx  = dy * inv - x * (sum(dy * x) * inv^3 / n)
// Rows of up to 1024 elements are owned by a warp, up to 8192 by a block (both keep the row in registers: one
// pass over HBM); longer rows take two passes of 16-byte loads.
// HBM-bound: 8 bytes per element forward, 12 backward.  Sums are f32 shuffle trees (the reference
// sums left to right), so parity is to rounding, not to the bit.
#include "common.cuh"

namespace {

constexpr int RN_MAXV = 8;      // float4 pieces per lane: rows of up to 32 * 8 * 4 = 1024 elements stay in registers

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    return v;
}

// BWD = false: y = x * inv, inv_out[row] = inv.   BWD = true: dx from x, dy and the saved inv.
template <bool BWD, bool VEC, bool VEC2 = false>
__global__ void __launch_bounds__(256) rmsnorm_kernel(const float* __restrict__ x, const float* __restrict__ dy,
                                                      const float* __restrict__ add, float* __restrict__ out,
                                                      float* __restrict__ inv_io, long long rows, int C, float eps,
                                                      float inv_n) {
    const int lane = threadIdx.x & 31;
    const long long warp = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
    const long long nwarps = (long long)gridDim.x * 8;
    for (long long row = warp; row < rows; row += nwarps) {
        const float* xr = x + row * C;
        float* orow = out + row * C;
        if (VEC) {
            const int nv = C / 4;                               // float4 pieces in the row (<= 32 * RN_MAXV)
            float4 xv[RN_MAXV], gv[RN_MAXV];
            float acc = 0.f;
#pragma unroll
            for (int i = 0; i < RN_MAXV; ++i) {
                const int p = lane + 32 * i;
                if (p < nv) {
                    xv[i] = reinterpret_cast<const float4*>(xr)[p];
                    if (BWD) {
                        gv[i] = reinterpret_cast<const float4*>(dy + row * C)[p];
                        acc += xv[i].x * gv[i].x + xv[i].y * gv[i].y + xv[i].z * gv[i].z + xv[i].w * gv[i].w;
                    } else {
                        acc += xv[i].x * xv[i].x + xv[i].y * xv[i].y + xv[i].z * xv[i].z + xv[i].w * xv[i].w;
                    }
                }
            }
            acc = warp_sum(acc);
            float inv, k = 0.f;
            if (BWD) {
                inv = inv_io[row];
                k = acc * inv * inv * inv * inv_n;
            } else {
                inv = 1.0f / sqrtf(acc * inv_n + eps);
                if (lane == 0) inv_io[row] = inv;
            }
#pragma unroll
            for (int i = 0; i < RN_MAXV; ++i) {
                const int p = lane + 32 * i;
                if (p < nv) {
                    float4 o;
                    if (BWD) {
                        o.x = gv[i].x * inv - xv[i].x * k; o.y = gv[i].y * inv - xv[i].y * k;
                        o.z = gv[i].z * inv - xv[i].z * k; o.w = gv[i].w * inv - xv[i].w * k;
                        if (add) {
                            const float4 r = reinterpret_cast<const float4*>(add + row * C)[p];
                            o.x = r.x + o.x; o.y = r.y + o.y; o.z = r.z + o.z; o.w = r.w + o.w;
                        }
                    } else {
                        o.x = xv[i].x * inv; o.y = xv[i].y * inv; o.z = xv[i].z * inv; o.w = xv[i].w * inv;
                    }
                    reinterpret_cast<float4*>(orow)[p] = o;
                }
            }
        } else if (VEC2) {                                      // long aligned rows: two passes of 16-byte loads
            const int nv = C / 4;
            const float4* x4 = reinterpret_cast<const float4*>(xr);
            const float4* g4 = BWD ? reinterpret_cast<const float4*>(dy + row * C) : nullptr;
            float acc = 0.f;
            for (int p = lane; p < nv; p += 32) {
                const float4 a = x4[p];
                if (BWD) {
                    const float4 b = g4[p];
                    acc += a.x * b.x + a.y * b.y + a.z * b.z + a.w * b.w;
                } else {
                    acc += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
                }
            }
            acc = warp_sum(acc);
            float inv, k = 0.f;
            if (BWD) {
                inv = inv_io[row];
                k = acc * inv * inv * inv * inv_n;
            } else {
                inv = 1.0f / sqrtf(acc * inv_n + eps);
                if (lane == 0) inv_io[row] = inv;
            }
            for (int p = lane; p < nv; p += 32) {               // the row (<= a few KB per lane group) is still in L1 / L2
                const float4 a = x4[p];
                float4 o;
                if (BWD) {
                    const float4 b = g4[p];
                    o.x = b.x * inv - a.x * k; o.y = b.y * inv - a.y * k; o.z = b.z * inv - a.z * k; o.w = b.w * inv - a.w * k;
                    if (add) {
                        const float4 r = reinterpret_cast<const float4*>(add + row * C)[p];
                        o.x = r.x + o.x; o.y = r.y + o.y; o.z = r.z + o.z; o.w = r.w + o.w;
                    }
                } else {
                    o.x = a.x * inv; o.y = a.y * inv; o.z = a.z * inv; o.w = a.w * inv;
                }
                reinterpret_cast<float4*>(orow)[p] = o;
            }
        } else {                                                // any C, any alignment: two passes over the row
            const float* gr = BWD ? dy + row * C : nullptr;
            float acc = 0.f;
            for (int c = lane; c < C; c += 32) acc += BWD ? xr[c] * gr[c] : xr[c] * xr[c];
            acc = warp_sum(acc);
            float inv, k = 0.f;
            if (BWD) {
                inv = inv_io[row];
                k = acc * inv * inv * inv * inv_n;
            } else {
                inv = 1.0f / sqrtf(acc * inv_n + eps);
                if (lane == 0) inv_io[row] = inv;
            }
            for (int c = lane; c < C; c += 32) {
                float o = BWD ? gr[c] * inv - xr[c] * k : xr[c] * inv;
                if (BWD && add) o = add[row * C + c] + o;
                orow[c] = o;
            }
        }
    }
}

// Rows of 1025 .. 8192 elements: a whole block owns a row, which still stays in registers (one pass over HBM).
template <bool BWD>
__global__ void __launch_bounds__(256) rmsnorm_block_kernel(const float* __restrict__ x, const float* __restrict__ dy,
                                                            const float* __restrict__ add, float* __restrict__ out,
                                                            float* __restrict__ inv_io, long long rows, int C, float eps,
                                                            float inv_n) {
    __shared__ float part[8];
    const int nv = C / 4;                                       // <= 256 * RN_MAXV
    for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
        const float4* x4 = reinterpret_cast<const float4*>(x + row * C);
        const float4* g4 = BWD ? reinterpret_cast<const float4*>(dy + row * C) : nullptr;
        float4 xv[RN_MAXV], gv[RN_MAXV];
        float acc = 0.f;
#pragma unroll
        for (int i = 0; i < RN_MAXV; ++i) {
            const int p = threadIdx.x + 256 * i;
            if (p < nv) {
                xv[i] = x4[p];
                if (BWD) {
                    gv[i] = g4[p];
                    acc += xv[i].x * gv[i].x + xv[i].y * gv[i].y + xv[i].z * gv[i].z + xv[i].w * gv[i].w;
                } else {
                    acc += xv[i].x * xv[i].x + xv[i].y * xv[i].y + xv[i].z * xv[i].z + xv[i].w * xv[i].w;
                }
            }
        }
        acc = warp_sum(acc);
        __syncthreads();                                        // part[] of the previous row has been read
        if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = acc;
        __syncthreads();
        float tot = 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w) tot += part[w];
        float inv, k = 0.f;
        if (BWD) {
            inv = inv_io[row];
            k = tot * inv * inv * inv * inv_n;
        } else {
            inv = 1.0f / sqrtf(tot * inv_n + eps);
            if (threadIdx.x == 0) inv_io[row] = inv;
        }
        float4* o4 = reinterpret_cast<float4*>(out + row * C);
#pragma unroll
        for (int i = 0; i < RN_MAXV; ++i) {
            const int p = threadIdx.x + 256 * i;
            if (p < nv) {
                float4 o;
                if (BWD) {
                    o.x = gv[i].x * inv - xv[i].x * k; o.y = gv[i].y * inv - xv[i].y * k;
                    o.z = gv[i].z * inv - xv[i].z * k; o.w = gv[i].w * inv - xv[i].w * k;
                    if (add) {
                        const float4 r = reinterpret_cast<const float4*>(add + row * C)[p];
                        o.x = r.x + o.x; o.y = r.y + o.y; o.z = r.z + o.z; o.w = r.w + o.w;
                    }
                } else {
                    o.x = xv[i].x * inv; o.y = xv[i].y * inv; o.z = xv[i].z * inv; o.w = xv[i].w * inv;
                }
                o4[p] = o;
            }
        }
    }
}

template <bool BWD>
int rms_launch(deers_ctx* ctx, long long rows, int C, float eps, const float* x, const float* dy, float* out, float* inv,
               const float* add = nullptr) {
    if (rows == 0) return DEERS_OK;
    uintptr_t bits = (uintptr_t)x | (uintptr_t)out | (BWD ? (uintptr_t)dy : 0) | (uintptr_t)add;
    const bool aligned = (C % 4) == 0 && (bits & 15u) == 0;
    const bool vec = aligned && C <= 32 * RN_MAXV * 4;
    const long long want = (rows + 7) / 8;
    const long long cap = 16LL * ctx->sm_count;
    const unsigned grid = (unsigned)(want < cap ? want : cap);
    const float inv_n = (float)(1.0 / (double)C);               // mean = sum * (1/n as f64 -> f32), src/tensor.rs:461-465
    {
        KernelTimerScope ts(ctx, DEERS_K_NORM);
        if (vec) rmsnorm_kernel<BWD, true><<<grid, 256, 0, ctx->stream>>>(x, dy, add, out, inv, rows, C, eps, inv_n);
        else if (aligned && C <= 256 * RN_MAXV * 4) {
            const unsigned bgrid = (unsigned)(rows < cap ? rows : cap);
            rmsnorm_block_kernel<BWD><<<bgrid, 256, 0, ctx->stream>>>(x, dy, add, out, inv, rows, C, eps, inv_n);
        } else if (aligned) rmsnorm_kernel<BWD, false, true><<<grid, 256, 0, ctx->stream>>>(x, dy, add, out, inv, rows, C, eps, inv_n);
        else rmsnorm_kernel<BWD, false><<<grid, 256, 0, ctx->stream>>>(x, dy, add, out, inv, rows, C, eps, inv_n);
    }
    ctx->launches += 1;
    DEERS_CUDA_TRY(ctx, cudaGetLastError());
    return DEERS_OK;
}

int rms_check(const deers_ctx* ctx, long long rows, int C, const void* a, const void* b, const void* c, const void* d) {
    if (!ctx || !a || !b || !c || !d) return DEERS_ERR_NULL;
    if (rows < 0 || C < 1) return DEERS_ERR_SHAPE;
    if (((uintptr_t)a | (uintptr_t)b | (uintptr_t)c | (uintptr_t)d) & 3u) return DEERS_ERR_LAYOUT;
    return DEERS_OK;
}

}  // namespace

extern "C" int deers_b200_rmsnorm_fwd(deers_ctx* ctx, int64_t rows, int32_t C, double eps, const float* x, float* y,
                                      float* inv_norm) {
    int rc = rms_check(ctx, rows, C, x, y, inv_norm, x);
    if (rc) return rc;
    DEERS_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    return rms_launch<false>(ctx, rows, C, (float)eps, x, nullptr, y, inv_norm);
}

// Internal launchers for the model step (gpt_model.cu).
int launch_rmsnorm_fwd(deers_ctx* ctx, long long rows, int C, double eps, const float* x, float* y, float* inv_norm) {
    return rms_launch<false>(ctx, rows, C, (float)eps, x, nullptr, y, inv_norm);
}
int launch_rmsnorm_bwd(deers_ctx* ctx, long long rows, int C, const float* x, const float* inv_norm, const float* dy,
                       const float* add, float* dx) {
    return rms_launch<true>(ctx, rows, C, 0.f, x, dy, dx, const_cast<float*>(inv_norm), add);
}

extern "C" int deers_b200_rmsnorm_bwd_add(deers_ctx* ctx, int64_t rows, int32_t C, const float* x, const float* inv_norm,
                                          const float* dy, const float* residual_grad, float* dx) {
    int rc = rms_check(ctx, rows, C, x, inv_norm, dy, dx);
    if (rc) return rc;
    if (!residual_grad) return DEERS_ERR_NULL;
    if ((uintptr_t)residual_grad & 3u) return DEERS_ERR_LAYOUT;
    DEERS_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    return rms_launch<true>(ctx, rows, C, 0.f, x, dy, dx, const_cast<float*>(inv_norm), residual_grad);
}

extern "C" int deers_b200_rmsnorm_bwd(deers_ctx* ctx, int64_t rows, int32_t C, const float* x, const float* inv_norm,
                                      const float* dy, float* dx) {
    int rc = rms_check(ctx, rows, C, x, inv_norm, dy, dx);
    if (rc) return rc;
    DEERS_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    return rms_launch<true>(ctx, rows, C, 0.f, x, dy, dx, const_cast<float*>(inv_norm));
}
