// Embedding lookup and cross-entropy for the f32 GPT step: the ops around the transformer blocks that
// the reference builds from index_select / index_add (src/nn.rs:214-221, src/storage/cuda.rs:359-413)
// and from log_softmax + gather + sum (src/loss.rs:11-24, src/tensor.rs:408-425).
//
//   embedding_fwd   out[n, :] = weight[ids[n], :]
//   embedding_bwd   dweight = 0; dweight[ids[n], :] += dout[n, :] in token order.  The reference adds
//                   with atomics (scatter order undefined); here the first occurrence of a token id
//                   owns the row and adds the later occurrences in order, so the result is reproducible
//                   and equals the CPU backend's left-to-right sum.
//   cross_entropy   one block per row reads the logits once (running maximum / sum of exponentials),
//                   writes lse[row] and the picked log-probability; a one-block kernel adds the rows in a
//                   fixed order: loss = sum * (float)(-1/rows).
//   cross_entropy_bwd  dlogits = (onehot * g - softmax * g) * upstream, g = (float)(-1/rows): the chain
//                   gather backward -> log_softmax backward of src/ops.rs:210-214, 777-799, 1162-1175 in one
//                   element-wise pass (in place over the logits if asked).
// A token id or target outside [0, vocab) sets the context's error word (reported by deers_b200_sync as
// DEERS_ERR_KERNEL) and is skipped; nothing traps.
#include "common.cuh"

#include <cuda_fp16.h>

namespace {

__global__ void __launch_bounds__(256) embedding_fwd_kernel(const float* __restrict__ w, const long long* __restrict__ ids,
                                                            long long n_ids, int C, long long V, float* __restrict__ out,
                                                            int vec, unsigned int* err) {
    const int lane = threadIdx.x & 31;
    const long long n = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (n >= n_ids) return;
    const long long id = ids[n];
    float* o = out + n * C;
    if (id < 0 || id >= V) {
        if (lane == 0) atomicCAS(err, 0u, (unsigned)DEERS_KERR_GPT | 1u);
        for (int c = lane; c < C; c += 32) o[c] = 0.f;
        return;
    }
    const float* s = w + id * C;
    if (vec) {
        for (int c = lane; c < C / 4; c += 32) reinterpret_cast<float4*>(o)[c] = reinterpret_cast<const float4*>(s)[c];
    } else {
        for (int c = lane; c < C; c += 32) o[c] = s[c];
    }
}

// One block per token n.  The block whose token is the first occurrence of its id writes the row.
__global__ void __launch_bounds__(256) embedding_bwd_kernel(const float* __restrict__ dout,
                                                            const long long* __restrict__ ids, long long n_ids, int C,
                                                            long long V, float* __restrict__ dw) {
    __shared__ unsigned char s_flag[256];
    const long long n = blockIdx.x;
    const long long id = ids[n];
    if (id < 0 || id >= V) return;                                     // reported by the forward
    int dup = 0;
    for (long long j = threadIdx.x; j < n; j += 256) dup |= (ids[j] == id);
    if (__syncthreads_or(dup)) return;
    for (int c0 = 0; c0 < C; c0 += 256 * 8) {                          // 8 channels per thread and sweep
        float acc[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const int c = c0 + k * 256 + threadIdx.x;
            acc[k] = c < C ? dout[n * C + c] : 0.f;
        }
        for (long long base = n + 1; base < n_ids; base += 256) {
            const long long j = base + threadIdx.x;
            const int flag = j < n_ids && ids[j] == id;
            if (!__syncthreads_or(flag)) continue;
            s_flag[threadIdx.x] = (unsigned char)flag;
            __syncthreads();
            for (int t = 0; t < 256; ++t) {
                if (!s_flag[t]) continue;
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    const int c = c0 + k * 256 + threadIdx.x;
                    if (c < C) acc[k] += dout[(base + t) * C + c];
                }
            }
            __syncthreads();
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const int c = c0 + k * 256 + threadIdx.x;
            if (c < C) dw[id * C + c] = acc[k];
        }
    }
}

// Row logsumexp + picked log-probability (src/storage/cpu.rs:759-770 computes the maximum first and then the
// sum of expf(x - max); the same value up to f32 rounding of a different summation order).
// Merges two (maximum, sum of exponentials relative to it) pairs.
__device__ __forceinline__ void lse_merge(float& m, float& s, float m2, float s2) {
    const float M = fmaxf(m, m2);
    if (M == -INFINITY) { s = 0.f; return; }                      // both parts empty
    s = s * expf(m - M) + s2 * expf(m2 - M);
    m = M;
}

// One pass over the row: every thread keeps a running maximum and the sum of exponentials relative to it (the
// sum is rescaled when the maximum grows), four values at a time when the row is 16-byte aligned; the 256 pairs
// are merged at the end.  A two-pass version (maximum, then sum) read the 206 MB of logits twice from DRAM.
__global__ void __launch_bounds__(256) cross_entropy_fwd_kernel(const float* __restrict__ logits, long long ld,
                                                                const long long* __restrict__ targets, long long V,
                                                                float* __restrict__ lse, float* __restrict__ picked,
                                                                unsigned int* err) {
    __shared__ float red_m[8], red_s[8];
    const long long row = blockIdx.x;
    const float* x = logits + row * ld;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float m = -INFINITY, s = 0.f;
    const bool vec = (((uintptr_t)x) & 15u) == 0;
    const long long V4 = vec ? V / 4 : 0;
    for (long long j = threadIdx.x; j < V4; j += 256) {
        const float4 v = *reinterpret_cast<const float4*>(x + 4 * j);
        const float vm = fmaxf(fmaxf(v.x, v.y), fmaxf(v.z, v.w));
        if (vm > m) { s *= expf(m - vm); m = vm; }                // m = -inf at first: s = 0 * 0
        s += expf(v.x - m) + expf(v.y - m) + expf(v.z - m) + expf(v.w - m);
    }
    for (long long j = 4 * V4 + threadIdx.x; j < V; j += 256) {
        const float v = x[j];
        if (v > m) { s *= expf(m - v); m = v; }
        s += expf(v - m);
    }
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1)
        lse_merge(m, s, __shfl_xor_sync(0xffffffffu, m, off), __shfl_xor_sync(0xffffffffu, s, off));
    if (lane == 0) { red_m[warp] = m; red_s[warp] = s; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < 8; ++w) lse_merge(m, s, red_m[w], red_s[w]);
        const float l = logf(s) + m;
        lse[row] = l;
        const long long t = targets[row];
        if (t < 0 || t >= V) {
            atomicCAS(err, 0u, (unsigned)DEERS_KERR_GPT | 2u);
            picked[row] = 0.f;
        } else {
            picked[row] = x[t] - l;
        }
    }
}

__global__ void __launch_bounds__(1024) cross_entropy_loss_kernel(const float* __restrict__ picked, long long rows,
                                                                  float neg_inv_rows, float* __restrict__ loss) {
    __shared__ float red[32];
    float s = 0.f;
    for (long long j = threadIdx.x; j < rows; j += 1024) s += picked[j];
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
    __syncthreads();
    if (threadIdx.x < 32) {
        s = red[threadIdx.x];
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
        if (threadIdx.x == 0) loss[0] = s * neg_inv_rows;
    }
}

__global__ void __launch_bounds__(256) cross_entropy_bwd_kernel(const float* __restrict__ logits, long long ld,
                                                                const long long* __restrict__ targets,
                                                                const float* __restrict__ lse, long long V, float g,
                                                                float upstream, float* __restrict__ dlogits,
                                                                long long ldd, int vec) {
    const long long row = blockIdx.y;
    const float* x = logits + row * ld;
    float* d = dlogits + row * ldd;
    const float l = lse[row];
    const long long t = targets[row];
    const long long stride = (long long)gridDim.x * 256;
    if (vec) {
        for (long long q = (long long)blockIdx.x * 256 + threadIdx.x; q * 4 < V; q += stride) {
            const long long j = q * 4;
            if (j + 4 <= V) {
                const float4 v = *reinterpret_cast<const float4*>(x + j);
                float o[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float p = expf(o[e] - l);
                    const float gj = (j + e == t) ? g : 0.f;
                    o[e] = __fmul_rn(__fsub_rn(gj, __fmul_rn(p, g)), upstream);
                }
                *reinterpret_cast<float4*>(d + j) = make_float4(o[0], o[1], o[2], o[3]);
            } else {
                for (long long e = j; e < V; ++e) {
                    const float p = expf(x[e] - l);
                    const float gj = (e == t) ? g : 0.f;
                    d[e] = __fmul_rn(__fsub_rn(gj, __fmul_rn(p, g)), upstream);
                }
            }
        }
    } else {
        for (long long j = (long long)blockIdx.x * 256 + threadIdx.x; j < V; j += stride) {
            const float p = expf(x[j] - l);
            const float gj = (j == t) ? g : 0.f;
            d[j] = __fmul_rn(__fsub_rn(gj, __fmul_rn(p, g)), upstream);
        }
    }
}

// The same gradient written as the f16 pair the tensor-core head products read (gemm_f16x3_sm100.cu):
// v = dlogit * scale, hi = f16(v), lo = f16((v - hi) * 2^11).  |dlogit| <= 1/rows, so scale = rows * 4096 keeps
// hi within +-4096 and the smallest probabilities that matter well inside the f16 range.
__global__ void __launch_bounds__(256) cross_entropy_bwd_split_kernel(const float* __restrict__ logits, long long ld,
                                                                      const long long* __restrict__ targets,
                                                                      const float* __restrict__ lse, long long V, float g,
                                                                      float upstream, float scale, __half* __restrict__ hi,
                                                                      __half* __restrict__ lo, long long ldd) {
    const long long row = blockIdx.y;
    const float* x = logits + row * ld;
    __half* dh = hi + row * ldd;
    __half* dl = lo + row * ldd;
    const float l = lse[row];
    const long long t = targets[row];
    const long long stride = (long long)gridDim.x * 256;
    const bool vec = (ld % 4 == 0) && (ldd % 8 == 0) && ((((uintptr_t)logits) & 15u) == 0) &&
                     ((((uintptr_t)hi | (uintptr_t)lo) & 15u) == 0);
    for (long long q = (long long)blockIdx.x * 256 + threadIdx.x; q * 8 < V; q += stride) {
        const long long j = q * 8;
        float o[8];
        if (vec && j + 8 <= V) {
            const float4 a = *reinterpret_cast<const float4*>(x + j), b = *reinterpret_cast<const float4*>(x + j + 4);
            o[0] = a.x; o[1] = a.y; o[2] = a.z; o[3] = a.w; o[4] = b.x; o[5] = b.y; o[6] = b.z; o[7] = b.w;
        } else {
#pragma unroll
            for (int e = 0; e < 8; ++e) o[e] = (j + e < V) ? x[j + e] : -INFINITY;
        }
        __half h8[8], l8[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const float pr = expf(o[e] - l);
            const float gj = (j + e == t) ? g : 0.f;
            const float d = __fmul_rn(__fsub_rn(gj, __fmul_rn(pr, g)), upstream) * scale;
            h8[e] = __float2half_rn(d);
            l8[e] = __float2half_rn((d - __half2float(h8[e])) * 2048.0f);
        }
        if (vec && j + 8 <= V) {
            *reinterpret_cast<uint4*>(dh + j) = *reinterpret_cast<const uint4*>(h8);
            *reinterpret_cast<uint4*>(dl + j) = *reinterpret_cast<const uint4*>(l8);
        } else {
            for (int e = 0; e < 8 && j + e < V; ++e) { dh[j + e] = h8[e]; dl[j + e] = l8[e]; }
        }
    }
}

}  // namespace

int launch_cross_entropy_bwd_split(deers_ctx* ctx, const float* logits, long long ld, const long long* targets,
                                   const float* lse, long long rows, long long V, float upstream, float scale, void* hi,
                                   void* lo, long long ldd) {
    long long per_row = (V / 8 + 255) / 256;
    if (per_row < 1) per_row = 1;
    if (per_row > 64) per_row = 64;
    const dim3 grid((unsigned)per_row, (unsigned)rows);
    {
        KernelTimerScope ts(ctx, DEERS_K_GPT);
        cross_entropy_bwd_split_kernel<<<grid, 256, 0, ctx->stream>>>(logits, ld, targets, lse, V, (float)(-1.0 / (double)rows),
                                                                      upstream, scale, (__half*)hi, (__half*)lo, ldd);
    }
    ctx->launches += 1;
    DEERS_CUDA_TRY(ctx, cudaGetLastError());
    return DEERS_OK;
}

int launch_embedding_fwd(deers_ctx* ctx, const float* weight, const long long* ids, long long n_ids, int C, long long V,
                         float* out) {
    if (n_ids == 0) return DEERS_OK;
    const int vec = C % 4 == 0 && (((uintptr_t)weight | (uintptr_t)out) & 15u) == 0;
    {
        KernelTimerScope ts(ctx, DEERS_K_GPT);
        embedding_fwd_kernel<<<(unsigned)((n_ids + 7) / 8), 256, 0, ctx->stream>>>(weight, ids, n_ids, C, V, out, vec,
                                                                                  ctx->dev_err);
    }
    ctx->launches += 1;
    DEERS_CUDA_TRY(ctx, cudaGetLastError());
    return DEERS_OK;
}

int launch_embedding_bwd(deers_ctx* ctx, const float* dout, const long long* ids, long long n_ids, int C, long long V,
                         float* dweight) {
    DEERS_CUDA_TRY(ctx, cudaMemsetAsync(dweight, 0, (size_t)V * C * sizeof(float), ctx->stream));
    if (n_ids == 0) return DEERS_OK;
    {
        KernelTimerScope ts(ctx, DEERS_K_GPT);
        embedding_bwd_kernel<<<(unsigned)n_ids, 256, 0, ctx->stream>>>(dout, ids, n_ids, C, V, dweight);
    }
    ctx->launches += 1;
    DEERS_CUDA_TRY(ctx, cudaGetLastError());
    return DEERS_OK;
}

int launch_cross_entropy_fwd(deers_ctx* ctx, const float* logits, long long ld, const long long* targets, long long rows,
                             long long V, float* lse, float* picked, float* loss) {
    {
        KernelTimerScope ts(ctx, DEERS_K_GPT);
        cross_entropy_fwd_kernel<<<(unsigned)rows, 256, 0, ctx->stream>>>(logits, ld, targets, V, lse, picked, ctx->dev_err);
        cross_entropy_loss_kernel<<<1, 1024, 0, ctx->stream>>>(picked, rows, (float)(-1.0 / (double)rows), loss);
    }
    ctx->launches += 2;
    DEERS_CUDA_TRY(ctx, cudaGetLastError());
    return DEERS_OK;
}

int launch_cross_entropy_loss(deers_ctx* ctx, const float* picked, long long rows, float* loss) {
    {
        KernelTimerScope ts(ctx, DEERS_K_GPT);
        cross_entropy_loss_kernel<<<1, 1024, 0, ctx->stream>>>(picked, rows, (float)(-1.0 / (double)rows), loss);
    }
    ctx->launches += 1;
    DEERS_CUDA_TRY(ctx, cudaGetLastError());
    return DEERS_OK;
}

int launch_cross_entropy_bwd(deers_ctx* ctx, const float* logits, long long ld, const long long* targets, const float* lse,
                             long long rows, long long V, float upstream, float* dlogits, long long ldd) {
    const int vec = ld % 4 == 0 && ldd % 4 == 0 && (((uintptr_t)logits | (uintptr_t)dlogits) & 15u) == 0;
    long long per_row = (V / 4 + 255) / 256;
    if (per_row < 1) per_row = 1;
    if (per_row > 64) per_row = 64;
    const dim3 grid((unsigned)per_row, (unsigned)rows);
    {
        KernelTimerScope ts(ctx, DEERS_K_GPT);
        cross_entropy_bwd_kernel<<<grid, 256, 0, ctx->stream>>>(logits, ld, targets, lse, V, (float)(-1.0 / (double)rows),
                                                                upstream, dlogits, ldd, vec);
    }
    ctx->launches += 1;
    DEERS_CUDA_TRY(ctx, cudaGetLastError());
    return DEERS_OK;
}

extern "C" int deers_b200_embedding_fwd(deers_ctx* ctx, const float* weight, const int64_t* ids, int64_t n_ids, int32_t C,
                                        int64_t vocab, float* out) {
    if (!ctx || !weight || !ids || !out) return DEERS_ERR_NULL;
    if (n_ids < 0 || C < 1 || vocab < 1 || n_ids > 0x7fffffffLL) return DEERS_ERR_SHAPE;
    if ((((uintptr_t)weight | (uintptr_t)out) & 3u) || ((uintptr_t)ids & 7u)) return DEERS_ERR_LAYOUT;
    DEERS_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    return launch_embedding_fwd(ctx, weight, (const long long*)ids, n_ids, C, vocab, out);
}

extern "C" int deers_b200_embedding_bwd(deers_ctx* ctx, const float* dout, const int64_t* ids, int64_t n_ids, int32_t C,
                                        int64_t vocab, float* dweight) {
    if (!ctx || !dout || !ids || !dweight) return DEERS_ERR_NULL;
    if (n_ids < 0 || C < 1 || vocab < 1 || n_ids > 0x7fffffffLL) return DEERS_ERR_SHAPE;
    if ((((uintptr_t)dout | (uintptr_t)dweight) & 3u) || ((uintptr_t)ids & 7u)) return DEERS_ERR_LAYOUT;
    DEERS_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    return launch_embedding_bwd(ctx, dout, (const long long*)ids, n_ids, C, vocab, dweight);
}

extern "C" size_t deers_b200_cross_entropy_scratch_bytes(int64_t rows) {
    return rows > 0 ? (size_t)rows * sizeof(float) : 0;
}

extern "C" int deers_b200_cross_entropy_fwd(deers_ctx* ctx, int64_t rows, int64_t vocab, const float* logits, int64_t ld,
                                            const int64_t* targets, float* lse, float* loss, void* scratch,
                                            size_t scratch_bytes) {
    if (!ctx || !logits || !targets || !lse || !loss) return DEERS_ERR_NULL;
    if (rows < 1 || vocab < 1 || rows > 0x7fffffffLL) return DEERS_ERR_SHAPE;
    if (ld < vocab || (((uintptr_t)logits | (uintptr_t)lse | (uintptr_t)loss) & 3u) || ((uintptr_t)targets & 7u))
        return DEERS_ERR_LAYOUT;
    if (!scratch || scratch_bytes < deers_b200_cross_entropy_scratch_bytes(rows) || ((uintptr_t)scratch & 3u))
        return DEERS_ERR_WORKSPACE;
    DEERS_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    return launch_cross_entropy_fwd(ctx, logits, ld, (const long long*)targets, rows, vocab, lse, (float*)scratch, loss);
}

extern "C" int deers_b200_cross_entropy_bwd(deers_ctx* ctx, int64_t rows, int64_t vocab, const float* logits, int64_t ld,
                                            const int64_t* targets, const float* lse, float upstream, float* dlogits,
                                            int64_t ld_dlogits) {
    if (!ctx || !logits || !targets || !lse || !dlogits) return DEERS_ERR_NULL;
    if (rows < 1 || vocab < 1 || rows > 65535) return DEERS_ERR_SHAPE;
    if (ld < vocab || ld_dlogits < vocab || (((uintptr_t)logits | (uintptr_t)lse | (uintptr_t)dlogits) & 3u) ||
        ((uintptr_t)targets & 7u))
        return DEERS_ERR_LAYOUT;
    DEERS_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    return launch_cross_entropy_bwd(ctx, logits, ld, (const long long*)targets, lse, rows, vocab, upstream, dlogits,
                                    ld_dlogits);
}
