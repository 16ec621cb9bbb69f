// Rotary embedding fused with the layout change that feeds (and leaves) the attention op.
//
// The reference rotates q and k as [B,T,H,D] tensors (apply_rotary_emb, src/models/gpt.rs:49-73:
// narrow, four multiplies, two adds, a cat built from two transposes, src/tensor.rs:428-440) and
// then permutes them to [B,H,T,D] (gpt.rs:135-136), which leaves head_dim as the slowest stride
// and forces a compaction copy before the batched GEMM.  Here one pass reads a row of D elements
// at its (b, t, h) source address, rotates it and writes it at its (b, t, h) destination address;
// both sides take arbitrary element strides (inner stride 1), so the same kernel packs
// [B,T,H,D] -> [B,H,T,D] on the way in and, with `inverse`, carries dQ / dK back to [B,T,H,D]
// through the transposed rotation.
//
//   forward:  y1 = x1*cos + x2*sin      y2 = x1*(-sin) + x2*cos       (x1 | x2 = halves of a row)
//   inverse:  x1 = y1*cos + y2*(-sin)   x2 = y1*sin + y2*cos
//
// Arithmetic follows the reference op by op: every multiply and add rounds to the storage type
// (f32: __fmul_rn / __fadd_rn, no contraction into FMA; f16: half-precision multiplies and adds),
// so results equal the reference's CPU path bit for bit.
//
// HBM-bound: 2 * N * sizeof(T) bytes per call plus the (L2-resident) cos / sin cache.
#include <cuda_fp16.h>

#include "common.cuh"

namespace {

struct RopeParams {
    const void* src;
    void* dst;
    const void* cosp;
    const void* sinp;
    long long s_b, s_t, s_h;        // source strides (elements) in (b, t, h) order
    long long d_b, d_t, d_h;        // destination strides
    int B, T, H, D;
    int inverse;
};

// One thread owns V elements of the first half of a row and the matching V of the second half.
// f16: V = 8 (16 bytes), f32: V = 4 (16 bytes); the scalar variant (V = 1) takes any even D and
// any alignment.

__device__ __forceinline__ void rotate(const float a, const float b, const float c, const float s, float& o1, float& o2) {
    // o1 = a*c + b*s ; o2 = a*(-s) + b*c, each product and sum rounded on its own
    o1 = __fadd_rn(__fmul_rn(a, c), __fmul_rn(b, s));
    o2 = __fadd_rn(__fmul_rn(a, -s), __fmul_rn(b, c));
}
__device__ __forceinline__ void rotate(const __half2 a, const __half2 b, const __half2 c, const __half2 s, __half2& o1,
                                       __half2& o2) {
    // the _rn forms are never contracted into a fused multiply-add
    o1 = __hadd2_rn(__hmul2_rn(a, c), __hmul2_rn(b, s));
    o2 = __hadd2_rn(__hmul2_rn(a, __hneg2(s)), __hmul2_rn(b, c));
}
__device__ __forceinline__ void rotate(const __half a, const __half b, const __half c, const __half s, __half& o1,
                                       __half& o2) {
    o1 = __hadd_rn(__hmul_rn(a, c), __hmul_rn(b, s));
    o2 = __hadd_rn(__hmul_rn(a, __hneg(s)), __hmul_rn(b, c));
}

template <typename T, int V>
__global__ void __launch_bounds__(256) rope_pack_kernel(const RopeParams p) {
    const int half = p.D / 2;
    const int cpr = half / V;                                   // chunks (threads) per row
    const long long rows = (long long)p.B * p.T * p.H;
    const long long total = rows * cpr;
    const T* __restrict__ src = static_cast<const T*>(p.src);
    T* __restrict__ dst = static_cast<T*>(p.dst);
    const T* __restrict__ cosp = static_cast<const T*>(p.cosp);
    const T* __restrict__ sinp = static_cast<const T*>(p.sinp);
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (long long)gridDim.x * blockDim.x) {
        const long long row = idx / cpr;                        // (b, t, h) in source order
        const int c = (int)(idx - row * cpr) * V;
        const int h = (int)(row % p.H);
        const long long bt = row / p.H;
        const int t = (int)(bt % p.T);
        const long long b = bt / p.T;
        const T* s1 = src + b * p.s_b + (long long)t * p.s_t + (long long)h * p.s_h + c;
        T* d1 = dst + b * p.d_b + (long long)t * p.d_t + (long long)h * p.d_h + c;
        const T* cs = cosp + (long long)t * half + c;
        const T* sn = sinp + (long long)t * half + c;
        if constexpr (V == 1) {
            T o1, o2;
            const T sv = p.inverse ? -sn[0] : sn[0];
            rotate(s1[0], s1[half], cs[0], sv, o1, o2);
            d1[0] = o1;
            d1[half] = o2;
        } else if constexpr (sizeof(T) == 2) {
            const uint4 a = *reinterpret_cast<const uint4*>(s1);
            const uint4 bq = *reinterpret_cast<const uint4*>(s1 + half);
            const uint4 cq = *reinterpret_cast<const uint4*>(cs);
            uint4 sq = *reinterpret_cast<const uint4*>(sn);
            if (p.inverse) { sq.x ^= 0x80008000u; sq.y ^= 0x80008000u; sq.z ^= 0x80008000u; sq.w ^= 0x80008000u; }
            uint4 o1, o2;
            const uint32_t av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {bq.x, bq.y, bq.z, bq.w};
            const uint32_t cv[4] = {cq.x, cq.y, cq.z, cq.w}, sv[4] = {sq.x, sq.y, sq.z, sq.w};
            uint32_t r1[4], r2[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                __half2 x1, x2;
                rotate(*reinterpret_cast<const __half2*>(&av[e]), *reinterpret_cast<const __half2*>(&bv[e]),
                       *reinterpret_cast<const __half2*>(&cv[e]), *reinterpret_cast<const __half2*>(&sv[e]), x1, x2);
                r1[e] = *reinterpret_cast<uint32_t*>(&x1);
                r2[e] = *reinterpret_cast<uint32_t*>(&x2);
            }
            o1 = make_uint4(r1[0], r1[1], r1[2], r1[3]);
            o2 = make_uint4(r2[0], r2[1], r2[2], r2[3]);
            *reinterpret_cast<uint4*>(d1) = o1;
            *reinterpret_cast<uint4*>(d1 + half) = o2;
        } else {
            const float4 a = *reinterpret_cast<const float4*>(s1);
            const float4 bq = *reinterpret_cast<const float4*>(s1 + half);
            const float4 cq = *reinterpret_cast<const float4*>(cs);
            float4 sq = *reinterpret_cast<const float4*>(sn);
            if (p.inverse) { sq.x = -sq.x; sq.y = -sq.y; sq.z = -sq.z; sq.w = -sq.w; }
            float4 o1, o2;
            rotate(a.x, bq.x, cq.x, sq.x, o1.x, o2.x);
            rotate(a.y, bq.y, cq.y, sq.y, o1.y, o2.y);
            rotate(a.z, bq.z, cq.z, sq.z, o1.z, o2.z);
            rotate(a.w, bq.w, cq.w, sq.w, o1.w, o2.w);
            *reinterpret_cast<float4*>(d1) = o1;
            *reinterpret_cast<float4*>(d1 + half) = o2;
        }
    }
}

bool aligned16(const void* p) { return ((uintptr_t)p & 15u) == 0; }

template <typename T, int VMAX>
int rope_launch(deers_ctx* ctx, const deers_rope_desc* d, const RopeParams& p) {
    const int half = d->D / 2;
    const size_t es = sizeof(T);
    // The 16-byte path needs every row start, both halves and the cache rows on 16-byte boundaries.
    bool vec = (half % VMAX) == 0 && aligned16(p.src) && aligned16(p.dst) && aligned16(p.cosp) && aligned16(p.sinp);
    const long long strides[6] = {p.s_b, p.s_t, p.s_h, p.d_b, p.d_t, p.d_h};
    for (long long s : strides) vec = vec && ((s * (long long)es) % 16 == 0);
    const long long rows = (long long)d->B * d->T * d->H;
    const long long total = rows * (vec ? half / VMAX : half);
    if (total == 0) return DEERS_OK;
    long long want = (total + 255) / 256;
    const long long cap = 16LL * ctx->sm_count;                  // grid-stride beyond 16 blocks per SM
    const unsigned grid = (unsigned)(want < cap ? want : cap);
    {
        KernelTimerScope ts(ctx, DEERS_K_ROPE);
        if (vec) rope_pack_kernel<T, VMAX><<<grid, 256, 0, ctx->stream>>>(p);
        else rope_pack_kernel<T, 1><<<grid, 256, 0, ctx->stream>>>(p);
    }
    ctx->launches += 1;
    DEERS_CUDA_TRY(ctx, cudaGetLastError());
    return DEERS_OK;
}

}  // namespace

extern "C" int deers_b200_rope_pack(deers_ctx* ctx, const deers_rope_desc* d, const void* src, const void* cosp,
                                    const void* sinp, void* dst) {
    if (!ctx || !d || !src || !cosp || !sinp || !dst) return DEERS_ERR_NULL;
    if (d->dtype != DEERS_F16 && d->dtype != DEERS_F32) return DEERS_ERR_DTYPE;
    if (d->B < 1 || d->T < 1 || d->H < 1 || d->D < 2 || (d->D & 1)) return DEERS_ERR_SHAPE;   // RoPE needs an even head_dim
    if (d->src_strides[3] != 1 || d->dst_strides[3] != 1) return DEERS_ERR_LAYOUT;
    for (int i = 0; i < 3; ++i)
        if (d->src_strides[i] < 0 || d->dst_strides[i] < 0) return DEERS_ERR_LAYOUT;
    const size_t es = d->dtype == DEERS_F16 ? 2 : 4;
    if (((uintptr_t)src | (uintptr_t)dst | (uintptr_t)cosp | (uintptr_t)sinp) & (es - 1)) return DEERS_ERR_LAYOUT;
    DEERS_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    RopeParams p;
    p.src = src; p.dst = dst; p.cosp = cosp; p.sinp = sinp;
    p.s_b = d->src_strides[0]; p.s_t = d->src_strides[1]; p.s_h = d->src_strides[2];
    p.d_b = d->dst_strides[0]; p.d_t = d->dst_strides[1]; p.d_h = d->dst_strides[2];
    p.B = d->B; p.T = d->T; p.H = d->H; p.D = d->D; p.inverse = d->inverse ? 1 : 0;
    return d->dtype == DEERS_F16 ? rope_launch<__half, 8>(ctx, d, p) : rope_launch<float, 4>(ctx, d, p);
}
