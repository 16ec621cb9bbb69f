// Decode-time attention: a few new query rows against a long key / value cache (split-KV).
//
// The reference's mask helper already models queries that sit `seqlen_offset` positions into a longer
// key sequence (causal_mask, src/nn/functional.rs:12-55: key j is masked for query i iff
// j > i + seqlen_offset), but its sampling loop re-runs the whole prefix for every token
// (src/bin/tinystories_train.rs sampling: O(T^2) per token).  With a KV cache the step is
// `softmax(scale * q K^T + mask) V` for Tq new rows against Tk = Tq + offset cached rows: no tensor-core
// shape (M = Tq is tiny), purely bound by reading K and V once.
//
//   decode_partial_vec_kernel  grid (splits, B*H): a block takes one chunk of the keys of one slice; its four
//                           warps stride over the chunk's keys; the lanes that share a key each own 16 bytes
//                           of its row (16-byte loads, four key groups in flight): dot product by shuffle
//                           reduction, online softmax, V accumulated in registers (f32); lane groups and
//                           warps are merged and the block writes (max, sum, unnormalised O) of its chunk
//                           to the workspace.
//   decode_partial_kernel   the same with element loads, for rows that are not a power-of-two number of
//                           aligned 16-byte pieces.
//   decode_combine_kernel   merges the chunks of a (slice, query) pair, normalises, writes O (and lse).
// K and V are read once per query row (Tq is 1 in sampling); 2 * Tk * D * sizeof(T) bytes per slice.
#include <cuda_fp16.h>

#include "common.cuh"

namespace {

constexpr int DEC_MAXC = 8;             // channels per lane: head_dim <= 256
constexpr float DEC_LOG2E = 1.4426950408889634f;

struct DecodeParams {
    const void* q; const void* k; const void* v; void* o;
    float* lse;                          // [B*H*Tq] or nullptr
    float* part;                         // [B*H][Tq][splits][D + 2]
    long long sq[3], sk[3], sv[3], so[3];   // (b, h, t) strides in elements
    int B, H, Tq, Tk, D, causal, splits, chunk;
    float scale;
};

__device__ __forceinline__ float ld(const float* p) { return *p; }
__device__ __forceinline__ float ld(const __half* p) { return __half2float(*p); }
__device__ __forceinline__ void st(float* p, float v) { *p = v; }
__device__ __forceinline__ void st(__half* p, float v) { *p = __float2half_rn(v); }

template <typename T>
__global__ void __launch_bounds__(128) decode_partial_kernel(const DecodeParams p) {
    const int split = blockIdx.x, bh = blockIdx.y;
    const int b = bh / p.H, h = bh % p.H;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nc = (p.D + 31) / 32;                              // channels of this lane: lane, lane + 32, ...
    const int k_begin = split * p.chunk, k_end = min(p.Tk, k_begin + p.chunk);
    const int offset = p.Tk - p.Tq;
    const T* kb = static_cast<const T*>(p.k) + b * p.sk[0] + h * p.sk[1];
    const T* vb = static_cast<const T*>(p.v) + b * p.sv[0] + h * p.sv[1];
    const float sl2 = p.scale * DEC_LOG2E;
    __shared__ float sm_m[4], sm_l[4];
    __shared__ float sm_o[4][32 * DEC_MAXC];

    for (int i = 0; i < p.Tq; ++i) {
        const T* qr = static_cast<const T*>(p.q) + b * p.sq[0] + h * p.sq[1] + (long long)i * p.sq[2];
        float qv[DEC_MAXC], acc[DEC_MAXC];
#pragma unroll
        for (int c = 0; c < DEC_MAXC; ++c) {
            const int d = lane + 32 * c;
            qv[c] = (c < nc && d < p.D) ? ld(qr + d) : 0.f;
            acc[c] = 0.f;
        }
        const int last = p.causal ? min(k_end, i + offset + 1) : k_end;      // keys j <= i + offset
        float m = -INFINITY, l = 0.f;
        for (int j0 = k_begin + warp * 4; j0 < last; j0 += 16) {             // four keys per warp iteration
            float s[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int j = j0 + u;
                float dot = 0.f;
                if (j < last) {
                    const T* kr = kb + (long long)j * p.sk[2];
#pragma unroll
                    for (int c = 0; c < DEC_MAXC; ++c) {
                        const int d = lane + 32 * c;
                        if (c < nc && d < p.D) dot = fmaf(qv[c], ld(kr + d), dot);
                    }
                }
                s[u] = dot;
            }
#pragma unroll
            for (int off = 16; off >= 1; off >>= 1) {
#pragma unroll
                for (int u = 0; u < 4; ++u) s[u] += __shfl_xor_sync(0xffffffffu, s[u], off);
            }
            float mx = m;
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                s[u] = (j0 + u < last) ? s[u] * sl2 : -INFINITY;
                mx = fmaxf(mx, s[u]);
            }
            const float corr = exp2f(m - mx);                                // 0 on the first keys (m = -inf)
            l *= corr;
#pragma unroll
            for (int c = 0; c < DEC_MAXC; ++c) acc[c] *= corr;
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int j = j0 + u;
                if (j < last) {
                    const float pj = exp2f(s[u] - mx);
                    l += pj;
                    const T* vr = vb + (long long)j * p.sv[2];
#pragma unroll
                    for (int c = 0; c < DEC_MAXC; ++c) {
                        const int d = lane + 32 * c;
                        if (c < nc && d < p.D) acc[c] = fmaf(pj, ld(vr + d), acc[c]);
                    }
                }
            }
            m = mx;
        }
        // merge the four warps (a warp without keys has m = -inf, l = 0)
        __syncthreads();                                                     // shared arrays of the previous query are free
        if (lane == 0) { sm_m[warp] = m; sm_l[warp] = l; }
#pragma unroll
        for (int c = 0; c < DEC_MAXC; ++c) sm_o[warp][lane + 32 * c] = acc[c];
        __syncthreads();
        if (warp == 0) {
            float mm = fmaxf(fmaxf(sm_m[0], sm_m[1]), fmaxf(sm_m[2], sm_m[3]));
            const float ms = (mm == -INFINITY) ? 0.f : mm;
            float w[4], ll = 0.f;
#pragma unroll
            for (int x = 0; x < 4; ++x) { w[x] = exp2f(sm_m[x] - ms); ll += w[x] * sm_l[x]; }
            float* out = p.part + (((long long)bh * p.Tq + i) * p.splits + split) * (p.D + 2);
#pragma unroll
            for (int c = 0; c < DEC_MAXC; ++c) {
                const int d = lane + 32 * c;
                if (c < nc && d < p.D) {
                    float o = 0.f;
#pragma unroll
                    for (int x = 0; x < 4; ++x) o += w[x] * sm_o[x][d];
                    out[d] = o;
                }
            }
            if (lane == 0) { out[p.D] = mm; out[p.D + 1] = ll; }
        }
    }
}

// 16-byte path: LPK lanes share a key (each owns 16 bytes of its row), so a warp instruction covers 32 / LPK
// keys; four such groups of keys are in flight per iteration.  Needs 16-byte aligned rows.
template <typename T, int LPK>
__global__ void __launch_bounds__(128) decode_partial_vec_kernel(const DecodeParams p) {
    constexpr int VEC = 16 / (int)sizeof(T);                     // channels per lane
    constexpr int KPW = 32 / LPK;                                // keys per warp instruction
    constexpr int U = 4;                                         // key groups in flight
    const int split = blockIdx.x, bh = blockIdx.y;
    const int b = bh / p.H, h = bh % p.H;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int sub = lane / LPK, cl = lane % LPK;
    const int k_begin = split * p.chunk, k_end = min(p.Tk, k_begin + p.chunk);
    const int offset = p.Tk - p.Tq;
    const T* kb = static_cast<const T*>(p.k) + b * p.sk[0] + h * p.sk[1] + cl * VEC;
    const T* vb = static_cast<const T*>(p.v) + b * p.sv[0] + h * p.sv[1] + cl * VEC;
    const float sl2 = p.scale * DEC_LOG2E;
    __shared__ float sm_m[4], sm_l[4];
    __shared__ float sm_o[4][32 * DEC_MAXC];

    auto unpack = [](const uint4& r, float (&f)[VEC]) {
        if constexpr (sizeof(T) == 2) {
            const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 t = __half22float2(*reinterpret_cast<const __half2*>(&w[e]));
                f[2 * e] = t.x; f[2 * e + 1] = t.y;
            }
        } else {
            f[0] = __uint_as_float(r.x); f[1] = __uint_as_float(r.y); f[2] = __uint_as_float(r.z); f[3] = __uint_as_float(r.w);
        }
    };

    for (int i = 0; i < p.Tq; ++i) {
        const T* qr = static_cast<const T*>(p.q) + b * p.sq[0] + h * p.sq[1] + (long long)i * p.sq[2] + cl * VEC;
        float qv[VEC], acc[VEC];
        unpack(*reinterpret_cast<const uint4*>(qr), qv);
#pragma unroll
        for (int c = 0; c < VEC; ++c) acc[c] = 0.f;
        const int last = p.causal ? min(k_end, i + offset + 1) : k_end;
        float m = -INFINITY, l = 0.f;
        // this lane group's keys: k_begin + (warp * U + u) * KPW + sub, stepping 4 warps * U * KPW
        for (int j0 = k_begin + warp * U * KPW; j0 < last; j0 += 4 * U * KPW) {
            uint4 kr[U], vr[U];
            bool ok[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int j = j0 + u * KPW + sub;
                ok[u] = j < last;
                kr[u] = make_uint4(0u, 0u, 0u, 0u);
                vr[u] = kr[u];
                if (ok[u]) {
                    kr[u] = *reinterpret_cast<const uint4*>(kb + (long long)j * p.sk[2]);
                    vr[u] = *reinterpret_cast<const uint4*>(vb + (long long)j * p.sv[2]);
                }
            }
            float s[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                float kf[VEC];
                unpack(kr[u], kf);
                float dot = 0.f;
#pragma unroll
                for (int c = 0; c < VEC; ++c) dot = fmaf(qv[c], kf[c], dot);
                s[u] = dot;
            }
#pragma unroll
            for (int off = LPK / 2; off >= 1; off >>= 1) {
#pragma unroll
                for (int u = 0; u < U; ++u) s[u] += __shfl_xor_sync(0xffffffffu, s[u], off);
            }
            float mx = m;
#pragma unroll
            for (int u = 0; u < U; ++u) {
                s[u] = ok[u] ? s[u] * sl2 : -INFINITY;
                mx = fmaxf(mx, s[u]);
            }
            if (mx != -INFINITY) {                               // at least one key of this lane group so far
                const float corr = exp2f(m - mx);
                l *= corr;
#pragma unroll
                for (int c = 0; c < VEC; ++c) acc[c] *= corr;
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const float pj = exp2f(s[u] - mx);           // 0 for keys that do not exist
                    l += pj;
                    float vf[VEC];
                    unpack(vr[u], vf);
#pragma unroll
                    for (int c = 0; c < VEC; ++c) acc[c] = fmaf(pj, vf[c], acc[c]);
                }
                m = mx;
            }
        }
        // merge the lane groups of the warp (they saw different keys), then the four warps
#pragma unroll
        for (int off = LPK; off < 32; off <<= 1) {
            const float mo = __shfl_xor_sync(0xffffffffu, m, off), lo = __shfl_xor_sync(0xffffffffu, l, off);
            const float mn = fmaxf(m, mo);
            const float ms = (mn == -INFINITY) ? 0.f : mn;
            const float wa = exp2f(m - ms), wb = exp2f(mo - ms);
#pragma unroll
            for (int c = 0; c < VEC; ++c) acc[c] = wa * acc[c] + wb * __shfl_xor_sync(0xffffffffu, acc[c], off);
            l = wa * l + wb * lo;
            m = mn;
        }
        __syncthreads();
        if (lane == 0) { sm_m[warp] = m; sm_l[warp] = l; }
        if (sub == 0) {
#pragma unroll
            for (int c = 0; c < VEC; ++c) sm_o[warp][cl * VEC + c] = acc[c];
        }
        __syncthreads();
        if (warp == 0) {
            const float mm = fmaxf(fmaxf(sm_m[0], sm_m[1]), fmaxf(sm_m[2], sm_m[3]));
            const float ms = (mm == -INFINITY) ? 0.f : mm;
            float w[4], ll = 0.f;
#pragma unroll
            for (int x = 0; x < 4; ++x) { w[x] = exp2f(sm_m[x] - ms); ll += w[x] * sm_l[x]; }
            float* out = p.part + (((long long)bh * p.Tq + i) * p.splits + split) * (p.D + 2);
            for (int d = lane; d < p.D; d += 32) {
                float o = 0.f;
#pragma unroll
                for (int x = 0; x < 4; ++x) o += w[x] * sm_o[x][d];
                out[d] = o;
            }
            if (lane == 0) { out[p.D] = mm; out[p.D + 1] = ll; }
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(128) decode_combine_kernel(const DecodeParams p) {
    const long long row = blockIdx.x;                                        // (bh, i)
    const int bh = (int)(row / p.Tq), i = (int)(row % p.Tq);
    const int b = bh / p.H, h = bh % p.H;
    const float* part = p.part + row * p.splits * (p.D + 2);
    float mm = -INFINITY;
    for (int s = 0; s < p.splits; ++s) mm = fmaxf(mm, part[s * (p.D + 2) + p.D]);
    const float ms = (mm == -INFINITY) ? 0.f : mm;
    float l = 0.f;
    for (int s = 0; s < p.splits; ++s) l += exp2f(part[s * (p.D + 2) + p.D] - ms) * part[s * (p.D + 2) + p.D + 1];
    T* orow = static_cast<T*>(p.o) + b * p.so[0] + h * p.so[1] + (long long)i * p.so[2];
    for (int d = threadIdx.x; d < p.D; d += blockDim.x) {
        float o = 0.f;
        for (int s = 0; s < p.splits; ++s) o += exp2f(part[s * (p.D + 2) + p.D] - ms) * part[s * (p.D + 2) + d];
        st(orow + d, o / l);
    }
    if (p.lse && threadIdx.x == 0) p.lse[row] = (mm + log2f(l)) * 0.6931471805599453f;   // natural log, like the forward op
}

int decode_splits(const deers_decode_desc* d, int* chunk) {
    const long long slices = (long long)d->B * d->H;
    long long want = (4LL * 148 + slices - 1) / slices;                        // about four blocks per SM in all
    const long long max_splits = (d->Tk + 255) / 256;                          // at least 256 keys per block
    if (want > max_splits) want = max_splits;
    if (want < 1) want = 1;
    long long c = (d->Tk + want - 1) / want;
    c = (c + 15) / 16 * 16;
    *chunk = (int)c;
    return (int)((d->Tk + c - 1) / c);
}

int decode_check(const deers_decode_desc* d) {
    if (!d) return DEERS_ERR_NULL;
    if (d->dtype != DEERS_F16 && d->dtype != DEERS_F32) return DEERS_ERR_DTYPE;
    if (d->B < 1 || d->H < 1 || d->Tq < 1 || d->Tk < d->Tq || d->D < 1) return DEERS_ERR_SHAPE;
    if (d->D > 32 * DEC_MAXC || d->Tq > 128 || d->Tk > (1 << 24)) return DEERS_ERR_UNSUPPORTED;
    if ((long long)d->B * d->H > 65535) return DEERS_ERR_UNSUPPORTED;           // grid.y
    if (!(d->scale == d->scale)) return DEERS_ERR_SHAPE;
    const int64_t* ss[4] = {d->q_strides, d->k_strides, d->v_strides, d->o_strides};
    for (const int64_t* s : ss) {
        if (s[3] != 1) return DEERS_ERR_LAYOUT;
        for (int i = 0; i < 3; ++i)
            if (s[i] < 0) return DEERS_ERR_LAYOUT;
    }
    return DEERS_OK;
}

}  // namespace

extern "C" size_t deers_b200_attn_decode_workspace_bytes(const deers_decode_desc* d) {
    if (decode_check(d) != DEERS_OK) return 0;
    int chunk;
    const int splits = decode_splits(d, &chunk);
    return (size_t)d->B * d->H * d->Tq * splits * (d->D + 2) * sizeof(float);
}

extern "C" int deers_b200_attn_decode(deers_ctx* ctx, const deers_decode_desc* d, const void* q, const void* k_cache,
                                      const void* v_cache, void* o, float* lse, void* workspace, size_t workspace_bytes) {
    if (!ctx || !q || !k_cache || !v_cache || !o) return DEERS_ERR_NULL;
    int rc = decode_check(d);
    if (rc) return rc;
    const size_t es = d->dtype == DEERS_F16 ? 2 : 4;
    if (((uintptr_t)q | (uintptr_t)k_cache | (uintptr_t)v_cache | (uintptr_t)o) & (es - 1)) return DEERS_ERR_LAYOUT;
    DecodeParams p;
    p.splits = decode_splits(d, &p.chunk);
    const size_t need = (size_t)d->B * d->H * d->Tq * p.splits * (d->D + 2) * sizeof(float);
    if (!workspace || workspace_bytes < need || ((uintptr_t)workspace & 3u)) return DEERS_ERR_WORKSPACE;
    DEERS_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    p.q = q; p.k = k_cache; p.v = v_cache; p.o = o; p.lse = lse; p.part = (float*)workspace;
    for (int i = 0; i < 3; ++i) { p.sq[i] = d->q_strides[i]; p.sk[i] = d->k_strides[i]; p.sv[i] = d->v_strides[i]; p.so[i] = d->o_strides[i]; }
    p.B = d->B; p.H = d->H; p.Tq = d->Tq; p.Tk = d->Tk; p.D = d->D; p.causal = d->causal; p.scale = d->scale;
    const dim3 grid(p.splits, d->B * d->H);
    const unsigned rows = (unsigned)((long long)d->B * d->H * d->Tq);
    // 16-byte path when every row of q, K and V starts on a 16-byte boundary and a row is 1..32 pieces long
    const int row_bytes = d->D * (int)es;
    bool vec = (row_bytes % 16) == 0 && row_bytes / 16 <= 32 && ((row_bytes / 16) & (row_bytes / 16 - 1)) == 0 &&
               (((uintptr_t)q | (uintptr_t)k_cache | (uintptr_t)v_cache) & 15u) == 0;
    for (int i = 0; i < 3; ++i)
        vec = vec && (d->q_strides[i] * (int64_t)es) % 16 == 0 && (d->k_strides[i] * (int64_t)es) % 16 == 0 &&
              (d->v_strides[i] * (int64_t)es) % 16 == 0;
    {
        KernelTimerScope ts(ctx, DEERS_K_DECODE);
        const int lpk = row_bytes / 16;
        if (d->dtype == DEERS_F16) {
            if (vec && lpk == 32) decode_partial_vec_kernel<__half, 32><<<grid, 128, 0, ctx->stream>>>(p);
            else if (vec && lpk == 16) decode_partial_vec_kernel<__half, 16><<<grid, 128, 0, ctx->stream>>>(p);
            else if (vec && lpk == 8) decode_partial_vec_kernel<__half, 8><<<grid, 128, 0, ctx->stream>>>(p);
            else if (vec && lpk == 4) decode_partial_vec_kernel<__half, 4><<<grid, 128, 0, ctx->stream>>>(p);
            else decode_partial_kernel<__half><<<grid, 128, 0, ctx->stream>>>(p);
            decode_combine_kernel<__half><<<rows, 128, 0, ctx->stream>>>(p);
        } else {
            if (vec && lpk == 32) decode_partial_vec_kernel<float, 32><<<grid, 128, 0, ctx->stream>>>(p);
            else if (vec && lpk == 16) decode_partial_vec_kernel<float, 16><<<grid, 128, 0, ctx->stream>>>(p);
            else if (vec && lpk == 8) decode_partial_vec_kernel<float, 8><<<grid, 128, 0, ctx->stream>>>(p);
            else if (vec && lpk == 4) decode_partial_vec_kernel<float, 4><<<grid, 128, 0, ctx->stream>>>(p);
            else decode_partial_kernel<float><<<grid, 128, 0, ctx->stream>>>(p);
            decode_combine_kernel<float><<<rows, 128, 0, ctx->stream>>>(p);
        }
    }
    ctx->launches += 2;
    DEERS_CUDA_TRY(ctx, cudaGetLastError());
    return DEERS_OK;
}
