// f32 causal attention for sm_100a: FFMA register tiling, no tensor cores and no
// TF32, so that the result holds 1e-4 against the CPU path of the reference
// (src/storage/cpu.rs:688-791 of deers).  Forward is one pass with an online
// softmax (row max / row sum reduced by warp shuffles); backward recomputes P
// from the saved lse and is split in two atomic-free kernels: a KV-tile-stationary
// one that owns dK/dV and a Q-tile-stationary one that owns dQ.  All three take
// [B,H,T,D] strides, so no compaction copy is needed around them.
#include "common.cuh"

namespace {

constexpr int BM = 64;        // query rows per tile
constexpr int BN = 64;        // key/value rows per tile
constexpr int NT = 256;       // threads per CTA: 16 x 16, each owns a 4 x 4 patch of a 64 x 64 tile
constexpr int PLD = BN + 4;   // leading dimension of the P / dS staging tiles
constexpr float LOG2E = 1.4426950408889634f;
constexpr float LN2 = 0.6931471805599453f;

struct Strides3 { long long b, h, t; };

struct F32Params {
    const float* q; const float* k; const float* v; const float* o; const float* d_o;
    float* out_o; float* lse_out; const float* lse; float* delta;
    float* dq; float* dk; float* dv;
    Strides3 sq, sk, sv, so, sdo, sdq, sdk, sdv;
    int B, H, T, D;
    int causal;
    int vec;            // 1: every row start is 16-byte aligned and D % 4 == 0
    float scale;
};

// Copies rows [row0, row0+64) x [0, DP) of a [T, D] matrix (row stride `st`) into
// shared memory with leading dimension DP+4, zero-filling rows >= T and columns >= D.
template <int DP>
__device__ __forceinline__ void load_tile(float* __restrict__ dst, const float* __restrict__ src,
                                          int row0, int T, int D, long long st, int vec) {
    constexpr int LD = DP + 4;
    constexpr int C4 = DP / 4;
    for (int idx = threadIdx.x; idx < BM * C4; idx += NT) {
        const int r = idx / C4, c = (idx % C4) * 4;
        const int row = row0 + r;
        float4 val = make_float4(0.f, 0.f, 0.f, 0.f);
        if (row < T) {
            const float* p = src + (long long)row * st + c;
            if (vec) {
                if (c < D) val = *reinterpret_cast<const float4*>(p);
            } else {
                if (c + 0 < D) val.x = p[0];
                if (c + 1 < D) val.y = p[1];
                if (c + 2 < D) val.z = p[2];
                if (c + 3 < D) val.w = p[3];
            }
        }
        *reinterpret_cast<float4*>(dst + r * LD + c) = val;
    }
}

// The same tile in two halves, global -> registers (fetch) and registers -> shared memory (put), so that the
// next tile of a walk is in flight while the current one is multiplied.  Used for head dims up to 64 (two or
// four float4 per thread and tile); at 128 the kernels have no registers to spare and load in place.
template <int DP>
struct TileRegs {
    static constexpr int C4 = DP / 4;
    static constexpr int NV = BM * C4 / NT;
    float4 v[NV];
    __device__ __forceinline__ void fetch(const float* __restrict__ src, int row0, int T, int D, long long st, int vec) {
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int idx = threadIdx.x + i * NT;
            const int r = idx / C4, c = (idx % C4) * 4;
            const int row = row0 + r;
            float4 val = make_float4(0.f, 0.f, 0.f, 0.f);
            if (row < T) {
                const float* p = src + (long long)row * st + c;
                if (vec) {
                    if (c < D) val = *reinterpret_cast<const float4*>(p);
                } else {
                    if (c + 0 < D) val.x = p[0];
                    if (c + 1 < D) val.y = p[1];
                    if (c + 2 < D) val.z = p[2];
                    if (c + 3 < D) val.w = p[3];
                }
            }
            v[i] = val;
        }
    }
    __device__ __forceinline__ void put(float* __restrict__ dst) const {
        constexpr int LD = DP + 4;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int idx = threadIdx.x + i * NT;
            *reinterpret_cast<float4*>(dst + (idx / C4) * LD + (idx % C4) * 4) = v[i];
        }
    }
};
__host__ __device__ constexpr bool prefetch_tiles(int DP) { return DP <= 64; }

// s[r][c] = sum_d A[ty*4+r][d] * Bm[tx+16c][d] for two [64][DP+4] shared tiles.
template <int DP>
__device__ __forceinline__ void tile_nt(const float* __restrict__ A, const float* __restrict__ Bm,
                                        int ty, int tx, float (&s)[4][4]) {
    constexpr int LD = DP + 4;
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
        for (int c = 0; c < 4; ++c) s[r][c] = 0.f;
#pragma unroll 4
    for (int d = 0; d < DP; d += 4) {
        float4 a[4], b[4];
#pragma unroll
        for (int r = 0; r < 4; ++r) a[r] = *reinterpret_cast<const float4*>(A + (ty * 4 + r) * LD + d);
#pragma unroll
        for (int c = 0; c < 4; ++c) b[c] = *reinterpret_cast<const float4*>(Bm + (tx + 16 * c) * LD + d);
#pragma unroll
        for (int r = 0; r < 4; ++r)
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                s[r][c] = fmaf(a[r].x, b[c].x, s[r][c]);
                s[r][c] = fmaf(a[r].y, b[c].y, s[r][c]);
                s[r][c] = fmaf(a[r].z, b[c].z, s[r][c]);
                s[r][c] = fmaf(a[r].w, b[c].w, s[r][c]);
            }
    }
}

// acc[r][c] += sum_k Ps[ty*4+r][k] * Vs[k][tx+16c]   (P row-major [64][PLD], V [64][DP+4])
template <int DP>
__device__ __forceinline__ void tile_pv(const float* __restrict__ Ps, const float* __restrict__ Vs,
                                        int ty, int tx, float (&acc)[4][DP / 16]) {
    constexpr int LD = DP + 4;
#pragma unroll 2
    for (int k = 0; k < BN; k += 4) {
        float4 p[4];
#pragma unroll
        for (int r = 0; r < 4; ++r) p[r] = *reinterpret_cast<const float4*>(Ps + (ty * 4 + r) * PLD + k);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
            float vv[DP / 16];
#pragma unroll
            for (int c = 0; c < DP / 16; ++c) vv[c] = Vs[(k + kk) * LD + tx + 16 * c];
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                const float pr = kk == 0 ? p[r].x : kk == 1 ? p[r].y : kk == 2 ? p[r].z : p[r].w;
#pragma unroll
                for (int c = 0; c < DP / 16; ++c) acc[r][c] = fmaf(pr, vv[c], acc[r][c]);
            }
        }
    }
}

// acc[r][c] += sum_q Ps[q][ty*4+r] * Xs[q][tx+16c]   (transposed use of a [64][PLD] tile)
template <int DP>
__device__ __forceinline__ void tile_tn(const float* __restrict__ Ps, const float* __restrict__ Xs,
                                        int ty, int tx, float (&acc)[4][DP / 16]) {
    constexpr int LD = DP + 4;
#pragma unroll 4
    for (int qi = 0; qi < BM; ++qi) {
        const float4 p = *reinterpret_cast<const float4*>(Ps + qi * PLD + ty * 4);
        float xv[DP / 16];
#pragma unroll
        for (int c = 0; c < DP / 16; ++c) xv[c] = Xs[qi * LD + tx + 16 * c];
#pragma unroll
        for (int c = 0; c < DP / 16; ++c) {
            acc[0][c] = fmaf(p.x, xv[c], acc[0][c]);
            acc[1][c] = fmaf(p.y, xv[c], acc[1][c]);
            acc[2][c] = fmaf(p.z, xv[c], acc[2][c]);
            acc[3][c] = fmaf(p.w, xv[c], acc[3][c]);
        }
    }
}

__device__ __forceinline__ float half_warp_max(float x) {
#pragma unroll
    for (int o = 8; o >= 1; o >>= 1) x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, o));
    return x;
}
__device__ __forceinline__ float half_warp_sum(float x) {
#pragma unroll
    for (int o = 8; o >= 1; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
    return x;
}

// ---------------------------------------------------------------------------
// Forward: one CTA per (batch*head, 64-row query tile).  Heavy (late) query
// tiles are scheduled first so that the causal triangle balances.
// ---------------------------------------------------------------------------
template <int DP>
__global__ void __launch_bounds__(NT) attn_fwd_f32_kernel(const F32Params p) {
    extern __shared__ __align__(16) float smem[];
    constexpr int LD = DP + 4;
    float* Qs = smem;
    float* Ks = Qs + BM * LD;
    float* Vs = Ks + BN * LD;
    float* Ps = Vs + BN * LD;

    const int nq = (p.T + BM - 1) / BM;
    const int qt = nq - 1 - (int)blockIdx.x;
    const int bh = blockIdx.y;
    const int b = bh / p.H, h = bh % p.H;
    const int ty = threadIdx.x / 16, tx = threadIdx.x % 16;
    const int q0 = qt * BM;

    const float* qb = p.q + b * p.sq.b + h * p.sq.h;
    const float* kb = p.k + b * p.sk.b + h * p.sk.h;
    const float* vb = p.v + b * p.sv.b + h * p.sv.h;

    load_tile<DP>(Qs, qb, q0, p.T, p.D, p.sq.t, p.vec);

    float m[4], l[4], acc[4][DP / 16];
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        m[r] = -INFINITY; l[r] = 0.f;
#pragma unroll
        for (int c = 0; c < DP / 16; ++c) acc[r][c] = 0.f;
    }
    const float sl2 = p.scale * LOG2E;
    const int last = p.causal ? qt : (p.T + BN - 1) / BN - 1;

    TileRegs<prefetch_tiles(DP) ? DP : 16> kr, vr;     // unused (and tiny) when the tiles are loaded in place
    if constexpr (prefetch_tiles(DP)) {
        kr.fetch(kb, 0, p.T, p.D, p.sk.t, p.vec);
        vr.fetch(vb, 0, p.T, p.D, p.sv.t, p.vec);
    }
    for (int j = 0; j <= last; ++j) {
        const int k0 = j * BN;
        __syncthreads();                       // previous tile fully consumed (and Q visible)
        if constexpr (prefetch_tiles(DP)) {
            kr.put(Ks); vr.put(Vs);
            if (j < last) {                    // the next tile travels while this one is multiplied
                kr.fetch(kb, k0 + BN, p.T, p.D, p.sk.t, p.vec);
                vr.fetch(vb, k0 + BN, p.T, p.D, p.sv.t, p.vec);
            }
        } else {
            load_tile<DP>(Ks, kb, k0, p.T, p.D, p.sk.t, p.vec);
            load_tile<DP>(Vs, vb, k0, p.T, p.D, p.sv.t, p.vec);
        }
        __syncthreads();

        float s[4][4];
        tile_nt<DP>(Qs, Ks, ty, tx, s);
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int row = q0 + ty * 4 + r;
            float mx = -INFINITY;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int col = k0 + tx + 16 * c;
                const bool masked = (col >= p.T) || (p.causal && col > row);
                s[r][c] = masked ? -INFINITY : s[r][c] * sl2;
                mx = fmaxf(mx, s[r][c]);
            }
            mx = half_warp_max(mx);
            const float m_new = fmaxf(m[r], mx);
            const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
            const float alpha = exp2f(m[r] - m_use);
            float rs = 0.f;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const float e = exp2f(s[r][c] - m_use);
                rs += e;
                Ps[(ty * 4 + r) * PLD + tx + 16 * c] = e;
            }
            rs = half_warp_sum(rs);
            l[r] = l[r] * alpha + rs;
            m[r] = m_new;
#pragma unroll
            for (int c = 0; c < DP / 16; ++c) acc[r][c] *= alpha;
        }
        __syncthreads();
        tile_pv<DP>(Ps, Vs, ty, tx, acc);
    }

    float* ob = p.out_o + b * p.so.b + h * p.so.h;
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        const int row = q0 + ty * 4 + r;
        if (row >= p.T) continue;
        const float inv = 1.f / l[r];
#pragma unroll
        for (int c = 0; c < DP / 16; ++c) {
            const int col = tx + 16 * c;
            if (col < p.D) ob[(long long)row * p.so.t + col] = acc[r][c] * inv;
        }
        if (tx == 0) p.lse_out[((long long)bh) * p.T + row] = (m[r] + log2f(l[r])) * LN2;
    }
}

// ---------------------------------------------------------------------------
// delta[bh][t] = sum_d dO[t][d] * O[t][d]  (= rowsum(dP * P)); one warp per row.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) attn_delta_f32_kernel(const F32Params p) {
    const long long row = (long long)blockIdx.x * 8 + threadIdx.x / 32;
    const int lane = threadIdx.x % 32;
    const long long rows = (long long)p.B * p.H * p.T;
    if (row >= rows) return;
    const int t = (int)(row % p.T);
    const int bh = (int)(row / p.T);
    const int b = bh / p.H, h = bh % p.H;
    const float* o = p.o + b * p.so.b + h * p.so.h + (long long)t * p.so.t;
    const float* g = p.d_o + b * p.sdo.b + h * p.sdo.h + (long long)t * p.sdo.t;
    float acc = 0.f;
    for (int d = lane; d < p.D; d += 32) acc = fmaf(o[d], g[d], acc);
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
    if (lane == 0) p.delta[row] = acc;
}

// Recomputes, for the 64 x 64 tile (q0, k0): P (0 where masked or out of range)
// and dS = scale * P * (dP - delta).  Patch layout as tile_nt.
template <int DP>
__device__ __forceinline__ void recompute_p_ds(const F32Params& p, const float* Qs, const float* Ks,
                                               const float* dOs, const float* Vs, const float* lse_s,
                                               const float* delta_s, int q0, int k0, int ty, int tx,
                                               float (&pp)[4][4], float (&ds)[4][4]) {
    float dp[4][4];
    tile_nt<DP>(Qs, Ks, ty, tx, pp);
    tile_nt<DP>(dOs, Vs, ty, tx, dp);
    const float sl2 = p.scale * LOG2E;
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        const int row = q0 + ty * 4 + r;
        const float l2 = lse_s[ty * 4 + r] * LOG2E;
        const float dl = delta_s[ty * 4 + r];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const int col = k0 + tx + 16 * c;
            const bool masked = (row >= p.T) || (col >= p.T) || (p.causal && col > row);
            const float e = masked ? 0.f : exp2f(pp[r][c] * sl2 - l2);
            pp[r][c] = e;
            ds[r][c] = e * (dp[r][c] - dl) * p.scale;
        }
    }
}

// ---------------------------------------------------------------------------
// Backward, dK/dV: one CTA per (batch*head, KV tile); it visits every query tile
// at or below its diagonal and keeps dK/dV in registers, so no atomics are needed.
// ---------------------------------------------------------------------------
template <int DP>
__device__ __forceinline__ void attn_bwd_dkdv_f32_body(const F32Params& p, float* smem) {
    constexpr int LD = DP + 4;
    float* Ks = smem;
    float* Vs = Ks + BN * LD;
    float* Qs = Vs + BN * LD;
    float* dOs = Qs + BM * LD;
    float* Ps = dOs + BM * LD;
    float* dSs = Ps + BM * PLD;
    float* lse_s = dSs + BM * PLD;
    float* delta_s = lse_s + BM;

    const int kt = blockIdx.x;                 // low KV tiles carry the most work: scheduled first
    const int bh = blockIdx.y;
    const int b = bh / p.H, h = bh % p.H;
    const int ty = threadIdx.x / 16, tx = threadIdx.x % 16;
    const int k0 = kt * BN;
    const int nq = (p.T + BM - 1) / BM;

    load_tile<DP>(Ks, p.k + b * p.sk.b + h * p.sk.h, k0, p.T, p.D, p.sk.t, p.vec);
    load_tile<DP>(Vs, p.v + b * p.sv.b + h * p.sv.h, k0, p.T, p.D, p.sv.t, p.vec);

    float dk[4][DP / 16], dv[4][DP / 16];
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
        for (int c = 0; c < DP / 16; ++c) { dk[r][c] = 0.f; dv[r][c] = 0.f; }

    const float* qb = p.q + b * p.sq.b + h * p.sq.h;
    const float* gb = p.d_o + b * p.sdo.b + h * p.sdo.h;
    const int i_first = p.causal ? kt : 0;
    TileRegs<prefetch_tiles(DP) ? DP : 16> qr, gr;
    if constexpr (prefetch_tiles(DP)) {
        if (i_first < nq) {
            qr.fetch(qb, i_first * BM, p.T, p.D, p.sq.t, p.vec);
            gr.fetch(gb, i_first * BM, p.T, p.D, p.sdo.t, p.vec);
        }
    }
    for (int i = i_first; i < nq; ++i) {
        const int q0 = i * BM;
        __syncthreads();
        if constexpr (prefetch_tiles(DP)) {
            qr.put(Qs); gr.put(dOs);
            if (i + 1 < nq) {
                qr.fetch(qb, q0 + BM, p.T, p.D, p.sq.t, p.vec);
                gr.fetch(gb, q0 + BM, p.T, p.D, p.sdo.t, p.vec);
            }
        } else {
            load_tile<DP>(Qs, qb, q0, p.T, p.D, p.sq.t, p.vec);
            load_tile<DP>(dOs, gb, q0, p.T, p.D, p.sdo.t, p.vec);
        }
        if (threadIdx.x < BM) {
            const int row = q0 + threadIdx.x;
            lse_s[threadIdx.x] = row < p.T ? p.lse[(long long)bh * p.T + row] : 0.f;
            delta_s[threadIdx.x] = row < p.T ? p.delta[(long long)bh * p.T + row] : 0.f;
        }
        __syncthreads();
        float pp[4][4], ds[4][4];
        recompute_p_ds<DP>(p, Qs, Ks, dOs, Vs, lse_s, delta_s, q0, k0, ty, tx, pp, ds);
#pragma unroll
        for (int r = 0; r < 4; ++r)
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                Ps[(ty * 4 + r) * PLD + tx + 16 * c] = pp[r][c];
                dSs[(ty * 4 + r) * PLD + tx + 16 * c] = ds[r][c];
            }
        __syncthreads();
        tile_tn<DP>(Ps, dOs, ty, tx, dv);      // dV += P^T dO
        tile_tn<DP>(dSs, Qs, ty, tx, dk);      // dK += dS^T Q
    }

    float* dkb = p.dk + b * p.sdk.b + h * p.sdk.h;
    float* dvb = p.dv + b * p.sdv.b + h * p.sdv.h;
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        const int row = k0 + ty * 4 + r;
        if (row >= p.T) continue;
#pragma unroll
        for (int c = 0; c < DP / 16; ++c) {
            const int col = tx + 16 * c;
            if (col < p.D) {
                dkb[(long long)row * p.sdk.t + col] = dk[r][c];
                dvb[(long long)row * p.sdv.t + col] = dv[r][c];
            }
        }
    }
}

// ---------------------------------------------------------------------------
// Backward, dQ: one CTA per (batch*head, query tile), looping over the KV tiles
// at or left of its diagonal.
// ---------------------------------------------------------------------------
template <int DP>
__device__ __forceinline__ void attn_bwd_dq_f32_body(const F32Params& p, float* smem) {
    constexpr int LD = DP + 4;
    float* Ks = smem;
    float* Vs = Ks + BN * LD;
    float* Qs = Vs + BN * LD;
    float* dOs = Qs + BM * LD;
    float* dSs = dOs + BM * LD;
    float* lse_s = dSs + BM * PLD;
    float* delta_s = lse_s + BM;

    const int nq = (p.T + BM - 1) / BM;
    const int qt = nq - 1 - (int)blockIdx.x;
    const int bh = blockIdx.y;
    const int b = bh / p.H, h = bh % p.H;
    const int ty = threadIdx.x / 16, tx = threadIdx.x % 16;
    const int q0 = qt * BM;

    load_tile<DP>(Qs, p.q + b * p.sq.b + h * p.sq.h, q0, p.T, p.D, p.sq.t, p.vec);
    load_tile<DP>(dOs, p.d_o + b * p.sdo.b + h * p.sdo.h, q0, p.T, p.D, p.sdo.t, p.vec);
    if (threadIdx.x < BM) {
        const int row = q0 + threadIdx.x;
        lse_s[threadIdx.x] = row < p.T ? p.lse[(long long)bh * p.T + row] : 0.f;
        delta_s[threadIdx.x] = row < p.T ? p.delta[(long long)bh * p.T + row] : 0.f;
    }

    float dq[4][DP / 16];
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
        for (int c = 0; c < DP / 16; ++c) dq[r][c] = 0.f;

    const float* kb = p.k + b * p.sk.b + h * p.sk.h;
    const float* vb = p.v + b * p.sv.b + h * p.sv.h;
    const int last = p.causal ? qt : (p.T + BN - 1) / BN - 1;
    TileRegs<prefetch_tiles(DP) ? DP : 16> kr, vr;
    if constexpr (prefetch_tiles(DP)) {
        kr.fetch(kb, 0, p.T, p.D, p.sk.t, p.vec);
        vr.fetch(vb, 0, p.T, p.D, p.sv.t, p.vec);
    }
    for (int j = 0; j <= last; ++j) {
        const int k0 = j * BN;
        __syncthreads();
        if constexpr (prefetch_tiles(DP)) {
            kr.put(Ks); vr.put(Vs);
            if (j < last) {
                kr.fetch(kb, k0 + BN, p.T, p.D, p.sk.t, p.vec);
                vr.fetch(vb, k0 + BN, p.T, p.D, p.sv.t, p.vec);
            }
        } else {
            load_tile<DP>(Ks, kb, k0, p.T, p.D, p.sk.t, p.vec);
            load_tile<DP>(Vs, vb, k0, p.T, p.D, p.sv.t, p.vec);
        }
        __syncthreads();
        float pp[4][4], ds[4][4];
        recompute_p_ds<DP>(p, Qs, Ks, dOs, Vs, lse_s, delta_s, q0, k0, ty, tx, pp, ds);
#pragma unroll
        for (int r = 0; r < 4; ++r)
#pragma unroll
            for (int c = 0; c < 4; ++c) dSs[(ty * 4 + r) * PLD + tx + 16 * c] = ds[r][c];
        __syncthreads();
        tile_pv<DP>(dSs, Ks, ty, tx, dq);      // dQ += dS K
    }

    float* dqb = p.dq + b * p.sdq.b + h * p.sdq.h;
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        const int row = q0 + ty * 4 + r;
        if (row >= p.T) continue;
#pragma unroll
        for (int c = 0; c < DP / 16; ++c) {
            const int col = tx + 16 * c;
            if (col < p.D) dqb[(long long)row * p.sdq.t + col] = dq[r][c];
        }
    }
}

// dK/dV and dQ in one launch: the two walks share nothing but their inputs, so blockIdx.z picks the role
// (z = 0: one KV tile per block, z = 1: one query tile per block) and both sets of blocks run side by side;
// at the model's shapes each alone fills well under one block per SM.
template <int DP>
__global__ void __launch_bounds__(NT) attn_bwd_f32_kernel(const F32Params p) {
    extern __shared__ __align__(16) float smem[];
    if (blockIdx.z == 0) attn_bwd_dkdv_f32_body<DP>(p, smem);
    else attn_bwd_dq_f32_body<DP>(p, smem);
}

Strides3 s3(const int64_t* s) { return Strides3{(long long)s[0], (long long)s[1], (long long)s[2]}; }

bool rows_vec_ok(const void* ptr, const int64_t* s) {
    return (((uintptr_t)ptr) & 15u) == 0 && (s[0] & 3) == 0 && (s[1] & 3) == 0 && (s[2] & 3) == 0;
}

template <typename K>
int set_smem(deers_ctx* ctx, K kernel, size_t bytes) {
    DEERS_CUDA_TRY(ctx, cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
    return DEERS_OK;
}

template <int DP>
int fwd_impl(deers_ctx* ctx, const F32Params& p) {
    const size_t smem = (size_t)(3 * BM * (DP + 4) + BM * PLD) * sizeof(float);
    int rc = set_smem(ctx, attn_fwd_f32_kernel<DP>, smem);
    if (rc) return rc;
    dim3 grid((p.T + BM - 1) / BM, p.B * p.H);
    {
        KernelTimerScope ts(ctx, DEERS_K_FWD);
        attn_fwd_f32_kernel<DP><<<grid, NT, smem, ctx->stream>>>(p);
    }
    ctx->launches += 1;
    DEERS_CUDA_TRY(ctx, cudaGetLastError());
    return DEERS_OK;
}

template <int DP>
int bwd_impl(deers_ctx* ctx, const F32Params& p) {
    const long long rows = (long long)p.B * p.H * p.T;
    {
        KernelTimerScope ts(ctx, DEERS_K_BWD_PREP);
        attn_delta_f32_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, ctx->stream>>>(p);
    }
    DEERS_CUDA_TRY(ctx, cudaGetLastError());
    const size_t smem_kv = (size_t)(4 * BM * (DP + 4) + 2 * BM * PLD + 2 * BM) * sizeof(float);
    const size_t smem_q = (size_t)(4 * BM * (DP + 4) + BM * PLD + 2 * BM) * sizeof(float);
    const size_t smem = smem_kv > smem_q ? smem_kv : smem_q;
    int rc = set_smem(ctx, attn_bwd_f32_kernel<DP>, smem);
    if (rc) return rc;
    dim3 grid((p.T + BM - 1) / BM, p.B * p.H, 2);
    {
        KernelTimerScope ts(ctx, DEERS_K_BWD_MAIN);
        attn_bwd_f32_kernel<DP><<<grid, NT, smem, ctx->stream>>>(p);
    }
    DEERS_CUDA_TRY(ctx, cudaGetLastError());
    ctx->launches += 2;
    return DEERS_OK;
}

F32Params base_params(const deers_attn_desc* d) {
    F32Params p;
    memset(&p, 0, sizeof(p));
    p.B = d->B; p.H = d->H; p.T = d->T; p.D = d->D;
    p.causal = d->causal; p.scale = d->scale;
    p.sq = s3(d->q_strides); p.sk = s3(d->k_strides); p.sv = s3(d->v_strides);
    p.so = s3(d->o_strides); p.sdo = s3(d->do_strides);
    p.sdq = s3(d->dq_strides); p.sdk = s3(d->dk_strides); p.sdv = s3(d->dv_strides);
    return p;
}

}  // namespace

int launch_attn_fwd_f32(deers_ctx* ctx, const deers_attn_desc* d, const float* q, const float* k,
                        const float* v, float* o, float* lse) {
    F32Params p = base_params(d);
    p.q = q; p.k = k; p.v = v; p.out_o = o; p.lse_out = lse;
    p.vec = (d->D % 4 == 0) && rows_vec_ok(q, d->q_strides) && rows_vec_ok(k, d->k_strides) &&
            rows_vec_ok(v, d->v_strides);
    if (d->D <= 32) return fwd_impl<32>(ctx, p);
    if (d->D <= 64) return fwd_impl<64>(ctx, p);
    return fwd_impl<128>(ctx, p);
}

int launch_attn_bwd_f32(deers_ctx* ctx, const deers_attn_desc* d, const float* q, const float* k,
                        const float* v, const float* o, const float* lse, const float* d_o, float* dq,
                        float* dk, float* dv, float* delta) {
    F32Params p = base_params(d);
    p.q = q; p.k = k; p.v = v; p.o = o; p.lse = lse; p.d_o = d_o;
    p.dq = dq; p.dk = dk; p.dv = dv; p.delta = delta;
    p.vec = (d->D % 4 == 0) && rows_vec_ok(q, d->q_strides) && rows_vec_ok(k, d->k_strides) &&
            rows_vec_ok(v, d->v_strides) && rows_vec_ok(d_o, d->do_strides);
    if (d->D <= 32) return bwd_impl<32>(ctx, p);
    if (d->D <= 64) return bwd_impl<64>(ctx, p);
    return bwd_impl<128>(ctx, p);
}
