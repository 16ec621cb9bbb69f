// f32 GEMM on the FFMA pipe (no TF32) for the projections of the f32 model: Linear::forward
// (src/nn.rs:184-190, weight stored [in, out]) and the two products of the matmul backward
// (src/ops.rs:1089-1101).  The reference sends these to cublasGemmStridedBatchedEx with
// CUBLAS_COMPUTE_32F (src/storage/cuda.rs:1098-1128), i.e. full f32 arithmetic; so does this kernel.
//
// One kernel template covers C[M,N] = A * B for either storage order of A and of B, arbitrary leading
// dimensions and alignments (16-byte loads when base and leading dimension allow, guarded scalar loads
// otherwise, zero fill beyond the edges), with an epilogue applied while the tile is still in registers:
//   NONE      C = acc
//   ADD       C = R + acc                 the residual connections of the block (gpt.rs:237-239)
//   RELU_SQ   r = max(acc, 0); C = r*r; AUX = r     relu and y*y of the MLP (gpt.rs:194-196)
//   MUL_AUX2  t = acc * AUX; C = t + t    the backward of y*y and relu in one (ops.rs:210-214, 560-568)
// 256 * KS threads own a BM x BN tile (register patches of TM x TN, operands double-buffered in shared
// memory, 16 * KS deep; with KS = 2 the two halves of the block each multiply 16 of a stage's 32 k and the
// patches are added through shared memory at the end: twice the warps per tile for the small shapes whose
// grids do not fill the SMs and that otherwise wait on shared-memory latency with two warps per scheduler).  Shapes with few output tiles and a long reduction (weight gradients, the head's
// input gradient) are split along K across gridDim.z: every part writes its partial tile to the
// workspace, the part that arrives last (one atomic counter per tile, no waiting) adds the parts in
// index order and runs the epilogue, so results do not depend on arrival order.
#include "common.cuh"

namespace {

constexpr int GK = 16;                                  // depth of one shared-memory stage

struct GemmArgs {
    const float* a; const float* b; float* c;
    const float* r;          // ADD: residual [M][ldr]
    float* aux;              // RELU_SQ: written; MUL_AUX2: read; [M][ldc]
    long long lda, ldb, ldc, ldr;
    int M, N, K;
    int a_mn, b_mn;          // 0: K contiguous, 1: M / N contiguous
    int a_vec, b_vec, c_vec; // 16-byte accesses allowed
    int epi;
    int k_chunk;             // K elements per gridDim.z part (multiple of GK)
    float* partial;          // split-K: [tile][part][BM*BN]
    unsigned int* counters;  // split-K: one per tile, zero on entry, left zero
};

__device__ __forceinline__ float4 ld4(const float* p, int valid, bool vec) {
    if (vec && valid >= 4) return *reinterpret_cast<const float4*>(p);
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (valid > 0) v.x = p[0];
    if (valid > 1) v.y = p[1];
    if (valid > 2) v.z = p[2];
    if (valid > 3) v.w = p[3];
    return v;
}

// Loads one BROWS x GKS operand tile into registers.  contiguous-K storage: rows = tile rows (m or n),
// GKS / 4 threads cover the k of a row; contiguous-MN storage: rows = k, float4 along m / n.
template <int BR, int KS>
struct TileLoader {
    static constexpr int GKS = GK * KS;
    static constexpr int NT = 256 * KS;
    static constexpr int NV = BR * GKS / 4 / NT;         // float4 per thread
    float4 v[NV];
    __device__ __forceinline__ void load(const float* base, long long ld, int mn_major, bool vec, int r0, int rmax,
                                         int k0, int kmax) {
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int idx = threadIdx.x + i * NT;
            if (!mn_major) {
                const int row = idx / (GKS / 4), kq = (idx % (GKS / 4)) * 4;
                const int gr = r0 + row, gk = k0 + kq;
                const int valid = gr < rmax ? kmax - gk : 0;
                v[i] = ld4(base + (long long)gr * ld + gk, valid, vec);
            } else {
                const int k = idx / (BR / 4), rq = (idx % (BR / 4)) * 4;
                const int gk = k0 + k, gr = r0 + rq;
                const int valid = gk < kmax ? rmax - gr : 0;
                v[i] = ld4(base + (long long)gk * ld + gr, valid, vec);
            }
        }
    }
    __device__ __forceinline__ void store(float (*s)[BR + 4], int mn_major) const {
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int idx = threadIdx.x + i * NT;
            if (!mn_major) {
                const int row = idx / (GKS / 4), kq = (idx % (GKS / 4)) * 4;
                s[kq + 0][row] = v[i].x; s[kq + 1][row] = v[i].y; s[kq + 2][row] = v[i].z; s[kq + 3][row] = v[i].w;
            } else {
                const int k = idx / (BR / 4), rq = (idx % (BR / 4)) * 4;
                *reinterpret_cast<float4*>(&s[k][rq]) = v[i];
            }
        }
    }
};

template <int BM, int BN, int TM, int TN, int KS>
__global__ void __launch_bounds__(256 * KS) gemm_f32_kernel(const GemmArgs g) {
    static_assert((BM / TM) * (BN / TN) == 256, "256 threads per tile and k half");
    constexpr int GKS = GK * KS;
    __shared__ __align__(16) float As[2][GKS][BM + 4];
    __shared__ __align__(16) float Bs[2][GKS][BN + 4];
    __shared__ int s_last;
    const int tid = threadIdx.x % 256, kh = threadIdx.x / 256;      // position in the tile, k half
    const int tx = tid % (BN / TN), ty = tid / (BN / TN);
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int kbeg = blockIdx.z * g.k_chunk;
    const int kend = min(g.K, kbeg + g.k_chunk);

    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

    TileLoader<BM, KS> la;
    TileLoader<BN, KS> lb;
    const int nk = (kend - kbeg + GKS - 1) / GKS;
    if (nk > 0) {
        la.load(g.a, g.lda, g.a_mn, g.a_vec, m0, g.M, kbeg, kend);
        lb.load(g.b, g.ldb, g.b_mn, g.b_vec, n0, g.N, kbeg, kend);
        la.store(As[0], g.a_mn);
        lb.store(Bs[0], g.b_mn);
    }
    __syncthreads();
    for (int kt = 0; kt < nk; ++kt) {
        const int cur = kt & 1;
        if (kt + 1 < nk) {
            la.load(g.a, g.lda, g.a_mn, g.a_vec, m0, g.M, kbeg + (kt + 1) * GKS, kend);
            lb.load(g.b, g.ldb, g.b_mn, g.b_vec, n0, g.N, kbeg + (kt + 1) * GKS, kend);
        }
#pragma unroll
        for (int k = kh * GK; k < (kh + 1) * GK; ++k) {
            float af[TM], bf[TN];
            // a thread's rows / columns come in groups of four, the groups BM/2 (BN/2) apart, so that the
            // lanes of a warp read consecutive 16-byte pieces
#pragma unroll
            for (int h = 0; h < TM / 4; ++h) {
                const float4 t = *reinterpret_cast<const float4*>(&As[cur][k][h * (BM / (TM / 4)) + ty * 4]);
                af[h * 4 + 0] = t.x; af[h * 4 + 1] = t.y; af[h * 4 + 2] = t.z; af[h * 4 + 3] = t.w;
            }
#pragma unroll
            for (int h = 0; h < TN / 4; ++h) {
                const float4 t = *reinterpret_cast<const float4*>(&Bs[cur][k][h * (BN / (TN / 4)) + tx * 4]);
                bf[h * 4 + 0] = t.x; bf[h * 4 + 1] = t.y; bf[h * 4 + 2] = t.z; bf[h * 4 + 3] = t.w;
            }
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(af[i], bf[j], acc[i][j]);
        }
        if (kt + 1 < nk) {
            la.store(As[cur ^ 1], g.a_mn);
            lb.store(Bs[cur ^ 1], g.b_mn);
        }
        __syncthreads();
    }

    // ---- the k halves of the block meet: the upper half hands its patch over through shared memory (the
    // operand buffers are free after the loop's last barrier) and only stays for the barriers below
    const bool owner = kh == 0;
    if (KS > 1) {
        static_assert(KS == 1 || sizeof(As) >= 256 * TM * TN * sizeof(float), "patch exchange fits in the A buffers");
        float4* red = reinterpret_cast<float4*>(&As[0][0][0]);
        if (!owner) {
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN / 4; ++j)
                    red[(i * (TN / 4) + j) * 256 + tid] =
                        make_float4(acc[i][j * 4], acc[i][j * 4 + 1], acc[i][j * 4 + 2], acc[i][j * 4 + 3]);
        }
        __syncthreads();
        if (owner) {
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN / 4; ++j) {
                    const float4 t = red[(i * (TN / 4) + j) * 256 + tid];
                    acc[i][j * 4] += t.x; acc[i][j * 4 + 1] += t.y; acc[i][j * 4 + 2] += t.z; acc[i][j * 4 + 3] += t.w;
                }
        }
    }

    // ---- split-K: park the partial tile; the last part to arrive adds all parts in index order
    if (gridDim.z > 1) {
        const int tile = blockIdx.y * gridDim.x + blockIdx.x;
        float4* mine = reinterpret_cast<float4*>(g.partial) +
                       ((size_t)tile * gridDim.z + blockIdx.z) * (BM * BN / 4);
        if (owner) {
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN / 4; ++j)
                    mine[(i * (TN / 4) + j) * 256 + tid] =
                        make_float4(acc[i][j * 4], acc[i][j * 4 + 1], acc[i][j * 4 + 2], acc[i][j * 4 + 3]);
        }
        __threadfence();
        __syncthreads();
        if (threadIdx.x == 0) {
            const unsigned int prev = atomicAdd(&g.counters[tile], 1u);
            s_last = prev == gridDim.z - 1;
            if (s_last) g.counters[tile] = 0;                     // ready for the next launch
        }
        __syncthreads();
        if (!s_last || !owner) return;
        __threadfence();
#pragma unroll
        for (int i = 0; i < TM; ++i)
#pragma unroll
            for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;
        const float4* parts = reinterpret_cast<const float4*>(g.partial) + (size_t)tile * gridDim.z * (BM * BN / 4);
        for (unsigned int z = 0; z < gridDim.z; ++z) {
            const float4* p = parts + (size_t)z * (BM * BN / 4);
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN / 4; ++j) {
                    const float4 t = __ldcg(&p[(i * (TN / 4) + j) * 256 + tid]);
                    acc[i][j * 4] += t.x; acc[i][j * 4 + 1] += t.y; acc[i][j * 4 + 2] += t.z; acc[i][j * 4 + 3] += t.w;
                }
        }
    }

    // ---- epilogue
    if (!owner) return;
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int m = m0 + (i / 4) * (BM / (TM / 4)) + ty * 4 + (i % 4);
        if (m >= g.M) continue;
#pragma unroll
        for (int h = 0; h < TN / 4; ++h) {
            const int n = n0 + h * (BN / (TN / 4)) + tx * 4;
            if (n >= g.N) continue;
            float o[4] = {acc[i][h * 4], acc[i][h * 4 + 1], acc[i][h * 4 + 2], acc[i][h * 4 + 3]};
            float x[4] = {0.f, 0.f, 0.f, 0.f};
            const int valid = g.N - n;
            float* cp = g.c + (long long)m * g.ldc + n;
            if (g.epi == DEERS_EPI_ADD) {
                const float4 t = ld4(g.r + (long long)m * g.ldr + n, valid, g.c_vec);
                o[0] = t.x + o[0]; o[1] = t.y + o[1]; o[2] = t.z + o[2]; o[3] = t.w + o[3];
            } else if (g.epi == DEERS_EPI_RELU_SQ) {
#pragma unroll
                for (int e = 0; e < 4; ++e) { x[e] = fmaxf(o[e], 0.f); o[e] = x[e] * x[e]; }
            } else if (g.epi == DEERS_EPI_MUL_AUX2) {
                const float4 t = ld4(g.aux + (long long)m * g.ldc + n, valid, g.c_vec);
                o[0] *= t.x; o[1] *= t.y; o[2] *= t.z; o[3] *= t.w;
#pragma unroll
                for (int e = 0; e < 4; ++e) o[e] = o[e] + o[e];
            }
            if (g.c_vec && valid >= 4) {
                *reinterpret_cast<float4*>(cp) = make_float4(o[0], o[1], o[2], o[3]);
                if (g.epi == DEERS_EPI_RELU_SQ)
                    *reinterpret_cast<float4*>(g.aux + (long long)m * g.ldc + n) = make_float4(x[0], x[1], x[2], x[3]);
            } else {
                for (int e = 0; e < 4 && e < valid; ++e) {
                    cp[e] = o[e];
                    if (g.epi == DEERS_EPI_RELU_SQ) g.aux[(long long)m * g.ldc + n + e] = x[e];
                }
            }
        }
    }
}

struct GemmPlan {
    int cfg;        // 0: 128x128, 1: 64x128, 2: 64x64
    int bm, bn;
    int tiles_m, tiles_n, parts, k_chunk;
};

GemmPlan plan_gemm(int M, int N, int K, int sm_count) {
    static const int kBM[3] = {128, 64, 64}, kBN[3] = {128, 128, 64}, kKS[3] = {1, 1, 2};
    GemmPlan p{};
    int pick = 2;
    for (int c = 0; c < 3; ++c) {
        const long long tiles = (long long)((M + kBM[c] - 1) / kBM[c]) * ((N + kBN[c] - 1) / kBN[c]);
        // the padding a tile shape adds to M (an [M=192] gradient wastes a quarter of a 128-row tile)
        const double waste = (double)((M + kBM[c] - 1) / kBM[c] * kBM[c]) * ((N + kBN[c] - 1) / kBN[c] * kBN[c]) /
                             ((double)M * N);
        if (tiles >= 2LL * sm_count && waste <= 1.15) { pick = c; break; }
    }
    p.cfg = pick; p.bm = kBM[pick]; p.bn = kBN[pick];
    p.tiles_m = (M + p.bm - 1) / p.bm;
    p.tiles_n = (N + p.bn - 1) / p.bn;
    const long long tiles = (long long)p.tiles_m * p.tiles_n;
    int parts = 1;
    if (tiles < 2LL * sm_count) {
        parts = (int)((3LL * sm_count + tiles - 1) / tiles);
        const int max_parts = K / (8 * GK) > 1 ? K / (8 * GK) : 1;      // at least 8 stages per part
        if (parts > max_parts) parts = max_parts;
        if (parts > 64) parts = 64;
    }
    const int gks = GK * kKS[pick];
    int chunk = ((K + parts - 1) / parts + gks - 1) / gks * gks;
    if (chunk < gks) chunk = gks;
    p.k_chunk = chunk;
    p.parts = (K + chunk - 1) / chunk;
    if (p.parts < 1) p.parts = 1;
    return p;
}

size_t plan_workspace(const GemmPlan& p) {
    if (p.parts <= 1) return 0;
    const size_t tiles = (size_t)p.tiles_m * p.tiles_n;
    return 256 + ((tiles * sizeof(unsigned int) + 255) / 256) * 256 + tiles * p.parts * p.bm * p.bn * sizeof(float);
}

}  // namespace

size_t gemm_f32_workspace_bytes(const deers_ctx* ctx, int M, int N, int K) {
    return plan_workspace(plan_gemm(M, N, K, ctx ? ctx->sm_count : 148));
}

// counters_zero: the caller guarantees that the counter words at the start of the workspace are zero (they
// are left zero by every launch); otherwise they are cleared on the stream first.
int launch_gemm_f32(deers_ctx* ctx, int M, int N, int K, const float* a, long long lda, int a_mn, const float* b,
                    long long ldb, int b_mn, float* c, long long ldc, int epi, const float* r, long long ldr, float* aux,
                    void* workspace, size_t ws_bytes, bool counters_zero) {
    if (M == 0 || N == 0) return DEERS_OK;
    const GemmPlan p = plan_gemm(M, N, K, ctx->sm_count);
    GemmArgs g{};
    g.a = a; g.b = b; g.c = c; g.r = r; g.aux = aux;
    g.lda = lda; g.ldb = ldb; g.ldc = ldc; g.ldr = ldr;
    g.M = M; g.N = N; g.K = K; g.a_mn = a_mn; g.b_mn = b_mn; g.epi = epi;
    g.a_vec = ((uintptr_t)a & 15u) == 0 && lda % 4 == 0;
    g.b_vec = ((uintptr_t)b & 15u) == 0 && ldb % 4 == 0;
    g.c_vec = ((uintptr_t)c & 15u) == 0 && ldc % 4 == 0 && (!r || (((uintptr_t)r & 15u) == 0 && ldr % 4 == 0)) &&
              (!aux || ((uintptr_t)aux & 15u) == 0);
    g.k_chunk = p.k_chunk;
    if (p.parts > 1) {
        if (!workspace || ws_bytes < plan_workspace(p) || ((uintptr_t)workspace & 255u) != 0) return DEERS_ERR_WORKSPACE;
        const size_t tiles = (size_t)p.tiles_m * p.tiles_n;
        const size_t cbytes = ((tiles * sizeof(unsigned int) + 255) / 256) * 256;
        g.counters = (unsigned int*)workspace;
        g.partial = (float*)((char*)workspace + cbytes);
        if (!counters_zero) DEERS_CUDA_TRY(ctx, cudaMemsetAsync(workspace, 0, cbytes, ctx->stream));
    }
    const dim3 grid(p.tiles_n, p.tiles_m, p.parts);
    {
        KernelTimerScope ts(ctx, DEERS_K_GEMM);
        if (p.cfg == 0) gemm_f32_kernel<128, 128, 8, 8, 1><<<grid, 256, 0, ctx->stream>>>(g);
        else if (p.cfg == 1) gemm_f32_kernel<64, 128, 4, 8, 1><<<grid, 256, 0, ctx->stream>>>(g);
        else gemm_f32_kernel<64, 64, 4, 4, 2><<<grid, 512, 0, ctx->stream>>>(g);
    }
    ctx->launches += 1;
    DEERS_CUDA_TRY(ctx, cudaGetLastError());
    return DEERS_OK;
}

extern "C" size_t deers_b200_gemm_f32_workspace_bytes(deers_ctx* ctx, int32_t M, int32_t N, int32_t K) {
    if (!ctx || M < 0 || N < 0 || K < 0) return 0;
    return gemm_f32_workspace_bytes(ctx, M, N, K);
}

extern "C" int deers_b200_gemm_f32(deers_ctx* ctx, int32_t M, int32_t N, int32_t K, const float* a, int64_t lda,
                                   int32_t a_mn_major, const float* b, int64_t ldb, int32_t b_mn_major, float* c,
                                   int64_t ldc, const deers_gemm_epilogue* epilogue, void* workspace,
                                   size_t workspace_bytes) {
    if (!ctx || !a || !b || !c) return DEERS_ERR_NULL;
    if (M < 0 || N < 0 || K < 0) return DEERS_ERR_SHAPE;
    if ((((uintptr_t)a | (uintptr_t)b | (uintptr_t)c) & 3u) != 0) return DEERS_ERR_LAYOUT;
    if (lda < (a_mn_major ? M : K) || ldb < (b_mn_major ? N : K) || ldc < N) return DEERS_ERR_LAYOUT;
    int epi = DEERS_EPI_NONE;
    const float* r = nullptr;
    long long ldr = 0;
    float* aux = nullptr;
    if (epilogue) {
        epi = epilogue->kind;
        if (epi < DEERS_EPI_NONE || epi > DEERS_EPI_MUL_AUX2) return DEERS_ERR_SHAPE;
        if (epi == DEERS_EPI_ADD) {
            if (!epilogue->residual) return DEERS_ERR_NULL;
            if (epilogue->ld_residual < N || ((uintptr_t)epilogue->residual & 3u)) return DEERS_ERR_LAYOUT;
            r = epilogue->residual; ldr = epilogue->ld_residual;
        } else if (epi != DEERS_EPI_NONE) {
            if (!epilogue->aux) return DEERS_ERR_NULL;
            if ((uintptr_t)epilogue->aux & 3u) return DEERS_ERR_LAYOUT;
            aux = epilogue->aux;
        }
    }
    DEERS_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    return launch_gemm_f32(ctx, M, N, K, a, lda, a_mn_major, b, ldb, b_mn_major, c, ldc, epi, r, ldr, aux, workspace,
                           workspace_bytes, false);
}
