// f32-accurate GEMM on the tensor core for the head of the f32 model: C[M,N] = A * B with every f32 operand
// carried as TWO f16 values,
//     x * s  =  hi + lo * 2^-11,     hi = f16(x * s),   lo = f16((x * s - hi) * 2^11)      (s: a power of two),
// and the product expanded into three `tcgen05.mma kind::f16` products with f32 accumulation in TMEM:
//     main += A_hi * B_hi        corr += A_hi * B_lo + A_lo * B_hi        C = (main + corr * 2^-11) * out_scale
// (the lo * lo term is below 2^-22 of the product).  hi and lo have 11 significant bits each, so an operand is
// carried to 2^-22 and a 192- or 50257-term sum comes out closer to the exact value than a sequential f32 sum
// does; the reference computes these products in full f32 (cuBLAS with CUBLAS_COMPUTE_32F,
// src/storage/cuda.rs:1098-1128), not in TF32, and this keeps that accuracy at tensor-core speed.
// It serves `lm_head` of src/models/gpt.rs:351 and the two products of its backward (src/ops.rs:1089-1101):
// 80 % of the FLOPs of a training step of the reference's GPT.
//
// Persistent kernel, 128 x 128 output tiles, 64-deep K blocks, 3-stage TMA ring of four operand tiles (A_hi,
// A_lo, B_hi, B_lo: 64 KB per stage, 128-byte swizzle, out-of-range rows / columns read as zero), twelve MMAs
// per K block, two pairs of TMEM accumulators so the epilogue of a tile overlaps the next tile's products.
// Either storage order of A and of B (the operand orders of forward, dgrad and wgrad), as in gemm_f16_sm100.cu.
// Long reductions with few output tiles (the head's input gradient: K = vocabulary) are split along K over the
// work units; every part writes its f32 partial tile, a second kernel adds the parts in index order.
#include "sm100_ptx.cuh"
#include "tma_host.cuh"

namespace {
using namespace sm100;

constexpr int XM = 128, XN = 128, XK = 64;
constexpr uint32_t X_TILE = 128 * XK * 2;          // 16 KB: one operand tile of a stage
constexpr uint32_t X_STAGE = 4 * X_TILE;           // A_hi | A_lo | B_hi | B_lo
constexpr int X_STAGES = 3;
constexpr uint32_t X_SMEM = X_STAGES * X_STAGE + 256;
constexpr uint32_t X_MN_BLOCK = XK * 128;          // 8 KB: 64 K-rows x 64 columns of an MN-major operand
constexpr float X_LO = 1.0f / 2048.0f;

// warp 0 TMA, warp 1 MMA, then two epilogue warpgroups that each take half of a tile's columns: with one, the
// head's forward product waits on its epilogue (206 MB of logits through 4 warps per SM), not on the tensor pipe
constexpr int X_EPI_WG = 2;
constexpr int X_THREADS = 64 + 128 * X_EPI_WG;

enum XBar { X_FULL = 0, X_EMPTY = 3, X_ACC_FULL = 6, X_ACC_EMPTY = 8, X_COUNT = 10 };

struct X3Params {
    float* c;                   // parts == 1: the output; parts > 1: partial tiles [part][M][N] (dense)
    long long ldc;
    int M, N, K;
    int parts, k_chunk;         // K range of part p: [p * k_chunk, min(K, (p + 1) * k_chunk)); k_chunk % 64 == 0
    float out_scale;
    int vec;                    // rows of c start on 16-byte boundaries: 16-byte stores
    unsigned int* err;
};

template <int A_MN, int B_MN>
__global__ void __launch_bounds__(X_THREADS, 1)
gemm_f16x3_kernel(const __grid_constant__ CUtensorMap tm_ah, const __grid_constant__ CUtensorMap tm_al,
                  const __grid_constant__ CUtensorMap tm_bh, const __grid_constant__ CUtensorMap tm_bl, const X3Params p) {
    extern __shared__ __align__(1024) uint8_t smem[];
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + X_STAGES * X_STAGE);
    uint32_t* tmem_base_s = reinterpret_cast<uint32_t*>(bars + X_COUNT);
    volatile uint32_t* abort_s = tmem_base_s + 1;
    uint32_t* skip_s = tmem_base_s + 2;

    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const int tiles_m = (p.M + XM - 1) / XM, tiles_n = (p.N + XN - 1) / XN;
    const int n_units = tiles_m * tiles_n * p.parts;

    if (threadIdx.x == 0) {
        *abort_s = 0;
        uint32_t skip = (*(volatile unsigned int*)p.err != 0) ? 1u : 0u;
        if ((smem_u32(smem) & 1023u) != 0) {
            atomicCAS(p.err, 0u, DEERS_KERR_GEMM | 0x21);
            skip = 1;
        }
        *skip_s = skip;
        for (int s = 0; s < X_STAGES; ++s) { mbar_init(&bars[X_FULL + s], 1); mbar_init(&bars[X_EMPTY + s], 1); }
        for (int s = 0; s < 2; ++s) { mbar_init(&bars[X_ACC_FULL + s], 1); mbar_init(&bars[X_ACC_EMPTY + s], 128 * X_EPI_WG); }
        fence_barrier_init();
        tma_prefetch_desc(&tm_ah); tma_prefetch_desc(&tm_al); tma_prefetch_desc(&tm_bh); tma_prefetch_desc(&tm_bl);
    }
    __syncthreads();
    if (*skip_s) return;
    if (warp == 1) {
        tmem_alloc(tmem_base_s, 512);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = *tmem_base_s;
    WaitState ws{abort_s, p.err};

    // unit u -> (tile, part); consecutive units are the parts of one tile, so they run at the same time on
    // neighbouring CTAs and share the B columns in L2
    auto unit = [&](int u, int& tm, int& tn, int& kb0, int& kb1) {
        const int part = u % p.parts, tile = u / p.parts;
        tm = tile % tiles_m; tn = tile / tiles_m;
        const int k0 = part * p.k_chunk;
        const int k1 = min(p.K, k0 + p.k_chunk);
        kb0 = k0 / XK; kb1 = (k1 + XK - 1) / XK;
    };

    if (warp == 0) {
        // ------------------------------ TMA producer ------------------------------
        if (lane == 0) {
            uint32_t g = 0;
            bool ok = true;
            for (int u = blockIdx.x; ok && u < n_units; u += gridDim.x) {
                int tm, tn, kb0, kb1;
                unit(u, tm, tn, kb0, kb1);
                for (int kb = kb0; kb < kb1; ++kb, ++g) {
                    const uint32_t s = g % X_STAGES;
                    if (!mbar_wait(ws, &bars[X_EMPTY + s], ((g / X_STAGES) & 1u) ^ 1u, DEERS_KERR_GEMM | 0x11)) { ok = false; break; }
                    mbar_arrive_expect_tx(&bars[X_FULL + s], X_STAGE);
                    uint8_t* st = smem + s * X_STAGE;
#pragma unroll
                    for (int half = 0; half < 2; ++half) {           // hi, lo
                        const CUtensorMap* ta = half ? &tm_al : &tm_ah;
                        const CUtensorMap* tb = half ? &tm_bl : &tm_bh;
                        uint8_t* a_dst = st + half * X_TILE;
                        uint8_t* b_dst = st + (2 + half) * X_TILE;
                        if (A_MN) {
#pragma unroll
                            for (int blk = 0; blk < XM / 64; ++blk)
                                tma_load_4d(a_dst + blk * X_MN_BLOCK, ta, &bars[X_FULL + s], tm * XM + blk * 64, kb * XK, 0, 0);
                        } else {
                            tma_load_4d(a_dst, ta, &bars[X_FULL + s], kb * XK, tm * XM, 0, 0);
                        }
                        if (B_MN) {
#pragma unroll
                            for (int blk = 0; blk < XN / 64; ++blk)
                                tma_load_4d(b_dst + blk * X_MN_BLOCK, tb, &bars[X_FULL + s], tn * XN + blk * 64, kb * XK, 0, 0);
                        } else {
                            tma_load_4d(b_dst, tb, &bars[X_FULL + s], kb * XK, tn * XN, 0, 0);
                        }
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer ------------------------------
        if (lane == 0) {
            constexpr uint32_t IDESC = idesc_f16(XM, XN, A_MN, B_MN);
            constexpr uint64_t TILE_STEP = X_TILE >> 4, STAGE_STEP = X_STAGE >> 4;
            const uint64_t a0 = A_MN ? desc_mnmajor(smem_u32(smem), 0, X_MN_BLOCK) : desc_kmajor(smem_u32(smem), 0, 0);
            const uint64_t b0 = B_MN ? desc_mnmajor(smem_u32(smem + 2 * X_TILE), 0, X_MN_BLOCK)
                                     : desc_kmajor(smem_u32(smem + 2 * X_TILE), 0, 0);
            uint32_t g = 0;
            int n = 0;
            bool ok = true;
            for (int u = blockIdx.x; ok && u < n_units; u += gridDim.x, ++n) {
                int tm, tn, kb0, kb1;
                unit(u, tm, tn, kb0, kb1);
                const uint32_t buf = (uint32_t)n & 1u;
                const uint32_t t_main = tmem + buf * 256u, t_corr = tmem + buf * 256u + 128u;
                if (!mbar_wait(ws, &bars[X_ACC_EMPTY + buf], (((uint32_t)n >> 1) & 1u) ^ 1u, DEERS_KERR_GEMM | 0x12)) break;
                for (int kb = kb0; kb < kb1; ++kb, ++g) {
                    const uint32_t s = g % X_STAGES;
                    if (!mbar_wait(ws, &bars[X_FULL + s], (g / X_STAGES) & 1u, DEERS_KERR_GEMM | 0x13)) { ok = false; break; }
                    tc_fence_after_sync();
                    const uint64_t ah = a0 + (uint64_t)s * STAGE_STEP, al = ah + TILE_STEP;
                    const uint64_t bh = b0 + (uint64_t)s * STAGE_STEP, bl = bh + TILE_STEP;
#pragma unroll
                    for (int ks = 0; ks < XK / 16; ++ks) {
                        const uint64_t sa = A_MN ? mnmajor_step(ks) : kmajor_step(ks, 0);
                        const uint64_t sb = B_MN ? mnmajor_step(ks) : kmajor_step(ks, 0);
                        const uint32_t first = (kb > kb0 || ks > 0);
                        umma_ss(t_main, ah + sa, bh + sb, IDESC, first);
                        umma_ss(t_corr, ah + sa, bl + sb, IDESC, first);
                        umma_ss(t_corr, al + sa, bh + sb, IDESC, 1u);
                    }
                    umma_commit(&bars[X_EMPTY + s]);
                }
                if (ok) umma_commit(&bars[X_ACC_FULL + buf]);
            }
        }
    } else {
        // ------------------------------ epilogue ------------------------------
        const int lane_base = (warp & 3) * 32;
        const uint32_t t_lane = (uint32_t)lane_base << 16;
        const int ewg = (warp - 2) >> 2;                         // which share of the columns
        constexpr int CHUNKS = XN / 32 / X_EPI_WG;
        int n = 0;
        for (int u = blockIdx.x; u < n_units; u += gridDim.x, ++n) {
            int tm, tn, kb0, kb1;
            unit(u, tm, tn, kb0, kb1);
            const int part = u % p.parts;
            const uint32_t buf = (uint32_t)n & 1u;
            if (!__all_sync(0xffffffffu, mbar_wait(ws, &bars[X_ACC_FULL + buf], ((uint32_t)n >> 1) & 1u, DEERS_KERR_GEMM | 0x14))) break;
            tc_fence_after_sync();
            float* cbase = p.c + (p.parts > 1 ? (long long)part * p.M * p.ldc : 0);
            const int row0 = tm * XM + lane_base + (lane & ~7);
#pragma unroll 1
            for (int chunk = ewg * CHUNKS; chunk < (ewg + 1) * CHUNKS; ++chunk) {      // 32 columns at a time
                uint32_t rm[32], rc[32];
                tmem_ld_x32(tmem + buf * 256u + t_lane + chunk * 32, rm);
                tmem_ld_x32(tmem + buf * 256u + 128u + t_lane + chunk * 32, rc);
                tmem_wait_ld();
                if (chunk == (ewg + 1) * CHUNKS - 1) {           // this warpgroup's share of both accumulators is in registers
                    tc_fence_before_sync();
                    mbar_arrive(&bars[X_ACC_EMPTY + buf]);
                }
                uint4 pc[8];
#pragma unroll
                for (int q = 0; q < 8; ++q) {
                    float o[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e)
                        o[e] = fmaf(__uint_as_float(rc[q * 4 + e]), X_LO, __uint_as_float(rm[q * 4 + e])) * p.out_scale;
                    pc[q] = make_uint4(__float_as_uint(o[0]), __float_as_uint(o[1]), __float_as_uint(o[2]), __float_as_uint(o[3]));
                }
                // 16-byte pieces transposed within 8-lane groups: a store instruction writes 128 contiguous bytes per row
                transpose_pieces<8>(pc, (uint32_t)lane);
                const int col = tn * XN + chunk * 32 + (lane & 7) * 4;
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    const int row = row0 + c;
                    if (row >= p.M || col >= p.N) continue;
                    float* dst = cbase + (long long)row * p.ldc + col;
                    if (p.vec && col + 4 <= p.N) {
                        *reinterpret_cast<uint4*>(dst) = pc[c];
                    } else {
                        const uint32_t v[4] = {pc[c].x, pc[c].y, pc[c].z, pc[c].w};
                        for (int e = 0; e < 4 && col + e < p.N; ++e) dst[e] = __uint_as_float(v[e]);
                    }
                }
            }
        }
    }
    __syncwarp();
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem, 512);
}

// c[m][n] = sum over parts (in index order) of partial[part][m][n]
__global__ void __launch_bounds__(256) x3_reduce_kernel(const float* __restrict__ partial, int parts, long long MN,
                                                        int N, float* __restrict__ c, long long ldc) {
    for (long long i = (long long)blockIdx.x * 256 + threadIdx.x; i < MN; i += (long long)gridDim.x * 256) {
        float acc = partial[i];
        for (int pz = 1; pz < parts; ++pz) acc += partial[(long long)pz * MN + i];
        c[(i / N) * ldc + (i % N)] = acc;
    }
}

// hi = f16(x * s), lo = f16((x * s - hi) * 2^11); 8 elements per thread (16-byte loads and stores when aligned)
__global__ void __launch_bounds__(256) x3_split_kernel(const float* __restrict__ src, long long ld_src, long long rows, int cols,
                                                       float scale, __half* __restrict__ hi, __half* __restrict__ lo,
                                                       long long ld_dst, int vec) {
    const int per_row = (cols + 7) / 8;
    const long long total = rows * per_row;
    for (long long t = (long long)blockIdx.x * 256 + threadIdx.x; t < total; t += (long long)gridDim.x * 256) {
        const long long r = t / per_row;
        const int c0 = (int)(t % per_row) * 8;
        const float* s = src + r * ld_src + c0;
        float x[8];
        if (vec && c0 + 8 <= cols) {
            const float4 a = *reinterpret_cast<const float4*>(s), b = *reinterpret_cast<const float4*>(s + 4);
            x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w; x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
        } else {
#pragma unroll
            for (int e = 0; e < 8; ++e) x[e] = (c0 + e < cols) ? s[e] : 0.f;
        }
        __half h[8], l[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const float v = x[e] * scale;
            h[e] = __float2half_rn(v);
            l[e] = __float2half_rn((v - __half2float(h[e])) * 2048.0f);
        }
        __half* dh = hi + r * ld_dst + c0;
        __half* dl = lo + r * ld_dst + c0;
        if (vec && c0 + 8 <= cols) {
            *reinterpret_cast<uint4*>(dh) = *reinterpret_cast<const uint4*>(h);
            *reinterpret_cast<uint4*>(dl) = *reinterpret_cast<const uint4*>(l);
        } else {
            for (int e = 0; e < 8 && c0 + e < cols; ++e) { dh[e] = h[e]; dl[e] = l[e]; }
        }
    }
}

// Tensor map over a row-major f16 matrix [rows][inner] with leading dimension ld (a multiple of 8 elements), as
// a 4-D map {inner, rows, 1, 1} with box {64, box_rows, 1, 1}, 128-byte swizzle, out-of-range elements read as zero.
int make_tmap_x3(deers_ctx* ctx, CUtensorMap* out, const void* base, long long rows, long long inner, long long ld, int box_rows) {
    if (!ctx->encode_tiled) {
        snprintf(ctx->last_error, sizeof(ctx->last_error), "cuTensorMapEncodeTiled not available");
        return DEERS_ERR_CUDA;
    }
    const cuuint64_t dims[4] = {(cuuint64_t)inner, (cuuint64_t)rows, 1, 1};
    const cuuint64_t row_bytes = (cuuint64_t)ld * 2;
    const cuuint64_t gstr[3] = {row_bytes, row_bytes * (cuuint64_t)rows, row_bytes * (cuuint64_t)rows};
    const cuuint32_t box[4] = {64u, (cuuint32_t)box_rows, 1u, 1u};
    const cuuint32_t estr[4] = {1u, 1u, 1u, 1u};
    const CUresult r = ((PFN_encodeTiled)ctx->encode_tiled)(
        out, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, const_cast<void*>(base), dims, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        snprintf(ctx->last_error, sizeof(ctx->last_error), "cuTensorMapEncodeTiled failed with CUresult %d (rows %lld, inner %lld, ld %lld)",
                 (int)r, rows, inner, ld);
        return DEERS_ERR_LAYOUT;
    }
    return DEERS_OK;
}

struct X3Plan { int parts, k_chunk; };

X3Plan x3_plan(int M, int N, int K, int sm_count) {
    const long long tiles = (long long)((M + XM - 1) / XM) * ((N + XN - 1) / XN);
    X3Plan pl{1, (K + XK - 1) / XK * XK};
    if (tiles < sm_count) {
        int parts = (int)(sm_count / tiles);                          // all (tile, part) units in one wave of CTAs
        const int kblocks = (K + XK - 1) / XK;
        const int max_parts = kblocks / 8 > 1 ? kblocks / 8 : 1;      // at least eight K blocks per part
        if (parts > max_parts) parts = max_parts;
        if (parts > 64) parts = 64;
        const int chunk_blocks = (kblocks + parts - 1) / parts;
        pl.k_chunk = chunk_blocks * XK;
        pl.parts = (kblocks + chunk_blocks - 1) / chunk_blocks;
    }
    return pl;
}

template <int A_MN, int B_MN>
int x3_launch(deers_ctx* ctx, const CUtensorMap* t, const X3Params& p, unsigned grid) {
    DEERS_CUDA_TRY(ctx, cudaFuncSetAttribute(gemm_f16x3_kernel<A_MN, B_MN>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)X_SMEM));
    {
        KernelTimerScope ts(ctx, DEERS_K_GEMM_X3);
        gemm_f16x3_kernel<A_MN, B_MN><<<grid, X_THREADS, X_SMEM, ctx->stream>>>(t[0], t[1], t[2], t[3], p);
    }
    ctx->launches += 1;
    DEERS_CUDA_TRY(ctx, cudaGetLastError());
    return DEERS_OK;
}

}  // namespace

size_t gemm_f16x3_workspace_bytes(const deers_ctx* ctx, int M, int N, int K) {
    const X3Plan pl = x3_plan(M, N, K, ctx ? ctx->sm_count : 148);
    return pl.parts > 1 ? (size_t)pl.parts * M * N * sizeof(float) : 0;
}

int launch_split_f16x3(deers_ctx* ctx, long long rows, int cols, const float* src, long long ld_src, float scale,
                       void* hi, void* lo, long long ld_dst) {
    if (rows == 0 || cols == 0) return DEERS_OK;
    const int vec = (((uintptr_t)src | (uintptr_t)hi | (uintptr_t)lo) & 15u) == 0 && ld_src % 4 == 0 && ld_dst % 8 == 0;
    const long long total = rows * ((cols + 7) / 8);
    long long want = (total + 255) / 256;
    const long long cap = 16LL * ctx->sm_count;
    {
        KernelTimerScope ts(ctx, DEERS_K_GEMM_X3);
        x3_split_kernel<<<(unsigned)(want < cap ? want : cap), 256, 0, ctx->stream>>>(src, ld_src, rows, cols, scale, (__half*)hi,
                                                                                      (__half*)lo, ld_dst, vec);
    }
    ctx->launches += 1;
    DEERS_CUDA_TRY(ctx, cudaGetLastError());
    return DEERS_OK;
}

int launch_gemm_f16x3(deers_ctx* ctx, int M, int N, int K, const void* a_hi, const void* a_lo, long long lda, int a_mn,
                      const void* b_hi, const void* b_lo, long long ldb, int b_mn, float* c, long long ldc, float out_scale,
                      void* workspace, size_t ws_bytes) {
    if (M == 0 || N == 0) return DEERS_OK;
    CUtensorMap t[4];
    int rc;
    // K-major operand: [rows = M or N][inner = K], box {64, 128}; MN-major: [rows = K][inner = M or N], box {64, 64}
    const void* ap[2] = {a_hi, a_lo};
    const void* bp[2] = {b_hi, b_lo};
    for (int h = 0; h < 2; ++h) {
        if ((rc = a_mn ? make_tmap_x3(ctx, &t[h], ap[h], K, M, lda, XK) : make_tmap_x3(ctx, &t[h], ap[h], M, K, lda, XM))) return rc;
        if ((rc = b_mn ? make_tmap_x3(ctx, &t[2 + h], bp[h], K, N, ldb, XK) : make_tmap_x3(ctx, &t[2 + h], bp[h], N, K, ldb, XN))) return rc;
    }
    const X3Plan pl = x3_plan(M, N, K, ctx->sm_count);
    X3Params p;
    p.M = M; p.N = N; p.K = K; p.parts = pl.parts; p.k_chunk = pl.k_chunk; p.err = ctx->dev_err;
    if (pl.parts > 1) {
        if (!workspace || ws_bytes < (size_t)pl.parts * M * N * sizeof(float) || ((uintptr_t)workspace & 15u)) return DEERS_ERR_WORKSPACE;
        p.c = (float*)workspace; p.ldc = N; p.out_scale = out_scale;
    } else {
        p.c = c; p.ldc = ldc; p.out_scale = out_scale;
    }
    p.vec = (p.ldc % 4 == 0) && (((uintptr_t)p.c & 15u) == 0);
    const long long units = (long long)((M + XM - 1) / XM) * ((N + XN - 1) / XN) * pl.parts;
    const unsigned grid = (unsigned)(units < ctx->sm_count ? units : ctx->sm_count);
    if (a_mn) rc = b_mn ? x3_launch<1, 1>(ctx, t, p, grid) : x3_launch<1, 0>(ctx, t, p, grid);
    else rc = b_mn ? x3_launch<0, 1>(ctx, t, p, grid) : x3_launch<0, 0>(ctx, t, p, grid);
    if (rc) return rc;
    if (pl.parts > 1) {
        const long long MN = (long long)M * N;
        long long want = (MN + 255) / 256;
        const long long cap = 8LL * ctx->sm_count;
        {
            KernelTimerScope ts(ctx, DEERS_K_GEMM_X3);
            x3_reduce_kernel<<<(unsigned)(want < cap ? want : cap), 256, 0, ctx->stream>>>((const float*)workspace, pl.parts, MN, N, c, ldc);
        }
        ctx->launches += 1;
        DEERS_CUDA_TRY(ctx, cudaGetLastError());
    }
    return DEERS_OK;
}

extern "C" int deers_b200_split_f16x3(deers_ctx* ctx, int64_t rows, int32_t cols, const float* src, int64_t ld_src, float scale,
                                      void* hi, void* lo, int64_t ld_dst) {
    if (!ctx || !src || !hi || !lo) return DEERS_ERR_NULL;
    if (rows < 0 || cols < 0) return DEERS_ERR_SHAPE;
    if (ld_src < cols || ld_dst < cols || ((uintptr_t)src & 3u) || (((uintptr_t)hi | (uintptr_t)lo) & 1u)) return DEERS_ERR_LAYOUT;
    if (!(scale > 0.f)) return DEERS_ERR_SHAPE;
    DEERS_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    return launch_split_f16x3(ctx, rows, cols, src, ld_src, scale, hi, lo, ld_dst);
}

extern "C" size_t deers_b200_gemm_f16x3_workspace_bytes(deers_ctx* ctx, int32_t M, int32_t N, int32_t K) {
    if (!ctx || M < 0 || N < 0 || K < 0) return 0;
    return gemm_f16x3_workspace_bytes(ctx, M, N, K);
}

extern "C" int deers_b200_gemm_f16x3(deers_ctx* ctx, int32_t M, int32_t N, int32_t K, const void* a_hi, const void* a_lo,
                                     int64_t lda, int32_t a_mn_major, const void* b_hi, const void* b_lo, int64_t ldb,
                                     int32_t b_mn_major, float* c, int64_t ldc, float out_scale, void* workspace,
                                     size_t workspace_bytes) {
    if (!ctx || !a_hi || !a_lo || !b_hi || !b_lo || !c) return DEERS_ERR_NULL;
    if (M < 1 || N < 1 || K < 1) return DEERS_ERR_SHAPE;
    // 16-byte rows for TMA (f16 operands) and for the epilogue's 16-byte stores (f32 output)
    if ((lda % 8) || (ldb % 8) || (ldc % 4) || lda < (a_mn_major ? M : K) || ldb < (b_mn_major ? N : K) || ldc < N)
        return DEERS_ERR_LAYOUT;
    if (((uintptr_t)a_hi | (uintptr_t)a_lo | (uintptr_t)b_hi | (uintptr_t)b_lo | (uintptr_t)c) & 15u) return DEERS_ERR_LAYOUT;
    DEERS_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    return launch_gemm_f16x3(ctx, M, N, K, a_hi, a_lo, lda, a_mn_major, b_hi, b_lo, ldb, b_mn_major, c, ldc, out_scale, workspace,
                             workspace_bytes);
}
