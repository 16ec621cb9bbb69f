// f16 GEMM with f32 accumulation on tcgen05 / TMEM / TMA, for the projections around the attention op.
//
// The reference runs `Linear::forward` (src/nn.rs:184-190: y = x.matmul(weight), weight stored
// [in_features, out_features]) and its backward (src/ops.rs:1089-1101: dx = dy @ W^T, dW = x^T @ dy)
// through cublasGemmStridedBatchedEx (src/storage/cuda.rs:1147-1177).  One kernel covers the three
// products through the two operand layouts of the tensor core:
//     C[M,N] = A * B,  A stored [M,K] (K contiguous: "K-major") or [K,M] (M contiguous: "MN-major"),
//                      B stored [N,K] (K-major)                or [K,N] (MN-major)
//     forward  y  = x   * W      : A = x  [M,K]  K-major,  B = W  [K,N] MN-major
//     dgrad    dx = dy  * W^T    : A = dy [M,N]  K-major,  B = W  [K,N] read as [N'=K, K'=N]: K-major
//     wgrad    dW = x^T * dy     : A = x  [m,K]  read as [K'=m, M'=K]: MN-major,  B = dy [m,N] MN-major
// Persistent: one CTA per SM walks 128 x 256 output tiles (consecutive CTAs share a B column block, which
// L2 then serves).  Warp 0 streams 64-deep K blocks of A (16 KB) and B (32 KB) through a 4-stage ring (TMA,
// 128-byte swizzle, out-of-range rows / columns read as zero), warp 1 issues four 128x256x16 tcgen05.mma
// per K block into one of two 256-column TMEM accumulators, warps 2-5 move a finished accumulator to
// registers 64 columns at a time, convert to f16 and store rows transposed within 8-lane groups
// (contiguous 128-byte segments), then release the accumulator.
// N = 256 because the instruction issue interval on this part is 166 cycles for 128x256x16 against 104 for
// 128x128x16 (128 / 64 would be the nominal rates): 20 % less time per flop.
#include "sm100_ptx.cuh"
#include "tma_host.cuh"

namespace {
using namespace sm100;

constexpr int GM = 128, GN = 256, GK = 64;      // output tile and K block
constexpr uint32_t G_A_BYTES = GM * GK * 2;     // 16 KB per stage
constexpr uint32_t G_B_BYTES = GN * GK * 2;     // 32 KB per stage
constexpr int G_STAGES = 4;
constexpr uint32_t G_SMEM = G_STAGES * (G_A_BYTES + G_B_BYTES) + 256;
// Shared-memory layouts of a stage (what the TMA boxes below write, 128-byte swizzle):
//   K-major operand of R rows (R = 128 for A, 256 for B): one block of R rows x 64 K-columns (R * 128 bytes)
//   MN-major operand of C columns (C = 128 / 256): C / 64 blocks of 64 K-rows x 64 columns (8 KB each)
constexpr uint32_t G_MN_BLOCK = GK * 128;       // 8 KB

enum GBar { G_FULL = 0, G_EMPTY = 4, G_ACC_FULL = 8, G_ACC_EMPTY = 10, G_COUNT = 12 };

struct GemmParams {
    __half* c;
    long long ldc;
    int M, N, K;
    unsigned int* err;
};

template <int A_MN, int B_MN>
__global__ void __launch_bounds__(192, 1)
gemm_f16_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b, const GemmParams p) {
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t* sA = smem;
    uint8_t* sB = smem + G_STAGES * G_A_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + G_STAGES * (G_A_BYTES + G_B_BYTES));
    uint32_t* tmem_base_s = reinterpret_cast<uint32_t*>(bars + G_COUNT);
    volatile uint32_t* abort_s = tmem_base_s + 1;
    uint32_t* skip_s = tmem_base_s + 2;

    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const int tiles_m = (p.M + GM - 1) / GM, tiles_n = (p.N + GN - 1) / GN;
    const int n_tiles = tiles_m * tiles_n;
    const int kblocks = (p.K + GK - 1) / GK;

    if (threadIdx.x == 0) {
        *abort_s = 0;
        uint32_t skip = (*(volatile unsigned int*)p.err != 0) ? 1u : 0u;
        if ((smem_u32(smem) & 1023u) != 0) {
            atomicCAS(p.err, 0u, DEERS_KERR_GEMM | 0x20);
            skip = 1;
        }
        *skip_s = skip;
        for (int s = 0; s < G_STAGES; ++s) { mbar_init(&bars[G_FULL + s], 1); mbar_init(&bars[G_EMPTY + s], 1); }
        for (int s = 0; s < 2; ++s) { mbar_init(&bars[G_ACC_FULL + s], 1); mbar_init(&bars[G_ACC_EMPTY + s], 128); }
        fence_barrier_init();
        tma_prefetch_desc(&tmap_a); tma_prefetch_desc(&tmap_b);
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

    if (warp == 0) {
        // ------------------------------ TMA producer ------------------------------
        if (lane == 0) {
            uint32_t g = 0;                                     // K blocks loaded so far (ring position)
            bool ok = true;
            for (int t = blockIdx.x; ok && t < n_tiles; t += gridDim.x) {
                const int tm = t % tiles_m, tn = t / tiles_m;
                for (int kb = 0; kb < kblocks; ++kb, ++g) {
                    const uint32_t s = g % G_STAGES;
                    if (!mbar_wait(ws, &bars[G_EMPTY + s], ((g / G_STAGES) & 1u) ^ 1u, DEERS_KERR_GEMM | 1)) { ok = false; break; }
                    mbar_arrive_expect_tx(&bars[G_FULL + s], G_A_BYTES + G_B_BYTES);
                    uint8_t* a_dst = sA + s * G_A_BYTES;
                    uint8_t* b_dst = sB + s * G_B_BYTES;
                    // K-major: box {64 of K, rows}; MN-major: boxes {64 of M / N, 64 rows of K}
                    if (A_MN) {
#pragma unroll
                        for (int blk = 0; blk < GM / 64; ++blk)
                            tma_load_4d(a_dst + blk * G_MN_BLOCK, &tmap_a, &bars[G_FULL + s], tm * GM + blk * 64, kb * GK, 0, 0);
                    } else {
                        tma_load_4d(a_dst, &tmap_a, &bars[G_FULL + s], kb * GK, tm * GM, 0, 0);
                    }
                    if (B_MN) {
#pragma unroll
                        for (int blk = 0; blk < GN / 64; ++blk)
                            tma_load_4d(b_dst + blk * G_MN_BLOCK, &tmap_b, &bars[G_FULL + s], tn * GN + blk * 64, kb * GK, 0, 0);
                    } else {
                        tma_load_4d(b_dst, &tmap_b, &bars[G_FULL + s], kb * GK, tn * GN, 0, 0);
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer ------------------------------
        if (lane == 0) {
            constexpr uint32_t IDESC = idesc_f16(GM, GN, A_MN, B_MN);
            constexpr uint64_t A_STEP = G_A_BYTES >> 4, B_STEP = G_B_BYTES >> 4;
            const uint64_t a0 = A_MN ? desc_mnmajor(smem_u32(sA), 0, G_MN_BLOCK) : desc_kmajor(smem_u32(sA), 0, 0);
            const uint64_t b0 = B_MN ? desc_mnmajor(smem_u32(sB), 0, G_MN_BLOCK) : desc_kmajor(smem_u32(sB), 0, 0);
            uint32_t g = 0;
            int n = 0;
            bool ok = true;
            for (int t = blockIdx.x; ok && t < n_tiles; t += gridDim.x, ++n) {
                const uint32_t buf = (uint32_t)n & 1u;
                if (!mbar_wait(ws, &bars[G_ACC_EMPTY + buf], (((uint32_t)n >> 1) & 1u) ^ 1u, DEERS_KERR_GEMM | 2)) break;
                for (int kb = 0; kb < kblocks; ++kb, ++g) {
                    const uint32_t s = g % G_STAGES;
                    if (!mbar_wait(ws, &bars[G_FULL + s], (g / G_STAGES) & 1u, DEERS_KERR_GEMM | 3)) { ok = false; break; }
                    tc_fence_after_sync();
                    const uint64_t a = a0 + (uint64_t)s * A_STEP, b = b0 + (uint64_t)s * B_STEP;
#pragma unroll
                    for (int ks = 0; ks < GK / 16; ++ks)                   // ks < 4: a K-major step stays inside its block
                        umma_ss(tmem + buf * 256u, a + (A_MN ? mnmajor_step(ks) : kmajor_step(ks, 0)),
                                b + (B_MN ? mnmajor_step(ks) : kmajor_step(ks, 0)), IDESC, (kb > 0 || ks > 0));
                    umma_commit(&bars[G_EMPTY + s]);
                }
                if (ok) umma_commit(&bars[G_ACC_FULL + buf]);
            }
        }
    } else {
        // ------------------------------ epilogue ------------------------------
        const int lane_base = (warp & 3) * 32;
        const uint32_t t_lane = (uint32_t)lane_base << 16;
        int n = 0;
        for (int t = blockIdx.x; t < n_tiles; t += gridDim.x, ++n) {
            const int tm = t % tiles_m, tn = t / tiles_m;
            const uint32_t buf = (uint32_t)n & 1u;
            if (!__all_sync(0xffffffffu, mbar_wait(ws, &bars[G_ACC_FULL + buf], ((uint32_t)n >> 1) & 1u, DEERS_KERR_GEMM | 4))) break;
            tc_fence_after_sync();
            const int row0 = tm * GM + lane_base + (lane & ~7);
#pragma unroll 1
            for (int part = 0; part < GN / 64; ++part) {        // 64 columns at a time
                uint32_t r[64];
                uint4 pc[8];
                tmem_ld_x32(tmem + buf * 256u + t_lane + part * 64, *reinterpret_cast<uint32_t(*)[32]>(&r[0]));
                tmem_ld_x32(tmem + buf * 256u + t_lane + part * 64 + 32, *reinterpret_cast<uint32_t(*)[32]>(&r[32]));
                tmem_wait_ld();
                if (part == GN / 64 - 1) {                      // accumulator is in registers: the next tile may use it
                    tc_fence_before_sync();
                    mbar_arrive(&bars[G_ACC_EMPTY + buf]);
                }
#pragma unroll
                for (int q8 = 0; q8 < 8; ++q8) pc[q8] = pack8_f16(r + q8 * 8, 1.0f);
                transpose_pieces<8>(pc, (uint32_t)lane);
                const int col = tn * GN + part * 64 + (lane & 7) * 8;
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    const int row = row0 + c;
                    if (row < p.M && col < p.N) *reinterpret_cast<uint4*>(p.c + (long long)row * p.ldc + col) = pc[c];
                }
            }
        }
    }
    __syncwarp();
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem, 512);
}

// 2-D tensor map over a row-major f16 matrix [rows][inner] with leading dimension ld (elements).
int make_tmap_matrix(deers_ctx* ctx, CUtensorMap* out, const void* base, long long rows, long long inner, long long ld,
                     int box_rows) {
    const int64_t strides[4] = {rows * ld, rows * ld, ld, 1};
    return make_tmap_bhtd_f16(ctx, out, base, 1, 1, (int)rows, (int)inner, strides, box_rows);
}

template <int A_MN, int B_MN>
int gemm_launch(deers_ctx* ctx, const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p) {
    DEERS_CUDA_TRY(ctx, cudaFuncSetAttribute(gemm_f16_kernel<A_MN, B_MN>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)G_SMEM));
    const long long tiles = (long long)((p.M + GM - 1) / GM) * ((p.N + GN - 1) / GN);
    const unsigned grid = (unsigned)(tiles < ctx->sm_count ? tiles : ctx->sm_count);
    {
        KernelTimerScope ts(ctx, DEERS_K_GEMM);
        gemm_f16_kernel<A_MN, B_MN><<<grid, 192, G_SMEM, ctx->stream>>>(ta, tb, p);
    }
    ctx->launches += 1;
    DEERS_CUDA_TRY(ctx, cudaGetLastError());
    return DEERS_OK;
}

}  // namespace

extern "C" int deers_b200_gemm_f16(deers_ctx* ctx, int32_t M, int32_t N, int32_t K, const void* a, int64_t lda, int32_t a_mn_major,
                                   const void* b, int64_t ldb, int32_t b_mn_major, void* c, int64_t ldc) {
    if (!ctx || !a || !b || !c) return DEERS_ERR_NULL;
    if (M < 1 || N < 1 || K < 1) return DEERS_ERR_SHAPE;
    // 16-byte rows for TMA and for the epilogue's 16-byte stores
    if ((N % 8) || (lda % 8) || (ldb % 8) || (ldc % 8) || lda < (a_mn_major ? M : K) || ldb < (b_mn_major ? N : K) || ldc < N)
        return DEERS_ERR_LAYOUT;
    if (((uintptr_t)a | (uintptr_t)b | (uintptr_t)c) & 15u) return DEERS_ERR_LAYOUT;
    DEERS_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    CUtensorMap ta, tb;
    int rc;
    // K-major A: [M rows][K inner], box {64, 128}; MN-major A: [K rows][M inner], box {64, 64}.  Same for B with
    // N (K-major box {64, 256}).
    if ((rc = a_mn_major ? make_tmap_matrix(ctx, &ta, a, K, M, lda, GK) : make_tmap_matrix(ctx, &ta, a, M, K, lda, GM))) return rc;
    if ((rc = b_mn_major ? make_tmap_matrix(ctx, &tb, b, K, N, ldb, GK) : make_tmap_matrix(ctx, &tb, b, N, K, ldb, GN))) return rc;
    GemmParams p;
    p.c = (__half*)c; p.ldc = ldc; p.M = M; p.N = N; p.K = K; p.err = ctx->dev_err;
    if (a_mn_major) return b_mn_major ? gemm_launch<1, 1>(ctx, ta, tb, p) : gemm_launch<1, 0>(ctx, ta, tb, p);
    return b_mn_major ? gemm_launch<0, 1>(ctx, ta, tb, p) : gemm_launch<0, 0>(ctx, ta, tb, p);
}
