// Self-test of the tcgen05 operand layouts the f16 attention kernels rely on.
// One CTA multiplies a 128 x 128 (f16) A by a 128 x N B into TMEM and writes the
// f32 product out; the host compares with its own product.  The cases cover
// TMA-written K-major operands (Q K^T), thread-written K-major A with an
// MN-major B (P V), MN-major A and B (the transposed products of the backward),
// the N = 64 shapes of head_dim 64, and an A operand that threads stored into
// TMEM (P^T kept in tensor memory for dV += P^T dO).
#include "sm100_ptx.cuh"
#include "tma_host.cuh"

#include <math.h>
#include <stdlib.h>
#include <vector>

namespace {
using namespace sm100;

struct SelftestParams {
    const __half* a_global;   // used when a_manual: row-major [128][128]
    float* out;               // [128][N]
    unsigned int* err;
    int N;
    int a_mn, b_mn, a_manual;  // a_manual: 1 = threads write A into shared memory, 2 = into TMEM
};

constexpr int ST_K = 128;

__global__ void __launch_bounds__(128) umma_selftest_kernel(const __grid_constant__ CUtensorMap tmap_a,
                                                            const __grid_constant__ CUtensorMap tmap_b,
                                                            const SelftestParams p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* sA = smem;                 // 2 blocks x 16 KB
    uint8_t* sB = smem + 32768;         // up to 2 blocks x 16 KB
    __shared__ uint64_t bar_tma, bar_mma;
    __shared__ uint32_t tmem_base_s;
    __shared__ uint32_t abort_s;

    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    WaitState ws{&abort_s, p.err};
    if (threadIdx.x == 0) {
        abort_s = 0;
        mbar_init(&bar_tma, 1);
        mbar_init(&bar_mma, 1);
        fence_barrier_init();
    }
    __syncwarp();
    if (warp == 0) {
        tmem_alloc(&tmem_base_s, 256);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = tmem_base_s;

    if (p.a_manual == 2) {
        // Thread r writes row r of A into TMEM lane r, columns 128..191: two f16 per 32-bit column.
        const uint32_t* src = reinterpret_cast<const uint32_t*>(p.a_global + (size_t)threadIdx.x * ST_K);
#pragma unroll
        for (int c = 0; c < 2; ++c) {
            uint32_t r[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = src[c * 32 + i];
            tmem_st_x32(tmem + ((uint32_t)(warp * 32) << 16) + 128u + (uint32_t)c * 32u, r);
        }
        tmem_wait_st();
        tc_fence_before_sync();
    } else if (p.a_manual) {
        // Thread r writes row r of A (K-major): 16 chunks of 8 f16 into two 64-column blocks.
        const int r = threadIdx.x;
        const uint4* src = reinterpret_cast<const uint4*>(p.a_global + (size_t)r * ST_K);
#pragma unroll
        for (int ch = 0; ch < 16; ++ch) {
            const uint4 v = src[ch];
            *reinterpret_cast<uint4*>(sA + (ch >> 3) * 16384 + sw128_chunk_offset(r, ch & 7)) = v;
        }
        fence_proxy_async_smem();
    }
    __syncthreads();

    const uint32_t b_block = p.b_mn ? 16384u : (uint32_t)p.N * 128u;
    if (threadIdx.x == 0) {
        const uint32_t bytes = (p.a_manual ? 0u : 32768u) + (uint32_t)p.N * ST_K * 2u;
        mbar_arrive_expect_tx(&bar_tma, bytes);
        if (!p.a_manual) {
            tma_load_4d(sA, &tmap_a, &bar_tma, 0, 0, 0, 0);
            tma_load_4d(sA + 16384, &tmap_a, &bar_tma, 64, 0, 0, 0);
        }
        if (p.b_mn) {
            for (int nb = 0; nb < p.N / 64; ++nb) tma_load_4d(sB + nb * 16384, &tmap_b, &bar_tma, nb * 64, 0, 0, 0);
        } else {
            for (int kb = 0; kb < 2; ++kb) tma_load_4d(sB + kb * b_block, &tmap_b, &bar_tma, kb * 64, 0, 0, 0);
        }
        if (mbar_wait(ws, &bar_tma, 0, DEERS_KERR_SELFTEST | 1)) {
            tc_fence_after_sync();
            const uint32_t idesc = idesc_f16(128, p.N, p.a_mn, p.b_mn);
            for (int ks = 0; ks < ST_K / 16; ++ks) {
                const uint64_t da = p.a_mn ? desc_mnmajor(smem_u32(sA), ks, 16384u) : desc_kmajor(smem_u32(sA), ks, 16384u);
                const uint64_t db = p.b_mn ? desc_mnmajor(smem_u32(sB), ks, b_block) : desc_kmajor(smem_u32(sB), ks, b_block);
                if (p.a_manual == 2) umma_ts(tmem, tmem + 128u + (uint32_t)ks * 8u, db, idesc, ks > 0);
                else umma_ss(tmem, da, db, idesc, ks > 0);
            }
        }
        umma_commit(&bar_mma);
    }
    __syncwarp();
    const bool ok = __all_sync(0xffffffffu, mbar_wait(ws, &bar_mma, 0, DEERS_KERR_SELFTEST | 2));
    tc_fence_after_sync();
    if (ok) {
        const int row = warp * 32 + lane;
        for (int c0 = 0; c0 < p.N; c0 += 32) {
            uint32_t r[32];
            tmem_ld_x32(tmem + ((uint32_t)(warp * 32) << 16) + (uint32_t)c0, r);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) p.out[(size_t)row * p.N + c0 + i] = __uint_as_float(r[i]);
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, 256);
}

int make_tmap_2d(deers_ctx* ctx, CUtensorMap* out, const __half* base, int rows, int cols, int box_rows) {
    const int64_t strides[4] = {(int64_t)rows * cols, (int64_t)rows * cols, cols, 1};
    return make_tmap_bhtd_f16(ctx, out, base, 1, 1, rows, cols, strides, box_rows);
}

}  // namespace

// Bounded-wait self-test: a barrier nobody arrives at.  Thread 0 waits on it through the same mbar_wait every
// kernel of the library uses, with a limit of a few milliseconds instead of two seconds; the wait must give
// up, raise the CTA's abort flag and record its code in the error word.  Thread 32 then waits on the same
// barrier and must return at once because of the flag.  The kernel ends normally: no trap, no hang.
__global__ void __launch_bounds__(64) wait_selftest_kernel(unsigned int* err, unsigned long long limit_ns, int* out) {
    __shared__ __align__(8) uint64_t bar;
    __shared__ uint32_t abort_s;
    if (threadIdx.x == 0) {
        abort_s = 0;
        mbar_init(&bar, 1);
        fence_barrier_init();
    }
    __syncthreads();
    WaitState ws{&abort_s, err, limit_ns};
    if (threadIdx.x == 0) {
        const uint64_t t0 = global_timer_ns();
        const bool ok = mbar_wait(ws, &bar, 0, DEERS_KERR_SELFTEST | 0x7f);
        out[0] = ok ? 0 : 1;                                   // 1: gave up, as it must
        out[2] = (int)((global_timer_ns() - t0) / 1000ull);    // microseconds spent waiting
    }
    __syncthreads();
    if (threadIdx.x == 32) {
        const uint64_t t0 = global_timer_ns();
        const bool ok = mbar_wait(ws, &bar, 0, DEERS_KERR_SELFTEST | 0x7e);
        out[1] = ok ? 0 : 1;
        out[3] = (int)((global_timer_ns() - t0) / 1000ull);
    }
}

int run_selftest_wait(deers_ctx* ctx, unsigned int limit_ms, int* result_host) {
    int* d = nullptr;
    DEERS_CUDA_TRY(ctx, cudaMalloc(&d, 4 * sizeof(int)));
    cudaMemsetAsync(d, 0xff, 4 * sizeof(int), ctx->stream);
    wait_selftest_kernel<<<1, 64, 0, ctx->stream>>>(ctx->dev_err, (unsigned long long)limit_ms * 1000000ull, d);
    ctx->launches += 1;
    cudaError_t e = cudaGetLastError();
    if (e == cudaSuccess) e = cudaMemcpyAsync(result_host, d, 4 * sizeof(int), cudaMemcpyDeviceToHost, ctx->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);      // the error word is left for deers_b200_sync
    cudaFree(d);
    DEERS_CUDA_TRY(ctx, e);
    return DEERS_OK;
}

int run_selftest_umma(deers_ctx* ctx, float* max_abs_err) {
    const int M = 128, K = ST_K;
    struct Case { int N, a_mn, b_mn, a_manual; };
    const Case cases[DEERS_SELFTEST_CASES] = {{128, 0, 0, 0}, {128, 0, 1, 1}, {128, 1, 1, 0}, {64, 0, 1, 0},
                                              {128, 0, 1, 2}, {64, 0, 0, 2}};
    for (int i = 0; i < DEERS_SELFTEST_CASES; ++i) max_abs_err[i] = INFINITY;

    __half *dA = nullptr, *dB = nullptr;
    float* dO = nullptr;
    DEERS_CUDA_TRY(ctx, cudaMalloc(&dA, (size_t)M * K * 2));
    DEERS_CUDA_TRY(ctx, cudaMalloc(&dB, (size_t)128 * K * 2));
    DEERS_CUDA_TRY(ctx, cudaMalloc(&dO, (size_t)M * 128 * 4));
    const size_t smem = 65536 + 1024;
    DEERS_CUDA_TRY(ctx, cudaFuncSetAttribute(umma_selftest_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));

    int rc = DEERS_OK;
    for (int ci = 0; ci < DEERS_SELFTEST_CASES && rc == DEERS_OK; ++ci) {
        const Case c = cases[ci];
        // Logical A[m][k], B[k][n]; storage depends on the operand's major-ness.
        std::vector<float> A((size_t)M * K), Bm((size_t)K * c.N);
        uint32_t s = 12345u + 977u * (uint32_t)ci;
        auto rnd = [&]() { s = s * 1664525u + 1013904223u; return ((int)((s >> 9) & 0xff) - 128) / 64.0f; };
        for (auto& x : A) x = rnd();
        for (auto& x : Bm) x = rnd();
        std::vector<__half> hA((size_t)M * K), hB((size_t)K * c.N);
        for (int m = 0; m < M; ++m)
            for (int k = 0; k < K; ++k)
                hA[c.a_mn ? (size_t)k * M + m : (size_t)m * K + k] = __float2half(A[(size_t)m * K + k]);
        for (int k = 0; k < K; ++k)
            for (int n = 0; n < c.N; ++n)
                hB[c.b_mn ? (size_t)k * c.N + n : (size_t)n * K + k] = __float2half(Bm[(size_t)k * c.N + n]);
        DEERS_CUDA_TRY(ctx, cudaMemcpyAsync(dA, hA.data(), hA.size() * 2, cudaMemcpyHostToDevice, ctx->stream));
        DEERS_CUDA_TRY(ctx, cudaMemcpyAsync(dB, hB.data(), hB.size() * 2, cudaMemcpyHostToDevice, ctx->stream));
        DEERS_CUDA_TRY(ctx, cudaMemsetAsync(dO, 0xff, (size_t)M * 128 * 4, ctx->stream));

        CUtensorMap ta, tb;
        // A: K-major storage [M][K] (rows = M) or MN-major storage [K][M] (rows = K); both 128 x 128.
        if ((rc = make_tmap_2d(ctx, &ta, dA, 128, 128, 128))) break;
        // B: K-major storage [N][K] (box rows = N) or MN-major storage [K][N] (box rows = K).
        if (c.b_mn) rc = make_tmap_2d(ctx, &tb, dB, K, c.N, 128);
        else rc = make_tmap_2d(ctx, &tb, dB, c.N, K, c.N);
        if (rc) break;

        SelftestParams p{dA, dO, ctx->dev_err, c.N, c.a_mn, c.b_mn, c.a_manual};
        umma_selftest_kernel<<<1, 128, smem, ctx->stream>>>(ta, tb, p);
        ctx->launches += 1;
        DEERS_CUDA_TRY(ctx, cudaGetLastError());
        std::vector<float> out((size_t)M * c.N);
        DEERS_CUDA_TRY(ctx, cudaMemcpyAsync(out.data(), dO, out.size() * 4, cudaMemcpyDeviceToHost, ctx->stream));
        rc = deers_b200_sync(ctx);
        if (rc) break;
        float worst = 0.f;
        for (int m = 0; m < M; ++m)
            for (int n = 0; n < c.N; ++n) {
                float acc = 0.f;
                for (int k = 0; k < K; ++k) acc += A[(size_t)m * K + k] * Bm[(size_t)k * c.N + n];
                const float e = fabsf(acc - out[(size_t)m * c.N + n]);
                worst = (e == e && e > worst) ? e : (e == e ? worst : INFINITY);
            }
        max_abs_err[ci] = worst;
    }
    cudaFree(dA); cudaFree(dB); cudaFree(dO);
    return rc;
}
