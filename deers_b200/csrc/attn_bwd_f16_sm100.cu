// f16 causal attention backward for sm_100a.
//
// Three launches, none of which uses atomics, so dQ, dK and dV are bitwise reproducible:
//   1. attn_bwd_prep_f16_kernel   delta[row] = sum_d dO*O (= rowsum(dP*P)) and lse*log2(e), both
//                                  padded to whole 128-row tiles so that the main kernels can
//                                  fetch a tile's values with one aligned bulk copy
//   2. attn_bwd_dkdv_f16_kernel   one CTA per (batch*head, KV tile of 128 rows), KV-stationary:
//                                  walks the query tiles at or below its diagonal with the dK and
//                                  dV accumulators resident in TMEM for the whole walk
//   3. attn_bwd_dq_f16_kernel     one CTA per (batch*head, query tile of 128 rows), Q-stationary:
//                                  walks the KV tiles at or left of its diagonal with the dQ
//                                  accumulator resident in TMEM
// Both main kernels recompute P from the saved lse.  Recomputing S and dP in the dQ kernel costs
// two extra products per tile pair (7 instead of 5), but the alternative - adding every
// 128 x D partial dQ tile into a float32 accumulator in global memory - was measured to be
// bound by the L2's reduction throughput (about 4 TB/s: 35 GB of reductions at B=64, H=32,
// T=2048, D=128) and needed two more memory passes to clear and convert that accumulator.
//
// dK/dV kernel: everything is computed transposed so that no operand needs a data movement
//   S^T  = K Q^T   (A = K, B = Q, both K-major as TMA writes them)      -> TMEM
//   dP^T = V dO^T  (A = V, B = dO)                                       -> TMEM
//   thread r (= KV row r) turns row r of S^T into P^T and row r of dP^T into
//   dS^T = P^T * (dP^T - delta), each stored back in place into TMEM as f16 pairs
//   dV += P^T dO   (A = P^T from TMEM, B = dO MN-major)
//   dK += dS^T Q   (A = dS^T from TMEM, B = Q MN-major)
// dQ kernel: thread r (= query row r)
//   S  = Q K^T, dP = dO V^T -> TMEM;  dS = P * (dP - delta) in place;  dQ += dS K (B = K MN-major)
// Warp roles in both: warp 0 TMA producer, warp 1 MMA issuer, warps 2-9 two compute
// warpgroups that split the 128 columns of S / dP (and the head_dim columns of the outputs).
#include "sm100_ptx.cuh"
#include "tma_host.cuh"

#include <stdlib.h>

#ifdef DEERS_TRACE
// Development aid: clock64() stamps of CTA 0's first iterations, read back by a debug entry point.
__device__ unsigned long long g_bwd_trace[16 * 3 * 8];
#define BWD_TRACE(role, ev)                                                                              \
    do {                                                                                                 \
        if (blockIdx.x == 0 && it < 16) g_bwd_trace[(it * 3 + (role)) * 8 + (ev)] = clock64();           \
    } while (0)
extern "C" __attribute__((visibility("default"))) int deers_b200_debug_bwd_trace(unsigned long long* out) {
    return (int)cudaMemcpyFromSymbol(out, g_bwd_trace, sizeof(g_bwd_trace));
}
#else
#define BWD_TRACE(role, ev) do {} while (0)
#endif
#if defined(DEERS_TRACE) && DEERS_TRACE == 1
#define TRACE_A(role, ev) BWD_TRACE(role, ev)
#else
#define TRACE_A(role, ev) do {} while (0)
#endif
#if defined(DEERS_TRACE) && DEERS_TRACE == 2
#define TRACE_B(role, ev) BWD_TRACE(role, ev)
#else
#define TRACE_B(role, ev) do {} while (0)
#endif

namespace {
using namespace sm100;

constexpr int BT = 128;                        // tile rows for both Q and KV
constexpr uint32_t BLOCK_BYTES = 128 * 128;    // one 64-column block of a 128-row tile
constexpr float LOG2E = 1.4426950408889634f;

struct BwdParams {
    const float* lse2;          // [B*H][Tpad] lse * log2(e), 0 beyond T
    const float* delta;         // [B*H][Tpad] rowsum(dO * O), 0 beyond T
    __half* dq; __half* dk; __half* dv;
    long long sdq_b, sdq_h, sdq_t, sdk_b, sdk_h, sdk_t, sdv_b, sdv_h, sdv_t;
    int B, H, T, Tpad;
    int causal;
    float scale;
    unsigned int* err;
};

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// 1-D bulk copy global -> shared, completion counted on an mbarrier (16-byte aligned, size % 16 == 0).
__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

// Launch order shared by both kernels: groups of 16 slices; inside a group the heaviest tiles
// of all its slices come first (balance) and the group's tensors (a few MB) stay in L2.
__device__ __forceinline__ void tile_of_block(int B, int H, int ntile, int& slot, int& bh) {
    const int BH = B * H;
    const int group = (int)(blockIdx.x / (16u * ntile));
    const int gsize = min(16, BH - group * 16);
    const int within = (int)(blockIdx.x - (unsigned)group * 16u * ntile);
    slot = within / gsize;                                   // 0 = heaviest
    bh = group * 16 + within % gsize;
}

// Stores 32 f32 TMEM columns of one row as 32 f16 values (64 bytes), scaled by s.
__device__ __forceinline__ void store_row32(__half* dst, const uint32_t (&r)[32], float s) {
#pragma unroll
    for (int q8 = 0; q8 < 4; ++q8) {
        uint4 a;
        a.x = pack_half2(__uint_as_float(r[q8 * 8 + 0]) * s, __uint_as_float(r[q8 * 8 + 1]) * s);
        a.y = pack_half2(__uint_as_float(r[q8 * 8 + 2]) * s, __uint_as_float(r[q8 * 8 + 3]) * s);
        a.z = pack_half2(__uint_as_float(r[q8 * 8 + 4]) * s, __uint_as_float(r[q8 * 8 + 5]) * s);
        a.w = pack_half2(__uint_as_float(r[q8 * 8 + 6]) * s, __uint_as_float(r[q8 * 8 + 7]) * s);
        *reinterpret_cast<uint4*>(dst + q8 * 8) = a;
    }
}

// ---------------------------------------------------------------------------------------------
// dK / dV kernel
// ---------------------------------------------------------------------------------------------
// Dynamic shared memory only; the base must be 1024-byte aligned for the 128-byte swizzle (checked).
template <int D>
struct DkvSmem {
    static constexpr uint32_t TILE = 128u * D * 2u;
    static constexpr uint32_t K = 0;
    static constexpr uint32_t V = K + TILE;
    static constexpr uint32_t Q = V + TILE;                  // two stages
    static constexpr uint32_t DO = Q + 2 * TILE;             // two stages
    static constexpr uint32_t LSE2 = DO + 2 * TILE;          // two stages of 128 floats
    static constexpr uint32_t DELTA = LSE2 + 2 * BT * 4;
    static constexpr uint32_t BARS = DELTA + 2 * BT * 4;
    static constexpr uint32_t TOTAL = BARS + 256;
};

enum DkvBar { A_KV = 0, A_QDO_FULL = 1, A_QDO_EMPTY = 3, A_S = 5, A_DP = 6, A_P = 7, A_DS = 8, A_DONE = 9, A_COUNT = 10 };

template <int D>
__global__ void __launch_bounds__(320, 1)
attn_bwd_dkdv_f16_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                         const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_do,
                         const BwdParams p) {
    using L = DkvSmem<D>;
    constexpr uint32_t TILE_BYTES = L::TILE;
    constexpr int DBLK = D / 64;
    constexpr int DH = D / 2;                               // output columns per compute warpgroup
    constexpr uint32_t TMEM_COLS = 512;
    // S^T (later P^T in place) | dP^T (later dS^T in place) | dV | dK
    constexpr uint32_t TM_S = 0, TM_DP = 128, TM_DV = 256, TM_DK = 256 + D;

    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t* sK = smem + L::K;
    uint8_t* sV = smem + L::V;
    uint8_t* sQ = smem + L::Q;
    uint8_t* sDO = smem + L::DO;
    float* lse2_s = reinterpret_cast<float*>(smem + L::LSE2);      // [2][BT]
    float* delta_s = reinterpret_cast<float*>(smem + L::DELTA);    // [2][BT]
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::BARS);
    uint32_t* tmem_base_s = reinterpret_cast<uint32_t*>(bars + A_COUNT);
    volatile uint32_t* abort_s = tmem_base_s + 1;
    uint32_t* skip_s = tmem_base_s + 2;

    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const int nq = (p.T + BT - 1) / BT;
    int kt, bh;
    tile_of_block(p.B, p.H, nq, kt, bh);                    // low KV tiles carry the most work
    const int b = bh / p.H, h = bh % p.H;
    const int k0 = kt * BT;
    const int i0 = p.causal ? kt : 0;
    const int niter = nq - i0;

    if (threadIdx.x == 0) {
        *abort_s = 0;
        uint32_t skip = (*(volatile unsigned int*)p.err != 0) ? 1u : 0u;   // an earlier CTA gave up
        if ((smem_u32(smem) & 1023u) != 0) {
            atomicCAS(p.err, 0u, DEERS_KERR_BWD_F16 | 0x20);
            skip = 1;
        }
        *skip_s = skip;
        mbar_init(&bars[A_KV], 1);
        for (int s = 0; s < 2; ++s) { mbar_init(&bars[A_QDO_FULL + s], 1); mbar_init(&bars[A_QDO_EMPTY + s], 1); }
        mbar_init(&bars[A_S], 1);
        mbar_init(&bars[A_DP], 1);
        mbar_init(&bars[A_P], 256);
        mbar_init(&bars[A_DS], 256);
        mbar_init(&bars[A_DONE], 1);
        fence_barrier_init();
        tma_prefetch_desc(&tmap_q); tma_prefetch_desc(&tmap_k); tma_prefetch_desc(&tmap_v); tma_prefetch_desc(&tmap_do);
    }
    __syncthreads();
    if (*skip_s) return;
    if (warp == 1) {
        tmem_alloc(tmem_base_s, TMEM_COLS);
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
            mbar_arrive_expect_tx(&bars[A_KV], 2 * TILE_BYTES);
#pragma unroll
            for (int blk = 0; blk < DBLK; ++blk) {
                tma_load_4d(sK + blk * BLOCK_BYTES, &tmap_k, &bars[A_KV], blk * 64, k0, h, b);
                tma_load_4d(sV + blk * BLOCK_BYTES, &tmap_v, &bars[A_KV], blk * 64, k0, h, b);
            }
            for (int it = 0; it < niter; ++it) {
                const int st = it & 1;
                const uint32_t ph = (uint32_t)(it >> 1) & 1u;
                if (!mbar_wait(ws, &bars[A_QDO_EMPTY + st], ph ^ 1u, DEERS_KERR_BWD_F16 | 1)) break;
                uint64_t* full = &bars[A_QDO_FULL + st];
                mbar_arrive_expect_tx(full, 2 * TILE_BYTES + 2 * BT * 4);
                const int q0 = (i0 + it) * BT;
                bulk_load(lse2_s + st * BT, p.lse2 + (long long)bh * p.Tpad + q0, BT * 4, full);
                bulk_load(delta_s + st * BT, p.delta + (long long)bh * p.Tpad + q0, BT * 4, full);
#pragma unroll
                for (int blk = 0; blk < DBLK; ++blk) {
                    tma_load_4d(sQ + st * TILE_BYTES + blk * BLOCK_BYTES, &tmap_q, full, blk * 64, q0, h, b);
                    tma_load_4d(sDO + st * TILE_BYTES + blk * BLOCK_BYTES, &tmap_do, full, blk * 64, q0, h, b);
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer ------------------------------
        if (lane == 0) {
            constexpr uint32_t IDESC_ST = idesc_f16(128, 128, 0, 0);   // S^T, dP^T: K-major A and B
            constexpr uint32_t IDESC_KV = idesc_f16(128, D, 0, 1);     // dV, dK: A from TMEM, MN-major B
            // Step-0 descriptors of every operand view, built once; each MMA adds a constant
            // (a single thread issues, so descriptor arithmetic must stay off the issue path).
            constexpr uint64_t STAGE_STEP = TILE_BYTES >> 4;           // next stage of Q / dO
            const uint64_t k_km = desc_kmajor(smem_u32(sK), 0, BLOCK_BYTES);
            const uint64_t v_km = desc_kmajor(smem_u32(sV), 0, BLOCK_BYTES);
            const uint64_t q_km0 = desc_kmajor(smem_u32(sQ), 0, BLOCK_BYTES), q_mn0 = desc_mnmajor(smem_u32(sQ), 0, BLOCK_BYTES);
            const uint64_t do_km0 = desc_kmajor(smem_u32(sDO), 0, BLOCK_BYTES), do_mn0 = desc_mnmajor(smem_u32(sDO), 0, BLOCK_BYTES);
            auto issue_st = [&](uint64_t q_km) {
#pragma unroll
                for (int ks = 0; ks < D / 16; ++ks)
                    umma_ss(tmem + TM_S, k_km + kmajor_step(ks, BLOCK_BYTES), q_km + kmajor_step(ks, BLOCK_BYTES), IDESC_ST, ks > 0);
                umma_commit(&bars[A_S]);
            };
            auto issue_dpt = [&](uint64_t do_km) {
#pragma unroll
                for (int ks = 0; ks < D / 16; ++ks)
                    umma_ss(tmem + TM_DP, v_km + kmajor_step(ks, BLOCK_BYTES), do_km + kmajor_step(ks, BLOCK_BYTES), IDESC_ST, ks > 0);
                umma_commit(&bars[A_DP]);
            };
            // A operand in TMEM: 32 packed columns per warpgroup half, halves 64 columns apart.
            auto a_tmem = [&](uint32_t base, int ks) { return tmem + base + (uint32_t)(ks >> 2) * 64u + (uint32_t)(ks & 3) * 8u; };
            bool ok = mbar_wait(ws, &bars[A_KV], 0, DEERS_KERR_BWD_F16 | 2) &&
                      mbar_wait(ws, &bars[A_QDO_FULL], 0, DEERS_KERR_BWD_F16 | 3);
            if (ok) {
                tc_fence_after_sync();
                issue_st(q_km0);
                issue_dpt(do_km0);
            }
            for (int it = 0; ok && it < niter; ++it) {
                const int st = it & 1, sn = st ^ 1;
                const uint32_t par = (uint32_t)it & 1u;
                const uint64_t q_mn = q_mn0 + (uint64_t)st * STAGE_STEP, do_mn = do_mn0 + (uint64_t)st * STAGE_STEP;
                const bool more = it + 1 < niter;
                // dV += P^T dO, then S^T of the next query tile: the pipe is in order, so the
                // new S^T lands only after dV has consumed P^T from the same columns.
                TRACE_A(0, 0);
                if (!mbar_wait(ws, &bars[A_P], par, DEERS_KERR_BWD_F16 | 4)) break;
                tc_fence_after_sync();
                TRACE_A(0, 1);
#pragma unroll
                for (int ks = 0; ks < BT / 16; ++ks)
                    umma_ts(tmem + TM_DV, a_tmem(TM_S, ks), do_mn + mnmajor_step(ks), IDESC_KV, (it > 0 || ks > 0));
                if (more) {
                    if (!mbar_wait(ws, &bars[A_QDO_FULL + sn], (uint32_t)((it + 1) >> 1) & 1u, DEERS_KERR_BWD_F16 | 6)) break;
                    tc_fence_after_sync();
                    issue_st(q_km0 + (uint64_t)sn * STAGE_STEP);
                }
                // dK += dS^T Q, then dP^T of the next query tile over the consumed dS^T columns.
                TRACE_A(0, 2);
                if (!mbar_wait(ws, &bars[A_DS], par, DEERS_KERR_BWD_F16 | 5)) break;
                tc_fence_after_sync();
                TRACE_A(0, 3);
#pragma unroll
                for (int ks = 0; ks < BT / 16; ++ks)
                    umma_ts(tmem + TM_DK, a_tmem(TM_DP, ks), q_mn + mnmajor_step(ks), IDESC_KV, (it > 0 || ks > 0));
                umma_commit(&bars[A_QDO_EMPTY + st]);                  // Q / dO of this stage are consumed
                if (more) issue_dpt(do_km0 + (uint64_t)sn * STAGE_STEP);
                TRACE_A(0, 4);
            }
            umma_commit(&bars[A_DONE]);
        }
    } else {
        // ------------------------------ compute threads ------------------------------
        // Warpgroup g owns query columns [64g, 64g+64) of S^T / dP^T and columns
        // [g*D/2, (g+1)*D/2) of dK and dV.  Thread r of a warpgroup owns TMEM lane r = KV row r.
        const int g = (warp - 2) >> 2;
        const int lane_base = (warp & 3) * 32;
        const int r = lane_base + lane;
        const uint32_t t_lane = (uint32_t)lane_base << 16;
        const float sl2 = p.scale * LOG2E;
        const bool kv_valid = (k0 + r) < p.T;               // rows past the sequence end contribute nothing
        bool alive = true;
#ifdef DEERS_TRACE
        const bool tr = lane == 0 && (warp == 2 || warp == 6);
#endif

        for (int it = 0; it < niter; ++it) {
            const int i = i0 + it;
            const int st = it & 1;
            const uint32_t par = (uint32_t)it & 1u;
            const float* lse2 = lse2_s + st * BT + 64 * g;
            const float* dlt = delta_s + st * BT + 64 * g;
            // The stage's lse / delta rows arrive with Q and dO: observe that barrier directly.
            if (!__all_sync(0xffffffffu, mbar_wait(ws, &bars[A_QDO_FULL + st], (uint32_t)(it >> 1) & 1u, DEERS_KERR_BWD_F16 | 8))) { alive = false; break; }
#ifdef DEERS_TRACE
            if (tr) TRACE_A(1 + g, 0);
#endif
            if (!__all_sync(0xffffffffu, mbar_wait(ws, &bars[A_S], par, DEERS_KERR_BWD_F16 | 9))) { alive = false; break; }
            tc_fence_after_sync();
#ifdef DEERS_TRACE
            if (tr) TRACE_A(1 + g, 1);
#endif
            const bool diag = p.causal && (i == kt);
            uint32_t pk[32];                                // P^T row, 64 query columns as f16 pairs
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                uint32_t sr[32];
                tmem_ld_x32(tmem + TM_S + t_lane + 64 * g + c * 32, sr);
                tmem_wait_ld();
                if (diag || !kv_valid) {                    // only the diagonal / tail tile pays for masking
#pragma unroll
                    for (int e = 0; e < 16; ++e) {
                        const int cl = c * 32 + e * 2;      // column inside this warpgroup's half
                        float p0 = ex2(fmaf(__uint_as_float(sr[e * 2]), sl2, -lse2[cl]));
                        float p1 = ex2(fmaf(__uint_as_float(sr[e * 2 + 1]), sl2, -lse2[cl + 1]));
                        if ((diag && (64 * g + cl) < r) || !kv_valid) p0 = 0.f;   // query index < key index: masked
                        if ((diag && (64 * g + cl + 1) < r) || !kv_valid) p1 = 0.f;
                        pk[c * 16 + e] = pack_half2(p0, p1);
                    }
                } else {
#pragma unroll
                    for (int e = 0; e < 16; ++e) {
                        const int cl = c * 32 + e * 2;
                        pk[c * 16 + e] = pack_half2(ex2(fmaf(__uint_as_float(sr[e * 2]), sl2, -lse2[cl])),
                                                    ex2(fmaf(__uint_as_float(sr[e * 2 + 1]), sl2, -lse2[cl + 1])));
                    }
                }
            }
            // P^T replaces this warpgroup's half of S^T in TMEM (32 packed columns).
            tmem_st_x32(tmem + TM_S + t_lane + 64 * g, pk);
            tmem_wait_st();
            tc_fence_before_sync();
            mbar_arrive(&bars[A_P]);
#ifdef DEERS_TRACE
            if (tr) TRACE_A(1 + g, 2);
#endif

            if (!__all_sync(0xffffffffu, mbar_wait(ws, &bars[A_DP], par, DEERS_KERR_BWD_F16 | 10))) { alive = false; break; }
            tc_fence_after_sync();
#ifdef DEERS_TRACE
            if (tr) TRACE_A(1 + g, 3);
#endif
            uint32_t dd[32];                                // dS^T row, 64 query columns as f16 pairs
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                uint32_t dr[32];
                tmem_ld_x32(tmem + TM_DP + t_lane + 64 * g + c * 32, dr);
                tmem_wait_ld();
#pragma unroll
                for (int e = 0; e < 16; ++e) {
                    const int cl = c * 32 + e * 2;
                    const float2 pf = __half22float2(*reinterpret_cast<const __half2*>(&pk[c * 16 + e]));
                    dd[c * 16 + e] = pack_half2(pf.x * (__uint_as_float(dr[e * 2]) - dlt[cl]),
                                                pf.y * (__uint_as_float(dr[e * 2 + 1]) - dlt[cl + 1]));
                }
            }
            tmem_st_x32(tmem + TM_DP + t_lane + 64 * g, dd);
            tmem_wait_st();
            tc_fence_before_sync();
            mbar_arrive(&bars[A_DS]);
#ifdef DEERS_TRACE
            if (tr) TRACE_A(1 + g, 4);
#endif
        }

        if (alive && __all_sync(0xffffffffu, mbar_wait(ws, &bars[A_DONE], 0, DEERS_KERR_BWD_F16 | 12))) {
            tc_fence_after_sync();
            const int krow = k0 + r;
            __half* dkrow = p.dk + b * p.sdk_b + h * p.sdk_h + (long long)krow * p.sdk_t + g * DH;
            __half* dvrow = p.dv + b * p.sdv_b + h * p.sdv_h + (long long)krow * p.sdv_t + g * DH;
#pragma unroll
            for (int c = 0; c < DH / 32; ++c) {
                uint32_t kr[32], vr[32];
                tmem_ld_x32(tmem + TM_DK + t_lane + g * DH + c * 32, kr);
                tmem_ld_x32(tmem + TM_DV + t_lane + g * DH + c * 32, vr);
                tmem_wait_ld();
                if (krow < p.T) {
                    store_row32(dkrow + c * 32, kr, p.scale);
                    store_row32(dvrow + c * 32, vr, 1.0f);
                }
            }
        }
    }

    __syncwarp();
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem, TMEM_COLS);
}

// ---------------------------------------------------------------------------------------------
// dQ kernel
// ---------------------------------------------------------------------------------------------
template <int D>
struct DqSmem {
    static constexpr uint32_t TILE = 128u * D * 2u;
    static constexpr uint32_t Q = 0;
    static constexpr uint32_t DO = Q + TILE;
    static constexpr uint32_t K = DO + TILE;                 // two stages
    static constexpr uint32_t V = K + 2 * TILE;              // two stages
    static constexpr uint32_t BARS = V + 2 * TILE;
    static constexpr uint32_t TOTAL = BARS + 256;
};

enum DqBar { Q_QDO = 0, Q_KV_FULL = 1, Q_KV_EMPTY = 3, Q_S = 5, Q_DP = 6, Q_PDONE = 7, Q_DS = 8, Q_DONE = 9, Q_COUNT = 10 };

template <int D>
__global__ void __launch_bounds__(320, 1)
attn_bwd_dq_f16_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                       const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_do,
                       const BwdParams p) {
    using L = DqSmem<D>;
    constexpr uint32_t TILE_BYTES = L::TILE;
    constexpr int DBLK = D / 64;
    constexpr int DH = D / 2;
    constexpr uint32_t TMEM_COLS = 512;
    // S | dP (later dS in place) | dQ
    constexpr uint32_t TM_S = 0, TM_DP = 128, TM_DQ = 256;

    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t* sQ = smem + L::Q;
    uint8_t* sDO = smem + L::DO;
    uint8_t* sK = smem + L::K;
    uint8_t* sV = smem + L::V;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::BARS);
    uint32_t* tmem_base_s = reinterpret_cast<uint32_t*>(bars + Q_COUNT);
    volatile uint32_t* abort_s = tmem_base_s + 1;
    uint32_t* skip_s = tmem_base_s + 2;

    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const int nq = (p.T + BT - 1) / BT;
    int slot, bh;
    tile_of_block(p.B, p.H, nq, slot, bh);
    const int qt = nq - 1 - slot;                           // late query tiles carry the most work
    const int b = bh / p.H, h = bh % p.H;
    const int q0 = qt * BT;
    const int ntiles = p.causal ? qt + 1 : nq;

    if (threadIdx.x == 0) {
        *abort_s = 0;
        uint32_t skip = (*(volatile unsigned int*)p.err != 0) ? 1u : 0u;
        if ((smem_u32(smem) & 1023u) != 0) {
            atomicCAS(p.err, 0u, DEERS_KERR_BWD_F16 | 0x21);
            skip = 1;
        }
        *skip_s = skip;
        mbar_init(&bars[Q_QDO], 1);
        for (int s = 0; s < 2; ++s) { mbar_init(&bars[Q_KV_FULL + s], 1); mbar_init(&bars[Q_KV_EMPTY + s], 1); }
        mbar_init(&bars[Q_S], 1);
        mbar_init(&bars[Q_DP], 1);
        mbar_init(&bars[Q_PDONE], 256);
        mbar_init(&bars[Q_DS], 256);
        mbar_init(&bars[Q_DONE], 1);
        fence_barrier_init();
        tma_prefetch_desc(&tmap_q); tma_prefetch_desc(&tmap_k); tma_prefetch_desc(&tmap_v); tma_prefetch_desc(&tmap_do);
    }
    __syncthreads();
    if (*skip_s) return;
    if (warp == 1) {
        tmem_alloc(tmem_base_s, TMEM_COLS);
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
            mbar_arrive_expect_tx(&bars[Q_QDO], 2 * TILE_BYTES);
#pragma unroll
            for (int blk = 0; blk < DBLK; ++blk) {
                tma_load_4d(sQ + blk * BLOCK_BYTES, &tmap_q, &bars[Q_QDO], blk * 64, q0, h, b);
                tma_load_4d(sDO + blk * BLOCK_BYTES, &tmap_do, &bars[Q_QDO], blk * 64, q0, h, b);
            }
            for (int j = 0; j < ntiles; ++j) {
                const int st = j & 1;
                const uint32_t ph = (uint32_t)(j >> 1) & 1u;
                if (!mbar_wait(ws, &bars[Q_KV_EMPTY + st], ph ^ 1u, DEERS_KERR_BWD_F16 | 0x11)) break;
                uint64_t* full = &bars[Q_KV_FULL + st];
                mbar_arrive_expect_tx(full, 2 * TILE_BYTES);
#pragma unroll
                for (int blk = 0; blk < DBLK; ++blk) {
                    tma_load_4d(sK + st * TILE_BYTES + blk * BLOCK_BYTES, &tmap_k, full, blk * 64, j * BT, h, b);
                    tma_load_4d(sV + st * TILE_BYTES + blk * BLOCK_BYTES, &tmap_v, full, blk * 64, j * BT, h, b);
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer ------------------------------
        if (lane == 0) {
            constexpr uint32_t IDESC_S = idesc_f16(128, 128, 0, 0);    // S, dP: K-major A and B
            constexpr uint32_t IDESC_DQ = idesc_f16(128, D, 0, 1);     // dQ: A from TMEM, MN-major B
            constexpr uint64_t STAGE_STEP = TILE_BYTES >> 4;
            const uint64_t q_km = desc_kmajor(smem_u32(sQ), 0, BLOCK_BYTES), do_km = desc_kmajor(smem_u32(sDO), 0, BLOCK_BYTES);
            const uint64_t k_km0 = desc_kmajor(smem_u32(sK), 0, BLOCK_BYTES), k_mn0 = desc_mnmajor(smem_u32(sK), 0, BLOCK_BYTES);
            const uint64_t v_km0 = desc_kmajor(smem_u32(sV), 0, BLOCK_BYTES);
            auto issue_s = [&](int st) {
                const uint64_t k_km = k_km0 + (uint64_t)st * STAGE_STEP;
#pragma unroll
                for (int ks = 0; ks < D / 16; ++ks)
                    umma_ss(tmem + TM_S, q_km + kmajor_step(ks, BLOCK_BYTES), k_km + kmajor_step(ks, BLOCK_BYTES), IDESC_S, ks > 0);
                umma_commit(&bars[Q_S]);
            };
            auto issue_dp = [&](int st) {
                const uint64_t v_km = v_km0 + (uint64_t)st * STAGE_STEP;
#pragma unroll
                for (int ks = 0; ks < D / 16; ++ks)
                    umma_ss(tmem + TM_DP, do_km + kmajor_step(ks, BLOCK_BYTES), v_km + kmajor_step(ks, BLOCK_BYTES), IDESC_S, ks > 0);
                umma_commit(&bars[Q_DP]);
            };
            bool ok = mbar_wait(ws, &bars[Q_QDO], 0, DEERS_KERR_BWD_F16 | 0x12) &&
                      mbar_wait(ws, &bars[Q_KV_FULL], 0, DEERS_KERR_BWD_F16 | 0x13);
            if (ok) {
                tc_fence_after_sync();
                issue_s(0);
                issue_dp(0);
            }
            for (int j = 0; ok && j < ntiles; ++j) {
#ifdef DEERS_TRACE
                const int it = j;
#endif
                const int st = j & 1, sn = st ^ 1;
                const uint32_t par = (uint32_t)j & 1u;
                const bool more = j + 1 < ntiles;
                // S of the next KV tile as soon as the compute threads have read this one.
                TRACE_B(0, 0);
                if (!mbar_wait(ws, &bars[Q_PDONE], par, DEERS_KERR_BWD_F16 | 0x14)) break;
                TRACE_B(0, 1);
                if (more) {
                    if (!mbar_wait(ws, &bars[Q_KV_FULL + sn], (uint32_t)((j + 1) >> 1) & 1u, DEERS_KERR_BWD_F16 | 0x15)) break;
                    tc_fence_after_sync();
                    issue_s(sn);
                }
                // dQ += dS K, then dP of the next KV tile over the consumed dS columns.
                TRACE_B(0, 2);
                if (!mbar_wait(ws, &bars[Q_DS], par, DEERS_KERR_BWD_F16 | 0x16)) break;
                tc_fence_after_sync();
                TRACE_B(0, 3);
                const uint64_t k_mn = k_mn0 + (uint64_t)st * STAGE_STEP;
#pragma unroll
                for (int ks = 0; ks < BT / 16; ++ks)
                    umma_ts(tmem + TM_DQ, tmem + TM_DP + (uint32_t)(ks >> 2) * 64u + (uint32_t)(ks & 3) * 8u,
                            k_mn + mnmajor_step(ks), IDESC_DQ, (j > 0 || ks > 0));
                umma_commit(&bars[Q_KV_EMPTY + st]);                   // K / V of this stage are consumed
                if (more) issue_dp(sn);
                TRACE_B(0, 4);
            }
            umma_commit(&bars[Q_DONE]);
        }
    } else {
        // ------------------------------ compute threads ------------------------------
        // Warpgroup g owns key columns [64g, 64g+64) of S / dP and columns [g*D/2, (g+1)*D/2) of
        // dQ.  Thread r of a warpgroup owns TMEM lane r = query row r.
        const int g = (warp - 2) >> 2;
        const int lane_base = (warp & 3) * 32;
        const int r = lane_base + lane;
        const uint32_t t_lane = (uint32_t)lane_base << 16;
        const float sl2 = p.scale * LOG2E;
        const float lse2_r = p.lse2[(long long)bh * p.Tpad + q0 + r];      // padded: 0 beyond T
        const float delta_r = p.delta[(long long)bh * p.Tpad + q0 + r];
        bool alive = true;
#ifdef DEERS_TRACE
        const bool tr = lane == 0 && (warp == 2 || warp == 6);
#endif

        for (int j = 0; j < ntiles; ++j) {
#ifdef DEERS_TRACE
            const int it = j;
            if (tr) TRACE_B(1 + g, 0);
#endif
            const uint32_t par = (uint32_t)j & 1u;
            if (!__all_sync(0xffffffffu, mbar_wait(ws, &bars[Q_S], par, DEERS_KERR_BWD_F16 | 0x17))) { alive = false; break; }
            tc_fence_after_sync();
#ifdef DEERS_TRACE
            if (tr) TRACE_B(1 + g, 1);
#endif
            const int k0 = j * BT;
            const bool edge = (p.causal && j == qt) || (k0 + BT > p.T);
            float pv[64];                                   // P row, this warpgroup's 64 key columns
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                uint32_t sr[32];
                tmem_ld_x32(tmem + TM_S + t_lane + 64 * g + c * 32, sr);
                tmem_wait_ld();
                if (edge) {
#pragma unroll
                    for (int e = 0; e < 32; ++e) {
                        const int col = 64 * g + c * 32 + e;                  // key index inside the tile
                        const bool masked = (p.causal && j == qt && col > r) || (k0 + col >= p.T);
                        pv[c * 32 + e] = masked ? 0.f : ex2(fmaf(__uint_as_float(sr[e]), sl2, -lse2_r));
                    }
                } else {
#pragma unroll
                    for (int e = 0; e < 32; ++e) pv[c * 32 + e] = ex2(fmaf(__uint_as_float(sr[e]), sl2, -lse2_r));
                }
            }
            tc_fence_before_sync();
            mbar_arrive(&bars[Q_PDONE]);                    // S has been read: the next S may land
#ifdef DEERS_TRACE
            if (tr) TRACE_B(1 + g, 2);
#endif

            if (!__all_sync(0xffffffffu, mbar_wait(ws, &bars[Q_DP], par, DEERS_KERR_BWD_F16 | 0x18))) { alive = false; break; }
            tc_fence_after_sync();
#ifdef DEERS_TRACE
            if (tr) TRACE_B(1 + g, 3);
#endif
            uint32_t dd[32];
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                uint32_t dr[32];
                tmem_ld_x32(tmem + TM_DP + t_lane + 64 * g + c * 32, dr);
                tmem_wait_ld();
#pragma unroll
                for (int e = 0; e < 16; ++e)
                    dd[c * 16 + e] = pack_half2(pv[c * 32 + e * 2] * (__uint_as_float(dr[e * 2]) - delta_r),
                                                pv[c * 32 + e * 2 + 1] * (__uint_as_float(dr[e * 2 + 1]) - delta_r));
            }
            // dS replaces this warpgroup's half of dP in TMEM (32 packed columns).
            tmem_st_x32(tmem + TM_DP + t_lane + 64 * g, dd);
            tmem_wait_st();
            tc_fence_before_sync();
            mbar_arrive(&bars[Q_DS]);
#ifdef DEERS_TRACE
            if (tr) TRACE_B(1 + g, 4);
#endif
        }

        if (alive && __all_sync(0xffffffffu, mbar_wait(ws, &bars[Q_DONE], 0, DEERS_KERR_BWD_F16 | 0x19))) {
            tc_fence_after_sync();
            const int qrow = q0 + r;
            __half* dqrow = p.dq + b * p.sdq_b + h * p.sdq_h + (long long)qrow * p.sdq_t + g * DH;
#pragma unroll
            for (int c = 0; c < DH / 32; ++c) {
                uint32_t qr[32];
                tmem_ld_x32(tmem + TM_DQ + t_lane + g * DH + c * 32, qr);
                tmem_wait_ld();
                if (qrow < p.T) store_row32(dqrow + c * 32, qr, p.scale);
            }
        }
    }

    __syncwarp();
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem, TMEM_COLS);
}

// delta[row] = sum_d dO[row][d] * O[row][d] and lse2[row] = lse[row] * log2(e) on the padded
// [B*H][Tpad] grid (0 beyond T).  One warp per row.
template <int D>
__global__ void __launch_bounds__(256)
attn_bwd_prep_f16_kernel(const __half* __restrict__ o, const __half* __restrict__ d_o, const float* __restrict__ lse,
                         float* __restrict__ delta, float* __restrict__ lse2, int B, int H, int T, int Tpad,
                         long long so_b, long long so_h, long long so_t, long long sdo_b, long long sdo_h,
                         long long sdo_t) {
    const long long row = (long long)blockIdx.x * 8 + threadIdx.x / 32;
    const int lane = threadIdx.x % 32;
    if (row >= (long long)B * H * Tpad) return;
    const int t = (int)(row % Tpad);
    const int bh = (int)(row / Tpad);
    constexpr int PER = D / 32;                              // 2 or 4 elements per lane
    if (t >= T) {
        if (lane == 0) { delta[row] = 0.f; lse2[row] = 0.f; }
        return;
    }
    const int b = bh / H, h = bh % H;
    const __half* orow = o + b * so_b + h * so_h + (long long)t * so_t + lane * PER;
    const __half* grow = d_o + b * sdo_b + h * sdo_h + (long long)t * sdo_t + lane * PER;
    float s = 0.f;
#pragma unroll
    for (int e = 0; e < PER; e += 2) {
        const float2 a = __half22float2(*reinterpret_cast<const __half2*>(orow + e));
        const float2 g = __half22float2(*reinterpret_cast<const __half2*>(grow + e));
        s = fmaf(a.x, g.x, s);
        s = fmaf(a.y, g.y, s);
    }
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
    if (lane == 0) {
        delta[row] = s;
        lse2[row] = lse[(long long)bh * T + t] * LOG2E;
    }
}

size_t bwd_stat_bytes(const deers_attn_desc* d) {
    const size_t Tpad = (size_t)((d->T + BT - 1) / BT) * BT;
    return ((size_t)d->B * d->H * Tpad * sizeof(float) + 255) / 256 * 256;
}

template <int D>
int bwd_launch(deers_ctx* ctx, const deers_attn_desc* d, const void* q, const void* k, const void* v, const void* o,
               const float* lse, const void* d_o, void* dq, void* dk, void* dv, void* workspace) {
    CUtensorMap tq, tk, tv, tdo;
    int rc;
    if ((rc = make_tmap_bhtd_f16(ctx, &tq, q, d->B, d->H, d->T, D, d->q_strides, BT))) return rc;
    if ((rc = make_tmap_bhtd_f16(ctx, &tk, k, d->B, d->H, d->T, D, d->k_strides, BT))) return rc;
    if ((rc = make_tmap_bhtd_f16(ctx, &tv, v, d->B, d->H, d->T, D, d->v_strides, BT))) return rc;
    if ((rc = make_tmap_bhtd_f16(ctx, &tdo, d_o, d->B, d->H, d->T, D, d->do_strides, BT))) return rc;
    const int nq = (d->T + BT - 1) / BT;
    const int Tpad = nq * BT;
    const long long BH = (long long)d->B * d->H;
    const size_t stat_bytes = bwd_stat_bytes(d);
    float* delta = (float*)workspace;
    float* lse2 = (float*)((char*)workspace + stat_bytes);

    const long long prep_rows = BH * Tpad;
    {
        KernelTimerScope ts(ctx, DEERS_K_BWD_PREP);
        attn_bwd_prep_f16_kernel<D><<<(unsigned)((prep_rows + 7) / 8), 256, 0, ctx->stream>>>(
            (const __half*)o, (const __half*)d_o, lse, delta, lse2, d->B, d->H, d->T, Tpad, d->o_strides[0],
            d->o_strides[1], d->o_strides[2], d->do_strides[0], d->do_strides[1], d->do_strides[2]);
    }
    DEERS_CUDA_TRY(ctx, cudaGetLastError());

    BwdParams p;
    p.lse2 = lse2; p.delta = delta;
    p.dq = (__half*)dq; p.dk = (__half*)dk; p.dv = (__half*)dv;
    p.sdq_b = d->dq_strides[0]; p.sdq_h = d->dq_strides[1]; p.sdq_t = d->dq_strides[2];
    p.sdk_b = d->dk_strides[0]; p.sdk_h = d->dk_strides[1]; p.sdk_t = d->dk_strides[2];
    p.sdv_b = d->dv_strides[0]; p.sdv_h = d->dv_strides[1]; p.sdv_t = d->dv_strides[2];
    p.B = d->B; p.H = d->H; p.T = d->T; p.Tpad = Tpad; p.causal = d->causal; p.scale = d->scale;
    p.err = ctx->dev_err;
    const long long grid = BH * nq;
    if (grid > 0x7fffffffLL) return DEERS_ERR_SHAPE;

    const size_t smem_a = DkvSmem<D>::TOTAL, smem_b = DqSmem<D>::TOTAL;
    DEERS_CUDA_TRY(ctx, cudaFuncSetAttribute(attn_bwd_dkdv_f16_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_a));
    DEERS_CUDA_TRY(ctx, cudaFuncSetAttribute(attn_bwd_dq_f16_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_b));
    {
        KernelTimerScope ts(ctx, DEERS_K_BWD_MAIN);
        attn_bwd_dkdv_f16_kernel<D><<<(unsigned)grid, 320, smem_a, ctx->stream>>>(tq, tk, tv, tdo, p);
    }
    DEERS_CUDA_TRY(ctx, cudaGetLastError());
    {
        KernelTimerScope ts(ctx, DEERS_K_BWD_DQ);
        attn_bwd_dq_f16_kernel<D><<<(unsigned)grid, 320, smem_b, ctx->stream>>>(tq, tk, tv, tdo, p);
    }
    DEERS_CUDA_TRY(ctx, cudaGetLastError());
    ctx->launches += 3;
    return DEERS_OK;
}

}  // namespace

// Workspace: delta [B*H][Tpad] | lse*log2e [B*H][Tpad], float32, Tpad = T rounded up to 128.
size_t attn_bwd_f16_workspace_bytes(const deers_attn_desc* d) { return 2 * bwd_stat_bytes(d); }

int launch_attn_bwd_f16(deers_ctx* ctx, const deers_attn_desc* d, const void* q, const void* k, const void* v,
                        const void* o, const float* lse, const void* d_o, void* dq, void* dk, void* dv,
                        void* workspace) {
    if (d->D == 64) return bwd_launch<64>(ctx, d, q, k, v, o, lse, d_o, dq, dk, dv, workspace);
    if (d->D == 128) return bwd_launch<128>(ctx, d, q, k, v, o, lse, d_o, dq, dk, dv, workspace);
    return DEERS_ERR_UNSUPPORTED;
}
