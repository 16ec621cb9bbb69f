// f16 causal attention backward for sm_100a.
//
// Three launches:
//   1. attn_bwd_prep_f16_kernel     delta[row] = sum_d dO*O (= rowsum(dP*P)) and lse*log2(e), both
//                                    padded to whole tiles so that the main kernel can fetch a
//                                    tile's 128 values with one aligned bulk copy, and zeroing of
//                                    the float32 dQ accumulator
//   2. attn_bwd_f16_kernel          one CTA per (batch*head, KV tile of 128 rows), KV-stationary:
//                                    walks the query tiles at or below its diagonal and keeps the
//                                    dK and dV accumulators in TMEM for the whole walk (no atomics,
//                                    bitwise reproducible); the per-tile dQ contribution is staged
//                                    through shared memory and added into the float32 accumulator
//                                    with bulk reduce-add copies (cp.reduce.async.bulk)
//   3. attn_bwd_dq_convert_kernel   dQ = f16(scale * accumulator)
//
// Inside the main kernel everything is computed transposed so that the tensor-core
// operands need no data movement:
//   S^T  = K Q^T   (A = K, B = Q, both K-major as TMA writes them)      -> TMEM
//   dP^T = V dO^T  (A = V, B = dO)                                       -> TMEM
//   thread r (= KV row r) turns row r of S^T into P^T, stored back into TMEM over S^T as f16
//   pairs, and row r of dP^T into dS^T = P^T * (dP^T - delta), an f16 K-major tile in shared memory
//   dV += P^T dO   (A = P^T from TMEM, B = dO MN-major)
//   dQ  = dS K     (A = dS^T read MN-major, B = K MN-major), overlaying the dP^T columns
//   dK += dS^T Q   (A = dS^T K-major, B = Q MN-major)
// Warp roles: warp 0 TMA producer, warp 1 MMA issuer, warps 2-9 two compute warpgroups that
// split the 128 query columns (and the head_dim columns of dQ/dK/dV) between them.  The MMA
// order S^T(i+1) -> dP^T(i+1) is issued while the warpgroups still reduce dQ(i), so the tensor
// core works on the next tile while the current one is being finished.
#include "sm100_ptx.cuh"
#include "tma_host.cuh"
#include <stdlib.h>

// Debug timeline (development aid): clock64() stamps of CTA 0's first iterations.
__device__ unsigned long long g_bwd_trace[16 * 3 * 8];
#define BWD_TRACE(role, ev)                                                                   \
    do {                                                                                      \
        if ((p.dbg & 2) && blockIdx.x == 0 && it < 16) g_bwd_trace[(it * 3 + (role)) * 8 + (ev)] = clock64(); \
    } while (0)

extern "C" __attribute__((visibility("default"))) int deers_b200_debug_bwd_trace(unsigned long long* out) {
    return (int)cudaMemcpyFromSymbol(out, g_bwd_trace, sizeof(g_bwd_trace));
}

namespace {
using namespace sm100;

constexpr int BT = 128;                        // tile rows for both Q and KV
constexpr uint32_t BLOCK_BYTES = 128 * 128;    // one 64-column block of a 128-row tile
constexpr float LOG2E = 1.4426950408889634f;

struct BwdParams {
    const float* lse2;          // [B*H][Tpad] lse * log2(e), 0 beyond T
    const float* delta;         // [B*H][Tpad] rowsum(dO * O), 0 beyond T
    float* dq_acc;              // [B*H][Tpad/128] tiles of 128 x D float32, in staging order
    __half* dk; __half* dv;
    long long sdk_b, sdk_h, sdk_t, sdv_b, sdv_h, sdv_t;
    int B, H, T, Tpad;
    int causal;
    float scale;
    unsigned int* err;
    int dbg;
};

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ void red_add_v4(float* addr, float a, float b, float c, float d) {
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d)
                 : "memory");
}

// 1-D bulk copy global -> shared, completion counted on an mbarrier (16-byte aligned, size % 16 == 0).
__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

// Shared-memory plan of the main kernel (dynamic shared memory only; the base must be
// 1024-byte aligned for the 128-byte swizzle, which the kernel verifies):
//   K, V            one tile each, resident for the CTA's whole walk
//   Q, dO           two stages each (the next query tile streams in while this one is used)
//   dS^T            128 x 128 f16, K-major
//   lse2, delta     two stages of 128 floats each
//   mbarriers, TMEM base, flags
template <int D>
struct BwdSmem {
    static constexpr uint32_t TILE = 128u * D * 2u;
    static constexpr uint32_t K = 0;
    static constexpr uint32_t V = K + TILE;
    static constexpr uint32_t Q = V + TILE;
    static constexpr uint32_t DO = Q + 2 * TILE;
    static constexpr uint32_t DS = DO + 2 * TILE;
    static constexpr uint32_t LSE2 = DS + 2 * BLOCK_BYTES;
    static constexpr uint32_t DELTA = LSE2 + 2 * BT * 4;
    static constexpr uint32_t BARS = DELTA + 2 * BT * 4;
    static constexpr uint32_t TOTAL = BARS + 256;
};

enum BwdBar { B_KV = 0, B_QDO_FULL = 1, B_QDO_EMPTY = 3, B_S = 5, B_DP = 6, B_P = 7, B_DS = 8, B_DQ = 9,
              B_DQ_READ = 10, B_DONE = 11, B_COUNT = 12 };

template <int D>
__global__ void __launch_bounds__(320, 1)
attn_bwd_f16_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                    const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_do,
                    const BwdParams p) {
    using L = BwdSmem<D>;
    constexpr uint32_t TILE_BYTES = L::TILE;
    constexpr int DBLK = D / 64;
    constexpr int DH = D / 2;                               // columns of dQ / dK / dV per compute warpgroup
    constexpr uint32_t TMEM_COLS = 512;
    // S^T (later P^T in place) | dP^T (later dQ in place) | dV | dK
    constexpr uint32_t TM_S = 0, TM_DP = 128, TM_DV = 256, TM_DK = 256 + D, TM_DQ = TM_DP;

    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t* sK = smem + L::K;
    uint8_t* sV = smem + L::V;
    uint8_t* sQ = smem + L::Q;
    uint8_t* sDO = smem + L::DO;
    uint8_t* sDS = smem + L::DS;
    float* lse2_s = reinterpret_cast<float*>(smem + L::LSE2);      // [2][BT]
    float* delta_s = reinterpret_cast<float*>(smem + L::DELTA);    // [2][BT]
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::BARS);
    uint32_t* tmem_base_s = reinterpret_cast<uint32_t*>(bars + B_COUNT);
    volatile uint32_t* abort_s = tmem_base_s + 1;
    uint32_t* skip_s = tmem_base_s + 2;

    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const int nq = (p.T + BT - 1) / BT;
    // Launch order: groups of 16 slices; inside a group the low KV tiles (most work) of all its
    // slices come first, and the group's Q, dO and dQ accumulator stay in L2 while it runs.
    const int BH = p.B * p.H;
    const int group = (int)(blockIdx.x / (16u * nq));
    const int gsize = min(16, BH - group * 16);
    const int within = (int)(blockIdx.x - (unsigned)group * 16u * nq);
    const int kt = within / gsize;
    const int bh = group * 16 + within % gsize;
    const int b = bh / p.H, h = bh % p.H;
    const int k0 = kt * BT;
    const int i0 = p.causal ? kt : 0;
    const int niter = nq - i0;

    if (threadIdx.x == 0) {
        *abort_s = 0;
        uint32_t skip = (*(volatile unsigned int*)p.err != 0) ? 1u : 0u;
        if ((smem_u32(smem) & 1023u) != 0) {                // swizzled tiles need a 1024-byte aligned base
            atomicCAS(p.err, 0u, DEERS_KERR_BWD_F16 | 0x20);
            skip = 1;
        }
        *skip_s = skip;
        mbar_init(&bars[B_KV], 1);
        for (int s = 0; s < 2; ++s) { mbar_init(&bars[B_QDO_FULL + s], 1); mbar_init(&bars[B_QDO_EMPTY + s], 1); }
        mbar_init(&bars[B_S], 1);
        mbar_init(&bars[B_DP], 1);
        mbar_init(&bars[B_P], 256);
        mbar_init(&bars[B_DS], 256);
        mbar_init(&bars[B_DQ], 1);
        mbar_init(&bars[B_DQ_READ], 256);
        mbar_init(&bars[B_DONE], 1);
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
            mbar_arrive_expect_tx(&bars[B_KV], 2 * TILE_BYTES);
#pragma unroll
            for (int blk = 0; blk < DBLK; ++blk) {
                tma_load_4d(sK + blk * BLOCK_BYTES, &tmap_k, &bars[B_KV], blk * 64, k0, h, b);
                tma_load_4d(sV + blk * BLOCK_BYTES, &tmap_v, &bars[B_KV], blk * 64, k0, h, b);
            }
            for (int it = 0; it < niter; ++it) {
                const int st = it & 1;
                const uint32_t ph = (uint32_t)(it >> 1) & 1u;
                if (!mbar_wait(ws, &bars[B_QDO_EMPTY + st], ph ^ 1u, DEERS_KERR_BWD_F16 | 1)) break;
                uint64_t* full = &bars[B_QDO_FULL + st];
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
            constexpr uint32_t IDESC_KV = idesc_f16(128, D, 0, 1);     // dV, dK: K-major A, MN-major B
            constexpr uint32_t IDESC_DQ = idesc_f16(128, D, 1, 1);     // dQ: MN-major A and B
            // Step-0 descriptors of every operand view, built once; each MMA adds a constant.
            const uint64_t k_km = desc_kmajor(smem_u32(sK), 0, BLOCK_BYTES), k_mn = desc_mnmajor(smem_u32(sK), 0, BLOCK_BYTES);
            const uint64_t v_km = desc_kmajor(smem_u32(sV), 0, BLOCK_BYTES);
            const uint64_t ds_km = desc_kmajor(smem_u32(sDS), 0, BLOCK_BYTES), ds_mn = desc_mnmajor(smem_u32(sDS), 0, BLOCK_BYTES);
            constexpr uint64_t STAGE_STEP = TILE_BYTES >> 4;           // next stage of Q / dO
            const uint64_t q_km0 = desc_kmajor(smem_u32(sQ), 0, BLOCK_BYTES), q_mn0 = desc_mnmajor(smem_u32(sQ), 0, BLOCK_BYTES);
            const uint64_t do_km0 = desc_kmajor(smem_u32(sDO), 0, BLOCK_BYTES), do_mn0 = desc_mnmajor(smem_u32(sDO), 0, BLOCK_BYTES);
            auto issue_st = [&](uint64_t q_km) {
#pragma unroll
                for (int ks = 0; ks < D / 16; ++ks)
                    umma_ss(tmem + TM_S, k_km + kmajor_step(ks, BLOCK_BYTES), q_km + kmajor_step(ks, BLOCK_BYTES), IDESC_ST, ks > 0);
                umma_commit(&bars[B_S]);
            };
            auto issue_dpt = [&](uint64_t do_km) {
#pragma unroll
                for (int ks = 0; ks < D / 16; ++ks)
                    umma_ss(tmem + TM_DP, v_km + kmajor_step(ks, BLOCK_BYTES), do_km + kmajor_step(ks, BLOCK_BYTES), IDESC_ST, ks > 0);
                umma_commit(&bars[B_DP]);
            };
            bool ok = mbar_wait(ws, &bars[B_KV], 0, DEERS_KERR_BWD_F16 | 2) &&
                      mbar_wait(ws, &bars[B_QDO_FULL], 0, DEERS_KERR_BWD_F16 | 3);
            if (ok) {
                tc_fence_after_sync();
                issue_st(q_km0);
                issue_dpt(do_km0);
            }
            for (int it = 0; ok && it < niter; ++it) {
                const int st = it & 1;
                const uint32_t par = (uint32_t)it & 1u;
                const uint64_t q_mn = q_mn0 + (uint64_t)st * STAGE_STEP, do_mn = do_mn0 + (uint64_t)st * STAGE_STEP;
                // dV += P^T dO: P^T sits in TMEM where S^T was, 32 packed columns per warpgroup half.
                BWD_TRACE(0, 0);
                if (!mbar_wait(ws, &bars[B_P], par, DEERS_KERR_BWD_F16 | 4)) break;
                tc_fence_after_sync();
                BWD_TRACE(0, 1);
#pragma unroll
                for (int ks = 0; ks < BT / 16; ++ks)
                    umma_ts(tmem + TM_DV, tmem + TM_S + (uint32_t)(ks >> 2) * 64u + (uint32_t)(ks & 3) * 8u,
                            do_mn + mnmajor_step(ks), IDESC_KV, (it > 0 || ks > 0));
                // S^T of the next query tile follows dV in the (in-order) pipe, which has consumed P^T.
                if (it + 1 < niter) {
                    const int sn = (it + 1) & 1;
                    BWD_TRACE(0, 2);
                    if (!mbar_wait(ws, &bars[B_QDO_FULL + sn], (uint32_t)((it + 1) >> 1) & 1u, DEERS_KERR_BWD_F16 | 6)) break;
                    tc_fence_after_sync();
                    issue_st(q_km0 + (uint64_t)sn * STAGE_STEP);
                }
                // dK += dS^T Q, then dQ = dS K over the consumed dP^T columns.
                BWD_TRACE(0, 3);
                if (!mbar_wait(ws, &bars[B_DS], par, DEERS_KERR_BWD_F16 | 5)) break;
                tc_fence_after_sync();
                BWD_TRACE(0, 4);
#pragma unroll
                for (int ks = 0; ks < BT / 16; ++ks)
                    umma_ss(tmem + TM_DK, ds_km + kmajor_step(ks, BLOCK_BYTES), q_mn + mnmajor_step(ks), IDESC_KV, (it > 0 || ks > 0));
#pragma unroll
                for (int ks = 0; ks < BT / 16; ++ks)
                    umma_ss(tmem + TM_DQ, ds_mn + mnmajor_step(ks), k_mn + mnmajor_step(ks), IDESC_DQ, ks > 0);
                umma_commit(&bars[B_DQ]);                               // dS^T in shared memory is free again, dQ is ready
                umma_commit(&bars[B_QDO_EMPTY + st]);
                if (it + 1 < niter) {
                    BWD_TRACE(0, 5);
                    if (!mbar_wait(ws, &bars[B_DQ_READ], par, DEERS_KERR_BWD_F16 | 7)) break;
                    tc_fence_after_sync();
                    BWD_TRACE(0, 6);
                    issue_dpt(do_km0 + (uint64_t)((it + 1) & 1) * STAGE_STEP);
                }
            }
            umma_commit(&bars[B_DONE]);
        }
    } else {
        // ------------------------------ compute threads ------------------------------
        // Two warpgroups; warpgroup g owns query columns [64g, 64g+64) of S^T / dP^T and columns
        // [g*D/2, (g+1)*D/2) of dQ, dK and dV.  Thread r of a warpgroup owns TMEM lane r.
        const int g = (warp - 2) >> 2;
        const int lane_base = (warp & 3) * 32;
        const int r = lane_base + lane;                     // KV row inside the tile (S^T, dK, dV); query row for dQ
        const uint32_t t_lane = (uint32_t)lane_base << 16;
        const float sl2 = p.scale * LOG2E;
        const bool kv_valid = (k0 + r) < p.T;               // rows past the sequence end contribute nothing
        bool alive = true;

        // dQ tile of iteration j: TMEM -> this thread's (idle) dS^T row slot in shared memory ->
        // one 4 KB bulk reduce-add per warp into the float32 accumulator, 32 columns per round.
        // The accumulator is stored tile by tile in exactly the staged order
        // [warpgroup][round][warp][32 rows][32 floats, 16-byte chunks XOR-swizzled by row & 7].
        uint8_t* my_slot = sDS + (uint32_t)g * BLOCK_BYTES + (uint32_t)r * 128u;
        uint8_t* warp_slot = sDS + (uint32_t)g * BLOCK_BYTES + (uint32_t)lane_base * 128u;
        auto dq_phase = [&](int j) -> bool {
            const int it = j;
            if (!__all_sync(0xffffffffu, mbar_wait(ws, &bars[B_DQ], (uint32_t)j & 1u, DEERS_KERR_BWD_F16 | 11))) return false;
            tc_fence_after_sync();
            if (lane == 0 && (warp == 2 || warp == 6)) BWD_TRACE(1 + g, 5);
            constexpr int ROUNDS = DH / 32;
            float* tile = p.dq_acc + ((long long)bh * nq + (i0 + j)) * (long long)(BT * D);
#pragma unroll
            for (int rnd = 0; rnd < ROUNDS; ++rnd) {
                uint32_t qr[32];
                tmem_ld_x32(tmem + TM_DQ + t_lane + g * DH + rnd * 32, qr);
                tmem_wait_ld();
                if (rnd > 0 && !(p.dbg & 4)) {
                    if (lane == 0) bulk_wait_group_read<0>();
                    __syncwarp();
                }
                if (!(p.dbg & 1)) {
#pragma unroll
                    for (int ch = 0; ch < 8; ++ch)
                        *reinterpret_cast<uint4*>(my_slot + ((ch ^ (r & 7)) << 4)) =
                            make_uint4(qr[ch * 4], qr[ch * 4 + 1], qr[ch * 4 + 2], qr[ch * 4 + 3]);
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) {
                        bulk_reduce_add_f32(tile + ((g * ROUNDS + rnd) * 4 + (warp & 3)) * 1024, warp_slot, 4096);
                        bulk_commit_group();
                    }
                }
            }
            tc_fence_before_sync();
            mbar_arrive(&bars[B_DQ_READ]);
            // The slot is written again by the next dS^T: the bulk engine must have read it.
            if (lane == 0 && !(p.dbg & 4)) bulk_wait_group_read<0>();
            __syncwarp();
            if (lane == 0 && (warp == 2 || warp == 6)) BWD_TRACE(1 + g, 6);
            return true;
        };

        for (int it = 0; it < niter; ++it) {
            const int i = i0 + it;
            const int q0 = i * BT;
            const int st = it & 1;
            const uint32_t par = (uint32_t)it & 1u;
            const float* lse2 = lse2_s + st * BT + 64 * g;
            const float* dlt = delta_s + st * BT + 64 * g;
            // The stage's lse / delta rows arrive with Q and dO: observe that barrier directly.
            if (!__all_sync(0xffffffffu, mbar_wait(ws, &bars[B_QDO_FULL + st], (uint32_t)(it >> 1) & 1u, DEERS_KERR_BWD_F16 | 8))) { alive = false; break; }
            const bool tr = lane == 0 && (warp == 2 || warp == 6);
            if (tr) BWD_TRACE(1 + g, 0);
            if (!__all_sync(0xffffffffu, mbar_wait(ws, &bars[B_S], par, DEERS_KERR_BWD_F16 | 9))) { alive = false; break; }
            tc_fence_after_sync();
            if (tr) BWD_TRACE(1 + g, 1);
            const bool diag = p.causal && (i == kt);
            uint32_t pk[32];                                // P^T row, 64 query columns as f16 pairs
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                uint32_t sr[32];
                tmem_ld_x32(tmem + TM_S + t_lane + 64 * g + c * 32, sr);
                tmem_wait_ld();
                if (diag || !kv_valid) {                        // warp-uniform except for the tail tile
#pragma unroll
                    for (int e = 0; e < 16; ++e) {
                        const int cl = c * 32 + e * 2;          // column inside this warpgroup's half
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
            // P^T replaces this warpgroup's half of S^T in TMEM (32 packed columns) for dV += P^T dO.
            tmem_st_x32(tmem + TM_S + t_lane + 64 * g, pk);
            tmem_wait_st();
            tc_fence_before_sync();
            mbar_arrive(&bars[B_P]);
            if (tr) BWD_TRACE(1 + g, 2);

            // The previous tile's dQ leaves while the tensor core works on this tile's products.
            if (it > 0 && !dq_phase(it - 1)) { alive = false; break; }

            if (!__all_sync(0xffffffffu, mbar_wait(ws, &bars[B_DP], par, DEERS_KERR_BWD_F16 | 10))) { alive = false; break; }
            tc_fence_after_sync();
            if (tr) BWD_TRACE(1 + g, 3);
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                uint32_t dr[32];
                tmem_ld_x32(tmem + TM_DP + t_lane + 64 * g + c * 32, dr);
                tmem_wait_ld();
                uint32_t dd[16];
#pragma unroll
                for (int e = 0; e < 16; ++e) {
                    const int cl = c * 32 + e * 2;
                    const float2 pf = __half22float2(*reinterpret_cast<const __half2*>(&pk[c * 16 + e]));
                    dd[e] = pack_half2(pf.x * (__uint_as_float(dr[e * 2]) - dlt[cl]),
                                       pf.y * (__uint_as_float(dr[e * 2 + 1]) - dlt[cl + 1]));
                }
                // 32 query columns = 4 chunks of 8 f16 inside column block g of the dS^T tile.
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4)
                    *reinterpret_cast<uint4*>(sDS + (uint32_t)g * BLOCK_BYTES + sw128_chunk_offset(r, c * 4 + q4)) =
                        make_uint4(dd[q4 * 4], dd[q4 * 4 + 1], dd[q4 * 4 + 2], dd[q4 * 4 + 3]);
            }
            fence_proxy_async_smem();
            tc_fence_before_sync();
            mbar_arrive(&bars[B_DS]);
            if (tr) BWD_TRACE(1 + g, 4);

        }
        if (alive) alive = dq_phase(niter - 1);
        if (lane == 0) bulk_wait_group_read<0>();

        if (alive && __all_sync(0xffffffffu, mbar_wait(ws, &bars[B_DONE], 0, DEERS_KERR_BWD_F16 | 12))) {
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
#pragma unroll
                    for (int q8 = 0; q8 < 4; ++q8) {
                        uint4 a, bq;
                        a.x = pack_half2(__uint_as_float(kr[q8 * 8 + 0]) * p.scale, __uint_as_float(kr[q8 * 8 + 1]) * p.scale);
                        a.y = pack_half2(__uint_as_float(kr[q8 * 8 + 2]) * p.scale, __uint_as_float(kr[q8 * 8 + 3]) * p.scale);
                        a.z = pack_half2(__uint_as_float(kr[q8 * 8 + 4]) * p.scale, __uint_as_float(kr[q8 * 8 + 5]) * p.scale);
                        a.w = pack_half2(__uint_as_float(kr[q8 * 8 + 6]) * p.scale, __uint_as_float(kr[q8 * 8 + 7]) * p.scale);
                        bq.x = pack_half2(__uint_as_float(vr[q8 * 8 + 0]), __uint_as_float(vr[q8 * 8 + 1]));
                        bq.y = pack_half2(__uint_as_float(vr[q8 * 8 + 2]), __uint_as_float(vr[q8 * 8 + 3]));
                        bq.z = pack_half2(__uint_as_float(vr[q8 * 8 + 4]), __uint_as_float(vr[q8 * 8 + 5]));
                        bq.w = pack_half2(__uint_as_float(vr[q8 * 8 + 6]), __uint_as_float(vr[q8 * 8 + 7]));
                        *reinterpret_cast<uint4*>(dkrow + c * 32 + q8 * 8) = a;
                        *reinterpret_cast<uint4*>(dvrow + c * 32 + q8 * 8) = bq;
                    }
                }
            }
        }
    }

    __syncwarp();
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem, TMEM_COLS);
}

// delta[row] = sum_d dO[row][d] * O[row][d] and lse2[row] = lse[row] * log2(e) on the padded
// [B*H][Tpad] grid (0 beyond T); also clears the row of the dQ accumulator.  One warp per row.
template <int D>
__global__ void __launch_bounds__(256)
attn_bwd_prep_f16_kernel(const __half* __restrict__ o, const __half* __restrict__ d_o, const float* __restrict__ lse,
                         float* __restrict__ delta, float* __restrict__ lse2, float* __restrict__ dq_acc, int B, int H,
                         int T, int Tpad, long long so_b, long long so_h, long long so_t, long long sdo_b,
                         long long sdo_h, long long sdo_t) {
    const long long row = (long long)blockIdx.x * 8 + threadIdx.x / 32;
    const int lane = threadIdx.x % 32;
    if (row >= (long long)B * H * Tpad) return;
    const int t = (int)(row % Tpad);
    const int bh = (int)(row / Tpad);
    constexpr int PER = D / 32;                              // 2 or 4 elements per lane
    float* acc = dq_acc + row * D + lane * PER;
#pragma unroll
    for (int e = 0; e < PER; ++e) acc[e] = 0.f;
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

template <int D>
__global__ void __launch_bounds__(256)
attn_bwd_dq_convert_kernel(const float* __restrict__ dq_acc, __half* __restrict__ dq, int B, int H, int T, int Tpad,
                           float scale, long long s_b, long long s_h, long long s_t) {
    // One thread per 8 consecutive elements of a row.
    constexpr int VEC = D / 8;
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long total = (long long)B * H * T * VEC;
    if (idx >= total) return;
    const int v = (int)(idx % VEC);
    const long long row = idx / VEC;
    const int t = (int)(row % T);
    const int bh = (int)(row / T);
    const int b = bh / H, h = bh % H;
    // The accumulator is tiled the way the main kernel stages it:
    // [slice][query tile][warpgroup][round][warp][32 rows][32 floats, chunks XOR-swizzled by row & 7].
    constexpr int DH = D / 2, ROUNDS = DH / 32;
    const int nq = Tpad / 128;
    const int i = t / 128, r = t % 128, wq = r / 32, ln = r % 32;
    const int d0 = v * 8;
    const int g = d0 / DH, rnd = (d0 % DH) / 32, ch = (d0 % 32) / 4;
    const float* base = dq_acc + ((long long)bh * nq + i) * (long long)(128 * D) +
                        ((g * ROUNDS + rnd) * 4 + wq) * 1024 + ln * 32;
    const float4 x = *reinterpret_cast<const float4*>(base + ((ch ^ (ln & 7)) << 2));
    const float4 y = *reinterpret_cast<const float4*>(base + (((ch + 1) ^ (ln & 7)) << 2));
    uint4 outv;
    outv.x = pack_half2(x.x * scale, x.y * scale);
    outv.y = pack_half2(x.z * scale, x.w * scale);
    outv.z = pack_half2(y.x * scale, y.y * scale);
    outv.w = pack_half2(y.z * scale, y.w * scale);
    *reinterpret_cast<uint4*>(dq + b * s_b + h * s_h + (long long)t * s_t + v * 8) = outv;
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
    float* dq_acc = (float*)((char*)workspace + 2 * stat_bytes);

    const long long prep_rows = BH * Tpad;
    {
        KernelTimerScope ts(ctx, DEERS_K_BWD_PREP);
        attn_bwd_prep_f16_kernel<D><<<(unsigned)((prep_rows + 7) / 8), 256, 0, ctx->stream>>>(
            (const __half*)o, (const __half*)d_o, lse, delta, lse2, dq_acc, d->B, d->H, d->T, Tpad, d->o_strides[0],
            d->o_strides[1], d->o_strides[2], d->do_strides[0], d->do_strides[1], d->do_strides[2]);
    }
    DEERS_CUDA_TRY(ctx, cudaGetLastError());

    BwdParams p;
    p.lse2 = lse2; p.delta = delta; p.dq_acc = dq_acc;
    p.dk = (__half*)dk; p.dv = (__half*)dv;
    p.sdk_b = d->dk_strides[0]; p.sdk_h = d->dk_strides[1]; p.sdk_t = d->dk_strides[2];
    p.sdv_b = d->dv_strides[0]; p.sdv_h = d->dv_strides[1]; p.sdv_t = d->dv_strides[2];
    p.B = d->B; p.H = d->H; p.T = d->T; p.Tpad = Tpad; p.causal = d->causal; p.scale = d->scale;
    p.err = ctx->dev_err;
    p.dbg = getenv("DEERS_DBG") ? atoi(getenv("DEERS_DBG")) : 0;
    const size_t smem = BwdSmem<D>::TOTAL;
    DEERS_CUDA_TRY(ctx, cudaFuncSetAttribute(attn_bwd_f16_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const long long grid = BH * nq;
    if (grid > 0x7fffffffLL) return DEERS_ERR_SHAPE;
    {
        KernelTimerScope ts(ctx, DEERS_K_BWD_MAIN);
        attn_bwd_f16_kernel<D><<<(unsigned)grid, 320, smem, ctx->stream>>>(tq, tk, tv, tdo, p);
    }
    DEERS_CUDA_TRY(ctx, cudaGetLastError());

    const long long total = BH * d->T * (D / 8);
    {
        KernelTimerScope ts(ctx, DEERS_K_BWD_DQ);
        attn_bwd_dq_convert_kernel<D><<<(unsigned)((total + 255) / 256), 256, 0, ctx->stream>>>(
            dq_acc, (__half*)dq, d->B, d->H, d->T, Tpad, d->scale, d->dq_strides[0], d->dq_strides[1], d->dq_strides[2]);
    }
    DEERS_CUDA_TRY(ctx, cudaGetLastError());
    ctx->launches += 3;
    return DEERS_OK;
}

}  // namespace

// Workspace: delta [B*H][Tpad] | lse*log2e [B*H][Tpad] | dQ accumulator [B*H][Tpad][D], all float32.
size_t attn_bwd_f16_workspace_bytes(const deers_attn_desc* d) {
    const size_t Tpad = (size_t)((d->T + BT - 1) / BT) * BT;
    return 2 * bwd_stat_bytes(d) + (size_t)d->B * d->H * Tpad * d->D * sizeof(float);
}

int launch_attn_bwd_f16(deers_ctx* ctx, const deers_attn_desc* d, const void* q, const void* k, const void* v,
                        const void* o, const float* lse, const void* d_o, void* dq, void* dk, void* dv,
                        void* workspace) {
    if (d->D == 64) return bwd_launch<64>(ctx, d, q, k, v, o, lse, d_o, dq, dk, dv, workspace);
    if (d->D == 128) return bwd_launch<128>(ctx, d, q, k, v, o, lse, d_o, dq, dk, dv, workspace);
    return DEERS_ERR_UNSUPPORTED;
}
