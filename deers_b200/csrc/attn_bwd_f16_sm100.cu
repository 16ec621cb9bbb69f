// f16 causal attention backward for sm_100a.
//
// Three launches, none of which uses atomics, so dQ, dK and dV are bitwise reproducible:
//   1. attn_bwd_prep_f16_kernel   delta[row] = sum_d dO*O (= rowsum(dP*P)) and lse*log2(e), both
//                                  padded to whole 128-row tiles so that the main kernels can
//                                  fetch a tile's values with one aligned bulk copy
//   2. attn_bwd_dkdv_f16_kernel   per (batch*head, KV tile of 128 rows), KV-stationary: walks the
//                                  query tiles at or below the diagonal with the dK and dV
//                                  accumulators resident in TMEM for the whole walk
//   3. attn_bwd_dq_f16_kernel     per (batch*head, query tile of 128 rows), Q-stationary: walks the
//                                  KV tiles at or left of the diagonal with the dQ accumulator
//                                  resident in TMEM
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
// Both kernels are persistent (one CTA per SM walking a strided list of tiles), so that the
// loads and first products of the next tile overlap the tail and the epilogue of the current one.
#include "sm100_ptx.cuh"
#include "tma_host.cuh"


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
    const int4* sched;          // balanced schedule table[n * grid + cta] = {slot, slice, batch, head} (or nullptr: strided)
    int sched_rows;
    // dS^T tiles kept between the two main kernels (nullptr: the dQ kernel recomputes S and dP instead).
    // Tile (slice, query tile i, KV tile j) is 32 KB at ((slice * ds_pairs + pair(i, j)) << 15): two blocks of
    // 128 KV rows x 64 query columns in the 128-byte-swizzled shared-memory image the tensor core reads.
    __half* ds;
    long long ds_pairs;         // tiles per slice: nq (nq + 1) / 2 causal, nq * nq otherwise
};

// Index of tile (query tile i, KV tile j) among its slice's dS^T tiles: all KV tiles of a query tile are adjacent.
__device__ __forceinline__ long long ds_pair(const BwdParams& p, int i, int j, int nq) {
    return p.causal ? (long long)i * (i + 1) / 2 + j : (long long)i * nq + j;
}

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

// The same with an L2 eviction-priority hint (a createpolicy value) for data that is read exactly once.
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}
__device__ __forceinline__ void bulk_load_hint(void* dst, const void* src, uint32_t bytes, uint64_t* bar, uint64_t pol) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
                 ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)), "l"(pol)
                 : "memory");
}

// Work order shared by both kernels: groups of 16 slices; inside a group the heaviest tiles
// of all its slices come first (balance) and the group's tensors (a few MB) stay in L2.
// Work item w -> (slot, slice); slot 0 is the heaviest tile of the slice.
__device__ __forceinline__ void item_tile(int B, int H, int ntile, int w, int& slot, int& bh) {
    const int BH = B * H;
    const int group = w / (16 * ntile);
    const int gsize = min(16, BH - group * 16);
    const int within = w - group * 16 * ntile;
    slot = within / gsize;
    bh = group * 16 + within % gsize;
}

// n-th work item of this CTA as {slot, slice, batch, head}; slot < 0 when its list is exhausted.  Callers
// fetch item n+1 when item n starts, so the table read (an L2 round trip) is never waited for at an item
// boundary; the table spares the single issuing threads the integer divisions of item_tile.
__device__ __forceinline__ int4 next_item(const BwdParams& p, int n, int n_items, int ntile) {
    if (p.sched) return n < p.sched_rows ? p.sched[n * (int)gridDim.x + (int)blockIdx.x] : make_int4(-1, 0, 0, 0);
    const int w = (int)blockIdx.x + n * (int)gridDim.x;
    if (w >= n_items) return make_int4(-1, 0, 0, 0);
    int slot, bh;
    item_tile(p.B, p.H, ntile, w, slot, bh);
    return make_int4(slot, bh, bh / p.H, bh % p.H);
}

// ---------------------------------------------------------------------------------------------
// dK / dV kernel (persistent: each CTA walks a strided list of KV tiles)
// ---------------------------------------------------------------------------------------------
// Dynamic shared memory only; the base must be 1024-byte aligned for the 128-byte swizzle (checked).
template <int D>
struct DkvSmem {
    static constexpr uint32_t TILE = 128u * D * 2u;
    static constexpr uint32_t K = 0;
    static constexpr uint32_t V = K + TILE;
    static constexpr uint32_t Q = V + TILE;                  // three stages: Q(i+1) feeds S^T while Q(i) still feeds dK
    static constexpr uint32_t DO = Q + 3 * TILE;             // two stages
    static constexpr uint32_t LSE2 = DO + 2 * TILE;          // two stages of 128 floats
    static constexpr uint32_t DELTA = LSE2 + 2 * BT * 4;
    static constexpr uint32_t BARS = DELTA + 2 * BT * 4;
    static constexpr uint32_t TOTAL = BARS + 192;
};

enum DkvBar { A_KV_FULL = 0, A_KV_EMPTY = 1, A_Q_FULL = 2, A_Q_EMPTY = 5, A_DO_FULL = 8, A_DO_EMPTY = 10,
              A_ST_FULL = 12, A_ST_EMPTY = 14, A_S = 16, A_DP = 17, A_P = 18, A_DS = 19, A_DONE = 20, A_ACC_FREE = 21,
              A_COUNT = 22 };

// Compute warpgroups of the dK / dV kernel: each owns 128 / DKV_NWG query columns of S^T / dP^T and
// D / DKV_NWG columns of dK and dV.  Four (four warps per scheduler) measure 3 % faster than two on the same
// GPU (6.36 against 6.56 ms at B64 H32 T2048 D128, both power-capped near 1.47 GHz).
constexpr int DKV_NWG = 4;
constexpr int DKV_THREADS = 64 + 128 * DKV_NWG;

__device__ __forceinline__ void tmem_ld(uint32_t taddr, uint32_t (&r)[32]) { tmem_ld_x32(taddr, r); }
__device__ __forceinline__ void tmem_ld(uint32_t taddr, uint32_t (&r)[16]) { tmem_ld_x16(taddr, r); }
__device__ __forceinline__ void tmem_st(uint32_t taddr, const uint32_t (&r)[32]) { tmem_st_x32(taddr, r); }
__device__ __forceinline__ void tmem_st(uint32_t taddr, const uint32_t (&r)[16]) { tmem_st_x16(taddr, r); }

template <int D>
__global__ void __launch_bounds__(DKV_THREADS, 1)
attn_bwd_dkdv_f16_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                         const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_do,
                         const BwdParams p) {
    using L = DkvSmem<D>;
    constexpr uint32_t TILE_BYTES = L::TILE;
    constexpr int DBLK = D / 64;
    constexpr int NWG = DKV_NWG;
    constexpr int NCT = 128 * NWG;                          // compute threads
    constexpr int CW = BT / NWG;                            // query columns of S^T / dP^T per compute warpgroup
    constexpr int DH = D / NWG;                             // output columns per compute warpgroup
    constexpr int EC = DH < 32 ? DH : 32;                   // columns per TMEM load in the epilogue
    static_assert(CW % 32 == 0 && (DH == 16 || DH % 32 == 0), "unsupported warpgroup split");
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
    const int n_items = p.B * p.H * nq;

    if (threadIdx.x == 0) {
        *abort_s = 0;
        uint32_t skip = (*(volatile unsigned int*)p.err != 0) ? 1u : 0u;   // an earlier CTA gave up
        if ((smem_u32(smem) & 1023u) != 0) {
            atomicCAS(p.err, 0u, DEERS_KERR_BWD_F16 | 0x20);
            skip = 1;
        }
        *skip_s = skip;
        mbar_init(&bars[A_KV_FULL], 1);
        mbar_init(&bars[A_KV_EMPTY], 1);
        for (int s = 0; s < 3; ++s) { mbar_init(&bars[A_Q_FULL + s], 1); mbar_init(&bars[A_Q_EMPTY + s], 1); }
        for (int s = 0; s < 2; ++s) {
            mbar_init(&bars[A_DO_FULL + s], 1); mbar_init(&bars[A_DO_EMPTY + s], 1);
            mbar_init(&bars[A_ST_FULL + s], NCT);
        }
        mbar_init(&bars[A_S], 1);
        mbar_init(&bars[A_DP], 1);
        mbar_init(&bars[A_P], NCT);
        mbar_init(&bars[A_DS], NCT);
        mbar_init(&bars[A_DONE], 1);
        mbar_init(&bars[A_ACC_FREE], NCT);
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
            uint32_t gi = 0;                                    // query-tile iterations so far (all items)
            bool ok = true;
            for (int4 cur = next_item(p, 0, n_items, nq), nxt = next_item(p, 1, n_items, nq), n4 = make_int4(0, 0, 0, 0); ok && cur.x >= 0;
                     ++n4.x, cur = nxt, nxt = next_item(p, n4.x + 1, n_items, nq)) {
                const int n = n4.x, kt = cur.x, bh = cur.y;
                const int b = cur.z, h = cur.w;
                const int i0 = p.causal ? kt : 0;
                const int niter = nq - i0;
                // K / V are single-buffered: wait until the previous item's S^T and dP^T products are done.
                if (!mbar_wait(ws, &bars[A_KV_EMPTY], ((uint32_t)n & 1u) ^ 1u, DEERS_KERR_BWD_F16 | 1)) break;
                mbar_arrive_expect_tx(&bars[A_KV_FULL], 2 * TILE_BYTES);
#pragma unroll
                for (int blk = 0; blk < DBLK; ++blk) {
                    tma_load_4d(sK + blk * BLOCK_BYTES, &tmap_k, &bars[A_KV_FULL], blk * 64, kt * BT, h, b);
                    tma_load_4d(sV + blk * BLOCK_BYTES, &tmap_v, &bars[A_KV_FULL], blk * 64, kt * BT, h, b);
                }
                for (int it = 0; it < niter; ++it, ++gi) {
                    const uint32_t qs = gi % 3u, ds = gi & 1u;
                    const int q0 = (i0 + it) * BT;
                    if (!mbar_wait(ws, &bars[A_Q_EMPTY + qs], ((gi / 3u) & 1u) ^ 1u, DEERS_KERR_BWD_F16 | 2)) { ok = false; break; }
                    mbar_arrive_expect_tx(&bars[A_Q_FULL + qs], TILE_BYTES);
#pragma unroll
                    for (int blk = 0; blk < DBLK; ++blk)
                        tma_load_4d(sQ + qs * TILE_BYTES + blk * BLOCK_BYTES, &tmap_q, &bars[A_Q_FULL + qs], blk * 64, q0, h, b);
                    if (!mbar_wait(ws, &bars[A_DO_EMPTY + ds], ((gi >> 1) & 1u) ^ 1u, DEERS_KERR_BWD_F16 | 4)) { ok = false; break; }
                    mbar_arrive_expect_tx(&bars[A_DO_FULL + ds], TILE_BYTES);
#pragma unroll
                    for (int blk = 0; blk < DBLK; ++blk)
                        tma_load_4d(sDO + ds * TILE_BYTES + blk * BLOCK_BYTES, &tmap_do, &bars[A_DO_FULL + ds], blk * 64, q0, h, b);
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
            auto issue_st = [&](uint32_t qs) {
                const uint64_t q_km = q_km0 + (uint64_t)qs * STAGE_STEP;
#pragma unroll
                for (int ks = 0; ks < D / 16; ++ks)
                    umma_ss(tmem + TM_S, k_km + kmajor_step(ks, BLOCK_BYTES), q_km + kmajor_step(ks, BLOCK_BYTES), IDESC_ST, ks > 0);
                umma_commit(&bars[A_S]);
            };
            auto issue_dpt = [&](uint32_t ds) {
                const uint64_t do_km = do_km0 + (uint64_t)ds * STAGE_STEP;
#pragma unroll
                for (int ks = 0; ks < D / 16; ++ks)
                    umma_ss(tmem + TM_DP, v_km + kmajor_step(ks, BLOCK_BYTES), do_km + kmajor_step(ks, BLOCK_BYTES), IDESC_ST, ks > 0);
                umma_commit(&bars[A_DP]);
            };
            // A operand in TMEM: CW / 2 packed columns per compute warpgroup, the groups CW columns apart.
            auto a_tmem = [&](uint32_t base, int ks) {
                return tmem + base + (uint32_t)(ks / (CW / 16)) * (uint32_t)CW + (uint32_t)(ks % (CW / 16)) * 8u;
            };
            uint32_t gi = 0;
            bool ok = true;
            for (int4 cur = next_item(p, 0, n_items, nq), nxt = next_item(p, 1, n_items, nq), n4 = make_int4(0, 0, 0, 0); ok && cur.x >= 0;
                     ++n4.x, cur = nxt, nxt = next_item(p, n4.x + 1, n_items, nq)) {
                const int n = n4.x, kt = cur.x, bh = cur.y;
                const int niter = nq - (p.causal ? kt : 0);
                if (!mbar_wait(ws, &bars[A_KV_FULL], (uint32_t)n & 1u, DEERS_KERR_BWD_F16 | 5)) break;
                if (!mbar_wait(ws, &bars[A_Q_FULL + gi % 3u], (gi / 3u) & 1u, DEERS_KERR_BWD_F16 | 6)) break;
                if (!mbar_wait(ws, &bars[A_DO_FULL + (gi & 1u)], (gi >> 1) & 1u, DEERS_KERR_BWD_F16 | 7)) break;
                tc_fence_after_sync();
                issue_st(gi % 3u);
                issue_dpt(gi & 1u);
                if (niter == 1) umma_commit(&bars[A_KV_EMPTY]);         // no further product reads K / V
                for (int it = 0; it < niter; ++it, ++gi) {
                    const uint32_t qs = gi % 3u, ds = gi & 1u, par = gi & 1u;
                    const uint64_t q_mn = q_mn0 + (uint64_t)qs * STAGE_STEP, do_mn = do_mn0 + (uint64_t)ds * STAGE_STEP;
                    const bool more = it + 1 < niter;
                    // dV += P^T dO, then S^T of the next query tile: the pipe is in order, so the
                    // new S^T lands only after dV has consumed P^T from the same columns.
                    if (!mbar_wait(ws, &bars[A_P], par, DEERS_KERR_BWD_F16 | 8)) { ok = false; break; }
                    // The previous item's dK / dV must have left TMEM before this item accumulates.
                    if (it == 0 && !mbar_wait(ws, &bars[A_ACC_FREE], ((uint32_t)n & 1u) ^ 1u, DEERS_KERR_BWD_F16 | 9)) { ok = false; break; }
                    tc_fence_after_sync();
#pragma unroll
                    for (int ks = 0; ks < BT / 16; ++ks)
                        umma_ts(tmem + TM_DV, a_tmem(TM_S, ks), do_mn + mnmajor_step(ks), IDESC_KV, (it > 0 || ks > 0));
                    if (more) {
                        if (!mbar_wait(ws, &bars[A_Q_FULL + (gi + 1u) % 3u], ((gi + 1u) / 3u) & 1u, DEERS_KERR_BWD_F16 | 10)) { ok = false; break; }
                        tc_fence_after_sync();
                        issue_st((gi + 1u) % 3u);
                    }
                    // dK += dS^T Q, then dP^T of the next query tile over the consumed dS^T columns.
                    if (!mbar_wait(ws, &bars[A_DS], par, DEERS_KERR_BWD_F16 | 11)) { ok = false; break; }
                    tc_fence_after_sync();
#pragma unroll
                    for (int ks = 0; ks < BT / 16; ++ks)
                        umma_ts(tmem + TM_DK, a_tmem(TM_DP, ks), q_mn + mnmajor_step(ks), IDESC_KV, (it > 0 || ks > 0));
                    umma_commit(&bars[A_Q_EMPTY + qs]);                 // S^T and dK have both read this Q tile
                    if (more) {
                        if (!mbar_wait(ws, &bars[A_DO_FULL + (ds ^ 1u)], ((gi + 1u) >> 1) & 1u, DEERS_KERR_BWD_F16 | 12)) { ok = false; break; }
                        tc_fence_after_sync();
                        issue_dpt(ds ^ 1u);
                        if (it + 2 == niter) umma_commit(&bars[A_KV_EMPTY]);   // the last S^T and dP^T are issued
                    }
                    // dO of this iteration was last read by dV (and dP^T before it): its stage is free once
                    // everything issued so far has finished.
                    umma_commit(&bars[A_DO_EMPTY + ds]);
                }
                umma_commit(&bars[A_DONE]);
            }
        }
    } else {
        // ------------------------------ compute threads ------------------------------
        // Warpgroup g owns query columns [CW*g, CW*g+CW) of S^T / dP^T and columns
        // [g*DH, (g+1)*DH) of dK and dV.  Thread r of a warpgroup owns TMEM lane r = KV row r.
        const int g = (warp - 2) >> 2;
        const int lane_base = (warp & 3) * 32;
        const int r = lane_base + lane;
        const uint32_t t_lane = (uint32_t)lane_base << 16;
        const float sl2 = p.scale * LOG2E;
        uint32_t gi = 0;
        bool alive = true;
        // The 128 lse * log2e and the 128 delta values of a query tile are staged in shared memory by the compute
        // threads themselves: thread ct < 256 fetches element ct of the NEXT iteration's 256 values one iteration
        // ahead (a plain global load, in flight during this iteration's products) and stores it at the top of that
        // iteration; every compute thread then arrives on the stage's barrier and waits for all before reading.  A stage is
        // rewritten two iterations after it was read, and nobody gets there before all threads have passed the
        // barrier of the iteration in between, i.e. have finished reading.  (An earlier version had the producer
        // warp bring these rows in with bulk copies; repeated full-size runs then showed, once in a few dozen, one
        // warp seeing a stale 32-byte piece of the delta row in the first iteration of an item.)
        const int ct = (warp - 2) * 32 + lane;
        const bool stager = ct < 2 * BT;
        const float* stat_src = (ct < BT) ? p.lse2 + ct : p.delta + (ct - BT);
        float* stat_dst = (ct < BT) ? lse2_s + ct : delta_s + (ct - BT);
        float stat_next = 0.f;
        {
            const int4 first = next_item(p, 0, n_items, nq);
            if (stager && first.x >= 0) stat_next = __ldg(stat_src + (long long)first.y * p.Tpad + (p.causal ? first.x : 0) * BT);
        }

        for (int4 cur = next_item(p, 0, n_items, nq), nxt = next_item(p, 1, n_items, nq), n4 = make_int4(0, 0, 0, 0); alive && cur.x >= 0;
                 ++n4.x, cur = nxt, nxt = next_item(p, n4.x + 1, n_items, nq)) {
            const int n = n4.x, kt = cur.x, bh = cur.y;
            const int b = cur.z, h = cur.w;
            const int k0 = kt * BT;
            const int i0 = p.causal ? kt : 0;
            const int niter = nq - i0;
            const bool kv_valid = (k0 + r) < p.T;           // rows past the sequence end contribute nothing

            for (int it = 0; it < niter; ++it, ++gi) {
                const int i = i0 + it;
                const uint32_t ss = gi & 1u, par = gi & 1u;
                const float* lse2 = lse2_s + ss * BT + CW * g;
                const float* dlt = delta_s + ss * BT + CW * g;
                if (stager) stat_dst[ss * BT] = stat_next;  // this iteration's value, fetched one iteration ago
                mbar_arrive(&bars[A_ST_FULL + ss]);
                // next iteration's value: the next query tile of this item, or the first one of the next item
                if (stager) {
                    if (it + 1 < niter) stat_next = __ldg(stat_src + (long long)bh * p.Tpad + (i + 1) * BT);
                    else if (nxt.x >= 0) stat_next = __ldg(stat_src + (long long)nxt.y * p.Tpad + (p.causal ? nxt.x : 0) * BT);
                }
                if (!__all_sync(0xffffffffu, mbar_wait(ws, &bars[A_ST_FULL + ss], (gi >> 1) & 1u, DEERS_KERR_BWD_F16 | 13))) { alive = false; break; }
                if (!__all_sync(0xffffffffu, mbar_wait(ws, &bars[A_S], par, DEERS_KERR_BWD_F16 | 14))) { alive = false; break; }
                tc_fence_after_sync();
                const bool diag = p.causal && (i == kt);
                uint32_t pk[CW / 2];                        // P^T row, CW query columns as f16 pairs
#pragma unroll
                for (int c = 0; c < CW / 32; ++c) {
                    uint32_t sr[32];
                    tmem_ld_x32(tmem + TM_S + t_lane + CW * g + c * 32, sr);
                    tmem_wait_ld();
                    if (diag || !kv_valid) {                // only the diagonal / tail tile pays for masking
#pragma unroll
                        for (int e = 0; e < 16; ++e) {
                            const int cl = c * 32 + e * 2;  // column inside this warpgroup's half
                            float p0 = ex2(fmaf(__uint_as_float(sr[e * 2]), sl2, -lse2[cl]));
                            float p1 = ex2(fmaf(__uint_as_float(sr[e * 2 + 1]), sl2, -lse2[cl + 1]));
                            if ((diag && (CW * g + cl) < r) || !kv_valid) p0 = 0.f;   // query index < key index: masked
                            if ((diag && (CW * g + cl + 1) < r) || !kv_valid) p1 = 0.f;
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
                // P^T replaces this warpgroup's part of S^T in TMEM (CW / 2 packed columns).
                tmem_st(tmem + TM_S + t_lane + CW * g, pk);
                tmem_wait_st();
                tc_fence_before_sync();
                mbar_arrive(&bars[A_P]);

                if (!__all_sync(0xffffffffu, mbar_wait(ws, &bars[A_DP], par, DEERS_KERR_BWD_F16 | 15))) { alive = false; break; }
                tc_fence_after_sync();
                uint32_t dd[CW / 2];                        // dS^T row, CW query columns as f16 pairs
#pragma unroll
                for (int c = 0; c < CW / 32; ++c) {
                    uint32_t dr[32];
                    tmem_ld_x32(tmem + TM_DP + t_lane + CW * g + c * 32, dr);
                    tmem_wait_ld();
#pragma unroll
                    for (int e = 0; e < 16; ++e) {
                        const int cl = c * 32 + e * 2;
                        const float2 pf = __half22float2(*reinterpret_cast<const __half2*>(&pk[c * 16 + e]));
                        dd[c * 16 + e] = pack_half2(pf.x * (__uint_as_float(dr[e * 2]) - dlt[cl]),
                                                    pf.y * (__uint_as_float(dr[e * 2 + 1]) - dlt[cl + 1]));
                    }
                }
                tmem_st(tmem + TM_DP + t_lane + CW * g, dd);
                tmem_wait_st();
                tc_fence_before_sync();
                mbar_arrive(&bars[A_DS]);
                if (p.ds) {
                    // The same dS^T row also goes to global memory, already swizzled, for the dQ kernel (off the
                    // critical path: the tensor core has what it needs).  The row's NCH 16-byte chunks are
                    // transposed within NCH-lane groups first, so that one store instruction writes whole
                    // NCH*16-byte row segments instead of 16 bytes in each of 32 rows.
                    constexpr int NCH = CW / 8;                 // this warpgroup's chunks of a row
                    uint8_t* tile = reinterpret_cast<uint8_t*>(p.ds) + (((long long)bh * p.ds_pairs + ds_pair(p, i, kt, nq)) << 15) +
                                    (CW * g / 64) * (int)BLOCK_BYTES;
                    const int ch0 = (CW * g % 64) / 8;          // first chunk inside the 64-column block
                    uint4 pc[NCH];
#pragma unroll
                    for (int ch = 0; ch < NCH; ++ch) pc[ch] = make_uint4(dd[4 * ch], dd[4 * ch + 1], dd[4 * ch + 2], dd[4 * ch + 3]);
                    transpose_pieces<NCH>(pc, (uint32_t)lane);
                    const int rbase = lane_base + (lane & ~(NCH - 1));  // pc[c] is now chunk (lane % NCH) of row rbase + c
#pragma unroll
                    for (int c = 0; c < NCH; ++c)     // streaming stores: the tiles are read once, by the next kernel
                        __stcs(reinterpret_cast<uint4*>(tile + sw128_chunk_offset(rbase + c, ch0 + (lane & (NCH - 1)))), pc[c]);
                }
            }
            if (!alive) break;

            // Epilogue: dK and dV of this KV tile leave TMEM; meanwhile the tensor core already
            // computes S^T and dP^T of the next item.
            if (!__all_sync(0xffffffffu, mbar_wait(ws, &bars[A_DONE], (uint32_t)n & 1u, DEERS_KERR_BWD_F16 | 16))) { alive = false; break; }
            tc_fence_after_sync();
            // The thread's half rows of dK and dV, as 16-byte pieces, are transposed within lane
            // groups so that every store instruction writes whole contiguous row segments.
            constexpr int NP = DH / 8;
            uint4 kc[NP], vc[NP];
#pragma unroll
            for (int c = 0; c < DH / EC; ++c) {
                uint32_t kr[EC], vr[EC];
                tmem_ld(tmem + TM_DK + t_lane + g * DH + c * EC, kr);
                tmem_ld(tmem + TM_DV + t_lane + g * DH + c * EC, vr);
                tmem_wait_ld();
                if (c == DH / EC - 1) {                     // accumulators are in registers: release TMEM early
                    tc_fence_before_sync();
                    mbar_arrive(&bars[A_ACC_FREE]);
                }
#pragma unroll
                for (int q8 = 0; q8 < EC / 8; ++q8) {
                    kc[c * (EC / 8) + q8] = pack8_f16(kr + q8 * 8, p.scale);
                    vc[c * (EC / 8) + q8] = pack8_f16(vr + q8 * 8, 1.0f);
                }
            }
            transpose_pieces<NP>(kc, (uint32_t)lane);
            transpose_pieces<NP>(vc, (uint32_t)lane);
            const int row0 = k0 + lane_base + (lane & ~(NP - 1));
            const int col = g * DH + (lane & (NP - 1)) * 8;
            __half* dkb = p.dk + b * p.sdk_b + h * p.sdk_h + col;
            __half* dvb = p.dv + b * p.sdv_b + h * p.sdv_h + col;
#pragma unroll
            for (int c = 0; c < NP; ++c) {
                const int row = row0 + c;
                if (row < p.T) {
                    *reinterpret_cast<uint4*>(dkb + (long long)row * p.sdk_t) = kc[c];
                    *reinterpret_cast<uint4*>(dvb + (long long)row * p.sdv_t) = vc[c];
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
// dQ kernel (persistent: each CTA walks a strided list of query tiles)
// ---------------------------------------------------------------------------------------------
template <int D>
struct DqSmem {
    static constexpr uint32_t TILE = 128u * D * 2u;
    static constexpr uint32_t Q = 0;
    static constexpr uint32_t DO = Q + TILE;
    static constexpr uint32_t K = DO + TILE;                 // three stages: K(j+1) feeds S while K(j) still feeds dQ
    static constexpr uint32_t V = K + 3 * TILE;              // two stages
    static constexpr uint32_t BARS = V + 2 * TILE;
    static constexpr uint32_t TOTAL = BARS + 256;
};

// Q_DP and Q_DS are pairs indexed by the parity of the KV step: dP runs one step ahead of its reader.
enum DqBar { Q_QDO_FULL = 0, Q_QDO_EMPTY = 1, Q_K_FULL = 2, Q_K_EMPTY = 5, Q_V_FULL = 8, Q_V_EMPTY = 10, Q_S = 12, Q_DP = 13,
             Q_PDONE = 15, Q_DS = 16, Q_DONE = 18, Q_DQ_FREE = 19, Q_COUNT = 20 };

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
    // S | dP of even KV steps (later dS in place) | dP of odd KV steps | dQ
    constexpr uint32_t TM_S = 0, TM_DP = 128, TM_DQ = 384;

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
    const int n_items = p.B * p.H * nq;

    if (threadIdx.x == 0) {
        *abort_s = 0;
        uint32_t skip = (*(volatile unsigned int*)p.err != 0) ? 1u : 0u;
        if ((smem_u32(smem) & 1023u) != 0) {
            atomicCAS(p.err, 0u, DEERS_KERR_BWD_F16 | 0x21);
            skip = 1;
        }
        *skip_s = skip;
        mbar_init(&bars[Q_QDO_FULL], 1);
        mbar_init(&bars[Q_QDO_EMPTY], 1);
        for (int s = 0; s < 3; ++s) { mbar_init(&bars[Q_K_FULL + s], 1); mbar_init(&bars[Q_K_EMPTY + s], 1); }
        for (int s = 0; s < 2; ++s) {
            mbar_init(&bars[Q_V_FULL + s], 1); mbar_init(&bars[Q_V_EMPTY + s], 1);
            mbar_init(&bars[Q_DP + s], 1); mbar_init(&bars[Q_DS + s], 256);
        }
        mbar_init(&bars[Q_S], 1);
        mbar_init(&bars[Q_PDONE], 256);
        mbar_init(&bars[Q_DONE], 1);
        mbar_init(&bars[Q_DQ_FREE], 256);
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
            uint32_t kvc = 0;                                   // K/V stage uses so far (all items)
            bool ok = true;
            for (int4 cur = next_item(p, 0, n_items, nq), nxt = next_item(p, 1, n_items, nq), n4 = make_int4(0, 0, 0, 0); ok && cur.x >= 0;
                     ++n4.x, cur = nxt, nxt = next_item(p, n4.x + 1, n_items, nq)) {
                const int n = n4.x, slot = cur.x, bh = cur.y;
                const int qt = nq - 1 - slot;                   // late query tiles carry the most work
                const int b = cur.z, h = cur.w;
                const int ntiles = p.causal ? qt + 1 : nq;
                // Q / dO are single-buffered: wait until the previous item's S and dP products are done.
                if (!mbar_wait(ws, &bars[Q_QDO_EMPTY], ((uint32_t)n & 1u) ^ 1u, DEERS_KERR_BWD_F16 | 0x10)) break;
                mbar_arrive_expect_tx(&bars[Q_QDO_FULL], 2 * TILE_BYTES);
#pragma unroll
                for (int blk = 0; blk < DBLK; ++blk) {
                    tma_load_4d(sQ + blk * BLOCK_BYTES, &tmap_q, &bars[Q_QDO_FULL], blk * 64, qt * BT, h, b);
                    tma_load_4d(sDO + blk * BLOCK_BYTES, &tmap_do, &bars[Q_QDO_FULL], blk * 64, qt * BT, h, b);
                }
                for (int j = 0; j < ntiles; ++j, ++kvc) {
                    const uint32_t ks = kvc % 3u, vs = kvc & 1u;
                    if (!mbar_wait(ws, &bars[Q_K_EMPTY + ks], ((kvc / 3u) & 1u) ^ 1u, DEERS_KERR_BWD_F16 | 0x11)) { ok = false; break; }
                    mbar_arrive_expect_tx(&bars[Q_K_FULL + ks], TILE_BYTES);
#pragma unroll
                    for (int blk = 0; blk < DBLK; ++blk)
                        tma_load_4d(sK + ks * TILE_BYTES + blk * BLOCK_BYTES, &tmap_k, &bars[Q_K_FULL + ks], blk * 64, j * BT, h, b);
                    if (!mbar_wait(ws, &bars[Q_V_EMPTY + vs], ((kvc >> 1) & 1u) ^ 1u, DEERS_KERR_BWD_F16 | 0x1b)) { ok = false; break; }
                    mbar_arrive_expect_tx(&bars[Q_V_FULL + vs], TILE_BYTES);
#pragma unroll
                    for (int blk = 0; blk < DBLK; ++blk)
                        tma_load_4d(sV + vs * TILE_BYTES + blk * BLOCK_BYTES, &tmap_v, &bars[Q_V_FULL + vs], blk * 64, j * BT, h, b);
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
            auto issue_s = [&](uint32_t st) {
                const uint64_t k_km = k_km0 + (uint64_t)st * STAGE_STEP;
#pragma unroll
                for (int ks = 0; ks < D / 16; ++ks)
                    umma_ss(tmem + TM_S, q_km + kmajor_step(ks, BLOCK_BYTES), k_km + kmajor_step(ks, BLOCK_BYTES), IDESC_S, ks > 0);
                umma_commit(&bars[Q_S]);
            };
            // The V stage and the dP buffer both alternate with the parity of the KV step.
            auto issue_dp = [&](uint32_t st) {
                const uint64_t v_km = v_km0 + (uint64_t)st * STAGE_STEP;
                const uint32_t tm_dp = tmem + TM_DP + st * 128u;
#pragma unroll
                for (int ks = 0; ks < D / 16; ++ks)
                    umma_ss(tm_dp, do_km + kmajor_step(ks, BLOCK_BYTES), v_km + kmajor_step(ks, BLOCK_BYTES), IDESC_S, ks > 0);
                umma_commit(&bars[Q_DP + st]);
                umma_commit(&bars[Q_V_EMPTY + st]);                    // dP is the only reader of a V tile
            };
            uint32_t kvc = 0;                                   // K/V stage uses == KV iterations so far
            bool ok = true;
            for (int4 cur = next_item(p, 0, n_items, nq), nxt = next_item(p, 1, n_items, nq), n4 = make_int4(0, 0, 0, 0); ok && cur.x >= 0;
                     ++n4.x, cur = nxt, nxt = next_item(p, n4.x + 1, n_items, nq)) {
                const int n = n4.x, slot = cur.x, bh = cur.y;
                const int qt = nq - 1 - slot;
                const int ntiles = p.causal ? qt + 1 : nq;
                const uint32_t tm_dq = tmem + TM_DQ;
                if (!mbar_wait(ws, &bars[Q_QDO_FULL], (uint32_t)n & 1u, DEERS_KERR_BWD_F16 | 0x12)) break;
                if (!mbar_wait(ws, &bars[Q_K_FULL + kvc % 3u], (kvc / 3u) & 1u, DEERS_KERR_BWD_F16 | 0x13)) break;
                if (!mbar_wait(ws, &bars[Q_V_FULL + (kvc & 1u)], (kvc >> 1) & 1u, DEERS_KERR_BWD_F16 | 0x1c)) break;
                tc_fence_after_sync();
                issue_s(kvc % 3u);
                issue_dp(kvc & 1u);
                for (int j = 0; j < ntiles; ++j, ++kvc) {
                    const uint32_t ks = kvc % 3u, ksn = (kvc + 1u) % 3u, vsn = (kvc + 1u) & 1u;
                    const uint32_t par = kvc & 1u;
                    const bool more = j + 1 < ntiles;
                    // S and dP of the next KV tile as soon as the compute threads have read this S:
                    // dP lands in the buffer whose dS the product issued one step ago has consumed
                    // (the pipe is in order), so the tensor core never waits for this step's dS.
                    if (!mbar_wait(ws, &bars[Q_PDONE], par, DEERS_KERR_BWD_F16 | 0x14)) { ok = false; break; }
                    if (more) {
                        if (!mbar_wait(ws, &bars[Q_K_FULL + ksn], ((kvc + 1u) / 3u) & 1u, DEERS_KERR_BWD_F16 | 0x15)) { ok = false; break; }
                        tc_fence_after_sync();
                        issue_s(ksn);
                        if (!mbar_wait(ws, &bars[Q_V_FULL + vsn], ((kvc + 1u) >> 1) & 1u, DEERS_KERR_BWD_F16 | 0x1d)) { ok = false; break; }
                        tc_fence_after_sync();
                        issue_dp(vsn);
                    } else {
                        umma_commit(&bars[Q_QDO_EMPTY]);               // every product reading Q / dO has been issued
                    }
                    // dQ += dS K
                    if (!mbar_wait(ws, &bars[Q_DS + par], (kvc >> 1) & 1u, DEERS_KERR_BWD_F16 | 0x16)) { ok = false; break; }
                    // The previous item's dQ must have left TMEM before this item accumulates.
                    if (j == 0 && n > 0 && !mbar_wait(ws, &bars[Q_DQ_FREE], ((uint32_t)n - 1u) & 1u, DEERS_KERR_BWD_F16 | 0x1a)) { ok = false; break; }
                    tc_fence_after_sync();
                    const uint64_t k_mn = k_mn0 + (uint64_t)ks * STAGE_STEP;
                    const uint32_t tm_ds = tmem + TM_DP + par * 128u;
#pragma unroll
                    for (int ks = 0; ks < BT / 16; ++ks)
                        umma_ts(tm_dq, tm_ds + (uint32_t)(ks >> 2) * 64u + (uint32_t)(ks & 3) * 8u,
                                k_mn + mnmajor_step(ks), IDESC_DQ, (j > 0 || ks > 0));
                    umma_commit(&bars[Q_K_EMPTY + ks]);                // S and dQ have both read this K tile
                }
                umma_commit(&bars[Q_DONE]);
            }
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
        uint32_t gi = 0;                                        // KV iterations so far (all items)
        bool alive = true;
        // The epilogue of item n (scale, convert, store its dQ tile, release the accumulator) is
        // deferred until the first dS of item n+1 has been handed over: the tensor core then still
        // has S and dP of the second KV tile to compute before it needs the accumulator.
        int pend_n = -1, pend_row = 0;
        __half* pend_ptr = nullptr;
        auto epilogue = [&]() -> bool {
            if (pend_n < 0) return true;
            const int n = pend_n;
            pend_n = -1;
            if (!__all_sync(0xffffffffu, mbar_wait(ws, &bars[Q_DONE], (uint32_t)n & 1u, DEERS_KERR_BWD_F16 | 0x19))) return false;
            tc_fence_after_sync();
            constexpr int NP = DH / 8;
            uint4 qc[NP];
#pragma unroll
            for (int c = 0; c < DH / 32; ++c) {
                uint32_t qr[32];
                tmem_ld_x32(tmem + TM_DQ + t_lane + g * DH + c * 32, qr);
                tmem_wait_ld();
#pragma unroll
                for (int q8 = 0; q8 < 4; ++q8) qc[c * 4 + q8] = pack8_f16(qr + q8 * 8, p.scale);
            }
            tc_fence_before_sync();
            mbar_arrive(&bars[Q_DQ_FREE]);
            // Pieces transposed within lane groups: every store writes contiguous row segments.
            transpose_pieces<NP>(qc, (uint32_t)lane);
            const int row0 = pend_row - lane + (lane & ~(NP - 1));
            __half* qb = pend_ptr + (lane & (NP - 1)) * 8;     // row 0 of the slice, this lane's piece
#pragma unroll
            for (int c = 0; c < NP; ++c) {
                const int row = row0 + c;
                if (row < p.T) *reinterpret_cast<uint4*>(qb + (long long)row * p.sdq_t) = qc[c];
            }
            return true;
        };

        for (int4 cur = next_item(p, 0, n_items, nq), nxt = next_item(p, 1, n_items, nq), n4 = make_int4(0, 0, 0, 0); alive && cur.x >= 0;
                 ++n4.x, cur = nxt, nxt = next_item(p, n4.x + 1, n_items, nq)) {
            const int n = n4.x, slot = cur.x, bh = cur.y;
            const int qt = nq - 1 - slot;
            const int b = cur.z, h = cur.w;
            const int q0 = qt * BT;
            const int ntiles = p.causal ? qt + 1 : nq;
            const float lse2_r = p.lse2[(long long)bh * p.Tpad + q0 + r];      // padded: 0 beyond T
            const float delta_r = p.delta[(long long)bh * p.Tpad + q0 + r];

            for (int j = 0; j < ntiles; ++j, ++gi) {
                const uint32_t par = gi & 1u;
                if (!__all_sync(0xffffffffu, mbar_wait(ws, &bars[Q_S], par, DEERS_KERR_BWD_F16 | 0x17))) { alive = false; break; }
                tc_fence_after_sync();
                const int k0 = j * BT;
                const bool edge = (p.causal && j == qt) || (k0 + BT > p.T);
                float pv[64];                               // P row, this warpgroup's 64 key columns
                {
                    uint32_t sr[64];
                    tmem_ld_x32(tmem + TM_S + t_lane + 64 * g, *reinterpret_cast<uint32_t(*)[32]>(&sr[0]));
                    tmem_ld_x32(tmem + TM_S + t_lane + 64 * g + 32, *reinterpret_cast<uint32_t(*)[32]>(&sr[32]));
                    tmem_wait_ld();
                    tc_fence_before_sync();
                    mbar_arrive(&bars[Q_PDONE]);            // S is in registers: the next S may land
                    if (edge) {
#pragma unroll
                        for (int e = 0; e < 64; ++e) {
                            const int col = 64 * g + e;                       // key index inside the tile
                            const bool masked = (p.causal && j == qt && col > r) || (k0 + col >= p.T);
                            pv[e] = masked ? 0.f : ex2(fmaf(__uint_as_float(sr[e]), sl2, -lse2_r));
                        }
                    } else {
#pragma unroll
                        for (int e = 0; e < 64; ++e) pv[e] = ex2(fmaf(__uint_as_float(sr[e]), sl2, -lse2_r));
                    }
                }

                if (!__all_sync(0xffffffffu, mbar_wait(ws, &bars[Q_DP + par], (gi >> 1) & 1u, DEERS_KERR_BWD_F16 | 0x18))) { alive = false; break; }
                tc_fence_after_sync();
                uint32_t dd[32];
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    uint32_t dr[32];
                    tmem_ld_x32(tmem + TM_DP + par * 128u + t_lane + 64 * g + c * 32, dr);
                    tmem_wait_ld();
#pragma unroll
                    for (int e = 0; e < 16; ++e)
                        dd[c * 16 + e] = pack_half2(pv[c * 32 + e * 2] * (__uint_as_float(dr[e * 2]) - delta_r),
                                                    pv[c * 32 + e * 2 + 1] * (__uint_as_float(dr[e * 2 + 1]) - delta_r));
                }
                // dS replaces this warpgroup's half of dP in TMEM (32 packed columns).
                tmem_st_x32(tmem + TM_DP + par * 128u + t_lane + 64 * g, dd);
                tmem_wait_st();
                tc_fence_before_sync();
                mbar_arrive(&bars[Q_DS + par]);
                if (j == 0 && !epilogue()) { alive = false; break; }       // previous item's dQ tile
            }
            if (!alive) break;

            pend_n = n;
            pend_row = q0 + r;
            pend_ptr = p.dq + b * p.sdq_b + h * p.sdq_h + g * DH;     // row 0 of the slice
        }
        if (alive) epilogue();
    }

    __syncwarp();
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem, TMEM_COLS);
}

// ---------------------------------------------------------------------------------------------
// dQ from stored dS^T tiles (persistent; used when the caller's workspace has room for them)
// ---------------------------------------------------------------------------------------------
// dQ tile i = scale * sum_j dS(i, j) K(j): a streaming product.  Warp 0 brings, per KV tile, the 32 KB dS^T tile
// (two bulk copies: it is already in shared-memory order) and the K tile (TMA) into a 3-stage ring; warp 1
// issues 8 tcgen05.mma per stage (A = dS^T read MN-major, B = K read MN-major) into one of two TMEM
// accumulators; warps 2-5 convert a finished accumulator to f16 and store it.  No exponentials, no second
// pass over Q, V, dO: the kernel is bound by reading the dS^T tiles once.
template <int D>
struct DqsSmem {
    static constexpr uint32_t DS = 128u * 128u * 2u;
    static constexpr uint32_t KT = 128u * D * 2u;
    static constexpr uint32_t STAGE = DS + KT;
    static constexpr int STAGES = 3;
    static constexpr uint32_t BARS = STAGES * STAGE;
    static constexpr uint32_t TOTAL = BARS + 256;
};

enum DqsBar { R_FULL = 0, R_EMPTY = 3, R_ACC_FULL = 6, R_ACC_EMPTY = 8, R_COUNT = 10 };

template <int D>
__global__ void __launch_bounds__(192, 1)
attn_bwd_dq_from_ds_f16_kernel(const __grid_constant__ CUtensorMap tmap_k, const BwdParams p) {
    using L = DqsSmem<D>;
    constexpr int DBLK = D / 64;
    constexpr uint32_t TMEM_COLS = 2 * D;                    // 128 or 256: a power of two

    extern __shared__ __align__(1024) uint8_t smem[];
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::BARS);
    uint32_t* tmem_base_s = reinterpret_cast<uint32_t*>(bars + R_COUNT);
    volatile uint32_t* abort_s = tmem_base_s + 1;
    uint32_t* skip_s = tmem_base_s + 2;

    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const int nq = (p.T + BT - 1) / BT;
    const int n_items = p.B * p.H * nq;

    if (threadIdx.x == 0) {
        *abort_s = 0;
        uint32_t skip = (*(volatile unsigned int*)p.err != 0) ? 1u : 0u;
        if ((smem_u32(smem) & 1023u) != 0) {
            atomicCAS(p.err, 0u, DEERS_KERR_BWD_F16 | 0x20);
            skip = 1;
        }
        *skip_s = skip;
        for (int s = 0; s < L::STAGES; ++s) { mbar_init(&bars[R_FULL + s], 1); mbar_init(&bars[R_EMPTY + s], 1); }
        for (int s = 0; s < 2; ++s) { mbar_init(&bars[R_ACC_FULL + s], 1); mbar_init(&bars[R_ACC_EMPTY + s], 128); }
        fence_barrier_init();
        tma_prefetch_desc(&tmap_k);
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
        // ------------------------------ producer ------------------------------
        if (lane == 0) {
            uint32_t gi = 0;                                    // KV steps so far (ring position)
            bool ok = true;
            const uint64_t pol = l2_policy_evict_first();
            for (int4 cur = next_item(p, 0, n_items, nq), nxt = next_item(p, 1, n_items, nq), n4 = make_int4(0, 0, 0, 0); ok && cur.x >= 0;
                     ++n4.x, cur = nxt, nxt = next_item(p, n4.x + 1, n_items, nq)) {
                const int qt = nq - 1 - cur.x, bh = cur.y, b = cur.z, h = cur.w;
                const int ntiles = p.causal ? qt + 1 : nq;
                const uint8_t* ds_src = reinterpret_cast<const uint8_t*>(p.ds) + (((long long)bh * p.ds_pairs + ds_pair(p, qt, 0, nq)) << 15);
                for (int j = 0; j < ntiles; ++j, ++gi) {
                    const uint32_t s = gi % (uint32_t)L::STAGES;
                    if (!mbar_wait(ws, &bars[R_EMPTY + s], ((gi / (uint32_t)L::STAGES) & 1u) ^ 1u, DEERS_KERR_BWD_F16 | 0x30)) { ok = false; break; }
                    mbar_arrive_expect_tx(&bars[R_FULL + s], L::STAGE);
                    uint8_t* stage = smem + s * L::STAGE;
                    // dS^T tiles are read exactly once: first to leave L2, so that the K tiles the slice's other
                    // query tiles share stay there
                    bulk_load_hint(stage, ds_src + ((long long)j << 15), BLOCK_BYTES, &bars[R_FULL + s], pol);
                    bulk_load_hint(stage + BLOCK_BYTES, ds_src + ((long long)j << 15) + BLOCK_BYTES, BLOCK_BYTES, &bars[R_FULL + s], pol);
#pragma unroll
                    for (int blk = 0; blk < DBLK; ++blk)
                        tma_load_4d(stage + L::DS + blk * BLOCK_BYTES, &tmap_k, &bars[R_FULL + s], blk * 64, j * BT, h, b);
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer ------------------------------
        if (lane == 0) {
            constexpr uint32_t IDESC = idesc_f16(128, D, 1, 1);        // both operands MN-major
            constexpr uint64_t STAGE_STEP = L::STAGE >> 4;
            const uint64_t a0 = desc_mnmajor(smem_u32(smem), 0, BLOCK_BYTES);
            const uint64_t b0 = desc_mnmajor(smem_u32(smem + L::DS), 0, BLOCK_BYTES);
            uint32_t gi = 0;
            bool ok = true;
            for (int4 cur = next_item(p, 0, n_items, nq), nxt = next_item(p, 1, n_items, nq), n4 = make_int4(0, 0, 0, 0); ok && cur.x >= 0;
                     ++n4.x, cur = nxt, nxt = next_item(p, n4.x + 1, n_items, nq)) {
                const uint32_t n = (uint32_t)n4.x, buf = n & 1u;
                const int qt = nq - 1 - cur.x;
                const int ntiles = p.causal ? qt + 1 : nq;
                if (!mbar_wait(ws, &bars[R_ACC_EMPTY + buf], ((n >> 1) & 1u) ^ 1u, DEERS_KERR_BWD_F16 | 0x31)) break;
                for (int j = 0; j < ntiles; ++j, ++gi) {
                    const uint32_t s = gi % (uint32_t)L::STAGES;
                    if (!mbar_wait(ws, &bars[R_FULL + s], (gi / (uint32_t)L::STAGES) & 1u, DEERS_KERR_BWD_F16 | 0x32)) { ok = false; break; }
                    tc_fence_after_sync();
                    const uint64_t a = a0 + (uint64_t)s * STAGE_STEP, bd = b0 + (uint64_t)s * STAGE_STEP;
#pragma unroll
                    for (int ks = 0; ks < BT / 16; ++ks)
                        umma_ss(tmem + buf * (uint32_t)D, a + mnmajor_step(ks), bd + mnmajor_step(ks), IDESC, (j > 0 || ks > 0));
                    umma_commit(&bars[R_EMPTY + s]);
                }
                if (ok) umma_commit(&bars[R_ACC_FULL + buf]);
            }
        }
    } else {
        // ------------------------------ epilogue ------------------------------
        const int lane_base = (warp & 3) * 32;
        const uint32_t t_lane = (uint32_t)lane_base << 16;
        for (int4 cur = next_item(p, 0, n_items, nq), nxt = next_item(p, 1, n_items, nq), n4 = make_int4(0, 0, 0, 0); cur.x >= 0;
                 ++n4.x, cur = nxt, nxt = next_item(p, n4.x + 1, n_items, nq)) {
            const uint32_t n = (uint32_t)n4.x, buf = n & 1u;
            const int qt = nq - 1 - cur.x, b = cur.z, h = cur.w;
            if (!__all_sync(0xffffffffu, mbar_wait(ws, &bars[R_ACC_FULL + buf], (n >> 1) & 1u, DEERS_KERR_BWD_F16 | 0x33))) break;
            tc_fence_after_sync();
            const int row0 = qt * BT + lane_base + (lane & ~7);
            __half* qb = p.dq + b * p.sdq_b + h * p.sdq_h + (lane & 7) * 8;
#pragma unroll 1
            for (int part = 0; part < D / 64; ++part) {          // 64 columns at a time
                uint32_t r[64];
                uint4 pc[8];
                tmem_ld_x32(tmem + buf * (uint32_t)D + t_lane + part * 64, *reinterpret_cast<uint32_t(*)[32]>(&r[0]));
                tmem_ld_x32(tmem + buf * (uint32_t)D + t_lane + part * 64 + 32, *reinterpret_cast<uint32_t(*)[32]>(&r[32]));
                tmem_wait_ld();
                if (part == D / 64 - 1) {                        // accumulator is in registers: the next item may use it
                    tc_fence_before_sync();
                    mbar_arrive(&bars[R_ACC_EMPTY + buf]);
                }
#pragma unroll
                for (int q8 = 0; q8 < 8; ++q8) pc[q8] = pack8_f16(r + q8 * 8, p.scale);
                transpose_pieces<8>(pc, (uint32_t)lane);
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    const int row = row0 + c;
                    if (row < p.T) *reinterpret_cast<uint4*>(qb + (long long)row * p.sdq_t + part * 64) = pc[c];
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
// [B*H][Tpad] grid (0 beyond T).  D/8 lanes share a row (16-byte loads); a warp takes 4 * 256 / D
// consecutive rows per step with all eight loads of a lane in flight before the first is used;
// grid-stride over such row groups.  The row count fits 32 bits (checked by the launcher).
template <int D>
__global__ void __launch_bounds__(256)
attn_bwd_prep_f16_kernel(const __half* __restrict__ o, const __half* __restrict__ d_o, const float* __restrict__ lse,
                         float* __restrict__ delta, float* __restrict__ lse2, int B, int H, int T, int Tpad,
                         long long so_b, long long so_h, long long so_t, long long sdo_b, long long sdo_h,
                         long long sdo_t) {
    constexpr int LPR = D / 8;                               // lanes per row
    constexpr int RPW = 32 / LPR;                            // rows per warp load
    constexpr int U = 4;                                     // loads in flight per lane and tensor
    const int lane = threadIdx.x % 32;
    const int sub = lane % LPR, rw = lane / LPR;
    const unsigned rows = (unsigned)B * (unsigned)H * (unsigned)Tpad;
    const unsigned warp_global = blockIdx.x * (blockDim.x / 32) + threadIdx.x / 32;
    const unsigned warp_count = gridDim.x * (blockDim.x / 32);
    const unsigned ngroups = (rows + RPW * U - 1) / (RPW * U);
    for (unsigned grp = warp_global; grp < ngroups; grp += warp_count) {
        uint4 a[U], g[U];
        unsigned row[U];
        bool valid[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            row[u] = grp * (RPW * U) + u * RPW + rw;
            const unsigned t = row[u] % (unsigned)Tpad, bh = row[u] / (unsigned)Tpad;
            valid[u] = row[u] < rows && t < (unsigned)T;
            a[u] = make_uint4(0u, 0u, 0u, 0u);
            g[u] = a[u];
            if (valid[u]) {
                const unsigned b = bh / (unsigned)H, h = bh % (unsigned)H;
                a[u] = *reinterpret_cast<const uint4*>(o + b * so_b + h * so_h + (long long)t * so_t + sub * 8);
                g[u] = *reinterpret_cast<const uint4*>(d_o + b * sdo_b + h * sdo_h + (long long)t * sdo_t + sub * 8);
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const uint32_t av[4] = {a[u].x, a[u].y, a[u].z, a[u].w}, gv[4] = {g[u].x, g[u].y, g[u].z, g[u].w};
            float s = 0.f;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 af = __half22float2(*reinterpret_cast<const __half2*>(&av[e]));
                const float2 gf = __half22float2(*reinterpret_cast<const __half2*>(&gv[e]));
                s = fmaf(af.x, gf.x, s);
                s = fmaf(af.y, gf.y, s);
            }
#pragma unroll
            for (int off = LPR / 2; off >= 1; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
            if (row[u] < rows && sub == 0) {
                const unsigned t = row[u] % (unsigned)Tpad, bh = row[u] / (unsigned)Tpad;
                delta[row[u]] = valid[u] ? s : 0.f;
                lse2[row[u]] = valid[u] ? lse[(long long)bh * T + t] * LOG2E : 0.f;
            }
        }
    }
}

size_t bwd_stat_bytes(const deers_attn_desc* d) {
    const size_t Tpad = (size_t)((d->T + BT - 1) / BT) * BT;
    return ((size_t)d->B * d->H * Tpad * sizeof(float) + 255) / 256 * 256;
}

template <int D>
int bwd_launch(deers_ctx* ctx, const deers_attn_desc* d, const void* q, const void* k, const void* v, const void* o,
               const float* lse, const void* d_o, void* dq, void* dk, void* dv, void* workspace, bool keep_ds) {
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
        if (prep_rows > 0x7fffffffLL) return DEERS_ERR_SHAPE;      // 32-bit row indices in the kernel
        const long long per_block = 8LL * 4 * (256 / D);           // 8 warps x 4 loads x rows per load
        const long long want = (prep_rows + per_block - 1) / per_block;
        const unsigned prep_grid = (unsigned)(want < 8LL * ctx->sm_count ? want : 8LL * ctx->sm_count);
        attn_bwd_prep_f16_kernel<D><<<prep_grid, 256, 0, ctx->stream>>>(
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
    p.ds_pairs = d->causal ? (long long)nq * (nq + 1) / 2 : (long long)nq * nq;
    p.ds = keep_ds ? (__half*)((char*)workspace + 2 * stat_bytes) : nullptr;
    const long long grid = BH * nq;
    if (grid > 0x7fffffffLL) return DEERS_ERR_SHAPE;

    const unsigned persistent = (unsigned)(grid < ctx->sm_count ? grid : ctx->sm_count);
    p.sched = deers_get_schedule(ctx, d->B, d->H, nq, d->causal, (int)persistent, &p.sched_rows);
    const size_t smem_a = DkvSmem<D>::TOTAL, smem_b = DqSmem<D>::TOTAL;
    DEERS_CUDA_TRY(ctx, cudaFuncSetAttribute(attn_bwd_dkdv_f16_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_a));
    DEERS_CUDA_TRY(ctx, cudaFuncSetAttribute(attn_bwd_dq_f16_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_b));
    {
        KernelTimerScope ts(ctx, DEERS_K_BWD_MAIN);
        attn_bwd_dkdv_f16_kernel<D><<<persistent, DKV_THREADS, smem_a, ctx->stream>>>(tq, tk, tv, tdo, p);
    }
    DEERS_CUDA_TRY(ctx, cudaGetLastError());
    if (keep_ds) {
        const size_t smem_c = DqsSmem<D>::TOTAL;
        DEERS_CUDA_TRY(ctx, cudaFuncSetAttribute(attn_bwd_dq_from_ds_f16_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_c));
        KernelTimerScope ts(ctx, DEERS_K_BWD_DQ);
        attn_bwd_dq_from_ds_f16_kernel<D><<<persistent, 192, smem_c, ctx->stream>>>(tk, p);
    } else {
        KernelTimerScope ts(ctx, DEERS_K_BWD_DQ);
        attn_bwd_dq_f16_kernel<D><<<persistent, 320, smem_b, ctx->stream>>>(tq, tk, tv, tdo, p);
    }
    DEERS_CUDA_TRY(ctx, cudaGetLastError());
    ctx->launches += 3;
    return DEERS_OK;
}

}  // namespace

// Workspace: delta [B*H][Tpad] | lse*log2e [B*H][Tpad], float32, Tpad = T rounded up to 128; with keep_ds
// also one 32 KB dS^T tile per (slice, query tile, KV tile) pair the mask leaves.
size_t attn_bwd_f16_workspace_bytes(const deers_attn_desc* d, bool keep_ds) {
    size_t bytes = 2 * bwd_stat_bytes(d);
    if (keep_ds) {
        const size_t nq = (size_t)((d->T + BT - 1) / BT);
        bytes += (size_t)d->B * d->H * (d->causal ? nq * (nq + 1) / 2 : nq * nq) * 32768u;
    }
    return bytes;
}

int launch_attn_bwd_f16(deers_ctx* ctx, const deers_attn_desc* d, const void* q, const void* k, const void* v,
                        const void* o, const float* lse, const void* d_o, void* dq, void* dk, void* dv,
                        void* workspace, bool keep_ds) {
    if (d->D == 64) return bwd_launch<64>(ctx, d, q, k, v, o, lse, d_o, dq, dk, dv, workspace, keep_ds);
    if (d->D == 128) return bwd_launch<128>(ctx, d, q, k, v, o, lse, d_o, dq, dk, dv, workspace, keep_ds);
    return DEERS_ERR_UNSUPPORTED;
}

// ---------------------------------------------------------------------------------------------
// Backward without a caller-provided workspace
// ---------------------------------------------------------------------------------------------
// Some hosts of this library cannot hand it scratch memory: code running inside a stream-ordered
// or pooled allocator's callback, a plugin whose host forbids cudaMalloc after start-up, or a caller
// in the middle of building its own memory plan.  For them the f16 backward is also offered with
// its scratch (the per-row delta and lse*log2e arrays) placed in a fixed array that is part of the
// library image.  Every GPU that loads the library carries these 8 MiB until the process exits.
constexpr size_t kStaticScratchFloats = 2u * 1024u * 1024u;            // 8 MiB: B*H*Tpad <= 1 Mi rows
static __device__ __align__(256) float g_bwd_static_scratch[kStaticScratchFloats];

// In host code the array's name is only a handle; kernels need its device address, which differs
// per device and is looked up once per device with that device current.  Two host threads that make
// the first call on one device at the same time both store the same address: harmless.
static void* g_static_scratch_addr[64] = {nullptr};

extern "C" __attribute__((visibility("default")))
int deers_b200_attn_bwd_f16_static(deers_ctx* ctx, const deers_attn_desc* d, const void* q, const void* k,
                                   const void* v, const void* o, const float* lse, const void* d_o, void* dq,
                                   void* dk, void* dv) {
    if (!ctx) return DEERS_ERR_NULL;
    // the same checks, in the same order, as deers_b200_attn_bwd: both accept and refuse the same descriptors
    const int rc = deers_check_bwd_args(d, q, k, v, o, lse, d_o, dq, dk, dv);
    if (rc) return rc;
    if (d->dtype != DEERS_F16) return DEERS_ERR_DTYPE;
    if (d->D != 64 && d->D != 128) return DEERS_ERR_UNSUPPORTED;      // the zero-padded path needs room for copies
    if (ctx->device < 0 || ctx->device >= 64) return DEERS_ERR_DEVICE;
    const size_t need = attn_bwd_f16_workspace_bytes(d, false);
    if (need > sizeof(float) * kStaticScratchFloats) {
        snprintf(ctx->last_error, sizeof(ctx->last_error),
                 "deers_b200_attn_bwd_f16_static: needs %zu bytes of scratch, the built-in array holds %zu "
                 "(B*H*ceil(T/128)*128 must not exceed %zu rows); use deers_b200_attn_bwd with a workspace",
                 need, sizeof(float) * kStaticScratchFloats, kStaticScratchFloats / 2);
        return DEERS_ERR_WORKSPACE;
    }
    DEERS_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    if (!g_static_scratch_addr[ctx->device]) {
        void* addr = nullptr;
        DEERS_CUDA_TRY(ctx, cudaGetSymbolAddress(&addr, g_bwd_static_scratch));
        g_static_scratch_addr[ctx->device] = addr;
    }
    void* scratch = g_static_scratch_addr[ctx->device];
    // Nothing needs clearing: the first kernel of the backward writes every element of both arrays
    // (zeros beyond T included) before the other two read them.
    if (d->D == 64) return bwd_launch<64>(ctx, d, q, k, v, o, lse, d_o, dq, dk, dv, scratch, false);
    return bwd_launch<128>(ctx, d, q, k, v, o, lse, d_o, dq, dk, dv, scratch, false);
}
