// f16 causal attention forward for sm_100a, two query tiles per CTA.
//
// Persistent kernel: one CTA per SM walks a balanced list of work items; an item is 256 query rows of one
// (batch, head) slice, handled as two 128-row tiles A and B that share every key / value tile.  While the
// softmax of one tile runs on the CUDA cores, the tensor core works on the other tile, so neither waits for
// the other in steady state:
//   warp 0        TMA producer: Q_A, Q_B per item, K and V tiles through rings
//   warp 1        the single MMA issuer.  Per key tile j:  O_A += P_A(j) V(j);  S_A(j+1) = Q_A K(j+1)^T;
//                 O_B += P_B(j) V(j);  S_B(j+1) = Q_B K(j+1)^T.  The tensor pipe executes in order, so a
//                 product may overwrite the TMEM columns the product issued just before it reads (S over P).
//                 The first S of the next item is issued as soon as a tile's last P V is.
//   warps 4-7     softmax of tile A, warps 8-11 softmax of tile B: thread r owns query row r (TMEM lane r)
//                 and all 128 key columns of a step, so the row maximum and the row sum are plain loops in
//                 registers: no exchange between threads.  P (f16 pairs) goes back into TMEM over the scores.
//                 O is rescaled (by the same threads, in TMEM) only when a row's maximum grew by more than 2^8.
//                 When a tile's last product has landed, the same threads read O from TMEM, normalise by the row
//                 sum, convert, store and write the row lse; with the causal mask tile A does this while tile B
//                 runs its extra (diagonal) step, and tile B while tile A already works on the next item.
//   warps 2-3     idle (they keep the softmax warps on TMEM lane quadrants 0-3: a warp reaches lanes 32*(warp%4)...)
// TMEM: S_A | S_B | O_A | O_B, 128 columns each (O: head_dim columns).  Scale, causal mask, softmax and both
// products happen in this one pass; the T x T scores never reach global memory.
#include <type_traits>

#include "sm100_ptx.cuh"
#include "tma_host.cuh"

namespace {
using namespace sm100;

constexpr int BM = 128;
constexpr int BN = 128;
constexpr uint32_t BLOCK_BYTES = 128 * 128;   // one 64-column block of a 128-row tile
constexpr float LOG2E = 1.4426950408889634f;
constexpr float LN2 = 0.6931471805599453f;
constexpr float RESCALE_THRESHOLD = 8.0f;     // log2 units: P stays below 2^8, safe in f16
constexpr int FWD2_THREADS = 384;

struct Fwd2Params {
    __half* o;
    float* lse;
    long long so_b, so_h, so_t;
    int B, H, T;
    int causal;
    float scale;
    unsigned int* err;
    const int4* sched;          // table[n * grid + cta] = {slot, slice, batch, head} over nq2 double tiles per slice
    int sched_rows;
};

__device__ __forceinline__ float ex2f(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

template <int D>
struct Fwd2Smem {
    static constexpr uint32_t TILE = 128u * D * 2u;
    static constexpr int KS = (D == 128) ? 2 : 3;            // K ring stages
    static constexpr int VS = (D == 128) ? 2 : 3;            // V ring stages
    static constexpr uint32_t Q = 0;                         // Q_A, Q_B
    static constexpr uint32_t K = Q + 2 * TILE;
    static constexpr uint32_t V = K + KS * TILE;
    static constexpr uint32_t BARS = V + VS * TILE;
    static constexpr uint32_t TOTAL = BARS + 320;
};

// per-tile barriers come in pairs (index + tile)
enum Fwd2Bar { G_Q_FULL = 0, G_Q_EMPTY = 2, G_S_FULL = 4, G_P_FULL = 6, G_PV_DONE = 8, G_O_DONE = 10, G_O_FREE = 12,
               G_K_FULL = 14, G_K_EMPTY = 17, G_V_FULL = 20, G_V_EMPTY = 23, G_COUNT = 26 };

// One work item as every role sees it.
struct Item2 {
    int valid;
    int qt2, bh, b, h;
    int hasB;
    int ntA, ntB, nt;           // key tiles for tile A, for tile B (0 when absent), and their maximum
};

__device__ __forceinline__ int4 table2(const Fwd2Params& p, int idx, int nq2, int n_items) {
    if (p.sched) return idx < p.sched_rows ? p.sched[idx * (int)gridDim.x + (int)blockIdx.x] : make_int4(-1, 0, 0, 0);
    const int v = (int)blockIdx.x + idx * (int)gridDim.x;
    if (v >= n_items) return make_int4(-1, 0, 0, 0);
    const int BH = p.B * p.H;
    const int group = v / (16 * nq2);
    const int gsize = min(16, BH - group * 16);
    const int within = v - group * 16 * nq2;
    const int s = group * 16 + within % gsize;
    return make_int4(within / gsize, s, s / p.H, s % p.H);
}

__device__ __forceinline__ Item2 decode2(const Fwd2Params& p, int4 e, int nq, int nq2);

// This CTA's item list, one entry ahead: the table read for item n+1 (an L2 round trip) is issued when item n
// becomes current and not looked at before the next advance.
struct Cursor2 {
    int n;
    int4 e_next;
    Item2 it;
    __device__ __forceinline__ void init(const Fwd2Params& p, int nq, int nq2, int n_items);
    __device__ __forceinline__ void advance(const Fwd2Params& p, int nq, int nq2, int n_items);
};

__device__ __forceinline__ Item2 decode2(const Fwd2Params& p, int4 e, int nq, int nq2) {
    Item2 it;
    it.valid = e.x >= 0;
    it.qt2 = nq2 - 1 - e.x;                                  // heaviest (latest) double tiles first
    it.bh = e.y; it.b = e.z; it.h = e.w;
    it.hasB = (2 * it.qt2 + 1) < nq;
    it.ntA = p.causal ? 2 * it.qt2 + 1 : nq;
    it.ntB = it.hasB ? (p.causal ? 2 * it.qt2 + 2 : nq) : 0;
    it.nt = it.ntA > it.ntB ? it.ntA : it.ntB;
    return it;
}

__device__ __forceinline__ void Cursor2::init(const Fwd2Params& p, int nq, int nq2, int n_items) {
    n = 0;
    it = decode2(p, table2(p, 0, nq2, n_items), nq, nq2);
    e_next = table2(p, 1, nq2, n_items);
}
__device__ __forceinline__ void Cursor2::advance(const Fwd2Params& p, int nq, int nq2, int n_items) {
    it = decode2(p, e_next, nq, nq2);
    ++n;
    e_next = table2(p, n + 1, nq2, n_items);
}

template <int D>
__global__ void __launch_bounds__(FWD2_THREADS, 1)
attn_fwd2_f16_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                     const __grid_constant__ CUtensorMap tmap_v, const Fwd2Params p) {
    using L = Fwd2Smem<D>;
    constexpr uint32_t TILE_BYTES = L::TILE;
    constexpr int DBLK = D / 64;
    constexpr int KS = L::KS, VS = L::VS;
    constexpr uint32_t TMEM_COLS = 512;
    constexpr uint32_t TM_S = 0, TM_O = 256;                 // S_A, S_B at 0, 128; O_A, O_B at 256, 256 + D

    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t* sQ = smem + L::Q;
    uint8_t* sK = smem + L::K;
    uint8_t* sV = smem + L::V;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::BARS);
    uint32_t* tmem_base_s = reinterpret_cast<uint32_t*>(bars + G_COUNT);
    volatile uint32_t* abort_s = tmem_base_s + 1;
    uint32_t* skip_s = tmem_base_s + 2;

    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const int nq = (p.T + BM - 1) / BM;
    const int nq2 = (nq + 1) / 2;
    const int n_items = p.B * p.H * nq2;

    if (threadIdx.x == 0) {
        *abort_s = 0;
        uint32_t skip = (*(volatile unsigned int*)p.err != 0) ? 1u : 0u;   // an earlier kernel gave up: exit at once
        if ((smem_u32(smem) & 1023u) != 0) {
            atomicCAS(p.err, 0u, DEERS_KERR_FWD_F16 | 0x20);
            skip = 1;
        }
        *skip_s = skip;
        for (int x = 0; x < 2; ++x) {
            mbar_init(&bars[G_Q_FULL + x], 1); mbar_init(&bars[G_Q_EMPTY + x], 1);
            mbar_init(&bars[G_S_FULL + x], 1); mbar_init(&bars[G_P_FULL + x], 128);
            mbar_init(&bars[G_PV_DONE + x], 1);
            mbar_init(&bars[G_O_DONE + x], 1); mbar_init(&bars[G_O_FREE + x], 128);
        }
        for (int s = 0; s < 3; ++s) {
            mbar_init(&bars[G_K_FULL + s], 1); mbar_init(&bars[G_K_EMPTY + s], 1);
            mbar_init(&bars[G_V_FULL + s], 1); mbar_init(&bars[G_V_EMPTY + s], 1);
        }
        fence_barrier_init();
        tma_prefetch_desc(&tmap_q); tma_prefetch_desc(&tmap_k); tma_prefetch_desc(&tmap_v);
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

    if (warp < 4) {
        if (warp == 0 && lane == 0) {
            // ------------------------------ TMA producer ------------------------------
            uint32_t gk = 0, gv = 0, useB = 0;
            bool ok = true;
            Cursor2 c;
            for (c.init(p, nq, nq2, n_items); ok && c.it.valid; c.advance(p, nq, nq2, n_items)) {
                const Item2& it = c.it;
                const int n = c.n;
                if (!mbar_wait(ws, &bars[G_Q_EMPTY + 0], ((uint32_t)n & 1u) ^ 1u, DEERS_KERR_FWD_F16 | 0x41)) break;
                mbar_arrive_expect_tx(&bars[G_Q_FULL + 0], TILE_BYTES);
#pragma unroll
                for (int blk = 0; blk < DBLK; ++blk)
                    tma_load_4d(sQ + blk * BLOCK_BYTES, &tmap_q, &bars[G_Q_FULL + 0], blk * 64, (2 * it.qt2) * BM, it.h, it.b);
                if (it.hasB) {
                    if (!mbar_wait(ws, &bars[G_Q_EMPTY + 1], (useB & 1u) ^ 1u, DEERS_KERR_FWD_F16 | 0x42)) break;
                    mbar_arrive_expect_tx(&bars[G_Q_FULL + 1], TILE_BYTES);
#pragma unroll
                    for (int blk = 0; blk < DBLK; ++blk)
                        tma_load_4d(sQ + TILE_BYTES + blk * BLOCK_BYTES, &tmap_q, &bars[G_Q_FULL + 1], blk * 64,
                                    (2 * it.qt2 + 1) * BM, it.h, it.b);
                    ++useB;
                }
                for (int j = 0; j < it.nt; ++j) {
                    const uint32_t sk = gk % (uint32_t)KS, sv = gv % (uint32_t)VS;
                    if (!mbar_wait(ws, &bars[G_K_EMPTY + sk], ((gk / (uint32_t)KS) & 1u) ^ 1u, DEERS_KERR_FWD_F16 | 0x43)) { ok = false; break; }
                    mbar_arrive_expect_tx(&bars[G_K_FULL + sk], TILE_BYTES);
#pragma unroll
                    for (int blk = 0; blk < DBLK; ++blk)
                        tma_load_4d(sK + sk * TILE_BYTES + blk * BLOCK_BYTES, &tmap_k, &bars[G_K_FULL + sk], blk * 64, j * BN, it.h, it.b);
                    ++gk;
                    if (!mbar_wait(ws, &bars[G_V_EMPTY + sv], ((gv / (uint32_t)VS) & 1u) ^ 1u, DEERS_KERR_FWD_F16 | 0x44)) { ok = false; break; }
                    mbar_arrive_expect_tx(&bars[G_V_FULL + sv], TILE_BYTES);
#pragma unroll
                    for (int blk = 0; blk < DBLK; ++blk)
                        tma_load_4d(sV + sv * TILE_BYTES + blk * BLOCK_BYTES, &tmap_v, &bars[G_V_FULL + sv], blk * 64, j * BN, it.h, it.b);
                    ++gv;
                }
            }
        } else if (warp == 1 && lane == 0) {
            // ------------------------------ MMA issuer ------------------------------
            constexpr uint32_t IDESC_S = idesc_f16(BM, BN, 0, 0);      // S: K-major A (Q) and B (K)
            constexpr uint32_t IDESC_O = idesc_f16(BM, D, 0, 1);       // O: A = P from TMEM, B = V MN-major
            constexpr uint64_t STAGE_STEP = TILE_BYTES >> 4;
            const uint64_t q_km0 = desc_kmajor(smem_u32(sQ), 0, BLOCK_BYTES);
            const uint64_t k_km0 = desc_kmajor(smem_u32(sK), 0, BLOCK_BYTES);
            const uint64_t v_mn0 = desc_mnmajor(smem_u32(sV), 0, BLOCK_BYTES);
            uint32_t gk = 0, gv = 0;                 // ring positions of the next K tile to use for S, next V for P V
            uint32_t cnt[2] = {0, 0};                // tile-steps so far per tile: phase of S_FULL / P_FULL / PV_DONE
            uint32_t use[2] = {0, 0};                // items so far that had this tile: phase of Q / O barriers
            bool ok = true;

            // S_X(item, j) = Q_X K(j)^T into S_X; the K tile is at ring position `kpos` and must have landed.
            auto issue_s = [&](int x, const Item2& it, int j, uint32_t kpos) {
                const uint32_t sk = kpos % (uint32_t)KS;
                const uint64_t q_km = q_km0 + (uint64_t)x * STAGE_STEP, k_km = k_km0 + (uint64_t)sk * STAGE_STEP;
                const uint32_t d_tmem = tmem + TM_S + (uint32_t)x * 128u;
#pragma unroll
                for (int ks = 0; ks < D / 16; ++ks)
                    umma_ss(d_tmem, q_km + kmajor_step(ks, BLOCK_BYTES), k_km + kmajor_step(ks, BLOCK_BYTES), IDESC_S, ks > 0);
                umma_commit(&bars[G_S_FULL + x]);
                if (j == (x ? it.ntB : it.ntA) - 1) umma_commit(&bars[G_Q_EMPTY + x]);   // last product reading this Q
            };
            auto issue_pv = [&](int x, const Item2& it, int j, uint32_t vpos) {
                const uint32_t sv = vpos % (uint32_t)VS;
                const uint64_t v_mn = v_mn0 + (uint64_t)sv * STAGE_STEP;
                const uint32_t o_tmem = tmem + TM_O + (uint32_t)x * D;
                const uint32_t p_tmem = tmem + TM_S + (uint32_t)x * 128u;      // P sits where this step's S was
#pragma unroll
                for (int ks = 0; ks < BN / 16; ++ks)
                    umma_ts(o_tmem, p_tmem + (uint32_t)ks * 8u, v_mn + mnmajor_step(ks), IDESC_O, (j > 0 || ks > 0));
                umma_commit(&bars[G_PV_DONE + x]);
                if (j == (x ? it.ntB : it.ntA) - 1) umma_commit(&bars[G_O_DONE + x]);
            };

            int n = 0;
            Item2 cur = decode2(p, table2(p, 0, nq2, n_items), nq, nq2);
            int4 e_nxt = table2(p, 1, nq2, n_items);
            bool pre = false;                        // the first S of `cur` went out during the previous item's last step
            while (ok && cur.valid) {
                const Item2 nxt = decode2(p, e_nxt, nq, nq2);
                e_nxt = table2(p, n + 2, nq2, n_items);          // looked at one item from now
                if (!pre) {
                    // ---- first S of the item (only the very first item of this CTA comes this way)
                    const uint32_t sk = gk % (uint32_t)KS;
                    if (!mbar_wait(ws, &bars[G_K_FULL + sk], (gk / (uint32_t)KS) & 1u, DEERS_KERR_FWD_F16 | 0x51)) break;
                    if (!mbar_wait(ws, &bars[G_Q_FULL + 0], use[0] & 1u, DEERS_KERR_FWD_F16 | 0x52)) break;
                    tc_fence_after_sync();
                    issue_s(0, cur, 0, gk);
                    if (cur.hasB) {
                        if (!mbar_wait(ws, &bars[G_Q_FULL + 1], use[1] & 1u, DEERS_KERR_FWD_F16 | 0x53)) break;
                        tc_fence_after_sync();
                        issue_s(1, cur, 0, gk);
                    }
                    umma_commit(&bars[G_K_EMPTY + sk]);          // every tile has issued its reads of K(0)
                    ++gk;
                }
                for (int j = 0; j < cur.nt; ++j) {
                    const bool last = (j == cur.nt - 1);
                    const bool more = !last;                     // K(j+1) of this item follows
                    const bool ahead = last && nxt.valid;        // K(0) of the next item follows
                    const uint32_t sv = gv % (uint32_t)VS, sk = gk % (uint32_t)KS;
                    bool v_ready = false;
                    // ---- tile A: O_A += P_A(j) V(j)
                    if (j < cur.ntA) {
                        if (!mbar_wait(ws, &bars[G_P_FULL + 0], cnt[0] & 1u, DEERS_KERR_FWD_F16 | 0x54)) { ok = false; break; }
                        if (!mbar_wait(ws, &bars[G_V_FULL + sv], (gv / (uint32_t)VS) & 1u, DEERS_KERR_FWD_F16 | 0x55)) { ok = false; break; }
                        v_ready = true;
                        if (j == 0 && !mbar_wait(ws, &bars[G_O_FREE + 0], (use[0] & 1u) ^ 1u, DEERS_KERR_FWD_F16 | 0x56)) { ok = false; break; }
                        tc_fence_after_sync();
                        issue_pv(0, cur, j, gv);
                        ++cnt[0];
                    }
                    // ---- the key tile both tiles' next S needs: K(j+1), or K(0) of the next item
                    if (more || ahead) {
                        if (!mbar_wait(ws, &bars[G_K_FULL + sk], (gk / (uint32_t)KS) & 1u, DEERS_KERR_FWD_F16 | 0x57)) { ok = false; break; }
                        tc_fence_after_sync();
                    }
                    if (j + 1 < cur.ntA) {
                        issue_s(0, cur, j + 1, gk);
                    } else if (ahead) {
                        // tile A is done with this item: the first S of its next item runs under this step's softmax
                        if (!mbar_wait(ws, &bars[G_Q_FULL + 0], (use[0] + 1u) & 1u, DEERS_KERR_FWD_F16 | 0x59)) { ok = false; break; }
                        tc_fence_after_sync();
                        issue_s(0, nxt, 0, gk);
                    }
                    // ---- tile B: O_B += P_B(j) V(j)
                    if (j < cur.ntB) {
                        if (!mbar_wait(ws, &bars[G_P_FULL + 1], cnt[1] & 1u, DEERS_KERR_FWD_F16 | 0x5a)) { ok = false; break; }
                        if (!v_ready && !mbar_wait(ws, &bars[G_V_FULL + sv], (gv / (uint32_t)VS) & 1u, DEERS_KERR_FWD_F16 | 0x5b)) { ok = false; break; }
                        if (j == 0 && !mbar_wait(ws, &bars[G_O_FREE + 1], (use[1] & 1u) ^ 1u, DEERS_KERR_FWD_F16 | 0x5c)) { ok = false; break; }
                        tc_fence_after_sync();
                        issue_pv(1, cur, j, gv);
                        ++cnt[1];
                    }
                    umma_commit(&bars[G_V_EMPTY + sv]);          // every product reading V(j) has been issued
                    ++gv;
                    if (j + 1 < cur.ntB) {
                        issue_s(1, cur, j + 1, gk);
                    } else if (ahead && nxt.hasB) {
                        if (!mbar_wait(ws, &bars[G_Q_FULL + 1], (use[1] + (cur.hasB ? 1u : 0u)) & 1u, DEERS_KERR_FWD_F16 | 0x5d)) { ok = false; break; }
                        tc_fence_after_sync();
                        issue_s(1, nxt, 0, gk);
                    }
                    if (more || ahead) {
                        umma_commit(&bars[G_K_EMPTY + sk]);      // every tile has issued its reads of this key tile
                        ++gk;
                    }
                }
                if (!ok) break;
                ++use[0];
                if (cur.hasB) ++use[1];
                pre = nxt.valid;
                cur = nxt;
                ++n;
            }
        }
    } else {
        // ------------------------------ softmax and epilogue of tile x ------------------------------
        const int x = (warp - 4) >> 2;                          // 0: tile A, 1: tile B
        const int lane_base = (warp & 3) * 32;
        const int row = lane_base + lane;                       // row inside the query tile == TMEM lane
        const uint32_t t_lane = (uint32_t)lane_base << 16;
        const float sl2 = p.scale * LOG2E;
        const uint32_t ts = tmem + TM_S + (uint32_t)x * 128u + t_lane;
        const uint32_t to = tmem + TM_O + (uint32_t)x * D + t_lane;
        uint32_t cnt = 0, use = 0;
        bool alive = true;
        Cursor2 c;
        for (c.init(p, nq, nq2, n_items); alive && c.it.valid; c.advance(p, nq, nq2, n_items)) {
            const Item2& it = c.it;
            if (x == 1 && !it.hasB) continue;
            const int qt = 2 * it.qt2 + x;
            const int ntiles = x ? it.ntB : it.ntA;
            float m_used = -INFINITY, l = 0.f;
            for (int j = 0; j < ntiles; ++j, ++cnt) {
                if (!__all_sync(0xffffffffu, mbar_wait(ws, &bars[G_S_FULL + x], cnt & 1u, DEERS_KERR_FWD_F16 | 0x61))) { alive = false; break; }
                tc_fence_after_sync();
                // Two sweeps over the row's 128 scores, 32 columns at a time (the next chunk's TMEM load is in
                // flight while this one is worked on): the row maximum first, then exponentials, row sum and P.
                // Reading the scores twice keeps a thread at a few dozen live registers instead of 128 + 64.
                // Steps that touch the diagonal or the end of the sequence mask with -inf (columns beyond `lim`);
                // the scale is folded into the exponent's FFMA.
                const int k0 = j * BN;
                int lim = BN - 1;
                if (k0 + BN > p.T) lim = p.T - 1 - k0;              // keys end at T
                if (p.causal && j == qt) lim = min(lim, row);       // diagonal tile (k0 == q0): key <= query
                const bool pos = sl2 >= 0.f;
                const bool edge = lim < BN - 1;                     // warp-uniform on all but the diagonal tile
                const bool warp_edge = __any_sync(0xffffffffu, edge);
                float mx;
                auto sweep_max = [&](auto mask_tag) {
                    constexpr bool MASK = decltype(mask_tag)::value;
                    uint32_t a[32], b[32];
                    float m0 = pos ? -INFINITY : INFINITY, m1 = m0, m2 = m0, m3 = m0;
                    tmem_ld_x32(ts, a);
                    tmem_wait_ld();
#pragma unroll
                    for (int ch = 0; ch < BN / 32; ch += 2) {
                        tmem_ld_x32(ts + (ch + 1) * 32, b);
#pragma unroll
                        for (int i = 0; i < 32; i += 4) {
                            const int c0 = ch * 32 + i;
                            const float v0 = __uint_as_float(a[i]), v1 = __uint_as_float(a[i + 1]);
                            const float v2 = __uint_as_float(a[i + 2]), v3 = __uint_as_float(a[i + 3]);
                            if (pos) {
                                m0 = (!MASK || c0 <= lim) ? fmaxf(m0, v0) : m0; m1 = (!MASK || c0 + 1 <= lim) ? fmaxf(m1, v1) : m1;
                                m2 = (!MASK || c0 + 2 <= lim) ? fmaxf(m2, v2) : m2; m3 = (!MASK || c0 + 3 <= lim) ? fmaxf(m3, v3) : m3;
                            } else {
                                m0 = (!MASK || c0 <= lim) ? fminf(m0, v0) : m0; m1 = (!MASK || c0 + 1 <= lim) ? fminf(m1, v1) : m1;
                                m2 = (!MASK || c0 + 2 <= lim) ? fminf(m2, v2) : m2; m3 = (!MASK || c0 + 3 <= lim) ? fminf(m3, v3) : m3;
                            }
                        }
                        tmem_wait_ld();
                        if (ch + 2 < BN / 32) tmem_ld_x32(ts + (ch + 2) * 32, a);
#pragma unroll
                        for (int i = 0; i < 32; i += 4) {
                            const int c0 = (ch + 1) * 32 + i;
                            const float v0 = __uint_as_float(b[i]), v1 = __uint_as_float(b[i + 1]);
                            const float v2 = __uint_as_float(b[i + 2]), v3 = __uint_as_float(b[i + 3]);
                            if (pos) {
                                m0 = (!MASK || c0 <= lim) ? fmaxf(m0, v0) : m0; m1 = (!MASK || c0 + 1 <= lim) ? fmaxf(m1, v1) : m1;
                                m2 = (!MASK || c0 + 2 <= lim) ? fmaxf(m2, v2) : m2; m3 = (!MASK || c0 + 3 <= lim) ? fmaxf(m3, v3) : m3;
                            } else {
                                m0 = (!MASK || c0 <= lim) ? fminf(m0, v0) : m0; m1 = (!MASK || c0 + 1 <= lim) ? fminf(m1, v1) : m1;
                                m2 = (!MASK || c0 + 2 <= lim) ? fminf(m2, v2) : m2; m3 = (!MASK || c0 + 3 <= lim) ? fminf(m3, v3) : m3;
                            }
                        }
                        if (ch + 2 < BN / 32) tmem_wait_ld();
                    }
                    mx = (pos ? fmaxf(fmaxf(m0, m1), fmaxf(m2, m3)) : fminf(fminf(m0, m1), fminf(m2, m3))) * sl2;
                };
                if (warp_edge) sweep_max(std::true_type{}); else sweep_max(std::false_type{});
                const float m_new = fmaxf(m_used, mx);
                // Lazy rescale: keep the old reference max unless this row grew by more than 2^8.
                const bool grow = (j > 0) && (m_new - m_used > RESCALE_THRESHOLD);
                const float m_cur = (j == 0 || grow) ? m_new : m_used;
                const float m_safe = (m_cur == -INFINITY) ? 0.f : m_cur;
                const float alpha = (j == 0) ? 0.f : ex2f(m_used - m_safe);
                const bool warp_grow = __any_sync(0xffffffffu, grow);
                if (j > 0 && warp_grow) {
                    // O += P V of the previous step must have landed before O is rescaled.
                    if (!__all_sync(0xffffffffu, mbar_wait(ws, &bars[G_PV_DONE + x], (cnt - 1u) & 1u, DEERS_KERR_FWD_F16 | 0x62))) { alive = false; break; }
                    tc_fence_after_sync();
#pragma unroll
                    for (int cc = 0; cc < D / 32; ++cc) {
                        uint32_t r[32];
                        tmem_ld_x32(to + cc * 32, r);
                        tmem_wait_ld();
#pragma unroll
                        for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
                        tmem_st_x32(to + cc * 32, r);
                    }
                }
                // Second sweep.  P (f16 pairs) replaces the first 64 columns of this tile's S, sixteen packed columns
                // per chunk: a chunk of P lands on score columns that have already been read.
                float rs0 = 0.f, rs1 = 0.f;
                auto sweep_exp = [&](auto mask_tag) {
                    constexpr bool MASK = decltype(mask_tag)::value;
                    uint32_t a[32], b[32];
                    tmem_ld_x32(ts, a);
                    tmem_wait_ld();
#pragma unroll
                    for (int ch = 0; ch < BN / 32; ch += 2) {
                        tmem_ld_x32(ts + (ch + 1) * 32, b);
                        uint32_t pk[16];
#pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            const int c0 = ch * 32 + 2 * i;
                            float e0 = ex2f(fmaf(__uint_as_float(a[2 * i]), sl2, -m_safe));
                            float e1 = ex2f(fmaf(__uint_as_float(a[2 * i + 1]), sl2, -m_safe));
                            if (MASK) {
                                e0 = (c0 <= lim) ? e0 : 0.f;
                                e1 = (c0 + 1 <= lim) ? e1 : 0.f;
                            }
                            rs0 += e0; rs1 += e1;
                            pk[i] = pack_half2(e0, e1);
                        }
                        tmem_wait_ld();                              // chunk ch+1 is in registers
                        tmem_st_x16(ts + ch * 16, pk);
                        if (ch + 2 < BN / 32) tmem_ld_x32(ts + (ch + 2) * 32, a);
#pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            const int c0 = (ch + 1) * 32 + 2 * i;
                            float e0 = ex2f(fmaf(__uint_as_float(b[2 * i]), sl2, -m_safe));
                            float e1 = ex2f(fmaf(__uint_as_float(b[2 * i + 1]), sl2, -m_safe));
                            if (MASK) {
                                e0 = (c0 <= lim) ? e0 : 0.f;
                                e1 = (c0 + 1 <= lim) ? e1 : 0.f;
                            }
                            rs0 += e0; rs1 += e1;
                            pk[i] = pack_half2(e0, e1);
                        }
                        if (ch + 2 < BN / 32) tmem_wait_ld();        // chunk ch+2 is in registers: its columns may be overwritten later
                        tmem_st_x16(ts + (ch + 1) * 16, pk);
                    }
                };
                if (warp_edge) sweep_exp(std::true_type{}); else sweep_exp(std::false_type{});
                l = l * alpha + (rs0 + rs1);
                m_used = m_cur;
                tmem_wait_st();
                tc_fence_before_sync();
                mbar_arrive(&bars[G_P_FULL + x]);
            }
            if (!alive) break;
            // ---- epilogue of this tile: its last product has been issued right after the hand-over above
            if (!__all_sync(0xffffffffu, mbar_wait(ws, &bars[G_O_DONE + x], use & 1u, DEERS_KERR_FWD_F16 | 0x72))) { alive = false; break; }
            tc_fence_after_sync();
            ++use;
            const float inv = 1.f / l;
            const int q0 = qt * BM;
            // The thread's row of O, 64 columns at a time, as 16-byte pieces transposed within 8-lane groups so
            // that every store instruction writes whole 128-byte row segments.
            const int grow0 = q0 + lane_base + (lane & ~7);
            __half* ob = p.o + it.b * p.so_b + it.h * p.so_h + (lane & 7) * 8;
#pragma unroll 1
            for (int part = 0; part < D / 64; ++part) {
                uint32_t r[64];
                uint4 pc[8];
                tmem_ld_x32(to + part * 64, *reinterpret_cast<uint32_t(*)[32]>(&r[0]));
                tmem_ld_x32(to + part * 64 + 32, *reinterpret_cast<uint32_t(*)[32]>(&r[32]));
                tmem_wait_ld();
                if (part == D / 64 - 1) {                        // the accumulator is in registers: release it
                    tc_fence_before_sync();
                    mbar_arrive(&bars[G_O_FREE + x]);
                }
#pragma unroll
                for (int q8 = 0; q8 < 8; ++q8) pc[q8] = pack8_f16(r + q8 * 8, inv);
                transpose_pieces<8>(pc, (uint32_t)lane);
#pragma unroll
                for (int cc = 0; cc < 8; ++cc) {
                    const int grow = grow0 + cc;
                    if (grow < p.T) *reinterpret_cast<uint4*>(ob + (long long)grow * p.so_t + part * 64) = pc[cc];
                }
            }
            if (q0 + row < p.T) p.lse[(long long)it.bh * p.T + q0 + row] = (m_used + log2f(l)) * LN2;
        }
    }

    __syncwarp();
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem, TMEM_COLS);
}

template <int D>
int fwd2_launch(deers_ctx* ctx, const deers_attn_desc* d, const void* q, const void* k, const void* v, void* o,
                float* lse) {
    CUtensorMap tq, tk, tv;
    int rc;
    if ((rc = make_tmap_bhtd_f16(ctx, &tq, q, d->B, d->H, d->T, D, d->q_strides, BM))) return rc;
    if ((rc = make_tmap_bhtd_f16(ctx, &tk, k, d->B, d->H, d->T, D, d->k_strides, BN))) return rc;
    if ((rc = make_tmap_bhtd_f16(ctx, &tv, v, d->B, d->H, d->T, D, d->v_strides, BN))) return rc;
    Fwd2Params p;
    p.o = (__half*)o; p.lse = lse;
    p.so_b = d->o_strides[0]; p.so_h = d->o_strides[1]; p.so_t = d->o_strides[2];
    p.B = d->B; p.H = d->H; p.T = d->T; p.causal = d->causal; p.scale = d->scale; p.err = ctx->dev_err;
    const size_t smem = Fwd2Smem<D>::TOTAL;
    DEERS_CUDA_TRY(ctx, cudaFuncSetAttribute(attn_fwd2_f16_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const long long nq = (d->T + BM - 1) / BM;
    const long long nq2 = (nq + 1) / 2;
    const long long items = nq2 * d->B * d->H;
    if (items > 0x7fffffffLL) return DEERS_ERR_SHAPE;
    const unsigned grid = (unsigned)(items < ctx->sm_count ? items : ctx->sm_count);
    p.sched = deers_get_schedule(ctx, d->B, d->H, (int)nq2, d->causal, (int)grid, &p.sched_rows);
    {
        KernelTimerScope ts(ctx, DEERS_K_FWD);
        attn_fwd2_f16_kernel<D><<<grid, FWD2_THREADS, smem, ctx->stream>>>(tq, tk, tv, p);
    }
    ctx->launches += 1;
    DEERS_CUDA_TRY(ctx, cudaGetLastError());
    return DEERS_OK;
}

}  // namespace

int launch_attn_fwd2_f16(deers_ctx* ctx, const deers_attn_desc* d, const void* q, const void* k, const void* v,
                         void* o, float* lse) {
    if (d->D == 64) return fwd2_launch<64>(ctx, d, q, k, v, o, lse);
    if (d->D == 128) return fwd2_launch<128>(ctx, d, q, k, v, o, lse);
    return DEERS_ERR_UNSUPPORTED;
}
