// f16 causal attention forward for sm_100a.
//
// Persistent kernel: one CTA per SM walks a strided, heaviest-first list of work items, an item
// being 128 query rows of one (batch, head) slice together with the key/value tiles (128 rows
// each) at or left of its diagonal.  The whole list is treated as ONE stream of (item, KV tile)
// steps, so loads and the S product run two steps ahead across item boundaries.
//   warp 0      TMA producer: Q per item (2 buffers), K and V tiles through 2-stage rings
//   last warp   issues the S = Q K^T products into a double-buffered TMEM tile, two steps ahead
//   warp 1      issues the O += P V products, with P read from TMEM and the accumulator resident
//               in TMEM (two O accumulators alternate between items).  One thread cannot issue
//               both streams fast enough: its barrier waits and commits between the batches of
//               eight instructions left the tensor core idle a third of the time.  The two
//               streams are ordered by barriers only (S of step g+2 overwrites P of step g once
//               the product that read it has completed).
//   warps 2-17  four softmax warpgroups that split the 128 key columns of a step (32 each); thread r
//               of a warpgroup owns query row r (= TMEM lane r).  Per step a thread reads its 32
//               scores, exchanges its partial row max with the twin threads of the other
//               warpgroups, keeps the running max / partial sum, stores P (f16 pairs) back into
//               TMEM over the scores it has just read, and rescales its quarter of O only when the
//               row max grew by more than 2^8.  At the end of an item the partial sums are
//               combined, O is normalised and O and the row lse are stored.
// Scale, causal mask, softmax and both products happen in this one pass; the T x T scores
// never reach global memory.
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
// Softmax warpgroups per CTA.  Four (32 key columns each) rather than two: the softmax threads are bound by
// instruction latency, not by any one pipe, and four resident warps per scheduler hide it better than two.
constexpr int NWG = 4;
constexpr int CW = 128 / NWG;                 // key columns of a step per warpgroup
constexpr int FWD_THREADS = 32 * (2 + 4 * NWG + 1);
constexpr int S_WARP = 2 + 4 * NWG;           // the warp that issues S

struct FwdParams {
    __half* o;
    float* lse;
    long long so_b, so_h, so_t;
    int B, H, T;
    int causal;
    float scale;
    unsigned int* err;
    const int4* sched;          // balanced schedule table[n * grid + cta] = {slot, slice, batch, head} (or nullptr: strided)
    int sched_rows;
};

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Dynamic shared memory only; the base must be 1024-byte aligned for the 128-byte swizzle (checked).
template <int D>
struct FwdSmem {
    static constexpr uint32_t TILE = 128u * D * 2u;
    static constexpr uint32_t Q = 0;                         // two buffers (alternate between items)
    static constexpr uint32_t K = Q + 2 * TILE;              // two stages
    static constexpr uint32_t V = K + 2 * TILE;              // two stages
    static constexpr uint32_t XCH = V + 2 * TILE;            // [2 parities][NWG warpgroups][128] partial row max
    static constexpr uint32_t LX = XCH + 2 * NWG * BM * 4;   // [2 parities][NWG warpgroups][128] partial row sum
    static constexpr uint32_t BARS = LX + 2 * NWG * BM * 4;
    static constexpr uint32_t TOTAL = BARS + 256;
};

// P_FULL is split by step parity: S runs two steps ahead of P V, so the softmax threads can hand over
// P of steps g and g+1 before the MMA thread has looked at step g; one barrier per parity keeps each
// barrier at most one phase ahead of its waiter.
// S_FULL (all S products of a step have finished) also tells the producer that the step's K stage is
// free; PV_DONE (all P V products of a step have finished) also frees the V stage, tells the S
// issuer that the step's P has been consumed and orders a rescale of O behind the product.
enum FwdBar { F_Q_FULL = 0, F_Q_EMPTY = 2, F_K_FULL = 4, F_V_FULL = 6, F_PV_DONE = 8, F_S_FULL = 10,
              F_P_FULL = 12, F_XCH = 14, F_LX = 15, F_O_DONE = 16, F_O_FREE = 18, F_COUNT = 20 };

// Work order: groups of 16 slices; inside a group the heaviest (latest) query tiles of all its
// slices come first (balance) and the group's K and V (a few MB) stay in L2.
struct WorkCursor {
    int n;          // index of the item inside this CTA's list
    int w;          // >= 0 while the cursor points at an item
    int4 e_next;    // table entry of the item after this one (prefetched)
    int j;          // KV tile inside the item
    int ntiles, qt, bh, b, h;
    // {slot, slice, batch, head} of this CTA's idx-th item; slot < 0 past the end.  With a host-built table
    // this is one load; the strided fallback pays the integer divisions.
    __device__ __forceinline__ int4 table(const FwdParams& p, int idx, int nq, int n_items) const {
        if (p.sched) return idx < p.sched_rows ? p.sched[idx * (int)gridDim.x + (int)blockIdx.x] : make_int4(-1, 0, 0, 0);
        const int v = (int)blockIdx.x + idx * (int)gridDim.x;
        if (v >= n_items) return make_int4(-1, 0, 0, 0);
        const int BH = p.B * p.H;
        const int group = v / (16 * nq);
        const int gsize = min(16, BH - group * 16);
        const int within = v - group * 16 * nq;
        const int s = group * 16 + within % gsize;
        return make_int4(within / gsize, s, s / p.H, s % p.H);
    }
    // Item n becomes current; the table entry of item n+1 is requested now and not looked at before the
    // next call, so its L2 round trip is off the item boundary.
    __device__ __forceinline__ void fetch(const FwdParams& p, int nq, int n_items) {
        const int4 e = e_next;
        e_next = table(p, n + 1, nq, n_items);
        w = e.x;
        if (e.x >= 0) {
            qt = nq - 1 - e.x;                              // heaviest (latest) query tiles first
            bh = e.y; b = e.z; h = e.w;
            ntiles = p.causal ? qt + 1 : nq;
        }
    }
    __device__ __forceinline__ void init(const FwdParams& p, int nq, int n_items) {
        n = 0; j = 0;
        e_next = table(p, 0, nq, n_items);
        fetch(p, nq, n_items);
    }
    __device__ __forceinline__ bool valid(int) const { return w >= 0; }
    __device__ __forceinline__ void advance(const FwdParams& p, int nq, int n_items) {
        if (++j == ntiles) {
            j = 0; ++n;
            fetch(p, nq, n_items);
        }
    }
};

template <int D>
__global__ void __launch_bounds__(FWD_THREADS, 1)
attn_fwd_f16_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                    const __grid_constant__ CUtensorMap tmap_v, const FwdParams p) {
    using L = FwdSmem<D>;
    constexpr uint32_t TILE_BYTES = L::TILE;
    constexpr int DBLK = D / 64;
    constexpr int DH = D / NWG;                              // O columns per softmax warpgroup
    constexpr uint32_t TMEM_COLS = 512;
    // S of even steps (P in place) | S of odd steps | O of even items | O of odd items
    constexpr uint32_t TM_S = 0, TM_O = 256;

    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t* sQ = smem + L::Q;
    uint8_t* sK = smem + L::K;
    uint8_t* sV = smem + L::V;
    float* xch = reinterpret_cast<float*>(smem + L::XCH);
    float* lx = reinterpret_cast<float*>(smem + L::LX);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::BARS);
    uint32_t* tmem_base_s = reinterpret_cast<uint32_t*>(bars + F_COUNT);
    volatile uint32_t* abort_s = tmem_base_s + 1;
    uint32_t* skip_s = tmem_base_s + 2;

    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const int nq = (p.T + BM - 1) / BM;
    const int n_items = p.B * p.H * nq;

    if (threadIdx.x == 0) {
        *abort_s = 0;
        uint32_t skip = (*(volatile unsigned int*)p.err != 0) ? 1u : 0u;   // an earlier CTA gave up: exit at once
        if ((smem_u32(smem) & 1023u) != 0) {
            atomicCAS(p.err, 0u, DEERS_KERR_FWD_F16 | 0x20);
            skip = 1;
        }
        *skip_s = skip;
        for (int s = 0; s < 2; ++s) {
            mbar_init(&bars[F_Q_FULL + s], 1); mbar_init(&bars[F_Q_EMPTY + s], 1);
            mbar_init(&bars[F_K_FULL + s], 1);
            mbar_init(&bars[F_V_FULL + s], 1); mbar_init(&bars[F_PV_DONE + s], 1);
            mbar_init(&bars[F_S_FULL + s], 1);
            mbar_init(&bars[F_P_FULL + s], 128 * NWG);
            mbar_init(&bars[F_O_DONE + s], 1); mbar_init(&bars[F_O_FREE + s], 128 * NWG);
        }
        mbar_init(&bars[F_XCH], 128 * NWG);
        mbar_init(&bars[F_LX], 128 * NWG);
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

    if (warp == 0) {
        // ------------------------------ TMA producer ------------------------------
        if (lane == 0) {
            WorkCursor c;
            c.init(p, nq, n_items);
            for (uint32_t g = 0; c.valid(n_items); ++g) {      // g: global step = K / V stage use
                const int b = c.b, h = c.h;
                if (c.j == 0) {
                    const int qb = c.n & 1;
                    if (!mbar_wait(ws, &bars[F_Q_EMPTY + qb], (((uint32_t)c.n >> 1) & 1u) ^ 1u, DEERS_KERR_FWD_F16 | 1)) break;
                    mbar_arrive_expect_tx(&bars[F_Q_FULL + qb], TILE_BYTES);
#pragma unroll
                    for (int blk = 0; blk < DBLK; ++blk)
                        tma_load_4d(sQ + qb * TILE_BYTES + blk * BLOCK_BYTES, &tmap_q, &bars[F_Q_FULL + qb], blk * 64, c.qt * BM, h, b);
                }
                const uint32_t st = g & 1u, ph = ((g >> 1) & 1u) ^ 1u;
                if (!mbar_wait(ws, &bars[F_S_FULL + st], ph, DEERS_KERR_FWD_F16 | 2)) break;      // S of step g-2 done
                mbar_arrive_expect_tx(&bars[F_K_FULL + st], TILE_BYTES);
#pragma unroll
                for (int blk = 0; blk < DBLK; ++blk)
                    tma_load_4d(sK + st * TILE_BYTES + blk * BLOCK_BYTES, &tmap_k, &bars[F_K_FULL + st], blk * 64, c.j * BN, h, b);
                if (!mbar_wait(ws, &bars[F_PV_DONE + st], ph, DEERS_KERR_FWD_F16 | 3)) break;     // P V of step g-2 done
                mbar_arrive_expect_tx(&bars[F_V_FULL + st], TILE_BYTES);
#pragma unroll
                for (int blk = 0; blk < DBLK; ++blk)
                    tma_load_4d(sV + st * TILE_BYTES + blk * BLOCK_BYTES, &tmap_v, &bars[F_V_FULL + st], blk * 64, c.j * BN, h, b);
                c.advance(p, nq, n_items);
            }
        }
    } else if (warp == 1) {
        // ------------------------------ P V issuer ------------------------------
        if (lane == 0) {
            constexpr uint32_t IDESC_O = idesc_f16(BM, D, 0, 1);       // O: A = P from TMEM, B = V MN-major
            constexpr uint64_t STAGE_STEP = TILE_BYTES >> 4;
            const uint64_t v_mn0 = desc_mnmajor(smem_u32(sV), 0, BLOCK_BYTES);
            WorkCursor pc;
            pc.init(p, nq, n_items);
            for (uint32_t gp = 0; pc.valid(n_items); ++gp) {
                const uint32_t st = gp & 1u;
                if (!mbar_wait(ws, &bars[F_P_FULL + st], (gp >> 1) & 1u, DEERS_KERR_FWD_F16 | 6)) break;
                if (!mbar_wait(ws, &bars[F_V_FULL + st], (gp >> 1) & 1u, DEERS_KERR_FWD_F16 | 7)) break;
                // The accumulator of item n was last used by item n-2: its epilogue must be over.
                if (pc.j == 0 && !mbar_wait(ws, &bars[F_O_FREE + (pc.n & 1)], (((uint32_t)pc.n >> 1) & 1u) ^ 1u, DEERS_KERR_FWD_F16 | 8)) break;
                tc_fence_after_sync();
                const uint64_t v_mn = v_mn0 + (uint64_t)st * STAGE_STEP;
                const uint32_t o_tmem = tmem + TM_O + (uint32_t)(pc.n & 1) * D;
                const uint32_t p_tmem = tmem + TM_S + st * 128u;       // P sits where this step's S was
#pragma unroll
                for (int ks = 0; ks < BN / 16; ++ks)
                    umma_ts(o_tmem, p_tmem + (uint32_t)(ks / (CW / 16)) * CW + (uint32_t)(ks % (CW / 16)) * 8u, v_mn + mnmajor_step(ks),
                            IDESC_O, (pc.j > 0 || ks > 0));
                umma_commit(&bars[F_PV_DONE + st]);
                if (pc.j == pc.ntiles - 1) umma_commit(&bars[F_O_DONE + (pc.n & 1)]);
                pc.advance(p, nq, n_items);
            }
        }
    } else if (warp == S_WARP) {
        // ------------------------------ S issuer ------------------------------
        if (lane == 0) {
            constexpr uint32_t IDESC_S = idesc_f16(BM, BN, 0, 0);      // S: K-major A (Q) and B (K)
            constexpr uint64_t STAGE_STEP = TILE_BYTES >> 4;
            const uint64_t q_km0 = desc_kmajor(smem_u32(sQ), 0, BLOCK_BYTES);
            const uint64_t k_km0 = desc_kmajor(smem_u32(sK), 0, BLOCK_BYTES);
            WorkCursor sc;
            sc.init(p, nq, n_items);
            for (uint32_t gs = 0; sc.valid(n_items); ++gs) {
                const uint32_t st = gs & 1u;
                const int qb = sc.n & 1;
                if (sc.j == 0 && !mbar_wait(ws, &bars[F_Q_FULL + qb], ((uint32_t)sc.n >> 1) & 1u, DEERS_KERR_FWD_F16 | 4)) break;
                if (!mbar_wait(ws, &bars[F_K_FULL + st], (gs >> 1) & 1u, DEERS_KERR_FWD_F16 | 5)) break;
                // This S tile still holds P of step gs-2 until the product reading it has finished.
                if (!mbar_wait(ws, &bars[F_PV_DONE + st], ((gs >> 1) & 1u) ^ 1u, DEERS_KERR_FWD_F16 | 0x15)) break;
                tc_fence_after_sync();
                const uint64_t q_km = q_km0 + (uint64_t)qb * STAGE_STEP, k_km = k_km0 + (uint64_t)st * STAGE_STEP;
                const uint32_t d_tmem = tmem + TM_S + st * 128u;
#pragma unroll
                for (int ks = 0; ks < D / 16; ++ks)
                    umma_ss(d_tmem, q_km + kmajor_step(ks, BLOCK_BYTES), k_km + kmajor_step(ks, BLOCK_BYTES), IDESC_S, ks > 0);
                umma_commit(&bars[F_S_FULL + st]);
                if (sc.j == sc.ntiles - 1) umma_commit(&bars[F_Q_EMPTY + qb]);     // last product reading this Q
                sc.advance(p, nq, n_items);
            }
        }
    } else if (warp < S_WARP) {
        // ------------------------------ softmax + epilogue ------------------------------
        const int g = (warp - 2) >> 2;                          // warpgroup: key columns [CW*g, CW*g + CW)
        const int lane_base = (warp & 3) * 32;
        const int row = lane_base + lane;                       // row inside the query tile == TMEM lane
        const uint32_t t_lane = (uint32_t)lane_base << 16;
        const float sl2 = p.scale * LOG2E;
        uint32_t gstep = 0;                                     // global step counter
        bool alive = true;

        // Deferred epilogue of the previous item (runs after this item's first P has been handed over).
        int pend_n = -1, pend_grow = 0, pend_bh = 0, pend_b = 0, pend_h = 0;
        float pend_m = 0.f, pend_l = 0.f;
        auto epilogue = [&]() -> bool {
            if (pend_n < 0) return true;
            const int n = pend_n;
            pend_n = -1;
            // Combine the partial row sums of the warpgroups (published when the item's last step ended,
            // so this wait has long been satisfied).
            float* lxp = lx + (n & 1) * NWG * BM;
            if (!__all_sync(0xffffffffu, mbar_wait(ws, &bars[F_LX], (uint32_t)n & 1u, DEERS_KERR_FWD_F16 | 9))) return false;
            float l = 0.f;
#pragma unroll
            for (int w = 0; w < NWG; ++w) l += lxp[w * BM + row];        // same order in every warpgroup
            if (!__all_sync(0xffffffffu, mbar_wait(ws, &bars[F_O_DONE + (n & 1)], ((uint32_t)n >> 1) & 1u, DEERS_KERR_FWD_F16 | 10))) return false;
            tc_fence_after_sync();
            const float inv = 1.f / l;
            const int b = pend_b, h = pend_h;
            // The thread's half row of O, as 16-byte pieces, is transposed within lane groups so
            // that every store instruction writes whole contiguous row segments.
            constexpr int NP = DH / 8;
            uint4 oc[NP];
            {
                uint32_t r[DH];
                const uint32_t to = tmem + TM_O + (uint32_t)(n & 1) * D + t_lane + g * DH;
                if constexpr (DH == 64) {
                    tmem_ld_x32(to, *reinterpret_cast<uint32_t(*)[32]>(&r[0]));
                    tmem_ld_x32(to + 32, *reinterpret_cast<uint32_t(*)[32]>(&r[DH - 32]));
                } else if constexpr (DH == 32) {
                    tmem_ld_x32(to, *reinterpret_cast<uint32_t(*)[32]>(&r[0]));
                } else {
                    tmem_ld_x16(to, *reinterpret_cast<uint32_t(*)[16]>(&r[0]));
                }
                tmem_wait_ld();
                tc_fence_before_sync();
                mbar_arrive(&bars[F_O_FREE + (n & 1)]);         // accumulator is in registers: release it
#pragma unroll
                for (int q8 = 0; q8 < NP; ++q8) oc[q8] = pack8_f16(r + q8 * 8, inv);
            }
            transpose_pieces<NP>(oc, (uint32_t)lane);
            const int grow0 = pend_grow - lane + (lane & ~(NP - 1));
            __half* ob = p.o + b * p.so_b + h * p.so_h + g * DH + (lane & (NP - 1)) * 8;
#pragma unroll
            for (int c = 0; c < NP; ++c) {
                const int grow = grow0 + c;
                if (grow < p.T) *reinterpret_cast<uint4*>(ob + (long long)grow * p.so_t) = oc[c];
            }
            if (g == 0 && pend_grow < p.T) p.lse[(long long)pend_bh * p.T + pend_grow] = (pend_m + log2f(l)) * LN2;
            return true;
        };

        WorkCursor c;
        c.init(p, nq, n_items);
        while (alive && c.valid(n_items)) {
            const int n = c.n, qt = c.qt, ntiles = c.ntiles, bh = c.bh;
            const int q0 = qt * BM;
            float m_used = -INFINITY, l = 0.f;                  // l: partial sum over this warpgroup's columns
            for (int j = 0; j < ntiles; ++j, ++gstep) {
                const uint32_t sb = gstep & 1u;
                if (!__all_sync(0xffffffffu, mbar_wait(ws, &bars[F_S_FULL + sb], (gstep >> 1) & 1u, DEERS_KERR_FWD_F16 | 11))) { alive = false; break; }
                tc_fence_after_sync();
                float s[CW];
                const uint32_t ts = tmem + TM_S + sb * 128u + t_lane + CW * g;
#pragma unroll
                for (int cc = 0; cc < CW / 32; ++cc) tmem_ld_x32(ts + cc * 32, *reinterpret_cast<uint32_t(*)[32]>(&s[cc * 32]));
                tmem_wait_ld();
                // Steps that touch the diagonal or the end of the sequence are scaled here and
                // masked with -inf; all others keep raw scores and fold the scale into the
                // exponent's FFMA.
                const int k0 = j * BN;
                const bool edge = (p.causal && j == qt) || (k0 + BN > p.T);
                float c1 = sl2;
                if (edge) {
                    // Column CW*g + i of this tile is valid iff i <= lim: on the diagonal tile (where
                    // k0 == q0) the key may not lie right of the query, and keys end at T.
                    int lim = p.T - 1 - k0 - CW * g;
                    if (p.causal && j == qt) lim = min(lim, row - CW * g);
#pragma unroll
                    for (int i = 0; i < CW; ++i) s[i] = (i > lim) ? -INFINITY : s[i] * sl2;
                    c1 = 1.0f;
                }
                float mx = s[0];
                if (c1 >= 0.f) {
#pragma unroll
                    for (int i = 1; i < CW; ++i) mx = fmaxf(mx, s[i]);
                } else {
#pragma unroll
                    for (int i = 1; i < CW; ++i) mx = fminf(mx, s[i]);
                }
                mx *= c1;
                // Exchange the partial row max with the twin threads of the other warpgroups.
                float* xp = xch + sb * NWG * BM;
                xp[g * BM + row] = mx;
                mbar_arrive(&bars[F_XCH]);
                if (!__all_sync(0xffffffffu, mbar_wait(ws, &bars[F_XCH], gstep & 1u, DEERS_KERR_FWD_F16 | 12))) { alive = false; break; }
#pragma unroll
                for (int w = 0; w < NWG; ++w) mx = fmaxf(mx, xp[w * BM + row]);

                const float m_new = fmaxf(m_used, mx);
                // Lazy rescale: keep the old reference max unless this row grew by more than 2^8.
                const bool grow = (j > 0) && (m_new - m_used > RESCALE_THRESHOLD);
                const float m_cur = (j == 0 || grow) ? m_new : m_used;
                const float m_safe = (m_cur == -INFINITY) ? 0.f : m_cur;
                const float alpha = (j == 0) ? 0.f : ex2(m_used - m_safe);
                const bool warp_grow = __any_sync(0xffffffffu, grow);

                uint32_t pk[CW / 2];
                float rs = 0.f;
#pragma unroll
                for (int i = 0; i < CW / 2; ++i) {
                    const float e0 = ex2(fmaf(s[2 * i], c1, -m_safe));
                    const float e1 = ex2(fmaf(s[2 * i + 1], c1, -m_safe));
                    rs += e0 + e1;
                    pk[i] = pack_half2(e0, e1);
                }
                l = l * alpha + rs;
                m_used = m_cur;

                if (j > 0 && warp_grow) {
                    // O += P V of the previous step must have landed before O is rescaled.
                    if (!__all_sync(0xffffffffu, mbar_wait(ws, &bars[F_PV_DONE + ((gstep - 1u) & 1u)], ((gstep - 1u) >> 1) & 1u, DEERS_KERR_FWD_F16 | 13))) { alive = false; break; }
                    tc_fence_after_sync();
                    const uint32_t to = tmem + TM_O + (uint32_t)(n & 1) * D + t_lane + g * DH;
                    if constexpr (DH % 32 == 0) {
#pragma unroll
                        for (int cc = 0; cc < DH / 32; ++cc) {
                            uint32_t r[32];
                            tmem_ld_x32(to + cc * 32, r);
                            tmem_wait_ld();
#pragma unroll
                            for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
                            tmem_st_x32(to + cc * 32, r);
                        }
                    } else {
                        uint32_t r[16];
                        tmem_ld_x16(to, r);
                        tmem_wait_ld();
#pragma unroll
                        for (int i = 0; i < 16; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
                        tmem_st_x16(to, r);
                    }
                }
                // P replaces this warpgroup's part of S in TMEM (CW / 2 packed columns).
                if constexpr (CW == 64) tmem_st_x32(ts, *reinterpret_cast<uint32_t(*)[32]>(&pk[0]));
                else tmem_st_x16(ts, *reinterpret_cast<uint32_t(*)[16]>(&pk[0]));
                tmem_wait_st();
                tc_fence_before_sync();
                mbar_arrive(&bars[F_P_FULL + sb]);
                if (j == 0 && !epilogue()) { alive = false; break; }          // previous item's O tile
            }
            if (!alive) break;
            pend_n = n; pend_grow = q0 + row; pend_bh = bh; pend_b = c.b; pend_h = c.h; pend_m = m_used; pend_l = l;
            lx[(n & 1) * NWG * BM + g * BM + row] = l;                       // partial row sum for the epilogue
            mbar_arrive(&bars[F_LX]);
            // advance the cursor by a whole item
            c.j = ntiles - 1;
            c.advance(p, nq, n_items);
        }
        if (alive) epilogue();
    }

    __syncwarp();
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem, TMEM_COLS);
}

template <int D>
int fwd_launch(deers_ctx* ctx, const deers_attn_desc* d, const void* q, const void* k, const void* v, void* o,
               float* lse) {
    CUtensorMap tq, tk, tv;
    int rc;
    if ((rc = make_tmap_bhtd_f16(ctx, &tq, q, d->B, d->H, d->T, D, d->q_strides, BM))) return rc;
    if ((rc = make_tmap_bhtd_f16(ctx, &tk, k, d->B, d->H, d->T, D, d->k_strides, BN))) return rc;
    if ((rc = make_tmap_bhtd_f16(ctx, &tv, v, d->B, d->H, d->T, D, d->v_strides, BN))) return rc;
    FwdParams p;
    p.o = (__half*)o; p.lse = lse;
    p.so_b = d->o_strides[0]; p.so_h = d->o_strides[1]; p.so_t = d->o_strides[2];
    p.B = d->B; p.H = d->H; p.T = d->T; p.causal = d->causal; p.scale = d->scale; p.err = ctx->dev_err;
    const size_t smem = FwdSmem<D>::TOTAL;
    DEERS_CUDA_TRY(ctx, cudaFuncSetAttribute(attn_fwd_f16_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const long long nq = (d->T + BM - 1) / BM;
    const long long items = nq * d->B * d->H;
    if (items > 0x7fffffffLL) return DEERS_ERR_SHAPE;
    const unsigned grid = (unsigned)(items < ctx->sm_count ? items : ctx->sm_count);
    p.sched = deers_get_schedule(ctx, d->B, d->H, (int)nq, d->causal, (int)grid, &p.sched_rows);
    {
        KernelTimerScope ts(ctx, DEERS_K_FWD);
        attn_fwd_f16_kernel<D><<<grid, FWD_THREADS, smem, ctx->stream>>>(tq, tk, tv, p);
    }
    ctx->launches += 1;
    DEERS_CUDA_TRY(ctx, cudaGetLastError());
    return DEERS_OK;
}

}  // namespace

int launch_attn_fwd_f16(deers_ctx* ctx, const deers_attn_desc* d, const void* q, const void* k, const void* v,
                        void* o, float* lse) {
    if (d->D == 64) return fwd_launch<64>(ctx, d, q, k, v, o, lse);
    if (d->D == 128) return fwd_launch<128>(ctx, d, q, k, v, o, lse);
    return DEERS_ERR_UNSUPPORTED;
}
