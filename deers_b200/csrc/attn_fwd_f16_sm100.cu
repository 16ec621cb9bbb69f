// f16 causal attention forward for sm_100a.
//
// One CTA owns 128 query rows of one (batch, head) slice and walks the key/value
// tiles (128 rows each) at or left of its diagonal:
//   warp 0      TMA producer: Q once, then K and V tiles through a 2-stage ring
//   warp 1      issues tcgen05.mma: S = Q K^T into a double-buffered TMEM tile,
//               then O += P V with the accumulator resident in TMEM
//   warps 2-5   softmax: one thread per query row reads its S row from TMEM,
//               keeps the running max / sum, writes P (f16) into shared memory in
//               the swizzled K-major layout the second MMA reads, rescales O in
//               TMEM only when the row max grew by more than 2^8, and at the end
//               normalises O and stores O and the row lse.
// Scale, causal mask, softmax and both products happen in this one pass; the
// T x T scores never reach global memory.
#include "sm100_ptx.cuh"
#include "tma_host.cuh"

namespace {
using namespace sm100;

constexpr int BM = 128;
constexpr int BN = 128;
constexpr int KV_STAGES = 2;
constexpr uint32_t BLOCK_BYTES = 128 * 128;   // one 64-column block of a 128-row tile
constexpr float LOG2E = 1.4426950408889634f;
constexpr float LN2 = 0.6931471805599453f;
constexpr float RESCALE_THRESHOLD = 8.0f;     // log2 units: P stays below 2^8, safe in f16

struct FwdParams {
    __half* o;
    float* lse;
    long long so_b, so_h, so_t;
    int B, H, T;
    int causal;
    float scale;
    unsigned int* err;
};

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

template <int D>
__global__ void __launch_bounds__(192, 1)
attn_fwd_f16_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                    const __grid_constant__ CUtensorMap tmap_v, const FwdParams p) {
    constexpr uint32_t TILE_BYTES = 128u * D * 2u;
    constexpr int DBLK = D / 64;
    constexpr uint32_t TMEM_COLS = 512;
    constexpr uint32_t TM_S0 = 0, TM_O = 256;

    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* sQ = smem;
    uint8_t* sK = sQ + TILE_BYTES;
    uint8_t* sV = sK + KV_STAGES * TILE_BYTES;
    uint8_t* sP = sV + KV_STAGES * TILE_BYTES;          // 128 x 128 f16

    __shared__ uint64_t q_full, k_full[KV_STAGES], v_full[KV_STAGES], k_empty[KV_STAGES], v_empty[KV_STAGES];
    __shared__ uint64_t s_full[2], p_full, pv_done;
    __shared__ uint32_t tmem_base_s, abort_s, skip_s;

    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const int nq = (p.T + BM - 1) / BM;
    // Launch order: groups of 16 slices; inside a group the heaviest tiles of all its slices
    // come first (balance), and the group's K and V (a few MB) fit in L2 together.
    const int BH = p.B * p.H;
    const int group = (int)(blockIdx.x / (16u * nq));
    const int gsize = min(16, BH - group * 16);
    const int within = (int)(blockIdx.x - (unsigned)group * 16u * nq);
    const int qt = nq - 1 - within / gsize;
    const int bh = group * 16 + within % gsize;
    const int b = bh / p.H, h = bh % p.H;
    const int q0 = qt * BM;
    const int ntiles = p.causal ? qt + 1 : (p.T + BN - 1) / BN;

    if (threadIdx.x == 0) {
        abort_s = 0;
        skip_s = (*(volatile unsigned int*)p.err != 0) ? 1u : 0u;   // an earlier CTA gave up: exit at once
        mbar_init(&q_full, 1);
        for (int s = 0; s < KV_STAGES; ++s) {
            mbar_init(&k_full[s], 1); mbar_init(&v_full[s], 1);
            mbar_init(&k_empty[s], 1); mbar_init(&v_empty[s], 1);
        }
        mbar_init(&s_full[0], 1); mbar_init(&s_full[1], 1);
        mbar_init(&p_full, 128);
        mbar_init(&pv_done, 1);
        fence_barrier_init();
        tma_prefetch_desc(&tmap_q); tma_prefetch_desc(&tmap_k); tma_prefetch_desc(&tmap_v);
    }
    __syncthreads();
    if (skip_s) return;
    if (warp == 1) {
        tmem_alloc(&tmem_base_s, TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = tmem_base_s;
    WaitState ws{&abort_s, p.err};

    if (warp == 0) {
        // ------------------------------ TMA producer ------------------------------
        if (lane == 0) {
            mbar_arrive_expect_tx(&q_full, TILE_BYTES);
#pragma unroll
            for (int blk = 0; blk < DBLK; ++blk) tma_load_4d(sQ + blk * BLOCK_BYTES, &tmap_q, &q_full, blk * 64, q0, h, b);
            for (int j = 0; j < ntiles; ++j) {
                const int st = j % KV_STAGES;
                const uint32_t ph = (uint32_t)(j / KV_STAGES) & 1u;
                if (!mbar_wait(ws, &k_empty[st], ph ^ 1u, DEERS_KERR_FWD_F16 | 1)) break;
                mbar_arrive_expect_tx(&k_full[st], TILE_BYTES);
#pragma unroll
                for (int blk = 0; blk < DBLK; ++blk)
                    tma_load_4d(sK + st * TILE_BYTES + blk * BLOCK_BYTES, &tmap_k, &k_full[st], blk * 64, j * BN, h, b);
                if (!mbar_wait(ws, &v_empty[st], ph ^ 1u, DEERS_KERR_FWD_F16 | 2)) break;
                mbar_arrive_expect_tx(&v_full[st], TILE_BYTES);
#pragma unroll
                for (int blk = 0; blk < DBLK; ++blk)
                    tma_load_4d(sV + st * TILE_BYTES + blk * BLOCK_BYTES, &tmap_v, &v_full[st], blk * 64, j * BN, h, b);
            }
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer ------------------------------
        if (lane == 0) {
            constexpr uint32_t IDESC_S = idesc_f16(BM, BN, 0, 0);
            constexpr uint32_t IDESC_O = idesc_f16(BM, D, 0, 1);
            // Step-0 descriptors built once; each MMA adds a constant (single-thread issue must
            // stay faster than MMA execution).
            constexpr uint64_t STAGE_STEP = TILE_BYTES >> 4;
            const uint64_t q_km = desc_kmajor(smem_u32(sQ), 0, BLOCK_BYTES), p_km = desc_kmajor(smem_u32(sP), 0, BLOCK_BYTES);
            const uint64_t k_km0 = desc_kmajor(smem_u32(sK), 0, BLOCK_BYTES), v_mn0 = desc_mnmajor(smem_u32(sV), 0, BLOCK_BYTES);
            auto issue_s = [&](int j) {
                const uint64_t k_km = k_km0 + (uint64_t)(j % KV_STAGES) * STAGE_STEP;
                const uint32_t d_tmem = tmem + TM_S0 + (uint32_t)(j & 1) * 128u;
#pragma unroll
                for (int ks = 0; ks < D / 16; ++ks)
                    umma_ss(d_tmem, q_km + kmajor_step(ks, BLOCK_BYTES), k_km + kmajor_step(ks, BLOCK_BYTES), IDESC_S, ks > 0);
                umma_commit(&s_full[j & 1]);
                umma_commit(&k_empty[j % KV_STAGES]);
            };
            bool ok = mbar_wait(ws, &q_full, 0, DEERS_KERR_FWD_F16 | 3) &&
                      mbar_wait(ws, &k_full[0], 0, DEERS_KERR_FWD_F16 | 4);
            if (ok) {
                tc_fence_after_sync();
                issue_s(0);
            }
            for (int j = 0; ok && j < ntiles; ++j) {
                if (j + 1 < ntiles) {
                    const int jn = j + 1;
                    if (!mbar_wait(ws, &k_full[jn % KV_STAGES], (uint32_t)(jn / KV_STAGES) & 1u, DEERS_KERR_FWD_F16 | 5)) break;
                    tc_fence_after_sync();
                    issue_s(jn);
                }
                if (!mbar_wait(ws, &p_full, (uint32_t)j & 1u, DEERS_KERR_FWD_F16 | 6)) break;
                if (!mbar_wait(ws, &v_full[j % KV_STAGES], (uint32_t)(j / KV_STAGES) & 1u, DEERS_KERR_FWD_F16 | 7)) break;
                tc_fence_after_sync();
                const uint64_t v_mn = v_mn0 + (uint64_t)(j % KV_STAGES) * STAGE_STEP;
#pragma unroll
                for (int ks = 0; ks < BN / 16; ++ks)
                    umma_ss(tmem + TM_O, p_km + kmajor_step(ks, BLOCK_BYTES), v_mn + mnmajor_step(ks), IDESC_O, (j > 0 || ks > 0));
                umma_commit(&pv_done);
                umma_commit(&v_empty[j % KV_STAGES]);
            }
        }
    } else {
        // ------------------------------ softmax + epilogue ------------------------------
        const int lane_base = (warp & 3) * 32;
        const int row = lane_base + lane;                       // row inside the query tile == TMEM lane
        const uint32_t t_lane = (uint32_t)lane_base << 16;
        const float sl2 = p.scale * LOG2E;
        float m_used = -INFINITY, l = 0.f;
        bool alive = true;

        for (int j = 0; j < ntiles; ++j) {
            if (!__all_sync(0xffffffffu, mbar_wait(ws, &s_full[j & 1], (uint32_t)(j >> 1) & 1u, DEERS_KERR_FWD_F16 | 8))) { alive = false; break; }
            tc_fence_after_sync();
            float s[128];
            {
                const uint32_t ts = tmem + TM_S0 + (uint32_t)(j & 1) * 128u + t_lane;
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    uint32_t r[32];
                    tmem_ld_x32(ts + c * 32, r);
#pragma unroll
                    for (int i = 0; i < 32; ++i) s[c * 32 + i] = __uint_as_float(r[i]);
                }
                tmem_wait_ld();
            }
            // Tiles that touch the diagonal or the end of the sequence are scaled
            // here and masked with -inf; all others keep raw scores and fold the
            // scale into the exponent's FFMA.
            const int k0 = j * BN;
            const bool edge = (p.causal && j == qt) || (k0 + BN > p.T);
            float c1 = sl2;
            if (edge) {
#pragma unroll
                for (int i = 0; i < 128; ++i) {
                    const int col = k0 + i;
                    const bool masked = (col >= p.T) || (p.causal && col > q0 + row);
                    s[i] = masked ? -INFINITY : s[i] * sl2;
                }
                c1 = 1.0f;
            }
            float mx;
            if (c1 >= 0.f) {
                mx = s[0];
#pragma unroll
                for (int i = 1; i < 128; ++i) mx = fmaxf(mx, s[i]);
            } else {
                mx = s[0];
#pragma unroll
                for (int i = 1; i < 128; ++i) mx = fminf(mx, s[i]);
            }
            mx *= c1;
            const float m_new = fmaxf(m_used, mx);
            // Lazy rescale: keep the old reference max unless this row grew by more than 2^8.
            const bool grow = (j > 0) && (m_new - m_used > RESCALE_THRESHOLD);
            const float m_cur = (j == 0 || grow) ? m_new : m_used;
            const float m_safe = (m_cur == -INFINITY) ? 0.f : m_cur;
            const float alpha = (j == 0) ? 0.f : ex2(m_used - m_safe);
            const bool warp_grow = __any_sync(0xffffffffu, grow);

            uint32_t pk[64];
            float rs = 0.f;
#pragma unroll
            for (int i = 0; i < 64; ++i) {
                const float e0 = ex2(fmaf(s[2 * i], c1, -m_safe));
                const float e1 = ex2(fmaf(s[2 * i + 1], c1, -m_safe));
                rs += e0 + e1;
                pk[i] = pack_half2(e0, e1);
            }
            l = l * alpha + rs;
            m_used = m_cur;

            if (j > 0) {
                // P's buffer and the O accumulator are free once PV(j-1) has finished.
                if (!__all_sync(0xffffffffu, mbar_wait(ws, &pv_done, (uint32_t)(j - 1) & 1u, DEERS_KERR_FWD_F16 | 9))) { alive = false; break; }
                tc_fence_after_sync();
                if (warp_grow) {
#pragma unroll
                    for (int c = 0; c < D / 32; ++c) {
                        uint32_t r[32];
                        tmem_ld_x32(tmem + TM_O + t_lane + c * 32, r);
                        tmem_wait_ld();
#pragma unroll
                        for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
                        tmem_st_x32(tmem + TM_O + t_lane + c * 32, r);
                    }
                    tmem_wait_st();
                }
            }
            // P row -> shared memory, K-major with the 128-byte swizzle: 16 chunks of 8 f16.
#pragma unroll
            for (int ch = 0; ch < 16; ++ch) {
                uint4 v = make_uint4(pk[ch * 4], pk[ch * 4 + 1], pk[ch * 4 + 2], pk[ch * 4 + 3]);
                *reinterpret_cast<uint4*>(sP + (ch >> 3) * BLOCK_BYTES + sw128_chunk_offset(row, ch & 7)) = v;
            }
            fence_proxy_async_smem();
            tc_fence_before_sync();
            mbar_arrive(&p_full);
        }

        if (alive && __all_sync(0xffffffffu, mbar_wait(ws, &pv_done, (uint32_t)(ntiles - 1) & 1u, DEERS_KERR_FWD_F16 | 10))) {
            tc_fence_after_sync();
            const float inv = 1.f / l;
            const int grow_ = q0 + row;
            __half* orow = p.o + b * p.so_b + h * p.so_h + (long long)grow_ * p.so_t;
#pragma unroll
            for (int c = 0; c < D / 32; ++c) {
                uint32_t r[32];
                tmem_ld_x32(tmem + TM_O + t_lane + c * 32, r);
                tmem_wait_ld();
                if (grow_ < p.T) {
#pragma unroll
                    for (int g = 0; g < 4; ++g) {
                        uint4 v;
                        v.x = pack_half2(__uint_as_float(r[g * 8 + 0]) * inv, __uint_as_float(r[g * 8 + 1]) * inv);
                        v.y = pack_half2(__uint_as_float(r[g * 8 + 2]) * inv, __uint_as_float(r[g * 8 + 3]) * inv);
                        v.z = pack_half2(__uint_as_float(r[g * 8 + 4]) * inv, __uint_as_float(r[g * 8 + 5]) * inv);
                        v.w = pack_half2(__uint_as_float(r[g * 8 + 6]) * inv, __uint_as_float(r[g * 8 + 7]) * inv);
                        *reinterpret_cast<uint4*>(orow + c * 32 + g * 8) = v;
                    }
                }
            }
            if (grow_ < p.T) p.lse[(long long)bh * p.T + grow_] = (m_used + log2f(l)) * LN2;
        }
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
    const size_t smem = (size_t)(1 + 2 * KV_STAGES) * 128 * D * 2 + 128 * 128 * 2 + 1024;
    DEERS_CUDA_TRY(ctx, cudaFuncSetAttribute(attn_fwd_f16_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const long long nq = (d->T + BM - 1) / BM;
    const long long grid = nq * d->B * d->H;
    if (grid > 0x7fffffffLL) return DEERS_ERR_SHAPE;
    {
        KernelTimerScope ts(ctx, DEERS_K_FWD);
        attn_fwd_f16_kernel<D><<<(unsigned)grid, 192, smem, ctx->stream>>>(tq, tk, tv, p);
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
