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
//                                    bitwise reproducible); the per-tile dQ contribution is added
//                                    into the float32 accumulator with vector reductions
//   3. attn_bwd_dq_convert_kernel   dQ = f16(scale * accumulator)
//
// Inside the main kernel everything is computed transposed so that the tensor-core
// operands need no data movement:
//   S^T  = K Q^T   (A = K, B = Q, both K-major as TMA writes them)      -> TMEM
//   dP^T = V dO^T  (A = V, B = dO)                                       -> TMEM
//   thread r (= KV row r) turns row r of S^T / dP^T into P^T and dS^T = P^T * (dP^T - delta)
//   and writes them as f16 K-major tiles in shared memory
//   dV += P^T dO   (A = P^T K-major, B = dO MN-major)
//   dK += dS^T Q   (A = dS^T K-major, B = Q MN-major)
//   dQ  = dS K     (A = dS^T read MN-major, B = K MN-major), overlaying the S^T columns
// Warp roles: warp 0 TMA producer, warp 1 MMA issuer, warps 2-5 the 128 compute threads.
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
    float* dq_acc;              // [B*H][Tpad][D] float32
    __half* dk; __half* dv;
    long long sdk_b, sdk_h, sdk_t, sdv_b, sdv_h, sdv_t;
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

template <int D, int STAGES>
__global__ void __launch_bounds__(192, 1)
attn_bwd_f16_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                    const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_do,
                    const BwdParams p) {
    constexpr uint32_t TILE_BYTES = 128u * D * 2u;
    constexpr int DBLK = D / 64;
    constexpr uint32_t TMEM_COLS = 512;
    constexpr uint32_t TM_S = 0, TM_DP = 128, TM_DV = 256, TM_DK = 256 + D, TM_DQ = 0;

    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* sK = smem;
    uint8_t* sV = sK + TILE_BYTES;
    uint8_t* sQ = sV + TILE_BYTES;                          // STAGES tiles
    uint8_t* sDO = sQ + STAGES * TILE_BYTES;                // STAGES tiles
    uint8_t* sP = sDO + STAGES * TILE_BYTES;                // P^T  : 128 (kv) x 128 (q) f16
    uint8_t* sDS = sP + 2 * BLOCK_BYTES;                    // dS^T : 128 (kv) x 128 (q) f16

    __shared__ uint64_t kv_full, qdo_full[STAGES], qdo_empty[STAGES], s_full, pds_full, dq_full, dq_read;
    __shared__ uint32_t tmem_base_s, abort_s, skip_s;
    __shared__ __align__(16) float lse2_s[STAGES][BT], delta_s[STAGES][BT];

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
        abort_s = 0;
        skip_s = (*(volatile unsigned int*)p.err != 0) ? 1u : 0u;
        mbar_init(&kv_full, 1);
        for (int s = 0; s < STAGES; ++s) { mbar_init(&qdo_full[s], 1); mbar_init(&qdo_empty[s], 1); }
        mbar_init(&s_full, 1);
        mbar_init(&pds_full, 128);
        mbar_init(&dq_full, 1);
        mbar_init(&dq_read, 128);
        fence_barrier_init();
        tma_prefetch_desc(&tmap_q); tma_prefetch_desc(&tmap_k); tma_prefetch_desc(&tmap_v); tma_prefetch_desc(&tmap_do);
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
            mbar_arrive_expect_tx(&kv_full, 2 * TILE_BYTES);
#pragma unroll
            for (int blk = 0; blk < DBLK; ++blk) {
                tma_load_4d(sK + blk * BLOCK_BYTES, &tmap_k, &kv_full, blk * 64, k0, h, b);
                tma_load_4d(sV + blk * BLOCK_BYTES, &tmap_v, &kv_full, blk * 64, k0, h, b);
            }
            for (int it = 0; it < niter; ++it) {
                const int st = it % STAGES;
                const uint32_t ph = (uint32_t)(it / STAGES) & 1u;
                if (!mbar_wait(ws, &qdo_empty[st], ph ^ 1u, DEERS_KERR_BWD_F16 | 1)) break;
                mbar_arrive_expect_tx(&qdo_full[st], 2 * TILE_BYTES + 2 * BT * 4);
                const int q0 = (i0 + it) * BT;
                bulk_load(lse2_s[st], p.lse2 + (long long)bh * p.Tpad + q0, BT * 4, &qdo_full[st]);
                bulk_load(delta_s[st], p.delta + (long long)bh * p.Tpad + q0, BT * 4, &qdo_full[st]);
#pragma unroll
                for (int blk = 0; blk < DBLK; ++blk) {
                    tma_load_4d(sQ + st * TILE_BYTES + blk * BLOCK_BYTES, &tmap_q, &qdo_full[st], blk * 64, q0, h, b);
                    tma_load_4d(sDO + st * TILE_BYTES + blk * BLOCK_BYTES, &tmap_do, &qdo_full[st], blk * 64, q0, h, b);
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer ------------------------------
        if (lane == 0) {
            constexpr uint32_t IDESC_ST = idesc_f16(128, 128, 0, 0);   // S^T, dP^T: K-major A and B
            constexpr uint32_t IDESC_KV = idesc_f16(128, D, 0, 1);     // dV, dK: K-major A, MN-major B
            constexpr uint32_t IDESC_DQ = idesc_f16(128, D, 1, 1);     // dQ: MN-major A and B
            const uint32_t k_addr = smem_u32(sK), v_addr = smem_u32(sV);
            const uint32_t p_addr = smem_u32(sP), ds_addr = smem_u32(sDS);
            bool ok = mbar_wait(ws, &kv_full, 0, DEERS_KERR_BWD_F16 | 2);
            for (int it = 0; ok && it < niter; ++it) {
                const int st = it % STAGES;
                const uint32_t q_addr = smem_u32(sQ + st * TILE_BYTES);
                const uint32_t do_addr = smem_u32(sDO + st * TILE_BYTES);
                if (!mbar_wait(ws, &qdo_full[st], (uint32_t)(it / STAGES) & 1u, DEERS_KERR_BWD_F16 | 3)) break;
                if (it > 0 && !mbar_wait(ws, &dq_read, (uint32_t)(it - 1) & 1u, DEERS_KERR_BWD_F16 | 4)) break;
                tc_fence_after_sync();
#pragma unroll
                for (int ks = 0; ks < D / 16; ++ks)
                    umma_ss(tmem + TM_S, desc_kmajor(k_addr, ks, BLOCK_BYTES), desc_kmajor(q_addr, ks, BLOCK_BYTES),
                            IDESC_ST, ks > 0);
#pragma unroll
                for (int ks = 0; ks < D / 16; ++ks)
                    umma_ss(tmem + TM_DP, desc_kmajor(v_addr, ks, BLOCK_BYTES), desc_kmajor(do_addr, ks, BLOCK_BYTES),
                            IDESC_ST, ks > 0);
                umma_commit(&s_full);
                if (!mbar_wait(ws, &pds_full, (uint32_t)it & 1u, DEERS_KERR_BWD_F16 | 5)) break;
                tc_fence_after_sync();
#pragma unroll
                for (int ks = 0; ks < BT / 16; ++ks)
                    umma_ss(tmem + TM_DV, desc_kmajor(p_addr, ks, BLOCK_BYTES), desc_mnmajor(do_addr, ks, BLOCK_BYTES),
                            IDESC_KV, (it > 0 || ks > 0));
#pragma unroll
                for (int ks = 0; ks < BT / 16; ++ks)
                    umma_ss(tmem + TM_DK, desc_kmajor(ds_addr, ks, BLOCK_BYTES), desc_mnmajor(q_addr, ks, BLOCK_BYTES),
                            IDESC_KV, (it > 0 || ks > 0));
#pragma unroll
                for (int ks = 0; ks < BT / 16; ++ks)
                    umma_ss(tmem + TM_DQ, desc_mnmajor(ds_addr, ks, BLOCK_BYTES), desc_mnmajor(k_addr, ks, BLOCK_BYTES),
                            IDESC_DQ, ks > 0);
                umma_commit(&dq_full);
                umma_commit(&qdo_empty[st]);
            }
        }
    } else {
        // ------------------------------ compute threads ------------------------------
        const int lane_base = (warp & 3) * 32;
        const int r = lane_base + lane;                     // KV row inside the tile == TMEM lane
        const uint32_t t_lane = (uint32_t)lane_base << 16;
        const float sl2 = p.scale * LOG2E;
        bool alive = true;

        for (int it = 0; it < niter; ++it) {
            const int i = i0 + it;
            const int q0 = i * BT;
            const int buf = it % STAGES;                    // stats travel with the Q/dO stage
            // The stage's lse / delta rows arrive with Q and dO: observe that barrier directly.
            if (!__all_sync(0xffffffffu, mbar_wait(ws, &qdo_full[buf], (uint32_t)(it / STAGES) & 1u, DEERS_KERR_BWD_F16 | 8))) { alive = false; break; }
            if (!__all_sync(0xffffffffu, mbar_wait(ws, &s_full, (uint32_t)it & 1u, DEERS_KERR_BWD_F16 | 6))) { alive = false; break; }
            tc_fence_after_sync();
            const bool diag = p.causal && (i == kt);
            const bool kv_valid = (k0 + r) < p.T;           // rows past the sequence end contribute nothing
#pragma unroll
            for (int c = 0; c < 4; ++c) {                  // 32 query columns at a time
                uint32_t sr[32], dr[32];
                tmem_ld_x32(tmem + TM_S + t_lane + c * 32, sr);
                tmem_ld_x32(tmem + TM_DP + t_lane + c * 32, dr);
                tmem_wait_ld();
                uint32_t pp[16], dd[16];
#pragma unroll
                for (int e = 0; e < 16; ++e) {
                    float pv[2], dv[2];
#pragma unroll
                    for (int u = 0; u < 2; ++u) {
                        const int col = c * 32 + e * 2 + u;
                        float pe = ex2(fmaf(__uint_as_float(sr[e * 2 + u]), sl2, -lse2_s[buf][col]));
                        if ((diag && col < r) || !kv_valid) pe = 0.f;   // query index < key index: masked
                        pv[u] = pe;
                        dv[u] = pe * (__uint_as_float(dr[e * 2 + u]) - delta_s[buf][col]);
                    }
                    pp[e] = pack_half2(pv[0], pv[1]);
                    dd[e] = pack_half2(dv[0], dv[1]);
                }
                // 32 columns = 4 chunks of 8 f16 inside column block c/2.
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                    const uint32_t off = (uint32_t)(c >> 1) * BLOCK_BYTES + sw128_chunk_offset(r, (c & 1) * 4 + g);
                    *reinterpret_cast<uint4*>(sP + off) = make_uint4(pp[g * 4], pp[g * 4 + 1], pp[g * 4 + 2], pp[g * 4 + 3]);
                    *reinterpret_cast<uint4*>(sDS + off) = make_uint4(dd[g * 4], dd[g * 4 + 1], dd[g * 4 + 2], dd[g * 4 + 3]);
                }
            }
            fence_proxy_async_smem();
            tc_fence_before_sync();
            mbar_arrive(&pds_full);

            if (!__all_sync(0xffffffffu, mbar_wait(ws, &dq_full, (uint32_t)it & 1u, DEERS_KERR_BWD_F16 | 7))) { alive = false; break; }
            tc_fence_after_sync();
            {
                // Row r of the dQ tile belongs to query q0 + r.
                const int qrow = q0 + r;
                float* acc = p.dq_acc + ((long long)bh * p.Tpad + qrow) * D;
#pragma unroll
                for (int c = 0; c < D / 32; ++c) {
                    uint32_t qr[32];
                    tmem_ld_x32(tmem + TM_DQ + t_lane + c * 32, qr);
                    tmem_wait_ld();
                    if (qrow < p.T) {
#pragma unroll
                        for (int g = 0; g < 8; ++g)
                            red_add_v4(acc + c * 32 + g * 4, __uint_as_float(qr[g * 4]), __uint_as_float(qr[g * 4 + 1]),
                                       __uint_as_float(qr[g * 4 + 2]), __uint_as_float(qr[g * 4 + 3]));
                    }
                }
            }
            tc_fence_before_sync();
            mbar_arrive(&dq_read);
        }

        if (alive) {
            // dq_full of the last iteration covers every MMA: dK and dV are final.
            const int krow = k0 + r;
            __half* dkrow = p.dk + b * p.sdk_b + h * p.sdk_h + (long long)krow * p.sdk_t;
            __half* dvrow = p.dv + b * p.sdv_b + h * p.sdv_h + (long long)krow * p.sdv_t;
#pragma unroll
            for (int c = 0; c < D / 32; ++c) {
                uint32_t kr[32], vr[32];
                tmem_ld_x32(tmem + TM_DK + t_lane + c * 32, kr);
                tmem_ld_x32(tmem + TM_DV + t_lane + c * 32, vr);
                tmem_wait_ld();
                if (krow < p.T) {
#pragma unroll
                    for (int g = 0; g < 4; ++g) {
                        uint4 a, bq;
                        a.x = pack_half2(__uint_as_float(kr[g * 8 + 0]) * p.scale, __uint_as_float(kr[g * 8 + 1]) * p.scale);
                        a.y = pack_half2(__uint_as_float(kr[g * 8 + 2]) * p.scale, __uint_as_float(kr[g * 8 + 3]) * p.scale);
                        a.z = pack_half2(__uint_as_float(kr[g * 8 + 4]) * p.scale, __uint_as_float(kr[g * 8 + 5]) * p.scale);
                        a.w = pack_half2(__uint_as_float(kr[g * 8 + 6]) * p.scale, __uint_as_float(kr[g * 8 + 7]) * p.scale);
                        bq.x = pack_half2(__uint_as_float(vr[g * 8 + 0]), __uint_as_float(vr[g * 8 + 1]));
                        bq.y = pack_half2(__uint_as_float(vr[g * 8 + 2]), __uint_as_float(vr[g * 8 + 3]));
                        bq.z = pack_half2(__uint_as_float(vr[g * 8 + 4]), __uint_as_float(vr[g * 8 + 5]));
                        bq.w = pack_half2(__uint_as_float(vr[g * 8 + 6]), __uint_as_float(vr[g * 8 + 7]));
                        *reinterpret_cast<uint4*>(dkrow + c * 32 + g * 8) = a;
                        *reinterpret_cast<uint4*>(dvrow + c * 32 + g * 8) = bq;
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
    const float4* src = reinterpret_cast<const float4*>(dq_acc + ((long long)bh * Tpad + t) * D + v * 8);
    const float4 x = src[0], y = src[1];
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

template <int D, int STAGES>
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
    const size_t smem = (size_t)(2 + 2 * STAGES) * 128 * D * 2 + 4 * BLOCK_BYTES + 1024;
    DEERS_CUDA_TRY(ctx, cudaFuncSetAttribute(attn_bwd_f16_kernel<D, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const long long grid = BH * nq;
    if (grid > 0x7fffffffLL) return DEERS_ERR_SHAPE;
    {
        KernelTimerScope ts(ctx, DEERS_K_BWD_MAIN);
        attn_bwd_f16_kernel<D, STAGES><<<(unsigned)grid, 192, smem, ctx->stream>>>(tq, tk, tv, tdo, p);
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
    if (d->D == 64) return bwd_launch<64, 2>(ctx, d, q, k, v, o, lse, d_o, dq, dk, dv, workspace);
    if (d->D == 128) return bwd_launch<128, 1>(ctx, d, q, k, v, o, lse, d_o, dq, dk, dv, workspace);
    return DEERS_ERR_UNSUPPORTED;
}
