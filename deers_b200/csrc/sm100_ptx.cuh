// Thin inline-PTX layer for the Blackwell (sm_100a) features the f16 kernels use:
// mbarriers with bounded waits, TMA tile loads, tensor memory (TMEM) allocation,
// tcgen05.mma with shared-memory operand descriptors, tcgen05.ld/st and the
// fences between the generic, async and tensor-core proxies.
#pragma once
#include <cuda_fp16.h>
#include <stdint.h>

namespace sm100 {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}

// ---------------------------------------------------------------------------
// mbarrier
// ---------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_barrier_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ uint64_t global_timer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

// State every bounded wait of a CTA shares: once one wait gives up, `abort`
// (shared memory) makes every later wait of the CTA return at once, and the
// first code is recorded in the context's error word (global) so that CTAs not
// yet started exit immediately and the host learns of it at the next sync.
constexpr uint64_t kWaitLimitNs = 2000000000ull;   // 2 s without progress = give up

struct WaitState {
    volatile uint32_t* abort;   // shared memory flag
    unsigned int* err;          // error word in device memory
    uint64_t limit_ns = kWaitLimitNs;
};

// Waits for the phase with the given parity.  Returns false if this or an
// earlier wait of the CTA gave up; callers then fall through to the teardown.
__device__ __forceinline__ bool mbar_wait(const WaitState& ws, uint64_t* bar, uint32_t parity,
                                          uint32_t code) {
    if (mbar_try_wait(bar, parity)) return true;
    uint64_t t0 = 0;
    for (uint32_t it = 1;; ++it) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((it & 255u) == 0) {
            if (*ws.abort) return false;
            const uint64_t now = global_timer_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > ws.limit_ns) {
                *ws.abort = 1;
                atomicCAS(ws.err, 0u, code);
                return false;
            }
        }
    }
}

// ---------------------------------------------------------------------------
// Proxy fences
// ---------------------------------------------------------------------------
// Makes generic-proxy writes to shared memory visible to the async proxy (TMA, tcgen05.mma).
__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// ---------------------------------------------------------------------------
// TMA: 4-D tiled load (innermost coordinate first), completion on an mbarrier
// ---------------------------------------------------------------------------
__device__ __forceinline__ void tma_load_4d(void* dst, const void* tmap, uint64_t* bar, int c0, int c1,
                                            int c2, int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(smem_u32(dst)), "l"(tmap), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}
__device__ __forceinline__ void tma_prefetch_desc(const void* tmap) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(tmap) : "memory");
}

// Bulk (untiled) reduce-add of f32 from shared to global memory; both addresses
// 16-byte aligned, size a multiple of 16.  Tracked by the bulk async-group.
__device__ __forceinline__ void bulk_reduce_add_f32(float* gdst, const void* ssrc, uint32_t bytes) {
    asm volatile("cp.reduce.async.bulk.global.shared::cta.bulk_group.add.f32 [%0], [%1], %2;"
                 ::"l"(gdst), "r"(smem_u32(ssrc)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void bulk_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void bulk_wait_group_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N>
__device__ __forceinline__ void bulk_wait_group() {
    asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

// ---------------------------------------------------------------------------
// Tensor memory
// ---------------------------------------------------------------------------
// Whole-warp calls.  `cols` is a power of two in [32, 512].
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32(smem_result)), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}

// ---------------------------------------------------------------------------
// tcgen05.mma operand descriptors
// ---------------------------------------------------------------------------
// Shared-memory matrix descriptor, 128-byte swizzle (layout type 2), version 1.
// Offsets are in bytes; the hardware fields drop the 4 low bits.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32;
    d |= (uint64_t)1 << 46;     // descriptor version for sm_100
    d |= (uint64_t)2 << 61;     // SWIZZLE_128B
    return d;
}

// Tiles are stored as column blocks of 64 f16 (128 bytes) by R rows, rows 128
// bytes apart, the 16-byte chunks of a row XOR-swizzled with (row % 8): what a
// TMA box {64, R} with CU_TENSOR_MAP_SWIZZLE_128B writes.  Blocks follow one
// another R*128 bytes apart.
//
// K-major operand (rows = M or N index, the 64 columns of a block = K):
//   one MMA consumes K=16 = 32 bytes of each row; step k lives in block k/4 at
//   byte (k%4)*32.  8-row groups are 1024 bytes apart (SBO); LBO is unused.
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t tile_saddr, int kstep, uint32_t block_bytes) {
    return smem_desc_sw128(tile_saddr + (uint32_t)(kstep >> 2) * block_bytes + (uint32_t)(kstep & 3) * 32u,
                           16u, 1024u);
}
// MN-major operand (rows = K index, the columns = M or N index):
//   one MMA consumes 16 rows = two 8-row groups 1024 bytes apart (SBO); the 64-wide
//   column blocks are block_bytes apart (LBO).
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t tile_saddr, int kstep, uint32_t block_bytes) {
    return smem_desc_sw128(tile_saddr + (uint32_t)kstep * 2048u, block_bytes, 1024u);
}

// Descriptor increments for step k relative to the descriptor of step 0 (added to the 64-bit
// descriptor; the address field never carries out).  The issuing thread is a single thread,
// so building every descriptor from scratch would make MMA issue slower than MMA execution.
__host__ __device__ constexpr uint64_t kmajor_step(int kstep, uint32_t block_bytes) {
    return (uint64_t)(((uint32_t)(kstep >> 2) * block_bytes + (uint32_t)(kstep & 3) * 32u) >> 4);
}
__host__ __device__ constexpr uint64_t mnmajor_step(int kstep) { return (uint64_t)kstep * (2048u >> 4); }

// Instruction descriptor for kind::f16 with f16 inputs and f32 accumulation.
__host__ __device__ constexpr uint32_t idesc_f16(int M, int N, int a_mn_major, int b_mn_major) {
    return (1u << 4)                       // D format: f32
           | (0u << 7) | (0u << 10)        // A, B format: f16
           | ((uint32_t)a_mn_major << 15) | ((uint32_t)b_mn_major << 16)
           | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

// D[tmem] (+)= A[smem] * B[smem]; issued by ONE thread.
__device__ __forceinline__ void umma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                        uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]; A holds f16 pairs packed in 32-bit columns.
__device__ __forceinline__ void umma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                        uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// The mbarrier receives one arrival when every MMA this thread issued so far has finished.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
                 ::"r"(smem_u32(bar)) : "memory");
}

// ---------------------------------------------------------------------------
// TMEM <-> registers.  32x32b: thread i of the warp owns lane (base + i) and
// receives N consecutive 32-bit columns.  A warp may only touch the 32 lanes
// starting at 32 * (warp index % 4).
// ---------------------------------------------------------------------------
__device__ __forceinline__ void tmem_ld_x32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_st_x32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
        "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
        ::"r"(taddr),
          "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
          "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
          "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void tmem_ld_x16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_st_x16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
        ::"r"(taddr),
          "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Byte offset of 16-byte chunk `chunk` (0..7) of row `row` inside one 64-column
// block of a 128-byte-swizzled tile.
__device__ __forceinline__ uint32_t sw128_chunk_offset(int row, int chunk) {
    return (uint32_t)row * 128u + (uint32_t)((chunk ^ (row & 7)) << 4);
}

__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}

// Packs 8 f32 values (scaled by s) into eight f16 values: one 16-byte piece of an output row.
__device__ __forceinline__ uint4 pack8_f16(const uint32_t* r, float s) {
    uint4 a;
    a.x = pack_half2(__uint_as_float(r[0]) * s, __uint_as_float(r[1]) * s);
    a.y = pack_half2(__uint_as_float(r[2]) * s, __uint_as_float(r[3]) * s);
    a.z = pack_half2(__uint_as_float(r[4]) * s, __uint_as_float(r[5]) * s);
    a.w = pack_half2(__uint_as_float(r[6]) * s, __uint_as_float(r[7]) * s);
    return a;
}

// N x N transpose (N = 4 or 8) of 16-byte pieces among the N lanes of each aligned lane group:
// on return v[c] of the group's lane j holds what v[j] of the group's lane c held.  A thread that
// owns one row of a tile (the TMEM lane layout) enters with pieces 0..N-1 of its row and leaves
// with piece j of rows 0..N-1 of its group, so that the group's N lanes together store N*16
// contiguous bytes of one row per instruction instead of 16 bytes in each of N rows.
template <int N>
__device__ __forceinline__ void transpose_pieces(uint4 (&v)[N], uint32_t lane) {
#pragma unroll
    for (int s = 1; s < N; s <<= 1) {
        const bool upper = (lane & (uint32_t)s) != 0;
#pragma unroll
        for (int c = 0; c < N; ++c) {
            if (c & s) continue;
            // lanes l (bit s clear) and l|s exchange element (l, c|s) with element (l|s, c)
            const uint4 send = upper ? v[c] : v[c | s];
            uint4 recv;
            recv.x = __shfl_xor_sync(0xffffffffu, send.x, s);
            recv.y = __shfl_xor_sync(0xffffffffu, send.y, s);
            recv.z = __shfl_xor_sync(0xffffffffu, send.z, s);
            recv.w = __shfl_xor_sync(0xffffffffu, send.w, s);
            if (upper) v[c] = recv; else v[c | s] = recv;
        }
    }
}

}  // namespace sm100
