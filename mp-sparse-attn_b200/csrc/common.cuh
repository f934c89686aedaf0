// Shared device-side building blocks for the sm_100a kernels: mbarrier, TMA (bulk and tiled, each
// CTA fetching its own tiles), tcgen05 (TMEM allocation, block-scaled MMA, scale-factor copy, loads and
// stores) and the descriptors they consume.  Every wait has an upper bound: when it expires the
// waiter records a code in a global status word and the kernel unwinds normally.
#pragma once
#include <cstdint>
#include <cuda_runtime.h>
#include <cuda.h>

#ifndef MPSA_WAIT_MODE
#define MPSA_WAIT_MODE 0
#endif

namespace mpsa {

// ---- status word written by kernels -----------------------------------------------------
enum KernelStatus : int {
  KS_OK = 0,
  KS_TIMEOUT_TMA = 1,     // a wait for TMA bytes expired
  KS_TIMEOUT_MMA = 2,     // a wait for tcgen05.commit expired
  KS_TIMEOUT_PIPE = 3,    // a wait between roles (consumer released / producer filled) expired
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}

// ---- mbarrier ---------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
// One probe of the barrier phase (the hardware may hold the thread for a short, implementation
// defined time before answering).
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
#if MPSA_WAIT_MODE == 1
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, 0x989680;\n\t"
#else
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
#endif
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Wait limit for any single barrier phase, in SM clock cycles (about two seconds at 2 GHz).
// Kernels here finish a phase in microseconds; hitting the limit means something upstream never
// arrived.
constexpr long long kWaitLimitCycles = 4000000000ll;

// Bounded wait.  Returns false when the limit expired (and records `code` in *status) or when
// another role already recorded a failure, so that every role unwinds promptly.
// BACKOFF = false is for pipelines whose phases last a few hundred cycles, where the back-off below would
// cost more than the wait itself.  `limit` (SM clock cycles) defaults to kWaitLimitCycles.
template <bool BACKOFF = true>
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int* status, int code,
                                          long long limit = kWaitLimitCycles) {
  if (mbar_try_wait(bar, parity)) return true;
#if MPSA_WAIT_MODE == 0
  // Reading the global nanosecond timer is slow; doing it once after the first unsuccessful probe
  // doubles as a back-off that keeps a waiting warp out of its scheduler's way.
  if (BACKOFF) {
    unsigned long long g0;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(g0));
    (void)g0;
  }
#endif
  const long long t0 = clock64();
  uint32_t spins = 0;
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
#if MPSA_WAIT_MODE == 2
    __nanosleep(40);
#endif
    if ((++spins & 0x3ff) == 0) {
      if (*(volatile int*)status != KS_OK) return false;
      if (clock64() - t0 > limit) {
        atomicCAS(status, KS_OK, code);
        return false;
      }
    }
  }
}

// ---- TMA --------------------------------------------------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(m) : "memory");
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* m, uint64_t* bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(m), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* m, uint64_t* bar, int x, int y,
                                            int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(dst)), "l"(m), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z)
      : "memory");
}
// Untiled bulk copy global -> shared; both addresses 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ---- tcgen05 / TMEM ---------------------------------------------------------------------
// Allocation is done by one full warp; the base address lands in *slot (shared memory).
__device__ __forceinline__ void tmem_alloc(uint32_t* slot, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot)),
               "r"(ncols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t base, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(base), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// Arrive (count 1) on `bar` when every tcgen05 operation issued so far by this thread is done.
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   smem_u32(bar))
               : "memory");
}
// 32 rows x 16 bytes of shared memory -> 32 lanes x 4 columns of TMEM, replicated into the four
// 32-lane quarters.  This is the move that places one 128x4 scale-factor tile.
__device__ __forceinline__ void tc_cp_32x128b_warpx4(uint32_t tmem, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(tmem), "l"(sdesc) : "memory");
}

// Shared-memory matrix descriptor (64 bit):
//   [0,14)  start address >> 4          [16,30) leading-dimension byte offset >> 4
//   [32,46) stride byte offset >> 4     [46,48) version = 1 on sm_100
//   [49,52) base offset (0: tiles are aligned to their swizzle period)
//   [61,64) layout: 0 none, 2 = 128-byte swizzle, 4 = 64-byte, 6 = 32-byte
// K-major operand tile stored as rows of SW bytes (SW = swizzle span): 8 rows form one
// swizzle period of 8*SW bytes, so the stride between 8-row groups is 8*SW.
__device__ __forceinline__ uint64_t make_sdesc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes,
                                               uint32_t layout) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr >> 4) & 0x3fff);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3fff) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3fff) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)(layout & 7) << 61;
  return d;
}
constexpr uint32_t kLayoutNone = 0, kLayoutSw128 = 2, kLayoutSw64 = 4;

__device__ __forceinline__ uint64_t sdesc_kmajor_sw128(uint32_t saddr) {
  return make_sdesc(saddr, 16, 1024, kLayoutSw128);
}
__device__ __forceinline__ uint64_t sdesc_kmajor_sw64(uint32_t saddr) {
  return make_sdesc(saddr, 16, 512, kLayoutSw64);
}
// One 512-byte scale-factor tile: 32 rows of 16 bytes, unswizzled; 8-row groups 128 bytes apart.
__device__ __forceinline__ uint64_t sdesc_sf_tile(uint32_t saddr) {
  return make_sdesc(saddr, 0, 128, kLayoutNone);
}

// Instruction descriptor of the block-scaled kinds (32 bit):
//   [4,6) B scale id   [7,10) A format   [10,13) B format   15/16 A/B major (0 = K-major)
//   [17,23) N>>3   23 scale format (1 = E8M0, 0 = E4M3)   [24,29) M>>4   [29,31) A scale id
// Formats for kind::mxf8f6f4: E4M3 0, E5M2 1, E2M1 5.  For kind::mxf4 / mxf4nvf4: E2M1 1.
__host__ __device__ constexpr uint32_t idesc_block_scaled(uint32_t afmt, uint32_t bfmt, uint32_t M, uint32_t N,
                                                          uint32_t sf_e8m0) {
  return (afmt << 7) | (bfmt << 10) | ((N >> 3) << 17) | (sf_e8m0 << 23) | ((M >> 4) << 24);
}
__host__ __device__ constexpr uint32_t idesc_with_sf_id(uint32_t idesc, uint32_t a_id, uint32_t b_id) {
  return idesc | (b_id << 4) | (a_id << 29);
}
// Instruction descriptor of kind::f16: [4,6) accumulator format (1 = f32), [7,10) A format
// (0 f16, 1 bf16), [10,13) B format, 15/16 majors, [17,23) N>>3, [24,29) M>>4.
__host__ __device__ constexpr uint32_t idesc_f16(uint32_t afmt, uint32_t bfmt, uint32_t M, uint32_t N) {
  return (1u << 4) | (afmt << 7) | (bfmt << 10) | ((N >> 3) << 17) | ((M >> 4) << 24);
}

// D[tmem] (+)= A[smem] * B[smem] with per-block scales read from TMEM.  One thread issues.
__device__ __forceinline__ void mma_mxf8f6f4(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t sfa,
                                             uint32_t sfb, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %6, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale.scale_vec::1X [%0], %1, %2, %3, [%4], [%5], p;\n\t}"
      ::"r"(d), "l"(a), "l"(b), "r"(idesc), "r"(sfa), "r"(sfb), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void mma_mxf4(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t sfa,
                                         uint32_t sfb, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %6, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf4.block_scale.scale_vec::2X [%0], %1, %2, %3, [%4], [%5], p;\n\t}"
      ::"r"(d), "l"(a), "l"(b), "r"(idesc), "r"(sfa), "r"(sfb), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void mma_nvf4(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t sfa,
                                         uint32_t sfb, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %6, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%4], [%5], p;\n\t}"
      ::"r"(d), "l"(a), "l"(b), "r"(idesc), "r"(sfa), "r"(sfb), "r"(accumulate)
      : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem], 16-bit floating operands.
__device__ __forceinline__ void mma_f16_ts(uint32_t d, uint32_t a_tmem, uint64_t b, uint32_t idesc,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d), "r"(a_tmem), "l"(b), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void mma_f16_ss(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d), "l"(a), "l"(b), "r"(idesc), "r"(accumulate)
      : "memory");
}

// TMEM -> registers: this thread's lane (warp quarter * 32 + lane id), 32 consecutive columns.
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
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
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// registers -> TMEM, 32 consecutive columns of this thread's lane.
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
      "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
        "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
        "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}

}  // namespace mpsa
