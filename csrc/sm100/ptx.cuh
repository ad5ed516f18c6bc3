// Thin inline-PTX wrappers for the sm_100a features the kernels in this tree use:
// mbarrier, TMA (cp.async.bulk[.tensor]), tcgen05 (TMEM alloc / mma / commit / ld) and
// system-scope flag traffic. Everything here is header-only device code.
//
// Conventions
//   * "bar", "smem_dst" ... are 32-bit shared-window addresses (see smem_u32()).
//   * every wait in this tree is bounded: see BoundedWait below.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace fluxb {
namespace ptx {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}


__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// barrier over all threads of the cluster, with release/acquire ordering
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of `saddr` (a shared::cta address) in CTA `cta_rank` of the cluster
__device__ __forceinline__ uint32_t mapa_u32(uint32_t saddr, uint32_t cta_rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(cta_rank));
  return r;
}

__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// ----------------------------------------------------------------------------------------
// mbarrier
// ----------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// Arrive without release ordering: for a hand-over whose data is already safe when the arrive is
// issued (TMEM reads completed by tcgen05.wait::ld). A release arrive also waits for the warp's
// global loads in flight.
__device__ __forceinline__ void mbar_arrive_relaxed(uint32_t bar) {
  asm volatile("mbarrier.arrive.relaxed.cta.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
// Arrive on the barrier at the same smem offset in another CTA of the cluster.
__device__ __forceinline__ void mbar_arrive_remote(uint32_t bar, uint32_t cta_rank) {
  asm volatile(
      "{\n"
      " .reg .b32 ra;\n"
      " mapa.shared::cluster.u32 ra, %0, %1;\n"
      " mbarrier.arrive.release.cluster.shared::cluster.b64 _, [ra];\n"
      "}\n" ::"r"(bar),
      "r"(cta_rank)
      : "memory");
}
// The same without release ordering: for a hand-over whose data is already safe when the arrive is
// issued (TMEM reads completed by tcgen05.wait::ld), so that the arrive does not wait for the warp's
// unrelated global loads in flight.
__device__ __forceinline__ void mbar_arrive_remote_relaxed(uint32_t bar, uint32_t cta_rank) {
  asm volatile(
      "{\n"
      " .reg .b32 ra;\n"
      " mapa.shared::cluster.u32 ra, %0, %1;\n"
      " mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [ra];\n"
      "}\n" ::"r"(bar),
      "r"(cta_rank)
      : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      " .reg .pred p;\n"
      " mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      " selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// ----------------------------------------------------------------------------------------
// fences
// ----------------------------------------------------------------------------------------
// generic-proxy writes to shared memory -> visible to the async proxy (TMA store / UMMA reads)
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
// generic <-> async proxy ordering for global memory (flag acquire -> TMA load of the data,
// TMA store completion -> flag release)
__device__ __forceinline__ void fence_proxy_async_all() {
  asm volatile("fence.proxy.async;" ::: "memory");
}
__device__ __forceinline__ void fence_acq_rel_sys() {
  asm volatile("fence.acq_rel.sys;" ::: "memory");
}

// ----------------------------------------------------------------------------------------
// TMA
// ----------------------------------------------------------------------------------------
__device__ __forceinline__ void prefetch_tmap(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}

// 2-D tiled load global -> shared, completion on an mbarrier of this CTA. No multicast.
__device__ __forceinline__ void tma_load_2d(uint32_t smem_dst, const CUtensorMap* m, uint32_t bar,
                                            int32_t x, int32_t y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];" ::"r"(smem_dst),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(x), "r"(y)
      : "memory");
}
// Same, for one CTA of a cta_group::2 pair: `bar` may be a shared::cluster address of the
// peer CTA's barrier (the pair leader collects the bytes of both CTAs).
__device__ __forceinline__ void tma_load_2d_cg2(uint32_t smem_dst, const CUtensorMap* m,
                                                uint32_t bar_cluster_addr, int32_t x, int32_t y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];" ::"r"(smem_dst),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(bar_cluster_addr), "r"(x), "r"(y)
      : "memory");
}
// L2 eviction policies for loads whose reuse pattern is known (operand band kept across waves:
// evict_last; operand streamed once per wave: evict_first)
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
  uint64_t pol;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}
__device__ __forceinline__ uint64_t l2_policy_evict_last() {
  uint64_t pol;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}
__device__ __forceinline__ void tma_load_2d_hint(uint32_t smem_dst, const CUtensorMap* m, uint32_t bar,
                                                 int32_t x, int32_t y, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
      " [%0], [%1, {%3, %4}], [%2], %5;" ::"r"(smem_dst),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(x), "r"(y), "l"(policy)
      : "memory");
}
__device__ __forceinline__ void tma_load_2d_cg2_hint(uint32_t smem_dst, const CUtensorMap* m,
                                                     uint32_t bar_cluster_addr, int32_t x, int32_t y,
                                                     uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
      " [%0], [%1, {%3, %4}], [%2], %5;" ::"r"(smem_dst),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(bar_cluster_addr), "r"(x), "r"(y), "l"(policy)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t smem_dst, const CUtensorMap* m, uint32_t bar,
                                            int32_t x, int32_t y, int32_t z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5}], [%2];" ::"r"(smem_dst),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(x), "r"(y), "r"(z)
      : "memory");
}
__device__ __forceinline__ void tma_load_4d(uint32_t smem_dst, const CUtensorMap* m, uint32_t bar,
                                            int32_t x, int32_t y, int32_t z, int32_t w) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6}], [%2];" ::"r"(smem_dst),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(x), "r"(y), "r"(z), "r"(w)
      : "memory");
}
__device__ __forceinline__ void tma_load_4d_cg2(uint32_t smem_dst, const CUtensorMap* m,
                                                uint32_t bar_cluster_addr, int32_t x, int32_t y,
                                                int32_t z, int32_t w) {
  asm volatile(
      "cp.async.bulk.tensor.4d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6}], [%2];" ::"r"(smem_dst),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(bar_cluster_addr), "r"(x), "r"(y), "r"(z), "r"(w)
      : "memory");
}
__device__ __forceinline__ void tma_store_4d(const CUtensorMap* m, uint32_t smem_src, int32_t x,
                                             int32_t y, int32_t z, int32_t w) {
  asm volatile(
      "cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];" ::"l"(
          reinterpret_cast<uint64_t>(m)),
      "r"(smem_src), "r"(x), "r"(y), "r"(z), "r"(w)
      : "memory");
}
// Four rows of a 2-D tensor picked by index (y0..y3), `box` columns starting at x, written as four
// consecutive rows at smem_dst. The tensor map's box is {columns, 1}.
__device__ __forceinline__ void tma_gather4_2d(uint32_t smem_dst, const CUtensorMap* m, uint32_t bar,
                                               int32_t x, int32_t y0, int32_t y1, int32_t y2, int32_t y3) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile::gather4.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6, %7}], [%2];" ::"r"(smem_dst),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(x), "r"(y0), "r"(y1), "r"(y2), "r"(y3)
      : "memory");
}
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* m, uint32_t smem_src, int32_t x,
                                             int32_t y, int32_t z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(
          reinterpret_cast<uint64_t>(m)),
      "r"(smem_src), "r"(x), "r"(y), "r"(z)
      : "memory");
}
__device__ __forceinline__ void bulk_commit() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
// wait until at most N of this thread's bulk groups still READ their shared source
template <int N>
__device__ __forceinline__ void bulk_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
// wait until at most N of this thread's bulk groups are incomplete (writes performed)
template <int N>
__device__ __forceinline__ void bulk_wait() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}
// untiled bulk copies (16-byte aligned addresses, size multiple of 16)
__device__ __forceinline__ void bulk_load(uint32_t smem_dst, const void* gsrc, uint32_t bytes,
                                          uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::
          "r"(smem_dst),
      "l"(reinterpret_cast<uint64_t>(gsrc)), "r"(bytes), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void bulk_store(void* gdst, uint32_t smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(
                   reinterpret_cast<uint64_t>(gdst)),
               "r"(smem_src), "r"(bytes)
               : "memory");
}

// 16-byte asynchronous copy global -> shared (generic proxy); bytes past src_size are zero-filled
__device__ __forceinline__ void cp_async_16(uint32_t smem_dst, const void* gsrc, uint32_t src_size) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_dst),
               "l"(reinterpret_cast<uint64_t>(gsrc)), "r"(src_size)
               : "memory");
}
// the barrier receives one arrival (already counted in its init value) once all cp.async issued
// so far by this thread have landed
__device__ __forceinline__ void cp_async_mbar_arrive_noinc(uint32_t bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}

// ----------------------------------------------------------------------------------------
// tcgen05 / TMEM
// ----------------------------------------------------------------------------------------
// Shared-memory matrix descriptor, K-major operand stored as rows of 128 bytes with the
// 128-byte swizzle (the layout a SWIZZLE_128B TMA box of 64 x 16-bit or 128 x 8-bit elements
// produces): 8-row groups are 1024 bytes apart (SBO), LBO unused, descriptor version 1.
// Stepping along K inside the 128-byte row is done by adding the byte offset to `saddr`.
__device__ __forceinline__ uint64_t umma_desc_k_sw128(uint32_t saddr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>(1024u >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}
// MN-major operand (rows of 64 16-bit elements along M/N, SWIZZLE_128B): consecutive
// 64-element column groups are LBO apart, 8-k-row groups SBO apart.
__device__ __forceinline__ uint64_t umma_desc_mn_sw128(uint32_t saddr, uint32_t lbo_bytes,
                                                       uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}

// Instruction descriptor: D fp32; A/B formats: kind::f16 -> 0 = f16, 1 = bf16;
// kind::f8f6f4 -> 0 = e4m3, 1 = e5m2. Majors: 0 = K-major, 1 = MN-major.
// kind::i8 -> 0 = u8, 1 = s8 with D s32 (c_fmt 2).
__host__ __device__ constexpr uint32_t umma_idesc(uint32_t a_fmt, uint32_t b_fmt, uint32_t m,
                                                  uint32_t n, uint32_t a_major = 0,
                                                  uint32_t b_major = 0, uint32_t c_fmt = 1) {
  return (c_fmt << 4) | (a_fmt << 7) | (b_fmt << 10) | (a_major << 15) | (b_major << 16) |
         ((n >> 3) << 17) | ((m >> 4) << 24);
}

template <int CG>
__device__ __forceinline__ void tmem_alloc(uint32_t smem_result, uint32_t ncols) {
  if constexpr (CG == 1)
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_result),
                 "r"(ncols)
                 : "memory");
  else
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_result),
                 "r"(ncols)
                 : "memory");
}
template <int CG>
__device__ __forceinline__ void tmem_relinquish() {
  if constexpr (CG == 1)
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  else
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
template <int CG>
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  if constexpr (CG == 1)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
                 : "memory");
  else
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// D[tmem] (+)= A[smem] * B[smem]; one thread issues. kind: 0 = f16/bf16, 1 = f8f6f4.
template <int CG, int KIND>
__device__ __forceinline__ void umma_ss(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc,
                                        uint32_t idesc, uint32_t accumulate) {
  if constexpr (CG == 1 && KIND == 0)
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
        " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
  else if constexpr (CG == 2 && KIND == 0)
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
        " tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
  else if constexpr (CG == 1 && KIND == 1)
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
        " tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n}\n" ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
  else if constexpr (CG == 2 && KIND == 1)
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
        " tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n}\n" ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
  else if constexpr (CG == 1 && KIND == 2)
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
        " tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n}\n" ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
  else
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
        " tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n}\n" ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// mbarrier arrive once all previously issued tcgen05.mma of this thread have completed.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   bar)
               : "memory");
}
// cta_group::2: signal the barrier at this smem offset in every CTA named in cta_mask.
__device__ __forceinline__ void umma_commit_cg2(uint32_t bar, uint16_t cta_mask) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64"
      " [%0], %1;" ::"r"(bar),
      "h"(cta_mask)
      : "memory");
}

// TMEM -> registers: this warp's 32 lanes x 32 consecutive fp32 columns (thread = lane/row).
__device__ __forceinline__ void tmem_ld_32x32b_x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
// per-warpgroup register reallocation (all four warps of the group execute it)
template <int N>
__device__ __forceinline__ void setmaxnreg_inc() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N));
}
template <int N>
__device__ __forceinline__ void setmaxnreg_dec() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N));
}
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// ----------------------------------------------------------------------------------------
// flags in (peer) global memory
// ----------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// gpu-scope arrival counting between CTAs of this GPU (the flag that follows carries sys scope)
__device__ __forceinline__ uint32_t atom_add_acq_rel_gpu(uint32_t* p, uint32_t v) {
  uint32_t old;
  asm volatile("atom.add.acq_rel.gpu.global.u32 %0, [%1], %2;" : "=r"(old) : "l"(p), "r"(v) : "memory");
  return old;
}
__device__ __forceinline__ uint32_t atom_add_acq_rel_sys(uint32_t* p, uint32_t v) {
  uint32_t old;
  asm volatile("atom.acq_rel.sys.global.add.u32 %0, [%1], %2;" : "=r"(old) : "l"(p), "r"(v) : "memory");
  return old;
}
__device__ __forceinline__ void st_global_v4(void* p, uint4 v) {
  asm volatile("st.global.v4.b32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z),
               "r"(v.w)
               : "memory");
}
__device__ __forceinline__ uint4 ld_global_v4(const void* p) {
  uint4 v;
  asm volatile("ld.global.v4.b32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
// streaming (evict-first) 16-byte load for data read exactly once
__device__ __forceinline__ uint4 ld_global_cs_v4(const void* p) {
  uint4 v;
  asm volatile("ld.global.cs.v4.b32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ uint32_t pack_f16x2(float lo, float hi) {
  __half2 v = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// packed fp32 pairs (sm_100 has a two-wide fp32 FMA)
__device__ __forceinline__ uint64_t pack_b32x2(uint32_t lo, uint32_t hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(lo), "r"(hi));
  return r;
}
__device__ __forceinline__ uint64_t pack_f32x2(float lo, float hi) {
  return pack_b32x2(__float_as_uint(lo), __float_as_uint(hi));
}
__device__ __forceinline__ uint64_t ffma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}

// epilogue activations: 1 gelu (tanh form), 2 relu, 3 silu
__device__ __forceinline__ float activate(float x, int kind) {
  if (kind == 1) {
    const float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
    // tanh(u) = 1 - 2 / (exp(2u) + 1)
    const float t = 1.f - 2.f / (__expf(2.f * u) + 1.f);
    return 0.5f * x * (1.f + t);
  }
  if (kind == 2) return fmaxf(x, 0.f);
  if (kind == 3) return x / (1.f + __expf(-x));
  return x;
}

// 16-bit float (bf16 or fp16, chosen at run time) helpers for epilogues
__device__ __forceinline__ float half_bits_to_float(uint16_t b, bool f16) {
  if (f16) return __half2float(__ushort_as_half(b));
  return __uint_as_float(static_cast<uint32_t>(b) << 16);
}
__device__ __forceinline__ uint32_t pack_half2(bool f16, float lo, float hi) {
  return f16 ? pack_f16x2(lo, hi) : pack_bf16x2(lo, hi);
}

}  // namespace ptx

// ----------------------------------------------------------------------------------------
// Bounded waits. A kernel owns one Status record in global memory (written by the device,
// read by the host after the op) and one abort word in shared memory. The first wait that
// runs out of time records where it gave up and raises the abort word; every later wait in
// the CTA then returns at once, so the kernel drains through its normal exit path (TMEM
// freed, barriers invalidated) with garbage results and a non-zero status instead of
// hanging the GPU.
// ----------------------------------------------------------------------------------------
struct Status {
  uint32_t code;      // 0 = ok, else (site id) of the first wait that timed out
  uint32_t block;     // blockIdx.x that recorded it
  uint32_t detail0;   // site-specific (e.g. value seen)
  uint32_t detail1;   // site-specific (e.g. value expected)
};

enum WaitSite : uint32_t {
  kSiteNone = 0,
  kSiteSmemEmpty = 1,
  kSiteSmemFull = 2,
  kSiteTmemEmpty = 3,
  kSiteTmemFull = 4,
  kSiteStartBarrier = 5,
  kSiteShardFlag = 6,
  kSiteTileCounter = 7,
  kSiteBarrierAll = 8,
  kSiteInplaceCast = 9,
  kSiteA2AFlag = 10,
  kSiteMoeFlag = 11,
  kSiteTest = 12,
  kSiteCapacity = 13,   // not a wait: more rows were routed to a rank than its receive buffer holds
};

struct WaitCtx {
  Status* status;          // global
  volatile uint32_t* abort;  // shared
  uint64_t timeout_ns;
};

__device__ __forceinline__ void wait_give_up(const WaitCtx& w, uint32_t site, uint32_t d0,
                                             uint32_t d1) {
  *w.abort = 1;
  if (w.status != nullptr && atomicCAS(&w.status->code, 0u, site) == 0u) {
    w.status->block = blockIdx.x;
    w.status->detail0 = d0;
    w.status->detail1 = d1;
  }
}

// Self-checks of the kernels, compiled in with -DFLUXB_DEBUG_CHECKS (the debug build of the
// library): a failed check records its site (100 + id) and two details in the status record,
// raises the CTA's abort word and tells the caller to skip the access it guards. In the normal
// build dcheck() is the constant true and the checks cost nothing.
enum CheckSite : uint32_t {
  kCheckTileDecode = 101,   // tile coordinates outside the problem
  kCheckAgPush = 102,       // all-gather push: piece outside the shard / misaligned
  kCheckA2APush = 103,      // post-attention push: piece outside the source or the landing slab
  kCheckMoeGather = 104,    // MoE row gather: token index outside the token matrix
  kCheckFlagEpoch = 105,    // a flag carries a call number far ahead of the current call
  kCheckStore = 106,        // epilogue store outside the output
};
#ifdef FLUXB_DEBUG_CHECKS
__device__ __forceinline__ bool dcheck(const WaitCtx& w, bool ok, uint32_t site, uint32_t d0, uint32_t d1) {
  if (!ok) wait_give_up(w, site, d0, d1);
  return ok;
}
#else
__device__ __forceinline__ constexpr bool dcheck(const WaitCtx&, bool, uint32_t, uint32_t, uint32_t) {
  return true;
}
#endif

// Wait for the mbarrier phase with the given parity. Returns false if it gave up.
__device__ __forceinline__ bool mbar_wait(const WaitCtx& w, uint32_t bar, uint32_t parity,
                                          uint32_t site) {
  if (ptx::mbar_try_wait(bar, parity)) return true;
  if (*w.abort) return false;
  const uint64_t t0 = ptx::globaltimer_ns();
  uint32_t spins = 0;
  while (!ptx::mbar_try_wait(bar, parity)) {
    if ((++spins & 63u) == 0u) {
      if (*w.abort) return false;
      if (ptx::globaltimer_ns() - t0 > w.timeout_ns) {
        wait_give_up(w, site, bar, parity);
        return false;
      }
    }
  }
  return true;
}

// Wait until *flag >= expected (system-scope acquire; flags only ever grow). One thread.
__device__ __forceinline__ bool flag_wait_ge(const WaitCtx& w, const uint32_t* flag,
                                             uint32_t expected, uint32_t site) {
  uint32_t v = ptx::ld_acquire_sys(flag);
  if (static_cast<int32_t>(v - expected) >= 0)
    return dcheck(w, v - expected < (1u << 24), kCheckFlagEpoch, v, expected);
  if (*w.abort) return false;
  const uint64_t t0 = ptx::globaltimer_ns();
  uint32_t spins = 0;
  while (true) {
    v = ptx::ld_acquire_sys(flag);
    if (static_cast<int32_t>(v - expected) >= 0)
      return dcheck(w, v - expected < (1u << 24), kCheckFlagEpoch, v, expected);
    if ((++spins & 31u) == 0u) {
      if (*w.abort) return false;
      if (ptx::globaltimer_ns() - t0 > w.timeout_ns) {
        wait_give_up(w, site, v, expected);
        return false;
      }
    }
    __nanosleep(40);
  }
}

}  // namespace fluxb
