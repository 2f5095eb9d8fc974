// Thin inline-PTX wrappers for the sm_100a features the contraction kernels use:
// mbarriers, TMA (cp.async.bulk.tensor, tiled and im2col), tcgen05 (TMEM
// allocation, MMA issue, commit, TMEM loads) and the proxy fences between them.
//
// Every wait in this file is bounded: `mbar_wait` gives up after a wall-clock
// limit read from %globaltimer, raises a CTA-wide abort flag in shared memory and
// returns false, so that a kernel whose pipeline is mis-programmed ends with an
// error status instead of spinning forever.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace pmlb {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ bool elect_one() {
  uint32_t pred = 0;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "elect.sync _|p, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}\n"
      : "=r"(pred));
  return pred != 0;
}

// ---------------------------------------------------------------- programmatic dependent launch
//
// A kernel launched with the programmatic-stream-serialization attribute may start while the kernel
// before it in the stream is still running, once every CTA of that kernel has executed
// `launch_dependents` (or exited).  Its CTAs then run their set-up (barriers, TMEM, descriptor prefetch)
// on SMs the earlier kernel has already left and block in `grid_dependency_wait` until the earlier kernel
// has completed and its memory operations are visible.  Nothing that depends on, or could disturb, the
// earlier kernel's data may happen before that wait.  Without the launch attribute both are no-ops.

__device__ __forceinline__ void grid_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

__device__ __forceinline__ void grid_dependency_wait() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
}

// ---------------------------------------------------------------- mbarrier

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// Non-blocking probe of the same condition (try_wait may suspend the thread for a while before it
// answers; this form answers at once).
__device__ __forceinline__ bool mbar_test_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// The same probe with one answer for the warp (all 32 lanes call it): true only if every lane saw the phase
// complete, so that the lanes agree on whether a wait follows.
__device__ __forceinline__ bool mbar_test_wait_warp(uint32_t bar, uint32_t parity) {
  return __all_sync(0xffffffffu, mbar_test_wait(bar, parity)) != 0;
}

// Wall-clock limit of one barrier wait.  A healthy pipeline waits microseconds.
constexpr uint64_t kWaitLimitNs = 2000000000ull;

// Waits for the phase with the given parity.  Returns false when the CTA-wide
// abort flag is up or when the wait ran out of time (in which case it raises the
// flag itself).  `abort_flag` lives in shared memory: word 0 is the flag, word 1 the code of
// the role that gave up first (written by the callers), word 2 the wait limit of this launch in
// microseconds (0 = kWaitLimitNs).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
#pragma unroll 1
  for (int i = 0; i < 128; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
  }
  const uint64_t t0 = global_timer_ns();
#pragma unroll 1
  while (true) {
#pragma unroll 1
    for (int i = 0; i < 64; ++i) {
      if (mbar_try_wait(bar, parity)) return true;
    }
    if (*abort_flag != 0) return false;
    const uint64_t limit_us = static_cast<uint64_t>(abort_flag[2]);
    if (global_timer_ns() - t0 > (limit_us != 0 ? limit_us * 1000ull : kWaitLimitNs)) {
      *abort_flag = 1;
      return false;
    }
  }
}

// The same wait made by all 32 lanes of a warp, with one answer for the warp: false if any
// lane gave up.
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity,
                                               volatile int* abort_flag) {
  return __all_sync(0xffffffffu, mbar_wait(bar, parity, abort_flag)) != 0;
}

// ---------------------------------------------------------------- CTA pairs (clusters of two)

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}

// All threads of all CTAs of the cluster.
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::
                   : "memory");
}

// The shared::cluster address of the same shared-memory offset in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t mapa_rank(uint32_t cta_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(cta_addr), "r"(rank));
  return r;
}

// Arrive (count 1) on a barrier named by a shared::cluster address (possibly another CTA's).
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}

// ---------------------------------------------------------------- fences

__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// ---------------------------------------------------------------- TMA

__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

// Tiled 3-D load: coordinates innermost first.  x * element size must be a
// multiple of 16 bytes.
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, uint32_t bar,
                                            int x, int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5}], [%2];"
      :
      : "r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y), "r"(z)
      : "memory");
}

// Tiled 4-D load (coordinates innermost first; same alignment rule for x).  Coordinates other
// than x may lie outside the tensor: those elements arrive as zeros.
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, uint32_t bar,
                                            int x, int y, int z, int w) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6}], [%2];"
      :
      : "r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y), "r"(z), "r"(w)
      : "memory");
}

// The same issued by one CTA of a pair working on one tile (cta_group::2): the data lands in
// this CTA's shared memory, the bytes are counted on `bar_cluster`, a shared::cluster address
// that may name the other CTA's barrier.  No multicast: each CTA fetches its own part.
__device__ __forceinline__ void tma_load_3d_pair(uint32_t dst, const CUtensorMap* map,
                                                 uint32_t bar_cluster, int x, int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5}], [%2];"
      :
      : "r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster), "r"(x), "r"(y), "r"(z)
      : "memory");
}

__device__ __forceinline__ void tma_load_4d_pair(uint32_t dst, const CUtensorMap* map, uint32_t bar_cluster, int x,
                                                 int y, int z, int w) {
  asm volatile(
      "cp.async.bulk.tensor.4d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6}], [%2];"
      :
      : "r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster), "r"(x), "r"(y), "r"(z), "r"(w)
      : "memory");
}

// im2col 4-D load over an NHWC activation tensor described as (C, W, H, N):
// (w, h, n) is the base pixel inside the bounding box, (off_w, off_h) the filter
// tap offset added to every pixel; `pixelsPerColumn` pixels are walked W-then-H-
// then-N with the traversal strides recorded in the tensor map.
__device__ __forceinline__ void tma_load_im2col_4d(uint32_t dst, const CUtensorMap* map,
                                                   uint32_t bar, int c, int w, int h, int n,
                                                   uint16_t off_w, uint16_t off_h) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.im2col.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6}], [%2], {%7, %8};"
      :
      : "r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c), "r"(w), "r"(h), "r"(n),
        "h"(off_w), "h"(off_h)
      : "memory");
}

// The same from either CTA of a pair, completing on a barrier of the cluster (an address made
// with mapa): both CTAs' loads count on the first CTA's barrier.
__device__ __forceinline__ void tma_load_im2col_4d_pair(uint32_t dst, const CUtensorMap* map,
                                                        uint32_t bar_cluster, int c, int w, int h,
                                                        int n, uint16_t off_w, uint16_t off_h) {
  asm volatile(
      "cp.async.bulk.tensor.4d.cta_group::2.shared::cluster.global.im2col.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6}], [%2], {%7, %8};"
      :
      : "r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster), "r"(c), "r"(w), "r"(h),
        "r"(n), "h"(off_w), "h"(off_h)
      : "memory");
}

// Tiled 3-D store from shared memory (bulk async-group completion).  Elements outside the
// tensor are not written.  Coordinates must not be negative.
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* map, uint32_t src, int x, int y,
                                             int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
      :
      : "l"(reinterpret_cast<uint64_t>(map)), "r"(src), "r"(x), "r"(y), "r"(z)
      : "memory");
}

__device__ __forceinline__ void tma_store_4d(const CUtensorMap* map, uint32_t src, int x, int y,
                                             int z, int w) {
  asm volatile(
      "cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
      :
      : "l"(reinterpret_cast<uint64_t>(map)), "r"(src), "r"(x), "r"(y), "r"(z), "r"(w)
      : "memory");
}

// Untiled copy of `bytes` (a multiple of 16, both addresses 16-byte aligned) from global to
// shared memory, completing on an mbarrier.
__device__ __forceinline__ void bulk_load_1d(uint32_t dst_smem, const void* src, uint32_t bytes,
                                             uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(dst_smem), "l"(src), "r"(bytes), "r"(bar)
      : "memory");
}

__device__ __forceinline__ void bulk_commit_group() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}

// Waits until at most N of this thread's bulk groups still read their shared-memory source.
template <int N>
__device__ __forceinline__ void bulk_wait_group_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}

// Waits until at most N of this thread's bulk groups are incomplete.
template <int N>
__device__ __forceinline__ void bulk_wait_group() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

__device__ __forceinline__ uint4 ld_shared_v4(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "r"(addr)
               : "memory");
  return v;
}

__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint4 v) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y),
               "r"(v.z), "r"(v.w)
               : "memory");
}

// ---------------------------------------------------------------- tcgen05 / TMEM

// Whole-warp call.  Writes the TMEM base address of `ncols` columns (a power of
// two, >= 32) to the shared-memory word at `dst`.
__device__ __forceinline__ void tmem_alloc(uint32_t dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst),
               "r"(ncols)
               : "memory");
}

__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}

// CTA-pair variants: executed by one warp of each CTA of the pair.
__device__ __forceinline__ void tmem_alloc_pair(uint32_t dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst),
               "r"(ncols)
               : "memory");
}

__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}

// Pair variant of the commit below: arrives on the barrier at the same shared-memory offset
// in every CTA of `cta_mask` once the pair's MMAs issued so far by this thread have completed.
__device__ __forceinline__ void tc_commit_pair(uint32_t bar, uint16_t cta_mask) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64"
      " [%0], %1;" ::"r"(bar),
      "h"(cta_mask)
      : "memory");
}

// Arrives (count 1) on `bar` once every tcgen05.mma issued so far by this thread
// has completed.  Implies tcgen05.fence::before_thread_sync.
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   bar)
               : "memory");
}

// Shared-memory operand descriptor (64 bit) for a 128-byte-swizzled tile whose
// base is 1024-byte aligned.
//   bits [0,14)  start address >> 4        bits [16,30) leading byte offset >> 4
//   bits [32,46) stride byte offset >> 4   bits [46,48) version (1 on sm_100)
//   bits [61,64) layout type (2 = 128-byte swizzle)
__device__ __forceinline__ uint64_t make_smem_desc_sw128(uint32_t saddr, uint32_t lbo_bytes,
                                                         uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}

// The same for 32-byte rows in the 32-byte swizzle (16-byte chunk index ^ address bit 7): eight
// rows every 256 bytes.
__device__ __forceinline__ uint64_t make_smem_desc_sw32(uint32_t saddr, uint32_t lbo_bytes,
                                                        uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(6) << 61;
  return d;
}

// Two floats -> packed 16-bit pair (lo in the low half), round to nearest even; the RELU forms
// turn negative values into +0 in the same instruction (NaN stays NaN).
template <bool BF16, bool RELU>
__device__ __forceinline__ uint32_t cvt_pack16(float lo, float hi) {
  uint32_t d;
  if constexpr (BF16) {
    if constexpr (RELU) {
      asm("cvt.rn.relu.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
    } else {
      asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
    }
  } else {
    if constexpr (RELU) {
      asm("cvt.rn.relu.f16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
    } else {
      asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
    }
  }
  return d;
}

// max(x, 0) that keeps NaN (one instruction; -0 becomes +0)
__device__ __forceinline__ float relu_keep_nan(float x) {
  float d;
  asm("max.NaN.f32 %0, %1, 0f00000000;" : "=f"(d) : "f"(x));
  return d;
}

// 32-byte global store (one whole sector per lane); the address must be 32-byte aligned.
__device__ __forceinline__ void st_global_v8(void* ptr, const uint4& lo, const uint4& hi) {
  asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
               :
               : "l"(ptr), "r"(lo.x), "r"(lo.y), "r"(lo.z), "r"(lo.w), "r"(hi.x), "r"(hi.y), "r"(hi.z), "r"(hi.w)
               : "memory");
}

enum : int { kMmaF16 = 0, kMmaTf32 = 1, kMmaI8 = 2 };

// D[tmem] (+)= A[smem] * B[smem]; `accumulate` == 0 overwrites D.
template <int KIND>
__device__ __forceinline__ void tc_mma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                       uint32_t idesc, uint32_t accumulate) {
  if constexpr (KIND == kMmaF16) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
        "}\n"
        :
        : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
  } else if constexpr (KIND == kMmaTf32) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t"
        "}\n"
        :
        : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
  } else {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t"
        "}\n"
        :
        : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
  }
}

// The CTA-pair MMA: issued by one thread of the pair's first CTA; rows 0..127 of D / A belong
// to that CTA, rows 128..255 to the second, each CTA holds half of B's N rows, and the
// descriptors name the same shared-memory offsets in both.
template <int KIND>
__device__ __forceinline__ void tc_mma_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                            uint32_t idesc, uint32_t accumulate) {
  if constexpr (KIND == kMmaF16) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t"
        "}\n"
        :
        : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
  } else if constexpr (KIND == kMmaTf32) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, p;\n\t"
        "}\n"
        :
        : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
  } else {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t"
        "}\n"
        :
        : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
  }
}

// Four MMAs over one 128-byte k-block in a single statement: the operand descriptors are given
// as their low words (start address >> 4, which is all that changes from MMA to MMA) plus the
// constant high words; MMA j uses a_lo + j * a_step and b_lo + j * b_step.  Only the first
// MMA's accumulate flag is a run-time value.  The issuing thread has ~48 cycles per 64-wide
// MMA: every instruction saved here is tensor-pipe time gained.
template <int KIND, int CTAS>
__device__ __forceinline__ void tc_mma_x4(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t a_hi,
                                          uint32_t b_hi, uint32_t idesc, uint32_t accumulate_first,
                                          uint32_t a_step, uint32_t b_step) {
#define PMLB_MMA_X4(OPCODE)                                                            \
  asm volatile(                                                                        \
      "{\n\t"                                                                          \
      ".reg .pred p, q;\n\t"                                                           \
      ".reg .b64 da, db;\n\t"                                                          \
      ".reg .b32 ta, tb;\n\t"                                                          \
      "setp.ne.b32 p, %6, 0;\n\t"                                                      \
      "setp.eq.b32 q, %6, %6;\n\t"                                                     \
      "mov.b64 da, {%1, %3};\n\t"                                                      \
      "mov.b64 db, {%2, %4};\n\t" OPCODE " [%0], da, db, %5, p;\n\t"                   \
      "add.u32 ta, %1, %7;\n\t"                                                        \
      "add.u32 tb, %2, %8;\n\t"                                                        \
      "mov.b64 da, {ta, %3};\n\t"                                                      \
      "mov.b64 db, {tb, %4};\n\t" OPCODE " [%0], da, db, %5, q;\n\t"                   \
      "add.u32 ta, ta, %7;\n\t"                                                        \
      "add.u32 tb, tb, %8;\n\t"                                                        \
      "mov.b64 da, {ta, %3};\n\t"                                                      \
      "mov.b64 db, {tb, %4};\n\t" OPCODE " [%0], da, db, %5, q;\n\t"                   \
      "add.u32 ta, ta, %7;\n\t"                                                        \
      "add.u32 tb, tb, %8;\n\t"                                                        \
      "mov.b64 da, {ta, %3};\n\t"                                                      \
      "mov.b64 db, {tb, %4};\n\t" OPCODE " [%0], da, db, %5, q;\n\t"                   \
      "}\n"                                                                            \
      :                                                                                \
      : "r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(a_hi), "r"(b_hi), "r"(idesc),           \
        "r"(accumulate_first), "r"(a_step), "r"(b_step)                                \
      : "memory")
  if constexpr (CTAS == 2) {
    if constexpr (KIND == kMmaF16) {
      PMLB_MMA_X4("tcgen05.mma.cta_group::2.kind::f16");
    } else if constexpr (KIND == kMmaTf32) {
      PMLB_MMA_X4("tcgen05.mma.cta_group::2.kind::tf32");
    } else {
      PMLB_MMA_X4("tcgen05.mma.cta_group::2.kind::i8");
    }
  } else {
    if constexpr (KIND == kMmaF16) {
      PMLB_MMA_X4("tcgen05.mma.cta_group::1.kind::f16");
    } else if constexpr (KIND == kMmaTf32) {
      PMLB_MMA_X4("tcgen05.mma.cta_group::1.kind::tf32");
    } else {
      PMLB_MMA_X4("tcgen05.mma.cta_group::1.kind::i8");
    }
  }
#undef PMLB_MMA_X4
}

// 32 lanes x 32 columns of 32-bit accumulators: thread t of the warp receives
// lane (lane_base + t), columns [col, col + 32).
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]),
        "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]),
        "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]),
        "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]),
        "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
}

__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

}  // namespace pmlb
