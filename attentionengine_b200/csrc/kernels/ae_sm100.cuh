// Device-side building blocks for sm_100a kernels: mbarrier, TMA (non-multicast),
// tcgen05 MMA / TMEM, UMMA descriptors.  Self-contained: compiles under NVRTC and
// nvcc without any CUDA or C++ standard header.
//
// Every wait in this file is bounded.  A wait that runs out records a code in the
// CTA's abort word (shared memory) and in the global status word, after which all
// later waits of the CTA return at once, so every warp still reaches the common
// exit path (TMEM dealloc included) and the context stays usable.
#pragma once

typedef unsigned char u8;
typedef unsigned short u16;
typedef unsigned int u32;
typedef unsigned long long u64;
typedef long long i64;

#define AE_DEVICE __device__ __forceinline__

struct alignas(64) AeTmaDesc {
  u64 opaque[16];
};

// ---------------------------------------------------------------------------
// status codes written to the global status word (0 = ok)
// ---------------------------------------------------------------------------
#define AE_ST_OK 0u
#define AE_ST_TIMEOUT_BASE 0x100u  // + site id of the wait that gave up

AE_DEVICE u32 smem_u32(const void* p) { return (u32)__cvta_generic_to_shared(p); }

AE_DEVICE u32 lane_id() {
  u32 r;
  asm volatile("mov.u32 %0, %%laneid;" : "=r"(r));
  return r;
}

AE_DEVICE bool elect_one() {
  u32 pred = 0;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "elect.sync _|p, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}\n"
      : "=r"(pred));
  return pred != 0;
}

// ---------------------------------------------------------------------------
// mbarrier
// ---------------------------------------------------------------------------
AE_DEVICE void mbar_init(u64* bar, u32 count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
AE_DEVICE void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
AE_DEVICE void mbar_arrive(u64* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// One arrival per warp: all lanes have finished their part (their own fences included), lane 0 arrives for
// the warp.  Barriers used this way are initialised with the number of warps, not threads: a few arrivals
// on the shared-memory word instead of 128 or 256 serialised ones.
AE_DEVICE void mbar_arrive_warp(u64* bar) {
  __syncwarp();
  if (lane_id() == 0) mbar_arrive(bar);
}
AE_DEVICE void mbar_arrive_expect_tx(u64* bar, u32 bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
// One poll of an mbarrier phase.  AE_WAIT_MODE selects the instruction:
//   0  mbarrier.try_wait with a suspend-time hint (the thread may be parked by the hardware; fewest issue slots)
//   1  mbarrier.try_wait without a hint
//   2  mbarrier.test_wait (never blocks; lowest wake-up latency, most issue slots)
#ifndef AE_WAIT_MODE
#define AE_WAIT_MODE 0
#endif
AE_DEVICE bool mbar_try_wait(u64* bar, u32 parity) {
  u32 ok;
#if AE_WAIT_MODE == 0
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity), "r"(20000u)
      : "memory");
#elif AE_WAIT_MODE == 1
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
#else
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
#endif
  return ok != 0;
}

struct AeTrue {
  static constexpr bool value = true;
};
struct AeFalse {
  static constexpr bool value = false;
};
template <int N>
struct AeInt {
  static constexpr int value = N;
};

// Shared per-CTA control block used by the bounded waits.
struct AeCtaCtl {
  volatile u32 abort;  // != 0 once any wait of this CTA has given up
  u32 tmem_base;       // written by tcgen05.alloc
};

#ifndef AE_WAIT_CYCLES
#define AE_WAIT_CYCLES 2000000000ll  // about one second at B200 clocks
#endif

// Bounded wait on an mbarrier phase.  Returns false when the CTA is aborting.
// mbarrier.try_wait may itself block for a system-dependent time, so the clock and the abort
// word are checked after every failed poll.
AE_DEVICE bool mbar_wait(u64* bar, u32 parity, AeCtaCtl* ctl, u32* g_status, u32 site) {
  if (mbar_try_wait(bar, parity)) return true;
  const i64 t0 = clock64();
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
    if (ctl->abort) return false;
    if (clock64() - t0 > AE_WAIT_CYCLES) {
      ctl->abort = 1;
      if (g_status) atomicCAS(g_status, 0u, AE_ST_TIMEOUT_BASE + site);
      return false;
    }
  }
}

// The same wait run by every lane of a warp; the result is made warp-uniform by a vote.
AE_DEVICE bool mbar_wait_w(u64* bar, u32 parity, AeCtaCtl* ctl, u32* g_status, u32 site) {
  return __all_sync(0xffffffffu, mbar_wait(bar, parity, ctl, g_status, site));
}

// ---------------------------------------------------------------------------
// proxies / fences
// ---------------------------------------------------------------------------
AE_DEVICE void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
AE_DEVICE void tc_fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
AE_DEVICE void tc_fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
AE_DEVICE void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
AE_DEVICE void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// Non-blocking arrival on a named barrier (the waiting side calls named_bar_sync with the same id and count).
// A named barrier costs the waiting warp about 20 clk, an mbarrier wait 100 - 400 clk; it has no time-out, so it is
// only used where the arriving side is guaranteed to arrive (row threads arrive in every iteration, aborted or not).
AE_DEVICE void named_bar_arrive(u32 id, u32 nthreads) {
  asm volatile("bar.arrive %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}
AE_DEVICE void named_bar_sync(u32 id, u32 nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// ---------------------------------------------------------------------------
// TMA (cp.async.bulk.tensor), never multicast: each CTA issues its own loads
// ---------------------------------------------------------------------------
AE_DEVICE void tma_prefetch_desc(const AeTmaDesc* d) {
  asm volatile("prefetch.tensormap [%0];" ::"l"((u64)d) : "memory");
}
// Bring a box into L2 only (no shared-memory destination, no barrier): for tiles that will be loaded a few steps later.
AE_DEVICE void tma_prefetch_l2_4d(const AeTmaDesc* d, int c0, int c1, int c2, int c3) {
  asm volatile("cp.async.bulk.prefetch.tensor.4d.L2.global.tile [%0, {%1, %2, %3, %4}];" ::"l"((u64)d), "r"(c0), "r"(c1),
               "r"(c2), "r"(c3)
               : "memory");
}
AE_DEVICE void tma_load_4d(void* smem_dst, const AeTmaDesc* d, u64* bar, int c0, int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"((u64)d), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
// A [rows x 64 elements] box of a [B, S, H, D] tensor (any strides): the tensor map's dimensions are ordered
// (d, s, h, b), so the box is {64, rows, 1, 1} and its rows are the map's second dimension.
AE_DEVICE void tma_load_bshd(void* smem_dst, const AeTmaDesc* d, u64* bar, int d0, int h, int s0, int b) {
  tma_load_4d(smem_dst, d, bar, d0, s0, h, b);
}
AE_DEVICE void tma_load_3d(void* smem_dst, const AeTmaDesc* d, u64* bar, int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"((u64)d), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
AE_DEVICE void tma_load_2d(void* smem_dst, const AeTmaDesc* d, u64* bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"((u64)d), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
      : "memory");
}
AE_DEVICE void tma_store_4d(const AeTmaDesc* d, const void* smem_src, int c0, int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
      ::"l"((u64)d), "r"(smem_u32(smem_src)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
AE_DEVICE void tma_store_3d(const AeTmaDesc* d, const void* smem_src, int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
      ::"l"((u64)d), "r"(smem_u32(smem_src)), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
AE_DEVICE void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
AE_DEVICE void tma_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
AE_DEVICE void tma_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }

// ---------------------------------------------------------------------------
// TMEM allocation (one warp, all 32 lanes)
// ---------------------------------------------------------------------------
AE_DEVICE void tmem_alloc(u32* smem_out, u32 ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_out)),
               "r"(ncols)
               : "memory");
}
AE_DEVICE void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
AE_DEVICE void tmem_dealloc(u32 taddr, u32 ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

// ---------------------------------------------------------------------------
// UMMA descriptors
// ---------------------------------------------------------------------------
// Shared-memory operand descriptor, 128-byte swizzle, descriptor version 1.
//   K-major tile  (rows of 64 x 16-bit = 128 B, 8-row groups 1024 B apart): sbo = 1024, lbo unused.
//   MN-major tile (K rows of 128 B holding 64 MN elements, 8-row groups 1024 B
//   apart, next 64 MN elements `lbo` bytes away): sbo = 1024, lbo = bytes between 64-wide MN blocks.
AE_DEVICE u64 umma_smem_desc_sw128(u32 smem_addr, u32 lbo_bytes, u32 sbo_bytes) {
  u64 d = 0;
  d |= (u64)((smem_addr & 0x3ffffu) >> 4);
  d |= (u64)((lbo_bytes >> 4) & 0x3fffu) << 16;
  d |= (u64)((sbo_bytes >> 4) & 0x3fffu) << 32;
  d |= (u64)1 << 46;  // descriptor version (Blackwell)
  d |= (u64)2 << 61;  // SWIZZLE_128B
  return d;
}

// Instruction descriptor for kind::f16 (fp16 or bf16 inputs, fp32 accumulate).
//   ab_fmt: 0 = f16, 1 = bf16.  a_mn / b_mn: 1 = operand is MN-major in shared memory.
AE_DEVICE constexpr u32 umma_idesc_f16(u32 M, u32 N, u32 ab_fmt, u32 a_mn, u32 b_mn) {
  return (1u << 4)            // D format f32
         | (ab_fmt << 7)      // A format
         | (ab_fmt << 10)     // B format
         | (a_mn << 15)       // A major
         | (b_mn << 16)       // B major
         | ((N >> 3) << 17)   // N / 8
         | ((M >> 4) << 24);  // M / 16
}

// D[tmem] (+)= A[smem] * B[smem]; issued by one thread.
AE_DEVICE void umma_ss(u32 tmem_d, u64 desc_a, u64 desc_b, u32 idesc, u32 accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n" ::"r"(tmem_d),
      "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]; issued by one thread.
AE_DEVICE void umma_ts(u32 tmem_d, u32 tmem_a, u64 desc_b, u32 idesc, u32 accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
      "}\n" ::"r"(tmem_d),
      "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Warp-level forms for an MMA-issuing warp whose 32 lanes all run the control flow: operands (descriptors, TMEM
// addresses, loop counters) then stay warp-uniform, which lets them live in uniform registers, the operand class
// tcgen05.mma takes; only the instruction itself is issued by one elected lane.
AE_DEVICE void umma_ss_w(u32 tmem_d, u64 desc_a, u64 desc_b, u32 idesc, u32 accumulate) {
  if (elect_one()) umma_ss(tmem_d, desc_a, desc_b, idesc, accumulate);
}
AE_DEVICE void umma_ts_w(u32 tmem_d, u32 tmem_a, u64 desc_b, u32 idesc, u32 accumulate) {
  if (elect_one()) umma_ts(tmem_d, tmem_a, desc_b, idesc, accumulate);
}
// All MMAs issued so far by this thread arrive on `bar` when they complete.
AE_DEVICE void umma_commit(u64* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
AE_DEVICE void umma_commit_w(u64* bar) {
  if (elect_one()) umma_commit(bar);
}

// ---------------------------------------------------------------------------
// CTA pairs (cluster of two CTAs on one TPC, tcgen05 ... .cta_group::2)
// One MMA of the pair covers 256 rows: each CTA holds its own 128 rows of A (shared memory or TMEM) and of D (TMEM),
// and half of B (N / 2 columns) in its own shared memory; the even CTA of the pair issues.  All tcgen05 instructions
// of a kernel that take a .cta_group use the same one, so a pair kernel uses only the wrappers below.
// ---------------------------------------------------------------------------
AE_DEVICE u32 cluster_ctarank() {
  u32 r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// every thread of every CTA of the cluster (no time-out: placed where all threads arrive whatever happened before)
AE_DEVICE void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of this CTA's shared-memory address `addr` in the CTA of rank `rank`
AE_DEVICE u32 mapa_u32(u32 addr, u32 rank) {
  u32 r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
// AE_PAIR_SCOPE 1: arrivals and waits between the CTAs of a pair carry release / acquire at cluster scope; 0 (default):
// the instructions' default scope.  What crosses between the CTAs of the pair kernels is TMEM and shared memory read
// and written by the tensor cores and TMA, ordered by tcgen05.fence / tcgen05.commit and the mbarrier itself, not
// generic-proxy memory; cluster-scope acquires on every wait cost the pair forward 20 % and changed no result.
#ifndef AE_PAIR_SCOPE
#define AE_PAIR_SCOPE 0
#endif
AE_DEVICE void mbar_arrive_cluster(u32 cluster_addr) {
#if AE_PAIR_SCOPE
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
#else
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
#endif
}
// Bounded wait on a barrier that the other CTA of the pair (its threads or its tensor core) arrives on.
AE_DEVICE bool mbar_try_wait_cl(u64* bar, u32 parity) {
#if !AE_PAIR_SCOPE
  return mbar_try_wait(bar, parity);
#endif
  u32 ok;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity), "r"(20000u)
      : "memory");
  return ok != 0;
}
AE_DEVICE bool mbar_wait_cl(u64* bar, u32 parity, AeCtaCtl* ctl, u32* g_status, u32 site) {
  if (mbar_try_wait_cl(bar, parity)) return true;
  const i64 t0 = clock64();
  while (true) {
    if (mbar_try_wait_cl(bar, parity)) return true;
    if (ctl->abort) return false;
    if (clock64() - t0 > AE_WAIT_CYCLES) {
      ctl->abort = 1;
      if (g_status) atomicCAS(g_status, 0u, AE_ST_TIMEOUT_BASE + site);
      return false;
    }
  }
}
// TMEM allocation of a pair: one warp of EACH CTA runs it (a collective of the two); both get the same base.
AE_DEVICE void tmem_alloc2(u32* smem_out, u32 ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_out)),
               "r"(ncols)
               : "memory");
}
AE_DEVICE void tmem_relinquish2() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
AE_DEVICE void tmem_dealloc2(u32 taddr, u32 ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
AE_DEVICE void umma_ss2(u32 tmem_d, u64 desc_a, u64 desc_b, u32 idesc, u32 accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n" ::"r"(tmem_d),
      "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
AE_DEVICE void umma_ts2(u32 tmem_d, u32 tmem_a, u64 desc_b, u32 idesc, u32 accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], [%1], %2, %3, p;\n\t"
      "}\n" ::"r"(tmem_d),
      "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// All MMAs issued so far by this thread arrive, when complete, on the barrier at this offset in BOTH CTAs of the pair.
AE_DEVICE void umma_commit2(u64* bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
                   smem_u32(bar)),
               "h"((u16)3)
               : "memory");
}

// ---------------------------------------------------------------------------
// TMEM <-> registers.  Shape 32x32b: lane i of the warp owns TMEM lane
// (32 * (warp_id % 4) + i); register j holds column (col0 + j).
// ---------------------------------------------------------------------------
AE_DEVICE void tmem_ld32(u32 taddr, u32 (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
AE_DEVICE void tmem_ld16(u32 taddr, u32 (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
AE_DEVICE void tmem_st32(u32 taddr, const u32 (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
      "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
      "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
      "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
AE_DEVICE void tmem_st16(u32 taddr, const u32 (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
      "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}

// ---------------------------------------------------------------------------
// numeric helpers
// ---------------------------------------------------------------------------
// Pack two fp32 into one 32-bit word of 16-bit floats; `lo` lands in bits [0,16).
template <int kBf16>
AE_DEVICE u32 pack2(float lo, float hi) {
  u32 r;
  if (kBf16) {
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  } else {
    asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  }
  return r;
}
template <int kBf16>
AE_DEVICE float unpack_lo(u32 w) {
  if (kBf16) return __uint_as_float(w << 16);
  float f;
  asm("{ .reg .b16 l, h; mov.b32 {l, h}, %1; cvt.f32.f16 %0, l; }" : "=f"(f) : "r"(w));
  return f;
}
template <int kBf16>
AE_DEVICE float unpack_hi(u32 w) {
  if (kBf16) return __uint_as_float(w & 0xffff0000u);
  float f;
  asm("{ .reg .b16 l, h; mov.b32 {l, h}, %1; cvt.f32.f16 %0, h; }" : "=f"(f) : "r"(w));
  return f;
}
AE_DEVICE float ae_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
AE_DEVICE float ae_log2(float x) {
  float y;
  asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
AE_DEVICE float ae_tanh(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
AE_DEVICE float ae_rcp(float x) {
  float y;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// Two fp32 operations per instruction (packed f32x2, sm_100): the row passes are bound by instruction issue, and these
// halve the count of their multiply-add and add instructions.
AE_DEVICE void ae_fma2(float& d0, float& d1, float x0, float x1, u64 a2, u64 b2) {
  u64 x, d;
  asm("mov.b64 %0, {%1, %2};" : "=l"(x) : "f"(x0), "f"(x1));
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(x), "l"(a2), "l"(b2));
  asm("mov.b64 {%0, %1}, %2;" : "=f"(d0), "=f"(d1) : "l"(d));
}
AE_DEVICE u64 ae_pack2f(float lo, float hi) {
  u64 r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
AE_DEVICE void ae_unpack2f(u64 v, float& lo, float& hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
AE_DEVICE u64 ae_add2(u64 acc, float x0, float x1) {
  u64 x, d;
  asm("mov.b64 %0, {%1, %2};" : "=l"(x) : "f"(x0), "f"(x1));
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(acc), "l"(x));
  return d;
}
#define AE_LOG2E 1.4426950408889634f
#define AE_LN2 0.6931471805599453f
AE_DEVICE float ae_exp(float x) { return ae_exp2(x * AE_LOG2E); }
// 2^x on the FMA / ALU pipes instead of the XU (ex2) pipe: round-to-nearest range reduction with the
// 1.5 * 2^23 trick, degree-3 polynomial for 2^f on [-0.5, 0.5] (max relative error 7.7e-5, below half an
// ulp of fp16), exponent added in integer arithmetic.  Valid for x in [-126, 126]; smaller x is clamped.
AE_DEVICE float ae_exp2_poly(float x) {
  x = fmaxf(x, -126.0f);
  const float xi = x + 12582912.0f;
  const float f = x - (xi - 12582912.0f);
  float p = fmaf(0.05508868396282196f, f, 0.24260404706001282f);
  p = fmaf(p, f, 0.6932762265205383f);
  p = fmaf(p, f, 0.9999289512634277f);
  return __uint_as_float(__float_as_uint(p) + (__float_as_uint(xi) << 23));
}
// Every AE_EXP_POLY_PERIOD-th element (by its compile-time index) takes the polynomial, the rest ex2.approx:
// spreads the exponentials of a tile over two pipes.  0 = always ex2.approx.
#ifndef AE_EXP_POLY_PERIOD
#define AE_EXP_POLY_PERIOD 0
#endif
AE_DEVICE float ae_exp2_mix(float x, int idx) {
#if AE_EXP_POLY_PERIOD > 0
  if ((idx % AE_EXP_POLY_PERIOD) == AE_EXP_POLY_PERIOD - 1) return ae_exp2_poly(x);
#endif
  return ae_exp2(x);
}
AE_DEVICE float ae_log(float x) { return ae_log2(x) * AE_LN2; }
// Running maximum that is only replaced when it would grow by more than AE_LAZY_TAU: with the softmax family of
// recurrences every result is unchanged (the states enter through differences that cancel), the rescale factor of the
// output accumulator is exactly 1 on most tiles, and P stays below e^AE_LAZY_TAU.  Used only where the lowering has
// verified that invariance numerically on the traced recurrence.
#ifndef AE_LAZY_TAU
#define AE_LAZY_TAU 5.0f
#endif
AE_DEVICE float ae_lazy_max(float old_v, float x) { return (x - old_v > AE_LAZY_TAU) ? x : old_v; }

// 4 x (32 lanes x 32 columns) TMEM load followed by tcgen05.wait::ld in ONE asm statement, so the
// compiler cannot schedule a use of the destination registers before the wait.
AE_DEVICE void tmem_ld_f32x128(u32 taddr, float (&r)[128]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%128];\n\t"
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%32, %33, %34, %35, %36, %37, %38, %39, %40, %41, %42, %43, %44, %45, %46, %47, %48, %49, %50, %51, %52, %53, %54, %55, %56, %57, %58, %59, %60, %61, %62, %63}, [%129];\n\t"
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%64, %65, %66, %67, %68, %69, %70, %71, %72, %73, %74, %75, %76, %77, %78, %79, %80, %81, %82, %83, %84, %85, %86, %87, %88, %89, %90, %91, %92, %93, %94, %95}, [%130];\n\t"
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%96, %97, %98, %99, %100, %101, %102, %103, %104, %105, %106, %107, %108, %109, %110, %111, %112, %113, %114, %115, %116, %117, %118, %119, %120, %121, %122, %123, %124, %125, %126, %127}, [%131];\n\t"
      "tcgen05.wait::ld.sync.aligned;"
      : "=f"(r[0]), "=f"(r[1]), "=f"(r[2]), "=f"(r[3]), "=f"(r[4]), "=f"(r[5]), "=f"(r[6]), "=f"(r[7]), "=f"(r[8]), "=f"(r[9]), "=f"(r[10]), "=f"(r[11]), "=f"(r[12]), "=f"(r[13]), "=f"(r[14]), "=f"(r[15]), "=f"(r[16]), "=f"(r[17]), "=f"(r[18]), "=f"(r[19]), "=f"(r[20]), "=f"(r[21]), "=f"(r[22]), "=f"(r[23]), "=f"(r[24]), "=f"(r[25]), "=f"(r[26]), "=f"(r[27]), "=f"(r[28]), "=f"(r[29]), "=f"(r[30]), "=f"(r[31]), "=f"(r[32]), "=f"(r[33]), "=f"(r[34]), "=f"(r[35]), "=f"(r[36]), "=f"(r[37]), "=f"(r[38]), "=f"(r[39]), "=f"(r[40]), "=f"(r[41]), "=f"(r[42]), "=f"(r[43]), "=f"(r[44]), "=f"(r[45]), "=f"(r[46]), "=f"(r[47]), "=f"(r[48]), "=f"(r[49]), "=f"(r[50]), "=f"(r[51]), "=f"(r[52]), "=f"(r[53]), "=f"(r[54]), "=f"(r[55]), "=f"(r[56]), "=f"(r[57]), "=f"(r[58]), "=f"(r[59]), "=f"(r[60]), "=f"(r[61]), "=f"(r[62]), "=f"(r[63]), "=f"(r[64]), "=f"(r[65]), "=f"(r[66]), "=f"(r[67]), "=f"(r[68]), "=f"(r[69]), "=f"(r[70]), "=f"(r[71]), "=f"(r[72]), "=f"(r[73]), "=f"(r[74]), "=f"(r[75]), "=f"(r[76]), "=f"(r[77]), "=f"(r[78]), "=f"(r[79]), "=f"(r[80]), "=f"(r[81]), "=f"(r[82]), "=f"(r[83]), "=f"(r[84]), "=f"(r[85]), "=f"(r[86]), "=f"(r[87]), "=f"(r[88]), "=f"(r[89]), "=f"(r[90]), "=f"(r[91]), "=f"(r[92]), "=f"(r[93]), "=f"(r[94]), "=f"(r[95]), "=f"(r[96]), "=f"(r[97]), "=f"(r[98]), "=f"(r[99]), "=f"(r[100]), "=f"(r[101]), "=f"(r[102]), "=f"(r[103]), "=f"(r[104]), "=f"(r[105]), "=f"(r[106]), "=f"(r[107]), "=f"(r[108]), "=f"(r[109]), "=f"(r[110]), "=f"(r[111]), "=f"(r[112]), "=f"(r[113]), "=f"(r[114]), "=f"(r[115]), "=f"(r[116]), "=f"(r[117]), "=f"(r[118]), "=f"(r[119]), "=f"(r[120]), "=f"(r[121]), "=f"(r[122]), "=f"(r[123]), "=f"(r[124]), "=f"(r[125]), "=f"(r[126]), "=f"(r[127])
      : "r"(taddr + 0u), "r"(taddr + 32u), "r"(taddr + 64u), "r"(taddr + 96u)
      : "memory");
}
// 2 x (32 lanes x 32 columns) TMEM load followed by tcgen05.wait::ld in ONE asm statement, so the
// compiler cannot schedule a use of the destination registers before the wait.
AE_DEVICE void tmem_ld_f32x64(u32 taddr, float (&r)[64]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%64];\n\t"
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%32, %33, %34, %35, %36, %37, %38, %39, %40, %41, %42, %43, %44, %45, %46, %47, %48, %49, %50, %51, %52, %53, %54, %55, %56, %57, %58, %59, %60, %61, %62, %63}, [%65];\n\t"
      "tcgen05.wait::ld.sync.aligned;"
      : "=f"(r[0]), "=f"(r[1]), "=f"(r[2]), "=f"(r[3]), "=f"(r[4]), "=f"(r[5]), "=f"(r[6]), "=f"(r[7]), "=f"(r[8]), "=f"(r[9]), "=f"(r[10]), "=f"(r[11]), "=f"(r[12]), "=f"(r[13]), "=f"(r[14]), "=f"(r[15]), "=f"(r[16]), "=f"(r[17]), "=f"(r[18]), "=f"(r[19]), "=f"(r[20]), "=f"(r[21]), "=f"(r[22]), "=f"(r[23]), "=f"(r[24]), "=f"(r[25]), "=f"(r[26]), "=f"(r[27]), "=f"(r[28]), "=f"(r[29]), "=f"(r[30]), "=f"(r[31]), "=f"(r[32]), "=f"(r[33]), "=f"(r[34]), "=f"(r[35]), "=f"(r[36]), "=f"(r[37]), "=f"(r[38]), "=f"(r[39]), "=f"(r[40]), "=f"(r[41]), "=f"(r[42]), "=f"(r[43]), "=f"(r[44]), "=f"(r[45]), "=f"(r[46]), "=f"(r[47]), "=f"(r[48]), "=f"(r[49]), "=f"(r[50]), "=f"(r[51]), "=f"(r[52]), "=f"(r[53]), "=f"(r[54]), "=f"(r[55]), "=f"(r[56]), "=f"(r[57]), "=f"(r[58]), "=f"(r[59]), "=f"(r[60]), "=f"(r[61]), "=f"(r[62]), "=f"(r[63])
      : "r"(taddr + 0u), "r"(taddr + 32u)
      : "memory");
}
// 1 x (32 lanes x 32 columns) TMEM load followed by tcgen05.wait::ld in ONE asm statement, so the
// compiler cannot schedule a use of the destination registers before the wait.
AE_DEVICE void tmem_ld_f32x32(u32 taddr, float (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n\t"
      "tcgen05.wait::ld.sync.aligned;"
      : "=f"(r[0]), "=f"(r[1]), "=f"(r[2]), "=f"(r[3]), "=f"(r[4]), "=f"(r[5]), "=f"(r[6]), "=f"(r[7]), "=f"(r[8]), "=f"(r[9]), "=f"(r[10]), "=f"(r[11]), "=f"(r[12]), "=f"(r[13]), "=f"(r[14]), "=f"(r[15]), "=f"(r[16]), "=f"(r[17]), "=f"(r[18]), "=f"(r[19]), "=f"(r[20]), "=f"(r[21]), "=f"(r[22]), "=f"(r[23]), "=f"(r[24]), "=f"(r[25]), "=f"(r[26]), "=f"(r[27]), "=f"(r[28]), "=f"(r[29]), "=f"(r[30]), "=f"(r[31])
      : "r"(taddr + 0u)
      : "memory");
}

// Dynamic shared memory rounded up to the 1024-byte alignment the 128-byte swizzle needs.
AE_DEVICE u8* smem_align1024(u8* raw) { return raw + ((1024u - (smem_u32(raw) & 1023u)) & 1023u); }

// Two independent 32-column loads (e.g. S and dP chunks) with a single wait.
AE_DEVICE void tmem_ld_2xf32x32(u32 taddr_a, u32 taddr_b, float (&a)[32], float (&b)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%64];\n\t"
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%32, %33, %34, %35, %36, %37, %38, %39, %40, %41, %42, %43, %44, %45, %46, %47, %48, %49, %50, %51, %52, %53, %54, %55, %56, %57, %58, %59, %60, %61, %62, %63}, [%65];\n\t"
      "tcgen05.wait::ld.sync.aligned;"
      : "=f"(a[0]), "=f"(a[1]), "=f"(a[2]), "=f"(a[3]), "=f"(a[4]), "=f"(a[5]), "=f"(a[6]), "=f"(a[7]), "=f"(a[8]), "=f"(a[9]), "=f"(a[10]), "=f"(a[11]), "=f"(a[12]), "=f"(a[13]), "=f"(a[14]), "=f"(a[15]), "=f"(a[16]), "=f"(a[17]), "=f"(a[18]), "=f"(a[19]), "=f"(a[20]), "=f"(a[21]), "=f"(a[22]), "=f"(a[23]), "=f"(a[24]), "=f"(a[25]), "=f"(a[26]), "=f"(a[27]), "=f"(a[28]), "=f"(a[29]), "=f"(a[30]), "=f"(a[31]), "=f"(b[0]), "=f"(b[1]), "=f"(b[2]), "=f"(b[3]), "=f"(b[4]), "=f"(b[5]), "=f"(b[6]), "=f"(b[7]), "=f"(b[8]), "=f"(b[9]), "=f"(b[10]), "=f"(b[11]), "=f"(b[12]), "=f"(b[13]), "=f"(b[14]), "=f"(b[15]), "=f"(b[16]), "=f"(b[17]), "=f"(b[18]), "=f"(b[19]), "=f"(b[20]), "=f"(b[21]), "=f"(b[22]), "=f"(b[23]), "=f"(b[24]), "=f"(b[25]), "=f"(b[26]), "=f"(b[27]), "=f"(b[28]), "=f"(b[29]), "=f"(b[30]), "=f"(b[31])
      : "r"(taddr_a), "r"(taddr_b)
      : "memory");
}

// UMMA operand descriptors over tiles stored as 64-element-wide column blocks of [rows][128 B] with the
// 128-byte swizzle (what a TMA box {64, rows} produces, and what the row threads write with swz128()).
//   K-major : the contraction dim is the contiguous one; k-step kk covers 16 elements.
//   MN-major: the contraction dim is the row index; k-step kk covers 16 rows.
// The MMA-issuing thread is a single thread, so every instruction between two tcgen05.mma is on the critical
// path: a tile's descriptor is built once (umma_base_*), each k-step only adds a compile-time constant to it
// (the address field holds bytes / 16 and never carries out of its 14 bits inside one CTA's shared memory).
AE_DEVICE u64 umma_base_k(u32 addr) { return umma_smem_desc_sw128(addr, 16, 1024); }
AE_DEVICE u64 umma_base_mn(u32 addr, int rows) { return umma_smem_desc_sw128(addr, rows * 128, 1024); }
AE_DEVICE u64 umma_step_k(u64 d0, int kk, int rows) {
  return d0 + (u64)(((kk >> 2) * (rows * 128) + (kk & 3) * 32) >> 4);
}
AE_DEVICE u64 umma_step_mn(u64 d0, int kk) { return d0 + (u64)(kk * 128); }
// byte offset of the 16-byte chunk `ch` of row `r` inside a [rows][128 B] swizzled block
AE_DEVICE u32 swz128(u32 r, u32 ch) { return r * 128 + ((ch ^ (r & 7)) << 4); }
// byte offset of element column `col` (multiple of 8) of row `r` in a tile of 64-wide blocks of `rows` rows
AE_DEVICE u32 tile_off(u32 r, u32 col, u32 rows) { return (col >> 6) * (rows * 128) + swz128(r, (col & 63) >> 3); }
