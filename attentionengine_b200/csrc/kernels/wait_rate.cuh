// Micro-benchmark of what one wait on an mbarrier whose phase has ALREADY completed costs a warp (tuning aid).
// One CTA, one warp, `reps` waits per form; out[form] = clocks per wait.
//   form 0: lane 0 alone runs mbar_wait                                (the single-lane issuer of attn_fwd.cuh)
//   form 1: all 32 lanes run mbar_wait, then a vote                     (mbar_wait_w)
//   form 2: lane 0 runs mbar_wait inside a branch, then a vote
//   form 3: all lanes mbar_try_wait once (no loop), then a vote
//   form 4: form 1 followed by tcgen05.fence::after_thread_sync
//   form 5: a dependent volatile shared-memory load (baseline latency of shared memory)
//   form 6: bar.sync on a named barrier of this warp alone
//   form 7: lane 0 mbarrier.arrive on a second barrier (count 1: every arrive completes a phase)
//   form 8: lane 0 mbarrier.test_wait issued back to back, results summed without branching (throughput, not latency)
// Launched through ae_launch_probe with mode = reps.

struct AeWaitBars {
  u64 bar;
  u64 bar2;
  volatile u32 word[32];
  AeCtaCtl ctl;
};

extern "C" __global__ void __launch_bounds__(32, 1) ae_wait_rate(const __grid_constant__ AeProbeArgs args) {
  extern __shared__ u8 smem_raw[];
  u8* smem = smem_align1024(smem_raw);
  AeWaitBars* bars = (AeWaitBars*)smem;
  AeCtaCtl* ctl = &bars->ctl;
  const u32 lane = threadIdx.x & 31;
  if (lane == 0) {
    ctl->abort = 0;
    mbar_init(&bars->bar, 1);
    mbar_init(&bars->bar2, 1);
    for (int i = 0; i < 32; ++i) bars->word[i] = 0;
    mbar_fence_init();
    mbar_arrive(&bars->bar);  // phase 0 completes here and stays complete
  }
  __syncwarp();
  const int reps = args.mode;
  u32 acc = 0;
  auto run = [&](auto F) {
    constexpr int form = decltype(F)::value;  // compile-time, so that the loop holds nothing but the measured form
    __syncwarp();
    const i64 t0 = clock64();
#pragma unroll 4
    for (int r = 0; r < reps; ++r) {
      bool ok;
      if (form == 0) {
        ok = true;
        if (lane == 0) ok = mbar_wait(&bars->bar, 0, ctl, args.status, 84);
      } else if (form == 1) {
        ok = mbar_wait_w(&bars->bar, 0, ctl, args.status, 84);
      } else if (form == 2) {
        bool x = false;
        if (lane == 0) x = mbar_wait(&bars->bar, 0, ctl, args.status, 84);
        ok = __any_sync(0xffffffffu, x);
      } else if (form == 3) {
        ok = __all_sync(0xffffffffu, mbar_try_wait(&bars->bar, 0));
      } else if (form == 4) {
        ok = mbar_wait_w(&bars->bar, 0, ctl, args.status, 84);
        tc_fence_after_sync();
      } else if (form == 5) {
        ok = bars->word[acc & 31] == 0;  // the address depends on the previous result
      } else if (form == 6) {
        named_bar_sync(3, 32);
        ok = true;
      } else if (form == 7) {
        if (lane == 0) mbar_arrive(&bars->bar2);
        ok = true;
      } else {
        ok = true;
        if (lane == 0) {
          u32 a0;
          asm volatile("{ .reg .pred p; mbarrier.test_wait.parity.shared::cta.b64 p, [%1], 0; selp.u32 %0, 1, 0, p; }"
                       : "=r"(a0) : "r"(smem_u32(&bars->bar)));
          acc += a0;
        }
      }
      acc += ok;
    }
    const i64 t1 = clock64();
    if (lane == 0) args.d[form] = (float)(t1 - t0) / reps;
  };
  run(AeInt<0>{});
  run(AeInt<1>{});
  run(AeInt<2>{});
  run(AeInt<3>{});
  run(AeInt<4>{});
  run(AeInt<5>{});
  run(AeInt<6>{});
  run(AeInt<7>{});
  run(AeInt<8>{});
  if (lane == 0) args.d[15] = (float)acc;
}
