// Micro-benchmark of the TMA fill rate of one SM (tuning aid): one CTA, one thread.  The same [128 x 128] 16-bit
// tile (32 KB, two 128-byte-swizzled boxes of {64, 128}, L2-resident after the first pass) is loaded `reps` times
// into a ring of shared-memory slots with `depth` loads kept in flight; out[depth - 1] = bytes per clock.
// With several CTAs (one per SM) every CTA streams the same tile and CTA 0 reports.
// Launched through ae_launch_probe with mode = reps (the launcher builds the B map for every mode, so the tile is read through it).  Expects nothing from the prelude.

#define AE_TR_SLOTS 6
#define AE_TR_TILE 32768

struct AeTmaRateBars {
  u64 full[AE_TR_SLOTS];
  AeCtaCtl ctl;
};

extern "C" __global__ void __launch_bounds__(32, 1) ae_tma_rate(const __grid_constant__ AeProbeArgs args) {
  extern __shared__ u8 smem_raw[];
  u8* smem = smem_align1024(smem_raw);
  AeTmaRateBars* bars = (AeTmaRateBars*)(smem + AE_TR_SLOTS * AE_TR_TILE);
  AeCtaCtl* ctl = &bars->ctl;
  if (threadIdx.x == 0) {
    ctl->abort = 0;
    for (int i = 0; i < AE_TR_SLOTS; ++i) mbar_init(&bars->full[i], 1);
    mbar_fence_init();
    tma_prefetch_desc(&args.tm_b);
    const int reps = args.mode;
    u32 n_use[AE_TR_SLOTS];
    for (int i = 0; i < AE_TR_SLOTS; ++i) n_use[i] = 0;
    auto issue = [&](int slot) {
      mbar_arrive_expect_tx(&bars->full[slot], AE_TR_TILE);
      tma_load_2d(smem + slot * AE_TR_TILE, &args.tm_b, &bars->full[slot], 0, 0);
      tma_load_2d(smem + slot * AE_TR_TILE + 16384, &args.tm_b, &bars->full[slot], 64, 0);
    };
    bool ok = true;
    for (int depth = 1; depth <= AE_TR_SLOTS && ok; ++depth) {
      // warm pass (brings the tile into L2), then the timed passes
      issue(0);
      ok = mbar_wait(&bars->full[0], n_use[0]++ & 1, ctl, args.status, 80);
      const i64 t0 = clock64();
      int issued = 0, done = 0;
      while (done < reps && ok) {
        while (issued < reps && issued - done < depth) {
          issue(issued % depth);
          ++issued;
        }
        const int slot = done % depth;
        ok = mbar_wait(&bars->full[slot], n_use[slot]++ & 1, ctl, args.status, 81);
        ++done;
      }
      const i64 t1 = clock64();
      if (blockIdx.x == 0) {
        args.d[depth - 1] = (float)((double)reps * AE_TR_TILE / (double)(t1 - t0));
        args.d[8 + depth - 1] = (float)(t1 - t0) / reps;  // clocks per 32 KB tile
      }
    }
  }
}
