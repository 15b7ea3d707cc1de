// Micro-benchmark of the K / V streaming of the attention kernels without any compute (tuning aid): same grid,
// same tensor maps and same tile walk as ae_attn_fwd (launched through ae_launch_attn_fwd), but each CTA only
// loads its kv-head's K and V tiles (64 KB per step at head dim 128) into a ring of AE_TS_SLOTS slots with
// AE_TS_DEPTH steps in flight and reports bytes per clock in final_rs[0][linear CTA index].
// AE_TS_MMA = 1 / 2 adds a second warp that issues TS / SS MMAs (M = 128, N = 128, operands in a shared-memory
// region of its own, results discarded) for as long as the loads run: does tensor-core operand traffic slow the fill?
// AE_TS_LD = 1 adds a third warp that times tcgen05.ld (32 lanes x 32 columns, with its wait) in a loop while the
// other two run: what a row thread's TMEM read costs under tensor-pipe load (reported in final_rs[1]).
// Expects AE_D, AE_DV, AE_TS_DEPTH, AE_TS_ROTATE, AE_TS_MMA, AE_TS_LD.

#define AE_TS_SLOTS 3
#define AE_TS_K_BYTES (128 * AE_D * 2)
#define AE_TS_V_BYTES (128 * AE_DV * 2)
#define AE_TS_STEP (AE_TS_K_BYTES + AE_TS_V_BYTES)

struct AeTsBars {
  u64 full[AE_TS_SLOTS];
  u64 mma_done;
  volatile u32 stop;
  AeCtaCtl ctl;
};
#define AE_TS_OPER (AE_TS_SLOTS * AE_TS_STEP)  // 32 KB of MMA operands behind the ring

extern "C" __global__ void __launch_bounds__(96, 1) ae_attn_fwd(const __grid_constant__ AeAttnFwdArgs args) {
  extern __shared__ u8 smem_raw[];
  u8* smem = smem_align1024(smem_raw);
  AeTsBars* bars = (AeTsBars*)(smem + AE_TS_OPER + 32768);
  AeCtaCtl* ctl = &bars->ctl;
  const u32 warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) {
    ctl->abort = 0;
    bars->stop = 0;
    for (int i = 0; i < AE_TS_SLOTS; ++i) mbar_init(&bars->full[i], 1);
    mbar_init(&bars->mma_done, 1);
    mbar_fence_init();
  }
#if AE_TS_MMA
  if (warp == 1) {
    tmem_alloc(&ctl->tmem_base, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
#endif
  __syncthreads();
#if AE_TS_MMA
  tc_fence_after_sync();
  if (warp == 1) {
    const u32 tmem = ctl->tmem_base;
    const u32 idesc = umma_idesc_f16(128, 128, 0, 0, 0);
    const u64 da = umma_base_k(smem_u32(smem + AE_TS_OPER)), db = umma_base_k(smem_u32(smem + AE_TS_OPER + 16384));
    // batches of 8 MMAs until the loading thread says stop (bounded: at most 1 << 16 batches)
    u32 phase = 0;
    for (int it = 0; it < (1 << 16) && !bars->stop; ++it) {
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {
#if AE_TS_MMA == 1
        umma_ts_w(tmem + 256, tmem + kk * 8, umma_step_k(db, kk, 128), idesc, 1);
        umma_ts_w(tmem + 384, tmem + kk * 8, umma_step_k(db, kk, 128), idesc, 1);
#else
        umma_ss_w(tmem + 256, umma_step_k(da, kk, 128), umma_step_k(db, kk, 128), idesc, 1);
        umma_ss_w(tmem + 384, umma_step_k(da, kk, 128), umma_step_k(db, kk, 128), idesc, 1);
#endif
      }
      umma_commit_w(&bars->mma_done);
      if (!mbar_wait_w(&bars->mma_done, phase, ctl, args.status, 83)) break;
      phase ^= 1;
    }
    tc_fence_before_sync();
#if AE_TS_LD
    named_bar_sync(5, 64);  // the reading warp has issued its last TMEM load
    tc_fence_after_sync();
#endif
    __syncwarp();
    tmem_dealloc(tmem, 512);
    return;
  }
#endif
#if AE_TS_MMA && AE_TS_LD
  if (warp == 2) {
    const u32 tmem = ctl->tmem_base;
    const u32 lane_base = (2u * 32u) << 16;  // warp 2 reads TMEM lanes 64..95
    float acc = 0.f;
    i64 total = 0;
    int n = 0;
    for (int it = 0; it < 4096 && !bars->stop; ++it) {
      float r[32];
      const i64 t0 = clock64();
      tmem_ld_f32x32(tmem + lane_base + (it & 3) * 32, r);
      const i64 t1 = clock64();
      acc += r[it & 31];
      total += t1 - t0;
      ++n;
    }
    if ((threadIdx.x & 31) == 0) {
      const i64 cta = ((i64)blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x;
      args.final_rs[1][cta] = n ? (float)total / n + 0.f * acc : 0.f;
    }
    tc_fence_before_sync();
    named_bar_sync(5, 64);  // lets the allocating warp free TMEM
    return;
  }
#endif
  if (threadIdx.x != 0) return;
  const int hq = blockIdx.y, b = blockIdx.z;
  const int hk = hq / (args.Hq / args.Hkv);
  const int n = args.n_kt;
  // same starting tile for every CTA (rot = 0) or a CTA-dependent one
#if AE_TS_ROTATE
  const int rot = (int)(((u32)blockIdx.x * 2654435761u + (u32)hq * 40503u + (u32)b * 9973u) >> 8) % n;
#else
  const int rot = 0;
#endif
  auto issue = [&](int step, int slot) {
    int kt = step + rot;
    if (kt >= n) kt -= n;
    u8* dst = smem + slot * AE_TS_STEP;
    mbar_arrive_expect_tx(&bars->full[slot], AE_TS_STEP);
    for (int dh = 0; dh < AE_D / 64; ++dh)
      tma_load_bshd(dst + dh * (128 * 128), &args.tm_k, &bars->full[slot], dh * 64, hk, kt * 128, b);
    for (int dh = 0; dh < AE_DV / 64; ++dh)
      tma_load_bshd(dst + AE_TS_K_BYTES + dh * (128 * 128), &args.tm_v, &bars->full[slot], dh * 64, hk, kt * 128, b);
  };
  bool ok = true;
  const i64 t0 = clock64();
  int issued = 0, done = 0;
  u32 use0 = 0, use1 = 0, use2 = 0;
  while (done < n && ok) {
    while (issued < n && issued - done < AE_TS_DEPTH) {
      issue(issued, issued % AE_TS_DEPTH);
      ++issued;
    }
    const int slot = done % AE_TS_DEPTH;
    u32& use = slot == 0 ? use0 : (slot == 1 ? use1 : use2);
    ok = mbar_wait(&bars->full[slot], use & 1, ctl, args.status, 82);
    ++use;
    ++done;
  }
  const i64 t1 = clock64();
  bars->stop = 1;
  const i64 cta = ((i64)b * gridDim.y + hq) * gridDim.x + blockIdx.x;
  args.final_rs[0][cta] = (float)((double)n * AE_TS_STEP / (double)(t1 - t0));
}
