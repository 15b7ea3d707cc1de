// Micro-benchmark of raw tcgen05.mma issue / execution rate for the operand forms the kernels use (tuning aid;
// results are garbage numerically: operands are whatever shared memory / TMEM holds).  One CTA, one issuing
// thread; `reps` back-to-back MMAs of one form, then a commit and a wait; cycles go to out[form].
//   form 0: SS  M=128 N=128 K=16, A and B K-major          (S = Q K^T at BN=128)
//   form 1: SS  M=128 N=64  K=16, K-major                   (S at BN=64)
//   form 2: TS  M=128 N=128 K=16, B MN-major                (O += P V, dQ += dS K)
//   form 3: TS  M=128 N=256 K=16, B MN-major                (MLA O half)
//   form 4: SS  M=128 N=128 K=16, A and B MN-major          (linear backward)
//   form 5: SS  M=128 N=32  K=16, K-major
//   form 6: TS  M=128 N=64  K=16, B K-major                 (S = Q K^T with Q resident in TMEM, BN=64)
//   form 7: TS  M=128 N=32  K=16, B K-major
//   form 8: TS  M=128 N=128 K=16, B K-major
//   form 9: SS  M=64  N=128 K=16, K-major
// Expects AE_BF16.

struct AeRateBars {
  u64 done;
  AeCtaCtl ctl;
};

extern "C" __global__ void __launch_bounds__(64, 1) ae_mma_rate(const __grid_constant__ AeProbeArgs args) {
  extern __shared__ u8 smem_raw[];
  u8* smem = smem_align1024(smem_raw);
  AeRateBars* bars = (AeRateBars*)(smem + 131072);
  AeCtaCtl* ctl = &bars->ctl;
  const u32 warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // zero the operand area so that no NaN patterns slow anything down
  for (int i = threadIdx.x; i < 131072 / 16; i += 64) ((uint4*)smem)[i] = make_uint4(0, 0, 0, 0);
  if (threadIdx.x == 0) {
    ctl->abort = 0;
    mbar_init(&bars->done, 1);
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(&ctl->tmem_base, 512);
    tmem_relinquish();
  }
  fence_proxy_async_smem();
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const u32 tmem = ctl->tmem_base;
  if (warp == 0 && lane == 0) {
    const u32 A = smem_u32(smem), B = smem_u32(smem + 65536);
    const int reps = args.mode;
    u32 phase = 0;
    auto run = [&](auto F) {
      constexpr int form = decltype(F)::value;
      constexpr u32 n = (form == 1 || form == 6) ? 64 : (form == 3 ? 256 : ((form == 5 || form == 7) ? 32 : 128));
      constexpr u32 idesc = umma_idesc_f16(form == 9 ? 64 : 128, n, AE_BF16, form == 4, form >= 2 && form <= 4);
      const u64 da = form == 4 ? umma_base_mn(A, 128) : umma_base_k(A);
      const u64 db = (form >= 2 && form <= 4) ? umma_base_mn(B, 128) : umma_base_k(B);
      const i64 t0 = clock64();
      for (int r = 0; r < reps; ++r) {
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          if (form == 2 || form == 3)
            umma_ts(tmem + 256, tmem + kk * 8, umma_step_mn(db, kk), idesc, 1);
          else if (form >= 6 && form <= 8)
            umma_ts(tmem + 256, tmem + kk * 8, umma_step_k(db, kk, 128), idesc, 1);
          else if (form == 4)
            umma_ss(tmem + 256, umma_step_mn(da, kk), umma_step_mn(db, kk), idesc, 1);
          else
            umma_ss(tmem + 256, umma_step_k(da, kk, 128), umma_step_k(db, kk, 128), idesc, 1);
        }
      }
      const i64 t1 = clock64();
      umma_commit(&bars->done);
      mbar_wait(&bars->done, phase, ctl, args.status, 90 + form);
      phase ^= 1;
      const i64 t2 = clock64();
      args.d[form * 2 + 0] = (float)(t1 - t0) / (reps * 8);  // issue cycles per MMA
      args.d[form * 2 + 1] = (float)(t2 - t0) / (reps * 8);  // cycles per MMA until all completed
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
    run(AeInt<9>{});
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, 512);
  }
}
