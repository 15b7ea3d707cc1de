// Bring-up probe for the tcgen05 building blocks the attention kernels rely on:
//   mode 0: D = A * B^T  with A, B [128, 128] 16-bit, both K-major in shared memory
//           (TMA 128-byte swizzle -> UMMA SS descriptors, k advance inside the swizzle atom)
//   mode 1: D = P * B    with P [128, 128] 16-bit staged through TMEM as the A operand
//           (tcgen05.st packing) and B [k = 128, n = 128] MN-major in shared memory
//           (the layout of a V tile).
// Expects AE_BF16 to be defined.  160 threads: warps 0-3 own TMEM lanes, warp 4 loads and issues.

struct AeProbeBars {
  u64 full;
  u64 done;
  AeCtaCtl ctl;
};

extern "C" __global__ void __launch_bounds__(160, 1) ae_probe(const __grid_constant__ AeProbeArgs args) {
  extern __shared__ u8 smem_raw[];
  u8* smem = smem_align1024(smem_raw);
  u8* sA = smem;            // 2 x [128 rows x 128 B]
  u8* sB = smem + 32768;    // 2 x [128 rows x 128 B]
  AeProbeBars* bars = (AeProbeBars*)(smem + 65536);
  AeCtaCtl* ctl = &bars->ctl;
  const u32 warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    ctl->abort = 0;
    mbar_init(&bars->full, 1);
    mbar_init(&bars->done, 1);
    mbar_fence_init();
  }
  if (warp == 4) {
    tmem_alloc(&ctl->tmem_base, 256);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const u32 tmem = ctl->tmem_base;
  const u32 TM_D = 0, TM_A = 128;

  if (warp < 4 && args.mode == 1) {
    // stage P through TMEM: thread = row, 64 words of two 16-bit values
    const u32* prow = (const u32*)args.p + (threadIdx.x & 127) * 64;
    const u32 taddr = tmem + TM_A + (((warp & 3) * 32) << 16);
    u32 w[32];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
#pragma unroll
      for (int i = 0; i < 32; ++i) w[i] = prow[h * 32 + i];
      tmem_st32(taddr + h * 32, w);
    }
    tc_wait_st();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();

  if (warp == 4 && lane == 0) {
    const u32 bytes = (args.mode == 0) ? 65536u : 32768u;
    mbar_arrive_expect_tx(&bars->full, bytes);
    if (args.mode == 0) {
      tma_load_2d(sA, &args.tm_a, &bars->full, 0, 0);
      tma_load_2d(sA + 16384, &args.tm_a, &bars->full, 64, 0);
    }
    tma_load_2d(sB, &args.tm_b, &bars->full, 0, 0);
    tma_load_2d(sB + 16384, &args.tm_b, &bars->full, 64, 0);
    if (mbar_wait(&bars->full, 0, ctl, args.status, 1)) {
      tc_fence_after_sync();
      if (args.mode == 0) {
        const u32 idesc = umma_idesc_f16(128, 128, AE_BF16, 0, 0);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const u32 off = (kk >> 2) * 16384 + (kk & 3) * 32;
          umma_ss(tmem + TM_D, umma_smem_desc_sw128(smem_u32(sA) + off, 16, 1024),
                  umma_smem_desc_sw128(smem_u32(sB) + off, 16, 1024), idesc, kk > 0);
        }
      } else {
        const u32 idesc = umma_idesc_f16(128, 128, AE_BF16, 0, 1);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          umma_ts(tmem + TM_D, tmem + TM_A + kk * 8, umma_smem_desc_sw128(smem_u32(sB) + kk * 2048, 16384, 1024),
                  idesc, kk > 0);
        }
      }
      umma_commit(&bars->done);
    }
  }
  if (warp < 4) {
    if (mbar_wait(&bars->done, 0, ctl, args.status, 2)) {
      tc_fence_after_sync();
      float r[128];
      tmem_ld_f32x128(tmem + TM_D + (((warp & 3) * 32) << 16), r);
      float* drow = args.d + (threadIdx.x & 127) * 128;
#pragma unroll
      for (int i = 0; i < 128; ++i) drow[i] = r[i];
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 4) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, 256);
  }
}
