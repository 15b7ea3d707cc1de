// Chunk start-states of the linear-attention / SSD recurrence, recomputed for the backward pass
// (reference: `chunk_fwd_h` called again from LinearAttention.backward,
// attention_engine/core/template/tl_template/linear/linear_tl.py:1187, kernel :114-233).
// Same walk as linear_fwd.cuh without the output path: per chunk the incoming state H [DK x DV] is
// written to HBM in 16-bit, decayed by exp(g_last) and updated with k^T (v * exp(g_last - g)).
// Roles: warps 0-3 row threads (thread r = step r = state row r), warp 4 TMA producer, warp 5 MMA issuer.
// The kernel is a chain of short dependent steps per chunk, so two CTAs share an SM: 98 KB of shared memory (the
// rescaled values overwrite the V tile they came from) and 128 TMEM columns each.
// Expects AE_BF16, AE_LIN_DV, AE_LIN_STAGES.

#define AE_LS_C 128
#define AE_LS_DK 128
#define AE_LS_K_BYTES (AE_LS_C * AE_LS_DK * 2)
#define AE_LS_V_BYTES (AE_LS_C * AE_LIN_DV * 2)
#define AE_LS_STAGE_BYTES (AE_LS_K_BYTES + AE_LS_V_BYTES)
#define AE_LS_SMEM_G (AE_LIN_STAGES * AE_LS_STAGE_BYTES)
#define AE_LS_SMEM_BAR (AE_LS_SMEM_G + 1024)

struct AeLsBars {
  u64 full[AE_LIN_STAGES];
  u64 empty[AE_LIN_STAGES];
  u64 prep_done;
  u64 h_done;
  AeCtaCtl ctl;
};

extern "C" __global__ void __launch_bounds__(192, 2) ae_linear_states(const __grid_constant__ AeLinearBwdArgs args) {
  extern __shared__ u8 smem_raw[];
  u8* smem = smem_align1024(smem_raw);
  AeLsBars* bars = (AeLsBars*)(smem + AE_LS_SMEM_BAR);
  float* gs = (float*)(smem + AE_LS_SMEM_G);
  AeCtaCtl* ctl = &bars->ctl;
  const u32 warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.x, b = blockIdx.y;
  const int hk = h / (args.H / args.HK);
  const int n_chunks = (args.T + AE_LS_C - 1) / AE_LS_C;

  if (threadIdx.x == 0) {
    ctl->abort = 0;
    for (int i = 0; i < AE_LIN_STAGES; ++i) {
      mbar_init(&bars->full[i], 1);
      mbar_init(&bars->empty[i], 1);
    }
    mbar_init(&bars->prep_done, 4);
    mbar_init(&bars->h_done, 1);
    mbar_fence_init();
  }
  if (warp == 5) {
    tmem_alloc(&ctl->tmem_base, 128);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const u32 tmem = ctl->tmem_base;

  if (warp == 4) {
    if (lane == 0) {
      tma_prefetch_desc(&args.tm_k);
      tma_prefetch_desc(&args.tm_v);
      for (int c = 0; c < n_chunks; ++c) {
        const int stage = c % AE_LIN_STAGES;
        if (!mbar_wait(&bars->empty[stage], ((c / AE_LIN_STAGES) & 1) ^ 1, ctl, args.status, 61)) break;
        u8* st = smem + stage * AE_LS_STAGE_BYTES;
        mbar_arrive_expect_tx(&bars->full[stage], AE_LS_STAGE_BYTES);
        for (int dh = 0; dh < AE_LS_DK / 64; ++dh)
          tma_load_4d(st + dh * (AE_LS_C * 128), &args.tm_k, &bars->full[stage], dh * 64, c * AE_LS_C, hk, b);
        for (int dh = 0; dh < AE_LIN_DV / 64; ++dh)
          tma_load_4d(st + AE_LS_K_BYTES + dh * (AE_LS_C * 128), &args.tm_v, &bars->full[stage], dh * 64, c * AE_LS_C,
                      h, b);
      }
    }
  } else if (warp == 5) {
    if (lane == 0) {
      const u32 idesc_h = umma_idesc_f16(AE_LS_DK, AE_LIN_DV, AE_BF16, 1, 1);
      const u64 bk_mn = umma_base_mn(smem_u32(smem), AE_LS_C);
      const u64 bv_mn = umma_base_mn(smem_u32(smem + AE_LS_K_BYTES), AE_LS_C);  // the stage's V tile, rescaled in place
      bool ok = true;
      for (int c = 0; c < n_chunks && ok; ++c) {
        const int stage = c % AE_LIN_STAGES;
        const u64 so = (u64)((stage * AE_LS_STAGE_BYTES) >> 4);
        ok = mbar_wait(&bars->prep_done, c & 1, ctl, args.status, 62);
        if (!ok) break;
        tc_fence_after_sync();
#pragma unroll
        for (int kk = 0; kk < AE_LS_C / 16; ++kk)
          umma_ss(tmem, umma_step_mn(bk_mn + so, kk), umma_step_mn(bv_mn + so, kk), idesc_h, (c > 0) | (kk > 0));
        umma_commit(&bars->h_done);
        umma_commit(&bars->empty[stage]);
      }
    }
  } else {
    const u32 r = threadIdx.x & 127;
    const u32 lane_base = ((warp & 3) * 32) << 16;
    const float* a_row = args.a + ((i64)b * args.H + h) * args.T;
    u16* hs_base = (u16*)args.h_states + ((i64)b * args.H + h) * (i64)n_chunks * AE_LS_DK * AE_LIN_DV;
    bool ok = true;
    for (int c = 0; c < n_chunks; ++c) {
      const int stage = c % AE_LIN_STAGES;
      const int t = c * AE_LS_C + (int)r;
      float g = t < args.T ? a_row[t] * (args.ascale ? args.ascale[h] : 1.f) : 0.f;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const float n = __shfl_up_sync(0xffffffffu, g, o);
        if (lane >= (u32)o) g += n;
      }
      if (lane == 31) gs[128 + (warp & 3)] = g;
      named_bar_sync(1, 128);
      {
        float pre = 0.f;
#pragma unroll
        for (int w = 0; w < 3; ++w)
          if ((u32)w < (warp & 3)) pre += gs[128 + w];
        g += pre;
      }
      if (r == AE_LS_C - 1) gs[0] = g;
      named_bar_sync(1, 128);
      const float g_last = gs[0];
      // incoming state: out to HBM in 16-bit (row r of H), then decay it in place
      u16* hrow = hs_base + ((i64)c * AE_LS_DK + r) * AE_LIN_DV;
      if (c > 0) {
        ok = ok && mbar_wait(&bars->h_done, (c - 1) & 1, ctl, args.status, 63);
        tc_fence_after_sync();
        const float dec = ae_exp(g_last);
#pragma unroll
        for (int cc = 0; cc < AE_LIN_DV / 32; ++cc) {
          float f[32];
          u32 w[32];
          tmem_ld_f32x32(tmem + lane_base + cc * 32, f);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint4 pk;
            pk.x = pack2<AE_BF16>(f[i * 8 + 0], f[i * 8 + 1]);
            pk.y = pack2<AE_BF16>(f[i * 8 + 2], f[i * 8 + 3]);
            pk.z = pack2<AE_BF16>(f[i * 8 + 4], f[i * 8 + 5]);
            pk.w = pack2<AE_BF16>(f[i * 8 + 6], f[i * 8 + 7]);
            *(uint4*)(hrow + cc * 32 + i * 8) = pk;
          }
#pragma unroll
          for (int i = 0; i < 32; ++i) w[i] = __float_as_uint(f[i] * dec);
          tmem_st32(tmem + lane_base + cc * 32, w);
        }
      } else {
#pragma unroll
        for (int i = 0; i < AE_LIN_DV / 8; ++i) *(uint4*)(hrow + i * 8) = make_uint4(0, 0, 0, 0);
      }
      // v' = v * exp(g_last - g)
      ok = ok && mbar_wait(&bars->full[stage], (c / AE_LIN_STAGES) & 1, ctl, args.status, 64);
      {
        const float wgt = ae_exp(g_last - g);
        u8* vt = smem + stage * AE_LS_STAGE_BYTES + AE_LS_K_BYTES;  // row r of the tile is this thread's alone
#pragma unroll
        for (int ch = 0; ch < AE_LIN_DV / 8; ++ch) {
          const u32 off = tile_off(r, ch * 8, AE_LS_C);
          uint4 x = *(const uint4*)(vt + off);
          u32* xw = (u32*)&x;
#pragma unroll
          for (int i = 0; i < 4; ++i)
            xw[i] = pack2<AE_BF16>(unpack_lo<AE_BF16>(xw[i]) * wgt, unpack_hi<AE_BF16>(xw[i]) * wgt);
          *(uint4*)(vt + off) = x;
        }
      }
      tc_wait_st();
      fence_proxy_async_smem();
      tc_fence_before_sync();
      mbar_arrive_warp(&bars->prep_done);
      // the stage (K and the rescaled V) goes back to the producer with the commit that follows this chunk's MMAs
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 5) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, 128);
  }
}
