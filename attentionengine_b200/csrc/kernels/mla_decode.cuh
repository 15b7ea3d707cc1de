// MLA (multi-head latent attention) split-KV decode for sm_100a.  Replaces the reference's
// `flash_attn` / `flash_attn_split` kernels (attention_engine/core/template/tl_template/attn/
// mla_decode_tl.py:38-177; CuTe variant cute_template_kvshared/kernels/splitkv_mla.cu:1061-1391).
//
// All H = 128 query heads of one batch row share one latent KV stream: rows of the MMA are heads.
//   S = [q | q_pe] [kv | k_pe]^T   over 512 + 64 dims (9 K blocks of 64)        TS / SS MMAs, M = 128, N = BN
//   row threads (thread = head): fused score_mod + online recurrence, P -> TMEM
//   O_half += P kv[:, half]          over this CTA's 256 of the 512 value dims     TS MMA, N = 256
// A [128 x 512] fp32 accumulator would fill all 512 TMEM columns, so the value dims are split
// over two CTAs (blockIdx.x) that each recompute S; both read the same KV tiles, the second read
// is an L2 hit.  blockIdx.y is the kv split, blockIdx.z the batch row.  With more than one split
// the CTA stores its normalised partial O (fp32) and its final row scales; ae_mla_combine merges.
// The first AE_MLA_QT (= 4) 64-wide blocks of the query block live in TMEM (16-bit pairs, the A-operand layout of a
// TS MMA), the other five in shared memory: that leaves room for two KV stages and two S regions, so the loads of
// tile s+1, its S GEMM and the row work of tile s overlap.  The TMEM-resident blocks first land in KV stage 0.
// TMEM columns: S0 | S1 | O half (256) | Q blocks 0-3 (128) = 512.
// Roles: warps 0-3 row threads, warp 4 TMA producer, warp 5 MMA issuer.
// Expects AE_BF16, AE_NFINAL, AE_O_SCALE_ONE, AE_MLA_BN (64), AE_MLA_ALIGN_SLACK, struct AeRow, ae_online_fwd(),
// ae_epilogue_o(), ae_final_rowscales().

// Optional phase trace of CTA (0, 0, 0): 32-bit clock stamps behind the status word (bring-up / tuning only).
#ifdef AE_TRACE
#define AE_TRM(cond, region, slot) \
  if (trace_on && (cond) && (slot) < 2048) args.status[64 + (region) * 4096 + (slot)] = (u32)clock64();
#else
#define AE_TRM(cond, region, slot)
#endif
#define AE_MLA_H 128
#define AE_MLA_DV 512
#define AE_MLA_DPE 64
#define AE_MLA_NBV (AE_MLA_DV / 64)
#define AE_MLA_NBK (AE_MLA_NBV + AE_MLA_DPE / 64)
#define AE_MLA_DVH (AE_MLA_DV / 2)
#define AE_MLA_QT 4        // query blocks resident in TMEM
#define AE_MLA_STAGES 2
#if AE_MLA_BN != 64
#error "the MLA decode kernel streams 64-row KV tiles"
#endif

#define AE_MLA_QS_BYTES ((AE_MLA_NBK - AE_MLA_QT) * AE_MLA_H * 128)  // query blocks kept in shared memory
#define AE_MLA_KV_BYTES (AE_MLA_NBK * AE_MLA_BN * 128)
#define AE_MLA_SMEM_QS 0
#define AE_MLA_SMEM_KV (AE_MLA_QS_BYTES)
#define AE_MLA_SMEM_BAR (AE_MLA_SMEM_KV + AE_MLA_STAGES * AE_MLA_KV_BYTES)

struct AeMlaBars {
  u64 q_full;   // the whole query block landed in shared memory
  u64 q_tmem;   // its first blocks were copied to TMEM (KV stage 0 is free)
  // A KV stage is two parts with their own barriers: the CTA's own half of the value dims (4 blocks, held until the
  // tile's P V GEMM has run) and the rest (the other half and the rope block, 5 blocks, free as soon as the S GEMM has
  // read them).  With two stages the refill of a stage used to wait for P V of the tile before; now 40 of its 72 KB
  // are requested one S GEMM earlier, and only the value part's 32 KB sit on the chain P V -> load -> next S GEMM.
  u64 kv_full[AE_MLA_STAGES];    // the value part landed
  u64 kv_empty[AE_MLA_STAGES];   // ... and was read by P V
  u64 kx_full[AE_MLA_STAGES];    // the rest landed
  u64 kx_empty[AE_MLA_STAGES];   // ... and was read by the S GEMM
  u64 s_full[2];
  u64 o_done;
  AeCtaCtl ctl;
};

extern "C" __global__ void __launch_bounds__(192, 1) ae_mla_decode(const __grid_constant__ AeMlaArgs args) {
  extern __shared__ u8 smem_raw[];
  u8* smem = smem_align1024(smem_raw);
  AeMlaBars* bars = (AeMlaBars*)(smem + AE_MLA_SMEM_BAR);
  AeCtaCtl* ctl = &bars->ctl;
  const u32 warp = threadIdx.x >> 5;
  const u32 lane = threadIdx.x & 31;
  const int dvh = blockIdx.x;    // which half of the value dims
  const int split = blockIdx.y;
  const int b = blockIdx.z;

#ifdef AE_TRACE
  const bool trace_on = blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && (threadIdx.x & 31) == 0;
#endif
  const int S_b = args.seqlens ? args.seqlens[b] : args.S;  // keys of this batch row
  const int n_tiles = (S_b + AE_MLA_BN - 1) / AE_MLA_BN;
  const int t_begin = split * args.tiles_per_split;
  int t_end = t_begin + args.tiles_per_split;
  if (t_end > n_tiles) t_end = n_tiles;
  const int n_steps = t_end > t_begin ? t_end - t_begin : 0;

  if (threadIdx.x == 0) {
    ctl->abort = 0;
    mbar_init(&bars->q_full, 1);
    mbar_init(&bars->q_tmem, 4);
    mbar_init(&bars->o_done, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars->kv_full[i], 1);
      mbar_init(&bars->kv_empty[i], 1);
      mbar_init(&bars->kx_full[i], 1);
      mbar_init(&bars->kx_empty[i], 1);
      mbar_init(&bars->s_full[i], 1);
    }
    mbar_fence_init();
  }
  if (warp == 5) {
    tmem_alloc(&ctl->tmem_base, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const u32 tmem = ctl->tmem_base;
  const u32 TM_S = 0, TM_O = 128, TM_Q = 384;  // S buffer i at TM_S + 64 i

  if (warp == 4) {
    // =============================== TMA producer ===============================
    if (lane == 0 && n_steps > 0) {
      tma_prefetch_desc(&args.tm_q);
      tma_prefetch_desc(&args.tm_qpe);
      tma_prefetch_desc(&args.tm_kv);
      tma_prefetch_desc(&args.tm_kpe);
      mbar_arrive_expect_tx(&bars->q_full, AE_MLA_NBK * AE_MLA_H * 128);
      // blocks 0 .. QT-1 pass through KV stage 0 on their way to TMEM, the rest stay in their own area
      for (int blk = 0; blk < AE_MLA_QT; ++blk)
        tma_load_3d(smem + AE_MLA_SMEM_KV + blk * (AE_MLA_H * 128), &args.tm_q, &bars->q_full, blk * 64, 0, b);
      for (int blk = AE_MLA_QT; blk < AE_MLA_NBV; ++blk)
        tma_load_3d(smem + AE_MLA_SMEM_QS + (blk - AE_MLA_QT) * (AE_MLA_H * 128), &args.tm_q, &bars->q_full, blk * 64, 0, b);
      tma_load_3d(smem + AE_MLA_SMEM_QS + (AE_MLA_NBV - AE_MLA_QT) * (AE_MLA_H * 128), &args.tm_qpe, &bars->q_full, 0, 0, b);
      for (int s = 0; s < n_steps; ++s) {
        const int stage = s % AE_MLA_STAGES;
        if (s == 0 && !mbar_wait(&bars->q_tmem, 0, ctl, args.status, 40)) break;
        if (!mbar_wait(&bars->kx_empty[stage], ((s / AE_MLA_STAGES) & 1) ^ 1, ctl, args.status, 41)) break;
        // dense: rows (tile * 64 ..) of batch b; paged: the tile's page in the pool (a page index outside the pool
        // reads the fill value, it cannot fault)
        int kv0 = (t_begin + s) * AE_MLA_BN, kb = b;
        if (args.block_table) {
          kv0 = args.block_table[(i64)b * args.max_pages + (t_begin + s)] * AE_MLA_BN;
          kb = 0;
        }
        u8* dst = smem + AE_MLA_SMEM_KV + stage * AE_MLA_KV_BYTES;
        const int v_lo = dvh * (AE_MLA_NBV / 2), v_hi = v_lo + AE_MLA_NBV / 2;  // this CTA's value blocks
        mbar_arrive_expect_tx(&bars->kx_full[stage], (AE_MLA_NBK - AE_MLA_NBV / 2) * (AE_MLA_BN * 128));
        for (int blk = 0; blk < AE_MLA_NBV; ++blk)
          if (blk < v_lo || blk >= v_hi)
            tma_load_3d(dst + blk * (AE_MLA_BN * 128), &args.tm_kv, &bars->kx_full[stage], blk * 64, kv0, kb);
        tma_load_3d(dst + AE_MLA_NBV * (AE_MLA_BN * 128), &args.tm_kpe, &bars->kx_full[stage], 0, kv0, kb);
        if (!mbar_wait(&bars->kv_empty[stage], ((s / AE_MLA_STAGES) & 1) ^ 1, ctl, args.status, 41)) break;
        mbar_arrive_expect_tx(&bars->kv_full[stage], (AE_MLA_NBV / 2) * (AE_MLA_BN * 128));
        for (int blk = v_lo; blk < v_hi; ++blk)
          tma_load_3d(dst + blk * (AE_MLA_BN * 128), &args.tm_kv, &bars->kv_full[stage], blk * 64, kv0, kb);
      }
    }
  } else if (warp == 5) {
    // =============================== MMA issuer =================================
    if (n_steps > 0) {  // all 32 lanes run the control flow; MMAs and commits are issued by an elected lane
      const u32 idesc_s = umma_idesc_f16(AE_MLA_H, AE_MLA_BN, AE_BF16, 0, 0);
      const u32 idesc_o = umma_idesc_f16(AE_MLA_H, AE_MLA_DVH, AE_BF16, 0, 1);
      const u32 qs_addr = smem_u32(smem + AE_MLA_SMEM_QS);
      const u32 kv_addr = smem_u32(smem + AE_MLA_SMEM_KV);
      const u64 dq0 = umma_base_k(qs_addr), dk0 = umma_base_k(kv_addr);
      const u64 dv0 = umma_base_mn(kv_addr + dvh * (AE_MLA_NBV / 2) * (AE_MLA_BN * 128), AE_MLA_BN);
      auto issue_s = [&](int s, bool landed) -> bool {  // S_s into region s & 1
        const int stage = s % AE_MLA_STAGES;
        AE_TRM(true, 0, s * 8 + 0)
        if (!landed) {
          if (!mbar_wait_w(&bars->kx_full[stage], (s / AE_MLA_STAGES) & 1, ctl, args.status, 43)) return false;
          if (!mbar_wait_w(&bars->kv_full[stage], (s / AE_MLA_STAGES) & 1, ctl, args.status, 44)) return false;
        }
        tc_fence_after_sync();
        AE_TRM(true, 0, s * 8 + 1)
        const u32 d = tmem + TM_S + (s & 1) * 64;
        const u64 dks = dk0 + (u64)((stage * AE_MLA_KV_BYTES) >> 4);
#pragma unroll
        for (int blk = 0; blk < AE_MLA_NBK; ++blk) {
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) {
            const u64 db = dks + (u64)((blk * (AE_MLA_BN * 128) + kk * 32) >> 4);
            if (blk < AE_MLA_QT)
              umma_ts_w(d, tmem + TM_Q + blk * 32 + kk * 8, db, idesc_s, (blk | kk) > 0);
            else
              umma_ss_w(d, dq0 + (u64)(((blk - AE_MLA_QT) * (AE_MLA_H * 128) + kk * 32) >> 4), db, idesc_s, 1);
          }
        }
        umma_commit_w(&bars->kx_empty[stage]);  // the five blocks that only the S GEMM reads can be refilled
        umma_commit_w(&bars->s_full[s & 1]);
        AE_TRM(true, 0, s * 8 + 2)
        return true;
      };
      // the blocks that stay in shared memory are read by the MMAs themselves: this warp waits for the TMA barrier
      // too, not only for the row threads that saw it
      bool ok = mbar_wait_w(&bars->q_full, 0, ctl, args.status, 49);
      ok = ok && mbar_wait_w(&bars->q_tmem, 0, ctl, args.status, 42);
      tc_fence_after_sync();
      if (ok) ok = issue_s(0, false);
      for (int s = 0; s < n_steps && ok; ++s) {
        const int stage = s % AE_MLA_STAGES;
        // The next S GEMM goes first if both parts of its KV tile have already landed (the other S region held P of tile
        // s-1, whose P V GEMM was issued in the previous iteration); otherwise P V of this tile must not wait behind the
        // load.
        bool early = false;
        if (s + 1 < n_steps) {
          const int ns = (s + 1) % AE_MLA_STAGES;
          const u32 np = ((s + 1) / AE_MLA_STAGES) & 1;
          early = __all_sync(0xffffffffu, mbar_try_wait(&bars->kx_full[ns], np) && mbar_try_wait(&bars->kv_full[ns], np));
          if (early) ok = issue_s(s + 1, true);
        }
        if (!ok) break;
        AE_TRM(true, 0, s * 8 + 3)
        // P of tile s: a named barrier (the four row warps arrive in every iteration, whatever happened; about 20 clk
        // for this warp against 100 - 400 clk for an mbarrier wait)
        named_bar_sync(1 + (s & 1), 128 + 32);
        tc_fence_after_sync();
        AE_TRM(true, 0, s * 8 + 4)
        // V = this half's four 64-wide blocks of the same tile, read MN-major
        const u64 dvs = dv0 + (u64)((stage * AE_MLA_KV_BYTES) >> 4);
#pragma unroll
        for (int kk = 0; kk < AE_MLA_BN / 16; ++kk)
          umma_ts_w(tmem + TM_O, tmem + TM_S + (s & 1) * 64 + kk * 8, umma_step_mn(dvs, kk), idesc_o, (s > 0) | (kk > 0));
        umma_commit_w(&bars->o_done);
        umma_commit_w(&bars->kv_empty[stage]);
        AE_TRM(true, 0, s * 8 + 5)
        if (s + 1 < n_steps && !early) ok = issue_s(s + 1, false);
      }
    }
  } else {
    // =============================== row threads (one per head) =================
    const u32 row = threadIdx.x & 127;
    const u32 lane_base = ((warp & 3) * 32) << 16;
    const u32 tm_o = tmem + TM_O + lane_base;
    const int h = (int)row;
    bool ok = true;
    // ---- query blocks 0 .. QT-1 of this head: shared memory (KV stage 0) -> TMEM, once -----------------
    if (n_steps > 0) {
      ok = mbar_wait(&bars->q_full, 0, ctl, args.status, 48);
      const u8* src = smem + AE_MLA_SMEM_KV;
      for (int blk = 0; blk < AE_MLA_QT; ++blk) {
        u32 w[32];
#pragma unroll
        for (int ch = 0; ch < 8; ++ch) {
          const uint4 v = *(const uint4*)(src + blk * (AE_MLA_H * 128) + swz128(row, ch));
          w[ch * 4 + 0] = v.x;
          w[ch * 4 + 1] = v.y;
          w[ch * 4 + 2] = v.z;
          w[ch * 4 + 3] = v.w;
        }
        tmem_st32(tmem + TM_Q + lane_base + blk * 32, w);  // column c holds elements 2c, 2c + 1 of the row
      }
      tc_wait_st();
      tc_fence_before_sync();
      mbar_arrive_warp(&bars->q_tmem);
    }
    AeCustom cu;
#pragma unroll
    for (int i = 0; i < AE_MAX_CUSTOM; ++i) {
      cu.p[i] = nullptr;
#pragma unroll
      for (int k = 0; k < 4; ++k) cu.st[i][k] = 0;
    }
    AeRow st;
    st.init();
    for (int s = 0; s < n_steps; ++s) {
      const u32 tm_s = tmem + TM_S + (s & 1) * 64 + lane_base;
      AE_TRM(warp == 0, 1, s * 8 + 0)
      ok = ok && mbar_wait(&bars->s_full[s & 1], (s >> 1) & 1, ctl, args.status, 45);
      tc_fence_after_sync();
      AE_TRM(warp == 0, 1, s * 8 + 1)
      float sc[AE_MLA_BN];
      tmem_ld_f32x64(tm_s, sc);
      const int kv0 = (t_begin + s) * AE_MLA_BN;
      if (kv0 + AE_MLA_BN > S_b) {
#pragma unroll
        for (int c = 0; c < AE_MLA_BN; ++c)
          if (kv0 + c >= S_b) sc[c] = -__int_as_float(0x7f800000);
      }
      const float o_scale = ae_online_fwd<AE_MLA_BN>(sc, st, b, h, 0, kv0, cu);
      {
        u32 pk[32];
#pragma unroll
        for (int half = 0; half < AE_MLA_BN / 64; ++half) {
#pragma unroll
          for (int i = 0; i < 32; ++i) pk[i] = pack2<AE_BF16>(sc[half * 64 + 2 * i], sc[half * 64 + 2 * i + 1]);
          tmem_st32(tm_s + half * 32, pk);
        }
      }
#if !AE_O_SCALE_ONE
      // O is rescaled only when some row of the warp needs it; only then must the previous P V GEMM have completed.
      // Phase bookkeeping of the skipped waits: S_s may be issued before P V of tile s-1, so s_full(s) only implies
      // that P V of tile s-2 has completed: o_done has then completed s-1 or s phases, and a parity wait for phase
      // s-1 cannot alias.  The wait after the loop asks for phase n-1 and would alias if only n-2 had completed, so
      // the last step always waits for its predecessor.
      const bool rescale = __any_sync(0xffffffffu, o_scale != 1.0f);
      if (s > 0 && (rescale || s + 1 == n_steps)) {
        ok = ok && mbar_wait(&bars->o_done, (s - 1) & 1, ctl, args.status, 46);
        tc_fence_after_sync();
        if (rescale) {
#pragma unroll
          for (int c = 0; c < AE_MLA_DVH / 32; ++c) {
            float f[32];
            u32 r[32];
            tmem_ld_f32x32(tm_o + c * 32, f);
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(f[i] * o_scale);
            tmem_st32(tm_o + c * 32, r);
          }
        }
      }
#else
      if (s > 0 && s + 1 == n_steps) {  // same phase bookkeeping: the wait after the loop must not find o_done two phases behind
        ok = ok && mbar_wait(&bars->o_done, (s - 1) & 1, ctl, args.status, 46);
        tc_fence_after_sync();
      }
#endif
      tc_wait_st();
      tc_fence_before_sync();
      named_bar_arrive(1 + (s & 1), 128 + 32);
      AE_TRM(warp == 0, 1, s * 8 + 2)
    }

    if (n_steps > 0) {
      ok = ok && mbar_wait(&bars->o_done, (n_steps - 1) & 1, ctl, args.status, 47);
      tc_fence_after_sync();
      const bool store = ok && h < args.H;
      const int hs = store ? h : 0;
      if (args.n_split == 1) {
        u16* orow = (u16*)args.o + ((i64)b * args.H + hs) * AE_MLA_DV + dvh * AE_MLA_DVH;
#pragma unroll
        for (int c = 0; c < AE_MLA_DVH / 32; ++c) {
          float r[32];
          tmem_ld_f32x32(tm_o + c * 32, r);
          if (store) {
            uint4* dst = (uint4*)(orow + c * 32);
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              uint4 w;
              w.x = pack2<AE_BF16>(ae_epilogue_o(r[v * 8 + 0], st), ae_epilogue_o(r[v * 8 + 1], st));
              w.y = pack2<AE_BF16>(ae_epilogue_o(r[v * 8 + 2], st), ae_epilogue_o(r[v * 8 + 3], st));
              w.z = pack2<AE_BF16>(ae_epilogue_o(r[v * 8 + 4], st), ae_epilogue_o(r[v * 8 + 5], st));
              w.w = pack2<AE_BF16>(ae_epilogue_o(r[v * 8 + 6], st), ae_epilogue_o(r[v * 8 + 7], st));
              dst[v] = w;
            }
          }
        }
      } else {
        float* prow = args.o_part + (((i64)b * args.n_split + split) * args.H + hs) * AE_MLA_DV + dvh * AE_MLA_DVH;
#pragma unroll
        for (int c = 0; c < AE_MLA_DVH / 32; ++c) {
          float r[32];
          tmem_ld_f32x32(tm_o + c * 32, r);
          if (store) {
            float4* dst = (float4*)(prow + c * 32);
#pragma unroll
            for (int v = 0; v < 8; ++v)
              dst[v] = make_float4(ae_epilogue_o(r[v * 4 + 0], st), ae_epilogue_o(r[v * 4 + 1], st),
                                   ae_epilogue_o(r[v * 4 + 2], st), ae_epilogue_o(r[v * 4 + 3], st));
          }
        }
      }
#if AE_NFINAL > 0
      if (store && dvh == 0) {
        float fr[AE_NFINAL];
        ae_final_rowscales(st, fr);
#pragma unroll
        for (int i = 0; i < AE_NFINAL; ++i)
          if (args.fr_part[i]) args.fr_part[i][((i64)b * args.n_split + split) * args.H + h] = fr[i];
      }
#endif
    } else if (args.n_split > 1 && h < args.H) {
      // rows of different lengths: this split starts past the row's last tile.  Its partial is zero with -inf row
      // scales, which the combine pass weighs with exp(-inf - ...) = 0.
      float4* dst = (float4*)(args.o_part + (((i64)b * args.n_split + split) * args.H + h) * AE_MLA_DV + dvh * AE_MLA_DVH);
      for (int v = 0; v < AE_MLA_DVH / 4; ++v) dst[v] = make_float4(0.f, 0.f, 0.f, 0.f);
#if AE_NFINAL > 0
      if (dvh == 0)
        for (int i = 0; i < AE_NFINAL; ++i)
          if (args.fr_part[i]) args.fr_part[i][((i64)b * args.n_split + split) * args.H + h] = -__int_as_float(0x7f800000);
#endif
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 5) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, 512);
  }
}
