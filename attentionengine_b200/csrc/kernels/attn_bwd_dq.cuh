// Attention backward, dQ pass, for sm_100a.  Together with attn_bwd_dkv.cuh it replaces
// the reference's `flash_bwd` + `flash_bwd_post` kernels
// (attention_engine/core/template/tl_template/attn/attn_tl.py:239-415, 436-455): instead of
// one kv-stationary kernel that atomically adds fp32 dQ tiles into a staging buffer, dQ is
// produced here by a q-stationary kernel that owns its output rows, so there are no
// atomics, no fp32 dQ buffer and no conversion kernel; the price is that S and dP are
// recomputed in both passes.
//
// One CTA owns one 128-row q tile of one (batch, q-head) and streams K/V tiles of AE_BWD_BN
// rows.  Per kv tile:
//   S  = Q  K^T   (SS MMA)        dP = dO V^T   (SS MMA)
//   row threads: T = score_mod(S); P = OnlineFunc.forward(T); mask; dT = OnlineFunc.backward(dP, P);
//                dS = score_mod'(S) dT  -> 16-bit pairs written over S in TMEM
//   dQ += dS K    (TS MMA, K tile read MN-major)
// TMEM columns: AE_BWD_NBUF x (S | dP) then dQ.  With two buffers the tensor pipe computes the
// next tile's S / dP while the row threads work on the current one.
// Roles: warps 0-3 and 4-7 row threads (thread = q row = TMEM lane; the two groups take alternate
// 32-column chunks of every tile), warp 8 TMA producer, warp 9 MMA issuer.  The 16-bit dS pairs of a
// chunk are written over the first 16 columns of that chunk, so a group only overwrites what it has read.

#define AE_BM 128
#define AE_NTHREADS_BWD 320
// Optional phase trace of CTA (0, 0, 0): 32-bit clock stamps behind the status word (bring-up / tuning only).
#ifdef AE_TRACE
#define AE_TR(cond, region, slot) \
  if (trace_on && (cond) && (slot) < 1024) args.status[64 + (region) * 4096 + (slot)] = (u32)clock64();
#else
#define AE_TR(cond, region, slot)
#endif
#define AE_NSUB (128 / AE_BWD_BN)

#define AE_DQ_Q_BYTES (AE_BM * AE_D * 2)
#define AE_DQ_DO_BYTES (AE_BM * AE_DV * 2)
#define AE_DQ_K_BYTES (AE_BWD_BN * AE_D * 2)
#define AE_DQ_V_BYTES (AE_BWD_BN * AE_DV * 2)
#define AE_DQ_SMEM_Q 0
#define AE_DQ_SMEM_DO (AE_DQ_Q_BYTES)
#define AE_DQ_SMEM_K (AE_DQ_SMEM_DO + AE_DQ_DO_BYTES)
#define AE_DQ_SMEM_V (AE_DQ_SMEM_K + AE_BWD_STAGES * AE_DQ_K_BYTES)
#define AE_DQ_SMEM_BAR (AE_DQ_SMEM_V + AE_BWD_STAGES * AE_DQ_V_BYTES)

struct AeDqBars {
  u64 qdo_full;
  u64 k_full[AE_BWD_STAGES];
  u64 k_empty[AE_BWD_STAGES];
  u64 v_full[AE_BWD_STAGES];
  u64 v_empty[AE_BWD_STAGES];
  u64 sp_full[AE_BWD_NBUF];
  u64 ds_full[AE_BWD_NBUF];
  u64 dq_done;
  AeCtaCtl ctl;
};

extern "C" __global__ void __launch_bounds__(AE_NTHREADS_BWD, 1)
ae_attn_bwd_dq(const __grid_constant__ AeAttnBwdArgs args) {
  extern __shared__ u8 smem_raw[];
  u8* smem = smem_align1024(smem_raw);
  AeDqBars* bars = (AeDqBars*)(smem + AE_DQ_SMEM_BAR);
  AeCtaCtl* ctl = &bars->ctl;
  const u32 warp = threadIdx.x >> 5;
  const u32 lane = threadIdx.x & 31;

  const int qt = (int)gridDim.x - 1 - (int)blockIdx.x;  // heavy tiles first under a causal mask
  const int hq = blockIdx.y;
  const int b = blockIdx.z;
  const int hk = hq / (args.Hq / args.Hkv);
  const int q0 = qt * AE_BM;
  const int n_kt_bn = (args.Skv + AE_BWD_BN - 1) / AE_BWD_BN;
#ifdef AE_TRACE
  const bool trace_on = blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && (threadIdx.x & 31) == 0;
#endif

  // ---- kv schedule ------------------------------------------------------------------
  int n_steps;
#if AE_MASK_MODE == 1
  n_steps = (q0 + AE_BM + AE_BWD_BN - 1) / AE_BWD_BN;
  if (n_steps > n_kt_bn) n_steps = n_kt_bn;
#elif AE_MASK_MODE == 2
  const int n_list = args.blk_cnt[((i64)b * args.Hq + hq) * args.n_qt + qt];
  const int* list = args.blk_idx + (((i64)b * args.Hq + hq) * args.n_qt + qt) * (i64)args.n_kt;
  n_steps = n_list * AE_NSUB;
#else
  n_steps = n_kt_bn;
#endif
  // step -> (first kv column, needs element mask)
  auto step_info = [&](int s, int& kv0, bool& partial) {
#if AE_MASK_MODE == 2
    const int e = list[s / AE_NSUB];
    kv0 = (e & 0x3fffffff) * 128 + (s % AE_NSUB) * AE_BWD_BN;
    partial = ((u32)e >> 30) & 1u;
#else
    kv0 = s * AE_BWD_BN;
#if AE_MASK_MODE == 1
    partial = kv0 + AE_BWD_BN - 1 > q0;
#elif AE_MASK_MODE == 3
    partial = true;
#else
    partial = false;
#endif
#endif
  };

  if (threadIdx.x == 0) {
    ctl->abort = 0;
    mbar_init(&bars->qdo_full, 1);
    mbar_init(&bars->dq_done, 1);
    for (int i = 0; i < AE_BWD_STAGES; ++i) {
      mbar_init(&bars->k_full[i], 1);
      mbar_init(&bars->k_empty[i], 1);
      mbar_init(&bars->v_full[i], 1);
      mbar_init(&bars->v_empty[i], 1);
    }
    for (int i = 0; i < AE_BWD_NBUF; ++i) {
      mbar_init(&bars->sp_full[i], 1);
      mbar_init(&bars->ds_full[i], 8);
    }
    mbar_fence_init();
  }
  if (warp == 9) {
    tmem_alloc(&ctl->tmem_base, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const u32 tmem = ctl->tmem_base;
  const u32 TM_DQ = AE_BWD_NBUF * 2 * AE_BWD_BN;

  if (warp == 8) {
    // =============================== TMA producer ===============================
    if (lane == 0 && n_steps > 0) {
      tma_prefetch_desc(&args.tm_q);
      tma_prefetch_desc(&args.tm_k);
      tma_prefetch_desc(&args.tm_v);
      tma_prefetch_desc(&args.tm_do);
      mbar_arrive_expect_tx(&bars->qdo_full, AE_DQ_Q_BYTES + AE_DQ_DO_BYTES);
      for (int dh = 0; dh < AE_D / 64; ++dh)
        tma_load_4d(smem + AE_DQ_SMEM_Q + dh * (AE_BM * 128), &args.tm_q, &bars->qdo_full, dh * 64, hq, q0, b);
      for (int dh = 0; dh < AE_DV / 64; ++dh)
        tma_load_4d(smem + AE_DQ_SMEM_DO + dh * (AE_BM * 128), &args.tm_do, &bars->qdo_full, dh * 64, hq, q0, b);
      for (int s = 0; s < n_steps; ++s) {
        int kv0;
        bool partial;
        step_info(s, kv0, partial);
        const int stage = s % AE_BWD_STAGES;
        const u32 par = ((s / AE_BWD_STAGES) & 1) ^ 1;
        if (!mbar_wait(&bars->k_empty[stage], par, ctl, args.status, 21)) break;
        mbar_arrive_expect_tx(&bars->k_full[stage], AE_DQ_K_BYTES);
        for (int dh = 0; dh < AE_D / 64; ++dh)
          tma_load_4d(smem + AE_DQ_SMEM_K + stage * AE_DQ_K_BYTES + dh * (AE_BWD_BN * 128), &args.tm_k,
                      &bars->k_full[stage], dh * 64, hk, kv0, b);
        if (!mbar_wait(&bars->v_empty[stage], par, ctl, args.status, 22)) break;
        mbar_arrive_expect_tx(&bars->v_full[stage], AE_DQ_V_BYTES);
        for (int dh = 0; dh < AE_DV / 64; ++dh)
          tma_load_4d(smem + AE_DQ_SMEM_V + stage * AE_DQ_V_BYTES + dh * (AE_BWD_BN * 128), &args.tm_v,
                      &bars->v_full[stage], dh * 64, hk, kv0, b);
      }
    }
  } else if (warp == 9) {
    // =============================== MMA issuer =================================
    if (n_steps > 0) {  // all 32 lanes run the control flow; single MMAs and commits are issued by an elected lane
      const u32 idesc_s = umma_idesc_f16(AE_BM, AE_BWD_BN, AE_BF16, 0, 0);
      const u32 idesc_dq = umma_idesc_f16(AE_BM, AE_D, AE_BF16, 0, 1);
      const u32 q_addr = smem_u32(smem + AE_DQ_SMEM_Q);
      const u32 do_addr = smem_u32(smem + AE_DQ_SMEM_DO);
      const u32 k_addr = smem_u32(smem + AE_DQ_SMEM_K);
      const u32 v_addr = smem_u32(smem + AE_DQ_SMEM_V);
      bool ok = mbar_wait_w(&bars->qdo_full, 0, ctl, args.status, 23);
      const u64 dq0 = umma_base_k(q_addr), ddo0 = umma_base_k(do_addr);
      const u64 dk0 = umma_base_k(k_addr), dv0 = umma_base_k(v_addr);
      const u64 dkmn0 = umma_base_mn(k_addr, AE_BWD_BN);

      auto issue_sp = [&](int s) -> bool {
        const int stage = s % AE_BWD_STAGES;
        const u32 par = (s / AE_BWD_STAGES) & 1;
        const int buf = s % AE_BWD_NBUF;
        const u32 tm_s = tmem + buf * 2 * AE_BWD_BN;
        const u32 tm_dp = tm_s + AE_BWD_BN;
        AE_TR(true, 3, s * 8 + 0)
        if (!mbar_wait_w(&bars->k_full[stage], par, ctl, args.status, 24)) return false;
        tc_fence_after_sync();
        AE_TR(true, 3, s * 8 + 1)
        const u64 dkk = dk0 + (u64)((stage * AE_DQ_K_BYTES) >> 4);
#pragma unroll
        for (int kk = 0; kk < AE_D / 16; ++kk)
          umma_ss_w(tm_s, umma_step_k(dq0, kk, AE_BM), umma_step_k(dkk, kk, AE_BWD_BN), idesc_s, kk > 0);
        AE_TR(true, 3, s * 8 + 2)
        if (!mbar_wait_w(&bars->v_full[stage], par, ctl, args.status, 25)) return false;
        tc_fence_after_sync();
        AE_TR(true, 3, s * 8 + 3)
        const u64 dvv = dv0 + (u64)((stage * AE_DQ_V_BYTES) >> 4);
#pragma unroll
        for (int kk = 0; kk < AE_DV / 16; ++kk)
          umma_ss_w(tm_dp, umma_step_k(ddo0, kk, AE_BM), umma_step_k(dvv, kk, AE_BWD_BN), idesc_s, kk > 0);
        AE_TR(true, 3, s * 8 + 4)
        umma_commit_w(&bars->sp_full[buf]);
        umma_commit_w(&bars->v_empty[stage]);
        AE_TR(true, 3, s * 8 + 5)
        return true;
      };

      if (ok) ok = issue_sp(0);
      for (int s = 0; s < n_steps && ok; ++s) {
        const int stage = s % AE_BWD_STAGES;
        const int buf = s % AE_BWD_NBUF;
        if (AE_BWD_NBUF > 1 && s + 1 < n_steps) ok = issue_sp(s + 1);
        if (!ok) break;
        AE_TR(true, 0, s * 4 + 0)
        ok = mbar_wait_w(&bars->ds_full[buf], (s / AE_BWD_NBUF) & 1, ctl, args.status, 26);
        if (!ok) break;
        AE_TR(true, 0, s * 4 + 1)
        tc_fence_after_sync();
        const u32 tm_ds = tmem + buf * 2 * AE_BWD_BN;  // dS pairs over the S columns
        const u64 dkm = dkmn0 + (u64)((stage * AE_DQ_K_BYTES) >> 4);
#pragma unroll
        for (int kk = 0; kk < AE_BWD_BN / 16; ++kk)
          umma_ts_w(tmem + TM_DQ, tm_ds + (kk >> 1) * 32 + (kk & 1) * 8, umma_step_mn(dkm, kk), idesc_dq, (s > 0) | (kk > 0));
        umma_commit_w(&bars->k_empty[stage]);
        if (s + 1 == n_steps) umma_commit_w(&bars->dq_done);
        AE_TR(true, 0, s * 4 + 2)
        if (AE_BWD_NBUF == 1 && s + 1 < n_steps) ok = issue_sp(s + 1);
      }
    }
  } else {
    // =============================== row threads ================================
    const int wg = warp >> 2;  // the two row warpgroups split every tile by 32-column chunks
    const u32 row = threadIdx.x & 127;
    const u32 lane_base = ((warp & 3) * 32) << 16;
    const int q_idx = q0 + (int)row;
    const bool row_valid = q_idx < args.Sq;
    const i64 rs_off = ((i64)b * args.Hq + hq) * args.Sq + (row_valid ? q_idx : 0);

    AeCustom cu;
#pragma unroll
    for (int i = 0; i < AE_MAX_CUSTOM; ++i) {
      cu.p[i] = args.custom[i];
#pragma unroll
      for (int k = 0; k < 4; ++k) cu.st[i][k] = args.custom_st[i][k];
    }
    float fr[AE_NFINAL > 0 ? AE_NFINAL : 1];
#pragma unroll
    for (int i = 0; i < AE_NFINAL; ++i) fr[i] = args.final_rs[i][rs_off];
#if AE_USES_DOOSUM
    const float delta = args.delta[rs_off];
#else
    const float delta = 0.f;
#endif

    bool ok = true;
    for (int s = 0; s < n_steps; ++s) {
      int kv0;
      bool partial;
      step_info(s, kv0, partial);
      const int buf = s % AE_BWD_NBUF;
      const u32 tm_s = tmem + buf * 2 * AE_BWD_BN + lane_base;
      const u32 tm_dp = tm_s + AE_BWD_BN;
      AE_TR((warp & 3) == 0, 1 + wg, s * 4 + 0)
      ok = ok && mbar_wait(&bars->sp_full[buf], (s / AE_BWD_NBUF) & 1, ctl, args.status, 27);
      tc_fence_after_sync();
      AE_TR((warp & 3) == 0, 1 + wg, s * 4 + 1)
      const bool tail = kv0 + AE_BWD_BN > args.Skv;
      auto chunk = [&](auto masked_tag, int c) {
        constexpr bool kMasked = decltype(masked_tag)::value;
        float sv[32], dp[32];
        tmem_ld_2xf32x32(tm_s + c * 32, tm_dp + c * 32, sv, dp);
        u32 pk[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float ds2[2];
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int kv_idx = kv0 + c * 32 + i + e;
            const float sraw = sv[i + e];
            float p = ae_bwd_p(sraw, fr, b, hq, q_idx, kv_idx, cu, i + e);
            float dpv = dp[i + e];
            bool keep = true;
            if (kMasked) {
              keep = kv_idx < args.Skv;
#if AE_MASK_MODE != 0
              if (partial) keep = keep && ae_mask(b, hq, q_idx, kv_idx);
#endif
              if (!keep) {
                p = 0.f;
                dpv = 0.f;
              }
            }
            float dsv = ae_bwd_ds(sraw, dpv, p, fr, delta, b, hq, q_idx, kv_idx, cu);
            if (kMasked && !keep) dsv = 0.f;
            ds2[e] = dsv;
          }
          pk[i >> 1] = pack2<AE_BF16>(ds2[0], ds2[1]);
        }
        tmem_st16(tm_s + c * 32, pk);  // pairs go over this chunk's own first 16 columns
      };
      if (partial || tail) {
        for (int c = wg; c < AE_BWD_BN / 32; c += 2) chunk(AeTrue{}, c);
      } else {
        for (int c = wg; c < AE_BWD_BN / 32; c += 2) chunk(AeFalse{}, c);
      }
      AE_TR((warp & 3) == 0, 1 + wg, s * 4 + 2)
      tc_wait_st();
      tc_fence_before_sync();
      mbar_arrive_warp(&bars->ds_full[buf]);
      AE_TR((warp & 3) == 0, 1 + wg, s * 4 + 3)
    }

    // ---- epilogue: dQ rows -------------------------------------------------------------
    if (n_steps > 0) {
      ok = ok && mbar_wait(&bars->dq_done, 0, ctl, args.status, 28);
      tc_fence_after_sync();
    }
    {
      // tcgen05.ld is warp-collective: every lane runs it; only the stores are per-row
      const bool store = row_valid && ok;
      u16* drow = (u16*)args.dq + (i64)b * args.dq_sb + (i64)(store ? q_idx : 0) * args.dq_ss + (i64)hq * args.dq_sh;
#pragma unroll
      for (int c = wg * (AE_D / 64); c < (wg + 1) * (AE_D / 64); ++c) {
        float r[32];
        if (n_steps > 0) {
          tmem_ld_f32x32(tmem + TM_DQ + lane_base + c * 32, r);
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] = 0.f;
        }
        if (store) {
          uint4* dst = (uint4*)(drow + c * 32);
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            uint4 w;
            w.x = pack2<AE_BF16>(r[v * 8 + 0], r[v * 8 + 1]);
            w.y = pack2<AE_BF16>(r[v * 8 + 2], r[v * 8 + 3]);
            w.z = pack2<AE_BF16>(r[v * 8 + 4], r[v * 8 + 5]);
            w.w = pack2<AE_BF16>(r[v * 8 + 6], r[v * 8 + 7]);
            dst[v] = w;
          }
        }
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 9) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, 512);
  }
}
