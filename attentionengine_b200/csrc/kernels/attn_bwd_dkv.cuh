// Attention backward, dK/dV pass, for sm_100a (see attn_bwd_dq.cuh for how the two passes
// split the reference's `flash_bwd`, attn_tl.py:239-415; GQA variant attn_gqa_tl.py:190-350).
//
// One CTA owns one 128-row kv tile of one (batch, kv-head) and streams the Q / dO tiles
// (AE_BWD_BN rows) of every q-head of that kv-head's group, so dK / dV of a group are summed
// in the CTA's own TMEM accumulators: no atomics (the reference adds half-precision atomics
// across the group, attn_gqa_tl.py:345-348).  Per q tile, with rows = kv and columns = q:
//   S^T  = K  Q^T  (SS MMA)      dP^T = V dO^T  (SS MMA)
//   row threads: P^T = forward(score_mod(S^T)); dS^T = score_mod'(S^T) * backward(dP^T, P^T)
//                (per-column lse / delta come from shared memory); both written back to TMEM
//                as 16-bit pairs over S^T and dP^T
//   dV += P^T dO   (TS MMA, dO tile read MN-major)     dK += dS^T Q  (TS MMA, Q tile read MN-major)
// TMEM columns: dK | dV | AE_BWD_NBUF x (S^T | dP^T).
// Roles: warps 0-3 and 4-7 row threads (thread = kv row = TMEM lane; the two groups take alternate
// 32-column chunks of every tile), warp 8 TMA producer, warp 9 MMA issuer.  The 16-bit pairs of a chunk
// are written over the first 16 columns of that chunk, so a group only overwrites what it has read.

#define AE_KV_BM 128
#define AE_NSUBQ (128 / AE_BWD_BN)
#define AE_NCS (AE_NFINAL + 1)

#define AE_KV_K_BYTES (AE_KV_BM * AE_D * 2)
#define AE_KV_V_BYTES (AE_KV_BM * AE_DV * 2)
#define AE_KV_Q_BYTES (AE_BWD_BN * AE_D * 2)
#define AE_KV_DO_BYTES (AE_BWD_BN * AE_DV * 2)
#define AE_KV_SMEM_K 0
#define AE_KV_SMEM_V (AE_KV_K_BYTES)
#define AE_KV_SMEM_Q (AE_KV_SMEM_V + AE_KV_V_BYTES)
#define AE_KV_SMEM_DO (AE_KV_SMEM_Q + AE_BWD_STAGES * AE_KV_Q_BYTES)
#define AE_KV_SMEM_CS (AE_KV_SMEM_DO + AE_BWD_STAGES * AE_KV_DO_BYTES)
#define AE_KV_CS_BYTES (2 * AE_BWD_BN * AE_NCS * 4)
#define AE_KV_SMEM_BAR (AE_KV_SMEM_CS + ((AE_KV_CS_BYTES + 15) / 16) * 16)

struct AeDkvBars {
  u64 kv_full;
  u64 q_full[AE_BWD_STAGES];
  u64 do_full[AE_BWD_STAGES];
  u64 qdo_empty[AE_BWD_STAGES];
  u64 sp_full[AE_BWD_NBUF];
  u64 pds_full[AE_BWD_NBUF];
  u64 acc_done;
  AeCtaCtl ctl;
};

struct AeDkvStep {
  int hq;       // q head
  int q0;       // first q row of the tile
  bool partial; // needs the element-wise mask
};

extern "C" __global__ void __launch_bounds__(320, 1)
ae_attn_bwd_dkv(const __grid_constant__ AeAttnBwdArgs args) {
  extern __shared__ u8 smem_raw[];
  u8* smem = smem_align1024(smem_raw);
  AeDkvBars* bars = (AeDkvBars*)(smem + AE_KV_SMEM_BAR);
  float* cs = (float*)(smem + AE_KV_SMEM_CS);  // [2][AE_NCS][AE_BWD_BN]: final rowscales..., delta, per q column
  AeCtaCtl* ctl = &bars->ctl;
  const u32 warp = threadIdx.x >> 5;
  const u32 lane = threadIdx.x & 31;

  const int kt = blockIdx.x;
  const int hk = blockIdx.y;
  const int b = blockIdx.z;
  const int G = args.Hq / args.Hkv;
  const int kv0 = kt * AE_KV_BM;
  const int n_q_bn = (args.Sq + AE_BWD_BN - 1) / AE_BWD_BN;

  // ---- q schedule: heads of the group outer, q tiles inner ---------------------------
#if AE_MASK_MODE == 1
  int i_start = kv0 / AE_BWD_BN;
  if (i_start > n_q_bn) i_start = n_q_bn;
#else
  const int i_start = 0;
#endif
  struct Walk {
    int g, e, sub;
  } walk = {0, 0, 0};
  auto next_step = [&](AeDkvStep& st) -> bool {
#if AE_MASK_MODE == 2
    while (walk.g < G) {
      const int hq = hk * G + walk.g;
      const i64 base = ((i64)b * args.Hq + hq) * args.n_kt + kt;
      const int n = args.blkT_cnt[base];
      if (walk.e < n) {
        const int ent = args.blkT_idx[base * args.n_qt + walk.e];
        st.hq = hq;
        st.q0 = (ent & 0x3fffffff) * 128 + walk.sub * AE_BWD_BN;
        st.partial = ((u32)ent >> 30) & 1u;
        if (++walk.sub == AE_NSUBQ) {
          walk.sub = 0;
          walk.e++;
        }
        if (st.q0 >= args.Sq) continue;  // second half of a ragged last tile
        return true;
      }
      walk.g++;
      walk.e = 0;
      walk.sub = 0;
    }
    return false;
#else
    const int n_i = n_q_bn - i_start;
    if (n_i <= 0 || walk.g >= G) return false;
    const int i = i_start + walk.e;
    st.hq = hk * G + walk.g;
    st.q0 = i * AE_BWD_BN;
#if AE_MASK_MODE == 1
    st.partial = st.q0 < kv0 + AE_KV_BM - 1;
#elif AE_MASK_MODE == 3
    st.partial = true;
#else
    st.partial = false;
#endif
    if (++walk.e == n_i) {
      walk.e = 0;
      walk.g++;
    }
    return true;
#endif
  };

  if (threadIdx.x == 0) {
    ctl->abort = 0;
    mbar_init(&bars->kv_full, 1);
    mbar_init(&bars->acc_done, 1);
    for (int i = 0; i < AE_BWD_STAGES; ++i) {
      mbar_init(&bars->q_full[i], 1);
      mbar_init(&bars->do_full[i], 1);
      mbar_init(&bars->qdo_empty[i], 1);
    }
    for (int i = 0; i < AE_BWD_NBUF; ++i) {
      mbar_init(&bars->sp_full[i], 1);
      mbar_init(&bars->pds_full[i], 8);
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
  const u32 TM_DK = 0, TM_DV = AE_D, TM_BUF = AE_D + AE_DV;

  if (warp == 8) {
    // =============================== TMA producer ===============================
    if (lane == 0) {
      tma_prefetch_desc(&args.tm_q);
      tma_prefetch_desc(&args.tm_k);
      tma_prefetch_desc(&args.tm_v);
      tma_prefetch_desc(&args.tm_do);
      mbar_arrive_expect_tx(&bars->kv_full, AE_KV_K_BYTES + AE_KV_V_BYTES);
      for (int dh = 0; dh < AE_D / 64; ++dh)
        tma_load_4d(smem + AE_KV_SMEM_K + dh * (AE_KV_BM * 128), &args.tm_k, &bars->kv_full, dh * 64, hk, kv0, b);
      for (int dh = 0; dh < AE_DV / 64; ++dh)
        tma_load_4d(smem + AE_KV_SMEM_V + dh * (AE_KV_BM * 128), &args.tm_v, &bars->kv_full, dh * 64, hk, kv0, b);
      AeDkvStep st;
      int s = 0;
      while (next_step(st)) {
        const int stage = s % AE_BWD_STAGES;
        const u32 par = ((s / AE_BWD_STAGES) & 1) ^ 1;
        if (!mbar_wait(&bars->qdo_empty[stage], par, ctl, args.status, 31)) break;
        mbar_arrive_expect_tx(&bars->q_full[stage], AE_KV_Q_BYTES);
        for (int dh = 0; dh < AE_D / 64; ++dh)
          tma_load_4d(smem + AE_KV_SMEM_Q + stage * AE_KV_Q_BYTES + dh * (AE_BWD_BN * 128), &args.tm_q,
                      &bars->q_full[stage], dh * 64, st.hq, st.q0, b);
        mbar_arrive_expect_tx(&bars->do_full[stage], AE_KV_DO_BYTES);
        for (int dh = 0; dh < AE_DV / 64; ++dh)
          tma_load_4d(smem + AE_KV_SMEM_DO + stage * AE_KV_DO_BYTES + dh * (AE_BWD_BN * 128), &args.tm_do,
                      &bars->do_full[stage], dh * 64, st.hq, st.q0, b);
        ++s;
      }
    }
  } else if (warp == 9) {
    // =============================== MMA issuer =================================
    if (lane == 0) {
      const u32 idesc_s = umma_idesc_f16(AE_KV_BM, AE_BWD_BN, AE_BF16, 0, 0);
      const u32 idesc_dk = umma_idesc_f16(AE_KV_BM, AE_D, AE_BF16, 0, 1);
      const u32 idesc_dv = umma_idesc_f16(AE_KV_BM, AE_DV, AE_BF16, 0, 1);
      const u32 k_addr = smem_u32(smem + AE_KV_SMEM_K);
      const u32 v_addr = smem_u32(smem + AE_KV_SMEM_V);
      const u32 q_addr = smem_u32(smem + AE_KV_SMEM_Q);
      const u32 do_addr = smem_u32(smem + AE_KV_SMEM_DO);

      const u64 dk0 = umma_base_k(k_addr), dv0 = umma_base_k(v_addr);
      const u64 dq0 = umma_base_k(q_addr), ddo0 = umma_base_k(do_addr);
      const u64 dqmn0 = umma_base_mn(q_addr, AE_BWD_BN), ddomn0 = umma_base_mn(do_addr, AE_BWD_BN);
      auto issue_sp = [&](int s) -> bool {
        const int stage = s % AE_BWD_STAGES;
        const u32 par = (s / AE_BWD_STAGES) & 1;
        const int buf = s % AE_BWD_NBUF;
        const u32 tm_s = tmem + TM_BUF + buf * 2 * AE_BWD_BN;
        const u32 tm_dp = tm_s + AE_BWD_BN;
        if (!mbar_wait(&bars->q_full[stage], par, ctl, args.status, 32)) return false;
        tc_fence_after_sync();
        const u64 dqq = dq0 + (u64)((stage * AE_KV_Q_BYTES) >> 4);
#pragma unroll
        for (int kk = 0; kk < AE_D / 16; ++kk)
          umma_ss(tm_s, umma_step_k(dk0, kk, AE_KV_BM), umma_step_k(dqq, kk, AE_BWD_BN), idesc_s, kk > 0);
        if (!mbar_wait(&bars->do_full[stage], par, ctl, args.status, 33)) return false;
        tc_fence_after_sync();
        const u64 ddd = ddo0 + (u64)((stage * AE_KV_DO_BYTES) >> 4);
#pragma unroll
        for (int kk = 0; kk < AE_DV / 16; ++kk)
          umma_ss(tm_dp, umma_step_k(dv0, kk, AE_KV_BM), umma_step_k(ddd, kk, AE_BWD_BN), idesc_s, kk > 0);
        umma_commit(&bars->sp_full[buf]);
        return true;
      };

      // count the steps first (the walk is cheap and identical in every role)
      int n_steps = 0;
      {
        AeDkvStep st;
        while (next_step(st)) ++n_steps;
      }
      bool ok = n_steps > 0 && mbar_wait(&bars->kv_full, 0, ctl, args.status, 34);
      if (ok) ok = issue_sp(0);
      for (int s = 0; s < n_steps && ok; ++s) {
        const int stage = s % AE_BWD_STAGES;
        const int buf = s % AE_BWD_NBUF;
        if (AE_BWD_NBUF > 1 && s + 1 < n_steps) ok = issue_sp(s + 1);
        if (!ok) break;
        ok = mbar_wait(&bars->pds_full[buf], (s / AE_BWD_NBUF) & 1, ctl, args.status, 35);
        if (!ok) break;
        tc_fence_after_sync();
        const u32 tm_p = tmem + TM_BUF + buf * 2 * AE_BWD_BN;
        const u32 tm_ds = tm_p + AE_BWD_BN;
        const u64 dqm = dqmn0 + (u64)((stage * AE_KV_Q_BYTES) >> 4);
        const u64 ddm = ddomn0 + (u64)((stage * AE_KV_DO_BYTES) >> 4);
#pragma unroll
        for (int kk = 0; kk < AE_BWD_BN / 16; ++kk)
          umma_ts(tmem + TM_DV, tm_p + (kk >> 1) * 32 + (kk & 1) * 8, umma_step_mn(ddm, kk), idesc_dv, (s > 0) | (kk > 0));
#pragma unroll
        for (int kk = 0; kk < AE_BWD_BN / 16; ++kk)
          umma_ts(tmem + TM_DK, tm_ds + (kk >> 1) * 32 + (kk & 1) * 8, umma_step_mn(dqm, kk), idesc_dk, (s > 0) | (kk > 0));
        umma_commit(&bars->qdo_empty[stage]);
        if (s + 1 == n_steps) umma_commit(&bars->acc_done);
        if (AE_BWD_NBUF == 1 && s + 1 < n_steps) ok = issue_sp(s + 1);
      }
    }
  } else {
    // =============================== row threads ================================
    const int wg = warp >> 2;  // the two row warpgroups split every tile by 32-column chunks
    const u32 row = threadIdx.x & 127;
    const u32 lane_base = ((warp & 3) * 32) << 16;
    const int kv_idx = kv0 + (int)row;
    const bool row_valid = kv_idx < args.Skv;

    AeCustom cu;
#pragma unroll
    for (int i = 0; i < AE_MAX_CUSTOM; ++i) {
      cu.p[i] = args.custom[i];
#pragma unroll
      for (int k = 0; k < 4; ++k) cu.st[i][k] = args.custom_st[i][k];
    }

    bool ok = true;
    int s = 0;
    AeDkvStep st;
    // per-column row scales (final row scales..., delta) of a q tile, fetched by the first AE_BWD_BN threads
    float cs_next[AE_NCS];
    auto fetch_cs = [&](const AeDkvStep& w) {
      if (threadIdx.x < AE_BWD_BN) {
        const int q = w.q0 + (int)row;
        const i64 off = ((i64)b * args.Hq + w.hq) * args.Sq + (q < args.Sq ? q : args.Sq - 1);
#pragma unroll
        for (int i = 0; i < AE_NFINAL; ++i) cs_next[i] = args.final_rs[i][off];
#if AE_USES_DOOSUM
        cs_next[AE_NFINAL] = args.delta[off];
#else
        cs_next[AE_NFINAL] = 0.f;
#endif
      }
    };
    // the walk is consumed one step ahead so that the next tile's scales can be requested early
    AeDkvStep st_next;
    bool have = next_step(st_next);
    if (have) fetch_cs(st_next);
    while (have) {
      st = st_next;
      const int buf = s % AE_BWD_NBUF;
      const u32 tm_s = tmem + TM_BUF + buf * 2 * AE_BWD_BN + lane_base;
      const u32 tm_dp = tm_s + AE_BWD_BN;
      float* csb = cs + (s & 1) * (AE_BWD_BN * AE_NCS);
      // stage the per-column row scales of this q tile
      if (threadIdx.x < AE_BWD_BN) {
        // values were fetched from HBM one step ahead (below); only the shared-memory store is on the path
#pragma unroll
        for (int i = 0; i < AE_NCS; ++i) csb[i * AE_BWD_BN + row] = cs_next[i];
      }
      named_bar_sync(1, 256);
      have = next_step(st_next);
      if (have) fetch_cs(st_next);  // in flight while this tile is processed
      ok = ok && mbar_wait(&bars->sp_full[buf], (s / AE_BWD_NBUF) & 1, ctl, args.status, 36);
      tc_fence_after_sync();
      const bool tail = (st.q0 + AE_BWD_BN > args.Sq) || (kv0 + AE_KV_BM > args.Skv);
      auto chunk = [&](auto masked_tag, int c) {
        constexpr bool kMasked = decltype(masked_tag)::value;
        float sv[32], dp[32];
        tmem_ld_2xf32x32(tm_s + c * 32, tm_dp + c * 32, sv, dp);
        u32 pk[16], dk[16];
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
          // per-column row scales of four q columns: one 128-bit broadcast load per scale
          float4 cv[AE_NCS];
#pragma unroll
          for (int j = 0; j < AE_NCS; ++j) cv[j] = *(const float4*)(csb + j * AE_BWD_BN + c * 32 + i);
          float p4[4], ds4[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int col = c * 32 + i + e;
            const int q_idx = st.q0 + col;
            float fr[AE_NCS];
#pragma unroll
            for (int j = 0; j < AE_NCS; ++j) fr[j] = e == 0 ? cv[j].x : (e == 1 ? cv[j].y : (e == 2 ? cv[j].z : cv[j].w));
            const float sraw = sv[i + e];
            float p = ae_bwd_p(sraw, fr, b, st.hq, q_idx, kv_idx, cu, i + e);
            float dpv = dp[i + e];
            bool keep = true;
            if (kMasked) {
              keep = row_valid && q_idx < args.Sq;
#if AE_MASK_MODE != 0
              if (st.partial) keep = keep && ae_mask(b, st.hq, q_idx, kv_idx);
#endif
              if (!keep) {
                p = 0.f;
                dpv = 0.f;
              }
            }
            float dsv = ae_bwd_ds(sraw, dpv, p, fr, fr[AE_NFINAL], b, st.hq, q_idx, kv_idx, cu);
            if (kMasked && !keep) dsv = 0.f;
            p4[e] = p;
            ds4[e] = dsv;
          }
          pk[(i >> 1) + 0] = pack2<AE_BF16>(p4[0], p4[1]);
          pk[(i >> 1) + 1] = pack2<AE_BF16>(p4[2], p4[3]);
          dk[(i >> 1) + 0] = pack2<AE_BF16>(ds4[0], ds4[1]);
          dk[(i >> 1) + 1] = pack2<AE_BF16>(ds4[2], ds4[3]);
        }
        tmem_st16(tm_s + c * 32, pk);  // pairs go over this chunk's own first 16 columns
        tmem_st16(tm_dp + c * 32, dk);
      };
      if (st.partial || tail) {
        for (int c = wg; c < AE_BWD_BN / 32; c += 2) chunk(AeTrue{}, c);
      } else {
        for (int c = wg; c < AE_BWD_BN / 32; c += 2) chunk(AeFalse{}, c);
      }
      tc_wait_st();
      tc_fence_before_sync();
      mbar_arrive_warp(&bars->pds_full[buf]);
      ++s;
    }

    // ---- epilogue: dK / dV rows ----------------------------------------------------------
    if (s > 0) {
      ok = ok && mbar_wait(&bars->acc_done, 0, ctl, args.status, 37);
      tc_fence_after_sync();
    }
    {
      // tcgen05.ld is warp-collective: every lane runs it; only the stores are per-row
      const bool store = row_valid && ok;
      const int kv_s = store ? kv_idx : 0;
      u16* dkrow = (u16*)args.dk + (i64)b * args.dk_sb + (i64)kv_s * args.dk_ss + (i64)hk * args.dk_sh;
      u16* dvrow = (u16*)args.dv + (i64)b * args.dv_sb + (i64)kv_s * args.dv_ss + (i64)hk * args.dv_sh;
      {
        const int which = wg;  // group 0 stores dK, group 1 stores dV
        const int ncol = which ? AE_DV : AE_D;
        u16* drow = which ? dvrow : dkrow;
        const u32 tm = tmem + (which ? TM_DV : TM_DK) + lane_base;
        for (int c = 0; c < ncol / 32; ++c) {
          float r[32];
          if (s > 0) {
            tmem_ld_f32x32(tm + c * 32, r);
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
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 9) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, 512);
  }
}
