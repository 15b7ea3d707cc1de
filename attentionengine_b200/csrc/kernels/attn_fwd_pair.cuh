// Fused attention forward over CTA pairs for sm_100a: the forward of attn_fwd.cuh (which replaces the reference's
// generated kernel, attention_engine/core/template/tl_template/attn/attn_tl.py:76-174, GQA variant
// attn_gqa_tl.py:38-133) with every MMA issued for two CTAs at once (tcgen05.mma.cta_group::2).
//
// Why: the single-CTA forward is bound by the bytes an SM moves through its shared-memory datapath per kv tile, and a
// third of them are B operands (K, V) that two neighbouring CTAs both stream.  A pair shares them: each CTA loads and
// holds 64 of the 128 kv rows of a K tile and 64 of the 128 value columns of a V tile, and the tensor cores of the
// two SMs exchange the halves.
//
// A cluster of two CTAs owns two query tiles of one (batch, q-head): the CTA of rank r holds tile 2p + r, and every
// MMA covers both (256 rows).  Hand-offs between the CTAs of a pair are slow (an arrival on the other CTA's barrier,
// a commit that arrives in both), so the score tiles are not chained through them: each CTA keeps TWO score regions
// in TMEM, the scores of kv tile n go to region n & 1, and the S GEMM runs two kv tiles ahead of P V.  The row
// threads then always find the next tile's scores waiting.  Roles per CTA (320 threads):
//   warps 0-7 : row threads, two per score row (warps w and w + 4 share rows, 64 columns each; the row reductions
//               of the generated recurrence are completed between them by ae_row_xchg).  The second half keeps its P in
//               the second half of its own score columns, so no thread writes TMEM columns another thread still reads.
//   warp 8    : TMA producer of this CTA's Q tile and K / V halves.
//   warp 9    : rank 0: issues the MMAs of the pair; rank 1: forwards "my half has landed" to rank 0's barriers.
// Barriers with arrivals from the other CTA: rank 0's kv_full (its own TMA bytes + rank 1's forwarder, count 2) and
// q_peer, p_full (the row warps of both CTAs -> rank 0, count 16), and every tcgen05.commit, which arrives at the
// same barrier in both CTAs.  The issuing thread is the scarce resource (every wait costs it a few hundred clocks even
// when the phase is long complete), so K and V of a kv tile share one barrier, waited for once, before the S GEMM.
// No load is multicast: each CTA issues plain TMA loads into its own shared memory.
// TMEM columns: S region 0 | S region 1 | O (P aliases its region: first half's pairs at +0, second half's at +96).
//
// Expects the same generated prelude as attn_fwd.cuh, built with AE_RSPLIT = 2; AE_MASK_MODE 0, 1 or 3 (block lists
// take the single-CTA kernel), AE_DV == 128, AE_D 64 or 128.

#define AE_BM 128
#define AE_BN 128
#define AE_NTHREADS 320
#ifdef AE_PAIR_STAGES  // ring depth of the K / V halves (the prelude's AE_STAGES is the single-CTA kernel's)
#undef AE_STAGES
#define AE_STAGES AE_PAIR_STAGES
#endif
#if AE_MASK_MODE == 2
#error "block lists run on the single-CTA forward"
#endif
#if AE_DV != 128 || (AE_D != 64 && AE_D != 128)
#error "pair forward: value head dim 128, head dim 64 or 128"
#endif
#if AE_RSPLIT != 2
#error "pair forward: the prelude is built for two threads per score row"
#endif
#if AE_STAGES < 3
#error "the two-ahead S GEMM needs three K / V stages"
#endif

#ifdef AE_TRACE  // clock stamps of one pair's roles into the status buffer (experiments; needs a status buffer that large)
#define AE_TRP(cond, region, slot) \
  if ((cond) && (slot) < 2048) args.status[64 + (region) * 4096 + (slot)] = (u32)clock64();
#else
#define AE_TRP(cond, region, slot)
#endif
#define AE_NC (AE_BN / 2)  // score columns per row thread
#define AE_Q_BYTES (AE_BM * AE_D * 2)
#define AE_KH_BYTES (64 * AE_D * 2)   // this CTA's 64 kv rows of a K tile
#define AE_VH_BYTES (AE_BN * 64 * 2)  // this CTA's 64 value columns of a V tile
#define AE_SMEM_Q 0
#define AE_SMEM_K AE_Q_BYTES
#define AE_SMEM_V (AE_SMEM_K + AE_STAGES * AE_KH_BYTES)
#define AE_SMEM_BAR (AE_SMEM_V + AE_STAGES * AE_VH_BYTES)
#define AE_SMEM_XCH (AE_SMEM_BAR + 512)  // [phase][half][row] partial row reductions (ae_row_xchg)

struct AePairBars {
  u64 q_full, q_peer;
  u64 kv_full[AE_STAGES], kv_empty[AE_STAGES];
  u64 s_full[2], p_full[2], o_done;
  AeCtaCtl ctl;
};

extern "C" __global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(AE_NTHREADS, 1)
ae_attn_fwd_pair(const __grid_constant__ AeAttnFwdArgs args) {
  extern __shared__ u8 smem_raw[];
  u8* smem = smem_align1024(smem_raw);
  AePairBars* bars = (AePairBars*)(smem + AE_SMEM_BAR);
  AeCtaCtl* ctl = &bars->ctl;
  const u32 warp = threadIdx.x >> 5;
  const u32 lane = threadIdx.x & 31;
  const u32 rank = cluster_ctarank();

  // heaviest (latest) q tiles first: better tail under a causal mask
  const int pair = (int)(gridDim.x >> 1) - 1 - (int)(blockIdx.x >> 1);
  const int hq = blockIdx.y;
  const int b = blockIdx.z;
  const int hk = hq / (args.Hq / args.Hkv);

  // ---- kv schedule (uniform over the pair) ----------------------------------------------------------------------
  auto n_of = [&](int qt) {
    if (qt >= args.n_qt) return 0;
#if AE_MASK_MODE == 1
    return qt + 1 < args.n_kt ? qt + 1 : args.n_kt;  // rows [qt*128, qt*128+127] see kv columns [0, qt*128+127]
#else
    return args.n_kt;
#endif
  };
#ifdef AE_TRACE
  const bool tr_cta = (blockIdx.x >> 1) == 0 && blockIdx.y == 0 && blockIdx.z == 0;
  const bool tr_mma = tr_cta && rank == 0 && threadIdx.x == 9 * 32;
  const int tr_row = (tr_cta && lane == 0 && (warp == 0 || warp == 4)) ? (int)(1 + rank * 2 + (warp >> 2)) : -1;
#endif
  const int qt = pair * 2 + (int)rank;  // this CTA's q tile
  const int own_n = n_of(qt), peer_n = n_of(pair * 2 + (int)(rank ^ 1u));
  const int n_steps = own_n > peer_n ? own_n : peer_n;

  // ---- setup -----------------------------------------------------------------------------------------------------
  if (threadIdx.x == 0) {
    ctl->abort = 0;
    mbar_init(&bars->q_full, 1);
    mbar_init(&bars->q_peer, 1);
    mbar_init(&bars->o_done, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars->s_full[i], 1);
      mbar_init(&bars->p_full[i], 16);  // the eight row warps of each CTA
    }
    for (int i = 0; i < AE_STAGES; ++i) {
      mbar_init(&bars->kv_full[i], rank == 0 ? 2 : 1);  // rank 0: its own K / V halves and rank 1's "mine have landed"
      mbar_init(&bars->kv_empty[i], 1);
    }
    mbar_fence_init();
  }
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers exist before anything can arrive on them
  if (warp == 9) {
    tmem_alloc2(&ctl->tmem_base, 512);
    tmem_relinquish2();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const u32 tmem = ctl->tmem_base;
  const u32 TM_S0 = 0, TM_S1 = 128, TM_O = 256;

  if (warp == 8) {
    // =============================== TMA producer ===============================
    if (lane == 0) {
      tma_prefetch_desc(&args.tm_q);
      tma_prefetch_desc(&args.tm_k);
      tma_prefetch_desc(&args.tm_v);
      if (own_n > 0) {  // a q tile past the end is never waited for
        mbar_arrive_expect_tx(&bars->q_full, AE_Q_BYTES);
        for (int dh = 0; dh < AE_D / 64; ++dh)
          tma_load_bshd(smem + AE_SMEM_Q + dh * (AE_BM * 128), &args.tm_q, &bars->q_full, dh * 64, hq, qt * AE_BM, b);
      }
      bool ok = true;
      for (int j = 0; j < n_steps; ++j) {
        const int stage = j % AE_STAGES;
        const u32 par = ((j / AE_STAGES) & 1) ^ 1;
        if (!(ok = mbar_wait_cl(&bars->kv_empty[stage], par, ctl, args.status, 1))) break;
        mbar_arrive_expect_tx(&bars->kv_full[stage], AE_KH_BYTES + AE_VH_BYTES);
        for (int dh = 0; dh < AE_D / 64; ++dh)  // tm_k has 64-row boxes in this build
          tma_load_bshd(smem + AE_SMEM_K + stage * AE_KH_BYTES + dh * (64 * 128), &args.tm_k, &bars->kv_full[stage],
                        dh * 64, hk, j * AE_BN + (int)rank * 64, b);
        tma_load_bshd(smem + AE_SMEM_V + stage * AE_VH_BYTES, &args.tm_v, &bars->kv_full[stage], (int)rank * 64, hk,
                      j * AE_BN, b);
      }
      // the last release of every slot used has arrived in this CTA before it may retire
      for (int l = (n_steps > AE_STAGES ? n_steps - AE_STAGES : 0); l < n_steps && ok; ++l) {
        const int stage = l % AE_STAGES;
        const u32 par = (l / AE_STAGES) & 1;
        ok = mbar_wait_cl(&bars->kv_empty[stage], par, ctl, args.status, 12);
      }
    }
  } else if (warp == 9 && rank == 1) {
    // =============================== forwarder (rank 1) ==========================
    // Tells rank 0, whose thread issues the pair's MMAs, that this CTA's half of an operand has landed.
    if (lane == 0) {
      bool ok = true;
      if (own_n > 0) {
        ok = mbar_wait(&bars->q_full, 0, ctl, args.status, 20);
        if (ok) mbar_arrive_cluster(mapa_u32(smem_u32(&bars->q_peer), 0));
      }
      for (int j = 0; j < n_steps && ok; ++j) {
        const int stage = j % AE_STAGES;
        const u32 par = (j / AE_STAGES) & 1;
        ok = mbar_wait(&bars->kv_full[stage], par, ctl, args.status, 21);
        if (!ok) break;
        mbar_arrive_cluster(mapa_u32(smem_u32(&bars->kv_full[stage]), 0));
      }
    }
  } else if (warp == 9) {
    // =============================== MMA issuer (rank 0) =========================
    if (lane == 0) {
      const u32 idesc_s = umma_idesc_f16(2 * AE_BM, AE_BN, AE_BF16, 0, 0);
      const u32 idesc_o = umma_idesc_f16(2 * AE_BM, AE_DV, AE_BF16, 0, 1);
      const u64 dq0 = umma_base_k(smem_u32(smem + AE_SMEM_Q));
      const u64 dk0 = umma_base_k(smem_u32(smem + AE_SMEM_K));
      const u64 dv0 = umma_base_mn(smem_u32(smem + AE_SMEM_V), AE_BN);
      bool ok = true;
      // kv tile n: K / V stage n % AE_STAGES, score region n & 1, phase n >> 1 of that region's s_full / p_full
      auto s_into = [&](int n) {
        const int stage = n % AE_STAGES;
        const u32 par = (n / AE_STAGES) & 1;
        ok = ok && mbar_wait_cl(&bars->kv_full[stage], par, ctl, args.status, 3);  // K and V of tile n, both CTAs' halves
        if (!ok) return;
        AE_TRP(tr_mma && n >= 2, 0, (n - 2) * 8 + 4);
        const u64 db = dk0 + (u64)((stage * AE_KH_BYTES) >> 4);
        const u32 d = tmem + ((n & 1) ? TM_S1 : TM_S0);
#pragma unroll
        for (int kk = 0; kk < AE_D / 16; ++kk)
          umma_ss2(d, umma_step_k(dq0, kk, AE_BM), umma_step_k(db, kk, 64), idesc_s, kk > 0);
        umma_commit2(&bars->s_full[n & 1]);
      };
      if (n_steps > 0) {
        if (own_n > 0) ok = ok && mbar_wait(&bars->q_full, 0, ctl, args.status, 4);
        if (peer_n > 0) ok = ok && mbar_wait_cl(&bars->q_peer, 0, ctl, args.status, 8);
        tc_fence_after_sync();
      }
      for (int n = 0; n < 2 && n < n_steps && ok; ++n) s_into(n);
      for (int n = 0; n < n_steps && ok; ++n) {
        const int stage = n % AE_STAGES;  // V of tile n landed with its K (waited for before S of tile n)
        AE_TRP(tr_mma, 0, n * 8 + 0);
        ok = mbar_wait_cl(&bars->p_full[n & 1], (n >> 1) & 1, ctl, args.status, 5);
        if (!ok) break;
        AE_TRP(tr_mma, 0, n * 8 + 1);
        tc_fence_after_sync();
        {
          const u64 db = dv0 + (u64)((stage * AE_VH_BYTES) >> 4);
          const u32 a = tmem + ((n & 1) ? TM_S1 : TM_S0);
#pragma unroll
          for (int kk = 0; kk < AE_BN / 16; ++kk)  // the second half of a row's P sits at column 96 of the region
            umma_ts2(tmem + TM_O, a + kk * 8 + (kk >= AE_BN / 32 ? 64 : 0), umma_step_mn(db, kk), idesc_o,
                     (u32)(n > 0) | (kk > 0));
        }
        umma_commit2(&bars->o_done);
        umma_commit2(&bars->kv_empty[stage]);  // releases the K half too: its S GEMM was issued two tiles ago
        AE_TRP(tr_mma, 0, n * 8 + 2);
        // the region of tile n is free once its P V (just issued) has read P: MMAs run in issue order
        if (n + 2 < n_steps) s_into(n + 2);
        AE_TRP(tr_mma, 0, n * 8 + 3);
      }
    }
  } else {
    // =============================== row threads ================================
    const u32 half = warp >> 2;         // which 64 columns of the row
    const u32 row = threadIdx.x & 127;  // row inside the tile == TMEM lane
    const u32 lane_base = ((warp & 3) * 32) << 16;
    const u32 tm_o = tmem + TM_O + lane_base;
    const bool tile_valid = qt < args.n_qt;
    const int q_idx = qt * AE_BM + (int)row;
    const bool row_valid = q_idx < args.Sq;
    const int h_row = hq;
    const u32 p_remote[2] = {mapa_u32(smem_u32(&bars->p_full[0]), 0), mapa_u32(smem_u32(&bars->p_full[1]), 0)};

    AeCustom cu;
#pragma unroll
    for (int i = 0; i < AE_MAX_CUSTOM; ++i) {
      cu.p[i] = args.custom[i];
#pragma unroll
      for (int k = 0; k < 4; ++k) cu.st[i][k] = args.custom_st[i][k];
    }

    AeRow st;
    st.init();
    st.xch = (volatile float*)(smem + AE_SMEM_XCH);
    st.xme = half * 128 + row;
    st.xother = (half ^ 1u) * 128 + row;
    st.xbar = 3;
    st.xn = 256;
    st.xphase = 0;
    bool ok = true;
    for (int n = 0; n < n_steps; ++n) {
      const u32 rgn = (u32)n & 1u;
      const u32 tm_s = tmem + (rgn ? TM_S1 : TM_S0) + lane_base;
      AE_TRP(tr_row > 0, tr_row, n * 8 + 0);
      ok = ok && mbar_wait_cl(&bars->s_full[rgn], ((u32)n >> 1) & 1u, ctl, args.status, 9);
      AE_TRP(tr_row > 0, tr_row, n * 8 + 1);
      tc_fence_after_sync();
      if (n >= own_n) {
        // kv tile of the other CTA's q tile only: P = 0, the row state and O stay as they are
        u32 z[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) z[i] = 0u;
        tmem_st32(tm_s + half * 96, z);
      } else {
        float s[AE_NC];
        tmem_ld_f32x64(tm_s + half * AE_NC, s);
        AE_TRP(tr_row > 0, tr_row, n * 8 + 2);
        const int kv0 = n * AE_BN + (int)half * AE_NC;  // first kv column of this thread
        const bool tail = (n * AE_BN + AE_BN > args.Skv);
#if AE_MASK_MODE == 1
        const bool partial = n * AE_BN + AE_BN - 1 > qt * AE_BM;
#elif AE_MASK_MODE == 3
        const bool partial = true;
#else
        const bool partial = false;
#endif
        if (partial || tail) {
#pragma unroll
          for (int c = 0; c < AE_NC; ++c) {
            const int kv_idx = kv0 + c;
            bool keep = kv_idx < args.Skv;
#if AE_MASK_MODE != 0
            if (partial) keep = keep && ae_mask(b, h_row, q_idx, kv_idx);
#endif
#if AE_MASK_NEG_INF
            if (!keep) s[c] = -__int_as_float(0x7f800000);
#else
            if (kv_idx >= args.Skv) s[c] = 0.f;  // additive mask value 0: scores stay as they are
            (void)keep;
#endif
          }
        }
        const float o_scale = ae_online_fwd<AE_NC>(s, st, b, h_row, q_idx, kv0, cu);

        AE_TRP(tr_row > 0, tr_row, n * 8 + 3);
        // P -> TMEM (16-bit pairs; this thread's 32 pair columns)
        {
          u32 pk[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) pk[i] = pack2<AE_BF16>(s[2 * i], s[2 * i + 1]);
          tmem_st32(tm_s + half * 96, pk);
        }
#if !AE_O_SCALE_ONE
        // O is rescaled only when some row of the warp needs it; only then must the previous tile's P V have completed.
        // (P V of this tile is not issued before this warp's arrival below, so O is quiet meanwhile.)
        if (n > 0 && __any_sync(0xffffffffu, o_scale != 1.0f)) {
          ok = ok && mbar_wait_cl(&bars->o_done, ((u32)n - 1) & 1u, ctl, args.status, 10);
          tc_fence_after_sync();
#pragma unroll
          for (int c = (int)half; c < AE_DV / 32; c += 2) {  // the two threads of a row share its O columns
            float f[32];
            u32 r[32];
            tmem_ld_f32x32(tm_o + c * 32, f);
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(f[i] * o_scale);
            tmem_st32(tm_o + c * 32, r);
          }
        }
#endif
      }
      tc_wait_st();
      AE_TRP(tr_row > 0, tr_row, n * 8 + 4);
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        if (rank == 0)
          mbar_arrive(&bars->p_full[rgn]);
        else
          mbar_arrive_cluster(p_remote[rgn]);
      }
      AE_TRP(tr_row > 0, tr_row, n * 8 + 5);
    }

    // ---- epilogue ------------------------------------------------------------------
    // The S GEMM of the last tile was issued before the P V of the tile before it, so o_done may still be two phases
    // short here: a parity wait can only tell neighbouring phases apart, hence one wait per missing phase.
    if (n_steps > 1) ok = ok && mbar_wait_cl(&bars->o_done, ((u32)n_steps - 2) & 1u, ctl, args.status, 14);
    if (n_steps > 0) {
      ok = ok && mbar_wait_cl(&bars->o_done, ((u32)n_steps - 1) & 1u, ctl, args.status, 11);
      tc_fence_after_sync();
    }
    // tcgen05.ld is warp-collective: every lane of the warp runs it; only the stores are per-row.
    if (tile_valid) {
      const bool store = row_valid && ok;
      u16* orow = (u16*)args.o + (i64)b * args.o_sb + (i64)(store ? q_idx : 0) * args.o_ss + (i64)h_row * args.o_sh;
#pragma unroll
      for (int c = (int)half; c < AE_DV / 32; c += 2) {
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
#if AE_NFINAL > 0
      if (store && half == 0) {
        float fr[AE_NFINAL];
        ae_final_rowscales(st, fr);
#pragma unroll
        for (int i = 0; i < AE_NFINAL; ++i) args.final_rs[i][((i64)b * args.Hq + hq) * args.Sq + q_idx] = fr[i];
      }
#endif
    }
  }

  // ---- teardown --------------------------------------------------------------------
  // Both CTAs stay until the pair is done: rank 0's MMAs read rank 1's shared memory and write its TMEM, and arrivals
  // cross in both directions.
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();
  if (warp == 9) {
    tc_fence_after_sync();
    tmem_dealloc2(tmem, 512);
  }
}
