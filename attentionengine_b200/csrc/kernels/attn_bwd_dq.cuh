// Attention backward, dQ pass, for sm_100a.  Together with attn_bwd_dkv.cuh it replaces
// the reference's `flash_bwd` + `flash_bwd_post` kernels
// (attention_engine/core/template/tl_template/attn/attn_tl.py:239-415, 436-455): instead of
// one kv-stationary kernel that atomically adds fp32 dQ tiles into a staging buffer, dQ is
// produced here by a q-stationary kernel that owns its output rows, so there are no
// atomics, no fp32 dQ buffer and no conversion kernel; the price is that S and dP are
// recomputed in both passes.
//
// One CTA owns one 128-row q tile of one (batch, q-head) and streams K/V tiles of AE_BWD_BN
// (= 128) rows.  Q and dO are copied once from shared memory into TMEM as 16-bit pairs, so every MMA
// of the loop takes its A operand from TMEM and only the streamed K / V tile is read from shared
// memory (an MMA with both operands there is bound by shared-memory bandwidth).  Per kv tile s:
//   S  = Q  K^T   (TS MMA)        dP = dO V^T   (TS MMA)
//   row threads, phase A: S -> registers (S is released at once); T = score_mod(S); P = OnlineFunc.forward(T), kept
//                in registers;
//                phase B: dT = OnlineFunc.backward(dP, P); dS = score_mod'(S) dT -> 16-bit pairs over dP
//   dQ += dS K    (TS MMA, K tile read MN-major)
// TMEM columns: Q | dO | S | dP | dQ.  The tensor pipe executes MMAs in issue order; the issue order is
//   S_{s+1} (after phase A of s has read S_s) , dQ_s (after phase B of s) , dP_{s+1}
// so the row threads run phase B of s under S_{s+1} and phase A of s+1 under dQ_s / dP_{s+1}.
// Roles: warps 0-3 and 4-7 row threads (thread = q row = TMEM lane; the two groups take alternate
// 32-column chunks of every tile), warp 8 TMA producer, warp 9 MMA issuer.  The 16-bit dS pairs of a
// chunk are written over the first 16 columns of that chunk of dP, so a group only overwrites what it has read.
// Shared memory: AE_DQ_KSTAGES slots for K and AE_DQ_VSTAGES for V (3 each by default); the last slot of each is
// where Q and dO land first and becomes a ring slot once they have been copied to TMEM.  With equal depths K and V
// of a step share one barrier pair; otherwise a V slot is released after the dP GEMM and a K slot after the dQ GEMM.

#define AE_BM 128
#define AE_NTHREADS_BWD 320
// Row warps -> MMA warp hand-offs (S read, dS written) through named barriers instead of mbarriers.  The MMA warp
// stops syncing when it aborts; the row warps never block on these barriers, and they arrive in every iteration.
#ifndef AE_DQ_NAMED_BAR
#define AE_DQ_NAMED_BAR 1
#endif
// Optional phase trace of CTA (0, 0, 0): 32-bit clock stamps behind the status word (bring-up / tuning only).
#ifdef AE_TRACE
#define AE_TR(cond, region, slot) \
  if (trace_on && (cond) && (slot) < 2048) args.status[64 + (region) * 4096 + (slot)] = (u32)clock64();
#else
#define AE_TR(cond, region, slot)
#endif
#define AE_NSUB (128 / AE_BWD_BN)

#define AE_DQ_K_BYTES (AE_BWD_BN * AE_D * 2)
#define AE_DQ_V_BYTES (AE_BWD_BN * AE_DV * 2)
#define AE_DQ_SMEM_K 0
#define AE_DQ_SMEM_V (AE_DQ_KSTAGES * AE_DQ_K_BYTES)
#define AE_DQ_SMEM_Q (AE_DQ_SMEM_K + (AE_DQ_KSTAGES - 1) * AE_DQ_K_BYTES)   // = last K slot
#define AE_DQ_SMEM_DO (AE_DQ_SMEM_V + (AE_DQ_VSTAGES - 1) * AE_DQ_V_BYTES)  // = last V slot
#define AE_DQ_SMEM_BAR (AE_DQ_SMEM_V + AE_DQ_VSTAGES * AE_DQ_V_BYTES)
#if AE_BWD_BN != 128
#error "the dQ pass streams 128-row K / V tiles"
#endif

struct AeDqBars {
  u64 qdo_full;   // Q and dO landed in shared memory
  u64 qdo_tmem;   // ... and were copied to TMEM (their shared-memory slots are free)
  u64 k_full[AE_DQ_KSTAGES];
  u64 k_empty[AE_DQ_KSTAGES];
  u64 v_full[AE_DQ_VSTAGES];
  u64 v_empty[AE_DQ_VSTAGES];
  u64 s_full, dp_full;  // S / dP of a step are in TMEM
  u64 a_done, ds_full;  // the row threads have read S / written dS
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
  // a count outside [0, n_kt] would walk past the list: such a tile gets an empty walk and status 0x400, as in the forward
  int n_list = args.blk_cnt[((i64)b * args.Hq + hq) * args.n_qt + qt];
  if (n_list < 0 || n_list > args.n_kt) {
    if (threadIdx.x == 0 && args.status) atomicCAS(args.status, 0u, 0x400u);
    n_list = 0;
  }
  const int* list = args.blk_idx + (((i64)b * args.Hq + hq) * args.n_qt + qt) * (i64)args.n_kt;
  n_steps = n_list * AE_NSUB;
#else
  n_steps = n_kt_bn;
#endif
  // step -> (first kv column, needs element mask).  dQ is a plain sum over the kv tiles, so every CTA walks them
  // from its own starting point (AE_DQ_ROTATE): CTAs that run together then read different tiles at any one time
  // instead of all asking L2 for the same lines.
#ifndef AE_DQ_ROTATE
#define AE_DQ_ROTATE 1
#endif
#if AE_DQ_ROTATE
  const int rot = n_steps > 0 ? (int)(((u32)qt * 2654435761u + (u32)hq * 40503u + (u32)b * 9973u) >> 8) % n_steps : 0;
#else
  const int rot = 0;
#endif
  auto step_info = [&](int s, int& kv0, bool& partial) {
    s += rot;
    if (s >= n_steps) s -= n_steps;
#if AE_MASK_MODE == 2
    const int e = list[s / AE_NSUB];
    int kt = e & 0x3fffffff;
    if (kt >= args.n_kt) {  // an entry outside the tile grid: keep every access in range, report status 0x400
      if (args.status) atomicCAS(args.status, 0u, 0x400u);
      kt = args.n_kt - 1;
    }
    kv0 = kt * 128 + (s % AE_NSUB) * AE_BWD_BN;
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
    mbar_init(&bars->qdo_tmem, 8);
    mbar_init(&bars->dq_done, 1);
    for (int i = 0; i < AE_DQ_KSTAGES; ++i) {
      mbar_init(&bars->k_full[i], 1);
      mbar_init(&bars->k_empty[i], 1);
    }
    for (int i = 0; i < AE_DQ_VSTAGES; ++i) {
      mbar_init(&bars->v_full[i], 1);
      mbar_init(&bars->v_empty[i], 1);
    }
    mbar_init(&bars->s_full, 1);
    mbar_init(&bars->dp_full, 1);
    mbar_init(&bars->a_done, 8);
    mbar_init(&bars->ds_full, 8);
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
  const u32 TM_Q = 0, TM_DO = AE_D / 2, TM_S = (AE_D + AE_DV) / 2, TM_DP = TM_S + AE_BWD_BN, TM_DQ = TM_DP + AE_BWD_BN;

  if (warp == 8) {
    // =============================== TMA producer ===============================
    if (lane == 0 && n_steps > 0) {
      tma_prefetch_desc(&args.tm_q);
      tma_prefetch_desc(&args.tm_k);
      tma_prefetch_desc(&args.tm_v);
      tma_prefetch_desc(&args.tm_do);
      mbar_arrive_expect_tx(&bars->qdo_full, AE_BM * (AE_D + AE_DV) * 2);
      for (int dh = 0; dh < AE_D / 64; ++dh)
        tma_load_bshd(smem + AE_DQ_SMEM_Q + dh * (AE_BM * 128), &args.tm_q, &bars->qdo_full, dh * 64, hq, q0, b);
      for (int dh = 0; dh < AE_DV / 64; ++dh)
        tma_load_bshd(smem + AE_DQ_SMEM_DO + dh * (AE_BM * 128), &args.tm_do, &bars->qdo_full, dh * 64, hq, q0, b);
      for (int s = 0; s < n_steps; ++s) {
        int kv0;
        bool partial;
        step_info(s, kv0, partial);
        const int ks = s % AE_DQ_KSTAGES, vs = s % AE_DQ_VSTAGES;
        // the last slots hold Q / dO until the row threads have moved them to TMEM
        if ((s == AE_DQ_KSTAGES - 1 || s == AE_DQ_VSTAGES - 1) && !mbar_wait(&bars->qdo_tmem, 0, ctl, args.status, 20)) break;
        AE_TR(true, 3, s * 8 + 0)
        if (!mbar_wait(&bars->k_empty[ks], ((s / AE_DQ_KSTAGES) & 1) ^ 1, ctl, args.status, 21)) break;
        AE_TR(true, 3, s * 8 + 1)
#if AE_DQ_KSTAGES == AE_DQ_VSTAGES
        // equal ring depths: K and V of a step share one barrier pair, which saves the MMA warp a wait per step
        // (a wait costs it 200 - 400 clk even when the data is there)
        mbar_arrive_expect_tx(&bars->k_full[ks], AE_DQ_K_BYTES + AE_DQ_V_BYTES);
#else
        mbar_arrive_expect_tx(&bars->k_full[ks], AE_DQ_K_BYTES);
#endif
        for (int dh = 0; dh < AE_D / 64; ++dh)
          tma_load_bshd(smem + AE_DQ_SMEM_K + ks * AE_DQ_K_BYTES + dh * (AE_BWD_BN * 128), &args.tm_k,
                      &bars->k_full[ks], dh * 64, hk, kv0, b);
        AE_TR(true, 3, s * 8 + 2)
#if AE_DQ_KSTAGES == AE_DQ_VSTAGES
        u64* vbar = &bars->k_full[ks];
#else
        if (!mbar_wait(&bars->v_empty[vs], ((s / AE_DQ_VSTAGES) & 1) ^ 1, ctl, args.status, 22)) break;
        u64* vbar = &bars->v_full[vs];
        mbar_arrive_expect_tx(vbar, AE_DQ_V_BYTES);
#endif
        AE_TR(true, 3, s * 8 + 3)
        for (int dh = 0; dh < AE_DV / 64; ++dh)
          tma_load_bshd(smem + AE_DQ_SMEM_V + vs * AE_DQ_V_BYTES + dh * (AE_BWD_BN * 128), &args.tm_v, vbar, dh * 64, hk,
                      kv0, b);
      }
    }
  } else if (warp == 9) {
    // =============================== MMA issuer =================================
    if (n_steps > 0) {  // all 32 lanes run the control flow; single MMAs and commits are issued by an elected lane
      const u32 idesc_s = umma_idesc_f16(AE_BM, AE_BWD_BN, AE_BF16, 0, 0);
      const u32 idesc_dq = umma_idesc_f16(AE_BM, AE_D, AE_BF16, 0, 1);
      const u32 k_addr = smem_u32(smem + AE_DQ_SMEM_K);
      const u32 v_addr = smem_u32(smem + AE_DQ_SMEM_V);
      const u64 dk0 = umma_base_k(k_addr), dv0 = umma_base_k(v_addr);
      const u64 dkmn0 = umma_base_mn(k_addr, AE_BWD_BN);

      auto issue_s = [&](int s) -> bool {  // S_s = Q K_s^T
        const int stage = s % AE_DQ_KSTAGES;
        // (no tcgen05 fence here: the operands waited for are in shared memory; the TMEM hazard of this GEMM, the row
        // threads' reads of the previous S, was fenced with the a_done wait)
        if (!mbar_wait_w(&bars->k_full[stage], (s / AE_DQ_KSTAGES) & 1, ctl, args.status, 24)) return false;
        AE_TR(s > 0, 0, (s - 1) * 8 + 6)
        AE_TR(s > 0, 0, (s - 1) * 8 + 7)
        const u64 dkk = dk0 + (u64)((stage * AE_DQ_K_BYTES) >> 4);
#pragma unroll
        for (int kk = 0; kk < AE_D / 16; ++kk)
          umma_ts_w(tmem + TM_S, tmem + TM_Q + kk * 8, umma_step_k(dkk, kk, AE_BWD_BN), idesc_s, kk > 0);
        umma_commit_w(&bars->s_full);
        return true;
      };
      auto issue_dp = [&](int s) -> bool {  // dP_s = dO V_s^T
        const int stage = s % AE_DQ_VSTAGES;
#if AE_DQ_KSTAGES != AE_DQ_VSTAGES
        if (!mbar_wait_w(&bars->v_full[stage], (s / AE_DQ_VSTAGES) & 1, ctl, args.status, 25)) return false;
        tc_fence_after_sync();
#endif
        const u64 dvv = dv0 + (u64)((stage * AE_DQ_V_BYTES) >> 4);
#pragma unroll
        for (int kk = 0; kk < AE_DV / 16; ++kk)
          umma_ts_w(tmem + TM_DP, tmem + TM_DO + kk * 8, umma_step_k(dvv, kk, AE_BWD_BN), idesc_s, kk > 0);
        umma_commit_w(&bars->dp_full);
#if AE_DQ_KSTAGES != AE_DQ_VSTAGES
        umma_commit_w(&bars->v_empty[stage]);
#endif
        return true;
      };

      bool ok = mbar_wait_w(&bars->qdo_tmem, 0, ctl, args.status, 23);
      tc_fence_after_sync();
      if (ok) ok = issue_s(0);
      if (ok) ok = issue_dp(0);
      for (int s = 0; s < n_steps && ok; ++s) {
        const int stage = s % AE_DQ_KSTAGES;
        const u32 par = s & 1;
        AE_TR(true, 0, s * 8 + 0)
        // the next S goes over S_s once the row threads have read it
#if AE_DQ_NAMED_BAR
        named_bar_sync(1, 256 + 32);  // the 8 row warps arrive in every iteration, whatever happened: no time-out needed
#else
        ok = mbar_wait_w(&bars->a_done, par, ctl, args.status, 26);
        if (!ok) break;
#endif
        tc_fence_after_sync();
        AE_TR(true, 0, s * 8 + 1)
        if (s + 1 < n_steps) ok = issue_s(s + 1);
        if (!ok) break;
        AE_TR(true, 0, s * 8 + 2)
        // dQ += dS_s K_s, then the next dP goes over dS_s
#if AE_DQ_NAMED_BAR
        named_bar_sync(2, 256 + 32);
#else
        ok = mbar_wait_w(&bars->ds_full, par, ctl, args.status, 29);
        if (!ok) break;
#endif
        tc_fence_after_sync();
        AE_TR(true, 0, s * 8 + 3)
        const u64 dkm = dkmn0 + (u64)((stage * AE_DQ_K_BYTES) >> 4);
#pragma unroll
        for (int kk = 0; kk < AE_BWD_BN / 16; ++kk)
          umma_ts_w(tmem + TM_DQ, tmem + TM_DP + (kk >> 1) * 32 + (kk & 1) * 8, umma_step_mn(dkm, kk), idesc_dq,
                    (s > 0) | (kk > 0));
        umma_commit_w(&bars->k_empty[stage]);
        if (s + 1 == n_steps) umma_commit_w(&bars->dq_done);
        AE_TR(true, 0, s * 8 + 4)
        if (s + 1 < n_steps) ok = issue_dp(s + 1);
        AE_TR(true, 0, s * 8 + 5)
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
    bool ok = true;

    // ---- Q (group 0) and dO (group 1) rows: shared memory -> TMEM, once ------------------------
    if (n_steps > 0) {
      ok = mbar_wait(&bars->qdo_full, 0, ctl, args.status, 19);
      const u8* src = smem + (wg ? AE_DQ_SMEM_DO : AE_DQ_SMEM_Q);
      const int nblk = (wg ? AE_DV : AE_D) / 64;
      const u32 tm = tmem + (wg ? TM_DO : TM_Q) + lane_base;
      for (int blk = 0; blk < nblk; ++blk) {
        u32 w[32];
#pragma unroll
        for (int ch = 0; ch < 8; ++ch) {
          const uint4 v = *(const uint4*)(src + blk * (AE_BM * 128) + swz128(row, ch));
          w[ch * 4 + 0] = v.x;
          w[ch * 4 + 1] = v.y;
          w[ch * 4 + 2] = v.z;
          w[ch * 4 + 3] = v.w;
        }
        tmem_st32(tm + blk * 32, w);  // column c of a row holds its elements 2c, 2c + 1: the A-operand layout
      }
      tc_wait_st();
      tc_fence_before_sync();
      mbar_arrive_warp(&bars->qdo_tmem);
    }

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

    constexpr int NCH = AE_BWD_BN / 64;  // 32-column chunks per group and tile
    const u32 tm_s = tmem + TM_S + lane_base;
    const u32 tm_dp = tmem + TM_DP + lane_base;
    for (int s = 0; s < n_steps; ++s) {
      int kv0;
      bool partial;
      step_info(s, kv0, partial);
      const bool masked = partial || (kv0 + AE_BWD_BN > args.Skv);
      float pkeep[NCH][32];
#if AE_DS_USES_S
      float skeep[NCH][32];
#endif
      auto keep_of = [&](int kv_idx) -> bool {
        bool keep = kv_idx < args.Skv;
#if AE_MASK_MODE != 0
        if (partial) keep = keep && ae_mask(b, hq, q_idx, kv_idx);
#endif
        return keep;
      };

      // ---- phase A: P from S -------------------------------------------------------------------
      AE_TR((warp & 3) == 0, 1 + wg, s * 8 + 0)
      ok = ok && mbar_wait(&bars->s_full, s & 1, ctl, args.status, 27);
      tc_fence_after_sync();
      AE_TR((warp & 3) == 0, 1 + wg, s * 8 + 1)
      // S_s goes to registers first and is released at once (the next S GEMM then runs under this tile's row work);
      // P is computed from the registers afterwards.
      static_assert(NCH == 2, "phase A loads its two chunks with one paired TMEM load");
      float sv[NCH][32];
      tmem_ld_2xf32x32(tm_s + wg * 32, tm_s + (wg + 2) * 32, sv[0], sv[1]);
      tc_fence_before_sync();
#if AE_DQ_NAMED_BAR
      named_bar_arrive(1, 256 + 32);  // S_s has been read: the next S may overwrite it
#else
      mbar_arrive_warp(&bars->a_done);
#endif
      AE_TR((warp & 3) == 0, 1 + wg, s * 8 + 2)
      auto phase_a = [&](auto masked_tag) {
        constexpr bool kMasked = decltype(masked_tag)::value;
#pragma unroll
        for (int ci = 0; ci < NCH; ++ci) {
          const int c = wg + 2 * ci;
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int kv_idx = kv0 + c * 32 + i;
            float p = ae_bwd_p(sv[ci][i], fr, b, hq, q_idx, kv_idx, cu, i);
            if (kMasked && !keep_of(kv_idx)) p = 0.f;
            pkeep[ci][i] = p;
#if AE_DS_USES_S
            skeep[ci][i] = sv[ci][i];
#endif
          }
        }
      };
      if (masked) phase_a(AeTrue{}); else phase_a(AeFalse{});

      // ---- phase B: dS from dP and the P kept in registers ----------------------------------------
      ok = ok && mbar_wait(&bars->dp_full, s & 1, ctl, args.status, 18);
      tc_fence_after_sync();
      AE_TR((warp & 3) == 0, 1 + wg, s * 8 + 3)
      auto phase_b = [&](auto masked_tag) {
        constexpr bool kMasked = decltype(masked_tag)::value;
#pragma unroll
        for (int ci = 0; ci < NCH; ++ci) {
          const int c = wg + 2 * ci;
          float dp[32];
          tmem_ld_f32x32(tm_dp + c * 32, dp);
          u32 pk[16];
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            float ds2[2];
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              const int kv_idx = kv0 + c * 32 + i + e;
#if AE_DS_USES_S
              const float sraw = skeep[ci][i + e];
#else
              const float sraw = 0.f;
#endif
              bool keep = true;
              if (kMasked) keep = keep_of(kv_idx);
              float dsv = ae_bwd_ds(sraw, keep ? dp[i + e] : 0.f, pkeep[ci][i + e], fr, delta, b, hq, q_idx, kv_idx, cu);
              if (kMasked && !keep) dsv = 0.f;
              ds2[e] = dsv;
            }
            pk[i >> 1] = pack2<AE_BF16>(ds2[0], ds2[1]);
          }
          tmem_st16(tm_dp + c * 32, pk);  // pairs go over this chunk's own first 16 columns
        }
      };
      if (masked) phase_b(AeTrue{}); else phase_b(AeFalse{});
      AE_TR((warp & 3) == 0, 1 + wg, s * 8 + 4)
      tc_wait_st();
      tc_fence_before_sync();
#if AE_DQ_NAMED_BAR
      named_bar_arrive(2, 256 + 32);
#else
      mbar_arrive_warp(&bars->ds_full);
#endif
      AE_TR((warp & 3) == 0, 1 + wg, s * 8 + 5)
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
