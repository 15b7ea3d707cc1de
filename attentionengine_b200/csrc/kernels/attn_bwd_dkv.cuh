// Attention backward, dK/dV pass, for sm_100a (see attn_bwd_dq.cuh for how the two passes
// split the reference's `flash_bwd`, attn_tl.py:239-415; GQA variant attn_gqa_tl.py:190-350).
//
// One CTA owns one 128-row kv tile of one (batch, kv-head) and streams the Q / dO tiles
// (AE_BWD_BN rows) of every q-head of that kv-head's group, so dK / dV of a group are summed
// in the CTA's own TMEM accumulators: no atomics (the reference adds half-precision atomics
// across the group, attn_gqa_tl.py:345-348).  Per q tile, with rows = kv and columns = q:
//   S^T  = K  Q^T  (SS MMA)      dP^T = V dO^T  (SS MMA)
//   row threads, phase A: P^T = forward(score_mod(S^T)), written over S^T as 16-bit pairs and kept in
//                registers; phase B: dS^T = score_mod'(S^T) * backward(dP^T, P^T), written over dP^T
//                (per-column lse / delta come from shared memory)
//   dV += P^T dO   (TS MMA, dO tile read MN-major)     dK += dS^T Q  (TS MMA, Q tile read MN-major)
// TMEM columns: dK | dV | S^T | dP^T.  The tensor pipe executes MMAs in issue order, so one S^T and one
// dP^T region are enough to keep it busy: the issue order per q tile s is
//   dV_s (after phase A of s) , S^T_{s+1} , dK_s (after phase B of s) , dP^T_{s+1}
// and the row threads run phase B of s under dV_s / S^T_{s+1} and phase A of s+1 under dK_s / dP^T_{s+1}.
// Roles: AE_KV_NWG row warpgroups (thread = kv row = TMEM lane; the groups take alternate 32-column chunks
// of every tile), then one producer warp (TMA loads of Q / dO by one lane, per-column row scales by all
// lanes) and one MMA-issuing warp.  The 16-bit pairs of a chunk are written over the first 16 columns of
// that chunk, so a group only overwrites what it has read.
// Expects AE_BWD_BN (q rows per tile), AE_KV_QSTAGES / AE_KV_DOSTAGES (ring depths), AE_KV_NWG (2 or 4),
// AE_KV_TS (1: K and V resident in TMEM, needs AE_BWD_BN = 64 at head dim 128 for the TMEM budget).

#define AE_KV_BM 128
// Optional phase trace of CTA (0, 0, 0): 32-bit clock stamps behind the status word (bring-up / tuning only).
#ifdef AE_TRACE
#define AE_TRK(cond, region, slot) \
  if (trace_on && (cond) && (slot) < 2048) args.status[64 + (region) * 4096 + (slot)] = (u32)clock64();
#else
#define AE_TRK(cond, region, slot)
#endif
#define AE_NSUBQ (128 / AE_BWD_BN)
#define AE_NCS (AE_NFINAL + 1)

#define AE_KV_K_BYTES (AE_KV_BM * AE_D * 2)
#define AE_KV_V_BYTES (AE_KV_BM * AE_DV * 2)
#define AE_KV_Q_BYTES (AE_BWD_BN * AE_D * 2)
#define AE_KV_DO_BYTES (AE_BWD_BN * AE_DV * 2)
#ifndef AE_KV_TS
#define AE_KV_TS 0
#endif
#if AE_KV_TS
// K and V go to TMEM once (S^T and dP^T become TS MMAs, which leave the shared-memory bandwidth to the streamed
// tiles); they land in the last ring slots of Q / dO, which join the rings after the copy.
#define AE_KV_SLOTS (AE_KV_BM / AE_BWD_BN)  // ring slots one resident tile covers
#define AE_KV_SMEM_Q 0
#define AE_KV_SMEM_DO (AE_KV_QSTAGES * AE_KV_Q_BYTES)
#define AE_KV_SMEM_K (AE_KV_SMEM_Q + (AE_KV_QSTAGES - AE_KV_SLOTS) * AE_KV_Q_BYTES)
#define AE_KV_SMEM_V (AE_KV_SMEM_DO + (AE_KV_DOSTAGES - AE_KV_SLOTS) * AE_KV_DO_BYTES)
#else
#define AE_KV_SMEM_K 0
#define AE_KV_SMEM_V (AE_KV_K_BYTES)
#define AE_KV_SMEM_Q (AE_KV_SMEM_V + AE_KV_V_BYTES)
#define AE_KV_SMEM_DO (AE_KV_SMEM_Q + AE_KV_QSTAGES * AE_KV_Q_BYTES)
#endif
#define AE_KV_SMEM_CS (AE_KV_SMEM_DO + AE_KV_DOSTAGES * AE_KV_DO_BYTES)
#define AE_KV_CS_BYTES (2 * AE_BWD_BN * AE_NCS * 4)
// equal ring depths: Q and dO of a step share one barrier pair (one wait less per step for the MMA warp)
#define AE_KV_ONE_BAR (AE_KV_QSTAGES == AE_KV_DOSTAGES && !AE_KV_TS)
// Row warps -> MMA warp hand-offs (P^T written, dS^T written) through named barriers instead of mbarriers: the MMA
// warp stops syncing when it aborts, the row warps never block on them and arrive in every iteration.
#ifndef AE_KV_NAMED_BAR
#define AE_KV_NAMED_BAR 1
#endif
#define AE_KV_NROW (AE_KV_NWG * 128)
#define AE_KV_NTHREADS (AE_KV_NROW + 64)
#define AE_KV_SMEM_BAR (AE_KV_SMEM_CS + ((AE_KV_CS_BYTES + 15) / 16) * 16)

struct AeDkvBars {
  u64 kv_full;
  u64 kv_tmem;  // K and V were copied to TMEM (AE_KV_TS)
  u64 q_full[AE_KV_QSTAGES];
  u64 cs_full[2], cs_empty[2];  // per-column row scales of a q tile (two slots)
  u64 q_empty[AE_KV_QSTAGES];
  u64 do_full[AE_KV_DOSTAGES];
  u64 do_empty[AE_KV_DOSTAGES];
  u64 s_full, dp_full;  // S^T / dP^T of a step are in TMEM
  u64 p_full, ds_full;  // the row threads have written P^T / dS^T
  u64 acc_done;
  AeCtaCtl ctl;
};

struct AeDkvStep {
  int hq;       // q head
  int q0;       // first q row of the tile
  bool partial; // needs the element-wise mask
};

extern "C" __global__ void __launch_bounds__(AE_KV_NTHREADS, 1)
ae_attn_bwd_dkv(const __grid_constant__ AeAttnBwdArgs args) {
  extern __shared__ u8 smem_raw[];
#if AE_KV_ALIGN_SLACK
  u8* smem = smem_align1024(smem_raw);
#else
  // the carve-up fills the CTA's shared memory: the launch gave no slack, so the base must be aligned already
  u8* smem = smem_raw;
  if (smem_u32(smem_raw) & 1023u) {
    if (threadIdx.x == 0 && args.status) atomicCAS(args.status, 0u, 0x200u);
    return;
  }
#endif
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
#ifdef AE_TRACE
  const bool trace_on = blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && (threadIdx.x & 31) == 0;
#endif

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
      int n = args.blkT_cnt[base];
      if (n < 0 || n > args.n_qt) {  // a count that would walk past the list: empty walk, status 0x400
        if (args.status) atomicCAS(args.status, 0u, 0x400u);
        n = 0;
      }
      if (walk.e < n) {
        const int ent = args.blkT_idx[base * args.n_qt + walk.e];
        st.hq = hq;
        int qt = ent & 0x3fffffff;
        if (qt >= args.n_qt) {  // an entry outside the tile grid: keep every access in range, report status 0x400
          if (args.status) atomicCAS(args.status, 0u, 0x400u);
          qt = args.n_qt - 1;
        }
        st.q0 = qt * 128 + walk.sub * AE_BWD_BN;
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
    mbar_init(&bars->kv_tmem, 8);
    mbar_init(&bars->acc_done, 1);
    for (int i = 0; i < AE_KV_QSTAGES; ++i) {
      mbar_init(&bars->q_full[i], 1);
      mbar_init(&bars->q_empty[i], 1);
    }
    for (int i = 0; i < AE_KV_DOSTAGES; ++i) {
      mbar_init(&bars->do_full[i], 1);
      mbar_init(&bars->do_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars->cs_full[i], 32);
      mbar_init(&bars->cs_empty[i], AE_KV_NWG * 4);
    }
    mbar_init(&bars->s_full, 1);
    mbar_init(&bars->dp_full, 1);
    mbar_init(&bars->p_full, AE_KV_NWG * 4);
    mbar_init(&bars->ds_full, AE_KV_NWG * 4);
    mbar_fence_init();
  }
  if (warp == AE_KV_NWG * 4 + 1) {
    tmem_alloc(&ctl->tmem_base, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const u32 tmem = ctl->tmem_base;
#if AE_KV_TS
  const u32 TM_K = 0, TM_V = AE_D / 2, TM_DK = (AE_D + AE_DV) / 2;
#else
  const u32 TM_DK = 0;
#endif
  const u32 TM_DV = TM_DK + AE_D, TM_S = TM_DV + AE_DV, TM_DP = TM_S + AE_BWD_BN;

  if (warp == AE_KV_NWG * 4) {
    // =============================== producer ====================================
    // All lanes walk the schedule; lane 0 issues the TMA loads, every lane fetches the row scales of four q columns.
    if (lane == 0) {
      tma_prefetch_desc(&args.tm_q);
      tma_prefetch_desc(&args.tm_k);
      tma_prefetch_desc(&args.tm_v);
      tma_prefetch_desc(&args.tm_do);
      mbar_arrive_expect_tx(&bars->kv_full, AE_KV_K_BYTES + AE_KV_V_BYTES);
      for (int dh = 0; dh < AE_D / 64; ++dh)
        tma_load_bshd(smem + AE_KV_SMEM_K + dh * (AE_KV_BM * 128), &args.tm_k, &bars->kv_full, dh * 64, hk, kv0, b);
      for (int dh = 0; dh < AE_DV / 64; ++dh)
        tma_load_bshd(smem + AE_KV_SMEM_V + dh * (AE_KV_BM * 128), &args.tm_v, &bars->kv_full, dh * 64, hk, kv0, b);
    }
    AeDkvStep st;
    int s = 0;
    while (next_step(st)) {
      const int sq = s % AE_KV_QSTAGES, sd = s % AE_KV_DOSTAGES;
#if AE_KV_TS
      if (s == AE_KV_QSTAGES - AE_KV_SLOTS && !mbar_wait_w(&bars->kv_tmem, 0, ctl, args.status, 43)) break;
#endif
      if (!mbar_wait_w(&bars->q_empty[sq], ((s / AE_KV_QSTAGES) & 1) ^ 1, ctl, args.status, 31)) break;
      if (lane == 0) {
        mbar_arrive_expect_tx(&bars->q_full[sq], AE_KV_ONE_BAR ? AE_KV_Q_BYTES + AE_KV_DO_BYTES : AE_KV_Q_BYTES);
        for (int dh = 0; dh < AE_D / 64; ++dh)
          tma_load_bshd(smem + AE_KV_SMEM_Q + sq * AE_KV_Q_BYTES + dh * (AE_BWD_BN * 128), &args.tm_q, &bars->q_full[sq],
                      dh * 64, st.hq, st.q0, b);
      }
      {
        if (!mbar_wait_w(&bars->cs_empty[s & 1], ((s >> 1) & 1) ^ 1, ctl, args.status, 42)) break;
        float* csb = cs + (s & 1) * (AE_BWD_BN * AE_NCS);
        const i64 base = ((i64)b * args.Hq + st.hq) * args.Sq;
#pragma unroll
        for (int j = 0; j < AE_BWD_BN / 32; ++j) {
          const int col = j * 32 + (int)lane;
          const int q = st.q0 + col;
          const i64 off = base + (q < args.Sq ? q : args.Sq - 1);
#pragma unroll
          for (int i = 0; i < AE_NFINAL; ++i) csb[i * AE_BWD_BN + col] = args.final_rs[i][off];
#if AE_USES_DOOSUM
          csb[AE_NFINAL * AE_BWD_BN + col] = args.delta[off];
#else
          csb[AE_NFINAL * AE_BWD_BN + col] = 0.f;
#endif
        }
        mbar_arrive(&bars->cs_full[s & 1]);
      }
#if AE_KV_TS
      if (s == AE_KV_DOSTAGES - AE_KV_SLOTS && !mbar_wait_w(&bars->kv_tmem, 0, ctl, args.status, 44)) break;
#endif
#if AE_KV_ONE_BAR
      if (lane == 0) {  // the slot pair was released by q_empty; dO completes the same barrier as Q
        for (int dh = 0; dh < AE_DV / 64; ++dh)
          tma_load_bshd(smem + AE_KV_SMEM_DO + sd * AE_KV_DO_BYTES + dh * (AE_BWD_BN * 128), &args.tm_do,
                      &bars->q_full[sq], dh * 64, st.hq, st.q0, b);
      }
#else
      if (!mbar_wait_w(&bars->do_empty[sd], ((s / AE_KV_DOSTAGES) & 1) ^ 1, ctl, args.status, 38)) break;
      if (lane == 0) {
        mbar_arrive_expect_tx(&bars->do_full[sd], AE_KV_DO_BYTES);
        for (int dh = 0; dh < AE_DV / 64; ++dh)
          tma_load_bshd(smem + AE_KV_SMEM_DO + sd * AE_KV_DO_BYTES + dh * (AE_BWD_BN * 128), &args.tm_do,
                      &bars->do_full[sd], dh * 64, st.hq, st.q0, b);
      }
#endif
      ++s;
    }
  } else if (warp == AE_KV_NWG * 4 + 1) {
    // =============================== MMA issuer =================================
    {  // all 32 lanes run the control flow; single MMAs and commits are issued by an elected lane
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
      auto issue_s = [&](int s) -> bool {  // S^T_s = K Q_s^T
        const int stage = s % AE_KV_QSTAGES;
        // (no tcgen05 fence after a wait for shared-memory operands: the TMEM hazards of this GEMM were fenced with
        // the p_full / ds_full waits that precede it in program order)
        if (!mbar_wait_w(&bars->q_full[stage], (s / AE_KV_QSTAGES) & 1, ctl, args.status, 32)) return false;
        const u64 dqq = dq0 + (u64)((stage * AE_KV_Q_BYTES) >> 4);
#pragma unroll
        for (int kk = 0; kk < AE_D / 16; ++kk)
#if AE_KV_TS
          umma_ts_w(tmem + TM_S, tmem + TM_K + kk * 8, umma_step_k(dqq, kk, AE_BWD_BN), idesc_s, kk > 0);
#else
          umma_ss_w(tmem + TM_S, umma_step_k(dk0, kk, AE_KV_BM), umma_step_k(dqq, kk, AE_BWD_BN), idesc_s, kk > 0);
#endif
        umma_commit_w(&bars->s_full);
        return true;
      };
      auto issue_dp = [&](int s) -> bool {  // dP^T_s = V dO_s^T
        const int stage = s % AE_KV_DOSTAGES;
#if !AE_KV_ONE_BAR
        if (!mbar_wait_w(&bars->do_full[stage], (s / AE_KV_DOSTAGES) & 1, ctl, args.status, 33)) return false;
#endif
        const u64 ddd = ddo0 + (u64)((stage * AE_KV_DO_BYTES) >> 4);
#pragma unroll
        for (int kk = 0; kk < AE_DV / 16; ++kk)
#if AE_KV_TS
          umma_ts_w(tmem + TM_DP, tmem + TM_V + kk * 8, umma_step_k(ddd, kk, AE_BWD_BN), idesc_s, kk > 0);
#else
          umma_ss_w(tmem + TM_DP, umma_step_k(dv0, kk, AE_KV_BM), umma_step_k(ddd, kk, AE_BWD_BN), idesc_s, kk > 0);
#endif
        umma_commit_w(&bars->dp_full);
        return true;
      };

      // count the steps first (the walk is cheap and identical in every role)
      int n_steps = 0;
      {
        AeDkvStep st;
        while (next_step(st)) ++n_steps;
      }
#if AE_KV_TS
      bool ok = n_steps > 0 && mbar_wait_w(&bars->kv_tmem, 0, ctl, args.status, 34);
      tc_fence_after_sync();
#else
      bool ok = n_steps > 0 && mbar_wait_w(&bars->kv_full, 0, ctl, args.status, 34);
#endif
      if (ok) ok = issue_s(0);
      if (ok) ok = issue_dp(0);
      for (int s = 0; s < n_steps && ok; ++s) {
        const int sq = s % AE_KV_QSTAGES, sd = s % AE_KV_DOSTAGES;
        const u32 par = s & 1;
        (void)par;
        // dV += P^T dO_s, then the next S^T goes over P^T (in issue order, so after it has been read)
        AE_TRK(true, 0, s * 8 + 0)
#if AE_KV_NAMED_BAR
        named_bar_sync(1, AE_KV_NROW + 32);
#else
        ok = mbar_wait_w(&bars->p_full, par, ctl, args.status, 35);
        if (!ok) break;
#endif
        tc_fence_after_sync();
        AE_TRK(true, 0, s * 8 + 1)
        const u64 ddm = ddomn0 + (u64)((sd * AE_KV_DO_BYTES) >> 4);
#pragma unroll
        for (int kk = 0; kk < AE_BWD_BN / 16; ++kk)
          umma_ts_w(tmem + TM_DV, tmem + TM_S + (kk >> 1) * 32 + (kk & 1) * 8, umma_step_mn(ddm, kk), idesc_dv,
                  (s > 0) | (kk > 0));
#if !AE_KV_ONE_BAR
        umma_commit_w(&bars->do_empty[sd]);
#endif
        AE_TRK(true, 0, s * 8 + 2)
        if (s + 1 < n_steps) ok = issue_s(s + 1);
        if (!ok) break;
        AE_TRK(true, 0, s * 8 + 3)
        // dK += dS^T Q_s, then the next dP^T goes over dS^T
#if AE_KV_NAMED_BAR
        named_bar_sync(2, AE_KV_NROW + 32);
#else
        ok = mbar_wait_w(&bars->ds_full, par, ctl, args.status, 39);
        if (!ok) break;
#endif
        tc_fence_after_sync();
        AE_TRK(true, 0, s * 8 + 4)
        const u64 dqm = dqmn0 + (u64)((sq * AE_KV_Q_BYTES) >> 4);
#pragma unroll
        for (int kk = 0; kk < AE_BWD_BN / 16; ++kk)
          umma_ts_w(tmem + TM_DK, tmem + TM_DP + (kk >> 1) * 32 + (kk & 1) * 8, umma_step_mn(dqm, kk), idesc_dk,
                  (s > 0) | (kk > 0));
        umma_commit_w(&bars->q_empty[sq]);
        if (s + 1 == n_steps) umma_commit_w(&bars->acc_done);
        AE_TRK(true, 0, s * 8 + 5)
        if (s + 1 < n_steps) ok = issue_dp(s + 1);
        AE_TRK(true, 0, s * 8 + 6)
      }
    }
  } else {
    // =============================== row threads ================================
    const int wg = warp >> 2;  // the row warpgroups split every tile by 32-column chunks
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
#if AE_KV_TS
    // ---- K (group 0) and V (group 1) rows: shared memory -> TMEM, once ------------------------------
    {
      ok = mbar_wait(&bars->kv_full, 0, ctl, args.status, 45);
      const u8* src = smem + (wg ? AE_KV_SMEM_V : AE_KV_SMEM_K);
      const int nblk = (wg ? AE_DV : AE_D) / 64;
      const u32 tm = tmem + (wg ? TM_V : TM_K) + lane_base;
      if (wg < 2) {
        for (int blk = 0; blk < nblk; ++blk) {
          u32 w[32];
#pragma unroll
          for (int ch = 0; ch < 8; ++ch) {
            const uint4 v = *(const uint4*)(src + blk * (AE_KV_BM * 128) + swz128(row, ch));
            w[ch * 4 + 0] = v.x;
            w[ch * 4 + 1] = v.y;
            w[ch * 4 + 2] = v.z;
            w[ch * 4 + 3] = v.w;
          }
          tmem_st32(tm + blk * 32, w);  // column c of a row holds its elements 2c, 2c + 1: the A-operand layout
        }
        tc_wait_st();
        tc_fence_before_sync();
        mbar_arrive_warp(&bars->kv_tmem);
      }
    }
#endif
    int s = 0;
    AeDkvStep st;
    AeDkvStep st_next;
    bool have = next_step(st_next);
    constexpr int NCH = AE_BWD_BN / 32 / AE_KV_NWG;  // 32-column chunks per group and tile
    const u32 tm_s = tmem + TM_S + lane_base;
    const u32 tm_dp = tmem + TM_DP + lane_base;
    while (have) {
      st = st_next;
      const float* csb = cs + (s & 1) * (AE_BWD_BN * AE_NCS);
      have = next_step(st_next);
      const bool tail = (st.q0 + AE_BWD_BN > args.Sq) || (kv0 + AE_KV_BM > args.Skv);
      const bool masked = st.partial || tail;
      float pkeep[NCH][32];
#if AE_DS_USES_S
      float skeep[NCH][32];
#endif
      auto col_scales = [&](int c, int i, int e, float (&fr)[AE_NCS], const float4 (&cv)[AE_NCS]) {
#pragma unroll
        for (int j = 0; j < AE_NCS; ++j) fr[j] = e == 0 ? cv[j].x : (e == 1 ? cv[j].y : (e == 2 ? cv[j].z : cv[j].w));
      };
      auto keep_of = [&](int q_idx) -> bool {
        bool keep = row_valid && q_idx < args.Sq;
#if AE_MASK_MODE != 0
        if (st.partial) keep = keep && ae_mask(b, st.hq, q_idx, kv_idx);
#endif
        return keep;
      };

      // ---- phase A: P^T from S^T ---------------------------------------------------------------
      AE_TRK((warp & 3) == 0, 1 + wg, s * 8 + 0)
      ok = ok && mbar_wait(&bars->cs_full[s & 1], (s >> 1) & 1, ctl, args.status, 41);
      ok = ok && mbar_wait(&bars->s_full, s & 1, ctl, args.status, 36);
      tc_fence_after_sync();
      AE_TRK((warp & 3) == 0, 1 + wg, s * 8 + 1)
      auto phase_a = [&](auto masked_tag) {
        constexpr bool kMasked = decltype(masked_tag)::value;
#pragma unroll
        for (int ci = 0; ci < NCH; ++ci) {
          const int c = wg + AE_KV_NWG * ci;
          float sv[32];
          tmem_ld_f32x32(tm_s + c * 32, sv);
          u32 pk[16];
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
            float4 cv[AE_NCS];
#pragma unroll
            for (int j = 0; j < AE_NCS; ++j) cv[j] = *(const float4*)(csb + j * AE_BWD_BN + c * 32 + i);
            float p4[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int q_idx = st.q0 + c * 32 + i + e;
              float fr[AE_NCS];
              col_scales(c, i, e, fr, cv);
              float p = ae_bwd_p(sv[i + e], fr, b, st.hq, q_idx, kv_idx, cu, i + e);
              if (kMasked && !keep_of(q_idx)) p = 0.f;
              p4[e] = p;
              pkeep[ci][i + e] = p;
#if AE_DS_USES_S
              skeep[ci][i + e] = sv[i + e];
#endif
            }
            pk[(i >> 1) + 0] = pack2<AE_BF16>(p4[0], p4[1]);
            pk[(i >> 1) + 1] = pack2<AE_BF16>(p4[2], p4[3]);
          }
          tmem_st16(tm_s + c * 32, pk);  // pairs go over this chunk's own first 16 columns
        }
      };
      if (masked) phase_a(AeTrue{}); else phase_a(AeFalse{});
      AE_TRK((warp & 3) == 0, 1 + wg, s * 8 + 2)
      tc_wait_st();
      tc_fence_before_sync();
#if AE_KV_NAMED_BAR
      named_bar_arrive(1, AE_KV_NROW + 32);
#else
      mbar_arrive_warp(&bars->p_full);
#endif
      AE_TRK((warp & 3) == 0, 1 + wg, s * 8 + 3)

      // ---- phase B: dS^T from dP^T and the P^T kept in registers --------------------------------
      ok = ok && mbar_wait(&bars->dp_full, s & 1, ctl, args.status, 40);
      tc_fence_after_sync();
      AE_TRK((warp & 3) == 0, 1 + wg, s * 8 + 4)
      auto phase_b = [&](auto masked_tag) {
        constexpr bool kMasked = decltype(masked_tag)::value;
#pragma unroll
        for (int ci = 0; ci < NCH; ++ci) {
          const int c = wg + AE_KV_NWG * ci;
          float dp[32];
          tmem_ld_f32x32(tm_dp + c * 32, dp);
          u32 dk[16];
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
            float4 cv[AE_NCS];
#pragma unroll
            for (int j = 0; j < AE_NCS; ++j) cv[j] = *(const float4*)(csb + j * AE_BWD_BN + c * 32 + i);
            float ds4[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int q_idx = st.q0 + c * 32 + i + e;
              float fr[AE_NCS];
              col_scales(c, i, e, fr, cv);
#if AE_DS_USES_S
              const float sraw = skeep[ci][i + e];
#else
              const float sraw = 0.f;
#endif
              bool keep = true;
              if (kMasked) keep = keep_of(q_idx);
              float dsv = ae_bwd_ds(sraw, keep ? dp[i + e] : 0.f, pkeep[ci][i + e], fr, fr[AE_NFINAL], b, st.hq, q_idx,
                                    kv_idx, cu);
              if (kMasked && !keep) dsv = 0.f;
              ds4[e] = dsv;
            }
            dk[(i >> 1) + 0] = pack2<AE_BF16>(ds4[0], ds4[1]);
            dk[(i >> 1) + 1] = pack2<AE_BF16>(ds4[2], ds4[3]);
          }
          tmem_st16(tm_dp + c * 32, dk);
        }
      };
      if (masked) phase_b(AeTrue{}); else phase_b(AeFalse{});
      AE_TRK((warp & 3) == 0, 1 + wg, s * 8 + 5)
      tc_wait_st();
      tc_fence_before_sync();
#if AE_KV_NAMED_BAR
      named_bar_arrive(2, AE_KV_NROW + 32);
#else
      mbar_arrive_warp(&bars->ds_full);
#endif
      mbar_arrive_warp(&bars->cs_empty[s & 1]);
      AE_TRK((warp & 3) == 0, 1 + wg, s * 8 + 6)
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
      // the groups take alternate 32-column chunks of [dK | dV] (adjacent in TMEM)
      for (int cc = wg; cc < (AE_D + AE_DV) / 32; cc += AE_KV_NWG) {
        const bool is_dv = cc * 32 >= AE_D;
        u16* drow = is_dv ? dvrow + (cc * 32 - AE_D) : dkrow + cc * 32;
        float r[32];
        if (s > 0) {
          tmem_ld_f32x32(tmem + TM_DK + lane_base + cc * 32, r);
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] = 0.f;
        }
        if (store) {
          uint4* dst = (uint4*)drow;
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
  if (warp == AE_KV_NWG * 4 + 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, 512);
  }
}
