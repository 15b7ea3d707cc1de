// Attention backward in ONE kv-stationary pass: dK, dV and dQ from five contractions per tile, the count the
// reference's `flash_bwd` runs (attn_tl.py:239-415: kv-stationary, dQ through fp32 atomics into a staging buffer
// that a post kernel converts, :406-411, 436-455).  The two-pass backward of attn_bwd_dq.cuh / attn_bwd_dkv.cuh
// recomputes S and dP in both passes (seven contractions) but needs no atomics and is bit-reproducible; this kernel
// trades that for the two contractions.
//
// One CTA owns one 128-row kv tile of one (batch, kv-head) and streams the 128-row Q / dO tiles of every q-head of
// that kv-head's group.  Per q tile s, with rows = kv and columns = q:
//   S^T  = K Q^T (SS)       dP^T = V dO^T (SS)
//   row threads, phase A: P^T = forward(score_mod(S^T)) -> TMEM over S^T (16-bit pairs), kept in registers
//   dV  += P^T dO (TS, dO read MN-major)
//   row threads, phase B: dS^T = score_mod'(S^T) * backward(dP^T, P^T) -> SHARED memory, 16-bit, [kv][q] swizzled
//   dQ_s = dS K   (SS: the dS^T tile read MN-major as A, K read MN-major as B) -> the TMEM columns of dP^T
//   dK  += dS^T Q (SS: the same dS^T tile read K-major as A, Q read MN-major as B)
//   drain warps: dQ_s (lanes = q rows) -> fp32 staging boxes in shared memory -> TMA reduce-add
//                (`cp.reduce.async.bulk.tensor ... .add`) into dq_acc [B, Sq, Hq, D].
// Why TMA and warps of their own: the adds of a tile are 64 KB of fp32 and the L2 atomic units take about 16 bytes per
// clock and SM of them (measured: `red.global.add.f32` from the 16 row warps, 128-byte coalesced, 4200 clk per tile
// during which those warps do nothing else; from 4 dedicated warps 10500 clk, each warp waits ~80 clk per
// instruction; 16-byte vector adds per thread 2x worse again).  A bulk reduce costs the issuing lane one instruction
// per 4 KB and runs behind the row work.
// TMEM columns: dK | dV | S^T / P^T | dP^T / dQ_s = 512 at head dim 128: dQ_s aliases dP^T, so dP^T of the next tile
// is issued once the row threads have drained dQ_s.  Issue order of the MMA warp per tile s:
//   [P^T written]  dV_s , S^T_{s+1}   [dS^T written]  dQ_s , dK_s   [dQ_s drained]  dP^T_{s+1}
// and of the row threads: phase B(s), phase A(s+1) (under dQ_s / dK_s), phase B(s+1).
// The fp32 accumulator dq_acc must be zero when the kernel starts (the launcher clears it); ae_attn_bwd_dq_cast turns
// it into the 16-bit dQ.  Accumulation order across CTAs varies from run to run, so dQ is not bit-reproducible.
// Roles: AE_FU_NWG row warpgroups (thread = kv row = TMEM lane; the groups take alternate 32-column chunks), one
// producer warp, one MMA-issuing warp, four drain warps (one per 32 TMEM lanes).
// Expects AE_FU_QSTAGES / AE_FU_DOSTAGES (ring depths), AE_FU_NWG (2 or 4), AE_FU_SMEM (the launch's dynamic bytes).

#ifndef AE_FU_DEFER_ADDS
#define AE_FU_DEFER_ADDS 1  // 0: the drain warps issue their reduce-adds as soon as the boxes are staged
#endif
#ifndef AE_FU_L2_AHEAD
#define AE_FU_L2_AHEAD 0  // > 0: the producer prefetches the Q / dO tiles of that many steps ahead into L2
#endif
#define AE_FU_BM 128  // kv rows per CTA
#define AE_FU_BN 128  // q rows per streamed tile
#ifdef AE_TRACE
#define AE_TRF(cond, region, slot) \
  if (trace_on && (cond) && (slot) < 2048) args.status[64 + (region) * 4096 + (slot)] = (u32)clock64();
#else
#define AE_TRF(cond, region, slot)
#endif
#define AE_NCS (AE_NFINAL + 1)

#define AE_FU_K_BYTES (AE_FU_BM * AE_D * 2)
#define AE_FU_V_BYTES (AE_FU_BM * AE_DV * 2)
#define AE_FU_Q_BYTES (AE_FU_BN * AE_D * 2)
#define AE_FU_DO_BYTES (AE_FU_BN * AE_DV * 2)
#define AE_FU_DS_BYTES (AE_FU_BM * AE_FU_BN * 2)
#define AE_FU_SMEM_K 0
#define AE_FU_SMEM_V (AE_FU_K_BYTES)
#define AE_FU_SMEM_Q (AE_FU_SMEM_V + AE_FU_V_BYTES)
#define AE_FU_SMEM_DO (AE_FU_SMEM_Q + AE_FU_QSTAGES * AE_FU_Q_BYTES)
#define AE_FU_SMEM_DS (AE_FU_SMEM_DO + AE_FU_DOSTAGES * AE_FU_DO_BYTES)
// dQ staging: per drain warp two boxes of [32 q rows][32 floats] (128-byte rows, 128-byte swizzle: what the TMA reduce reads)
#define AE_FU_DQS_BOX 4096
#define AE_FU_SMEM_DQS (AE_FU_SMEM_DS + AE_FU_DS_BYTES)
#define AE_FU_TILE_BYTES (AE_FU_SMEM_DQS + 4 * 2 * AE_FU_DQS_BOX)
#define AE_FU_CS_BYTES (2 * AE_FU_BN * AE_NCS * 4)
#define AE_FU_BAR_BYTES 256
#define AE_FU_NROW (AE_FU_NWG * 128)
#define AE_FU_NDRAIN 128  // threads of the drain warps
#define AE_FU_NTHREADS (AE_FU_NROW + 64 + AE_FU_NDRAIN)

struct AeFuBars {
  u64 kv_full;
  u64 q_full[AE_FU_QSTAGES], q_empty[AE_FU_QSTAGES];
  u64 do_full[AE_FU_DOSTAGES], do_empty[AE_FU_DOSTAGES];
  u64 cs_full[2], cs_empty[2];  // per-column row scales of a q tile (two slots)
  u64 q_req;  // step s: dK_s has completed and the producer has requested the Q tile that takes its place (if any)
  u64 s_full, dp_full, dq_full;  // S^T / dP^T / dQ of a step are in TMEM
  u64 acc_done;
  AeCtaCtl ctl;
};
static_assert(sizeof(AeFuBars) <= AE_FU_BAR_BYTES, "barrier block");

struct AeFuStep {
  int hq;        // q head
  int q0;        // first q row of the tile
  bool partial;  // needs the element-wise mask
};

extern "C" __global__ void __launch_bounds__(AE_FU_NTHREADS, 1)
ae_attn_bwd_fused(const __grid_constant__ AeAttnBwdArgs args) {
  extern __shared__ __align__(16) u8 smem_raw[];
  // Carve-up that holds for ANY 16-byte aligned base: the tiles start at the next 1024-byte boundary (`gap` bytes in),
  // the row-scale slots follow them, the barrier block follows those when it still fits and otherwise sits in the gap
  // (the launch asks for tiles + slots + 1008 bytes, which covers both cases).
  const u32 gap = (1024u - (smem_u32(smem_raw) & 1023u)) & 1023u;
  u8* smem = smem_raw + gap;
  u8* bar_mem = smem + AE_FU_TILE_BYTES + AE_FU_CS_BYTES;
  if (gap + AE_FU_TILE_BYTES + AE_FU_CS_BYTES + AE_FU_BAR_BYTES > (u32)AE_FU_SMEM) {
    bar_mem = smem_raw;
    if (gap < AE_FU_BAR_BYTES || gap + AE_FU_TILE_BYTES + AE_FU_CS_BYTES > (u32)AE_FU_SMEM) {
      if (threadIdx.x == 0 && args.status) atomicCAS(args.status, 0u, 0x200u);
      return;
    }
  }
  AeFuBars* bars = (AeFuBars*)bar_mem;
  float* cs = (float*)(smem + AE_FU_TILE_BYTES);  // [2][AE_NCS][AE_FU_BN]: final rowscales..., delta, per q column
  AeCtaCtl* ctl = &bars->ctl;
  const u32 warp = threadIdx.x >> 5;
  const u32 lane = threadIdx.x & 31;

  const int kt = blockIdx.x;
  const int hk = blockIdx.y;
  const int b = blockIdx.z;
  const int G = args.Hq / args.Hkv;
  const int kv0 = kt * AE_FU_BM;
  const int n_q_bn = (args.Sq + AE_FU_BN - 1) / AE_FU_BN;
#ifdef AE_TRACE
  const bool trace_on = blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && (threadIdx.x & 31) == 0;
#endif

  // ---- q schedule: heads of the group outer, q tiles inner (identical in every role) ---------------------
#if AE_MASK_MODE == 1
  int i_start = kv0 / AE_FU_BN;
  if (i_start > n_q_bn) i_start = n_q_bn;
#else
  const int i_start = 0;
#endif
  struct Walk {
    int g, e;
  } walk = {0, 0};
  auto next_step = [&](AeFuStep& st) -> bool {
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
        int qt = ent & 0x3fffffff;
        if (qt >= args.n_qt) {  // an entry outside the tile grid: keep every access in range, report status 0x400
          if (args.status) atomicCAS(args.status, 0u, 0x400u);
          qt = args.n_qt - 1;
        }
        st.hq = hq;
        st.q0 = qt * AE_FU_BN;
        st.partial = ((u32)ent >> 30) & 1u;
        walk.e++;
        return true;
      }
      walk.g++;
      walk.e = 0;
    }
    return false;
#else
    const int n_i = n_q_bn - i_start;
    if (n_i <= 0 || walk.g >= G) return false;
    st.hq = hk * G + walk.g;
    st.q0 = (i_start + walk.e) * AE_FU_BN;
#if AE_MASK_MODE == 1
    st.partial = st.q0 < kv0 + AE_FU_BM - 1;
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
    for (int i = 0; i < AE_FU_QSTAGES; ++i) {
      mbar_init(&bars->q_full[i], 1);
      mbar_init(&bars->q_empty[i], 1);
    }
    for (int i = 0; i < AE_FU_DOSTAGES; ++i) {
      mbar_init(&bars->do_full[i], 1);
      mbar_init(&bars->do_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars->cs_full[i], 32);
      mbar_init(&bars->cs_empty[i], AE_FU_NWG * 4);
      if (i == 0) mbar_init(&bars->q_req, 1);
    }
    mbar_init(&bars->s_full, 1);
    mbar_init(&bars->dp_full, 1);
    mbar_init(&bars->dq_full, 1);
    mbar_fence_init();
  }
  if (warp == AE_FU_NWG * 4 + 1) {
    tmem_alloc(&ctl->tmem_base, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const u32 tmem = ctl->tmem_base;
  const u32 TM_DK = 0, TM_DV = AE_D, TM_S = AE_D + AE_DV, TM_DP = TM_S + AE_FU_BN;  // dQ_s aliases TM_DP

  if (warp == AE_FU_NWG * 4) {
    // =============================== producer ====================================
    // All lanes walk the schedule; lane 0 issues the TMA loads, every lane fetches the row scales of four q columns.
    AeFuStep st;
    int s = 0;
    bool have = next_step(st);
    // K and V are only fetched when the walk has a step: a CTA must not retire with a bulk copy into its shared
    // memory still in flight
    if (have && lane == 0) {
      tma_prefetch_desc(&args.tm_q);
      tma_prefetch_desc(&args.tm_k);
      tma_prefetch_desc(&args.tm_v);
      tma_prefetch_desc(&args.tm_do);
      mbar_arrive_expect_tx(&bars->kv_full, AE_FU_K_BYTES + AE_FU_V_BYTES);
      for (int dh = 0; dh < AE_D / 64; ++dh)
        tma_load_bshd(smem + AE_FU_SMEM_K + dh * (AE_FU_BM * 128), &args.tm_k, &bars->kv_full, dh * 64, hk, kv0, b);
      for (int dh = 0; dh < AE_DV / 64; ++dh)
        tma_load_bshd(smem + AE_FU_SMEM_V + dh * (AE_FU_BM * 128), &args.tm_v, &bars->kv_full, dh * 64, hk, kv0, b);
    }
    // The walk plus AE_FU_QSTAGES closing iterations: iteration s waits for the Q slot of step s - AE_FU_QSTAGES to
    // fall free (its dK has completed), requests the Q tile of step s if there is one, and tells the drain warps of
    // step s - AE_FU_QSTAGES that the request is out (q_req), so that their reduce-adds queue up behind it.
    int tail = 0;
    while (have || tail < AE_FU_QSTAGES) {
      const int sq = s % AE_FU_QSTAGES, sd = s % AE_FU_DOSTAGES;
      if (!mbar_wait_w(&bars->q_empty[sq], ((s / AE_FU_QSTAGES) & 1) ^ 1, ctl, args.status, 31)) break;
      AE_TRF(true, 6, s * 8 + 2)
#if AE_MASK_MODE != 2 && AE_FU_L2_AHEAD > 0
      if (lane == 0 && have) {
        // the Q and dO tiles of the step AE_FU_L2_AHEAD ahead, into L2: their loads then pay the L2 latency, not HBM's
        const int n_i = n_q_bn - i_start, sa = s + AE_FU_L2_AHEAD;
        if (n_i > 0 && sa < n_i * G) {
          const int hqa = hk * G + sa / n_i, q0a = (i_start + sa % n_i) * AE_FU_BN;
          for (int dh = 0; dh < AE_D / 64; ++dh) tma_prefetch_l2_4d(&args.tm_q, dh * 64, q0a, hqa, b);
          for (int dh = 0; dh < AE_DV / 64; ++dh) tma_prefetch_l2_4d(&args.tm_do, dh * 64, q0a, hqa, b);
        }
      }
#endif
      if (lane == 0) {
        if (have) {
          mbar_arrive_expect_tx(&bars->q_full[sq], AE_FU_Q_BYTES);
          for (int dh = 0; dh < AE_D / 64; ++dh)
            tma_load_bshd(smem + AE_FU_SMEM_Q + sq * AE_FU_Q_BYTES + dh * (AE_FU_BN * 128), &args.tm_q, &bars->q_full[sq],
                          dh * 64, st.hq, st.q0, b);
        }
        if (s >= AE_FU_QSTAGES) mbar_arrive(&bars->q_req);
      }
      if (!have) {
        ++tail;
        ++s;
        continue;
      }
      {
        if (!mbar_wait_w(&bars->cs_empty[s & 1], ((s >> 1) & 1) ^ 1, ctl, args.status, 42)) break;
        float* csb = cs + (s & 1) * (AE_FU_BN * AE_NCS);
        const i64 base = ((i64)b * args.Hq + st.hq) * args.Sq;
#pragma unroll
        for (int j = 0; j < AE_FU_BN / 32; ++j) {
          const int col = j * 32 + (int)lane;
          const int q = st.q0 + col;
          const i64 off = base + (q < args.Sq ? q : args.Sq - 1);
#pragma unroll
          for (int i = 0; i < AE_NFINAL; ++i) csb[i * AE_FU_BN + col] = args.final_rs[i][off];
#if AE_USES_DOOSUM
          csb[AE_NFINAL * AE_FU_BN + col] = args.delta[off];
#else
          csb[AE_NFINAL * AE_FU_BN + col] = 0.f;
#endif
        }
        mbar_arrive(&bars->cs_full[s & 1]);
      }
      if (!mbar_wait_w(&bars->do_empty[sd], ((s / AE_FU_DOSTAGES) & 1) ^ 1, ctl, args.status, 38)) break;
      if (lane == 0) {
        mbar_arrive_expect_tx(&bars->do_full[sd], AE_FU_DO_BYTES);
        for (int dh = 0; dh < AE_DV / 64; ++dh)
          tma_load_bshd(smem + AE_FU_SMEM_DO + sd * AE_FU_DO_BYTES + dh * (AE_FU_BN * 128), &args.tm_do,
                        &bars->do_full[sd], dh * 64, st.hq, st.q0, b);
      }
      ++s;
      have = next_step(st);
    }
  } else if (warp == AE_FU_NWG * 4 + 1) {
    // =============================== MMA issuer =================================
    // all 32 lanes run the control flow; single MMAs and commits are issued by an elected lane
    const u32 idesc_s = umma_idesc_f16(AE_FU_BM, AE_FU_BN, AE_BF16, 0, 0);
    const u32 idesc_dk = umma_idesc_f16(AE_FU_BM, AE_D, AE_BF16, 0, 1);
    const u32 idesc_dv = umma_idesc_f16(AE_FU_BM, AE_DV, AE_BF16, 0, 1);
    const u32 idesc_dq = umma_idesc_f16(AE_FU_BN, AE_D, AE_BF16, 1, 1);
    const u32 k_addr = smem_u32(smem + AE_FU_SMEM_K);
    const u32 v_addr = smem_u32(smem + AE_FU_SMEM_V);
    const u32 q_addr = smem_u32(smem + AE_FU_SMEM_Q);
    const u32 do_addr = smem_u32(smem + AE_FU_SMEM_DO);
    const u32 ds_addr = smem_u32(smem + AE_FU_SMEM_DS);
    const u64 dk0 = umma_base_k(k_addr), dv0 = umma_base_k(v_addr);
    const u64 dq0 = umma_base_k(q_addr), ddo0 = umma_base_k(do_addr);
    const u64 dqmn0 = umma_base_mn(q_addr, AE_FU_BN), ddomn0 = umma_base_mn(do_addr, AE_FU_BN);
    const u64 dkmn0 = umma_base_mn(k_addr, AE_FU_BM);
    const u64 dds_k = umma_base_k(ds_addr), dds_mn = umma_base_mn(ds_addr, AE_FU_BM);
    auto issue_s = [&](int s) -> bool {  // S^T_s = K Q_s^T
      const int stage = s % AE_FU_QSTAGES;
      AE_TRF(true, 6, s * 8 + 0)
      if (!mbar_wait_w(&bars->q_full[stage], (s / AE_FU_QSTAGES) & 1, ctl, args.status, 32)) return false;
      AE_TRF(true, 6, s * 8 + 1)
      const u64 dqq = dq0 + (u64)((stage * AE_FU_Q_BYTES) >> 4);
#pragma unroll
      for (int kk = 0; kk < AE_D / 16; ++kk)
        umma_ss_w(tmem + TM_S, umma_step_k(dk0, kk, AE_FU_BM), umma_step_k(dqq, kk, AE_FU_BN), idesc_s, kk > 0);
      umma_commit_w(&bars->s_full);
      return true;
    };
    auto issue_dp = [&](int s) -> bool {  // dP^T_s = V dO_s^T
      const int stage = s % AE_FU_DOSTAGES;
      if (!mbar_wait_w(&bars->do_full[stage], (s / AE_FU_DOSTAGES) & 1, ctl, args.status, 33)) return false;
      const u64 ddd = ddo0 + (u64)((stage * AE_FU_DO_BYTES) >> 4);
#pragma unroll
      for (int kk = 0; kk < AE_DV / 16; ++kk)
        umma_ss_w(tmem + TM_DP, umma_step_k(dv0, kk, AE_FU_BM), umma_step_k(ddd, kk, AE_FU_BN), idesc_s, kk > 0);
      umma_commit_w(&bars->dp_full);
      return true;
    };

    int n_steps = 0;
    {
      AeFuStep st;
      while (next_step(st)) ++n_steps;
    }
    bool ok = n_steps > 0 && mbar_wait_w(&bars->kv_full, 0, ctl, args.status, 34);
    if (ok) ok = issue_s(0);
    if (ok) ok = issue_dp(0);
    for (int s = 0; s < n_steps && ok; ++s) {
      const int sq = s % AE_FU_QSTAGES, sd = s % AE_FU_DOSTAGES;
      // dV += P^T dO_s, then the next S^T goes over P^T (in issue order, so after it has been read)
      AE_TRF(true, 0, s * 8 + 0)
      named_bar_sync(1, AE_FU_NROW + 32);
      tc_fence_after_sync();
      AE_TRF(true, 0, s * 8 + 1)
      const u64 ddm = ddomn0 + (u64)((sd * AE_FU_DO_BYTES) >> 4);
#pragma unroll
      for (int kk = 0; kk < AE_FU_BN / 16; ++kk)
        umma_ts_w(tmem + TM_DV, tmem + TM_S + (kk >> 1) * 32 + (kk & 1) * 8, umma_step_mn(ddm, kk), idesc_dv,
                  (s > 0) | (kk > 0));
      umma_commit_w(&bars->do_empty[sd]);  // dO_s was also read by dP^T_s, issued earlier
      AE_TRF(true, 0, s * 8 + 7)
      if (s + 1 < n_steps) ok = issue_s(s + 1);
      if (!ok) break;
      AE_TRF(true, 0, s * 8 + 2)
      // dS^T_s is in shared memory (and dP^T_s has been read): dQ_s over dP^T's columns, then dK
      named_bar_sync(2, AE_FU_NROW + 32);
      tc_fence_after_sync();
      AE_TRF(true, 0, s * 8 + 3)
#pragma unroll
      for (int kk = 0; kk < AE_FU_BM / 16; ++kk)
        umma_ss_w(tmem + TM_DP, umma_step_mn(dds_mn, kk), umma_step_mn(dkmn0, kk), idesc_dq, kk > 0);
      umma_commit_w(&bars->dq_full);
      const u64 dqm = dqmn0 + (u64)((sq * AE_FU_Q_BYTES) >> 4);
#pragma unroll
      for (int kk = 0; kk < AE_FU_BN / 16; ++kk)
        umma_ss_w(tmem + TM_DK, umma_step_k(dds_k, kk, AE_FU_BM), umma_step_mn(dqm, kk), idesc_dk, (s > 0) | (kk > 0));
      umma_commit_w(&bars->q_empty[sq]);
      if (s + 1 == n_steps) umma_commit_w(&bars->acc_done);
      AE_TRF(true, 0, s * 8 + 4)
      if (s + 1 < n_steps) {
        named_bar_sync(3, AE_FU_NDRAIN + 32);  // dQ_s has left TMEM
        tc_fence_after_sync();
        AE_TRF(true, 0, s * 8 + 5)
        ok = issue_dp(s + 1);
      }
      AE_TRF(true, 0, s * 8 + 6)
    }
    // Every commit of this warp has arrived before the CTA may retire (the last steps' slot releases have no other
    // waiter): an arrival that lands on a retired CTA's shared memory would hit whoever owns it next.
    if (ok) {
      const int l = n_steps - 1;
      ok = mbar_wait_w(&bars->acc_done, 0, ctl, args.status, 44) &&
           mbar_wait_w(&bars->q_empty[l % AE_FU_QSTAGES], (l / AE_FU_QSTAGES) & 1, ctl, args.status, 45) &&
           mbar_wait_w(&bars->do_empty[l % AE_FU_DOSTAGES], (l / AE_FU_DOSTAGES) & 1, ctl, args.status, 46);
    }
  } else if (warp >= AE_FU_NWG * 4 + 2) {
    // =============================== drain warps ================================
    // dQ_s out of TMEM into the fp32 accumulator in global memory.  Warp w owns TMEM lanes 32 (w % 4) ... = 32 q rows of
    // the tile and moves them as AE_D / 32 boxes of [32 rows][32 floats]: registers -> one of its two staging boxes ->
    // TMA reduce-add, one bulk group per box.  A box is rewritten once the group that read it two boxes earlier has
    // finished reading (wait_group.read 1).  The first two boxes go through staging at once, the others wait in
    // registers, so the TMEM columns are handed back (named barrier 3) after two issues, not after the whole tile.
    const u32 wq = warp & 3;
    const u32 tm_dp = tmem + TM_DP + ((wq * 32) << 16);
    u8* box0 = smem + AE_FU_SMEM_DQS + wq * (2 * AE_FU_DQS_BOX);
    constexpr int NBOX = AE_D / 32;
    constexpr int NKEEP = NBOX > 2 ? NBOX - 2 : 0;
    bool ok = true;
    AeFuStep st, st_next;
    bool have = next_step(st);
    if (lane == 0) tma_prefetch_desc(&args.tm_dqacc);
    // A box goes out in two steps: into its staging slot (c & 1), then as a TMA reduce-add of its own bulk group.
    auto stage_box = [&](const float (&v)[32], int c) {
      u8* box = box0 + (c & 1) * AE_FU_DQS_BOX;
#pragma unroll
      for (int ch = 0; ch < 8; ++ch)
        *(float4*)(box + swz128(lane, ch)) = make_float4(v[ch * 4 + 0], v[ch * 4 + 1], v[ch * 4 + 2], v[ch * 4 + 3]);
    };
    auto issue_box = [&](int c, const AeFuStep& stp) {
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        if (ok)
          asm volatile(
              "cp.reduce.async.bulk.tensor.4d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3, %4, %5}], [%1];" ::"l"(
                  (u64)&args.tm_dqacc),
              "r"(smem_u32(box0 + (c & 1) * AE_FU_DQS_BOX)), "r"(c * 32), "r"(stp.q0 + (int)wq * 32), "r"(stp.hq), "r"(b)
              : "memory");
        tma_store_commit();  // an empty group when the CTA is aborting: the slot accounting stays the same
      }
    };
    auto slot_free = [&](int pending) {  // the bulk group issued `pending + 1` boxes ago has read its slot
      if (lane == 0) {
        if (pending)
          asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
        else
          asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
      }
      __syncwarp();
    };
    for (int s = 0; have; ++s) {
      const bool more = next_step(st_next);
      ok = ok && mbar_wait(&bars->dq_full, s & 1, ctl, args.status, 43);
      tc_fence_after_sync();
      AE_TRF(lane == 0, 5, s * 8 + wq * 2)
      float keep[NKEEP > 0 ? NKEEP : 1][32];
      slot_free(0);  // the last two boxes of the tile before have left both slots
#pragma unroll
      for (int c = 0; c < NBOX && c < 2; ++c) {
        float v[32];
        tmem_ld_f32x32(tm_dp + c * 32, v);
        stage_box(v, c);
      }
#pragma unroll
      for (int c = 2; c < NBOX; ++c) tmem_ld_f32x32(tm_dp + c * 32, keep[c - 2]);
      tc_fence_before_sync();
      if (more) named_bar_arrive(3, AE_FU_NDRAIN + 32);  // the columns may be overwritten by the next dP^T
      // The reduce-adds are slow (the L2 reduce units) and share the SM's bulk-copy queue with the loads: a Q tile
      // requested behind a tile's worth of them arrives late for the next S GEMM.  The producer requests the next Q tile
      // the moment dK_s has completed and then arrives on q_req: the adds of this tile are held back until then.
#if AE_FU_DEFER_ADDS
      ok = ok && mbar_wait(&bars->q_req, s & 1, ctl, args.status, 47);
#endif
#pragma unroll
      for (int c = 0; c < NBOX && c < 2; ++c) issue_box(c, st);
#pragma unroll
      for (int c = 2; c < NBOX; ++c) {
        slot_free(1);
        stage_box(keep[c - 2], c);
        issue_box(c, st);
      }
      AE_TRF(lane == 0, 5, s * 8 + wq * 2 + 1)
      st = st_next;
      have = more;
    }
    // the staging boxes belong to this CTA until the bulk engine has read them; the adds themselves complete on their own
    if (lane == 0) tma_store_wait_read();
    __syncwarp();
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
    constexpr int NCH = AE_FU_BN / 32 / AE_FU_NWG;  // 32-column chunks per group and tile
    const u32 tm_s = tmem + TM_S + lane_base;
    const u32 tm_dp = tmem + TM_DP + lane_base;
    u8* ds_tile = smem + AE_FU_SMEM_DS;
    float pkeep[NCH][32];
#if AE_DS_USES_S
    float skeep[NCH][32];
#endif

    auto col_scales = [&](int e, float (&fr)[AE_NCS], const float4 (&cv)[AE_NCS]) {
#pragma unroll
      for (int j = 0; j < AE_NCS; ++j) fr[j] = e == 0 ? cv[j].x : (e == 1 ? cv[j].y : (e == 2 ? cv[j].z : cv[j].w));
    };

    // ---- phase A of step s: P^T from S^T, kept in registers and written over S^T as 16-bit pairs ----------
    auto phase_a_step = [&](const AeFuStep& st, int s) {
      const float* csb = cs + (s & 1) * (AE_FU_BN * AE_NCS);
      const bool tail = (st.q0 + AE_FU_BN > args.Sq) || (kv0 + AE_FU_BM > args.Skv);
      const bool masked = st.partial || tail;
      AE_TRF((warp & 3) == 0, 1 + wg, s * 8 + 0)
      ok = ok && mbar_wait(&bars->cs_full[s & 1], (s >> 1) & 1, ctl, args.status, 41);
      ok = ok && mbar_wait(&bars->s_full, s & 1, ctl, args.status, 36);
      tc_fence_after_sync();
      AE_TRF((warp & 3) == 0, 1 + wg, s * 8 + 1)
      auto body = [&](auto masked_tag) {
        constexpr bool kMasked = decltype(masked_tag)::value;
#pragma unroll
        for (int ci = 0; ci < NCH; ++ci) {
          const int c = wg + AE_FU_NWG * ci;
          float sv[32];
          tmem_ld_f32x32(tm_s + c * 32, sv);
          u32 pk[16];
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
            float4 cv[AE_NCS];
#pragma unroll
            for (int j = 0; j < AE_NCS; ++j) cv[j] = *(const float4*)(csb + j * AE_FU_BN + c * 32 + i);
            float p4[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int q_idx = st.q0 + c * 32 + i + e;
              float fr[AE_NCS];
              col_scales(e, fr, cv);
              float p = ae_bwd_p(sv[i + e], fr, b, st.hq, q_idx, kv_idx, cu, i + e);
              if (kMasked) {
                bool keep = row_valid && q_idx < args.Sq;
#if AE_MASK_MODE != 0
                if (st.partial) keep = keep && ae_mask(b, st.hq, q_idx, kv_idx);
#endif
                if (!keep) p = 0.f;
              }
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
      if (masked) body(AeTrue{}); else body(AeFalse{});
      tc_wait_st();
      tc_fence_before_sync();
      named_bar_arrive(1, AE_FU_NROW + 32);
      AE_TRF((warp & 3) == 0, 1 + wg, s * 8 + 2)
    };

    // ---- phase B of step s: dS^T from dP^T and the P^T kept in registers, into shared memory -------------
    auto phase_b_step = [&](const AeFuStep& st, int s) {
      const float* csb = cs + (s & 1) * (AE_FU_BN * AE_NCS);
      const bool tail = (st.q0 + AE_FU_BN > args.Sq) || (kv0 + AE_FU_BM > args.Skv);
      const bool masked = st.partial || tail;
      ok = ok && mbar_wait(&bars->dp_full, s & 1, ctl, args.status, 40);
      tc_fence_after_sync();
      AE_TRF((warp & 3) == 0, 1 + wg, s * 8 + 3)
      auto body = [&](auto masked_tag) {
        constexpr bool kMasked = decltype(masked_tag)::value;
#pragma unroll
        for (int ci = 0; ci < NCH; ++ci) {
          const int c = wg + AE_FU_NWG * ci;
          float dp[32];
          tmem_ld_f32x32(tm_dp + c * 32, dp);
          u32 dk[16];
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
            float4 cv[AE_NCS];
#pragma unroll
            for (int j = 0; j < AE_NCS; ++j) cv[j] = *(const float4*)(csb + j * AE_FU_BN + c * 32 + i);
            float ds4[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int q_idx = st.q0 + c * 32 + i + e;
              float fr[AE_NCS];
              col_scales(e, fr, cv);
#if AE_DS_USES_S
              const float sraw = skeep[ci][i + e];
#else
              const float sraw = 0.f;
#endif
              bool keep = true;
              if (kMasked) {
                keep = row_valid && q_idx < args.Sq;
#if AE_MASK_MODE != 0
                if (st.partial) keep = keep && ae_mask(b, st.hq, q_idx, kv_idx);
#endif
              }
              float dsv = ae_bwd_ds(sraw, keep ? dp[i + e] : 0.f, pkeep[ci][i + e], fr, fr[AE_NFINAL], b, st.hq, q_idx,
                                    kv_idx, cu);
              if (kMasked && !keep) dsv = 0.f;
              ds4[e] = dsv;
            }
            dk[(i >> 1) + 0] = pack2<AE_BF16>(ds4[0], ds4[1]);
            dk[(i >> 1) + 1] = pack2<AE_BF16>(ds4[2], ds4[3]);
          }
          // row `row` of the [kv][q] tile, q columns c * 32 .. c * 32 + 31: four 16-byte pieces of one 64-column block
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const u32 col = (u32)c * 32u + (u32)i * 8u;
            *(uint4*)(ds_tile + tile_off(row, col, AE_FU_BM)) = make_uint4(dk[i * 4 + 0], dk[i * 4 + 1], dk[i * 4 + 2], dk[i * 4 + 3]);
          }
        }
      };
      if (masked) body(AeTrue{}); else body(AeFalse{});
      fence_proxy_async_smem();  // the tile is read by tcgen05.mma (async proxy)
      tc_fence_before_sync();
      named_bar_arrive(2, AE_FU_NROW + 32);
      mbar_arrive_warp(&bars->cs_empty[s & 1]);
      AE_TRF((warp & 3) == 0, 1 + wg, s * 8 + 4)
    };

    int s = 0;
    AeFuStep st, st_next;
    bool have = next_step(st);
    if (have) phase_a_step(st, 0);
    while (have) {
      phase_b_step(st, s);
      const bool more = next_step(st_next);
      if (more) phase_a_step(st_next, s + 1);
      st = st_next;
      have = more;
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
      for (int cc = wg; cc < (AE_D + AE_DV) / 32; cc += AE_FU_NWG) {
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
  if (warp == AE_FU_NWG * 4 + 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, 512);
  }
}

// dq[b, s, h, :] (16-bit, any strides) = dq_acc[b, s, h, :] (fp32, contiguous [B, Sq, Hq, D]): the conversion pass after
// ae_attn_bwd_fused, the `flash_bwd_post` of the reference (attn_tl.py:436-455).  Eight elements per thread.
extern "C" __global__ void __launch_bounds__(256) ae_attn_bwd_dq_cast(const __grid_constant__ AeAttnBwdArgs args) {
  const i64 n_vec = (i64)args.B * args.Sq * args.Hq * (AE_D / 8);
  for (i64 i = (i64)blockIdx.x * 256 + threadIdx.x; i < n_vec; i += (i64)gridDim.x * 256) {
    const int dv = (int)(i % (AE_D / 8));
    i64 r = i / (AE_D / 8);
    const int h = (int)(r % args.Hq);
    r /= args.Hq;
    const int sq = (int)(r % args.Sq);
    const int b = (int)(r / args.Sq);
    const float4* src = (const float4*)(args.dq_acc + i * 8);
    const float4 lo = src[0], hi = src[1];
    uint4 w;
    w.x = pack2<AE_BF16>(lo.x, lo.y);
    w.y = pack2<AE_BF16>(lo.z, lo.w);
    w.z = pack2<AE_BF16>(hi.x, hi.y);
    w.w = pack2<AE_BF16>(hi.z, hi.w);
    *(uint4*)((u16*)args.dq + (i64)b * args.dq_sb + (i64)sq * args.dq_ss + (i64)h * args.dq_sh + dv * 8) = w;
  }
}
