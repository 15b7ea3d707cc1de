// Chunked linear-attention / SSD scan, backward, for sm_100a.  Replaces the reference's
// `chunk_bwd_kernel_dh`, `chunk_bwd_dqkg`, `chunk_bwd_kernel_dv` and `compute_final_dg` kernels
// (attention_engine/core/template/tl_template/linear/linear_tl.py:447-545, 584-788, 827-930, 52-65).
//
// One CTA owns one (batch, head) and walks its 128-step chunks from the last to the first, carrying
// dH, the gradient with respect to the state, as an fp32 TMEM accumulator.  With g the inclusive
// cumulative log-decay inside the chunk, E_ij = exp(g_i - g_j) [i >= j], w_j = exp(g_last - g_j),
// h the chunk's incoming state (recomputed by linear_states.cuh) and dH' the gradient of its outgoing state:
//     A  = q k^T          dPr = dO v^T                          (SS MMAs into R0, R1)
//     row threads: P = E o A, dS = E o dPr  -> 16-bit tiles in shared memory
//     dq_i = exp(g_i) (dO h^T)_i + (dS k)_i                      (R0: inter MMA on the copy of dO that carries exp(g_i),
//                                                                 intra MMA on top; no row scaling)
//     dk_j = w_j (v dH'^T)_j + (dS^T q)_j                        (R2: inter MMA early, rows scale by w_j, intra on top)
//     dv_j = w_j (k dH')_j + (P^T dO)_j
//     dH   = exp(g_last) dH' + q^T (dO o exp(g))
//     d a_t = sum over s >= t of (q_s . dq_s - k_s . dk_s): a suffix sum inside the chunk; what the later chunks add
//             is <dH, h> of the next chunk (the state that crosses the boundary times its gradient), computed there
//             directly.  Carrying the running sum across chunks instead lets the rounding of the 16-bit operands
//             random-walk over the whole sequence (28 % error on dA at 8192 steps).
// dq / dk are written per head; the caller sums them over a head group when q / k have fewer heads.
// All transposed products read the same 16-bit tiles through MN-major descriptors: nothing is transposed in
// registers.  Roles: warps 0-3 row threads (thread r = step r = state row r), warp 4 TMA, warp 5 MMA.
// The row threads are the critical path (one warp per sub-partition, every phase of a chunk waits for them), so the
// chunk's dq / dk / dv rows do not leave through their per-row global stores: they are written as 16-bit tiles over the
// P, dS and dO-copy tiles (dead once the chunk's last MMAs have completed) and the TMA warp sends them out as bulk
// stores while the next chunk is under way.
// AE_LB_MODS = 1 (the Mamba2 block: v = x * s[b, h, t] before the scan, y += x * d[h] after it): the gradients that
// meet at x leave this kernel instead of a streaming pass of their own.  The chunk's x tile is loaded next to q and k;
// the row threads keep their piece of the dO row from phase C in registers (the dO tile is refilled before the output
// phase) and write gx = dv * s + dO * d[h] where dv went, the row sums gs = <dv, x> (dv rounded to 16 bits first, as
// the separate kernel saw it) per step, and one sum of <dO, x> per (batch, head) for the gradient of d.
// Expects AE_BF16, AE_LIN_DV (64).

#ifdef AE_TRACE  // clock stamps of CTA (0, 0)'s row warp 0 and MMA warp into the status buffer (experiments)
#define AE_TRL(cond, region, slot) \
  if (blockIdx.x == 0 && blockIdx.y == 0 && lane == 0 && (cond) && (slot) < 4096) \
    args.status[64 + (region) * 4096 + (slot)] = (u32)clock64();
#else
#define AE_TRL(cond, region, slot)
#endif
// AE_LB_NWG = 2: a second row warpgroup takes half of the columns of every row phase (same rows, other 32-column
// blocks); the cumulative sum and the suffix sums of the decay gradient stay with the first group.  The groups meet
// at named barrier 2 (the chunk's cumulative decays are ready) and 3 (the second group's share of q.dq - k.dk is in
// shared memory).
#ifndef AE_LB_NWG
#define AE_LB_NWG 1
#endif
#ifndef AE_LB_MODS
#define AE_LB_MODS 0
#endif
#define AE_LB_ROWW (4 * AE_LB_NWG)  // row warps; then the TMA warp and the MMA warp
#define AE_LB_C 128
#define AE_LB_DK 128
#define AE_LB_QK_BYTES (AE_LB_C * AE_LB_DK * 2)
#define AE_LB_V_BYTES (AE_LB_C * AE_LIN_DV * 2)
#define AE_LB_H_BYTES (AE_LB_DK * AE_LIN_DV * 2)
#define AE_LB_PP_BYTES (AE_LB_C * AE_LB_C * 2)
#define AE_LB_SMEM_Q 0
#define AE_LB_SMEM_K (AE_LB_SMEM_Q + AE_LB_QK_BYTES)
#define AE_LB_SMEM_V (AE_LB_SMEM_K + AE_LB_QK_BYTES)
#define AE_LB_SMEM_DO (AE_LB_SMEM_V + AE_LB_V_BYTES)
#define AE_LB_SMEM_HC (AE_LB_SMEM_DO + AE_LB_V_BYTES)
#define AE_LB_SMEM_P (AE_LB_SMEM_HC + AE_LB_H_BYTES)
#define AE_LB_SMEM_DS (AE_LB_SMEM_P + AE_LB_PP_BYTES)
#define AE_LB_SMEM_DHB (AE_LB_SMEM_DS + AE_LB_PP_BYTES)
#define AE_LB_SMEM_DO2 (AE_LB_SMEM_DHB + AE_LB_H_BYTES)
#define AE_LB_SMEM_X (AE_LB_SMEM_DO2 + AE_LB_V_BYTES)  // AE_LB_MODS: the chunk's rows of x
#define AE_LB_SMEM_G (AE_LB_SMEM_X + AE_LB_MODS * AE_LB_V_BYTES)
#define AE_LB_SMEM_BAR (AE_LB_SMEM_G + 1024)
#define AE_LB_SMEM_XG (AE_LB_SMEM_BAR + 256)  // AE_LB_NWG = 2: [128] fp32, the second group's partial dG per row
#define AE_LB_LOAD_BYTES (2 * AE_LB_QK_BYTES + 2 * AE_LB_V_BYTES + AE_LB_H_BYTES)

struct AeLbBars {
  u64 full;     // q, k of the chunk (requested when the chunk before hands its tiles back)
  u64 full_vd;  // v, dO (requested earlier: at the chunk before's last MMA, nothing reads those two tiles after it)
  u64 full_h;   // the chunk's start state (same request as q, k; first needed by the dq MMA, late in the chunk)
  u64 empty;    // the row threads are done with the chunk's start state (and x)
  u64 qk_free;  // ... and, earlier, with its q and k tiles
  u64 s_full;
  u64 prep_done;
  u64 pds_full;
  u64 inter_full;
  u64 scaled_done;
  u64 out_full;
  u64 o_ready;  // the chunk's dq / dk / dv tiles are in shared memory
  u64 o_free;   // ... and the bulk store of dv has read its tile (the dO copy, rewritten early in the next chunk)
  u64 o_free2;  // ... and those of dq, dk theirs (the P and dS tiles, rewritten by the next chunk's P / dS pass)
  AeCtaCtl ctl;
};

extern "C" __global__ void __launch_bounds__(AE_LB_ROWW * 32 + 64, 1) ae_linear_bwd(const __grid_constant__ AeLinearBwdArgs args) {
  extern __shared__ u8 smem_raw[];
  u8* smem = smem_align1024(smem_raw);
  AeLbBars* bars = (AeLbBars*)(smem + AE_LB_SMEM_BAR);
  // Two buffers of 128 cumulative log-decays: the chunk at hand reads one (after its P / dS pass it carries the second
  // group's <dv, x>) while the first group already fills the other for the next chunk.
  float* gs = (float*)(smem + AE_LB_SMEM_G);
  // [0..3] warp totals of the cumulative sum, [4..7] warp sums of dG, [8..23] warp sums of <dH, h> (two chunks' worth,
  // by chunk parity), [24..31] warp sums of <dO, x> at the end
  float* misc = (float*)(smem + AE_LB_SMEM_BAR + 128);
  AeCtaCtl* ctl = &bars->ctl;
  const u32 warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.x, b = blockIdx.y;
  const int hq = h / (args.H / args.HQ);
  const int hk = h / (args.H / args.HK);
  const int n_chunks = (args.T + AE_LB_C - 1) / AE_LB_C;

  if (threadIdx.x == 0) {
    ctl->abort = 0;
    mbar_init(&bars->full, 1);
    mbar_init(&bars->full_vd, 1);
    mbar_init(&bars->full_h, 1);
    mbar_init(&bars->empty, AE_LB_ROWW);
    mbar_init(&bars->qk_free, AE_LB_ROWW);
    mbar_init(&bars->s_full, 1);
    mbar_init(&bars->prep_done, AE_LB_ROWW);
    mbar_init(&bars->pds_full, AE_LB_ROWW);
    mbar_init(&bars->inter_full, 1);
    mbar_init(&bars->scaled_done, AE_LB_ROWW);
    mbar_init(&bars->out_full, 1);
    mbar_init(&bars->o_ready, AE_LB_ROWW);
    mbar_init(&bars->o_free, 1);
    mbar_init(&bars->o_free2, 1);
    mbar_fence_init();
  }
  if (warp == AE_LB_ROWW + 1) {
    tmem_alloc(&ctl->tmem_base, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const u32 tmem = ctl->tmem_base;
  // R0: A = q k^T, then dq.  R1: dPr = dO v^T.  R2: dk.  The inter-chunk parts of dk and dv do not wait for the row
  // threads' P / dS pass: they go to regions that pass does not read.
  const u32 TM_R0 = 0, TM_R1 = 128, TM_DV = 256, TM_DH = 256 + AE_LIN_DV, TM_R2 = 384;

  if (warp == AE_LB_ROWW) {
    // =============================== TMA producer ===============================
    if (lane == 0) {
      tma_prefetch_desc(&args.tm_q);
      tma_prefetch_desc(&args.tm_k);
      tma_prefetch_desc(&args.tm_v);
      tma_prefetch_desc(&args.tm_do);
      tma_prefetch_desc(&args.tm_h);
      tma_prefetch_desc(&args.tm_dq);
      tma_prefetch_desc(&args.tm_dk);
      tma_prefetch_desc(&args.tm_dv);
#if AE_LB_MODS
      tma_prefetch_desc(&args.tm_x);
#endif
      bool ok = true;
      // Shared memory holds one chunk, so the loads of the next one can only be requested as its tiles fall free: v and
      // dO (the two that come from HBM and are not read by the row threads' output phase) at the chunk's last MMA, the
      // rest when the row threads hand the tiles back.  The output tiles of the chunk before go out in between.
      for (int it = 0; it <= n_chunks && ok; ++it) {
        const int c = n_chunks - 1 - it;
        if (it >= 1) {
          ok = mbar_wait(&bars->out_full, (it - 1) & 1, ctl, args.status, 82);
          if (!ok) break;
        }
        if (it < n_chunks) {
          mbar_arrive_expect_tx(&bars->full_vd, 2 * AE_LB_V_BYTES);
          for (int dh = 0; dh < AE_LIN_DV / 64; ++dh) {
            tma_load_4d(smem + AE_LB_SMEM_V + dh * (AE_LB_C * 128), &args.tm_v, &bars->full_vd, dh * 64, c * AE_LB_C, h, b);
            tma_load_4d(smem + AE_LB_SMEM_DO + dh * (AE_LB_C * 128), &args.tm_do, &bars->full_vd, dh * 64, c * AE_LB_C, h, b);
          }
        }
        if (it < n_chunks) {
          // q and k: handed back by the row threads as soon as their dq / dk rows are done, ahead of the rest of the
          // output phase - the next chunk's first MMA waits for these two
          if (it >= 1 && !mbar_wait(&bars->qk_free, (it - 1) & 1, ctl, args.status, 88)) break;
          mbar_arrive_expect_tx(&bars->full, 2 * AE_LB_QK_BYTES);
          for (int dh = 0; dh < AE_LB_DK / 64; ++dh) {
            tma_load_4d(smem + AE_LB_SMEM_Q + dh * (AE_LB_C * 128), &args.tm_q, &bars->full, dh * 64, c * AE_LB_C, hq, b);
            tma_load_4d(smem + AE_LB_SMEM_K + dh * (AE_LB_C * 128), &args.tm_k, &bars->full, dh * 64, c * AE_LB_C, hk, b);
          }
        }
        if (it >= 1) {
          // the output tiles of the chunk before: ready a little before its last tiles are handed back
          const int co = n_chunks - it;
          ok = mbar_wait(&bars->o_ready, (it - 1) & 1, ctl, args.status, 80);
          if (!ok) break;
          // dv now (a small group of its own: its tile is rewritten early in the next chunk); dq and dk go out after
          // the loads of q and k below, which the next chunk needs first
          for (int dh = 0; dh < AE_LIN_DV / 64; ++dh)
            tma_store_4d(&args.tm_dv, smem + AE_LB_SMEM_DO2 + dh * (AE_LB_C * 128), dh * 64, co * AE_LB_C, h, b);
          tma_store_commit();
        }
        if (it < n_chunks) {
          if (!mbar_wait(&bars->empty, (it & 1) ^ 1, ctl, args.status, 71)) break;
          mbar_arrive_expect_tx(&bars->full_h, AE_LB_H_BYTES + AE_LB_MODS * AE_LB_V_BYTES);
          for (int dh = 0; dh < AE_LIN_DV / 64; ++dh)
            tma_load_3d(smem + AE_LB_SMEM_HC + dh * (AE_LB_DK * 128), &args.tm_h, &bars->full_h, dh * 64, 0,
                        (b * args.H + h) * n_chunks + c);
#if AE_LB_MODS
          // x is first read by the output phase, at the far end of the chunk: it travels with the start state, behind
          // q and k, which the chunk's first MMA waits for
          for (int dh = 0; dh < AE_LIN_DV / 64; ++dh)
            tma_load_4d(smem + AE_LB_SMEM_X + dh * (AE_LB_C * 128), &args.tm_x, &bars->full_h, dh * 64, c * AE_LB_C, h, b);
#endif
        }
        if (it >= 1) {
          const int co = n_chunks - it;
          for (int dh = 0; dh < AE_LB_DK / 64; ++dh) {
            tma_store_4d(&args.tm_dq, smem + AE_LB_SMEM_P + dh * (AE_LB_C * 128), dh * 64, co * AE_LB_C, h, b);
            tma_store_4d(&args.tm_dk, smem + AE_LB_SMEM_DS + dh * (AE_LB_C * 128), dh * 64, co * AE_LB_C, h, b);
          }
          tma_store_commit();
          asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");  // the dv group has read its tile
          mbar_arrive(&bars->o_free);
          tma_store_wait_read();  // the row threads of the next chunk write these tiles again
          mbar_arrive(&bars->o_free2);
        }
      }
      tma_store_wait_read();
    }
  } else if (warp == AE_LB_ROWW + 1) {
    // =============================== MMA issuer =================================
    {  // all 32 lanes run the control flow; MMAs and commits are issued by an elected lane
      const u32 Q = smem_u32(smem + AE_LB_SMEM_Q), K = smem_u32(smem + AE_LB_SMEM_K), V = smem_u32(smem + AE_LB_SMEM_V);
      const u32 DO = smem_u32(smem + AE_LB_SMEM_DO), HC = smem_u32(smem + AE_LB_SMEM_HC);
      const u32 P = smem_u32(smem + AE_LB_SMEM_P), DS = smem_u32(smem + AE_LB_SMEM_DS);
      const u32 DHB = smem_u32(smem + AE_LB_SMEM_DHB), DO2 = smem_u32(smem + AE_LB_SMEM_DO2);
      const u64 kQ = umma_base_k(Q), kK = umma_base_k(K), kV = umma_base_k(V), kDO = umma_base_k(DO), kHC = umma_base_k(HC);
      const u64 kDHB = umma_base_k(DHB), kDS = umma_base_k(DS), kDO2 = umma_base_k(DO2);
      const u64 mQ = umma_base_mn(Q, 128), mK = umma_base_mn(K, 128), mDO = umma_base_mn(DO, 128), mDO2 = umma_base_mn(DO2, 128);
      const u64 mDHB = umma_base_mn(DHB, 128), mDS = umma_base_mn(DS, 128), mP = umma_base_mn(P, 128);
      const u32 id_kk_128 = umma_idesc_f16(128, 128, AE_BF16, 0, 0);
      const u32 id_kmn_dv = umma_idesc_f16(128, AE_LIN_DV, AE_BF16, 0, 1);
      const u32 id_mnmn_dv = umma_idesc_f16(128, AE_LIN_DV, AE_BF16, 1, 1);
      const u32 id_kmn_128 = umma_idesc_f16(128, 128, AE_BF16, 0, 1);
      const u32 id_mnmn_128 = umma_idesc_f16(128, 128, AE_BF16, 1, 1);
      bool ok = true;
      for (int it = 0; it < n_chunks && ok; ++it) {
        const u32 par = it & 1;
        ok = mbar_wait_w(&bars->full, par, ctl, args.status, 72) && mbar_wait_w(&bars->full_vd, par, ctl, args.status, 83);
        if (!ok) break;
        tc_fence_after_sync();
        // A = q k^T -> R0 ; dPr = dO v^T -> R1
#pragma unroll
        for (int kk = 0; kk < AE_LB_DK / 16; ++kk)
          umma_ss_w(tmem + TM_R0, umma_step_k(kQ, kk, 128), umma_step_k(kK, kk, 128), id_kk_128, kk > 0);
#pragma unroll
        for (int kk = 0; kk < AE_LIN_DV / 16; ++kk)
          umma_ss_w(tmem + TM_R1, umma_step_k(kDO, kk, 128), umma_step_k(kV, kk, 128), id_kk_128, kk > 0);
        umma_commit_w(&bars->s_full);
        ok = mbar_wait_w(&bars->prep_done, par, ctl, args.status, 73);
        if (!ok) break;
        tc_fence_after_sync();
        // inter-chunk parts of dk and dv (their regions are not read by the P / dS pass under way), then the state
        // gradient; the row threads scale the two by w_j once they are done with P / dS
#pragma unroll
        for (int kk = 0; kk < AE_LIN_DV / 16; ++kk)
          umma_ss_w(tmem + TM_R2, umma_step_k(kV, kk, 128), umma_step_k(kDHB, kk, 128), id_kk_128, kk > 0);
#pragma unroll
        for (int kk = 0; kk < AE_LB_DK / 16; ++kk)
          umma_ss_w(tmem + TM_DV, umma_step_k(kK, kk, 128), umma_step_mn(mDHB, kk), id_kmn_dv, kk > 0);
        umma_commit_w(&bars->inter_full);
        // dH (+)= q^T (dO o exp(g))
#pragma unroll
        for (int kk = 0; kk < AE_LB_C / 16; ++kk)
          umma_ss_w(tmem + TM_DH, umma_step_mn(mQ, kk), umma_step_mn(mDO2, kk), id_mnmn_dv, (it > 0) | (kk > 0));
        ok = mbar_wait_w(&bars->pds_full, par, ctl, args.status, 74) && mbar_wait_w(&bars->full_h, par, ctl, args.status, 84);
        if (!ok) break;
        tc_fence_after_sync();
        // dq: the inter-chunk part over A (the copy of dO whose rows already carry exp(g_i): no row scaling), the
        // intra-chunk part on top, back to back
#pragma unroll
        for (int kk = 0; kk < AE_LIN_DV / 16; ++kk)
          umma_ss_w(tmem + TM_R0, umma_step_k(kDO2, kk, 128), umma_step_k(kHC, kk, 128), id_kk_128, kk > 0);
#pragma unroll
        for (int kk = 0; kk < AE_LB_C / 16; ++kk)
          umma_ss_w(tmem + TM_R0, umma_step_k(kDS, kk, 128), umma_step_mn(mK, kk), id_kmn_128, 1);
        ok = mbar_wait_w(&bars->scaled_done, par, ctl, args.status, 75);
        if (!ok) break;
        tc_fence_after_sync();
        // intra-chunk parts of dk and dv on top of the scaled inter-chunk parts
#pragma unroll
        for (int kk = 0; kk < AE_LB_C / 16; ++kk)
          umma_ss_w(tmem + TM_R2, umma_step_mn(mDS, kk), umma_step_mn(mQ, kk), id_mnmn_128, 1);
#pragma unroll
        for (int kk = 0; kk < AE_LB_C / 16; ++kk)
          umma_ss_w(tmem + TM_DV, umma_step_mn(mP, kk), umma_step_mn(mDO, kk), id_mnmn_dv, 1);
        umma_commit_w(&bars->out_full);
      }
    }
  } else {
    // =============================== row threads ================================
    const u32 r = threadIdx.x & 127;
    const u32 lane_base = ((warp & 3) * 32) << 16;
    const u32 wg = warp >> 2;  // 0: the group that also runs phases A, B, C, E and the suffix sums
    float* xg = (float*)(smem + AE_LB_SMEM_XG);
    const i64 bh = (i64)b * args.H + h;
    const float* a_row = args.a + bh * args.T;
    float carry = 0.f;  // sum of dG over all later chunks = <dH, h> at the boundary to the next chunk
    bool ok = true;
    // this thread's log-decay of the chunk at hand, requested one chunk ahead (the load would otherwise sit at the top
    // of every chunk's chain)
    float a_next = ((n_chunks - 1) * AE_LB_C + (int)r) < args.T ? a_row[(n_chunks - 1) * AE_LB_C + (int)r] : 0.f;
    // a decay mod of the form decay * custom[heads] (applied where the prefetched value is used): da leaves as the
    // gradient of the decay as passed, and sum_t (gradient of the scaled decay) * decay is the gradient of the scale
    const float asc = args.ascale ? args.ascale[h] : 1.f;
    float acc_a = 0.f, araw_nxt = 0.f, araw_pend = 0.f;
#if AE_LB_MODS
    // the row scale of v, requested a chunk ahead like the log-decay; the raw bits are kept until they are used
    // (converting at once would wait for the load right here)
    const bool vs16 = args.vscale_16 != 0;
    auto load_vs = [&](int tt) -> u32 {
      if (tt < 0 || tt >= args.T) return 0u;
      return vs16 ? (u32)((const u16*)args.vscale)[bh * args.T + tt] : ((const u32*)args.vscale)[bh * args.T + tt];
    };
    u32 vs_next = load_vs((n_chunks - 1) * AE_LB_C + (int)r);
    const float dsk = args.dskip[h];
    float acc_o = 0.f;  // this thread's share of <dO, x> over all chunks
#endif
    // The two scans over the chunk's steps (cumulative log-decay; suffix sums of dG) are shuffles, shared-memory round
    // trips and a barrier of the first group.  At the chunk boundary they sat in the burst of bulk copies (the chunk's
    // output tiles leave, the next chunk's tiles arrive) and took 2700 clk of the chain for a few dozen instructions.
    // Both now run in the idle time before the output phase: the cumulative sum of the NEXT chunk into the other
    // buffer, the suffix sums of the chunk BEFORE from values kept in registers.
    auto cum_sum = [&](float g, float* gb) -> float {  // first group only
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const float n = __shfl_up_sync(0xffffffffu, g, o);
        if (lane >= (u32)o) g += n;
      }
      if (lane == 31) misc[warp & 3] = g;
      named_bar_sync(1, 128);
      float pre = 0.f;
#pragma unroll
      for (int w = 0; w < 3; ++w)
        if ((u32)w < (warp & 3)) pre += misc[w];
      g += pre;
      gb[r] = g;
      return g;  // the others read gb[] after the barrier at the top of the chunk
    };
    float dg_pend = 0.f;
    int t_pend = 0;
    bool store_pend = false;
    auto finish_da = [&](u32 hp) {  // first group only: da of the chunk whose dG is in dg_pend, <dH, h> sums in misc[8 + hp * 8 ..]
      float sfx = dg_pend;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const float n = __shfl_down_sync(0xffffffffu, sfx, o);
        if (lane + (u32)o < 32) sfx += n;
      }
      if (lane == 0) misc[4 + (warp & 3)] = sfx;
      named_bar_sync(1, 128);
      float after = 0.f, next_carry = 0.f;
#pragma unroll
      for (int w = 0; w < 4; ++w)
        if ((u32)w > (warp & 3)) after += misc[4 + w];
#pragma unroll
      for (int w = 0; w < AE_LB_ROWW; ++w) next_carry += misc[8 + hp * 8 + w];
      if (store_pend) {
        const float da = sfx + after + carry;
        args.da[bh * args.T + t_pend] = da * asc;
        acc_a = fmaf(da, araw_pend, acc_a);
      }
      carry = next_carry;
    };
    float g_nxt = 0.f;
    if (wg == 0) {
      g_nxt = cum_sum(a_next * asc, gs);
      araw_nxt = a_next;
      a_next = n_chunks >= 2 ? a_row[(n_chunks - 2) * AE_LB_C + (int)r] : 0.f;  // chunks before the last one are full
    }
    for (int it = 0; it < n_chunks; ++it) {
      const int c = n_chunks - 1 - it;
      const u32 par = it & 1;
      const int t = c * AE_LB_C + (int)r;
      const bool row_ok = t < args.T;
      float* gc = gs + par * 128;  // this chunk's cumulative log-decays
      AE_TRL(warp == 0, 1, it * 16 + 0)
      float g = g_nxt, eg = 0.f, wj = 0.f;
      const float araw_cur = araw_nxt;  // this row's decay as passed (first group)
#if AE_LB_MODS
      const float vsc = vs16 ? unpack_lo<AE_BF16>(vs_next) : __uint_as_float(vs_next);
      vs_next = load_vs(t - AE_LB_C);
      uint4 dos[AE_LIN_DV / 8 / AE_LB_NWG];  // this thread's piece of the dO row, for the output phase
#endif
      // ---- A: the chunk's cumulative log-decays were summed during the chunk before ------------------
#if AE_LB_NWG > 1
      named_bar_sync(2, 128 * AE_LB_NWG);
      if (wg != 0) g = gc[r];
#else
      named_bar_sync(1, 128);
#endif
      const float g_last = gc[AE_LB_C - 1];
      eg = ae_exp(g);
      wj = ae_exp(g_last - g);
      AE_TRL(warp == 0, 1, it * 16 + 1)
      // ---- B: dH' -> 16-bit copy, then decay dH in place ------------------------------------------
      {
        u8* dhb = smem + AE_LB_SMEM_DHB;
        if (it > 0) {
          const float dec = ae_exp(g_last);
#pragma unroll
          for (int c2 = 0; c2 < AE_LIN_DV / 32 / AE_LB_NWG; ++c2) {
            const int cc = (int)wg * (AE_LIN_DV / 32 / AE_LB_NWG) + c2;
            float f[32];
            u32 w[32];
            tmem_ld_f32x32(tmem + TM_DH + lane_base + cc * 32, f);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              uint4 pk;
              pk.x = pack2<AE_BF16>(f[i * 8 + 0], f[i * 8 + 1]);
              pk.y = pack2<AE_BF16>(f[i * 8 + 2], f[i * 8 + 3]);
              pk.z = pack2<AE_BF16>(f[i * 8 + 4], f[i * 8 + 5]);
              pk.w = pack2<AE_BF16>(f[i * 8 + 6], f[i * 8 + 7]);
              *(uint4*)(dhb + tile_off(r, cc * 32 + i * 8, AE_LB_DK)) = pk;
            }
#pragma unroll
            for (int i = 0; i < 32; ++i) w[i] = __float_as_uint(f[i] * dec);
            tmem_st32(tmem + TM_DH + lane_base + cc * 32, w);
          }
        } else {
#pragma unroll
          for (int c2 = 0; c2 < AE_LIN_DV / 8 / AE_LB_NWG; ++c2) {
            const int ch = (int)wg * (AE_LIN_DV / 8 / AE_LB_NWG) + c2;
            *(uint4*)(dhb + tile_off(r, ch * 8, AE_LB_DK)) = make_uint4(0, 0, 0, 0);
          }
        }
      }
      AE_TRL(warp == 0, 1, it * 16 + 2)
      // ---- C: dO2 = dO * exp(g) -----------------------------------------------------------------------
      ok = ok && mbar_wait(&bars->full_vd, par, ctl, args.status, 76);
      AE_TRL(warp == 0, 1, it * 16 + 3)
      // the bulk store of the chunk before's dv has read the dO-copy tile this phase writes again
      if (it > 0) ok = ok && mbar_wait(&bars->o_free, (it - 1) & 1, ctl, args.status, 81);
      {
        const u8* dsrc = smem + AE_LB_SMEM_DO;
        u8* d2 = smem + AE_LB_SMEM_DO2;
#pragma unroll
        for (int c2 = 0; c2 < AE_LIN_DV / 8 / AE_LB_NWG; ++c2) {
          const int ch = (int)wg * (AE_LIN_DV / 8 / AE_LB_NWG) + c2;
          const u32 off = tile_off(r, ch * 8, AE_LB_C);
          uint4 x = *(const uint4*)(dsrc + off);
#if AE_LB_MODS
          dos[c2] = x;
#endif
          u32* xw = (u32*)&x;
#pragma unroll
          for (int i = 0; i < 4; ++i)
            xw[i] = pack2<AE_BF16>(unpack_lo<AE_BF16>(xw[i]) * eg, unpack_hi<AE_BF16>(xw[i]) * eg);
          *(uint4*)(d2 + off) = x;
        }
      }
      tc_wait_st();
      fence_proxy_async_smem();
      tc_fence_before_sync();
      mbar_arrive_warp(&bars->prep_done);
      AE_TRL(warp == 0, 1, it * 16 + 4)
      // ---- D: P = E o A, dS = E o dPr -> shared memory ------------------------------------------------
      ok = ok && mbar_wait(&bars->s_full, par, ctl, args.status, 77);
      if (it > 0) ok = ok && mbar_wait(&bars->o_free2, (it - 1) & 1, ctl, args.status, 87);  // P and dS tiles are free
      AE_TRL(warp == 0, 1, it * 16 + 5)
      tc_fence_after_sync();
      {
        u8* pt = smem + AE_LB_SMEM_P;
        u8* dst = smem + AE_LB_SMEM_DS;
#pragma unroll
        for (int c2 = 0; c2 < AE_LB_C / 32 / AE_LB_NWG; ++c2) {
          const int cc = (int)wg * (AE_LB_C / 32 / AE_LB_NWG) + c2;  // this group's 32-column blocks
          float av[32], dv[32];
          tmem_ld_2xf32x32(tmem + TM_R0 + lane_base + cc * 32, tmem + TM_R1 + lane_base + cc * 32, av, dv);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            u32 pw[4], dw[4];
#pragma unroll
            for (int e2 = 0; e2 < 4; ++e2) {
              const int j0 = cc * 32 + i * 8 + e2 * 2;
              const float2 gj = *(const float2*)(gc + j0);
              const float e0 = ((u32)j0 <= r) ? ae_exp(g - gj.x) : 0.f;
              const float e1 = ((u32)(j0 + 1) <= r) ? ae_exp(g - gj.y) : 0.f;
              pw[e2] = pack2<AE_BF16>(av[i * 8 + e2 * 2] * e0, av[i * 8 + e2 * 2 + 1] * e1);
              dw[e2] = pack2<AE_BF16>(dv[i * 8 + e2 * 2] * e0, dv[i * 8 + e2 * 2 + 1] * e1);
            }
            const u32 off = tile_off(r, cc * 32 + i * 8, AE_LB_C);
            *(uint4*)(pt + off) = make_uint4(pw[0], pw[1], pw[2], pw[3]);
            *(uint4*)(dst + off) = make_uint4(dw[0], dw[1], dw[2], dw[3]);
          }
        }
      }
      fence_proxy_async_smem();
      tc_fence_before_sync();
      mbar_arrive_warp(&bars->pds_full);
      AE_TRL(warp == 0, 1, it * 16 + 6)
      // ---- E: row scaling of the inter-chunk parts ------------------------------------------------------
      {
      ok = ok && mbar_wait(&bars->inter_full, par, ctl, args.status, 78);
      AE_TRL(warp == 0, 1, it * 16 + 7)
      tc_fence_after_sync();
#pragma unroll
      for (int which = 1; which < 3; ++which) {  // R2 (dk) and DV by w_j; dq needs no scaling
        const u32 base = tmem + lane_base + (which == 1 ? TM_R2 : TM_DV);
        const int ncol = which == 2 ? AE_LIN_DV : 128;
        const float sc = wj;
#pragma unroll
        for (int c2 = 0; c2 < ncol / 32 / AE_LB_NWG; ++c2) {
          const int cc = (int)wg * (ncol / 32 / AE_LB_NWG) + c2;
          float f[32];
          u32 w[32];
          tmem_ld_f32x32(base + cc * 32, f);
#pragma unroll
          for (int i = 0; i < 32; ++i) w[i] = __float_as_uint(f[i] * sc);
          tmem_st32(base + cc * 32, w);
        }
      }
      tc_wait_st();
      tc_fence_before_sync();
      mbar_arrive_warp(&bars->scaled_done);
      }
      AE_TRL(warp == 0, 1, it * 16 + 8)
      if (wg == 0) {  // under the chunk's last MMAs
        if (it > 0) finish_da((it - 1) & 1);
        if (c > 0) {
          g_nxt = cum_sum(a_next * asc, gs + (par ^ 1) * 128);
          araw_nxt = a_next;
          a_next = c >= 2 ? a_row[t - 2 * AE_LB_C] : 0.f;
        }
      }
      AE_TRL(warp == 0, 1, it * 16 + 13)
      // ---- F: outputs -------------------------------------------------------------------------------------
      ok = ok && mbar_wait(&bars->out_full, par, ctl, args.status, 79);
      // q, k and the start state are read below with ordinary loads: this thread has to have seen their barriers too
      ok = ok && mbar_wait(&bars->full, par, ctl, args.status, 85) && mbar_wait(&bars->full_h, par, ctl, args.status, 86);
      AE_TRL(warp == 0, 1, it * 16 + 9)
      tc_fence_after_sync();
      float dg = 0.f;
      {
        const bool store = ok && row_ok;
        // rows past T are clipped by the bulk stores
        u8* dv_tile = smem + AE_LB_SMEM_DO2;
#if AE_LB_MODS
        float dot_v = 0.f, dot_o = 0.f;
#endif
#pragma unroll
        for (int which = 0; which < 2; ++which) {
          const u8* src = smem + (which == 0 ? AE_LB_SMEM_Q : AE_LB_SMEM_K);
          u8* otile = smem + (which == 0 ? AE_LB_SMEM_P : AE_LB_SMEM_DS);
          float dot = 0.f;
#pragma unroll
          for (int c2 = 0; c2 < AE_LB_DK / 32 / AE_LB_NWG; ++c2) {
            const int cc = (int)wg * (AE_LB_DK / 32 / AE_LB_NWG) + c2;
            float f[32];
            tmem_ld_f32x32(tmem + (which == 0 ? TM_R0 : TM_R2) + lane_base + cc * 32, f);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const uint4 x = *(const uint4*)(src + tile_off(r, cc * 32 + i * 8, AE_LB_C));
              const u32 xw[4] = {x.x, x.y, x.z, x.w};
              uint4 pk;
              u32* pw = (u32*)&pk;
#pragma unroll
              for (int e2 = 0; e2 < 4; ++e2) {
                dot += unpack_lo<AE_BF16>(xw[e2]) * f[i * 8 + e2 * 2] + unpack_hi<AE_BF16>(xw[e2]) * f[i * 8 + e2 * 2 + 1];
                pw[e2] = pack2<AE_BF16>(f[i * 8 + e2 * 2], f[i * 8 + e2 * 2 + 1]);
              }
              *(uint4*)(otile + tile_off(r, cc * 32 + i * 8, AE_LB_C)) = pk;
            }
          }
          dg += which == 0 ? dot : -dot;
        }
        tc_fence_before_sync();
        mbar_arrive_warp(&bars->qk_free);  // last read of the q and k tiles (their MMAs completed before this phase)
#pragma unroll
        for (int c2 = 0; c2 < AE_LIN_DV / 32 / AE_LB_NWG; ++c2) {
          const int cc = (int)wg * (AE_LIN_DV / 32 / AE_LB_NWG) + c2;
          float f[32];
          tmem_ld_f32x32(tmem + TM_DV + lane_base + cc * 32, f);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint4 pk;
            pk.x = pack2<AE_BF16>(f[i * 8 + 0], f[i * 8 + 1]);
            pk.y = pack2<AE_BF16>(f[i * 8 + 2], f[i * 8 + 3]);
            pk.z = pack2<AE_BF16>(f[i * 8 + 4], f[i * 8 + 5]);
            pk.w = pack2<AE_BF16>(f[i * 8 + 6], f[i * 8 + 7]);
#if AE_LB_MODS
            // gx = dv * s + dO * d[h] over the 16-bit dv; <dv, x> and <dO, x> on the way
            const uint4 xr = *(const uint4*)(smem + AE_LB_SMEM_X + tile_off(r, cc * 32 + i * 8, AE_LB_C));
            const uint4 gr = dos[c2 * 4 + i];
            const u32 xw[4] = {xr.x, xr.y, xr.z, xr.w}, gw[4] = {gr.x, gr.y, gr.z, gr.w};
            u32* pw = (u32*)&pk;
#pragma unroll
            for (int e2 = 0; e2 < 4; ++e2) {
              const float v0 = unpack_lo<AE_BF16>(pw[e2]), v1 = unpack_hi<AE_BF16>(pw[e2]);
              const float g0 = unpack_lo<AE_BF16>(gw[e2]), g1 = unpack_hi<AE_BF16>(gw[e2]);
              const float x0 = unpack_lo<AE_BF16>(xw[e2]), x1 = unpack_hi<AE_BF16>(xw[e2]);
              dot_v = fmaf(v0, x0, dot_v);
              dot_v = fmaf(v1, x1, dot_v);
              dot_o = fmaf(g0, x0, dot_o);
              dot_o = fmaf(g1, x1, dot_o);
              pw[e2] = pack2<AE_BF16>(fmaf(v0, vsc, g0 * dsk), fmaf(v1, vsc, g1 * dsk));
            }
#endif
            *(uint4*)(dv_tile + tile_off(r, cc * 32 + i * 8, AE_LB_C)) = pk;
          }
        }
#if AE_LB_MODS
        if (row_ok) acc_o += dot_o;
#endif
        fence_proxy_async_smem();
        mbar_arrive_warp(&bars->o_ready);
        AE_TRL(warp == 0, 1, it * 16 + 10)
        if (!row_ok) dg = 0.f;
        // <dH, h> of this chunk (row r of both), the carry for the chunk before it
        float hd = 0.f;
        {
          const u8* hc = smem + AE_LB_SMEM_HC;
#pragma unroll
          for (int c2 = 0; c2 < AE_LIN_DV / 32 / AE_LB_NWG; ++c2) {
            const int cc = (int)wg * (AE_LIN_DV / 32 / AE_LB_NWG) + c2;
            float f[32];
            tmem_ld_f32x32(tmem + TM_DH + lane_base + cc * 32, f);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const uint4 x = *(const uint4*)(hc + tile_off(r, cc * 32 + i * 8, AE_LB_DK));
              const u32 xw[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
              for (int e2 = 0; e2 < 4; ++e2)
                hd += unpack_lo<AE_BF16>(xw[e2]) * f[i * 8 + e2 * 2] + unpack_hi<AE_BF16>(xw[e2]) * f[i * 8 + e2 * 2 + 1];
            }
          }
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) hd += __shfl_xor_sync(0xffffffffu, hd, o);
          if (lane == 0) misc[8 + par * 8 + warp] = hd;  // one slot per row warp of either group
        }
        // last read of this chunk's tiles and accumulators: the next chunk's loads start under the sums below
        tc_fence_before_sync();
        mbar_arrive_warp(&bars->empty);
        AE_TRL(warp == 0, 1, it * 16 + 11)
#if AE_LB_NWG > 1
        // the second group's share of q.dq - k.dk (and its <dH, h> slot, written above) reaches the first group
        if (wg != 0) xg[r] = dg;
#if AE_LB_MODS
        if (wg != 0) gc[r] = dot_v;  // the chunk's cumulative decays are dead since the P / dS pass
#endif
        named_bar_sync(3, 128 * AE_LB_NWG);
        AE_TRL(warp == 0, 1, it * 16 + 12)
        if (wg != 0) continue;
        dg += xg[r];
#if AE_LB_MODS
        dot_v += gc[r];
#endif
#endif
#if AE_LB_MODS
        if (store) {
          if (vs16) ((u16*)args.gs)[bh * args.T + t] = (u16)(pack2<AE_BF16>(dot_v, 0.f) & 0xffffu);
          else ((float*)args.gs)[bh * args.T + t] = dot_v;
        }
#endif
        // the suffix sums of dG (-> da) follow under the next chunk's last MMAs
        dg_pend = dg;
        araw_pend = araw_cur;
        t_pend = t;
        store_pend = store;
      }
    }
    if (wg == 0) {
      finish_da((n_chunks - 1) & 1);
      if (args.ascale) {  // gradient of the decay scale of this (batch, head)
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) acc_a += __shfl_xor_sync(0xffffffffu, acc_a, o);
        if (lane == 0) misc[warp & 3] = acc_a;
        named_bar_sync(1, 128);
        if (threadIdx.x == 0) args.gasc[bh] = misc[0] + misc[1] + misc[2] + misc[3];
      }
    }
#if AE_LB_MODS
    // <dO, x> of this (batch, head): the row threads' sums meet in shared memory
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc_o += __shfl_xor_sync(0xffffffffu, acc_o, o);
    if (lane == 0) misc[24 + warp] = acc_o;
    named_bar_sync(4, 128 * AE_LB_NWG);
    if (threadIdx.x == 0) {
      float tot = 0.f;
#pragma unroll
      for (int w = 0; w < AE_LB_ROWW; ++w) tot += misc[24 + w];
      args.gd[bh] = tot;
    }
#endif
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == AE_LB_ROWW + 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, 512);
  }
}
