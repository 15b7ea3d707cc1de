// Chunked linear-attention / SSD scan, forward, for sm_100a.  Replaces the reference's
// `chunk_local_cumsum_scalar_kernel` + `chunk_fwd_h` + `chunk_o` kernels
// (attention_engine/core/template/tl_template/linear/linear_tl.py:25-49, 114-233, 283-410) with one
// kernel that does not need the per-chunk states in HBM (it writes them, 16-bit, only when the caller asks for them for
// the backward: args.h_out; the reference always stores and re-reads them).
//
// Recurrence per (batch, head), with a_t <= 0 the log-decay of step t:
//     S_t = exp(a_t) S_{t-1} + k_t^T v_t ,      o_t = q_t S_t
// One CTA owns one (batch, head) and walks its chunks of 128 steps in order; the state S [DK x DV]
// lives in TMEM as an fp32 accumulator for the whole sequence.  Per chunk, with g the inclusive
// cumulative sum of a inside the chunk:
//     A   = q k^T                                   (SS MMA)
//     Oi  = q h                                     (SS MMA, h = bf16 copy of the incoming state)
//     H   = exp(g_last) H + k^T (v * exp(g_last - g))    (SS MMA, k read MN-major as A)
//     row threads: P_ij = A_ij exp(g_i - g_j) [i >= j] -> TMEM ; Oi_i *= exp(g_i)
//     O   = Oi + P v                                (TS MMA)
// The exponent g_i - g_j is only evaluated for j <= i (where it is <= 0), so nothing overflows; the
// reference evaluates it everywhere and masks afterwards (linear_tl.py:372-378).
// Roles: warps 0-3 row threads (thread r = step r of the chunk = state row r), warp 4 TMA producer,
// warp 5 MMA issuer.  Expects AE_BF16, AE_LIN_DV (64 or 128), AE_LIN_STAGES; DK is 128.
//
// AE_LIN_MODS = 1 builds the Mamba2 block's two mods into the kernel (the reference runs them as eager PyTorch
// statements around its kernels, linear_tl.py:1136-1144; mamba2_ngroup1.py:31-33 is `v * dt`): the tensor behind tm_v
// is x, the scan runs on v = x * vscale[b, h, t] (the row thread that rescales its row of the V tile for the state
// update anyway also scales it in place for P v and writes v out for the backward), and the output row gets
// + x * dskip[h] from a copy of the raw row kept in shared memory.  Two streaming passes over x and one over o less.
#ifndef AE_LIN_MODS
#define AE_LIN_MODS 0
#endif

#ifdef AE_TRACE  // clock stamps of CTA (0, 0)'s row warp 0 into the status buffer (experiments)
#define AE_TRL(cond, region, slot) \
  if (blockIdx.x == 0 && blockIdx.y == 0 && lane == 0 && (cond) && (slot) < 4096) \
    args.status[64 + (region) * 4096 + (slot)] = (u32)clock64();
#else
#define AE_TRL(cond, region, slot)
#endif
// AE_LIN_NWG = 2: a second row warpgroup takes half of the columns of every row phase (same rows, other 32-column
// blocks); the cumulative sum stays with the first group, which runs it one chunk ahead into the other of two buffers.
// The groups meet at named barrier 2 at the top of every chunk.  The second group keeps its P in the second half of
// its own score columns (16-bit pairs at column 96 ...), so neither group writes TMEM columns the other still reads.
#ifndef AE_LIN_NWG
#define AE_LIN_NWG 1
#endif
#define AE_LIN_ROWW (4 * AE_LIN_NWG)  // row warps; then the TMA warp and the MMA warp
#define AE_LIN_C 128
#define AE_LIN_DK 128

#define AE_LIN_Q_BYTES (AE_LIN_C * AE_LIN_DK * 2)
#define AE_LIN_V_BYTES (AE_LIN_C * AE_LIN_DV * 2)
#define AE_LIN_STAGE_BYTES (2 * AE_LIN_Q_BYTES + AE_LIN_V_BYTES)
#define AE_LIN_SMEM_STAGE 0
#define AE_LIN_SMEM_V2 (AE_LIN_STAGES * AE_LIN_STAGE_BYTES)
#define AE_LIN_SMEM_H (AE_LIN_SMEM_V2 + AE_LIN_V_BYTES)
#define AE_LIN_SMEM_G (AE_LIN_SMEM_H + AE_LIN_DK * AE_LIN_DV * 2)
#define AE_LIN_SMEM_BAR (AE_LIN_SMEM_G + 1024)
// Output staging tile [128 rows][DV] 16-bit in the layout of a 128-byte-swizzled TMA box (64-column blocks): row r is
// written by thread r alone and the tile leaves through one bulk store per chunk.  In the AE_LIN_MODS build the same
// rows first hold the raw x of the chunk (phase C) for the skip term of phase F.
#define AE_LIN_SMEM_Y (AE_LIN_SMEM_BAR + 2048)

struct AeLinBars {
  u64 full[AE_LIN_STAGES];
  u64 empty[AE_LIN_STAGES];
  u64 s_full;
  u64 prep_done;
  u64 oi_full;
  u64 p_full;
  u64 o_done;
  u64 h_done;
  u64 hb_free;  // the bulk store of the previous chunk's state copy has read it (h_out builds)
  u64 y_full;   // the chunk's output tile is in shared memory
  u64 y_free;   // ... and its bulk store has read it
  AeCtaCtl ctl;
};

extern "C" __global__ void __launch_bounds__(AE_LIN_ROWW * 32 + 64, 1) ae_linear_fwd(const __grid_constant__ AeLinearArgs args) {
  extern __shared__ u8 smem_raw[];
  u8* smem = smem_align1024(smem_raw);
  AeLinBars* bars = (AeLinBars*)(smem + AE_LIN_SMEM_BAR);
  float* gs = (float*)(smem + AE_LIN_SMEM_G);  // [128] cumulative log-decay of the chunk, [128..131] warp totals
  AeCtaCtl* ctl = &bars->ctl;
  const u32 warp = threadIdx.x >> 5;
  const u32 lane = threadIdx.x & 31;
  const int h = blockIdx.x;
  const int b = blockIdx.y;
  const int hq = h / (args.H / args.HQ);
  const int hk = h / (args.H / args.HK);
  const int n_chunks = (args.T + AE_LIN_C - 1) / AE_LIN_C;

  if (threadIdx.x == 0) {
    ctl->abort = 0;
    for (int i = 0; i < AE_LIN_STAGES; ++i) {
      mbar_init(&bars->full[i], 1);
      mbar_init(&bars->empty[i], 1);
    }
    mbar_init(&bars->s_full, 1);
    mbar_init(&bars->prep_done, AE_LIN_ROWW);
    mbar_init(&bars->oi_full, 1);
    mbar_init(&bars->p_full, AE_LIN_ROWW);
    mbar_init(&bars->o_done, 1);
    mbar_init(&bars->h_done, 1);
    mbar_init(&bars->hb_free, 1);
    mbar_init(&bars->y_full, AE_LIN_ROWW);
    mbar_init(&bars->y_free, 1);
    mbar_fence_init();
  }
  if (warp == AE_LIN_ROWW + 1) {
    tmem_alloc(&ctl->tmem_base, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const u32 tmem = ctl->tmem_base;
  const u32 TM_S = 0, TM_O = 128, TM_H = 128 + AE_LIN_DV;

  if (warp == AE_LIN_ROWW) {
    // =============================== TMA producer ===============================
    if (lane == 0) {
      tma_prefetch_desc(&args.tm_q);
      tma_prefetch_desc(&args.tm_k);
      tma_prefetch_desc(&args.tm_v);
      // Outputs that are whole shared-memory tiles leave through bulk stores issued here, one chunk behind the loads,
      // instead of through per-row stores of the row threads (who are this kernel's critical path): the 16-bit copy of
      // each chunk's incoming state (h_out) and, in the build with the mods inside, the scaled V tile (v_out).
      const bool st_h = args.h_out != nullptr;
      const bool st_v = AE_LIN_MODS && args.v_out != nullptr;
      if (st_h) tma_prefetch_desc(&args.tm_hout);
      if (st_v) tma_prefetch_desc(&args.tm_vout);
      tma_prefetch_desc(&args.tm_o);
      bool ok = true;
      for (int c = 0; c <= n_chunks && ok; ++c) {
        // first the stores of chunk c - 1, then the loads of chunk c: the row threads cannot reach prep_done of chunk c
        // without those loads, so the parity wait below can never be two phases behind
        if ((st_h || st_v) && c >= 1) {
          const int cs = c - 1;  // its row threads have written and fenced the state copy and the scaled V tile
          ok = mbar_wait(&bars->prep_done, cs & 1, ctl, args.status, 60);
          if (!ok) break;
          if (st_h && cs >= 1) {
            for (int dh = 0; dh < AE_LIN_DV / 64; ++dh)
              tma_store_3d(&args.tm_hout, smem + AE_LIN_SMEM_H + dh * (AE_LIN_DK * 128), dh * 64, 0,
                           (b * args.H + h) * n_chunks + cs);
          }
          if (st_v) {
            const u8* vt = smem + AE_LIN_SMEM_STAGE + (cs % AE_LIN_STAGES) * AE_LIN_STAGE_BYTES + 2 * AE_LIN_Q_BYTES;
            for (int dh = 0; dh < AE_LIN_DV / 64; ++dh)
              tma_store_4d(&args.tm_vout, vt + dh * (AE_LIN_C * 128), dh * 64, cs * AE_LIN_C, h, b);
          }
          tma_store_commit();
          if (st_h && cs >= 1) {
            tma_store_wait_read();  // the state copy is rewritten by the row threads of the next chunk
            mbar_arrive(&bars->hb_free);
          }
        }
        if (c < n_chunks) {
          const int stage = c % AE_LIN_STAGES;
          const u32 par = ((c / AE_LIN_STAGES) & 1) ^ 1;
          if (!mbar_wait(&bars->empty[stage], par, ctl, args.status, 51)) break;
          if (st_v) tma_store_wait_read();  // no bulk store still reads the V tile about to be refilled
          u8* st = smem + AE_LIN_SMEM_STAGE + stage * AE_LIN_STAGE_BYTES;
          mbar_arrive_expect_tx(&bars->full[stage], AE_LIN_STAGE_BYTES);
          for (int dh = 0; dh < AE_LIN_DK / 64; ++dh) {
            tma_load_4d(st + dh * (AE_LIN_C * 128), &args.tm_q, &bars->full[stage], dh * 64, c * AE_LIN_C, hq, b);
            tma_load_4d(st + AE_LIN_Q_BYTES + dh * (AE_LIN_C * 128), &args.tm_k, &bars->full[stage], dh * 64,
                        c * AE_LIN_C, hk, b);
          }
          for (int dh = 0; dh < AE_LIN_DV / 64; ++dh)
            tma_load_4d(st + 2 * AE_LIN_Q_BYTES + dh * (AE_LIN_C * 128), &args.tm_v, &bars->full[stage], dh * 64,
                        c * AE_LIN_C, h, b);
        }
        if (c >= 1) {
          // the output tile of chunk c - 1 (complete at the end of that chunk; the loads of chunk c are already out)
          const int cy = c - 1;
          ok = mbar_wait(&bars->y_full, cy & 1, ctl, args.status, 62);
          if (!ok) break;
          for (int dh = 0; dh < AE_LIN_DV / 64; ++dh)
            tma_store_4d(&args.tm_o, smem + AE_LIN_SMEM_Y + dh * (AE_LIN_C * 128), dh * 64, cy * AE_LIN_C, h, b);
          tma_store_commit();
          tma_store_wait_read();  // the rows of the next chunk write the tile again
          mbar_arrive(&bars->y_free);
        }
      }
      tma_store_wait_read();  // the tiles belong to this CTA until the bulk engine has read them
    }
  } else if (warp == AE_LIN_ROWW + 1) {
    // =============================== MMA issuer =================================
    if (n_chunks > 0) {  // all 32 lanes run the control flow; MMAs and commits are issued by an elected lane
      const u32 idesc_s = umma_idesc_f16(128, AE_LIN_C, AE_BF16, 0, 0);          // q k^T
      const u32 idesc_oi = umma_idesc_f16(128, AE_LIN_DV, AE_BF16, 0, 1);        // q h, P v
      const u32 idesc_h = umma_idesc_f16(AE_LIN_DK, AE_LIN_DV, AE_BF16, 1, 1);   // k^T v'
      const u32 v2_addr = smem_u32(smem + AE_LIN_SMEM_V2);
      const u32 h_addr = smem_u32(smem + AE_LIN_SMEM_H);
      const u32 st_addr = smem_u32(smem + AE_LIN_SMEM_STAGE);
      const u64 bq = umma_base_k(st_addr), bk = umma_base_k(st_addr + AE_LIN_Q_BYTES);
      const u64 bk_mn = umma_base_mn(st_addr + AE_LIN_Q_BYTES, AE_LIN_C);
      const u64 bv_mn = umma_base_mn(st_addr + 2 * AE_LIN_Q_BYTES, AE_LIN_C);
      const u64 bh_mn = umma_base_mn(h_addr, AE_LIN_DK), bv2_mn = umma_base_mn(v2_addr, AE_LIN_C);
      auto issue_s = [&](int c) -> bool {
        const int stage = c % AE_LIN_STAGES;
        if (!mbar_wait_w(&bars->full[stage], (c / AE_LIN_STAGES) & 1, ctl, args.status, 52)) return false;
        tc_fence_after_sync();
        const u64 so = (u64)((stage * AE_LIN_STAGE_BYTES) >> 4);
#pragma unroll
        for (int kk = 0; kk < AE_LIN_DK / 16; ++kk)
          umma_ss_w(tmem + TM_S, umma_step_k(bq + so, kk, AE_LIN_C), umma_step_k(bk + so, kk, AE_LIN_C), idesc_s, kk > 0);
        umma_commit_w(&bars->s_full);
        return true;
      };
      bool ok = issue_s(0);
      for (int c = 0; c < n_chunks && ok; ++c) {
        const int stage = c % AE_LIN_STAGES;
        const u64 so = (u64)((stage * AE_LIN_STAGE_BYTES) >> 4);
        ok = mbar_wait_w(&bars->prep_done, c & 1, ctl, args.status, 53);
        if (!ok) break;
        tc_fence_after_sync();
        if (c > 0) {
          // Oi = q h   (h: [DK rows][DV contiguous], MN-major B)
#pragma unroll
          for (int kk = 0; kk < AE_LIN_DK / 16; ++kk)
            umma_ss_w(tmem + TM_O, umma_step_k(bq + so, kk, AE_LIN_C), umma_step_mn(bh_mn, kk), idesc_oi, kk > 0);
        }
        umma_commit_w(&bars->oi_full);
        // H (+)= k^T v'   (k tile read MN-major as A: [chunk rows][DK contiguous]; v' likewise as B)
#pragma unroll
        for (int kk = 0; kk < AE_LIN_C / 16; ++kk)
          umma_ss_w(tmem + TM_H, umma_step_mn(bk_mn + so, kk), umma_step_mn(bv2_mn, kk), idesc_h, (c > 0) | (kk > 0));
        umma_commit_w(&bars->h_done);
        ok = mbar_wait_w(&bars->p_full, c & 1, ctl, args.status, 54);
        if (!ok) break;
        tc_fence_after_sync();
#pragma unroll
        for (int kk = 0; kk < AE_LIN_C / 16; ++kk)
          umma_ts_w(tmem + TM_O, tmem + TM_S + kk * 8 + ((AE_LIN_NWG > 1 && kk >= AE_LIN_C / 32) ? 64 : 0),
                    umma_step_mn(bv_mn + so, kk), idesc_oi, (c > 0) | (kk > 0));
        umma_commit_w(&bars->o_done);
        umma_commit_w(&bars->empty[stage]);
        if (c + 1 < n_chunks) ok = issue_s(c + 1);
      }
    }
  } else {
    // =============================== row threads ================================
    const u32 r = threadIdx.x & 127;
    const u32 lane_base = ((warp & 3) * 32) << 16;
    const float* a_row = args.a + ((i64)b * args.H + h) * args.T;
    u8* y_tile = smem + AE_LIN_SMEM_Y;
    // [2][128] column factors of the chunk's decay matrix; like the cumulative log-decays (gs, [2][128]) by chunk parity:
    // the first group fills the next chunk's while the chunk at hand still reads its own
    float* cf_all = (float*)(smem + AE_LIN_SMEM_BAR + 1024);
    float* misc = (float*)(smem + AE_LIN_SMEM_BAR + 512);  // [0..3] warp totals of the cumulative sum
#if AE_LIN_MODS
    const float dsk = args.dskip ? args.dskip[h] : 0.f;
#endif
    bool ok = true;
    // The per-step scalars of a chunk (log-decay; the row scale of v in the AE_LIN_MODS build) are requested one chunk
    // ahead: a global load at the top of every chunk would sit on the chain of dependent phases.
    auto load_a = [&](int tt) { return tt < args.T ? a_row[tt] : 0.f; };
    const u32 wg = warp >> 2;  // 0: the group that also runs the cumulative sum
    float a_next = load_a((int)r);
    // a decay mod of the form decay * custom[heads]; applied where the prefetched value is used, not where it is loaded
    const float asc = args.ascale ? args.ascale[h] : 1.f;
#if AE_LIN_MODS
    // the raw bits are kept until the value is used a chunk later: converting at once would wait for the load right here
    const bool vs16 = args.vscale_16 != 0;
    auto load_vs = [&](int tt) -> u32 {
      if (!args.vscale || tt >= args.T) return vs16 ? (AE_BF16 ? 0x3f80u : 0x3c00u) : 0x3f800000u;  // 1.0
      const i64 si = ((i64)b * args.H + h) * args.T + tt;
      return vs16 ? (u32)((const u16*)args.vscale)[si] : ((const u32*)args.vscale)[si];
    };
    u32 vs_next = load_vs((int)r);
#endif
    // Inclusive cumulative sum of the log-decay over a chunk and the column factors of its decay matrix (first group
    // only).  It runs one chunk ahead, while the P v MMAs of the chunk at hand are under way: at the top of the chunk
    // its shuffles, shared-memory round trips and barrier were 500 to 800 clk of the chain.
    auto cum_sum = [&](float g, float* gb, float* cb) -> float {
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
      // column factor of the decay matrix: exp(g at the end of this step's 32-step block - g) <= 1, see phase D
      cb[r] = ae_exp(__shfl_sync(0xffffffffu, g, 31) - g);
      return g;
    };
    float g_nxt = 0.f;
    if (wg == 0) {
      g_nxt = cum_sum(a_next * asc, gs, cf_all);
      a_next = load_a(AE_LIN_C + (int)r);
    }
    for (int c = 0; c < n_chunks; ++c) {
      const int stage = c % AE_LIN_STAGES;
      const int t = c * AE_LIN_C + (int)r;
      AE_TRL(warp == 0, 1, c * 16 + 0)
      // ---- A: the chunk's cumulative log-decays were summed during the chunk before (cum_sum) -----
      float* gc = gs + (c & 1) * 128;
      const float* cf = cf_all + (c & 1) * 128;
      float g = g_nxt;
#if AE_LIN_MODS
      const float vsc = vs16 ? unpack_lo<AE_BF16>(vs_next) : __uint_as_float(vs_next);
#endif
      // all row threads are done with the chunk before; its sums (written by the first group) are visible
#if AE_LIN_NWG > 1
      named_bar_sync(2, 128 * AE_LIN_NWG);
      if (wg != 0) g = gc[r];
#else
      named_bar_sync(1, 128);
#endif
      const float g_last = gc[AE_LIN_C - 1];
#if AE_LIN_MODS
      vs_next = load_vs(t + AE_LIN_C);
#endif
      AE_TRL(warp == 0, 1, c * 16 + 1)
      // ---- B: incoming state -> bf16 copy for q h, and decay it in place --------------------
      if (c == 0 && args.h_out && wg == 0) {  // the first chunk starts from zero; the later ones leave through the producer's bulk stores
        u16* hrow = (u16*)args.h_out + (((i64)b * args.H + h) * n_chunks * AE_LIN_DK + r) * AE_LIN_DV;
#pragma unroll
        for (int i = 0; i < AE_LIN_DV / 8; ++i) *(uint4*)(hrow + i * 8) = make_uint4(0, 0, 0, 0);
      }
      if (c > 0) {
        // the bulk store of the previous chunk's copy has read it (long ago: it was issued a chunk earlier)
        if (args.h_out && c >= 2) ok = ok && mbar_wait(&bars->hb_free, (c - 2) & 1, ctl, args.status, 61);
        ok = ok && mbar_wait(&bars->h_done, (c - 1) & 1, ctl, args.status, 55);
        tc_fence_after_sync();
        const float dec = ae_exp(g_last);
        u8* hb = smem + AE_LIN_SMEM_H;
#pragma unroll
        for (int c2 = 0; c2 < AE_LIN_DV / 32 / AE_LIN_NWG; ++c2) {
          const int cc = (int)wg * (AE_LIN_DV / 32 / AE_LIN_NWG) + c2;  // this group's 32-column chunks
          float f[32];
          u32 w[32];
          tmem_ld_f32x32(tmem + TM_H + lane_base + cc * 32, f);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint4 pk;
            pk.x = pack2<AE_BF16>(f[i * 8 + 0], f[i * 8 + 1]);
            pk.y = pack2<AE_BF16>(f[i * 8 + 2], f[i * 8 + 3]);
            pk.z = pack2<AE_BF16>(f[i * 8 + 4], f[i * 8 + 5]);
            pk.w = pack2<AE_BF16>(f[i * 8 + 6], f[i * 8 + 7]);
            const u32 col = cc * 32 + i * 8;  // element column of this 16-byte chunk
            *(uint4*)(hb + (col >> 6) * (AE_LIN_DK * 128) + swz128(r, (col & 63) >> 3)) = pk;
          }
#pragma unroll
          for (int i = 0; i < 32; ++i) w[i] = __float_as_uint(f[i] * dec);
          tmem_st32(tmem + TM_H + lane_base + cc * 32, w);
        }
      }
      AE_TRL(warp == 0, 1, c * 16 + 2)
      // ---- C: v' = v * exp(g_last - g), second copy of the v tile ---------------------------
      ok = ok && mbar_wait(&bars->full[stage], (c / AE_LIN_STAGES) & 1, ctl, args.status, 56);
      // the bulk store of the previous chunk's output tile has read it (this chunk writes its rows again)
      if (c > 0) ok = ok && mbar_wait(&bars->y_free, (c - 1) & 1, ctl, args.status, 63);
      AE_TRL(warp == 0, 1, c * 16 + 3)
      {
        const float wgt = ae_exp(g_last - g);
        u8* vt = smem + AE_LIN_SMEM_STAGE + stage * AE_LIN_STAGE_BYTES + 2 * AE_LIN_Q_BYTES;
        u8* v2 = smem + AE_LIN_SMEM_V2;
#if AE_LIN_MODS
        // v = x * vscale: in place for P v (row r of the tile is this thread's alone; the producer's bulk store sends
        // the tile to v_out for the backward); the raw row is kept for the skip term of phase F (the stage may be
        // refilled by then)
#endif
#pragma unroll
        for (int c2 = 0; c2 < AE_LIN_DV / 8 / AE_LIN_NWG; ++c2) {
          const int ch = (int)wg * (AE_LIN_DV / 8 / AE_LIN_NWG) + c2;
          const u32 off = (ch >> 3) * (AE_LIN_C * 128) + swz128(r, ch & 7);
          uint4 x = *(const uint4*)(vt + off);
          u32* xw = (u32*)&x;
#if AE_LIN_MODS
          *(uint4*)(y_tile + off) = x;  // the raw row, for the skip term (same swizzled layout as the V tile)
#pragma unroll
          for (int i = 0; i < 4; ++i)
            xw[i] = pack2<AE_BF16>(unpack_lo<AE_BF16>(xw[i]) * vsc, unpack_hi<AE_BF16>(xw[i]) * vsc);
          *(uint4*)(vt + off) = x;
#endif
#pragma unroll
          for (int i = 0; i < 4; ++i)
            xw[i] = pack2<AE_BF16>(unpack_lo<AE_BF16>(xw[i]) * wgt, unpack_hi<AE_BF16>(xw[i]) * wgt);
          *(uint4*)(v2 + off) = x;
        }
      }
      tc_wait_st();
      fence_proxy_async_smem();
      tc_fence_before_sync();
      mbar_arrive_warp(&bars->prep_done);
      AE_TRL(warp == 0, 1, c * 16 + 4)
      // ---- D: P = A * exp(g_i - g_j) for j <= i -------------------------------------------------
      ok = ok && mbar_wait(&bars->s_full, c & 1, ctl, args.status, 57);
      AE_TRL(warp == 0, 1, c * 16 + 5)
      tc_fence_after_sync();
      {
        // this group's columns: all 128, or its 64 (two 32-column blocks); s[] is indexed from the first of them
        constexpr int NCOL = AE_LIN_C / AE_LIN_NWG;
        const int col0 = (int)wg * NCOL;
        float s[NCOL];
#if AE_LIN_NWG > 1
        tmem_ld_f32x64(tmem + TM_S + lane_base + col0, s);
#else
        tmem_ld_f32x128(tmem + TM_S + lane_base, s);
#endif
        // exp(g_i - g_j) per 32-column block (the rows of a warp share the block that holds their diagonal): blocks
        // left of it take exp(g_i - g_end) * exp(g_end - g_j) with g_end the block's last step - one exponential per
        // row and block, the column factors computed once per chunk in phase A, both <= 1 - the diagonal block is
        // evaluated element by element, the blocks right of it are zero.  128 exponentials per row become 35.
        const u32 wq = warp & 3;
        u32 pk[32];
#pragma unroll
        for (int half = 0; half < NCOL / 64; ++half) {
#pragma unroll
          for (int q2 = 0; q2 < 2; ++q2) {
            const int lc = half * 64 + q2 * 32;  // first of the block's columns in s[]
            const int cc = (col0 + lc) / 32;     // 32-column block of the chunk
            if ((u32)cc < wq) {
              const float rf = ae_exp(g - gc[cc * 32 + 31]);
#pragma unroll
              for (int i = 0; i < 32; i += 4) {
                const float4 c4 = *(const float4*)(cf + cc * 32 + i);
                s[lc + i + 0] *= rf * c4.x;
                s[lc + i + 1] *= rf * c4.y;
                s[lc + i + 2] *= rf * c4.z;
                s[lc + i + 3] *= rf * c4.w;
              }
            } else if ((u32)cc == wq) {
#pragma unroll
              for (int i = 0; i < 32; i += 4) {
                const float4 gj = *(const float4*)(gc + cc * 32 + i);
                const float gv[4] = {gj.x, gj.y, gj.z, gj.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  const int j = cc * 32 + i + e;
                  s[lc + i + e] = ((u32)j <= r) ? s[lc + i + e] * ae_exp(g - gv[e]) : 0.f;
                }
              }
            } else {
#pragma unroll
              for (int i = 0; i < 32; ++i) s[lc + i] = 0.f;
            }
#pragma unroll
            for (int i = 0; i < 16; ++i) pk[q2 * 16 + i] = pack2<AE_BF16>(s[lc + 2 * i], s[lc + 2 * i + 1]);
          }
          // 16-bit pairs: columns half * 32 ... of the region; the second group's at column 96 (inside its own scores)
          tmem_st32(tmem + TM_S + lane_base + (AE_LIN_NWG > 1 ? (int)wg * 96 : half * 32), pk);
        }
      }
      AE_TRL(warp == 0, 1, c * 16 + 6)
      // ---- E: scale the inter-chunk part of O by exp(g_i) ---------------------------------------
      ok = ok && mbar_wait(&bars->oi_full, c & 1, ctl, args.status, 58);
      AE_TRL(warp == 0, 1, c * 16 + 7)
      tc_fence_after_sync();
      if (c > 0) {
        const float eg = ae_exp(g);
#pragma unroll
        for (int c2 = 0; c2 < AE_LIN_DV / 32 / AE_LIN_NWG; ++c2) {
          const int cc = (int)wg * (AE_LIN_DV / 32 / AE_LIN_NWG) + c2;
          float f[32];
          u32 w[32];
          tmem_ld_f32x32(tmem + TM_O + lane_base + cc * 32, f);
#pragma unroll
          for (int i = 0; i < 32; ++i) w[i] = __float_as_uint(f[i] * eg);
          tmem_st32(tmem + TM_O + lane_base + cc * 32, w);
        }
      }
      tc_wait_st();
      tc_fence_before_sync();
      mbar_arrive_warp(&bars->p_full);
      AE_TRL(warp == 0, 1, c * 16 + 8)
      if (wg == 0 && c + 1 < n_chunks) {  // under the P v MMAs
        g_nxt = cum_sum(a_next * asc, gs + ((c + 1) & 1) * 128, cf_all + ((c + 1) & 1) * 128);
        a_next = load_a(t + 2 * AE_LIN_C);
      }
      AE_TRL(warp == 0, 1, c * 16 + 11)
      // ---- F: O rows out ---------------------------------------------------------------------------
      ok = ok && mbar_wait(&bars->o_done, c & 1, ctl, args.status, 59);
      AE_TRL(warp == 0, 1, c * 16 + 9)
      tc_fence_after_sync();
      {
#pragma unroll
        for (int c2 = 0; c2 < AE_LIN_DV / 32 / AE_LIN_NWG; ++c2) {
          const int cc = (int)wg * (AE_LIN_DV / 32 / AE_LIN_NWG) + c2;
          float f[32];
          tmem_ld_f32x32(tmem + TM_O + lane_base + cc * 32, f);
#if AE_LIN_MODS
          if (args.dskip) {  // + x * dskip[h], x = the raw row saved in phase C
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const uint4 xr = *(const uint4*)(y_tile + tile_off(r, cc * 32 + i * 8, AE_LIN_C));
              const u32 xw[4] = {xr.x, xr.y, xr.z, xr.w};
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                f[i * 8 + 2 * e] = fmaf(unpack_lo<AE_BF16>(xw[e]), dsk, f[i * 8 + 2 * e]);
                f[i * 8 + 2 * e + 1] = fmaf(unpack_hi<AE_BF16>(xw[e]), dsk, f[i * 8 + 2 * e + 1]);
              }
            }
          }
#endif
#pragma unroll
          for (int i = 0; i < 4; ++i) {  // rows past T hold zeros or leftovers: the bulk store clips them
            uint4 pk;
            pk.x = pack2<AE_BF16>(f[i * 8 + 0], f[i * 8 + 1]);
            pk.y = pack2<AE_BF16>(f[i * 8 + 2], f[i * 8 + 3]);
            pk.z = pack2<AE_BF16>(f[i * 8 + 4], f[i * 8 + 5]);
            pk.w = pack2<AE_BF16>(f[i * 8 + 6], f[i * 8 + 7]);
            *(uint4*)(y_tile + tile_off(r, cc * 32 + i * 8, AE_LIN_C)) = pk;
          }
        }
      }
      fence_proxy_async_smem();
      tc_fence_before_sync();
      mbar_arrive_warp(&bars->y_full);
      // no barrier here: the next chunk's q h MMA (which overwrites O) waits for every row warp's prep_done arrival,
      // and each warp arrives there only after this point
      AE_TRL(warp == 0, 1, c * 16 + 10)
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == AE_LIN_ROWW + 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, 512);
  }
}
