// Fused attention forward for sm_100a (replaces the reference's generated forward
// kernel, attention_engine/core/template/tl_template/attn/attn_tl.py:76-174, GQA
// variant attn_gqa_tl.py:38-133, block-sparse variant blockattn_tl.py:48-162).
//
// One CTA owns two query tiles of 128 rows of one (batch, q-head) and streams the
// K/V tiles of the matching kv-head once for both.  Roles:
//   warps 0-3 / 4-7 : "row" warpgroups, one per query tile.  Thread i of a group owns
//                     row i: it reads its 128 scores from TMEM, applies mask,
//                     score_mod and the online recurrence in registers (no shuffles),
//                     writes P back to TMEM as 16-bit pairs, rescales O when needed
//                     and runs the epilogue.  (AE_RSPLIT = 2: four row warpgroups, two
//                     threads per row with 64 columns each; the roles below move up.)
//   warp 8          : TMA producer (Q once, K/V ring of AE_STAGES stages).
//   warp 9          : tcgen05.mma issuer; owns the TMEM allocation.
// TMEM columns: S0 | S1 | O0 | O1 (P_t aliases the first half of S_t).
// While one group runs its recurrence the tensor pipe runs the other tile's MMAs.
//
// Expects the generated prelude to define:
//   AE_D, AE_DV (multiples of 64, <= 128), AE_BF16 (0/1), AE_STAGES,
//   AE_MASK_MODE (0 none, 1 causal bounds, 2 block list), AE_NFINAL, AE_O_SCALE_ONE,
//   struct AeRow, ae_mask(), ae_online_fwd() (score_mod fused in), ae_epilogue_o(),
//   ae_final_rowscales().

#define AE_BM 128
#define AE_BN 128
#ifndef AE_DECODE
#define AE_DECODE 0  // 1: split-KV decode (reference: attn_decode_tl.py:34-141 / attn_gqa_decode_tl.py), see AeAttnFwdArgs
#endif
#if AE_DECODE && AE_MASK_MODE != 0 && AE_MASK_MODE != 3
#error "the decode build takes no mask, or an element-wise one (mask mode 3)"
#endif
#ifndef AE_NQ
#define AE_NQ 2  // q tiles held in shared memory; 1 in a decode build whose head units have at most 128 rows (the
                 // space goes to a third K / V stage: more bytes in flight per SM while a tile's chain runs)
#endif
// One q tile per CTA leaves the second S region of TMEM free: the scores of kv tile n go to region n & 1 and the S GEMM
// runs two tiles ahead of P V, so the row threads find the next tile's scores ready when they finish a tile
// (S MMA -> row pass -> P V MMA is no longer one chain per tile).
#define AE_PINGPONG (AE_DECODE && AE_NQ == 1)
// AE_TURNS = 1: the two row warpgroups take turns (named barriers 1 and 2 as a token), so that one group's row pass
// runs while the tensor pipe works on the other tile.  Off by default: measured slower with all exponentials on the
// special-function unit (a group's row pass is then longer than the other tile's two MMAs); a sweep candidate together
// with AE_EXP_POLY_PERIOD.
#ifndef AE_TURNS
#define AE_TURNS 0
#endif
#if AE_TURNS && AE_DECODE
#error "turn-taking is for the two-tile forward"
#endif
// AE_RSPLIT = 2: two threads per score row (warpgroups 2t and 2t + 1 work on q tile t, 64 kv columns each).  A row
// pass is then half as long, which is what lets the two tiles alternate (AE_TURNS) with the tensor pipe busy on one
// while the other's rows run.  Row reductions are completed between the two threads of a row by the generated
// ae_row_xchg (shared memory slot + named barrier 3 + t).  The second half keeps its P in the second half of its own
// score columns (16-bit pairs at column 96 ...), so that no thread writes TMEM columns another thread still reads.
#ifndef AE_RSPLIT
#define AE_RSPLIT 1
#endif
#if AE_RSPLIT != 1 && (AE_RSPLIT != 2 || AE_DECODE)
#error "rows are split over two threads in the two-tile forward only"
#endif
#define AE_ROW_WARPS (8 * AE_RSPLIT)
#define AE_NTHREADS (AE_ROW_WARPS * 32 + 64)
#define AE_NC (AE_BN / AE_RSPLIT)  // score columns per row thread
#if AE_PINGPONG && AE_STAGES < 3
#error "the two-ahead S GEMM needs three K / V stages"
#endif

#ifdef AE_TRACE  // clock stamps of CTA (0, 0, 0)'s roles into the status buffer (experiments; needs a buffer that large)
#define AE_TRW(cond, region, slot) \
  if (tr_cta && (cond) && (slot) < 2048) args.status[64 + (region) * 4096 + (slot)] = (u32)clock64();
#else
#define AE_TRW(cond, region, slot)
#endif
// shared memory carve-up (dynamic, 1024-byte aligned by the launch)
#define AE_Q_BYTES (AE_BM * AE_D * 2)
#define AE_K_BYTES (AE_BN * AE_D * 2)
#define AE_V_BYTES (AE_BN * AE_DV * 2)
#define AE_SMEM_Q 0
#define AE_SMEM_K (AE_NQ * AE_Q_BYTES)
#define AE_SMEM_V (AE_SMEM_K + AE_STAGES * AE_K_BYTES)
#define AE_SMEM_BAR (AE_SMEM_V + AE_STAGES * AE_V_BYTES)
#define AE_SMEM_XCH (AE_SMEM_BAR + 512)  // AE_RSPLIT = 2 only: [q tile][phase][half][row] partial row reductions
#define AE_SMEM_STEPS (AE_SMEM_XCH + (AE_RSPLIT > 1 ? 2 * 2 * AE_RSPLIT * 128 * 4 : 0))  // mask mode 2 only: one word per kv tile
#define AE_MAX_KT 2048                    // kv tiles a block list may cover (4 * AE_MAX_KT bytes of shared memory)

struct AeFwdBars {
  u64 q_full[2];
  u64 k_full[AE_STAGES];
  u64 k_empty[AE_STAGES];
  u64 v_full[AE_STAGES];
  u64 v_empty[AE_STAGES];
  u64 s_full[2];
  u64 p_full[2];
  u64 o_done[2];
  AeCtaCtl ctl;
  int n_steps;  // mask mode 2: length of the merged walk
};

// kv tile schedule of one q tile --------------------------------------------------
// The CTA walks the union of its two tiles' lists; entry `j` of the walk gives the kv
// tile index and, per q tile, whether it takes part and whether it needs the
// element-wise mask.  With block lists (mask mode 2) the union is built once per CTA in
// shared memory (a flag word per kv tile, then compacted in place), so that the roles
// read the same table instead of each merging the two lists from global memory.
struct AeKvStep {
  int kt;        // kv tile index
  u32 flags;     // bit t: tile t active; bit 2+t: tile t needs element mask; bit 4+t: tile t's P is zero
};

AE_DEVICE int ae_causal_ntiles(int qt, int n_kt) {
  // rows [qt*128, qt*128+127] see kv columns [0, qt*128+127]
  int n = qt + 1;
  return n < n_kt ? n : n_kt;
}

extern "C" __global__ void __launch_bounds__(AE_NTHREADS, 1)
ae_attn_fwd(const __grid_constant__ AeAttnFwdArgs args) {
  extern __shared__ u8 smem_raw[];
  u8* smem = smem_align1024(smem_raw);
  AeFwdBars* bars = (AeFwdBars*)(smem + AE_SMEM_BAR);
  AeCtaCtl* ctl = &bars->ctl;
  const u32 warp = threadIdx.x >> 5;
  const u32 lane = threadIdx.x & 31;

#if AE_DECODE
  // Uniform split: CTA (split, head unit, batch row).  With a work list (rows of different lengths, args.work): CTA
  // (item, head unit), item = {batch row, split of that row, first kv tile, kv tiles}; the row's length comes from
  // args.seqlens and its partial results go to slot args.part_off[row] + split.
  const int hq = blockIdx.y;  // head unit: a kv head (gq > 1) or a head with its own K/V (gq == 1)
  const int hk = hq;
  const int qt0 = 0;
  int split, b, kt_off, dec_tiles, skv, part_slot;
  bool staged;
  if (args.work) {
    const AeWorkItem w = args.work[blockIdx.x];
    b = w.row;
    split = w.split;
    kt_off = w.tile_begin;
    dec_tiles = w.n_tiles;
    skv = args.seqlens[b];
    part_slot = args.part_off[b] + split;
    staged = args.part_off[b + 1] - args.part_off[b] > 1;
  } else {
    split = blockIdx.x;
    b = blockIdx.z;
    kt_off = split * args.tiles_per_split;
    dec_tiles = args.n_kt - kt_off < args.tiles_per_split ? args.n_kt - kt_off : args.tiles_per_split;
    skv = args.Skv;
    part_slot = b * args.n_split + split;
    staged = args.n_split > 1;
  }
#define AE_SKV skv
#else
#define AE_SKV args.Skv
  // heaviest (latest) q tiles first: better tail under a causal mask
  const int qpair = (int)gridDim.x - 1 - (int)blockIdx.x;
  const int hq = blockIdx.y;
  const int b = blockIdx.z;
  const int hk = hq / (args.Hq / args.Hkv);
  const int qt0 = qpair * 2;
  const int kt_off = 0;
#endif

#ifdef AE_TRACE
  const bool tr_cta = blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0;
#endif
  // ---- kv schedule (uniform over the CTA) ---------------------------------------
  int n_steps;
#if AE_MASK_MODE == 1
  int n_t0 = ae_causal_ntiles(qt0, args.n_kt);
  int n_t1 = (qt0 + 1 < args.n_qt) ? ae_causal_ntiles(qt0 + 1, args.n_kt) : 0;
  n_steps = n_t0 > n_t1 ? n_t0 : n_t1;
#elif AE_MASK_MODE == 2
  const u32* steps = (const u32*)(smem + AE_SMEM_STEPS);
  n_steps = 0;  // read from shared memory after the set-up barrier
#elif AE_DECODE
  int n_t0 = dec_tiles;
  int n_t1 = (1 < args.n_qt) ? n_t0 : 0;
  n_steps = n_t0;
#else
  int n_t0 = args.n_kt;
  int n_t1 = (qt0 + 1 < args.n_qt) ? args.n_kt : 0;
  n_steps = args.n_kt;
#endif

  // step iterator: all roles call next() in lockstep order
  struct Walk {
    int j;
  } walk = {0};
  auto next_step = [&](AeKvStep& st) -> bool {
#if AE_MASK_MODE == 2
    if (walk.j >= n_steps) return false;
    const u32 e = steps[walk.j];
    st.kt = (int)(e & 0xffffffu);
    st.flags = e >> 24;
    walk.j++;
    return true;
#else
    if (walk.j >= n_steps) return false;
    st.kt = kt_off + walk.j;
    st.flags = 0;
    if (walk.j < n_t0) st.flags |= 1u;
    if (walk.j < n_t1) st.flags |= 2u;
#if AE_MASK_MODE == 3
    st.flags |= 12u;  // no block information: every tile is masked element-wise
#endif
#if AE_MASK_MODE == 1
    // partial when the tile's last column exceeds the tile's first row
    if (walk.j * AE_BN + AE_BN - 1 > qt0 * AE_BM) st.flags |= 4u;
    if (walk.j * AE_BN + AE_BN - 1 > (qt0 + 1) * AE_BM) st.flags |= 8u;
#endif
    walk.j++;
    return true;
#endif
  };

  // ---- setup ---------------------------------------------------------------------
  if (threadIdx.x == 0) {
    ctl->abort = 0;
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars->q_full[i], 1);
      mbar_init(&bars->s_full[i], 1);
      mbar_init(&bars->p_full[i], 4 * AE_RSPLIT);
      mbar_init(&bars->o_done[i], 1);
    }
    for (int i = 0; i < AE_STAGES; ++i) {
      mbar_init(&bars->k_full[i], 1);
      mbar_init(&bars->k_empty[i], 1);
      mbar_init(&bars->v_full[i], 1);
      mbar_init(&bars->v_empty[i], 1);
    }
    mbar_fence_init();
  }
#if AE_MASK_MODE == 2
  {
    // flag word per kv tile: bit t = tile t takes part, bit 2+t = it needs the element mask.  The lists come from the
    // caller: a count or an entry outside the tile grid empties this CTA's walk and is reported through the status word.
    u32* tab = (u32*)(smem + AE_SMEM_STEPS);
    const int* cnt_base = args.blk_cnt + ((i64)b * args.Hq + hq) * args.n_qt;
    const int* idx_base = args.blk_idx + ((i64)b * args.Hq + hq) * args.n_qt * (i64)args.n_kt;
    const int n_t0 = cnt_base[qt0];
    const int n_t1 = (qt0 + 1 < args.n_qt) ? cnt_base[qt0 + 1] : 0;
    const int* list0 = idx_base + (i64)qt0 * args.n_kt;
    const int* list1 = idx_base + (i64)(qt0 + 1) * args.n_kt;
    bool bad = args.n_kt > AE_MAX_KT || n_t0 < 0 || n_t0 > args.n_kt || n_t1 < 0 || n_t1 > args.n_kt;
    if (!bad)
      for (int i = threadIdx.x; i < args.n_kt; i += AE_NTHREADS) tab[i] = 0u;
    __syncthreads();
    if (!bad) {
      for (int i = threadIdx.x; i < n_t0 + n_t1; i += AE_NTHREADS) {
        const bool second = i >= n_t0;
        const u32 e = (u32)(second ? list1[i - n_t0] : list0[i]);
        const u32 kt = e & 0x3fffffffu;
        const u32 part = (e >> 30) & 1u;
        if (kt >= (u32)args.n_kt)
          bad = true;
        else
          atomicOr(&tab[kt], second ? (2u | part << 3) : (1u | part << 2));
      }
    }
    const int any_bad = __syncthreads_or(bad ? 1 : 0);
    if (warp == 0) {
      int n = 0;
      if (!any_bad) {
        // in-place compaction: entry kt moves to a position <= kt, and a chunk is read by every lane before it is written
        for (int base = 0; base < args.n_kt; base += 32) {
          const int kt = base + (int)lane;
          const u32 f = kt < args.n_kt ? tab[kt] : 0u;
          const u32 m = __ballot_sync(0xffffffffu, f != 0u);
          if (f) {
            // A kv tile listed for one q tile only is still run for both (bits 4, 5: the other tile's P is zero):
            // the MMA and TMA roles then see the step pattern of an unmasked walk, whatever the lists hold.
            u32 g = f;
            if (!(f & 1u)) g |= 1u | 16u;
            if (!(f & 2u) && qt0 + 1 < args.n_qt) g |= 2u | 32u;
            tab[n + __popc(m & ((1u << lane) - 1u))] = (u32)kt | g << 24;
          }
          n += __popc(m);
          __syncwarp();
        }
      }
      if (lane == 0) {
        bars->n_steps = n;
        if (any_bad && args.status) atomicCAS(args.status, 0u, 0x400u);
      }
    }
  }
#endif
  if (warp == AE_ROW_WARPS + 1) {
    tmem_alloc(&ctl->tmem_base, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const u32 tmem = ctl->tmem_base;
#if AE_MASK_MODE == 2
  n_steps = bars->n_steps;
#endif
  const u32 TM_S0 = 0, TM_S1 = 128, TM_O0 = 256, TM_O1 = 256 + AE_DV;

  if (warp == AE_ROW_WARPS) {
    // =============================== TMA producer ===============================
    if (lane == 0) {
      tma_prefetch_desc(&args.tm_q);
      tma_prefetch_desc(&args.tm_k);
      tma_prefetch_desc(&args.tm_v);
      for (int t = 0; t < AE_NQ; ++t) {
        // a q tile past the end is never waited for: fetching it would leave a bulk copy in flight when the CTA retires
#if AE_DECODE
        if (t > 0 && t * AE_BM >= args.rows) break;
#else
        if (qt0 + t >= args.n_qt) break;
#endif
        mbar_arrive_expect_tx(&bars->q_full[t], AE_Q_BYTES);
        for (int dh = 0; dh < AE_D / 64; ++dh)
          tma_load_bshd(smem + AE_SMEM_Q + t * AE_Q_BYTES + dh * (AE_BM * 128), &args.tm_q, &bars->q_full[t], dh * 64,
                      hq, (qt0 + t) * AE_BM, b);
      }
      AeKvStep st;
      int it = 0;
      while (next_step(st)) {
        const int stage = it % AE_STAGES;
        const u32 par = ((it / AE_STAGES) & 1) ^ 1;
#if AE_DECODE
        // paged K / V (args.block_table): the pool is one batch of num_pages * 128 rows, tile kt of row b is a page
        const int kv_row0 = args.block_table ? args.block_table[(i64)b * args.max_pages + st.kt] * AE_BN : st.kt * AE_BN;
        const int kv_b = args.block_table ? 0 : b;
#else
        const int kv_row0 = st.kt * AE_BN;
        const int kv_b = b;
#endif
        if (!mbar_wait(&bars->k_empty[stage], par, ctl, args.status, 1)) break;
        mbar_arrive_expect_tx(&bars->k_full[stage], AE_K_BYTES);
        for (int dh = 0; dh < AE_D / 64; ++dh)
          tma_load_bshd(smem + AE_SMEM_K + stage * AE_K_BYTES + dh * (AE_BN * 128), &args.tm_k, &bars->k_full[stage],
                      dh * 64, hk, kv_row0, kv_b);
        if (!mbar_wait(&bars->v_empty[stage], par, ctl, args.status, 2)) break;
        mbar_arrive_expect_tx(&bars->v_full[stage], AE_V_BYTES);
        for (int dh = 0; dh < AE_DV / 64; ++dh)
          tma_load_bshd(smem + AE_SMEM_V + stage * AE_V_BYTES + dh * (AE_BN * 128), &args.tm_v, &bars->v_full[stage],
                      dh * 64, hk, kv_row0, kv_b);
        ++it;
      }
    }
  } else if (warp == AE_ROW_WARPS + 1) {
    // =============================== MMA issuer =================================
    if (lane == 0) {
      const u32 idesc_s = umma_idesc_f16(AE_BM, AE_BN, AE_BF16, 0, 0);
      const u32 idesc_o = umma_idesc_f16(AE_BM, AE_DV, AE_BF16, 0, 1);
      const u32 q_addr = smem_u32(smem + AE_SMEM_Q);
      const u32 k_addr = smem_u32(smem + AE_SMEM_K);
      const u32 v_addr = smem_u32(smem + AE_SMEM_V);
      const u64 dk0 = umma_base_k(k_addr);
      const u64 dv0 = umma_base_mn(v_addr, AE_BN);
      // q tile index as a compile-time constant: every per-tile quantity stays in a named register
      auto issue_s = [&](auto T, int stage) {
        constexpr int t = decltype(T)::value;
        const u64 da = umma_base_k(q_addr + t * AE_Q_BYTES);
        const u64 db = dk0 + (u64)((stage * AE_K_BYTES) >> 4);
        const u32 d = tmem + (t ? TM_S1 : TM_S0);
#pragma unroll
        for (int kk = 0; kk < AE_D / 16; ++kk)
          umma_ss(d, umma_step_k(da, kk, AE_BM), umma_step_k(db, kk, AE_BN), idesc_s, kk > 0);
      };
      auto issue_pv = [&](auto T, int stage, u32 acc) {
        constexpr int t = decltype(T)::value;
        const u64 db = dv0 + (u64)((stage * AE_V_BYTES) >> 4);
        const u32 d = tmem + (t ? TM_O1 : TM_O0);
        const u32 a = tmem + (t ? TM_S1 : TM_S0);
#pragma unroll
        for (int kk = 0; kk < AE_BN / 16; ++kk)
          umma_ts(d, a + kk * 8 + ((AE_RSPLIT > 1 && kk >= AE_BN / 32) ? 64 : 0), umma_step_mn(db, kk), idesc_o, acc | (kk > 0));
      };

#if AE_PINGPONG
      // kv tiles kt_off .. kt_off + n_steps - 1 in order (no mask in a decode build); tile n uses K / V stage n % AE_STAGES,
      // S region n & 1 and phase n >> 1 of that region's s_full / p_full; O (region 0) takes every P V.
      auto s_into = [&](int n) {
        const int stage = n % AE_STAGES;
        const u64 da = umma_base_k(q_addr);
        const u64 db = dk0 + (u64)((stage * AE_K_BYTES) >> 4);
        const u32 d = tmem + ((n & 1) ? TM_S1 : TM_S0);
#pragma unroll
        for (int kk = 0; kk < AE_D / 16; ++kk)
          umma_ss(d, umma_step_k(da, kk, AE_BM), umma_step_k(db, kk, AE_BN), idesc_s, kk > 0);
        umma_commit(&bars->s_full[n & 1]);
        umma_commit(&bars->k_empty[stage]);
      };
      bool ok = mbar_wait(&bars->q_full[0], 0, ctl, args.status, 4);
      for (int n = 0; n < 2 && n < n_steps && ok; ++n) {
        ok = mbar_wait(&bars->k_full[n % AE_STAGES], 0, ctl, args.status, 3);
        if (!ok) break;
        tc_fence_after_sync();
        s_into(n);
      }
      for (int n = 0; n < n_steps && ok; ++n) {
        const int stage = n % AE_STAGES;
        const u32 par = (n / AE_STAGES) & 1;
        ok = mbar_wait(&bars->p_full[n & 1], (n >> 1) & 1, ctl, args.status, 5);
        if (!ok) break;
        ok = mbar_wait(&bars->v_full[stage], par, ctl, args.status, 6);
        if (!ok) break;
        tc_fence_after_sync();
        {
          const u64 db = dv0 + (u64)((stage * AE_V_BYTES) >> 4);
          const u32 d = tmem + TM_O0;
          const u32 a = tmem + ((n & 1) ? TM_S1 : TM_S0);
#pragma unroll
          for (int kk = 0; kk < AE_BN / 16; ++kk)
            umma_ts(d, a + kk * 8, umma_step_mn(db, kk), idesc_o, (u32)(n > 0) | (kk > 0));
        }
        umma_commit(&bars->o_done[0]);
        umma_commit(&bars->v_empty[stage]);
        if (n + 2 < n_steps) {
          // the region of tile n is free once its P V (just issued) has read P: MMAs run in issue order
          ok = mbar_wait(&bars->k_full[(n + 2) % AE_STAGES], ((n + 2) / AE_STAGES) & 1, ctl, args.status, 7);
          if (!ok) break;
          s_into(n + 2);
        }
      }
      // every commit of this thread has arrived before the CTA may retire (the last slot releases have no other waiter)
      if (ok && n_steps > 0) {
        const int l = n_steps - 1;
        ok = mbar_wait(&bars->v_empty[l % AE_STAGES], (l / AE_STAGES) & 1, ctl, args.status, 12) &&
             mbar_wait(&bars->k_empty[l % AE_STAGES], (l / AE_STAGES) & 1, ctl, args.status, 13);
      }
#else
      // The walk is consumed one step ahead for the S GEMMs.
      AeKvStep cur, nxt;
      bool ok = true;
      bool have = next_step(cur);
      int it = 0;
      u32 np0 = 0, np1 = 0;  // P tiles consumed per q tile
      u32 q_ready = 0;       // bit t: Q tile t has landed
      auto first_s = [&](auto T) {
        constexpr int t = decltype(T)::value;
        if (!ok || !(cur.flags & (1u << t))) return;
        ok = mbar_wait(&bars->q_full[t], 0, ctl, args.status, 4);
        q_ready |= 1u << t;
        tc_fence_after_sync();
        issue_s(T, 0);
        umma_commit(&bars->s_full[t]);
      };
      if (have) {
        ok = mbar_wait(&bars->k_full[0], 0, ctl, args.status, 3);
        tc_fence_after_sync();
        first_s(AeInt<0>{});
        first_s(AeInt<1>{});
        umma_commit(&bars->k_empty[0]);
      }
      while (have && ok) {
        const int stage = it % AE_STAGES;
        const u32 par = (it / AE_STAGES) & 1;
        const bool have_n = next_step(nxt);
        const int nstage = (it + 1) % AE_STAGES;
        const u32 npar = ((it + 1) / AE_STAGES) & 1;
        bool v_ready = false, k_ready = false;
        auto tile_step = [&](auto T, u32& np) {
          constexpr int t = decltype(T)::value;
          if (!ok) return;
          AE_TRW(true, 0, it * 8 + t * 4 + 0);
          if (cur.flags & (1u << t)) {
            ok = mbar_wait(&bars->p_full[t], np & 1, ctl, args.status, 5);
            if (!ok) return;
            AE_TRW(true, 0, it * 8 + t * 4 + 1);
            if (!v_ready) {
              ok = mbar_wait(&bars->v_full[stage], par, ctl, args.status, 6);
              if (!ok) return;
              v_ready = true;
            }
            tc_fence_after_sync();
            issue_pv(T, stage, np > 0);
            umma_commit(&bars->o_done[t]);
            np++;
            AE_TRW(true, 0, it * 8 + t * 4 + 2);
          }
          if (have_n && (nxt.flags & (1u << t))) {
            if (!k_ready) {
              ok = mbar_wait(&bars->k_full[nstage], npar, ctl, args.status, 7);
              if (!ok) return;
              k_ready = true;
            }
            if (!(q_ready & (1u << t))) {  // Q of this tile is awaited once
              ok = mbar_wait(&bars->q_full[t], 0, ctl, args.status, 8);
              if (!ok) return;
              q_ready |= 1u << t;
            }
            // (no tcgen05 fence: the waits above are for shared-memory operands; the S region's last TMEM accesses by
            // other threads were fenced with the p_full wait of the step that made them)
            issue_s(T, nstage);
            umma_commit(&bars->s_full[t]);
            AE_TRW(true, 0, it * 8 + t * 4 + 3);
          }
        };
        tile_step(AeInt<0>{}, np0);
        tile_step(AeInt<1>{}, np1);
        if (!ok) break;
        umma_commit(&bars->v_empty[stage]);
        if (have_n) umma_commit(&bars->k_empty[nstage]);
        cur = nxt;
        have = have_n;
        ++it;
      }
      // every commit of this thread has arrived before the CTA may retire (the last slot releases have no other waiter)
      if (ok && it > 0) {
        const int l = it - 1;
        ok = mbar_wait(&bars->v_empty[l % AE_STAGES], (l / AE_STAGES) & 1, ctl, args.status, 12) &&
             mbar_wait(&bars->k_empty[l % AE_STAGES], (l / AE_STAGES) & 1, ctl, args.status, 13);
      }
#endif  // AE_PINGPONG
    }
  } else {
    // =============================== row warpgroups =============================
    const int t = warp / (4 * AE_RSPLIT);    // q tile of this group
    const u32 half = (warp >> 2) & (AE_RSPLIT - 1);  // which columns of the row this thread takes
    const u32 row = threadIdx.x & 127;       // row inside the tile == TMEM lane
    const u32 lane_base = ((warp & 3) * 32) << 16;
    const u32 tm_s = tmem + (t ? TM_S1 : TM_S0) + lane_base;
    const u32 tm_o = tmem + (t ? TM_O1 : TM_O0) + lane_base;
    const bool tile_valid = (qt0 + t) < args.n_qt;
#if AE_DECODE
    // packed rows: the query heads of the kv head's group (one query position), or the positions of one head;
    // rows past the last valid one compute on zero-filled Q with the indices of row 0 and are never stored
    const int r_idx = t * AE_BM + (int)row;
    const bool row_valid = r_idx < args.rows;
    const int h_row = (args.gq > 1) ? hq * args.gq + (row_valid ? r_idx : 0) : hq;
    const int q_idx = (args.gq > 1 || !row_valid) ? 0 : r_idx;
#else
    const int q_idx = (qt0 + t) * AE_BM + (int)row;
    const bool row_valid = q_idx < args.Sq;
    const int h_row = hq;
#endif

    AeCustom cu;
#pragma unroll
    for (int i = 0; i < AE_MAX_CUSTOM; ++i) {
      cu.p[i] = args.custom[i];
#pragma unroll
      for (int k = 0; k < 4; ++k) cu.st[i][k] = args.custom_st[i][k];
    }

    AeRow st;
    st.init();
#if AE_RSPLIT > 1
    st.xch = (volatile float*)(smem + AE_SMEM_XCH) + t * (2 * AE_RSPLIT * 128);
    st.xme = half * 128 + row;
    st.xother = (half ^ 1u) * 128 + row;
    st.xbar = 3 + t;
    st.xn = AE_RSPLIT * 128;
    st.xphase = 0;
#endif
    u32 n_done = 0;
    bool ok = true;
    AeKvStep step;
#if AE_TURNS
    // group 0 goes first: group 1 hands it the token once before the walk.  Every group passes the token at every
    // step of the walk, also at steps its tile sits out, so the two sides stay in step whatever the masks are.
    if (t == 1) named_bar_arrive(1, AE_RSPLIT * 256);
#endif
    while (next_step(step)) {
#if AE_TURNS
      if (!(step.flags & (1u << t))) {
        named_bar_sync(1 + t, AE_RSPLIT * 256);
        named_bar_arrive(2 - t, AE_RSPLIT * 256);
        continue;
      }
#else
      if (!(step.flags & (1u << t))) continue;
#endif
#if AE_PINGPONG
      // scores of this group's n-th tile: region n & 1, phase n >> 1 of that region's barriers
      const u32 rgn = n_done & 1u;
      const u32 tm_s_n = tmem + (rgn ? TM_S1 : TM_S0) + lane_base;
      u64* const s_bar = &bars->s_full[rgn];
      u64* const p_bar = &bars->p_full[rgn];
      const u32 s_par = (n_done >> 1) & 1u;
#else
      const u32 tm_s_n = tm_s;
      u64* const s_bar = &bars->s_full[t];
      u64* const p_bar = &bars->p_full[t];
      const u32 s_par = n_done & 1u;
#endif
      AE_TRW((warp & 3) == 0 && half == 0 && lane == 0, 1 + t, n_done * 8 + 0);
      ok = ok && mbar_wait(s_bar, s_par, ctl, args.status, 9);
      AE_TRW((warp & 3) == 0 && half == 0 && lane == 0, 1 + t, n_done * 8 + 1);
#if AE_TURNS
      named_bar_sync(1 + t, AE_RSPLIT * 256);  // this group's turn
#endif
      tc_fence_after_sync();
#if AE_MASK_MODE == 2
      if ((step.flags >> (4 + t)) & 1u) {
        // kv tile of the other q tile's list: P = 0, the row state and O stay as they are
        u32 z[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) z[i] = 0u;
#pragma unroll
        for (int hh = (int)half; hh < AE_BN / 64; hh += AE_RSPLIT) tmem_st32(tm_s_n + hh * 32 + (AE_RSPLIT > 1 ? hh * 64 : 0), z);
        tc_wait_st();
        tc_fence_before_sync();
        mbar_arrive_warp(p_bar);
#if AE_TURNS
        named_bar_arrive(2 - t, AE_RSPLIT * 256);
#endif
        ++n_done;
        continue;
      }
#endif
      float s[AE_NC];
#if AE_RSPLIT > 1
      tmem_ld_f32x64(tm_s_n + half * AE_NC, s);
#else
      tmem_ld_f32x128(tm_s_n, s);
#endif
      AE_TRW((warp & 3) == 0 && half == 0 && lane == 0, 1 + t, n_done * 8 + 2);
      const int kv0 = step.kt * AE_BN + (int)half * AE_NC;  // first kv column of this thread
      const bool tail = (step.kt * AE_BN + AE_BN > AE_SKV);
      const bool partial = (step.flags >> (2 + t)) & 1u;
      if (partial || tail) {
#pragma unroll
        for (int c = 0; c < AE_NC; ++c) {
          const int kv_idx = kv0 + c;
          bool keep = kv_idx < AE_SKV;
#if AE_MASK_MODE != 0
          if (partial) keep = keep && ae_mask(b, h_row, q_idx, kv_idx);
#endif
#if AE_MASK_NEG_INF
          if (!keep) s[c] = -__int_as_float(0x7f800000);
#else
          if (kv_idx >= AE_SKV) s[c] = 0.f;  // additive mask value 0: scores stay as they are
          (void)keep;
#endif
        }
      }
      const float o_scale = ae_online_fwd<AE_NC>(s, st, b, h_row, q_idx, kv0, cu);
#if AE_TURNS
      named_bar_arrive(2 - t, AE_RSPLIT * 256);  // the exponentials are done: the other group's turn
#endif

      AE_TRW((warp & 3) == 0 && half == 0 && lane == 0, 1 + t, n_done * 8 + 3);
      // P -> TMEM (16-bit pairs, column c/2 holds kv columns c, c+1)
      {
        u32 pk[32];
#pragma unroll
        for (int hh = 0; hh < AE_NC / 64; ++hh) {
#pragma unroll
          for (int i = 0; i < 32; ++i) pk[i] = pack2<AE_BF16>(s[hh * 64 + 2 * i], s[hh * 64 + 2 * i + 1]);
          tmem_st32(tm_s_n + hh * 32 + (AE_RSPLIT > 1 ? half * 96 : 0), pk);
        }
      }
#if !AE_O_SCALE_ONE
      // O is rescaled only when some row of the warp needs it; only then must the previous step's P V have
      // completed.  (A skipped wait cannot alias: o_done runs at most one phase ahead of this warp's arrivals.)
      if (n_done > 0 && __any_sync(0xffffffffu, o_scale != 1.0f)) {
        ok = ok && mbar_wait(&bars->o_done[t], (n_done - 1) & 1, ctl, args.status, 10);
        tc_fence_after_sync();
#pragma unroll
        for (int c = (int)half; c < AE_DV / 32; c += AE_RSPLIT) {  // the threads of a row share its O columns
          float f[32];
          u32 r[32];
          tmem_ld_f32x32(tm_o + c * 32, f);
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(f[i] * o_scale);
          tmem_st32(tm_o + c * 32, r);
        }
      }
#endif
      tc_wait_st();
      AE_TRW((warp & 3) == 0 && half == 0 && lane == 0, 1 + t, n_done * 8 + 4);
      tc_fence_before_sync();
      mbar_arrive_warp(p_bar);
      AE_TRW((warp & 3) == 0 && half == 0 && lane == 0, 1 + t, n_done * 8 + 5);
      ++n_done;
    }

    // ---- epilogue ------------------------------------------------------------------
#if AE_PINGPONG
    // The S GEMM of the last tile was issued before the P V of the tile before it, so o_done may still be two phases
    // short here: a parity wait can only tell neighbouring phases apart, hence one wait per missing phase.
    if (n_done > 1) ok = ok && mbar_wait(&bars->o_done[t], (n_done - 2) & 1, ctl, args.status, 14);
#endif
    if (n_done > 0) {
      ok = ok && mbar_wait(&bars->o_done[t], (n_done - 1) & 1, ctl, args.status, 11);
      tc_fence_after_sync();
    }
    // tcgen05.ld is warp-collective: every lane of the warp runs it; only the stores are per-row.
    if (tile_valid) {
      const bool store = row_valid && ok;
      u16* orow = (u16*)args.o + (i64)b * args.o_sb + (i64)(store ? q_idx : 0) * args.o_ss + (i64)h_row * args.o_sh;
#if AE_DECODE
      // more than one split: this split's normalised O and final row scales go to fp32 staging, merged by the combine pass
      const i64 part_row = (i64)part_slot * ((i64)args.Sq * args.Hq) + (i64)q_idx * args.Hq + h_row;
      float* prow = args.o_part + part_row * AE_DV;
#endif
#pragma unroll
      for (int c = (int)half; c < AE_DV / 32; c += AE_RSPLIT) {
        float r[32];
        if (n_done > 0) {
          tmem_ld_f32x32(tm_o + c * 32, r);
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] = 0.f;
        }
#if AE_DECODE
        if (store && staged) {
          float4* dst = (float4*)(prow + c * 32);
#pragma unroll
          for (int v = 0; v < 8; ++v)
            dst[v] = make_float4(ae_epilogue_o(r[v * 4 + 0], st), ae_epilogue_o(r[v * 4 + 1], st),
                                 ae_epilogue_o(r[v * 4 + 2], st), ae_epilogue_o(r[v * 4 + 3], st));
        } else
#endif
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
        for (int i = 0; i < AE_NFINAL; ++i) {
#if AE_DECODE
          if (staged)
            args.fr_part[i][part_row] = fr[i];
          else if (args.final_rs[i])
            args.final_rs[i][((i64)b * args.Hq + h_row) * args.Sq + q_idx] = fr[i];
#else
          args.final_rs[i][((i64)b * args.Hq + hq) * args.Sq + q_idx] = fr[i];
#endif
        }
      }
#endif
    }
  }

  // ---- teardown --------------------------------------------------------------------
  tc_fence_before_sync();
  __syncthreads();
  if (warp == AE_ROW_WARPS + 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, 512);
  }
}
