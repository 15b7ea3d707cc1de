// Kernel argument blocks shared by the host launcher (compiled with g++) and the
// kernel sources (compiled with NVRTC / nvcc).  Plain C layout, no CUDA headers.
#ifndef AE_ARGS_H_
#define AE_ARGS_H_

#ifndef AE_DEVICE
typedef unsigned char u8;
typedef unsigned short u16;
typedef unsigned int u32;
typedef unsigned long long u64;
typedef long long i64;
struct alignas(64) AeTmaDesc {
  u64 opaque[16];
};
#endif

#define AE_MAX_CUSTOM 4
#define AE_MAX_FINAL 4

struct alignas(16) AeWorkItem {  // one CTA's share of a split-KV decode over rows of different lengths
  int row;         // batch row
  int split;       // index of this share among the row's splits
  int tile_begin;  // first 128-key tile
  int n_tiles;     // tiles of this share (>= 1)
};

#ifdef AE_DEVICE
// custom inputs as seen by the generated functors
struct AeCustom {
  const void* p[AE_MAX_CUSTOM];
  i64 st[AE_MAX_CUSTOM][4];
};
#endif

// ---- fused attention forward (kernel ae_attn_fwd) --------------------------------
struct AeAttnFwdArgs {
  AeTmaDesc tm_q;  // dims (d, s, h, b), box {64, 128, 1, 1}, 128-byte swizzle
  AeTmaDesc tm_k;
  AeTmaDesc tm_v;
  void* o;
  i64 o_sb, o_ss, o_sh;           // element strides of O [B, S, H, DV]
  float* final_rs[AE_MAX_FINAL];  // each [B, Hq, Sq] fp32
  const void* custom[AE_MAX_CUSTOM];
  i64 custom_st[AE_MAX_CUSTOM][4];  // element strides over (b, h, q, kv); 0 = broadcast
  const int* blk_cnt;  // [B, Hq, n_qt] number of listed kv tiles            (mask mode 2)
  const int* blk_idx;  // [B, Hq, n_qt, n_kt] kv tile index | (partial << 30)  (mask mode 2)
  int B, Hq, Hkv, Sq, Skv;
  int n_qt, n_kt;  // number of 128-row q tiles / 128-column kv tiles
  u32* status;
  // Split-KV decode (the same kernel built with AE_DECODE): one CTA per (split, head unit, batch) owns ALL query rows
  // of its unit (at most 256) and the kv tiles [split * tiles_per_split, ...).  gq > 1: the unit is a kv head and the
  // rows are the gq query heads of its group (Sq == 1; tm_q is built over (d, head in group, kv head, b)); gq == 1:
  // the unit is a head and the rows are its Sq query positions.
  float* o_part;                 // [B, n_split, Sq * Hq, DV] fp32, after the epilogue (n_split > 1)
  float* fr_part[AE_MAX_FINAL];  // each [B, n_split, Sq * Hq]
  int n_split, tiles_per_split;
  int gq, rows;
  // Rows of different lengths and paged K / V (decode build; all null = one length, dense K / V):
  const AeWorkItem* work;  // [n_items]: one CTA per item and head unit
  const int* seqlens;      // [B] keys of each row
  const int* part_off;     // [B + 1] first partial-result slot of each row (its splits are consecutive slots)
  const int* block_table;  // [B, max_pages] page of each 128-key tile of a row; K / V are then pools [pages * 128, Hkv, D]
  int max_pages;
};

// ---- attention backward ------------------------------------------------------------
// Pre-pass: delta[b, h, s] = sum_d O * dO                     (kernel ae_attn_bwd_prep)
struct AeAttnBwdPrepArgs {
  const void* o;
  const void* d_o;
  float* delta;  // [B, Hq, Sq]
  i64 o_sb, o_ss, o_sh;
  i64 do_sb, do_ss, do_sh;
  int B, Hq, Sq, DV;
};

// dQ pass (kernel ae_attn_bwd_dq): one CTA per 128-row q tile, streams K/V tiles.
// dK/dV pass (kernel ae_attn_bwd_dkv): one CTA per 128-row kv tile, streams Q/dO tiles
// of every q-head of the kv-head's group.
struct AeAttnBwdArgs {
  AeTmaDesc tm_q;
  AeTmaDesc tm_k;
  AeTmaDesc tm_v;
  AeTmaDesc tm_do;
  void* dq;
  void* dk;
  void* dv;
  i64 dq_sb, dq_ss, dq_sh;
  i64 dk_sb, dk_ss, dk_sh;
  i64 dv_sb, dv_ss, dv_sh;
  const float* final_rs[AE_MAX_FINAL];  // each [B, Hq, Sq]
  const float* delta;                   // [B, Hq, Sq]
  const void* custom[AE_MAX_CUSTOM];
  i64 custom_st[AE_MAX_CUSTOM][4];
  const int* blk_cnt;   // per q tile lists (dQ pass)
  const int* blk_idx;
  const int* blkT_cnt;  // per kv tile lists of q tiles (dK/dV pass)
  const int* blkT_idx;
  int B, Hq, Hkv, Sq, Skv;
  int n_qt, n_kt;
  u32* status;
  float* dq_acc;  // [B, Sq, Hq, D] fp32, contiguous: dQ accumulator of the one-pass backward (ae_attn_bwd_fused)
  AeTmaDesc tm_dqacc;  // the same buffer as (d, s, h, b) fp32, box {32, 32, 1, 1}, 128-byte swizzle (TMA reduce-add)
};

// ---- MLA split-KV decode (kernels ae_mla_decode, ae_mla_combine) --------------------------
struct AeMlaArgs {
  AeTmaDesc tm_q;    // dims (512, H, B), box {64, 128, 1}
  AeTmaDesc tm_qpe;  // dims (64, H, B),  box {64, 128, 1}
  AeTmaDesc tm_kv;   // dims (512, S, B), box {64, BN, 1}
  AeTmaDesc tm_kpe;  // dims (64, S, B),  box {64, BN, 1}
  void* o;           // [B, H, 512] 16-bit                       (n_split == 1)
  float* o_part;     // [B, n_split, H, 512] fp32, normalised   (n_split > 1)
  float* fr_part[AE_MAX_FINAL];  // each [B, n_split, H]
  int B, H, S, n_split, tiles_per_split;
  u32* status;
  // paged KV (null = the dense layout above): tm_kv / tm_kpe then cover the page pool as rows (page * 64 + r) of one
  // batch, tile i of batch row b is page block_table[b * max_pages + i], and row b holds seqlens[b] keys
  // (S = the longest row; a split that starts past a row's last tile writes zero partials with -inf row scales).
  const int* block_table;
  const int* seqlens;
  int max_pages;
};
struct AeMlaCombineArgs {
  void* o;
  const float* o_part;
  const float* fr_part[AE_MAX_FINAL];
  int B, H, DV, n_split;
  const int* part_off;  // [B + 1] or null: row b owns the partial slots part_off[b] .. part_off[b + 1] - 1 (at most 32);
                        // null = n_split slots per row.  A row with a single slot was written directly and is skipped.
};

// ---- chunked linear attention / SSD scan forward (kernel ae_linear_fwd) -------------------
struct AeLinearArgs {
  AeTmaDesc tm_q;  // [B, HQ, T, DK] seen as (d, t, h, b), box {64, 128, 1, 1}
  AeTmaDesc tm_k;  // [B, HK, T, DK]
  AeTmaDesc tm_v;  // [B, H, T, DV]
  const float* a;  // [B, H, T] fp32 log-decay per step (<= 0)
  void* o;         // [B, H, T, DV] 16-bit
  int B, H, HQ, HK, T;
  u32* status;
  // Build with AE_LIN_MODS (the Mamba2 block's mods inside the kernel): the scan runs on v = x * vscale[b, h, t] with x
  // the tensor behind tm_v, the output is scan + x * dskip[h], and v is written out for the backward when v_out is set.
  const void* vscale;  // [B, H, T] fp32, or the 16-bit type when vscale_16 != 0
  const float* dskip;  // [H] fp32, or null
  void* v_out;         // [B, H, T, DV] 16-bit, or null
  int vscale_16;
  // Any build: when set, the state each chunk starts from is written here in 16-bit, [B, H, n_chunks, DK, DV] (what
  // ae_linear_states would recompute for the backward).
  void* h_out;
  AeTmaDesc tm_hout;  // h_out as [B * H * n_chunks, DK, DV], dims (dv, dk, n), box {64, 128, 1}   (when h_out is set)
  AeTmaDesc tm_vout;  // v_out like tm_v                                                       (when v_out is set)
  AeTmaDesc tm_o;     // o like tm_v: the output tile leaves through a bulk store
  const float* ascale;  // [H] or null: the scan runs on a * ascale[h] (a decay mod of the form decay * custom[heads])
};

// ---- chunked linear attention backward (kernels ae_linear_states, ae_linear_bwd) ---------
struct AeLinearBwdArgs {
  AeTmaDesc tm_q;   // [B, HQ, T, DK]
  AeTmaDesc tm_k;   // [B, HK, T, DK]
  AeTmaDesc tm_v;   // [B, H, T, DV]
  AeTmaDesc tm_do;  // [B, H, T, DV]
  AeTmaDesc tm_h;   // chunk start-states [B * H * n_chunks, DK, DV] 16-bit, dims (dv, dk, n), box {64, 128, 1}
  const float* a;   // [B, H, T]
  void* h_states;   // written by ae_linear_states, read (through tm_h) by ae_linear_bwd
  void* dq;         // [B, H, T, DK] 16-bit, per head
  void* dk;         // [B, H, T, DK] 16-bit, per head
  void* dv;         // [B, H, T, DV] 16-bit
  float* da;        // [B, H, T] fp32
  int B, H, HQ, HK, T;
  u32* status;
  AeTmaDesc tm_dq;  // dq, dk, dv as store targets: like tm_q / tm_v with H heads (ae_linear_bwd stages each chunk's tiles in
  AeTmaDesc tm_dk;  // shared memory and sends them out as bulk stores)
  AeTmaDesc tm_dv;
  // AE_LB_MODS build (v = x * vscale before the scan, y += x * dskip[h] after it): dv receives gx
  AeTmaDesc tm_x;       // [B, H, T, DV]
  const void* vscale;   // [B, H, T] fp32 or 16-bit
  const float* dskip;   // [H]
  void* gs;             // [B, H, T] in the type of vscale: sum_d dv * x
  float* gd;            // [B, H]: sum over t, d of dO * x
  int vscale_16;
  // Any build: a decay mod of the form decay * custom[heads] inside the kernels.  The scan runs on a * ascale[h]; da is
  // then the gradient of a as passed (times ascale[h]) and gasc [B, H] receives sum_t (gradient of the scaled decay) * a.
  const float* ascale;  // [H] or null
  float* gasc;          // [B, H] (required with ascale)
};

// ---- row-scale mod and its backward (kernels ae_rowscale_fwd, ae_rowscale_bwd) ---------------
struct AeRowScaleArgs {
  const void* x;  // [n_rows, D] 16-bit
  const void* s;  // [n_rows] fp32 or 16-bit
  void* y;        // forward:  x * s
  const void* g;  // backward: gradient of y
  void* gx;       // backward: g * s
  void* gs;       // backward: sum_d g * x, in the type of s
  i64 n_rows;
  // per-head skip kernels (ae_skip_fwd / ae_skip_bwd): s is [n_heads] fp32, a row's head is (row / rows_per_head) % n_heads
  i64 rows_per_head;
  int n_heads;
  // ae_vskip_bwd (row scale and skip of one block, both gradients in one pass): g2 = gradient of the scaled rows,
  // d [n_heads] fp32 skip weights, gs2 [n_rows] fp32 = sum_d g * x
  const void* g2;
  const float* d;
  float* gs2;
};

// ---- UMMA / TMA probe kernels (bring-up checks, kernel ae_probe) -------------------
struct AeProbeArgs {
  AeTmaDesc tm_a;  // [128 rows, KD] 16-bit, box {64, 128}
  AeTmaDesc tm_b;  // [128 rows, KD] 16-bit, box {64, 128}
  const void* p;   // [128, 128] 16-bit row-major (mode 1: A operand staged through TMEM)
  float* d;        // [128, 128] fp32 out
  int mode;        // 0: D = A * B^T (both K-major, smem)  1: D = P * B (P via TMEM, B MN-major)
  u32* status;
};

#endif  // AE_ARGS_H_
