/* C ABI of libae_b200.so: the B200 (sm_100a) back end behind AttentionEngine's
 * operator API.
 *
 * The reference has no C interface for this path: its Python front end renders a
 * TileLang module and lets TileLang/TVM compile and launch it
 * (attention_engine/attn_engine/attn_engine.py:334-395), or binds the CuTe kernels
 * with pybind11 (attention_engine/core/template/cute_template/flash_api.cpp:696-697,
 * cute_template_kvshared/flash_api.cpp:212-216).  The entry points below are what a
 * ctypes / cffi stub in that front end binds instead.  Each comment names the
 * reference interface the entry point stands in for.
 *
 * Conventions
 *  - plain pointers and sizes only; device pointers are raw CUDA device addresses;
 *  - every function returns 0 on success or an AE_ERR_* code (ae_strerror() gives
 *    text); nothing here calls exit() or traps;
 *  - `stream` is a cudaStream_t / CUstream passed as void*;
 *  - all tensors are owned by the caller; the library allocates no device memory (the one exception is the
 *    fixed 32 MiB array behind ae_launch_attn_bwd_static_scratch, which is part of the library image);
 *  - runtime tensors are [B, S, H, D] with the last dimension contiguous; strides
 *    are in elements, ordered (batch, seq, head);
 *  - `status` is an optional device word the kernels write when a bounded wait gives
 *    up (0 = ok); the caller clears and reads it.
 */
#ifndef AE_B200_H_
#define AE_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
  AE_OK = 0,
  AE_ERR_INVALID = 1,     /* bad argument (null pointer, unsupported shape / dtype / stride) */
  AE_ERR_COMPILE = 2,     /* NVRTC reported errors; see the log buffer */
  AE_ERR_NO_NVRTC = 3,    /* libnvrtc could not be loaded */
  AE_ERR_NO_DRIVER = 4,   /* libcuda could not be loaded / no CUDA context */
  AE_ERR_CUDA = 5,        /* a driver call failed; ae_last_error() has the text */
  AE_ERR_UNSUPPORTED = 6, /* kernel kind does not match the entry point */
};

enum { AE_DTYPE_F16 = 0, AE_DTYPE_BF16 = 1 };

enum {
  AE_KIND_PROBE = 0,
  AE_KIND_ATTN_FWD = 1,
  AE_KIND_ATTN_BWD_PREP = 2,
  AE_KIND_ATTN_BWD_DQ = 3,
  AE_KIND_ATTN_BWD_DKV = 4,
  AE_KIND_MLA_DECODE = 5,
  AE_KIND_MLA_COMBINE = 6,
  AE_KIND_LINEAR_FWD = 7,
  AE_KIND_LINEAR_BWD = 8,
  AE_KIND_LINEAR_STATES = 9,
  AE_KIND_ATTN_DECODE = 10,
  AE_KIND_ROWSCALE = 11,
  AE_KIND_ATTN_BWD_FUSED = 12,
  AE_KIND_ATTN_BWD_CAST = 13,
  AE_KIND_ATTN_FWD_PAIR = 14, /* kernel "ae_attn_fwd_pair": launched through ae_launch_attn_fwd */
};

#define AE_MAX_CUSTOM_INPUTS 4
#define AE_MAX_FINAL_ROWSCALES 4

/* Static facts about one compiled kernel, given by whoever generated its source. */
typedef struct AeKernelConfig {
  int kind;       /* AE_KIND_* */
  int dtype;      /* AE_DTYPE_* */
  int head_dim;   /* D  */
  int head_dim_v; /* DV */
  int threads;    /* block size */
  int smem_bytes; /* dynamic shared memory */
  int stages;     /* depth of the K/V (or Q/dO) ring */
  int mask_mode;  /* 0 none, 1 causal loop bounds, 2 block list */
  int reserved[8];
} AeKernelConfig;

/* Resource usage read back from the driver after loading. */
typedef struct AeKernelInfo {
  int num_regs;
  int static_smem_bytes;
  int max_dynamic_smem_bytes;
  int local_bytes; /* spill / stack bytes per thread */
  int max_threads;
} AeKernelInfo;

/* Compile CUDA C++ source to an sm_100a cubin with NVRTC and wrap it in a module
 * handle.  No GPU is needed; the cubin is loaded into the current context on the
 * first launch.  Replaces the reference's JIT step `tl.compile(...)` run when the
 * rendered module is imported (core/template/tl_template/attn/attn_tl.py:523-561)
 * and `torch.utils.cpp_extension.load` (cute_template/flash_attn_interface.py:136-147). */
int ae_compile(const char* cuda_src, const char* kernel_name, const char* arch, const char** opts, int nopts,
               const AeKernelConfig* cfg, void** out_module, char* log, size_t log_cap);

/* Wrap a cubin produced earlier (content-addressed cache).  Replaces the
 * reference's md5-keyed source cache (attn_engine/attn_engine.py:369-382). */
int ae_module_from_cubin(const void* cubin, size_t size, const char* kernel_name, const AeKernelConfig* cfg,
                         void** out_module);
/* Borrow the module's cubin image (valid until ae_release). */
int ae_module_cubin(void* module, const void** data, size_t* size);
/* Load (if needed) and report registers / shared memory / spills.  Needs a GPU. */
int ae_query(void* module, AeKernelInfo* info);
void ae_release(void* module);
const char* ae_strerror(int code);
/* Text of the last driver / NVRTC failure on the calling thread. */
const char* ae_last_error(void);

/* ---- fused attention forward --------------------------------------------------
 * Stands in for the generated `_attention.forward` -> `mod(q, k, v, *custom)`
 * (core/template/tl_template/attn/attn_tl.py:567-580; GQA attn_gqa_tl.py:354-380;
 * block-sparse blockattn_tl.py). */
typedef struct AeAttnParams {
  const void* q; /* [B, Sq, Hq, D]   */
  const void* k; /* [B, Skv, Hkv, D] */
  const void* v; /* [B, Skv, Hkv, DV]*/
  void* o;       /* [B, Sq, Hq, DV]  */
  int64_t q_stride[3], k_stride[3], v_stride[3], o_stride[3]; /* (batch, seq, head) */
  float* final_rowscales[AE_MAX_FINAL_ROWSCALES];             /* each [B, Hq, Sq] fp32 */
  const void* custom[AE_MAX_CUSTOM_INPUTS];
  int64_t custom_stride[AE_MAX_CUSTOM_INPUTS][4]; /* over (b, h, q, kv); 0 = broadcast */
  const int32_t* block_count; /* [B, Hq, n_qt]        (mask_mode 2) */
  const int32_t* block_index; /* [B, Hq, n_qt, n_kt]  (mask_mode 2): kv tile | partial << 30; the first block_count
                                 entries of a row count, in any order; at most 2048 kv tiles (AE_ERR_INVALID beyond);
                                 an entry outside the grid sets status 0x400 and that CTA writes nothing useful */
  int32_t B, Hq, Hkv, Sq, Skv;
  uint32_t* status;
} AeAttnParams;

/* Module kind AE_KIND_ATTN_FWD (kernel "ae_attn_fwd", one CTA per two q tiles) or AE_KIND_ATTN_FWD_PAIR (kernel
 * "ae_attn_fwd_pair": a cluster of two CTAs per two q tiles on tcgen05 cta_group::2; mask_mode 0, 1 or 3, head_dim_v 128,
 * head_dim 64 or 128, AE_ERR_INVALID otherwise).  Same parameter block and results for both. */
int ae_launch_attn_fwd(void* module, const AeAttnParams* p, void* stream);

/* ---- attention backward -----------------------------------------------------------
 * Stands in for `_attention.backward` (attn_tl.py:582-601): `mod_prep(o, dO)` (K2,
 * attn_tl.py:196-223), `mod_bwd(...)` (K3, :239-415) and `mod_post(dq)` (K4, :436-455).
 * Two forms.  Two-pass (ae_launch_attn_bwd_dq + _dkv): the dQ and the dK/dV parts are two
 * launches with no atomics and no fp32 dQ staging buffer, bit-reproducible, at the cost of
 * computing S and dP in both.  One-pass (ae_launch_attn_bwd_fused + _dq_cast): the reference's
 * own scheme, one kv-stationary kernel that adds dQ in fp32 into `dq_accum`, and the post
 * kernel that converts it; five contractions per tile instead of seven, dQ not bit-reproducible. */
typedef struct AeAttnBwdParams {
  const void* q;
  const void* k;
  const void* v;
  const void* o;
  const void* d_o;
  void* dq;
  void* dk;
  void* dv;
  int64_t q_stride[3], k_stride[3], v_stride[3], o_stride[3], do_stride[3];
  int64_t dq_stride[3], dk_stride[3], dv_stride[3];
  const float* final_rowscales[AE_MAX_FINAL_ROWSCALES];
  float* delta; /* [B, Hq, Sq] fp32 scratch: rowsum(O * dO) */
  const void* custom[AE_MAX_CUSTOM_INPUTS];
  int64_t custom_stride[AE_MAX_CUSTOM_INPUTS][4];
  const int32_t* block_count;
  const int32_t* block_index;
  const int32_t* block_count_t; /* transposed lists: per kv tile, the q tiles */
  const int32_t* block_index_t;
  int32_t B, Hq, Hkv, Sq, Skv;
  uint32_t* status;
  float* dq_accum; /* [B, Sq, Hq, D] fp32 contiguous scratch (one-pass form only; 16-byte aligned) */
} AeAttnBwdParams;

int ae_launch_attn_bwd_prep(void* module, const AeAttnBwdParams* p, void* stream);
int ae_launch_attn_bwd_dq(void* module, const AeAttnBwdParams* p, void* stream);
int ae_launch_attn_bwd_dkv(void* module, const AeAttnBwdParams* p, void* stream);
/* One-pass form (`mod_bwd` with its fp32 dQ atomics, attn_tl.py:239-415): clears p->dq_accum on `stream`, then runs
 * the kv-stationary kernel, which writes dk, dv and adds dQ into dq_accum.  Module kind AE_KIND_ATTN_BWD_FUSED
 * (kernel "ae_attn_bwd_fused"); p->delta as for the two-pass form. */
int ae_launch_attn_bwd_fused(void* module, const AeAttnBwdParams* p, void* stream);
/* `mod_post` (attn_tl.py:436-455): dq = p->dq_accum converted to the 16-bit type.  Module kind
 * AE_KIND_ATTN_BWD_CAST (kernel "ae_attn_bwd_dq_cast"). */
int ae_launch_attn_bwd_dq_cast(void* module, const AeAttnBwdParams* p, void* stream);

/* ---- attention backward without a caller-provided scratch buffer --------------------
 * No counterpart in the reference (there PyTorch allocates `delta` inside the generated
 * autograd function).  For callers that cannot allocate device memory: programs that bind
 * this ABI directly and own nothing but the input / output buffers they were handed, and
 * serving runtimes whose memory plan is frozen (cudaMalloc would synchronise the device).
 * Runs pre-pass + dQ pass + dK/dV pass like the three entry points above, but keeps
 * delta = rowsum(O * dO) in a fixed device array inside the library image
 * (AE_STATIC_SCRATCH_MAX_ROWS fp32 words = 32 MiB, held by every GPU that loads the
 * library until the process exits).  `p->delta` is ignored.
 *  - B * Hq * Sq above AE_STATIC_SCRATCH_MAX_ROWS is refused with AE_ERR_INVALID
 *    (ae_last_error() names both numbers).
 *  - Calls no cudaMalloc / cudaFree and no allocating library routine.  The array is part of
 *    the library image all the same: with CUDA's default lazy module loading the FIRST call
 *    on a device (cudaGetSymbolAddress, made with that device current) loads that image,
 *    which reserves the 32 MiB on that GPU, may synchronise the device and can fail with
 *    AE_ERR_CUDA on a GPU with no memory left.  Make that first call during start-up, as a
 *    warm-up, and outside any stream capture; later calls only launch kernels.
 *  - The target device must be current for every call (as for every entry point here).
 *  - The pre-pass always runs, so all three modules must be given, also for an OnlineFunc
 *    whose backward does not read delta.
 *  - All calls on a device share the one array.  It keeps the previous call's contents;
 *    every word a call reads is first rewritten by that call's pre-pass, so nothing needs
 *    clearing, but two calls that overlap on the GPU (different streams) race on it. */
#define AE_STATIC_SCRATCH_MAX_ROWS (8 * 1024 * 1024)
int ae_launch_attn_bwd_static_scratch(void* prep_module, void* dq_module, void* dkv_module, const AeAttnBwdParams* p,
                                      void* stream);

/* ---- MLA split-KV decode ------------------------------------------------------------
 * Stands in for the generated MLA op `mod(q, q_pe, kv, k_pe) -> o`
 * (core/template/tl_template/attn/mla_decode_tl.py:218-229, 326-335: `flash_attn_split` +
 * `combine` with `glse` / `Output_partial` scratch) and for the CuTe path's
 * `fwd_kvcache_mla` (cute_template_kvshared/flash_api.cpp:212-216).  All tensors contiguous. */
typedef struct AeMlaParams {
  const void* q;    /* [B, 1, H, 512] */
  const void* q_pe; /* [B, 1, H, 64]  */
  const void* kv;   /* [B, S, 1, 512] */
  const void* k_pe; /* [B, S, 1, 64]  */
  void* o;          /* [B, 1, H, 512] */
  float* o_partial; /* [B, n_split, H, 512] fp32 scratch, used when n_split > 1 */
  float* rowscale_partial[AE_MAX_FINAL_ROWSCALES]; /* each [B, n_split, H] fp32 scratch */
  int32_t B, H, S, n_split;
  uint32_t* status;
} AeMlaParams;

int ae_launch_mla_decode(void* module, const AeMlaParams* p, void* stream);
int ae_launch_mla_combine(void* module, const AeMlaParams* p, void* stream);

/* The same decode over a paged KV pool with one length per batch row: the call of the reference's CuTe kv-shared
 * path, `flash_mla_with_kvcache(q, k_cache, block_table, cache_seqlens, ...)`
 * (core/template/cute_template_kvshared/flash_mla_interface.py:73-113; script attn_script/mla_decode_cute.py:295-303),
 * whose scheduler metadata (`get_mla_metadata`) has no counterpart here: every batch row gets the same n_split over
 * the longest row's tiles, and a split that starts past a shorter row's end contributes nothing.  Pages hold 64 keys.
 * The merge is `ae_launch_mla_combine` with q / kv unused (fill o, o_partial, rowscale_partial, B, H, n_split). */
typedef struct AeMlaPagedParams {
  const void* q;                /* [B, H, 512] contiguous: the latent part of the query */
  const void* q_pe;             /* [B, H, 64]  contiguous: its rope part */
  const void* kcache;           /* [num_pages, 64, 576]: dims 0..511 latent kv (keys and values), 512..575 rope keys */
  const int32_t* block_table;   /* [B, max_pages]: page of the i-th 64-key tile of a batch row */
  const int32_t* cache_seqlens; /* [B]: keys of each batch row, 1 <= len <= max_pages * 64 */
  void* o;                      /* [B, H, 512] */
  float* o_partial;             /* [B, n_split, H, 512] fp32 (n_split > 1) */
  float* rowscale_partial[AE_MAX_FINAL_ROWSCALES]; /* each [B, n_split, H]; with n_split == 1 the final row scales */
  int32_t B, H, num_pages, max_pages, max_seqlen, n_split;
  uint32_t* status;
} AeMlaPagedParams;

int ae_launch_mla_decode_paged(void* module, const AeMlaPagedParams* p, void* stream);

/* ---- split-KV decode for MHA / GQA -----------------------------------------------------
 * Stands in for the reference's decode modules: `flashattn_gqa_decode` / `flashattn` split + `combine`
 * (core/template/tl_template/attn/attn_decode_tl.py:34-206, attn_gqa_decode_tl.py; dispatch
 * attn_engine/attn_engine.py:252-286; scripts attn_script/gqa_inference.py, mha_inference.py).
 * Query rows of one head unit share a tile: Hq > Hkv needs Sq == 1 (the Hq / Hkv query heads of a kv
 * head are the rows), Hq == Hkv takes Sq <= 256 query positions.  n_split CTAs per unit each walk
 * ceil(n_kv_tiles / n_split) kv tiles of 128 keys (the caller chooses n_split so that no split is
 * empty); n_split == 1 writes `o` directly, otherwise the splits write normalised fp32 partials and
 * their final row scales, and `ae_launch_decode_combine` (module kind AE_KIND_MLA_COMBINE, the traced
 * `OnlineFunc.combine`) merges them into `o`.  `o` is contiguous.  A module built with mask mode 3 applies the
 * traced mask_mod element by element (the dense mask input of the reference's TL decode,
 * core/lower/lower_decode_gqa.py:390-396).
 * Rows of different lengths (the varlen scheduling of the reference's kv-shared path,
 * cute_template_kvshared/kernels/get_mla_metadata.cu:8-75, flash_mla_interface.py:73-113): give `seqlens`, a
 * work list and `part_off`.  Each work item is one CTA's share {row, split of that row, first 128-key tile,
 * tiles}; row b's shares write the partial slots part_off[b] .. part_off[b + 1] - 1 (at most 32), a row with one
 * share writes `o` directly.  Build the list so that every share has about the same number of tiles
 * (attentionengine_b200/attn_engine/attn_decode.py: `schedule`).  Skv is then the longest row.
 * Paged K / V: give `block_table` [B, max_pages] (page = 128 keys = one tile); k / v are then pools
 * [num_pages, 128, Hkv, D] and k_stride / v_stride their (page, key, head) strides. */
typedef struct AeDecodeWorkItem {
  int32_t row, split, tile_begin, n_tiles;
} AeDecodeWorkItem;
typedef struct AeDecodeParams {
  const void* q; /* [B, Sq, Hq, D]    */
  const void* k; /* [B, Skv, Hkv, D]  */
  const void* v; /* [B, Skv, Hkv, DV] */
  void* o;       /* [B, Sq, Hq, DV] contiguous */
  int64_t q_stride[3], k_stride[3], v_stride[3]; /* (batch, seq, head) */
  float* o_partial;                                /* [B, n_split, Sq * Hq, DV] fp32 (n_split > 1) */
  float* rowscale_partial[AE_MAX_FINAL_ROWSCALES]; /* each [B, n_split, Sq * Hq]    (n_split > 1) */
  const void* custom[AE_MAX_CUSTOM_INPUTS];
  int64_t custom_stride[AE_MAX_CUSTOM_INPUTS][4];
  int32_t B, Hq, Hkv, Sq, Skv, n_split;
  uint32_t* status;
  /* optional (all null / 0 = one length, dense K / V, n_split shares per row) */
  const AeDecodeWorkItem* work; /* [n_items] */
  int32_t n_items;
  const int32_t* seqlens;     /* [B] */
  const int32_t* part_off;    /* [B + 1]; o_partial / rowscale_partial then hold part_off[B] slots */
  const int32_t* block_table; /* [B, max_pages] */
  int32_t max_pages, num_pages;
} AeDecodeParams;

int ae_launch_attn_decode(void* module, const AeDecodeParams* p, void* stream);
int ae_launch_decode_combine(void* module, const AeDecodeParams* p, void* stream);

/* ---- chunked linear attention / SSD scan, forward ----------------------------------------
 * Stands in for `LinearAttention.forward` after the q/k/v/decay mods
 * (core/template/tl_template/linear/linear_tl.py:1129-1156): `chunk_local_cumsum_scalar`,
 * `chunk_fwd_h_mod`, `chunk_fwd_o_mod`.  Layout [B, H, T, D] contiguous (as the reference);
 * q has HQ heads, k has HK heads, v / a / o have H heads (H a multiple of HQ and HK);
 * `a` is the per-step log-decay (fp32, <= 0).  DK = 128, DV = 64 or 128. */
typedef struct AeLinearParams {
  const void* q;  /* [B, HQ, T, DK] */
  const void* k;  /* [B, HK, T, DK] */
  const void* v;  /* [B, H, T, DV]  */
  const float* a; /* [B, H, T]      */
  void* o;        /* [B, H, T, DV]  */
  int32_t B, H, HQ, HK, T;
  uint32_t* status;
  /* Modules compiled with AE_LIN_MODS (config reserved[0] = 1) only, each optional: the scan runs on
   * v * vscale[b, h, t], the output is scan + v * dskip[h] (v as passed, unscaled), and the scaled v is written to v_out
   * (what the backward entry points take as v).  The Mamba2 block's `v * dt` and `+ D x` (attn_script/
   * mamba2_ngroup1.py:31-33; the reference runs such mods as eager PyTorch, linear_tl.py:1136-1144). */
  const void* vscale;   /* [B, H, T] fp32, or the 16-bit type when vscale_16bit != 0 */
  const float* dskip;   /* [H] */
  void* v_out;          /* [B, H, T, DV] 16-bit */
  int32_t vscale_16bit;
  /* Any module, optional: the state every chunk starts from, [B, H, ceil(T/128), DK, DV] 16-bit - the h_states operand of
   * ae_launch_linear_bwd, which then needs no ae_launch_linear_states (the reference's forward stores the same tensor,
   * linear_tl.py:142, 185-186). */
  void* h_states_out;
  /* Any module, optional: a decay mod of the form `decay * custom[heads]` (Mamba2's `decay_mod = dt * A`,
   * attn_script/mamba2_ngroup1.py:26-29) inside the kernel - the scan runs on a * ascale[h]. */
  const float* ascale; /* [H] */
} AeLinearParams;

int ae_launch_linear_fwd(void* module, const AeLinearParams* p, void* stream);

/* ---- row-scale mod of the linear-attention operator ---------------------------------------
 * Stands in for the eager PyTorch statements the reference generates for a mod of the form
 * `v * custom[b, h, t]` and for their hand-chained derivatives in `LinearAttention.forward / backward`
 * (core/template/tl_template/linear/linear_tl.py:1136-1144, 1203-1214; Mamba2's `v_mod = v * dt`,
 * attn_script/mamba2_ngroup1.py:31-33).  x, y, g, gx: [n_rows, head_dim] 16-bit contiguous (head_dim of the
 * module: 64, 128 or 256); s, gs: one value per row, fp32 or (module config reserved[0] = 1) the 16-bit type.
 * The module's kernel name selects the direction: "ae_rowscale_fwd" writes y = x * s; "ae_rowscale_bwd"
 * writes gx = g * s and gs = sum_d g * x.
 * Two more kernels of the same module kind add the per-head skip connection of the Mamba2 block (benchmark config 4:
 * o += D_skip[h] * x; no counterpart in the reference, whose harness passes D=None, benchmark/bench_utils.py:304-308),
 * for rows ordered (batch, head, step): s is then [n_heads] fp32 and a row's head is (row / rows_per_head) % n_heads.
 * "ae_skip_fwd" writes y = g + x * s[head] (g carries the scan output); "ae_skip_bwd" writes gx = g * s[head] and
 * gs[row] = sum_d g * x in fp32 (summed over batch and steps by the caller for the gradient of s).
 * "ae_vskip_bwd" is the backward of a block that uses both (v' = x * s[row] into the scan, y = o + x * d[head] after
 * it) in one pass over x: gx = g2 * s[row] + g * d[head], gs[row] = sum_d g2 * x (type of s), gs2[row] = sum_d g * x
 * (fp32), with g the gradient of y and g2 the gradient of v'.
 * "ae_head_sum" sums x [groups, G, T, D] over G into y [groups, T, D] with fp32 accumulation (n_rows = groups * T,
 * rows_per_head = T, n_heads = G; s unused): the sum of the per-head dq / dk of the reverse pass when q / k have fewer
 * heads than v (linear_tl.py:1198-1201). */
typedef struct AeRowScaleParams {
  const void* x;
  const void* s;
  void* y;
  const void* g;
  void* gx;
  void* gs;
  int64_t n_rows;
  int64_t rows_per_head; /* skip kernels only */
  int32_t n_heads;       /* skip kernels only */
  const void* g2;        /* ae_vskip_bwd only: gradient of the scaled rows */
  const float* d;        /* ae_vskip_bwd only: [n_heads] skip weights */
  float* gs2;            /* ae_vskip_bwd only: [n_rows] */
} AeRowScaleParams;

int ae_launch_rowscale(void* module, const AeRowScaleParams* p, void* stream);

/* ---- chunked linear attention / SSD scan, backward -------------------------------------
 * Stands in for the kernel part of `LinearAttention.backward`
 * (core/template/tl_template/linear/linear_tl.py:1158-1216): `chunk_fwd_h_mod_2` (state
 * recompute) = ae_launch_linear_states; `chunk_bwd_dh_mod` + `chunk_bwd_dqkg_mod` +
 * `chunk_bwd_dv_mod` + `compute_final_dg` = ae_launch_linear_bwd.  Gradients are with respect
 * to the kernel inputs (after the mods); dq / dk are per head of v and are summed by the
 * caller when q / k have fewer heads, as the reference does (:1198-1201).  DK = 128, DV = 64. */
typedef struct AeLinearBwdParams {
  const void* q;   /* [B, HQ, T, DK] */
  const void* k;   /* [B, HK, T, DK] */
  const void* v;   /* [B, H, T, DV]  */
  const float* a;  /* [B, H, T]      */
  const void* d_o; /* [B, H, T, DV]  */
  void* h_states;  /* scratch [B, H, ceil(T/128), DK, DV] 16-bit: chunk start-states */
  void* dq;        /* [B, H, T, DK] 16-bit */
  void* dk;        /* [B, H, T, DK] 16-bit */
  void* dv;        /* [B, H, T, DV] 16-bit */
  float* da;       /* [B, H, T] fp32 */
  int32_t B, H, HQ, HK, T;
  uint32_t* status;
  /* Only read by a reverse-pass module compiled with the block's mods inside (AeKernelConfig.reserved[0] = 1; the
   * forward's counterpart is AeLinearParams.vscale / dskip): v was x * vscale[b, h, t] and the output had
   * x * dskip[h] added.  `dv` then receives the gradient of x, dv * vscale + d_o * dskip[h], instead of dv. */
  const void* x;      /* [B, H, T, DV] 16-bit, 16-byte aligned */
  const void* vscale; /* [B, H, T] fp32, or 16-bit when vscale_16bit != 0 */
  const float* dskip; /* [H] */
  void* gs;           /* out [B, H, T] in the type of vscale: sum over DV of dv * x */
  float* gd;          /* out [B, H]: sum over t and DV of d_o * x (sum it over B for the gradient of dskip) */
  int32_t vscale_16bit;
  /* Any module, optional (both or neither): the forward ran with AeLinearParams.ascale.  `a` is the decay as passed
   * there; `da` then receives the gradient of that tensor and gasc [B, H] the per-(batch, head) sums of
   * (gradient of a * ascale[h]) * a - sum them over B for the gradient of ascale. */
  const float* ascale; /* [H] */
  float* gasc;         /* out [B, H] */
} AeLinearBwdParams;

int ae_launch_linear_states(void* module, const AeLinearBwdParams* p, void* stream);
int ae_launch_linear_bwd(void* module, const AeLinearBwdParams* p, void* stream);

/* ---- bring-up probe (tests only): one 128x128x128 tcgen05 GEMM -------------------
 * mode 0: d = a * b^T (a, b [128,128] 16-bit row-major);
 * mode 1: d = p * b   (p, b [128,128] 16-bit row-major). d is [128,128] fp32.
 * No counterpart in the reference. */
int ae_launch_probe(void* module, const void* a, const void* b, const void* p, float* d, int mode, uint32_t* status,
                    void* stream);

#ifdef __cplusplus
}
#endif
#endif /* AE_B200_H_ */
