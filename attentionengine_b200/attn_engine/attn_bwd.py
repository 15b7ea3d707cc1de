"""Backward launches of AttentionEngine.

Stands in for the generated ``_attention.backward`` of the reference
(attention_engine/core/template/tl_template/attn/attn_tl.py:582-601): ``mod_prep`` (only when
``OnlineFunc.backward`` reads doosum), ``mod_bwd`` and ``mod_post``.  Two forms:

* ``"fused"``: the reference's scheme.  One kv-stationary kernel (attn_bwd_fused.cuh) computes dK and dV and adds its
  dQ tiles in fp32 into a [B, S, Hq, D] buffer, a cast kernel converts that buffer: five contractions per tile.
  dQ is summed in an order that varies from run to run.
* ``"split"``: a dQ pass and a dK/dV pass that each recompute S and dP (seven contractions), no atomics,
  bit-reproducible, no fp32 buffer.

``AttentionEngine.bwd_mode`` picks one per engine; the tuned-config table (attentionengine_b200/tune.py) can name
one per problem; otherwise the default comes from ``AE_B200_BWD`` (``fused`` unless set: measured faster on every swept
shape, 4 % at head dim 128 and 16 % at head dim 64).
"""
from __future__ import annotations

import ctypes as C
import os
from dataclasses import dataclass

import torch

from .. import runtime as rt


DEFAULT_MODE = os.environ.get("AE_B200_BWD", "fused")
SMEM_MAX = 232448  # dynamic shared memory a CTA can have on sm_100 (227 KiB)


@dataclass
class BwdKernels:
    prep: rt.Module
    dq: rt.Module
    dkv: rt.Module
    bn: int      # kv rows per streamed tile of the dQ pass
    stages: int  # its K / V ring depth
    sources: dict | None = None  # kernel name -> generated CUDA source (kept for inspection and build checks)


@dataclass
class FusedBwdKernels:
    prep: rt.Module
    fused: rt.Module
    cast: rt.Module
    config: tuple  # (Q ring depth, dO ring depth, row warpgroups)
    sources: dict | None = None


def fused_tile_config(D: int, DV: int, ncs: int, tuned: dict | None = None):
    """(Q ring depth, dO ring depth, row warpgroups) of the one-pass backward.  K, V, the 128 x 128 dS tile and the
    32 KB of dQ staging boxes are resident; a Q tile is needed first in a step (S^T of the next tile) and released last
    (dK), a dO tile is read by dP^T and dV only, so at head dim 128 what is left holds two Q slots and one dO slot;
    smaller heads take deeper rings."""
    cfg = os.environ.get("AE_B200_FUSED_TILE")  # "Q stages,dO stages,row groups": tuning override
    if cfg:
        return tuple(int(x) for x in cfg.split(","))
    if tuned and tuned.get("fused_tile"):
        return tuple(tuned["fused_tile"])
    for qst, dost in ((4, 2), (3, 2), (3, 1), (2, 1)):
        if fused_smem_bytes(D, DV, ncs, qst, dost) <= SMEM_MAX:
            return qst, dost, 4
    raise NotImplementedError("one-pass backward: the tiles do not fit in shared memory")


def fused_smem_bytes(D, DV, ncs, qst, dost):
    """tiles + row-scale slots + 1008: enough for the kernel's carve-up from any 16-byte aligned base (the barrier
    block sits behind the slots or in the alignment gap)."""
    tiles = 128 * (D + DV) * 2 + 128 * (qst * D + dost * DV) * 2 + 128 * 128 * 2 + 4 * 2 * 4096  # + dQ staging boxes
    return tiles + 2 * 128 * ncs * 4 + 1008


def compile_fused(k) -> FusedBwdKernels:
    D, DV, low = k.D, k.DV, k.low
    ncs = len(low.final_names) + 1
    qst, dost, nwg = fused_tile_config(D, DV, ncs, k.tuned)
    smem = fused_smem_bytes(D, DV, ncs, qst, dost)
    cfg = rt.KernelConfig(kind=rt.KIND_ATTN_BWD_PREP, dtype=k.dtype_tag, head_dim=D, head_dim_v=DV, threads=256,
                          smem_bytes=0, stages=0, mask_mode=k.mask_mode)
    src_prep = rt.kernel_source("attn_bwd_prep.cuh", prelude=low.prelude_bwd)
    prep = rt.compile_module(src_prep, "ae_attn_bwd_prep", cfg)
    prelude = low.prelude_bwd + (f"#define AE_FU_QSTAGES {qst}\n#define AE_FU_DOSTAGES {dost}\n#define AE_FU_NWG {nwg}\n"
                                 f"#define AE_FU_SMEM {smem}\n"
                                 f"#define AE_FU_DEFER_ADDS {int(os.environ.get('AE_B200_BWD_DEFER', '1'))}\n"
                                 f"#define AE_FU_L2_AHEAD {int(os.environ.get('AE_B200_BWD_L2_AHEAD', k.tuned.get('fused_l2_ahead', 0)))}\n")
    src = rt.kernel_source("attn_bwd_fused.cuh", prelude=prelude)
    cfg = rt.KernelConfig(kind=rt.KIND_ATTN_BWD_FUSED, dtype=k.dtype_tag, head_dim=D, head_dim_v=DV,
                          threads=nwg * 128 + 64 + 128, smem_bytes=smem, stages=qst, mask_mode=k.mask_mode)
    fused = rt.compile_module(src, "ae_attn_bwd_fused", cfg)
    cfg = rt.KernelConfig(kind=rt.KIND_ATTN_BWD_CAST, dtype=k.dtype_tag, head_dim=D, head_dim_v=DV, threads=256,
                          smem_bytes=0, stages=0, mask_mode=k.mask_mode)
    cast = rt.compile_module(src, "ae_attn_bwd_dq_cast", cfg)
    return FusedBwdKernels(prep, fused, cast, (qst, dost, nwg), {"attn_bwd_prep": src_prep, "attn_bwd_fused": src})


def dq_tile_config(D: int, DV: int, tuned: dict | None = None):
    """(streamed kv-tile rows, K ring depth, V ring depth) of the dQ pass: Q and dO live in TMEM next to one S and one
    dP region of 128 columns and the dQ accumulator; three 128-row K and V slots fill 192 KB of shared memory at head
    dim 128.  With equal depths K and V of a step share one barrier pair (one wait less per step for the MMA warp);
    4 / 3 slots with separate barriers measured 3 % slower."""
    cfg = os.environ.get("AE_B200_BWD_TILE")  # "bn,K stages,V stages": tuning override
    if cfg:
        return tuple(int(x) for x in cfg.split(","))
    if tuned and tuned.get("dq_tile"):
        return tuple(tuned["dq_tile"])
    return 128, 3, 3


def dkv_tile_config(D: int, DV: int, tuned: dict | None = None):
    """(streamed q-tile rows, Q ring depth, dO ring depth, row warpgroups) of the dK/dV pass: one 128 x 128 S^T and
    dP^T region next to the two accumulators fill the 512 TMEM columns; K, V, three Q and two dO stages fill shared
    memory at head dim 128 (a Q slot is released last in a step and needed first, so it gets the extra stage)."""
    cfg = os.environ.get("AE_B200_DKV_TILE")  # "bn,q stages,dO stages,row groups,ts": tuning override
    if cfg:
        return tuple(int(x) for x in cfg.split(","))
    if tuned and tuned.get("dkv_tile"):
        return tuple(tuned["dkv_tile"])
    return (128, 3, 2, 4, 0) if max(D, DV) > 64 else (128, 3, 3, 4, 0)


def compile_bwd(k) -> BwdKernels:
    D, DV, low = k.D, k.DV, k.low
    bn, kst, vst = dq_tile_config(D, DV, k.tuned)
    defs = f"#define AE_BWD_BN {bn}\n#define AE_DQ_KSTAGES {kst}\n#define AE_DQ_VSTAGES {vst}\n"
    prelude = low.prelude_bwd + defs
    cfg = rt.KernelConfig(kind=rt.KIND_ATTN_BWD_PREP, dtype=k.dtype_tag, head_dim=D, head_dim_v=DV, threads=256,
                          smem_bytes=0, stages=0, mask_mode=k.mask_mode)
    src_prep = rt.kernel_source("attn_bwd_prep.cuh", prelude=prelude)
    prep = rt.compile_module(src_prep, "ae_attn_bwd_prep", cfg)
    smem_dq = bn * (kst * D + vst * DV) * 2 + 512 + 1024  # Q / dO land in the last K / V slot
    cfg = rt.KernelConfig(kind=rt.KIND_ATTN_BWD_DQ, dtype=k.dtype_tag, head_dim=D, head_dim_v=DV, threads=320,
                          smem_bytes=smem_dq, stages=kst, mask_mode=k.mask_mode)
    cfg.reserved[0] = bn
    # every 4th exponential of the dQ pass runs on the FMA pipe (measured 3 % faster there, slower in the other kernels)
    src_dq = rt.kernel_source("attn_bwd_dq.cuh", prelude=prelude, exp_poly=4)
    dq = rt.compile_module(src_dq, "ae_attn_bwd_dq", cfg)
    ncs = len(low.final_names) + 1
    bn_kv, qst, dost, nwg, ts = dkv_tile_config(D, DV, k.tuned)
    prelude_kv = low.prelude_bwd + (f"#define AE_BWD_BN {bn_kv}\n#define AE_KV_QSTAGES {qst}\n"
                                    f"#define AE_KV_DOSTAGES {dost}\n#define AE_KV_NWG {nwg}\n#define AE_KV_TS {ts}\n")
    # with K / V resident in TMEM they only pass through the last ring slots
    smem_kv = (0 if ts else 128 * (D + DV) * 2) + bn_kv * (qst * D + dost * DV) * 2 + 2 * bn_kv * ncs * 4 + 256
    # 1 KiB of slack lets the kernel align its base itself; where that would exceed the 227 KiB a CTA can have, the
    # base must already be aligned (the kernel checks and reports status 0x200 instead of running misaligned)
    slack = smem_kv + 1024 <= 232448
    if smem_kv > 232448:
        raise NotImplementedError("dK/dV pass: the streamed tiles do not fit in shared memory")
    smem_kv += 1024 if slack else 0
    prelude_kv += f"#define AE_KV_ALIGN_SLACK {int(slack)}\n"
    cfg = rt.KernelConfig(kind=rt.KIND_ATTN_BWD_DKV, dtype=k.dtype_tag, head_dim=D, head_dim_v=DV,
                          threads=nwg * 128 + 64, smem_bytes=smem_kv, stages=qst, mask_mode=k.mask_mode)
    cfg.reserved[0] = bn_kv
    src_dkv = rt.kernel_source("attn_bwd_dkv.cuh", prelude=prelude_kv)
    dkv = rt.compile_module(src_dkv, "ae_attn_bwd_dkv", cfg)
    return BwdKernels(prep, dq, dkv, bn, kst,
                      {"attn_bwd_prep": src_prep, "attn_bwd_dq": src_dq, "attn_bwd_dkv": src_dkv})


def _s3(t):
    return (C.c_int64 * 3)(t.stride(0), t.stride(1), t.stride(2))


# Batch ranges of the one-pass backward on streams of their own (see launch_bwd; 1: one launch).  Measured at the
# Llama-3.1-8B GQA 8K problem, alternating in one process under the power cap: 18.74 ms per step with 1, 18.79 with 2,
# 18.45 with 4.
BWD_PARTS = 4


def batch_ranges(B: int, ctas_per_batch_row: int, sms: int, want: int, min_rounds: int = 1) -> int:
    """Into how many equal batch ranges (4, 2 or 1) a pass over B batch rows is launched: at most ``want``, the batch
    has to divide, and a range must still bring ``min_rounds`` CTAs per SM."""
    for n in (4, 2):
        if n <= want and B % n == 0 and (B // n) * ctas_per_batch_row >= min_rounds * sms:
            return n
    return 1


def _batch_parts(B, Hq, Sq, dev):
    want = int(os.environ.get("AE_B200_BWD_PARTS", BWD_PARTS))
    sms = torch.cuda.get_device_properties(dev).multi_processor_count
    return batch_ranges(B, Hq * ((Sq + 127) // 128), sms, want, min_rounds=8)


def _side_streams(eng, dev, n):
    cache = eng.__dict__.setdefault("_bwd_streams", {})
    key = (dev.index if dev.index is not None else torch.cuda.current_device(), n)
    if key not in cache:
        cache[key] = ([torch.cuda.Stream(device=dev) for _ in range(n)], torch.cuda.Event(),
                      [torch.cuda.Event() for _ in range(n)])
    return cache[key]


def launch_bwd(eng, q, k, v, o, d_o, finals, custom, lists=None):
    mode = getattr(eng, "bwd_mode", None) or DEFAULT_MODE
    if mode not in ("fused", "split"):
        raise ValueError(f"bwd_mode {mode!r}: 'fused' or 'split'")
    kern = eng.kernels.bwd_fused if mode == "fused" else eng.kernels.bwd
    B, Sq, Hq, Skv, Hkv = eng._check_qkv(q, k, v)
    dev = q.device
    if d_o.stride(3) != 1 or d_o.stride(2) % 8 or d_o.stride(1) % 8 or d_o.data_ptr() % 16:
        d_o = d_o.contiguous()
    dq = torch.empty_like(q)
    dk = torch.empty_like(k)
    dv = torch.empty_like(v)
    p = rt.AttnBwdParams()
    p.q, p.k, p.v, p.o, p.d_o = q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), d_o.data_ptr()
    p.dq, p.dk, p.dv = dq.data_ptr(), dk.data_ptr(), dv.data_ptr()
    p.q_stride, p.k_stride, p.v_stride, p.o_stride, p.do_stride = _s3(q), _s3(k), _s3(v), _s3(o), _s3(d_o)
    p.dq_stride, p.dk_stride, p.dv_stride = _s3(dq), _s3(dk), _s3(dv)
    for i, f in enumerate(finals):
        p.final_rowscales[i] = f.data_ptr()
    delta = None
    if eng.lowered.uses_doosum:
        delta = torch.empty(B, Hq, Sq, dtype=torch.float32, device=dev)
        p.delta = delta.data_ptr()
    p.custom, p.custom_stride, keep = eng._custom_args(custom, Sq, Skv)
    if lists is None:  # direct callers; the autograd path hands over the lists its forward walked
        lists = eng._ensure_lists(dev, eng.block_mask if eng.extern_block_mask else None, B, Hq, Sq, Skv)
    if lists is not None:
        p.block_count, p.block_index = lists[0].data_ptr(), lists[1].data_ptr()
        p.block_count_t, p.block_index_t = lists[2].data_ptr(), lists[3].data_ptr()
    p.B, p.Hq, p.Hkv, p.Sq, p.Skv = B, Hq, Hkv, Sq, Skv
    p.status = eng._get_status(dev).data_ptr()
    stream = C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    L = rt.lib()
    # custom tensors may come along when none of them is indexed by the batch (stride slot 0): the kernels of a range
    # then see the same pointers and strides
    batch_free = all(p.custom_stride[i][0] == 0 for i in range(rt.AE_MAX_CUSTOM))
    n_parts = _batch_parts(B, Hq, Sq, dev) if (mode == "fused" and lists is None and batch_free) else 1
    if n_parts > 1:
        # Batch ranges on streams of their own: the HBM-bound kernels around the main one (clearing the fp32 dQ buffer,
        # delta = rowsum(O dO), the cast of dQ) of one range run next to the tensor-bound main kernel of another
        # instead of in front of and behind the whole pass.
        acc = torch.empty(B, Sq, Hq, eng.D, dtype=torch.float32, device=dev)
        main = torch.cuda.current_stream(dev)
        side, start, done = _side_streams(eng, dev, n_parts - 1)
        start.record(main)
        nb = B // n_parts
        for i in range(n_parts):
            st = main if i == 0 else side[i - 1]
            if i:
                st.wait_event(start)
            sl = slice(i * nb, (i + 1) * nb)
            p.q, p.k, p.v, p.o, p.d_o = (t[sl].data_ptr() for t in (q, k, v, o, d_o))
            p.dq, p.dk, p.dv, p.dq_accum = (t[sl].data_ptr() for t in (dq, dk, dv, acc))
            for j, f in enumerate(finals):
                p.final_rowscales[j] = f[sl].data_ptr()
            if delta is not None:
                p.delta = delta[sl].data_ptr()
            p.B = nb
            sp = C.c_void_p(st.cuda_stream)
            if delta is not None:
                rt.check(L.ae_launch_attn_bwd_prep(kern.prep.handle, C.byref(p), sp), "ae_launch_attn_bwd_prep")
            rt.check(L.ae_launch_attn_bwd_fused(kern.fused.handle, C.byref(p), sp), "ae_launch_attn_bwd_fused")
            rt.check(L.ae_launch_attn_bwd_dq_cast(kern.cast.handle, C.byref(p), sp), "ae_launch_attn_bwd_dq_cast")
            if i:
                done[i - 1].record(st)
                main.wait_event(done[i - 1])
        return dq, dk, dv
    if delta is not None:
        rt.check(L.ae_launch_attn_bwd_prep(kern.prep.handle, C.byref(p), stream), "ae_launch_attn_bwd_prep")
    if mode == "fused":
        acc = torch.empty(B, Sq, Hq, eng.D, dtype=torch.float32, device=dev)  # cleared by the launcher on the stream
        p.dq_accum = acc.data_ptr()
        rt.check(L.ae_launch_attn_bwd_fused(kern.fused.handle, C.byref(p), stream), "ae_launch_attn_bwd_fused")
        rt.check(L.ae_launch_attn_bwd_dq_cast(kern.cast.handle, C.byref(p), stream), "ae_launch_attn_bwd_dq_cast")
    else:
        rt.check(L.ae_launch_attn_bwd_dq(kern.dq.handle, C.byref(p), stream), "ae_launch_attn_bwd_dq")
        rt.check(L.ae_launch_attn_bwd_dkv(kern.dkv.handle, C.byref(p), stream), "ae_launch_attn_bwd_dkv")
    return dq, dk, dv
