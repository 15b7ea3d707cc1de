"""AttentionEngine / OnlineFunc: the operator API, re-pointed at the sm_100a back end.

Same constructor and call signature as the reference (attention_engine/attn_engine/attn_engine.py:
``OnlineFunc`` :16-105, ``AttentionEngine.__init__`` :109-115, shape-class dispatch
``_select_lower_template`` :218-332, ``__call__`` :388-395).  Instead of rendering a TileLang module
the constructor traces the user callables, lowers them to CUDA functor fragments
(``lower.cuda_lower``), splices them into the kernel templates under ``csrc/kernels`` and compiles
them with NVRTC through the C ABI; the call launches those kernels on the current CUDA stream.
"""
from __future__ import annotations

import os
import ctypes as C
from typing import Optional

import torch

from .. import runtime as rt
from ..core.transform.core import (CustomIO, SymbolicArray, SymbolScalar, Var, block_mask_counts)
from ..lower.cuda_lower import LoweredAttention, lower_attention


class OnlineFunc:
    """User-defined online (streaming) row normalisation, as in the reference
    (attn_engine.py:16-105):

    * ``online_fwd(scores, online_rowscales, b, h, q_idx) -> (scores, new_rowscales, o_scale)``
    * ``online_fwd_epilogue(o, online_rowscales, b, h, q_idx) -> (o, final_rowscales)``
    * ``forward(scores, final_rowscales, b, h, q_idx, kv_idx) -> p`` (recompute for backward)
    * ``backward(dp, scores, final_rowscales, doosum_rowscales, b, h, q_idx, kv_idx) -> dscores``
    * ``combine(final_rowscales) -> o_scale`` (split-KV merge)
    """

    def __init__(self, online_rowscales: dict, final_rowscales: dict, external_fwd_tensors: CustomIO):
        self.online_rowscales = online_rowscales
        self.final_rowscales = final_rowscales
        self.vars = {"scores": SymbolicArray(), "o_scale": None}
        self.external_fwd_tensors = external_fwd_tensors
        self.doosum_rowscales = SymbolicArray("doosum", Var("doosum"), shape_idx=["block_M"])

    @staticmethod
    def online_fwd(scores, online_rowscales, b, h, q_idx):
        return scores, online_rowscales, SymbolScalar("o_scale", Var("1"))

    @staticmethod
    def online_fwd_epilogue(o, online_rowscales, b, h, q_idx):
        return o, online_rowscales

    @staticmethod
    def forward(scores, final_rowscales, b, h, q_idx, kv_idx):
        return scores

    @staticmethod
    def backward(dp, scores, final_rowscales, doosum_rowscales, b, h, q_idx, kv_idx):
        return dp

    @staticmethod
    def combine(final_rowscales):
        return SymbolScalar("o_scale", Var("1"))


class H100:
    """Placeholder accepted for the reference's ``device=`` argument (autotuner/arch); the back end
    always targets B200."""


_DYN_PROBE = 1024  # sequence length on which a dynamic-shape engine classifies its mask
MAX_LIST_KV_TILES = 2048  # kv tiles a block list may cover (AE_MAX_KT of attn_fwd.cuh): 262,144 keys

_TORCH_DTYPES = {torch.float16: rt.DTYPE_F16, torch.bfloat16: rt.DTYPE_BF16}


def _strides3(t: torch.Tensor):
    # [B, S, H, D] -> (batch, seq, head) element strides
    return (C.c_int64 * 3)(t.stride(0), t.stride(1), t.stride(2))


def _block_lists(cnt: torch.Tensor, q_blk: int, kv_blk: int, Sq: int, Skv: int, B: int, H: int, device):
    """Per (b, h, q tile): ascending list of kept kv tiles, entry = tile | partial << 30.
    Returns (count [B,H,nq] int32, index [B,H,nq,nk] int32) and the transposed pair.  Runs where ``cnt`` lives: a
    call-time block mask on the GPU is turned into lists there, without a copy to the host."""
    b_, h_, nq, nk = cnt.shape
    dev = cnt.device
    rows = torch.clamp(Sq - torch.arange(nq, device=dev) * q_blk, max=q_blk).view(1, 1, nq, 1)
    cols = torch.clamp(Skv - torch.arange(nk, device=dev) * kv_blk, max=kv_blk).view(1, 1, 1, nk)
    full = cnt == rows * cols
    keep = cnt > 0

    def lists(keep_m, full_m):
        order = torch.argsort((~keep_m).to(torch.int8), dim=-1, stable=True)
        part = (~torch.gather(full_m, -1, order)).to(torch.int32)
        idx = (order.to(torch.int32) | (part << 30))
        return keep_m.sum(-1, dtype=torch.int32), idx

    c, i = lists(keep, full)
    ct, it = lists(keep.transpose(2, 3), full.transpose(2, 3))

    def ex(t):
        return t.expand(B, H, *t.shape[2:]).contiguous().to(device)

    return ex(c), ex(i), ex(ct), ex(it)


FWD_PAIR = 0  # 1: the forward over CTA pairs where it applies
FWD_FORM = (1, 0)  # (threads per score row, turn-taking) of the forward kernel when no tuned entry says otherwise


class _AttnKernels:
    """Compiled kernels of one engine instance."""

    def __init__(self, low: LoweredAttention, D: int, DV: int, dtype_tag: int, mask_mode: int, stages: int,
                 tuned: Optional[dict] = None):
        self.low = low
        self.D, self.DV, self.dtype_tag, self.mask_mode, self.stages = D, DV, dtype_tag, mask_mode, stages
        self.tuned = tuned or {}  # tile choices of the backward kernels (attentionengine_b200/tune.py)
        # forward form: threads per score row (1 or 2) and whether the two q tiles take turns; from the tuned table,
        # AE_B200_FWD_RSPLIT / AE_B200_FWD_TURNS override (experiments)
        rsplit, turns = self.tuned.get("fwd_form", FWD_FORM)
        rsplit = int(os.environ.get("AE_B200_FWD_RSPLIT", rsplit))
        turns = int(os.environ.get("AE_B200_FWD_TURNS", turns))
        self.fwd_form = (rsplit, turns)
        smem = 2 * 128 * D * 2 + stages * 128 * (D + DV) * 2 + 512 + 1024
        if rsplit > 1:
            smem += 2 * 2 * rsplit * 128 * 4  # partial row reductions exchanged between the threads of a row
        if mask_mode == 2:
            smem += 4 * MAX_LIST_KV_TILES  # the CTA's merged tile walk
        # forward over CTA pairs (tcgen05 cta_group::2): for the shapes it is written for, when the tuned entry or
        # AE_B200_FWD_PAIR asks for it
        pair = int(os.environ.get("AE_B200_FWD_PAIR", self.tuned.get("fwd_pair", FWD_PAIR)))
        self.fwd_pair = bool(pair) and mask_mode in (0, 1, 3) and DV == 128 and D in (64, 128)
        if self.fwd_pair:
            pstages = int(os.environ.get("AE_B200_FWD_PAIR_STAGES", self.tuned.get("fwd_pair_stages", 5)))
            smem = 128 * D * 2 + pstages * (64 * D * 2 + 128 * 64 * 2) + 512 + 2048 + 1024
            cfg = rt.KernelConfig(kind=rt.KIND_ATTN_FWD_PAIR, dtype=dtype_tag, head_dim=D, head_dim_v=DV, threads=320,
                                  smem_bytes=smem, stages=pstages, mask_mode=mask_mode)
            self.fwd_src = rt.kernel_source("attn_fwd_pair.cuh", prelude=low.prelude_fwd,
                                            defines={"AE_PAIR_STAGES": pstages, "AE_RSPLIT": 2,
                                                     "AE_PAIR_SCOPE": int(os.environ.get("AE_B200_PAIR_SCOPE", "0"))})
            self.fwd = rt.compile_module(self.fwd_src, "ae_attn_fwd_pair", cfg)
        else:
            cfg = rt.KernelConfig(kind=rt.KIND_ATTN_FWD, dtype=dtype_tag, head_dim=D, head_dim_v=DV,
                                  threads=rsplit * 256 + 64, smem_bytes=smem, stages=stages, mask_mode=mask_mode)
            self.fwd_src = rt.kernel_source("attn_fwd.cuh", prelude=low.prelude_fwd,
                                            defines={"AE_RSPLIT": rsplit, "AE_TURNS": turns})
            self.fwd = rt.compile_module(self.fwd_src, "ae_attn_fwd", cfg)
        self._bwd = None
        self._bwd_fused = None

    @property
    def bwd(self):
        """The two-pass backward (dQ pass + dK/dV pass)."""
        if self._bwd is None:
            from .attn_bwd import compile_bwd
            self._bwd = compile_bwd(self)
        return self._bwd

    @property
    def bwd_fused(self):
        """The one-pass backward (kv-stationary kernel with fp32 dQ accumulation + cast)."""
        if self._bwd_fused is None:
            from .attn_bwd import compile_fused
            self._bwd_fused = compile_fused(self)
        return self._bwd_fused


class _AttentionFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, eng, q, k, v, *custom):
        eng._check_qkv(q, k, v)
        with torch.cuda.device(q.device):  # the C ABI launches on the current device's context
            o, finals, lists = eng._launch_fwd(q, k, v, custom, block_mask=eng._call_block_mask, return_lists=True)
        ctx.eng = eng
        ctx.lists = lists  # the tile lists this forward walked: its backward walks the same ones
        ctx.n_custom = len(custom)
        ctx.save_for_backward(q, k, v, o, *finals, *custom)
        ctx.n_final = len(finals)
        return o

    @staticmethod
    def backward(ctx, d_o):
        eng = ctx.eng
        saved = ctx.saved_tensors
        q, k, v, o = saved[:4]
        finals = saved[4:4 + ctx.n_final]
        custom = saved[4 + ctx.n_final:]
        with torch.cuda.device(q.device):
            dq, dk, dv = eng._launch_bwd(q, k, v, o, d_o, finals, custom, ctx.lists)
        return (None, dq, dk, dv) + (None,) * ctx.n_custom


class AttentionEngine:
    def __init__(self, qkv_meta, custom_fwd_inputs, score_mod, mask_mod, online_func, mask_value="-inf",
                 device=None, backend="tl", tune=False, tune_file="", tune_bwd=False, tune_file_bwd="",
                 infer_mask=True, infer_mask_block_M=128, infer_mask_block_N=128, extern_block_mask=False,
                 kv_shared=False, tuned_config=None):
        if backend not in ("tl", "b200"):
            raise NotImplementedError(f"backend={backend!r}: only the B200 back end exists here "
                                      "(the reference's 'cute' sm_90a path is not part of it)")
        qm, km, vm = qkv_meta
        self.dtype = qm.dtype
        if self.dtype not in _TORCH_DTYPES:
            raise NotImplementedError(f"dtype {self.dtype}: fp16 and bf16 only")
        B, Hq, Sq, D = qm.shape
        _, Hkv, Skv, _ = km.shape
        DV = vm.shape[3]
        self.B, self.Hq, self.Hkv, self.Sq, self.Skv, self.D, self.DV = B, Hq, Hkv, Sq, Skv, D, DV
        self.custom_fwd_inputs = custom_fwd_inputs if custom_fwd_inputs is not None else CustomIO()
        self.score_mod, self.mask_mod, self.online_func = score_mod, mask_mod, online_func
        self.mask_value = mask_value
        self.extern_block_mask = extern_block_mask
        self.bwd_mode = None  # "fused" | "split"; None = the package default (attn_bwd.DEFAULT_MODE)
        self.block_mask = None
        self._call_block_mask = None
        self._lists = None
        self._status = None
        dynamic = any(isinstance(x, str) for x in (B, Hq, Sq, Skv))
        self._dynamic = dynamic
        self._lists_by_shape = {}

        # shape-class dispatch, as attn_engine.py:218-332
        self._mla = None
        self._decode = None
        if kv_shared:
            from .mla_decode import MlaDecode
            self._mla = MlaDecode(score_mod, online_func, self.custom_fwd_inputs, Hq, D, DV, self.dtype)
            self.tl_code = self._mla.src
            self.mask_mode = 0
            return
        ints = all(isinstance(x, int) for x in (Hq, Hkv, Sq))
        if ints and Sq != Skv and (isinstance(Skv, str) or not dynamic):
            # decode shape classes (reference: attn_engine.py:252-286): split-KV kernel + OnlineFunc.combine.  The KV
            # length (and the batch) may be named dims: a serving loop calls one engine with a growing cache.
            if isinstance(Skv, int) and Sq > Skv:
                raise NotImplementedError("q_len > kv_len is not an attention shape the reference defines")
            from .attn_decode import AttnDecode
            self._decode = AttnDecode(score_mod, mask_mod, online_func, self.custom_fwd_inputs, Hq, Hkv, Sq, D, DV,
                                      self.dtype, mask_value)
            self.tl_code = self._decode.src
            self.mask_mode = 0
            return
        # Value head dims above 128 run as independent 128-wide value blocks: O[:, block] depends on V[:, block] only, and
        # the backward is linear in dO, so the blocks' dQ / dK add up (torch autograd sums them) and dV is per block.
        # Each block recomputes the scores.  (The reference's lowering has a DV > 256 path of its own, lower.py:648-654.)
        self.DV_total = DV
        if isinstance(DV, int) and DV > 128:
            if DV % 128:
                raise NotImplementedError(f"value head dim {DV}: above 128 it must be a multiple of 128")
            DV = self.DV = 128
        if isinstance(D, str) or isinstance(DV, str) or D % 64 or DV % 64 or D > 128 or DV > 128:
            raise NotImplementedError(f"head dims D={D}, DV={DV}: the query / key head dim is a multiple of 64 up to 128, "
                                      "the value head dim a multiple of 64 up to 128 or a multiple of 128 above")
        if not isinstance(Hq, str) and not isinstance(Hkv, str):
            assert Hq % Hkv == 0, "query heads must be a multiple of kv heads"

        # mask classification (reference: lower.py:708-738)
        mask_mode = 0
        self._mask_counts = None
        if extern_block_mask:
            mask_mode = 2
        elif mask_mod is not None:
            if infer_mask and not dynamic:
                cnt = block_mask_counts(mask_mod, B, Hq, Sq, Skv, "cpu", 128, 128)
                causal_cnt = block_mask_counts(lambda b, h, q, kv: q >= kv, 1, 1, Sq, Skv, "cpu", 128, 128)
                if cnt.shape[:2] == (1, 1) and torch.equal(cnt, causal_cnt):
                    mask_mode = 1
                else:
                    rows = torch.clamp(Sq - torch.arange(cnt.shape[2]) * 128, max=128).view(1, 1, -1, 1)
                    cols = torch.clamp(Skv - torch.arange(cnt.shape[3]) * 128, max=128).view(1, 1, 1, -1)
                    mask_mode = 0 if bool((cnt == rows * cols).all()) else 2
                    self._mask_counts = cnt
                if infer_mask_block_M == 128 and infer_mask_block_N == 128:
                    self.block_mask = (cnt > 0).to(torch.int8).expand(B, Hq, cnt.shape[2], cnt.shape[3])
            elif infer_mask:
                # Dynamic shapes (named dims, reference: lower.py:626-629): the kernels do not depend on B, H or S, only
                # the tile lists do.  The mask is classified on a probe shape: exactly causal there -> analytic bounds
                # for every length; anything else -> lists, built per runtime shape at the first call with it.
                probe = block_mask_counts(mask_mod, 2, 2, _DYN_PROBE, _DYN_PROBE, "cpu", 128, 128)
                causal_cnt = block_mask_counts(lambda b, h, q, kv: q >= kv, 1, 1, _DYN_PROBE, _DYN_PROBE, "cpu", 128, 128)
                mask_mode = 1 if probe.shape[:2] == (1, 1) and torch.equal(probe, causal_cnt) else 2
            else:
                mask_mode = 3  # no block information: visit every tile, mask every element
        self.mask_mode = mask_mode

        # tile / stage choices (reference: the tuned-config json of attn_tl.py:474-500).  `tuned_config` is what the
        # sweep itself passes; otherwise the caller's tune_file (filled by a sweep when tune=True), then the package's
        # own table, then the built-in defaults.
        if tuned_config is None:
            from .. import tune as _tune
            keys = _tune.problem_keys(B, Hq, Hkv, Sq, Skv, D, DV, self.dtype, mask_mode)
            tuned_config = _tune.resolve(dict(score_mod=score_mod, mask_mod=mask_mod, online_func=online_func,
                                              custom_io=self.custom_fwd_inputs, mask_value=mask_value), keys,
                                         bool(tune) and not dynamic, tune_file)
        self.tuned_config = tuned_config
        stages = int(tuned_config.get("stages", 2))
        low = lower_attention(score_mod, mask_mod, online_func, self.custom_fwd_inputs, D=D, DV=DV,
                              bf16=self.dtype == torch.bfloat16, mask_mode=mask_mode, stages=stages,
                              mask_value=mask_value)
        self.lowered = low
        self.kernels = _AttnKernels(low, D, DV, _TORCH_DTYPES[self.dtype], mask_mode, stages, tuned_config)
        if tuned_config.get("mode") in ("fused", "split"):
            self.bwd_mode = tuned_config["mode"]
        self.tl_code = self.kernels.fwd_src  # name kept from the reference (attn_engine.py:365): generated source

    # ------------------------------------------------------------------------------------------
    def _get_status(self, device):
        if self._status is None or self._status.device != device:
            self._status = torch.zeros(1, dtype=torch.int32, device=device)
        return self._status

    def check_status(self):
        """Raise if a kernel of this engine recorded a bounded-wait timeout."""
        if self._mla is not None:
            self._status = self._mla._status
        if self._decode is not None:
            self._status = self._decode._status
        if self._status is not None:
            code = int(self._status.item())
            if code:
                self._status.zero_()
                raise rt.AeError(f"kernel reported status 0x{code:x} (a bounded wait gave up)")

    def _ensure_lists(self, device, block_mask: Optional[torch.Tensor], B, Hq, Sq, Skv):
        """Tile lists (count, index, transposed count, transposed index) of a mode-2 engine for one call, or None.
        The kernels index the lists with the runtime tile grid, so every source is checked against it here."""
        if self.mask_mode != 2:
            return None
        nq, nk = -(-Sq // 128), -(-Skv // 128)
        if block_mask is not None:
            if block_mask.dim() != 4 or tuple(block_mask.shape[2:]) != (nq, nk) or \
                    block_mask.shape[0] not in (1, B) or block_mask.shape[1] not in (1, Hq):
                raise ValueError(f"block_mask has shape {tuple(block_mask.shape)}; expected [1 or {B}, 1 or {Hq}, {nq}, {nk}] "
                                 f"(one entry per 128 x 128 tile of the {Sq} x {Skv} score matrix)")
            cnt = block_mask.to(torch.int32)  # stays on the mask's device: no host round trip per call
            if self.mask_mod is None:
                # listed blocks are complete blocks
                rows = torch.clamp(Sq - torch.arange(nq, device=cnt.device) * 128, max=128).view(1, 1, nq, 1)
                cols = torch.clamp(Skv - torch.arange(nk, device=cnt.device) * 128, max=128).view(1, 1, 1, nk)
                cnt = (cnt > 0).to(torch.int32) * rows * cols
            return _block_lists(cnt, 128, 128, Sq, Skv, B, Hq, device)
        if self._dynamic and self.mask_mod is not None:
            key = (B, Hq, Sq, Skv, str(device))
            if key not in self._lists_by_shape:
                if len(self._lists_by_shape) >= 16:  # a serving loop over many lengths must not grow without bound
                    self._lists_by_shape.pop(next(iter(self._lists_by_shape)))
                cnt = block_mask_counts(self.mask_mod, B, Hq, Sq, Skv, "cpu", 128, 128)
                self._lists_by_shape[key] = _block_lists(cnt, 128, 128, Sq, Skv, B, Hq, device)
            return self._lists_by_shape[key]
        if self._mask_counts is None:
            raise ValueError("this engine needs block_mask= at call time (extern_block_mask=True)")
        if (B, Hq, Sq, Skv) != (self.B, self.Hq, self.Sq, self.Skv):
            raise ValueError(f"this engine's tile lists were inferred for (B, Hq, Sq, Skv) = "
                             f"{(self.B, self.Hq, self.Sq, self.Skv)}; the call has {(B, Hq, Sq, Skv)}. "
                             "Build the engine with named dims (meta_tensor('B', 'H', 'S', D)) for varying shapes")
        if self._lists is None or self._lists[0].device != device:
            self._lists = _block_lists(self._mask_counts, 128, 128, Sq, Skv, B, Hq, device)
        return self._lists

    def _custom_args(self, custom, Sq, Skv):
        specs = self.lowered.custom
        if len(custom) != len(specs):
            raise TypeError(f"expected {len(specs)} custom input(s) {[s.name for s in specs]}, got {len(custom)}")
        ptrs = (C.c_void_p * rt.AE_MAX_CUSTOM)()
        strides = ((C.c_int64 * 4) * rt.AE_MAX_CUSTOM)()
        keep = []
        for sp, t in zip(specs, custom):
            want = self.dtype if sp.is_16bit else torch.float32
            if t.dtype != want:
                t = t.to(want)
            if t.dim() != len(sp.shape):
                raise ValueError(f"custom input {sp.name}: expected {len(sp.shape)} dims, got {tuple(t.shape)}")
            if sp.is_16bit and (Sq % 128 or Skv % 128):
                raise NotImplementedError("tile-shaped custom inputs need sequence lengths that are multiples of 128")
            keep.append(t)
            ptrs[sp.slot] = t.data_ptr()
            for d, slot in enumerate(sp.dim_slots):
                if slot >= 0 and t.shape[d] > 1:
                    strides[sp.slot][slot] = t.stride(d)
        return ptrs, strides, keep

    def _check_qkv(self, q, k, v):
        for name, t in (("q", q), ("k", k), ("v", v)):
            if not t.is_cuda:
                raise rt.AeError(f"{name} must be a CUDA tensor: this back end has no CPU path")
            if t.dtype != self.dtype:
                raise TypeError(f"{name} has dtype {t.dtype}, engine was built for {self.dtype}")
            if t.dim() != 4 or t.stride(3) != 1:
                raise ValueError(f"{name} must be [B, S, H, D] with a contiguous last dimension")
        B, Sq, Hq, D = q.shape
        _, Skv, Hkv, _ = k.shape
        if (D, v.shape[3]) != (self.D, self.DV):
            raise ValueError(f"head dims {(D, v.shape[3])} differ from the engine's {(self.D, self.DV)}")
        if Hq % Hkv or v.shape[1] != Skv or v.shape[2] != Hkv or k.shape[0] != B or v.shape[0] != B:
            raise ValueError("inconsistent q/k/v shapes")
        return B, Sq, Hq, Skv, Hkv

    def _launch_fwd(self, q, k, v, custom, block_mask=None, return_lists=False):
        B, Sq, Hq, Skv, Hkv = self._check_qkv(q, k, v)
        dev = q.device
        o = torch.empty(B, Sq, Hq, self.DV, dtype=self.dtype, device=dev)
        finals = [torch.empty(B, Hq, Sq, dtype=torch.float32, device=dev) for _ in self.lowered.final_names]
        p = rt.AttnParams()
        p.q, p.k, p.v, p.o = q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr()
        p.q_stride, p.k_stride, p.v_stride, p.o_stride = _strides3(q), _strides3(k), _strides3(v), _strides3(o)
        for i, f in enumerate(finals):
            p.final_rowscales[i] = f.data_ptr()
        p.custom, p.custom_stride, keep = self._custom_args(custom, Sq, Skv)
        lists = self._ensure_lists(dev, block_mask if block_mask is not None else (
            self.block_mask if self.extern_block_mask else None), B, Hq, Sq, Skv)
        if lists is not None:
            p.block_count, p.block_index = lists[0].data_ptr(), lists[1].data_ptr()
        p.B, p.Hq, p.Hkv, p.Sq, p.Skv = B, Hq, Hkv, Sq, Skv
        p.status = self._get_status(dev).data_ptr()
        stream = torch.cuda.current_stream(dev).cuda_stream
        rt.check(rt.lib().ae_launch_attn_fwd(self.kernels.fwd.handle, C.byref(p), C.c_void_p(stream)),
                 "ae_launch_attn_fwd")
        return (o, finals, lists) if return_lists else (o, finals)

    def decode_paged(self, q, kcache, block_table, cache_seqlens, num_split=None):
        """kv_shared engines: decode over a paged KV pool with one length per batch row, returns (out, lse)."""
        if self._mla is None:
            raise NotImplementedError("paged decode is built for kv_shared (MLA) engines")
        return self._mla.paged(q, kcache, block_table, cache_seqlens, num_split)

    def decode_schedule(self, cache_seqlens, device=None):
        """Decode engines: the work list for rows of these lengths (see AttnDecode.schedule); reuse it across layers."""
        if self._decode is None:
            raise NotImplementedError("decode_schedule belongs to decode engines (q_len != kv_len)")
        return self._decode.schedule(cache_seqlens, device)

    def decode_varlen(self, q, k, v, cache_seqlens, *custom, block_table=None, metadata=None):
        """Decode engines (MHA / GQA): one length per batch row, dense or paged (128-key pages) K / V."""
        if self._decode is None:
            raise NotImplementedError("decode_varlen belongs to decode engines (q_len != kv_len)")
        return self._decode.decode_varlen(q, k, v, cache_seqlens, *custom, block_table=block_table, metadata=metadata)

    def _launch_bwd(self, q, k, v, o, d_o, finals, custom, lists=None):
        from .attn_bwd import launch_bwd
        return launch_bwd(self, q, k, v, o, d_o, finals, custom, lists)

    def __call__(self, *args, **kargs):
        if self._mla is not None:
            if len(args) == 2:
                # mod(q [B, 1, H, 576], kcache [B * S / 64, 64, 1, 576]) -> (out, lse): the call of the reference's
                # CuTe kv-shared script (attn_script/mla_decode_cute.py:295-303), pages in batch order, full rows
                q, kcache = args
                B = q.shape[0]
                pages = kcache.shape[0] // B
                table = torch.arange(B * pages, dtype=torch.int32, device=q.device).view(B, pages)
                lens = torch.full((B,), pages * 64, dtype=torch.int32, device=q.device)
                return self._mla.paged(q, kcache, table, lens)
            return self._mla(*args)
        if self._decode is not None:
            return self._decode(*args)
        block_mask = kargs.get("block_mask")
        if block_mask is not None:
            if self.mask_mode != 2:
                raise ValueError("block_mask= needs an engine built with extern_block_mask=True")
            self.block_mask = block_mask  # kept as the reference keeps it; the call below uses its own copy
            self.extern_block_mask = True
        q, k, v, *custom = args
        self._call_block_mask = block_mask if block_mask is not None else (
            self.block_mask if self.extern_block_mask else None)
        try:
            if getattr(self, "DV_total", self.DV) != self.DV:
                if v.shape[-1] != self.DV_total:
                    raise ValueError(f"v has head dim {v.shape[-1]}, engine was built for {self.DV_total}")
                outs = [_AttentionFn.apply(self, q, k, v[..., i:i + self.DV], *custom)
                        for i in range(0, self.DV_total, self.DV)]
                return torch.cat(outs, dim=-1)
            return _AttentionFn.apply(self, q, k, v, *custom)
        finally:
            self._call_block_mask = None
