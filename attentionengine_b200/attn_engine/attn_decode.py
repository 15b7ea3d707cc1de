"""Split-KV decode for MHA / GQA: ``mod(q, k, v, *custom) -> o`` with ``q_len != kv_len``.

Reference: shape-class dispatch attention_engine/attn_engine/attn_engine.py:252-286 (GQA decode needs
``q_len == 1``), lowering core/lower/lower_decode.py / lower_decode_gqa.py, templates
core/template/tl_template/attn/attn_decode_tl.py:34-206 (split kernel + ``combine``), scripts
attn_script/gqa_inference.py and mha_inference.py.  Forward only, as in the reference.

The kernel is the forward attention kernel built with ``AE_DECODE``: the query rows of one head unit (the
query heads of a kv head's group, or the positions of one head) fill one tile, so K / V of a kv head are read
once per split whatever the group size; the splits' results are merged by the traced ``OnlineFunc.combine``.
The reference fixes ``num_split = 4`` (attn_decode_tl.py:230-236); here it is chosen so that the CTAs cover the
GPU once.
"""
from __future__ import annotations

import ctypes as C

import torch

from .. import runtime as rt
from ..lower.cuda_lower import lower_attention, lower_combine

N_SM = 148
MAX_ROWS = 256  # two 128-row tiles per CTA


class AttnDecode:
    def __init__(self, score_mod, mask_mod, online_func, custom_fwd_inputs, Hq: int, Hkv: int, Sq: int, D: int, DV: int,
                 dtype, mask_value="-inf"):
        if mask_mod is not None:
            raise NotImplementedError("decode takes no mask_mod: every query row sees the whole KV range")
        if Hq % Hkv:
            raise ValueError("query heads must be a multiple of kv heads")
        if Hq > Hkv and Sq != 1:
            raise NotImplementedError("decode with grouped query heads takes q_len == 1 (as the reference does)")
        self.rows = Hq // Hkv if Hq > Hkv else Sq
        if self.rows > MAX_ROWS:
            raise NotImplementedError(f"decode packs at most {MAX_ROWS} query rows per head unit, got {self.rows}")
        if D % 64 or DV % 64 or D > 128 or DV > 128:
            raise NotImplementedError(f"head dims D={D}, DV={DV}: multiples of 64 up to 128 are supported")
        self.Hq, self.Hkv, self.Sq, self.D, self.DV, self.dtype = Hq, Hkv, Sq, D, DV, dtype
        bf16 = dtype == torch.bfloat16
        tag = rt.DTYPE_BF16 if bf16 else rt.DTYPE_F16
        self.low = lower_attention(score_mod, None, online_func, custom_fwd_inputs, D=D, DV=DV, bf16=bf16, mask_mode=0,
                                   stages=2, mask_value=mask_value)
        # at most 128 rows: one q tile in shared memory, its space goes to a third K / V stage
        nq, stages = (1, 3) if self.rows <= 128 else (2, 2)
        smem = nq * 128 * D * 2 + stages * 128 * (D + DV) * 2 + 512 + 1024
        cfg = rt.KernelConfig(kind=rt.KIND_ATTN_DECODE, dtype=tag, head_dim=D, head_dim_v=DV, threads=320,
                              smem_bytes=smem, stages=stages, mask_mode=0)
        cfg.reserved[1] = len(self.low.final_names)
        prelude = self.low.prelude_fwd.replace("#define AE_STAGES 2\n", f"#define AE_STAGES {stages}\n")
        assert f"#define AE_STAGES {stages}\n" in prelude
        self.src = rt.kernel_source("attn_fwd.cuh", prelude=prelude + f"#define AE_DECODE 1\n#define AE_NQ {nq}\n")
        self.kernel = rt.compile_module(self.src, "ae_attn_fwd", cfg)
        self.combine = None
        self.combine_src = None
        from .attn_engine import OnlineFunc
        overridden = getattr(type(online_func), "combine", None) is not OnlineFunc.combine
        # OnlineFunc.combine left at its default gives every split the weight 1: right for online functions without
        # row state (their partial outputs add up); with row state and no combine of its own the engine keeps one split.
        if overridden or not self.low.final_names:
            functor = lower_combine(online_func)
            if functor is not None:
                comb = (rt.KERNEL_DIR / "mla_combine.cuh").read_text().replace("//%%AE_COMBINE_FUNCTOR%%", functor)
                head = (rt.KERNEL_DIR / "ae_sm100.cuh").read_text().replace("#pragma once\n", "") + \
                    (rt.KERNEL_DIR / "ae_args.h").read_text()
                defs = f"#define AE_BF16 {int(bf16)}\n#define AE_NFINAL {len(self.low.final_names)}\n"
                self.combine_src = head + defs + comb
                cfg2 = rt.KernelConfig(kind=rt.KIND_MLA_COMBINE, dtype=tag, head_dim=D, head_dim_v=DV, threads=128,
                                       smem_bytes=0)
                self.combine = rt.compile_module(self.combine_src, "ae_mla_combine", cfg2)
        self.num_split = None  # None = choose per call
        self.last_num_split = None
        self._status = None

    def pick_splits(self, B: int, Skv: int) -> int:
        """Split count that minimises waves x (kv tiles per split + 3): a CTA occupies an SM alone, so the CTAs run in
        waves of 148, and each CTA pays about three tile periods to fill its pipeline and write its partials (measured
        at B = 16: 2 splits 0.131 ms, 8 splits 0.139 ms).  No empty split; one split when the online function has row
        state but no combine of its own."""
        if self.combine is None:
            return 1
        units = B * (self.Hkv if self.Hq > self.Hkv else self.Hq)
        n_tiles = -(-Skv // 128)
        best, best_cost = 1, None
        for n in range(1, min(32, n_tiles) + 1):
            tps = -(-n_tiles // n)
            if (n - 1) * tps >= n_tiles:
                continue
            cost = -(-units * n // N_SM) * (tps + 3)
            if best_cost is None or cost < best_cost:
                best, best_cost = n, cost
        return best

    def __call__(self, q, k, v, *custom):
        for name, t in (("q", q), ("k", k), ("v", v)):
            if not t.is_cuda:
                raise rt.AeError(f"{name} must be a CUDA tensor: this back end has no CPU path")
            if t.dtype != self.dtype:
                raise TypeError(f"{name} has dtype {t.dtype}, engine was built for {self.dtype}")
            if t.dim() != 4 or t.stride(3) != 1:
                raise ValueError(f"{name} must be [B, S, H, D] with a contiguous last dimension")
        B, Sq, Hq, D = q.shape
        _, Skv, Hkv, _ = k.shape
        if (Sq, Hq, Hkv, D, v.shape[3]) != (self.Sq, self.Hq, self.Hkv, self.D, self.DV) or v.shape[:3] != k.shape[:3]:
            raise ValueError("q / k / v shapes differ from the engine's")
        specs = self.low.custom
        if len(custom) != len(specs):
            raise TypeError(f"expected {len(specs)} custom input(s) {[s.name for s in specs]}, got {len(custom)}")
        dev = q.device
        n_split = self.num_split or self.pick_splits(B, Skv)
        if n_split > 1 and self.combine is None:
            raise ValueError("more than one split needs OnlineFunc.combine")
        o = torch.empty(B, Sq, Hq, self.DV, dtype=self.dtype, device=dev)
        p = rt.DecodeParams()
        p.q, p.k, p.v, p.o = q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr()
        for name, t in (("q_stride", q), ("k_stride", k), ("v_stride", v)):
            setattr(p, name, (C.c_int64 * 3)(t.stride(0), t.stride(1), t.stride(2)))
        keep = []
        for sp, t in zip(specs, custom):
            if sp.is_16bit:
                raise NotImplementedError("tile-shaped custom inputs are not wired into the decode kernel")
            t = t.to(torch.float32)
            keep.append(t)
            p.custom[sp.slot] = t.data_ptr()
            for d, slot in enumerate(sp.dim_slots):
                if slot >= 0 and t.shape[d] > 1:
                    p.custom_stride[sp.slot][slot] = t.stride(d)
        if n_split > 1:
            part = torch.empty(B, n_split, Sq * Hq, self.DV, dtype=torch.float32, device=dev)
            p.o_partial = part.data_ptr()
            keep.append(part)
            for i in range(len(self.low.final_names)):
                f = torch.empty(B, n_split, Sq * Hq, dtype=torch.float32, device=dev)
                p.rowscale_partial[i] = f.data_ptr()
                keep.append(f)
        p.B, p.Hq, p.Hkv, p.Sq, p.Skv, p.n_split = B, Hq, Hkv, Sq, Skv, n_split
        if self._status is None or self._status.device != dev:
            self._status = torch.zeros(1, dtype=torch.int32, device=dev)
        p.status = self._status.data_ptr()
        stream = C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
        rt.check(rt.lib().ae_launch_attn_decode(self.kernel.handle, C.byref(p), stream), "ae_launch_attn_decode")
        if n_split > 1:
            rt.check(rt.lib().ae_launch_decode_combine(self.combine.handle, C.byref(p), stream), "ae_launch_decode_combine")
        self.last_num_split = n_split
        return o
