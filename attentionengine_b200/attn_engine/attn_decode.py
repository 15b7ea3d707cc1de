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

Rows of different lengths and paged K / V (the serving call of the reference's kv-shared path,
core/template/cute_template_kvshared/flash_mla_interface.py:73-113 with its scheduler
kernels/get_mla_metadata.cu:8-75) are ``decode_varlen``: ``schedule(cache_seqlens)`` cuts every row into shares of
about equal size, one CTA each, and the result is reused by every layer of a decode step.
A ``mask_mod`` is applied element by element (mask mode 3), the dense mask input of the reference's TL decode
(core/lower/lower_decode_gqa.py:390-396); the query position it sees is the row's index among the engine's q_len
positions.
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
        mask_mode = 0 if mask_mod is None else 3
        self.low = lower_attention(score_mod, mask_mod, online_func, custom_fwd_inputs, D=D, DV=DV, bf16=bf16,
                                   mask_mode=mask_mode, stages=2, mask_value=mask_value)
        # at most 128 rows: one q tile in shared memory, its space goes to a third K / V stage
        nq, stages = (1, 3) if self.rows <= 128 else (2, 2)
        smem = nq * 128 * D * 2 + stages * 128 * (D + DV) * 2 + 512 + 1024
        cfg = rt.KernelConfig(kind=rt.KIND_ATTN_DECODE, dtype=tag, head_dim=D, head_dim_v=DV, threads=320,
                              smem_bytes=smem, stages=stages, mask_mode=mask_mode)
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

    # ------------------------------------------------------------------------------------------------------
    # rows of different lengths
    # ------------------------------------------------------------------------------------------------------
    def schedule(self, cache_seqlens, device=None, waves: int = 1):
        """Work list for a batch whose rows hold ``cache_seqlens[b]`` keys: every row is cut into shares of at most
        ``g`` 128-key tiles, ``g`` chosen so that the shares of all rows and head units fill the GPU ``waves`` times
        (at least 2 tiles per share, at most 32 shares per row).  Returns a dict of device tensors that
        ``decode_varlen`` takes; compute it once per decode step and reuse it for every layer (the reference's
        ``get_mla_metadata`` is used the same way).  Reads the lengths on the host (one small copy)."""
        lens = torch.as_tensor(cache_seqlens).to("cpu", torch.int64)
        if lens.dim() != 1 or int(lens.min()) < 1:
            raise ValueError("cache_seqlens must be a 1-D tensor of positive lengths")
        B = lens.numel()
        units = self.Hkv if self.Hq > self.Hkv else self.Hq
        tiles = (lens + 127) // 128
        if self.combine is None:
            g = int(tiles.max())  # no combine: one share per row
        else:
            total = int(tiles.sum()) * units
            g = max(2, -(-total // (N_SM * waves)))
            g = max(g, -(-int(tiles.max()) // 32))
        items, part_off = [], [0]
        for b in range(B):
            nt = int(tiles[b])
            n = -(-nt // g)
            per = -(-nt // n)
            n = -(-nt // per)  # no empty share
            for sidx in range(n):
                items.append((b, sidx, sidx * per, min(per, nt - sidx * per)))
            part_off.append(part_off[-1] + n)
        dev = device if device is not None else (cache_seqlens.device if isinstance(cache_seqlens, torch.Tensor)
                                                 and cache_seqlens.is_cuda else torch.device("cuda"))
        return {"work": torch.tensor(items, dtype=torch.int32).to(dev), "n_items": len(items),
                "part_off": torch.tensor(part_off, dtype=torch.int32).to(dev), "n_slots": part_off[-1],
                "seqlens": lens.to(torch.int32).to(dev), "max_seqlen": int(lens.max()), "tiles_per_share": g, "B": B}

    def decode_varlen(self, q, k, v, cache_seqlens, *custom, block_table=None, metadata=None):
        """``q`` [B, q_len, Hq, D]; dense ``k`` / ``v`` [B, S_max, Hkv, D] of which row b uses its first
        ``cache_seqlens[b]`` keys, or, with ``block_table`` [B, max_pages] int32, pools [num_pages, 128, Hkv, D]
        whose pages a row lists in order.  ``metadata`` = ``schedule(cache_seqlens)`` (computed here when absent)."""
        meta = metadata if metadata is not None else self.schedule(cache_seqlens, q.device)
        return self._run(q, k, v, custom, meta, block_table)

    def __call__(self, q, k, v, *custom):
        return self._run(q, k, v, custom, None, None)

    def _run(self, q, k, v, custom, meta, block_table):
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
        if block_table is not None:
            if meta is None:
                raise ValueError("paged K / V go through decode_varlen")
            if Skv != 128 or k.stride(0) != 128 * k.stride(1) or v.stride(0) != 128 * v.stride(1):
                raise ValueError("paged K / V pools are [num_pages, 128, Hkv, D] with the keys of a page contiguous")
            if block_table.dtype != torch.int32 or block_table.dim() != 2 or block_table.shape[0] != B or \
                    not block_table.is_contiguous() or block_table.shape[1] * 128 < meta["max_seqlen"]:
                raise ValueError("block_table must be contiguous int32 [B, max_pages] covering the longest row")
        elif k.shape[0] != B:
            raise ValueError("q / k / v shapes differ from the engine's")
        if meta is not None and (meta["B"] != B or (block_table is None and meta["max_seqlen"] > Skv)):
            raise ValueError("the schedule was made for other lengths than these tensors hold")
        specs = self.low.custom
        if len(custom) != len(specs):
            raise TypeError(f"expected {len(specs)} custom input(s) {[s.name for s in specs]}, got {len(custom)}")
        dev = q.device
        n_split = 1 if meta is not None else (self.num_split or self.pick_splits(B, Skv))
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
        n_slots = meta["n_slots"] if meta is not None else (B * n_split if n_split > 1 else 0)
        if n_slots:
            part = torch.empty(n_slots, Sq * Hq, self.DV, dtype=torch.float32, device=dev)
            p.o_partial = part.data_ptr()
            keep.append(part)
            for i in range(len(self.low.final_names)):
                f = torch.empty(n_slots, Sq * Hq, dtype=torch.float32, device=dev)
                p.rowscale_partial[i] = f.data_ptr()
                keep.append(f)
        p.B, p.Hq, p.Hkv, p.Sq, p.Skv, p.n_split = B, Hq, Hkv, Sq, Skv, n_split
        if meta is not None:
            p.work, p.n_items = meta["work"].data_ptr(), meta["n_items"]
            p.seqlens, p.part_off = meta["seqlens"].data_ptr(), meta["part_off"].data_ptr()
            p.Skv = meta["max_seqlen"]
            if block_table is not None:
                p.block_table, p.max_pages, p.num_pages = block_table.data_ptr(), block_table.shape[1], k.shape[0]
        if self._status is None or self._status.device != dev:
            self._status = torch.zeros(1, dtype=torch.int32, device=dev)
        p.status = self._status.data_ptr()
        stream = C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
        rt.check(rt.lib().ae_launch_attn_decode(self.kernel.handle, C.byref(p), stream), "ae_launch_attn_decode")
        if n_split > 1 or (meta is not None and meta["n_slots"] > B):
            rt.check(rt.lib().ae_launch_decode_combine(self.combine.handle, C.byref(p), stream), "ae_launch_decode_combine")
        self.last_num_split = n_split if meta is None else meta["n_slots"] / B
        return o
