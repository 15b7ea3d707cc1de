"""MLA (kv_shared) decode path of AttentionEngine: ``mod(q, q_pe, kv, k_pe) -> o``.

Reference: shape-class dispatch ``kv_shared`` (attention_engine/attn_engine/attn_engine.py:235-250),
lowering core/lower/lower_decode_mla.py:25-38 and template core/template/tl_template/attn/mla_decode_tl.py.
Unlike the reference, which ignores ``score_mod`` / ``online_func`` on this path and hard-codes
softmax with scale 1/sqrt(576) (mla_decode_tl.py:30), the traced callables are honoured here, so the
user's ``score * softmax_scale`` decides the scale.  Forward only, as in the reference (:337-339).
"""
from __future__ import annotations

import ctypes as C

import torch

from .. import runtime as rt
from ..lower.cuda_lower import lower_attention, lower_combine

MLA_BN = 64  # kv rows per tile: five of the nine query blocks (80 KB) and two 72 KB KV stages fill shared memory
N_SM = 148


class MlaDecode:
    def __init__(self, score_mod, online_func, custom_fwd_inputs, H: int, D: int, DV: int, dtype):
        if (D, DV) != (576, 512):
            raise NotImplementedError(f"MLA decode is built for D = 512 + 64, DV = 512; got D={D}, DV={DV}")
        if H > 128:
            raise NotImplementedError("MLA decode handles up to 128 query heads per latent KV")
        if custom_fwd_inputs.input_tensors:
            raise NotImplementedError("custom inputs are not wired into the MLA decode kernel")
        self.dtype = dtype
        bf16 = dtype == torch.bfloat16
        self.low = lower_attention(score_mod, None, online_func, custom_fwd_inputs, D=D, DV=DV, bf16=bf16, mask_mode=0)
        tag = rt.DTYPE_BF16 if bf16 else rt.DTYPE_F16
        prelude = self.low.prelude_fwd + f"#define AE_MLA_BN {MLA_BN}\n"
        smem = 5 * 128 * 128 + 2 * 9 * MLA_BN * 128 + 256 + 1024  # 230,656 B of the 232,448 a CTA can have
        cfg = rt.KernelConfig(kind=rt.KIND_MLA_DECODE, dtype=tag, head_dim=D, head_dim_v=DV, threads=192,
                              smem_bytes=smem, stages=1, mask_mode=0)
        cfg.reserved[0] = MLA_BN
        self.src = rt.kernel_source("mla_decode.cuh", prelude=prelude)
        self.decode = rt.compile_module(self.src, "ae_mla_decode", cfg)
        comb = (rt.KERNEL_DIR / "mla_combine.cuh").read_text().replace("//%%AE_COMBINE_FUNCTOR%%", lower_combine(online_func))
        cfg2 = rt.KernelConfig(kind=rt.KIND_MLA_COMBINE, dtype=tag, head_dim=D, head_dim_v=DV, threads=128, smem_bytes=0)
        head = (rt.KERNEL_DIR / "ae_sm100.cuh").read_text().replace("#pragma once\n", "") + (rt.KERNEL_DIR / "ae_args.h").read_text()
        defs = f"#define AE_BF16 {int(bf16)}\n#define AE_NFINAL {len(self.low.final_names)}\n"
        self.combine_src = head + defs + comb
        self.combine = rt.compile_module(self.combine_src, "ae_mla_combine", cfg2)
        self.num_split = None  # None = choose per call
        self._status = None

    @staticmethod
    def pick_splits(B: int, S: int) -> int:
        """Enough CTAs (2 per batch row and split) to cover the 148 SMs once, never an empty split: a second split
        re-reads nothing but adds the combine pass, which measured slower as soon as one wave was full."""
        n_tiles = -(-S // MLA_BN)
        want = max(1, -(-N_SM // (2 * B)))
        n = min(want, 32, n_tiles)
        while n > 1 and (n - 1) * (-(-n_tiles // n)) >= n_tiles:
            n -= 1
        return n

    def __call__(self, q, q_pe, kv, k_pe):
        for name, t in (("q", q), ("q_pe", q_pe), ("kv", kv), ("k_pe", k_pe)):
            if not t.is_cuda:
                raise rt.AeError(f"{name} must be a CUDA tensor: this back end has no CPU path")
            if t.dtype != self.dtype:
                raise TypeError(f"{name} has dtype {t.dtype}, engine was built for {self.dtype}")
        B, one, H, DV = q.shape
        S = kv.shape[1]
        if one != 1 or DV != 512 or q_pe.shape != (B, 1, H, 64) or kv.shape != (B, S, 1, 512) or k_pe.shape != (B, S, 1, 64):
            raise ValueError("expected q [B,1,H,512], q_pe [B,1,H,64], kv [B,S,1,512], k_pe [B,S,1,64]")
        q, q_pe, kv, k_pe = (t.contiguous() for t in (q, q_pe, kv, k_pe))
        dev = q.device
        n_split = self.num_split or self.pick_splits(B, S)
        o = torch.empty(B, 1, H, 512, dtype=self.dtype, device=dev)
        p = rt.MlaParams()
        p.q, p.q_pe, p.kv, p.k_pe, p.o = q.data_ptr(), q_pe.data_ptr(), kv.data_ptr(), k_pe.data_ptr(), o.data_ptr()
        keep = []
        if n_split > 1:
            part = torch.empty(B, n_split, H, 512, dtype=torch.float32, device=dev)
            p.o_partial = part.data_ptr()
            keep.append(part)
            for i in range(len(self.low.final_names)):
                f = torch.empty(B, n_split, H, dtype=torch.float32, device=dev)
                p.rowscale_partial[i] = f.data_ptr()
                keep.append(f)
        p.B, p.H, p.S, p.n_split = B, H, S, n_split
        if self._status is None or self._status.device != dev:
            self._status = torch.zeros(1, dtype=torch.int32, device=dev)
        p.status = self._status.data_ptr()
        stream = C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
        rt.check(rt.lib().ae_launch_mla_decode(self.decode.handle, C.byref(p), stream), "ae_launch_mla_decode")
        if n_split > 1:
            rt.check(rt.lib().ae_launch_mla_combine(self.combine.handle, C.byref(p), stream), "ae_launch_mla_combine")
        self.last_num_split = n_split
        return o

    def paged(self, q, kcache, block_table, cache_seqlens, num_split=None):
        """Decode over a paged KV pool with one length per batch row; returns (o [B, 1, H, 512], lse [B, H] fp32).

        The call of the reference's CuTe kv-shared path (core/template/cute_template_kvshared/flash_mla_interface.py:73-113,
        attn_script/mla_decode_cute.py:295-303): q [B, 1, H, 576] (latent 512 + rope 64), kcache [num_pages, 64, 1, 576]
        or [num_pages, 64, 576], block_table [B, max_pages] int32 (page of each 64-key tile), cache_seqlens [B] int32.
        Every row gets the same split count over the longest row's tiles."""
        if list(self.low.final_names) != ["lse"]:
            raise NotImplementedError("the paged call returns the log-sum-exp: the online function must have the final row scale 'lse'")
        for name, t in (("q", q), ("kcache", kcache)):
            if not t.is_cuda:
                raise rt.AeError(f"{name} must be a CUDA tensor: this back end has no CPU path")
            if t.dtype != self.dtype:
                raise TypeError(f"{name} has dtype {t.dtype}, engine was built for {self.dtype}")
        B, one, H, D = q.shape
        if one != 1 or D != 576 or H > 128:
            raise ValueError("expected q [B, 1, H <= 128, 576]")
        if kcache.dim() == 4:
            if kcache.shape[2] != 1:
                raise ValueError("expected kcache [num_pages, 64, 1, 576]")
            kcache = kcache[:, :, 0]
        if kcache.shape[1:] != (64, 576) or not kcache.is_contiguous():
            raise ValueError("expected a contiguous kcache of 64-key pages, [num_pages, 64, (1,) 576]")
        dev = q.device
        block_table = block_table.to(device=dev, dtype=torch.int32).contiguous()
        cache_seqlens = cache_seqlens.to(device=dev, dtype=torch.int32).contiguous()
        if block_table.shape[0] != B or cache_seqlens.shape != (B,):
            raise ValueError("block_table is [B, max_pages], cache_seqlens is [B]")
        max_pages = block_table.shape[1]
        max_seqlen = int(cache_seqlens.max().item())  # host read: the grid and the split ranges depend on it
        if max_seqlen < 1 or int(cache_seqlens.min().item()) < 1 or max_seqlen > max_pages * 64:
            raise ValueError("cache_seqlens must lie in [1, max_pages * 64]")
        q_nope = q[:, 0, :, :512].contiguous()
        q_pe = q[:, 0, :, 512:].contiguous()
        n_split = num_split or self.num_split or self.pick_splits(B, max_seqlen)
        o = torch.empty(B, 1, H, 512, dtype=self.dtype, device=dev)
        fr = torch.empty(B, n_split, H, dtype=torch.float32, device=dev)
        p = rt.MlaPagedParams()
        p.q, p.q_pe, p.kcache, p.o = q_nope.data_ptr(), q_pe.data_ptr(), kcache.data_ptr(), o.data_ptr()
        p.block_table, p.cache_seqlens = block_table.data_ptr(), cache_seqlens.data_ptr()
        p.rowscale_partial[0] = fr.data_ptr()
        part = None
        if n_split > 1:
            part = torch.empty(B, n_split, H, 512, dtype=torch.float32, device=dev)
            p.o_partial = part.data_ptr()
        p.B, p.H, p.num_pages, p.max_pages, p.max_seqlen, p.n_split = B, H, kcache.shape[0], max_pages, max_seqlen, n_split
        if self._status is None or self._status.device != dev:
            self._status = torch.zeros(1, dtype=torch.int32, device=dev)
        p.status = self._status.data_ptr()
        stream = C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
        rt.check(rt.lib().ae_launch_mla_decode_paged(self.decode.handle, C.byref(p), stream), "ae_launch_mla_decode_paged")
        if n_split > 1:
            pc = rt.MlaParams()
            pc.o, pc.o_partial = o.data_ptr(), part.data_ptr()
            pc.rowscale_partial[0] = fr.data_ptr()
            pc.B, pc.H, pc.S, pc.n_split = B, H, max_seqlen, n_split
            rt.check(rt.lib().ae_launch_mla_combine(self.combine.handle, C.byref(pc), stream), "ae_launch_mla_combine")
        self.last_num_split = n_split
        return o, torch.logsumexp(fr, dim=1)
