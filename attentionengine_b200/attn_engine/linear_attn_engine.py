"""LinearAttentionEngine: operator API of the chunked linear-attention / SSD scan.

Same constructor and call as the reference (attention_engine/attn_engine/linear_attn_engine.py:10-52):
``LinearAttentionEngine(qkv_meta, q_mod, k_mod, v_mod, decay_mod, custom_io, ...)`` and
``mod(q, k, v, decay, *custom)`` with [B, H, T, D] tensors, decay [B, H, T] fp32, returning O [B, H, T, DV].

One keyword beyond the reference: ``o_mod(o, v, custom_io)``, applied to the scan output with the un-modded v at
hand.  The benchmark's Mamba2 configuration has a skip connection ``o + D_skip[h] * x`` that the reference's operator
cannot express (its harness passes D=None, benchmark/bench_utils.py:304-308); ``o_mod = lambda o, v, io: o + v *
io.input_tensors["D"]`` with ``"D": (1, "heads")`` states it, and that form runs as one streaming kernel each way.

As in the reference (core/template/tl_template/linear/linear_tl.py:1136-1144) the mods are traced once and
run as eager PyTorch on the inputs; the scan itself (chunk cumulative sum, state recurrence, intra-chunk
products) is one sm_100a kernel (csrc/kernels/linear_fwd.cuh); its backward is a state-recompute pass
(linear_states.cuh) and a reverse pass (linear_bwd.cuh) on value blocks of 64; heads larger than one block of
128 key dims x 64 / 128 value dims are decomposed into blocks (``_scan``).
"""
from __future__ import annotations

import ctypes as C
import os

import torch

from .. import runtime as rt
from ..core.transform.core import CustomIO, SymbolScalar
from ..core.transform.graph import Var
from ..lower.torch_eval import evaluate

LIN_FWD_NWG = 2  # row warpgroups of the scan's forward kernel (measured: cfg4 3.72 against 4.14 ms)
LIN_BWD_PARTS = 2  # batch ranges of the reverse pass on streams of their own when a head sum follows (1: one launch;
                   # measured at cfg4: 3.31 ms with 1, 3.10 with 2, 3.11 with 4)
LIN_DECAY_SCALE = 1  # a decay mod `decay * c[heads]` inside the scan kernels of the Mamba2 block (0: eager PyTorch)
LIN_BWD_MODS = 1  # the row scale of v and the skip term inside the reverse pass (0: a streaming kernel after it)
LIN_BWD_NWG = 2  # row warpgroups of the reverse pass of the scan (measured: 4.05 against 4.33 ms at cfg4)

_DIM_POS = {"batch": 0, "heads": 1, "seq_len": 2}


def _align(t: torch.Tensor, names: tuple, ndim: int) -> torch.Tensor:
    """View a custom tensor so that its named dims line up with [batch, heads, seq_len, (feature)]."""
    shape = [1] * ndim
    for size, name in zip(t.shape, names):
        name = str(name)
        if name in _DIM_POS:
            shape[_DIM_POS[name]] = size
        elif size != 1:
            raise ValueError(f"custom input dim {name!r} of size {size} cannot be broadcast")
    return t.reshape(shape)


class _Scan(torch.autograd.Function):
    """The scan on the mod-ed tensors; gradients flow on into the eager mods through torch autograd
    (the reference chains the traced mod derivatives by hand, linear_tl.py:1203-1214)."""

    @staticmethod
    def forward(ctx, eng, q, k, v, a):
        q, k, v, a = q.contiguous(), k.contiguous(), v.contiguous(), a.float().contiguous()
        ctx.eng = eng
        # with a backward to come (value blocks of 64), the forward also writes the chunk start-states it has at hand
        hs = eng._new_states(v) if (any(ctx.needs_input_grad) and v.shape[3] == 64) else None
        o = eng._launch(q, k, v, a, h_out=hs)
        ctx.has_states = hs is not None
        ctx.save_for_backward(q, k, v, a, *([hs] if hs is not None else []))
        return o

    @staticmethod
    def backward(ctx, d_o):
        q, k, v, a = ctx.saved_tensors[:4]
        hs = ctx.saved_tensors[4] if ctx.has_states else None
        dq, dk, dv, da = ctx.eng._launch_bwd(q, k, v, a, d_o.contiguous(), hs=hs)
        return None, dq, dk, dv, da


class _RowScale(torch.autograd.Function):
    """y = x * s[..., None] for x [B, H, T, D] 16-bit and s [B, H, T]: the `v * dt` shape of mod, as one streaming
    kernel each way (csrc/kernels/rowscale.cuh) instead of PyTorch's broadcast multiply and 64-wide reduction."""

    @staticmethod
    def forward(ctx, eng, x, s):
        x, s = x.contiguous(), s.contiguous()
        ctx.eng = eng
        ctx.save_for_backward(x, s)
        y = torch.empty_like(x)
        eng._rowscale("fwd", x, s, y=y)
        return y

    @staticmethod
    def backward(ctx, g):
        x, s = ctx.saved_tensors
        gx, gs = torch.empty_like(x), torch.empty_like(s)
        ctx.eng._rowscale("bwd", x, s, g=g.contiguous(), gx=gx, gs=gs)
        return None, gx, gs


class _Skip(torch.autograd.Function):
    """y = o + x * d[head] for o, x [B, H, T, D] 16-bit and d [1, H] or [H] fp32 (csrc/kernels/rowscale.cuh)."""

    @staticmethod
    def forward(ctx, eng, o, x, d):
        o, x = o.contiguous(), x.contiguous()
        df = d.detach().float().reshape(-1).contiguous()
        ctx.eng, ctx.d_shape, ctx.d_dtype = eng, d.shape, d.dtype
        ctx.save_for_backward(x, df)
        y = torch.empty_like(o)
        eng._rowscale("skip_fwd", x, df, g=o, y=y, rows_per_head=x.shape[2], n_heads=x.shape[1])
        return y

    @staticmethod
    def backward(ctx, g):
        x, df = ctx.saved_tensors
        g = g.contiguous()
        gx = torch.empty_like(x)
        rows = torch.empty(x.shape[:3], dtype=torch.float32, device=x.device)
        ctx.eng._rowscale("skip_bwd", x, df, g=g, gx=gx, gs=rows, rows_per_head=x.shape[2], n_heads=x.shape[1])
        gd = rows.sum(dim=(0, 2)).reshape(ctx.d_shape).to(ctx.d_dtype)
        return None, g, gx, gd


class _ScaleScanSkip(torch.autograd.Function):
    """y = scan(q, k, x * s[..., None], a) + x * d[head] as one node.  Forward: one launch of the scan kernel built
    with the two mods inside.  Backward: the two gradients that meet at x (through the scaled rows and through the
    skip) and the row sums for s and d come out of one pass over x (ae_vskip_bwd) instead of two kernels and an add."""

    @staticmethod
    def forward(ctx, eng, q, k, x, a, s, d, asc=None):
        q, k, x, a, s = q.contiguous(), k.contiguous(), x.contiguous(), a.float().contiguous(), s.contiguous()
        df = d.detach().float().reshape(-1).contiguous()
        # a decay mod of the form decay * custom[heads]: a is the decay as passed, the kernels scale it
        af = None if asc is None else asc.detach().float().reshape(-1).contiguous()
        ctx.asc_meta = None if asc is None else (asc.shape, asc.dtype)
        # one kernel: the scan scales its V rows by s, adds x * d[head] to its output rows and writes the scaled v
        # for the backward (only when a gradient is wanted)
        need_v = any(ctx.needs_input_grad)
        v = torch.empty_like(x) if need_v else None
        hs = eng._new_states(x) if need_v else None  # the chunk start-states, for the reverse pass
        y = eng._launch(q, k, x, a, vscale=s, dskip=df, v_out=v, h_out=hs, ascale=af)
        ctx.eng, ctx.d_shape, ctx.d_dtype = eng, d.shape, d.dtype
        if not need_v:
            return y
        ctx.save_for_backward(q, k, v, a, x, s, df, hs, af)
        return y

    @staticmethod
    def backward(ctx, g):
        q, k, v, a, x, s, df, hs, af = ctx.saved_tensors
        g = g.contiguous()
        gasc = None
        if int(os.environ.get("AE_B200_LIN_BWD_MODS", LIN_BWD_MODS)):
            # the reverse pass built with the two mods inside: no pass over x of its own
            res = ctx.eng._launch_bwd(q, k, v, a, g, hs=hs, mods=(x, s, df), ascale=af)
            dq, dk, gx, da, gs, rows = res[:6]
            if af is not None:
                gasc = res[6].sum(dim=0).reshape(ctx.asc_meta[0]).to(ctx.asc_meta[1])
            return None, dq, dk, gx, da, gs, rows.sum(dim=0).reshape(ctx.d_shape).to(ctx.d_dtype), gasc
        res = ctx.eng._launch_bwd(q, k, v, a, g, hs=hs, ascale=af)
        dq, dk, dv, da = res[:4]
        if af is not None:
            gasc = res[4].sum(dim=0).reshape(ctx.asc_meta[0]).to(ctx.asc_meta[1])
        gx, gs = torch.empty_like(x), torch.empty_like(s)
        rows = torch.empty(x.shape[:3], dtype=torch.float32, device=x.device)
        ctx.eng._rowscale("vskip_bwd", x, s, g=g, g2=dv, d=df, gx=gx, gs=gs, gs2=rows, rows_per_head=x.shape[2],
                          n_heads=x.shape[1])
        gd = rows.sum(dim=(0, 2)).reshape(ctx.d_shape).to(ctx.d_dtype)
        return None, dq, dk, gx, da, gs, gd, gasc


class LinearAttentionEngine:
    def __init__(self, qkv_meta, q_mod=None, k_mod=None, v_mod=None, decay_mod=None, custom_io=None, tune=False,
                 tune_filename="tune_result", tune_bwd=False, o_mod=None):
        qm, km, vm = qkv_meta
        self.dtype = qm.dtype
        if self.dtype not in (torch.float16, torch.bfloat16):
            raise NotImplementedError("fp16 / bf16 only")
        self.B, self.HQ, self.T, self.DK = qm.shape
        self.HK = km.shape[1]
        self.H, self.DV = vm.shape[1], vm.shape[3]
        if self.DK % 128 or self.DK > 512 or self.DV % 64 or self.DV > 1024:
            raise NotImplementedError("linear attention takes DK in (128, 256, 384, 512) and DV a multiple of 64 up to "
                                      f"1024; got {self.DK}, {self.DV}")
        self.custom_io = custom_io if custom_io is not None else CustomIO()
        self.mods = {"q": q_mod, "k": k_mod, "v": v_mod, "decay": decay_mod}
        self._traced = {}
        for name, fn in self.mods.items():
            if fn is None:
                continue
            leaf = SymbolScalar(name, Var(name), shape_idx=["batch", "heads", "seq_len"] + ([] if name == "decay" else ["dim"]))
            self._traced[name] = (leaf, fn(leaf, self.custom_io))
        self.o_mod = o_mod
        if o_mod is not None:
            dims = ["batch", "heads", "seq_len", "dim"]
            self._o_leaves = (SymbolScalar("o", Var("o"), shape_idx=dims), SymbolScalar("v", Var("v"), shape_idx=dims))
            self._o_traced = o_mod(*self._o_leaves, self.custom_io)
        self._bf16 = self.dtype == torch.bfloat16
        self._status = None
        self._bwd = None
        self._bwd_mods = None
        self._streams = {}
        self._fwd_by_dv = {}
        self._rowscale_mods = {}
        # The kernels work on blocks of 128 key dims x 64 or 128 value dims.  Larger heads (simple_gla / retention_linear
        # of the reference use D = 256, DV = 512) are sums over key blocks of independent value blocks, see _scan().
        self._dv_block = self.DV if self.DV in (64, 128) else (128 if self.DV % 128 == 0 else 64)
        self.fwd, self.tl_code = self._fwd_kernel(self._dv_block)

    def _fwd_kernel(self, dv: int, mods: bool = False):
        """The forward kernel for value blocks of ``dv``; ``mods``: the build with the row scale of v and the skip
        connection inside."""
        key = (dv, mods)
        if key not in self._fwd_by_dv:
            stages = 2 if dv == 64 else 1
            nwg = int(os.environ.get("AE_B200_LIN_FWD_NWG", LIN_FWD_NWG))
            prelude = (f"#define AE_BF16 {int(self._bf16)}\n#define AE_LIN_DV {dv}\n#define AE_LIN_STAGES {stages}\n"
                       f"#define AE_LIN_MODS {int(mods)}\n#define AE_LIN_NWG {nwg}\n")
            # K/V ring, rescaled V, state copy, cumulative decays, barriers, output staging tile, alignment slack
            smem = stages * (2 * 128 * 128 * 2 + 128 * dv * 2) + 3 * 128 * dv * 2 + 1024 + 2048 + 1024
            cfg = rt.KernelConfig(kind=rt.KIND_LINEAR_FWD, dtype=rt.DTYPE_BF16 if self._bf16 else rt.DTYPE_F16,
                                  head_dim=128, head_dim_v=dv, threads=nwg * 128 + 64, smem_bytes=smem, stages=stages,
                                  mask_mode=0)
            cfg.reserved[0] = int(mods)
            src = rt.kernel_source("linear_fwd.cuh", prelude=prelude)
            self._fwd_by_dv[key] = (rt.compile_module(src, "ae_linear_fwd", cfg), src)
        return self._fwd_by_dv[key]

    def _bwd_kernels(self, mods: bool = False):
        """(state recompute, reverse pass).  ``mods``: the reverse pass built with the block's row scale of v and skip
        term inside (it then writes the gradient of x where dv went, the row sums for the scale and the per-head sum
        for the skip weight)."""
        if mods:
            if self._bwd_mods is None:
                self._bwd_mods = (self._bwd_kernels()[0], self._build_bwd(True))
            return self._bwd_mods
        if self._bwd is None:
            DV = 64  # the backward kernels are built for value blocks of 64
            tag = rt.DTYPE_BF16 if self._bf16 else rt.DTYPE_F16
            pre = f"#define AE_BF16 {int(self._bf16)}\n#define AE_LIN_DV {DV}\n#define AE_LIN_STAGES 2\n"
            smem_s = 2 * (128 * 128 * 2 + 128 * DV * 2) + 1024 + 256 + 1024  # two CTAs per SM
            cfg = rt.KernelConfig(kind=rt.KIND_LINEAR_STATES, dtype=tag, head_dim=128, head_dim_v=DV, threads=192,
                                  smem_bytes=smem_s, stages=2, mask_mode=0)
            states = rt.compile_module(rt.kernel_source("linear_states.cuh", prelude=pre), "ae_linear_states", cfg)
            self._bwd = (states, self._build_bwd(False))
        return self._bwd

    def _build_bwd(self, mods: bool):
        DV = 64
        tag = rt.DTYPE_BF16 if self._bf16 else rt.DTYPE_F16
        # row warpgroups of the reverse pass (2: the second one takes half of the P / dS pass and of the output phase)
        nwg = int(os.environ.get("AE_B200_LIN_BWD_NWG", LIN_BWD_NWG))
        pre = (f"#define AE_BF16 {int(self._bf16)}\n#define AE_LIN_DV {DV}\n#define AE_LIN_STAGES 2\n"
               f"#define AE_LB_NWG {nwg}\n#define AE_LB_MODS {int(mods)}\n")
        smem_b = (2 * 128 * 128 * 2 + 2 * 128 * DV * 2 + 128 * DV * 2 + 2 * 128 * 128 * 2
                  + 128 * DV * 2 + 128 * DV * 2 + int(mods) * 128 * DV * 2 + 1024 + 256 + 512 + 1024)
        cfg = rt.KernelConfig(kind=rt.KIND_LINEAR_BWD, dtype=tag, head_dim=128, head_dim_v=DV,
                              threads=nwg * 128 + 64, smem_bytes=smem_b, stages=1, mask_mode=0)
        cfg.reserved[0] = int(mods)
        return rt.compile_module(rt.kernel_source("linear_bwd.cuh", prelude=pre), "ae_linear_bwd", cfg)

    def _new_states(self, v):
        """Storage for the chunk start-states of a scan over v [B, H, T, DV]: [B, H, ceil(T / 128), 128, DV]."""
        B, H, T, DV = v.shape
        return torch.empty(B, H, -(-T // 128), 128, DV, dtype=self.dtype, device=v.device)

    def _launch_bwd(self, q, k, v, a, d_o, hs=None, mods=None, ascale=None):
        """State recompute (unless the forward saved the states in ``hs``) and the reverse pass -> dq, dk, dv, da.
        ``mods`` = (x, s, d) with v = x * s[..., None] and the output's skip term x * d[head]: the reverse pass built
        with the two inside returns dq, dk, gx, da, gs, gd (gd per (batch, head), fp32).  ``ascale`` [H] fp32: the
        forward ran on a * ascale[h]; da is then the gradient of ``a`` as passed and one more result, [B, H] fp32, holds
        the per-(batch, head) sums for the gradient of ascale."""
        if v.shape[3] != 64:
            raise NotImplementedError("backward of the linear-attention scan runs on value blocks of 64")
        states, bwd = self._bwd_kernels(mods is not None)
        B, HQ, T, DK = q.shape
        HK = k.shape[1]
        H, DV = v.shape[1], v.shape[3]
        dev = q.device
        recompute = hs is None
        if recompute:
            hs = self._new_states(v)
        dq_h = torch.empty(B, H, T, DK, dtype=self.dtype, device=dev)
        dk_h = torch.empty(B, H, T, DK, dtype=self.dtype, device=dev)
        dv = torch.empty(B, H, T, DV, dtype=self.dtype, device=dev)
        da = torch.empty(B, H, T, dtype=torch.float32, device=dev)
        p = rt.LinearBwdParams()
        p.q, p.k, p.v, p.a, p.d_o = q.data_ptr(), k.data_ptr(), v.data_ptr(), a.data_ptr(), d_o.data_ptr()
        p.h_states, p.dq, p.dk, p.dv, p.da = hs.data_ptr(), dq_h.data_ptr(), dk_h.data_ptr(), dv.data_ptr(), da.data_ptr()
        p.B, p.H, p.HQ, p.HK, p.T = B, H, HQ, HK, T
        if self._status is None or self._status.device != dev:
            self._status = torch.zeros(1, dtype=torch.int32, device=dev)
        p.status = self._status.data_ptr()
        if mods is not None:
            x, s, d = mods
            gs = torch.empty_like(s)
            gd = torch.empty(B, H, dtype=torch.float32, device=dev)
            p.x, p.vscale, p.dskip, p.gs, p.gd = x.data_ptr(), s.data_ptr(), d.data_ptr(), gs.data_ptr(), gd.data_ptr()
            p.vscale_16bit = int(s.dtype != torch.float32)
        gasc = None
        if ascale is not None:
            gasc = torch.empty(B, H, dtype=torch.float32, device=dev)
            p.ascale, p.gasc = ascale.data_ptr(), gasc.data_ptr()
        dq = dq_h if HQ == H else torch.empty(B, HQ, T, DK, dtype=self.dtype, device=dev)
        dk = dk_h if HK == H else torch.empty(B, HK, T, DK, dtype=self.dtype, device=dev)
        # Batch ranges on streams of their own when a head sum follows: the (batch, head) CTAs of all ranges fill the
        # SMs in launch order as before, and the head sums of a range that is complete run under the later ranges'
        # chunk walks (a latency-bound kernel next to an HBM-bound one) instead of after the whole pass.
        n_parts = self._bwd_batch_parts(B, H, dev) if (HQ != H or HK != H) else 1
        main = torch.cuda.current_stream(dev)
        if n_parts > 1:
            side, start, done = self._side_streams(dev, n_parts - 1)
            start.record(main)
        nb = B // n_parts
        for i in range(n_parts):
            st = main if i == 0 else side[i - 1]
            if i:
                st.wait_event(start)
            sl = slice(i * nb, (i + 1) * nb)
            p.q, p.k, p.v, p.a, p.d_o = (t[sl].data_ptr() for t in (q, k, v, a, d_o))
            p.h_states, p.dq, p.dk, p.dv, p.da = (t[sl].data_ptr() for t in (hs, dq_h, dk_h, dv, da))
            if mods is not None:
                p.x, p.vscale, p.gs, p.gd = x[sl].data_ptr(), s[sl].data_ptr(), gs[sl].data_ptr(), gd[sl].data_ptr()
            if ascale is not None:
                p.gasc = gasc[sl].data_ptr()
            p.B = nb
            stream = C.c_void_p(st.cuda_stream)
            if recompute:
                rt.check(rt.lib().ae_launch_linear_states(states.handle, C.byref(p), stream), "ae_launch_linear_states")
            rt.check(rt.lib().ae_launch_linear_bwd(bwd.handle, C.byref(p), stream), "ae_launch_linear_bwd")
            if HQ != H:
                self._head_sum(dq_h[sl], HQ, out=dq[sl], stream=st)
            if HK != H:
                self._head_sum(dk_h[sl], HK, out=dk[sl], stream=st)
            if i:
                done[i - 1].record(st)
                main.wait_event(done[i - 1])
        out = (dq, dk, dv, da) + ((gs, gd) if mods is not None else ())
        return out + ((gasc,) if ascale is not None else ())

    def _bwd_batch_parts(self, B, H, dev):
        """Into how many batch ranges the reverse pass is split (see _launch_bwd): 4 or 2 when the batch divides and a
        range still has one CTA per SM, else 1."""
        from .attn_bwd import batch_ranges
        want = int(os.environ.get("AE_B200_LIN_BWD_PARTS", LIN_BWD_PARTS))
        return batch_ranges(B, H, torch.cuda.get_device_properties(dev).multi_processor_count, want)

    def _side_streams(self, dev, n):
        """n side streams of this engine on ``dev`` with an event to start them after the caller's stream and one each
        to join them back."""
        key = (dev.index if dev.index is not None else torch.cuda.current_device(), n)
        if key not in self._streams:
            self._streams[key] = ([torch.cuda.Stream(device=dev) for _ in range(n)], torch.cuda.Event(),
                                  [torch.cuda.Event() for _ in range(n)])
        return self._streams[key]

    def _head_sum(self, x, n_out, out=None, stream=None):
        """[B, H, T, D] -> [B, n_out, T, D]: sum over the H / n_out heads of each group, fp32 accumulation, one pass."""
        B, H, T, D = x.shape
        y = out if out is not None else torch.empty(B, n_out, T, D, dtype=x.dtype, device=x.device)
        key = ("head_sum", D, False)
        if key not in self._rowscale_mods:
            pre = f"#define AE_BF16 {int(self._bf16)}\n#define AE_RS_D {D}\n#define AE_RS_S16 0\n"
            cfg = rt.KernelConfig(kind=rt.KIND_ROWSCALE, dtype=rt.DTYPE_BF16 if self._bf16 else rt.DTYPE_F16, head_dim=D,
                                  head_dim_v=D, threads=256, smem_bytes=0, stages=1, mask_mode=0)
            self._rowscale_mods[key] = rt.compile_module(rt.kernel_source("rowscale.cuh", prelude=pre), "ae_head_sum", cfg)
        p = rt.RowScaleParams()
        p.x, p.y, p.n_rows, p.rows_per_head, p.n_heads = x.data_ptr(), y.data_ptr(), B * n_out * T, T, H // n_out
        stream = C.c_void_p((stream if stream is not None else torch.cuda.current_stream(x.device)).cuda_stream)
        rt.check(rt.lib().ae_launch_rowscale(self._rowscale_mods[key].handle, C.byref(p), stream), "ae_launch_rowscale")
        return y

    def _rowscale(self, which, x, s, rows_per_head=0, n_heads=0, **out):
        """Launch one of the streaming kernels of rowscale.cuh: "fwd" / "bwd" (one scale per row) or "skip_fwd" /
        "skip_bwd" (one fp32 scale per head)."""
        D = x.shape[-1]
        skip = which.startswith("skip")  # s is the per-head fp32 weight vector
        s16 = s.dtype == self.dtype and not skip
        key = (which, D, s16)
        if key not in self._rowscale_mods:
            pre = f"#define AE_BF16 {int(self._bf16)}\n#define AE_RS_D {D}\n#define AE_RS_S16 {int(s16)}\n"
            cfg = rt.KernelConfig(kind=rt.KIND_ROWSCALE, dtype=rt.DTYPE_BF16 if self._bf16 else rt.DTYPE_F16, head_dim=D,
                                  head_dim_v=D, threads=256, smem_bytes=0, stages=1, mask_mode=0)
            cfg.reserved[0] = int(s16)
            name = f"ae_{which}" if (skip or which == "vskip_bwd") else f"ae_rowscale_{which}"
            self._rowscale_mods[key] = rt.compile_module(rt.kernel_source("rowscale.cuh", prelude=pre), name, cfg)
        p = rt.RowScaleParams()
        p.x, p.s, p.n_rows = x.data_ptr(), s.data_ptr(), x.numel() // D
        p.rows_per_head, p.n_heads = rows_per_head, n_heads
        for k_, t in out.items():
            setattr(p, k_, t.data_ptr())
        stream = C.c_void_p(torch.cuda.current_stream(x.device).cuda_stream)
        rt.check(rt.lib().ae_launch_rowscale(self._rowscale_mods[key].handle, C.byref(p), stream), "ae_launch_rowscale")

    def _rowscale_operand(self, name, x, custom):
        """The custom tensor s when the traced mod is exactly ``x * s`` with s indexed by (batch, heads, seq_len) and of
        x's leading shape in fp32 or x's dtype; None otherwise (the mod then runs as eager PyTorch)."""
        leaf, out = self._traced[name]
        if name == "decay" or out.code.type != "Mul" or len(out.prev) != 2 or x.shape[-1] not in (64, 128, 256):
            return None
        other = out.prev[1] if out.prev[0] is leaf else out.prev[0] if out.prev[1] is leaf else None
        if other is None:
            return None
        for (cname, sym), t in zip(self.custom_io.input_tensors.items(), custom):
            if sym is other:
                names = tuple(str(n) for n in sym.shape_idx)
                if names == ("batch", "heads", "seq_len") and tuple(t.shape) == tuple(x.shape[:3]) and \
                        t.dtype in (torch.float32, self.dtype) and x.dtype == self.dtype:
                    return t
        return None

    def _apply_mod(self, name, x, custom):
        if name not in self._traced:
            return x
        s = self._rowscale_operand(name, x, custom)
        if s is not None:
            return _RowScale.apply(self, x, s)
        leaf, out = self._traced[name]
        env = {id(leaf): x.float() if name == "decay" else x}
        for (cname, sym), t in zip(self.custom_io.input_tensors.items(), custom):
            env[id(sym)] = _align(t, tuple(sym.shape_idx), x.dim())
        y = evaluate(out, env)
        return y if name == "decay" else y.to(x.dtype)

    def _decay_scale_operand(self, decay, custom):
        """The custom tensor c when the traced decay_mod is exactly ``decay * c`` with c indexed by heads only (fp32,
        [1, H] or [H]); None otherwise (the mod then runs as eager PyTorch)."""
        if "decay" not in self._traced or decay.dtype != torch.float32:
            return None
        leaf, out = self._traced["decay"]
        if out.code.type != "Mul" or len(out.prev) != 2:
            return None
        other = out.prev[1] if out.prev[0] is leaf else out.prev[0] if out.prev[1] is leaf else None
        if other is None:
            return None
        for (cname, sym), t in zip(self.custom_io.input_tensors.items(), custom):
            if sym is other:
                names = tuple(str(n) for n in sym.shape_idx if str(n) != "1")
                if names == ("heads",) and t.numel() == self.H and t.dtype == torch.float32:
                    return t
        return None

    def _skip_operand(self, custom):
        """The custom tensor d when the traced o_mod is exactly ``o + v * d`` with d indexed by heads only (fp32,
        [1, H] or [H]); None otherwise (the mod then runs as eager PyTorch)."""
        o_leaf, v_leaf = self._o_leaves
        out = self._o_traced
        if out.code.type != "Add" or len(out.prev) != 2:
            return None
        mul = out.prev[1] if out.prev[0] is o_leaf else out.prev[0] if out.prev[1] is o_leaf else None
        if mul is None or mul.code.type != "Mul" or len(mul.prev) != 2:
            return None
        other = mul.prev[1] if mul.prev[0] is v_leaf else mul.prev[0] if mul.prev[1] is v_leaf else None
        for (cname, sym), t in zip(self.custom_io.input_tensors.items(), custom):
            if sym is other:
                names = tuple(str(n) for n in sym.shape_idx if str(n) != "1")
                if names == ("heads",) and t.numel() == self.H and t.dtype == torch.float32 and self.DV in (64, 128, 256):
                    return t
        return None

    def _apply_o_mod(self, o, v, custom):
        d = self._skip_operand(custom)
        if d is not None and v.dtype == self.dtype:
            return _Skip.apply(self, o, v, d)
        env = {id(self._o_leaves[0]): o, id(self._o_leaves[1]): v}
        for (cname, sym), t in zip(self.custom_io.input_tensors.items(), custom):
            env[id(sym)] = _align(t, tuple(sym.shape_idx), o.dim())
        return evaluate(self._o_traced, env).to(o.dtype)

    def _launch(self, q, k, v, a, vscale=None, dskip=None, v_out=None, h_out=None, ascale=None):
        """The scan kernel.  With ``vscale`` [B, H, T] / ``dskip`` [H] fp32 the build with the mods inside runs: scan of
        v * vscale plus v * dskip[h]; ``v_out`` receives the scaled v."""
        B, HQ, T, DK = q.shape
        H, DV = v.shape[1], v.shape[3]
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        a = a.float().contiguous()
        o = torch.empty(B, H, T, DV, dtype=self.dtype, device=q.device)
        p = rt.LinearParams()
        p.q, p.k, p.v, p.a, p.o = q.data_ptr(), k.data_ptr(), v.data_ptr(), a.data_ptr(), o.data_ptr()
        mods = vscale is not None or dskip is not None
        if mods:
            if vscale is not None:
                p.vscale, p.vscale_16bit = vscale.data_ptr(), int(vscale.dtype != torch.float32)
            if dskip is not None:
                p.dskip = dskip.data_ptr()
            if v_out is not None:
                p.v_out = v_out.data_ptr()
        if h_out is not None:
            p.h_states_out = h_out.data_ptr()
        if ascale is not None:  # [H] fp32: the scan runs on a * ascale[h]
            p.ascale = ascale.data_ptr()
        p.B, p.H, p.HQ, p.HK, p.T = B, H, HQ, k.shape[1], T
        if self._status is None or self._status.device != q.device:
            self._status = torch.zeros(1, dtype=torch.int32, device=q.device)
        p.status = self._status.data_ptr()
        stream = C.c_void_p(torch.cuda.current_stream(q.device).cuda_stream)
        rt.check(rt.lib().ae_launch_linear_fwd(self._fwd_kernel(DV, mods)[0].handle, C.byref(p), stream),
                 "ae_launch_linear_fwd")
        return o

    def _scan(self, q, k, v, a):
        """The scan on heads of any supported size, from kernels that take 128 key dims and 64 / 128 value dims.
        Value blocks are independent problems sharing q, k and the decay (o[:, block] depends on v[:, block] only): they
        become extra heads.  Key blocks add up: S = [S_1; S_2] row-wise and o = q_1 S_1 + q_2 S_2, one launch per key
        block, summed in fp32.  Blocks of 64 value dims when gradients are wanted (the backward kernels' size)."""
        B, H, T, DV = v.shape
        DK = q.shape[3]
        want_grad = torch.is_grad_enabled() and any(t.requires_grad for t in (q, k, v, a))
        dvb = 64 if (want_grad or DV % 128) else 128
        if DK == 128 and DV == dvb:
            return _Scan.apply(self, q, k, v, a)
        n_dv = DV // dvb
        if n_dv > 1:
            v = v.view(B, H, T, n_dv, dvb).permute(0, 1, 3, 2, 4).reshape(B, H * n_dv, T, dvb)
            a = a.repeat_interleave(n_dv, dim=1)
        o = None
        for j in range(DK // 128):
            oj = _Scan.apply(self, q[..., j * 128:(j + 1) * 128], k[..., j * 128:(j + 1) * 128], v, a)
            o = oj.float() if o is None else o + oj.float()
        o = o.to(self.dtype)
        if n_dv > 1:
            o = o.view(B, H, n_dv, T, dvb).permute(0, 1, 3, 2, 4).reshape(B, H, T, DV)
        return o

    def check_status(self):
        if self._status is not None:
            code = int(self._status.item())
            if code:
                self._status.zero_()
                raise rt.AeError(f"kernel reported status 0x{code:x} (a bounded wait gave up)")

    def __call__(self, q, k, v, decay, *custom):
        for name, t in (("q", q), ("k", k), ("v", v), ("decay", decay)):
            if not t.is_cuda:
                raise rt.AeError(f"{name} must be a CUDA tensor: this back end has no CPU path")
        with torch.cuda.device(q.device):  # the C ABI launches on the current device's context
            return self._call(q, k, v, decay, *custom)

    def _call(self, q, k, v, decay, *custom):
        if q.dtype != self.dtype or k.dtype != self.dtype or v.dtype != self.dtype:
            raise TypeError(f"q/k/v must be {self.dtype}")
        if len(custom) != len(self.custom_io.input_tensors):
            raise TypeError(f"expected {len(self.custom_io.input_tensors)} custom input(s), got {len(custom)}")
        if q.shape[3] != self.DK or v.shape[3] != self.DV or v.shape[1] % q.shape[1] or v.shape[1] % k.shape[1]:
            raise ValueError("inconsistent q/k/v shapes")
        qm = self._apply_mod("q", q, custom)
        km = self._apply_mod("k", k, custom)
        if self.o_mod is not None and "v" in self._traced and self.DK == 128 and self.DV == 64 and v.dtype == self.dtype:
            # `v * s[b, h, t]` into the scan and `o + v * d[h]` after it (the Mamba2 block): one autograd node, which
            # also takes a decay mod of the form `decay * c[h]` into the kernels
            s, d = self._rowscale_operand("v", v, custom), self._skip_operand(custom)
            if s is not None and d is not None:
                c = self._decay_scale_operand(decay, custom) if LIN_DECAY_SCALE else None
                if c is not None:
                    return _ScaleScanSkip.apply(self, qm, km, v, decay, s, d, c)
                return _ScaleScanSkip.apply(self, qm, km, v, self._apply_mod("decay", decay, custom), s, d, None)
        a = self._apply_mod("decay", decay, custom)
        vm = self._apply_mod("v", v, custom)
        o = self._scan(qm, km, vm, a)
        return o if self.o_mod is None else self._apply_o_mod(o, v, custom)
