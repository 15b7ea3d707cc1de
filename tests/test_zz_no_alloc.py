"""The attention backward entry point that takes its scratch from the library instead of the caller.

Who needs it: a program that drives the C ABI directly with nothing but the input and output buffers it
was handed (no tensor library to ask for memory), or a serving runtime whose device-memory plan is frozen
and where cudaMalloc is off limits because it stalls the whole device.  The regular backward wants a
[B, Hq, Sq] fp32 `delta` buffer from such a caller; `ae_launch_attn_bwd_static_scratch` keeps it in a fixed
device array inside libae_b200.so.

Checked here, through the C ABI: its dQ / dK / dV equal those of the regular three-launch backward bit for
bit (same kernels, same inputs, only the scratch address differs), on two calls in a row with different
data, so that contents left behind by the first call cannot leak into the second; and a shape beyond the
array's size is refused with a message instead of being launched.  Collected last on purpose.
"""
import ctypes as C

import pytest
import torch

from attentionengine_b200 import runtime as rt
from attentionengine_b200.attn_engine import attn_bwd as ab

import helpers

pytestmark = pytest.mark.gpu


def _params(eng, q, k, v, o, d_o, finals, dq, dk, dv, delta):
    p = rt.AttnBwdParams()
    p.q, p.k, p.v, p.o, p.d_o = q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), d_o.data_ptr()
    p.dq, p.dk, p.dv = dq.data_ptr(), dk.data_ptr(), dv.data_ptr()
    s3 = ab._s3
    p.q_stride, p.k_stride, p.v_stride, p.o_stride, p.do_stride = s3(q), s3(k), s3(v), s3(o), s3(d_o)
    p.dq_stride, p.dk_stride, p.dv_stride = s3(dq), s3(dk), s3(dv)
    for i, f in enumerate(finals):
        p.final_rowscales[i] = f.data_ptr()
    p.delta = delta.data_ptr() if delta is not None else None
    B, S, Hq, _ = q.shape
    p.B, p.Hq, p.Hkv, p.Sq, p.Skv = B, Hq, k.shape[2], S, k.shape[1]
    p.status = eng._get_status(q.device).data_ptr()
    return p


@pytest.mark.parametrize("S", [384, 200])
def test_static_scratch_backward_matches_regular_backward_twice(S):
    """S = 200 is ragged: the last tile's rows past the end read clamped delta words of the shared array."""
    B, Hq, Hkv, D = 2, 4, 2, 128
    eng = helpers.softmax_engine(B, Hq, Hkv, S, D, D, torch.float16, True)
    kern = eng.kernels.bwd
    L = rt.lib()
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    for call, seed in enumerate((101, 202)):
        q, k, v, d_o = helpers.seeded_qkv(B, Hq, Hkv, S, D, D, torch.float16, seed=seed, device="cuda")
        o, finals = eng._launch_fwd(q, k, v, ())
        # regular path: the caller provides delta
        ref = [torch.empty_like(t) for t in (q, k, v)]
        delta = torch.empty(B, Hq, S, dtype=torch.float32, device="cuda")
        p = _params(eng, q, k, v, o, d_o, finals, *ref, delta)
        rt.check(L.ae_launch_attn_bwd_prep(kern.prep.handle, C.byref(p), stream), "prep")
        rt.check(L.ae_launch_attn_bwd_dq(kern.dq.handle, C.byref(p), stream), "dq")
        rt.check(L.ae_launch_attn_bwd_dkv(kern.dkv.handle, C.byref(p), stream), "dkv")
        # new path: no delta, nothing allocated between here and the launch
        got = [torch.full_like(t, float("nan")) for t in (q, k, v)]
        p2 = _params(eng, q, k, v, o, d_o, finals, *got, None)
        rt.check(L.ae_launch_attn_bwd_static_scratch(kern.prep.handle, kern.dq.handle, kern.dkv.handle, C.byref(p2),
                                                     stream), "static scratch backward")
        torch.cuda.synchronize()
        eng.check_status()
        for name, a, b in zip(("dq", "dk", "dv"), got, ref):
            assert torch.equal(a, b), f"call {call}: {name} differs from the regular backward"
        assert not torch.isnan(got[0]).any()


def test_static_scratch_refuses_oversize():
    eng = helpers.softmax_engine(1, 4, 2, 256, 64, 64, torch.float16, True)
    kern = eng.kernels.bwd
    p = rt.AttnBwdParams()
    p.B, p.Hq, p.Hkv, p.Sq, p.Skv = 64, 64, 64, 4096, 4096   # 16 Mi rows > 8 Mi
    rc = rt.lib().ae_launch_attn_bwd_static_scratch(kern.prep.handle, kern.dq.handle, kern.dkv.handle, C.byref(p), None)
    assert rc == 1
    msg = rt.lib().ae_last_error().decode()
    assert str(rt.STATIC_SCRATCH_MAX_ROWS) in msg and "exceeds" in msg
    p.B = 0
    rc = rt.lib().ae_launch_attn_bwd_static_scratch(kern.prep.handle, kern.dq.handle, kern.dkv.handle, C.byref(p), None)
    assert rc == 1 and "positive" in rt.lib().ae_last_error().decode()
