"""Parity at the benchmark's own sizes, gradients included.  The kernels run the full sequence length (and head
count) of each benchmark configuration; the CPU oracle, which needs the whole score matrix, is evaluated on
self-contained slices: one (batch, kv-group) for softmax attention (dK / dV of a kv head depend on its own query
heads only), one (batch, head) for sigmoid / relu attention, two heads of the SSD scan, two batch rows of MLA decode.
Acceptance rule: tests/parity.py."""
import math

import pytest
import torch

from oracle import attention_oracle as orc

import helpers
from parity import check

pytestmark = pytest.mark.gpu


def test_cfg2_llama_gqa_s8192_slice_forward_and_gradients():
    """Config 2 at batch 2 of 8: Hq=32, Hkv=8, S=8192, D=128, fp16, causal, dO ~ N(0,1).  64 q tiles per head, four
    query heads accumulated per kv head in the dK / dV pass.  Oracle on (batch 1, kv head 5) = query heads 20..23."""
    B, Hq, Hkv, S, D, dt = 2, 32, 8, 8192, 128, torch.float16
    q, k, v, d_o = helpers.seeded_qkv(B, Hq, Hkv, S, D, D, dt, seed=2)
    eng = helpers.softmax_engine(B, Hq, Hkv, S, D, D, dt, True)
    qd, kd, vd = (t.cuda().requires_grad_() for t in (q, k, v))
    o = eng(qd, kd, vd)
    o.backward(d_o.cuda())
    torch.cuda.synchronize()
    eng.check_status()
    b, hk = 1, 5
    hs = slice(hk * 4, hk * 4 + 4)
    ro, (rq, rk, rv) = orc.fwd_bwd(lambda a, b_, c: orc.softmax_attention(a, b_, c, True),
                                   (q[b:b + 1, :, hs], k[b:b + 1, :, hk:hk + 1], v[b:b + 1, :, hk:hk + 1]),
                                   d_o[b:b + 1, :, hs])
    check("cfg2.o", o[b:b + 1, :, hs], ro, dt)
    check("cfg2.dq", qd.grad[b:b + 1, :, hs], rq, dt)
    check("cfg2.dk", kd.grad[b:b + 1, :, hk:hk + 1], rk, dt)
    check("cfg2.dv", vd.grad[b:b + 1, :, hk:hk + 1], rv, dt)


@pytest.mark.parametrize("kind", ["sigmoid", "relu"])
def test_cfg3_sigmoid_relu_s4096_slices(kind):
    """Config 3 in full: B=4, H=32, S=4096, D=128, bf16, non-causal.  Oracle on (batch 3, head 17) and (batch 0, head 0).
    bf16 stages: o = P (rounded) V -> 2; dV = P^T dO -> 2; dQ, dK = dS (rounded) K / Q -> 2."""
    B, H, S, D, dt = 4, 32, 4096, 128, torch.bfloat16
    q, k, v, d_o = helpers.seeded_qkv(B, H, H, S, D, D, dt, seed=3)
    if kind == "sigmoid":
        eng = helpers.sigmoid_engine(B, H, S, D, dt, False)
        custom = (torch.tensor([-math.log(S)], dtype=torch.float32).cuda(),)
        fn = lambda a, b_, c: orc.sigmoid_attention(a, b_, c, bias=-math.log(S))  # noqa: E731
    else:
        eng = helpers.relu_engine(B, H, S, D, dt, False, post_scale=1.0 / S)
        custom = ()
        fn = lambda a, b_, c: orc.relu_attention(a, b_, c, post_scale=1.0 / S)  # noqa: E731
    qd, kd, vd = (t.cuda().requires_grad_() for t in (q, k, v))
    o = eng(qd, kd, vd, *custom)
    o.backward(d_o.cuda())
    torch.cuda.synchronize()
    eng.check_status()
    for b, h in ((3, 17), (0, 0)):
        sl = (slice(b, b + 1), slice(None), slice(h, h + 1))
        ro, (rq, rk, rv) = orc.fwd_bwd(fn, (q[sl], k[sl], v[sl]), d_o[sl])
        for name, got, ref in (("o", o, ro), ("dq", qd.grad, rq), ("dk", kd.grad, rk), ("dv", vd.grad, rv)):
            check(f"cfg3.{kind}.b{b}h{h}.{name}", got[sl], ref, dt, stages=2)


def test_cfg4_mamba2_l8192_with_d_skip():
    """Config 4's length and distributions (L=8192, P=64, N=128, chunk-independent recurrence, bf16; x, B, C ~ N(0,1),
    dt = softplus(N(0,1) - 4), A = -exp(U(ln 1, ln 16)), D_skip ~ N(0,1)) on one batch row and two heads, against fp64
    autograd through the step-by-step recurrence, every gradient included.
    bf16 stages: y = scan output (P, v', carried state: 3 rounded operands) stored (1) plus the skip term -> 4;
    dx: dS, the carried dH, v'-gradient stored, dt product -> 4; dB, dC: dS / P, states, result -> 4.  The gradients of
    dt, A and D are fp32 sums over 64 (and L) cancelling terms of those bf16 quantities: rel-L2 <= 2e-2 is asked of them."""
    B, H, T, N, P, dt_ = 1, 2, 8192, 128, 64, torch.bfloat16
    x, dt, A, Bm, Cm = helpers.mamba2_inputs(B, H, T, N, P, dt_, seed=4)
    g = torch.Generator().manual_seed(44)
    Dk = torch.randn(1, H, generator=g)
    d_o = (0.1 * torch.randn(B, H, T, P, generator=g)).to(dt_)
    eng = helpers.mamba2_engine(B, H, T, N, P, dt_, d_skip=True)
    leaves = [t.cuda().requires_grad_() for t in (Cm, Bm, x, dt, A.view(1, H))]
    dtb = dt.to(dt_).cuda().requires_grad_()
    Dd = Dk.cuda().requires_grad_()
    y = eng(*leaves, dtb, Dd)
    y.backward(d_o.cuda())
    torch.cuda.synchronize()
    eng.check_status()
    C2, B2, x2, dt2, A2, dtb2, D2 = [t.detach().double().cpu().requires_grad_() for t in (*leaves, dtb, Dd)]
    # the operator's mapping: decay = dt * A (fp32 dt), v = x * dt (the 16-bit dt), skip on the raw x
    from oracle.linear_oracle import linear_scan
    yref = linear_scan(C2, B2, x2 * dtb2[..., None], dt2 * A2.view(1, H, 1)) + D2.view(1, H, 1, 1) * x2
    yref.backward(d_o.double())
    check("cfg4.y", y, yref.detach(), dt_, stages=4, unnormalised=True)
    check("cfg4.dx", leaves[2].grad, x2.grad, dt_, stages=4, unnormalised=True)
    check("cfg4.dC", leaves[0].grad, C2.grad, dt_, stages=4, unnormalised=True)
    check("cfg4.dB", leaves[1].grad, B2.grad, dt_, stages=4, unnormalised=True)
    for name, got, ref in (("d(dt) via decay", leaves[3].grad, dt2.grad), ("dA", leaves[4].grad, A2.grad),
                           ("d(dt) via v_mod", dtb.grad, dtb2.grad), ("dD", Dd.grad, D2.grad)):
        check(f"cfg4.{name}", got, ref, dt_, rel_limit=2e-2)


def test_cfg4_full_head_count_agrees_with_the_two_head_run():
    """B=2, H=80 (the configuration's head count, ngroups = 1) at L=8192: y, dx of two heads are what the same kernels
    give when those two heads run alone, and dB / dC are the sum over all 80 heads of per-head terms, checked through
    their linearity in dO (gradients for dO and 2 dO differ by the factor 2)."""
    B, H, T, N, P, dt_ = 2, 80, 8192, 128, 64, torch.bfloat16
    x, dt, A, Bm, Cm = helpers.mamba2_inputs(B, H, T, N, P, dt_, seed=5)
    g = torch.Generator().manual_seed(45)
    Dk = torch.randn(1, H, generator=g)
    d_o = (0.1 * torch.randn(B, H, T, P, generator=g)).to(dt_)
    eng = helpers.mamba2_engine(B, H, T, N, P, dt_, d_skip=True)

    def run(eng_, Cm_, Bm_, x_, dt_f, A_, D_, do_):
        leaves = [t.cuda().requires_grad_() for t in (Cm_, Bm_, x_, dt_f, A_)]
        dtb = dt_f.to(dt_).cuda().requires_grad_()
        y = eng_(*leaves, dtb, D_.cuda())
        y.backward(do_.cuda())
        torch.cuda.synchronize()
        eng_.check_status()
        return y.detach(), [t.grad for t in leaves]

    y, gr = run(eng, Cm, Bm, x, dt, A.view(1, H), Dk, d_o)
    y2, gr2 = run(eng, Cm, Bm, x, dt, A.view(1, H), Dk, 2 * d_o)
    torch.testing.assert_close(gr2[0].float(), 2 * gr[0].float(), rtol=2e-2, atol=2e-2 * gr[0].float().abs().max().item())
    torch.testing.assert_close(gr2[1].float(), 2 * gr[1].float(), rtol=2e-2, atol=2e-2 * gr[1].float().abs().max().item())
    hs = [7, 63]
    small = helpers.mamba2_engine(1, 2, T, N, P, dt_, d_skip=True)
    ys, gs = run(small, Cm[1:2], Bm[1:2], x[1:2, hs], dt[1:2, hs], A[hs].view(1, 2), Dk[:, hs], d_o[1:2, hs])
    assert torch.equal(y[1:2, hs], ys)
    assert torch.equal(gr[2][1:2, hs], gs[2])


def test_cfg5_mla_decode_s8192():
    """Config 5's shape at batch 2 of 128: 128 heads, latent KV length 8192, D = 512 + 64, fp16, scale 1/sqrt(192)."""
    B, H, S, dt = 2, 128, 8192, torch.float16
    scale = 1 / math.sqrt(192)
    g = torch.Generator().manual_seed(6)
    q, q_pe = torch.randn(B, 1, H, 512, generator=g).to(dt), torch.randn(B, 1, H, 64, generator=g).to(dt)
    kv, k_pe = torch.randn(B, S, 1, 512, generator=g).to(dt), torch.randn(B, S, 1, 64, generator=g).to(dt)
    eng = helpers.mla_engine(B, H, S, dt, scale)
    o = eng(q.cuda(), q_pe.cuda(), kv.cuda(), k_pe.cuda())
    torch.cuda.synchronize()
    eng.check_status()
    assert eng._mla.last_num_split > 1
    check("cfg5.o", o[:, 0], orc.mla_decode(q[:, 0], q_pe[:, 0], kv, k_pe, scale=scale), dt)
