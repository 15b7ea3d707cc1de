"""The CPU oracle against the golden vectors produced by the reference's own reference functions
(tests/golden/make_golden.py).  No GPU."""
import math
import os

import numpy as np
import pytest
import torch

import attentionengine_b200 as ae
from oracle import attention_oracle as orc
from oracle.ir_eval import evaluate, online_attention

from helpers import OnlineSoftmax, causal_mask

TIGHT = dict(rtol=2e-5, atol=2e-5)


def _t(a):
    return torch.from_numpy(np.asarray(a))


@pytest.mark.parametrize("case", ["cfg1", "gqa_causal", "gqa_full", "mha_d128"])
def test_softmax_oracle_matches_reference(golden_dir, case):
    z = np.load(os.path.join(golden_dir, "softmax.npz"))
    q, k, v, d_o = (_t(z[f"{case}.{n}"]) for n in ("q", "k", "v", "do"))
    causal = bool(z[f"{case}.causal"])
    D = q.shape[-1]
    o, (dq, dk, dv) = orc.fwd_bwd(lambda a, b, c: orc.softmax_attention(a, b, c, causal, 1 / math.sqrt(D)), (q, k, v), d_o)
    for name, got in (("o", o), ("dq", dq), ("dk", dk), ("dv", dv)):
        torch.testing.assert_close(got, _t(z[f"{case}.{name}"]), **TIGHT, msg=lambda m: f"{case}.{name}: {m}")


def test_relu_oracle_matches_reference(golden_dir):
    z = np.load(os.path.join(golden_dir, "relu.npz"))
    q, k, v, d_o = (_t(z[n]) for n in ("q", "k", "v", "do"))
    o, (dq, dk, dv) = orc.fwd_bwd(lambda a, b, c: orc.relu_attention(a, b, c), (q, k, v), d_o)
    for name, got in (("o", o), ("dq", dq), ("dk", dk), ("dv", dv)):
        torch.testing.assert_close(got, _t(z[name]), rtol=2e-5, atol=1e-4)


def test_retention_oracle_matches_reference(golden_dir):
    z = np.load(os.path.join(golden_dir, "retention.npz"))
    o = orc.retention_parallel(_t(z["q"]), _t(z["k"]), _t(z["v"]), _t(z["mask"]))
    torch.testing.assert_close(o, _t(z["o"]), **TIGHT)


def test_mla_oracle_matches_reference(golden_dir):
    z = np.load(os.path.join(golden_dir, "mla_decode.npz"))
    o = orc.mla_decode(_t(z["q"]), _t(z["q_pe"]), _t(z["kv"]), _t(z["k_pe"]))
    torch.testing.assert_close(o, _t(z["o"]), **TIGHT)


def test_online_recurrence_equals_closed_form(golden_dir):
    """The tile-by-tile restatement of the forward kernel gives the same O and lse as the naive reference."""
    z = np.load(os.path.join(golden_dir, "softmax.npz"))
    q, k, v = (_t(z[f"gqa_causal.{n}"]) for n in ("q", "k", "v"))
    D = q.shape[-1]

    def score_mod(score, custom, b, h, q_idx, kv_idx):
        return score * (1 / math.sqrt(D))

    o, fin = online_attention(ae, q, k, v, score_mod, causal_mask, OnlineSoftmax(), block_n=128)
    # P is rounded to fp16 before P V, as in the kernel: tolerance of that rounding
    torch.testing.assert_close(o, _t(z["gqa_causal.o"]), rtol=2e-3, atol=2e-3)
    _, lse = orc.softmax_attention(q, k, v, True, 1 / math.sqrt(D), return_lse=True)
    torch.testing.assert_close(fin["lse"], lse, rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("name", ["scale", "sigmoid", "relu", "div_log"])
def test_symbolic_autodiff_matches_reference(golden_dir, name):
    """This package's reverse-mode differentiation of a score_mod equals the reference's and autograd's."""
    z = np.load(os.path.join(golden_dir, "autodiff.npz"))
    x, seed, bias = _t(z["x"]), _t(z["seed"]), float(z["bias"])
    fns = {
        "scale": lambda s, T: s * 0.125,
        "sigmoid": lambda s, T: (((s + T) * 0.5).tanh() + 1) * 0.5,
        "relu": lambda s, T: (s * 0.125).max(0),
        "div_log": lambda s, T: (s * s + 1.0).log() * s / (s * s + 2.0),
    }
    s = ae.SymbolicArray("scores", ae.Var("scores"), shape_idx=["block_M", "block_N"])
    T = ae.SymbolicTensor("T", (1,))
    y = fns[name](s, T)
    d = ae.SymbolicArray("d", ae.Var("d"), shape_idx=["block_M", "block_N"])
    d.require_grad = False
    y.backward(d)
    env = {id(s): x, id(T): torch.tensor(bias), id(d): seed}
    torch.testing.assert_close(torch.as_tensor(evaluate(y, env)).expand_as(x), _t(z[f"{name}.y"]), rtol=1e-6, atol=1e-6)
    torch.testing.assert_close(torch.as_tensor(evaluate(s.grad, env)).expand_as(x), _t(z[f"{name}.dx"]), rtol=1e-5, atol=1e-6)


def test_autodiff_ops_the_reference_lacks():
    """Sub, Neg, Exp, Abs have no derivative in the reference (core/transform/core.py:193-195); here they do."""
    x = torch.linspace(-2, 2, 41).view(1, -1).clone().requires_grad_()
    s = ae.SymbolicArray("scores", ae.Var("scores"), shape_idx=["block_M", "block_N"])
    y = (-(s - 0.5)).exp() * s.abs() + (2.0 - s) / 3.0
    d = ae.SymbolicArray("d", ae.Var("d"), shape_idx=["block_M", "block_N"])
    d.require_grad = False
    y.backward(d)
    seed = torch.ones_like(x)
    yt = torch.exp(-(x - 0.5)) * x.abs() + (2.0 - x) / 3.0
    yt.backward(seed)
    got = torch.as_tensor(evaluate(s.grad, {id(s): x.detach(), id(d): seed}))
    keep = x.detach().abs() > 1e-6  # |x| is not differentiable at 0
    torch.testing.assert_close(got[keep], x.grad[keep], rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("name", ["causal", "causal_less", "sliding", "head_dep"])
@pytest.mark.parametrize("blk", [(128, 128), (128, 64)])
def test_block_mask_matches_reference(golden_dir, name, blk):
    z = np.load(os.path.join(golden_dir, "block_masks.npz"))
    fns = {
        "causal": lambda b, h, q, kv: q >= kv,
        "causal_less": lambda b, h, q, kv: q >= kv + 128,
        "sliding": lambda b, h, q, kv: torch.logical_and(q >= kv, q - kv <= 100),
        "head_dep": lambda b, h, q, kv: q >= kv + h * 64,
    }
    bm, bn = blk
    got = ae.create_block_mask(fns[name], 2, 4, 512, 512, "cpu", bm, bn)
    ref = _t(z[f"{name}.{bm}x{bn}.block"])
    assert got.dtype == torch.int8 and torch.equal(got, ref)
    from attentionengine_b200.core import is_causal_mask, is_less_causal_mask
    assert bool(is_causal_mask(got, bm, bn)) == bool(z[f"{name}.{bm}x{bn}.is_causal"])
    assert bool(is_less_causal_mask(got, bm, bn)) == bool(z[f"{name}.{bm}x{bn}.is_less_causal"])


def test_create_mask_dense_matches_blockwise():
    m = ae.core.create_mask(lambda b, h, q, kv: q >= kv, 1, 2, 200, 300, "cpu")
    assert m.shape == (1, 2, 200, 300)
    assert torch.equal(m[0, 0], torch.ones(200, 300, dtype=torch.bool).tril())


def test_linear_scan_oracle_matches_fla_naive(golden_dir):
    from oracle.linear_oracle import linear_scan
    z = np.load(os.path.join(golden_dir, "linear_scan.npz"))
    o = linear_scan(_t(z["q"]), _t(z["k"]), _t(z["v"]), _t(z["a"]))
    torch.testing.assert_close(o.float(), _t(z["o"]), rtol=1e-4, atol=1e-4)


def test_sigmoid_oracle_matches_reference_score_mod(golden_dir):
    """sigmoid.npz: the score_mod of the reference's attn_script/sigmoidattn.py, traced and differentiated by the
    reference's own IR, inside the un-normalised P V composition; the oracle writes the same function in torch."""
    z = np.load(os.path.join(golden_dir, "sigmoid.npz"))
    q, k, v, d_o = (_t(z[n]) for n in ("q", "k", "v", "do"))
    o, (dq, dk, dv) = orc.fwd_bwd(lambda a, b, c: orc.sigmoid_attention(a, b, c, scale=1.0, bias=float(z["bias"])),
                                  (q, k, v), d_o)
    for name, got in (("o", o), ("dq", dq), ("dk", dk), ("dv", dv)):
        torch.testing.assert_close(got, _t(z[name]), rtol=1e-4, atol=1e-4, msg=lambda m: f"{name}: {m}")
    # and the textbook form: (tanh(x / 2) + 1) / 2 is the logistic function
    x = torch.linspace(-12, 12, 97)
    torch.testing.assert_close((torch.tanh(x * 0.5) + 1) * 0.5, torch.sigmoid(x), rtol=1e-6, atol=1e-7)


def test_mamba2_mapping_matches_reference_mods(golden_dir):
    """mamba2.npz: decay_mod / v_mod of the reference's attn_script/mamba2_ngroup1.py evaluated by the reference's IR
    and fed to flash-linear-attention's naive recurrence with q = C, k = B; the oracle's mamba2_ssd is the same map."""
    from oracle.linear_oracle import mamba2_ssd
    z = np.load(os.path.join(golden_dir, "mamba2.npz"))
    x, dt, A, Bm, Cm = (_t(z[n]) for n in ("x", "dt", "A", "Bm", "Cm"))
    o = mamba2_ssd(x, dt, A, Bm, Cm)
    torch.testing.assert_close(o.float(), _t(z["o"]), rtol=1e-4, atol=1e-4)
    # the skip connection is a per-head multiple of the raw input added to that output
    Dk = torch.tensor([0.5, -1.25, 2.0])
    torch.testing.assert_close(mamba2_ssd(x, dt, A, Bm, Cm, Dk), o + Dk.view(1, -1, 1, 1) * x.double())
