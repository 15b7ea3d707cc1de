"""CPU oracle for the attention paths: plain PyTorch, fp32 compute on the (fp16 / bf16 rounded)
inputs, gradients by autograd.  TEST INFRASTRUCTURE ONLY (see oracle/__init__.py).

Each function restates the reference's own checker for that variant; citations are paths inside
microsoft/AttentionEngine.  Pinning: ``tests/golden/*.npz`` hold outputs of the reference's own
reference functions executed from its source tree by ``tests/golden/make_golden.py``;
``tests/test_oracle_golden.py`` compares this file against them.  Sigmoid attention, whose checker in the
reference is the third-party flash_sigmoid package, is pinned through the reference's own score_mod instead:
``sigmoid.npz`` holds that score_mod and its symbolic derivative evaluated by the reference's IR front end.
"""
from __future__ import annotations

import math

import torch


def _expand_kv(x: torch.Tensor, groups: int) -> torch.Tensor:
    # query head i reads kv head i // groups (attention_engine/core/template/tl_template/attn/attn_gqa_tl.py:80)
    return x if groups == 1 else x.repeat_interleave(groups, dim=2)


def softmax_attention(q, k, v, causal: bool, scale: float | None = None, return_lse: bool = False):
    """Naive softmax attention, [B, S, H, D] layout, GQA by head grouping.
    Restates the fallback ``flash_attn_func`` of attention_engine/benchmark/bench_utils.py:1250-1275:
    scores = q k^T; causal -> masked_fill(-inf) below-diagonal kept; softmax(scores * scale); attn v."""
    q, k, v = q.float(), k.float(), v.float()
    D = q.shape[-1]
    scale = 1.0 / math.sqrt(D) if scale is None else scale
    g = q.shape[2] // k.shape[2]
    kf, vf = _expand_kv(k, g), _expand_kv(v, g)
    s = torch.einsum("bqhd,bkhd->bhqk", q, kf)
    if causal:
        keep = torch.ones(q.shape[1], k.shape[1], dtype=torch.bool, device=q.device).tril()
        s = s.masked_fill(~keep, float("-inf"))
    s = s * scale
    p = torch.softmax(s, dim=-1)
    o = torch.einsum("bhqk,bkhd->bqhd", p, vf)
    if return_lse:
        return o, torch.logsumexp(s, dim=-1)
    return o


def relu_attention(q, k, v, scale: float | None = None, post_scale: float = 1.0, causal: bool = False):
    """P = relu(q k^T * scale) * post_scale; O = P v.  Restates ``ref_program`` of
    attention_engine/benchmark/bench_utils.py:979-984 (post_scale = 1 there; the 1/S factor of the
    non-causal benchmark config is a score_mod change in the style of attn_script/reluattn.py:14-17)."""
    q, k, v = q.float(), k.float(), v.float()
    scale = 1.0 / math.sqrt(q.shape[-1]) if scale is None else scale
    g = q.shape[2] // k.shape[2]
    s = torch.einsum("bqhd,bkhd->bhqk", q, _expand_kv(k, g)) * scale
    p = torch.relu(s) * post_scale
    if causal:
        keep = torch.ones(q.shape[1], k.shape[1], dtype=torch.bool, device=q.device).tril()
        p = p * keep
    return torch.einsum("bhqk,bkhd->bqhd", p, _expand_kv(v, g))


def sigmoid_attention(q, k, v, scale: float | None = None, bias: float = 0.0, causal: bool = False):
    """P = sigmoid(q k^T * scale + bias) written as (tanh(x / 2) + 1) / 2 as in
    attn_script/sigmoidattn.py:14-18; no row normalisation.  Pinned by tests/golden/sigmoid.npz (the reference's
    score_mod and its derivative evaluated by the reference's IR); the reference itself checks this variant against
    the third-party flash_sigmoid package only (bench_utils.py:736-744)."""
    q, k, v = q.float(), k.float(), v.float()
    scale = 1.0 / math.sqrt(q.shape[-1]) if scale is None else scale
    g = q.shape[2] // k.shape[2]
    x = torch.einsum("bqhd,bkhd->bhqk", q, _expand_kv(k, g)) * scale + bias
    p = (torch.tanh(x * 0.5) + 1.0) * 0.5
    if causal:
        keep = torch.ones(q.shape[1], k.shape[1], dtype=torch.bool, device=q.device).tril()
        p = p * keep
    return torch.einsum("bhqk,bkhd->bqhd", p, _expand_kv(v, g))


def retention_parallel(q, k, v, mask):
    """Parallel retention: qk * decay mask, rows normalised by max(sum |.|, 1) with the normaliser
    detached.  Restates ``ref_program`` of attention_engine/benchmark/bench_utils.py:1062-1067."""
    q, k, v = q.float(), k.float(), v.float()
    qkm = torch.einsum("bqhd,bkhd->bhqk", q, k) * mask.float()
    r = qkm.detach().abs().sum(dim=-1, keepdim=True).clamp(min=1.0)
    return torch.einsum("bhqk,bkhd->bqhd", qkm / r, v)


def mla_decode(q, q_pe, kv, k_pe, scale: float | None = None, return_lse: bool = False):
    """Absorbed-MLA decode.  q [B, H, 512], q_pe [B, H, 64], kv [B, S, 1, 512], k_pe [B, S, 1, 64].
    Restates ``ref_program`` of attention_engine/core/template/tl_template/attn/mla_decode_tl.py:266-306
    (scores over the concatenated 576 dims, softmax, output over the first 512 dims).  ``scale``
    defaults to the reference's 1/sqrt(576); the benchmark config passes 1/sqrt(192)."""
    q, q_pe, kv, k_pe = q.float(), q_pe.float(), kv.float(), k_pe.float()
    scale = 1.0 / math.sqrt(q.shape[-1] + q_pe.shape[-1]) if scale is None else scale
    query = torch.cat([q, q_pe], dim=-1)                     # [B, H, 576]
    key = torch.cat([kv, k_pe], dim=-1)[:, :, 0]              # [B, S, 576]
    s = torch.einsum("bhd,bsd->bhs", query, key) * scale
    p = torch.softmax(s, dim=-1)
    o = torch.einsum("bhs,bsd->bhd", p, kv[:, :, 0])
    if return_lse:
        return o, torch.logsumexp(s, dim=-1)
    return o


def fwd_bwd(fn, inputs, d_out):
    """Run ``fn(*inputs)`` on fp32 leaf copies and return (out, grads) for the given upstream gradient."""
    leaves = [t.detach().float().requires_grad_() for t in inputs]
    out = fn(*leaves)
    out.backward(d_out.float())
    return out.detach(), [t.grad for t in leaves]


def error_stats(actual: torch.Tensor, expected: torch.Tensor):
    """(max-abs error, relative L2 error), both in fp64."""
    a, e = actual.double().cpu(), expected.double().cpu()
    return (a - e).abs().max().item(), ((a - e).norm() / e.norm().clamp_min(1e-30)).item()
