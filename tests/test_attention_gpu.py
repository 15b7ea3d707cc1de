"""Parity of the CUDA attention path (through AttentionEngine -> C ABI -> sm_100a kernels) against the
CPU oracle and the golden vectors.  Acceptance rule (tests/parity.py): max-abs <= 2e-2 and rel-L2 <= 1e-3 for fp16
outputs and gradients, as the benchmark specification states; bf16 results are held to a multiple of the bf16
rounding floor measured on the tensor itself."""
import math
import os

import numpy as np
import pytest
import torch

from oracle import attention_oracle as orc

import helpers
import parity
from attentionengine_b200 import AttentionEngine, CustomIO

pytestmark = pytest.mark.gpu

MAX_ABS, REL_L2 = parity.MAX_ABS, parity.REL_L2


@pytest.fixture(params=["split", "fused"], autouse=True)
def bwd_mode(request, monkeypatch):
    """Every test of this file runs with both forms of the attention backward (two-pass / one-pass)."""
    from attentionengine_b200 import tune
    from attentionengine_b200.attn_engine import attn_bwd
    monkeypatch.setattr(attn_bwd, "DEFAULT_MODE", request.param)
    monkeypatch.setattr(tune, "PACKAGE_FILE", tune.PACKAGE_FILE.with_name("no_table_in_these_tests.json"))
    return request.param


@pytest.fixture(params=["single", "pair"])
def fwd_form(request, monkeypatch):
    """A test that takes this fixture also runs with the forward over CTA pairs (tcgen05 cta_group::2) wherever the
    engine's shape allows it (value head dim 128, no block lists)."""
    from attentionengine_b200.attn_engine import attn_engine as ae
    monkeypatch.setattr(ae, "FWD_PAIR", int(request.param == "pair"))
    return request.param


@pytest.fixture(params=[2, 1])
def scan_groups(request, monkeypatch):
    """A test that takes this fixture runs the scan's forward and reverse kernels with two row warpgroups (the default)
    and with one."""
    from attentionengine_b200.attn_engine import linear_attn_engine as le
    monkeypatch.setattr(le, "LIN_FWD_NWG", request.param)
    monkeypatch.setattr(le, "LIN_BWD_NWG", request.param)
    return request.param


def _check(name, got, ref, dtype, unnormalised=False, stages=None):
    """bf16 rounding stages of the attention kernels: O and dV = (P rounded) x operand, stored -> 2; dQ and dK =
    (dS rounded) x operand, stored, with dS built from delta = rowsum(O dO) of the rounded O -> 3.  The linear-attention
    results (``unnormalised``) pass through P / dS, the carried state, the rescaled values and the store -> 4."""
    if stages is None:
        stages = 4 if unnormalised else (3 if name.split(".")[-1].split()[-1] in ("dq", "dk") else 2)
    parity.check(name, got, ref, dtype, stages=stages, unnormalised=unnormalised)


def _run(eng, q, k, v, d_o, custom=()):
    qd, kd, vd = (t.cuda().requires_grad_() for t in (q, k, v))
    o = eng(qd, kd, vd, *[c.cuda() for c in custom])
    o.backward(d_o.cuda())
    torch.cuda.synchronize()
    eng.check_status()
    return o.detach().cpu(), qd.grad.cpu(), kd.grad.cpu(), vd.grad.cpu()


@pytest.mark.parametrize("case", ["cfg1", "gqa_causal", "gqa_full", "mha_d128"])
def test_softmax_against_reference_golden(golden_dir, case):
    """Config 1 of the benchmark (B=1, H=4, S=512, D=64, causal, dO = ones) and three small variants,
    against outputs of the reference's own naive attention."""
    z = np.load(os.path.join(golden_dir, "softmax.npz"))
    q, k, v, d_o = (torch.from_numpy(z[f"{case}.{n}"]) for n in ("q", "k", "v", "do"))
    causal = bool(z[f"{case}.causal"])
    B, S, Hq, D = q.shape
    eng = helpers.softmax_engine(B, Hq, k.shape[2], S, D, D, torch.float16, causal)
    got = _run(eng, q, k, v, d_o)
    for name, g in zip(("o", "dq", "dk", "dv"), got):
        _check(f"{case}.{name}", g, torch.from_numpy(z[f"{case}.{name}"]), torch.float16)


SHAPES = [
    # B, Hq, Hkv, S, D, causal, dtype
    (2, 8, 2, 1024, 128, True, torch.float16),
    (1, 4, 4, 512, 128, False, torch.bfloat16),
    (1, 2, 2, 384, 64, True, torch.float16),
    (1, 2, 2, 300, 64, True, torch.float16),      # ragged: last tile partly out of range
    (1, 2, 1, 200, 128, False, torch.float16),    # ragged, non-causal, GQA
    (1, 1, 1, 64, 64, True, torch.float16),       # shorter than one tile
    (2, 4, 2, 129, 128, True, torch.bfloat16),    # one row past a tile
]


@pytest.mark.parametrize("B,Hq,Hkv,S,D,causal,dtype", SHAPES)
def test_softmax_shapes_against_oracle(B, Hq, Hkv, S, D, causal, dtype):
    q, k, v, d_o = helpers.seeded_qkv(B, Hq, Hkv, S, D, D, dtype, seed=S)
    eng = helpers.softmax_engine(B, Hq, Hkv, S, D, D, dtype, causal)
    got = _run(eng, q, k, v, d_o)
    o, (dq, dk, dv) = orc.fwd_bwd(lambda a, b, c: orc.softmax_attention(a, b, c, causal), (q, k, v), d_o)
    for name, g, r in zip(("o", "dq", "dk", "dv"), got, (o, dq, dk, dv)):
        _check(name, g, r, dtype)


@pytest.mark.parametrize("B,Hq,Hkv,S,D,causal,dtype", [
    (2, 8, 2, 1024, 128, True, torch.float16),    # four pairs per head, the even tile of each idles on the last step
    (1, 4, 4, 512, 128, False, torch.bfloat16),
    (1, 2, 1, 200, 128, False, torch.float16),    # ragged: the second CTA's K half is partly out of range
    (2, 4, 2, 129, 128, True, torch.bfloat16),    # the second tile has one row
    (1, 2, 2, 640, 64, True, torch.float16),      # odd tile count: the last pair's second CTA has no tile
])
def test_forward_over_cta_pairs(B, Hq, Hkv, S, D, causal, dtype):
    """The forward built on tcgen05 cta_group::2 (tuned entry ``fwd_pair``): output, saved LSE (through the gradients of
    the backward that consumes it) against the oracle, and the output against the single-CTA forward's."""
    q, k, v, d_o = helpers.seeded_qkv(B, Hq, Hkv, S, D, 128, dtype, seed=S + 1)
    eng = helpers.softmax_engine(B, Hq, Hkv, S, D, 128, dtype, causal, tuned_config={"fwd_pair": 1})
    assert eng.kernels.fwd_pair
    got = _run(eng, q, k, v, d_o)
    o, (dq, dk, dv) = orc.fwd_bwd(lambda a, b, c: orc.softmax_attention(a, b, c, causal), (q, k, v), d_o)
    for name, g, r in zip(("o", "dq", "dk", "dv"), got, (o, dq, dk, dv)):
        _check(name, g, r, dtype)
    single = helpers.softmax_engine(B, Hq, Hkv, S, D, 128, dtype, causal)
    assert not single.kernels.fwd_pair
    o1, _ = single._launch_fwd(q.cuda(), k.cuda(), v.cuda(), ())
    torch.cuda.synchronize()
    torch.testing.assert_close(got[0].float(), o1.cpu().float(), rtol=0, atol=2e-3 if dtype == torch.float16 else 1.6e-2)


def test_lse_is_saved_like_the_reference():
    """final_rowscales['lse'] is the natural-log LSE of the scaled scores, [B, H, S] fp32 (lower.py:385-392)."""
    B, Hq, Hkv, S, D = 1, 4, 2, 256, 64
    q, k, v, _ = helpers.seeded_qkv(B, Hq, Hkv, S, D, D, torch.float16, seed=5)
    eng = helpers.softmax_engine(B, Hq, Hkv, S, D, D, torch.float16, True)
    o, finals = eng._launch_fwd(q.cuda(), k.cuda(), v.cuda(), ())
    torch.cuda.synchronize()
    _, lse = orc.softmax_attention(q, k, v, True, return_lse=True)
    assert finals[0].shape == (B, Hq, S) and finals[0].dtype == torch.float32
    torch.testing.assert_close(finals[0].cpu(), lse, rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("causal", [False, True])
def test_sigmoid_attention(causal, fwd_form):
    B, H, S, D, dtype = 1, 4, 512, 128, torch.bfloat16
    q, k, v, d_o = helpers.seeded_qkv(B, H, H, S, D, D, dtype, seed=11)
    bias = torch.tensor([-math.log(S)], dtype=torch.float32)
    eng = helpers.sigmoid_engine(B, H, S, D, dtype, causal)
    got = _run(eng, q, k, v, d_o, custom=(bias,))
    o, (dq, dk, dv) = orc.fwd_bwd(lambda a, b, c: orc.sigmoid_attention(a, b, c, bias=float(bias), causal=causal),
                                  (q, k, v), d_o)
    for name, g, r in zip(("o", "dq", "dk", "dv"), got, (o, dq, dk, dv)):
        _check(name, g, r, dtype)


def test_relu_attention_against_reference_golden(golden_dir):
    z = np.load(os.path.join(golden_dir, "relu.npz"))
    q, k, v, d_o = (torch.from_numpy(z[n]) for n in ("q", "k", "v", "do"))
    B, S, H, D = q.shape
    eng = helpers.relu_engine(B, H, S, D, torch.float16)
    got = _run(eng, q, k, v, d_o)
    for name, g in zip(("o", "dq", "dk", "dv"), got):
        ref = torch.from_numpy(z[name])
        mx, rel = orc.error_stats(g, ref)
        # un-normalised relu attention has outputs of magnitude ~S/2: the absolute bound scales with it
        assert rel <= REL_L2 and mx <= MAX_ABS * max(1.0, ref.abs().max().item()), f"{name}: {mx:.3e} {rel:.3e}"


def test_relu_attention_benchmark_form(fwd_form):
    """P = relu(S / sqrt(D)) / S_len, non-causal, bf16 (config 3 of the benchmark, small)."""
    B, H, S, D, dtype = 1, 2, 512, 128, torch.bfloat16
    q, k, v, d_o = helpers.seeded_qkv(B, H, H, S, D, D, dtype, seed=12)
    eng = helpers.relu_engine(B, H, S, D, dtype, post_scale=1.0 / S)
    got = _run(eng, q, k, v, d_o)
    o, (dq, dk, dv) = orc.fwd_bwd(lambda a, b, c: orc.relu_attention(a, b, c, post_scale=1.0 / S), (q, k, v), d_o)
    for name, g, r in zip(("o", "dq", "dk", "dv"), got, (o, dq, dk, dv)):
        _check(name, g, r, dtype)


def test_sliding_window_block_sparse():
    """mask_mod that is not causal-shaped: block lists skip empty tiles, partial tiles are masked per element."""
    B, H, S, D, dtype = 1, 2, 1024, 64, torch.float16
    W = 200

    def window(b, h, q_idx, kv_idx):
        return torch.logical_and(q_idx >= kv_idx, q_idx - kv_idx <= W)

    def score_mod(score, custom, b, h, q_idx, kv_idx):
        return score * (1 / math.sqrt(D))

    from attentionengine_b200 import AttentionEngine, CustomIO
    eng = AttentionEngine(helpers.metas(B, H, H, S, D, D, dtype), CustomIO({}), score_mod=score_mod, mask_mod=window,
                          online_func=helpers.OnlineSoftmax())
    assert eng.mask_mode == 2
    q, k, v, d_o = helpers.seeded_qkv(B, H, H, S, D, D, dtype, seed=13)
    got = _run(eng, q, k, v, d_o)

    def ref(a, b, c):
        s = torch.einsum("bqhd,bkhd->bhqk", a, b) / math.sqrt(D)
        i = torch.arange(S)
        keep = (i.view(-1, 1) >= i.view(1, -1)) & (i.view(-1, 1) - i.view(1, -1) <= W)
        s = s.masked_fill(~keep, float("-inf"))
        return torch.einsum("bhqk,bkhd->bqhd", torch.softmax(s, -1), c)

    o, (dq, dk, dv) = orc.fwd_bwd(ref, (q, k, v), d_o)
    for name, g, r in zip(("o", "dq", "dk", "dv"), got, (o, dq, dk, dv)):
        _check(name, g, r, dtype)


def test_dynamic_shape_engine_runs_several_lengths(fwd_form):
    """One engine built from named dims serves different batch sizes and lengths: causal (analytic bounds) and a
    sliding window (tile lists rebuilt per shape)."""
    from attentionengine_b200 import AttentionEngine, CustomIO, meta_tensor
    D, H, dtype, W = 64, 2, torch.float16, 150
    scale = 1 / math.sqrt(D)
    metas = tuple(meta_tensor("B", "H", "S", D, dtype=dtype) for _ in range(3))
    masks = {"causal": lambda b, h, q_idx, kv_idx: q_idx >= kv_idx,
             "window": lambda b, h, q_idx, kv_idx: torch.logical_and(q_idx >= kv_idx, q_idx - kv_idx <= W)}
    for kind, mask in masks.items():
        eng = AttentionEngine(metas, CustomIO({}), score_mod=lambda s, c, b, h, q, kv: s * scale, mask_mod=mask,
                              online_func=helpers.OnlineSoftmax())
        assert eng.mask_mode == (1 if kind == "causal" else 2)
        for B, S in ((1, 300), (2, 640)):
            q, k, v, d_o = helpers.seeded_qkv(B, H, H, S, D, D, dtype, seed=40 + S)
            got = _run(eng, q, k, v, d_o)
            i = torch.arange(S)
            keep = i.view(-1, 1) >= i.view(1, -1)
            if kind == "window":
                keep = keep & (i.view(-1, 1) - i.view(1, -1) <= W)

            def ref(a, b, c):
                s_ = (torch.einsum("bqhd,bkhd->bhqk", a, b) * scale).masked_fill(~keep, float("-inf"))
                return torch.einsum("bhqk,bkhd->bqhd", torch.softmax(s_, -1), c)

            o, grads = orc.fwd_bwd(ref, (q, k, v), d_o)
            for name, g, r in zip(("o", "dq", "dk", "dv"), got, (o, *grads)):
                _check(f"{kind} S={S} {name}", g, r, dtype)


@pytest.mark.parametrize("n_split", [1, None, 5])
def test_gqa_decode_split_kv(n_split):
    """attn_script/gqa_inference.py: one query position, Hq > Hkv, K / V of a kv head streamed once for its group;
    1 split (no combine), the default split count and a forced ragged one (1000 keys = 8 tiles over 5 splits -> 4)."""
    B, Hq, Hkv, S, D, dtype = 2, 32, 8, 1000, 128, torch.float16
    eng = helpers.decode_engine(B, Hq, Hkv, 1, S, D, dtype)
    eng._decode.num_split = 4 if n_split == 5 else n_split
    g = torch.Generator().manual_seed(50)
    q = torch.randn(B, 1, Hq, D, generator=g).to(dtype)
    k = torch.randn(B, S, Hkv, D, generator=g).to(dtype)
    v = torch.randn(B, S, Hkv, D, generator=g).to(dtype)
    o = eng(q.cuda(), k.cuda(), v.cuda())
    torch.cuda.synchronize()
    eng.check_status()
    assert eng._decode.last_num_split == (1 if n_split == 1 else 4 if n_split == 5 else eng._decode.pick_splits(B, S))
    _check("o", o.cpu(), orc.softmax_attention(q, k, v, False), dtype)


def test_decode_engine_with_a_named_kv_length_serves_a_growing_cache():
    """meta_tensor(B, Hkv, "S_kv", D): one decode engine, calls with different KV lengths and batch sizes."""
    Hq, Hkv, D, dtype = 16, 4, 128, torch.float16
    eng = helpers.decode_engine("B", Hq, Hkv, 1, "S_kv", D, dtype)
    g = torch.Generator().manual_seed(53)
    for B, S in ((1, 300), (3, 1500), (2, 64)):
        q = torch.randn(B, 1, Hq, D, generator=g).to(dtype)
        k = torch.randn(B, S, Hkv, D, generator=g).to(dtype)
        v = torch.randn(B, S, Hkv, D, generator=g).to(dtype)
        o = eng(q.cuda(), k.cuda(), v.cuda())
        torch.cuda.synchronize()
        eng.check_status()
        _check(f"B={B} S={S} o", o.cpu(), orc.softmax_attention(q, k, v, False), dtype)


@pytest.mark.parametrize("Sq", [1, 3, 200])
def test_mha_decode_split_kv(Sq):
    """attn_script/mha_inference.py shape class: Hq == Hkv, a few query positions against a long KV range; 200 rows
    use both row tiles of the CTA.  bf16, D = 64."""
    B, H, S, D, dtype = 2, 4, 2048 + 77, 64, torch.bfloat16
    eng = helpers.decode_engine(B, H, H, Sq, S, D, dtype)
    g = torch.Generator().manual_seed(51)
    q = torch.randn(B, Sq, H, D, generator=g).to(dtype)
    k = torch.randn(B, S, H, D, generator=g).to(dtype)
    v = torch.randn(B, S, H, D, generator=g).to(dtype)
    o = eng(q.cuda(), k.cuda(), v.cuda())
    torch.cuda.synchronize()
    eng.check_status()
    assert eng._decode.last_num_split > 1
    _check("o", o.cpu(), orc.softmax_attention(q, k, v, False), dtype)


def test_decode_with_identity_online_func_sums_the_splits():
    """OnlineFunc.combine left at its default (weight 1 per split): relu attention, whose partial outputs add up."""
    B, Hq, Hkv, S, D, dtype = 1, 8, 2, 1536, 128, torch.float16
    scale = 1 / math.sqrt(D)
    metas = (helpers.meta_tensor(B, Hq, 1, D, dtype=dtype), helpers.meta_tensor(B, Hkv, S, D, dtype=dtype),
             helpers.meta_tensor(B, Hkv, S, D, dtype=dtype))
    eng = AttentionEngine(metas, CustomIO({}), score_mod=lambda s, c, b, h, q, kv: (s * scale).max(0) * (1.0 / S),
                          mask_mod=None, online_func=helpers.OnlineIdentity(), mask_value="0")
    g = torch.Generator().manual_seed(52)
    q = torch.randn(B, 1, Hq, D, generator=g).to(dtype)
    k = torch.randn(B, S, Hkv, D, generator=g).to(dtype)
    v = torch.randn(B, S, Hkv, D, generator=g).to(dtype)
    o = eng(q.cuda(), k.cuda(), v.cuda())
    torch.cuda.synchronize()
    eng.check_status()
    assert eng._decode.last_num_split > 1
    _check("o", o.cpu(), orc.relu_attention(q, k, v, post_scale=1.0 / S), dtype)


def test_run_to_run_determinism(bwd_mode):
    """The forward and the two-pass backward use no atomics: two runs give bit-identical outputs and gradients.  The
    one-pass backward adds its dQ tiles with fp32 atomics: o, dK, dV are still bit-identical, dQ agrees to rounding."""
    B, Hq, Hkv, S, D = 1, 4, 2, 512, 128
    q, k, v, d_o = helpers.seeded_qkv(B, Hq, Hkv, S, D, D, torch.float16, seed=21)
    eng = helpers.softmax_engine(B, Hq, Hkv, S, D, D, torch.float16, True)
    a = _run(eng, q, k, v, d_o)
    b = _run(eng, q, k, v, d_o)
    for name, x, y in zip(("o", "dq", "dk", "dv"), a, b):
        if bwd_mode == "fused" and name == "dq":
            torch.testing.assert_close(x.float(), y.float(), rtol=2e-3, atol=2e-4)
        else:
            assert torch.equal(x, y), name


def test_one_pass_and_two_pass_backward_agree():
    """Same inputs through both backward forms: dV comes from identical tensor-core products, dK and dQ differ only
    in summation order and in where the rounded dS tile is read from."""
    B, Hq, Hkv, S, D = 2, 8, 2, 640, 128
    q, k, v, d_o = helpers.seeded_qkv(B, Hq, Hkv, S, D, D, torch.float16, seed=22)
    res = {}
    for mode in ("split", "fused"):
        eng = helpers.softmax_engine(B, Hq, Hkv, S, D, D, torch.float16, True)
        eng.bwd_mode = mode
        res[mode] = _run(eng, q, k, v, d_o)
    assert torch.equal(res["split"][0], res["fused"][0]) and torch.equal(res["split"][3], res["fused"][3])
    for i in (1, 2):
        torch.testing.assert_close(res["split"][i].float(), res["fused"][i].float(), rtol=4e-3, atol=4e-4)


def test_probe_gemms():
    """The two tcgen05 operand paths the kernels rely on, in isolation."""
    import ctypes as C
    from attentionengine_b200 import runtime as rt
    for bf16, dt in ((0, torch.float16), (1, torch.bfloat16)):
        cfg = rt.KernelConfig(kind=rt.KIND_PROBE, dtype=bf16, head_dim=128, head_dim_v=128, threads=160,
                              smem_bytes=65536 + 256 + 1024, stages=1, mask_mode=0)
        m = rt.compile_module(rt.kernel_source("probe.cuh", prelude=f"#define AE_BF16 {bf16}\n"), "ae_probe", cfg)
        g = torch.Generator().manual_seed(1)
        a, b, p = (torch.randn(128, 128, generator=g).to(dt).cuda() for _ in range(3))
        for mode in (0, 1):
            d = torch.zeros(128, 128, device="cuda")
            st = torch.zeros(1, dtype=torch.int32, device="cuda")
            rt.check(rt.lib().ae_launch_probe(m.handle, a.data_ptr(), b.data_ptr(), p.data_ptr(), d.data_ptr(), mode,
                                              st.data_ptr(), C.c_void_p(torch.cuda.current_stream().cuda_stream)))
            torch.cuda.synchronize()
            assert st.item() == 0
            ref = a.float() @ b.float().T if mode == 0 else p.float() @ b.float()
            torch.testing.assert_close(d, ref, rtol=1e-4, atol=1e-3)


def test_full_size_properties():
    """At the benchmark's full shape the oracle is too slow; check size-independent properties instead:
    rows of P sum to one (O of constant V is that constant), linearity in V and dO, and agreement of a
    (batch, kv-group) slice with the oracle."""
    B, Hq, Hkv, S, D = 2, 8, 2, 8192, 128
    dt = torch.float16
    eng = helpers.softmax_engine(B, Hq, Hkv, S, D, D, dt, True)
    g = torch.Generator().manual_seed(3)
    q = torch.randn(B, S, Hq, D, generator=g).to(dt).cuda()
    k = torch.randn(B, S, Hkv, D, generator=g).to(dt).cuda()
    v1 = torch.randn(B, S, Hkv, D, generator=g).to(dt).cuda()
    ones = torch.ones_like(v1)
    o_ones, _ = eng._launch_fwd(q, k, ones, ())
    torch.testing.assert_close(o_ones.float(), torch.ones_like(o_ones).float(), rtol=2e-3, atol=2e-3)
    o1, _ = eng._launch_fwd(q, k, v1, ())
    o2, _ = eng._launch_fwd(q, k, (2 * v1), ())
    torch.testing.assert_close(o2.float(), 2 * o1.float(), rtol=2e-3, atol=2e-3)
    # one slice against the oracle (batch 1, kv head 1 -> q heads 4..7), first 1024 rows are self-contained
    sl = slice(0, 1024)
    qs, ks, vs = q[1:2, sl, 4:8].cpu(), k[1:2, sl, 1:2].cpu(), v1[1:2, sl, 1:2].cpu()
    ref = orc.softmax_attention(qs, ks, vs, True)
    _check("slice.o", o1[1:2, sl, 4:8].cpu(), ref, dt)
    eng.check_status()


# ---------------------------------------------------------------------------------------------------
# MLA split-KV decode
# ---------------------------------------------------------------------------------------------------
def _mla_inputs(B, H, S, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(B, 1, H, 512, generator=g).to(dtype), torch.randn(B, 1, H, 64, generator=g).to(dtype),
            torch.randn(B, S, 1, 512, generator=g).to(dtype), torch.randn(B, S, 1, 64, generator=g).to(dtype))


@pytest.mark.parametrize("n_split", [1, 3])
def test_mla_decode_against_reference_golden(golden_dir, n_split):
    """Output of the reference's own `ref_program` (scale 1/sqrt(576)), H = 16 heads, S = 320."""
    z = np.load(os.path.join(golden_dir, "mla_decode.npz"))
    q, q_pe, kv, k_pe = (torch.from_numpy(z[n]) for n in ("q", "q_pe", "kv", "k_pe"))
    B, H, _ = q.shape
    S = kv.shape[1]
    eng = helpers.mla_engine(B, H, S, torch.float16, 1 / math.sqrt(576))
    eng._mla.num_split = n_split
    o = eng(q.view(B, 1, H, 512).cuda(), q_pe.view(B, 1, H, 64).cuda(), kv.cuda(), k_pe.cuda())
    torch.cuda.synchronize()
    eng.check_status()
    _check("mla.o", o.view(B, H, 512).cpu(), torch.from_numpy(z["o"]), torch.float16)


@pytest.mark.parametrize("B,H,S,dtype,n_split", [
    (2, 128, 1024, torch.float16, None),   # benchmark head count, automatic split
    (3, 128, 333, torch.float16, 2),       # ragged kv length
    (1, 64, 2048, torch.bfloat16, 1),
    (4, 128, 4096, torch.float16, 1),
])
def test_mla_decode_against_oracle(B, H, S, dtype, n_split):
    """DeepSeek-V3 absorbed shape with the benchmark's scale 1/sqrt(192), honoured through score_mod."""
    scale = 1 / math.sqrt(192)
    q, q_pe, kv, k_pe = _mla_inputs(B, H, S, dtype, seed=S)
    eng = helpers.mla_engine(B, H, S, dtype, scale)
    eng._mla.num_split = n_split
    o = eng(q.cuda(), q_pe.cuda(), kv.cuda(), k_pe.cuda())
    torch.cuda.synchronize()
    eng.check_status()
    ref = orc.mla_decode(q[:, 0], q_pe[:, 0], kv, k_pe, scale=scale)
    _check("mla.o", o[:, 0].cpu(), ref, dtype)


# ---------------------------------------------------------------------------------------------------
# chunked linear attention / SSD scan (forward)
# ---------------------------------------------------------------------------------------------------
def test_linear_scan_against_fla_golden(golden_dir):
    """Plain gated linear attention (no mods) against flash-linear-attention's naive recurrence."""
    from attentionengine_b200 import LinearAttentionEngine, meta_tensor
    z = np.load(os.path.join(golden_dir, "linear_scan.npz"))
    q, k, v, a = (torch.from_numpy(z[n]) for n in ("q", "k", "v", "a"))
    B, H, T, DK = q.shape
    DV = v.shape[-1]
    dt = torch.bfloat16
    eng = LinearAttentionEngine((meta_tensor(B, H, T, DK, dtype=dt), meta_tensor(B, H, T, DK, dtype=dt),
                                 meta_tensor(B, H, T, DV, dtype=dt)))
    o = eng(q.to(dt).cuda(), k.to(dt).cuda(), v.to(dt).cuda(), a.cuda())
    torch.cuda.synchronize()
    eng.check_status()
    _check("linear.o", o.cpu(), torch.from_numpy(z["o"]), dt, unnormalised=True)


@pytest.mark.parametrize("B,H,T,DV", [(2, 4, 512, 64), (1, 3, 200, 64), (1, 2, 1024, 128)])
def test_mamba2_ssd_forward_against_oracle(B, H, T, DV, scan_groups):
    dt_ = torch.bfloat16
    x, dt, A, Bm, Cm = helpers.mamba2_inputs(B, H, T, 128, DV, dt_, seed=T)
    eng = helpers.mamba2_engine(B, H, T, 128, DV, dt_)
    o = eng(Cm.cuda(), Bm.cuda(), x.cuda(), dt.cuda(), A.view(1, H).cuda(), dt.to(dt_).cuda())
    torch.cuda.synchronize()
    eng.check_status()
    # the engine applies v_mod with the bf16 dt it was given and rounds v * dt to bf16, as the reference does
    from oracle.linear_oracle import linear_scan
    a = dt.double() * A.double().view(1, -1, 1)
    v_mod = (x.float() * dt.to(dt_).float()[..., None]).to(dt_)
    ref = linear_scan(Cm, Bm, v_mod, a)
    _check("ssd.o", o.cpu(), ref.float(), dt_, unnormalised=True)


@pytest.mark.parametrize("B,H,T", [(1, 2, 256), (2, 4, 512), (1, 3, 200), (1, 2, 64), (2, 1, 128), (1, 2, 129)])
def test_mamba2_ssd_backward_against_oracle(B, H, T, scan_groups):
    """Gradients of the Mamba2 mapping (q = C, k = B, v = x * dt, a = dt * A, one q/k head shared by all heads)
    against fp64 autograd through the step-by-step recurrence.  The tensor gradients follow the bf16 rule of
    tests/parity.py with four rounding stages (P / dS, v', the carried states, the stored result); the gradients of dt
    are asked rel-L2 <= 2e-2 and dA, a sum of B * T cancelling terms per head, 5e-2."""
    from oracle.linear_oracle import linear_scan
    dt_ = torch.bfloat16
    x, dt, A, Bm, Cm = helpers.mamba2_inputs(B, H, T, 128, 64, dt_, seed=T)
    g = torch.Generator().manual_seed(7)
    d_o = (0.1 * torch.randn(B, H, T, 64, generator=g)).to(dt_)
    eng = helpers.mamba2_engine(B, H, T, 128, 64, dt_)
    leaves = [t.cuda().requires_grad_() for t in (Cm, Bm, x, dt, A.view(1, H))]
    dtb = dt.to(dt_).cuda().requires_grad_()
    o = eng(*leaves, dtb)
    o.backward(d_o.cuda())
    torch.cuda.synchronize()
    eng.check_status()
    C2, B2, x2, dt2, A2, dtb2 = [t.detach().double().cpu().requires_grad_() for t in (*leaves, dtb)]
    oref = linear_scan(C2, B2, x2 * dtb2[..., None], dt2 * A2.view(1, H, 1))
    oref.backward(d_o.double())
    names = ("dC", "dB", "dx", "d(dt) via decay", "dA", "d(dt) via v_mod")
    for name, got, ref in zip(names, [t.grad for t in leaves] + [dtb.grad], [C2.grad, B2.grad, x2.grad, dt2.grad, A2.grad, dtb2.grad]):
        if name in ("dC", "dB", "dx"):
            parity.check(f"ssd T={T} {name}", got, ref, dt_, stages=4, unnormalised=True)
        else:  # fp32 sums of many cancelling bf16 terms (per step over 64 dims, per head over B * T steps)
            parity.check(f"ssd T={T} {name}", got, ref, dt_, rel_limit=5e-2 if name == "dA" else 2e-2)


@pytest.mark.parametrize("dt_", [torch.bfloat16, torch.float16])
def test_streaming_kernels_of_the_scan_against_torch(dt_):
    """The row-scale / skip / head-sum kernels of rowscale.cuh one by one (bit-exact where the arithmetic is a single
    rounding of an fp32 result, otherwise within one 16-bit rounding of the fp32 reference)."""
    B, H, T, D = 2, 6, 300, 64
    g = torch.Generator().manual_seed(31)
    x = torch.randn(B, H, T, D, generator=g).to(dt_).cuda()
    go = torch.randn(B, H, T, D, generator=g).to(dt_).cuda()
    gv = torch.randn(B, H, T, D, generator=g).to(dt_).cuda()
    s = torch.rand(B, H, T, generator=g).to(dt_).cuda()
    d = torch.randn(H, generator=g).cuda()
    eng = helpers.mamba2_engine(B, H, T, 128, D, dt_, d_skip=True)
    # y = x * s
    y = torch.empty_like(x)
    eng._rowscale("fwd", x, s, y=y)
    assert torch.equal(y, (x.float() * s.float()[..., None]).to(dt_))
    # both backward passes in one: gx = gv * s + go * d[h], gs = sum gv * x, rows = sum go * x
    gx, gs = torch.empty_like(x), torch.empty_like(s)
    rows = torch.empty(B, H, T, dtype=torch.float32, device="cuda")
    eng._rowscale("vskip_bwd", x, s, g=go, g2=gv, d=d, gx=gx, gs=gs, gs2=rows, rows_per_head=T, n_heads=H)
    ref_gx = gv.float() * s.float()[..., None] + go.float() * d.view(1, H, 1, 1)
    torch.testing.assert_close(gx.float(), ref_gx, rtol=1e-2, atol=1e-2)
    torch.testing.assert_close(gs.float(), (gv.float() * x.float()).sum(-1), rtol=1e-2, atol=6e-2)
    torch.testing.assert_close(rows, (go.float() * x.float()).sum(-1), rtol=1e-5, atol=1e-4)
    # the separate kernels give the same numbers
    gx1, gs1 = torch.empty_like(x), torch.empty_like(s)
    eng._rowscale("bwd", x, s, g=gv, gx=gx1, gs=gs1)
    gx2, rows2 = torch.empty_like(x), torch.empty_like(rows)
    eng._rowscale("skip_bwd", x, d, g=go, gx=gx2, gs=rows2, rows_per_head=T, n_heads=H)
    assert torch.equal(gs1, gs) and torch.equal(rows2, rows)
    torch.testing.assert_close(gx.float(), gx1.float() + gx2.float(), rtol=1e-2, atol=2e-2)
    # head sums: [B, H, T, D] -> [B, n_out, T, D]
    for n_out in (1, 2, 3):
        got = eng._head_sum(x, n_out)
        ref = x.view(B, n_out, H // n_out, T, D).float().sum(2).to(dt_)
        assert torch.equal(got, ref), n_out


def test_scan_forward_with_the_block_mods_inside_against_the_separate_kernels(scan_groups):
    """y = scan(q, k, x * s, a) + x * d[h] from the kernel built with the mods inside, its v_out and its chunk states
    against the same engine's plain scan on the row-scaled input and the separate skip kernel."""
    B, H, T, dt_ = 2, 4, 456, torch.bfloat16
    x, dt, A, Bm, Cm = helpers.mamba2_inputs(B, H, T, 128, 64, dt_, seed=13)
    eng = helpers.mamba2_engine(B, H, T, 128, 64, dt_, d_skip=True)
    q, k, xc = Cm.cuda(), Bm.cuda(), x.cuda()
    s = dt.to(dt_).cuda()
    a = (dt * A.view(1, H, 1)).float().cuda()
    d = torch.randn(H, generator=torch.Generator().manual_seed(14)).cuda()
    v = torch.empty_like(xc)
    eng._rowscale("fwd", xc, s, y=v)
    hs_ref = eng._new_states(v)
    o = eng._launch(q, k, v, a, h_out=hs_ref)
    y_ref = torch.empty_like(o)
    eng._rowscale("skip_fwd", xc, d, g=o, y=y_ref, rows_per_head=T, n_heads=H)
    v_out, hs = torch.empty_like(xc), eng._new_states(xc)
    y = eng._launch(q, k, xc, a, vscale=s, dskip=d, v_out=v_out, h_out=hs)
    torch.cuda.synchronize()
    eng.check_status()
    assert torch.equal(v_out, v) and torch.equal(hs, hs_ref)
    # the fused kernel adds the skip term to the fp32 accumulator, the separate kernel to the stored 16-bit output
    torch.testing.assert_close(y.float(), y_ref.float(), rtol=2e-2, atol=2e-2 * y_ref.float().abs().max().item())
    # fp32 row scales take the other load path
    y32 = eng._launch(q, k, xc, a, vscale=s.float(), dskip=d)
    assert torch.equal(y32, y)


def test_scan_states_from_the_forward_equal_the_recompute_pass():
    """The chunk start-states the forward writes for the backward are the ones ae_linear_states recomputes, and the
    reverse pass gives the same gradients from either (T not a multiple of the chunk, several heads per q / k head)."""
    B, H, T, dt_ = 2, 4, 456, torch.bfloat16
    x, dt, A, Bm, Cm = helpers.mamba2_inputs(B, H, T, 128, 64, dt_, seed=11)
    g = torch.Generator().manual_seed(12)
    d_o = (0.1 * torch.randn(B, H, T, 64, generator=g)).to(dt_).cuda()
    eng = helpers.mamba2_engine(B, H, T, 128, 64, dt_)
    q, k, v = Cm.cuda(), Bm.cuda(), (x.float() * dt[..., None]).to(dt_).cuda()
    a = (dt * A.view(1, H, 1)).float().cuda()
    hs = eng._new_states(v)
    o = eng._launch(q, k, v, a, h_out=hs)
    with_saved = eng._launch_bwd(q, k, v, a, d_o, hs=hs)
    recomputed = eng._launch_bwd(q, k, v, a, d_o, hs=None)
    torch.cuda.synchronize()
    eng.check_status()
    assert torch.equal(o, eng._launch(q, k, v, a))  # writing the states does not change the output
    for name, x1, x2 in zip(("dq", "dk", "dv", "da"), with_saved, recomputed):
        assert torch.equal(x1, x2), name


@pytest.mark.parametrize("T,s_dtype", [(456, torch.bfloat16), (128, torch.float32), (1000, torch.bfloat16)])
def test_scan_reverse_pass_with_the_block_mods_inside_against_the_separate_kernels(T, s_dtype, scan_groups):
    """The reverse pass built with v = x * s and the skip term inside (it writes the gradient of x where dv went, the
    row sums <dv, x> for s and <dO, x> per (batch, head) for the skip weight) against the plain reverse pass followed
    by the streaming kernel: the gradient of x bit for bit (same inputs, same arithmetic per element), the sums within
    fp32 summation-order noise (and one 16-bit rounding where s is 16-bit)."""
    B, H, dt_ = 2, 3, torch.bfloat16
    x, dt, A, Bm, Cm = helpers.mamba2_inputs(B, H, T, 128, 64, dt_, seed=T)
    eng = helpers.mamba2_engine(B, H, T, 128, 64, dt_, d_skip=True)
    q, k, xc = Cm.cuda(), Bm.cuda(), x.cuda()
    s = dt.to(s_dtype).cuda()
    a = (dt * A.view(1, H, 1)).float().cuda()
    d = torch.randn(H, generator=torch.Generator().manual_seed(15)).cuda()
    d_o = (0.1 * torch.randn(B, H, T, 64, generator=torch.Generator().manual_seed(16))).to(dt_).cuda()
    v, hs = torch.empty_like(xc), eng._new_states(xc)
    eng._launch(q, k, xc, a, vscale=s, dskip=d, v_out=v, h_out=hs)
    dq, dk, dv, da = eng._launch_bwd(q, k, v, a, d_o, hs=hs)
    gx, gs = torch.empty_like(xc), torch.empty_like(s)
    rows = torch.empty(B, H, T, dtype=torch.float32, device="cuda")
    eng._rowscale("vskip_bwd", xc, s, g=d_o, g2=dv, d=d, gx=gx, gs=gs, gs2=rows, rows_per_head=T, n_heads=H)
    fdq, fdk, fgx, fda, fgs, fgd = eng._launch_bwd(q, k, v, a, d_o, hs=hs, mods=(xc, s, d))
    torch.cuda.synchronize()
    eng.check_status()
    for name, x1, x2 in (("dq", fdq, dq), ("dk", fdk, dk), ("gx", fgx, gx), ("da", fda, da)):
        assert torch.equal(x1, x2), name
    assert fgs.dtype == s.dtype and fgd.shape == (B, H)
    scale = gs.float().abs().max().item()
    tol = 2e-5 * scale if s_dtype == torch.float32 else 1e-2 * scale  # 16-bit: a sum on a rounding edge moves one ulp
    assert (fgs.float() - gs.float()).abs().max().item() <= tol
    ref_gd = rows.double().sum(dim=2)
    assert (fgd.double() - ref_gd).abs().max().item() <= 1e-4 * ref_gd.abs().max().item() + 1e-4


@pytest.mark.parametrize("T", [456, 128, 1000])
def test_decay_scale_inside_the_scan_kernels_against_the_eager_mod(T, monkeypatch):
    """Mamba2's ``decay_mod = decay * A[heads]`` taken into the scan kernels (the forward scales the log-decay where it
    uses it, the reverse pass returns the gradient of the decay as passed and the per-head sums for A) against the same
    engine with the mod run as eager PyTorch: output and every tensor gradient bit for bit (the same fp32 products feed
    the same kernels), the gradient of A within fp32 summation-order noise."""
    from attentionengine_b200.attn_engine import linear_attn_engine as le
    B, H, dt_ = 2, 3, torch.bfloat16
    x, dt, A, Bm, Cm = helpers.mamba2_inputs(B, H, T, 128, 64, dt_, seed=T + 1)
    Dk = torch.randn(1, H, generator=torch.Generator().manual_seed(17))
    d_o = (0.1 * torch.randn(B, H, T, 64, generator=torch.Generator().manual_seed(18))).to(dt_).cuda()

    def run(inside):
        monkeypatch.setattr(le, "LIN_DECAY_SCALE", inside)
        eng = helpers.mamba2_engine(B, H, T, 128, 64, dt_, d_skip=True)
        leaves = [t.cuda().requires_grad_() for t in (Cm, Bm, x, dt, A.view(1, H), dt.to(dt_), Dk)]
        y = eng(*leaves)
        y.backward(d_o)
        torch.cuda.synchronize()
        eng.check_status()
        return y.detach(), [t.grad for t in leaves]

    y1, g1 = run(1)
    y0, g0 = run(0)
    assert torch.equal(y1, y0)
    for name, a1, a0 in zip(("dC", "dB", "dx", "d(dt) through the decay", "dA", "d(dt) through v", "dD"), g1, g0):
        if name == "dA":
            assert (a1 - a0).abs().max().item() <= 1e-4 * a0.abs().max().item() + 1e-6, name
        else:
            assert torch.equal(a1, a0), name


@pytest.mark.parametrize("kind", ["softmax", "sigmoid"])
@pytest.mark.parametrize("parts", [2, 4])
def test_attention_backward_in_batch_ranges_on_side_streams(parts, kind, monkeypatch):
    """The one-pass attention backward launched as batch ranges on streams of their own (what the engine does at sizes
    where a range still fills the SMs several times over) against one launch: dK and dV bit for bit, dQ within the
    order noise of its fp32 accumulation.  The sigmoid case carries a custom tensor that has no batch index (the
    scalar bias), which travels with every range."""
    from attentionengine_b200.attn_engine import attn_bwd as ab
    B, Hq, Hkv, S, D = 4, 4, 2, 384, 64
    g = torch.Generator().manual_seed(40 + parts)
    if kind == "softmax":
        dtype = torch.float16
        eng, custom = helpers.softmax_engine(B, Hq, Hkv, S, D, D, dtype, True), ()
    else:
        dtype, Hkv = torch.bfloat16, Hq
        eng, custom = helpers.sigmoid_engine(B, Hq, S, D, dtype, False), (torch.tensor([-math.log(S)], device="cuda"),)
    q, k, v, d_o = (torch.randn(B, S, h, D, generator=g).to(dtype).cuda() for h in (Hq, Hkv, Hkv, Hq))
    eng.bwd_mode = "fused"

    def run(n):
        monkeypatch.setattr(ab, "_batch_parts", lambda B_, Hq_, Sq_, dev: n)
        leaves = [t.clone().requires_grad_() for t in (q, k, v)]
        for _ in range(2):
            for t in leaves:
                t.grad = None
            eng(*leaves, *custom).backward(d_o)
        torch.cuda.synchronize()
        eng.check_status()
        return [t.grad for t in leaves]

    one, split = run(1), run(parts)
    assert torch.equal(split[1], one[1]) and torch.equal(split[2], one[2])
    assert (split[0].float() - one[0].float()).abs().max().item() <= 2e-3 * one[0].float().abs().max().item()


@pytest.mark.parametrize("parts", [2, 4])
def test_reverse_pass_in_batch_ranges_on_side_streams_equals_one_launch(parts, monkeypatch):
    """The reverse pass split into batch ranges, each on a stream of its own with its head sums behind it (what the
    engine does at sizes where a range still fills the SMs), against one launch: every gradient bit for bit - a
    (batch, head) CTA does the same work either way - also when the caller's stream is not the default one."""
    from attentionengine_b200.attn_engine import linear_attn_engine as le
    B, H, T, dt_ = 4, 2, 300, torch.bfloat16
    x, dt, A, Bm, Cm = helpers.mamba2_inputs(B, H, T, 128, 64, dt_, seed=parts)
    Dk = torch.randn(1, H, generator=torch.Generator().manual_seed(19))
    d_o = (0.1 * torch.randn(B, H, T, 64, generator=torch.Generator().manual_seed(20))).to(dt_).cuda()

    def run(n, stream):
        monkeypatch.setattr(le.LinearAttentionEngine, "_bwd_batch_parts", lambda self, B_, H_, dev: n)
        eng = helpers.mamba2_engine(B, H, T, 128, 64, dt_, d_skip=True)
        leaves = [t.cuda().requires_grad_() for t in (Cm, Bm, x, dt, A.view(1, H), dt.to(dt_), Dk)]
        torch.cuda.synchronize()
        with torch.cuda.stream(stream):
            for _ in range(2):  # the second call reuses the engine's side streams and events
                for t in leaves:
                    t.grad = None
                eng(*leaves).backward(d_o)
        torch.cuda.synchronize()
        eng.check_status()
        return [t.grad for t in leaves]

    one = run(1, torch.cuda.current_stream())
    split = run(parts, torch.cuda.Stream())
    for name, a1, a0 in zip(("dC", "dB", "dx", "d(dt) through the decay", "dA", "d(dt) through v", "dD"), split, one):
        assert torch.equal(a1, a0), name


@pytest.mark.parametrize("n_split", [None, 1, 3])
def test_mla_decode_paged_kv_with_ragged_lengths(n_split):
    """The call of the reference's CuTe kv-shared path (flash_mla_interface.py:73-113): a pool of 64-key pages in
    shuffled order, a block table per batch row, one length per row (one row a single key, one exactly full pages, one
    shorter than the splits reach).  Output and log-sum-exp per row against the oracle on that row's gathered keys."""
    B, H, dtype, scale = 4, 128, torch.float16, 1 / math.sqrt(192)
    lens = [1, 640, 1000, 130]
    max_pages = 16
    g = torch.Generator().manual_seed(70)
    n_pages = B * max_pages + 3
    kcache = torch.randn(n_pages, 64, 1, 576, generator=g).to(dtype)
    perm = torch.randperm(n_pages, generator=g)[:B * max_pages].to(torch.int32).view(B, max_pages)
    q = torch.randn(B, 1, H, 576, generator=g).to(dtype)
    eng = helpers.mla_engine(B, H, max_pages * 64, dtype, scale)
    o, lse = eng.decode_paged(q.cuda(), kcache.cuda(), perm.cuda(), torch.tensor(lens, dtype=torch.int32).cuda(),
                              num_split=n_split)
    torch.cuda.synchronize()
    eng.check_status()
    if n_split:
        assert eng._mla.last_num_split == n_split
    for b, L in enumerate(lens):
        rows = kcache[perm[b].long(), :, 0].reshape(-1, 576)[:L]          # [L, 576] in logical order
        ro, rl = orc.mla_decode(q[b:b + 1, 0, :, :512], q[b:b + 1, 0, :, 512:], rows[None, :, None, :512],
                                rows[None, :, None, 512:], scale=scale, return_lse=True)
        _check(f"row {b} o", o[b:b + 1, 0].cpu(), ro, dtype)
        assert (lse[b].cpu() - rl[0]).abs().max().item() <= 2e-3, f"row {b} lse"


def test_mla_two_argument_call_reads_the_cache_in_batch_order():
    """mod(q, kcache) as in attn_script/mla_decode_cute.py:295-303: pages of a batch row are consecutive, rows full."""
    B, H, S, dtype, scale = 2, 64, 512, torch.bfloat16, 1 / math.sqrt(576)
    g = torch.Generator().manual_seed(71)
    kcache = torch.randn(B * S // 64, 64, 1, 576, generator=g).to(dtype)
    q = torch.randn(B, 1, H, 576, generator=g).to(dtype)
    eng = helpers.mla_engine(B, H, S, dtype, scale)
    o, lse = eng(q.cuda(), kcache.cuda())
    torch.cuda.synchronize()
    eng.check_status()
    kv = kcache.view(B, S, 1, 576)
    ro, rl = orc.mla_decode(q[:, 0, :, :512], q[:, 0, :, 512:], kv[..., :512], kv[..., 512:], scale=scale, return_lse=True)
    _check("o", o[:, 0].cpu(), ro, dtype)
    assert (lse.cpu() - rl).abs().max().item() <= 2e-2


@pytest.mark.parametrize("variant", ["simple_gla", "retention_linear"])
def test_linear_variants_with_large_heads(variant):
    """attn_script/simple_gla.py (q_mod = q * scale, the decay input is already a log-decay) and retention_linear.py
    (decay_mod = log of a per-head decay factor) at their head sizes class: D = 256 (two key blocks, summed) and
    DV = 256 (value blocks as extra heads).  Forward without gradients (128-wide value blocks) and forward + backward
    (64-wide value blocks) against fp64 autograd through the step-by-step recurrence; bf16 protocol as for the SSD
    backward test."""
    from attentionengine_b200 import LinearAttentionEngine, meta_tensor
    from oracle.linear_oracle import linear_scan
    B, H, T, D, DV, dt_ = 1, 2, 384, 256, 256, torch.bfloat16
    scale = 1 / math.sqrt(D)
    metas = (meta_tensor(B, H, T, D, dtype=dt_), meta_tensor(B, H, T, D, dtype=dt_), meta_tensor(B, H, T, DV, dtype=dt_))
    mods = {"q_mod": lambda q, io: q * scale}
    g = torch.Generator().manual_seed(60)
    if variant == "retention_linear":
        mods["decay_mod"] = lambda decay, io: decay.log()
        decay = (1 - torch.exp2(-5 - torch.arange(H, dtype=torch.float32))).view(1, H, 1).expand(B, H, T).contiguous()
        to_log = torch.log
    else:
        decay = torch.nn.functional.logsigmoid(torch.randn(B, H, T, generator=g)) / 16
        to_log = lambda x: x  # noqa: E731
    eng = LinearAttentionEngine(metas, custom_io=CustomIO({}), **mods)
    q, k = (torch.randn(B, H, T, D, generator=g).to(dt_) for _ in range(2))
    v = torch.randn(B, H, T, DV, generator=g).to(dt_)
    d_o = (0.1 * torch.randn(B, H, T, DV, generator=g)).to(dt_)

    with torch.no_grad():
        o_ng = eng(q.cuda(), k.cuda(), v.cuda(), decay.cuda())
    leaves = [t.cuda().requires_grad_() for t in (q, k, v, decay)]
    o = eng(*leaves)
    o.backward(d_o.cuda())
    torch.cuda.synchronize()
    eng.check_status()

    q2, k2, v2, g2 = [t.detach().double().cpu().requires_grad_() for t in leaves]
    # the engine rounds the mod-ed q to bf16 before the scan: the rounded value, with the gradient of the exact product
    q_round = (q2 * scale).detach().to(dt_).double()
    oref = linear_scan(q_round + (q2 * scale - (q2 * scale).detach()), k2, v2, to_log(g2))
    oref.backward(d_o.double())
    _check("o (no grad, 128-wide value blocks)", o_ng.cpu(), oref.detach().float(), dt_, unnormalised=True)
    _check("o", o.detach().cpu(), oref.detach().float(), dt_, unnormalised=True)
    for name, got, ref in zip(("dq", "dk", "dv", "d(decay)"), [t.grad for t in leaves], [q2.grad, k2.grad, v2.grad, g2.grad]):
        if name == "d(decay)":
            parity.check(f"{variant} {name}", got, ref, dt_, rel_limit=5e-2)
        else:  # two key blocks are summed in fp32 and stored once more -> one stage on top of the scan's four
            parity.check(f"{variant} {name}", got, ref, dt_, stages=5, unnormalised=True)


@pytest.mark.parametrize("D", [64, 128])
def test_extern_block_mask_given_at_call_time(D):
    """attn_script/blocksparseattn.py: the engine is built with extern_block_mask=True and no mask_mod, the int8 block
    mask [B, H, S/128, S/128] arrives with the call; listed blocks are complete blocks.  Forward and gradients
    against dense softmax attention under the expanded mask."""
    B, H, S, dtype = 1, 2, 640, torch.float16
    g = torch.Generator().manual_seed(5)
    n = S // 128
    bm = (torch.rand(B, H, n, n, generator=g) < 0.5)
    bm |= torch.eye(n, dtype=torch.bool)          # no empty row: a row without blocks is 0 / 0 in the softmax epilogue
    scale = 1.0 / math.sqrt(D)
    eng = AttentionEngine(helpers.metas(B, H, H, S, D, D, dtype), CustomIO({}),
                          score_mod=lambda s, c, b, h, q, kv: s * scale, mask_mod=None,
                          online_func=helpers.OnlineSoftmax(), extern_block_mask=True)
    q, k, v, d_o = helpers.seeded_qkv(B, H, H, S, D, D, dtype, seed=31)
    qd, kd, vd = (t.cuda().requires_grad_() for t in (q, k, v))
    o = eng(qd, kd, vd, block_mask=bm.to(torch.int8).cuda())
    o.backward(d_o.cuda())
    torch.cuda.synchronize()
    eng.check_status()
    dense = bm.repeat_interleave(128, 2).repeat_interleave(128, 3)  # [B, H, S, S]

    def ref(a, b_, c):
        s_ = torch.einsum("bqhd,bkhd->bhqk", a, b_) * scale
        s_ = s_.masked_fill(~dense, float("-inf"))
        p = torch.softmax(s_, -1)
        p = torch.nan_to_num(p, nan=0.0)               # rows with no block at all
        return torch.einsum("bhqk,bkhd->bqhd", p, c)

    ro, (rq, rk, rv) = orc.fwd_bwd(ref, (q, k, v), d_o)
    for name, got, r in zip(("o", "dq", "dk", "dv"), (o, qd.grad, kd.grad, vd.grad), (ro, rq, rk, rv)):
        _check(name, got.detach().cpu(), r, dtype)


@pytest.mark.gpu
def test_element_mask_without_block_inference(fwd_form):
    """infer_mask=False: every tile is visited and masked element by element (mask mode 3); a banded mask that the
    block inference would have turned into tile lists."""
    B, H, S, D, dtype, W = 1, 2, 384, 64, torch.float16, 100
    scale = 1.0 / math.sqrt(D)
    band = lambda b, h, q_idx, kv_idx: torch.logical_and(q_idx >= kv_idx, q_idx - kv_idx < W)  # noqa: E731
    eng = AttentionEngine(helpers.metas(B, H, H, S, D, D, dtype), CustomIO({}),
                          score_mod=lambda s, c, b, h, q, kv: s * scale, mask_mod=band,
                          online_func=helpers.OnlineSoftmax(), infer_mask=False)
    assert eng.mask_mode == 3
    q, k, v, d_o = helpers.seeded_qkv(B, H, H, S, D, D, dtype, seed=32)
    got = _run(eng, q, k, v, d_o)
    i = torch.arange(S)
    keep = (i[:, None] >= i[None, :]) & (i[:, None] - i[None, :] < W)

    def ref(a, b_, c):
        s_ = torch.einsum("bqhd,bkhd->bhqk", a, b_) * scale
        return torch.einsum("bhqk,bkhd->bqhd", torch.softmax(s_.masked_fill(~keep, float("-inf")), -1), c)

    ro, grads = orc.fwd_bwd(ref, (q, k, v), d_o)
    for name, g_, r in zip(("o", "dq", "dk", "dv"), got, (ro,) + tuple(grads)):
        _check(name, g_, r, dtype)


@pytest.mark.gpu
@pytest.mark.parametrize("S,causal", [(384, True), (200, False)])
def test_softcap_score_mod_keeps_the_raw_score_for_the_backward(S, causal, fwd_form):
    """score_mod = cap * tanh(score * scale / cap): its derivative needs the raw score again, so the backward passes
    keep it next to P between their two row phases (the autodiff of Tanh is the reference's, core.py:129-195)."""
    B, Hq, Hkv, D, dtype, cap = 1, 4, 2, 128, torch.float16, 20.0
    scale = 1.0 / math.sqrt(D)

    def score_mod(score, custom_fwd_inputs, b, h, q_idx, kv_idx):
        return (score * (scale / cap)).tanh() * cap

    eng = AttentionEngine(helpers.metas(B, Hq, Hkv, S, D, D, dtype), CustomIO({}), score_mod=score_mod,
                          mask_mod=helpers.causal_mask if causal else None, online_func=helpers.OnlineSoftmax())
    assert eng.lowered.defines["AE_DS_USES_S"] == 1
    q, k, v, d_o = helpers.seeded_qkv(B, Hq, Hkv, S, D, D, dtype, seed=77)
    q = q * 3.0  # scores large enough for the cap to bend them
    got = _run(eng, q, k, v, d_o)

    def ref(a, b_, c):
        g = Hq // Hkv
        s = torch.einsum("bqhd,bkhd->bhqk", a, b_.repeat_interleave(g, dim=2)) * scale
        s = torch.tanh(s / cap) * cap
        if causal:
            i = torch.arange(S)
            s = s.masked_fill(i[:, None] < i[None, :], float("-inf"))
        return torch.einsum("bhqk,bkhd->bqhd", torch.softmax(s, -1), c.repeat_interleave(g, dim=2))

    o, (dq, dk, dv) = orc.fwd_bwd(ref, (q, k, v), d_o)
    for name, g_, r in zip(("o", "dq", "dk", "dv"), got, (o, dq, dk, dv)):
        _check(name, g_, r, dtype)


@pytest.mark.gpu
@pytest.mark.parametrize("S", [256, 384])
def test_retention_parallel_with_tile_shaped_custom_input(S, fwd_form):
    """attn_script/retention.py: score * decay mask (custom input [1, H, S, S] in the input dtype), rows normalised by
    max(sum |.|, 1); forward and the three gradients against the oracle (bench_utils.py:1062-1067)."""
    B, H, D, DV, dtype = 1, 2, 128, 128, torch.float16
    q, k, v, d_o = helpers.seeded_qkv(B, H, H, S, D, DV, dtype, seed=21)
    q, k = q * 0.25, k * 0.25
    idx = torch.arange(S)
    gamma = 1.0 - 2.0 ** (-5.0 - torch.arange(H, dtype=torch.float32))
    dist = (idx[:, None] - idx[None, :]).clamp(min=0).float()
    mask = (gamma.view(H, 1, 1) ** dist) * (idx[:, None] >= idx[None, :])
    mask = mask.view(1, H, S, S).to(dtype)
    eng = helpers.retention_engine(B, H, S, D, DV, dtype)
    qd, kd, vd = (t.cuda().requires_grad_() for t in (q, k, v))
    o = eng(qd, kd, vd, mask.cuda())
    o.backward(d_o.cuda())
    torch.cuda.synchronize()
    eng.check_status()
    ro, (rq, rk, rv) = orc.fwd_bwd(lambda a, b, c: orc.retention_parallel(a, b, c, mask), (q, k, v), d_o)
    for name, g, r in zip(("o", "dq", "dk", "dv"), (o, qd.grad, kd.grad, vd.grad), (ro, rq, rk, rv)):
        _check(name, g.detach().cpu(), r, dtype)




def test_backward_uses_the_block_mask_of_its_own_forward():
    """Two forward calls with different call-time block masks, then both backward calls: each gradient must follow the
    mask its own forward walked, not the one the engine saw last."""
    B, H, S, D, dtype = 1, 2, 512, 64, torch.float16
    n = S // 128
    scale = 1.0 / math.sqrt(D)
    eng = AttentionEngine(helpers.metas(B, H, H, S, D, D, dtype), CustomIO({}),
                          score_mod=lambda s, c, b, h, q, kv: s * scale, mask_mod=None,
                          online_func=helpers.OnlineSoftmax(), extern_block_mask=True)
    g = torch.Generator().manual_seed(8)
    masks = [torch.eye(n, dtype=torch.bool).expand(B, H, n, n) | (torch.rand(B, H, n, n, generator=g) < p) for p in (0.3, 0.7)]
    q, k, v, d_o = helpers.seeded_qkv(B, H, H, S, D, D, dtype, seed=33)
    runs = []
    for bm in masks:
        leaves = [t.cuda().requires_grad_() for t in (q, k, v)]
        runs.append((leaves, eng(*leaves, block_mask=bm.to(torch.int8).cuda())))
    for leaves, o in runs:          # backward calls only after both forwards
        o.backward(d_o.cuda())
    torch.cuda.synchronize()
    eng.check_status()
    for bm, (leaves, o) in zip(masks, runs):
        dense = bm.repeat_interleave(128, 2).repeat_interleave(128, 3)

        def ref(a, b_, c):
            s_ = (torch.einsum("bqhd,bkhd->bhqk", a, b_) * scale).masked_fill(~dense, float("-inf"))
            return torch.einsum("bhqk,bkhd->bqhd", torch.softmax(s_, -1), c)

        ro, grads = orc.fwd_bwd(ref, (q, k, v), d_o)
        for name, got, r in zip(("o", "dq", "dk", "dv"), (o, *[t.grad for t in leaves]), (ro, *grads)):
            _check(name, got.detach().cpu(), r, dtype)


# ---------------------------------------------------------------------------------------------------
# split-KV decode: rows of different lengths, paged K / V, mask
# ---------------------------------------------------------------------------------------------------
def _ragged_ref(q, k, v, lens, keep=None):
    outs = []
    for b, L in enumerate(lens):
        qb, kb, vb = q[b:b + 1].float(), k[b:b + 1, :L].float(), v[b:b + 1, :L].float()
        g = qb.shape[2] // kb.shape[2]
        s = torch.einsum("bqhd,bkhd->bhqk", qb, kb.repeat_interleave(g, 2)) / math.sqrt(qb.shape[-1])
        if keep is not None:
            s = s.masked_fill(~keep(L), float("-inf"))
        outs.append(torch.einsum("bhqk,bkhd->bqhd", torch.softmax(s, -1), vb.repeat_interleave(g, 2)))
    return torch.cat(outs)


@pytest.mark.parametrize("paged", [False, True])
def test_gqa_decode_rows_of_different_lengths(paged, bwd_mode):
    """Lengths from one key to 4000 in one batch: the schedule gives long rows several shares and short rows one;
    dense K / V [B, S_max, ...] or a shuffled pool of 128-key pages with a block table."""
    if bwd_mode == "fused":
        pytest.skip("forward only")
    B, Hq, Hkv, D, dtype = 5, 32, 8, 128, torch.float16
    lens = [1, 4000, 129, 1000, 2048]
    S_max = 4096
    eng = helpers.decode_engine("B", Hq, Hkv, 1, "S_kv", D, dtype)
    g = torch.Generator().manual_seed(90)
    q = torch.randn(B, 1, Hq, D, generator=g).to(dtype)
    k = torch.randn(B, S_max, Hkv, D, generator=g).to(dtype)
    v = torch.randn(B, S_max, Hkv, D, generator=g).to(dtype)
    meta = eng.decode_schedule(torch.tensor(lens), device="cuda")
    assert meta["n_slots"] > B and int(meta["part_off"][2] - meta["part_off"][1]) > 1
    if paged:
        n_pages = B * (S_max // 128)
        perm = torch.randperm(n_pages, generator=g)
        table = perm.view(B, S_max // 128).to(torch.int32)
        kp = torch.empty(n_pages, 128, Hkv, D, dtype=dtype)
        vp = torch.empty(n_pages, 128, Hkv, D, dtype=dtype)
        kp[perm] = k.view(n_pages, 128, Hkv, D)
        vp[perm] = v.view(n_pages, 128, Hkv, D)
        o = eng.decode_varlen(q.cuda(), kp.cuda(), vp.cuda(), None, block_table=table.cuda(), metadata=meta)
    else:
        o = eng.decode_varlen(q.cuda(), k.cuda(), v.cuda(), None, metadata=meta)
    torch.cuda.synchronize()
    eng.check_status()
    _check("o", o.cpu(), _ragged_ref(q, k, v, lens), dtype)


def test_mha_decode_with_a_mask_and_ragged_rows(bwd_mode):
    """mha_inference.py shape class (Hq == Hkv, several query positions) with a mask_mod applied element by element:
    a sliding window over the keys, rows of different lengths."""
    if bwd_mode == "fused":
        pytest.skip("forward only")
    B, H, Sq, D, dtype, W = 3, 4, 3, 64, torch.bfloat16, 300
    lens = [700, 77, 1500]
    scale = 1 / math.sqrt(D)
    metas = (helpers.meta_tensor(B, H, Sq, D, dtype=dtype), helpers.meta_tensor(B, H, 2048, D, dtype=dtype),
             helpers.meta_tensor(B, H, 2048, D, dtype=dtype))
    eng = AttentionEngine(metas, CustomIO({}), score_mod=lambda s, c, b, h, q, kv: s * scale,
                          mask_mod=lambda b, h, q_idx, kv_idx: kv_idx % 512 < W, online_func=helpers.OnlineSoftmaxSplit())
    g = torch.Generator().manual_seed(91)
    q = torch.randn(B, Sq, H, D, generator=g).to(dtype)
    k = torch.randn(B, 2048, H, D, generator=g).to(dtype)
    v = torch.randn(B, 2048, H, D, generator=g).to(dtype)
    o = eng.decode_varlen(q.cuda(), k.cuda(), v.cuda(), torch.tensor(lens))
    torch.cuda.synchronize()
    eng.check_status()
    keep = lambda L: (torch.arange(L) % 512 < W).view(1, 1, 1, L)  # noqa: E731
    _check("o", o.cpu(), _ragged_ref(q, k, v, lens, keep), dtype)
    # the same engine, one length for all rows, through the plain call
    o2 = eng(q.cuda(), k.cuda(), v.cuda())
    torch.cuda.synchronize()
    _check("o", o2.cpu(), _ragged_ref(q, k, v, [2048] * B, keep), dtype)


def test_value_head_dim_above_128_runs_as_value_blocks():
    """DV = 256 with D = 128: two 128-wide value blocks through the same kernels, dQ / dK summed over the blocks."""
    B, Hq, Hkv, S, D, DV, dtype = 1, 4, 2, 384, 128, 256, torch.float16
    eng = helpers.softmax_engine(B, Hq, Hkv, S, D, DV, dtype, True)
    q, k, v, d_o = helpers.seeded_qkv(B, Hq, Hkv, S, D, DV, dtype, seed=17)
    got = _run(eng, q, k, v, d_o)
    assert got[0].shape == (B, S, Hq, DV)
    o, (dq, dk, dv) = orc.fwd_bwd(lambda a, b, c: orc.softmax_attention(a, b, c, True), (q, k, v), d_o)
    for name, g, r in zip(("o", "dq", "dk", "dv"), got, (o, dq, dk, dv)):
        _check(name, g, r, dtype)
