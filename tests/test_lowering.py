"""Host-side logic: tracing, mask classification, lowering to CUDA functors, NVRTC compile (no GPU)."""
import math

import pytest
import torch

import attentionengine_b200 as ae
from attentionengine_b200 import AttentionEngine, CustomIO, meta_tensor
from attentionengine_b200.lower.cuda_lower import lower_attention

import helpers


def test_softmax_lowering_has_expected_pieces():
    eng = helpers.softmax_engine(1, 4, 4, 512, 64, 64, torch.float16, True)
    low = eng.lowered
    assert eng.mask_mode == 1 and low.final_names == ["lse"] and low.uses_doosum and not low.o_scale_one
    for piece in ("struct AeRow", "ae_score_mod", "ae_online_fwd", "ae_epilogue_o", "ae_final_rowscales",
                  "ae_bwd_p", "ae_bwd_ds", "st_m = -1e38f"):
        assert piece in low.prelude_bwd
    assert "(q_idx >= kv_idx)" in low.prelude_fwd
    assert eng.tl_code.count("tcgen05.mma") >= 2 and "cp.async.bulk.tensor" in eng.tl_code


def test_identity_online_func_needs_no_rescale_and_no_delta():
    eng = helpers.relu_engine(1, 2, 256, 64, torch.float16)
    assert eng.lowered.o_scale_one and not eng.lowered.uses_doosum and eng.lowered.final_names == []
    assert eng.mask_mode == 0


def test_custom_input_binding():
    eng = helpers.sigmoid_engine(1, 2, 256, 128, torch.bfloat16, True)
    (spec,) = eng.lowered.custom
    assert spec.name == "softmax_bias" and not spec.is_16bit and spec.dim_slots == [-1]
    assert "((const float*)cu.p[0])[0]" in eng.lowered.prelude_fwd
    assert "ae_tanh" in eng.lowered.prelude_fwd


def test_mask_classification():
    D = 64

    def sm(score, c, b, h, q, kv):
        return score * 0.125

    def mk(mask, **kw):
        return AttentionEngine(helpers.metas(1, 2, 2, 512, D, D, torch.float16), CustomIO({}), score_mod=sm,
                               mask_mod=mask, online_func=helpers.OnlineSoftmax(), **kw)

    assert mk(None).mask_mode == 0
    assert mk(lambda b, h, q, kv: q >= kv).mask_mode == 1
    assert mk(lambda b, h, q, kv: q >= kv + 128).mask_mode == 2
    assert mk(lambda b, h, q, kv: q >= kv, infer_mask=False).mask_mode == 3
    always = mk(lambda b, h, q, kv: q + kv >= 0)
    assert always.mask_mode == 0
    e = mk(lambda b, h, q, kv: torch.logical_and(q >= kv, q - kv <= 100))
    assert e.mask_mode == 2 and e.block_mask.shape == (1, 2, 4, 4)
    assert "&&" in e.lowered.prelude_fwd


def test_dynamic_shape_engine_classifies_on_a_probe_and_builds_lists_per_shape():
    """meta_tensor with named dims (reference: attn_script/mha.py:92-94, lower.py:626-629): one engine for every
    batch / length; the mask is classified once, the tile lists are built per runtime shape."""
    from attentionengine_b200 import meta_tensor
    D = 64
    metas = tuple(meta_tensor("B", "H", "S", D, dtype=torch.float16) for _ in range(3))

    def mk(mask):
        return AttentionEngine(metas, CustomIO({}), score_mod=lambda s, c, b, h, q, kv: s * 0.125, mask_mod=mask,
                               online_func=helpers.OnlineSoftmax())

    assert mk(None).mask_mode == 0
    assert mk(lambda b, h, q, kv: q >= kv).mask_mode == 1
    e = mk(lambda b, h, q, kv: torch.logical_and(q >= kv, q - kv <= 100))
    assert e.mask_mode == 2
    c1 = e._ensure_lists("cpu", None, 1, 2, 256, 256)[0]
    c2 = e._ensure_lists("cpu", None, 2, 2, 640, 640)[0]
    assert c1.shape == (1, 2, 2) and c1[0, 0].tolist() == [1, 2]
    assert c2.shape == (2, 2, 5) and c2[1, 1].tolist() == [1, 2, 2, 2, 2]
    assert e._ensure_lists("cpu", None, 1, 2, 256, 256)[0] is c1  # cached per shape


def test_decode_shapes_dispatch_to_the_split_kv_path():
    """q_len != kv_len (reference: attn_engine.py:252-286): grouped heads need one query position; the split count never
    leaves a split empty and is 1 when a stateful online function has no combine of its own."""
    e = helpers.decode_engine(1, 32, 8, 1, 8192, 128, torch.float16)
    assert e._decode is not None and e._decode.rows == 4 and e._decode.combine is not None
    assert "AE_DECODE 1" in e.tl_code and "AE_NQ 1" in e.tl_code and "#define AE_STAGES 3" in e.tl_code
    for B, S in ((1, 8192), (16, 8192), (64, 8192), (2, 1000), (3, 130)):
        n = e._decode.pick_splits(B, S)
        tiles = -(-S // 128)
        assert 1 <= n <= min(32, tiles) and (n - 1) * (-(-tiles // n)) < tiles
    two_tiles = helpers.decode_engine(1, 4, 4, 200, 4096, 64, torch.bfloat16)
    assert two_tiles._decode.rows == 200 and "AE_NQ 2" in two_tiles.tl_code
    no_combine = helpers.decode_engine(1, 8, 2, 1, 4096, 64, torch.float16, online=helpers.OnlineSoftmax())
    assert no_combine._decode.combine is None and no_combine._decode.pick_splits(1, 4096) == 1
    growing = helpers.decode_engine("B", 32, 8, 1, "S_kv", 128, torch.float16)  # named batch and KV length
    assert growing._decode is not None and growing._decode.rows == 4
    with pytest.raises(NotImplementedError):
        helpers.decode_engine(1, 8, 2, 2, 4096, 64, torch.float16)       # grouped heads with two query positions
    with pytest.raises(NotImplementedError):
        helpers.decode_engine(1, 4, 4, 300, 4096, 64, torch.float16)     # more than 256 rows per head unit


def test_row_scale_mod_is_recognised_in_the_trace():
    """`v * custom[batch, heads, seq_len]` (Mamba2's v_mod) goes to the row-scale kernels; other mods stay eager."""
    e = helpers.mamba2_engine(2, 4, 256, 128, 64, torch.bfloat16)
    x = torch.zeros(2, 4, 256, 64, dtype=torch.bfloat16)
    A, dt = torch.zeros(1, 4), torch.zeros(2, 4, 256, dtype=torch.bfloat16)
    assert e._rowscale_operand("v", x, (A, dt)) is dt
    assert e._rowscale_operand("decay", torch.zeros(2, 4, 256), (A, dt)) is None
    assert e._rowscale_operand("v", x, (A, dt[:1])) is None  # a broadcast batch dim is left to PyTorch


def test_decay_scale_and_skip_are_recognised_in_the_trace():
    """`decay * custom[1, heads]` (Mamba2's decay_mod) and `o + v * custom[1, heads]` (the skip) are taken into the
    scan kernels when their operands are fp32 with one value per head; anything else stays eager PyTorch."""
    from attentionengine_b200.attn_engine import LinearAttentionEngine
    from attentionengine_b200.core import CustomIO, meta_tensor
    e = helpers.mamba2_engine(2, 4, 256, 128, 64, torch.bfloat16, d_skip=True)
    decay = torch.zeros(2, 4, 256)
    A, dt, D = torch.zeros(1, 4), torch.zeros(2, 4, 256, dtype=torch.bfloat16), torch.zeros(1, 4)
    assert e._decay_scale_operand(decay, (A, dt, D)) is A
    assert e._skip_operand((A, dt, D)) is D
    assert e._decay_scale_operand(decay.double(), (A, dt, D)) is None          # the kernels read an fp32 decay
    assert e._decay_scale_operand(decay, (A.to(torch.bfloat16), dt, D)) is None  # ... and an fp32 scale
    metas = (meta_tensor(2, 1, 256, 128, dtype=torch.bfloat16),) * 2 + (meta_tensor(2, 4, 256, 64, dtype=torch.bfloat16),)
    other = LinearAttentionEngine(metas, decay_mod=lambda decay, io: decay + io.input_tensors["A"],
                                  custom_io=CustomIO({"A": (1, "heads")}))
    assert other._decay_scale_operand(decay, (A,)) is None                     # not a product
    per_step = LinearAttentionEngine(metas, decay_mod=lambda decay, io: decay * io.input_tensors["w"],
                                     custom_io=CustomIO({"w": ("batch", "heads", "seq_len")}))
    assert per_step._decay_scale_operand(decay, (torch.zeros(2, 4, 256),)) is None  # one value per step: eager


def test_block_lists_layout():
    from attentionengine_b200.attn_engine.attn_engine import _block_lists
    cnt = torch.tensor([[[[128 * 128, 0, 5], [0, 0, 0], [1, 128 * 128, 128 * 128]]]], dtype=torch.int32)
    c, i, ct, it = _block_lists(cnt, 128, 128, 384, 384, 1, 1, "cpu")
    assert c.tolist() == [[[2, 0, 3]]]
    assert (i[0, 0, 0, :2] & 0x3fffffff).tolist() == [0, 2] and (i[0, 0, 0, :2] >> 30).tolist() == [0, 1]
    assert (i[0, 0, 2, :3] >> 30).tolist() == [1, 0, 0]
    assert ct.tolist() == [[[2, 1, 2]]] and (it[0, 0, 2, :2] & 0x3fffffff).tolist() == [0, 2]


def test_unsupported_requests_fail_loudly():
    with pytest.raises(NotImplementedError):
        helpers.softmax_engine(1, 2, 2, 256, 256, 256, torch.float16, True)  # head dim > 128
    with pytest.raises(NotImplementedError):
        AttentionEngine(helpers.metas(1, 2, 2, 256, 64, 64, torch.float32), CustomIO({}),
                        score_mod=lambda s, c, b, h, q, kv: s, mask_mod=None, online_func=helpers.OnlineSoftmax())
    eng = helpers.softmax_engine(1, 2, 2, 256, 64, 64, torch.float16, True)
    q = torch.zeros(1, 256, 2, 64, dtype=torch.float16)
    with pytest.raises(Exception) as e:
        eng(q, q, q)
    assert "CUDA" in str(e.value)  # no CPU path


def test_reference_import_names():
    ae.install_reference_aliases()
    from attn_engine import AttentionEngine as A2, OnlineFunc as O2  # noqa: F401
    from core import CustomIO as C2, SymbolicArray, SymbolScalar, SymbolicTensor, Var, create_block_mask  # noqa: F401
    from core.utils import meta_tensor as m2
    assert A2 is AttentionEngine and m2 is meta_tensor


def test_block_mask_of_the_wrong_shape_is_refused_on_the_host():
    """The kernels index the tile lists with the runtime tile grid: a call-time block_mask with other dimensions, or a
    non-dynamic engine called at a shape other than the one its lists were inferred for, must not reach a launch."""
    B, H, S, D = 1, 2, 640, 64
    eng = AttentionEngine(helpers.metas(B, H, H, S, D, D, torch.float16), CustomIO({}),
                          score_mod=lambda s, c, b, h, q, kv: s * 0.125, mask_mod=None,
                          online_func=helpers.OnlineSoftmax(), extern_block_mask=True)
    ok = torch.ones(B, H, 5, 5, dtype=torch.int8)
    lists = eng._ensure_lists("cpu", ok, B, H, S, S)
    assert lists[0].shape == (B, H, 5) and lists[1].shape == (B, H, 5, 5)
    for bad in (torch.ones(B, H, 4, 5, dtype=torch.int8), torch.ones(B, H, 5, 6, dtype=torch.int8),
                torch.ones(3, H, 5, 5, dtype=torch.int8), torch.ones(H, 5, 5, dtype=torch.int8)):
        with pytest.raises(ValueError, match="block_mask has shape"):
            eng._ensure_lists("cpu", bad, B, H, S, S)
    win = AttentionEngine(helpers.metas(B, H, H, 1024, D, D, torch.float16), CustomIO({}),
                          score_mod=lambda s, c, b, h, q, kv: s * 0.125,
                          mask_mod=lambda b, h, q, kv: torch.logical_and(q >= kv, q - kv <= 200),
                          online_func=helpers.OnlineSoftmax())
    assert win.mask_mode == 2
    assert win._ensure_lists("cpu", None, B, H, 1024, 1024)[0].shape == (B, H, 8)
    with pytest.raises(ValueError, match="inferred for"):
        win._ensure_lists("cpu", None, B, H, 2048, 2048)
