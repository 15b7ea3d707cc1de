"""The reference's own example programs as acceptance inputs: the definitions part of each
``attn_script/*.py`` (everything above its ``eval()`` / ``__main__`` section) is executed unchanged, with
``import attn_engine`` / ``import core`` resolved to this package by ``install_reference_aliases()``, and an engine
is built from the names the script defines, which traces, lowers and compiles its callables for sm_100a.

Needs the reference's source tree (``AE_REFERENCE_ROOT``, default: a directory ``reference`` beside this repository);
skipped where it is absent.
No GPU: NVRTC compiles without one."""
import os

import pytest
import torch

import attentionengine_b200 as ae

REF = os.environ.get("AE_REFERENCE_ROOT",
                     os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "reference"))
pytestmark = pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "attn_script")),
                                reason="reference source tree not present")


def _defs(name):
    ae.install_reference_aliases()
    src = open(os.path.join(REF, "attn_script", name)).read()
    cut = min(i for i in (src.find("\ndef eval("), src.find("\nif __name__"), len(src)) if i >= 0)
    env = {"__name__": "attn_script_defs"}
    exec(compile(src[:cut], name, "exec"), env)
    return env


def _metas(B, Hq, Hkv, Sq, Skv, D, DV, dtype=torch.float16):
    return (ae.meta_tensor(B, Hq, Sq, D, dtype=dtype), ae.meta_tensor(B, Hkv, Skv, D, dtype=dtype),
            ae.meta_tensor(B, Hkv, Skv, DV, dtype=dtype))


ATTENTION = [
    # script, mask name, online class, custom inputs name, (B, Hq, Hkv, Sq, Skv, D, DV), expected mask mode, extra kwargs
    ("mha.py", "causal_mask", "OnlineSoftmax", None, (1, 2, 2, 256, 256, 128, 128), 1, {}),
    ("gqa.py", None, "OnlineSoftmax", None, (1, 4, 2, 256, 256, 128, 128), 0, {}),
    ("sigmoidattn.py", "causal_mask", "OnlineIdentity", "custom_fwd_inputs", (1, 2, 2, 256, 256, 128, 128), 1, {}),
    ("reluattn.py", None, "OnlineIdentity", "custom_fwd_inputs", (1, 2, 2, 256, 256, 64, 64), 0, {}),
    ("sparseattn.py", "block_sparse_mask", "OnlineSoftmax", None, (1, 2, 2, 1024, 1024, 128, 128), 2, {}),
    ("blocksparseattn.py", "true_mask_mod", "OnlineSoftmax", None, (1, 2, 2, 512, 512, 128, 128), 2,
     {"extern_block_mask": True}),
    ("mha_inference.py", None, "OnlineSoftmax", None, (1, 2, 2, 128, 1024, 128, 128), 0, {}),
    ("gqa_inference.py", None, "OnlineSoftmax", None, (1, 8, 2, 1, 1024, 128, 128), 0, {}),
    ("mla_decode.py", None, "OnlineSoftmax", None, (2, 128, 1, 1, 1024, 576, 512), 0, {"kv_shared": True}),
    ("retention.py", "causal_mask", "OnlineRetention", None, (1, 2, 2, 256, 256, 128, 128), 1, {"mask_value": "0"}),
]


@pytest.mark.parametrize("script,mask,online,custom,shape,mode,kw", ATTENTION, ids=[a[0] for a in ATTENTION])
def test_attention_script_definitions_build_an_engine(script, mask, online, custom, shape, mode, kw):
    env = _defs(script)
    cio = env[custom] if custom else ae.CustomIO({})
    if script == "retention.py":
        cio = ae.CustomIO({"mask": (1, "heads", "seq_len", "seq_len_kv")})  # built inside the script's eval()
    eng = ae.AttentionEngine(_metas(*shape), cio, score_mod=env["score_mod"], mask_mod=env[mask] if mask else None,
                             online_func=env[online](), **kw)
    assert "tcgen05" in eng.tl_code and eng.mask_mode == mode
    if not kw.get("kv_shared") and shape[3] == shape[4]:
        assert eng.kernels.bwd.dkv.handle  # the backward kernels compile from the traced forward / backward too


LINEAR = [
    ("mamba2_ngroup1.py", {"decay_mod", "v_mod"}, {"A": (1, "heads"), "dt": ("batch", "heads", "seq_len")}, 128, 64, 1),
    ("mamba2.py", {"decay_mod", "k_mod"}, {"A": (1, "heads"), "dt": ("batch", "heads", "seq_len")}, 128, 64, 4),
    ("simple_gla.py", {"q_mod"}, {}, 256, 256, 4),
    ("retention_linear.py", {"decay_mod", "q_mod"}, {}, 256, 512, 4),
]


@pytest.mark.parametrize("script,mods,custom,DK,DV,HQ", LINEAR, ids=[a[0] for a in LINEAR])
def test_linear_script_definitions_build_an_engine(script, mods, custom, DK, DV, HQ):
    env = _defs(script)
    B, H, T, dt = 1, 4, 512, torch.bfloat16
    metas = (ae.meta_tensor(B, HQ, T, DK, dtype=dt), ae.meta_tensor(B, HQ, T, DK, dtype=dt),
             ae.meta_tensor(B, H, T, DV, dtype=dt))
    eng = ae.LinearAttentionEngine(metas, custom_io=ae.CustomIO(custom), **{m: env[m] for m in mods})
    assert "tcgen05" in eng.tl_code and set(eng._traced) == {m[:-4] for m in mods}
