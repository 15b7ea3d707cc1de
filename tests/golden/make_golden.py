"""Generate the golden fixtures in this directory from the reference's own source tree.

Run once, where the reference checkout is available:

    python tests/golden/make_golden.py /path/to/AttentionEngine

Nothing here is needed at test time: the tests read the ``.npz`` files only.  The script executes the
reference's *own* functions, taken from its files as text (they are closures nested inside benchmark
harnesses that need a GPU and matplotlib, so they cannot be imported), and the reference's own IR /
mask front end imported from ``<ref>/attention_engine``:

* softmax / GQA      ``flash_attn_func`` fallback      benchmark/bench_utils.py  (nested in do_bench_attention)
* relu               ``ref_program``                   benchmark/bench_utils.py  (nested in do_bench_reluattn)
* retention          ``ref_program``                   benchmark/bench_utils.py  (nested in do_bench_retention)
* MLA decode         ``ref_program``                   core/template/tl_template/attn/mla_decode_tl.py
* block masks        create_block_mask, is_causal_mask, is_less_causal_mask   core/transform/core.py
* symbolic autodiff  SymbolScalar.backward on the example score_mods          core/transform/core.py
* linear scan        fla.ops.simple_gla.naive (the library the reference checks simple_gla against, bench_utils.py:552-566)
* sigmoid attention  score_mod of attn_script/sigmoidattn.py traced and differentiated by the reference's IR, inside
                     the un-normalised P V composition its OnlineIdentity defines
* Mamba2 mapping     decay_mod / v_mod of attn_script/mamba2_ngroup1.py traced by the reference's IR, fed to fla's naive
                     recurrence (q = C, k = B)

Inputs are seeded; inputs and outputs are stored together so the fixtures do not depend on the
random-number generator of the machine that reads them.
"""
import math
import os
import sys
import textwrap

import numpy as np
import torch
import torch.nn.functional as F
from einops import einsum, rearrange

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", ".."))


def extract_def(path: str, header: str, occurrence: int = 0) -> str:
    """Source text of the (possibly nested) function whose ``def`` line starts with ``header``."""
    lines = open(path).read().split("\n")
    hits = [i for i, l in enumerate(lines) if l.strip().startswith(header)]
    i = hits[occurrence]
    indent = len(lines[i]) - len(lines[i].lstrip())
    out = [lines[i]]
    for l in lines[i + 1:]:
        if l.strip() and (len(l) - len(l.lstrip())) <= indent:
            break
        out.append(l)
    return textwrap.dedent("\n".join(out))


def load_fn(path, header, name, occurrence=0, **ns):
    env = {"torch": torch, "F": F, "einsum": einsum, "rearrange": rearrange, "math": math}
    env.update(ns)
    exec(extract_def(path, header, occurrence), env)
    return env[name]


def randn(g, *shape, dtype=torch.float16):
    return torch.randn(*shape, generator=g).to(dtype)


def grads(fn, inputs, d_out):
    leaves = [t.detach().float().requires_grad_() for t in inputs]
    out = fn(*leaves)
    out.float().backward(d_out.float())
    return out.detach().float(), [t.grad for t in leaves]


def np16(t):
    return t.detach().to(torch.float16).numpy() if t.dtype in (torch.float16,) else t.detach().float().numpy()


def script_defs(ref_root: str, name: str) -> dict:
    """The definitions part of one of the reference's example programs (everything above its ``eval()`` /
    ``__main__`` section), executed against the reference's own ``attn_engine`` / ``core`` packages."""
    src = open(os.path.join(ref_root, "attn_script", name)).read()
    cut = min(i for i in (src.find("\ndef eval("), src.find("\nif __name__"), len(src)) if i >= 0)
    env = {"__name__": "attn_script_defs"}
    exec(compile(src[:cut], name, "exec"), env)
    return env


def main(ref_root: str):
    bench = os.path.join(ref_root, "attention_engine", "benchmark", "bench_utils.py")
    mla = os.path.join(ref_root, "attention_engine", "core", "template", "tl_template", "attn", "mla_decode_tl.py")

    # ---------------- softmax (MHA causal at the benchmark's config 1, and small GQA cases) ---------------
    fa = load_fn(bench, "def flash_attn_func(query, key, value, softmax_scale, causal)", "flash_attn_func")
    cases = {"cfg1": (1, 4, 4, 512, 64, True, "ones"), "gqa_causal": (1, 4, 2, 256, 64, True, "randn"),
             "gqa_full": (1, 4, 2, 128, 64, False, "randn"), "mha_d128": (1, 2, 2, 128, 128, True, "randn")}
    out = {}
    for name, (B, Hq, Hkv, S, D, causal, dmode) in cases.items():
        g = torch.Generator().manual_seed(0)
        q, k, v = randn(g, B, S, Hq, D), randn(g, B, S, Hkv, D), randn(g, B, S, Hkv, D)
        d_o = torch.ones(B, S, Hq, D) if dmode == "ones" else randn(g, B, S, Hq, D).float()
        o, (dq, dk, dv) = grads(lambda a, b, c: fa(a, b, c, 1 / D ** 0.5, causal), (q, k, v), d_o)
        for nm, t in (("q", q), ("k", k), ("v", v), ("do", d_o.to(torch.float16)), ("o", o), ("dq", dq), ("dk", dk), ("dv", dv)):
            out[f"{name}.{nm}"] = np16(t)
        out[f"{name}.causal"] = np.array(causal)
    np.savez_compressed(os.path.join(HERE, "softmax.npz"), **out)

    # ---------------- relu ---------------------------------------------------------------------------------
    B, H, S, D = 1, 2, 256, 64
    relu = load_fn(bench, "def ref_program(query, key, value):", "ref_program", D=D)
    g = torch.Generator().manual_seed(1)
    q, k, v, d_o = randn(g, B, S, H, D), randn(g, B, S, H, D), randn(g, B, S, H, D), randn(g, B, S, H, D)
    o, (dq, dk, dv) = grads(relu, (q, k, v), d_o)
    np.savez_compressed(os.path.join(HERE, "relu.npz"), q=np16(q), k=np16(k), v=np16(v), do=np16(d_o), o=np16(o),
                        dq=np16(dq), dk=np16(dk), dv=np16(dv))

    # ---------------- retention (parallel form) ------------------------------------------------------------------
    B, H, S, D, DV = 1, 2, 256, 64, 64
    ret = load_fn(bench, "def ref_program(query, key, value, mask):", "ref_program", dtype=torch.float32)
    g = torch.Generator().manual_seed(2)
    q, k, v = randn(g, B, S, H, D), randn(g, B, S, H, D), randn(g, B, S, H, DV)
    gamma = 1 - 2.0 ** (-5 - torch.arange(H, dtype=torch.float32))
    idx = torch.arange(S)
    dist = (idx.view(-1, 1) - idx.view(1, -1)).float()
    mask = torch.where(dist >= 0, gamma.view(H, 1, 1) ** dist.clamp(min=0), torch.zeros(())).unsqueeze(0).to(torch.float16)
    o = ret(q.float(), k.float(), v.float(), mask.float())
    np.savez_compressed(os.path.join(HERE, "retention.npz"), q=np16(q), k=np16(k), v=np16(v), mask=np16(mask), o=np16(o))

    # ---------------- MLA decode ---------------------------------------------------------------------------------
    mla_ref = load_fn(mla, "def ref_program(q, q_pe, kv, k_pe, glse, Output_partial):", "ref_program")
    B, H, S, DV, DPE = 1, 16, 320, 512, 64
    g = torch.Generator().manual_seed(3)
    q, q_pe, kv, k_pe = randn(g, B, H, DV), randn(g, B, H, DPE), randn(g, B, S, 1, DV), randn(g, B, S, 1, DPE)
    o = mla_ref(q.float(), q_pe.float(), kv.float(), k_pe.float(), None, None)
    np.savez_compressed(os.path.join(HERE, "mla_decode.npz"), q=np16(q), q_pe=np16(q_pe), kv=np16(kv), k_pe=np16(k_pe),
                        o=np16(o))

    # ---------------- block masks and symbolic autodiff from the reference front end -----------------------------
    sys.path.insert(0, os.path.join(ref_root, "attention_engine"))
    from core.transform import core as rcore  # the reference's module

    def causal(b, h, q_idx, kv_idx):
        return q_idx >= kv_idx

    def causal_less(b, h, q_idx, kv_idx):
        return q_idx >= kv_idx + 128

    def sliding(b, h, q_idx, kv_idx):
        return torch.logical_and(q_idx >= kv_idx, q_idx - kv_idx <= 100)

    def head_dep(b, h, q_idx, kv_idx):
        return q_idx >= kv_idx + h * 64

    masks = {"causal": causal, "causal_less": causal_less, "sliding": sliding, "head_dep": head_dep}
    out = {}
    for nm, fn in masks.items():
        for (bm, bn) in ((128, 128), (128, 64)):
            bmask = rcore.create_block_mask(fn, 2, 4, 512, 512, "cpu", bm, bn)
            out[f"{nm}.{bm}x{bn}.block"] = bmask.numpy()
            out[f"{nm}.{bm}x{bn}.is_causal"] = np.array(bool(rcore.is_causal_mask(bmask, bm, bn)))
            out[f"{nm}.{bm}x{bn}.is_less_causal"] = np.array(bool(rcore.is_less_causal_mask(bmask, bm, bn)))
    np.savez_compressed(os.path.join(HERE, "block_masks.npz"), **out)

    # ---------------- linear scan: flash-linear-attention's naive recurrent form (the reference's checker library) --
    from fla.ops.simple_gla.naive import naive_recurrent_simple_gla
    g = torch.Generator().manual_seed(5)
    B, H, T, DK, DV = 1, 2, 320, 128, 64
    q, k, v = randn(g, B, H, T, DK, dtype=torch.bfloat16), randn(g, B, H, T, DK, dtype=torch.bfloat16), randn(g, B, H, T, DV, dtype=torch.bfloat16)
    a = -torch.nn.functional.softplus(torch.randn(B, H, T, generator=g) - 2.0)
    o, _ = naive_recurrent_simple_gla(q.float().transpose(1, 2), k.float().transpose(1, 2), v.float().transpose(1, 2),
                                      a.transpose(1, 2), scale=1.0)
    np.savez_compressed(os.path.join(HERE, "linear_scan.npz"), q=q.float().numpy(), k=k.float().numpy(),
                        v=v.float().numpy(), a=a.numpy(), o=o.transpose(1, 2).float().numpy())

    from oracle.ir_eval import evaluate
    g = torch.Generator().manual_seed(4)
    x = torch.randn(64, 64, generator=g) * 3
    seed = torch.randn(64, 64, generator=g)
    bias = 0.37

    def sm_scale(s, T):
        return s * 0.125

    def sm_sigmoid(s, T):
        s = s + T
        return ((s * 0.5).tanh() + 1) * 0.5

    def sm_relu(s, T):
        return (s * 0.125).max(0)

    def sm_div_log(s, T):
        return (s * s + 1.0).log() * s / (s * s + 2.0)

    out = {"x": x.numpy(), "seed": seed.numpy(), "bias": np.array(bias)}
    for nm, fn in (("scale", sm_scale), ("sigmoid", sm_sigmoid), ("relu", sm_relu), ("div_log", sm_div_log)):
        s = rcore.SymbolicArray("scores", rcore.Var("scores"), shape_idx=["block_M", "block_N"])
        T = rcore.SymbolicTensor("T", (1,))
        y = fn(s, T)
        d = rcore.SymbolScalar("d", rcore.Var("d"), shape_idx=["block_M", "block_N"])
        y.backward(d)
        env = {id(s): x, id(T): torch.tensor(bias), id(d): seed}
        out[f"{nm}.y"] = torch.as_tensor(evaluate(y, env)).expand_as(x).numpy()
        out[f"{nm}.dx"] = torch.as_tensor(evaluate(s.grad, env)).expand_as(x).numpy()
    np.savez_compressed(os.path.join(HERE, "autodiff.npz"), **out)

    # ---------------- sigmoid attention: the reference's score_mod and its symbolic derivative ----------------------
    defs = script_defs(ref_root, "sigmoidattn.py")
    B, H, S, D = 1, 2, 256, 64
    g = torch.Generator().manual_seed(6)
    q, k, v, d_o = (randn(g, B, S, H, D) for _ in range(4))
    q = (q.float() * D ** -0.5).to(torch.float16)   # the script's score_mod has no scale of its own
    bias = -math.log(S)
    s_sym = rcore.SymbolicArray("scores", rcore.Var("scores"), shape_idx=["block_M", "block_N"])
    cio = defs["custom_fwd_inputs"]
    y = defs["score_mod"](s_sym, cio, None, None, None, None)
    d_sym = rcore.SymbolScalar("d", rcore.Var("d"), shape_idx=["block_M", "block_N"])
    y.backward(d_sym)
    sc = torch.einsum("bqhd,bkhd->bhqk", q.float(), k.float())
    dp = torch.einsum("bqhd,bkhd->bhqk", d_o.float(), v.float())
    env = {id(s_sym): sc, id(cio.input_tensors["softmax_bias"]): torch.tensor(bias), id(d_sym): dp}
    p = torch.as_tensor(evaluate(y, env))
    ds = torch.as_tensor(evaluate(s_sym.grad, env))
    np.savez_compressed(os.path.join(HERE, "sigmoid.npz"), q=np16(q), k=np16(k), v=np16(v), do=np16(d_o),
                        bias=np.array(bias), o=torch.einsum("bhqk,bkhd->bqhd", p, v.float()).numpy(),
                        dq=torch.einsum("bhqk,bkhd->bqhd", ds, k.float()).numpy(),
                        dk=torch.einsum("bhqk,bqhd->bkhd", ds, q.float()).numpy(),
                        dv=torch.einsum("bhqk,bqhd->bkhd", p, d_o.float()).numpy())

    # ---------------- Mamba2 operator mapping: the reference's decay_mod / v_mod in front of fla's recurrence --------
    defs = script_defs(ref_root, "mamba2_ngroup1.py")
    B, H, T, N, P = 1, 3, 320, 128, 64
    g = torch.Generator().manual_seed(7)
    x = randn(g, B, H, T, P, dtype=torch.bfloat16)
    Bm, Cm = randn(g, B, 1, T, N, dtype=torch.bfloat16), randn(g, B, 1, T, N, dtype=torch.bfloat16)
    dt = F.softplus(torch.randn(B, H, T, generator=g) - 4.0)
    A = -torch.exp(torch.rand(H, generator=g) * math.log(16.0))
    cio = rcore.CustomIO({"A": (1, "heads"), "dt": ("batch", "heads", "seq_len")})
    dec_sym = rcore.SymbolicArray("decay", rcore.Var("decay"), shape_idx=["B", "H", "T"])
    v_sym = rcore.SymbolicArray("v", rcore.Var("v"), shape_idx=["B", "H", "T", "D"])
    a = torch.as_tensor(evaluate(defs["decay_mod"](dec_sym, cio),
                                 {id(dec_sym): dt, id(cio.input_tensors["A"]): A.view(1, H, 1)}))
    vm = torch.as_tensor(evaluate(defs["v_mod"](v_sym, cio),
                                  {id(v_sym): x.float(), id(cio.input_tensors["dt"]): dt[..., None]}))
    o, _ = naive_recurrent_simple_gla(Cm.float().expand(B, H, T, N).transpose(1, 2), Bm.float().expand(B, H, T, N).transpose(1, 2),
                                      vm.transpose(1, 2), a.transpose(1, 2), scale=1.0)
    np.savez_compressed(os.path.join(HERE, "mamba2.npz"), x=x.float().numpy(), dt=dt.numpy(), A=A.numpy(),
                        Bm=Bm.float().numpy(), Cm=Cm.float().numpy(), o=o.transpose(1, 2).float().numpy())
    print("wrote", sorted(f for f in os.listdir(HERE) if f.endswith(".npz")))


if __name__ == "__main__":
    if len(sys.argv) < 2:
        sys.exit("usage: make_golden.py <path to the AttentionEngine source tree>")
    main(sys.argv[1])
