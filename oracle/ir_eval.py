"""Evaluate a traced IR expression with PyTorch, and run the online attention recurrence on CPU the
way the reference forward kernel does.  TEST INFRASTRUCTURE ONLY (see oracle/__init__.py).

``evaluate`` only relies on ``.prev`` and ``.code.type`` / ``.code.name`` / ``.code.value``, which the
reference's SymbolScalar (attention_engine/core/transform/core.py:36-251) and this repository's share,
so the same evaluator is used on both (tests/golden/make_golden.py runs it on the reference's graphs).
"""
from __future__ import annotations

import math

import torch


def evaluate(v, env: dict, cache: dict | None = None):
    """Value of symbolic value ``v``.  ``env`` maps id(leaf) or a leaf's varname / Var name to a tensor
    or number.  Tile values are [..., M, N]; row values [..., M, 1]; reductions keep the last dim."""
    cache = {} if cache is None else cache
    key = id(v)
    if key in cache:
        return cache[key]
    t = v.code.type
    if not v.prev:
        if key in env:
            r = env[key]
        elif t == "Const":
            r = float(v.code.value)
        elif v.varname in env:
            r = env[v.varname]
        elif t == "Var" and v.code.name in env:
            r = env[v.code.name]
        elif t == "Var":
            nm = v.code.name.strip()
            r = -math.inf if nm == "-inf" else float(nm)
        else:
            raise KeyError(v.varname)
        cache[key] = r
        return r
    a = [evaluate(p, env, cache) for p in v.prev]
    T = torch.as_tensor
    if t == "Add":
        r = a[0] + a[1]
    elif t == "Sub":
        r = a[0] - a[1]
    elif t == "Mul":
        r = a[0] * a[1]
    elif t == "Div":
        r = a[0] / a[1]
    elif t == "Neg":
        r = -a[0]
    elif t == "Abs":
        r = T(a[0]).abs()
    elif t == "Exp":
        r = T(a[0]).exp()
    elif t == "Exp2":
        r = T(a[0]).exp2()
    elif t == "Log":
        r = T(a[0]).log()
    elif t == "Log2":
        r = T(a[0]).log2()
    elif t == "Tanh":
        r = T(a[0]).tanh()
    elif t == "Max":
        r = torch.maximum(T(a[0], dtype=torch.float32), T(a[1], dtype=torch.float32))
    elif t == "MaxBwd":  # grad where out > other else 0 (core/codegen/tl_gen.py:118-121)
        r = torch.where(T(a[1]) > T(a[2]), T(a[0], dtype=torch.float32), torch.zeros(()))
    elif t == "ReduceSum":
        r = T(a[0]).sum(dim=-1, keepdim=True)
    elif t == "ReduceMax":
        r = T(a[0]).amax(dim=-1, keepdim=True)
    elif t == "ReduceAbsSum":
        r = T(a[0]).abs().sum(dim=-1, keepdim=True)
    else:
        raise NotImplementedError(t)
    cache[key] = r
    return r


def online_attention(ae, q, k, v, score_mod, mask_mod, online_func, custom: dict | None = None, block_n: int = 128,
                     mask_value: float = -math.inf):
    """Forward of the reference kernel, tile by tile (attention_engine/core/template/tl_template/attn/
    attn_tl.py:117-172): per kv tile  S = mask_value-or-0 + q k^T  ->  score_mod  ->  online_fwd (new row
    scales, o_scale)  ->  acc_o *= o_scale  ->  acc_o += P v ; then online_fwd_epilogue.  fp32 throughout,
    P rounded to the input dtype before P v as the kernel does (attn_tl.py:153).  ``ae`` is the package
    providing SymbolicArray / SymbolScalar / Var (this repository's or the reference's).
    Returns (o [B, S, H, DV] fp32, {name: final rowscale [B, H, S]})."""
    SymbolicArray, SymbolScalar, Var = ae.SymbolicArray, ae.SymbolScalar, ae.Var
    B, Sq, Hq, D = q.shape
    Skv, Hkv = k.shape[1], k.shape[2]
    g = Hq // Hkv
    qf = q.float().permute(0, 2, 1, 3)                      # [B, H, Sq, D]
    kf = k.float().repeat_interleave(g, dim=2).permute(0, 2, 1, 3)
    vf = v.float().repeat_interleave(g, dim=2).permute(0, 2, 1, 3)
    custom = custom or {}
    bi = torch.arange(B).view(B, 1, 1, 1)
    hi = torch.arange(Hq).view(1, Hq, 1, 1)
    qi = torch.arange(Sq).view(1, 1, Sq, 1)

    def sym(name, shape):
        return SymbolScalar(name, Var(name), shape_idx=shape)

    # state
    state = {}
    for name, s in online_func.online_rowscales.items():
        init = s.code.name.strip()
        val = -1e38 if init == "-inf" else float(init)      # finite sentinel, core/lower/lower.py:23-29
        state[name] = torch.full((B, Hq, Sq, 1), val)
    acc = torch.zeros(B, Hq, Sq, v.shape[-1])

    class _CI:  # stand-in for CustomIO inside score_mod
        def __init__(self, tensors):
            self.input_tensors = tensors

    for n0 in range(0, Skv, block_n):
        n1 = min(n0 + block_n, Skv)
        ki = torch.arange(n0, n1).view(1, 1, 1, -1)
        s = torch.einsum("bhqd,bhkd->bhqk", qf, kf[:, :, n0:n1])
        if mask_mod is not None:
            keep = mask_mod(bi, hi, qi, ki)
            s = s + torch.where(keep, torch.zeros(()), torch.full((), mask_value))
        # score_mod
        sc = SymbolicArray("scores", Var("scores"), shape_idx=["block_M", "block_N"])
        ci = {}
        env = {id(sc): s, "b": bi.float(), "h": hi.float(), "q_idx": qi.float(), "kv_idx": ki.float()}
        for nm, (shape, t) in custom.items():
            st = SymbolScalar(nm, Var(nm), shape_idx=[str(x) for x in shape])
            ci[nm] = st
            tt = t.float()
            view = [1, 1, 1, 1]
            sl = [slice(None)] * tt.dim()
            for d, dn in enumerate(shape):
                if str(dn) == "seq_len_kv":
                    sl[d] = slice(n0, n1)
            tt = tt[tuple(sl)]
            dims = {"batch": 0, "heads": 1, "seq_len": 2, "seq_len_kv": 3}
            shp = [1, 1, 1, 1]
            for d, dn in enumerate(shape):
                if str(dn) in dims:
                    shp[dims[str(dn)]] = tt.shape[d]
            env[id(st)] = tt.reshape(shp)
        out = score_mod(sc, _CI(ci), sym("b", ["1"]), sym("h", ["1"]), sym("q_idx", ["block_M"]),
                        sym("kv_idx", ["block_N"]))
        s = torch.as_tensor(evaluate(out, env)).expand(B, Hq, Sq, n1 - n0)
        # online_fwd
        sc2 = SymbolicArray("scores", Var("scores"), shape_idx=["block_M", "block_N"])
        rs = {nm: sym(nm, ["block_M"]) for nm in state}
        env = {id(sc2): s, "b": bi.float(), "h": hi.float(), "q_idx": qi.float()}
        for nm in state:
            env[id(rs[nm])] = state[nm]
        p_sym, new_rs, o_scale = online_func.online_fwd(sc2, dict(rs), sym("b", ["1"]), sym("h", ["1"]),
                                                        sym("q_idx", ["block_M"]))
        cache = {}
        p = torch.as_tensor(evaluate(p_sym, env, cache)).expand(B, Hq, Sq, n1 - n0)
        osc = torch.as_tensor(evaluate(o_scale, env, cache), dtype=torch.float32)
        new_state = {nm: torch.as_tensor(evaluate(x, env, cache), dtype=torch.float32).expand(B, Hq, Sq, 1).clone()
                     for nm, x in new_rs.items()}
        acc = acc * osc
        acc = acc + torch.einsum("bhqk,bhkd->bhqd", p.to(q.dtype).float(), vf[:, :, n0:n1])
        state.update(new_state)
    # epilogue
    o_sym = SymbolicArray("o", Var("o"), shape_idx=["block_M", "dimv"])
    rs = {nm: sym(nm, ["block_M"]) for nm in state}
    env = {id(o_sym): acc}
    for nm in state:
        env[id(rs[nm])] = state[nm]
    o_new, finals = online_func.online_fwd_epilogue(o_sym, rs, sym("b", ["1"]), sym("h", ["1"]), sym("q_idx", ["block_M"]))
    cache = {}
    o = torch.as_tensor(evaluate(o_new, env, cache)).expand_as(acc)
    fin = {nm: torch.as_tensor(evaluate(x, env, cache), dtype=torch.float32).expand(B, Hq, Sq, 1)[..., 0] for nm, x in finals.items()}
    return o.permute(0, 2, 1, 3).contiguous(), fin
