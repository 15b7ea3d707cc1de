"""Evaluate a traced IR expression with torch ops (differentiable by torch autograd).

Used for the q / k / v / decay mods of LinearAttentionEngine, which the reference also runs as eager
PyTorch statements generated from the trace (``to_pytorch_op``, core/codegen/tl_gen.py:236-303, spliced at
core/template/tl_template/linear/linear_tl.py:1136-1144).
"""
from __future__ import annotations

import torch


def evaluate(v, env: dict, cache: dict | None = None, hooks: dict | None = None):
    """`hooks` maps id(node) -> callable(list of evaluated operands) that replaces the node's own rule."""
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
        elif t == "Var" and v.code.name.strip().lstrip("-").replace(".", "", 1).isdigit():
            r = float(v.code.name)
        else:
            raise KeyError(f"unbound symbolic value {v.varname!r}")
        cache[key] = r
        return r
    a = [evaluate(p, env, cache, hooks) for p in v.prev]
    T = torch.as_tensor
    if hooks and key in hooks:
        r = hooks[key](a)
    elif t == "ReduceSum":
        r = T(a[0]).sum(-1, keepdim=True)
    elif t == "ReduceMax":
        r = T(a[0]).amax(-1, keepdim=True)
    elif t == "ReduceAbsSum":
        r = T(a[0]).abs().sum(-1, keepdim=True)
    elif t == "Add":
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
        x, y = a
        if not isinstance(x, torch.Tensor):
            x, y = y, x
        r = torch.clamp(x, min=y) if not isinstance(y, torch.Tensor) else torch.maximum(x, y)
    else:
        raise NotImplementedError(f"mod uses IR op {t}, which has no eager evaluation")
    cache[key] = r
    return r
