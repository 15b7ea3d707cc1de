"""Symbolic values traced through user callables (score_mod, OnlineFunc.*, q/k/v/decay mods).

Host-side mirror of the reference's IR front end (attention_engine/core/transform/core.py):
``SymbolScalar`` (:36-251), ``SymbolicArray`` (:253-278), ``SymbolicColReduceArray`` (:280-304),
``SymbolicTensor`` (:306-316), ``SymbolicConst`` (:319-328), ``CustomIO`` (:331-349) and the mask
helpers ``create_mask`` / ``create_block_mask`` / ``is_causal_mask`` / ``is_less_causal_mask`` /
``create_block_idx`` (:352-512).  Same names, constructor arguments and method surface; the
implementation differs:

* values are proper SSA: the result shape of a binary op is the broadcast of both operands, so
  ``a * b`` and ``b * a`` lower identically (the reference inherits the left operand's name/shape);
* reverse-mode differentiation walks the DAG once in topological order and also covers Sub, Neg,
  Exp, Exp2, Log2 and Abs, for which the reference raises NotImplementedError (:193-195);
* block masks are built one query-block row at a time from broadcast index tensors, never from a
  dense [B, H, S, S] mask.
"""
from __future__ import annotations

import math
from typing import Callable, Literal, Optional

import torch

from .graph import *  # noqa: F401,F403
from .graph import (Abs, Add, ColReduceAbsSum, ColReduceMax, ColReduceSum, Const, Div, Exp, Exp2, Log, Log2, Max,
                    MaxBwd, Mul, Neg, Node, ReduceAbsSum, ReduceMax, ReduceSum, Sub, Tanh, Var)

# dimension names that make a value vary along the kv (column) direction of a score tile
_COL_DIMS = {"block_N", "seq_len_kv", "kv_idx"}
_ROW_DIMS = {"block_M", "seq_len", "q_idx"}
_UNIFORM_DIMS = {"batch", "heads", "1"}

_uid = [0]


def _fresh(prefix: str) -> str:
    _uid[0] += 1
    return f"{prefix}_{_uid[0]}"


class SymbolScalar:
    """A symbolic scalar / row vector / tile, identified by its defining expression."""

    def __init__(self, varname: str, value: Node, prev=(), shape_idx=("block_M",), require_grad: bool = True,
                 dtype="float"):
        self.varname = varname
        self.code = value
        self.prev = list(prev)
        self.shape_idx = [str(i) for i in shape_idx]
        self.require_grad = require_grad
        self.dtype = dtype
        self.grad: Optional[SymbolScalar] = None
        # bookkeeping fields kept for scripts that poke at them
        self.count = 0
        self.use_list = []
        self.allow_reuse = True
        self.lowered = False
        self.visit_count = 0

    # -- introspection ---------------------------------------------------------------
    def __repr__(self):
        return f"{type(self).__name__}({self.varname}, {self.code.type}, shape={self.shape_idx})"

    @property
    def name(self):
        return self.varname

    @property
    def shape(self):
        return list(self.shape_idx)

    @property
    def kind(self) -> str:
        """'const' | 'uniform' | 'row' | 'tile' : how the value varies over a score tile."""
        dims = set(self.shape_idx)
        if dims & _COL_DIMS:
            return "tile"
        if dims & _ROW_DIMS:
            return "row"
        if self.code.type == "Const" or not dims:
            return "const"
        return "uniform"

    def set_allow_reuse(self, allow_reuse: bool):
        self.allow_reuse = allow_reuse

    def clear_usecount(self):
        self.count = 0
        self.use_list.clear()

    def clear_visit(self):
        self.visit_count = 0
        self.lowered = False

    def clear_codegen(self):
        self.clear_usecount()
        self.clear_visit()

    # -- construction of new values ----------------------------------------------------
    @staticmethod
    def _wrap(x) -> "SymbolScalar":
        if isinstance(x, SymbolScalar):
            return x
        if isinstance(x, (int, float)):
            return SymbolicConst(x)
        raise TypeError(f"cannot use {type(x).__name__} in a symbolic expression")

    def op(self, code, others=(), shape_idx=None, varname_suffix: Optional[str] = None):
        operands = [self] + [self._wrap(o) for o in others]
        if shape_idx is None:
            rank = {"const": 0, "uniform": 1, "row": 2, "tile": 3}
            widest = max(operands, key=lambda v: (rank[v.kind], len(v.shape_idx)))
            shape_idx = widest.shape_idx
        cls = SymbolicArray if isinstance(self, SymbolicArray) or any(
            isinstance(o, SymbolicArray) for o in operands) else SymbolScalar
        if isinstance(self, SymbolicColReduceArray):
            cls = SymbolicColReduceArray
        base = self.varname if not isinstance(self, SymbolicConst) else "c"
        if varname_suffix:
            base = f"{base}_{varname_suffix}"
        node = code(*[o.code for o in operands])
        out = cls(_fresh(base), node, operands, shape_idx)
        out.require_grad = any(o.require_grad for o in operands)
        for o in operands:
            o.use_list.append(out)
            o.count += 1
        return out

    def __add__(self, other):
        return self.op(Add, [other])

    def __radd__(self, other):
        return self._wrap(other).op(Add, [self])

    def __sub__(self, other):
        return self.op(Sub, [other])

    def __rsub__(self, other):
        return self._wrap(other).op(Sub, [self])

    def __mul__(self, other):
        return self.op(Mul, [other])

    def __rmul__(self, other):
        return self._wrap(other).op(Mul, [self])

    def __truediv__(self, other):
        return self.op(Div, [other])

    def __rtruediv__(self, other):
        return self._wrap(other).op(Div, [self])

    def __neg__(self):
        return self.op(Neg)

    def abs(self):
        return self.op(Abs)

    def tanh(self):
        return self.op(Tanh)

    def exp(self):
        return self.op(Exp)

    def exp2(self):
        return self.op(Exp2)

    def log(self):
        return self.op(Log)

    def log2(self):
        return self.op(Log2)

    def max(self, other):
        return self.op(Max, [other])

    def maxbwd(self, out, other):
        return self.op(MaxBwd, [out, other])

    # -- reverse-mode differentiation -------------------------------------------------------
    def backward(self, grad: Optional["SymbolScalar"] = None):
        """Propagate ``grad`` (d loss / d self) to every value this one depends on; results
        land in ``.grad``.  One pass over the DAG in reverse topological order."""
        if grad is not None:
            self.grad = grad
        if self.grad is None:
            raise ValueError("backward() needs a seed gradient")
        order, seen = [], set()

        def visit(v):
            if id(v) in seen:
                return
            seen.add(id(v))
            for p in v.prev:
                visit(p)
            order.append(v)

        visit(self)
        for v in order:
            if v is not self:
                v.grad = None
        for v in reversed(order):
            if v.grad is None or not v.prev:
                continue
            v._push_grad(v.grad)

    def _accumulate(self, g: "SymbolScalar"):
        if not self.require_grad:
            return
        self.grad = g if self.grad is None else self.grad + g

    def _push_grad(self, g: "SymbolScalar"):
        t = self.code.type
        p = self.prev
        if t == "Add":
            p[0]._accumulate(g)
            p[1]._accumulate(g)
        elif t == "Sub":
            p[0]._accumulate(g)
            if p[1].require_grad:
                p[1]._accumulate(-g)
        elif t == "Neg":
            p[0]._accumulate(-g)
        elif t == "Mul":
            if p[0].require_grad:
                p[0]._accumulate(g * p[1])
            if p[1].require_grad:
                p[1]._accumulate(g * p[0])
        elif t == "Div":
            if p[0].require_grad or p[1].require_grad:
                g0 = g / p[1]
                p[0]._accumulate(g0)
                if p[1].require_grad:
                    p[1]._accumulate(-(g0 * self))
        elif t == "Tanh":
            if p[0].require_grad:
                p[0]._accumulate(g - g * self * self)
        elif t == "Exp":
            if p[0].require_grad:
                p[0]._accumulate(g * self)
        elif t == "Exp2":
            if p[0].require_grad:
                p[0]._accumulate(g * self * math.log(2.0))
        elif t == "Log":
            if p[0].require_grad:
                p[0]._accumulate(g / p[0])
        elif t == "Log2":
            if p[0].require_grad:
                p[0]._accumulate(g / (p[0] * math.log(2.0)))
        elif t == "Abs":
            if p[0].require_grad:
                # d|x| = sign(x): g where x > 0, -g where -x > 0
                p[0]._accumulate(g.maxbwd(p[0], SymbolicConst(0.0)) - g.maxbwd(-p[0], SymbolicConst(0.0)))
        elif t == "Max":
            if p[0].require_grad:
                p[0]._accumulate(g.maxbwd(self, p[1]))
            if p[1].require_grad:
                p[1]._accumulate(g.maxbwd(self, p[0]))
        else:
            raise NotImplementedError(f"backward for {t} is not implemented")


class SymbolicArray(SymbolScalar):
    """A [block_M, block_N] score tile inside ``OnlineFunc`` (reference: core.py:253-278)."""

    def __init__(self, varname: str = "", code: Node = None, prev=(), shape_idx=("block_M", "block_N")):
        super().__init__(varname, code if code is not None else Var(" "), prev, shape_idx)

    def get_reduce(self, op: Literal["sum", "max", "abssum"]):
        node = {"sum": ReduceSum, "max": ReduceMax, "abssum": ReduceAbsSum}.get(op)
        if node is None:
            raise NotImplementedError(op)
        out = self.op(node, shape_idx=self.shape_idx[:-1], varname_suffix=op)
        return out


class SymbolicColReduceArray(SymbolScalar):
    """Per-split row scales inside ``OnlineFunc.combine``; reductions run over the split
    dimension (reference: core.py:280-304)."""

    def __init__(self, varname: str = "", code: Node = None, prev=(), shape_idx=("block_M", "block_N")):
        super().__init__(varname, code if code is not None else Var(" "), prev, shape_idx)

    def get_reduce(self, op: Literal["sum", "max", "abssum"]):
        node = {"sum": ColReduceSum, "max": ColReduceMax, "abssum": ColReduceAbsSum}.get(op)
        if node is None:
            raise NotImplementedError(op)
        return self.op(node, shape_idx=self.shape_idx[:-2] + [self.shape_idx[-1]], varname_suffix=op)


class SymbolicTensor(SymbolScalar):
    """A named runtime tensor declared through ``CustomIO`` (reference: core.py:306-316)."""

    def __init__(self, varname: str, shape: tuple):
        super().__init__(varname, Var(varname), shape_idx=[str(i) for i in shape], require_grad=False)


class SymbolicConst(SymbolScalar):
    """A python number folded into the expression (reference: core.py:319-328)."""

    def __init__(self, value):
        super().__init__(f"float({value})", Const(value), prev=[], shape_idx=[], require_grad=False)


class CustomIO:
    """Named extra inputs of the operator: ``{name: shape}`` with shapes made of ints or the
    dimension names "batch", "heads", "seq_len", "seq_len_kv", "1" (reference: core.py:331-349,
    shape vocabulary core/lower/lower.py:31-56)."""

    def __init__(self, input_tensors: Optional[dict] = None):
        self.input_tensors: dict[str, SymbolicTensor] = {}
        for k, v in (input_tensors or {}).items():
            self.input_tensors[k] = SymbolicTensor(k, tuple(v))

    def __call__(self, tensor_name: str, tensor_shape: tuple):
        """Decorator form ``@io("name", shape)``: declares the tensor and returns the function."""
        if tensor_name in self.input_tensors:
            raise ValueError(f"Tensor {tensor_name} already exists")
        self.input_tensors[tensor_name] = SymbolicTensor(tensor_name, tuple(tensor_shape))

        def decorator(func):
            return func

        return decorator


# =====================================================================================
# mask utilities
# =====================================================================================

def _broadcast_indices(B, H, q, kv, device):
    b = torch.arange(B, device=device).view(B, 1, 1, 1)
    h = torch.arange(H, device=device).view(1, H, 1, 1)
    return b, h, q.view(1, 1, -1, 1), kv.view(1, 1, 1, -1)


def _eval_mask(mod_fn: Callable, B, H, q, kv, device) -> torch.Tensor:
    """mask_mod over broadcast index tensors; falls back to vmap for callables that need scalars."""
    b, h, qq, kk = _broadcast_indices(B, H, q, kv, device)
    try:
        m = mod_fn(b, h, qq, kk)
        if not isinstance(m, torch.Tensor):
            raise TypeError
        return m.to(torch.bool)
    except Exception:
        fn = mod_fn
        for dims in ((None, None, None, 0), (None, None, 0, None), (None, 0, None, None), (0, None, None, None)):
            fn = torch.vmap(fn, in_dims=dims, out_dims=0)
        return fn(torch.arange(B, device=device), torch.arange(H, device=device), q, kv).to(torch.bool)


def create_mask(mod_fn, B: Optional[int], H: Optional[int], Q_LEN: int, KV_LEN: int, device: str = "cuda"):
    """Dense boolean mask [B, H, Q_LEN, KV_LEN] of ``mod_fn(b, h, q_idx, kv_idx)`` (reference: core.py:352-398)."""
    B = 1 if B is None else B
    H = 1 if H is None else H
    m = _eval_mask(mod_fn, B, H, torch.arange(Q_LEN, device=device), torch.arange(KV_LEN, device=device), device)
    return m.expand(B, H, Q_LEN, KV_LEN)


_DEFAULT_SPARSE_BLOCK_SIZE = 128
BLOCK_SIZE = 128


def _convert_mask_to_block_mask(mask: torch.Tensor, Q_BLOCK_SIZE=_DEFAULT_SPARSE_BLOCK_SIZE,
                                KV_BLOCK_SIZE=_DEFAULT_SPARSE_BLOCK_SIZE, separate_full_blocks: bool = False):
    """Pool a dense boolean mask into per-block int8 flags (reference: core.py:410-453)."""
    assert mask.dtype == torch.bool
    while mask.dim() < 4:
        mask = mask.unsqueeze(0)
    B, H, Q, KV = mask.shape
    pq, pk = (-Q) % Q_BLOCK_SIZE, (-KV) % KV_BLOCK_SIZE
    mask = torch.nn.functional.pad(mask, (0, pk, 0, pq))
    nq, nk = (Q + pq) // Q_BLOCK_SIZE, (KV + pk) // KV_BLOCK_SIZE
    cnt = mask.reshape(B, H, nq, Q_BLOCK_SIZE, nk, KV_BLOCK_SIZE).sum(dim=(3, 5))
    if separate_full_blocks:
        full = cnt == Q_BLOCK_SIZE * KV_BLOCK_SIZE
        return ((cnt > 0) & ~full).to(torch.int8), full.to(torch.int8)
    return (cnt > 0).to(torch.int8), None


def block_mask_counts(mask_mod, B, H, QLen, KVLen, device, Q_BLOCK_SIZE=None, KV_BLOCK_SIZE=None) -> torch.Tensor:
    """Number of kept positions per block, int32 [b, h, nq, nk] with b in {1, B}, h in {1, H}
    (size 1 when the mask does not depend on that index).  One query-block row at a time."""
    qb = Q_BLOCK_SIZE or BLOCK_SIZE
    kb = KV_BLOCK_SIZE or BLOCK_SIZE
    nq, nk = -(-QLen // qb), -(-KVLen // kb)
    B = 1 if B is None else B
    H = 1 if H is None else H
    kv = torch.arange(nk * kb, device=device)
    rows = []
    for i in range(nq):
        q = torch.arange(i * qb, (i + 1) * qb, device=device)
        m = _eval_mask(mask_mod, B, H, q, kv, device)  # [b?, h?, qb, nk*kb] (broadcastable)
        m = m & (q.view(1, 1, -1, 1) < QLen) & (kv.view(1, 1, 1, -1) < KVLen)
        m = m.expand(m.shape[0], m.shape[1], qb, nk * kb)
        rows.append(m.reshape(m.shape[0], m.shape[1], qb, nk, kb).sum(dim=(2, 4), dtype=torch.int32))
    b = max(r.shape[0] for r in rows)
    h = max(r.shape[1] for r in rows)
    return torch.stack([r.expand(b, h, nk) for r in rows], dim=2)


def create_block_mask(mask_mod, B, H, QLen, KVLen, device, Q_BLOCK_SIZE=None, KV_BLOCK_SIZE=None):
    """int8 [B, H, QLen/Q_BLOCK, KVLen/KV_BLOCK]: 1 where the block keeps at least one position
    (reference: core.py:492-506).  Never materialises the dense mask."""
    B_ = 1 if B is None else B
    H_ = 1 if H is None else H
    cnt = block_mask_counts(mask_mod, B_, H_, QLen, KVLen, device, Q_BLOCK_SIZE, KV_BLOCK_SIZE)
    return (cnt > 0).to(torch.int8).expand(B_, H_, cnt.shape[2], cnt.shape[3]).contiguous()


def create_block_idx(mask_mod, B, H, QLen, KVLen, device, Q_BLOCK_SIZE=None, KV_BLOCK_SIZE=None):
    """Coordinates (b, h, q_block, kv_block) of the kept blocks (reference: core.py:508-512)."""
    return torch.nonzero(create_block_mask(mask_mod, B, H, QLen, KVLen, device, Q_BLOCK_SIZE, KV_BLOCK_SIZE),
                         as_tuple=False)


def is_causal_mask(mask_tensor, block_M, block_N):
    """True when the block mask equals the block pattern of ``q_idx >= kv_idx`` (reference: core.py:455-470)."""
    _, _, M, N = mask_tensor.shape
    q = torch.arange(M, device=mask_tensor.device).view(-1, 1)
    k = torch.arange(N, device=mask_tensor.device).view(1, -1)
    return torch.all(mask_tensor.bool() == ((q + 1) * block_M > k * block_N))


def is_less_causal_mask(mask_tensor, block_M, block_N):
    """True when no block strictly above the causal block diagonal is kept (reference: core.py:472-488)."""
    _, _, M, N = mask_tensor.shape
    q = torch.arange(M, device=mask_tensor.device).view(-1, 1)
    k = torch.arange(N, device=mask_tensor.device).view(1, -1)
    above = (q + 1) * block_M - 1 < k * block_N
    return torch.all(mask_tensor[..., above] == 0)
