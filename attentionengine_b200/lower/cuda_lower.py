"""Lower traced IR expressions to CUDA C++ functor fragments.

Replaces the reference's lowering + codegen layers for the attention path
(attention_engine/core/lower/lower.py:318-614 ``lower_online_func`` / ``lower_score_mod`` /
``lower_custom_inputs`` and core/codegen/tl_gen.py:7-132,306-370), which emit TileLang statements
over tile buffers.  Here one query row is owned by one thread, so

* tile values ([block_M, block_N]) become ``float x[N]`` register arrays indexed by the column,
* row values ([block_M]) become scalars,
* row reductions become in-thread loops (no shuffles),

and the result is a *prelude*: ``#define``s plus ``__device__`` functions that the hand-written
kernel templates in ``csrc/kernels`` call.  Evaluation order follows the DAG (SSA), so the result
does not depend on operand order the way the reference's in-place buffer reuse does.
"""
from __future__ import annotations

import os

import math
import re
from dataclasses import dataclass, field
from typing import Callable, Optional

import torch

from ..core.transform.core import (CustomIO, SymbolicArray, SymbolicConst, SymbolicTensor, SymbolScalar)
from ..core.transform.graph import Var

NEG_INF_SENTINEL = "-1e38f"  # finite stand-in for a "-inf" initial row scale (reference: lower.py:23-29)


def _flit(x: float) -> str:
    if isinstance(x, str):
        x = x.strip()
        if x in ("-inf", "-float('inf')"):
            return NEG_INF_SENTINEL
        if x in ("inf", "float('inf')"):
            return "1e38f"
        x = float(x)
    if math.isinf(x):
        return NEG_INF_SENTINEL if x < 0 else "1e38f"
    r = repr(float(x))
    if "e" not in r and "." not in r:
        r += ".0"
    return r + "f"


def _is_number(s: str) -> bool:
    try:
        float(s)
        return True
    except ValueError:
        return s.strip() in ("-inf", "inf")


_RANK = {"const": 0, "uniform": 1, "row": 2, "tile": 3}


class Scal:
    """A non-tile scalar operand of an affine form: C++ expression plus its value when it is a
    compile-time constant (None otherwise)."""
    __slots__ = ("expr", "val")

    def __init__(self, expr: str, val=None):
        self.expr, self.val = expr, val


class Emitter:
    """Emits C++ for a set of root values.  ``env`` maps id(leaf SymbolScalar) or a leaf's Var
    name to a (C++ expression, kind) pair; tile-kind leaf expressions contain ``{c}`` where the
    column index goes.

    Tile values that are affine in another tile (x * a + b with row / uniform / constant a, b)
    are carried symbolically and only materialised when a non-affine consumer needs them, so that
    ``exp(score * scale - m)`` becomes one FFMA feeding ``ex2`` and ``rowmax(score * scale)``
    becomes ``scale * rowmax(score)``.  Row reductions use four interleaved accumulators.
    """

    def __init__(self, env_by_id: dict, env_by_name: dict, n_cols: str = "N", tile_mode: str = "array"):
        self.by_id = env_by_id
        self.by_name = env_by_name
        self.n = n_cols
        self.tile_mode = tile_mode  # "array": tiles are float[N]; "scalar": inside a per-element function
        self.lines: list[str] = []
        self.names: dict[int, tuple[str, str]] = {}   # id(value) -> (expr, kind), materialised
        self.aff: dict[int, tuple] = {}               # id(value) -> (base (expr, kind), a Scal|None, b Scal|None)
        self.used_leaves: set[str] = set()
        self.lazy_max: dict[int, int] = {}  # id(Max node) -> index of the operand that is the previous state
        # packed f32x2 multiply-add / add in the tile loops: off unless AE_B200_PACKED=1 (measured 1 - 4 % slower in the
        # forward kernel: the pack / unpack moves cost what the halved instruction count saves)
        self.packed = tile_mode == "array" and os.environ.get("AE_B200_PACKED", "0") == "1"
        self.k = 0

    # -- helpers -------------------------------------------------------------------------------
    def _tmp(self) -> str:
        self.k += 1
        return f"t{self.k}"

    def _scal(self, expr: str) -> Scal:
        try:
            return Scal(expr, float(expr.rstrip("f")))
        except ValueError:
            return Scal(expr, None)

    def _emit_scalar(self, expr: str) -> Scal:
        name = self._tmp()
        self.lines.append(f"const float {name} = {expr};")
        return Scal(name, None)

    def _s_mul(self, x, y):
        if x is None:
            return y
        if y is None:
            return x
        if x.val is not None and y.val is not None:
            return Scal(_flit(x.val * y.val), x.val * y.val)
        return self._emit_scalar(f"({x.expr} * {y.expr})")

    def _s_add(self, x, y):
        if x is None:
            return y
        if y is None:
            return x
        if x.val is not None and y.val is not None:
            return Scal(_flit(x.val + y.val), x.val + y.val)
        return self._emit_scalar(f"({x.expr} + {y.expr})")

    def _s_neg(self, x):
        if x is None:
            return None
        if x.val is not None:
            return Scal(_flit(-x.val), -x.val)
        return self._emit_scalar(f"(-{x.expr})")

    def _s_div(self, x, y):
        # x / y with x possibly None (= 1 for slope, = 0 for offset is handled by the caller)
        if x.val is not None and y.val is not None:
            return Scal(_flit(x.val / y.val), x.val / y.val)
        return self._emit_scalar(f"__fdividef({x.expr}, {y.expr})")

    # -- public ------------------------------------------------------------------------------------
    def ref(self, v: SymbolScalar, col: str = "c") -> str:
        expr, kind = self.value(v)
        if kind == "tile" and self.tile_mode == "array":
            return expr.replace("{c}", col)
        return expr

    def value(self, v: SymbolScalar) -> tuple[str, str]:
        """Materialised (expression, kind) of ``v``."""
        if id(v) in self.names:
            return self.names[id(v)]
        if id(v) not in self.aff:
            self._lower(v)
        if id(v) in self.names:
            return self.names[id(v)]
        base, a, b = self.aff[id(v)]
        res = self._materialise(base, a, b)
        self.names[id(v)] = res
        return res

    def affine(self, v: SymbolScalar):
        """(base, a, b) with base a materialised tile, for tile-kind ``v``."""
        if id(v) not in self.aff and id(v) not in self.names:
            self._lower(v)
        if id(v) in self.aff:
            return self.aff[id(v)]
        return (self.names[id(v)], None, None)

    def _tile_ref(self, base, col="c"):
        expr, _ = base
        return expr.replace("{c}", col) if self.tile_mode == "array" else expr

    def _affine_expr(self, base, a, b, col="c") -> str:
        x = self._tile_ref(base, col)
        if a is None and b is None:
            return x
        if a is None:
            return f"({x} + {b.expr})"
        if b is None:
            return f"({x} * {a.expr})"
        return f"fmaf({x}, {a.expr}, {b.expr})"

    def _new_tile(self, expr_of_c: str) -> tuple[str, str]:
        name = self._tmp()
        if self.tile_mode == "array":
            self.lines.append(f"float {name}[{self.n}];")
            self.lines.append(f"#pragma unroll\nfor (int c = 0; c < {self.n}; ++c) {name}[c] = {expr_of_c};")
            return name + "[{c}]", "tile"
        self.lines.append(f"const float {name} = {expr_of_c};")
        return name, "tile"

    def _materialise(self, base, a, b):
        if a is None and b is None:
            return base
        return self._new_tile(self._affine_expr(base, a, b))

    # -- lowering ------------------------------------------------------------------------------------
    def _leaf(self, v: SymbolScalar) -> tuple[str, str]:
        if id(v) in self.by_id:
            e = self.by_id[id(v)]
            self.used_leaves.add(v.varname)
            return e
        t = v.code.type
        if t == "Const":
            return _flit(v.code.value), "const"
        if t == "Var":
            nm = v.code.name
            if v.varname in self.by_name:
                self.used_leaves.add(v.varname)
                return self.by_name[v.varname]
            if nm in self.by_name:
                self.used_leaves.add(nm)
                return self.by_name[nm]
            if _is_number(nm):
                return _flit(nm), "const"
        raise KeyError(f"unbound symbolic value {v.varname!r} ({v.code})")

    def _kind_of(self, v: SymbolScalar) -> str:
        if id(v) in self.names:
            return self.names[id(v)][1]
        if id(v) in self.aff:
            return "tile"
        self._lower(v)
        return "tile" if id(v) in self.aff else self.names[id(v)][1]

    def _reduce(self, t: str, src_of_c) -> str:
        """Row reduction over the N columns with four interleaved accumulators.  With ``packed`` (N a multiple of 8) the
        sum takes two elements per instruction (packed f32x2 add): the row passes are issue-bound."""
        if self.tile_mode != "array":
            raise NotImplementedError("row reduction outside of online_fwd")
        name = self._tmp()
        if self.packed and t == "ReduceSum":  # N is a multiple of 8 (asserted in the functor)
            # (the three-input max of PTX assembles under nvcc 12.9 but not under NVRTC 12.9, so the maximum stays scalar)
            if True:
                self.lines.append("u64 " + ", ".join(f"{name}_{i} = 0ull" for i in range(4)) + ";")
                body = " ".join(f"{name}_{i} = ae_add2({name}_{i}, {src_of_c(f'c + {2 * i}')}, {src_of_c(f'c + {2 * i + 1}')});"
                                for i in range(4))
                self.lines.append(f"#pragma unroll\nfor (int c = 0; c < {self.n}; c += 8) {{ {body} }}")
                self.lines.append(f"float {name}_s[8];")
                for i in range(4):
                    self.lines.append(f"ae_unpack2f({name}_{i}, {name}_s[{2 * i}], {name}_s[{2 * i + 1}]);")
                self.lines.append(f"const float {name} = (({name}_s[0] + {name}_s[1]) + ({name}_s[2] + {name}_s[3])) + "
                                  f"(({name}_s[4] + {name}_s[5]) + ({name}_s[6] + {name}_s[7]));")
            return self._row_exchange(name, t)
        op = {"ReduceMax": "{a} = fmaxf({a}, {x});", "ReduceSum": "{a} += {x};", "ReduceAbsSum": "{a} += fabsf({x});"}[t]
        if t == "ReduceMax":
            inits = [src_of_c(str(i)) for i in range(4)]
            start = 4
        else:
            inits = ["0.f"] * 4
            start = 0
        self.lines.append("float " + ", ".join(f"{name}_{i} = {inits[i]}" for i in range(4)) + ";")
        body = " ".join(op.format(a=f"{name}_{i}", x=src_of_c(f"c + {i}")) for i in range(4))
        self.lines.append(f"#pragma unroll\nfor (int c = {start}; c < {self.n}; c += 4) {{ {body} }}")
        if t == "ReduceMax":
            self.lines.append(f"const float {name} = fmaxf(fmaxf({name}_0, {name}_1), fmaxf({name}_2, {name}_3));")
        else:
            self.lines.append(f"const float {name} = ({name}_0 + {name}_1) + ({name}_2 + {name}_3);")
        return self._row_exchange(name, t)

    def _row_exchange(self, name: str, t: str) -> str:
        """A kernel that gives one row's columns to several threads (AE_RSPLIT > 1) completes every row reduction across
        them; in every other build AE_ROW_XCHG is the identity."""
        self.lines.append(f"const float {name}x = AE_ROW_XCHG(st, {name}, {int(t == 'ReduceMax')});")
        return name + "x"

    def _lower(self, v: SymbolScalar):
        if not v.prev:
            self.names[id(v)] = self._leaf(v)
            return
        t = v.code.type
        kinds = [self._kind_of(p) for p in v.prev]
        # ---- row reductions ------------------------------------------------------------------
        if t in ("ReduceSum", "ReduceMax", "ReduceAbsSum"):
            if kinds[0] != "tile":
                raise NotImplementedError("row reduction of a non-tile value")
            base, a, b = self.affine(v.prev[0])
            if t == "ReduceMax" and (a is None or (a.val is not None and a.val > 0)):
                r = self._reduce(t, lambda col: self._tile_ref(base, col))
                if a is None and b is None:
                    self.names[id(v)] = (r, "row")
                else:
                    self.names[id(v)] = (self._emit_scalar(self._affine_expr((r, "row"), a, b)).expr, "row")
                return
            src = self.value(v.prev[0])
            r = self._reduce(t, lambda col: self._tile_ref(src, col))
            self.names[id(v)] = (r, "row")
            return
        if t in ("ColReduceSum", "ColReduceMax", "ColReduceAbsSum"):
            # split-KV merge: one split per lane, reductions over the split dimension are warp reductions
            if self.tile_mode != "lane":
                raise NotImplementedError("column reductions only exist in OnlineFunc.combine")
            x = self.ref(v.prev[0])
            fn = {"ColReduceSum": f"ae_warp_sum({x})", "ColReduceMax": f"ae_warp_max({x})",
                  "ColReduceAbsSum": f"ae_warp_sum(fabsf({x}))"}[t]
            name = self._tmp()
            self.lines.append(f"const float {name} = {fn};")
            self.names[id(v)] = (name, "row")
            return
        kind = max(kinds, key=lambda k: _RANK[k])
        if kind == "const":
            kind = "uniform"
        # ---- tile results: keep affine forms symbolic -----------------------------------------------------
        if kind == "tile":
            tiles = [i for i, k in enumerate(kinds) if k == "tile"]
            if len(tiles) == 1 and t in ("Mul", "Add", "Sub", "Div", "Neg"):
                i = tiles[0]
                base, a, b = self.affine(v.prev[i])
                if t == "Neg":
                    one = Scal("1.0f", 1.0)
                    self.aff[id(v)] = (base, self._s_neg(a if a is not None else one), self._s_neg(b))
                    return
                k = self._scal(self.ref(v.prev[1 - i]))
                if t == "Mul":
                    self.aff[id(v)] = (base, self._s_mul(a, k), self._s_mul(b, k) if b is not None else None)
                    return
                if t == "Add":
                    self.aff[id(v)] = (base, a, self._s_add(b, k))
                    return
                if t == "Sub":
                    if i == 0:
                        self.aff[id(v)] = (base, a, self._s_add(b, self._s_neg(k)))
                    else:
                        one = Scal("1.0f", 1.0)
                        self.aff[id(v)] = (base, self._s_neg(a if a is not None else one), self._s_add(k, self._s_neg(b)))
                    return
                if t == "Div" and i == 0:
                    one = Scal("1.0f", 1.0)
                    self.aff[id(v)] = (base, self._s_div(a if a is not None else one, k),
                                       self._s_div(b, k) if b is not None else None)
                    return
            if t in ("Exp", "Exp2"):
                base, a, b = self.affine(v.prev[0])
                if t == "Exp":
                    l2e = Scal("AE_LOG2E", 1.4426950408889634)
                    a = self._s_mul(a if a is not None else Scal("1.0f", 1.0), l2e)
                    b = self._s_mul(b, l2e) if b is not None else None
                idx = "c" if self.tile_mode == "array" else "sel"
                if self.packed and self.tile_mode == "array" and a is not None and b is not None:
                    # exp2(x * a + b) over the tile: the multiply-add on two elements per instruction
                    name = self._tmp()
                    x0, x1 = self._tile_ref(base, "c"), self._tile_ref(base, "c + 1")
                    self.lines.append(f"float {name}[{self.n}];")
                    self.lines.append(f"{{ const u64 {name}_a = ae_pack2f({a.expr}, {a.expr}), {name}_b = ae_pack2f({b.expr}, {b.expr});")
                    self.lines.append(f"#pragma unroll\nfor (int c = 0; c < {self.n}; c += 2) {{ float y0, y1; "
                                      f"ae_fma2(y0, y1, {x0}, {x1}, {name}_a, {name}_b); "
                                      f"{name}[c] = ae_exp2_mix(y0, c); {name}[c + 1] = ae_exp2_mix(y1, c + 1); }} }}")
                    self.names[id(v)] = (name + "[{c}]", "tile")
                    return
                self.names[id(v)] = self._new_tile(f"ae_exp2_mix({self._affine_expr(base, a, b)}, {idx})")
                return
            args = [self.ref(p, "c") for p in v.prev]
            self.names[id(v)] = self._new_tile(self._expr(t, args))
            return
        # ---- row / uniform scalars -----------------------------------------------------------------
        args = [self.ref(p, "c") for p in v.prev]
        name = self._tmp()
        if id(v) in self.lazy_max:  # running maximum kept while it grows by less than AE_LAZY_TAU
            i_old = self.lazy_max[id(v)]
            self.lines.append(f"const float {name} = ae_lazy_max({args[i_old]}, {args[1 - i_old]});")
        else:
            self.lines.append(f"const float {name} = {self._expr(t, args)};")
        self.names[id(v)] = (name, kind)

    @staticmethod
    def _expr(t: str, a: list[str]) -> str:
        if t == "Add":
            return f"({a[0]} + {a[1]})"
        if t == "Sub":
            return f"({a[0]} - {a[1]})"
        if t == "Mul":
            return f"({a[0]} * {a[1]})"
        if t == "Div":
            return f"__fdividef({a[0]}, {a[1]})"
        if t == "Neg":
            return f"(-{a[0]})"
        if t == "Abs":
            return f"fabsf({a[0]})"
        if t == "Max":
            return f"fmaxf({a[0]}, {a[1]})"
        if t == "Exp":
            return f"ae_exp({a[0]})"
        if t == "Exp2":
            return f"ae_exp2({a[0]})"
        if t == "Log":
            return f"ae_log({a[0]})"
        if t == "Log2":
            return f"ae_log2({a[0]})"
        if t == "Tanh":
            return f"ae_tanh({a[0]})"
        if t == "MaxBwd":
            return f"(({a[1]} > {a[2]}) ? {a[0]} : 0.f)"
        raise NotImplementedError(f"no CUDA lowering for IR op {t}")

    def body(self, indent: str = "  ") -> str:
        return "".join(indent + l + "\n" for l in self.lines)


# -------------------------------------------------------------------------------------------
# custom inputs
# -------------------------------------------------------------------------------------------
_DIM_SLOT = {"batch": 0, "heads": 1, "seq_len": 2, "seq_len_kv": 3}


@dataclass
class CustomSpec:
    name: str
    shape: tuple
    slot: int
    is_16bit: bool            # tile-shaped inputs travel in the q/k/v dtype, the rest in fp32
    dim_slots: list           # per tensor dim: index slot (0 b, 1 h, 2 q, 3 kv) or -1 for broadcast


def custom_specs(custom: CustomIO) -> list[CustomSpec]:
    specs = []
    for slot, (name, t) in enumerate(custom.input_tensors.items()):
        shape = tuple(t.shape_idx)
        dims = [(_DIM_SLOT[s] if s in _DIM_SLOT else -1) for s in shape]
        for s in shape:
            if s not in _DIM_SLOT and not (s.isdigit() and int(s) == 1):
                raise NotImplementedError(f"custom input {name}: dimension {s!r} is not one of "
                                          f"{sorted(_DIM_SLOT)} or 1")
        is16 = (2 in dims) and (3 in dims)
        specs.append(CustomSpec(name, shape, slot, is16, dims))
    if len(specs) > 4:
        raise NotImplementedError("at most 4 custom inputs are supported")
    return specs


def _custom_env(specs: list[CustomSpec], custom: CustomIO, bf16: bool, tile_mode: str, transposed: bool = False):
    env = {}
    for sp in specs:
        t = custom.input_tensors[sp.name]
        kind = "tile" if 3 in sp.dim_slots else ("row" if 2 in sp.dim_slots else "uniform")
        kv = "(kv0 + {c})" if tile_mode == "array" else "kv_idx"
        names = {0: "b", 1: "h", 2: "q_idx", 3: kv}
        terms = [f"(i64){names[d]} * cu.st[{sp.slot}][{d}]" for d in sorted(set(sp.dim_slots)) if d >= 0]
        idx = " + ".join(terms) if terms else "0"
        if sp.is_16bit:
            expr = f"ae_ld16<{1 if bf16 else 0}>(cu.p[{sp.slot}], {idx})"
        else:
            expr = f"((const float*)cu.p[{sp.slot}])[{idx}]"
        env[id(t)] = (expr, kind)
    return env


# -------------------------------------------------------------------------------------------
# the lowered bundle
# -------------------------------------------------------------------------------------------
@dataclass
class LoweredAttention:
    prelude_fwd: str
    prelude_bwd: str
    final_names: list[str]
    custom: list[CustomSpec]
    o_scale_one: bool
    uses_doosum: bool
    has_mask: bool
    defines: dict = field(default_factory=dict)


def _trace_mask(mask_mod: Optional[Callable]) -> Optional[str]:
    """C++ boolean expression over (b, h, q_idx, kv_idx) for ``mask_mod`` (reference: fx trace of
    the mask restricted to python operators and logical_and, core/codegen/common.py:124-152).
    Traced with a tiny operator-overloading value instead of torch.fx."""
    if mask_mod is None:
        return None

    class E:
        def __init__(self, s):
            self.s = s

        def _b(self, o, op):
            return E(f"({self.s} {op} {_e(o)})")

        def _rb(self, o, op):
            return E(f"({_e(o)} {op} {self.s})")

        __add__ = lambda a, o: a._b(o, "+")
        __radd__ = lambda a, o: a._rb(o, "+")
        __sub__ = lambda a, o: a._b(o, "-")
        __rsub__ = lambda a, o: a._rb(o, "-")
        __mul__ = lambda a, o: a._b(o, "*")
        __rmul__ = lambda a, o: a._rb(o, "*")
        __floordiv__ = lambda a, o: a._b(o, "/")
        __mod__ = lambda a, o: a._b(o, "%")
        __ge__ = lambda a, o: a._b(o, ">=")
        __gt__ = lambda a, o: a._b(o, ">")
        __le__ = lambda a, o: a._b(o, "<=")
        __lt__ = lambda a, o: a._b(o, "<")
        __eq__ = lambda a, o: a._b(o, "==")
        __ne__ = lambda a, o: a._b(o, "!=")
        __and__ = lambda a, o: a._b(o, "&&")
        __rand__ = lambda a, o: a._rb(o, "&&")
        __or__ = lambda a, o: a._b(o, "||")
        __ror__ = lambda a, o: a._rb(o, "||")
        __invert__ = lambda a: E(f"(!{a.s})")
        __neg__ = lambda a: E(f"(-{a.s})")
        __hash__ = None

        def __bool__(self):
            raise TypeError("mask_mod must not branch on index values; combine conditions with & and |")

        @classmethod
        def __torch_function__(cls, func, types, args=(), kwargs=None):
            nm = getattr(func, "__name__", "")
            if nm == "logical_and":
                return E(f"({_e(args[0])} && {_e(args[1])})")
            if nm == "logical_or":
                return E(f"({_e(args[0])} || {_e(args[1])})")
            if nm == "logical_not":
                return E(f"(!{_e(args[0])})")
            if nm == "abs":
                return E(f"abs({_e(args[0])})")
            raise NotImplementedError(f"mask_mod uses torch.{nm}, which has no CUDA lowering")

    def _e(o):
        if isinstance(o, E):
            return o.s
        if isinstance(o, bool):
            return "true" if o else "false"
        if isinstance(o, int):
            return str(o)
        raise TypeError(f"mask_mod mixes index values with {type(o).__name__}")

    out = mask_mod(E("b"), E("h"), E("q_idx"), E("kv_idx"))
    return _e(out)


_LD16 = """
template <int kBf16>
AE_DEVICE float ae_ld16(const void* p, i64 idx) {
  const u16 w = ((const u16*)p)[idx];
  return unpack_lo<kBf16>((u32)w);
}
"""


def lower_combine(online_func) -> str:
    """``OnlineFunc.combine`` (split-KV merge weights) as a per-lane functor: lane k holds the final row
    scales of split k; reductions over the split dimension become warp reductions.  Reference:
    core/lower/lower_decode.py:287-317."""
    from ..core.transform.core import SymbolicColReduceArray
    fr, env = {}, {}
    for i, (k, v) in enumerate(online_func.final_rowscales.items()):
        s = SymbolicColReduceArray(k, Var(k), shape_idx=["num_split", "block_M2"])
        fr[k] = s
        env[id(s)] = (f"fr[{i}]", "tile")
    w = online_func.combine(fr)
    em = Emitter(env, {}, tile_mode="lane")
    res = em.ref(w)
    return ("AE_DEVICE float ae_combine(const float* fr) {\n  const int sel = 0; (void)sel;\n" + em.body() + f"  return {res};\n}}\n")


LAZY_TAU = 5.0  # a running maximum is kept while it would grow by less than this (P then stays below e^5 = 148)


def _lazy_max_candidates(rs_in: dict, new_rs: dict) -> dict[int, int]:
    """Row states updated as max(previous value, something): id(Max node) -> operand index of the previous value."""
    out = {}
    for k, v in new_rs.items():
        if isinstance(v, SymbolScalar) and v.code.type == "Max" and len(v.prev) == 2 and k in rs_in:
            for i in (0, 1):
                if v.prev[i] is rs_in[k]:
                    out[id(v)] = i
    return out


def _lazy_max_is_invariant(online_func, raw, t_scores, rs_in, new_scores, new_rs, o_scale, lazy) -> bool:
    """Numerical test, on the traced recurrence itself, that keeping a stale running maximum changes no result:
    runs the tile-by-tile recurrence (O = O * o_scale + P V) on random scores with and without the lazy rule and
    compares the epilogue's outputs and final row scales.  True for the softmax family (the states are only used
    through differences that cancel), False for anything else, which then keeps the exact maximum."""
    from .torch_eval import evaluate
    try:
        g = torch.Generator().manual_seed(7)
        R, N, T, DV = 16, 32, 6, 8
        scores = [torch.randn(R, N, generator=g, dtype=torch.float64) * (1.0 + 3.0 * t) for t in range(T)]
        vals = [torch.randn(N, DV, generator=g, dtype=torch.float64) for _ in range(T)]
        init = {k: float(str(v.code.name if v.code.type == "Var" else v.code.value).replace("inf", "1e30"))
                for k, v in online_func.online_rowscales.items()}
        zero = {id(x): torch.zeros(1, dtype=torch.float64) for x in ()}

        def run(lazy_on: bool):
            st = {k: torch.full((R, 1), init[k], dtype=torch.float64) for k in rs_in}
            o = torch.zeros(R, DV, dtype=torch.float64)
            hooks = None
            if lazy_on:
                def mk(i_old):
                    return lambda a: torch.where(a[1 - i_old] - a[i_old] > LAZY_TAU, a[1 - i_old] + 0 * a[i_old], a[i_old] + 0 * a[1 - i_old])
                hooks = {nid: mk(i) for nid, i in lazy.items()}
            for t in range(T):
                env = {id(rs_in[k]): st[k] for k in rs_in}
                env[id(raw)] = scores[t]
                cache = {}
                p = evaluate(new_scores, env, cache, hooks)
                osc = evaluate(o_scale, env, cache, hooks)
                st = {k: torch.as_tensor(evaluate(v, env, cache, hooks), dtype=torch.float64).expand(R, 1).clone()
                      for k, v in new_rs.items()}
                o = o * osc + torch.as_tensor(p) @ vals[t]
            o_sym = SymbolicArray("o", Var("o"), shape_idx=["block_M", "dimv"])
            rs_ep = {k: SymbolScalar(k, Var(k), shape_idx=["block_M"]) for k in rs_in}
            o_new, finals = online_func.online_fwd_epilogue(o_sym, rs_ep, None, None, None)
            env = {id(rs_ep[k]): st[k] for k in rs_in}
            env[id(o_sym)] = o
            return [torch.as_tensor(evaluate(o_new, env))] + [torch.as_tensor(evaluate(f, env)) for f in finals.values()]

        a, b_ = run(False), run(True)
        return all(torch.isfinite(x).all() and torch.allclose(x, y, rtol=1e-9, atol=1e-9) for x, y in zip(a, b_))
    except Exception:  # anything the eager evaluator cannot run keeps the exact maximum
        return False


def lower_attention(score_mod, mask_mod, online_func, custom_fwd_inputs: CustomIO, *, D: int, DV: int, bf16: bool,
                    mask_mode: int, stages: int = 2, mask_value: str = "-inf") -> LoweredAttention:
    """Trace the user callables and produce the kernel preludes.

    Order of operations per score tile follows the reference forward kernel
    (core/template/tl_template/attn/attn_tl.py:124-164): mask (to ``mask_value``) -> score_mod ->
    online_fwd -> rescale O by o_scale -> O += P V; after the loop online_fwd_epilogue.  The backward
    fragments follow attn_tl.py:348-403: score_mod, OnlineFunc.forward with the saved final
    rowscales, OnlineFunc.backward (its ``scores`` argument is P), score_mod's derivative.
    """
    specs = custom_specs(custom_fwd_inputs)
    idx_env = {"b": ("(float)b", "uniform"), "h": ("(float)h", "uniform"), "q_idx": ("(float)q_idx", "row"),
               "kv_idx": ("(float)kv_idx", "tile")}

    def sym_idx(name):
        return SymbolScalar(name, Var(name), shape_idx=["block_N"] if name == "kv_idx" else (
            ["block_M"] if name == "q_idx" else ["1"]), require_grad=False)

    src = []
    src.append(_LD16)

    # ---- mask ---------------------------------------------------------------------------------
    mask_expr = _trace_mask(mask_mod)
    src.append("AE_DEVICE bool ae_mask(int b, int h, int q_idx, int kv_idx) { return %s; }\n" %
               (mask_expr if mask_expr is not None else "true"))

    # ---- score_mod (per element; kept for kernels that want the plain composition) ---------------------
    def trace_score_mod(scores=None):
        scores = scores if scores is not None else SymbolicArray("scores", Var("scores"), shape_idx=["block_M", "block_N"])
        out = score_mod(scores, custom_fwd_inputs, sym_idx("b"), sym_idx("h"), sym_idx("q_idx"), sym_idx("kv_idx"))
        if not isinstance(out, SymbolScalar):
            out = SymbolScalar._wrap(out)
        return scores, out

    scores, out = trace_score_mod()
    env = _custom_env(specs, custom_fwd_inputs, bf16, "scalar")
    env[id(scores)] = ("s", "tile")
    em = Emitter(env, idx_env, tile_mode="scalar")
    res = em.ref(out)
    src.append("AE_DEVICE float ae_score_mod(float s, int b, int h, int q_idx, int kv_idx, const AeCustom& cu) {\n  const int sel = 0; (void)sel;\n"
               + em.body() + f"  return {res};\n}}\n")

    # ---- online_fwd fused with score_mod (per row, N columns) --------------------------------------------
    state_names = list(online_func.online_rowscales.keys())
    state_init = {k: v.code.name if v.code.type == "Var" else str(v.code.value)
                  for k, v in online_func.online_rowscales.items()}
    row_struct = "struct AeRow {\n"
    if state_names:
        row_struct += "  float " + ", ".join(f"st_{k}" for k in state_names) + ";\n"
    row_struct += ("#if AE_RSPLIT > 1\n  volatile float* xch; u32 xme, xother, xbar, xn, xphase;\n#endif\n")
    row_struct += "  AE_DEVICE void init() {" + " ".join(
        f"st_{k} = {_flit(state_init[k])};" for k in state_names) + " }\n};\n"
    # the threads that share a row publish their partial reduction in shared memory (two alternating slot sets, so that
    # the next exchange cannot overwrite a value a slower partner has yet to read), meet at a named barrier and combine
    row_struct += (
        "#if AE_RSPLIT > 1\n"
        "AE_DEVICE float ae_row_xchg(AeRow& st, float x, int is_max) {\n"
        "  volatile float* slot = st.xch + (st.xphase & 1u) * (AE_RSPLIT * 128);\n"
        "  slot[st.xme] = x;\n"
        "  named_bar_sync(st.xbar, st.xn);\n"
        "  const float y = slot[st.xother];\n"
        "  st.xphase++;\n"
        "  return is_max ? fmaxf(x, y) : x + y;\n"
        "}\n"
        "#define AE_ROW_XCHG(st, x, is_max) ae_row_xchg(st, x, is_max)\n"
        "#else\n"
        "#define AE_ROW_XCHG(st, x, is_max) (x)\n"
        "#endif\n")
    src.append(row_struct)

    raw, t_scores = trace_score_mod()
    rs_in = {}
    env = _custom_env(specs, custom_fwd_inputs, bf16, "array")
    for k in state_names:
        v = SymbolScalar(k, Var(k), shape_idx=["block_M"])
        rs_in[k] = v
        env[id(v)] = (f"st.st_{k}", "row")
    env[id(raw)] = ("s[{c}]", "tile")
    new_scores, new_rs, o_scale = online_func.online_fwd(t_scores, dict(rs_in), sym_idx("b"), sym_idx("h"),
                                                          sym_idx("q_idx"))
    arr_idx_env = dict(idx_env)
    arr_idx_env["kv_idx"] = ("(float)(kv0 + {c})", "tile")
    em = Emitter(env, arr_idx_env, n_cols="N")
    lazy = _lazy_max_candidates(rs_in, new_rs)
    if lazy and not specs and _lazy_max_is_invariant(online_func, raw, t_scores, rs_in, new_scores, new_rs, o_scale, lazy):
        em.lazy_max = lazy
    o_expr, o_kind = em.value(o_scale)
    o_scale_one = (o_kind == "const" and float(o_expr.rstrip("f")) == 1.0)
    new_exprs = {k: em.ref(v) for k, v in new_rs.items()}
    p_expr = em.ref(new_scores, "c")
    body = em.body()
    body += "".join(f"  const float n_{k} = {e};\n" for k, e in new_exprs.items())
    body += f"  const float o_scale_ = {o_expr};\n"
    if p_expr != "s[c]":
        body += f"  #pragma unroll\nfor (int c = 0; c < N; ++c) s[c] = {p_expr};\n"
    body += "".join(f"  st.st_{k} = n_{k};\n" for k in new_exprs)
    src.append("// s[] holds the raw (masked) scores q.k on entry and P on exit: score_mod and online_fwd in one pass\n"
               "template <int N>\nAE_DEVICE float ae_online_fwd(float (&s)[N], AeRow& st, int b, int h, int q_idx, "
               "int kv0, const AeCustom& cu) {\n  static_assert(N % 8 == 0, \"tile loops take eight columns at a time\");\n"
               + body + "  return o_scale_;\n}\n")

    # ---- epilogue --------------------------------------------------------------------------------------
    o_sym = SymbolicArray("o", Var("o"), shape_idx=["block_M", "dimv"])
    rs_ep = {}
    env = {}
    for k in state_names:
        v = SymbolScalar(k, Var(k), shape_idx=["block_M"])
        rs_ep[k] = v
        env[id(v)] = (f"st.st_{k}", "row")
    env[id(o_sym)] = ("o", "row")
    o_new, finals = online_func.online_fwd_epilogue(o_sym, rs_ep, sym_idx("b"), sym_idx("h"), sym_idx("q_idx"))
    em = Emitter(env, {}, tile_mode="scalar")
    res = em.ref(o_new)
    src.append("AE_DEVICE float ae_epilogue_o(float o, const AeRow& st) {\n  const int sel = 0; (void)sel;\n" + em.body() + f"  return {res};\n}}\n")
    final_names = list(finals.keys())
    if len(final_names) > 4:
        raise NotImplementedError("at most 4 final rowscales are supported")
    em = Emitter(env, {}, tile_mode="scalar")
    fl = [em.ref(v) for v in finals.values()]
    src.append("AE_DEVICE void ae_final_rowscales(const AeRow& st, float* out) {\n  const int sel = 0; (void)sel;\n" + em.body()
               + "".join(f"  out[{i}] = {e};\n" for i, e in enumerate(fl)) + "}\n")

    # ---- backward fragments: P = forward(score_mod(S)); dS = score_mod'(S) * backward(dP, P) ---------------------
    bsrc = []
    fr = {}
    fr_env = {}
    for i, k in enumerate(final_names):
        v = SymbolScalar(k, Var(k), shape_idx=["block_M"], require_grad=False)
        fr[k] = v
        fr_env[id(v)] = (f"fr[{i}]", "row")
    raw_p, t_p = trace_score_mod()
    env = _custom_env(specs, custom_fwd_inputs, bf16, "scalar")
    env.update(fr_env)
    env[id(raw_p)] = ("s", "tile")
    p_out = online_func.forward(t_p, fr, sym_idx("b"), sym_idx("h"), sym_idx("q_idx"), sym_idx("kv_idx"))
    em = Emitter(env, idx_env, tile_mode="scalar")
    res = em.ref(p_out)
    bsrc.append("// P from the raw score: OnlineFunc.forward(score_mod(s)) with the saved final row scales\n"
                "AE_DEVICE float ae_bwd_p(float s, const float* fr, int b, int h, int q_idx, int kv_idx, "
                "const AeCustom& cu, const int sel = 0) {\n" + em.body() + f"  return {res};\n}}\n")

    dp = SymbolScalar("dp", Var("dp"), shape_idx=["block_M", "block_N"], require_grad=False)
    pp = SymbolScalar("p", Var("p"), shape_idx=["block_M", "block_N"], require_grad=False)
    doosum = SymbolScalar("doosum", Var("doosum"), shape_idx=["block_M"], require_grad=False)
    d_t = online_func.backward(dp, pp, fr, doosum, sym_idx("b"), sym_idx("h"), sym_idx("q_idx"), sym_idx("kv_idx"))
    if not isinstance(d_t, SymbolScalar):
        d_t = SymbolScalar._wrap(d_t)
    raw_b, out_b = trace_score_mod()
    d_t.require_grad = False
    out_b.backward(d_t)
    env = _custom_env(specs, custom_fwd_inputs, bf16, "scalar")
    env.update(fr_env)
    env[id(raw_b)] = ("s", "tile")
    env[id(dp)] = ("dp", "tile")
    env[id(pp)] = ("p", "tile")
    env[id(doosum)] = ("doosum", "row")
    em = Emitter(env, idx_env, tile_mode="scalar")
    gres = em.ref(raw_b.grad) if raw_b.grad is not None else "0.f"
    uses_doosum = "doosum" in em.used_leaves
    ds_body = em.body()
    # score_mod'(s) needs the raw score again only when score_mod is not affine in it
    ds_uses_s = re.search(r"\bs\b", ds_body + str(gres)) is not None
    bsrc.append("// dS from dP and P: score_mod'(s) * OnlineFunc.backward(dp, p, final row scales, doosum)\n"
                "AE_DEVICE float ae_bwd_ds(float s, float dp, float p, const float* fr, float doosum, int b, int h, "
                "int q_idx, int kv_idx, const AeCustom& cu) {\n  const int sel = 0; (void)sel;\n" + em.body() + f"  return {gres};\n}}\n")

    defines = {
        "AE_D": D, "AE_DV": DV, "AE_BF16": int(bf16), "AE_STAGES": stages, "AE_MASK_MODE": mask_mode,
        "AE_NFINAL": len(final_names), "AE_O_SCALE_ONE": int(o_scale_one), "AE_USES_DOOSUM": int(uses_doosum),
        "AE_DS_USES_S": int(ds_uses_s),
        "AE_MASK_NEG_INF": int(str(mask_value).strip() in ("-inf", "-float('inf')")),
    }
    head = ("".join(f"#define {k} {v}\n" for k, v in defines.items())
            + "#ifndef AE_RSPLIT\n#define AE_RSPLIT 1  // threads per score row in the kernel that includes this\n#endif\n"
            + "struct AeCustom;\n")
    fwd = head + "".join(src)
    bwd = fwd + "".join(bsrc)
    return LoweredAttention(prelude_fwd=fwd, prelude_bwd=bwd, final_names=final_names, custom=specs,
                            o_scale_one=o_scale_one, uses_doosum=uses_doosum, has_mask=mask_mod is not None,
                            defines=defines)
