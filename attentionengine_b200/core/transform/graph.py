"""Expression nodes of the symbolic IR.

Mirrors the node vocabulary of the reference (attention_engine/core/transform/graph.py:2-243:
Var, Const, Add, Sub, Mul, Div, Neg, Exp, Exp2, Log, Log2, Tanh, Abs, Max, MaxBwd,
ReduceSum/Max/AbsSum, ColReduceSum/Max/AbsSum) so that user scripts and isinstance / ``.type``
checks keep working.  A node only records its kind and operands; differentiation lives in
``core.SymbolScalar.backward`` and code generation in ``lower.cuda_lower``.
"""


class Node:
    arity = None  # number of operands, None = leaf

    def __init__(self, type: str, inputs=()):
        self.type = type
        self.inputs = list(inputs)
        self.grad = None

    def __str__(self):
        return f"{self.type}(" + "".join(f"{i}, " for i in self.inputs) + ")"

    __repr__ = __str__


class Var(Node):
    def __init__(self, name: str):
        super().__init__("Var")
        self.name = name

    def __str__(self):
        return f'Var("{self.name}")'


class Const(Node):
    def __init__(self, value: float):
        super().__init__("Const")
        self.value = value

    def __str__(self):
        return f"Const({self.value})"


def _make_op(name: str, arity: int):
    def __init__(self, *operands):
        if len(operands) != arity:
            raise TypeError(f"{name} takes {arity} operand(s), got {len(operands)}")
        Node.__init__(self, name, operands)

    return type(name, (Node,), {"__init__": __init__, "arity": arity})


ELEMENTWISE_UNARY = ("Neg", "Exp", "Exp2", "Log", "Log2", "Tanh", "Abs")
ELEMENTWISE_BINARY = ("Add", "Sub", "Mul", "Div", "Max")
ROW_REDUCE = ("ReduceSum", "ReduceMax", "ReduceAbsSum")
COL_REDUCE = ("ColReduceSum", "ColReduceMax", "ColReduceAbsSum")

for _n in ELEMENTWISE_UNARY + ROW_REDUCE + COL_REDUCE:
    globals()[_n] = _make_op(_n, 1)
for _n in ELEMENTWISE_BINARY:
    globals()[_n] = _make_op(_n, 2)
# MaxBwd(grad, out, other) = grad where out > other else 0  (reference emit: core/codegen/tl_gen.py:118-121)
MaxBwd = _make_op("MaxBwd", 3)

__all__ = ["Node", "Var", "Const", "MaxBwd"] + list(
    ELEMENTWISE_UNARY + ELEMENTWISE_BINARY + ROW_REDUCE + COL_REDUCE
)
