"""Small helpers kept for API compatibility with the reference (attention_engine/core/utils.py)."""


class IndentedCode:
    """Accumulates lines of text at a running indentation level (reference: core/utils.py:4-33)."""

    def __init__(self, indent: int = 0, unit: str = "    "):
        self.indent = indent
        self.unit = unit
        self.lines = []

    @property
    def code(self) -> str:
        return "".join(l + "\n" for l in self.lines)

    def __str__(self):
        return self.code

    def add_line(self, line: str):
        self.lines.append(self.unit * self.indent + line)

    def __iadd__(self, other):
        if isinstance(other, str):
            self.add_line(other)
        elif isinstance(other, IndentedCode):
            for l in other.lines:
                if l.strip():
                    self.add_line(l)
        else:
            raise TypeError(type(other))
        return self

    def more_indent(self, n: int = 1):
        self.indent += n

    def less_indent(self, n: int = 1):
        self.indent -= n


class meta_tensor:
    """Shape/dtype record in (B, H, S, D) order; dims may be ints or names for dynamic
    shapes (reference: core/utils.py:40-47)."""

    def __init__(self, *shape, **kwargs):
        self.shape = shape
        self.kargs = kwargs

    @property
    def dtype(self):
        return self.kargs["dtype"]

    def __repr__(self):
        return f"meta_tensor{self.shape}"
