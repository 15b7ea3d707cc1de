"""B200 (sm_100a) back end behind AttentionEngine's operator API.

``AttentionEngine``, ``OnlineFunc``, ``LinearAttentionEngine`` and the symbolic IR keep the
reference's names and signatures; the kernels underneath are hand-written tcgen05 / TMA CUDA,
compiled with NVRTC and launched through the C ABI in ``include/ae_b200.h``.
"""
import sys as _sys

from . import attn_engine, core
from .attn_engine import AttentionEngine, LinearAttentionEngine, OnlineFunc
from .core import (CustomIO, SymbolicArray, SymbolicTensor, SymbolScalar, Var, create_block_mask, meta_tensor)


def install_reference_aliases():
    """Make ``import attn_engine`` / ``import core`` (the reference's top-level package names, used by
    its attn_script/*.py examples) resolve to this package's modules."""
    _sys.modules.setdefault("attn_engine", attn_engine)
    _sys.modules.setdefault("core", core)
    _sys.modules.setdefault("core.utils", core.utils)
    _sys.modules.setdefault("core.transform", core.transform)


__all__ = ["AttentionEngine", "OnlineFunc", "LinearAttentionEngine", "CustomIO", "SymbolicArray", "SymbolicTensor",
           "SymbolScalar", "Var", "create_block_mask", "meta_tensor", "install_reference_aliases"]
