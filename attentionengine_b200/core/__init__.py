"""Symbolic IR front end.  Same import surface as the reference's ``core`` package
(attention_engine/core/__init__.py:1-2) plus ``create_block_mask``, which the reference README
imports from here (README.md:63) although its ``core/__init__.py`` forgets to export it."""
from .transform.core import (CustomIO, SymbolicArray, SymbolicColReduceArray, SymbolicConst, SymbolicTensor,
                             SymbolScalar, Var, create_block_idx, create_block_mask, create_mask, is_causal_mask,
                             is_less_causal_mask)
from .utils import IndentedCode, meta_tensor

__all__ = ["CustomIO", "SymbolicArray", "SymbolicColReduceArray", "SymbolicConst", "SymbolicTensor", "SymbolScalar",
           "Var", "create_block_idx", "create_block_mask", "create_mask", "is_causal_mask", "is_less_causal_mask",
           "IndentedCode", "meta_tensor"]
