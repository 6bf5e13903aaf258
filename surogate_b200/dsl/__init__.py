"""Python model DSL: nn-style modules traced to an explicit graph IR with ahead-of-time autodiff.

Parity: surogate/dsl/ (nn.py, graph_builder.py, py_compiler.py, hf.py, ir_builder.py).
"""
from . import nn, functional, hf, autodiff, ir  # noqa: F401
from . import models  # noqa: F401  (registers architectures)
from .compiler import build_dsl_ir_for_model, compile_model, CompiledModel  # noqa: F401
