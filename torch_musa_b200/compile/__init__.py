"""Compile stack of the blackwell backend: FX passes, CUDA C++ code generation for fused element-wise
groups, a native graph runner, graph trees, and ahead-of-time packages (``export``)."""
from . import codegen, lower, graph_trees, backend  # noqa: F401
from .backend import blackwell, register, stats  # noqa: F401
from .graph_trees import mark_static  # noqa: F401
