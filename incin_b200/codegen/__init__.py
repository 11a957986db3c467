"""Kernel fuser: pointwise expression trees -> one specialised sm_100a kernel per (expression, dtype, layout)."""
from .pointwise import (Arg, Binary, Const, KernelKey, Layout, PointwiseExpr, Scalar, Ternary, Unary, render_cuda)  # noqa: F401
from .runtime import FusedKernel, compile_pointwise, fused  # noqa: F401
from .shading import render_msl, render_wgsl  # noqa: F401,E402
from .rows import Col, Norm, fused_rows, reference_rows, render_row_cuda  # noqa: F401,E402
