"""Hand-written sm_100a ops (CUDA) with PyTorch-CPU twins."""
from . import functional  # noqa: F401
from .functional import (causal_attention, cross_entropy, embedding, layer_norm, layernorm_fork, linear, mlp,  # noqa: F401
                         rms_norm, rmsnorm_fork, rope, swiglu)
