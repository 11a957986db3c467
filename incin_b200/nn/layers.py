"""Layers.  Modules are ``torch.nn.Module``s (PyTorch is the framework layer) whose forward goes through
:mod:`incin_b200.ops.functional`, so bf16 CUDA tensors hit the hand-written sm_100a kernels and
everything else runs the PyTorch twin.

Surface and conventions follow crates/incin-core/src/nn: Linear stores ``weight [out, in]`` and
``bias [out]`` (linear.rs:46-53) with Kaiming-uniform init, Embedding initialises N(0,1)
(embedding.rs:59-90), LayerNorm/RMSNorm (layer_norm.rs, rms_norm.rs), Dropout, Flatten, pools, RNN/LSTM
cells, activations (ReLU, GELU exact-erf, Swish, Mish, ELU, Softmax, Sigmoid, Tanh), ``Sequential`` with
flat PyTorch-style numbering (module.rs:18-33) and ``ComputeStats`` (parameter / FLOP accounting).
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn.functional as TF
from torch import nn

from ..ops import functional as F
from .init import Init, initialize

_default_generator: torch.Generator | None = None


def manual_seed(seed: int) -> None:
    """Seed the generator module initialisers draw from (defines "seed 0" for every builder below)."""
    global _default_generator
    _default_generator = torch.Generator().manual_seed(seed)


def _gen() -> torch.Generator | None:
    return _default_generator


class Param(nn.Parameter):
    """A trainable tensor; ``Buffer`` is its non-trainable counterpart (nn/param.rs)."""


def Buffer(t: torch.Tensor) -> torch.Tensor:
    t.requires_grad_(False)
    return t


class Linear(nn.Module):
    def __init__(self, in_features: int, out_features: int, bias: bool = True, init: Init = Init.KAIMING_UNIFORM,
                 act: str | None = None):
        super().__init__()
        self.in_features, self.out_features, self.act = in_features, out_features, act
        self.weight = Param(initialize(torch.empty(out_features, in_features), init, generator=_gen()))
        self.bias = Param(initialize(torch.empty(out_features), Init.KAIMING_UNIFORM, generator=_gen(),
                                     fan_in=in_features)) if bias else None

    def forward(self, x, residual=None):
        return F.linear(x, self.weight, self.bias, act=self.act, residual=residual)

    def flops(self, rows: int) -> int:
        return 2 * rows * self.in_features * self.out_features


class LayerNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-5, bias: bool = True):
        super().__init__()
        self.eps = eps
        self.weight = Param(torch.ones(dim))
        self.bias = Param(torch.zeros(dim)) if bias else None

    def forward(self, x):
        return F.layer_norm(x, self.weight, self.bias, self.eps)


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-5):
        super().__init__()
        self.eps = eps
        self.weight = Param(torch.ones(dim))

    def forward(self, x):
        return F.rms_norm(x, self.weight, self.eps)


class Embedding(nn.Module):
    def __init__(self, num: int, dim: int, init: Init = Init.RANDN, std: float = 0.02):
        super().__init__()
        self.weight = Param(initialize(torch.empty(num, dim), init, generator=_gen(), std=std))

    def forward(self, tokens):
        if tokens.dim() == 2:
            return F.embedding(tokens, self.weight, None)
        return TF.embedding(tokens, self.weight)


class Dropout(nn.Module):
    """Inverted dropout; on CUDA/bf16 the mask is regenerated from (seed, offset) by the Philox kernel."""

    def __init__(self, p: float = 0.5, seed: int = 0):
        super().__init__()
        if not 0.0 <= p < 1.0:
            raise ValueError("dropout probability must be in [0, 1)")
        self.p, self.seed, self._calls = p, seed, 0

    def forward(self, x):
        if not self.training or self.p == 0.0:
            return x
        self._calls += 1
        return F.dropout(x, self.p, self.seed, self._calls)


class Flatten(nn.Module):
    def __init__(self, start_dim: int = 1):
        super().__init__()
        self.start_dim = start_dim

    def forward(self, x):
        return x.flatten(self.start_dim)


class _Act(nn.Module):
    fn = staticmethod(lambda x: x)

    def forward(self, x):
        return type(self).fn(x)


class ReLU(_Act):
    fn = staticmethod(TF.relu)


class GELU(_Act):
    fn = staticmethod(lambda x: F.activation(x, "gelu"))   # exact erf form: the CPU/CUDA contract


class GELUTanh(_Act):
    fn = staticmethod(lambda x: TF.gelu(x, approximate="tanh"))  # the WGSL shader's approximation, restated


class Swish(_Act):
    fn = staticmethod(lambda x: F.activation(x, "silu"))


class Mish(_Act):
    fn = staticmethod(TF.mish)


class ELU(_Act):
    fn = staticmethod(TF.elu)


class Sigmoid(_Act):
    fn = staticmethod(torch.sigmoid)


class Tanh(_Act):
    fn = staticmethod(torch.tanh)


class Softmax(nn.Module):
    def __init__(self, dim: int = -1):
        super().__init__()
        self.dim = dim

    def forward(self, x):
        from ..ops.tensor_ops import softmax
        return softmax(x, self.dim)


class Conv2d(nn.Conv2d):
    """NCHW convolution (conv2d.rs); CPU and fp32 run ATen, the bf16 CUDA path lowers to im2col + tcgen05 GEMM."""

    def forward(self, x):
        if x.is_cuda and x.dtype == torch.bfloat16 and self.groups == 1 and self.padding_mode == "zeros" and \
                not isinstance(self.padding, str):
            from ..ops.tensor_ops import conv2d
            return conv2d(x, self.weight, self.bias, self.stride, self.padding, self.dilation)
        return super().forward(x)


class Conv1d(nn.Conv1d):
    """``[N, C, L]`` convolution; the bf16 CUDA path is the 2-D lowering over a height of 1 (conv1d in
    crates/incin-backends/src/cuda/backend.rs:1576)."""

    def forward(self, x):
        if x.is_cuda and x.dtype == torch.bfloat16 and self.groups == 1 and self.padding_mode == "zeros" and \
                not isinstance(self.padding, str):
            from ..ops.tensor_ops import conv1d
            return conv1d(x, self.weight, self.bias, self.stride[0], self.padding[0], self.dilation[0])
        return super().forward(x)


class ConvTranspose2d(nn.ConvTranspose2d):
    """Transposed NCHW convolution (crates/incin-backends/src/cuda/backend.rs:1604); bf16 CUDA tensors run GEMM + fold."""

    def forward(self, x, output_size=None):
        if x.is_cuda and x.dtype == torch.bfloat16 and self.groups == 1 and output_size is None:
            from ..ops.tensor_ops import conv_transpose2d
            return conv_transpose2d(x, self.weight, self.bias, self.stride, self.padding, self.output_padding, self.dilation)
        return super().forward(x, output_size)

class BatchNorm2d(nn.Module):
    """Per-channel batch normalisation over ``[N, C, H, W]`` (crates/incin-core/src/nn/batch_norm.rs): fp32 affine
    parameters and running statistics, training forward + backward and the inference form on the native kernels."""

    def __init__(self, num_features: int, eps: float = 1e-5, momentum: float = 0.1, affine: bool = True):
        super().__init__()
        self.num_features, self.eps, self.momentum = num_features, eps, momentum
        self.weight = nn.Parameter(torch.ones(num_features)) if affine else None
        self.bias = nn.Parameter(torch.zeros(num_features)) if affine else None
        self.register_buffer("running_mean", torch.zeros(num_features))
        self.register_buffer("running_var", torch.ones(num_features))

    def forward(self, x):
        from ..ops.tensor_ops import batch_norm
        return batch_norm(x, self.weight, self.bias, self.running_mean, self.running_var, self.training, self.momentum,
                          self.eps)


class MaxPool2d(nn.Module):
    def __init__(self, kernel_size, stride=None, padding=0):
        super().__init__()
        self.kernel_size, self.stride, self.padding = kernel_size, stride, padding

    def forward(self, x):
        from ..ops.tensor_ops import max_pool2d
        return max_pool2d(x, self.kernel_size, self.stride, self.padding)


class AvgPool2d(nn.Module):
    def __init__(self, kernel_size, stride=None, padding=0):
        super().__init__()
        self.kernel_size, self.stride, self.padding = kernel_size, stride, padding

    def forward(self, x):
        from ..ops.tensor_ops import avg_pool2d
        return avg_pool2d(x, self.kernel_size, self.stride, self.padding)


class AdaptiveAvgPool2d(nn.Module):
    def __init__(self, output_size):
        super().__init__()
        self.output_size = output_size

    def forward(self, x):
        from ..ops.tensor_ops import adaptive_avg_pool2d
        return adaptive_avg_pool2d(x, self.output_size)


class RNNCell(nn.Module):
    def __init__(self, input_size: int, hidden_size: int):
        super().__init__()
        self.ih, self.hh = Linear(input_size, hidden_size), Linear(hidden_size, hidden_size)

    def forward(self, x, h):
        return torch.tanh(self.ih(x) + self.hh(h))


class LSTMCell(nn.Module):
    def __init__(self, input_size: int, hidden_size: int):
        super().__init__()
        self.hidden_size = hidden_size
        self.ih, self.hh = Linear(input_size, 4 * hidden_size), Linear(hidden_size, 4 * hidden_size)

    def forward(self, x, state):
        h, c = state
        i, f, g, o = (self.ih(x) + self.hh(h)).chunk(4, dim=-1)
        c = torch.sigmoid(f) * c + torch.sigmoid(i) * torch.tanh(g)
        h = torch.sigmoid(o) * torch.tanh(c)
        return h, c


class RNN(nn.Module):
    def __init__(self, input_size: int, hidden_size: int):
        super().__init__()
        self.cell, self.hidden_size = RNNCell(input_size, hidden_size), hidden_size

    def forward(self, x, h=None):   # x: [B, T, I]
        h = x.new_zeros(x.shape[0], self.hidden_size) if h is None else h
        out = []
        for t in range(x.shape[1]):
            h = self.cell(x[:, t], h)
            out.append(h)
        return torch.stack(out, 1), h


class LSTM(nn.Module):
    def __init__(self, input_size: int, hidden_size: int):
        super().__init__()
        self.cell, self.hidden_size = LSTMCell(input_size, hidden_size), hidden_size

    def forward(self, x, state=None):
        if state is None:
            z = x.new_zeros(x.shape[0], self.hidden_size)
            state = (z, z)
        out = []
        for t in range(x.shape[1]):
            state = self.cell(x[:, t], state)
            out.append(state[0])
        return torch.stack(out, 1), state


class Sequential(nn.Sequential):
    """Flat numbering like PyTorch: ``seq(Linear(..), ReLU(), Linear(..))`` names parameters ``0.weight``,
    ``2.bias`` (crates/incin-core/src/nn/module.rs:18-33)."""


def seq(*layers: nn.Module) -> Sequential:
    return Sequential(*layers)


@dataclass
class ComputeStats:
    parameters: int
    trainable: int
    bytes: int
    linear_flops_per_row: int

    @staticmethod
    def of(module: nn.Module) -> "ComputeStats":
        ps = list(module.parameters())
        fl = sum(m.flops(1) for m in module.modules() if isinstance(m, Linear))
        return ComputeStats(sum(p.numel() for p in ps), sum(p.numel() for p in ps if p.requires_grad),
                            sum(p.numel() * p.element_size() for p in ps), fl)
