"""Parameter initialisers (crates/incin-core/src/nn/init.rs:3-48, nn/param.rs:29-35).

The default for Linear/Conv is Kaiming-uniform with a = sqrt(5) over fan_in, i.e. U(-1/sqrt(fan_in),
1/sqrt(fan_in)); the bias uses the same bound.  Randomness comes from an explicit seeded generator: the
reference has no seeding API (CPU rand/randn use thread_rng), so "seed 0" is defined here as
``torch.Generator().manual_seed(0)`` on the CPU for module initialisers and as the Philox4x32-10 stream
``(seed, offset)`` for device-side generation (bit-identical on CPU and GPU).
"""
from __future__ import annotations

import enum
import math

import torch


class Init(enum.Enum):
    ZEROS = "zeros"
    ONES = "ones"
    KAIMING_UNIFORM = "kaiming_uniform"
    KAIMING_NORMAL = "kaiming_normal"
    XAVIER_UNIFORM = "xavier_uniform"
    XAVIER_NORMAL = "xavier_normal"
    NORMAL = "normal"        # N(0, std)
    UNIFORM = "uniform"      # U(-bound, bound)
    RANDN = "randn"          # N(0, 1): the reference's Embedding default


def fans(shape) -> tuple[int, int]:
    if len(shape) < 2:
        return shape[0], shape[0]
    rf = 1
    for d in shape[2:]:
        rf *= d
    return shape[1] * rf, shape[0] * rf


def initialize(t: torch.Tensor, how: Init, *, generator: torch.Generator | None = None, std: float = 0.02,
               bound: float | None = None, fan_in: int | None = None) -> torch.Tensor:
    fi, fo = fans(t.shape)
    fi = fan_in or fi
    with torch.no_grad():
        if how is Init.ZEROS:
            t.zero_()
        elif how is Init.ONES:
            t.fill_(1.0)
        elif how is Init.KAIMING_UNIFORM:
            b = 1.0 / math.sqrt(fi)            # gain sqrt(2/(1+5)) * sqrt(3/fan_in)
            t.uniform_(-b, b, generator=generator)
        elif how is Init.KAIMING_NORMAL:
            t.normal_(0.0, math.sqrt(2.0 / fi), generator=generator)
        elif how is Init.XAVIER_UNIFORM:
            b = math.sqrt(6.0 / (fi + fo))
            t.uniform_(-b, b, generator=generator)
        elif how is Init.XAVIER_NORMAL:
            t.normal_(0.0, math.sqrt(2.0 / (fi + fo)), generator=generator)
        elif how is Init.NORMAL:
            t.normal_(0.0, std, generator=generator)
        elif how is Init.UNIFORM:
            b = bound if bound is not None else 1.0
            t.uniform_(-b, b, generator=generator)
        elif how is Init.RANDN:
            t.normal_(0.0, 1.0, generator=generator)
    return t
