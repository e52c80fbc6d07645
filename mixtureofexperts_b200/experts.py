"""GatedExpert and StandardExpert with the reference's constructors and fields
(src/experts/gated.jl, src/experts/standard.jl)."""
from __future__ import annotations

import math

import numpy as np


class Expert:
    """abstract type Expert (src/experts/standard.jl:6)."""


def silu(x):
    """silu(x) = x * sigmoid(x) (src/experts/gated.jl:36).  Only its identity matters: the
    layer maps the callable to the activation enum of the C ABI."""
    return x / (1.0 + np.exp(-x))


def gelu(x):
    """NNlib.gelu (tanh approximation), the MoEConfig default activation."""
    return 0.5 * x * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (x + 0.044715 * x ** 3)))


def relu(x):
    return np.maximum(x, 0)


def identity(x):
    return x


swish = silu


class GatedExpert(Expert):
    """GatedExpert(input_dim, hidden_dim, output_dim, activation) (src/experts/gated.jl:6-27):
    three bias-free projections w1, w3 (hidden x input) and w2 (output x hidden), all drawn
    randn * sqrt(2/input_dim); forward w2(act.(w1 x) .* (w3 x)).

    Weights are float32 arrays of logical shape (out, in) (Flux's Dense.weight), held either
    as NumPy arrays or as torch tensors (possibly on the GPU).  ``rng`` seeds the draw."""

    def __init__(self, input_dim: int, hidden_dim: int, output_dim: int, activation=silu, *, rng=None,
                 device=None, dtype=None):
        self.input_dim, self.hidden_dim, self.output_dim = int(input_dim), int(hidden_dim), int(output_dim)
        self.activation = activation
        sigma = math.sqrt(2.0 / input_dim)
        if device is not None:
            import torch

            gen = rng if isinstance(rng, torch.Generator) else None
            dt = dtype or torch.float32
            mk = lambda o, i: (torch.randn((o, i), device=device, dtype=torch.float32, generator=gen) * sigma).to(dt)
        else:
            g = rng if isinstance(rng, np.random.Generator) else np.random.default_rng(rng)
            mk = lambda o, i: (g.standard_normal((o, i), dtype=np.float32) * np.float32(sigma))
        self.w1 = mk(hidden_dim, input_dim)
        self.w2 = mk(output_dim, hidden_dim)
        self.w3 = mk(hidden_dim, input_dim)


class StandardExpert(Expert):
    """StandardExpert(input_dim, hidden_dim, output_dim, activation; dropout=0, bias=true)
    (src/experts/standard.jl:8-36): w1 (hidden x input) drawn randn * sqrt(2/input_dim), w2
    (output x hidden) drawn randn * sqrt(2/hidden_dim), b1 / b2 zero vectors (None when
    ``bias=False``); forward w2(act.(w1 x .+ b1)) .+ b2 (:38-55).

    The reference applies Dropout to the hidden activations when training; that draw lives in
    Flux's RNG and is not offered here: ``dropout`` must be 0."""

    def __init__(self, input_dim: int, hidden_dim: int, output_dim: int, activation=gelu, *, dropout: float = 0.0,
                 bias: bool = True, rng=None, device=None, dtype=None):
        if dropout > 0:
            raise ValueError("StandardExpert dropout is not accelerated: pass dropout=0")
        self.input_dim, self.hidden_dim, self.output_dim = int(input_dim), int(hidden_dim), int(output_dim)
        self.activation = activation
        self.dropout = None
        s1, s2 = math.sqrt(2.0 / input_dim), math.sqrt(2.0 / hidden_dim)
        if device is not None:
            import torch

            gen = rng if isinstance(rng, torch.Generator) else None
            dt = dtype or torch.float32
            mk = lambda o, i, s: (torch.randn((o, i), device=device, dtype=torch.float32, generator=gen) * s).to(dt)
            zeros = lambda n: torch.zeros(n, device=device, dtype=torch.float32)
        else:
            g = rng if isinstance(rng, np.random.Generator) else np.random.default_rng(rng)
            mk = lambda o, i, s: (g.standard_normal((o, i), dtype=np.float32) * np.float32(s))
            zeros = lambda n: np.zeros(n, dtype=np.float32)
        self.w1 = mk(hidden_dim, input_dim, s1)
        self.w2 = mk(output_dim, hidden_dim, s2)
        self.b1 = zeros(hidden_dim) if bias else None
        self.b2 = zeros(output_dim) if bias else None
