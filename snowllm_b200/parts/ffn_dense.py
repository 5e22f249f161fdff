"""Dense SwiGLU feed-forward: down(silu(gate x) * up x)
(snowllm/models/lfm2/layers.py:76-88; snowllm/ops/mlp.py:12-20).  Gate and up are one fused
product [2I, H] (rows interleaved by 8, so that the product's store applies SwiGLU); the down product leaves a float delta for the residual sum."""
from __future__ import annotations

import torch

from ..errors import ConfigError
from ..ops import interleave_gate_up, kernels, linear, linear_glu, linear_swiglu
from .base import Part
from .registry import register_ffn
from .spec import TensorSpec


class SwiGLU(Part):
    libraries = ("gemm", "gemm_skinny", "gemm_tc", "gemm_tc2", "elementwise")

    def __init__(self, dtype, names, *, hidden_size: int, intermediate_size: int):
        super().__init__(dtype, names)
        self.hidden_size, self.intermediate_size = hidden_size, intermediate_size
        self.w13 = self.w2 = None

    def declare(self, has):
        H, I = self.hidden_size, self.intermediate_size
        return [TensorSpec("gate", self.names["gate"], (I, H)),
                TensorSpec("up", self.names["up"], (I, H)),
                TensorSpec("down", self.names["down"], (H, I))]

    def bind(self, tensors):
        # gate and up rows interleaved by 8 where the width allows: the product then applies SwiGLU itself
        self.interleaved = self.intermediate_size % 8 == 0
        self.w13 = (interleave_gate_up(tensors["gate"], tensors["up"]) if self.interleaved
                    else torch.cat((tensors["gate"], tensors["up"]), 0).contiguous())
        self.w2 = tensors["down"]

    def forward(self, ctx, x):
        act = linear_swiglu(x, self.w13, self.interleaved)
        return linear(act, self.w2, out_dtype=torch.float32)


class GatedFFN(SwiGLU):
    """down(act(gate x) * up x) with ``activation`` one of silu, relu, gelu_tanh, or ``swish_clamp`` with its
    ``limit`` (g = min(gate, limit), u = clamp(up, -limit, limit), g * sigmoid(1.702 g) * (u + 1)): the
    bfloat16 products apply the gate at their store (gate and up rows interleaved by 8); float32, and widths
    that are no multiple of 8, run the product and then one elementwise kernel."""
    libraries = SwiGLU.libraries + ("sublayer",)

    def __init__(self, dtype, names, *, hidden_size: int, intermediate_size: int, activation: str = "silu",
                 limit: float | None = None):
        super().__init__(dtype, names, hidden_size=hidden_size, intermediate_size=intermediate_size)
        if activation not in kernels.GATED_ACTIVATIONS or activation == "relu2":
            raise ConfigError(f"activation {activation!r} (known: silu, relu, gelu_tanh, swish_clamp)")
        if activation == "swish_clamp" and not (limit and limit > 0):
            raise ConfigError("the clamped activation needs a positive limit")
        self.activation, self.limit = activation, float(limit or 0.0)

    def forward(self, ctx, x):
        act = linear_glu(x, self.w13, self.interleaved, self.activation, self.limit)
        return linear(act, self.w2, out_dtype=torch.float32)


class MLP(Part):
    """down(act(up x)) without a gate, ``activation`` one of silu, relu, gelu_tanh, relu2 (the square of
    relu).  The activation is evaluated in float on the up product's output and rounded once."""
    libraries = ("gemm", "gemm_skinny", "gemm_tc", "gemm_tc2", "sublayer")

    def __init__(self, dtype, names, *, hidden_size: int, intermediate_size: int, activation: str = "relu2"):
        super().__init__(dtype, names)
        if activation not in kernels.ACTIVATIONS:
            raise ConfigError(f"activation {activation!r} (known: {', '.join(kernels.ACTIVATIONS)})")
        self.hidden_size, self.intermediate_size, self.activation = hidden_size, intermediate_size, activation
        self.w1 = self.w2 = None

    def declare(self, has):
        H, I = self.hidden_size, self.intermediate_size
        return [TensorSpec("up", self.names["up"], (I, H)), TensorSpec("down", self.names["down"], (H, I))]

    def bind(self, tensors):
        self.w1, self.w2 = tensors["up"], tensors["down"]

    def forward(self, ctx, x):
        u = linear(x, self.w1)
        return linear(kernels.act_rows(u, self.activation), self.w2, out_dtype=torch.float32)


register_ffn("swiglu", SwiGLU)
register_ffn("mlp", MLP)
register_ffn("gated", GatedFFN)
