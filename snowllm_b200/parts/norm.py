"""Norms over the hidden size, fused with the residual sum that precedes them: RMSNorm
(snowllm/ops/norm.py:11-30; snowllm/models/lfm2/layers.py:99-104) and Dynamic Tanh, which computes no
statistics at all: tanh(alpha * x) * weight + bias with one learned number alpha; and the RMS norm in groups,
which also reads a residual stream that is kept as several streams."""
from __future__ import annotations

import torch

from ..errors import ConfigError
from ..ops import kernels
from .base import Part
from .registry import register_norm
from .spec import INIT_BIAS, INIT_ONES, KEEP_SMALL, TensorSpec


class RMSNorm(Part):
    libraries = ("elementwise",)
    fusable_rms = True     # x * rsqrt(mean(x^2) + eps) * weight over the whole width: what a part that fuses
                           # the norm before it into its own first kernel may take over (weight, eps)

    def __init__(self, dtype, names, *, size: int, eps: float):
        super().__init__(dtype, names)
        self.size, self.eps = size, eps
        self.weight = None

    def declare(self, has):
        return [TensorSpec("weight", self.names["weight"], (self.size,), INIT_ONES, KEEP_SMALL)]

    def bind(self, tensors):
        self.weight = tensors["weight"]

    def forward(self, ctx, residual, delta=None, rows=None):
        """``residual += delta`` in float, then the norm of the sum in the compute dtype.  With
        ``rows`` (int32 row numbers) only those rows come out and the residual stays untouched."""
        return kernels.add_rmsnorm(residual, delta, self.weight, self.eps, self.dtype, rows=rows)

    def add_normed(self, ctx, residual, y):
        """``residual += norm(y)`` for a sublayer's float output ``y`` (the norm on the output side);
        returns the new residual in the compute dtype (the residual itself when that is float)."""
        same = residual.dtype == self.dtype
        x = kernels.norm_add(residual, y, self.weight, self.eps, self.dtype, want_x=not same)
        return residual if same else x


class DynamicTanh(Part):
    """tanh(alpha * x) * weight + bias, elementwise, in float: no mean, no variance, no eps.  Tensors:
    ``weight`` [size], ``bias`` [size], ``alpha`` (one number)."""
    libraries = ("sublayer",)
    fusable_rms = False

    def __init__(self, dtype, names, *, size: int):
        super().__init__(dtype, names)
        self.size = size
        self.weight = self.bias = self.alpha = None

    def declare(self, has):
        n = self.names
        return [TensorSpec("weight", n["weight"], (self.size,), INIT_ONES, KEEP_SMALL),
                TensorSpec("bias", n["bias"], (self.size,), INIT_BIAS, KEEP_SMALL),
                TensorSpec("alpha", n["alpha"], (), INIT_ONES, KEEP_SMALL)]

    def bind(self, tensors):
        self.weight, self.bias, self.alpha = tensors["weight"], tensors["bias"], tensors["alpha"]

    def forward(self, ctx, residual, delta=None, rows=None):
        """``residual += delta`` in float (a tensor, an ``ExpertSum`` or the ``DeltaSum`` of a layer whose
        two sublayers ran side by side), then the norm of the sum in the compute dtype.  With ``rows`` only
        those rows come out and the residual stays untouched."""
        return kernels.add_dyt(residual, delta, self.weight, self.bias, self.alpha, self.dtype, rows=rows)


class GroupRMSNorm(Part):
    """RMS norm in ``groups`` equal consecutive parts of the width: each part over its own
    sqrt(mean(part^2) + eps), the whole times ``weight``.  ``groups`` 1 is the plain RMS norm.  It reads a plain
    float residual (``residual += delta`` first) or, when ``delta`` is a ``kernels.StreamsDelta``, a stream
    kept as several streams: the pending update is applied and the streams are read with ``read`` weights
    (None: their plain sum), all in the one kernel."""
    libraries = ("streams",)
    fusable_rms = False

    def __init__(self, dtype, names, *, size: int, eps: float, groups: int = 1):
        super().__init__(dtype, names)
        if groups < 1 or size % groups:
            raise ConfigError(f"a norm over {size} in {groups} groups: the width must be a multiple of the groups")
        self.size, self.eps, self.groups = size, float(eps), int(groups)
        self.weight = None

    def declare(self, has):
        return [TensorSpec("weight", self.names["weight"], (self.size,), INIT_ONES, KEEP_SMALL)]

    def bind(self, tensors):
        self.weight = tensors["weight"]

    def read_streams(self, ctx, streams, *, init=None, update=None, read=None, rows=None):
        """The norm of sum_s read[s] X[s] after ``init`` and the pending ``update`` have been applied."""
        return kernels.streams_norm(streams, self.weight, self.groups, self.eps, self.dtype, init=init,
                                    update=update, read=read, rows=rows)

    def forward(self, ctx, residual, delta=None, rows=None):
        if isinstance(delta, kernels.StreamsDelta):
            return self.read_streams(ctx, delta.streams, update=delta, rows=rows)
        # one stream: the residual itself, with the identity as its update
        M, W = residual.shape
        one = ctx.memo.get("streams_identity")
        if one is None:
            one = ctx.memo["streams_identity"] = torch.ones(1, 1, dtype=torch.float32, device=residual.device)
        streams, update = residual.view(M, 1, W), None
        if delta is not None:
            update = kernels.StreamsDelta(streams, delta, one, one.view(1))
        return self.read_streams(ctx, streams, update=update, rows=rows)


register_norm("rmsnorm", RMSNorm)
register_norm("group_rmsnorm", GroupRMSNorm)
register_norm("dyt", DynamicTanh)
