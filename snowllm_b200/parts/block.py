"""How a layer's parts sit around the residual stream.

``prenorm`` (snowllm/models/lfm2/layers.py:91-104): x += mixer(norm(x)); x += ffn(norm(x)).
The float residual sum is fused into the norm that follows it, so a block takes the delta that the
previous block left and returns its own last delta; the model adds the final one.

``output_norm``: x += norm(mixer(x)); x += norm(ffn(x)).  The sums are made at once (nothing is left for
the next block), and the block hands on the stream's copy in the compute dtype.

``parallel``: h = norm(x); x += mixer(h) + ffn(h).  One norm, both sublayers read its output; the sum of
their outputs is left to the norm that follows (``kernels.DeltaSum``).

``hyper``: the stream is kept as S streams (hyper-connections).  Sublayer q reads u = sum_s in_q[s] X[s]
through its norm and leaves y; then X'[t] = sum_s mix_q[s, t] X[s] + out_q[t] y for all t at once.  The
update stays pending (``kernels.StreamsDelta``) until the next norm applies it in its own kernel."""
from __future__ import annotations

import torch

from ..errors import ConfigError
from ..ops import kernels
from ..trace import span
from .base import Part
from .registry import register_block
from .spec import KEEP_F32, TensorSpec


class PreNormBlock:
    """``residual_scale`` m (a constant of the arrangement): x += m * mixer(norm(x)); x += m * ffn(norm(x)).
    The factor travels with the delta (``kernels.ScaledDelta``) to the norm that adds it."""

    def __init__(self, mixer, ffn, mixer_norm, ffn_norm, *, dtype=None, residual_scale: float = 1.0):
        self.mixer, self.ffn, self.mixer_norm, self.ffn_norm = mixer, ffn, mixer_norm, ffn_norm
        self.residual_scale = float(residual_scale)
        self._names = tuple(f"{what}:{type(part).__name__}" for what, part in
                            (("norm", mixer_norm), ("mixer", mixer), ("norm", ffn_norm), ("ffn", ffn)))

    def parts(self):
        return tuple(p for p in (self.mixer_norm, self.mixer, self.ffn_norm, self.ffn) if p is not None)

    def forward(self, ctx, residual, delta, cache, owns_cache=True):
        with span(self._names[0]):
            x = self.mixer_norm.forward(ctx, residual, delta)
        ctx.tap("mixer_in", x)
        with span(self._names[1]):
            delta = self.mixer.forward(ctx, x, cache, owns_cache)
        ctx.tap("mixer_out", delta)
        if self.residual_scale != 1.0:
            return self._scaled(ctx, residual, delta)
        if self.ffn is None:
            self._tap_layer(ctx, residual, delta)
            return delta
        fused = getattr(self.ffn, "forward_from_residual", None)
        if fused is not None:          # a feed-forward that can take the norm before it into its first kernel
            with span(self._names[3]):
                out = fused(ctx, residual, delta, self.ffn_norm)
            if out is not None:
                ctx.tap("ffn_out", out)
                self._tap_layer(ctx, residual, out)
                return out
        with span(self._names[2]):
            x = self.ffn_norm.forward(ctx, residual, delta)
        ctx.tap("ffn_in", x)
        with span(self._names[3]):
            delta = self.ffn.forward(ctx, x)
        ctx.tap("ffn_out", delta)
        self._tap_layer(ctx, residual, delta)
        return delta

    @staticmethod
    def _tap_layer(ctx, residual, delta):
        if ctx.taps is not None:
            ctx.tap("layer_out", residual + (delta.dense() if hasattr(delta, "dense") else delta))

    def _scaled(self, ctx, residual, delta):
        """The rest of the layer when the sublayers' outputs enter the stream times a constant."""
        delta = kernels.ScaledDelta(delta, self.residual_scale)
        if self.ffn is not None:
            with span(self._names[2]):
                x = self.ffn_norm.forward(ctx, residual, delta)
            ctx.tap("ffn_in", x)
            with span(self._names[3]):
                delta = kernels.ScaledDelta(self.ffn.forward(ctx, x), self.residual_scale)
            ctx.tap("ffn_out", delta.delta)
        self._tap_layer(ctx, residual, delta)
        return delta


class OutputNormBlock:
    """x += norm(mixer(x)); x += norm(ffn(x)): each norm sits on its sublayer's OUTPUT, and the sublayers
    read the residual stream itself.  The stream is float; its copy in the compute dtype, which the next
    sublayer reads, comes out of the kernel that adds the normalised output (``norm.add_normed``) and is
    handed from block to block through the step's memo.  A layer may have the mixer's sublayer alone."""

    def __init__(self, mixer, ffn, mixer_norm, ffn_norm):
        self.mixer, self.ffn, self.mixer_norm, self.ffn_norm = mixer, ffn, mixer_norm, ffn_norm
        self._names = tuple(f"{what}:{type(part).__name__}" for what, part in
                            (("mixer", mixer), ("norm", mixer_norm), ("ffn", ffn), ("norm", ffn_norm)))

    def parts(self):
        return tuple(p for p in (self.mixer_norm, self.mixer, self.ffn_norm, self.ffn) if p is not None)

    def forward(self, ctx, residual, delta, cache, owns_cache=True):
        if delta is not None:                      # a block of another arrangement left its sum to us
            kernels.residual_add(residual, delta.dense() if hasattr(delta, "dense") else delta)
        key = ("stream_copy", id(residual))
        x = ctx.memo.get(key)
        if x is None or delta is not None:
            x = residual if ctx.dtype == residual.dtype else kernels.cast_rows(residual, ctx.dtype)
        ctx.tap("mixer_in", x)
        with span(self._names[0]):
            y = self.mixer.forward(ctx, x, cache, owns_cache)
        ctx.tap("mixer_out", y)
        with span(self._names[1]):
            x = self.mixer_norm.add_normed(ctx, residual, y)
        if self.ffn is not None:
            ctx.tap("ffn_in", x)
            with span(self._names[2]):
                y = self.ffn.forward(ctx, x)
            y = y.dense() if hasattr(y, "dense") else y
            ctx.tap("ffn_out", y)
            with span(self._names[3]):
                x = self.ffn_norm.add_normed(ctx, residual, y)
        ctx.memo[key] = x
        if ctx.taps is not None:
            ctx.tap("layer_out", residual.clone())
        return None


class ParallelBlock:
    """h = norm(x); x += mixer(h) + ffn(h): the layer has ONE norm and both sublayers read its output.  The
    block leaves the two outputs as a ``kernels.DeltaSum``: the next norm forms a + b, adds it into the float
    residual and normalises in one kernel.  A layer may have the mixer alone."""
    single_norm = True         # the model builds it without a second norm

    def __init__(self, mixer, ffn, mixer_norm, ffn_norm=None):
        if ffn_norm is not None:
            raise ValueError("a parallel layer has one norm")
        self.mixer, self.ffn, self.mixer_norm, self.ffn_norm = mixer, ffn, mixer_norm, None
        self._names = tuple(f"{what}:{type(part).__name__}" for what, part in
                            (("norm", mixer_norm), ("mixer", mixer), ("ffn", ffn)))

    def parts(self):
        return tuple(p for p in (self.mixer_norm, self.mixer, self.ffn) if p is not None)

    def forward(self, ctx, residual, delta, cache, owns_cache=True):
        with span(self._names[0]):
            x = self.mixer_norm.forward(ctx, residual, delta)
        ctx.tap("mixer_in", x)
        with span(self._names[1]):
            out = self.mixer.forward(ctx, x, cache, owns_cache)
        ctx.tap("mixer_out", out)
        if self.ffn is not None:
            ctx.tap("ffn_in", x)
            with span(self._names[2]):
                f = self.ffn.forward(ctx, x)
            ctx.tap("ffn_out", f)
            out = kernels.DeltaSum(out, f)
        if ctx.taps is not None:
            ctx.tap("layer_out", residual + (out.dense() if hasattr(out, "dense") else out))
        return out


class StreamWeights(Part):
    """The learned numbers of one sublayer's hyper-connection: ``in`` [S] (how the sublayer reads the
    streams), ``out`` [S] (how its output enters each stream) and ``mix`` [S, S] (indexed [from, to]: how the
    streams pass into one another), kept in float."""

    def __init__(self, dtype, names, *, streams: int):
        super().__init__(dtype, names)
        self.streams = streams
        self.read = self.out = self.mix = None

    def declare(self, has):
        S, n = self.streams, self.names
        return [TensorSpec("in", n["in"], (S,), keep=KEEP_F32), TensorSpec("out", n["out"], (S,), keep=KEEP_F32),
                TensorSpec("mix", n["mix"], (S, S), keep=KEEP_F32)]

    def bind(self, tensors):
        self.read, self.out, self.mix = (tensors[k].float().contiguous() for k in ("in", "out", "mix"))


class HyperBlock:
    """A pre-norm layer over ``streams`` streams instead of one residual.  The norms must be able to read
    streams (``read_streams``: ``group_rmsnorm``).  The first block of a model finds a plain residual (the
    embedding output, with whatever delta a block of another arrangement left) and starts every stream as
    a copy of it; every block leaves its last update pending for the norm that follows, in the next block
    or at the model's end.  ``names`` None (with ``streams`` 1): no learned numbers, which is the plain
    pre-norm layer x += sublayer(norm(x)) on these norms."""

    def __init__(self, mixer, ffn, mixer_norm, ffn_norm, *, dtype=torch.float32, streams: int = 1, names=None):
        self.mixer, self.ffn, self.mixer_norm, self.ffn_norm = mixer, ffn, mixer_norm, ffn_norm
        for norm in (mixer_norm, ffn_norm):
            if norm is not None and not hasattr(norm, "read_streams"):
                raise ConfigError(f"a hyper layer needs norms that read streams, not {type(norm).__name__}")
        if streams < 1 or streams > 8:
            raise ConfigError(f"streams={streams}: the kernel keeps 1 to 8")
        if names is None and streams != 1:
            raise ConfigError("several streams need their learned weights")
        self.streams = streams
        self.hc = [StreamWeights(dtype, n, streams=streams) for n in names] if names is not None else None
        if self.hc is not None and len(self.hc) != (1 if ffn is None else 2):
            raise ConfigError("a hyper layer has one set of stream weights per sublayer")
        self._fixed = None
        self._names = tuple(f"{what}:{type(part).__name__}" for what, part in
                            (("norm", mixer_norm), ("mixer", mixer), ("norm", ffn_norm), ("ffn", ffn)))

    def parts(self):
        own = tuple(p for p in (self.mixer_norm, self.mixer, self.ffn_norm, self.ffn) if p is not None)
        return own + tuple(self.hc or ())

    def _weights(self, q: int, device):
        """(read, out, mix) of sublayer q."""
        if self.hc is not None:
            return self.hc[q].read, self.hc[q].out, self.hc[q].mix
        if self._fixed is None or self._fixed[0].device != device:
            one = torch.ones(1, dtype=torch.float32, device=device)
            self._fixed = (one, one, one.view(1, 1))
        return self._fixed

    def forward(self, ctx, residual, delta, cache, owns_cache=True):
        M, W = residual.shape
        S = self.streams
        init = None
        if isinstance(delta, kernels.StreamsDelta):
            streams, pending = delta.streams, delta
            if streams.shape[1] != S:
                raise ConfigError(f"a layer of {S} streams follows one of {streams.shape[1]}")
        else:
            if delta is not None:                  # a block of another arrangement left its sum to us
                kernels.residual_add(residual, delta.dense() if hasattr(delta, "dense") else delta)
            pending = None
            if S == 1:
                streams = residual.view(M, 1, W)
            else:
                streams = torch.empty(M, S, W, dtype=torch.float32, device=residual.device)
                init = residual
        read, out, mix = self._weights(0, residual.device)
        with span(self._names[0]):
            x = self.mixer_norm.read_streams(ctx, streams, init=init, update=pending, read=read)
        ctx.tap("mixer_in", x)
        with span(self._names[1]):
            y = self.mixer.forward(ctx, x, cache, owns_cache)
        ctx.tap("mixer_out", y)
        pending = kernels.StreamsDelta(streams, y, mix, out)
        if self.ffn is not None:
            read, out, mix = self._weights(1, residual.device)
            with span(self._names[2]):
                x = self.ffn_norm.read_streams(ctx, streams, update=pending, read=read)
            ctx.tap("ffn_in", x)
            with span(self._names[3]):
                y = self.ffn.forward(ctx, x)
            ctx.tap("ffn_out", y)
            pending = kernels.StreamsDelta(streams, y, mix, out)
        if ctx.taps is not None:
            ctx.tap("layer_out", pending.total())
        return pending


register_block("prenorm", PreNormBlock)
register_block("hyper", HyperBlock)
register_block("parallel", ParallelBlock)
register_block("output_norm", OutputNormBlock)
