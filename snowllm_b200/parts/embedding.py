"""Token embedding and output head (snowllm/models/embedding.py:10-19;
snowllm/models/qwen3_5/layers.py:209-228: logits are float whatever the compute dtype)."""
from __future__ import annotations

import torch

from ..ops import kernels, linear
from .base import Part
from .registry import register_embedding, register_head
from ..errors import ConfigError
from .spec import SlotStateSpec, TensorSpec


class Embedding(Part):
    libraries = ("elementwise",)

    def __init__(self, dtype, names, *, vocab_size: int, hidden_size: int, scale: float = 1.0):
        """``scale``: a constant that multiplies every row on its way into the stream."""
        super().__init__(dtype, names)
        self.vocab_size, self.hidden_size, self.scale = vocab_size, hidden_size, float(scale)
        self.weight = None

    def declare(self, has):
        return [TensorSpec("weight", self.names["weight"], (self.vocab_size, self.hidden_size))]

    def bind(self, tensors):
        self.weight = tensors["weight"]

    def bytes_read(self, bound, picked=None):
        return 0        # a step gathers one row per token: nothing beside the matrices

    def forward(self, ctx):
        """The float residual stream [M, H] of the step's tokens."""
        return kernels.embedding(ctx.token_ids, self.weight, pending=ctx.pending_tokens, scale=self.scale)


class PairHashEmbedding(Embedding):
    """The embedding plus a row of a second table chosen by a hash of the token and the one before it:
    ``pairs[(previous * mul_prev + token * mul_cur) mod buckets]``; a sequence's first token reads the table's
    extra last row (number ``buckets``).  The last token of a request's earlier steps is state of fixed size
    (one int32 per slot), which the cache manager keeps like a mixer's."""

    def __init__(self, dtype, names, *, vocab_size: int, hidden_size: int, buckets: int, mul_prev: int,
                 mul_cur: int, scale: float = 1.0):
        super().__init__(dtype, names, vocab_size=vocab_size, hidden_size=hidden_size, scale=scale)
        if buckets < 1 or mul_prev < 0 or mul_cur < 0:
            raise ConfigError(f"a pair table of {buckets} buckets with multipliers {mul_prev}, {mul_cur}")
        self.buckets, self.mul_prev, self.mul_cur = int(buckets), int(mul_prev), int(mul_cur)
        self.pairs = None

    def cache_spec(self):
        return SlotStateSpec(((),), ("i32",))

    def declare(self, has):
        return super().declare(has) + [TensorSpec("pairs", self.names["pairs"], (self.buckets + 1, self.hidden_size))]

    def bind(self, tensors):
        super().bind(tensors)
        self.pairs = tensors["pairs"]

    def forward(self, ctx, cache):
        return kernels.pair_embedding(ctx.token_ids, self.weight, self.pairs, self.buckets, self.mul_prev,
                                      self.mul_cur, ctx.row_seg, ctx.cu_seqlens, ctx.seg_start, ctx.seg_slot,
                                      cache.tensors[0], pending=ctx.pending_tokens, scale=self.scale)


class LinearHead(Part):
    """logits = x . W^T in float.  ``tied``: W is the embedding table, and no tensor is declared.
    ``softcap`` c: the logits are then c * tanh(logits / c)."""
    libraries = ("gemm", "gemm_skinny", "gemm_tc", "gemm_tc2", "elementwise")

    def __init__(self, dtype, names, *, vocab_size: int, hidden_size: int, tied: bool, softcap: float | None = None):
        super().__init__(dtype, names)
        self.vocab_size, self.hidden_size, self.tied = vocab_size, hidden_size, tied
        if softcap is not None and not softcap > 0:
            raise ConfigError(f"a logit cap of {softcap}: want a positive number")
        self.softcap = softcap
        self.weight = None

    def declare(self, has):
        if self.tied:
            return []
        return [TensorSpec("weight", self.names["weight"], (self.vocab_size, self.hidden_size))]

    def bind(self, tensors):
        self.weight = tensors["weight"]

    def bytes_read(self, bound, picked=None):
        # tied: nothing was declared here, yet the whole table is read as the head
        return self.weight.numel() * self.weight.element_size() if self.weight is not None else 0

    def forward(self, ctx, x):
        logits = linear(x, self.weight, out_dtype=torch.float32)
        return kernels.softcap(logits, self.softcap) if self.softcap else logits


register_embedding("embedding", Embedding)
register_embedding("pair_hash_embedding", PairHashEmbedding)
register_head("linear_head", LinearHead)
