"""Windowed grouped-query attention mixers whose keys and values have widths of their own
(csrc/attention_split.cu): keys of ``head_dim``, values of ``v_head_dim``, kept in two pools.

Five kinds are built on one class:

* ``bias_attention``: one softmax map per head; a learned bias is added to the scaled score, chosen by
  head and by a bucket of the distance i - j (``DistanceBuckets``).  No rotation.
* ``diff_attention``: two softmax maps per head over the same values (q and k hold the maps' halves side
  by side, head by head); the second map's output is taken off the first with one weight per layer,
  lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + offset; each head of the difference is divided by its root
  mean square and scaled by (1 - offset); the heads are gated by sigmoid(W_g x) before the output
  product.  Rotary positions (plain or stretched) on the first ``rot_dim`` elements of every map.

* ``sink_attention``: one map per head, no positions at all; biased projections; q and k over their root
  mean square per head without a weight; a learned factor per head on the scale (``temp``); a learned sink
  per head, one more term exp(sink) in the softmax's sum that has no key and no value; and a block-local
  mask: position i reads j <= i of its own block of ``block`` positions only (blocks counted from position
  0 of the sequence, whatever the cut into steps).

* ``slope_attention``: one map per head, no rotation; q and k each over ONE root mean square taken over all
  heads at once (weights of the projections' sizes); slope[h] * (i - j) is taken off the scaled score, with
  slope[h] = 2^(-slope_range * (h + 1) / heads); a sliding window.
* ``conv_gate_attention``: q, k and v pass a short causal convolution over time right after their projection
  (depthwise, ``conv_taps`` taps; the last taps - 1 projected rows of a request are state of fixed size);
  per-head RMS norm of q and k with one weight shared by all heads; rotary positions on the first
  ``rot_dim`` elements; a sliding window beside the sequence's first ``keep_first`` positions, which stay
  reachable at their true positions; one more term 1 in the softmax's denominator (``one_more``: a sink whose
  score is 0 and which has no value); each head's output times sigmoid of the head's own logit from a gate
  projection [heads, hidden] that reads the mixer's input.

The first two: per-head RMS norm of q and k with one weight of ``head_dim`` shared by all heads (and maps), before
the rotation; ``window`` keeps the last ``window`` keys.  Scores, softmax weights and the per-head
statistics are float whatever the compute dtype.  A layer that reads another layer's cache
(``reads_cache``) has no key and value tensors at all: it projects q (and the gate) alone and attends
over the keys as the owner wrote them.  ``cache_window`` is how many positions the owner of the cache
keeps: its own window or the widest window among its readers."""
from __future__ import annotations

import math

import numpy as np
import torch

from ..errors import ConfigError, KernelError
from ..ops import kernels, linear
from . import attention_plan as plan
from .base import Part
from .registry import lookup, register_mixer
from .spec import INIT_BIAS, INIT_CONV, INIT_ONES, KEEP_F32, KEEP_SMALL, PagedKVSpec, SlotStateSpec, TensorSpec


class DistanceBuckets:
    """Which row of a bias table a key ``n`` positions back reads: one row per distance below rows/2, then
    logarithmic steps that reach the last row at distance ``far``:
    bucket(n) = n for n < rows/2, else min(rows - 1, rows/2 + floor(ln(n / (rows/2)) / ln(far / (rows/2))
    * (rows - rows/2))).  From some distance on the bucket is the last row."""

    def __init__(self, rows: int, far: float):
        if rows < 2 or far <= rows // 2:
            raise ConfigError(f"a distance bias of {rows} rows reaching to {far}: want rows >= 2 and far > rows/2")
        self.rows, self.far = int(rows), float(far)

    def bucket(self, n: int) -> int:
        half = self.rows // 2
        if n < half:
            return n
        # the logarithms in double precision; an exact step (n/half a whole power of the ratio) must not
        # fall below its bucket by a rounding error
        step = math.log(n / half) / math.log(self.far / half) * (self.rows - half)
        return min(self.rows - 1, half + int(math.floor(step + 1e-9)))

    def saturation(self) -> int:
        """The first distance whose bucket is the last row (every longer distance reads it too)."""
        n = self.rows // 2
        while self.bucket(n) < self.rows - 1:
            n += 1
        return n

    def table(self, length: int) -> list:
        return [self.bucket(n) for n in range(length)]


def pad_rows(w: torch.Tensor, multiple: int) -> torch.Tensor:
    extra = -w.shape[0] % multiple
    if not extra:
        return w.contiguous()
    return torch.cat((w, w.new_zeros(extra, w.shape[1])), 0).contiguous()


def attention_tiles(ctx, tile_rows: int):
    """The step's rows cut into runs of up to ``tile_rows`` consecutive rows of one request: int32 [n, 2] =
    (first row, rows) on the device, uploaded once per step; None when every row stands alone (decode
    steps: a captured step then holds nothing that changes)."""
    if tile_rows <= 1 or max(ctx.host_seg_len) <= 1:
        return None
    key = ("attention_maps_tiles", tile_rows)
    if key not in ctx.memo:
        tiles, first = [], 0
        for n in ctx.host_seg_len:
            for r in range(0, n, tile_rows):
                tiles.append((first + r, min(tile_rows, n - r)))
            first += n
        host = torch.tensor(tiles, dtype=torch.int32).pin_memory()
        ctx.memo[key] = host.to(ctx.device, non_blocking=True)
    return ctx.memo[key]


def single_row_tiles(ctx, rows):
    """``rows`` (host list of row numbers) as tiles of one row each, int32 [n, 2] on the device; once per step."""
    key = ("attention_maps_single_rows", len(rows))
    if key not in ctx.memo:
        host = torch.tensor([[r, 1] for r in rows], dtype=torch.int32).pin_memory()
        ctx.memo[key] = host.to(ctx.device, non_blocking=True)
    return ctx.memo[key]


class MapsAttention(Part):
    libraries = ("gemm", "gemm_skinny", "gemm_tc", "gemm_tc2", "attention_split", "attention", "sublayer")
    maps = 1
    norm_weights = True        # the per-head norm of q and k has a weight (False: the plain root mean square)
    whole_norm = False         # True: ONE root mean square over all heads of q (of k), weights of that size
    keep_first = 0             # positions at the sequence's start that stay reachable beside the window

    def __init__(self, dtype, names, *, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 v_head_dim: int, scale: float, qk_norm_eps: float | None, window: int | None = None,
                 cache_window: int | None = None, position: dict | None = None, reads_cache: bool = False,
                 block: int | None = None, keep_first: int = 0):
        super().__init__(dtype, names)
        if keep_first and (not window or keep_first < 0 or reads_cache or cache_window not in (None, window)):
            raise ConfigError("kept first positions go with a sliding window on a cache of the layer's own")
        self.keep_first = int(keep_first or 0)
        if block is not None and (window is not None or cache_window is not None or reads_cache or block < 1):
            raise ConfigError("a block-local mask stands alone: no window, no shared cache, a positive size")
        self.block = block
        self.proj_bias = self.head_scale = self.sink = self.slopes = None      # float tensors a kind may bind
        if num_heads % num_kv_heads:
            raise ConfigError(f"num_heads={num_heads} is no multiple of num_kv_heads={num_kv_heads}")
        if (num_heads // num_kv_heads) * self.maps > 32:
            raise ConfigError(f"{num_heads // num_kv_heads} query heads per kv head with {self.maps} maps: "
                              f"the attention kernel serves up to 32 per kv head")
        if v_head_dim > 256:
            raise ConfigError(f"v_head_dim={v_head_dim}: the attention kernel takes up to 256")
        self.hidden_size, self.num_heads, self.num_kv_heads = hidden_size, num_heads, num_kv_heads
        self.head_dim, self.v_head_dim, self.scale = head_dim, v_head_dim, float(scale)
        self.qk_norm_eps, self.window, self.reads_cache = qk_norm_eps, window, reads_cache
        self.cache_window = cache_window if cache_window is not None or window is None else window
        if window is None and cache_window is not None:
            raise ConfigError("a layer that sees every key cannot live on a cache that keeps a window")
        if window is not None and self.cache_window is not None and self.cache_window < window:
            raise ConfigError(f"cache_window={cache_window} is shorter than the layer's window {window}")
        pos = dict(position or {"kind": "none"})
        self.position = lookup("position", pos.pop("kind"))(**pos)
        self.w_in = self.wo = self.q_norm = self.k_norm = None
        self.bias = None

    # -- sizes of the fused projection ----------------------------------------------------------
    @property
    def nq(self) -> int:
        return self.num_heads * self.maps

    def _columns(self):
        """(q, k, v, gate) column offsets of the fused projection, and its width."""
        q = 0
        k = q + self.nq * self.head_dim
        v = k + (0 if self.reads_cache else self.num_kv_heads * self.maps * self.head_dim)
        g = v + (0 if self.reads_cache else self.num_kv_heads * self.v_head_dim)
        return q, k, v, g, g + self._gate_width()

    def _gate_width(self) -> int:
        return 0

    def cache_spec(self):
        return PagedKVSpec(self.num_kv_heads, self.maps * self.head_dim, self.cache_window, self.v_head_dim,
                           separate=True, block=self.block, keep_first=self.keep_first)

    def declare(self, has):
        H, dk, dv, n = self.hidden_size, self.head_dim, self.v_head_dim, self.names
        specs = [TensorSpec("q_proj", n["q_proj"], (self.nq * dk, H))]
        if not self.reads_cache:
            specs += [TensorSpec("k_proj", n["k_proj"], (self.num_kv_heads * self.maps * dk, H)),
                      TensorSpec("v_proj", n["v_proj"], (self.num_kv_heads * dv, H))]
        specs.append(TensorSpec("out_proj", n["out_proj"], (H, self.num_heads * dv)))
        if self.qk_norm_eps is not None and self.norm_weights:
            nq, nk = (self.nq * dk, self.num_kv_heads * self.maps * dk) if self.whole_norm else (dk, dk)
            specs.append(TensorSpec("q_norm", n["q_norm"], (nq,), INIT_ONES, KEEP_SMALL))
            if not self.reads_cache:
                specs.append(TensorSpec("k_norm", n["k_norm"], (nk,), INIT_ONES, KEEP_SMALL))
        return specs

    def _projection_rows(self, tensors) -> list:
        rows = [tensors["q_proj"]]
        if not self.reads_cache:
            rows += [tensors["k_proj"], tensors["v_proj"]]
        return rows

    def bind(self, tensors):
        self._decode_chunk = kernels.split_attention_decode_chunk(self.nq, self.num_kv_heads, self.maps, self.head_dim,
                                                                  self.v_head_dim, self.dtype) \
            if tensors["q_proj"].is_cuda else kernels.SPLIT_ATTENTION_CHUNK
        self.w_in = pad_rows(torch.cat(self._projection_rows(tensors), 0), 16)
        self.wo = tensors["out_proj"]
        self.q_norm = tensors.get("q_norm")
        self.k_norm = tensors.get("k_norm", self.q_norm)      # a reader of another layer's cache normalises q alone

    # -- the step -----------------------------------------------------------------------------
    def _attend(self, ctx, x, cache, owns_cache, out_dtype):
        if owns_cache == self.reads_cache:
            raise KernelError("a layer without key and value tensors must read another layer's cache, "
                              "and one with them must own its cache")
        proj = linear(x, self.w_in)
        q_off, k_off, v_off, g_off, _ = self._columns()
        cache, rows = self._convolved(ctx, proj, cache)      # the rows that are normalised, turned and cached
        kpool, vpool = cache.pools
        inv_freq, rot_dim = self.position.rotary(x.device)
        q = kernels.split_prepare(rows, q_off, k_off, v_off, self.q_norm, self.k_norm, self.qk_norm_eps or 0.0,
                                  inv_freq, rot_dim, getattr(self.position, "magnitude", 1.0), ctx.positions,
                                  ctx.row_seg, cache.block_table, cache.page_size, kpool, vpool, self.nq,
                                  self.num_kv_heads, self.maps, self.head_dim, self.v_head_dim,
                                  write_kv=owns_cache, proj_bias=self.proj_bias,
                                  plain_norm=self.qk_norm_eps is not None and not self.norm_weights,
                                  whole_norm=self.whole_norm)
        ctx.tap("attention_q", q)
        if self._prompt_kernel_ok(ctx, q, cache, out_dtype):
            # prompt portions on the tcgen05 kernel; the rows of short segments (decoded tokens beside them) below
            tc_tiles, rows_dev, rows_host = plan.split(ctx, kernels.PREFILL_TC_TILE_ROWS)
            out = torch.empty(ctx.M, self.nq, self.v_head_dim, dtype=out_dtype, device=q.device)
            kernels.attention_prefill_tc_split(q, kpool, vpool, cache.block_table, cache.page_size, tc_tiles, self.scale,
                                               out, window=self.window, keep=self.keep_first, slopes=self.slopes,
                                               sink=self.sink, gate=proj if self._gate_in_kernel() else None,
                                               gate_col=g_off)
            if not rows_host:
                ctx.tap("attention_o", out)
                return proj, out
            if self._decode_kernel_ok(q, cache, out_dtype):
                # the rows of short segments (decoded tokens beside the portions) on the TMA decode kernel
                self._alone(ctx, q, cache, proj, g_off, out, rows_dev, rows_host)
                ctx.tap("attention_o", out)
                return proj, out
            tiles = single_row_tiles(ctx, rows_host)
            return proj, self._rows(ctx, q, cache, proj, g_off, out_dtype, tiles, 1, out)
        return proj, self._rows(ctx, q, cache, proj, g_off, out_dtype, None, None, None)

    def _prompt_kernel_ok(self, ctx, q, cache, out_dtype) -> bool:
        """Whether the step's long segments go to the tcgen05 prompt kernel: bfloat16, one map, heads of 64 for
        keys and values alike, a mask and a bias it knows (causal, a window with or without kept first keys, a
        slope per head, a sink per head, a gate per head)."""
        return (self.maps == 1 and self.head_dim == 64 and self.v_head_dim == 64 and self.bias is None
                and self.block is None and self.head_scale is None and out_dtype == torch.bfloat16
                and kernels.attention_prefill_tc_ok(q, cache.page_size)
                and max(ctx.host_seg_len) >= plan.PREFILL_MIN_ROWS)

    def _decode_kernel_ok(self, q, cache, out_dtype) -> bool:
        """Whether rows that stand alone go to the TMA decode kernel: bfloat16, one map, heads of 64 or 128 for
        keys and values alike, up to 16 heads per kv head, a mask and a bias it knows."""
        return (self.maps == 1 and self.head_dim == self.v_head_dim and self.head_dim in kernels.PREFILL_HEAD_DIMS
                and self.bias is None and self.block is None and self.head_scale is None
                and out_dtype == torch.bfloat16 and q.dtype == torch.bfloat16
                and self.nq // self.num_kv_heads <= kernels.DECODE_MMA_MAX_GROUP
                and kernels.DECODE_TMA and kernels.decode_tma_page_ok(cache.page_size))

    def _alone(self, ctx, q, cache, proj, g_off, out, rows_dev, rows_host):
        """Rows that stand alone (all of the step, or ``rows_host``) on the tensor cores, their keys and values by
        TMA in chunks of 256, written into ``out``."""
        kpool, vpool = cache.pools
        chunk = kernels.DECODE_MMA_CHUNK
        num_chunks = plan.chunks(ctx, self.window, rows_host, chunk, keep=self.keep_first)
        if self.window:                    # a captured step plans for its longest sequence; a window spans fewer
            num_chunks = min(num_chunks, (self.window - 1) // chunk + 2 + -(-self.keep_first // chunk))
        served = ctx.M if rows_host is None else len(rows_host)
        scratch = ctx.scratch(kernels.attention_scratch_bytes(served, self.nq, self.v_head_dim, num_chunks)) \
            if num_chunks > 1 else None
        kernels.attention_decode_tma_split(q, kpool, vpool, cache.block_table, cache.page_size, ctx.positions,
                                           ctx.row_seg, self.scale, num_chunks, out, window=self.window,
                                           keep=self.keep_first, slopes=self.slopes, sink=self.sink,
                                           gate=proj if self._gate_in_kernel() else None, gate_col=g_off,
                                           scratch=scratch, rows=rows_dev)

    def _rows(self, ctx, q, cache, proj, g_off, out_dtype, tiles, tile_rows, out):
        """The kernels of csrc/attention_split.cu: every row of the step (``tiles`` None), or the rows that
        ``tiles`` names, written into ``out``."""
        kpool, vpool = cache.pools
        decode_only = tiles is None and max(ctx.host_seg_len) <= 1
        if decode_only and self._decode_kernel_ok(q, cache, out_dtype):
            out = torch.empty(ctx.M, self.nq, self.v_head_dim, dtype=out_dtype, device=q.device)
            self._alone(ctx, q, cache, proj, g_off, out, None, None)
            ctx.tap("attention_o", out)
            return out
        if tiles is None:
            tile_rows = kernels.split_attention_tile_rows(self.nq, self.num_kv_heads, self.maps, self.head_dim,
                                                          self.v_head_dim, self.dtype, decode_only)
            tiles = attention_tiles(ctx, tile_rows)
        num_chunks, scratch, chunk = 1, None, kernels.SPLIT_ATTENTION_CHUNK
        if decode_only:
            # rows of decoded tokens: their keys in chunks, one block each, merged in chunk order
            chunk = self._decode_chunk
            num_chunks = plan.chunks(ctx, self.window, None, chunk, block=self.block, keep=self.keep_first)
            if self.window:                # a captured step plans for its longest sequence; a window spans fewer
                num_chunks = min(num_chunks, (self.window - 1) // chunk + 2 + -(-self.keep_first // chunk))
            if num_chunks > 1:
                scratch = ctx.scratch(kernels.attention_scratch_bytes(ctx.M, self.nq, self.v_head_dim, num_chunks))
        out = kernels.split_attention(q, kpool, vpool, cache.block_table, cache.page_size, ctx.positions,
                                      ctx.row_seg, self.scale, maps=self.maps, window=self.window, bias=self.bias,
                                      tiles=tiles, tile_rows=tile_rows, out=out,
                                      out_dtype=out_dtype, num_chunks=num_chunks, scratch=scratch, chunk=chunk,
                                      block=self.block, head_scale=self.head_scale, sink=self.sink,
                                      keep=self.keep_first, slopes=self.slopes,
                                      gate=proj if self._gate_in_kernel() else None, gate_col=g_off)
        ctx.tap("attention_o", out)
        return out

    def _convolved(self, ctx, proj, cache):
        """(the paged view, the rows split_prepare reads): a kind whose projections pass something on their
        way (a convolution with state of its own) does it here."""
        return cache, proj

    def _gate_in_kernel(self) -> bool:
        """Whether the gate columns of the projection hold one logit per head that the attention kernel
        applies itself."""
        return False


class BiasAttention(MapsAttention):
    """One map per head and a learned bias per (distance bucket, head)."""

    DEFAULT_ROWS = 16          # rows of a drawn table when the configuration names none

    def __init__(self, dtype, names, *, bias_far: float, bias_rows: int | None = None, **kw):
        super().__init__(dtype, names, **kw)
        self.bias_rows, self.bias_far = bias_rows, float(bias_far)
        self.buckets = None

    def declare(self, has):
        # the table's rows are the checkpoint's to say (its first dimension), unless the configuration does
        rows = self.bias_rows if self.bias_rows is not None else -1
        return super().declare(has) + [TensorSpec("rel", self.names["rel"], (rows, self.num_heads), keep=KEEP_F32,
                                                  free_default=self.DEFAULT_ROWS)]

    def bind(self, tensors):
        super().bind(tensors)
        self.buckets = DistanceBuckets(tensors["rel"].shape[0], self.bias_far)
        # the bias by distance: [heads, L] with L the window, or where the buckets reach their last row
        length = self.buckets.saturation() + 1
        if self.window is not None:
            length = min(length, self.window)
        rel = tensors["rel"].float()
        index = torch.as_tensor(np.asarray(self.buckets.table(length), dtype=np.int64), device=rel.device)
        self.bias = rel[index].t().contiguous()

    def forward(self, ctx, x, cache, owns_cache=True):
        _, out = self._attend(ctx, x, cache, owns_cache, self.dtype)
        return linear(out.view(ctx.M, -1), self.wo, out_dtype=torch.float32)


class DiffAttention(MapsAttention):
    """Two maps per head; the second is taken off the first; normalised, gated heads."""
    maps = 2

    def __init__(self, dtype, names, *, offset: float, head_norm_eps: float, **kw):
        super().__init__(dtype, names, **kw)
        self.offset, self.head_norm_eps = float(offset), float(head_norm_eps)
        self.lam = None

    def _gate_width(self) -> int:
        return self.num_heads * self.v_head_dim

    def declare(self, has):
        n, dk = self.names, self.head_dim
        return super().declare(has) + [
            TensorSpec("gate_proj", n["gate_proj"], (self.num_heads * self.v_head_dim, self.hidden_size)),
            *(TensorSpec(v, n[v], (dk,), keep=KEEP_F32) for v in ("lq1", "lk1", "lq2", "lk2"))]

    def _projection_rows(self, tensors) -> list:
        return super()._projection_rows(tensors) + [tensors["gate_proj"]]

    def bind(self, tensors):
        super().bind(tensors)
        t = {k: tensors[k].float() for k in ("lq1", "lk1", "lq2", "lk2")}
        self.lam = float(torch.exp((t["lq1"] * t["lk1"]).sum()) - torch.exp((t["lq2"] * t["lk2"]).sum())) + self.offset

    def forward(self, ctx, x, cache, owns_cache=True):
        proj, maps = self._attend(ctx, x, cache, owns_cache, torch.float32)     # [M, heads * 2, dv] float
        dv = self.v_head_dim
        gate_col = self._columns()[3]
        heads = kernels.head_norm_gate(maps, self.num_heads, dv, self.head_norm_eps, self.dtype, second=dv,
                                       lam=self.lam, gate=proj, gate_col=gate_col, mult=1.0 - self.offset)
        ctx.tap("attention_heads", heads)
        return linear(heads, self.wo, out_dtype=torch.float32)


class SinkAttention(MapsAttention):
    """One map per head, no positions; biased projections, weightless q/k norms, a factor and a sink per
    head, a block-local mask (``block`` None: plain causal)."""
    norm_weights = False

    def __init__(self, dtype, names, *, biased: bool = True, **kw):
        super().__init__(dtype, names, **kw)
        self.biased = biased

    def declare(self, has):
        n, dk, dv = self.names, self.head_dim, self.v_head_dim
        specs = super().declare(has) + [TensorSpec("temp", n["temp"], (self.num_heads,), INIT_ONES, KEEP_F32),
                                        TensorSpec("sink", n["sink"], (self.num_heads,), INIT_BIAS, KEEP_F32)]
        if self.biased:
            specs += [TensorSpec("q_bias", n["q_bias"], (self.num_heads * dk,), INIT_BIAS, KEEP_F32),
                      TensorSpec("k_bias", n["k_bias"], (self.num_kv_heads * dk,), INIT_BIAS, KEEP_F32),
                      TensorSpec("v_bias", n["v_bias"], (self.num_kv_heads * dv,), INIT_BIAS, KEEP_F32)]
        return specs

    def bind(self, tensors):
        super().bind(tensors)
        self.head_scale = tensors["temp"].float().contiguous()
        self.sink = tensors["sink"].float().contiguous()
        if self.biased:
            bias = torch.cat([tensors[k].float() for k in ("q_bias", "k_bias", "v_bias")])
            self.proj_bias = torch.cat((bias, bias.new_zeros(self.w_in.shape[0] - bias.numel()))).contiguous()

    def forward(self, ctx, x, cache, owns_cache=True):
        _, out = self._attend(ctx, x, cache, owns_cache, self.dtype)
        return linear(out.view(ctx.M, -1), self.wo, out_dtype=torch.float32)


class SlopeAttention(MapsAttention):
    """One map per head, no rotation; q and k over one root mean square each, taken over all heads at once;
    a distance penalty slope[h] * (i - j) with slope[h] = 2^(-slope_range * (h + 1) / heads)."""
    libraries = MapsAttention.libraries + ("attention_tc", "attention_mma")
    whole_norm = True

    def __init__(self, dtype, names, *, slope_range: float = 8.0, **kw):
        super().__init__(dtype, names, **kw)
        self.slope_range = float(slope_range)

    def bind(self, tensors):
        super().bind(tensors)
        H = self.num_heads
        slopes = [2.0 ** (-self.slope_range * (h + 1) / H) for h in range(H)]
        self.slopes = torch.tensor(slopes, dtype=torch.float64).to(torch.float32).to(self.w_in.device)

    def forward(self, ctx, x, cache, owns_cache=True):
        _, out = self._attend(ctx, x, cache, owns_cache, self.dtype)
        return linear(out.view(ctx.M, -1), self.wo, out_dtype=torch.float32)


class ConvGateAttention(MapsAttention):
    """Convolved projections, kept first positions, one more term in the softmax's sum, gated heads."""
    libraries = MapsAttention.libraries + ("attention_tc", "attention_mma", "short_conv")

    def __init__(self, dtype, names, *, conv_taps: int | None = None, one_more: bool = True, **kw):
        super().__init__(dtype, names, **kw)
        if self.reads_cache:
            raise ConfigError("a layer with convolved projections owns its cache")
        self.conv_taps = int(conv_taps) if conv_taps else 0
        if self.conv_taps > 16:
            raise ConfigError(f"conv taps {self.conv_taps}: the kernel takes up to 16")
        self.one_more = bool(one_more)
        self.conv_w = None

    @property
    def conv_channels(self) -> int:
        return self.num_heads * self.head_dim + self.num_kv_heads * (self.head_dim + self.v_head_dim)

    def _gate_width(self) -> int:
        return self.num_heads

    def _gate_in_kernel(self) -> bool:
        return True

    def cache_spec(self):
        pages = super().cache_spec()
        if self.conv_taps <= 1:
            return pages
        return (pages, SlotStateSpec(((self.conv_taps - 1, self.conv_channels),), ("compute",)))

    def declare(self, has):
        n, dk, dv = self.names, self.head_dim, self.v_head_dim
        specs = super().declare(has) + [TensorSpec("gate_proj", n["gate_proj"], (self.num_heads, self.hidden_size))]
        if self.conv_taps:
            L = self.conv_taps
            specs += [TensorSpec("q_conv", n["q_conv"], (self.num_heads * dk, L), INIT_CONV, KEEP_SMALL),
                      TensorSpec("k_conv", n["k_conv"], (self.num_kv_heads * dk, L), INIT_CONV, KEEP_SMALL),
                      TensorSpec("v_conv", n["v_conv"], (self.num_kv_heads * dv, L), INIT_CONV, KEEP_SMALL)]
        return specs

    def _projection_rows(self, tensors) -> list:
        return super()._projection_rows(tensors) + [tensors["gate_proj"]]

    def bind(self, tensors):
        super().bind(tensors)
        if self.conv_taps:
            self.conv_w = torch.cat([tensors[k] for k in ("q_conv", "k_conv", "v_conv")], 0).contiguous()
        if self.one_more:          # a sink whose score is 0: exp(0) = 1 joins every row's sum
            self.sink = torch.zeros(self.nq, dtype=torch.float32, device=self.w_in.device)

    def _convolved(self, ctx, proj, cache):
        if not self.conv_taps:
            return cache, proj
        if self.conv_taps == 1:            # one tap: a factor per channel, and no history to keep
            pages, state = cache, proj.new_empty(1, 0, self.conv_channels)
        else:
            pages, state = cache[0], cache[1].tensors[0]
        rows = kernels.causal_conv(proj, self.conv_channels, self.conv_w, state, ctx.cu_seqlens,
                                   ctx.seg_start, ctx.seg_slot, ctx.row_seg)
        ctx.tap("attention_conv", rows)
        return pages, rows

    def forward(self, ctx, x, cache, owns_cache=True):
        _, out = self._attend(ctx, x, cache, owns_cache, self.dtype)
        return linear(out.view(ctx.M, -1), self.wo, out_dtype=torch.float32)


register_mixer("sink_attention", SinkAttention)
register_mixer("slope_attention", SlopeAttention)
register_mixer("conv_gate_attention", ConvGateAttention)
register_mixer("bias_attention", BiasAttention)
register_mixer("diff_attention", DiffAttention)
