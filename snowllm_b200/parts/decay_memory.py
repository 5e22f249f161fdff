"""Linear-attention mixers on a decayed matrix memory with a state of fixed size per request
(csrc/decay_memory.cu): per head a float matrix S [head_dim, v_head_dim], zero for a fresh request,

    S_t = diag(a_t) S_(t-1) + k_t v_t^T,      o_t = S_t^T q_t.

* ``hgrn2``: the forget gate also decides what is written.  f = low + (1 - low) * sigmoid(W_f x + b) per head
  and channel with a learned lower bound ``low``; a_t = f, k_t = 1 - f; q = silu(W_q x), v = W_v x.  Each
  head's o is divided by its root mean square and weighted by ``norm`` [v_head_dim] (one weight, shared by
  the heads), then the output product.
* ``retention``: one fixed decay per head (a_t = decay[head] for every row), no softmax and no
  denominator.  q = W_q x and k = W_k x turn with the position on their first ``rot_dim`` elements (split
  halves), k times head_dim^(-1/2) after the rotation.  Each head's o is divided by its root mean square
  (no weight), the heads are multiplied by silu(W_g x), then the output product.

One fused product leaves the projections in float; gates, decays, angles, state, sums and the per-head
statistics are float whatever the compute dtype."""
from __future__ import annotations

import functools
import os

import torch

from ..errors import ConfigError
from ..ops import kernels, linear
from .attention_maps import pad_rows
from .base import Part
from .registry import lookup, register_mixer
from .spec import INIT_BIAS, INIT_ONES, KEEP_F32, KEEP_SMALL, SlotStateSpec, TensorSpec

MAX_HEAD_DIM = 256
PIECE_ROWS = 64        # rows of a prompt portion that one block walks when the step holds a long portion


PIECE_CHOICES = (48, 56, 64, 72, 80, 96)
FIXED_PIECE_ROWS = int(os.environ.get("SNOWLLM_B200_PIECE_ROWS", "0"))    # one size for every layer (A/B runs)
BLOCKS_PER_SM = 2      # of the memory kernel with heads of 128 rows, by its registers


def piece_rows_for(seg_lens, blocks_per_piece: int, sms: int) -> int:
    """The piece size among PIECE_CHOICES whose blocks fill the SMs in the fewest and shortest rounds: a launch
    takes about (rounds of blocks) x (rows a block walks), and 512 blocks on 296 places wait for a second round
    that is a quarter empty where 592 smaller ones fill two.  Ties go to PIECE_ROWS, then to the larger piece."""
    places = max(sms * BLOCKS_PER_SM, 1)

    def cost(rows):
        blocks = sum(-(-n // rows) for n in seg_lens) * blocks_per_piece
        return -(-blocks // places) * rows
    return min(PIECE_CHOICES, key=lambda rows: (cost(rows), rows != PIECE_ROWS, -rows))


@functools.lru_cache(maxsize=None)
def _sm_count(device) -> int:
    return torch.cuda.get_device_properties(device).multi_processor_count


def memory_pieces(ctx, piece_rows: int | None = None):
    """The step's segments cut into pieces of up to ``piece_rows`` rows for the memory kernel: (int32 [n, 4] =
    segment, first row, rows, flags with 1 for a segment's first piece and 2 for its last; int32 [B+1] = first
    piece of each segment), on the device, uploaded once per step.  None when no segment is longer than two
    pieces: one block per (segment, head, columns) then walks its whole segment, and a captured step holds
    nothing that changes."""
    piece_rows = piece_rows or PIECE_ROWS
    if ctx.capture_max_len is not None or max(ctx.host_seg_len) <= 2 * piece_rows:
        return None
    key = ("memory_pieces", piece_rows)
    if key not in ctx.memo:
        table, first_piece, first = [], [0], 0
        for b, n in enumerate(ctx.host_seg_len):
            cuts = list(range(0, n, piece_rows)) or [0]
            for r in cuts:
                table.append((b, first + r, min(piece_rows, n - r), (r == 0) | ((r == cuts[-1]) << 1)))
            first_piece.append(len(table))
            first += n
        flat = [v for row in table for v in row] + first_piece
        dev = torch.tensor(flat, dtype=torch.int32).pin_memory().to(ctx.device, non_blocking=True)
        ctx.memo[key] = (dev[:4 * len(table)].view(-1, 4), dev[4 * len(table):])
    return ctx.memo[key]


class _DecayMemory(Part):
    libraries = ("gemm", "gemm_skinny", "gemm_tc", "gemm_tc2", "decay_memory", "sublayer")

    def __init__(self, dtype, names, *, hidden_size: int, num_heads: int, head_dim: int, v_head_dim: int,
                 head_norm_eps: float):
        super().__init__(dtype, names)
        if head_dim > MAX_HEAD_DIM:
            raise ConfigError(f"memory heads of {head_dim} rows: the kernel keeps up to {MAX_HEAD_DIM}")
        self.hidden_size, self.num_heads, self.head_dim, self.v_head_dim = hidden_size, num_heads, head_dim, v_head_dim
        self.head_norm_eps = float(head_norm_eps)
        self.w_in = self.wo = None

    def cache_spec(self):
        return SlotStateSpec(((self.num_heads, self.head_dim, self.v_head_dim),), ("f32",))

    def _pieces(self, ctx):
        """The step's pieces at the size that suits this layer's heads (a block serves 128 columns of a wide
        head, 32 of a narrow one)."""
        if ctx.capture_max_len is not None or PIECE_ROWS not in PIECE_CHOICES:
            return memory_pieces(ctx)
        if FIXED_PIECE_ROWS:
            return memory_pieces(ctx, FIXED_PIECE_ROWS)
        cols = 128 if self.v_head_dim > 64 else 32
        per_piece = self.num_heads * -(-self.v_head_dim // cols)
        return memory_pieces(ctx, piece_rows_for(ctx.host_seg_len, per_piece, _sm_count(ctx.device)))


class Hgrn2(_DecayMemory):
    def declare(self, has):
        W, H, dk, dv, n = self.hidden_size, self.num_heads, self.head_dim, self.v_head_dim, self.names
        return [TensorSpec("q_proj", n["q_proj"], (H * dk, W)), TensorSpec("f_proj", n["f_proj"], (H * dk, W)),
                TensorSpec("v_proj", n["v_proj"], (H * dv, W)), TensorSpec("out_proj", n["out_proj"], (W, H * dv)),
                TensorSpec("f_bias", n["f_bias"], (H * dk,), INIT_BIAS, KEEP_F32),
                TensorSpec("lower", n["lower"], (H * dk,), INIT_BIAS, KEEP_F32),
                TensorSpec("norm", n["norm"], (dv,), INIT_ONES, KEEP_SMALL)]

    def bind(self, tensors):
        self.w_in = pad_rows(torch.cat([tensors[k] for k in ("q_proj", "f_proj", "v_proj")], 0), 16)
        self.wo = tensors["out_proj"]
        self.f_bias, self.lower = tensors["f_bias"].float().contiguous(), tensors["lower"].float().contiguous()
        self.norm = tensors["norm"].repeat(self.num_heads).contiguous()      # one weight for every head

    def forward(self, ctx, x, cache, owns_cache=True):
        H, dk, dv = self.num_heads, self.head_dim, self.v_head_dim
        proj = linear(x, self.w_in, out_dtype=torch.float32)
        raw = kernels.decay_memory(proj, 0, H * dk, 2 * H * dk, ctx.cu_seqlens, ctx.seg_start, ctx.seg_slot,
                                   cache.tensors[0], H, dk, dv, gate_bias=self.f_bias, gate_low=self.lower,
                                   pieces=self._pieces(ctx))
        ctx.tap("memory_raw", raw)
        heads = kernels.head_norm_gate(raw, H, dv, self.head_norm_eps, self.dtype, weight=self.norm)
        return linear(heads, self.wo, out_dtype=torch.float32)


class Retention(_DecayMemory):
    def __init__(self, dtype, names, *, decay, position: dict | None = None, **kw):
        super().__init__(dtype, names, **kw)
        decay = [float(d) for d in decay]
        if len(decay) != self.num_heads:
            raise ConfigError(f"{len(decay)} decays for {self.num_heads} heads")
        self.decay_values = decay
        pos = dict(position or {"kind": "none"})
        self.position = lookup("position", pos.pop("kind"))(**pos)
        if getattr(self.position, "layout", "halves") != "halves":
            raise ConfigError("the memory kernel rotates split halves")
        self.decay = None

    def declare(self, has):
        W, H, dk, dv, n = self.hidden_size, self.num_heads, self.head_dim, self.v_head_dim, self.names
        return [TensorSpec("q_proj", n["q_proj"], (H * dk, W)), TensorSpec("k_proj", n["k_proj"], (H * dk, W)),
                TensorSpec("v_proj", n["v_proj"], (H * dv, W)), TensorSpec("gate_proj", n["gate_proj"], (H * dv, W)),
                TensorSpec("out_proj", n["out_proj"], (W, H * dv))]

    def bind(self, tensors):
        self.w_in = pad_rows(torch.cat([tensors[k] for k in ("q_proj", "k_proj", "v_proj", "gate_proj")], 0), 16)
        self.wo = tensors["out_proj"]
        self.decay = torch.tensor(self.decay_values, dtype=torch.float32, device=self.wo.device)

    def forward(self, ctx, x, cache, owns_cache=True):
        H, dk, dv = self.num_heads, self.head_dim, self.v_head_dim
        proj = linear(x, self.w_in, out_dtype=torch.float32)
        inv_freq, rot_dim = self.position.rotary(x.device)
        raw = kernels.decay_memory(proj, 0, H * dk, 2 * H * dk, ctx.cu_seqlens, ctx.seg_start, ctx.seg_slot,
                                   cache.tensors[0], H, dk, dv, decay=self.decay, inv_freq=inv_freq, rot_dim=rot_dim,
                                   k_scale=dk ** -0.5, positions=ctx.positions, pieces=self._pieces(ctx))
        ctx.tap("memory_raw", raw)
        heads = kernels.head_norm_gate(raw, H, dv, self.head_norm_eps, self.dtype, gate=proj,
                                       gate_col=2 * H * dk + H * dv, gate_act="silu")
        return linear(heads, self.wo, out_dtype=torch.float32)


register_mixer("hgrn2", Hgrn2)
register_mixer("retention", Retention)
