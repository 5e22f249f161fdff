"""Position encodings of the rotary family: a table of inverse frequencies and how many of a
head's elements rotate.  inv_freq[i] = theta^(-2i/rot_dim) in float
(snowllm/models/lfm2/layers.py:116-117); the angle pos * inv_freq[i] is formed in float inside the
kernel that applies it."""
from __future__ import annotations

import math

import torch

from .registry import register_position


class RotaryPosition:
    """``precise``: the table is worked out in double precision on the host and rounded to float once
    (otherwise in float, as SnowLLM forms it)."""

    def __init__(self, *, head_dim: int, theta: float, rot_dim: int | None = None, precise: bool = False):
        self.head_dim, self.theta, self.precise = head_dim, float(theta), precise
        self.rot_dim = head_dim if rot_dim is None else rot_dim
        if self.rot_dim % 2 or self.rot_dim > head_dim:
            raise ValueError(f"rot_dim={self.rot_dim} must be even and at most head_dim={head_dim}")
        self._inv_freq = None

    def rotary(self, device):
        if self._inv_freq is None or self._inv_freq.device != torch.device(device):
            if self.precise:
                inv = torch.tensor([self.theta ** (-2.0 * i / self.rot_dim) for i in range(self.rot_dim // 2)],
                                   dtype=torch.float64).to(torch.float32)
            else:
                inv = 1.0 / (self.theta ** (torch.arange(0, self.rot_dim, 2, dtype=torch.float32) / self.rot_dim))
            self._inv_freq = inv.to(device)
        return self._inv_freq, self.rot_dim


class PairedRotaryPosition:
    """Rotary positions in the interleaved layout: element 2i turns with element 2i + 1 (not with the one
    half a head away), f_i = theta^(-2i/rot_dim).  The table is worked out in double precision on the host
    and kept in float; a kernel that rotates pairs asks for it (``layout``)."""
    layout = "pairs"

    def __init__(self, *, head_dim: int, theta: float, rot_dim: int | None = None):
        self.head_dim, self.theta = head_dim, float(theta)
        self.rot_dim = head_dim if rot_dim is None else rot_dim
        if self.rot_dim % 2 or self.rot_dim > head_dim:
            raise ValueError(f"rot_dim={self.rot_dim} must be even and at most head_dim={head_dim}")
        self._inv_freq = None

    def frequencies(self) -> list:
        return [self.theta ** (-2.0 * i / self.rot_dim) for i in range(self.rot_dim // 2)]

    def rotary(self, device):
        if self._inv_freq is None or self._inv_freq.device != torch.device(device):
            self._inv_freq = torch.tensor(self.frequencies(), dtype=torch.float64).to(torch.float32).to(device)
        return self._inv_freq, self.rot_dim


class YarnRotaryPosition:
    """Rotary frequencies stretched for contexts longer than the ``original`` one (YaRN).  With
    f_i = theta^(-2i/rot_dim) and place(t) = rot_dim * ln(original / (2 pi t)) / (2 ln theta), the
    dimensions between lo = floor(place(fast)) and hi = ceil(place(slow)) go over from f_i (fast turning
    ones, kept) to f_i / factor (slow ones, stretched): f = f_i / factor * ramp + f_i * (1 - ramp) with
    ramp = clamp((i - lo) / max(hi - lo, 0.001), 0, 1).  cos and sin are scaled by
    ``magnitude`` = 0.1 ln(factor) + 1.  The table is worked out in double precision on the host and kept
    in float; the angle position * f is formed in float inside the kernel."""

    def __init__(self, *, head_dim: int, theta: float, rot_dim: int | None = None, factor: float = 1.0,
                 original: float | None = None, fast: float = 32.0, slow: float = 1.0):
        self.head_dim, self.theta = head_dim, float(theta)
        self.rot_dim = head_dim if rot_dim is None else rot_dim
        if self.rot_dim % 2 or self.rot_dim > head_dim:
            raise ValueError(f"rot_dim={self.rot_dim} must be even and at most head_dim={head_dim}")
        self.factor, self.original, self.fast, self.slow = float(factor), original, float(fast), float(slow)
        self.magnitude = 0.1 * math.log(self.factor) + 1.0 if original else 1.0
        self._inv_freq = None

    def frequencies(self) -> list:
        n, base = self.rot_dim, self.theta
        plain = [base ** (-2.0 * i / n) for i in range(n // 2)]
        if not self.original:
            return plain

        def place(turns):
            return n * math.log(self.original / (2 * math.pi * turns)) / (2 * math.log(base))
        lo = max(math.floor(place(self.fast)), 0)
        hi = min(math.ceil(place(self.slow)), n - 1)
        out = []
        for i, f in enumerate(plain):
            ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
            out.append(f / self.factor * ramp + f * (1.0 - ramp))
        return out

    def rotary(self, device):
        if self._inv_freq is None or self._inv_freq.device != torch.device(device):
            self._inv_freq = torch.tensor(self.frequencies(), dtype=torch.float64).to(torch.float32).to(device)
        return self._inv_freq, self.rot_dim


class NoPosition:
    """No position encoding (the mixer sees order only through its causal mask)."""

    def __init__(self, **_):
        pass

    def rotary(self, device):
        return None, 0


register_position("rope", RotaryPosition)
register_position("none", NoPosition)
register_position("yarn", YarnRotaryPosition)
register_position("rope_pairs", PairedRotaryPosition)
