"""Python side of the sm_100a kernels: checks of dtype, shape and contiguity, then one launch.

Every function launches on torch's current CUDA stream and returns without synchronising.
There is no other implementation behind these names: a tensor that is not on a CUDA device,
or a library that cannot be built, is an error (the role of snowllm/ops/_common.py:82-112).
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from ..csrc import build
from ..errors import KernelError

F32, BF16 = 0, 1
_DTYPE_CODE = {torch.float32: F32, torch.bfloat16: BF16}

P, I, F, LL = c_void_p, c_int, c_float, c_longlong
_SIGNATURES = {
    "elementwise": {
        "snk_embedding": [P, P, I, P, P, I, I, I, I, F, P],
        "snk_add_rmsnorm": [P, P, P, I, P, P, I, I, F, I, P, P, P, I, F, P, I, P],
        "snk_pair_embedding": [P, P, I, P, P, P, I, I, I, I, F, LL, LL, LL, P, P, P, P, P, P],
        "snk_softcap": [P, LL, F, P],
        "snk_residual_add": [P, P, LL, P],
        "snk_swiglu": [P, P, I, I, I, I, P],
    },
    "rope_cache": {
        "snk_qk_norm_rope_cache": [P, P, P, I, I, F, P, I, P, P, P, I, I, P, P, I, I, I, I, I, I, P],
    },
    "short_conv": {
        "snk_short_conv": [P, P, I, P, P, P, P, P, P, I, I, I, I, I, P],
        "snk_causal_conv": [P, LL, P, I, P, P, P, P, P, P, LL, I, I, I, I, I, P],
    },
    "attention": {
        "snk_paged_attention_scratch_bytes": [I, I, I, I],
        "snk_paged_attention": [P, P, P, I, I, P, P, P, P, I, I, I, I, I, I, I, F, I, P],
        "snk_paged_attention_rows": [P, P, P, I, I, P, P, P, P, I, I, I, I, I, I, I, F, I, P, P],
        "snk_attention_merge": [P, P, P, I, I, I, I, I, I, I, P, P],
        "snk_attention_merge_gated": [P, P, P, I, I, I, I, I, I, I, P, LL, I, P, P],
    },
    "attention_mma": {
        "snk_attention_prefill": [P, P, P, I, I, P, I, P, I, I, I, I, F, P],
        "snk_attention_decode_mma": [P, P, P, I, I, P, P, P, P, P, I, I, I, I, I, I, F, P],
        "snk_attention_prefill_tma": [P, P, LL, P, I, I, P, I, P, I, I, I, I, F, P],
        "snk_attention_decode_tma": [P, P, LL, P, I, I, P, P, P, P, P, I, I, I, I, I, I, F, P],
        "snk_attention_decode_tma_split": [P, P, P, LL, P, I, I, P, P, P, P, P, I, I, I, I, I, I, F, I, P, P, P, LL, P],
        "snk_attention_decode_status": [],
        "snk_attention_decode_status_peek": [P, P],
    },
    "attention_tc": {
        "snk_attention_prefill_tc": [P, LL, P, LL, P, I, I, P, I, P, I, I, I, I, F, P],
        "snk_attention_prefill_tc_split": [P, LL, P, P, LL, P, I, I, P, I, P, I, I, I, I, F, I, P, P, P, LL, P],
        "snk_attention_tc_status": [],
        "snk_attention_tc_status_peek": [P, P],
    },
    "gemm": {
        "snk_gemm_simt": [P, P, P, I, I, I, P, I, P, I, I, I, I, P],
    },
    "gemm_skinny": {
        "snk_gemm_skinny": [P, P, P, I, I, I, P, I, P, I, I, I, I, P],
    },
    "gemm_tc": {
        "snk_gemm_tc": [P, P, P, I, I, I, P, I, I, I, I, P, P],
        "snk_gemm_tc_scratch_bytes": [I, I, I, I],
        "snk_gemm_tc_status": [],
        "snk_gemm_tc_status_peek": [P, P],
        "snk_gemm_tc_test_lose_loads": [I],
        "snk_gemm_tc_parts": [P, P, P, I, I, I, P, P],
        "snk_gather_rows_bf16": [P, P, P, I, I, I, P],
    },
    "gemm_tc2": {
        "snk_gemm_tc2": [P, P, P, I, I, I, P, I, I, I, P],
        "snk_gemm_tc2_status": [P],
        "snk_gemm_tc2_status_peek": [P, P],
        "snk_gemm_tc2_test_lose_loads": [I],
    },
    "moe": {
        "snk_moe_route": [P, P, I, P, P, P, I, I, I, I, I, F, I, P],
        "snk_moe_topk": [P, P, P, P, I, I, I, I, F, I, I, P],
        "snk_moe_route_sort": [P, P, I, P, P, P, P, P, P, P, I, I, I, I, I, F, I, P],
        "snk_moe_sort": [P, P, P, P, I, I, P],
        "snk_norm_route_sort": [P, P, P, I, P, I, F, P, P, P, I, P, I, P, P, P, P, P, P, I, I, I, I, F, I, P, P],
        "snk_moe_combine": [P, P, P, P, I, I, I, P],
        "snk_moe_scaled_rows": [P, P, P, P, P, I, I, I, I, P],
        "snk_row_dot": [P, P, I, P, I, I, I, P],
    },
    "sublayer": {
        "snk_norm_add": [P, P, P, I, P, I, I, F, I, P],
        "snk_cast_rows": [P, P, LL, I, P],
        "snk_gated_act": [P, P, I, I, I, I, F, I, P],
        "snk_head_norm_gate": [P, I, I, F, P, I, P, I, LL, P, I, I, I, F, F, I, I, P],
        "snk_act_rows": [P, P, LL, I, I, P],
        "snk_rms_cols": [P, LL, I, P, I, P, I, I, F, I, P],
        "snk_add_dyt": [P, P, P, P, P, P, I, P, P, P, I, P, P, I, I, I, P],
    },
    "attention_latent": {
        "snk_latent_prepare": [P, LL, I, P, LL, I, P, I, F, P, I, P, P, P, I, I, P, P, P, I, I, I, I, I, I, I, P],
        "snk_latent_attention_tile_rows": [I, I, I, I],
        "snk_latent_attention": [P, P, P, P, I, I, P, P, P, I, I, P, I, I, I, I, I, F, P, I, I, P, I, P],
        "snk_heads_to_rows": [P, P, I, I, I, I, P],
    },
    "attention_split": {
        "snk_split_prepare": [P, LL, I, I, I, P, P, P, I, I, F, P, I, F, P, P, P, I, I, P, P, P, I, I, I, I, I, I, I, I, P],
        "snk_split_attention_tile_rows": [I, I, I, I, I, I, I],
        "snk_split_attention_decode_chunk": [I, I, I, I, I, I],
        "snk_split_attention": [P, P, P, P, I, I, P, P, P, I, I, P, I, I, I, I, I, I, I, F, P, I, P, P, I, P, LL, I, I, P,
                                I, P],
    },
    "mlstm": {
        "snk_mlstm": [P, LL, I, I, I, I, I, P, P, I, F, P, P, P, P, P, P, P, I, I, I, I, P],
    },
    "decay_memory": {
        "snk_decay_memory": [P, LL, I, I, I, I, P, P, I, P, P, I, F, P, P, P, P, P, P, I, I, I, I, P, P, I, P, P, P, I, P],
    },
    "streams": {
        "snk_streams_norm": [P, P, P, P, P, P, P, I, P, P, P, P, I, I, F, P, P, I, I, I, I, I, P],
        "snk_pair_norm_mix": [P, P, P, P, I, F, F, F, P, I, I, P],
    },
    "sampling": {
        "snk_argmax": [P, P, I, I, P],
        "snk_apply_penalties": [P, P, P, P, P, P, P, I, I, P],
        "snk_sample": [P, P, P, P, P, P, I, I, P],
    },
}
_RESTYPES = {"snk_paged_attention_scratch_bytes": LL, "snk_gemm_tc_scratch_bytes": LL}
_functions: dict[str, object] = {}
_library_of = {fn: lib for lib, fns in _SIGNATURES.items() for fn in fns}

_ERRORS = {20001: "unknown dtype code", 20002: "a size this kernel does not take",
           20003: "a pointer or pitch that is not aligned as the kernel needs"}


def register_signatures(library: str, signatures: dict, restypes: dict | None = None) -> None:
    """Let another source file of csrc/ be called through ``fn``."""
    _SIGNATURES.setdefault(library, {}).update(signatures)
    for name in signatures:
        _library_of[name] = library
    _RESTYPES.update(restypes or {})


def fn(name: str):
    f = _functions.get(name)
    if f is None:
        lib = build.load(_library_of[name])
        f = getattr(lib, name)
        f.argtypes = _SIGNATURES[_library_of[name]][name]
        f.restype = _RESTYPES.get(name, c_int)
        _functions[name] = f
    return f


def libraries_for(names) -> None:
    """Build (in parallel) the libraries that hold the named groups, before first use."""
    build.build(tuple(dict.fromkeys(names)))


def set_pdl(on: bool) -> None:
    """Switch programmatic dependent launch on or off for every library loaded so far (launches made from
    now on; a captured graph keeps what it was captured with)."""
    for name in list(_SIGNATURES):
        if build.is_loaded(name):
            f = build.load(name).snk_pdl_set
            f.argtypes, f.restype = [c_int], None
            f(int(bool(on)))


_launches = 0

# When a list: every wrapper appends (its name, kernels it launched, bytes it has to move, flops it has to do)
# for each call, in launch order: the ledger that a measurement lays beside a profiler's kernel times.  The
# bytes are the algorithmic ones (each operand and result once); None where a wrapper does not say.  Some
# figures need a look at device data (which experts own rows, how long each row's sequence is): with the
# ledger on, a wrapper may synchronise.  Off (None), it costs nothing.
ledger: list | None = None


def launch_count() -> int:
    """Kernels launched through this module so far (each wrapper reports how many it starts)."""
    return _launches


def _nbytes(*tensors) -> int:
    return sum(t.numel() * t.element_size() for t in tensors if t is not None)


def check(status: int, what: str, launches: int = 1, work=None) -> None:
    """``work``: a function giving (bytes, flops) of the call, or a list of them, one per launch in launch
    order; evaluated only when the ledger is on."""
    global _launches
    if status == 0:
        _launches += launches
        if ledger is not None and launches:
            done = work() if work is not None else (None, None)
            if isinstance(done, list):
                if len(done) != launches:
                    raise KernelError(f"{what}: work of {len(done)} launches for {launches}")
                ledger.extend((what, 1, nbytes, flops) for nbytes, flops in done)
            else:
                ledger.append((what, launches, done[0], done[1]))
        return
    if status in _ERRORS:
        raise KernelError(f"{what}: {_ERRORS[status]}")
    raise KernelError(f"{what}: CUDA error {status} ({_cuda_error_name(status)})")


def _cuda_error_name(code: int) -> str:
    try:
        rt = ctypes.CDLL("libcudart.so")
        rt.cudaGetErrorString.restype = ctypes.c_char_p
        return rt.cudaGetErrorString(code).decode()
    except OSError:
        return "?"


def _stream() -> c_void_p:
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t: torch.Tensor | None) -> c_void_p:
    return c_void_p(t.data_ptr()) if t is not None else c_void_p(0)


def _chk(t: torch.Tensor, what: str, dtype=None, shape=None) -> None:
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise KernelError(f"{what}: needs a CUDA tensor (this engine has no CPU path)")
    if dtype is not None and t.dtype not in (dtype if isinstance(dtype, tuple) else (dtype,)):
        raise KernelError(f"{what}: dtype {t.dtype}, want {dtype}")
    if not t.is_contiguous():
        raise KernelError(f"{what}: must be contiguous")
    if shape is not None and tuple(t.shape) != tuple(shape):
        raise KernelError(f"{what}: shape {tuple(t.shape)}, want {tuple(shape)}")


def code_of(dtype: torch.dtype) -> int:
    try:
        return _DTYPE_CODE[dtype]
    except KeyError:
        raise KernelError(f"compute dtype {dtype} is not supported (float32 or bfloat16)") from None


def _small(t: torch.Tensor, what: str, compute: torch.dtype) -> int:
    """A small weight may be float32 or the compute dtype; returns its is-float flag."""
    _chk(t, what, (torch.float32, compute))
    return int(t.dtype == torch.float32)


# --- elementwise -----------------------------------------------------------------------

def embedding(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor | None = None,
              pending: torch.Tensor | None = None, scale: float = 1.0) -> torch.Tensor:
    """Float rows of ``table`` (compute dtype) at int32 ``ids``, times ``scale``: the start of the residual stream.
    An id -(i + 1) reads its token from ``pending[i]`` (int32, on the device)."""
    M = ids.numel()
    V, H = table.shape
    _chk(ids, "embedding ids", torch.int32)
    if pending is not None:
        _chk(pending, "pending tokens", torch.int32)
    _chk(table, "embedding table", (torch.float32, torch.bfloat16))
    if out is None:
        out = torch.empty(M, H, dtype=torch.float32, device=table.device)
    _chk(out, "embedding output", torch.float32, (M, H))
    check(fn("snk_embedding")(_ptr(ids), _ptr(pending), pending.numel() if pending is not None else 0,
                              _ptr(table), _ptr(out), M, H, V, code_of(table.dtype), float(scale), _stream()),
          "embedding",
          work=lambda: (M * H * table.element_size() + _nbytes(out, ids), 0))
    return out


def pair_embedding(ids, table, pairs, buckets: int, mul_prev: int, mul_cur: int, row_seg, cu_seqlens, seg_start,
                   seg_slot, last_token, pending=None, scale: float = 1.0, out=None):
    """The embedding with a second table read by a hash of (previous token, token):
    ``table[id] * scale + pairs[(prev * mul_prev + id * mul_cur) % buckets]``; a sequence's first token reads
    ``pairs[buckets]``.  ``last_token`` int32 [slots]: the request's last token of earlier steps (read for a
    segment that continues a sequence, then set to the segment's last token)."""
    M = ids.numel()
    V, H = table.shape
    _chk(ids, "embedding ids", torch.int32)
    if pending is not None:
        _chk(pending, "pending tokens", torch.int32)
    _chk(table, "embedding table", (torch.float32, torch.bfloat16))
    _chk(pairs, "pair table", table.dtype, (buckets + 1, H))
    _chk(last_token, "last tokens", torch.int32)
    for name, t in (("row_seg", row_seg), ("cu_seqlens", cu_seqlens), ("seg_start", seg_start), ("seg_slot", seg_slot)):
        _chk(t, name, torch.int32)
    if out is None:
        out = torch.empty(M, H, dtype=torch.float32, device=table.device)
    _chk(out, "embedding output", torch.float32, (M, H))
    check(fn("snk_pair_embedding")(_ptr(ids), _ptr(pending), pending.numel() if pending is not None else 0,
                                   _ptr(table), _ptr(pairs), _ptr(out), M, H, V, code_of(table.dtype), float(scale),
                                   int(buckets), int(mul_prev), int(mul_cur), _ptr(row_seg), _ptr(cu_seqlens),
                                   _ptr(seg_start), _ptr(seg_slot), _ptr(last_token), _stream()), "pair_embedding",
          work=lambda: (2 * M * H * table.element_size() + _nbytes(out, ids), 0))
    return out


def softcap(logits, cap: float):
    """``logits <- cap * tanh(logits / cap)`` in place (float)."""
    _chk(logits, "logits", torch.float32)
    check(fn("snk_softcap")(_ptr(logits), logits.numel(), float(cap), _stream()), "softcap",
          work=lambda: (2 * _nbytes(logits), 0))
    return logits


class ExpertSum:
    """A residual delta that is still in pieces: the routed experts' outputs ``y`` [pairs, H] (float), where
    each (token, pick) pair's row lies (``pair_pos`` int32 [M*k]) and the picks' weights (``weights`` float
    [M, k]).  The norm that follows adds sum_j w[m, j] * y[pair_pos[m*k + j]] into the residual itself;
    ``dense()`` forms the sum for anyone else."""

    def __init__(self, y, pair_pos, weights):
        self.y, self.pair_pos, self.weights = y, pair_pos, weights
        self.shape = (weights.shape[0], y.shape[1])

    def dense(self) -> torch.Tensor:
        return moe_combine(self.y, self.pair_pos, self.weights)


class DeltaSum:
    """A residual delta that is the sum of two sublayers' outputs (a layer whose mixer and feed-forward
    read the same normalised input): ``a`` a float tensor [M, H], ``b`` a float tensor or an ``ExpertSum``.
    ``a_gate`` (float [M, n], its first column used): a logit per row whose sigmoid multiplies ``a``.
    A norm that knows it adds both into the residual itself; ``dense()`` forms the sum for anyone else."""

    def __init__(self, a, b, a_gate=None):
        self.a, self.b, self.a_gate = a, b, a_gate
        self.shape = tuple(a.shape)

    def dense(self) -> torch.Tensor:
        out = self.a.clone() if self.a_gate is None else self.a * torch.sigmoid(self.a_gate[:, :1])
        residual_add(out, self.b.dense() if isinstance(self.b, ExpertSum) else self.b)
        return out


class ScaledDelta:
    """A residual delta that enters the stream times a constant: ``residual += scale * delta`` (``delta`` a
    float tensor, an ``ExpertSum`` or a ``DeltaSum``).  The RMS norm's kernel applies the factor in its own
    sum; ``dense()`` forms the product for anyone else."""

    def __init__(self, delta, scale: float):
        self.delta, self.scale = delta, float(scale)
        self.shape = tuple(delta.shape)

    def dense(self) -> torch.Tensor:
        d = self.delta.dense() if hasattr(self.delta, "dense") else self.delta
        return d * self.scale


def add_rmsnorm(residual: torch.Tensor, delta, gamma: torch.Tensor, eps: float,
                dtype: torch.dtype, rows: torch.Tensor | None = None,
                out: torch.Tensor | None = None) -> torch.Tensor:
    """``residual += delta`` (if given), then RMSNorm of the sum into the compute dtype.  With
    ``rows`` only those rows are normalised and the residual is left as it is.  ``delta`` is a float
    tensor [M, H], an ``ExpertSum``, a ``DeltaSum`` of a tensor (with or without a gate per row) and an
    ``ExpertSum``, or any of these in a ``ScaledDelta``."""
    M, H = residual.shape
    _chk(residual, "residual", torch.float32)
    moe = gate = None
    dscale = 1.0
    if isinstance(delta, ScaledDelta):
        delta, dscale = delta.delta, delta.scale
    if isinstance(delta, DeltaSum):
        if H % 4 == 0 and isinstance(delta.b, ExpertSum) and isinstance(delta.a, torch.Tensor):
            moe, gate, delta = delta.b, delta.a_gate, delta.a
            _chk(moe.y, "expert outputs", torch.float32)
            _chk(moe.pair_pos, "pair positions", torch.int32, (M * moe.weights.shape[1],))
            _chk(moe.weights, "top-k weights", torch.float32)
            if gate is not None:
                _chk(gate, "row gate", torch.float32)
                if gate.dim() != 2 or gate.shape[0] != M:
                    raise KernelError(f"row gate of shape {tuple(gate.shape)}, want [{M}, n]")
        else:
            delta = delta.dense()
    if isinstance(delta, ExpertSum):
        if H % 4 == 0:
            moe, delta = delta, None
            _chk(moe.y, "expert outputs", torch.float32)
            _chk(moe.pair_pos, "pair positions", torch.int32, (M * moe.weights.shape[1],))
            _chk(moe.weights, "top-k weights", torch.float32)
        else:
            delta = delta.dense()
    if delta is not None:
        _chk(delta, "residual delta", torch.float32, (M, H))
    g32 = _small(gamma, "norm weight", dtype)
    _chk(gamma, "norm weight", shape=(H,))
    R = M if rows is None else rows.numel()
    if rows is not None:
        _chk(rows, "norm rows", torch.int32)
    if out is None:
        out = torch.empty(R, H, dtype=dtype, device=residual.device)
    _chk(out, "norm output", dtype, (R, H))
    check(fn("snk_add_rmsnorm")(_ptr(residual), _ptr(delta), _ptr(gamma), g32, _ptr(out), _ptr(rows),
                                R, H, float(eps), code_of(dtype), _ptr(moe.y if moe else None),
                                _ptr(moe.pair_pos if moe else None), _ptr(moe.weights if moe else None),
                                moe.weights.shape[1] if moe else 0, float(dscale), _ptr(gate),
                                gate.shape[1] if gate is not None else 0, _stream()), "add_rmsnorm",
          work=lambda: (R * H * 4 + _nbytes(out, gamma) + (_nbytes(delta) + M * H * 4 if delta is not None else 0)
                        + ((moe.weights.shape[1] + 1) * M * H * 4 if moe else 0), 0))
    return out


def residual_add(residual: torch.Tensor, delta: torch.Tensor) -> None:
    _chk(residual, "residual", torch.float32)
    _chk(delta, "residual delta", torch.float32, residual.shape)
    check(fn("snk_residual_add")(_ptr(residual), _ptr(delta), residual.numel(), _stream()), "residual_add")


def swiglu(gate_up: torch.Tensor, out: torch.Tensor | None = None, interleaved: bool = False) -> torch.Tensor:
    """[M, 2I] -> [M, I]: silu(gate) * up.  Columns are (gate | up), or with ``interleaved`` blocks of 8
    gate columns followed by the 8 up columns of the same features."""
    M, two_i = gate_up.shape
    _chk(gate_up, "swiglu input", (torch.float32, torch.bfloat16))
    if two_i % 2:
        raise KernelError("swiglu input needs an even width")
    inter = two_i // 2
    if out is None:
        out = torch.empty(M, inter, dtype=gate_up.dtype, device=gate_up.device)
    _chk(out, "swiglu output", gate_up.dtype, (M, inter))
    check(fn("snk_swiglu")(_ptr(gate_up), _ptr(out), M, inter, int(interleaved), code_of(gate_up.dtype), _stream()),
          "swiglu", work=lambda: (_nbytes(gate_up, out), 0))
    return out


# --- attention -------------------------------------------------------------------------

def qk_norm_rope_cache(qkv, q_gamma, k_gamma, eps, inv_freq, rot_dim, positions, row_seg, block_table,
                       page_size, pool, num_heads, num_kv_heads, head_dim, write_kv=True, q_out=None):
    """Per-head RMSNorm of q and k (if weights are given), rotary encoding (if ``inv_freq``), k and v
    written to the paged pool at each row's position; returns q as [M, heads, head_dim]."""
    M = qkv.shape[0]
    dtype = qkv.dtype
    width = (num_heads + (2 * num_kv_heads if write_kv else 0)) * head_dim
    _chk(qkv, "qkv", (torch.float32, torch.bfloat16), (M, width))
    has_norm = q_gamma is not None
    g32 = 0
    if has_norm:
        g32 = _small(q_gamma, "q norm weight", dtype)
        if _small(k_gamma, "k norm weight", dtype) != g32:
            raise KernelError("q and k norm weights must share a dtype")
        _chk(q_gamma, "q norm weight", shape=(head_dim,))
        _chk(k_gamma, "k norm weight", shape=(head_dim,))
    if inv_freq is not None:
        _chk(inv_freq, "inv_freq", torch.float32, (rot_dim // 2,))
    _chk(positions, "positions", torch.int32, (M,))
    _chk(row_seg, "row_seg", torch.int32, (M,))
    _chk(block_table, "block table", torch.int32)
    _chk(pool, "kv pool", dtype)
    if pool.dim() != 5 or tuple(pool.shape[1:]) != (2, num_kv_heads, page_size, head_dim):
        raise KernelError(f"kv pool shape {tuple(pool.shape)}, want [pages, 2, {num_kv_heads}, "
                          f"{page_size}, {head_dim}]")
    if q_out is None:
        q_out = torch.empty(M, num_heads, head_dim, dtype=dtype, device=qkv.device)
    _chk(q_out, "q output", dtype, (M, num_heads, head_dim))
    check(fn("snk_qk_norm_rope_cache")(
        _ptr(qkv), _ptr(q_gamma), _ptr(k_gamma), g32, int(has_norm), float(eps), _ptr(inv_freq),
        int(rot_dim if inv_freq is not None else 0), _ptr(positions), _ptr(row_seg), _ptr(block_table),
        block_table.shape[1], page_size, _ptr(pool), _ptr(q_out), M, num_heads, num_kv_heads, head_dim,
        int(write_kv), code_of(dtype), _stream()), "qk_norm_rope_cache",
        work=lambda: (2 * _nbytes(qkv), 0))
    return q_out


ATTENTION_TILE = 32


def _rows_attention_work(q, pool, positions, rows, window):
    """(bytes, flops) of attention for single rows: each row reads its keys and values of every kv head
    once (a look at the positions: only called with the ledger on)."""
    pos = positions.cpu().long()
    if rows is not None:
        pos = pos[rows.cpu().long()]
    keys = pos + 1
    if window:
        keys = keys.clamp(max=int(window))
    total = int(keys.sum())
    nh, hd = q.shape[1], q.shape[2]
    return (total * 2 * pool.shape[2] * hd * pool.element_size() + 2 * len(pos) * nh * hd * q.element_size(),
            4 * nh * hd * total)


def _tiles_attention_work(q, pool, tiles, window):
    """(bytes, flops) of attention for prompt tiles: the rows of a tile share their keys and values."""
    t = tiles.cpu().long()
    nh, hd = q.shape[1], q.shape[2]
    nbytes = flops = 0
    for _, _, n, p0 in t.tolist():
        last = p0 + n                                   # keys the tile's last row sees
        first = max(0, p0 - int(window) + 1) if window else 0
        pairs = sum(min(p + 1, int(window)) if window else p + 1 for p in range(p0, p0 + n))
        nbytes += (last - first) * 2 * pool.shape[2] * hd * pool.element_size() + 2 * n * nh * hd * q.element_size()
        flops += 4 * nh * hd * pairs
    return nbytes, flops


def attention_scratch_bytes(M: int, num_heads: int, head_dim: int, num_chunks: int) -> int:
    return int(fn("snk_paged_attention_scratch_bytes")(M, num_heads, head_dim, num_chunks))


def paged_attention(q, pool, block_table, page_size, positions, row_seg, scale, window=None,
                    chunk=None, num_chunks=1, scratch=None, out=None, rows=None):
    """Causal attention of each row of q [M, heads, head_dim] over its request's cached keys up to
    its own position.  ``chunk`` keys per block along the sequence (a multiple of 32) and
    ``num_chunks`` = the most chunks any row spans; more than one needs ``scratch`` bytes.
    ``rows`` (int32): serve only these rows of the batch; the others of ``out`` are left alone."""
    M, nh, hd = q.shape
    dtype = q.dtype
    _chk(q, "q", (torch.float32, torch.bfloat16))
    _chk(pool, "kv pool", dtype)
    nkv = pool.shape[2]
    _chk(positions, "positions", torch.int32, (M,))
    _chk(row_seg, "row_seg", torch.int32, (M,))
    _chk(block_table, "block table", torch.int32)
    if chunk is None:
        chunk = 1 << 30
        chunk -= chunk % ATTENTION_TILE
    if out is None:
        out = torch.empty(M, nh * hd, dtype=dtype, device=q.device)
    _chk(out, "attention output", dtype, (M, nh * hd))
    served = M
    if rows is not None:
        _chk(rows, "attention rows", torch.int32)
        served = rows.numel()
    if num_chunks > 1:
        need = attention_scratch_bytes(served, nh, hd, num_chunks)
        if scratch is None:
            scratch = torch.empty(need, dtype=torch.uint8, device=q.device)
        _chk(scratch, "attention scratch", torch.uint8)
        if scratch.numel() < need:
            raise KernelError(f"attention scratch holds {scratch.numel()} bytes, needs {need}")
    check(fn("snk_paged_attention_rows")(
        _ptr(q), _ptr(pool), _ptr(block_table), block_table.shape[1], page_size, _ptr(positions),
        _ptr(row_seg), _ptr(out), _ptr(scratch), served, nh, nkv, hd, int(window or 0), int(chunk),
        int(num_chunks), float(scale), code_of(dtype), _ptr(rows), _stream()), "paged_attention",
        launches=2 if num_chunks > 1 else 1, work=lambda: _rows_attention_work(q, pool, positions, rows, window))
    return out


PREFILL_TILE_ROWS = 64
PREFILL_HEAD_DIMS = (64, 128)


def attention_prefill_ok(q) -> bool:
    """Whether the tensor-core prompt kernel takes this q [M, heads, head_dim]."""
    return q.dtype == torch.bfloat16 and q.shape[2] in PREFILL_HEAD_DIMS


def prefill_tma_page_ok(page_size: int) -> bool:
    """Page sizes whose pages a TMA box brings into a 64-key tile whole (csrc/attention_mma.cu)."""
    return page_size in (8, 16, 32, 64)


PREFILL_TMA = os.environ.get("SNOWLLM_B200_PREFILL_TMA", "1") != "0"


def attention_prefill(q, pool, block_table, page_size, tiles, scale, out, window=None, tma=None):
    """Tensor-core causal attention for prompt portions: ``tiles`` int32 [n, 4] = (segment, first row,
    rows <= 64, position of the first row); writes those rows of ``out`` [M, heads*head_dim].
    ``tma``: bring keys and values in by TMA (default: wherever the page size allows); both ways give the
    same bits."""
    M, nh, hd = q.shape
    _chk(q, "q", torch.bfloat16)
    _chk(pool, "kv pool", torch.bfloat16)
    _chk(tiles, "attention tiles", torch.int32)
    _chk(block_table, "block table", torch.int32)
    _chk(out, "attention output", torch.bfloat16, (M, nh * hd))
    if tiles.dim() != 2 or tiles.shape[1] != 4:
        raise KernelError("attention tiles must be [n, 4]")
    if tma is None:
        tma = PREFILL_TMA and prefill_tma_page_ok(page_size)
    if tma:
        check(fn("snk_attention_prefill_tma")(
            _ptr(q), _ptr(pool), pool.shape[0], _ptr(block_table), block_table.shape[1], page_size, _ptr(tiles),
            tiles.shape[0], _ptr(out), nh, pool.shape[2], hd, int(window or 0), float(scale), _stream()),
            "attention_prefill_tma", work=lambda: _tiles_attention_work(q, pool, tiles, window))
    else:
        check(fn("snk_attention_prefill")(
            _ptr(q), _ptr(pool), _ptr(block_table), block_table.shape[1], page_size, _ptr(tiles), tiles.shape[0],
            _ptr(out), nh, pool.shape[2], hd, int(window or 0), float(scale), _stream()), "attention_prefill",
            work=lambda: _tiles_attention_work(q, pool, tiles, window))
    return out


PREFILL_TC_TILE_ROWS = 128
PREFILL_TC = os.environ.get("SNOWLLM_B200_PREFILL_TC", "1") != "0"


def attention_prefill_tc_ok(q, page_size: int) -> bool:
    """Whether the tcgen05 prompt kernel (csrc/attention_tc.cu) takes this q [M, heads, head_dim] and page size."""
    return (PREFILL_TC and q.dtype == torch.bfloat16 and q.shape[2] == 64
            and page_size in (8, 16, 32, 64, 128))


def attention_prefill_tc(q, pool, block_table, page_size, tiles, scale, out, window=None):
    """Causal attention for prompt portions on the tcgen05 tensor cores: ``tiles`` int32 [n, 4] = (segment,
    first row, rows <= 128, position of the first row); writes those rows of ``out`` [M, heads*64]."""
    M, nh, hd = q.shape
    _chk(q, "q", torch.bfloat16)
    _chk(pool, "kv pool", torch.bfloat16)
    _chk(tiles, "attention tiles", torch.int32)
    _chk(block_table, "block table", torch.int32)
    _chk(out, "attention output", torch.bfloat16, (M, nh * hd))
    if tiles.dim() != 2 or tiles.shape[1] != 4:
        raise KernelError("attention tiles must be [n, 4]")
    check(fn("snk_attention_prefill_tc")(
        _ptr(q), M, _ptr(pool), pool.shape[0], _ptr(block_table), block_table.shape[1], page_size, _ptr(tiles),
        tiles.shape[0], _ptr(out), nh, pool.shape[2], hd, int(window or 0), float(scale), _stream()),
        "attention_prefill_tc", work=lambda: _tiles_attention_work(q, pool, tiles, window))
    return out


def attention_prefill_tc_split(q, kpool, vpool, block_table, page_size, tiles, scale, out, *, window=None, keep=0,
                               slopes=None, sink=None, gate=None, gate_col=0):
    """``attention_prefill_tc`` over keys and values in pools of their own [pages, kv heads, page_size, 64], with
    the options of ``split_attention``: ``keep`` first positions beside the window, ``slopes`` and ``sink`` float
    [heads], ``gate`` [M, width] bfloat16 whose columns from ``gate_col`` hold a logit per head."""
    M, nh, hd = q.shape
    _chk(q, "q", torch.bfloat16)
    _chk(kpool, "key pool", torch.bfloat16)
    _chk(vpool, "value pool", torch.bfloat16, tuple(kpool.shape))
    _chk(tiles, "attention tiles", torch.int32)
    _chk(block_table, "block table", torch.int32)
    _chk(out, "attention output", torch.bfloat16)
    if out.numel() != M * nh * hd:
        raise KernelError(f"attention output of {out.numel()} elements for {M} rows of {nh} heads of {hd}")
    if tiles.dim() != 2 or tiles.shape[1] != 4:
        raise KernelError("attention tiles must be [n, 4]")
    if kpool.dim() != 4 or kpool.shape[2] != page_size or kpool.shape[3] != hd:
        raise KernelError(f"key pool {tuple(kpool.shape)}, want [pages, kv heads, {page_size}, {hd}]")
    for name, t in (("distance slopes", slopes), ("sink", sink)):
        if t is not None:
            _chk(t, name, torch.float32, (nh,))
    gate_ptr, gate_ld = c_void_p(0), 0
    if gate is not None:
        _chk(gate, "head gate", torch.bfloat16)
        if gate.dim() != 2 or gate.shape[0] != M or gate_col + nh > gate.shape[1]:
            raise KernelError(f"head gate of shape {tuple(gate.shape)} holds no {nh} columns from {gate_col} on")
        gate_ptr, gate_ld = c_void_p(gate.data_ptr() + gate_col * gate.element_size()), gate.shape[1]
    nkv = kpool.shape[1]

    def work():
        nbytes = flops = 0
        for _, _, n, p0 in tiles.cpu().tolist():
            first = max(0, p0 - int(window) + 1) if window else 0
            pairs = sum((min(p + 1, int(window)) if window else p + 1) + (min(max(p + 1 - int(window), 0), int(keep))
                                                                          if window else 0) for p in range(p0, p0 + n))
            nbytes += (p0 + n - first + min(int(keep), first)) * 2 * nkv * hd * 2 + 2 * n * nh * hd * 2
            flops += 4 * nh * hd * pairs
        return nbytes, flops
    check(fn("snk_attention_prefill_tc_split")(
        _ptr(q), M, _ptr(kpool), _ptr(vpool), kpool.shape[0], _ptr(block_table), block_table.shape[1], page_size,
        _ptr(tiles), tiles.shape[0], _ptr(out), nh, nkv, hd, int(window or 0), float(scale), int(keep or 0),
        _ptr(slopes), _ptr(sink), gate_ptr, gate_ld, _stream()), "attention_prefill_tc", work=work)
    return out


def attention_tc_status() -> int:
    """0, or the code of a wait that ran out inside the tcgen05 prompt kernel since the last call (clears it;
    synchronises the device)."""
    return int(fn("snk_attention_tc_status")())


DECODE_MMA_CHUNK = 256
DECODE_MMA_MAX_GROUP = 16


def attention_decode_mma_ok(q, num_kv_heads: int) -> bool:
    """Whether the tensor-core kernel for decoded rows takes this q [M, heads, head_dim]."""
    return (q.dtype == torch.bfloat16 and q.shape[2] in PREFILL_HEAD_DIMS
            and q.shape[1] // num_kv_heads <= DECODE_MMA_MAX_GROUP)


def decode_tma_page_ok(page_size: int) -> bool:
    """Page sizes whose pages a TMA box brings in whole (csrc/attention_mma.cu)."""
    return 8 <= page_size <= DECODE_MMA_CHUNK and page_size % 8 == 0 and DECODE_MMA_CHUNK % page_size == 0


DECODE_TMA = os.environ.get("SNOWLLM_B200_DECODE_TMA", "1") != "0"


def attention_decode_status() -> int:
    """0, or 1 when a block of the TMA decode kernel gave up waiting for its keys (clears it)."""
    return int(fn("snk_attention_decode_status")())


def attention_decode_mma(q, pool, block_table, page_size, positions, row_seg, scale, num_chunks, out,
                         window=None, scratch=None, rows=None, tma=None):
    """Tensor-core attention for rows with long runs of keys (decoded tokens): keys in chunks of 256, the
    q heads of a kv head as the rows of the MMA; chunks merged in order when there is more than one.
    ``tma``: bring keys and values in by TMA (default: wherever the page size allows); both ways give the
    same bits."""
    M, nh, hd = q.shape
    _chk(q, "q", torch.bfloat16)
    _chk(pool, "kv pool", torch.bfloat16)
    _chk(positions, "positions", torch.int32, (M,))
    _chk(row_seg, "row_seg", torch.int32, (M,))
    _chk(block_table, "block table", torch.int32)
    _chk(out, "attention output", torch.bfloat16, (M, nh * hd))
    served = M
    if rows is not None:
        _chk(rows, "attention rows", torch.int32)
        served = rows.numel()
    if num_chunks > 1:
        need = attention_scratch_bytes(served, nh, hd, num_chunks)
        if scratch is None:
            scratch = torch.empty(need, dtype=torch.uint8, device=q.device)
        _chk(scratch, "attention scratch", torch.uint8)
        if scratch.numel() < need:
            raise KernelError(f"attention scratch holds {scratch.numel()} bytes, needs {need}")
    if tma is None:
        tma = DECODE_TMA and decode_tma_page_ok(page_size)
    if tma:
        check(fn("snk_attention_decode_tma")(
            _ptr(q), _ptr(pool), pool.shape[0], _ptr(block_table), block_table.shape[1], page_size, _ptr(positions),
            _ptr(row_seg), _ptr(rows), _ptr(out), _ptr(scratch), served, nh, pool.shape[2], hd, int(window or 0),
            int(num_chunks), float(scale), _stream()), "attention_decode_tma",
            work=lambda: _rows_attention_work(q, pool, positions, rows, window))
    else:
        check(fn("snk_attention_decode_mma")(
            _ptr(q), _ptr(pool), _ptr(block_table), block_table.shape[1], page_size, _ptr(positions), _ptr(row_seg),
            _ptr(rows), _ptr(out), _ptr(scratch), served, nh, pool.shape[2], hd, int(window or 0), int(num_chunks),
            float(scale), _stream()), "attention_decode_mma",
            work=lambda: _rows_attention_work(q, pool, positions, rows, window))
    if num_chunks > 1:
        check(fn("snk_attention_merge")(_ptr(scratch), _ptr(positions), _ptr(out), served, nh, hd, int(window or 0),
                                        DECODE_MMA_CHUNK, int(num_chunks), BF16, _ptr(rows), _stream()),
              "attention_merge", work=lambda: (served * nh * (hd + 2) * 4 * int(num_chunks) + served * nh * hd * 2, 0))
    return out


def attention_decode_tma_split(q, kpool, vpool, block_table, page_size, positions, row_seg, scale, num_chunks, out, *,
                               window=None, keep=0, slopes=None, sink=None, gate=None, gate_col=0, scratch=None,
                               rows=None):
    """``attention_decode_mma`` by TMA over keys and values in pools of their own [pages, kv heads, page_size,
    64 or 128], with the options of ``split_attention``: ``keep`` first positions beside the window (a row's
    chunks of 256 keys are then the chunks of its kept keys followed by its window's; ``num_chunks`` counts
    both), ``slopes`` and ``sink`` float [heads], ``gate`` [M, width] bfloat16 whose columns from ``gate_col``
    hold a logit per head.  Every served row stands alone; ``rows`` (int32, on the device): the rows of the
    step to serve, when not all of them (the others' outputs are left as they are)."""
    M, nh, hd = q.shape
    served = M
    if rows is not None:
        _chk(rows, "attention rows", torch.int32)
        served = rows.numel()
    _chk(q, "q", torch.bfloat16)
    _chk(kpool, "key pool", torch.bfloat16)
    _chk(vpool, "value pool", torch.bfloat16, tuple(kpool.shape))
    _chk(positions, "positions", torch.int32, (M,))
    _chk(row_seg, "row_seg", torch.int32, (M,))
    _chk(block_table, "block table", torch.int32)
    _chk(out, "attention output", torch.bfloat16)
    if out.numel() != M * nh * hd:
        raise KernelError(f"attention output of {out.numel()} elements for {M} rows of {nh} heads of {hd}")
    if kpool.dim() != 4 or kpool.shape[2] != page_size or kpool.shape[3] != hd:
        raise KernelError(f"key pool {tuple(kpool.shape)}, want [pages, kv heads, {page_size}, {hd}]")
    for name, t in (("distance slopes", slopes), ("sink", sink)):
        if t is not None:
            _chk(t, name, torch.float32, (nh,))
    gate_ptr, gate_ld = c_void_p(0), 0
    if gate is not None:
        _chk(gate, "head gate", torch.bfloat16)
        if gate.dim() != 2 or gate.shape[0] != M or gate_col + nh > gate.shape[1]:
            raise KernelError(f"head gate of shape {tuple(gate.shape)} holds no {nh} columns from {gate_col} on")
        gate_ptr, gate_ld = c_void_p(gate.data_ptr() + gate_col * gate.element_size()), gate.shape[1]
    num_chunks = int(num_chunks)
    if num_chunks > 1:
        need = attention_scratch_bytes(served, nh, hd, num_chunks)
        if scratch is None:
            scratch = torch.empty(need, dtype=torch.uint8, device=q.device)
        _chk(scratch, "attention scratch", torch.uint8)
        if scratch.numel() < need:
            raise KernelError(f"attention scratch holds {scratch.numel()} bytes, needs {need}")
    nkv, keep = kpool.shape[1], int(keep or 0)

    def work():
        pos = positions.cpu().long()
        if rows is not None:
            pos = pos[rows.cpu().long()]
        keys = (pos + 1).clamp(max=int(window)) if window else pos + 1
        if keep:
            keys = keys + (pos + 1 - int(window)).clamp(min=0, max=keep)
        total = int(keys.sum())
        return total * 2 * nkv * hd * 2 + 2 * served * nh * hd * 2, 4 * nh * hd * total
    check(fn("snk_attention_decode_tma_split")(
        _ptr(q), _ptr(kpool), _ptr(vpool), kpool.shape[0], _ptr(block_table), block_table.shape[1], page_size,
        _ptr(positions), _ptr(row_seg), _ptr(rows), _ptr(out), _ptr(scratch), served, nh, nkv, hd, int(window or 0),
        num_chunks, float(scale), keep, _ptr(slopes), _ptr(sink), gate_ptr, gate_ld, _stream()),
        "attention_decode_tma", work=work)
    if num_chunks > 1:
        check(fn("snk_attention_merge_gated")(_ptr(scratch), _ptr(positions), _ptr(out), served, nh, hd,
                                              int(window or 0), keep, DECODE_MMA_CHUNK, num_chunks, gate_ptr, gate_ld,
                                              BF16, _ptr(rows), _stream()),
              "attention_merge", work=lambda: (served * nh * (hd + 2) * 4 * num_chunks + served * nh * hd * 2, 0))
    return out


class StatusWatch:
    """The error words of the kernels whose waits are bounded (TMA and tcgen05 kernels: a wait that runs out
    makes the block give up, and its rows of the output are then not to be trusted), read where the host
    synchronises with the stream anyway.

    ``peek()`` queues, on the current stream, a copy of every loaded library's status word into pinned host
    memory; it neither waits nor clears.  After the host has synchronised with the stream (an event, a
    read-back), ``check()`` raises KernelError if a word is set, and clears it on the device.  The words are
    sticky, so an error is never lost between a peek and a later check."""
    WORDS = (("gemm_tc", "snk_gemm_tc_status_peek", 1, lambda: gemm_tc_status()),
             ("gemm_tc2", "snk_gemm_tc2_status_peek", 1, lambda: gemm_tc2_status()[0]),
             ("attention_tc", "snk_attention_tc_status_peek", 1, lambda: attention_tc_status()),
             ("attention_mma", "snk_attention_decode_status_peek", 2, lambda: attention_decode_status()))

    def __init__(self):
        self.host = torch.zeros(sum(w[2] for w in self.WORDS), dtype=torch.int32).pin_memory()
        self._base = self.host.data_ptr()

    def peek(self) -> None:
        at = 0
        for library, peek, words, _ in self.WORDS:
            if build.is_loaded(library):
                check(fn(peek)(c_void_p(self._base + 4 * at), _stream()), peek, launches=0)
            at += words

    def check(self) -> None:
        """Call after the host has synchronised with a stream position behind a ``peek``."""
        if not bool(self.host.any()):
            return
        at, found = 0, []
        for library, _, words, clear in self.WORDS:
            codes = self.host[at:at + words].tolist()
            if any(codes):
                found.append(f"{library} (code {codes if words > 1 else codes[0]})")
                clear()
            at += words
        self.host.zero_()
        raise KernelError("a bounded wait ran out inside a kernel of " + ", ".join(found) +
                          ": the step's results are not to be trusted")


# --- short convolution -----------------------------------------------------------------

def short_conv(bcx, weight, state, cu_seqlens, seg_start, seg_slot, row_seg, out=None):
    """Gated causal depthwise convolution over [M, 3H] rows (B | C | x) of a flat batch of segments;
    ``state`` [slots, L-1, H] holds each request's history and is brought up to date."""
    M, three_h = bcx.shape
    dtype = bcx.dtype
    H = three_h // 3
    _chk(bcx, "conv input", (torch.float32, torch.bfloat16), (M, 3 * H))
    w32 = _small(weight, "conv weight", dtype)
    L = weight.shape[1]
    _chk(weight, "conv weight", shape=(H, L))
    _chk(state, "conv state", dtype)
    if state.dim() != 3 or tuple(state.shape[1:]) != (max(L - 1, 0), H):
        raise KernelError(f"conv state shape {tuple(state.shape)}, want [slots, {L - 1}, {H}]")
    B = seg_start.numel()
    _chk(cu_seqlens, "cu_seqlens", torch.int32, (B + 1,))
    _chk(seg_start, "seg_start", torch.int32, (B,))
    _chk(seg_slot, "seg_slot", torch.int32, (B,))
    _chk(row_seg, "row_seg", torch.int32, (M,))
    if out is None:
        out = torch.empty(M, H, dtype=dtype, device=bcx.device)
    _chk(out, "conv output", dtype, (M, H))
    check(fn("snk_short_conv")(_ptr(bcx), _ptr(weight), w32, _ptr(state), _ptr(cu_seqlens), _ptr(seg_start),
                               _ptr(seg_slot), _ptr(row_seg), _ptr(out), M, B, H, L, code_of(dtype),
                               _stream()), "short_conv", launches=2 if L > 1 and M != B else 1,
          work=lambda: (_nbytes(bcx, out, weight) + 2 * B * max(L - 1, 0) * H * state.element_size(), 2 * M * H * (L + 2)))
    return out


# --- matrix products -------------------------------------------------------------------

def causal_conv(u, channels: int, weight, state, cu_seqlens, seg_start, seg_slot, row_seg, out=None):
    """Depthwise causal convolution over time on the first ``channels`` columns of ``u`` [M, width]:
    y[t, c] = sum_j weight[c, j] * u~[t - taps + 1 + j, c], where u~ is the request's history (``state``
    [slots, taps-1, channels], the last taps-1 rows of earlier steps; zeros for a fresh request) followed by
    this step's rows; the state is brought up to date.  Returns y [M, channels]."""
    M, width = u.shape
    dtype = u.dtype
    _chk(u, "conv input", (torch.float32, torch.bfloat16))
    C, L = weight.shape
    if C != channels or channels > width:
        raise KernelError(f"conv weight {tuple(weight.shape)} over {channels} of {width} columns")
    w32 = _small(weight, "conv weight", dtype)
    _chk(state, "conv state", dtype)
    if tuple(state.shape[1:]) != (max(L - 1, 0), C):
        raise KernelError(f"conv state {tuple(state.shape)}, want [slots, {L - 1}, {C}]")
    B = seg_start.numel()
    if out is None:
        out = torch.empty(M, C, dtype=dtype, device=u.device)
    _chk(out, "conv output", dtype, (M, C))
    fused = M == B and L > 1
    check(fn("snk_causal_conv")(_ptr(u), width, _ptr(weight), w32, _ptr(state), _ptr(cu_seqlens), _ptr(seg_start),
                                _ptr(seg_slot), _ptr(row_seg), _ptr(out), C, M, B, C, L, code_of(dtype), _stream()),
          "causal_conv", launches=1 if fused or L == 1 else 2,
          work=(lambda: (2 * M * C * u.element_size(), 2 * M * C * L)) if fused or L == 1 else
          (lambda: [(2 * M * C * u.element_size(), 2 * M * C * L), (2 * B * (L - 1) * C * u.element_size(), 0)]))
    return out


def _gemm_work(rows, a, w, out, offsets):
    """(bytes, flops) of a product: a's rows and the result once, of a grouped W only the groups that own
    rows (a look at the offsets: only called with the ledger on)."""
    K = a.shape[1]
    N = w.shape[-2]
    wbytes = _nbytes(w)
    if offsets is not None:
        o = offsets.cpu()
        wbytes = wbytes // w.shape[0] * int((o[1:] > o[:-1]).sum())
    return rows * K * a.element_size() + wbytes + _nbytes(out), 2 * rows * N * K


def gemm_simt(a, w, out_dtype=None, out=None, a_rows=None, a_div=1, offsets=None, rows_out=None,
              max_rows_per_group=None):
    """a [M, K] times w [N, K]^T (or, grouped, w [G, N, K] over rows sorted by group) with float
    accumulation in k order on the CUDA cores."""
    dtype = a.dtype
    _chk(a, "gemm a", (torch.float32, torch.bfloat16))
    _chk(w, "gemm w", dtype)
    K = a.shape[1]
    grouped = offsets is not None
    if grouped:
        G, N, Kw = w.shape
        _chk(offsets, "group offsets", torch.int32, (G + 1,))
    else:
        G = 1
        N, Kw = w.shape
    if Kw != K:
        raise KernelError(f"gemm: a has K={K}, w has K={Kw}")
    M = rows_out if rows_out is not None else a.shape[0]
    if a_rows is not None:
        _chk(a_rows, "gemm row gather", torch.int32)
    out_dtype = out_dtype or dtype
    if out is None:
        out = torch.empty(M, N, dtype=out_dtype, device=a.device)
    _chk(out, "gemm out", out_dtype, (M, N))
    if out_dtype not in (dtype, torch.float32):
        raise KernelError("gemm output is the compute dtype or float32")
    check(fn("snk_gemm_simt")(_ptr(a), _ptr(w), _ptr(out), M, N, K, _ptr(a_rows), int(a_div), _ptr(offsets),
                              G, int(max_rows_per_group if grouped else M),
                              int(out_dtype == torch.float32), code_of(dtype), _stream()), "gemm_simt",
          work=lambda: _gemm_work(M, a, w, out, offsets))
    return out


def gemm_skinny_ok(a, w) -> bool:
    """Whether the few-rows bfloat16 kernel takes these operands."""
    return (a.dtype == torch.bfloat16 and a.shape[1] % 8 == 0 and a.data_ptr() % 16 == 0
            and w.data_ptr() % 16 == 0)


def gemm_skinny(a, w, out_dtype=None, out=None, a_rows=None, a_div=1, offsets=None, rows_out=None,
                rows_hint=None, swiglu=False):
    """bfloat16 a [M, K] times w [N, K]^T (or grouped w [G, N, K]) for few rows: W streams from memory
    once into tensor-core fragments.  ``rows_hint``: rows expected per group (sets the pass size)."""
    _chk(a, "gemm a", torch.bfloat16)
    _chk(w, "gemm w", torch.bfloat16)
    K = a.shape[1]
    grouped = offsets is not None
    if grouped:
        G, N, Kw = w.shape
        _chk(offsets, "group offsets", torch.int32, (G + 1,))
    else:
        G = 1
        N, Kw = w.shape
    if Kw != K:
        raise KernelError(f"gemm: a has K={K}, w has K={Kw}")
    M = rows_out if rows_out is not None else a.shape[0]
    if a_rows is not None:
        _chk(a_rows, "gemm row gather", torch.int32)
    out_dtype = out_dtype or torch.bfloat16
    cols = N // 2 if swiglu else N          # swiglu: w rows are gate/up interleaved by 8, out = silu(gate) * up
    if out is None:
        out = torch.empty(M, cols, dtype=out_dtype, device=a.device)
    _chk(out, "gemm out", out_dtype, (M, cols))
    if out_dtype not in (torch.bfloat16, torch.float32) or (swiglu and out_dtype != torch.bfloat16):
        raise KernelError("gemm output is bfloat16 or float32 (bfloat16 with swiglu)")
    check(fn("snk_gemm_skinny")(_ptr(a), _ptr(w), _ptr(out), M, N, K, _ptr(a_rows), int(a_div), _ptr(offsets),
                                G, int(rows_hint if rows_hint is not None else M),
                                int(out_dtype == torch.float32), int(swiglu), _stream()), "gemm_skinny",
          work=lambda: _gemm_work(M, a, w, out, offsets))
    return out


TC_TILE = 128


def gemm_tc_ok(a, w) -> bool:
    """Whether the tcgen05 kernel takes these operands (bfloat16, K a multiple of 8, 16-byte aligned)."""
    return (a.dtype == torch.bfloat16 and a.shape[1] % 8 == 0 and a.data_ptr() % 16 == 0
            and w.data_ptr() % 16 == 0)


def gemm_tc(a, w, out_dtype=None, out=None, offsets=None, swiglu=False):
    """bfloat16 a [M, K] times w [N, K]^T on the tcgen05 tensor cores, float accumulation in tensor
    memory.  Grouped: w [G, N, K], rows of ``a`` sorted by group, ``offsets`` int32 [G+1]."""
    _chk(a, "gemm a", torch.bfloat16)
    _chk(w, "gemm w", torch.bfloat16)
    M, K = a.shape
    grouped = offsets is not None
    if grouped:
        G, N, Kw = w.shape
        _chk(offsets, "group offsets", torch.int32, (G + 1,))
    else:
        G = 1
        N, Kw = w.shape
    if Kw != K:
        raise KernelError(f"gemm: a has K={K}, w has K={Kw}")
    out_dtype = out_dtype or torch.bfloat16
    cols = N // 2 if swiglu else N          # swiglu: w rows are gate/up interleaved by 8, out = silu(gate) * up
    if out is None:
        out = torch.empty(M, cols, dtype=out_dtype, device=a.device)
    _chk(out, "gemm out", out_dtype, (M, cols))
    if out_dtype not in (torch.bfloat16, torch.float32) or (swiglu and out_dtype != torch.bfloat16):
        raise KernelError("gemm output is bfloat16 or float32 (bfloat16 with swiglu)")
    row_tiles = -(-M // TC_TILE) + (G if grouped else 0)
    # few tiles: the product is split along K, and the parts' float planes need a place
    need = int(fn("snk_gemm_tc_scratch_bytes")(M, N, K, int(grouped)))
    scratch = torch.empty(need, dtype=torch.uint8, device=a.device) if need else None
    check(fn("snk_gemm_tc")(_ptr(a), _ptr(w), _ptr(out), M, N, K, _ptr(offsets), G, row_tiles,
                            int(out_dtype == torch.float32), int(swiglu), _ptr(scratch), _stream()), "gemm_tc",
          launches=2 if need else 1, work=lambda: _gemm_work(M, a, w, out, offsets))
    return out


def gemm_tc2(a, w, out_dtype=None, out=None, offsets=None, swiglu=False):
    """As ``gemm_tc``, on pairs of SMs (cta_group::2): 256 x 256 tiles of C, each block of a pair loading
    its 128 rows of ``a`` and half of the tile's rows of ``w``.  Grouped (``offsets``): the operands change
    places, each block loads 128 rows of the group's ``w`` and half of up to 256 of its rows of ``a``, and
    a group's last tile is as wide as its rows need (a multiple of 16); at most 256 groups."""
    _chk(a, "gemm a", torch.bfloat16)
    _chk(w, "gemm w", torch.bfloat16)
    M, K = a.shape
    grouped = offsets is not None
    if grouped:
        G, N, Kw = w.shape
        _chk(offsets, "group offsets", torch.int32, (G + 1,))
    else:
        G = 1
        N, Kw = w.shape
    if Kw != K:
        raise KernelError(f"gemm: a has K={K}, w has K={Kw}")
    out_dtype = out_dtype or torch.bfloat16
    cols = N // 2 if swiglu else N
    if out is None:
        out = torch.empty(M, cols, dtype=out_dtype, device=a.device)
    _chk(out, "gemm out", out_dtype, (M, cols))
    if out_dtype not in (torch.bfloat16, torch.float32) or (swiglu and out_dtype != torch.bfloat16):
        raise KernelError("gemm output is bfloat16 or float32 (bfloat16 with swiglu)")
    check(fn("snk_gemm_tc2")(_ptr(a), _ptr(w), _ptr(out), M, N, K, _ptr(offsets), G,
                             int(out_dtype == torch.float32), int(swiglu), _stream()), "gemm_tc2",
          work=lambda: _gemm_work(M, a, w, out, offsets))
    return out


def gemm_tc2_status():
    """(0 or the code of a wait that ran out inside the pair kernel since the last call, the tensor-memory
    addresses the two blocks of the first pair were given); synchronises the device."""
    addr = (ctypes.c_uint * 2)()
    return int(fn("snk_gemm_tc2_status")(addr)), (int(addr[0]), int(addr[1]))


def gemm_tc_is_split(M: int, N: int, K: int) -> bool:
    """Whether a plain tcgen05 product of these sizes is split along K (few tiles): its sums then have
    another order than the unsplit product's, so the same row may differ by rounding between the two."""
    return int(fn("snk_gemm_tc_scratch_bytes")(M, N, K, 0)) > 0


def gemm_tc_status() -> int:
    """0, or the code of a wait that ran out inside a tcgen05 kernel since the last call
    (synchronises the device; 1: operands never arrived, 2: a stage never came back, 3: the
    accumulator never became ready)."""
    return int(fn("snk_gemm_tc_status")())


def lose_loads(on: bool) -> None:
    """Test hook of the two tcgen05 product libraries: while on, their producers issue no loads, so the
    bounded waits inside the kernels run out and a launch returns with an error status (see
    ``gemm_tc_status``, ``gemm_tc2_status``, ``StatusWatch``) instead of a product."""
    check(fn("snk_gemm_tc_test_lose_loads")(int(on)), "gemm_tc test hook", 0)
    check(fn("snk_gemm_tc2_test_lose_loads")(int(on)), "gemm_tc2 test hook", 0)


def gather_rows(x, rows, div=1, out=None):
    """out[r] = x[rows[r] // div] for bfloat16 rows (the sorted copy the grouped tcgen05 product reads)."""
    _chk(x, "gather input", torch.bfloat16)
    _chk(rows, "gather rows", torch.int32)
    R, K = rows.numel(), x.shape[1]
    if out is None:
        out = torch.empty(R, K, dtype=x.dtype, device=x.device)
    _chk(out, "gather output", x.dtype, (R, K))
    check(fn("snk_gather_rows_bf16")(_ptr(x), _ptr(out), _ptr(rows), int(div), R, K, _stream()), "gather_rows",
          work=lambda: (2 * _nbytes(out), 0))
    return out


# --- routed experts --------------------------------------------------------------------

ROUTE_GEMM_MIN_ROWS = 64
ROUTER_SCORINGS = ("sigmoid", "softmax", "softmax_picked")


def _route_flags(norm_topk_prob, scoring: str) -> int:
    """The routing kernels' ``norm_topk`` argument: bit 0 renormalises the picks' weights by their sum, bit 1
    scores with a softmax over all experts instead of a sigmoid per expert, bit 2 ("softmax_picked") picks by
    the logits themselves (the bias then belongs to the logit) and weights by the softmax over the picked
    logits alone."""
    if scoring not in ROUTER_SCORINGS:
        raise KernelError(f"router scoring {scoring!r} (known: {', '.join(ROUTER_SCORINGS)})")
    if scoring == "softmax_picked":
        return 4
    return int(bool(norm_topk_prob)) | (2 if scoring == "softmax" else 0)


def moe_route(x, router_w, bias, top_k, norm_topk_prob, scaling, scoring: str = "sigmoid"):
    """(ids int32 [M, k], weights float [M, k]) of the router, computed in float: a sigmoid per expert, or
    (``scoring`` "softmax") a softmax over all experts' logits; the k largest scores are picked."""
    M, H = x.shape
    dtype = x.dtype
    _chk(x, "router input", (torch.float32, torch.bfloat16))
    w32 = _small(router_w, "router weight", dtype)
    E = router_w.shape[0]
    _chk(router_w, "router weight", shape=(E, H))
    if bias is not None:
        _chk(bias, "expert bias", torch.float32, (E,))
    ids = torch.empty(M, top_k, dtype=torch.int32, device=x.device)
    wts = torch.empty(M, top_k, dtype=torch.float32, device=x.device)
    if (M > ROUTE_GEMM_MIN_ROWS and router_w.dtype == torch.bfloat16 and gemm_tc_ok(x, router_w)
            and gemm_tc_is_split(M, E, H)):
        # many rows, few experts: a tcgen05 product split along K (float accumulation, float output)
        # whose partial sums the selection adds itself, in the order the product's own sum has
        nbytes = int(fn("snk_gemm_tc_scratch_bytes")(M, E, H, 0))
        parts = torch.empty(nbytes, dtype=torch.uint8, device=x.device)
        planes = ctypes.c_int(0)
        check(fn("snk_gemm_tc_parts")(_ptr(x), _ptr(router_w), _ptr(parts), M, E, H, ctypes.byref(planes),
                                      _stream()), "gemm_tc_parts",
              work=lambda: (_nbytes(x, router_w) + M * E * 4 * max(planes.value, 1), 2 * M * E * H))
        check(fn("snk_moe_topk")(_ptr(parts), _ptr(bias), _ptr(ids), _ptr(wts), M, E, top_k,
                                 _route_flags(norm_topk_prob, scoring), float(scaling), 0, planes.value, _stream()), "moe_topk")
        return ids, wts
    if M > ROUTE_GEMM_MIN_ROWS and router_w.dtype == torch.bfloat16 and gemm_skinny_ok(router_w, x):
        # many rows: the logits are a tensor-core product with float accumulation and float output.  The few
        # router rows take the place of the tokens in the few-rows kernel, which then streams x once and
        # leaves the logits transposed, [E, M].
        logits = gemm_skinny(router_w, x, out_dtype=torch.float32, rows_hint=min(E, 64))
        check(fn("snk_moe_topk")(_ptr(logits), _ptr(bias), _ptr(ids), _ptr(wts), M, E, top_k,
                                 _route_flags(norm_topk_prob, scoring), float(scaling), 1, 1, _stream()), "moe_topk")
        return ids, wts
    check(fn("snk_moe_route")(_ptr(x), _ptr(router_w), w32, _ptr(bias), _ptr(ids), _ptr(wts), M, H, E,
                              top_k, _route_flags(norm_topk_prob, scoring), float(scaling), code_of(dtype), _stream()),
          "moe_route", work=lambda: (_nbytes(x, router_w, ids, wts), 2 * M * E * H))
    return ids, wts


ROUTE_FUSED_MAX_ROWS = 32      # up to here: logits spread over the GPU, selection and sort in one block


def moe_route_sort(x, router_w, bias, top_k, norm_topk_prob, scaling, scoring: str = "sigmoid"):
    """Routing and the sort by expert together: (ids, weights, offsets, pair_pos, sorted_pair) as
    `moe_route` and `moe_sort` give them.  The few rows of a decode step take two launches made for
    them; a row's logits are the same numbers on every path but the tensor-core one."""
    M, H = x.shape
    E = router_w.shape[0]
    if M > ROUTE_FUSED_MAX_ROWS or 8 * E * min(M, 32) + 8 * M * top_k > 48 * 1024:
        ids, wts = moe_route(x, router_w, bias, top_k, norm_topk_prob, scaling, scoring)
        return (ids, wts) + moe_sort(ids, E)
    dtype = x.dtype
    _chk(x, "router input", (torch.float32, torch.bfloat16))
    w32 = _small(router_w, "router weight", dtype)
    _chk(router_w, "router weight", shape=(E, H))
    if bias is not None:
        _chk(bias, "expert bias", torch.float32, (E,))
    dev = x.device
    ints = torch.empty(M * top_k * 3 + E + 1, dtype=torch.int32, device=dev)
    floats = torch.empty(M * E + M * top_k, dtype=torch.float32, device=dev)
    pairs = M * top_k
    ids, pair_pos, sorted_pair = ints[:pairs].view(M, top_k), ints[pairs:2 * pairs], ints[2 * pairs:3 * pairs]
    offsets = ints[3 * pairs:]
    logits, wts = floats[:M * E], floats[M * E:].view(M, top_k)
    check(fn("snk_moe_route_sort")(_ptr(x), _ptr(router_w), w32, _ptr(bias), _ptr(logits), _ptr(ids), _ptr(wts),
                                   _ptr(offsets), _ptr(pair_pos), _ptr(sorted_pair), M, H, E, top_k,
                                   _route_flags(norm_topk_prob, scoring), float(scaling), code_of(dtype), _stream()),
          "moe_route_sort", launches=2, work=lambda: (_nbytes(x, router_w, ints, floats), 2 * M * E * H))
    return ids, wts, offsets, pair_pos, sorted_pair


NORM_ROUTE_MAX_ROWS = 32
# Off by default: measured in the decode step of the 8B-A1B sizes it gains nothing (batch 1: 1.488 ms against
# 1.471 ms with the three launches it replaces; batch 8: 3.012 against 2.966 ms).  Inside a captured step the
# three launches hide one another's start, and one block per row walks norm, 32 dot products, selection and
# sort one after the other (12.4 us against 3.3 + 4.2 + 5.4 us).
FUSE_ROUTER = os.environ.get("SNOWLLM_B200_FUSE_ROUTER", "0") != "0"


def norm_route_sort_ok(residual, delta, gamma, router_w, top_k) -> bool:
    """Whether the one-launch front of a routed feed-forward (csrc/moe.cu: norm_route_sort_kernel) takes these
    operands (the switch ``FUSE_ROUTER`` is the caller's business)."""
    M, H = residual.shape
    E = router_w.shape[0]
    plain = delta is None or isinstance(delta, ExpertSum) or (torch.is_tensor(delta) and delta.data_ptr() % 16 == 0)
    return (M <= NORM_ROUTE_MAX_ROWS and H % 4 == 0 and H <= 32768 and top_k <= 32 and plain
            and residual.data_ptr() % 16 == 0 and (max(H, 2 * E + 4) + 40 + 2 * E) * 4 <= 200 * 1024)


def norm_route_sort(residual, delta, gamma, eps, dtype, router_w, bias, top_k, norm_topk_prob, scaling, ticket):
    """``residual += delta`` (a float tensor, an ``ExpertSum`` or None), RMSNorm into ``dtype``, the sigmoid
    router on the normalised rows, and the sort of the (token, pick) pairs by expert, in one launch for the
    few rows of a decode step: (x, ids, weights, offsets, pair_pos, sorted_pair), the same values as
    ``add_rmsnorm`` followed by ``moe_route_sort`` give.  ``ticket``: one int32 on the device, zero before
    the first call; the kernel leaves it zero."""
    M, H = residual.shape
    E = router_w.shape[0]
    _chk(residual, "residual", torch.float32)
    moe = None
    if isinstance(delta, ExpertSum):
        moe, delta = delta, None
        _chk(moe.y, "expert outputs", torch.float32)
        _chk(moe.pair_pos, "pair positions", torch.int32, (M * moe.weights.shape[1],))
        _chk(moe.weights, "top-k weights", torch.float32)
    if delta is not None:
        _chk(delta, "residual delta", torch.float32, (M, H))
    g32 = _small(gamma, "norm weight", dtype)
    _chk(gamma, "norm weight", shape=(H,))
    w32 = _small(router_w, "router weight", dtype)
    _chk(router_w, "router weight", shape=(E, H))
    if bias is not None:
        _chk(bias, "expert bias", torch.float32, (E,))
    _chk(ticket, "ticket", torch.int32, (1,))
    dev = residual.device
    x = torch.empty(M, H, dtype=dtype, device=dev)
    pairs = M * top_k
    ints = torch.empty(pairs * 3 + E + 1, dtype=torch.int32, device=dev)
    wts = torch.empty(M, top_k, dtype=torch.float32, device=dev)
    ids, pair_pos, sorted_pair = ints[:pairs].view(M, top_k), ints[pairs:2 * pairs], ints[2 * pairs:3 * pairs]
    offsets = ints[3 * pairs:]
    check(fn("snk_norm_route_sort")(
        _ptr(residual), _ptr(delta), _ptr(gamma), g32, _ptr(x), H, float(eps), _ptr(moe.y if moe else None),
        _ptr(moe.pair_pos if moe else None), _ptr(moe.weights if moe else None), moe.weights.shape[1] if moe else 0,
        _ptr(router_w), w32, _ptr(bias), _ptr(ids), _ptr(wts), _ptr(offsets), _ptr(pair_pos), _ptr(sorted_pair),
        M, E, top_k, int(bool(norm_topk_prob)), float(scaling), code_of(dtype), _ptr(ticket), _stream()),
        "norm_route_sort",
        work=lambda: (2 * M * H * 4 + _nbytes(x, router_w, ints, wts) + (_nbytes(delta) if delta is not None else 0)
                      + (moe.weights.shape[1] * M * H * 4 if moe else 0), 2 * M * E * H))
    return x, ids, wts, offsets, pair_pos, sorted_pair


def row_dot(x, w):
    """One float logit per row: ``x`` [M, H] (compute dtype) . ``w`` [H] or [1, H] (float32 or the compute dtype);
    returns float [M, 1]."""
    M, H = x.shape
    _chk(x, "row gate input", (torch.float32, torch.bfloat16))
    w32 = _small(w, "row gate weight", x.dtype)
    if w.numel() != H:
        raise KernelError(f"row gate weight of {w.numel()} elements for rows of {H}")
    out = torch.empty(M, 1, dtype=torch.float32, device=x.device)
    check(fn("snk_row_dot")(_ptr(x), _ptr(w), w32, _ptr(out), M, H, code_of(x.dtype), _stream()), "row_dot",
          work=lambda: (_nbytes(x, w, out), 2 * M * H))
    return out


def moe_sort(topk_ids, num_experts):
    """(offsets int32 [E+1], pair_pos int32 [M*k], sorted_pair int32 [M*k]) of the pairs sorted by
    expert."""
    _chk(topk_ids, "top-k ids", torch.int32)
    pairs = topk_ids.numel()
    dev = topk_ids.device
    offsets = torch.empty(num_experts + 1, dtype=torch.int32, device=dev)
    pair_pos = torch.empty(pairs, dtype=torch.int32, device=dev)
    sorted_pair = torch.empty(pairs, dtype=torch.int32, device=dev)
    check(fn("snk_moe_sort")(_ptr(topk_ids), _ptr(offsets), _ptr(pair_pos), _ptr(sorted_pair), pairs,
                             num_experts, _stream()), "moe_sort")
    return offsets, pair_pos, sorted_pair


def moe_combine(y, pair_pos, topk_w, out=None):
    """out[m] = sum_j w[m, j] * y[pair_pos[m*k + j]] in float, j in order."""
    M, k = topk_w.shape
    H = y.shape[1]
    _chk(y, "expert outputs", torch.float32, (M * k, H))
    _chk(pair_pos, "pair positions", torch.int32, (M * k,))
    _chk(topk_w, "top-k weights", torch.float32)
    if out is None:
        out = torch.empty(M, H, dtype=torch.float32, device=y.device)
    _chk(out, "moe output", torch.float32, (M, H))
    check(fn("snk_moe_combine")(_ptr(y), _ptr(pair_pos), _ptr(topk_w), _ptr(out), M, H, k, _stream()),
          "moe_combine")
    return out


# --- sampling --------------------------------------------------------------------------

def argmax(logits, out=None):
    B, V = logits.shape
    _chk(logits, "logits", torch.float32)
    if out is None:
        out = torch.empty(B, dtype=torch.int32, device=logits.device)
    _chk(out, "argmax output", torch.int32, (B,))
    check(fn("snk_argmax")(_ptr(logits), _ptr(out), B, V, _stream()), "argmax", work=lambda: (_nbytes(logits), 0))
    return out


def apply_penalties(logits, row_offsets, ids, counts, presence, frequency, repetition):
    B, V = logits.shape
    _chk(logits, "logits", torch.float32)
    _chk(row_offsets, "penalty offsets", torch.int32, (B + 1,))
    _chk(ids, "penalty ids", torch.int32)
    _chk(counts, "penalty counts", torch.int32, ids.shape)
    for t, what in ((presence, "presence"), (frequency, "frequency"), (repetition, "repetition")):
        _chk(t, what + " penalty", torch.float32, (B,))
    check(fn("snk_apply_penalties")(_ptr(logits), _ptr(row_offsets), _ptr(ids), _ptr(counts), _ptr(presence),
                                    _ptr(frequency), _ptr(repetition), B, V, _stream()), "apply_penalties")


def sample(logits, temperature, top_k, top_p, uniform, out=None):
    B, V = logits.shape
    _chk(logits, "logits", torch.float32)
    _chk(temperature, "temperature", torch.float32, (B,))
    _chk(top_k, "top_k", torch.int32, (B,))
    _chk(top_p, "top_p", torch.float32, (B,))
    _chk(uniform, "uniform", torch.float32, (B,))
    if out is None:
        out = torch.empty(B, dtype=torch.int32, device=logits.device)
    _chk(out, "sample output", torch.int32, (B,))
    check(fn("snk_sample")(_ptr(logits), _ptr(temperature), _ptr(top_k), _ptr(top_p), _ptr(uniform),
                           _ptr(out), B, V, _stream()), "sample", work=lambda: (_nbytes(logits), 0))
    return out


# --- layers with norms on the sublayers' outputs; gated heads ---------------------------

ACTIVATIONS = {"silu": 0, "relu": 1, "gelu_tanh": 2, "relu2": 3}


def norm_add(residual, y, gamma, eps, dtype, x_out=None, want_x=True):
    """``residual += y / sqrt(mean(y^2) + eps) * gamma`` over rows of float ``y``; returns the new
    residual in the compute dtype (what the next sublayer reads), or None with ``want_x`` off."""
    M, H = residual.shape
    _chk(residual, "residual", torch.float32)
    _chk(y, "sublayer output", torch.float32, (M, H))
    g32 = _small(gamma, "norm weight", dtype)
    _chk(gamma, "norm weight", shape=(H,))
    if want_x and x_out is None:
        x_out = torch.empty(M, H, dtype=dtype, device=residual.device)
    if x_out is not None:
        _chk(x_out, "norm_add output", dtype, (M, H))
    check(fn("snk_norm_add")(_ptr(residual), _ptr(y), _ptr(gamma), g32, _ptr(x_out), M, H, float(eps),
                             code_of(dtype), _stream()), "norm_add",
          work=lambda: (3 * M * H * 4 + _nbytes(x_out, gamma), 0))
    return x_out


def cast_rows(x, dtype, out=None):
    """Float ``x`` in the compute dtype."""
    _chk(x, "cast input", torch.float32)
    if out is None:
        out = torch.empty(x.shape, dtype=dtype, device=x.device)
    _chk(out, "cast output", dtype, x.shape)
    check(fn("snk_cast_rows")(_ptr(x), _ptr(out), x.numel(), code_of(dtype), _stream()), "cast_rows",
          work=lambda: (_nbytes(x, out), 0))
    return out


GATED_ACTIVATIONS = dict(ACTIVATIONS, swish_clamp=4)


def gated_act(gate_up, activation: str, interleaved: bool = False, out=None, limit: float = 0.0):
    """[M, 2I] -> [M, I]: act(gate) * up with ``activation`` one of silu, relu, gelu_tanh, or ``swish_clamp``:
    g = min(gate, limit), u = clamp(up, -limit, limit), g * sigmoid(1.702 g) * (u + 1).  Columns are
    (gate | up), or with ``interleaved`` blocks of 8 gate columns followed by the 8 up columns."""
    M, two_i = gate_up.shape
    _chk(gate_up, "gated activation input", (torch.float32, torch.bfloat16))
    if activation not in GATED_ACTIVATIONS:
        raise KernelError(f"activation {activation!r} (known: {', '.join(GATED_ACTIVATIONS)})")
    if two_i % 2:
        raise KernelError("gated activation input needs an even width")
    inter = two_i // 2
    if out is None:
        out = torch.empty(M, inter, dtype=gate_up.dtype, device=gate_up.device)
    _chk(out, "gated activation output", gate_up.dtype, (M, inter))
    check(fn("snk_gated_act")(_ptr(gate_up), _ptr(out), M, inter, int(interleaved), GATED_ACTIVATIONS[activation],
                              float(limit), code_of(gate_up.dtype), _stream()), "gated_act",
          work=lambda: (_nbytes(gate_up, out), 0))
    return out


def head_norm_gate(a, heads, dv, eps, dtype, *, second=0, lam=0.0, weight=None, gate=None, gate_col=0,
                   mult=1.0, out=None, gate_act: str = "sigmoid"):
    """Per (row, head): o = a[..., :dv] - lam * a[..., second:second + dv] (the second term only with
    ``second``), o / sqrt(mean(o^2) + eps) * mult, times ``weight`` [heads*dv] and times
    sigmoid(gate[:, gate_col + head*dv + c]) where given (``gate_act`` "silu": times silu of it).  ``a``:
    float [M, heads, width]; ``gate``: a 2-D float or compute-dtype tensor whose columns from ``gate_col`` on
    hold the gate's pre-activation."""
    if gate_act not in ("sigmoid", "silu"):
        raise KernelError(f"gate activation {gate_act!r} (known: sigmoid, silu)")
    _chk(a, "head values", torch.float32)
    M = a.shape[0]
    stride = a.numel() // max(M * heads, 1)
    if a.numel() != M * heads * stride or stride < dv + second:
        raise KernelError(f"head values of shape {tuple(a.shape)} do not hold {heads} heads of {dv}")
    w32 = 0
    if weight is not None:
        w32 = _small(weight, "head norm weight", dtype)
        _chk(weight, "head norm weight", shape=(heads * dv,))
    g_ptr, g32, g_ld = c_void_p(0), 0, 0
    if gate is not None:
        _chk(gate, "gate", (torch.float32, dtype))
        if gate.dim() != 2 or gate.shape[0] != M or gate.shape[1] < gate_col + heads * dv:
            raise KernelError(f"gate of shape {tuple(gate.shape)} has no {heads * dv} columns from {gate_col} on")
        g32, g_ld = int(gate.dtype == torch.float32), gate.shape[1]
        g_ptr = c_void_p(gate.data_ptr() + gate_col * gate.element_size())
    if out is None:
        out = torch.empty(M, heads * dv, dtype=dtype, device=a.device)
    _chk(out, "gated heads", dtype, (M, heads * dv))
    check(fn("snk_head_norm_gate")(_ptr(a), stride, int(second), float(lam), _ptr(weight), w32, g_ptr, g32, g_ld,
                                   _ptr(out), M, heads, dv, float(eps), float(mult), int(gate_act == "silu"),
                                   code_of(dtype), _stream()),
          "head_norm_gate", work=lambda: (_nbytes(a, out) + M * heads * dv * (gate.element_size() if gate is not None else 0), 0))
    return out


def act_rows(x, activation: str, out=None):
    """``act(x)`` elementwise in x's dtype, ``activation`` one of silu, relu, gelu_tanh, relu2 (the square
    of relu); evaluated in float, rounded once at the store."""
    _chk(x, "activation input", (torch.float32, torch.bfloat16))
    if activation not in ACTIVATIONS:
        raise KernelError(f"activation {activation!r} (known: {', '.join(ACTIVATIONS)})")
    if out is None:
        out = torch.empty_like(x)
    _chk(out, "activation output", x.dtype, x.shape)
    check(fn("snk_act_rows")(_ptr(x), _ptr(out), x.numel(), ACTIVATIONS[activation], code_of(x.dtype), _stream()),
          "act_rows", work=lambda: (_nbytes(x, out), 0))
    return out


def rms_cols(x, off: int, n: int, weight, eps: float, out=None):
    """Columns [off, off + n) of every row of ``x`` [M, width] divided by their root mean square
    (eps inside the root) and multiplied by ``weight`` [n]; statistics in float; [M, n] in x's dtype."""
    _chk(x, "rms input", (torch.float32, torch.bfloat16))
    M, width = x.shape
    if off < 0 or off + n > width:
        raise KernelError(f"columns [{off}, {off + n}) of a matrix of width {width}")
    w32 = _small(weight, "rms weight", x.dtype)
    _chk(weight, "rms weight", shape=(n,))
    if out is None:
        out = torch.empty(M, n, dtype=x.dtype, device=x.device)
    _chk(out, "rms output", x.dtype, (M, n))
    check(fn("snk_rms_cols")(_ptr(x), width, int(off), _ptr(weight), w32, _ptr(out), M, int(n), float(eps),
                             code_of(x.dtype), _stream()), "rms_cols",
          work=lambda: (2 * M * n * x.element_size(), 0))
    return out


def add_dyt(residual, delta, weight, bias, alpha, dtype, rows=None, out=None):
    """``residual += delta`` (None, a float tensor, an ``ExpertSum`` or a ``DeltaSum``: its two parts are
    summed first, then added), then the Dynamic Tanh norm ``tanh(alpha * x) * weight + bias`` of the sum in
    the compute dtype.  With ``rows`` only those rows come out and the residual stays as it is."""
    M, H = residual.shape
    _chk(residual, "residual", torch.float32)
    da = db = moe = None
    if isinstance(delta, ScaledDelta) or (isinstance(delta, DeltaSum) and delta.a_gate is not None):
        delta = delta.dense()              # a factor or a gate per row: forms this kernel does not apply itself
    if isinstance(delta, DeltaSum):
        da, db = delta.a, delta.b
    elif delta is not None:
        da = delta
    if isinstance(da, ExpertSum):
        da, db = db, da
    if isinstance(db, ExpertSum):
        moe, db = db, None
        _chk(moe.y, "expert outputs", torch.float32)
        _chk(moe.pair_pos, "pair positions", torch.int32, (M * moe.weights.shape[1],))
        _chk(moe.weights, "top-k weights", torch.float32)
    for d in (da, db):
        if d is not None:
            _chk(d, "residual delta", torch.float32, (M, H))
    s32 = _small(weight, "norm weight", dtype)
    if _small(bias, "norm bias", dtype) != s32 or _small(alpha, "norm alpha", dtype) != s32:
        raise KernelError("the norm's weight, bias and alpha must share a dtype")
    _chk(weight, "norm weight", shape=(H,))
    _chk(bias, "norm bias", shape=(H,))
    if alpha.numel() != 1:
        raise KernelError("the norm's alpha is one number")
    R = M if rows is None else rows.numel()
    if rows is not None:
        _chk(rows, "norm rows", torch.int32)
    if out is None:
        out = torch.empty(R, H, dtype=dtype, device=residual.device)
    _chk(out, "norm output", dtype, (R, H))
    k = moe.weights.shape[1] if moe else 0
    check(fn("snk_add_dyt")(_ptr(residual), _ptr(da), _ptr(db), _ptr(moe.y if moe else None),
                            _ptr(moe.pair_pos if moe else None), _ptr(moe.weights if moe else None), k, _ptr(weight),
                            _ptr(bias), _ptr(alpha), s32, _ptr(out), _ptr(rows), R, H, code_of(dtype), _stream()),
          "add_dyt", work=lambda: (R * H * 4 * (1 + (rows is None and delta is not None) + (da is not None)
                                                + (db is not None) + k) + _nbytes(out), 0))
    return out


def moe_scaled_rows(x, sorted_pair, weights, top_k: int):
    """Rows for experts whose weight multiplies their input: (xs [pairs, K] with xs[r] = x[pair // k] *
    weights.flat[pair], pair = sorted_pair[r], in x's dtype; ones float [M, k])."""
    _chk(x, "expert input", (torch.float32, torch.bfloat16))
    _chk(sorted_pair, "sorted pairs", torch.int32)
    _chk(weights, "top-k weights", torch.float32)
    R, K = sorted_pair.numel(), x.shape[1]
    out = torch.empty(R, K, dtype=x.dtype, device=x.device)
    ones = torch.empty_like(weights)
    check(fn("snk_moe_scaled_rows")(_ptr(x), _ptr(sorted_pair), _ptr(weights), _ptr(out), _ptr(ones), R, K,
                                    int(top_k), code_of(x.dtype), _stream()), "moe_scaled_rows",
          work=lambda: (2 * _nbytes(out), 0))
    return out, ones


# --- latent attention -----------------------------------------------------------------------------

LATENT_ATTENTION_CHUNK = 256


def latent_prepare(q, q_off, kv, kv_off, c_gamma, eps, inv_freq, rot, positions, row_seg, block_table, page_size,
                   pool, H, dim, rd, r, write_kv=True):
    """The step's rows of a latent attention layer.  ``q`` [M, *] holds head h at column ``q_off`` + h *
    (dim + rd) as [dim unrotated, rd rotated]; ``kv`` [M, *] holds [r latent, rd shared rotated key part] at
    column ``kv_off`` (ignored without ``write_kv``).  The latent is divided by its root mean square and
    multiplied by ``c_gamma``; the first ``rot`` elements of every rotated part turn in pairs (2i, 2i+1) by
    position * inv_freq[i]; the row [r + rd] goes into its page of ``pool`` [pages, 1, page_size, r + rd].
    Returns (q_unrot [H, M, dim] head-major, q_rot [M, H, rd])."""
    dtype = q.dtype
    _chk(q, "queries", (torch.float32, torch.bfloat16))
    M = q.shape[0]
    if q.shape[1] < q_off + H * (dim + rd):
        raise KernelError(f"queries of width {q.shape[1]} hold no {H} heads of {dim + rd} from column {q_off}")
    g32 = 0
    if write_kv:
        _chk(kv, "latent projection", dtype)
        if kv.shape[0] != M or kv.shape[1] < kv_off + r + rd:
            raise KernelError(f"latent projection {tuple(kv.shape)} holds no {r + rd} columns from {kv_off}")
        g32 = _small(c_gamma, "latent norm weight", dtype)
        _chk(c_gamma, "latent norm weight", shape=(r,))
        _chk(pool, "latent pool", dtype)
        if tuple(pool.shape[1:]) != (1, page_size, r + rd):
            raise KernelError(f"latent pool {tuple(pool.shape)}, want [pages, 1, {page_size}, {r + rd}]")
    rot = int(rot) if inv_freq is not None else 0
    if rot:
        _chk(inv_freq, "inv_freq", torch.float32, (rot // 2,))
    _chk(positions, "positions", torch.int32, (M,))
    _chk(row_seg, "row_seg", torch.int32, (M,))
    _chk(block_table, "block table", torch.int32)
    q_unrot = torch.empty(H, M, dim, dtype=dtype, device=q.device)
    q_rot = torch.empty(M, H, rd, dtype=dtype, device=q.device)
    check(fn("snk_latent_prepare")(
        _ptr(q), q.shape[1], int(q_off), _ptr(kv if write_kv else None), kv.shape[1] if write_kv else 0, int(kv_off),
        _ptr(c_gamma if write_kv else None), g32, float(eps), _ptr(inv_freq), rot, _ptr(positions), _ptr(row_seg),
        _ptr(block_table), block_table.shape[1], page_size, _ptr(pool if write_kv else None), _ptr(q_unrot),
        _ptr(q_rot), M, H, dim, rd, r, int(write_kv), code_of(dtype), _stream()), "latent_prepare",
        work=lambda: ((2 * M * H * (dim + rd) + (2 * M * (r + rd) if write_kv else 0)) * q.element_size(), 0))
    return q_unrot, q_rot


def latent_attention_tile_rows(H: int, r: int, rd: int, dtype) -> int:
    """Rows of one request that a block of ``latent_attention`` serves beside each other for ``H`` heads over
    rows of r + rd (bfloat16 with r and rd multiples of 16 runs on the tensor cores, up to 64 (row, head) units a
    block; everything else on the CUDA cores, 16 units)."""
    return int(fn("snk_latent_attention_tile_rows")(int(H), int(r), int(rd), code_of(dtype)))


def latent_attention(q_abs, q_rot, pool, block_table, page_size, positions, row_seg, scale, *, window=None,
                     sink=None, tiles=None, tile_rows=1, out=None, num_chunks=1, scratch=None,
                     chunk=LATENT_ATTENTION_CHUNK):
    """Attention of all heads over one shared row per position: ``pool`` [pages, 1, page_size, r + rd] holds
    [latent r, rotated key part rd]; head h's score is (q_abs[h, m] . latent + q_rot[m, h] . key part) *
    scale, its value the latent.  ``q_abs`` [H, M, r] (head-major), ``q_rot`` [M, H, rd].  Causal, or with
    ``window`` the last ``window`` keys; ``sink`` float [H]: exp(sink[h]) joins the softmax's denominator.
    ``tiles`` int32 [n, 2] = (first row, rows <= tile_rows) of consecutive rows of one request covering the
    step, None: every row alone.  ``num_chunks`` > 1 (rows alone only): keys in chunks of ``chunk`` at
    absolute positions, merged in chunk order.  Returns the heads' weighted sums of the latent, [M, H, r]."""
    H, M, r = q_abs.shape
    rd = q_rot.shape[2]
    dtype = q_abs.dtype
    _chk(q_abs, "absorbed queries", (torch.float32, torch.bfloat16))
    _chk(q_rot, "rotated queries", dtype, (M, H, rd))
    _chk(pool, "latent pool", dtype)
    if pool.dim() != 4 or tuple(pool.shape[1:]) != (1, page_size, r + rd):
        raise KernelError(f"latent pool {tuple(pool.shape)}, want [pages, 1, {page_size}, {r + rd}]")
    _chk(positions, "positions", torch.int32, (M,))
    _chk(row_seg, "row_seg", torch.int32, (M,))
    _chk(block_table, "block table", torch.int32)
    if sink is not None:
        _chk(sink, "sink", torch.float32, (H,))
    n_tiles = M
    if tiles is not None:
        _chk(tiles, "attention tiles", torch.int32)
        if tiles.dim() != 2 or tiles.shape[1] != 2:
            raise KernelError("attention tiles must be [n, 2]")
        n_tiles = tiles.shape[0]
    if out is None:
        out = torch.empty(M, H, r, dtype=dtype, device=q_abs.device)
    _chk(out, "attention output", dtype, (M, H, r))
    num_chunks = int(num_chunks)
    if num_chunks > 1:
        if tiles is not None:
            raise KernelError("keys are cut into chunks for rows that stand alone only")
        need = attention_scratch_bytes(M, H, r, num_chunks)
        if scratch is None:
            scratch = torch.empty(need, dtype=torch.uint8, device=q_abs.device)
        _chk(scratch, "attention scratch", torch.uint8)
        if scratch.numel() < need:
            raise KernelError(f"attention scratch holds {scratch.numel()} bytes, needs {need}")

    def work():
        pos = positions.cpu().long()
        keys = (pos + 1).clamp(max=int(window)) if window else pos + 1
        total = int(keys.sum())
        groups = -(-H // 16)
        return (-(-total // max(tile_rows, 1)) * groups * (r + rd) * pool.element_size() + _nbytes(q_abs, q_rot, out),
                2 * H * (2 * r + rd) * total)
    check(fn("snk_latent_attention")(
        _ptr(q_abs), _ptr(q_rot), _ptr(pool), _ptr(block_table), block_table.shape[1], page_size, _ptr(positions),
        _ptr(row_seg), _ptr(tiles), n_tiles, int(tile_rows), _ptr(out), M, H, r, rd, int(window or 0), float(scale),
        _ptr(sink), int(chunk), num_chunks, _ptr(scratch), code_of(dtype), _stream()), "latent_attention", work=work)
    if num_chunks > 1:
        check(fn("snk_attention_merge")(_ptr(scratch), _ptr(positions), _ptr(out), M, H, r, int(window or 0),
                                        int(chunk), num_chunks, code_of(dtype), c_void_p(0), _stream()),
              "attention_merge", work=lambda: (M * H * (r + 2) * 4 * num_chunks + _nbytes(out), 0))
    return out


def heads_to_rows(x, out=None):
    """[H, M, d] (head-major) -> [M, H * d]."""
    _chk(x, "head-major values", (torch.float32, torch.bfloat16))
    H, M, d = x.shape
    if out is None:
        out = torch.empty(M, H * d, dtype=x.dtype, device=x.device)
    _chk(out, "row-major values", x.dtype, (M, H * d))
    check(fn("snk_heads_to_rows")(_ptr(x), _ptr(out), M, H, d, code_of(x.dtype), _stream()), "heads_to_rows",
          work=lambda: (2 * _nbytes(x), 0))
    return out


# --- attention over split pools ---------------------------------------------------------------

def split_prepare(proj, q_off, k_off, v_off, q_gamma, k_gamma, eps, inv_freq, rot_dim, rot_mult, positions,
                  row_seg, block_table, page_size, kpool, vpool, nq, nkv, maps, dk, dv, write_kv=True,
                  proj_bias=None, plain_norm=False, whole_norm=False):
    """Rows of a fused projection ``proj`` [M, width] (q at column ``q_off`` as [nq, dk], k at ``k_off`` as
    [nkv*maps, dk], v at ``v_off`` as [nkv, dv]): per-head RMS norm of q and k (if weights are given),
    rotation of the first ``rot_dim`` elements of each head by angle position * inv_freq with cos and sin
    times ``rot_mult`` (if ``inv_freq``), k and v written to their pools
    ([pages, nkv, page_size, maps*dk] and [pages, nkv, page_size, dv]); returns q [M, nq, dk].
    ``proj_bias`` (float [width]): added to the projection's columns first.  ``plain_norm``: q and k over
    their root mean square without a weight.  ``whole_norm``: ONE root mean square over all heads of q (and
    one over all of k), with weights of the projections' sizes [nq*dk] and [nkv*maps*dk]."""
    M, width = proj.shape
    dtype = proj.dtype
    _chk(proj, "projection", (torch.float32, torch.bfloat16))
    need = max(q_off + nq * dk, (k_off + nkv * maps * dk) if write_kv else 0, (v_off + nkv * dv) if write_kv else 0)
    if width < need:
        raise KernelError(f"projection of width {width} holds no {need} columns")
    has_norm = q_gamma is not None or plain_norm
    g32 = 0
    if proj_bias is not None:
        _chk(proj_bias, "projection bias", torch.float32, (width,))
    if q_gamma is not None:
        g32 = _small(q_gamma, "q norm weight", dtype)
        if _small(k_gamma, "k norm weight", dtype) != g32:
            raise KernelError("q and k norm weights must share a dtype")
        _chk(q_gamma, "q norm weight", shape=(nq * dk if whole_norm else dk,))
        _chk(k_gamma, "k norm weight", shape=(nkv * maps * dk if whole_norm else dk,))
    rot = int(rot_dim) if inv_freq is not None else 0
    if inv_freq is not None:
        _chk(inv_freq, "inv_freq", torch.float32, (rot // 2,))
    _chk(positions, "positions", torch.int32, (M,))
    _chk(row_seg, "row_seg", torch.int32, (M,))
    _chk(block_table, "block table", torch.int32)
    if write_kv:
        _chk(kpool, "key pool", dtype)
        _chk(vpool, "value pool", dtype)
        if tuple(kpool.shape[1:]) != (nkv, page_size, maps * dk) or tuple(vpool.shape[1:]) != (nkv, page_size, dv):
            raise KernelError(f"pools of shapes {tuple(kpool.shape)} and {tuple(vpool.shape)}, want [pages, {nkv}, "
                              f"{page_size}, {maps * dk}] and [pages, {nkv}, {page_size}, {dv}]")
    q_out = torch.empty(M, nq, dk, dtype=dtype, device=proj.device)
    check(fn("snk_split_prepare")(
        _ptr(proj), width, q_off, k_off, v_off, _ptr(proj_bias), _ptr(q_gamma), _ptr(k_gamma), g32,
        2 if whole_norm and has_norm else int(has_norm),
        float(eps),
        _ptr(inv_freq), rot, float(rot_mult), _ptr(positions), _ptr(row_seg), _ptr(block_table),
        block_table.shape[1], page_size, _ptr(kpool), _ptr(vpool), _ptr(q_out), M, nq, nkv * maps, nkv, dk, dv,
        int(write_kv), code_of(dtype), _stream()), "split_prepare",
        work=lambda: (2 * M * need * proj.element_size(), 0))
    return q_out


def split_attention_tile_rows(nq: int, nkv: int, maps: int, dk: int, dv: int, dtype, decode_only: bool) -> int:
    """Rows of one request that a block of ``split_attention`` serves for these sizes (0: too many heads per
    kv head).  bfloat16 with dk a multiple of 16 and dv a multiple of 8, both up to 128, runs on the tensor
    cores; everything else on the CUDA cores."""
    return int(fn("snk_split_attention_tile_rows")(int(nq), int(nkv), int(maps), int(dk), int(dv), code_of(dtype),
                                                   int(decode_only)))


SPLIT_ATTENTION_CHUNK = 256


def split_attention_decode_chunk(nq: int, nkv: int, maps: int, dk: int, dv: int, dtype) -> int:
    """Keys per chunk when rows stand alone (decoded tokens): 128 where the tensor-core kernel takes the
    sizes (a block brings its whole chunk in at once, 32 keys per warp), else 256."""
    return int(fn("snk_split_attention_decode_chunk")(int(nq), int(nkv), int(maps), int(dk), int(dv), code_of(dtype)))


def reach_code(window=None, block=None) -> int:
    """How the attention kernels are told which keys a query reaches: W > 0 the last W keys, -C < 0 the keys
    of the query's own block of C positions (counted from position 0), 0 every earlier key."""
    if window and block:
        raise KernelError("a sliding window and a block-local mask exclude one another")
    return int(window) if window else (-int(block) if block else 0)


def split_attention(q, kpool, vpool, block_table, page_size, positions, row_seg, scale, *, maps=1, window=None,
                    bias=None, tiles=None, tile_rows=1, out_dtype=None, out=None, num_chunks=1, scratch=None,
                    chunk=SPLIT_ATTENTION_CHUNK, block=None, head_scale=None, sink=None, keep=0, slopes=None,
                    gate=None, gate_col=0):
    """Causal attention of q [M, nq, dk] (nq = heads * maps) over keys [pages, nkv, page_size, maps*dk] and
    values [pages, nkv, page_size, dv]; query head (h, map) reads the key at offset map*dk of its kv head.
    ``window``: the last ``window`` keys only; ``block``: the keys of the query's own block of ``block``
    positions only.  ``head_scale`` float [nq]: a factor per query head on ``scale``.  ``sink`` float [nq]: one
    more term exp(sink) in each row's softmax sum, with no key and no value.  ``bias`` float [nq, L]: added to the scaled score by
    distance min(i - j, L - 1).  ``tiles`` int32 [n, 2] = (first row, rows <= tile_rows) of consecutive
    rows of one request, covering the step; None: every row alone.  ``num_chunks`` > 1 (rows alone only):
    a row's keys are cut into chunks of ``chunk`` (``split_attention_decode_chunk``) at absolute positions, one block each, and
    merged in chunk order (``num_chunks``: the most chunks a row spans; needs ``scratch`` bytes as
    ``attention_scratch_bytes`` says).  ``keep``: beside its window a query also reaches the positions below
    ``keep`` (``split_attention_chunks`` counts a row's chunks then).  ``slopes`` float [nq] (instead of
    ``bias``): slopes[head] * (i - j) is taken off the scaled score.  ``gate`` [M, width] in the compute dtype:
    head h's output is multiplied by sigmoid(gate[m, gate_col + h]).  Scores, weights and sums are float;
    returns [M, nq, dv] in ``out_dtype`` (float32 or the compute dtype)."""
    M, nq, dk = q.shape
    dtype = q.dtype
    _chk(q, "q", (torch.float32, torch.bfloat16))
    _chk(kpool, "key pool", dtype)
    _chk(vpool, "value pool", dtype)
    nkv, dv = vpool.shape[1], vpool.shape[3]
    if kpool.dim() != 4 or tuple(kpool.shape[1:]) != (nkv, page_size, maps * dk) or vpool.shape[2] != page_size:
        raise KernelError(f"key pool {tuple(kpool.shape)} and value pool {tuple(vpool.shape)} do not fit "
                          f"{nkv} kv heads, pages of {page_size} and {maps} maps of {dk}")
    _chk(positions, "positions", torch.int32, (M,))
    _chk(row_seg, "row_seg", torch.int32, (M,))
    _chk(block_table, "block table", torch.int32)
    if bias is not None:
        _chk(bias, "distance bias", torch.float32)
        if bias.dim() != 2 or bias.shape[0] != nq:
            raise KernelError(f"distance bias of shape {tuple(bias.shape)}, want [{nq}, distances]")
    for name, t in (("head scale", head_scale), ("sink", sink), ("distance slopes", slopes)):
        if t is not None:
            _chk(t, name, torch.float32, (nq,))
    if slopes is not None and bias is not None:
        raise KernelError("a bias table and distance slopes exclude one another")
    keep = int(keep or 0)
    if keep and not window:
        raise KernelError("kept first keys go with a sliding window")
    gate_ptr, gate_ld = c_void_p(0), 0
    if gate is not None:
        _chk(gate, "head gate", dtype)
        if gate.dim() != 2 or gate.shape[0] != M or gate_col + nq > gate.shape[1]:
            raise KernelError(f"head gate of shape {tuple(gate.shape)} holds no {nq} columns from {gate_col} on")
        gate_ptr, gate_ld = c_void_p(gate.data_ptr() + gate_col * gate.element_size()), gate.shape[1]
    reach = reach_code(window, block)
    n_tiles = M
    if tiles is not None:
        _chk(tiles, "attention tiles", torch.int32)
        if tiles.dim() != 2 or tiles.shape[1] != 2:
            raise KernelError("attention tiles must be [n, 2]")
        n_tiles = tiles.shape[0]
    out_dtype = out_dtype or dtype
    if out_dtype not in (dtype, torch.float32):
        raise KernelError("attention output is the compute dtype or float32")
    if gate is not None and out_dtype != dtype:
        raise KernelError("gated heads come out in the compute dtype")
    if out is None:
        out = torch.empty(M, nq, dv, dtype=out_dtype, device=q.device)
    _chk(out, "attention output", out_dtype, (M, nq, dv))
    num_chunks = int(num_chunks)
    if num_chunks > 1:
        if tiles is not None:
            raise KernelError("keys are cut into chunks for rows that stand alone only")
        need = attention_scratch_bytes(M, nq, dv, num_chunks)
        if scratch is None:
            scratch = torch.empty(need, dtype=torch.uint8, device=q.device)
        _chk(scratch, "attention scratch", torch.uint8)
        if scratch.numel() < need:
            raise KernelError(f"attention scratch holds {scratch.numel()} bytes, needs {need}")

    def work():
        pos = positions.cpu().long()
        keys = (pos + 1).clamp(max=int(window)) if window else (pos % int(block) + 1 if block else pos + 1)
        if keep:
            keys = keys + (pos + 1 - int(window)).clamp(min=0, max=keep)
        total = int(keys.sum())
        return (-(-total // max(tile_rows, 1)) * nkv * (maps * dk + dv) * kpool.element_size() + _nbytes(q, out),
                2 * nq * (dk + dv) * total)
    check(fn("snk_split_attention")(
        _ptr(q), _ptr(kpool), _ptr(vpool), _ptr(block_table), block_table.shape[1], page_size, _ptr(positions),
        _ptr(row_seg), _ptr(tiles), n_tiles, int(tile_rows), _ptr(out), int(out_dtype == torch.float32 and dtype != torch.float32),
        nq, nkv, int(maps), dk, dv, reach, float(scale), _ptr(bias if slopes is None else slopes),
        -1 if slopes is not None else (bias.shape[1] if bias is not None else 0), _ptr(head_scale), _ptr(sink),
        keep, gate_ptr, gate_ld, int(chunk), num_chunks, _ptr(scratch),
        code_of(dtype), _stream()), "split_attention", work=work)
    if num_chunks > 1:
        check(fn("snk_attention_merge_gated")(_ptr(scratch), _ptr(positions), _ptr(out), M, nq, dv, reach, keep,
                                              int(chunk), num_chunks, gate_ptr, gate_ld, code_of(out_dtype),
                                              c_void_p(0), _stream()),
              "attention_merge", work=lambda: (M * nq * (dv + 2) * 4 * num_chunks + _nbytes(out), 0))
    return out


# --- matrix memory --------------------------------------------------------------------------------

def mlstm(proj, q_off, k_off, v_off, i_off, f_off, bias_i, bias_f, cap, cu_seqlens, seg_start, seg_slot,
          state_s, state_n, state_m, heads, dk, dv, out=None):
    """The mLSTM recurrence over the segments of a flat batch.  ``proj``: float [M, width] with q, k
    ([heads, dk]), v ([heads, dv]) and the input and forget gates' pre-activations ([heads] each) at the
    given columns.  The states (float; [slots, heads, dk, dv], [slots, heads, dk], [slots, heads]) are read
    unless a segment starts at 0, and brought up to date.  Returns the raw head outputs, float [M, heads*dv]."""
    M, width = proj.shape
    _chk(proj, "mlstm projection", torch.float32)
    B = seg_start.numel()
    _chk(cu_seqlens, "cu_seqlens", torch.int32, (B + 1,))
    _chk(seg_start, "seg_start", torch.int32, (B,))
    _chk(seg_slot, "seg_slot", torch.int32, (B,))
    slots = state_s.shape[0]
    _chk(state_s, "mlstm matrix state", torch.float32, (slots, heads, dk, dv))
    _chk(state_n, "mlstm vector state", torch.float32, (slots, heads, dk))
    _chk(state_m, "mlstm maximum state", torch.float32, (slots, heads))
    if width < max(q_off + heads * dk, k_off + heads * dk, v_off + heads * dv, i_off + heads, f_off + heads):
        raise KernelError(f"mlstm projection of width {width} is too narrow")
    b32 = _small(bias_i, "input gate bias", torch.float32)
    if _small(bias_f, "forget gate bias", torch.float32) != b32:
        raise KernelError("gate biases must share a dtype")
    if out is None:
        out = torch.empty(M, heads * dv, dtype=torch.float32, device=proj.device)
    _chk(out, "mlstm output", torch.float32, (M, heads * dv))
    check(fn("snk_mlstm")(_ptr(proj), width, q_off, k_off, v_off, i_off, f_off, _ptr(bias_i), _ptr(bias_f), b32,
                          float(cap), _ptr(cu_seqlens), _ptr(seg_start), _ptr(seg_slot), _ptr(state_s),
                          _ptr(state_n), _ptr(state_m), _ptr(out), B, heads, dk, dv, _stream()), "mlstm",
          work=lambda: (M * (2 * heads * dk + 2 * heads * dv) * 4 + 2 * B * heads * dk * dv * 4,
                        4 * M * heads * dk * dv))
    return out


# --- decayed matrix memory (linear attention with a state of fixed size) ----------------------------

def decay_memory(proj, q_off, k_off, v_off, cu_seqlens, seg_start, seg_slot, state, heads, dk, dv, *,
                 gate_bias=None, gate_low=None, decay=None, inv_freq=None, rot_dim=0, k_scale=1.0, positions=None,
                 out=None, pieces=None):
    """S_t = diag(a_t) S_(t-1) + k_t v_t^T, o_t = S_t^T q_t per (segment, head) over a flat batch.  ``proj``:
    float [M, width] with q at ``q_off`` and k (or the gate's pre-activation) at ``k_off`` ([heads, dk] each)
    and v at ``v_off`` ([heads, dv]).  Gated form (``gate_bias`` and ``gate_low`` over [heads*dk]): f = low +
    (1 - low) * sigmoid(z + bias), a = f, k = 1 - f, q = silu(projection).  Fixed form (``decay`` float
    [heads]): a = decay[head] for every row; the first ``rot_dim`` elements of q and k of each head turn with
    ``positions`` (split halves, ``inv_freq`` float [rot_dim/2]); k times ``k_scale`` afterwards.  ``state``
    (float [slots, heads, dk, dv]) is read unless a segment starts at 0, and brought up to date.  Returns
    the raw head outputs, float [M, heads*dv].  ``pieces`` = (int32 [n, 4] = segment, first row, rows, flags
    with 1 for a segment's first piece and 2 for its last; int32 [B+1] = first piece of each segment): every
    piece is walked by blocks of its own, from the state that a scan over the pieces' own sums gives it."""
    M, width = proj.shape
    _chk(proj, "memory projection", torch.float32)
    B = seg_start.numel()
    _chk(cu_seqlens, "cu_seqlens", torch.int32, (B + 1,))
    _chk(seg_start, "seg_start", torch.int32, (B,))
    _chk(seg_slot, "seg_slot", torch.int32, (B,))
    _chk(state, "memory state", torch.float32, (state.shape[0], heads, dk, dv))
    if width < max(q_off + heads * dk, k_off + heads * dk, v_off + heads * dv):
        raise KernelError(f"memory projection of width {width} is too narrow")
    gated = gate_bias is not None
    g32 = 0
    if gated:
        g32 = _small(gate_bias, "gate bias", torch.float32)
        if gate_low is None or _small(gate_low, "gate lower bound", torch.float32) != g32:
            raise KernelError("gate bias and lower bound must both be given, in one dtype")
        _chk(gate_bias, "gate bias", shape=(heads * dk,))
        _chk(gate_low, "gate lower bound", shape=(heads * dk,))
    else:
        if decay is None:
            raise KernelError("a memory without a gate needs a decay per head")
        _chk(decay, "decay", torch.float32, (heads,))
        if inv_freq is not None and rot_dim:
            _chk(inv_freq, "inv_freq", torch.float32, (rot_dim // 2,))
            _chk(positions, "positions", torch.int32, (M,))
        else:
            inv_freq, rot_dim = None, 0
    if out is None:
        out = torch.empty(M, heads * dv, dtype=torch.float32, device=proj.device)
    _chk(out, "memory output", torch.float32, (M, heads * dv))
    table = cu_pieces = work = work_decay = prep = None
    n_pieces = 0
    if pieces is not None:
        table, cu_pieces = pieces
        n_pieces = table.shape[0]
        _chk(table, "memory pieces", torch.int32, (n_pieces, 4))
        _chk(cu_pieces, "first piece of each segment", torch.int32, (B + 1,))
        work = torch.empty(n_pieces, heads, dk, dv, dtype=torch.float32, device=proj.device)
        work_decay = torch.empty(n_pieces, heads, dk, dtype=torch.float32, device=proj.device)
        prep = torch.empty(3 if gated else 2, M, heads * dk, dtype=torch.float32, device=proj.device)
    check(fn("snk_decay_memory")(_ptr(proj), width, q_off, k_off, v_off, 0 if gated else 1, _ptr(gate_bias),
                                 _ptr(gate_low), g32, _ptr(decay), _ptr(inv_freq), int(rot_dim), float(k_scale),
                                 _ptr(positions), _ptr(cu_seqlens), _ptr(seg_start), _ptr(seg_slot), _ptr(state),
                                 _ptr(out), B, heads, dk, dv, _ptr(table), _ptr(cu_pieces), n_pieces, _ptr(work),
                                 _ptr(work_decay), _ptr(prep), M, _stream()), "decay_memory",
          launches=4 if n_pieces else 1, work=lambda: _decay_memory_work(M, B, heads, dk, dv, n_pieces, gated))
    return out


def _decay_memory_work(M, B, H, dk, dv, pieces, gated):
    """(bytes, flops) of the memory kernel; with pieces one pair per launch: prepare, collect, scan, emit.  A
    token's step on one element of S is three operations (a S, k v, their sum) and two more where o is formed."""
    rows_k, rows_v, cells = M * H * dk * 4, M * H * dv * 4, H * dk * dv
    if not pieces:
        return (2 * rows_k + 2 * rows_v + 2 * B * cells * 4, 5 * M * cells)
    prep = (3 if gated else 2) * rows_k
    return [(2 * rows_k + prep, 0),
            (prep - rows_k + rows_v + pieces * cells * 4, 3 * M * cells),
            (2 * pieces * cells * 4 + B * cells * 4, 2 * pieces * cells),
            (prep + 2 * rows_v + pieces * cells * 4 + B * cells * 4, 5 * M * cells)]


# --- several residual streams ------------------------------------------------------------------------

class StreamsDelta:
    """A residual stream kept as ``S`` streams (``streams`` float [M, S, W]) with the last sublayer's update
    still pending: its output ``y`` (a float tensor, an ``ExpertSum`` or a ``DeltaSum``), the matrix ``mix``
    (float [S, S], indexed [from, to]) and the weights ``out`` (float [S]): X'[t] = sum_s mix[s, t] X[s] +
    out[t] y.  The norm that follows applies it in its own kernel (``streams_norm``)."""

    def __init__(self, streams, y, mix, out):
        self.streams, self.y, self.mix, self.out = streams, y, mix, out
        self.shape = (streams.shape[0], streams.shape[2])

    def total(self) -> torch.Tensor:
        """The sum of the streams after the pending update, float [M, W] (for taps and tests; not a kernel path)."""
        y = self.y.dense() if hasattr(self.y, "dense") else self.y
        new = torch.einsum("st,msw->mtw", self.mix, self.streams) + self.out[None, :, None] * y[:, None, :]
        return new.sum(1)

    def dense(self):
        raise KernelError("several residual streams do not reduce to one delta: the norm that follows must be one "
                          "that reads streams (group_rmsnorm)")


def streams_norm(streams, weight, groups, eps, dtype, *, init=None, update: StreamsDelta | None = None,
                 read=None, rows=None, out=None):
    """The seam between two sublayers of a stream kept as ``streams`` float [M, S, W]: set the streams to S
    copies of ``init`` [M, W] (if given), apply the pending ``update`` (if given; its ``y`` may be in pieces),
    form u = sum_s read[s] X[s] (``read`` None: the plain sum) and normalise it in ``groups`` equal parts,
    times ``weight``.  With ``rows`` only those rows come out and the streams stay untouched."""
    M, S, W = streams.shape
    _chk(streams, "streams", torch.float32)
    if init is not None:
        _chk(init, "stream start", torch.float32, (M, W))
    da = db = moe = None
    mix = outw = None
    if update is not None:
        if update.streams is not streams:
            raise KernelError("the pending update belongs to other streams")
        y = update.y
        if isinstance(y, ScaledDelta) or (isinstance(y, DeltaSum) and y.a_gate is not None):
            y = y.dense()                  # a factor or a gate per row: forms this kernel does not apply itself
        if isinstance(y, DeltaSum):
            da, y = y.a, y.b
        if isinstance(y, ExpertSum):
            moe = y
            _chk(moe.y, "expert outputs", torch.float32)
            _chk(moe.pair_pos, "pair positions", torch.int32, (M * moe.weights.shape[1],))
            _chk(moe.weights, "top-k weights", torch.float32)
        elif da is None:
            da = y
        else:
            db = y
        for t in (da, db):
            if t is not None:
                _chk(t, "sublayer output", torch.float32, (M, W))
        mix, outw = update.mix, update.out
        _chk(mix, "stream mix", torch.float32, (S, S))
        _chk(outw, "stream out weights", torch.float32, (S,))
    if read is not None:
        _chk(read, "stream read weights", torch.float32, (S,))
    w32 = _small(weight, "norm weight", dtype)
    _chk(weight, "norm weight", shape=(W,))
    R = M if rows is None else rows.numel()
    if rows is not None:
        _chk(rows, "norm rows", torch.int32)
    if out is None:
        out = torch.empty(R, W, dtype=dtype, device=streams.device)
    _chk(out, "norm output", dtype, (R, W))
    k = moe.weights.shape[1] if moe else 0
    check(fn("snk_streams_norm")(_ptr(streams), _ptr(init), _ptr(da), _ptr(db), _ptr(moe.y if moe else None),
                                 _ptr(moe.pair_pos if moe else None), _ptr(moe.weights if moe else None), k,
                                 _ptr(mix), _ptr(outw), _ptr(read), _ptr(weight), w32, int(groups), float(eps),
                                 _ptr(out), _ptr(rows), R, S, W, int(update is not None), code_of(dtype), _stream()),
          "streams_norm",
          work=lambda: (R * W * 4 * ((S if init is None else 1) + (S if rows is None else 0)
                                     + (da is not None) + (db is not None) + k) + _nbytes(out), 0))
    return out


def pair_norm_mix(a, b, wa, wb, ca, cb, eps, out=None):
    """ca * a / rms(a) * wa + cb * b / rms(b) * wb over the width, float [M, W]: the outputs of two mixers
    side by side, each normalised with a weight of its own."""
    M, W = a.shape
    _chk(a, "left output", torch.float32)
    _chk(b, "right output", torch.float32, (M, W))
    w32 = _small(wa, "left weight", torch.bfloat16)
    if _small(wb, "right weight", torch.bfloat16) != w32:
        raise KernelError("the two weights must share a dtype")
    _chk(wa, "left weight", shape=(W,))
    _chk(wb, "right weight", shape=(W,))
    if out is None:
        out = torch.empty(M, W, dtype=torch.float32, device=a.device)
    _chk(out, "mixed output", torch.float32, (M, W))
    check(fn("snk_pair_norm_mix")(_ptr(a), _ptr(b), _ptr(wa), _ptr(wb), w32, float(ca), float(cb), float(eps),
                                  _ptr(out), M, W, _stream()), "pair_norm_mix",
          work=lambda: (_nbytes(a, b, out), 0))
    return out
