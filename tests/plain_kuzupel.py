"""A plain, slow implementation of the Kuzupel design on the CPU: one function per mechanism, written from the
design's equations, whole sequences at a time, no cache.  It shares nothing with the engine: the softmax is a
plain one over an explicit mask, the short convolution a loop over taps on a zero-padded sequence, the experts
are looped over.

Notation: W x means ``x @ W.T`` for a weight stored [out, in]; a sequence is [T, width] from position 0.
Everything runs in ``dtype`` (float64 by default).  A model is a dict: ``config`` (the parsed config.json) and
``tensors`` (name -> tensor)."""
from __future__ import annotations

import math

import torch

SWISH_SLOPE = 1.702          # the feed-forward's gate: g * sigmoid(1.702 g)
SLOPE_RANGE = 8.0            # distance slopes of the heads: 2^(-SLOPE_RANGE (h + 1) / heads)


def rms(x, eps):
    """x over the root of its mean square along the last axis (eps inside the root)."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def hashed_pair_rows(tokens, buckets: int, mul_prev: int, mul_cur: int):
    """Row of the pair table for each token: (previous * mul_prev + current * mul_cur) mod buckets; the first
    token of a sequence, which has no previous one, reads the table's extra last row (number ``buckets``)."""
    rows = [buckets]
    for prev, cur in zip(tokens[:-1], tokens[1:]):
        rows.append((prev * mul_prev + cur * mul_cur) % buckets)
    return torch.tensor(rows)


def embed(tokens, t, emb: dict):
    x = t["embed"][torch.tensor(tokens)] * emb.get("scale", 1.0)
    pair = emb.get("bigram")
    if pair is not None:
        x = x + t["bigram"][hashed_pair_rows(list(tokens), pair["buckets"], pair["mul_prev"], pair["mul_cur"])]
    return x


def causal_taps(u, w):
    """Depthwise causal convolution over time: u [T, C], w [C, taps];
    y[t] = sum_j w[:, j] * u[t - taps + 1 + j], zeros before the start."""
    T, C = u.shape
    taps = w.shape[1]
    padded = torch.cat((torch.zeros(taps - 1, C, dtype=u.dtype), u), 0)
    y = torch.zeros_like(u)
    for j in range(taps):
        y = y + w[:, j] * padded[j:j + T]
    return y


def rotate_halves(x, positions, base: float, dims: int):
    """x [T, heads, d]: element i < dims/2 turns with element i + dims/2 by positions * base^(-2i/dims);
    elements from dims on pass."""
    out = x.clone()
    half = dims // 2
    for i in range(half):
        a = positions.to(x.dtype) * base ** (-2.0 * i / dims)
        c, s = torch.cos(a)[:, None], torch.sin(a)[:, None]
        u, v = x[..., i], x[..., i + half]
        out[..., i] = u * c - v * s
        out[..., i + half] = v * c + u * s
    return out


def window_mask(T: int, size, keep_first: int = 0):
    """[T, T] bool: i sees j <= i with i - j < size (None: every j <= i), or j among the first ``keep_first``
    positions."""
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    if size is None:
        return j <= i
    return (j <= i) & ((i - j < size) | (j < keep_first))


def masked_softmax(s, mask, one_more: bool = False):
    """Rows of s [T, T] over their visible keys; ``one_more``: a term exp(0) = 1 joins the denominator."""
    s = s.masked_fill(~mask, -math.inf)
    m = s.max(-1, keepdim=True).values
    if one_more:
        m = torch.clamp(m, min=0.0)
    e = torch.exp(s - m)
    total = e.sum(-1, keepdim=True)
    if one_more:
        total = total + torch.exp(-m)
    return e / total


def slope_attention(h, t, m: dict, eps: float, p: str):
    """Windowed grouped-query attention without rotation: q and k each RMS-normed over the WHOLE projection
    (all heads at once) with a weight of that size; score = q.k * scale - slope[head] * (i - j)."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (rms(h @ t[p + "q"].T, eps) * t[p + "q.norm"]).view(T, H, d)
    k = (rms(h @ t[p + "k"].T, eps) * t[p + "k.norm"]).view(T, G, d)
    v = (h @ t[p + "v"].T).view(T, G, dv)
    mask = window_mask(T, (m.get("mask") or {}).get("size"))
    dist = (torch.arange(T)[:, None] - torch.arange(T)[None, :]).to(h.dtype)
    out = []
    for head in range(H):
        g = head // (H // G)
        slope = 2.0 ** (-SLOPE_RANGE * (head + 1) / H)
        s = q[:, head] @ k[:, g].T * m["scale"] - slope * dist
        out.append(masked_softmax(s, mask) @ v[:, g])
    return torch.cat(out, -1) @ t[p + "o"].T


def conv_gated_attention(h, t, m: dict, eps: float, p: str, positions):
    """Grouped-query attention whose projections pass a short causal convolution; q and k RMS-normed per head
    (one weight of ``dim`` for all heads), partly rotated; a window plus the first ``keep_first`` positions;
    one more term 1 in the softmax's denominator; each head times sigmoid of its own gate logit."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q, k, v = h @ t[p + "q"].T, h @ t[p + "k"].T, h @ t[p + "v"].T
    if m.get("conv"):
        q, k, v = (causal_taps(u, t[p + n + ".conv"]) for u, n in ((q, "q"), (k, "k"), (v, "v")))
    q = rms(q.view(T, H, d), eps) * t[p + "q.norm"]
    k = rms(k.view(T, G, d), eps) * t[p + "k.norm"]
    v = v.view(T, G, dv)
    rot = m.get("rot")
    if rot is not None:
        q = rotate_halves(q, positions, rot["base"], rot["dims"])
        k = rotate_halves(k, positions, rot["base"], rot["dims"])
    mask = window_mask(T, (m.get("mask") or {}).get("size"), (m.get("mask") or {}).get("keep_first", 0))
    gate = torch.sigmoid(h @ t[p + "g"].T)                       # [T, H]
    out = []
    for head in range(H):
        g = head // (H // G)
        s = q[:, head] @ k[:, g].T * m["scale"]
        out.append(masked_softmax(s, mask, one_more=True) @ v[:, g] * gate[:, head:head + 1])
    return torch.cat(out, -1) @ t[p + "o"].T


def clamped_glu(h, t, p: str, limit: float):
    g = torch.clamp(h @ t[p + "gate"].T, max=limit)
    u = torch.clamp(h @ t[p + "up"].T, -limit, limit)
    return (g * torch.sigmoid(SWISH_SLOPE * g) * (u + 1)) @ t[p + "down"].T


def picked_softmax_experts(h, t, mlp: dict, p: str, picks=None, router_input=None):
    """Router logits z = W_r h + b; the ``top`` largest logits are chosen (ties to the lower index) and
    weighted by the softmax over the chosen logits alone; a shared expert, times sigmoid(W_sg h), is added.
    ``picks`` [T, top] forces the choice."""
    E, top = mlp["router"]["experts"], mlp["router"]["top"]
    z = (h if router_input is None else router_input) @ t[p + "router"].T + t[p + "router.b"]
    if picks is None:
        picks = torch.sort(torch.argsort(-z, dim=-1, stable=True)[:, :top], -1).values
    w = torch.softmax(torch.gather(z, 1, picks), -1)
    out = torch.zeros(h.shape[0], t[p + "e0.down"].shape[0], dtype=h.dtype)
    for e in range(E):
        for slot in range(top):
            rows = picks[:, slot] == e
            if rows.any():
                out[rows] += w[rows, slot][:, None] * clamped_glu(h[rows], t, f"{p}e{e}.", mlp["expert"]["limit"])
    if mlp.get("shared") is not None:
        out = out + torch.sigmoid(h @ t[p + "shared.sg"].T) * clamped_glu(h, t, p + "shared.", mlp["shared"]["limit"])
    return out, picks


def soft_cap(z, cap):
    return z if not cap else cap * torch.tanh(z / cap)


def forward(model: dict, tokens, dtype=torch.float64, layers_out=None, picks=None, picks_out=None):
    """Logits [T, vocab] of one sequence from position 0.  ``layers_out``: a list that receives the residual
    stream after every layer.  ``picks``: {layer -> [T, top]} forces the experts' choice; ``picks_out``: a dict
    that receives {layer -> the choice made}."""
    cfg = model["config"]
    t = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in model["tensors"].items()}
    eps, mult = cfg["norm"]["eps"], cfg.get("residual_mult", 1.0)
    positions = torch.arange(len(tokens))
    x = embed(tokens, t, cfg.get("embedding") or {})
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = rms(x, eps) * t[p + "norm1"]
        if layer["type"] == "attention":
            y = slope_attention(h, t, layer["mixer"], eps, p + "mix.")
        else:
            y = conv_gated_attention(h, t, layer["mixer"], eps, p + "mix.", positions)
        x = x + mult * y
        mlp = layer.get("mlp")
        if mlp is not None:
            h = rms(x, eps) * t[p + "norm2"]
            if mlp["kind"] == "dense":
                y = clamped_glu(h, t, p + "mlp.", mlp["limit"])
            else:
                y, chosen = picked_softmax_experts(h, t, mlp, p + "mlp.", None if picks is None else picks.get(i))
                if picks_out is not None:
                    picks_out[i] = chosen
            x = x + mult * y
        if layers_out is not None:
            layers_out.append(x.clone())
    z = (rms(x, eps) * t["final.norm"]) @ t["head"].T
    return soft_cap(z, cfg.get("logit_softcap"))
