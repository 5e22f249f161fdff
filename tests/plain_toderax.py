"""A plain, slow implementation of the Toderax design on the CPU: one function per mechanism, written from
the design's equations, whole sequences at a time, no cache.  It shares nothing with the engine: recurrences
are loops over tokens with the state as a matrix, the softmax is a plain one over an explicit mask, the
experts are looped over, the streams of the hyper-connections are a list.

Notation: a sequence's streams are X[s] [T, width]; u = sum_s in[s] X[s] is what a sublayer reads through
its norm; W x means ``x @ W.T`` for a weight stored [out, in].  Everything runs in ``dtype`` (float64 by
default).  A model is a dict: ``config`` (the parsed config.json) and ``tensors`` (name -> tensor)."""
from __future__ import annotations

import math

import torch

SWISH_SLOPE = 1.702          # the experts' gate: g * sigmoid(1.702 g)


def rms(x, eps):
    """x over the root of its mean square along the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def group_rms_norm(x, w, groups: int, eps: float):
    """The last axis in ``groups`` equal consecutive parts, each over its own root mean square; then w."""
    T, W = x.shape
    parts = x.reshape(T, groups, W // groups)
    return rms(parts, eps).reshape(T, W) * w


def silu(z):
    return z * torch.sigmoid(z)


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


def same_chunk_causal(T: int, size):
    """[T, T] bool: i sees j <= i of its own chunk of ``size`` positions (None: every j <= i)."""
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    ok = j <= i
    return ok if size is None else ok & (i // size == j // size)


def softmax_with_sink(s, mask, sink):
    """Rows of s [T, T] over their visible keys, with one more term exp(sink) in the denominator."""
    s = s.masked_fill(~mask, -math.inf)
    m = torch.maximum(s.max(-1, keepdim=True).values, sink.expand(s.shape[0], 1))
    e = torch.exp(s - m)
    return e / (e.sum(-1, keepdim=True) + torch.exp(sink - m))


def chunk_sink_attention(h, t, m: dict, eps: float, p: str):
    """Grouped-query softmax attention without positions: biased projections, q and k over their root mean
    square per head, score = q.k * scale * temp[head], keys of the row's own chunk only, a sink per head."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ t[p + "q"].T + t[p + "q.b"]).view(T, H, d)
    k = (h @ t[p + "k"].T + t[p + "k.b"]).view(T, G, d)
    v = (h @ t[p + "v"].T + t[p + "v.b"]).view(T, G, dv)
    q, k = rms(q, eps), rms(k, eps)
    mask = same_chunk_causal(T, (m.get("mask") or {}).get("size"))
    out = []
    for head in range(H):
        g = head // (H // G)
        s = q[:, head] @ k[:, g].T * m["scale"] * t[p + "temp"][head]
        out.append(softmax_with_sink(s, mask, t[p + "sink"][head]) @ v[:, g])
    return torch.cat(out, -1) @ t[p + "o"].T


def decayed_memory(q, k, v, decay):
    """S_t = diag(decay_t) S_(t-1) + k_t v_t^T, o_t = S_t^T q_t, S_0 = 0, for one head.  q, k [T, d];
    v [T, dv]; decay [T, d] (one number per row of S and token)."""
    T, d = q.shape
    S = torch.zeros(d, v.shape[1], dtype=q.dtype)
    out = []
    for i in range(T):
        S = decay[i][:, None] * S + k[i][:, None] * v[i][None, :]
        out.append(S.T @ q[i])
    return torch.stack(out)


def retention(h, t, m: dict, eps: float, p: str, positions):
    """Linear attention with one fixed decay per head: rotated q and k, k * dim^(-1/2), no softmax; each
    head's output over its root mean square, the heads gated by silu(W_g h)."""
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    q = (h @ t[p + "q"].T).view(T, H, d)
    k = (h @ t[p + "k"].T).view(T, H, d)
    v = (h @ t[p + "v"].T).view(T, H, dv)
    rot = m.get("rot")
    if rot is not None:
        q = rotate_halves(q, positions, rot["base"], rot["dims"])
        k = rotate_halves(k, positions, rot["base"], rot["dims"])
    k = k * d ** -0.5
    out = []
    for head in range(H):
        decay = torch.full((T, d), m["decay"][head], dtype=h.dtype)
        out.append(rms(decayed_memory(q[:, head], k[:, head], v[:, head], decay), eps))
    return (torch.cat(out, -1) * silu(h @ t[p + "g"].T)) @ t[p + "o"].T


def hgrn2(h, t, m: dict, eps: float, p: str):
    """Linear attention whose forget gate f (per head and channel, bounded below by ``lower``) is the decay
    and whose complement 1 - f is the key."""
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ t[p + "q"].T).view(T, H, d)
    v = (h @ t[p + "v"].T).view(T, H, dv)
    low = t[p + "lower"]
    f = (low + (1 - low) * torch.sigmoid(h @ t[p + "f"].T + t[p + "f.b"])).view(T, H, d)
    out = []
    for head in range(H):
        o = decayed_memory(q[:, head], 1 - f[:, head], v[:, head], f[:, head])
        out.append(rms(o, eps) * t[p + "norm"])
    return torch.cat(out, -1) @ t[p + "o"].T


def side_by_side(h, t, m: dict, eps: float, p: str, positions):
    """Two mixers on the same input; the result is half the sum of their outputs, each RMS-normed over the
    width with a weight of its own."""
    a = chunk_sink_attention(h, t, m["left"], eps, p + "left.")
    b = retention(h, t, m["right"], eps, p + "right.", positions)
    return 0.5 * (rms(a, eps) * t[p + "left.out"] + rms(b, eps) * t[p + "right.out"])


def clamped_expert(h, t, p: str, limit: float):
    g = torch.clamp(h @ t[p + "gate"].T, max=limit)
    u = torch.clamp(h @ t[p + "up"].T, -limit, limit)
    return (g * torch.sigmoid(SWISH_SLOPE * g) * (u + 1)) @ t[p + "down"].T


def routed_experts(h, t, mlp: dict, p: str, picks=None, router_input=None):
    """softmax over all experts' logits, the ``top`` largest chosen (ties to the lower index), their scores
    used as they are; a shared expert is added for every token.  ``picks`` [T, top] forces the choice."""
    E, top = mlp["router"]["experts"], mlp["router"]["top"]
    z = (h if router_input is None else router_input) @ t[p + "router"].T
    s = torch.softmax(z, -1)
    if picks is None:
        picks = torch.sort(torch.argsort(-s, dim=-1, stable=True)[:, :top], -1).values
    out = torch.zeros(h.shape[0], t[p + "e0.down"].shape[0], dtype=h.dtype)
    for e in range(E):
        rows = (picks == e).any(-1)
        if rows.any():
            out[rows] += s[rows, e][:, None] * clamped_expert(h[rows], t, f"{p}e{e}.", mlp["expert"]["limit"])
    if mlp.get("shared") is not None:
        out = out + clamped_expert(h, t, p + "shared.", mlp["shared"]["limit"])
    return out, picks


def hyper_step(X, t, p: str, sublayer):
    """One sublayer over the streams: it reads u = sum_s in[s] X[s]; afterwards, all at once,
    X'[t] = sum_s mix[s, t] X[s] + out[t] * y."""
    S = len(X)
    u = sum(t[p + "in"][s] * X[s] for s in range(S))
    y = sublayer(u)
    return [sum(t[p + "mix"][s, j] * X[s] for s in range(S)) + t[p + "out"][j] * y for j in range(S)]


def forward(model: dict, tokens, dtype=torch.float64, layers_out=None, picks=None, picks_out=None):
    """Logits [T, vocab] of one sequence from position 0.  ``layers_out``: a list that receives the sum of
    the streams after every layer.  ``picks``: {layer -> [T, top]} forces the experts' choice; ``picks_out``:
    a dict that receives {layer -> the choice made}."""
    cfg = model["config"]
    t = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in model["tensors"].items()}
    eps, groups = cfg["norm"]["eps"], cfg["norm"].get("groups", 1)
    T = len(tokens)
    positions = torch.arange(T)
    x = t["embed"][torch.tensor(tokens)] * (cfg.get("embedding") or {}).get("scale", 1.0)
    streams = cfg.get("streams")
    X = [x.clone() for _ in range(streams)] if streams else [x]

    def norm(name):
        return lambda u: group_rms_norm(u, t[name], groups, eps)

    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        if layer["type"] == "hgrn2":
            mixer = lambda h: hgrn2(h, t, layer["mixer"], eps, p + "mix.")
        else:
            mixer = lambda h: side_by_side(h, t, layer["mixer"], eps, p + "mix.", positions)
        subs = [("hc1.", lambda u: mixer(norm(p + "norm1")(u)))]
        if layer.get("mlp") is not None:
            forced = None if picks is None else picks.get(i)

            def feed_forward(u):
                y, chosen = routed_experts(norm(p + "norm2")(u), t, layer["mlp"], p + "mlp.", forced)
                if picks_out is not None:
                    picks_out[i] = chosen
                return y
            subs.append(("hc2.", feed_forward))
        for hc, sub in subs:
            X = hyper_step(X, t, p + hc, sub) if streams else [X[0] + sub(X[0])]
        if layers_out is not None:
            layers_out.append(sum(X))
    return norm("final.norm")(sum(X)) @ t["head"].T
