"""Small Kuzupel configurations, weights that make faults show, and helpers to run a request through the
engine's step function (any cut into steps) and through the plain implementation."""
from __future__ import annotations

import copy

import torch

import plain_kuzupel as plain
from beledra_cases import cuts_of, relative_error, run_cuts, tokens_for, worst_row_error  # noqa: F401


def dense(ff=40, limit=1.5):
    return {"kind": "dense", "ff": ff, "limit": limit}


def moe(ff=24, experts=5, top=2, limit=1.2, shared=(16, 0.8)):
    out = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}
    if shared is not None:
        out["shared"] = {"ff": shared[0], "limit": shared[1]}
    return out


def slope_layer(heads=4, kv_heads=2, dim=12, vdim=20, scale=0.4, window=21, mlp="moe"):
    """attention: a window, q and k normalised over the whole projection, a distance slope per head."""
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if window is not None:
        m["mask"] = {"size": window}
    return {"type": "attention", "mixer": m, "mlp": moe() if mlp == "moe" else mlp}


def conv_layer(heads=3, kv_heads=1, dim=16, vdim=8, scale=0.3, window=13, keep_first=3, conv=3, rot_dims=8,
               base=700.0, mlp="dense"):
    """attention_2: convolved projections, a window beside the first tokens, one more term in the softmax's
    sum, gated heads."""
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if window is not None:
        m["mask"] = {"size": window}
        if keep_first is not None:
            m["mask"]["keep_first"] = keep_first
    if conv:
        m["conv"] = conv
    if rot_dims:
        m["rot"] = {"dims": rot_dims, "base": base}
    return {"type": "attention_2", "mixer": m, "mlp": dense() if mlp == "dense" else mlp}


def config(layers, vocab=96, width=40, eps=1e-5, mult=0.6, cap=9.0, scale=3.0, pair=(53, 5, 11)):
    out = {"architecture": "Kuzupel", "vocab": vocab, "width": width, "norm": {"eps": eps},
           "embedding": {"scale": scale}, "layers": copy.deepcopy(layers)}
    if mult is not None:
        out["residual_mult"] = mult
    if cap is not None:
        out["logit_softcap"] = cap
    if pair is not None:
        out["embedding"]["bigram"] = {"buckets": pair[0], "mul_prev": pair[1], "mul_cur": pair[2]}
    return out


# both mixers, dense and routed feed-forwards and none, windows that are no multiples of pages or tiles, kept
# first tokens within one page and over several, one and several picks, with and without a shared expert,
# part of the head and the whole head turning, layers of one kind with different sizes
MIXED = config([conv_layer(),
                slope_layer(),
                conv_layer(heads=4, kv_heads=4, dim=8, vdim=12, scale=0.7, window=33, keep_first=20, conv=2, rot_dims=8,
                           base=50.0, mlp=moe(16, 3, 1, 2.0, None)),
                slope_layer(heads=2, kv_heads=1, dim=16, vdim=4, scale=0.25, window=50, mlp=None),
                conv_layer(heads=2, kv_heads=2, dim=12, vdim=12, scale=0.5, window=19, keep_first=1, conv=5, rot_dims=4,
                           mlp=moe(8, 4, 4, 0.7, (24, 3.0)))])


# heads of 64 for keys and values: the sizes the tcgen05 prompt kernel takes in bfloat16
HEADS_OF_64 = config([conv_layer(heads=6, kv_heads=3, dim=64, vdim=64, scale=0.11, window=52, keep_first=10, conv=3,
                                 rot_dims=16),
                      slope_layer(heads=4, kv_heads=1, dim=64, vdim=64, scale=0.15, window=170),
                      conv_layer(heads=2, kv_heads=2, dim=64, vdim=64, scale=0.2, window=150, keep_first=140, conv=2,
                                 rot_dims=64, mlp=None)], width=64)


def draw_weights(cfg: dict, seed: int = 0, dtype=torch.bfloat16) -> dict:
    """name -> tensor (as stored: ``dtype``) from the framework's seeded generator, with the small tensors
    redrawn so that each mechanism carries weight: conv taps of size one, gates and routers whose logits are
    spread out, router biases that change the choice, a pair table as large as the embedding."""
    from snowllm_b200.loader import build_model
    from snowllm_b200.weights import random_tensors
    model = build_model(cfg, "float32")
    tensors = random_tensors(model, seed, torch.float32, fan_in_scaled=True, norm_jitter=0.2)
    gen = torch.Generator().manual_seed(seed + 1)
    for name, t in tensors.items():
        def randn(scale=1.0):
            return torch.randn(t.shape, generator=gen) * scale
        if name.endswith(".conv"):
            tensors[name] = randn(0.7)
        elif name.endswith((".mix.g", ".shared.sg")):
            tensors[name] = t * 3.0
        elif name.endswith(".router"):
            tensors[name] = t * 3.0
        elif name.endswith(".router.b"):
            tensors[name] = randn(1.0)
        elif name == "bigram":
            tensors[name] = randn(2.0)
    return {k: v.to(dtype) for k, v in tensors.items()}


def write_folder(path, cfg: dict, tensors: dict):
    from snowllm_b200.loader import build_model
    from snowllm_b200.weights import write_model_folder
    return write_model_folder(path, build_model(cfg, "float32").config.to_json_dict(), tensors)


def plain_logits(cfg, tensors, tokens, layers_out=None, **kw):
    return plain.forward({"config": cfg, "tensors": tensors}, list(tokens), torch.float64, layers_out, **kw)
