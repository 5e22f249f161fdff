"""Small Toderax configurations, weights that make faults show, and helpers to run a request through the
engine's step function (any cut into steps) and through the plain implementation."""
from __future__ import annotations

import copy

import torch

import plain_toderax as plain
from beledra_cases import cuts_of, relative_error, run_cuts, tokens_for, worst_row_error  # noqa: F401


def moe(ff=24, experts=5, top=2, limit=1.2, shared=(16, 0.8)):
    out = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}
    if shared is not None:
        out["shared"] = {"ff": shared[0], "limit": shared[1]}
    return out


def memory_layer(heads=3, dim=8, vdim=12, mlp="moe"):
    """hgrn2: a gated matrix memory."""
    return {"type": "hgrn2", "mixer": {"heads": heads, "dim": dim, "vdim": vdim}, "mlp": moe() if mlp == "moe" else mlp}


def pair_layer(heads=4, kv_heads=2, dim=12, vdim=20, scale=0.4, chunk=21, r_heads=3, r_dim=16, r_vdim=8,
               decay=(0.9, 0.99, 0.75), rot_dims=8, base=700.0, mlp="moe"):
    """parallel: block-local attention with sinks beside a retention memory."""
    left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if chunk is not None:
        left["mask"] = {"size": chunk}
    right = {"heads": r_heads, "dim": r_dim, "vdim": r_vdim, "decay": list(decay)}
    if rot_dims:
        right["rot"] = {"dims": rot_dims, "base": base}
    return {"type": "parallel", "mixer": {"left": left, "right": right}, "mlp": moe() if mlp == "moe" else mlp}


def config(layers, vocab=96, width=40, eps=1e-5, groups=5, streams=3, scale=3.0):
    out = {"architecture": "Toderax", "vocab": vocab, "width": width, "norm": {"eps": eps, "groups": groups},
           "embedding": {"scale": scale}, "layers": copy.deepcopy(layers)}
    if streams is not None:
        out["streams"] = streams
    return out


# both mixers, layers with and without a feed-forward, chunks that are no multiples of pages or tiles, one
# and several picks, with and without a shared expert, part of the head and the whole head turning, layers
# of one design with different sizes
MIXED = config([pair_layer(),
                memory_layer(),
                pair_layer(heads=3, kv_heads=3, dim=8, vdim=8, scale=0.7, chunk=33, r_heads=1, r_dim=8, r_vdim=24,
                           decay=(0.97,), rot_dims=8, base=50.0, mlp=moe(16, 3, 1, 2.0, None)),
                memory_layer(heads=2, dim=16, vdim=4, mlp=None),
                pair_layer(heads=2, kv_heads=1, dim=16, vdim=12, scale=0.25, chunk=19, r_heads=2, r_dim=12, r_vdim=12,
                           decay=(1.0, 0.5), rot_dims=4, mlp=None)])


def draw_weights(cfg: dict, seed: int = 0, dtype=torch.bfloat16) -> dict:
    """name -> tensor (as stored: ``dtype``) from the framework's seeded generator, with the small tensors
    redrawn so that each mechanism carries weight: sinks of spread 2, factors per head off 1, projection
    biases, lower bounds spread over (0, 0.9), gate biases that keep a long memory, stream weights that mix,
    routers whose scores are spread out."""
    from snowllm_b200.loader import build_model
    from snowllm_b200.weights import random_tensors
    model = build_model(cfg, "float32")
    tensors = random_tensors(model, seed, torch.float32, fan_in_scaled=True, norm_jitter=0.2)
    gen = torch.Generator().manual_seed(seed + 1)
    for name, t in tensors.items():
        leaf = name.split(".", 1)[1] if "." in name else name

        def randn(scale=1.0):
            return torch.randn(t.shape, generator=gen) * scale
        if leaf.endswith(".sink"):
            tensors[name] = randn(2.0)
        elif leaf.endswith(".temp"):
            tensors[name] = 0.5 + 1.5 * torch.rand(t.shape, generator=gen)
        elif leaf.endswith((".q.b", ".k.b", ".v.b")):
            tensors[name] = randn(0.5)
        elif leaf.endswith(".lower"):
            tensors[name] = 0.9 * torch.rand(t.shape, generator=gen)
        elif leaf.endswith(".f.b"):
            tensors[name] = 1.0 + randn()
        elif leaf.endswith(".mix.f"):
            tensors[name] = t * 2.0
        elif leaf.endswith(".router"):
            tensors[name] = t * 4.0
        elif ".hc" in name and leaf.endswith(".in"):
            tensors[name] = 1.0 / t.numel() + randn(0.3)
        elif ".hc" in name and leaf.endswith(".out"):
            tensors[name] = 1.0 + randn(0.4)
        elif ".hc" in name and leaf.endswith(".mix"):
            tensors[name] = torch.eye(t.shape[0]) * 0.8 + randn(0.15)
    return {k: v.to(dtype) for k, v in tensors.items()}


def write_folder(path, cfg: dict, tensors: dict):
    from snowllm_b200.loader import build_model
    from snowllm_b200.weights import write_model_folder
    return write_model_folder(path, build_model(cfg, "float32").config.to_json_dict(), tensors)


def plain_logits(cfg, tensors, tokens, layers_out=None, **kw):
    return plain.forward({"config": cfg, "tensors": tensors}, list(tokens), torch.float64, layers_out, **kw)
