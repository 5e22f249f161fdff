"""Typed configuration of the Toderax design, read from its config.json.

    {"architecture": "Toderax", "vocab": V, "width": W, "streams": S, "embedding": {"scale": c},
     "norm": {"eps": e, "groups": g}, "layers": [{"type": T, "mixer": {...}, "mlp": {...} | null}, ...]}

``type`` names the layer's mixer; ``mixer`` holds that mixer's sizes and constants:

* ``hgrn2``:    heads, dim, vdim
* ``parallel``: ``left`` {heads, kv_heads, dim, vdim, scale, mask.size (the block of the block-local mask;
                without it the layer is plainly causal)} and ``right`` {heads, dim, vdim, decay [one per
                head], rot {dims, base} (without it: no rotation)}

``mlp``: ``{"kind": "moe", "expert": {"ff", "limit"}, "router": {"experts", "top"}, "shared": {"ff", "limit"}
| absent}`` or null.  ``streams`` absent: one plain residual stream (no learned stream weights);
``norm.groups`` absent: 1; ``embedding.scale`` absent: 1.  Every size and constant comes from the file; what is
missing or unusable is reported in one ConfigError that lists every key."""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any

from ..errors import ConfigError
from .beledra import _is_num, _Reader

ARCHITECTURE = "Toderax"
LAYER_TYPES = ("hgrn2", "parallel")
MAX_STREAMS = 8


@dataclass(frozen=True)
class ToderaxLayer:
    type: str
    mixer: dict          # hgrn2: heads, dim, vdim; parallel: left {...}, right {...}
    mlp: dict | None     # {"ff", "limit", "experts", "top", "shared": {"ff", "limit"} | None}


@dataclass(frozen=True)
class ToderaxConfig:
    architecture: str
    vocab: int
    width: int
    streams: int | None
    embedding_scale: float
    norm_eps: float
    norm_groups: int
    layers: tuple

    def to_json_dict(self) -> dict[str, Any]:
        """config.json content that reads back to this configuration."""
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
               "embedding": {"scale": self.embedding_scale},
               "norm": {"eps": self.norm_eps, "groups": self.norm_groups},
               "layers": [{"type": l.type, "mixer": _mixer_json(l), "mlp": _mlp_json(l.mlp)} for l in self.layers]}
        if self.streams is not None:
            out["streams"] = self.streams
        return out


def _mixer_json(layer: ToderaxLayer) -> dict:
    m = copy.deepcopy(layer.mixer)
    if layer.type == "parallel":
        block = m["left"].pop("block", None)
        if block is not None:
            m["left"]["mask"] = {"size": block}
        if m["right"].get("rot") is None:
            m["right"].pop("rot", None)
    return m


def _mlp_json(mlp):
    if mlp is None:
        return None
    out = {"kind": "moe", "expert": {"ff": mlp["ff"], "limit": mlp["limit"]},
           "router": {"experts": mlp["experts"], "top": mlp["top"]}}
    if mlp.get("shared") is not None:
        out["shared"] = dict(mlp["shared"])
    return out


def _read_mixer(r: _Reader, kind: str, m: dict, w: str) -> dict:
    if kind == "hgrn2":
        return dict(heads=r.positive_int(m, "heads", w), dim=r.positive_int(m, "dim", w),
                    vdim=r.positive_int(m, "vdim", w))
    left, right = m.get("left"), m.get("right")
    lw, rw = w + "left.", w + "right."
    out_l = dict(heads=r.positive_int(left, "heads", lw), kv_heads=r.positive_int(left, "kv_heads", lw),
                 dim=r.positive_int(left, "dim", lw), vdim=r.positive_int(left, "vdim", lw),
                 scale=r.positive(left, "scale", lw), block=None)
    if out_l["heads"] and out_l["kv_heads"] and out_l["heads"] % out_l["kv_heads"]:
        r.bad.append(f"{lw}heads={out_l['heads']} is no multiple of kv_heads={out_l['kv_heads']}")
    mask = left.get("mask") if isinstance(left, dict) else None
    if mask is not None:
        out_l["block"] = r.positive_int(mask, "size", lw + "mask.") or None
    out_r = dict(heads=r.positive_int(right, "heads", rw), dim=r.positive_int(right, "dim", rw),
                 vdim=r.positive_int(right, "vdim", rw), decay=[], rot=None)
    decay = right.get("decay") if isinstance(right, dict) else None
    if decay is None:
        r.missing.append(rw + "decay")
    elif (not isinstance(decay, list) or len(decay) != out_r["heads"]
          or not all(_is_num(d) and 0 <= d <= 1 for d in decay)):
        r.bad.append(f"{rw}decay={decay!r} (want one number in [0, 1] per head)")
    else:
        out_r["decay"] = [float(d) for d in decay]
    rot = right.get("rot") if isinstance(right, dict) else None
    if rot is not None:
        out_r["rot"] = dict(dims=r.positive_int(rot, "dims", rw + "rot."), base=r.positive(rot, "base", rw + "rot."))
        dims = out_r["rot"]["dims"]
        if dims and (dims % 2 or (out_r["dim"] and dims > out_r["dim"])):
            r.bad.append(f"{rw}rot.dims={dims} (want an even number, at most dim={out_r['dim']})")
    return dict(left=out_l, right=out_r)


def _read_mlp(r: _Reader, mlp, where: str):
    if mlp is None:
        return None
    kind = mlp.get("kind") if isinstance(mlp, dict) else None
    if kind != "moe":
        r.bad.append(f"{where}mlp.kind={kind!r} (want 'moe')")
        return None
    e, ro = mlp.get("expert"), mlp.get("router")
    out = dict(ff=r.positive_int(e, "ff", where + "mlp.expert."), limit=r.positive(e, "limit", where + "mlp.expert."),
               experts=r.positive_int(ro, "experts", where + "mlp.router."),
               top=r.positive_int(ro, "top", where + "mlp.router."), shared=None)
    if out["experts"] and out["top"] > out["experts"]:
        r.bad.append(f"{where}mlp.router.top={out['top']} exceeds experts={out['experts']}")
    sh = mlp.get("shared")
    if sh is not None:
        out["shared"] = dict(ff=r.positive_int(sh, "ff", where + "mlp.shared."),
                             limit=r.positive(sh, "limit", where + "mlp.shared."))
    return out


def read_toderax_config(cfg: dict) -> ToderaxConfig:
    r = _Reader()
    vocab, width = r.positive_int(cfg, "vocab", ""), r.positive_int(cfg, "width", "")
    norm = cfg.get("norm")
    eps = r.positive(norm, "eps", "norm.")
    groups = 1
    if isinstance(norm, dict) and norm.get("groups") is not None:
        groups = r.positive_int(norm, "groups", "norm.")
        if groups and width and width % groups:
            r.bad.append(f"norm.groups={groups} does not divide width={width}")
    streams = None
    if cfg.get("streams") is not None:
        streams = r.positive_int(cfg, "streams", "")
        if streams > MAX_STREAMS:
            r.bad.append(f"streams={streams} (at most {MAX_STREAMS})")
    scale = 1.0
    if isinstance(cfg.get("embedding"), dict) and cfg["embedding"].get("scale") is not None:
        scale = r.positive(cfg["embedding"], "scale", "embedding.")
    raw_layers = cfg.get("layers")
    layers = []
    if not isinstance(raw_layers, list) or not raw_layers:
        r.missing.append("layers")
        raw_layers = []
    for i, layer in enumerate(raw_layers):
        where = f"layers[{i}]."
        kind = layer.get("type") if isinstance(layer, dict) else None
        if kind not in LAYER_TYPES:
            r.bad.append(f"{where}type={kind!r} (want one of {LAYER_TYPES})")
            continue
        m = layer.get("mixer")
        if not isinstance(m, dict):
            r.missing.append(where + "mixer")
            continue
        layers.append(ToderaxLayer(kind, _read_mixer(r, kind, m, where + "mixer."),
                                   _read_mlp(r, layer.get("mlp"), where)))
    if r.missing or r.bad:
        parts = []
        if r.missing:
            parts.append("missing keys: " + ", ".join(r.missing))
        if r.bad:
            parts.append("unusable values: " + "; ".join(r.bad))
        raise ConfigError(f"unsupported {ARCHITECTURE} configuration: " + " | ".join(parts))
    return ToderaxConfig(ARCHITECTURE, vocab, width, streams, scale, eps, groups, tuple(layers))
