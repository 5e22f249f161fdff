"""Typed configuration of the Kuzupel design, read from its config.json.

    {"architecture": "Kuzupel", "vocab": V, "width": W, "residual_mult": m, "logit_softcap": c,
     "embedding": {"scale": s, "bigram": {"buckets": B, "mul_prev": a, "mul_cur": b}},
     "norm": {"eps": e}, "layers": [{"type": T, "mixer": {...}, "mlp": {...} | null}, ...]}

``type`` names the layer's mixer; ``mixer`` holds that mixer's sizes and constants:

* ``attention``:   heads, kv_heads, dim, vdim, scale, mask {size}
* ``attention_2``: heads, kv_heads, dim, vdim, scale, mask {size, keep_first}, conv (taps), rot {dims, base}

``mlp``: ``{"kind": "dense", "ff", "limit"}``, or ``{"kind": "moe", "expert": {"ff", "limit"}, "router":
{"experts", "top"}, "shared": {"ff", "limit"} | absent}``, or null.  What a file leaves out is off:
``residual_mult`` 1, no ``logit_softcap``, ``embedding.scale`` 1, no ``embedding.bigram`` (no pair table), no
``mask`` (plainly causal; ``keep_first`` 0), no ``conv``, no ``rot``, no ``shared``.  Every size and constant
comes from the file; what is missing or unusable is reported in one ConfigError that lists every key."""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any

from ..errors import ConfigError
from .beledra import _Reader

ARCHITECTURE = "Kuzupel"
LAYER_TYPES = ("attention", "attention_2")
MAX_CONV_TAPS = 16


@dataclass(frozen=True)
class KuzupelLayer:
    type: str
    mixer: dict          # heads, kv_heads, dim, vdim, scale, window, keep_first, conv, rot
    mlp: dict | None     # {"kind": "dense", "ff", "limit"} | {"kind": "moe", "ff", "limit", "experts", "top", "shared"}


@dataclass(frozen=True)
class KuzupelConfig:
    architecture: str
    vocab: int
    width: int
    residual_mult: float
    logit_softcap: float | None
    embedding_scale: float
    pair_table: dict | None      # {"buckets", "mul_prev", "mul_cur"}
    norm_eps: float
    layers: tuple

    def to_json_dict(self) -> dict[str, Any]:
        """config.json content that reads back to this configuration."""
        emb: dict = {"scale": self.embedding_scale}
        if self.pair_table is not None:
            emb["bigram"] = dict(self.pair_table)
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
               "residual_mult": self.residual_mult, "embedding": emb, "norm": {"eps": self.norm_eps},
               "layers": [{"type": l.type, "mixer": _mixer_json(l), "mlp": _mlp_json(l.mlp)} for l in self.layers]}
        if self.logit_softcap is not None:
            out["logit_softcap"] = self.logit_softcap
        return out


def _mixer_json(layer: KuzupelLayer) -> dict:
    m = copy.deepcopy(layer.mixer)
    window, keep = m.pop("window"), m.pop("keep_first")
    if window is not None:
        m["mask"] = {"size": window}
        if keep:
            m["mask"]["keep_first"] = keep
    for k in ("conv", "rot"):
        if m.get(k) is None:
            m.pop(k, None)
    return m


def _mlp_json(mlp):
    if mlp is None:
        return None
    if mlp["kind"] == "dense":
        return {"kind": "dense", "ff": mlp["ff"], "limit": mlp["limit"]}
    out = {"kind": "moe", "expert": {"ff": mlp["ff"], "limit": mlp["limit"]},
           "router": {"experts": mlp["experts"], "top": mlp["top"]}}
    if mlp.get("shared") is not None:
        out["shared"] = dict(mlp["shared"])
    return out


def _read_mixer(r: _Reader, kind: str, m: dict, w: str) -> dict:
    out = dict(heads=r.positive_int(m, "heads", w), kv_heads=r.positive_int(m, "kv_heads", w),
               dim=r.positive_int(m, "dim", w), vdim=r.positive_int(m, "vdim", w),
               scale=r.positive(m, "scale", w), window=None, keep_first=0, conv=None, rot=None)
    if out["heads"] and out["kv_heads"] and out["heads"] % out["kv_heads"]:
        r.bad.append(f"{w}heads={out['heads']} is no multiple of kv_heads={out['kv_heads']}")
    mask = m.get("mask")
    if mask is not None:
        out["window"] = r.positive_int(mask, "size", w + "mask.") or None
        keep = mask.get("keep_first") if isinstance(mask, dict) else None
        if keep is not None:
            if isinstance(keep, bool) or not isinstance(keep, int) or keep < 0:
                r.bad.append(f"{w}mask.keep_first={keep!r} (want a count of positions)")
            else:
                out["keep_first"] = keep
    if kind == "attention_2":
        if m.get("conv") is not None:
            out["conv"] = r.positive_int(m, "conv", w)
            if out["conv"] > MAX_CONV_TAPS:
                r.bad.append(f"{w}conv={out['conv']} (at most {MAX_CONV_TAPS} taps)")
        rot = m.get("rot")
        if rot is not None:
            out["rot"] = dict(dims=r.positive_int(rot, "dims", w + "rot."), base=r.positive(rot, "base", w + "rot."))
            dims = out["rot"]["dims"]
            if dims and (dims % 2 or (out["dim"] and dims > out["dim"])):
                r.bad.append(f"{w}rot.dims={dims} (want an even number, at most dim={out['dim']})")
    return out


def _read_mlp(r: _Reader, mlp, where: str):
    if mlp is None:
        return None
    kind = mlp.get("kind") if isinstance(mlp, dict) else None
    w = where + "mlp."
    if kind == "dense":
        return dict(kind="dense", ff=r.positive_int(mlp, "ff", w), limit=r.positive(mlp, "limit", w))
    if kind != "moe":
        r.bad.append(f"{w}kind={kind!r} (want 'dense' or 'moe')")
        return None
    e, ro = mlp.get("expert"), mlp.get("router")
    out = dict(kind="moe", ff=r.positive_int(e, "ff", w + "expert."), limit=r.positive(e, "limit", w + "expert."),
               experts=r.positive_int(ro, "experts", w + "router."), top=r.positive_int(ro, "top", w + "router."),
               shared=None)
    if out["experts"] and out["top"] > out["experts"]:
        r.bad.append(f"{w}router.top={out['top']} exceeds experts={out['experts']}")
    sh = mlp.get("shared")
    if sh is not None:
        out["shared"] = dict(ff=r.positive_int(sh, "ff", w + "shared."), limit=r.positive(sh, "limit", w + "shared."))
    return out


def read_kuzupel_config(cfg: dict) -> KuzupelConfig:
    r = _Reader()
    vocab, width = r.positive_int(cfg, "vocab", ""), r.positive_int(cfg, "width", "")
    eps = r.positive(cfg.get("norm"), "eps", "norm.")
    mult = r.positive(cfg, "residual_mult", "") if cfg.get("residual_mult") is not None else 1.0
    cap = r.positive(cfg, "logit_softcap", "") if cfg.get("logit_softcap") is not None else None
    emb = cfg.get("embedding") if isinstance(cfg.get("embedding"), dict) else {}
    scale = r.positive(emb, "scale", "embedding.") if emb.get("scale") is not None else 1.0
    pair = None
    if emb.get("bigram") is not None:
        b = emb["bigram"]
        pair = dict(buckets=r.positive_int(b, "buckets", "embedding.bigram."))
        for k in ("mul_prev", "mul_cur"):
            v = b.get(k) if isinstance(b, dict) else None
            if isinstance(v, bool) or not isinstance(v, int) or v < 0:
                (r.missing if v is None else r.bad).append(f"embedding.bigram.{k}" + ("" if v is None else f"={v!r}"))
                v = 0
            pair[k] = v
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
        layers.append(KuzupelLayer(kind, _read_mixer(r, kind, m, where + "mixer."),
                                   _read_mlp(r, layer.get("mlp"), where)))
    if r.missing or r.bad:
        parts = []
        if r.missing:
            parts.append("missing keys: " + ", ".join(r.missing))
        if r.bad:
            parts.append("unusable values: " + "; ".join(r.bad))
        raise ConfigError(f"unsupported {ARCHITECTURE} configuration: " + " | ".join(parts))
    return KuzupelConfig(ARCHITECTURE, vocab, width, mult, cap, scale, pair, eps, tuple(layers))
