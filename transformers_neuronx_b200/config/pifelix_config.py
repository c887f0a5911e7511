"""Typed configuration of the Pifelix decoder, read from the keys of its own config.json.

    {"architecture": "Pifelix", "vocab": V, "width": W, "residual_mult": m, "embedding": {"scale": s},
     "norm": {"eps": e},
     "layers": [{"type": "attention", "mixer": {...}, "mlp": {"kind": "moe", ...} | null}, ...]}

An 'attention' layer's mixer holds heads, kv_heads, dim (queries and keys), vdim (values), scale, conv (taps of the
short convolution on the projections; absent or 0: none), mask {size} (chunked; absent: plain causal), rot {dims, base,
scaling {factor, original, fast, slow} (optional)} (absent: no rotation) and optionally kv_from: the index of an
earlier layer whose keys and values it reads instead of projecting its own.  A 'moe' feed-forward holds
router {experts, top} and expert {ff, limit}.  Every layer carries its own sizes, so layers of one model may differ.
Nothing has a default but `init_std` (the spread of random weights, used only when a folder is written from a seed)
and `max_positions` (the longest request the engine admits; the design itself has no limit).
"""
from __future__ import annotations

import copy
import json
import os
from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .model_config import ConfigError

LAYER_TYPES = ("attention",)


def _pos_int(d, key, where):
    v = d.get(key)
    if not isinstance(v, int) or isinstance(v, bool) or v <= 0:
        raise ConfigError(f"{where}: key {key!r} must be a positive integer, got {v!r}")
    return v


def _number(d, key, where):
    v = d.get(key)
    if not isinstance(v, (int, float)) or isinstance(v, bool):
        raise ConfigError(f"{where}: key {key!r} must be a number, got {v!r}")
    return float(v)


def _check_rot(m, where):
    r = m.get("rot")
    if r is None:
        return
    if not isinstance(r, dict):
        raise ConfigError(f"{where}: key 'rot' must hold 'dims' and 'base'")
    dims = r.get("dims")
    if not isinstance(dims, int) or isinstance(dims, bool) or dims < 0 or dims % 2 or dims > m["dim"]:
        raise ConfigError(f"{where}: rot.dims must be even and at most the head size {m['dim']}, got {dims!r}")
    if _number(r, "base", where + ".rot") <= 1:
        raise ConfigError(f"{where}: rot.base must be larger than 1")
    s = r.get("scaling")
    if s is not None:
        if not isinstance(s, dict):
            raise ConfigError(f"{where}.rot: key 'scaling' must hold factor, original, fast and slow")
        for k in ("factor", "original", "fast", "slow"):
            if _number(s, k, where + ".rot.scaling") <= 0:
                raise ConfigError(f"{where}.rot.scaling: {k} must be positive")


def _check_layer(i: int, layer: Dict[str, Any], layers) -> None:
    where = f"layers[{i}]"
    if not isinstance(layer, dict) or layer.get("type") not in LAYER_TYPES:
        t = layer.get("type") if isinstance(layer, dict) else layer
        raise ConfigError(f"{where}: unknown layer type {t!r}; known: {', '.join(LAYER_TYPES)}")
    m = layer.get("mixer")
    if not isinstance(m, dict):
        raise ConfigError(f"{where}: key 'mixer' must hold the mixer's sizes")
    mw = where + ".mixer"
    for k in ("heads", "kv_heads", "dim", "vdim"):
        _pos_int(m, k, mw)
    if m["heads"] % m["kv_heads"]:
        raise ConfigError(f"{mw}: {m['heads']} heads cannot share {m['kv_heads']} key/value heads")
    if _number(m, "scale", mw) <= 0:
        raise ConfigError(f"{mw}: scale must be positive")
    conv = m.get("conv", 0)
    if conv is not None and (not isinstance(conv, int) or isinstance(conv, bool) or conv < 0):
        raise ConfigError(f"{mw}: conv must be a number of taps, got {conv!r}")
    mask = m.get("mask")
    if mask is not None:
        if not isinstance(mask, dict):
            raise ConfigError(f"{mw}: key 'mask' must hold 'size'")
        _pos_int(mask, "size", mw + ".mask")
    _check_rot(m, mw)
    src = m.get("kv_from")
    if src is not None:
        if not isinstance(src, int) or isinstance(src, bool) or not (0 <= src < i):
            raise ConfigError(f"{mw}: kv_from must name an earlier layer, got {src!r}")
        o = layers[src]["mixer"]
        if "kv_from" in o and o["kv_from"] is not None:
            raise ConfigError(f"{mw}: kv_from names layer {src}, which has no keys and values of its own")
        for k in ("heads", "kv_heads", "dim", "vdim"):
            if o.get(k) != m[k]:
                raise ConfigError(f"{mw}: {k} differs from that of layer {src}, whose keys and values it reads")
        if o.get("rot") != m.get("rot"):
            raise ConfigError(f"{mw}: the rotation differs from that of layer {src}, whose keys it reads")
    mlp = layer.get("mlp")
    if mlp is not None:
        fw = where + ".mlp"
        if not isinstance(mlp, dict) or mlp.get("kind") != "moe":
            raise ConfigError(f"{fw}: kind must be 'moe' (or the layer's mlp null), got {mlp!r}")
        r, e = mlp.get("router"), mlp.get("expert")
        if not isinstance(r, dict) or not isinstance(e, dict):
            raise ConfigError(f"{fw}: keys 'router' and 'expert' must hold the experts' numbers and sizes")
        _pos_int(r, "experts", fw + ".router")
        _pos_int(r, "top", fw + ".router")
        if r["top"] > r["experts"]:
            raise ConfigError(f"{fw}.router: top {r['top']} exceeds the {r['experts']} experts")
        _pos_int(e, "ff", fw + ".expert")
        if _number(e, "limit", fw + ".expert") <= 0:
            raise ConfigError(f"{fw}.expert: limit must be positive")


@dataclass(frozen=True, eq=False)
class PifelixConfig:
    vocab: int
    width: int
    layers: Tuple[Dict[str, Any], ...]
    norm_eps: float
    residual_mult: float
    embedding_scale: float
    init_std: float = 0.05
    max_positions: int = 1 << 20
    architecture: str = "Pifelix"

    def __post_init__(self):
        for name in ("vocab", "width", "max_positions"):
            v = getattr(self, name)
            if not isinstance(v, int) or isinstance(v, bool) or v <= 0:
                raise ConfigError(f"config key {name!r} must be a positive integer, got {v!r}")
        if not (self.norm_eps > 0):
            raise ConfigError(f"norm.eps must be positive, got {self.norm_eps!r}")
        if not self.layers:
            raise ConfigError("config key 'layers' must list at least one layer")
        for i, layer in enumerate(self.layers):
            _check_layer(i, layer, self.layers)

    def __eq__(self, other):
        return isinstance(other, PifelixConfig) and self.to_dict() == other.to_dict()

    # what the engine's front door asks of any configuration
    @property
    def vocab_size(self) -> int:
        return self.vocab

    torch_dtype = "bfloat16"                 # the type the design's checkpoints are stored in

    @property
    def max_position_embeddings(self) -> int:
        return self.max_positions

    eos_token_id: Optional[int] = None
    bos_token_id: Optional[int] = None
    pad_token_id: Optional[int] = None

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "PifelixConfig":
        missing = [k for k in ("vocab", "width", "layers", "norm", "residual_mult", "embedding") if k not in d]
        if missing:
            raise ConfigError("config.json lacks required key(s): " + ", ".join(missing))
        if not isinstance(d["norm"], dict) or "eps" not in d["norm"]:
            raise ConfigError("config key 'norm' must hold 'eps'")
        if not isinstance(d["embedding"], dict):
            raise ConfigError("config key 'embedding' must hold 'scale'")
        if not isinstance(d["layers"], list):
            raise ConfigError("config key 'layers' must be a list")
        kw = dict(vocab=d["vocab"], width=d["width"], layers=tuple(copy.deepcopy(l) for l in d["layers"]),
                  norm_eps=float(d["norm"]["eps"]), residual_mult=_number(d, "residual_mult", "config"),
                  embedding_scale=_number(d["embedding"], "scale", "config.embedding"))
        for k in ("init_std", "max_positions"):
            if k in d:
                kw[k] = d[k]
        return cls(**kw)

    @classmethod
    def from_json(cls, path: str) -> "PifelixConfig":
        with open(path) as fp:
            return cls.from_dict(json.load(fp))

    @classmethod
    def from_pretrained(cls, folder: str) -> "PifelixConfig":
        return cls.from_json(os.path.join(folder, "config.json"))

    def to_dict(self) -> Dict[str, Any]:
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                "residual_mult": self.residual_mult, "embedding": {"scale": self.embedding_scale},
                "norm": {"eps": self.norm_eps}, "layers": [copy.deepcopy(l) for l in self.layers],
                "init_std": self.init_std, "max_positions": self.max_positions}

    def save(self, folder: str) -> None:
        os.makedirs(folder, exist_ok=True)
        with open(os.path.join(folder, "config.json"), "w") as fp:
            json.dump(self.to_dict(), fp, indent=1)
