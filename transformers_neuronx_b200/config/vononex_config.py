"""Typed configuration of the Vononex decoder, read from the keys of its own config.json.

    {"architecture": "Vononex", "vocab": V, "width": W, "postln_alpha": a, "norm": {"eps": e},
     "layers": [{"type": "parallel" | "mingru", "mixer": {...}, "mlp": {"kind": "dense", "ff": F} | null}, ...]}

A 'parallel' layer's mixer holds "left" (softmax attention: heads, kv_heads, dim, vdim, scale, rot {dims, base}),
"right" (retention: heads, dim, vdim, decay [one per head], rot {dims, base}) and the two scales; a 'mingru'
layer's mixer holds "width".  Every layer carries its own sizes, so layers of one model may differ.  Nothing has
a default but `init_std` (the spread of random weights, used only when a folder is written from a seed) and
`max_positions` (the longest request the engine admits; the design itself has no limit).
"""
from __future__ import annotations

import copy
import json
import os
from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .model_config import ConfigError

LAYER_TYPES = ("parallel", "mingru")


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


def _rot(d, where, dim):
    r = d.get("rot")
    if not isinstance(r, dict):
        raise ConfigError(f"{where}: key 'rot' must hold 'dims' and 'base'")
    dims = r.get("dims")
    if not isinstance(dims, int) or dims < 0 or dims % 2 or dims > dim:
        raise ConfigError(f"{where}: rot.dims must be even and at most the head size {dim}, got {dims!r}")
    if _number(r, "base", where + ".rot") <= 0:
        raise ConfigError(f"{where}: rot.base must be positive")


def _check_layer(i: int, layer: Dict[str, Any]) -> None:
    where = f"layers[{i}]"
    t = layer.get("type")
    if t not in LAYER_TYPES:
        raise ConfigError(f"{where}: unknown layer type {t!r}; known: {', '.join(LAYER_TYPES)}")
    m = layer.get("mixer")
    if not isinstance(m, dict):
        raise ConfigError(f"{where}: key 'mixer' must hold the mixer's sizes")
    if t == "parallel":
        for side in ("left", "right"):
            if not isinstance(m.get(side), dict):
                raise ConfigError(f"{where}.mixer: key {side!r} is missing")
            _number(m, side + "_scale", where + ".mixer")
        l, r = m["left"], m["right"]
        for k in ("heads", "kv_heads", "dim", "vdim"):
            _pos_int(l, k, where + ".mixer.left")
        if l["heads"] % l["kv_heads"]:
            raise ConfigError(f"{where}.mixer.left: {l['heads']} heads cannot share {l['kv_heads']} key/value heads")
        if l["vdim"] % 2:
            raise ConfigError(f"{where}.mixer.left: vdim must be even (values are rotated in pairs)")
        _number(l, "scale", where + ".mixer.left")
        _rot(l, where + ".mixer.left", l["dim"])
        for k in ("heads", "dim", "vdim"):
            _pos_int(r, k, where + ".mixer.right")
        dec = r.get("decay")
        if not isinstance(dec, list) or len(dec) != r["heads"] or not all(isinstance(x, (int, float)) for x in dec):
            raise ConfigError(f"{where}.mixer.right: 'decay' must list one number per head")
        _rot(r, where + ".mixer.right", r["dim"])
    else:
        _pos_int(m, "width", where + ".mixer")
    mlp = layer.get("mlp")
    if mlp is not None:
        if not isinstance(mlp, dict) or mlp.get("kind") != "dense":
            raise ConfigError(f"{where}.mlp: kind must be 'dense' (or the layer's mlp null), got {mlp!r}")
        _pos_int(mlp, "ff", where + ".mlp")


@dataclass(frozen=True, eq=False)
class VononexConfig:
    vocab: int
    width: int
    layers: Tuple[Dict[str, Any], ...]
    norm_eps: float
    postln_alpha: float
    init_std: float = 0.05
    max_positions: int = 1 << 20
    architecture: str = "Vononex"

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
            _check_layer(i, layer)

    def __eq__(self, other):
        return isinstance(other, VononexConfig) and self.to_dict() == other.to_dict()

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
    def from_dict(cls, d: Dict[str, Any]) -> "VononexConfig":
        missing = [k for k in ("vocab", "width", "layers", "norm", "postln_alpha") if k not in d]
        if missing:
            raise ConfigError("config.json lacks required key(s): " + ", ".join(missing))
        if not isinstance(d["norm"], dict) or "eps" not in d["norm"]:
            raise ConfigError("config key 'norm' must hold 'eps'")
        if not isinstance(d["layers"], list):
            raise ConfigError("config key 'layers' must be a list")
        kw = dict(vocab=d["vocab"], width=d["width"], layers=tuple(copy.deepcopy(l) for l in d["layers"]),
                  norm_eps=float(d["norm"]["eps"]), postln_alpha=_number(d, "postln_alpha", "config"))
        for k in ("init_std", "max_positions"):
            if k in d:
                kw[k] = d[k]
        return cls(**kw)

    @classmethod
    def from_json(cls, path: str) -> "VononexConfig":
        with open(path) as fp:
            return cls.from_dict(json.load(fp))

    @classmethod
    def from_pretrained(cls, folder: str) -> "VononexConfig":
        return cls.from_json(os.path.join(folder, "config.json"))

    def to_dict(self) -> Dict[str, Any]:
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                "postln_alpha": self.postln_alpha, "norm": {"eps": self.norm_eps},
                "layers": [copy.deepcopy(l) for l in self.layers], "init_std": self.init_std,
                "max_positions": self.max_positions}

    def save(self, folder: str) -> None:
        os.makedirs(folder, exist_ok=True)
        with open(os.path.join(folder, "config.json"), "w") as fp:
            json.dump(self.to_dict(), fp, indent=1)
