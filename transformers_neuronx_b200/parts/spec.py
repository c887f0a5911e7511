"""Descriptions of a model as data: which parts, with which sizes and constants, in which order.

An architecture (models/opt.py) turns its typed configuration into a ``ModelSpec``.  Every part
is named by a ``kind`` that the registries of parts/registry.py resolve to a class, so a model may
use different mixers and feed-forwards in different layers, and a test may register a kind of its
own.  The order in which layers run is the ``schedule``: a list of (layer, cache) pairs that may
name a layer twice, or give two entries the same cache so that one layer reads what another wrote.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Optional, Tuple


@dataclass(frozen=True)
class LinearSpec:
    in_features: int
    out_features: int
    weight: str                      # tensor name, [out_features, in_features]
    bias: Optional[str] = None       # tensor name, [out_features]; None: no bias


@dataclass(frozen=True)
class NormSpec:
    kind: str                        # 'layer_norm' | 'rms_norm'
    size: int
    eps: float
    weight: Optional[str] = None     # None: no elementwise scale
    bias: Optional[str] = None
    weight_offset: float = 0.0       # 'rms_norm': the scale is weight + weight_offset (1.0: "one plus" weights)


@dataclass(frozen=True)
class RotarySpec:
    """Rotation of pairs of dims by position: over the first `dims` dims of a head, dim i is paired with
    dim i + dims/2 and turned by position * base^(-2i/dims)."""
    dims: int
    base: float


@dataclass(frozen=True)
class PositionSpec:
    kind: str                        # 'learned' | 'none' | a registered kind
    table: Optional[str] = None      # tensor name, [rows, dim]
    rows: int = 0
    dim: int = 0
    offset: int = 0                  # row = position + offset
    extra: Tuple = ()


@dataclass(frozen=True)
class AttentionSpec:
    kind: str                        # 'attention'
    hidden: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    scale: float
    q: LinearSpec = None
    k: LinearSpec = None
    v: LinearSpec = None
    out: LinearSpec = None
    window: Optional[int] = None     # None: every earlier position is read
    position: Optional[PositionSpec] = None   # an encoding applied to queries and keys, if any


@dataclass(frozen=True)
class RotaryAttentionSpec:
    """Softmax attention over the paged cache whose queries and keys may be normalised over the whole
    projection, are rotated by position, and whose score is multiplied by a number per head; the values
    may be rotated as well (and each head's output turned back by the query's position)."""
    kind: str                        # 'rotary_attention'
    hidden: int
    n_heads: int
    n_kv_heads: int
    k_dim: int                       # per-head size of queries and keys
    v_dim: int                       # per-head size of values
    scale: float
    q: LinearSpec = None
    k: LinearSpec = None
    v: LinearSpec = None
    out: LinearSpec = None
    rotary: Optional[RotarySpec] = None
    rotate_values: bool = False      # values turned by their position over all v_dim dims (base of `rotary`)
    q_norm: Optional[str] = None     # tensor [n_heads * k_dim]: RMS norm over the whole projection, before rotation
    k_norm: Optional[str] = None     # tensor [n_kv_heads * k_dim]
    norm_eps: float = 1e-6
    head_scale: Optional[str] = None  # tensor [n_heads]: the score of head h is multiplied by its entry
    window: Optional[int] = None


@dataclass(frozen=True)
class RetentionSpec:
    """Linear attention with a fixed decay per head: S <- decay S + k v^T, o = S^T q; each head's o divided by
    its root mean square, gated by silu of a projection, then the output projection."""
    kind: str                        # 'retention'
    hidden: int
    n_heads: int
    k_dim: int
    v_dim: int
    decay: Tuple[float, ...] = ()    # one per head
    q: LinearSpec = None
    k: LinearSpec = None
    v: LinearSpec = None
    gate: Optional[LinearSpec] = None
    out: LinearSpec = None
    rotary: Optional[RotarySpec] = None
    k_scale: float = 1.0             # keys are multiplied by it after rotation
    norm_eps: float = 1e-6


@dataclass(frozen=True)
class ParallelMixerSpec:
    """Several mixers side by side on the same input; the result is the sum of scale_i * branch_i."""
    kind: str                        # 'parallel'
    branches: Tuple[Any, ...] = ()
    scales: Tuple[float, ...] = ()


@dataclass(frozen=True)
class MinGRUSpec:
    """S <- (1 - z) S + z cand with gates that read the current token only; output W_o (S * silu(gate))."""
    kind: str                        # 'mingru'
    hidden: int
    width: int
    z: LinearSpec = None             # update gate (sigmoid)
    x: LinearSpec = None             # candidate
    gate: Optional[LinearSpec] = None
    out: LinearSpec = None


@dataclass(frozen=True)
class GatedFeedForwardSpec:
    kind: str                        # 'gated_dense'
    gate: LinearSpec = None
    up: LinearSpec = None
    down: LinearSpec = None
    activation: str = "silu"         # applied to the gate's product


@dataclass(frozen=True)
class DenseFeedForwardSpec:
    kind: str                        # 'dense'
    fc1: LinearSpec = None
    fc2: LinearSpec = None
    activation: str = "relu"


@dataclass(frozen=True)
class LayerSpec:
    block: str                       # 'pre_norm' | 'post_norm' | 'post_norm_scaled' | a registered kind
    norm1: Any = None
    mixer: Any = None
    norm2: Any = None
    feed_forward: Any = None         # None: the layer has no feed-forward (and no second norm)
    residual_scale: float = 1.0      # 'post_norm_scaled': x <- norm(residual_scale * x + sublayer(x))


@dataclass(frozen=True)
class EmbeddingSpec:
    table: str                       # tensor name, [vocab, dim]
    vocab: int = 0
    dim: int = 0
    project_in: Optional[LinearSpec] = None
    position: Optional[PositionSpec] = None   # an encoding added to the hidden state, if any


@dataclass(frozen=True)
class HeadSpec:
    weight: str                      # tensor name of the output matrix [vocab, dim]
    vocab: int = 0
    dim: int = 0
    tied_to: Optional[str] = None    # used when the file does not store `weight`
    final_norm: Optional[NormSpec] = None
    project_out: Optional[LinearSpec] = None


@dataclass(frozen=True)
class ScheduleEntry:
    layer: int                       # index into ModelSpec.layers
    cache: int                       # which cache its mixer uses; entries may share one


@dataclass(frozen=True)
class ModelSpec:
    hidden_size: int
    vocab_size: int
    max_positions: int
    embedding: EmbeddingSpec
    layers: Tuple[LayerSpec, ...]
    schedule: Tuple[ScheduleEntry, ...]
    head: HeadSpec
    eos_token_id: Optional[int] = None
    pad_token_id: Optional[int] = None
    bos_token_id: Optional[int] = None
