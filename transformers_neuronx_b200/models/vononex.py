"""The Vononex architecture as data: its configuration -> a ModelSpec naming parts, sizes, constants and tensors.

A decoder whose layers are listed one by one in the configuration.  Every layer is post-norm with a scaled
residual, x <- norm(alpha x + sublayer(x)) with RMS norms, and has one of two mixers:

  'parallel'  softmax attention (grouped key/value heads, queries and keys normalised over the whole projection
              and rotated, a temperature per head, values rotated by their position and the output turned
              back) beside retention (a decaying outer-product state per head, gated), summed with two scales;
  'mingru'    a gated recurrence over `width` channels;

and an optional gated feed-forward (tanh-form gelu on the gate).  No position table: positions enter through
the rotations only.  The head is a matrix of its own (not tied to the embedding) behind a final RMS norm.

Tensor names: 'embed', 'final.norm', 'head', and for layer i the prefix 'l<i>.': 'norm1', 'norm2', 'mix.*'
('mix.left.*' / 'mix.right.*' in a parallel layer), 'mlp.gate|up|down'; a bias is the matrix's name + '.b'.
"""
from __future__ import annotations

from ..config.registry import Architecture, register_architecture
from ..config.vononex_config import VononexConfig
from ..parts.spec import (EmbeddingSpec, GatedFeedForwardSpec, HeadSpec, LayerSpec, LinearSpec, MinGRUSpec, ModelSpec,
                          NormSpec, ParallelMixerSpec, RetentionSpec, RotaryAttentionSpec, RotarySpec, ScheduleEntry)

FF_ACTIVATION = "gelu_pytorch_tanh"      # 0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3)))


def _lin(name: str, n_in: int, n_out: int, bias: bool) -> LinearSpec:
    return LinearSpec(n_in, n_out, name, name + ".b" if bias else None)


def _attention(p: str, W: int, m: dict, eps: float) -> RotaryAttentionSpec:
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    return RotaryAttentionSpec(
        kind="rotary_attention", hidden=W, n_heads=H, n_kv_heads=G, k_dim=d, v_dim=dv, scale=float(m["scale"]),
        q=_lin(p + ".q", W, H * d, True), k=_lin(p + ".k", W, G * d, True), v=_lin(p + ".v", W, G * dv, True),
        out=_lin(p + ".o", H * dv, W, True), rotary=RotarySpec(m["rot"]["dims"], float(m["rot"]["base"])),
        rotate_values=True, q_norm=p + ".q.norm", k_norm=p + ".k.norm", norm_eps=eps, head_scale=p + ".temp")


def _retention(p: str, W: int, m: dict, eps: float) -> RetentionSpec:
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    return RetentionSpec(
        kind="retention", hidden=W, n_heads=H, k_dim=d, v_dim=dv, decay=tuple(float(x) for x in m["decay"]),
        q=_lin(p + ".q", W, H * d, False), k=_lin(p + ".k", W, H * d, False), v=_lin(p + ".v", W, H * dv, False),
        gate=_lin(p + ".g", W, H * dv, False), out=_lin(p + ".o", H * dv, W, False),
        rotary=RotarySpec(m["rot"]["dims"], float(m["rot"]["base"])), k_scale=float(d) ** -0.5, norm_eps=eps)


def build_spec(cfg: VononexConfig) -> ModelSpec:
    W, eps = cfg.width, cfg.norm_eps
    layers = []
    for i, layer in enumerate(cfg.layers):
        p, m = f"l{i}", layer["mixer"]
        if layer["type"] == "parallel":
            mixer = ParallelMixerSpec("parallel",
                                      branches=(_attention(p + ".mix.left", W, m["left"], eps),
                                                _retention(p + ".mix.right", W, m["right"], eps)),
                                      scales=(float(m["left_scale"]), float(m["right_scale"])))
        else:
            n = m["width"]
            mixer = MinGRUSpec("mingru", hidden=W, width=n, z=_lin(p + ".mix.z", W, n, True),
                               x=_lin(p + ".mix.x", W, n, True), gate=_lin(p + ".mix.g", W, n, False),
                               out=_lin(p + ".mix.o", n, W, False))
        ff = norm2 = None
        if layer.get("mlp") is not None:
            F = layer["mlp"]["ff"]
            ff = GatedFeedForwardSpec("gated_dense", gate=_lin(p + ".mlp.gate", W, F, True),
                                      up=_lin(p + ".mlp.up", W, F, True), down=_lin(p + ".mlp.down", F, W, True),
                                      activation=FF_ACTIVATION)
            norm2 = NormSpec("rms_norm", W, eps, weight=p + ".norm2")
        layers.append(LayerSpec(block="post_norm_scaled", norm1=NormSpec("rms_norm", W, eps, weight=p + ".norm1"),
                                mixer=mixer, norm2=norm2, feed_forward=ff, residual_scale=float(cfg.postln_alpha)))
    return ModelSpec(hidden_size=W, vocab_size=cfg.vocab, max_positions=cfg.max_positions,
                     embedding=EmbeddingSpec(table="embed", vocab=cfg.vocab, dim=W),
                     layers=tuple(layers), schedule=tuple(ScheduleEntry(i, i) for i in range(len(layers))),
                     head=HeadSpec(weight="head", vocab=cfg.vocab, dim=W,
                                   final_norm=NormSpec("rms_norm", W, eps, weight="final.norm")))


register_architecture(Architecture(name="Vononex", model_type="vononex", config_class=VononexConfig,
                                   build_spec=build_spec))
