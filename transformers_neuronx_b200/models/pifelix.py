"""The Pifelix architecture as data: its configuration -> a ModelSpec naming parts, sizes, constants and tensors.

A decoder whose layers are listed one by one in the configuration.  The embedding's rows are multiplied by a
constant.  In every layer the norm sits on the sublayer's OUTPUT only and the sublayers read the stream itself:
x <- x + m * norm1(mixer(x)), then x <- x + m * norm2(ff(x)), with RMS norms and m = residual_mult.  The mixer is
softmax attention with grouped key/value heads whose projections (with biases) pass through a short causal
convolution over time, then a per-head RMS norm of queries and keys, then a rotation of interleaved pairs with
stretched frequencies; the mask is chunked (a query reads the keys of its own block of positions).  A layer may read
the keys and values of an earlier layer instead of projecting its own (`kv_from`).  The feed-forward is a mixture of
experts: sigmoid scores, the largest `top` choose, the score multiplies the expert's input; an expert is
down(g * sigmoid(1.702 g) * (u + 1)) with g and u clamped.  The head is a matrix of its own behind a final RMS norm.

Tensor names: 'embed', 'final.norm', 'head', and for layer i the prefix 'l<i>.': 'norm1', 'norm2',
'mix.q|k|v|o' (bias: + '.b'; convolution: + '.conv'; per-head norm: + '.norm'), 'mlp.router', 'mlp.e<j>.gate|up|down'.
"""
from __future__ import annotations

from ..config.pifelix_config import PifelixConfig
from ..config.registry import Architecture, register_architecture
from ..parts.spec import (ConvAttentionSpec, EmbeddingSpec, ExpertSpec, FrequencyRampSpec, HeadSpec, LayerSpec, LinearSpec,
                          ModelSpec, NormSpec, RotarySpec, RoutedFeedForwardSpec, ScheduleEntry)

EXPERT_ACT_ALPHA = 1.702       # y = g * sigmoid(1.702 g) * (u + 1)
EXPERT_UP_SHIFT = 1.0


def _lin(name: str, n_in: int, n_out: int, bias: bool) -> LinearSpec:
    return LinearSpec(n_in, n_out, name, name + ".b" if bias else None)


def _mask(m: dict):
    return m["mask"]["size"] if m.get("mask") is not None else None


def _attention(p: str, W: int, m: dict, eps: float, keep_all_pages: bool) -> ConvAttentionSpec:
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    taps = int(m.get("conv") or 0)
    own = m.get("kv_from") is None
    rot = None
    if m.get("rot") is not None and m["rot"]["dims"]:
        r = m["rot"]
        s = r.get("scaling")
        rot = RotarySpec(r["dims"], float(r["base"]), interleaved=True,
                         scaling=None if s is None else FrequencyRampSpec(float(s["factor"]), float(s["original"]),
                                                                          float(s["fast"]), float(s["slow"])))
    return ConvAttentionSpec(
        kind="conv_attention", hidden=W, n_heads=H, n_kv_heads=G, k_dim=d, v_dim=dv, scale=float(m["scale"]),
        q=_lin(p + ".q", W, H * d, True), k=_lin(p + ".k", W, G * d, True) if own else None,
        v=_lin(p + ".v", W, G * dv, True) if own else None, out=_lin(p + ".o", H * dv, W, False),
        conv_taps=taps, q_conv=p + ".q.conv" if taps else None, k_conv=p + ".k.conv" if taps and own else None,
        v_conv=p + ".v.conv" if taps and own else None, q_norm=p + ".q.norm", k_norm=p + ".k.norm" if own else None,
        norm_eps=eps, rotary=rot, chunk=_mask(m), kv_source=None if own else int(m["kv_from"]),
        keep_all_pages=keep_all_pages)


def _experts(p: str, W: int, mlp: dict) -> RoutedFeedForwardSpec:
    E, F = mlp["router"]["experts"], mlp["expert"]["ff"]
    lim = float(mlp["expert"]["limit"])
    return RoutedFeedForwardSpec(
        kind="routed_experts", hidden=W, ff=F, n_experts=E, top=mlp["router"]["top"], router=p + ".router",
        experts=tuple(ExpertSpec(f"{p}.e{j}.gate", f"{p}.e{j}.up", f"{p}.e{j}.down") for j in range(E)),
        scores="sigmoid", renormalize=False, weight_on_input=True, gate_limit=lim, up_limit=lim,
        act_alpha=EXPERT_ACT_ALPHA, up_shift=EXPERT_UP_SHIFT)


def build_spec(cfg: PifelixConfig) -> ModelSpec:
    W, eps = cfg.width, cfg.norm_eps
    # pages that another layer reads under another mask are not given back behind their own layer's mask
    lent_elsewhere = set()
    for layer in cfg.layers:
        m = layer["mixer"]
        if m.get("kv_from") is not None and _mask(m) != _mask(cfg.layers[m["kv_from"]]["mixer"]):
            lent_elsewhere.add(m["kv_from"])
    layers = []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}"
        ff = norm2 = None
        if layer.get("mlp") is not None:
            ff = _experts(p + ".mlp", W, layer["mlp"])
            norm2 = NormSpec("rms_norm", W, eps, weight=p + ".norm2")
        layers.append(LayerSpec(block="output_norm", norm1=NormSpec("rms_norm", W, eps, weight=p + ".norm1"),
                                mixer=_attention(p + ".mix", W, layer["mixer"], eps, i in lent_elsewhere), norm2=norm2,
                                feed_forward=ff, residual_scale=float(cfg.residual_mult)))
    return ModelSpec(hidden_size=W, vocab_size=cfg.vocab, max_positions=cfg.max_positions,
                     embedding=EmbeddingSpec(table="embed", vocab=cfg.vocab, dim=W, scale=float(cfg.embedding_scale)),
                     layers=tuple(layers), schedule=tuple(ScheduleEntry(i, i) for i in range(len(layers))),
                     head=HeadSpec(weight="head", vocab=cfg.vocab, dim=W,
                                   final_norm=NormSpec("rms_norm", W, eps, weight="final.norm")))


register_architecture(Architecture(name="Pifelix", model_type="pifelix", config_class=PifelixConfig,
                                   build_spec=build_spec))
