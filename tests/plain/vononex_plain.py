"""A plain, slow implementation of the Vononex decoder on the CPU in 64-bit, one function per mechanism,
written from the design's equations; it shares no code with the engine.  Weights come as a dict of
tensors by their checkpoint names, the configuration as the dict that config.json holds.

    rms(y)            = y / sqrt(mean(y^2) + eps)
    layer             : x <- rms(alpha x + mixer(x)) * w1 ;  x <- rms(alpha x + ff(x)) * w2 (when it has a feed-forward)
    logits            = head (rms(x) * w_final)
"""
from __future__ import annotations

import math

import torch

DT = torch.float64


def rms(y, eps, w=None):
    out = y / torch.sqrt((y * y).mean(-1, keepdim=True) + eps)
    return out if w is None else out * w


def turn(x, pos, dims, base, back=False):
    """x [T, heads, d]: over the first `dims` dims, dim i is paired with dim i + dims/2 and the pair turned by
    pos * base^(-2i/dims) (by minus that with back=True)."""
    if dims == 0:
        return x
    half = dims // 2
    freq = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=DT)
    ang = pos.to(DT)[:, None] * freq[None, :] * (-1.0 if back else 1.0)
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


def linear(h, w, name, bias=True):
    y = h @ w[name].to(DT).T
    if bias and name + ".b" in w:
        y = y + w[name + ".b"].to(DT)
    return y


def gelu_tanh(z):
    return 0.5 * z * (1 + torch.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z / (1 + torch.exp(-z))


def softmax_attention(h, w, p, m, eps):
    """The left mixer: causal softmax attention with whole-projection q/k norm, rotation, a temperature
    per head and rotated values."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    q = rms(linear(h, w, p + ".q"), eps, w[p + ".q.norm"].to(DT)).view(T, H, d)
    k = rms(linear(h, w, p + ".k"), eps, w[p + ".k.norm"].to(DT)).view(T, G, d)
    v = linear(h, w, p + ".v").view(T, G, dv)
    q = turn(q, pos, m["rot"]["dims"], m["rot"]["base"])
    k = turn(k, pos, m["rot"]["dims"], m["rot"]["base"])
    v = turn(v, pos, dv, m["rot"]["base"])
    out = torch.zeros(T, H, dv, dtype=DT)
    temp = w[p + ".temp"].to(DT)
    for hd in range(H):
        g = hd // (H // G)
        s = (q[:, hd] @ k[:, g].T) * m["scale"] * temp[hd]
        s = s.masked_fill(torch.ones(T, T, dtype=torch.bool).triu(1), float("-inf"))
        out[:, hd] = torch.softmax(s, -1) @ v[:, g]
    out = turn(out, pos, dv, m["rot"]["base"], back=True)
    return linear(out.reshape(T, H * dv), w, p + ".o")


def retention(h, w, p, m, eps):
    """The right mixer: S_t = decay S_(t-1) + k_t v_t^T, o_t = S_t^T q_t per head, token by token."""
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    q = turn(linear(h, w, p + ".q", False).view(T, H, d), pos, m["rot"]["dims"], m["rot"]["base"])
    k = turn(linear(h, w, p + ".k", False).view(T, H, d), pos, m["rot"]["dims"], m["rot"]["base"]) * d ** -0.5
    v = linear(h, w, p + ".v", False).view(T, H, dv)
    o = torch.zeros(T, H, dv, dtype=DT)
    for hd in range(H):
        S = torch.zeros(d, dv, dtype=DT)
        for t in range(T):
            S = m["decay"][hd] * S + torch.outer(k[t, hd], v[t, hd])
            o[t, hd] = S.T @ q[t, hd]
    o = rms(o, eps).reshape(T, H * dv)
    return linear(o * silu(linear(h, w, p + ".g", False)), w, p + ".o", False)


def mingru(h, w, p, m):
    T = h.shape[0]
    z = torch.sigmoid(linear(h, w, p + ".z"))
    u = linear(h, w, p + ".x")
    cand = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
    S = torch.zeros(m["width"], dtype=DT)
    states = []
    for t in range(T):
        S = (1 - z[t]) * S + z[t] * cand[t]
        states.append(S)
    return linear(torch.stack(states) * silu(linear(h, w, p + ".g", False)), w, p + ".o", False)


def feed_forward(h, w, p):
    return linear(gelu_tanh(linear(h, w, p + ".gate")) * linear(h, w, p + ".up"), w, p + ".down")


def forward_logits(ids, w, cfg, hidden=None):
    """[T, vocab] logits of every position in 64-bit; `hidden`, a list, receives the stream after every layer."""
    eps, alpha = cfg["norm"]["eps"], cfg["postln_alpha"]
    x = w["embed"].to(DT)[torch.tensor(list(ids))]
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}", layer["mixer"]
        if layer["type"] == "parallel":
            y = (m["left_scale"] * softmax_attention(x, w, p + ".mix.left", m["left"], eps)
                 + m["right_scale"] * retention(x, w, p + ".mix.right", m["right"], eps))
        else:
            y = mingru(x, w, p + ".mix", m)
        x = rms(alpha * x + y, eps, w[p + ".norm1"].to(DT))
        if layer.get("mlp") is not None:
            x = rms(alpha * x + feed_forward(x, w, p + ".mlp"), eps, w[p + ".norm2"].to(DT))
        if hidden is not None:
            hidden.append(x.clone())
    return rms(x, eps, w["final.norm"].to(DT)) @ w["head"].to(DT).T
