"""A plain, slow implementation of the Pifelix decoder in 64-bit: the oracle of the tests.

One function per mechanism, loops over tokens where a loop says it most directly, whole sequences only (no cache,
no state, no batches): the engine's answers under any cut of a request must equal these.  It shares no code with
the package.

  embedding      x_t = E[token_t] * s_emb
  layer          x <- x + m * rms(mixer(x)) * w1 ;  x <- x + m * rms(ff(x)) * w2        (the norm on the output only)
  mixer          q, k, v = projections with bias; each channel through `short_conv`; q, k: `rms` per head with one
                 shared weight; `turn_pairs` on the first rot.dims dims; `chunked_attention`; output projection.
                 A layer with kv_from reads the keys and values computed by that earlier layer.
  feed-forward   `routed_experts`
  head           rms(x) * w_final, then the output matrix
"""
import math

import torch

F64 = torch.float64


def rms(x, eps, w=None):
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if w is None else y * w


def short_conv(u, w):
    """u [T, C], w [C, taps]: y_t = sum_j w[:, j] u_(t - taps + 1 + j), with zeros before the first position."""
    T, taps = u.shape[0], w.shape[1]
    y = torch.zeros_like(u)
    for t in range(T):
        for j in range(taps):
            src = t - taps + 1 + j
            if src >= 0:
                y[t] += w[:, j] * u[src]
    return y


def pair_frequencies(dims, base, scaling=None):
    """Frequency of pair i = 0 .. dims/2 - 1, and what sines and cosines are multiplied by."""
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    if scaling is None:
        return f, 1.0
    def turns(t):
        return dims * math.log(scaling["original"] / (2 * math.pi * t)) / (2 * math.log(base))
    lo = max(math.floor(turns(scaling["fast"])), 0)
    hi = min(math.ceil(turns(scaling["slow"])), dims - 1)
    out = []
    for i, fi in enumerate(f):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(fi / scaling["factor"] * ramp + fi * (1 - ramp))
    return out, 0.1 * math.log(scaling["factor"]) + 1.0


def turn_pairs(x, positions, rot):
    """x [T, heads, d]: dims (2i, 2i + 1), i < rot.dims / 2, of every head turned by position * frequency_i."""
    if rot is None or not rot.get("dims"):
        return x
    f, mag = pair_frequencies(rot["dims"], float(rot["base"]), rot.get("scaling"))
    y = x.clone()
    for t, p in enumerate(positions):
        for i, fi in enumerate(f):
            c, s = math.cos(p * fi) * mag, math.sin(p * fi) * mag
            a, b = x[t, :, 2 * i], x[t, :, 2 * i + 1]
            y[t, :, 2 * i] = a * c - b * s
            y[t, :, 2 * i + 1] = b * c + a * s
    return y


def sees(i, j, chunk):
    return j <= i and (chunk is None or i // chunk == j // chunk)


def visibility(n_queries, n_keys, first_query, chunk):
    """[n_queries, n_keys] of booleans: query r sits at position first_query + r, key j at position j."""
    i = first_query + torch.arange(n_queries)[:, None]
    j = torch.arange(n_keys)[None, :]
    return (j <= i) if chunk is None else (j <= i) & (i // chunk == j // chunk)


def chunked_attention(q, k, v, scale, chunk, first_query=0):
    """q [Tq, H, d] at positions first_query.., k [Tk, G, d], v [Tk, G, dv] -> [Tq, H, dv]; query head h uses
    key/value head h // (H / G); ordinary softmax over the keys a query sees."""
    H, G = q.shape[1], k.shape[1]
    see = visibility(q.shape[0], k.shape[0], first_query, chunk)
    out = torch.zeros(q.shape[0], H, v.shape[2], dtype=F64)
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h].to(F64) @ k[:, g].to(F64).T) * scale
        s = s.masked_fill(~see, -math.inf)
        out[:, h] = torch.softmax(s, -1) @ v[:, g].to(F64)
    return out


def attention_mixer(h, t, p, m, eps, shared):
    """shared: {layer index: (keys, values)} of the layers that ran before; this layer adds its own."""
    T, H, G, d, dv = h.shape[0], m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    taps = m.get("conv") or 0
    pos = list(range(T))

    def projected(name, heads, width):
        u = h @ t[p + name].T + t[p + name + ".b"]
        if taps:
            u = short_conv(u, t[p + name + ".conv"])
        return u.view(T, heads, width)

    q = turn_pairs(rms(projected("q", H, d), eps, t[p + "q.norm"]), pos, m.get("rot"))
    if m.get("kv_from") is not None:
        k, v = shared[m["kv_from"]]
    else:
        k = turn_pairs(rms(projected("k", G, d), eps, t[p + "k.norm"]), pos, m.get("rot"))
        v = projected("v", G, dv)
    chunk = m["mask"]["size"] if m.get("mask") else None
    o = chunked_attention(q, k, v, float(m["scale"]), chunk)
    return o.reshape(T, H * dv) @ t[p + "o"].T, (k, v)


def routed_experts(h, t, p, mlp):
    E, top, lim = mlp["router"]["experts"], mlp["router"]["top"], float(mlp["expert"]["limit"])
    out = torch.zeros_like(h)
    for n in range(h.shape[0]):
        score = torch.sigmoid(t[p + "router"] @ h[n])
        order = sorted(range(E), key=lambda e: (-float(score[e]), e))[:top]
        for e in order:
            x = float(score[e]) * h[n]
            g = torch.clamp(t[f"{p}e{e}.gate"] @ x, max=lim)
            u = torch.clamp(t[f"{p}e{e}.up"] @ x, -lim, lim)
            out[n] += t[f"{p}e{e}.down"] @ (g * torch.sigmoid(1.702 * g) * (u + 1.0))
    return out


def forward_hidden(ids, tensors, cfg):
    """The residual stream after every layer, [layers, T, width], and the logits [T, vocab]."""
    t = {k: v.to(F64) for k, v in tensors.items()}
    eps, m_res = float(cfg["norm"]["eps"]), float(cfg["residual_mult"])
    x = t["embed"][list(ids)] * float(cfg["embedding"]["scale"])
    shared, after = {}, []
    for i, layer in enumerate(cfg["layers"]):
        y, kv = attention_mixer(x, t, f"l{i}.mix.", layer["mixer"], eps, shared)
        shared[i] = kv
        x = x + m_res * rms(y, eps, t[f"l{i}.norm1"])
        if layer.get("mlp") is not None:
            x = x + m_res * rms(routed_experts(x, t, f"l{i}.mlp.", layer["mlp"]), eps, t[f"l{i}.norm2"])
        after.append(x.clone())
    return torch.stack(after), rms(x, eps, t["final.norm"]) @ t["head"].T


def forward_logits(ids, tensors, cfg):
    return forward_hidden(ids, tensors, cfg)[1]
