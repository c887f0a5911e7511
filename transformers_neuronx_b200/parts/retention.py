"""Retention: linear attention with a fixed decay per head, no softmax and no denominator.

  q = W_q h, k = W_k h (heads x k_dim), v = W_v h (heads x v_dim), gate = W_g h
  q, k rotated by position on the first rotary.dims dims of each head; k then multiplied by k_scale
  per head:  S_t = decay_h S_(t-1) + k_t v_t^T,   o_t = S_t^T q_t
  each head's o divided by its root mean square (no weight), heads concatenated, times silu(gate), output projection

The state S (heads x k_dim x v_dim numbers per request) is state of fixed size in 32-bit: it lives in the
request's slot, starts at zero when a request takes the slot, and is carried from step to step.  What enters
the recurrence is 32-bit: the rotation is applied in 32-bit to the projection's output and not rounded again.
A step's tokens of one request are walked in order by one kernel, portions of prompts and single decoded
tokens alike, so the state after a token does not depend on how the prompt was cut.
"""
from __future__ import annotations

import torch

from ..cache.manager import FixedStateNeed
from ..kernels import ops
from .fusable import FusableMixer
from .linear import Linear
from .registry import register_mixer
from .rotary import inverse_frequencies
from .spec import RetentionSpec


class Retention(FusableMixer):
    extra_libraries = ("retention",)

    def __init__(self, spec: RetentionSpec):
        s = self.spec = spec
        if len(s.decay) != s.n_heads:
            raise ValueError(f"{len(s.decay)} decays for {s.n_heads} heads")
        if s.k_dim > 256:
            raise ValueError(f"key size {s.k_dim} is not supported: the scan keeps up to 256 rows of a column in a warp")
        if s.rotary is not None and (s.rotary.dims > s.k_dim or s.rotary.dims % 2):
            raise ValueError(f"{s.rotary.dims} rotated dims do not fit heads of {s.k_dim}")
        self.inputs = [Linear(s.q), Linear(s.k), Linear(s.v)] + ([Linear(s.gate)] if s.gate is not None else [])
        self.output = Linear(s.out)
        self.decay = self.inv_freq = None

    @property
    def inner_width(self):
        return self.spec.n_heads * self.spec.v_dim

    def load_extras(self, tensors, device, act_dtype):
        s = self.spec
        self.decay = torch.tensor([float(d) for d in s.decay], dtype=torch.float64).to(torch.float32).to(device)
        if s.rotary is not None and s.rotary.dims:
            self.inv_freq = inverse_frequencies(s.rotary.dims, s.rotary.base, device)

    def cache_need(self):
        s = self.spec
        return FixedStateNeed((s.n_heads, s.v_dim, s.k_dim), "float32")     # a column's rows side by side

    def mix(self, ctx, proj, col0, inner_out, out_scale, sub=None):
        s, N = self.spec, proj.shape[0]
        H, dk, dv = s.n_heads, s.k_dim, s.v_dim
        rot = s.rotary.dims if s.rotary is not None else 0
        v0 = col0 + 2 * H * dk
        # a step of single tokens: one kernel does the rotation, the state's update, the output and its norm
        if ctx.decode_only and ops.retention_decode(
                proj, col0, col0 + H * dk, v0, v0 + H * dv if s.gate is not None else None, ctx.positions, self.inv_freq,
                rot, s.k_scale, self.decay, ctx.cache(sub), ctx.q_start, ctx.q_len, ctx.state_slots, s.norm_eps, out_scale,
                inner_out, H, dk, dv):
            return
        qr = ctx.scratch(N, H * dk, torch.float32)
        kr = ctx.scratch(N, H * dk, torch.float32)
        ops.retention_prep(proj, col0, col0 + H * dk, ctx.token_request, ctx.positions, self.inv_freq,
                           s.rotary.dims if s.rotary is not None else 0, s.k_scale, qr, kr, H, dk)
        v0 = col0 + 2 * H * dk
        v = proj[:, v0:v0 + H * dv]
        gate = proj[:, v0 + H * dv:v0 + 2 * H * dv] if s.gate is not None else None
        o = ctx.scratch(N, H * dv, torch.float32)
        ops.retention_scan(qr, kr, v, self.decay, ctx.cache(sub), ctx.q_start, ctx.q_len, ctx.state_slots, o, H, dk, dv,
                           most_tokens=1 if ctx.decode_only else N)
        ops.headwise_gated_rms_norm(o, gate, ctx.token_request, None, s.norm_eps, out_scale, inner_out, H, dv)


register_mixer("retention", Retention)
