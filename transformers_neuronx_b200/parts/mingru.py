"""minGRU: a gated recurrence whose gates read only the current token.

  z = sigmoid(W_z h + b_z),  u = W_x h + b_x,  cand = u + 1/2 where u >= 0, sigmoid(u) where u < 0
  S_t = (1 - z) S_(t-1) + z cand          (element by element over `width` channels)
  result = W_o (S_t * silu(W_g h))

The state (width numbers per request, 32-bit) lives in the request's slot and starts at zero.  Gates,
candidate and state are computed in 32-bit from the projections' output.
"""
from __future__ import annotations

from ..cache.manager import FixedStateNeed
from ..kernels import ops
from .fusable import FusableMixer
from .linear import Linear
from .registry import register_mixer
from .spec import MinGRUSpec


class MinGRU(FusableMixer):
    extra_libraries = ("mingru",)

    def __init__(self, spec: MinGRUSpec):
        s = self.spec = spec
        self.inputs = [Linear(s.z), Linear(s.x)] + ([Linear(s.gate)] if s.gate is not None else [])
        self.output = Linear(s.out)

    @property
    def inner_width(self):
        return self.spec.width

    def cache_need(self):
        return FixedStateNeed((self.spec.width,), "float32")

    def mix(self, ctx, proj, col0, inner_out, out_scale, sub=None):
        W = self.spec.width
        ops.mingru_scan(proj, col0, col0 + W, col0 + 2 * W if self.spec.gate is not None else None, ctx.cache(sub),
                        ctx.q_start, ctx.q_len, ctx.state_slots, inner_out, W, out_scale=out_scale,
                        most_tokens=1 if ctx.decode_only else proj.shape[0])


register_mixer("mingru", MinGRU)
