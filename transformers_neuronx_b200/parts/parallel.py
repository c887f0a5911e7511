"""Several mixers side by side on the same input:  result = sum_i scale_i * branch_i(h).

Every branch is a FusableMixer (parts/fusable.py), so the whole part is three stages: ONE product for all
projections of all branches, each branch's own step between (attention over its pages, a recurrence over its
state, ...) writing scale_i times its activations into its columns of one buffer, and ONE product for all
output projections over the concatenated columns (the biases add up as sum_i scale_i * b_i).  Each branch
keeps its own cache: the part's cache_need() is the tuple of the branches' needs.
"""
from __future__ import annotations

from .fusable import FusableMixer, fuse_linears_along_k
from .linear import fuse_linears
from .registry import build_part, register_mixer
from .spec import ParallelMixerSpec


class ParallelMixer(FusableMixer):
    def __init__(self, spec: ParallelMixerSpec):
        self.spec = spec
        if len(spec.branches) != len(spec.scales) or not spec.branches:
            raise ValueError("a parallel mixer needs one scale per branch and at least one branch")
        self.branches = [build_part("mixer", b) for b in spec.branches]
        for b in self.branches:
            if not isinstance(b, FusableMixer):
                raise TypeError(f"{type(b).__name__} cannot be a branch of a parallel mixer: it does not describe "
                                "its projections (parts/fusable.py)")
        self.scales = [float(s) for s in spec.scales]

    @property
    def libraries(self):
        libs = []
        for b in self.branches:
            libs += list(b.libraries)
        return tuple(dict.fromkeys(libs))

    def tensor_specs(self):
        out = []
        for b in self.branches:
            out += b.tensor_specs()
        return out

    def load(self, tensors, device, act_dtype):
        for b in self.branches:
            b.load_parts(tensors, device, act_dtype)
        self._fused_in = fuse_linears([p for b in self.branches for p in b.inputs], device)
        self._fused_out = fuse_linears_along_k([b.output for b in self.branches], self.scales, device)
        self._extra_bytes = sum(b.extra_parameter_bytes() for b in self.branches)
        for b in self.branches:
            b.release_inputs()
            b.output.weight = b.output.bias = None

    def parameter_bytes(self):
        return self._fused_in.parameter_bytes() + self._fused_out.parameter_bytes() + self._extra_bytes

    def cache_need(self):
        return tuple(b.cache_need() for b in self.branches)

    def forward(self, ctx, h, out, accumulate=True):
        N = h.shape[0]
        proj = ctx.scratch(N, self._fused_in.spec.out_features)
        self._fused_in.forward(h, proj)
        inner = ctx.scratch(N, self._fused_out.spec.in_features)
        col = k0 = 0
        for j, (b, s) in enumerate(zip(self.branches, self.scales)):
            b.mix(ctx, proj, col, inner[:, k0:k0 + b.inner_width], s, sub=j)
            col += b.projection_width
            k0 += b.inner_width
        self._fused_out.forward(inner, out, residual=out if accumulate else None)


register_mixer("parallel", ParallelMixer)
