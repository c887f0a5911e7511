"""Mixers of the shape  projections of h -> something with state -> one output projection.

Such a mixer describes itself by its projections (all read the same h), its output projection and the step
between them (``mix``), which reads a slice of the projections' output and fills a buffer of activations.  That
is enough to run it alone (one fused product in, ``mix``, one product out) and to put several of them side by
side (parts/parallel.py): then ALL projections of ALL branches are one product, every branch's ``mix`` fills
its columns of one activation buffer (already multiplied by the branch's scale), and all output projections
are one product over the concatenated columns.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from .base import Mixer
from .linear import Linear, fuse_linears
from .spec import LinearSpec


def fuse_linears_along_k(parts: List[Linear], scales, device) -> Linear:
    """One Linear whose input is the concatenation of the given ones' inputs and whose output is
    sum_i (W_i a_i) + sum_i scales[i] * b_i: the callers put scales[i] * a_i into the concatenated input."""
    ws = [p.weight for p in parts]
    dtype = torch.float32 if any(w.dtype == torch.float32 for w in ws) else ws[0].dtype
    weight = torch.cat([w.to(dtype) for w in ws], dim=1).contiguous()
    bias = None
    for p, s in zip(parts, scales):
        if p.bias is not None:
            b = p.bias * float(s)
            bias = b if bias is None else bias + b
    spec = LinearSpec(sum(p.spec.in_features for p in parts), parts[0].spec.out_features, "<fused>",
                      "<fused>" if bias is not None else None)
    fused = Linear(spec)
    fused.set_weight(weight, bias)
    return fused


class FusableMixer(Mixer):
    """Subclasses set self.inputs (list of Linear reading h), self.output (Linear) and implement
    inner_width, load_extras(), mix()."""
    graph_safe = True
    can_overwrite = True
    inputs: List[Linear] = ()
    output: Optional[Linear] = None
    extra_libraries = ()

    @property
    def libraries(self):
        return ("gemm_simt", "gemm_tc", "gemv") + tuple(self.extra_libraries)

    @property
    def inner_width(self) -> int:
        raise NotImplementedError

    @property
    def projection_width(self) -> int:
        return sum(p.spec.out_features for p in self.inputs)

    def extra_tensor_specs(self):
        return []

    def load_extras(self, tensors, device, act_dtype) -> None:
        pass

    def extra_parameter_bytes(self) -> int:
        return 0

    def mix(self, ctx, proj, col0: int, inner_out, out_scale: float, sub=None) -> None:
        """proj: [N, *], this mixer's projections from column col0 on, in the order of self.inputs;
        inner_out: [N, inner_width] view to fill with out_scale * (the input of the output projection);
        sub: which of the running entry's caches is this mixer's (None: the only one)."""
        raise NotImplementedError

    # ---- alone -------------------------------------------------------------------------------------
    def tensor_specs(self):
        out = []
        for p in list(self.inputs) + [self.output]:
            out += p.tensor_specs()
        return out + list(self.extra_tensor_specs())

    def load(self, tensors, device, act_dtype):
        self.load_parts(tensors, device, act_dtype)
        self._fused_in = fuse_linears(list(self.inputs), device)
        self.release_inputs()

    def load_parts(self, tensors, device, act_dtype):
        for p in list(self.inputs) + [self.output]:
            p.load(tensors, device, act_dtype)
        self.load_extras(tensors, device, act_dtype)

    def release_inputs(self):
        for p in self.inputs:                       # the fused copy is the one that is used
            p.weight = p.bias = None

    def parameter_bytes(self):
        return self._fused_in.parameter_bytes() + self.output.parameter_bytes() + self.extra_parameter_bytes()

    def forward(self, ctx, h, out, accumulate=True):
        N = h.shape[0]
        proj = ctx.scratch(N, self.projection_width)
        self._fused_in.forward(h, proj)
        inner = ctx.scratch(N, self.inner_width)
        self.mix(ctx, proj, 0, inner, 1.0)
        self.output.forward(inner, out, residual=out if accumulate else None)
