"""Softmax attention over the paged cache whose projections pass through a short causal convolution over time.

  q = W_q h + b, k = W_k h + b, v = W_v h + b
  each channel of q, k and v: y_t = sum_j w[c, j] u_(t - taps + 1 + j), zeros before the sequence's start
  q, k: RMS norm per head (one weight vector of k_dim for all heads), then rotated by position on the first
        rotary.dims dims of each head (interleaved pairs or halves, optionally with stretched frequencies)
  score(i, j) = scale * <q_i, k_j>, causal, and windowed or chunked where the spec says; softmax in 32-bit
  output projection

What the mixer keeps between steps: the pages of its keys (after convolution, norm and rotation) and values (after
convolution), and per request the last taps - 1 projected values of every channel (a state slot, in the activation
type: exactly what a longer step would have read from its own rows).  cache_need() is the tuple (pages, state), pages
first; a mixer whose spec names `kv_source` has neither keys nor values: it keeps the state of its queries alone and
reads the pages of the schedule entry with that cache number, which ran earlier in the same step, so that the pages
already hold this step's tokens.

Queries/keys (k_dim) and values (v_dim) may differ in size: as in parts/rotary_attention.py they are written with
D = max(k_dim, v_dim) rounded up to 16 dims a head, the rest zero, and the attention kernels are those of every other
attention part.
"""
from __future__ import annotations

import torch

from ..cache.manager import FixedStateNeed, PagedKVNeed
from ..kernels import ops
from ..weights.loader import TensorSpec
from .base import to_device
from .fusable import FusableMixer
from .linear import Linear
from .registry import register_mixer
from .rotary import inverse_frequencies, rotation_magnitude
from .spec import ConvAttentionSpec

MAX_TAPS = 8           # csrc/conv_qkv.cu


class ConvAttention(FusableMixer):
    @property
    def extra_libraries(self):
        prefill = "attention_prefill_tc" if self.pad_dim in (64, 80, 96, 112, 128) else "attention_prefill"
        return ("conv_qkv", "rotary_qkv", "kv_cache", "attention_simt", prefill, "attention_decode")

    def __init__(self, spec: ConvAttentionSpec):
        s = self.spec = spec
        if s.n_heads % s.n_kv_heads:
            raise ValueError(f"{s.n_heads} heads cannot share {s.n_kv_heads} key/value heads")
        self.pad_dim = -(-max(s.k_dim, s.v_dim) // 16) * 16
        if self.pad_dim > 256:
            raise ValueError(f"head sizes {s.k_dim}/{s.v_dim} are not supported: the attention kernels take up to 256")
        if s.rotary is not None and (s.rotary.dims > s.k_dim or s.rotary.dims % 2):
            raise ValueError(f"{s.rotary.dims} rotated dims do not fit heads of {s.k_dim}")
        if not (0 <= s.conv_taps <= MAX_TAPS):
            raise ValueError(f"a convolution of {s.conv_taps} taps is not supported (at most {MAX_TAPS})")
        if s.window and s.chunk:
            raise ValueError("an attention mixer takes a sliding window or a chunked mask, not both")
        if not (s.scale > 0):
            raise ValueError(f"the scale of the scores must be positive, got {s.scale}")
        self.own_kv = s.kv_source is None
        if self.own_kv and (s.k is None or s.v is None):
            raise ValueError("an attention mixer without kv_source needs key and value projections")
        self.inputs = [Linear(s.q)] + ([Linear(s.k), Linear(s.v)] if self.own_kv else [])
        self.output = Linear(s.out)
        self.keep = max(0, s.conv_taps - 1)                  # projected values kept per channel and request
        self.channels = s.n_heads * s.k_dim + (s.n_kv_heads * (s.k_dim + s.v_dim) if self.own_kv else 0)
        self.conv_w = self.q_weight = self.k_weight = self.inv_freq = None
        self.magnitude = 1.0

    @property
    def inner_width(self):
        return self.spec.n_heads * self.spec.v_dim

    def _conv_names(self):
        s = self.spec
        return [(s.q_conv, s.n_heads * s.k_dim)] + ([(s.k_conv, s.n_kv_heads * s.k_dim),
                                                      (s.v_conv, s.n_kv_heads * s.v_dim)] if self.own_kv else [])

    def extra_tensor_specs(self):
        s, out = self.spec, []
        if s.q_norm:
            out.append(TensorSpec(s.q_norm, (s.k_dim,), "norm_weight"))
        if s.k_norm and self.own_kv:
            out.append(TensorSpec(s.k_norm, (s.k_dim,), "norm_weight"))
        if s.conv_taps:
            for name, ch in self._conv_names():
                if not name:
                    raise ValueError("a convolution needs a weight tensor for each of its projections")
                out.append(TensorSpec(name, (ch, s.conv_taps), "matrix"))
        return out

    def load_extras(self, tensors, device, act_dtype):
        s = self.spec
        f32 = lambda name: to_device(tensors[name], device, torch.float32) if name else None
        self.q_weight, self.k_weight = f32(s.q_norm), (f32(s.k_norm) if self.own_kv else None)
        if s.conv_taps:
            # [taps, channels]: the kernels read a tap's weights of consecutive channels together
            self.conv_w = torch.cat([f32(name) for name, _ in self._conv_names()], dim=0).t().contiguous()
        if s.rotary is not None and s.rotary.dims:
            self.inv_freq = inverse_frequencies(s.rotary.dims, s.rotary.base, device, s.rotary.scaling)
            self.magnitude = rotation_magnitude(s.rotary.scaling)

    def extra_parameter_bytes(self):
        return sum(t.numel() * 4 for t in (self.q_weight, self.k_weight, self.conv_w) if t is not None)

    def cache_need(self):
        s = self.spec
        state = (FixedStateNeed((self.keep, self.channels), "activation"),) if self.keep else ()
        if not self.own_kv:
            return state
        free = s.keep_all_pages
        return (PagedKVNeed(s.n_kv_heads, self.pad_dim, None if free else s.window, None if free else s.chunk),) + state

    def mix(self, ctx, proj, col0, inner_out, out_scale, sub=None):
        if sub is not None:
            raise NotImplementedError("this mixer keeps several caches of its own and cannot be a branch of another")
        s, D, N = self.spec, self.pad_dim, proj.shape[0]
        H, G = s.n_heads, s.n_kv_heads
        q = ctx.scratch(N, H * D)
        k = v = None
        if self.own_kv:
            k, v = ctx.scratch(N, G * D), ctx.scratch(N, G * D)
        state = ctx.cache(1 if self.own_kv else 0) if self.keep else None
        rot = s.rotary
        ops.conv_qkv_prep(proj, col0, self.conv_w, s.conv_taps, state, ctx, self.q_weight, self.k_weight, s.norm_eps,
                          self.inv_freq, rot.dims if rot is not None else 0, bool(rot is not None and rot.interleaved),
                          self.magnitude, q, k, v, H, G if self.own_kv else 0, s.k_dim, s.v_dim, D)
        if self.own_kv:
            cache, g = ctx.cache(0), ctx.cache_group(0)
            new_kv = (k, v, ctx.slot_mapping[g])
        else:
            cache, g = ctx.cache_of(s.kv_source, 0), ctx.cache_group_of(s.kv_source, 0)
            new_kv = None
            if cache.dim() != 5 or cache.shape[2] != G or cache.shape[4] != D:
                raise ValueError(f"cache {s.kv_source} does not hold pages of {G} key/value heads of {D} dims")
        direct = s.v_dim == D and out_scale == 1.0 and inner_out.is_contiguous()
        att = inner_out if direct else ctx.scratch(N, H * D)
        ops.attention(ctx, g, q, cache, att, H, s.scale, s.window or 0, new_kv=new_kv, chunk=s.chunk or 0)
        if not direct:
            ops.rotary_unrotate(att, ctx.token_request, ctx.positions, None, out_scale, inner_out, H, s.v_dim, D)


register_mixer("conv_attention", ConvAttention)
