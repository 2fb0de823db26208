"""The gated delta rule: a recurrent token mixer.  Per head it keeps a matrix ``S [key_dim,
value_dim]`` and, for every token, decays it, corrects what it returns for the token's key
towards the token's value, and reads it with the token's query:

    S <- g S;   u = b (v - S^T k);   S <- S + k u^T;   o = S^T q

q and k (``n_kv_heads`` heads of ``key_dim``, shared by ``n_heads / n_kv_heads`` heads each) and
v (``n_heads`` heads of ``value_dim``) are projections of the input that pass a short causal
convolution over time per channel (``conv_taps`` taps, the last one the current token's, no
bias) and silu; q and k are then unit vectors per head (``x / sqrt(sum x^2 + unit_norm_eps)``),
q scaled by ``key_dim ** -0.5``.  ``b = logistic(b_proj x)`` and
``g = exp(-exp(A_log) softplus(a_proj x + dt_bias))`` are one number per head and token.  The
read-out is normalised per head over ``value_dim`` (RMS, ``norm_eps``, one gain vector shared
by the heads), multiplied by ``silu(g_proj x)`` and projected back.

One product gives all six projections (weights concatenated ``[q; k; v; gate; b; a]``).  The
state per sequence, zero when a slot opens: S in float32 ``[n_heads, value_dim, key_dim]`` and
a ring of the last ``conv_taps`` raw q/k/v projections (the convolution's window).  Everything
that enters the recurrence after the projections is float32.  Kernels: csrc/delta_rule.cu.
"""

from __future__ import annotations

from typing import List

import torch

from .. import ops
from ..cache.sequence_cache import CacheNeed, StateSpec
from ..config.base import PartSpec, ScheduleEntry
from ..weights.loader import GAIN, MATRIX, TensorSpec
from .registry import register_part
from .runtime import Runtime, StepContext

PROJECTIONS = ("q", "k", "v", "g", "b", "a")     # the order of the fused product's columns
CONVOLVED = ("q", "k", "v")


@register_part("mixer", "gated_delta")
class GatedDelta:
    @staticmethod
    def _shape(spec: PartSpec) -> ops.DeltaShape:
        p = spec.params
        return ops.DeltaShape(int(p["n_heads"]), int(p["n_kv_heads"]), int(p["key_dim"]), int(p["value_dim"]),
                              int(p["conv_taps"]))

    @classmethod
    def _widths(cls, spec: PartSpec) -> dict:
        s = cls._shape(spec)
        return {"q": s.n_kv * s.key_dim, "k": s.n_kv * s.key_dim, "v": s.n_heads * s.value_dim,
                "g": s.n_heads * s.value_dim, "b": s.n_heads, "a": s.n_heads}

    @classmethod
    def tensor_specs(cls, spec: PartSpec) -> List[TensorSpec]:
        s, hidden, widths = cls._shape(spec), int(spec.params["hidden_size"]), cls._widths(spec)
        specs = [TensorSpec(spec.tensors[name], (widths[name], hidden), MATRIX) for name in PROJECTIONS]
        specs += [TensorSpec(spec.tensors[name + ".conv"], (widths[name], s.taps), GAIN, init="conv_taps")
                  for name in CONVOLVED]
        specs += [TensorSpec(spec.tensors["A_log"], (s.n_heads,), GAIN, init="log_rate"),
                  TensorSpec(spec.tensors["dt_bias"], (s.n_heads,), GAIN, init="unit_normal"),
                  TensorSpec(spec.tensors["norm"], (s.value_dim,), GAIN),
                  TensorSpec(spec.tensors["o"], (hidden, s.n_heads * s.value_dim), MATRIX)]
        return specs

    def __init__(self, spec: PartSpec, runtime: Runtime):
        self.shape = s = self._shape(spec)
        if s.n_heads % s.n_kv:
            raise ValueError(f"gated_delta: {s.n_heads} heads are not a multiple of {s.n_kv} key heads")
        self.norm_eps = float(spec.params["norm_eps"])
        self.unit_eps = float(spec.params["unit_norm_eps"])
        self.dtype = runtime.dtype
        self.w_in = torch.cat([runtime.tensor(spec, name) for name in PROJECTIONS], dim=0).contiguous()
        self.w_o = runtime.tensor(spec, "o")
        f32 = lambda t: t.to(torch.float32).contiguous()
        self.conv_w = f32(torch.cat([runtime.tensor(spec, name + ".conv") for name in CONVOLVED], dim=0))
        self.a_log, self.dt_bias = f32(runtime.tensor(spec, "A_log")), f32(runtime.tensor(spec, "dt_bias"))
        self.out_gain = f32(runtime.tensor(spec, "norm"))

    def cache_need(self) -> CacheNeed:
        s = self.shape
        return (StateSpec((s.n_heads, s.value_dim, s.key_dim), torch.float32),
                StateSpec((s.taps, s.conv_channels), self.dtype))

    def forward(self, x: torch.Tensor, ctx: StepContext, entry: ScheduleEntry) -> torch.Tensor:
        s = self.shape
        proj = ops.linear(x, self.w_in, err=ctx.err)
        o = ops.delta_rule(proj, self.conv_w, self.a_log, self.dt_bias, ctx.cache.state_view(entry.cache, 0),
                           ctx.cache.state_view(entry.cache, 1), ctx.rows, ctx.cache.seq_lens, s, self.unit_eps)
        y = ops.gated_head_norm(o, proj, s.gate_offset, self.out_gain, self.norm_eps, s.n_heads, s.value_dim, self.dtype)
        return ops.linear(y, self.w_o, err=ctx.err)
