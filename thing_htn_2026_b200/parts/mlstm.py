"""Matrix memory with exponential gating (the mLSTM of xLSTM): a recurrent token mixer.  Per
head it keeps a matrix ``S [key_dim, value_dim]``, a vector ``n [key_dim]`` and a running
maximum ``m``, all zero at the start of a sequence, and for every token

    i = cap tanh((W_i x + b_i) / cap)              f = logsigmoid(cap tanh((W_f x + b_f) / cap))
    m' = max(f + m, i)
    S <- exp(f + m - m') S + exp(i - m') k v^T     n <- exp(f + m - m') n + exp(i - m') k
    o  = S^T q / (max(|n . q|, exp(-m')) + 1e-6)

with ``q = W_q x * key_dim^-1/2``, ``k = W_k x``, ``v = W_v x`` per head.  Each head's ``o`` is
divided by its root mean square (``norm_eps``), the heads are concatenated, multiplied by a gain
over all heads' entries and by ``logistic(W_g x)``, and projected back.

One product gives q, k, v and the output gate (weights concatenated ``[q; k; v; g]``); the two
gates' pre-activations come from a second, narrow product whose result stays float32.  The state
per sequence is float32: ``S`` as ``[n_heads, value_dim, key_dim]`` and, per block of columns of
the kernel, a copy of ``n`` and ``m`` (``[n_heads, blocks, key_dim + 1]``).  Everything that enters
the recurrence after the projections is float32.  Kernels: csrc/mlstm.cu.
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

PROJECTIONS = ("q", "k", "v", "g")     # the order of the fused product's columns


@register_part("mixer", "mlstm")
class MatrixMemory:
    @staticmethod
    def _sizes(spec: PartSpec):
        p = spec.params
        return int(p["hidden_size"]), int(p["n_heads"]), int(p["key_dim"]), int(p["value_dim"])

    @classmethod
    def tensor_specs(cls, spec: PartSpec) -> List[TensorSpec]:
        hidden, h, d, e = cls._sizes(spec)
        widths = {"q": h * d, "k": h * d, "v": h * e, "g": h * e}
        specs = [TensorSpec(spec.tensors[name], (widths[name], hidden), MATRIX) for name in PROJECTIONS]
        specs += [TensorSpec(spec.tensors["i"], (h, hidden), MATRIX), TensorSpec(spec.tensors["i_bias"], (h,), GAIN, init="gate_bias"),
                  TensorSpec(spec.tensors["f"], (h, hidden), MATRIX), TensorSpec(spec.tensors["f_bias"], (h,), GAIN, init="gate_bias"),
                  TensorSpec(spec.tensors["norm"], (h * e,), GAIN),
                  TensorSpec(spec.tensors["o"], (hidden, h * e), MATRIX)]
        return specs

    def __init__(self, spec: PartSpec, runtime: Runtime):
        _, self.n_heads, self.key_dim, self.value_dim = self._sizes(spec)
        self.cap = float(spec.params["gate_cap"])
        self.norm_eps = float(spec.params["norm_eps"])
        self.floor = float(spec.params.get("denominator_floor", 1e-6))
        self.dtype = runtime.dtype
        self.w_in = torch.cat([runtime.tensor(spec, name) for name in PROJECTIONS], dim=0).contiguous()
        self.w_gates = torch.cat([runtime.tensor(spec, "i"), runtime.tensor(spec, "f")], dim=0).contiguous()
        self.w_o = runtime.tensor(spec, "o")
        f32 = lambda t: t.to(torch.float32).contiguous()
        self.bias_i, self.bias_f = f32(runtime.tensor(spec, "i_bias")), f32(runtime.tensor(spec, "f_bias"))
        self.out_gain = f32(runtime.tensor(spec, "norm"))
        self.gate_offset = self.n_heads * (2 * self.key_dim + self.value_dim)

    def cache_need(self) -> CacheNeed:
        blocks = -(-self.value_dim // ops.MLSTM_COLUMNS_PER_BLOCK)
        return (StateSpec((self.n_heads, self.value_dim, self.key_dim), torch.float32),
                StateSpec((self.n_heads, blocks, self.key_dim + 1), torch.float32))

    def forward(self, x: torch.Tensor, ctx: StepContext, entry: ScheduleEntry) -> torch.Tensor:
        proj = ops.linear(x, self.w_in, err=ctx.err)
        gate_pre = ops.linear(x, self.w_gates, out_dtype=torch.float32, err=ctx.err)
        o = ops.mlstm(proj, gate_pre, self.bias_i, self.bias_f, self.cap, ctx.cache.state_view(entry.cache, 0),
                      ctx.cache.state_view(entry.cache, 1), ctx.rows, self.n_heads, self.key_dim, self.value_dim,
                      self.key_dim ** -0.5, self.floor)
        y = ops.gated_head_norm(o, proj, self.gate_offset, self.out_gain, self.norm_eps, self.n_heads, self.value_dim,
                                self.dtype, gate_kind="logistic")
        return ops.linear(y, self.w_o, err=ctx.err)
