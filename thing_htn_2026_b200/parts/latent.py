"""Latent attention: keys and values of all heads are read out of one low-rank latent per token.

Per token, with ``n_heads`` heads, ``plain_dim`` unrotated and ``rot_dim`` rotated query/key
entries per head, values of ``value_dim`` and a latent of ``latent_rank``:

    q            = W_q x                      laid out head by head as [plain | rot]
    [l | r]      = W_dkv x                    latent_rank + rot_dim entries
    c            = l / sqrt(mean(l^2) + eps) * w_norm
    k_h          = [W_uk,h c | rotate(r)]     the rotated part is shared by the heads
    v_h          = W_uv,h c
    score        = (q_h . k_h) * scale        with the rot part of q_h rotated as well
    out          = W_o (concat_h softmax(score) v_h * logistic(W_g x))

The rotation pairs entries 2i and 2i + 1 of the rot part (the position part's "interleaved"
layout, with whatever frequency scaling its spec names).  ``window`` (None: all keys): position
i sees j with 0 <= i - j < window.  ``gated`` False leaves the output gate (and ``g_proj``) out.

One product gives q, the latent row and the gate (weights concatenated ``[q; dkv; g]``); a
second one, on the normalised latent, gives every head's unrotated key and value (``[uk; uv]``).
The cache holds per head the assembled key and the value (a window bounds what a sequence
holds), so the attention kernels of the other mixers serve this one unchanged.  Where the values
are smaller than the keys and the tensor-core attention kernels take the keys' size (bfloat16),
the cache's values are padded to that size with zeros, and the gate's rows and the output
projection's columns with them, so that those kernels serve such sizes too; the result is the
same, entry by entry.  Kernels: csrc/latent_prepare.cu.
"""

from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .. import ops
from ..cache.sequence_cache import PAGE_SIZE, CacheNeed, KVSpec
from ..config.base import PartSpec, ScheduleEntry
from ..weights.loader import GAIN, MATRIX, TensorSpec
from .registry import part_class, register_part
from .runtime import HostBatch, Runtime, StepContext


@register_part("mixer", "latent_attention")
class LatentAttention:
    @staticmethod
    def _sizes(spec: PartSpec):
        p = spec.params
        return (int(p["hidden_size"]), int(p["n_heads"]), int(p["plain_dim"]), int(p["rot_dim"]), int(p["value_dim"]),
                int(p["latent_rank"]))

    @classmethod
    def tensor_specs(cls, spec: PartSpec) -> List[TensorSpec]:
        hidden, h, d, r, e, c = cls._sizes(spec)
        specs = [TensorSpec(spec.tensors["q_proj"], (h * (d + r), hidden), MATRIX),
                 TensorSpec(spec.tensors["down_proj"], (c + r, hidden), MATRIX),
                 TensorSpec(spec.tensors["latent_norm"], (c,), GAIN),
                 TensorSpec(spec.tensors["up_k"], (h * d, c), MATRIX),
                 TensorSpec(spec.tensors["up_v"], (h * e, c), MATRIX)]
        if spec.params.get("gated", True):
            specs.append(TensorSpec(spec.tensors["g_proj"], (h * e, hidden), MATRIX))
        specs.append(TensorSpec(spec.tensors["o_proj"], (hidden, h * e), MATRIX))
        return specs

    def __init__(self, spec: PartSpec, runtime: Runtime):
        p = spec.params
        _, self.n_heads, self.plain, self.rot, self.value_dim, self.rank = self._sizes(spec)
        if self.rot % 2:
            raise ValueError(f"latent_attention: rot_dim {self.rot} must be even")
        self.scale = float(p["scale"])
        self.window: Optional[int] = None if p.get("window") is None else int(p["window"])
        self.eps = float(p["norm_eps"])
        self.gated = bool(p.get("gated", True))
        self.exact_weights = p.get("softmax_weights") == "float32"
        self.dtype = runtime.dtype
        # the size of a value in the cache and in the attention's output: its own, or the keys'
        key_dim, hidden = self.plain + self.rot, int(p["hidden_size"])
        self.out_dim = self.value_dim
        if runtime.dtype == torch.bfloat16 and self.value_dim < key_dim and p.get("pad_values", True) \
                and ops.lib().thn_attention_mma_supported(key_dim, PAGE_SIZE, self.n_heads, self.n_heads):
            self.out_dim = key_dim
        pad = self.out_dim - self.value_dim
        parts = [runtime.tensor(spec, "q_proj"), runtime.tensor(spec, "down_proj")]
        if self.gated:
            gate = runtime.tensor(spec, "g_proj")
            if pad:
                gate = torch.nn.functional.pad(gate.view(self.n_heads, self.value_dim, hidden), (0, 0, 0, pad))
                gate = gate.reshape(self.n_heads * self.out_dim, hidden)
            parts.append(gate)
        self.w_in = torch.cat(parts, dim=0).contiguous()
        self.w_up = torch.cat([runtime.tensor(spec, "up_k"), runtime.tensor(spec, "up_v")], dim=0).contiguous()
        self.w_o = runtime.tensor(spec, "o_proj")
        if pad:
            self.w_o = torch.nn.functional.pad(self.w_o.view(hidden, self.n_heads, self.value_dim), (0, pad))
            self.w_o = self.w_o.reshape(hidden, self.n_heads * self.out_dim).contiguous()
        self.latent_gain = runtime.tensor(spec, "latent_norm").to(torch.float32).contiguous()
        self.latent_offset = self.n_heads * (self.plain + self.rot)
        self.shared_offset = self.latent_offset + self.rank
        self.gate_offset = self.shared_offset + self.rot
        self.position = None
        position_spec = p.get("position")
        if self.rot:
            if position_spec is None:
                raise ValueError("latent_attention: a rotated part needs a position spec")
            key = "position:" + position_spec.key()
            if key not in runtime.shared:
                runtime.shared[key] = part_class("position", position_spec.kind)(position_spec, runtime)
            self.position = runtime.shared[key]

    def cache_need(self) -> CacheNeed:
        return KVSpec(self.n_heads, self.plain + self.rot, self.window, 0, None, self.out_dim)

    def _tile(self, page_size: int) -> int:
        return ops.prompt_attention_tile(self.dtype, self.plain + self.rot, page_size, self.n_heads, self.n_heads,
                                         self.out_dim)

    def step_inputs(self, batch: HostBatch, out: Dict[str, List[int]]) -> None:
        """Row tiles for the tensor-core prompt kernel, where keys and values have one size that it
        takes (the list is shared with every other attention that wants tiles of this size)."""
        size = self._tile(batch.page_size) if batch.max_count > 1 else 0
        if size and f"row_tiles/{size}/row0" not in out:
            out[f"row_tiles/{size}/row0"], out[f"row_tiles/{size}/rows"] = ops.row_tiles_of(
                batch.counts, batch.held, size)

    def forward(self, x: torch.Tensor, ctx: StepContext, entry: ScheduleEntry) -> torch.Tensor:
        kv = ctx.cache.kv_view(entry.cache)
        tiles = None
        if ctx.rows.max_q_len > 1:
            size = self._tile(kv.page_size)
            row0 = ctx.inputs.get(f"row_tiles/{size}/row0") if size else None
            if row0 is not None:
                tiles = ops.RowTiles(row0, ctx.inputs[f"row_tiles/{size}/rows"], row0.shape[0], size)
        proj = ops.linear(x, self.w_in, err=ctx.err)
        latent = ops.latent_norm(proj, self.latent_offset, self.rank, self.latent_gain, self.eps)
        up = ops.linear(latent, self.w_up, err=ctx.err)
        q = ops.latent_assemble(proj, 0, self.shared_offset, up, self.position.tables() if self.position else None,
                                ctx.rows, kv, self.n_heads, self.plain, self.rot, ctx.err, self.value_dim)
        a = ops.attention(q, ctx.rows, kv, self.n_heads, self.scale, self.window, ctx.err, tiles,
                          exact_weights=self.exact_weights)
        if self.gated:
            a = ops.logistic_gate(a, proj, self.gate_offset)
        return ops.linear(a, self.w_o, err=ctx.err)
