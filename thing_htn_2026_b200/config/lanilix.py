"""Typed configuration of the Lanilix decoder: a stack of layers given one by one, each with
a token mixer of one of two kinds and an optional gated feed-forward, norms before and after
every sublayer, and a residual stream kept in float32.

config.json keys::

    architecture   "Lanilix"
    vocab, width   sizes of the embedding table ``embed`` [vocab, width] and the head ``head``
    norm.eps       eps of every RMS norm of the model
    layers         a list; entry i has
        type        "delta" (gated delta rule) or "attention" (windowed softmax attention)
        mixer       the mixer's sizes and constants, see below
        mlp         {"kind": "dense", "ff", "limit"} or null (no feed-forward in this layer)
        weights_of  optional: the index of the layer whose tensors this layer uses; it then has
                    none of its own, but a cache or state of its own

    mixer of "delta":      heads, kv_heads, dim, vdim, conv (taps of the short convolutions)
    mixer of "attention":  heads, kv_heads, dim, vdim, scale,
                           rot {"base", "dims"} (rotation of the first dims entries of a head),
                           mask {"size", "keep_first"} (window, and first positions kept visible)

Tensor names: layer i's start with ``l<i>.``; its norms are ``norm1, norm1b, norm2, norm2b``
(gains stored around zero), its mixer's tensors ``mix.*``, its feed-forward's ``mlp.*``; the
model's last norm is ``final.norm``.

Constants that the design fixes (not in config.json) are parameters of the parts all the
same, set here: the unit norms' eps 1e-6, the feed-forward's logistic slope 1.702.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, List, Mapping, Optional, Tuple

from .base import ConfigError, LayerSpec, ModelConfig, ModelPlan, PartSpec, ScheduleEntry, _freeze, require

DELTA = "delta"
ATTENTION = "attention"

UNIT_NORM_EPS = 1e-6
GLU_SLOPE = 1.702


def _section(data: Mapping[str, Any], key: str, where: str) -> Mapping[str, Any]:
    value = data.get(key)
    if not isinstance(value, Mapping):
        raise ConfigError(f"config.json: {where}'{key}' must be an object")
    return value


def _int(data: Mapping[str, Any], key: str, where: str, minimum: int = 1) -> int:
    value = data.get(key)
    if isinstance(value, bool) or not isinstance(value, int) or value < minimum:
        raise ConfigError(f"config.json: {where}'{key}' must be an integer >= {minimum}, got {value!r}")
    return value


def _float(data: Mapping[str, Any], key: str, where: str) -> float:
    value = data.get(key)
    if isinstance(value, bool) or not isinstance(value, (int, float)) or not value > 0:
        raise ConfigError(f"config.json: {where}'{key}' must be a positive number, got {value!r}")
    return float(value)


@dataclass(frozen=True)
class LanilixConfig(ModelConfig):
    vocab: int
    width: int
    norm_eps: float
    layers: Tuple[Mapping[str, Any], ...]
    max_positions: int = 1 << 20

    architecture = "Lanilix"

    # ------------------------------------------------------------------ reading

    @classmethod
    def from_dict(cls, data: Mapping[str, Any]) -> "LanilixConfig":
        layers = data.get("layers")
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        config = cls(
            vocab=require(data, "vocab", int),
            width=require(data, "width", int),
            norm_eps=_float(_section(data, "norm", ""), "eps", "norm."),
            layers=tuple(_freeze(dict(layer)) for layer in layers),
            max_positions=int(data.get("max_positions", 1 << 20)),
        )
        config.validate()
        return config

    def validate(self) -> None:
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]."
            kind = layer.get("type")
            if kind not in (DELTA, ATTENTION):
                raise ConfigError(f"config.json: {where}'type' must be '{DELTA}' or '{ATTENTION}', got {kind!r}")
            mixer = _section(layer, "mixer", where)
            heads, kv_heads = _int(mixer, "heads", where + "mixer."), _int(mixer, "kv_heads", where + "mixer.")
            if heads % kv_heads:
                raise ConfigError(f"config.json: {where}mixer.heads {heads} is not a multiple of kv_heads {kv_heads}")
            dim, vdim = _int(mixer, "dim", where + "mixer."), _int(mixer, "vdim", where + "mixer.")
            if kind == DELTA:
                _int(mixer, "conv", where + "mixer.")
            else:
                _float(mixer, "scale", where + "mixer.")
                if vdim != dim:
                    raise ConfigError(f"config.json: {where}mixer.vdim {vdim} differs from dim {dim}; the values of "
                                      f"this attention are its keys")
                rot = mixer.get("rot")
                if rot is not None:
                    dims = _int(rot, "dims", where + "mixer.rot.", 0)
                    if dims % 2 or dims > dim:
                        raise ConfigError(f"config.json: {where}mixer.rot.dims {dims} must be even and at most dim {dim}")
                    if dims:
                        _float(rot, "base", where + "mixer.rot.")
                mask = mixer.get("mask")
                if mask is not None:
                    _int(mask, "size", where + "mixer.mask.")
                    _int(mask, "keep_first", where + "mixer.mask.", 0)
            mlp = layer.get("mlp")
            if mlp is not None:
                if mlp.get("kind") != "dense":
                    raise ConfigError(f"config.json: {where}mlp.kind must be 'dense', got {mlp.get('kind')!r}")
                _int(mlp, "ff", where + "mlp.")
                _float(mlp, "limit", where + "mlp.")
            owner = layer.get("weights_of")
            if owner is not None:
                if isinstance(owner, bool) or not isinstance(owner, int) or not 0 <= owner < len(self.layers) or owner == i:
                    raise ConfigError(f"config.json: {where}weights_of must name another layer, got {owner!r}")
                if self.layers[owner].get("weights_of") is not None:
                    raise ConfigError(f"config.json: {where}weights_of names layer {owner}, which has no tensors of its own")
                if self.layers[owner].get("type") != kind:
                    raise ConfigError(f"config.json: {where}weights_of names a layer of another type")

    def to_dict(self) -> dict:
        def thaw(value):
            if isinstance(value, Mapping):
                return {k: thaw(v) for k, v in value.items()}
            if isinstance(value, tuple):
                return [thaw(v) for v in value]
            return value
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                "norm": {"eps": self.norm_eps}, "layers": [thaw(layer) for layer in self.layers]}

    # ------------------------------------------------------------------ the plan

    def _norm(self, name: str) -> PartSpec:
        return PartSpec("rmsnorm", {"size": self.width, "eps": self.norm_eps, "gain_offset": 1.0,
                                    "residual": "float32"}, {"weight": name})

    def _mixer(self, layer: Mapping[str, Any], prefix: str) -> PartSpec:
        m = layer["mixer"]
        if layer["type"] == DELTA:
            return PartSpec(
                "gated_delta",
                {"hidden_size": self.width, "n_heads": m["heads"], "n_kv_heads": m["kv_heads"], "key_dim": m["dim"],
                 "value_dim": m["vdim"], "conv_taps": m["conv"], "norm_eps": self.norm_eps,
                 "unit_norm_eps": UNIT_NORM_EPS},
                {name: f"{prefix}mix.{name}" for name in
                 ("q", "k", "v", "q.conv", "k.conv", "v.conv", "b", "a", "A_log", "dt_bias", "g", "norm", "o")})
        rot, mask = m.get("rot"), m.get("mask")
        position = None
        if rot is not None and rot["dims"]:
            position = PartSpec("rope", {"head_dim": m["dim"], "rotary_dim": rot["dims"], "theta": float(rot["base"]),
                                         "layout": "interleaved", "frequency_precision": "float64"})
        return PartSpec(
            "attention",
            {"hidden_size": self.width, "n_heads": m["heads"], "n_kv_heads": m["kv_heads"], "head_dim": m["dim"],
             "scale": float(m["scale"]), "window": None if mask is None else mask["size"],
             "keep_first": 0 if mask is None else mask["keep_first"], "qk_norm_eps": self.norm_eps,
             "qk_norm_scope": "projection", "values": "keys", "position": position},
            {"q_proj": f"{prefix}mix.q", "k_proj": f"{prefix}mix.k", "o_proj": f"{prefix}mix.o",
             "q_norm": f"{prefix}mix.q.norm", "k_norm": f"{prefix}mix.k.norm"})

    def plan(self) -> ModelPlan:
        layers: List[LayerSpec] = []
        index_of = {}
        schedule: List[ScheduleEntry] = []
        for i, layer in enumerate(self.layers):
            if layer.get("weights_of") is None:
                prefix = f"l{i}."
                mlp = layer.get("mlp")
                parts = dict(norm_mixer=self._norm(prefix + "norm1"), mixer=self._mixer(layer, prefix),
                             post_norm_mixer=self._norm(prefix + "norm1b"))
                if mlp is not None:
                    parts.update(
                        norm_ffn=self._norm(prefix + "norm2"),
                        ffn=PartSpec("clamped_glu",
                                     {"hidden_size": self.width, "intermediate_size": mlp["ff"],
                                      "limit": float(mlp["limit"]), "slope": GLU_SLOPE},
                                     {"gate_proj": prefix + "mlp.gate", "up_proj": prefix + "mlp.up",
                                      "down_proj": prefix + "mlp.down"}),
                        post_norm_ffn=self._norm(prefix + "norm2b"))
                index_of[i] = len(layers)
                layers.append(LayerSpec.of("sandwich_norm", **parts))
        for i, layer in enumerate(self.layers):
            owner = layer.get("weights_of")
            schedule.append(ScheduleEntry(layer=index_of[i if owner is None else owner], cache=i))
        return ModelPlan(
            hidden_size=self.width,
            vocab_size=self.vocab,
            embedding=PartSpec("embedding", {"vocab_size": self.vocab, "hidden_size": self.width}, {"weight": "embed"}),
            layers=tuple(layers),
            schedule=tuple(schedule),
            final_norm=self._norm("final.norm"),
            head=PartSpec("lm_head", {"vocab_size": self.vocab, "hidden_size": self.width, "tied": False},
                          {"weight": "head"}),
            max_positions=self.max_positions,
        )
