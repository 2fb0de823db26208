"""Typed configuration of the Bunudra decoder: a stack of layers given one by one, each with a
token mixer of one of three kinds and an optional mixture-of-experts feed-forward.  The norm
(a layer norm with gain and bias) stands on a sublayer's output only; the sublayers read the
residual stream itself, which is kept in float32 and starts as the token's embedding times a
constant.

config.json keys::

    architecture      "Bunudra"
    vocab, width      sizes of the embedding table ``embed`` [vocab, width] and the head ``head``
    embedding.scale   the factor on the embedding
    norm.eps          eps of every norm of the model (layer norms, q/k norms, latent norm, read-out norm)
    layers            a list; entry i has
        type   "attention", "mlstm" or "latent_attention"
        mixer  the mixer's sizes and constants, see below
        mlp    {"kind": "moe", "expert": {"ff"}, "router": {"experts", "top", "scale", "groups": {"count", "keep"}},
                "shared": {"ff"}} or null (no feed-forward in this layer)

    mixer of "attention":         heads, kv_heads, dim, vdim, scale, rot {"base", "dims"} (rotation of the
                                  first dims entries of a head, entry i paired with i + dims/2),
                                  mask {"size"} (chunks of that many positions)
    mixer of "mlstm":             heads, dim, vdim, gate_cap
    mixer of "latent_attention":  heads, dim (unrotated), rot_dim (rotated), vdim, kv_rank, scale,
                                  rot {"base", "dims", "scaling": {"factor", "original", "fast", "slow"}}
                                  (entry 2i paired with 2i + 1), mask {"size"} (sliding window)

Tensor names: layer i's start with ``l<i>.``; its norms are ``norm1`` and ``norm2`` with biases
``norm1.b`` and ``norm2.b``, its mixer's tensors ``mix.*``, its feed-forward's ``mlp.*`` (experts
``mlp.e<j>.up`` / ``.down``, ``mlp.router``, ``mlp.shared.up`` / ``.down`` / ``.sg``); the model's last
norm is ``final.norm`` (+ ``.b``).

The floor 1e-6 of the matrix memory's denominator is a constant of the design; it is a
parameter of the part all the same, set here.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, List, Mapping, Optional, Tuple

from .base import ConfigError, LayerSpec, ModelConfig, ModelPlan, PartSpec, ScheduleEntry, _freeze, require

ATTENTION = "attention"
MLSTM = "mlstm"
LATENT = "latent_attention"

DENOMINATOR_FLOOR = 1e-6


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


def _rotation(mixer: Mapping[str, Any], where: str, limit: int, scaling_allowed: bool) -> None:
    rot = mixer.get("rot")
    if rot is None:
        return
    dims = _int(rot, "dims", where + "rot.", 0)
    if dims % 2 or dims > limit:
        raise ConfigError(f"config.json: {where}rot.dims {dims} must be even and at most {limit}")
    if dims:
        _float(rot, "base", where + "rot.")
    scaling = rot.get("scaling")
    if scaling is not None:
        if not scaling_allowed:
            raise ConfigError(f"config.json: {where}rot.scaling is not part of this mixer")
        for key in ("factor", "original", "fast", "slow"):
            _float(scaling, key, where + "rot.scaling.")


@dataclass(frozen=True)
class BunudraConfig(ModelConfig):
    vocab: int
    width: int
    embedding_scale: float
    norm_eps: float
    layers: Tuple[Mapping[str, Any], ...]
    max_positions: int = 1 << 20

    architecture = "Bunudra"

    # ------------------------------------------------------------------ reading

    @classmethod
    def from_dict(cls, data: Mapping[str, Any]) -> "BunudraConfig":
        layers = data.get("layers")
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        embedding = data.get("embedding") or {}
        config = cls(
            vocab=require(data, "vocab", int),
            width=require(data, "width", int),
            embedding_scale=_float(embedding, "scale", "embedding.") if "scale" in embedding else 1.0,
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
            if kind not in (ATTENTION, MLSTM, LATENT):
                raise ConfigError(f"config.json: {where}'type' must be '{ATTENTION}', '{MLSTM}' or '{LATENT}', got {kind!r}")
            mixer = _section(layer, "mixer", where)
            at = where + "mixer."
            heads, dim, vdim = _int(mixer, "heads", at), _int(mixer, "dim", at), _int(mixer, "vdim", at)
            if kind == MLSTM:
                _float(mixer, "gate_cap", at)
            else:
                _float(mixer, "scale", at)
                mask = mixer.get("mask")
                if mask is not None:
                    _int(mask, "size", at + "mask.")
            if kind == ATTENTION:
                kv_heads = _int(mixer, "kv_heads", at)
                if heads % kv_heads:
                    raise ConfigError(f"config.json: {at}heads {heads} is not a multiple of kv_heads {kv_heads}")
                _rotation(mixer, at, dim, scaling_allowed=False)
            if kind == LATENT:
                _int(mixer, "kv_rank", at)
                rot_dim = _int(mixer, "rot_dim", at, 0)
                _rotation(mixer, at, rot_dim, scaling_allowed=True)
                rot = mixer.get("rot")
                if rot_dim and (rot is None or rot.get("dims") != rot_dim):
                    raise ConfigError(f"config.json: {at}rot.dims must equal rot_dim {rot_dim}")
            mlp = layer.get("mlp")
            if mlp is not None:
                at = where + "mlp."
                if mlp.get("kind") != "moe":
                    raise ConfigError(f"config.json: {at}kind must be 'moe', got {mlp.get('kind')!r}")
                _int(_section(mlp, "expert", at), "ff", at + "expert.")
                router = _section(mlp, "router", at)
                experts, top = _int(router, "experts", at + "router."), _int(router, "top", at + "router.")
                if "scale" in router:
                    _float(router, "scale", at + "router.")
                count, keep = 1, 1
                groups = router.get("groups")
                if groups is not None:
                    count, keep = _int(groups, "count", at + "router.groups."), _int(groups, "keep", at + "router.groups.")
                if experts % count or keep > count or top > keep * (experts // count):
                    raise ConfigError(f"config.json: {at}router: top {top} of {experts} experts in {count} groups of "
                                      f"which {keep} are kept cannot be chosen")
                if mlp.get("shared") is not None:
                    _int(mlp["shared"], "ff", at + "shared.")

    def to_dict(self) -> dict:
        def thaw(value):
            if isinstance(value, Mapping):
                return {k: thaw(v) for k, v in value.items()}
            if isinstance(value, tuple):
                return [thaw(v) for v in value]
            return value
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                "embedding": {"scale": self.embedding_scale}, "norm": {"eps": self.norm_eps},
                "layers": [thaw(layer) for layer in self.layers]}

    # ------------------------------------------------------------------ the plan

    def _norm(self, name: str) -> PartSpec:
        return PartSpec("layernorm", {"size": self.width, "eps": self.norm_eps, "residual": "float32"},
                        {"weight": name, "bias": name + ".b"})

    def _mixer(self, layer: Mapping[str, Any], prefix: str) -> PartSpec:
        m, kind = layer["mixer"], layer["type"]
        t = lambda *names: {key: f"{prefix}mix.{name}" for key, name in names}
        if kind == MLSTM:
            return PartSpec(
                "mlstm",
                {"hidden_size": self.width, "n_heads": m["heads"], "key_dim": m["dim"], "value_dim": m["vdim"],
                 "gate_cap": float(m["gate_cap"]), "norm_eps": self.norm_eps, "denominator_floor": DENOMINATOR_FLOOR},
                t(("q", "q"), ("k", "k"), ("v", "v"), ("g", "g"), ("o", "o"), ("norm", "norm"), ("i", "i"),
                  ("i_bias", "i.b"), ("f", "f"), ("f_bias", "f.b")))
        rot, mask = m.get("rot"), m.get("mask")
        if kind == ATTENTION:
            position = None
            if rot is not None and rot["dims"]:
                position = PartSpec("rope", {"head_dim": m["dim"], "rotary_dim": rot["dims"], "theta": float(rot["base"]),
                                             "layout": "half", "frequency_precision": "float64"})
            return PartSpec(
                "attention",
                {"hidden_size": self.width, "n_heads": m["heads"], "n_kv_heads": m["kv_heads"], "head_dim": m["dim"],
                 "value_dim": m["vdim"], "scale": float(m["scale"]), "window": None,
                 "chunk": None if mask is None else mask["size"], "qk_norm_eps": self.norm_eps, "qk_norm_scope": "head",
                 "prepare": "float32", "softmax_weights": "float32", "position": position},
                t(("q_proj", "q"), ("k_proj", "k"), ("v_proj", "v"), ("o_proj", "o"), ("q_norm", "q.norm"),
                  ("k_norm", "k.norm")))
        position = None
        if m["rot_dim"]:
            scaling = rot.get("scaling")
            position = PartSpec("rope", {"head_dim": m["rot_dim"], "rotary_dim": m["rot_dim"], "theta": float(rot["base"]),
                                         "layout": "interleaved", "frequency_precision": "float64",
                                         "scaling": None if scaling is None else {k: float(scaling[k]) for k in
                                                                                  ("factor", "original", "fast", "slow")}})
        return PartSpec(
            "latent_attention",
            {"hidden_size": self.width, "n_heads": m["heads"], "plain_dim": m["dim"], "rot_dim": m["rot_dim"],
             "value_dim": m["vdim"], "latent_rank": m["kv_rank"], "scale": float(m["scale"]),
             "window": None if mask is None else mask["size"], "norm_eps": self.norm_eps, "gated": True,
             "softmax_weights": "float32", "position": position},
            t(("q_proj", "q"), ("down_proj", "dkv"), ("latent_norm", "dkv.norm"), ("up_k", "uk"), ("up_v", "uv"),
              ("g_proj", "g"), ("o_proj", "o")))

    def _ffn(self, mlp: Mapping[str, Any], prefix: str) -> PartSpec:
        router = mlp["router"]
        groups = router.get("groups") or {"count": 1, "keep": 1}
        shared = mlp.get("shared")
        tensors = {"router": prefix + "mlp.router"}
        for e in range(router["experts"]):
            tensors[f"up.{e}"] = f"{prefix}mlp.e{e}.up"
            tensors[f"down.{e}"] = f"{prefix}mlp.e{e}.down"
        if shared is not None:
            tensors.update(shared_up=prefix + "mlp.shared.up", shared_down=prefix + "mlp.shared.down",
                           shared_gate=prefix + "mlp.shared.sg")
        return PartSpec(
            "routed_experts",
            {"hidden_size": self.width, "n_experts": router["experts"], "expert_ff": mlp["expert"]["ff"],
             "top": router["top"], "scale": float(router.get("scale", 1.0)), "groups": groups["count"],
             "keep": groups["keep"], "shared_ff": 0 if shared is None else shared["ff"], "shared_gated": True},
            tensors)

    def plan(self) -> ModelPlan:
        layers: List[LayerSpec] = []
        schedule: List[ScheduleEntry] = []
        for i, layer in enumerate(self.layers):
            prefix = f"l{i}."
            parts = dict(mixer=self._mixer(layer, prefix), norm_mixer=self._norm(prefix + "norm1"))
            if layer.get("mlp") is not None:
                parts.update(ffn=self._ffn(layer["mlp"], prefix), norm_ffn=self._norm(prefix + "norm2"))
            layers.append(LayerSpec.of("branch_norm", **parts))
            schedule.append(ScheduleEntry(layer=i, cache=i))
        return ModelPlan(
            hidden_size=self.width,
            vocab_size=self.vocab,
            embedding=PartSpec("embedding", {"vocab_size": self.vocab, "hidden_size": self.width,
                                             "scale": self.embedding_scale, "stream": "float32"}, {"weight": "embed"}),
            layers=tuple(layers),
            schedule=tuple(schedule),
            final_norm=self._norm("final.norm"),
            head=PartSpec("lm_head", {"vocab_size": self.vocab, "hidden_size": self.width, "tied": False},
                          {"weight": "head"}),
            max_positions=self.max_positions,
        )
