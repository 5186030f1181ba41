"""Galodra: typed configuration, layer description and tensor names.

A decoder-only model of post-norm layers.  ``config.json`` lists the layers one by one (``layers``: ``type`` names the
mixer, ``mixer`` its sizes, ``mlp`` the feed-forward or null); everything else is a handful of model-wide constants
(``vocab``, ``width``, ``norm.eps``, ``postln_alpha``).  Per layer:

* mixer ``latent_attention``: attention over a cached low-rank latent with a shared rotated key part, a sink in the
  softmax's denominator and a sliding window (``iian_b200/parts/latent_attention.py``);
* feed-forward ``dense`` (gated, tanh-form gelu) or ``moe`` (sigmoid-routed experts with silu whose weight scales the
  expert's input; ``iian_b200/parts/experts.py``);
* arrangement ``post_norm_residual`` with a sigmoid gate on each sub-layer's output, a scaled skip path, LayerNorm with
  weight and bias after each sum, and a learned mix over the embedding output and all layer results as what the next
  layer reads (``iian_b200/parts/block.py``).

The output is the model's LayerNorm and the embedding table as the head.  Positions have no stated limit.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Mapping, Optional, Tuple

from ..config.registry import Architecture, register_architecture
from ..config.spec import LayerCall, LayerSpec, ModelSpec, PartSpec
from .qwen3 import ConfigError

MAX_POSITION = 1 << 24          # the design states no limit; angles are computed from float64 products


def _get(raw: Mapping[str, Any], key: str, kind, where: str, optional: bool = False):
    val = raw.get(key) if isinstance(raw, Mapping) else None
    if val is None:
        if optional:
            return None
        raise ConfigError(f"config.json: {where} lacks '{key}'")
    if kind is int:
        if isinstance(val, bool) or not isinstance(val, int) or val <= 0:
            raise ConfigError(f"config.json: {where} '{key}' must be a positive integer, got {val!r}")
    elif kind is float:
        if isinstance(val, bool) or not isinstance(val, (int, float)):
            raise ConfigError(f"config.json: {where} '{key}' must be a number, got {val!r}")
        val = float(val)
    elif kind is dict:
        if not isinstance(val, Mapping):
            raise ConfigError(f"config.json: {where} '{key}' must be an object")
    return val


@dataclass(frozen=True)
class LatentMixerConfig:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    scale: float
    rot_dims: int                  # how many of the rot_dim entries rotate (0: none)
    rot_base: float
    window: Optional[int]          # keys visible to a query, itself included; None: all


@dataclass(frozen=True)
class FeedForwardConfig:
    kind: str                      # "dense" | "moe"
    ff: int                        # intermediate size (of one expert for "moe")
    experts: int = 0
    top: int = 0


@dataclass(frozen=True)
class GalodraLayerConfig:
    type: str
    mixer: LatentMixerConfig
    mlp: Optional[FeedForwardConfig]


@dataclass(frozen=True)
class GalodraConfig:
    vocab: int
    width: int
    norm_eps: float
    postln_alpha: float
    layers: Tuple[GalodraLayerConfig, ...]
    eos_token_ids: Tuple[int, ...] = ()

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)


def _mixer_from_dict(raw: Mapping[str, Any], where: str) -> LatentMixerConfig:
    rot = raw.get("rot")
    rot_dim = _get(raw, "rot_dim", int, where)
    rot_dims, base = 0, 10000.0
    if rot is not None:
        rot_dims = _get(rot, "dims", int, where + " rot")
        base = _get(rot, "base", float, where + " rot")
        if rot_dims % 2 or rot_dims > rot_dim:
            raise ConfigError(f"config.json: {where} rot.dims must be even and at most rot_dim ({rot_dim}), got {rot_dims}")
    mask = raw.get("mask")
    window = _get(mask, "size", int, where + " mask", optional=True) if mask is not None else None
    return LatentMixerConfig(
        heads=_get(raw, "heads", int, where), dim=_get(raw, "dim", int, where), rot_dim=rot_dim,
        vdim=_get(raw, "vdim", int, where), kv_rank=_get(raw, "kv_rank", int, where),
        scale=_get(raw, "scale", float, where), rot_dims=rot_dims, rot_base=base, window=window)


def _mlp_from_dict(raw: Optional[Mapping[str, Any]], where: str) -> Optional[FeedForwardConfig]:
    if raw is None:
        return None
    kind = raw.get("kind")
    if kind == "dense":
        return FeedForwardConfig("dense", _get(raw, "ff", int, where))
    if kind == "moe":
        expert = _get(raw, "expert", dict, where)
        router = _get(raw, "router", dict, where)
        experts, top = _get(router, "experts", int, where + " router"), _get(router, "top", int, where + " router")
        if top > experts:
            raise ConfigError(f"config.json: {where} router takes {top} of {experts} experts")
        return FeedForwardConfig("moe", _get(expert, "ff", int, where + " expert"), experts, top)
    raise ConfigError(f"config.json: {where} has unknown kind {kind!r} (dense, moe)")


def galodra_config_from_dict(raw: Mapping[str, Any]) -> GalodraConfig:
    layers_raw = raw.get("layers")
    if not isinstance(layers_raw, list) or not layers_raw:
        raise ConfigError("config.json: 'layers' must be a non-empty list")
    layers = []
    for i, lr in enumerate(layers_raw):
        where = f"layer {i}"
        kind = lr.get("type") if isinstance(lr, Mapping) else None
        if kind != "latent_attention":
            raise ConfigError(f"config.json: {where} has unknown type {kind!r} (latent_attention)")
        layers.append(GalodraLayerConfig(kind, _mixer_from_dict(_get(lr, "mixer", dict, where), where + " mixer"),
                                         _mlp_from_dict(lr.get("mlp"), where + " mlp")))
    norm = _get(raw, "norm", dict, "the model")
    eos = raw.get("eos_token_id")
    eos_ids = () if eos is None else (eos,) if isinstance(eos, int) else tuple(eos)
    return GalodraConfig(vocab=_get(raw, "vocab", int, "the model"), width=_get(raw, "width", int, "the model"),
                         norm_eps=_get(norm, "eps", float, "norm"), postln_alpha=_get(raw, "postln_alpha", float, "the model"),
                         layers=tuple(layers), eos_token_ids=eos_ids)


@register_architecture
class Galodra(Architecture):
    name = "Galodra"

    def load_config(self, raw: Mapping[str, Any]) -> GalodraConfig:
        return galodra_config_from_dict(raw)

    def config_to_dict(self, c: GalodraConfig) -> Dict[str, Any]:
        layers = []
        for lc in c.layers:
            m = lc.mixer
            mixer: Dict[str, Any] = {"heads": m.heads, "dim": m.dim, "rot_dim": m.rot_dim, "vdim": m.vdim, "kv_rank": m.kv_rank,
                                     "scale": m.scale}
            if m.rot_dims:
                mixer["rot"] = {"dims": m.rot_dims, "base": m.rot_base}
            if m.window is not None:
                mixer["mask"] = {"size": m.window}
            if lc.mlp is None:
                mlp = None
            elif lc.mlp.kind == "dense":
                mlp = {"kind": "dense", "ff": lc.mlp.ff}
            else:
                mlp = {"kind": "moe", "expert": {"ff": lc.mlp.ff}, "router": {"experts": lc.mlp.experts, "top": lc.mlp.top}}
            layers.append({"type": lc.type, "mixer": mixer, "mlp": mlp})
        d: Dict[str, Any] = {"architecture": self.name, "vocab": c.vocab, "width": c.width, "norm": {"eps": c.norm_eps},
                             "postln_alpha": c.postln_alpha, "layers": layers}
        if c.eos_token_ids:
            d["eos_token_id"] = list(c.eos_token_ids)
        return d

    def build_spec(self, c: GalodraConfig) -> ModelSpec:
        def norm() -> PartSpec:
            return PartSpec("layer_norm", {"size": c.width, "eps": c.norm_eps})

        layers = []
        for i, lc in enumerate(c.layers):
            m = lc.mixer
            position = (PartSpec("rotary", {"dim": m.rot_dims, "base": m.rot_base, "style": "neox", "max_position": MAX_POSITION})
                        if m.rot_dims else PartSpec("none"))
            mixer = PartSpec("latent_attention", {
                "hidden_size": c.width, "num_heads": m.heads, "dim": m.dim, "rot_dim": m.rot_dim, "v_dim": m.vdim,
                "kv_rank": m.kv_rank, "scale": m.scale, "norm_eps": c.norm_eps, "window": m.window, "sink": True,
                "position": position})
            extra = [("alpha", PartSpec("constant", {"value": c.postln_alpha})),
                     ("mixer_gate", PartSpec("sigmoid_gate", {"size": c.width})),
                     ("depth_mix", PartSpec("depth_mix", {"terms": i + 2}))]
            ffn = None
            if lc.mlp is not None:
                extra.append(("feed_forward_gate", PartSpec("sigmoid_gate", {"size": c.width})))
                if lc.mlp.kind == "dense":
                    ffn = PartSpec("gated_mlp", {"hidden_size": c.width, "intermediate_size": lc.mlp.ff,
                                                 "activation": "gelu_tanh", "names": ("gate", "up", "down")})
                else:
                    ffn = PartSpec("routed_experts", {"hidden_size": c.width, "num_experts": lc.mlp.experts, "top": lc.mlp.top,
                                                      "intermediate_size": lc.mlp.ff, "activation": "silu", "score": "sigmoid",
                                                      "weight_on": "input"})
            layers.append(LayerSpec(mixer=mixer, feed_forward=ffn, mixer_norm=norm(),
                                    feed_forward_norm=norm() if ffn is not None else None,
                                    arrangement="post_norm_residual", extra=tuple(extra)))
        return ModelSpec(
            hidden_size=c.width, vocab_size=c.vocab, max_position=MAX_POSITION,
            embedding=PartSpec("token_embedding", {"vocab_size": c.vocab, "hidden_size": c.width}),
            layers=tuple(layers),
            order=tuple(LayerCall(layer=i, cache=i) for i in range(len(layers))),
            final_norm=norm(),
            head=PartSpec("lm_head", {"hidden_size": c.width, "vocab_size": c.vocab, "tied": True}))

    _LOCAL = {
        ("mixer_norm", "weight"): "norm1", ("mixer_norm", "bias"): "norm1.b",
        ("feed_forward_norm", "weight"): "norm2", ("feed_forward_norm", "bias"): "norm2.b",
        ("mixer_gate", "weight"): "rg1", ("mixer_gate", "bias"): "rg1.b",
        ("feed_forward_gate", "weight"): "rg2", ("feed_forward_gate", "bias"): "rg2.b",
        ("depth_mix", "weight"): "dwa",
    }

    def tensor_name(self, scope: tuple, local: str) -> str:
        if scope[0] == "embedding":
            return "embed"
        if scope[0] == "final_norm":
            return "final.norm" if local == "weight" else "final.norm.b"
        if scope[0] == "layer":
            i, slot = scope[1], scope[2]
            if slot == "mixer":
                return f"l{i}.mix.{local}"
            if slot == "feed_forward":
                return f"l{i}.mlp.{local}"
            return f"l{i}.{self._LOCAL[(slot, local)]}"
        raise KeyError(scope)
