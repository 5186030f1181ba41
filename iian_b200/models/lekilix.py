"""Lekilix: typed configuration, layer description and tensor names.

A decoder-only model of parallel layers: one norm per layer whose output feeds the mixer and the feed-forward side by
side, ``x += mixer(h) + ff(h)``.  ``config.json`` lists the layers one by one (``layers``: ``type`` names the mixer,
``mixer`` its sizes, ``mlp`` the feed-forward or null) besides a few model-wide values (``vocab``, ``width``,
``norm.eps``, ``embedding.scale``, ``loop``).  Per layer:

* mixer ``attention``: attention whose values are its keys, with a norm of q and k over the whole projection, a partial
  rotation of interleaved pairs, a sliding window, a sink in the softmax and a sigmoid gate on the output
  (``iian_b200/parts/shared_kv_attention.py``);
* mixer ``mlstm``: the matrix-memory recurrence with capped gates and a state per request
  (``iian_b200/parts/matrix_memory.py``);
* feed-forward ``dense`` (gated, silu) or ``moe`` (experts chosen by a table indexed with the token id, equal weights on
  the outputs, a clamped activation; ``iian_b200/parts/experts.py``);
* the norm is an RMS norm whose stored weight sits around zero (``weight_offset`` 1).

``loop`` makes the layers ``start .. stop - 1`` run ``times`` times in a row with the same weights; every run has caches
and states of its own (the run order names a layer several times, each call with its own cache id) and begins with
``x <- Win [x ; e]``, ``e`` being what the embedding left (``iian_b200/parts/stream.py``).  The embedding is multiplied by
``embedding.scale``; the output is the model's norm and an untied head.  Positions have no stated limit.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Mapping, Optional, Tuple

from ..config.registry import Architecture, register_architecture
from ..config.spec import LayerCall, LayerSpec, ModelSpec, PartSpec
from .galodra import FeedForwardConfig, _get
from .qwen3 import ConfigError

MAX_POSITION = 1 << 24          # the design states no limit; angles are float64 products


@dataclass(frozen=True)
class AttentionMixerConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot_dims: int                  # how many of a head's entries rotate (0: none)
    rot_base: float
    window: Optional[int]          # keys visible to a query, itself included; None: all


@dataclass(frozen=True)
class MemoryMixerConfig:
    heads: int
    dim: int
    vdim: int
    gate_cap: float


@dataclass(frozen=True)
class ExpertsConfig(FeedForwardConfig):
    limit: float = 0.0


@dataclass(frozen=True)
class LekilixLayerConfig:
    type: str                      # "attention" | "mlstm"
    mixer: object
    mlp: Optional[FeedForwardConfig]


@dataclass(frozen=True)
class LoopConfig:
    start: int
    stop: int
    times: int


@dataclass(frozen=True)
class LekilixConfig:
    vocab: int
    width: int
    norm_eps: float
    embedding_scale: float
    layers: Tuple[LekilixLayerConfig, ...]
    loop: Optional[LoopConfig] = None
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

    def run_order(self) -> Tuple[Tuple[int, bool], ...]:
        """(layer, whether a run of the looped stretch starts here) in the order the layers run."""
        n = len(self.layers)
        if self.loop is None:
            return tuple((i, False) for i in range(n))
        lp = self.loop
        order = [(i, False) for i in range(lp.start)]
        for _ in range(lp.times):
            order += [(i, i == lp.start) for i in range(lp.start, lp.stop)]
        order += [(i, False) for i in range(lp.stop, n)]
        return tuple(order)


def _attention_from_dict(raw: Mapping[str, Any], where: str) -> AttentionMixerConfig:
    dim = _get(raw, "dim", int, where)
    vdim = _get(raw, "vdim", int, where)
    if vdim != dim:
        raise ConfigError(f"config.json: {where} has values of size {vdim} but keys of size {dim}: the values are the keys")
    rot = raw.get("rot")
    rot_dims, base = 0, 10000.0
    if rot is not None:
        rot_dims = _get(rot, "dims", int, where + " rot")
        base = _get(rot, "base", float, where + " rot")
        if rot_dims % 2 or rot_dims > dim:
            raise ConfigError(f"config.json: {where} rot.dims must be even and at most dim ({dim}), got {rot_dims}")
    mask = raw.get("mask")
    window = _get(mask, "size", int, where + " mask", optional=True) if mask is not None else None
    heads = _get(raw, "heads", int, where)
    kv_heads = _get(raw, "kv_heads", int, where)
    if heads % kv_heads:
        raise ConfigError(f"config.json: {where} has {heads} heads for {kv_heads} key/value heads")
    return AttentionMixerConfig(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=_get(raw, "scale", float, where),
                                rot_dims=rot_dims, rot_base=base, window=window)


def _memory_from_dict(raw: Mapping[str, Any], where: str) -> MemoryMixerConfig:
    cap = _get(raw, "gate_cap", float, where)
    if cap <= 0:
        raise ConfigError(f"config.json: {where} gate_cap must be positive, got {cap}")
    return MemoryMixerConfig(heads=_get(raw, "heads", int, where), dim=_get(raw, "dim", int, where),
                             vdim=_get(raw, "vdim", int, where), gate_cap=cap)


def _mlp_from_dict(raw: Optional[Mapping[str, Any]], where: str) -> Optional[FeedForwardConfig]:
    if raw is None:
        return None
    kind = raw.get("kind") if isinstance(raw, Mapping) else None
    if kind == "dense":
        return FeedForwardConfig("dense", _get(raw, "ff", int, where))
    if kind == "moe":
        expert = _get(raw, "expert", dict, where)
        router = _get(raw, "router", dict, where)
        experts, top = _get(router, "experts", int, where + " router"), _get(router, "top", int, where + " router")
        if top > experts:
            raise ConfigError(f"config.json: {where} router takes {top} of {experts} experts")
        limit = _get(expert, "limit", float, where + " expert")
        if limit <= 0:
            raise ConfigError(f"config.json: {where} expert limit must be positive, got {limit}")
        return ExpertsConfig("moe", _get(expert, "ff", int, where + " expert"), experts, top, limit)
    raise ConfigError(f"config.json: {where} has unknown kind {kind!r} (dense, moe)")


def lekilix_config_from_dict(raw: Mapping[str, Any]) -> LekilixConfig:
    layers_raw = raw.get("layers")
    if not isinstance(layers_raw, list) or not layers_raw:
        raise ConfigError("config.json: 'layers' must be a non-empty list")
    layers = []
    for i, lr in enumerate(layers_raw):
        where = f"layer {i}"
        kind = lr.get("type") if isinstance(lr, Mapping) else None
        mixer_raw = _get(lr, "mixer", dict, where) if isinstance(lr, Mapping) else None
        if kind == "attention":
            mixer = _attention_from_dict(mixer_raw, where + " mixer")
        elif kind == "mlstm":
            mixer = _memory_from_dict(mixer_raw, where + " mixer")
        else:
            raise ConfigError(f"config.json: {where} has unknown type {kind!r} (attention, mlstm)")
        layers.append(LekilixLayerConfig(kind, mixer, _mlp_from_dict(lr.get("mlp"), where + " mlp")))
    norm = _get(raw, "norm", dict, "the model")
    emb = raw.get("embedding")
    scale = _get(emb, "scale", float, "embedding") if emb is not None else 1.0
    loop = None
    if raw.get("loop") is not None:
        lr = _get(raw, "loop", dict, "the model")
        start, stop, times = lr.get("start"), lr.get("stop"), lr.get("times")
        for name, v in (("start", start), ("stop", stop), ("times", times)):
            if isinstance(v, bool) or not isinstance(v, int) or v < 0:
                raise ConfigError(f"config.json: loop '{name}' must be a non-negative integer, got {v!r}")
        if not start < stop <= len(layers) or times < 1:
            raise ConfigError(f"config.json: loop runs layers {start} .. {stop} - 1 {times} times; the model has {len(layers)} layers")
        loop = LoopConfig(start, stop, times)
    eos = raw.get("eos_token_id")
    eos_ids = () if eos is None else (eos,) if isinstance(eos, int) else tuple(eos)
    return LekilixConfig(vocab=_get(raw, "vocab", int, "the model"), width=_get(raw, "width", int, "the model"),
                         norm_eps=_get(norm, "eps", float, "norm"), embedding_scale=scale, layers=tuple(layers), loop=loop,
                         eos_token_ids=eos_ids)


@register_architecture
class Lekilix(Architecture):
    name = "Lekilix"

    def load_config(self, raw: Mapping[str, Any]) -> LekilixConfig:
        return lekilix_config_from_dict(raw)

    def config_to_dict(self, c: LekilixConfig) -> Dict[str, Any]:
        layers = []
        for lc in c.layers:
            m = lc.mixer
            if lc.type == "attention":
                mixer: Dict[str, Any] = {"heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "scale": m.scale}
                if m.rot_dims:
                    mixer["rot"] = {"dims": m.rot_dims, "base": m.rot_base}
                if m.window is not None:
                    mixer["mask"] = {"size": m.window}
            else:
                mixer = {"heads": m.heads, "dim": m.dim, "vdim": m.vdim, "gate_cap": m.gate_cap}
            if lc.mlp is None:
                mlp = None
            elif lc.mlp.kind == "dense":
                mlp = {"kind": "dense", "ff": lc.mlp.ff}
            else:
                mlp = {"kind": "moe", "expert": {"ff": lc.mlp.ff, "limit": lc.mlp.limit},
                       "router": {"experts": lc.mlp.experts, "top": lc.mlp.top}}
            layers.append({"type": lc.type, "mixer": mixer, "mlp": mlp})
        d: Dict[str, Any] = {"architecture": self.name, "vocab": c.vocab, "width": c.width, "norm": {"eps": c.norm_eps},
                             "embedding": {"scale": c.embedding_scale}, "layers": layers}
        if c.loop is not None:
            d["loop"] = {"start": c.loop.start, "stop": c.loop.stop, "times": c.loop.times}
        if c.eos_token_ids:
            d["eos_token_id"] = list(c.eos_token_ids)
        return d

    def build_spec(self, c: LekilixConfig) -> ModelSpec:
        def norm() -> PartSpec:
            return PartSpec("rms_norm", {"size": c.width, "eps": c.norm_eps, "weight_offset": 1.0})

        layers = []
        for lc in c.layers:
            m = lc.mixer
            if lc.type == "attention":
                position = (PartSpec("rotary", {"dim": m.rot_dims, "base": m.rot_base, "style": "interleaved",
                                                "max_position": MAX_POSITION}) if m.rot_dims else PartSpec("none"))
                mixer = PartSpec("shared_kv_attention", {
                    "hidden_size": c.width, "num_heads": m.heads, "num_kv_heads": m.kv_heads, "head_dim": m.dim,
                    "scale": m.scale, "window": m.window, "qk_norm": True, "qk_norm_eps": c.norm_eps, "sink": True,
                    "output_gate": True, "position": position})
            else:
                mixer = PartSpec("matrix_memory", {"hidden_size": c.width, "num_heads": m.heads, "dim": m.dim, "v_dim": m.vdim,
                                                   "gate_cap": m.gate_cap, "norm_eps": c.norm_eps, "output_gate": True})
            ffn = None
            if lc.mlp is not None:
                if lc.mlp.kind == "dense":
                    ffn = PartSpec("gated_mlp", {"hidden_size": c.width, "intermediate_size": lc.mlp.ff, "activation": "silu",
                                                 "names": ("gate", "up", "down")})
                else:
                    ffn = PartSpec("routed_experts", {"hidden_size": c.width, "num_experts": lc.mlp.experts, "top": lc.mlp.top,
                                                      "intermediate_size": lc.mlp.ff, "activation": "clamped_swish",
                                                      "limit": lc.mlp.limit, "score": "table", "vocab_size": c.vocab,
                                                      "weight_on": "output"})
            layers.append(LayerSpec(mixer=mixer, feed_forward=ffn, mixer_norm=norm(), arrangement="parallel_residual"))
        stream_parts = (PartSpec("reinject_embedding", {"hidden_size": c.width}),) if c.loop is not None else ()
        order = tuple(LayerCall(layer=i, cache=idx, before=0 if starts else None)
                      for idx, (i, starts) in enumerate(c.run_order()))           # every run of a layer has a cache of its own
        return ModelSpec(
            hidden_size=c.width, vocab_size=c.vocab, max_position=MAX_POSITION,
            embedding=PartSpec("token_embedding", {"vocab_size": c.vocab, "hidden_size": c.width, "scale": c.embedding_scale}),
            layers=tuple(layers), order=order, final_norm=norm(),
            head=PartSpec("lm_head", {"hidden_size": c.width, "vocab_size": c.vocab, "tied": False}),
            stream_parts=stream_parts)

    def tensor_name(self, scope: tuple, local: str) -> str:
        if scope[0] == "embedding":
            return "embed"
        if scope[0] == "final_norm":
            return "final.norm"
        if scope[0] == "head":
            return "head"
        if scope[0] == "stream":
            return "loop.in"
        if scope[0] == "layer":
            i, slot = scope[1], scope[2]
            if slot == "mixer":
                return f"l{i}.mix.{local}"
            if slot == "feed_forward":
                return f"l{i}.mlp.{local}"
            if slot == "mixer_norm":
                return f"l{i}.norm1"
        raise KeyError(scope)
