"""Radapel: a decoder whose config.json lists its layers one by one, from typed config to a description made of registered parts.

Every layer is ``x += post_norm(mixer(pre_norm(x)))`` and, unless its ``mlp`` is null, ``x += post_norm(ff(pre_norm(x)))``. The mixer
of a layer is one of ``attention`` (grouped-query, chunk-masked, with a bucketed distance bias; no rotation), ``latent_attention``
(compressed key/value row, an interleaved rotary part, a sink in the softmax) and ``mamba2``. The feed-forward is a clamped gated unit.
``loop`` lets a stretch of layers run several times with the same weights; each pass has a cache or state of its own and is entered
through a linear map of [stream; embedding output] plus a per-pass vector. The embedding is scaled; the head is a tensor of its own.

Tensor names: ``embed``, ``head``, ``final.norm``, ``loop.in``, ``loop.step``, and per layer ``l<i>.norm1``, ``norm1b``, ``norm2``,
``norm2b``, ``l<i>.mix.*`` and ``l<i>.mlp.{gate,up,down}``.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping

from oxr_inference_b200.config.model_config import ConfigError
from oxr_inference_b200.config.registry import Architecture, register_architecture
from oxr_inference_b200.parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

MAX_POSITIONS = 1 << 20
"""The design has no table over positions and config.json gives no limit; this bounds a request's length for the scheduler."""
GATE_ALPHA = 1.702
"""Slope of the sigmoid that stands in for GELU in the feed-forward's gate; fixed by the design."""


def _need(d: Mapping[str, Any], key: str, where: str) -> Any:
    if not isinstance(d, Mapping) or key not in d:
        raise ConfigError(f"config.json: {where} lacks {key!r}")
    return d[key]


def _pos_int(d: Mapping[str, Any], key: str, where: str) -> int:
    v = _need(d, key, where)
    if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
        raise ConfigError(f"config.json: {where}.{key} must be a positive integer, got {v!r}")
    return v


@dataclass(frozen=True)
class RadapelLayer:
    type: str
    mixer: Mapping[str, Any]
    mlp: Mapping[str, Any] | None


@dataclass(frozen=True)
class RadapelConfig:
    width: int
    vocab: int
    eps: float
    embedding_scale: float
    layers: tuple[RadapelLayer, ...]
    loop_start: int
    loop_stop: int
    loop_times: int
    """0: no stretch of layers is repeated (config.json has no ``loop``)."""
    eos_token_ids: tuple[int, ...] = ()
    architecture: str = "Radapel"

    @staticmethod
    def from_dict(raw: Mapping[str, Any], generation: Mapping[str, Any] | None = None) -> "RadapelConfig":
        layers = []
        listed = _need(raw, "layers", "the top level")
        if not isinstance(listed, list) or not listed:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        for i, entry in enumerate(listed):
            where = f"layers[{i}]"
            kind = _need(entry, "type", where)
            if kind not in _MIXERS:
                raise ConfigError(f"config.json: {where}.type {kind!r} is not one of {sorted(_MIXERS)}")
            mlp = entry.get("mlp")
            if mlp is not None and _need(mlp, "kind", where + ".mlp") != "dense":
                raise ConfigError(f"config.json: {where}.mlp.kind {mlp['kind']!r} is not implemented (dense is)")
            layers.append(RadapelLayer(kind, dict(_need(entry, "mixer", where)), dict(mlp) if mlp is not None else None))
        loop = raw.get("loop")
        start = stop = times = 0
        if loop:
            times = _pos_int(loop, "times", "loop")
            start, stop = int(_need(loop, "start", "loop")), int(_need(loop, "stop", "loop"))
            if not 0 <= start < stop <= len(layers):
                raise ConfigError(f"config.json: loop {start}..{stop} does not lie within the {len(layers)} layers")
        eos = raw.get("eos_token_id", [])
        if generation is not None and generation.get("eos_token_id") is not None:
            eos = generation["eos_token_id"]
        eos = [] if eos is None else (list(eos) if isinstance(eos, list) else [eos])
        return RadapelConfig(
            width=_pos_int(raw, "width", "the top level"), vocab=_pos_int(raw, "vocab", "the top level"),
            eps=float(_need(_need(raw, "norm", "the top level"), "eps", "norm")),
            embedding_scale=float((raw.get("embedding") or {}).get("scale", 1.0)),
            layers=tuple(layers), loop_start=start, loop_stop=stop, loop_times=times,
            eos_token_ids=tuple(int(t) for t in eos), architecture=str(raw.get("architecture", "Radapel")))


# ---- one function per mixer kind: config.json's mixer entry -> (mixer part, position part or None)
def _attention(c: RadapelConfig, m: Mapping[str, Any], prefix: str):
    where = prefix + "mixer"
    mask = m.get("mask") or {}
    params = {"hidden_size": c.width, "num_heads": _pos_int(m, "heads", where), "num_kv_heads": _pos_int(m, "kv_heads", where),
              "key_dim": _pos_int(m, "dim", where), "value_dim": _pos_int(m, "vdim", where), "scale": float(_need(m, "scale", where)),
              "chunk": int(mask.get("size", 0) or 0), "bias_rows": 0, "bias_far": 0.0}
    if "bias_max" in m:
        params["bias_far"] = float(m["bias_max"])
        params["bias_rows"] = -1    # the table's height is the tensor's: filled in from the checkpoint's shape by the caller
    return PartSpec("masked_attention", params, prefix=prefix + "mix."), None


def _latent(c: RadapelConfig, m: Mapping[str, Any], prefix: str):
    where = prefix + "mixer"
    rot_dim = int(m.get("rot_dim", 0))
    position = None
    if rot_dim:
        rot = _need(m, "rot", where)
        position = PartSpec("rope_pairs", {"dims": _pos_int(rot, "dims", where + ".rot"), "base": float(_need(rot, "base", where + ".rot"))})
        if position.params["dims"] > rot_dim:
            raise ConfigError(f"config.json: {where}.rot.dims exceeds rot_dim")
    params = {"hidden_size": c.width, "num_heads": _pos_int(m, "heads", where), "key_dim": _pos_int(m, "dim", where), "rot_dim": rot_dim,
              "value_dim": _pos_int(m, "vdim", where), "rank": _pos_int(m, "kv_rank", where), "scale": float(_need(m, "scale", where)),
              "eps": c.eps, "sink": True}
    return PartSpec("latent_attention", params, prefix=prefix + "mix."), position


def _mamba2(c: RadapelConfig, m: Mapping[str, Any], prefix: str):
    where = prefix + "mixer"
    params = {"hidden_size": c.width, "num_heads": _pos_int(m, "heads", where), "value_dim": _pos_int(m, "vdim", where),
              "state": _pos_int(m, "state", where), "groups": _pos_int(m, "groups", where), "taps": _pos_int(m, "conv", where),
              "norm_groups": _pos_int(m, "norm_groups", where), "eps": c.eps}
    return PartSpec("mamba2", params, prefix=prefix + "mix."), None


_MIXERS = {"attention": _attention, "latent_attention": _latent, "mamba2": _mamba2}


def radapel_model_spec(c: RadapelConfig, tensor_shapes: Mapping[str, tuple[int, ...]] | None = None) -> ModelSpec:
    """``tensor_shapes`` (checkpoint name -> shape), when given, supplies the sizes that only a tensor's shape tells (the height of a
    distance-bias table); without it (random-weights mode) such a table takes the mixer entry's ``bias_rows`` if it has one, else
    :data:`DEFAULT_BIAS_ROWS`."""
    def norm(name: str) -> PartSpec:
        return PartSpec("rms_norm", {"size": c.width, "eps": c.eps}, prefix=name, names={"weight": ""})

    layers = []
    for i, layer in enumerate(c.layers):
        p = f"l{i}."
        mixer, position = _MIXERS[layer.type](c, layer.mixer, p)
        if mixer.params.get("bias_rows") == -1:
            shape = (tensor_shapes or {}).get(p + "mix.rel")
            mixer = PartSpec(mixer.kind, {**mixer.params, "bias_rows": int(shape[0]) if shape else int(layer.mixer.get("bias_rows", DEFAULT_BIAS_ROWS))},
                             prefix=mixer.prefix)
        ff = ff_norm = ff_post = None
        if layer.mlp is not None:
            ff = PartSpec("clamped_glu", {"hidden_size": c.width, "intermediate_size": _pos_int(layer.mlp, "ff", p + "mlp"),
                                          "limit": float(_need(layer.mlp, "limit", p + "mlp")), "alpha": GATE_ALPHA}, prefix=p + "mlp.")
            ff_norm, ff_post = norm(p + "norm2"), norm(p + "norm2b")
        layers.append(LayerSpec(mixer=mixer, mixer_norm=norm(p + "norm1"), feed_forward=ff, feed_forward_norm=ff_norm, arrangement="sandwich_norm",
                                position=position, mixer_post_norm=norm(p + "norm1b"), feed_forward_post_norm=ff_post))

    schedule, joints = [], ()
    n = len(c.layers)
    if c.loop_times:
        joints = (PartSpec("reentry_linear", {"hidden_size": c.width, "passes": c.loop_times}, prefix="loop."),)
        schedule += [ScheduleEntry(i) for i in range(c.loop_start)]
        for t in range(c.loop_times):   # every pass has a cache or state of its own: one schedule entry per run
            schedule += [ScheduleEntry(i, joint=0 if i == c.loop_start else None, joint_arg=t) for i in range(c.loop_start, c.loop_stop)]
        schedule += [ScheduleEntry(i) for i in range(c.loop_stop, n)]
    else:
        schedule = [ScheduleEntry(i) for i in range(n)]
    return ModelSpec(
        architecture=c.architecture, hidden_size=c.width, vocab_size=c.vocab,
        embedding=PartSpec("token_embedding", {"vocab_size": c.vocab, "hidden_size": c.width, "scale": c.embedding_scale, "whole_stream": True},
                           prefix="embed", names={"weight": ""}),
        layers=tuple(layers), schedule=tuple(schedule), joints=joints,
        final_norm=norm("final.norm"),
        head=PartSpec("linear_head", {"vocab_size": c.vocab, "hidden_size": c.width, "tied": False}, prefix="head", names={"weight": ""}),
        max_positions=MAX_POSITIONS, eos_token_ids=c.eos_token_ids)


DEFAULT_BIAS_ROWS = 16

RADAPEL = register_architecture(Architecture("Radapel", RadapelConfig.from_dict, radapel_model_spec, shapes_matter=True))
