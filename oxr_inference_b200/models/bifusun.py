"""Bifusun: a pre-norm decoder whose config.json lists its layers one by one, from typed config to a description made of registered parts.

Every layer is ``x += mixer(norm1(x))`` and, unless its ``mlp`` is null, ``x += ff(norm2(x))``. The mixer of a layer is ``attention``
(grouped-query softmax attention without rotation: projections with biases, a short causal convolution on every channel of q, k and v,
a query temperature that grows with the position, and, where ``v_mix`` is set, values blended with those of the first such layer) or
``mlstm`` (the matrix-memory recurrence of xLSTM). The feed-forward routes each token to ``top`` of ``experts`` small relu-squared
layers, chosen among the best ``groups.keep`` of ``groups.count`` groups of neighbouring experts by sigmoid scores. The embedding and
the logits are scaled.

Tensor names: ``embed``, ``head``, ``final.norm``, and per layer ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.mix.*`` and
``l<i>.mlp.{router, e<j>.up, e<j>.down}``.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping

from oxr_inference_b200.config.model_config import ConfigError
from oxr_inference_b200.config.registry import Architecture, register_architecture
from oxr_inference_b200.parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

MAX_POSITIONS = 1 << 20
"""The design has no table over positions and config.json gives no limit; this bounds a request's length for the scheduler."""
VALUE_MIX_KEY = "bifusun_first_values"


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
class BifusunLayer:
    type: str
    mixer: Mapping[str, Any]
    mlp: Mapping[str, Any] | None


@dataclass(frozen=True)
class BifusunConfig:
    width: int
    vocab: int
    eps: float
    embedding_scale: float
    logit_scale: float
    layers: tuple[BifusunLayer, ...]
    eos_token_ids: tuple[int, ...] = ()
    architecture: str = "Bifusun"

    @staticmethod
    def from_dict(raw: Mapping[str, Any], generation: Mapping[str, Any] | None = None) -> "BifusunConfig":
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
            if mlp is not None and _need(mlp, "kind", where + ".mlp") != "moe":
                raise ConfigError(f"config.json: {where}.mlp.kind {mlp['kind']!r} is not implemented (moe is)")
            layers.append(BifusunLayer(kind, dict(_need(entry, "mixer", where)), dict(mlp) if mlp is not None else None))
        eos = raw.get("eos_token_id", [])
        if generation is not None and generation.get("eos_token_id") is not None:
            eos = generation["eos_token_id"]
        eos = [] if eos is None else (list(eos) if isinstance(eos, list) else [eos])
        config = BifusunConfig(
            width=_pos_int(raw, "width", "the top level"), vocab=_pos_int(raw, "vocab", "the top level"),
            eps=float(_need(_need(raw, "norm", "the top level"), "eps", "norm")),
            embedding_scale=float((raw.get("embedding") or {}).get("scale", 1.0)), logit_scale=float(raw.get("logit_scale", 1.0)),
            layers=tuple(layers), eos_token_ids=tuple(int(t) for t in eos), architecture=str(raw.get("architecture", "Bifusun")))
        bifusun_model_spec(config)   # sizes that do not fit each other are config errors, found here
        return config


# ---- one function per mixer kind: config.json's mixer entry -> mixer part
def _attention(c: BifusunConfig, m: Mapping[str, Any], prefix: str, blending: str | None) -> PartSpec:
    where = prefix + "mixer"
    temp = m.get("q_temp") or {}
    params = {"hidden_size": c.width, "num_heads": _pos_int(m, "heads", where), "num_kv_heads": _pos_int(m, "kv_heads", where),
              "key_dim": _pos_int(m, "dim", where), "value_dim": _pos_int(m, "vdim", where), "scale": float(_need(m, "scale", where)),
              "biases": True, "conv_taps": int(m.get("conv", 0) or 0),
              "temp_coef": float(_need(temp, "coef", where + ".q_temp")) if temp else 0.0,
              "temp_every": _pos_int(temp, "every", where + ".q_temp") if temp else 0,
              "value_mix": blending, "value_mix_key": VALUE_MIX_KEY}
    if params["num_heads"] % params["num_kv_heads"]:
        raise ConfigError(f"config.json: {where}: {params['num_heads']} heads are not a multiple of {params['num_kv_heads']} kv_heads")
    if params["conv_taps"] < 0:
        raise ConfigError(f"config.json: {where}.conv must not be negative")
    return PartSpec("masked_attention", params, prefix=prefix + "mix.")


def _mlstm(c: BifusunConfig, m: Mapping[str, Any], prefix: str, blending: str | None) -> PartSpec:
    where = prefix + "mixer"
    params = {"hidden_size": c.width, "num_heads": _pos_int(m, "heads", where), "key_dim": _pos_int(m, "dim", where),
              "value_dim": _pos_int(m, "vdim", where), "gate_cap": float(_need(m, "gate_cap", where)), "eps": c.eps}
    if not params["gate_cap"] > 0:
        raise ConfigError(f"config.json: {where}.gate_cap must be positive")
    return PartSpec("mlstm", params, prefix=prefix + "mix.")


_MIXERS = {"attention": _attention, "mlstm": _mlstm}


def _experts(c: BifusunConfig, mlp: Mapping[str, Any], prefix: str) -> PartSpec:
    where = prefix + "mlp"
    router = _need(mlp, "router", where)
    groups = router.get("groups") or {}
    params = {"hidden_size": c.width, "intermediate_size": _pos_int(_need(mlp, "expert", where), "ff", where + ".expert"),
              "experts": _pos_int(router, "experts", where + ".router"), "top": _pos_int(router, "top", where + ".router"),
              "groups": _pos_int(groups, "count", where + ".router.groups") if groups else 1,
              "keep": _pos_int(groups, "keep", where + ".router.groups") if groups else 1,
              "scale": float(router.get("scale", 1.0))}
    E, G, K, top = params["experts"], params["groups"], params["keep"], params["top"]
    if E % G or K > G or top > K * (E // G):
        raise ConfigError(f"config.json: {where}.router: {top} of {E} experts in {K} of {G} groups do not fit each other")
    return PartSpec("routed_experts", params, prefix=prefix + "mlp.")


def bifusun_model_spec(c: BifusunConfig) -> ModelSpec:
    def norm(name: str) -> PartSpec:
        return PartSpec("rms_norm", {"size": c.width, "eps": c.eps}, prefix=name, names={"weight": ""})

    layers = []
    kept_width = None    # heads x size of the values that the first blending layer keeps for the later ones
    for i, layer in enumerate(c.layers):
        p = f"l{i}."
        blending = None
        if layer.type == "attention" and layer.mixer.get("v_mix"):
            width = (layer.mixer.get("kv_heads"), layer.mixer.get("vdim"))
            if kept_width is None:
                blending, kept_width = "keep", width
            elif width != kept_width:
                raise ConfigError(f"config.json: layers[{i}] blends its values with the first blending layer's, whose key/value heads and value "
                                  f"size {kept_width} differ from its {width}")
            else:
                blending = "blend"
        mixer = _MIXERS[layer.type](c, layer.mixer, p, blending)
        ff = ff_norm = None
        if layer.mlp is not None:
            ff, ff_norm = _experts(c, layer.mlp, p), norm(p + "norm2")
        layers.append(LayerSpec(mixer=mixer, mixer_norm=norm(p + "norm1"), feed_forward=ff, feed_forward_norm=ff_norm, arrangement="pre_norm"))
    return ModelSpec(
        architecture=c.architecture, hidden_size=c.width, vocab_size=c.vocab,
        embedding=PartSpec("token_embedding", {"vocab_size": c.vocab, "hidden_size": c.width, "scale": c.embedding_scale, "whole_stream": True},
                           prefix="embed", names={"weight": ""}),
        layers=tuple(layers), schedule=tuple(ScheduleEntry(i) for i in range(len(layers))),
        final_norm=norm("final.norm"),
        head=PartSpec("linear_head", {"vocab_size": c.vocab, "hidden_size": c.width, "tied": False, "scale": c.logit_scale}, prefix="head",
                      names={"weight": ""}),
        max_positions=MAX_POSITIONS, eos_token_ids=c.eos_token_ids,
        # tensors a checkpoint may carry for layers that do not use them (a blending weight where nothing is blended, the second norm of
        # a layer without a feed-forward); names that a part claims are never matched against these
        ignored_tensors=(r"l\d+\.mix\.vmix", r"l\d+\.norm2"))


BIFUSUN = register_architecture(Architecture("Bifusun", BifusunConfig.from_dict, bifusun_model_spec))
