"""Small Bifusun configurations and model folders for the tests: sizes unlike any real model's, values that differ where a coincidence
(heads == kv_heads, key size == value size, one group, top == 1) would hide a fault, and weights reshaped so that faults show."""

from __future__ import annotations

import json
from pathlib import Path

import torch


def moe(ff=24, experts=6, top=2, count=3, keep=2, scale=1.7):
    router = {"experts": experts, "top": top, "scale": scale}
    if count:
        router["groups"] = {"count": count, "keep": keep}
    return {"kind": "moe", "expert": {"ff": ff}, "router": router}


def attention_layer(heads=4, kv_heads=2, dim=16, vdim=24, conv=3, coef=0.4, every=7, scale=0.3, v_mix=False, mlp=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if conv:
        m["conv"] = conv
    if every:
        m["q_temp"] = {"coef": coef, "every": every}
    if v_mix:
        m["v_mix"] = True
    return {"type": "attention", "mixer": m, "mlp": mlp}


def mlstm_layer(heads=2, dim=16, vdim=24, cap=9.0, mlp=None):
    return {"type": "mlstm", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}, "mlp": mlp}


def model_config(layers, width=48, vocab=131, eps=1e-5, scale=3.0, logit_scale=0.5):
    return {"architecture": "Bifusun", "embedding": {"scale": scale}, "layers": layers, "logit_scale": logit_scale, "norm": {"eps": eps},
            "vocab": vocab, "width": width}


# Three whole models that differ in every size and option.
MODEL_P = model_config([attention_layer(v_mix=True, mlp=moe()), mlstm_layer(mlp=moe(ff=16, experts=8, top=3, count=4, keep=3, scale=0.8)),
                        attention_layer(v_mix=True, conv=2, every=5, coef=0.9), attention_layer(dim=16, vdim=16, kv_heads=4, conv=4, every=0),
                        attention_layer(v_mix=True, heads=2, kv_heads=2, dim=8, scale=0.5, mlp=moe(count=0, top=1)), mlstm_layer(heads=3, dim=8, vdim=16)])
MODEL_Q = model_config([mlstm_layer(heads=3, dim=40, vdim=24, cap=5.0, mlp=moe(ff=40, experts=4, top=4, count=2, keep=2, scale=1.0)),
                        attention_layer(heads=4, kv_heads=1, dim=64, vdim=64, conv=4, every=16, v_mix=True, scale=0.11,
                                        mlp=moe(ff=8, experts=10, top=3, count=10, keep=5, scale=2.2)),
                        attention_layer(heads=2, kv_heads=1, dim=64, vdim=64, conv=1, every=3, coef=0.25, v_mix=True, scale=0.2)],
                       width=64, vocab=200, eps=1e-6, scale=0.9, logit_scale=2.0)
MODEL_R = model_config([attention_layer(heads=6, kv_heads=3, dim=32, vdim=32, conv=0, every=1, coef=0.15, mlp=moe(ff=32, experts=9, top=2, count=3, keep=1)),
                        mlstm_layer(heads=1, dim=70, vdim=40, cap=15.0, mlp=moe(ff=12, experts=5, top=2, count=1, keep=1, scale=3.0))],
                       width=40, vocab=97, scale=1.0, logit_scale=1.0)


def make_folder(tmp: Path, config: dict, name: str, seed: int = 0, sharpen: float = 8.0) -> Path:
    """A model folder with random bfloat16 weights, then reshaped so that faults show: query and key weights of the attention layers are
    scaled up (peaked attention: a lost, doubled or wrongly placed key changes the output), biases, filters and blending weights get a
    visible size, the forget gates lean open (a long memory: a lost state shows many tokens later), the routers' scores are spread out."""
    from safetensors.torch import load_file, save_file

    from oxr_inference_b200.weights import write_random_model

    folder = write_random_model(config, tmp / name, seed, dtype="bfloat16", std=0.06)
    path = folder / "model.safetensors"
    tensors = load_file(str(path))
    kinds = {f"l{i}.": layer["type"] for i, layer in enumerate(config["layers"])}
    for k, t in tensors.items():
        f = t.float()
        kind = kinds.get(k.split("mix.")[0], "")
        if k.endswith((".mix.q", ".mix.k")) and kind == "attention":
            f = f * sharpen ** 0.5
        elif k.endswith((".mix.q", ".mix.k", ".mix.v")) and kind == "mlstm":
            f = f * 3
        elif k.endswith(".conv"):
            f = f * 6 + 0.3
        elif k.endswith((".q.b", ".k.b", ".v.b", ".o.b")):
            f = f * 5
        elif k.endswith(".vmix"):
            f = 0.35 + f * 2
        elif k.endswith(".f.b"):
            f = f * 20 + 3.0
        elif k.endswith((".mix.i", ".mix.f", ".i.b")):
            f = f * 10
        elif k.endswith(".router"):
            f = f * 3
        elif k.endswith(("head", "embed")):
            f = f * 4
        tensors[k] = f.to(t.dtype)
    save_file(tensors, str(path), metadata={"format": "pt"})
    (folder / "config.json").write_text(json.dumps(config, indent=1))
    return folder


def tokens(config: dict, n: int, seed: int) -> list[int]:
    g = torch.Generator().manual_seed(seed * 104729 + n)
    return torch.randint(0, config["vocab"], (n,), generator=g).tolist()


_cache: dict = {}


def plain_logits(folder: Path, ids: list[int]) -> torch.Tensor:
    from plain import bifusun_plain as BP

    key = (str(folder), tuple(ids))
    if key not in _cache:
        if str(folder) not in _cache:
            _cache[str(folder)] = BP.read_model(folder, torch.float64)
        cfg, w = _cache[str(folder)]
        margins: list = []
        _cache[key] = BP.forward(cfg, w, ids, margins=margins).float()
        _cache[("margin",) + key] = torch.stack(margins).min(0).values.float() if margins else torch.full((len(ids),), float("inf"))
    return _cache[key]


def router_margins(folder: Path, ids: list[int]) -> torch.Tensor:
    """Per position, the smallest margin by which any layer's router decided (``inf`` without routers)."""
    plain_logits(folder, ids)
    return _cache[("margin", str(folder), tuple(ids))]
