"""Small Radapel configurations and model folders for the tests: sizes unlike any real model's, values that differ where a
coincidence (heads == kv_heads, one group, rot.dims == rot_dim) would hide a fault, and weights reshaped so that faults show."""

from __future__ import annotations

import json
from pathlib import Path

import torch


def attention_layer(heads=4, kv_heads=2, dim=16, vdim=24, chunk=10, bias_max=40, bias_rows=12, scale=0.3, mlp=(40, 0.8)):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if chunk:
        m["mask"] = {"size": chunk}
    if bias_max:
        m.update(bias_max=bias_max, bias_rows=bias_rows)
    return {"type": "attention", "mixer": m, "mlp": {"kind": "dense", "ff": mlp[0], "limit": mlp[1]} if mlp else None}


def latent_layer(heads=2, dim=16, rot_dim=8, rot_dims=8, base=500.0, vdim=12, kv_rank=24, scale=0.25, mlp=(56, 1.5)):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "rot": {"dims": rot_dims, "base": base}, "vdim": vdim, "kv_rank": kv_rank, "scale": scale}
    return {"type": "latent_attention", "mixer": m, "mlp": {"kind": "dense", "ff": mlp[0], "limit": mlp[1]} if mlp else None}


def mamba_layer(heads=4, vdim=8, state=16, groups=2, conv=3, norm_groups=2, mlp=None):
    m = {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv, "norm_groups": norm_groups}
    return {"type": "mamba2", "mixer": m, "mlp": {"kind": "dense", "ff": mlp[0], "limit": mlp[1]} if mlp else None}


def model_config(layers, width=48, vocab=131, eps=1e-5, scale=0.7, loop=None):
    cfg = {"architecture": "Radapel", "embedding": {"scale": scale}, "layers": layers, "norm": {"eps": eps}, "vocab": vocab, "width": width}
    if loop:
        cfg["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return cfg


# Three whole models that differ in every size and option.
MODEL_X = model_config([mamba_layer(), attention_layer(), latent_layer(rot_dims=4), attention_layer(kv_heads=4, chunk=0, bias_rows=6, bias_max=9.5)],
                       loop=(1, 3, 3))
MODEL_Y = model_config([latent_layer(heads=3, dim=8, rot_dim=16, rot_dims=16, vdim=16, kv_rank=40, mlp=None),
                        attention_layer(heads=6, kv_heads=2, dim=16, vdim=16, chunk=7, bias_max=0, mlp=(24, 0.5)),
                        mamba_layer(heads=6, vdim=16, state=40, groups=3, conv=2, norm_groups=3, mlp=(72, 2.0))], width=64, vocab=200, eps=1e-6, scale=1.3)
MODEL_Z = model_config([attention_layer(heads=2, kv_heads=1, dim=32, vdim=16, chunk=33, bias_max=100, bias_rows=20),
                        mamba_layer(heads=2, vdim=4, state=70, groups=1, conv=4, norm_groups=1, mlp=(32, 1.0))], width=40, vocab=97, loop=(0, 2, 2))


def make_folder(tmp: Path, config: dict, name: str, seed: int = 0, sharpen: float = 8.0) -> Path:
    """A model folder with random bfloat16 weights, then reshaped so that faults show: query and key weights are scaled up (peaked
    attention: a lost, doubled or wrongly masked key changes the output), the decay's logarithm is moved down (a long memory: a lost
    state shows many tokens later), sinks and distance biases get a visible spread."""
    from safetensors.torch import load_file, save_file

    from oxr_inference_b200.weights import write_random_model

    folder = write_random_model(config, tmp / name, seed, dtype="bfloat16", std=0.06)
    path = folder / "model.safetensors"
    tensors = load_file(str(path))
    for k, t in tensors.items():
        f = t.float()
        if k.endswith((".mix.q", ".mix.k", ".mix.uk")):
            f = f * sharpen ** 0.5
        elif k.endswith(".mix.A_log"):
            f = f * 10 - 3.0
        elif k.endswith((".mix.sink", ".mix.rel", ".mix.dt_bias")):
            f = f * 15
        elif k.endswith(("head", "embed")):
            f = f * 4
        tensors[k] = f.to(t.dtype)
    save_file(tensors, str(path), metadata={"format": "pt"})
    (folder / "config.json").write_text(json.dumps({k: v for k, v in config.items()}, indent=1))
    return folder


def tokens(config: dict, n: int, seed: int) -> list[int]:
    g = torch.Generator().manual_seed(seed * 104729 + n)
    return torch.randint(0, config["vocab"], (n,), generator=g).tolist()


_cache: dict = {}


def plain_logits(folder: Path, ids: list[int]) -> torch.Tensor:
    from plain import radapel_plain as RP

    key = (str(folder), tuple(ids))
    if key not in _cache:
        if str(folder) not in _cache:
            _cache[str(folder)] = RP.read_model(folder, torch.float64)
        cfg, w = _cache[str(folder)]
        _cache[key] = RP.forward(cfg, w, ids).float()
    return _cache[key]
