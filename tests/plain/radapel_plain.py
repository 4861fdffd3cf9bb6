"""A plain, slow statement of the Radapel decoder: one function per mechanism, whole sequences at once, no cache.

Shares no code with the engine. Everything runs on the host in one floating-point type (float64 by default), so it
is the yardstick for both the 16-bit and the 32-bit engine. The network: scaled token embedding; a list of layers,
each ``x += post_norm(mixer(pre_norm(x)))`` and, when it has a feed-forward, ``x += post_norm(ff(pre_norm(x)))``; a
stretch of layers that may run several times in a row with the same weights, each pass entered through a linear
map of [stream; embedding output] plus a per-pass vector; a final norm and the output head. Mixers: chunk-masked
grouped-query attention with a bucketed distance bias, latent attention with an interleaved rotary part and a
sink in the softmax denominator, and a Mamba-2 recurrence.
"""

from __future__ import annotations

import json
import math
from pathlib import Path

import torch
from safetensors import safe_open


def read_model(folder: str | Path, dtype: torch.dtype = torch.float64):
    folder = Path(folder)
    cfg = json.loads((folder / "config.json").read_text())
    w = {}
    with safe_open(str(folder / "model.safetensors"), framework="pt", device="cpu") as f:
        for name in f.keys():  # noqa: SIM118
            t = f.get_tensor(name)
            w[name] = t.to(dtype) if t.is_floating_point() else t
    return cfg, w


# ------------------------------------------------------------------------------------------------ small pieces
def rms_norm(x: torch.Tensor, weight: torch.Tensor | None, eps: float) -> torch.Tensor:
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if weight is None else y * weight


def distance_bucket(n: int, rows: int, far: float) -> int:
    """Row of the distance-bias table for a key ``n`` positions back: exact below rows/2, logarithmic up to ``far``."""
    half = rows // 2
    if n < half:
        return n
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))


def rotate_pairs(x: torch.Tensor, positions: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """Rotary encoding of the first ``dims`` entries of the last axis, entry 2i paired with 2i+1. x: [T, ..., D]."""
    out = x.clone()
    i = torch.arange(dims // 2, dtype=x.dtype)
    freq = base ** (-2 * i / dims)
    ang = positions.to(x.dtype)[:, None] * freq[None, :]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [dims // 2]
    c, s = ang.cos().view(shape), ang.sin().view(shape)
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


# ------------------------------------------------------------------------------------------------ mixers
def chunked_attention(h: torch.Tensor, w: dict, p: str, m: dict) -> torch.Tensor:
    T = h.shape[0]
    H, G, D, DV = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T).view(T, H, D)
    k = (h @ w[p + "k"].T).view(T, G, D)
    v = (h @ w[p + "v"].T).view(T, G, DV)
    rel = w.get(p + "rel")
    chunk = (m.get("mask") or {}).get("size")
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    seen = j <= i
    if chunk is not None:
        seen = seen & (i // chunk == j // chunk)
    if rel is not None:
        row_of = torch.tensor([distance_bucket(n, rel.shape[0], m["bias_max"]) for n in range(T)])
        rows = row_of[(i - j).clamp(min=0)]
    out = torch.zeros(T, H, DV, dtype=h.dtype)
    for hd in range(H):
        g = hd // (H // G)
        s = (q[:, hd] @ k[:, g].T) * m["scale"]
        if rel is not None:
            s = s + rel[:, hd][rows]
        s = s.masked_fill(~seen, -math.inf)
        out[:, hd] = torch.softmax(s, dim=-1) @ v[:, g]
    return out.reshape(T, H * DV) @ w[p + "o"].T


def latent_attention(h: torch.Tensor, w: dict, p: str, m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, D, R, DV, L = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(T)
    q = (h @ w[p + "q"].T).view(T, H, D + R)
    down = h @ w[p + "dkv"].T
    c = rms_norm(down[:, :L], w[p + "dkv.norm"], eps)
    rot = m.get("rot") or {"dims": 0, "base": 1.0}
    k_rot = rotate_pairs(down[:, L:].view(T, 1, R), pos, rot["dims"], rot["base"])[:, 0]
    q_rot = rotate_pairs(q[..., D:], pos, rot["dims"], rot["base"])
    k_plain = (c @ w[p + "uk"].T).view(T, H, D)
    v = (c @ w[p + "uv"].T).view(T, H, DV)
    sink = w[p + "sink"]
    out = torch.zeros(T, H, DV, dtype=h.dtype)
    causal = torch.ones(T, T).tril().bool()
    for hd in range(H):
        s = (q[:, hd, :D] @ k_plain[:, hd].T + q_rot[:, hd] @ k_rot.T) * m["scale"]
        s = s.masked_fill(~causal, -math.inf)
        top = torch.maximum(s.max(-1, keepdim=True).values, sink[hd])
        e = torch.exp(s - top)
        out[:, hd] = (e / (e.sum(-1, keepdim=True) + torch.exp(sink[hd] - top))) @ v[:, hd]
    return out.reshape(T, H * DV) @ w[p + "o"].T


def mamba2(h: torch.Tensor, w: dict, p: str, m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, P, N, G, taps = m["heads"], m["vdim"], m["state"], m["groups"], m["conv"]
    inner = H * P
    proj = h @ w[p + "in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    padded = torch.cat([torch.zeros(taps - 1, xbc.shape[1], dtype=h.dtype), xbc])
    conv = w[p + "conv.b"].expand(T, -1).clone()
    for j in range(taps):
        conv = conv + padded[j:j + T] * w[p + "conv"][:, j]
    conv = conv * torch.sigmoid(conv)
    x = conv[:, :inner].view(T, H, P)
    B = conv[:, inner:inner + G * N].view(T, G, N)
    C = conv[:, inner + G * N:].view(T, G, N)
    dt = torch.nn.functional.softplus(dt + w[p + "dt_bias"], threshold=1e9)
    decay = torch.exp(-torch.exp(w[p + "A_log"]) * dt)
    y = torch.zeros(T, H, P, dtype=h.dtype)
    for hd in range(H):
        g = hd // (H // G)
        S = torch.zeros(N, P, dtype=h.dtype)
        for t in range(T):
            S = decay[t, hd] * S + dt[t, hd] * torch.outer(B[t, g], x[t, hd])
            y[t, hd] = S.T @ C[t, g] + w[p + "D"][hd] * x[t, hd]
    y = y.view(T, inner) * (z * torch.sigmoid(z))
    parts = m["norm_groups"]
    y = rms_norm(y.view(T, parts, inner // parts), None, eps).view(T, inner) * w[p + "norm"]
    return y @ w[p + "o"].T


def dense_ff(h: torch.Tensor, w: dict, p: str, f: dict) -> torch.Tensor:
    lim = f["limit"]
    g = (h @ w[p + "gate"].T).clamp(max=lim)
    u = (h @ w[p + "up"].T).clamp(-lim, lim)
    return (g * torch.sigmoid(1.702 * g) * (u + 1)) @ w[p + "down"].T


MIXERS = {
    "attention": lambda h, w, p, m, eps: chunked_attention(h, w, p, m),
    "latent_attention": latent_attention,
    "mamba2": mamba2,
}


# ------------------------------------------------------------------------------------------------ the network
def layer_runs(cfg: dict) -> list[tuple[int, int | None]]:
    """(layer, pass number if the run is the first of a pass) in execution order."""
    n, loop = len(cfg["layers"]), cfg.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    runs = [(i, None) for i in range(loop["start"])]
    for t in range(loop["times"]):
        runs += [(i, t if i == loop["start"] else None) for i in range(loop["start"], loop["stop"])]
    return runs + [(i, None) for i in range(loop["stop"], n)]


def forward(cfg: dict, w: dict, ids: list[int], trace: list | None = None) -> torch.Tensor:
    """Logits ``[tokens, vocab]`` of one sequence; ``trace`` collects the stream after every layer run."""
    dtype = w["embed"].dtype
    eps = cfg["norm"]["eps"]
    x0 = w["embed"][torch.tensor(ids)] * cfg["embedding"]["scale"]
    x = x0.clone()
    for i, enter in layer_runs(cfg):
        if enter is not None:
            x = torch.cat([x, x0], dim=-1) @ w["loop.in"].T + w["loop.step"][enter]
        layer, p = cfg["layers"][i], f"l{i}."
        a = MIXERS[layer["type"]](rms_norm(x, w[p + "norm1"], eps), w, p + "mix.", layer["mixer"], eps)
        x = x + rms_norm(a, w[p + "norm1b"], eps)
        if layer.get("mlp"):
            f = dense_ff(rms_norm(x, w[p + "norm2"], eps), w, p + "mlp.", layer["mlp"])
            x = x + rms_norm(f, w[p + "norm2b"], eps)
        if trace is not None:
            trace.append(x.clone())
    return rms_norm(x, w["final.norm"], eps).to(dtype) @ w["head"].T


def greedy(cfg: dict, w: dict, prompt: list[int], n: int) -> tuple[list[int], list[float]]:
    """``n`` greedy tokens after ``prompt`` (the whole sequence is run again for each), and for each the gap between the two
    largest logits, so that a caller can tell a real difference from a near-tie."""
    ids, out, gaps = list(prompt), [], []
    for _ in range(n):
        last = forward(cfg, w, ids)[-1]
        top = last.topk(2).values
        nxt = int(last.argmax())
        gaps.append(float(top[0] - top[1]))
        out.append(nxt)
        ids.append(nxt)
    return out, gaps
