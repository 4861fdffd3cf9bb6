"""A plain, slow statement of the Bifusun decoder: one function per mechanism, whole sequences at once, no cache.

Shares no code with the engine. Everything runs on the host in one floating-point type (float64 by default), so it is the
yardstick for both the 16-bit and the 32-bit engine. The network: a scaled token embedding; a list of pre-norm layers,
``x += mixer(norm1(x))`` and, when the layer has a feed-forward, ``x += ff(norm2(x))``; a final norm; an output head whose
logits are scaled. Mixers: grouped-query softmax attention whose projections have biases and pass a short causal
convolution, with a query temperature that grows with the position and a blend of the values with those of the first
blending layer; and the matrix-memory recurrence of xLSTM. The feed-forward routes each token to a few small experts.
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


def short_convolution(u: torch.Tensor, taps: torch.Tensor) -> torch.Tensor:
    """Causal per-channel filter over time. u: [T, C]; taps: [C, J]; the last tap meets the current token, zeros stand before
    the first token."""
    T, C = u.shape
    J = taps.shape[1]
    padded = torch.cat([torch.zeros(J - 1, C, dtype=u.dtype), u])
    out = torch.zeros_like(u)
    for j in range(J):
        out += padded[j:j + T] * taps[:, j]
    return out


def query_temperature(T: int, coef: float, every: int, dtype) -> torch.Tensor:
    """Factor on the query at positions 0..T-1: 1 + coef ln(floor((p + 1) / every) + 1)."""
    return torch.tensor([1.0 + coef * math.log((p + 1) // every + 1) for p in range(T)], dtype=dtype)


# ------------------------------------------------------------------------------------------------ mixers
def convolved_attention(h: torch.Tensor, w: dict, p: str, m: dict, shared: dict) -> torch.Tensor:
    """``shared``: carries the values of the first blending layer from layer to layer."""
    T = h.shape[0]
    H, G, D, DV = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    proj = {}
    for name in ("q", "k", "v"):
        u = h @ w[p + name].T
        if p + name + ".b" in w:
            u = u + w[p + name + ".b"]
        if m.get("conv"):
            u = short_convolution(u, w[p + name + ".conv"])
        proj[name] = u
    q = proj["q"].view(T, H, D)
    k = proj["k"].view(T, G, D)
    v = proj["v"].view(T, G, DV)
    temp = m.get("q_temp")
    if temp:
        q = q * query_temperature(T, temp["coef"], temp["every"], h.dtype)[:, None, None]
    if m.get("v_mix"):
        if "first_values" not in shared:
            shared["first_values"] = v
        else:
            lam = w[p + "vmix"]
            v = (1 - lam) * v + lam * shared["first_values"]
    seen = torch.arange(T)[None, :] <= torch.arange(T)[:, None]
    out = torch.zeros(T, H, DV, dtype=h.dtype)
    for hd in range(H):
        g = hd // (H // G)
        s = (q[:, hd] @ k[:, g].T) * m["scale"]
        s = s.masked_fill(~seen, float("-inf"))
        out[:, hd] = torch.softmax(s, dim=-1) @ v[:, g]
    y = out.reshape(T, H * DV) @ w[p + "o"].T
    if p + "o.b" in w:
        y = y + w[p + "o.b"]
    return y


def matrix_memory(h: torch.Tensor, w: dict, p: str, m: dict, eps: float) -> torch.Tensor:
    """Per head a matrix S [D, DV], a vector n [D] and a running maximum m_t (all start at 0), driven by a log input gate a and a log
    forget gate b, both squashed to (-cap, cap) before use:

        m_t = max(b_t + m_(t-1), a_t)
        S_t = exp(b_t + m_(t-1) - m_t) S_(t-1) + exp(a_t - m_t) k_t v_t^T         n_t likewise with k_t alone
        o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + 1e-6)
    """
    T = h.shape[0]
    H, D, DV, cap = m["heads"], m["dim"], m["vdim"], float(m["gate_cap"])
    q = (h @ w[p + "q"].T).view(T, H, D) * D ** -0.5
    k = (h @ w[p + "k"].T).view(T, H, D)
    v = (h @ w[p + "v"].T).view(T, H, DV)
    a = cap * torch.tanh((h @ w[p + "i"].T + w[p + "i.b"]) / cap)                                     # [T, H]
    b = torch.nn.functional.logsigmoid(cap * torch.tanh((h @ w[p + "f"].T + w[p + "f.b"]) / cap))
    S = torch.zeros(H, D, DV, dtype=h.dtype)
    n = torch.zeros(H, D, dtype=h.dtype)
    mx = torch.zeros(H, dtype=h.dtype)
    out = torch.zeros(T, H, DV, dtype=h.dtype)
    for t in range(T):
        new_mx = torch.maximum(b[t] + mx, a[t])
        keep = torch.exp(b[t] + mx - new_mx)
        take = torch.exp(a[t] - new_mx)
        S = keep[:, None, None] * S + take[:, None, None] * k[t][:, :, None] * v[t][:, None, :]
        n = keep[:, None] * n + take[:, None] * k[t]
        mx = new_mx
        num = torch.einsum("hdv,hd->hv", S, q[t])
        den = torch.maximum((n * q[t]).sum(-1).abs(), torch.exp(-mx)) + 1e-6
        out[t] = num / den[:, None]
    out = rms_norm(out, None, eps).reshape(T, H * DV) * w[p + "norm"]
    out = out * torch.sigmoid(h @ w[p + "g"].T)
    return out @ w[p + "o"].T


# ------------------------------------------------------------------------------------------------ feed-forward
def route(z: torch.Tensor, r: dict) -> tuple[torch.Tensor, torch.Tensor]:
    """Router logits [T, E] -> (chosen experts [T, top], their weights [T, top])."""
    E, top = r["experts"], r["top"]
    s = torch.sigmoid(z)
    allowed = torch.ones_like(s, dtype=torch.bool)
    groups = r.get("groups")
    if groups and groups["count"] > 1:
        per = E // groups["count"]
        by_group = s.view(-1, groups["count"], per)
        group_score = by_group.topk(min(2, per), dim=-1).values.sum(-1)                  # the two best of each group
        best = group_score.topk(groups["keep"], dim=-1).indices
        keep = torch.zeros_like(group_score, dtype=torch.bool).scatter_(1, best, True)
        allowed = keep[:, :, None].expand(-1, -1, per).reshape(-1, E)
    chosen = s.masked_fill(~allowed, float("-inf")).topk(top, dim=-1).indices
    weight = s.gather(1, chosen)
    weight = weight / (weight.sum(-1, keepdim=True) + 1e-20) * r["scale"]
    return chosen, weight


def route_margin(z: torch.Tensor, r: dict) -> torch.Tensor:
    """Per token, by how much the router's choice was decided: the smaller of the gap between the last group kept and the first one
    dropped and the gap between the last expert chosen and the best one left out. A choice with a small margin may fall the other way
    under another rounding, for no fault."""
    E, top = r["experts"], r["top"]
    s = torch.sigmoid(z)
    margin = torch.full((z.shape[0],), float("inf"), dtype=z.dtype)
    allowed = torch.ones_like(s, dtype=torch.bool)
    groups = r.get("groups")
    if groups and groups["count"] > 1:
        per = E // groups["count"]
        score = s.view(-1, groups["count"], per).topk(min(2, per), dim=-1).values.sum(-1)
        ranked = score.sort(-1, descending=True)
        if groups["keep"] < groups["count"]:
            margin = ranked.values[:, groups["keep"] - 1] - ranked.values[:, groups["keep"]]
        keep = torch.zeros_like(score, dtype=torch.bool).scatter_(1, ranked.indices[:, :groups["keep"]], True)
        allowed = keep[:, :, None].expand(-1, -1, per).reshape(-1, E)
    ranked = s.masked_fill(~allowed, -1.0).sort(-1, descending=True).values
    if top < E:
        gap = ranked[:, top - 1] - ranked[:, top].clamp_min(0.0)
        margin = torch.minimum(margin, torch.where(ranked[:, top] >= 0, gap, torch.full_like(gap, float("inf"))))
    return margin


def routed_experts(h: torch.Tensor, w: dict, p: str, mlp: dict, margins: list | None = None) -> torch.Tensor:
    r = mlp["router"]
    z = h @ w[p + "router"].T
    if margins is not None:
        margins.append(route_margin(z, r))
    chosen, weight = route(z, r)
    out = torch.zeros(h.shape[0], w[p + "e0.down"].shape[0], dtype=h.dtype)
    for t in range(h.shape[0]):
        for e, g in zip(chosen[t].tolist(), weight[t]):
            u = torch.relu(w[p + f"e{e}.up"] @ h[t]) ** 2
            out[t] += g * (w[p + f"e{e}.down"] @ u)
    return out


# ------------------------------------------------------------------------------------------------ the model
def forward(cfg: dict, w: dict, ids: list[int], trace: list | None = None, margins: list | None = None) -> torch.Tensor:
    """Logits [T, vocab] of one sequence. ``trace`` (a list) receives the stream after every layer, ``margins`` every router's
    :func:`route_margin` per token."""
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.tensor(ids)] * cfg.get("embedding", {}).get("scale", 1.0)
    shared: dict = {}
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = rms_norm(x, w[p + "norm1"], eps)
        if layer["type"] == "attention":
            x = x + convolved_attention(h, w, p + "mix.", layer["mixer"], shared)
        elif layer["type"] == "mlstm":
            x = x + matrix_memory(h, w, p + "mix.", layer["mixer"], eps)
        else:
            raise ValueError(layer["type"])
        if layer.get("mlp") is not None:
            x = x + routed_experts(rms_norm(x, w[p + "norm2"], eps), w, p + "mlp.", layer["mlp"], margins)
        if trace is not None:
            trace.append(x.clone())
    return (rms_norm(x, w["final.norm"], eps) @ w["head"].T) * cfg.get("logit_scale", 1.0)


def greedy(cfg: dict, w: dict, prompt: list[int], n: int) -> tuple[list[int], list[float]]:
    """``n`` greedy tokens after ``prompt``, and for each the gap between the two largest logits over the logits' spread (a near-tie
    may fall either way under another rounding)."""
    ids, gaps = list(prompt), []
    for _ in range(n):
        row = forward(cfg, w, ids)[-1]
        best = row.topk(2).values
        gaps.append(float((best[0] - best[1]) / row.std()))
        ids.append(int(row.argmax()))
    return ids[len(prompt):], gaps
