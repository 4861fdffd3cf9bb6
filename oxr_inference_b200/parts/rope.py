"""Rotary position encodings: the half-split (GPT-NeoX) table, and per-step angles for the interleaved-pairs form."""

from __future__ import annotations

import torch

from oxr_inference_b200 import ops
from oxr_inference_b200.parts.base import POSITION_ENCODINGS, PositionEncoding, Runtime, StepContext


@POSITION_ENCODINGS.register("rope_neox")
class RotaryTable(PositionEncoding):
    """fp32 ``cos`` and ``sin`` of ``position * theta^(-2i/dim)`` for i < dim/2, one row per position.

    Built exactly as the reference builds it: fp32 ``inv_freq``, fp32 outer product, then cos/sin
    (oxr_runtime/language.py:160-165). The reference then rounds the table to the model dtype
    (language.py:167-170); here the angles stay fp32 whatever the activation dtype. The table is computed on the
    host so that it does not depend on the device's math library, then copied once.
    """

    def __init__(self, runtime: Runtime, *, dim: int, theta: float):
        if dim % 2:
            raise ValueError(f"rotary dimension {dim} is odd")
        self.dim, self.theta = int(dim), float(theta)
        inv_freq = 1.0 / (self.theta ** (torch.arange(0, self.dim, 2, dtype=torch.float) / self.dim))
        freqs = torch.outer(torch.arange(runtime.max_positions, dtype=torch.float), inv_freq)
        self.cos = freqs.cos().to(runtime.device).contiguous()
        self.sin = freqs.sin().to(runtime.device).contiguous()

    def tables(self) -> tuple[torch.Tensor, torch.Tensor]:
        return self.cos, self.sin


@POSITION_ENCODINGS.register("rope_pairs")
class RotaryPairs(PositionEncoding):
    """Rotary encoding of entry pairs (2i, 2i+1) of the first ``dims`` entries of a vector: the pair (u, v) at position p becomes
    ``(u cos a - v sin a, v cos a + u sin a)`` with ``a = p * base^(-2i/dims)``. There is no table over all positions: each step
    computes cos and sin for its own tokens, once, shared by every layer with the same ``dims`` and ``base`` (the frequencies, the
    product with the position and the functions in fp64, rounded once to fp32), so no position limit comes from here."""

    def __init__(self, runtime: Runtime, *, dims: int, base: float):
        if dims % 2 or dims <= 0:
            raise ValueError(f"rotary dimension {dims} must be even and positive")
        self.dims, self.base = int(dims), float(base)
        freq = torch.tensor([self.base ** (-2.0 * i / self.dims) for i in range(self.dims // 2)], dtype=torch.float64)
        self.freq = freq.to(runtime.device)

    def tables(self):
        raise NotImplementedError("rope_pairs has per-step angles (step_angles), not a table over all positions")

    def step_angles(self, ctx: StepContext) -> tuple[torch.Tensor, torch.Tensor]:
        key = ("rope_pairs", self.dims, self.base)
        if key not in ctx.shared:
            ctx.shared[key] = ops.rotary_angles(ctx.positions, self.freq)
        return ctx.shared[key]
