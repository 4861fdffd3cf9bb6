"""The Mamba-2 mixer: a state-space recurrence with fixed-size per-request state instead of a cache that grows."""

from __future__ import annotations

import torch

from oxr_inference_b200 import ops
from oxr_inference_b200.parts.base import MIXERS, LayerCache, Mixer, ParamInfo, PositionEncoding, Runtime, StateNeed, StepContext
from oxr_inference_b200.parts.linear import StackedLinear


@MIXERS.register("mamba2")
class Mamba2(Mixer):
    """``W_in h = [z | x | B | C | dt]`` with ``inner = heads * value_dim`` entries of z and x, ``groups * state`` of B and of C and one dt
    per head. x, B and C pass a causal per-channel convolution of ``taps`` taps (with bias; the last tap is the current token's) and
    SiLU. ``dt <- softplus(dt + dt_bias)``; per head, with its group's B and C:

        S_t = exp(-exp(A_log) dt_t) S_(t-1) + dt_t B_t x_t^T        y_t = S_t^T C_t + D x_t

    then ``y * silu(z)``, RMS-normed in ``norm_groups`` equal parts (each by its own root mean square) times ``norm``, then ``W_o``.

    Per request the mixer keeps one fp32 state row: S ``[heads, state, value_dim]`` followed by the convolution's last ``taps - 1``
    inputs ``[channels, taps - 1]``; zero for a new request, carried from step to step whatever the cut."""

    def __init__(self, runtime: Runtime, position: PositionEncoding | None, *, hidden_size: int, num_heads: int, value_dim: int, state: int,
                 groups: int, taps: int, norm_groups: int, eps: float):
        if num_heads % groups:
            raise ValueError(f"{num_heads} heads are not a multiple of {groups} groups")
        self.runtime = runtime
        self.hidden, self.H, self.P, self.N, self.G = int(hidden_size), int(num_heads), int(value_dim), int(state), int(groups)
        self.taps, self.norm_groups, self.eps = int(taps), int(norm_groups), float(eps)
        self.inner = self.H * self.P
        if self.inner % self.norm_groups:
            raise ValueError(f"{self.inner} inner entries do not split into {self.norm_groups} equal parts")
        self.channels = self.inner + 2 * self.G * self.N
        self.ssm_size = self.H * self.P * self.N
        self.tail_size = self.channels * (self.taps - 1)
        self.in_proj = StackedLinear(runtime, self.hidden, {"in": 2 * self.inner + 2 * self.G * self.N + self.H})
        self.out = StackedLinear(runtime, self.inner, {"o": self.hidden})
        self.vectors: dict[str, torch.Tensor] = {}

    _VECTORS = ("conv", "conv.b", "dt_bias", "A_log", "D", "norm")

    def parameters(self) -> dict[str, ParamInfo]:
        return {**self.in_proj.parameters(), **self.out.parameters(),
                "conv": ParamInfo((self.channels, self.taps), role="vector"), "conv.b": ParamInfo((self.channels,), role="vector"),
                "dt_bias": ParamInfo((self.H,), role="vector"), "A_log": ParamInfo((self.H,), role="vector"),
                "D": ParamInfo((self.H,), init="around_one", role="vector"), "norm": ParamInfo((self.inner,), init="around_one", role="vector")}

    def assign(self, name: str, tensor: torch.Tensor) -> None:
        if name in self.in_proj.outs:
            self.in_proj.assign(name, tensor)
        elif name in self.out.outs:
            self.out.assign(name, tensor)
        elif name in self._VECTORS:
            self.vectors[name] = tensor.to(device=self.runtime.device, dtype=torch.float32).contiguous()
        else:
            raise KeyError(name)

    def cache_need(self) -> StateNeed:
        return StateNeed((self.ssm_size + self.tail_size,), torch.float32)

    def forward(self, h: torch.Tensor, ctx: StepContext, cache: LayerCache) -> torch.Tensor:
        v = self.vectors
        state = cache.state                       # [slots, ssm | tail]
        tail = state[:, self.ssm_size:]
        proj = self.in_proj(h)
        xbc = ops.mamba_conv(proj, self.inner, self.channels, v["conv"], v["conv.b"], tail, req_of_token=ctx.req_of_token, cu_q=ctx.cu_q,
                             state_slots=ctx.state_slots, n_requests=ctx.n_requests)
        y = ops.mamba_scan(xbc, proj, self.inner + self.channels, heads=self.H, vdim=self.P, state=self.N, groups=self.G, dt_bias=v["dt_bias"],
                           a_log=v["A_log"], d_skip=v["D"], ssm=state, cu_q=ctx.cu_q, state_slots=ctx.state_slots, n_requests=ctx.n_requests)
        return self.out(ops.gated_group_norm(y, proj, 0, v["norm"], self.norm_groups, self.eps))
