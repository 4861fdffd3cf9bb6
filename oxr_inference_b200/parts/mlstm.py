"""The matrix-memory mixer of xLSTM (mLSTM): a recurrence with fixed-size per-request state instead of a cache that grows."""

from __future__ import annotations

import torch

from oxr_inference_b200 import ops
from oxr_inference_b200.parts.base import MIXERS, LayerCache, Mixer, ParamInfo, PositionEncoding, Runtime, StateNeed, StepContext
from oxr_inference_b200.parts.linear import StackedLinear


@MIXERS.register("mlstm")
class MatrixMemory(Mixer):
    """``q = W_q h / sqrt(key_dim)``, ``k = W_k h`` (``heads x key_dim``), ``v = W_v h`` (``heads x value_dim``); per head a log input gate
    ``a = cap tanh((W_i h + i.b) / cap)`` and a log forget gate ``b = logsigmoid(cap tanh((W_f h + f.b) / cap))``. Per head, with S, n and a
    running maximum m that all start at zero:

        m_t = max(b_t + m_(t-1), a_t)
        S_t = exp(b_t + m_(t-1) - m_t) S_(t-1) + exp(a_t - m_t) k_t v_t^T        n_t likewise with k_t alone
        o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + 1e-6)

    then each head's o is divided by its root mean square, the heads side by side are multiplied by ``norm`` and by ``sigmoid(W_g h)``, then
    ``W_o``. q, k, v and the output gate are one product; the two gate projections are a second one whose result stays in fp32, as does
    everything that enters the recurrence behind the projections. Per request the mixer keeps one fp32 state row: S ``[heads, key_dim,
    value_dim]``, n ``[heads, key_dim]`` and m ``[heads]``; zero for a new request, carried from step to step whatever the cut."""

    def __init__(self, runtime: Runtime, position: PositionEncoding | None, *, hidden_size: int, num_heads: int, key_dim: int, value_dim: int,
                 gate_cap: float, eps: float):
        if position is not None:
            raise ValueError("mlstm takes no position encoding")
        if not gate_cap > 0:
            raise ValueError(f"the gates' cap must be positive, got {gate_cap}")
        if key_dim > 256:
            raise ValueError(f"the recurrence kernel keeps keys of up to 256 entries per head, got {key_dim}")
        self.runtime = runtime
        self.hidden, self.H, self.DK, self.DV = int(hidden_size), int(num_heads), int(key_dim), int(value_dim)
        self.cap, self.eps = float(gate_cap), float(eps)
        self.inner = self.H * self.DV
        self.in_proj = StackedLinear(runtime, self.hidden, {"q": self.H * self.DK, "k": self.H * self.DK, "v": self.inner, "g": self.inner})
        self.gates = StackedLinear(runtime, self.hidden, {"i": self.H, "f": self.H})
        self.out = StackedLinear(runtime, self.inner, {"o": self.hidden})
        self.vectors: dict[str, torch.Tensor] = {}
        self.gate_bias: torch.Tensor | None = None

    _VECTORS = ("i.b", "f.b", "norm")

    def parameters(self) -> dict[str, ParamInfo]:
        return {**self.in_proj.parameters(), **self.gates.parameters(), **self.out.parameters(),
                "i.b": ParamInfo((self.H,), role="vector"), "f.b": ParamInfo((self.H,), role="vector"),
                "norm": ParamInfo((self.inner,), init="around_one", role="vector")}

    def assign(self, name: str, tensor: torch.Tensor) -> None:
        for stack in (self.in_proj, self.gates, self.out):
            if name in stack.outs:
                stack.assign(name, tensor)
                return
        if name not in self._VECTORS:
            raise KeyError(name)
        self.vectors[name] = tensor.to(device=self.runtime.device, dtype=torch.float32).contiguous()

    def finish_loading(self) -> None:
        self.gate_bias = torch.cat([self.vectors["i.b"], self.vectors["f.b"]]).contiguous()

    def cache_need(self) -> StateNeed:
        return StateNeed((self.H * self.DK * self.DV + self.H * self.DK + self.H,), torch.float32)

    def forward(self, h: torch.Tensor, ctx: StepContext, cache: LayerCache) -> torch.Tensor:
        proj = self.in_proj(h)                              # [tokens, q | k | v | g]
        gates = self.gates(h, torch.float32)                # [tokens, i | f], kept in fp32
        k0 = self.H * self.DK
        o = ops.mlstm_scan(proj, 0, k0, 2 * k0, gates, self.gate_bias, heads=self.H, key_dim=self.DK, value_dim=self.DV, cap=self.cap,
                           q_scale=self.DK ** -0.5, state=cache.state, cu_q=ctx.cu_q, state_slots=ctx.state_slots, n_requests=ctx.n_requests)
        return self.out(ops.head_norm_gate(o, proj, 2 * k0 + self.inner, self.vectors["norm"], self.H, self.eps))
