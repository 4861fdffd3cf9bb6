"""Maps of the whole residual stream between layer runs."""

from __future__ import annotations

import torch

from oxr_inference_b200 import ops
from oxr_inference_b200.parts.base import JOINTS, Joint, ParamInfo, Runtime, StepContext
from oxr_inference_b200.parts.linear import StackedLinear


@JOINTS.register("reentry_linear")
class ReentryLinear(Joint):
    """Entry of a pass through a stretch of layers that runs several times with the same weights:
    ``stream <- W [stream; first] + step[pass]`` with ``W [hidden, 2 hidden]`` (the stream's columns first), ``first`` the embedding's
    output and ``step [passes, hidden]`` one learned vector per pass. The product reads activations in the runtime's dtype and
    leaves fp32; the vector is added in fp32."""

    def __init__(self, runtime: Runtime, *, hidden_size: int, passes: int):
        self.runtime, self.hidden, self.passes = runtime, int(hidden_size), int(passes)
        self.map = StackedLinear(runtime, 2 * self.hidden, {"in": self.hidden})
        self.step: torch.Tensor | None = None

    def parameters(self) -> dict[str, ParamInfo]:
        return {**self.map.parameters(), "step": ParamInfo((self.passes, self.hidden), role="vector")}

    def assign(self, name: str, tensor: torch.Tensor) -> None:
        if name == "in":
            self.map.assign(name, tensor)
        elif name == "step":
            self.step = tensor.to(device=self.runtime.device, dtype=torch.float32).contiguous()
        else:
            raise KeyError(name)

    def forward(self, stream: torch.Tensor, first: torch.Tensor, arg: int, ctx: StepContext) -> torch.Tensor:
        if not 0 <= arg < self.passes:
            raise ValueError(f"pass {arg} of {self.passes}")
        both = ops.concat2_cast(stream, first, self.runtime.dtype)
        return ops.add_row_(self.map(both, torch.float32), self.step[arg])
