"""Steps that change the whole stream before a layer runs (``LayerSpec.entry``).

``reinject``: x <- W [x; x0] + step[index], with x0 the embedding output of the same tokens, W [H, 2H] (the
columns of x first) and ``step`` one row per pass over a run of layers.  The product reads [x | x0] in the
products' number format and writes the float32 stream, the step's row added as the product's bias.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .base import STREAM_STEPS, ParamSpec, StepContext, StreamStep


@STREAM_STEPS.register("reinject")
class Reinject(StreamStep):
    """params: ``hidden_size``, ``index`` (which row of ``step`` this visit adds), ``count`` (rows of ``step``).
    weights: ``weight`` [hidden, 2 hidden], ``step`` (float32 [count, hidden])."""
    graph_safe = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.hidden = int(spec.params["hidden_size"])
        self.index = int(spec.params["index"])
        self.count = int(spec.params["count"])
        if self.hidden <= 0 or not 0 <= self.index < self.count:
            raise ValueError(f"reinject: row {self.index} of {self.count}, width {self.hidden}")
        self.weight: Optional[torch.Tensor] = None
        self.step: Optional[torch.Tensor] = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {"weight": ParamSpec((self.hidden, 2 * self.hidden)), "step": ParamSpec((self.count, self.hidden), role="vector")}

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.weight = tensors["weight"].contiguous()
        self.step = tensors["step"][self.index].contiguous()

    def param_bytes(self) -> int:
        return 2 * self.hidden * self.hidden * self.env.dtype.itemsize + 4 * self.hidden

    def flops(self, tokens: int, pairs: float) -> float:
        return 2.0 * tokens * 2 * self.hidden * self.hidden

    def forward(self, x: torch.Tensor, x0: torch.Tensor, ctx: StepContext) -> None:
        both = self.ops.concat_rows(x, x0, self.env.dtype)
        self.ops.linear(both, self.weight, self.step, self.ops.GEMM_STORE_F32, out=x)
