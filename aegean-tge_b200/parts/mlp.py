"""Dense gated feed-forward (SwiGLU).

Reference order (src/models/qwen2.cpp:2105-2118,
src/cpu/scalar/norm_rope_scalar.cpp:43-51): ``g = Wg h``, ``u = Wu h``,
``a_i = g_i / (1 + exp(-g_i)) * u_i``, ``d = Wd a``, added to the stream.  No
biases.  Gate and up rows are interleaved at load (row 2i = gate_i, row 2i+1
= up_i) so that one product yields both and its epilogue applies the gate.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .base import FEED_FORWARDS, FeedForward, ParamSpec, StepContext


@FEED_FORWARDS.register("swiglu")
class SwiGLU(FeedForward):
    """params: ``hidden_size``, ``intermediate_size``.  weights: ``gate|up|down.weight``."""
    graph_safe = True
    can_defer_norm = True
    takes_deferred_rows = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.hidden = int(spec.params["hidden_size"])
        self.inner = int(spec.params["intermediate_size"])
        if self.hidden <= 0 or self.inner <= 0:
            raise ValueError("swiglu: sizes must be positive")
        self.w_gate_up: Optional[torch.Tensor] = None
        self.w_down: Optional[torch.Tensor] = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {
            "gate.weight": ParamSpec((self.inner, self.hidden)),
            "up.weight": ParamSpec((self.inner, self.hidden)),
            "down.weight": ParamSpec((self.hidden, self.inner)),
        }

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        gate, up = tensors["gate.weight"], tensors["up.weight"]
        self.w_gate_up = torch.stack([gate, up], dim=1).reshape(2 * self.inner, self.hidden).contiguous()
        self.w_down = tensors["down.weight"].contiguous()

    def flops(self, tokens: int, pairs: float) -> float:
        return 2.0 * tokens * 3 * self.inner * self.hidden

    def forward(self, h: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        a = self.ops.linear(h, self.w_gate_up, None, self.ops.GEMM_SWIGLU)
        return self.ops.linear(a, self.w_down, None, self.ops.GEMM_STORE)

    def forward_f32(self, h: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        a = self.ops.linear(h, self.w_gate_up, None, self.ops.GEMM_SWIGLU)
        return self.ops.linear(a, self.w_down, None, self.ops.GEMM_STORE_F32)

    def forward_add(self, h: torch.Tensor, x: torch.Tensor, ctx: StepContext, next_norm=None, defer: bool = False):
        a = self.ops.linear(h, self.w_gate_up, None, self.ops.GEMM_SWIGLU)
        fused = next_norm.fusable() if next_norm is not None else None
        if fused is not None:
            return self.ops.linear_add_norm(a, self.w_down, None, x, fused[0], fused[1], self.env.dtype, defer=defer)
        self.ops.linear(a, self.w_down, None, self.ops.GEMM_ADD_F32, out=x)
        return None


@FEED_FORWARDS.register("dense_mlp")
class DenseMLP(FeedForward):
    """The ungated feed-forward: d = Wdown act(Wup h + bup) + bdown.

    params: ``hidden_size``, ``intermediate_size``, ``activation`` (``"gelu"``: 0.5 z (1 + erf(z / sqrt 2)), the
    default; ``"gelu_tanh"``: 0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3))); ``"xielu"``: with two learned numbers
    (p, q), z > 0: softplus(p) z^2 + z/2, else (1/2 + softplus(q)) (exp(z) - 1 - z) + z/2; ``"relu_squared"``:
    max(z, 0)^2), ``bias`` (bool, default
    False: both products have one).  weights: ``up|down.weight``, with ``bias`` ``up|down.bias``, with xielu ``act``
    (float32 [2]).  The GELUs are the epilogue of the up product; xielu is a kernel behind it.
    """
    graph_safe = True
    can_defer_norm = True
    takes_deferred_rows = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.hidden = int(spec.params["hidden_size"])
        self.inner_size = int(spec.params["intermediate_size"])
        activation = str(spec.params.get("activation", "gelu"))
        if activation not in ("gelu", "gelu_tanh", "xielu", "relu_squared"):
            raise ValueError(f"dense_mlp: unknown activation '{activation}'")
        if self.hidden <= 0 or self.inner_size <= 0:
            raise ValueError("dense_mlp: sizes must be positive")
        self.activation = activation
        self.bias = bool(spec.params.get("bias", False))
        self.w_up: Optional[torch.Tensor] = None
        self.w_down: Optional[torch.Tensor] = None
        self.b_up: Optional[torch.Tensor] = None
        self.b_down: Optional[torch.Tensor] = None
        self.act: Optional[torch.Tensor] = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        specs = {"up.weight": ParamSpec((self.inner_size, self.hidden)),
                 "down.weight": ParamSpec((self.hidden, self.inner_size))}
        if self.bias:
            specs["up.bias"] = ParamSpec((self.inner_size,), role="vector")
            specs["down.bias"] = ParamSpec((self.hidden,), role="vector")
        if self.activation == "xielu":
            specs["act"] = ParamSpec((2,), role="vector")
        return specs

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.w_up = tensors["up.weight"].contiguous()
        self.w_down = tensors["down.weight"].contiguous()
        if self.bias:
            self.b_up = tensors["up.bias"].contiguous()
            self.b_down = tensors["down.bias"].contiguous()
        if self.activation == "xielu":
            self.act = tensors["act"].contiguous()

    def flops(self, tokens: int, pairs: float) -> float:
        return 2.0 * tokens * 2 * self.inner_size * self.hidden

    def epilogue(self) -> int:
        return {"gelu": self.ops.GEMM_GELU, "gelu_tanh": self.ops.GEMM_GELU_TANH, "xielu": self.ops.GEMM_STORE,
                "relu_squared": self.ops.GEMM_STORE}[self.activation]

    def input_projection(self) -> torch.Tensor:
        return self.w_up

    def adopt_input_projection(self, view: torch.Tensor) -> None:
        """The up rows now live inside a tensor that another part shares (same values): use that copy."""
        self.w_up = view

    def inner(self, h, ctx: StepContext, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        rows = self.ops.linear(h, self.w_up, self.b_up, self.epilogue(), out=out)
        if self.activation == "xielu":
            self.ops.activation(rows, self.ops.ACT_XIELU, self.act)
        elif self.activation == "relu_squared":
            self.ops.activation(rows, self.ops.ACT_RELU_SQUARED)
        return rows

    def output_projection(self):
        return self.w_down, self.b_down

    def forward(self, h: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        return self.ops.linear(self.inner(h, ctx), self.w_down, self.b_down, self.ops.GEMM_STORE)

    def forward_add(self, h: torch.Tensor, x: torch.Tensor, ctx: StepContext, next_norm=None, defer: bool = False):
        a = self.inner(h, ctx)
        fused = next_norm.fusable() if next_norm is not None else None
        if fused is not None:
            return self.ops.linear_add_norm(a, self.w_down, self.b_down, x, fused[0], fused[1], self.env.dtype, defer=defer)
        self.ops.linear(a, self.w_down, self.b_down, self.ops.GEMM_ADD_F32, out=x)
        return None


@FEED_FORWARDS.register("clamped_glu")
class ClampedGLU(FeedForward):
    """A gated feed-forward whose two halves are clamped: g = min(Wgate h, L), u = clamp(Wup h, -L, L),
    a = g sigmoid(alpha g) (u + offset), d = Wdown a.  No biases.

    params: ``hidden_size``, ``intermediate_size``, ``limit`` (L), optional ``alpha`` (default 1.702) and ``up_offset``
    (default 1).  weights: ``gate|up|down.weight``.  Gate and up rows are interleaved at load so that one product
    yields both; with alpha 1.702 and offset 1 its epilogue clamps and gates, otherwise the product is stored in
    float32 and one kernel clamps, gates and writes the rows the down product reads.
    """
    graph_safe = True
    can_defer_norm = True
    takes_deferred_rows = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.hidden = int(spec.params["hidden_size"])
        self.inner_size = int(spec.params["intermediate_size"])
        self.limit = float(spec.params["limit"])
        self.alpha = float(spec.params.get("alpha", 1.702))
        self.offset = float(spec.params.get("up_offset", 1.0))
        if self.hidden <= 0 or self.inner_size <= 0 or not self.limit > 0.0:
            raise ValueError("clamped_glu: sizes and the limit must be positive")
        self.w_gate_up: Optional[torch.Tensor] = None
        self.w_down: Optional[torch.Tensor] = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {"gate.weight": ParamSpec((self.inner_size, self.hidden)), "up.weight": ParamSpec((self.inner_size, self.hidden)),
                "down.weight": ParamSpec((self.hidden, self.inner_size))}

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        gate, up = tensors["gate.weight"], tensors["up.weight"]
        self.w_gate_up = torch.stack([gate, up], dim=1).reshape(2 * self.inner_size, self.hidden).contiguous()
        self.w_down = tensors["down.weight"].contiguous()

    def flops(self, tokens: int, pairs: float) -> float:
        return 2.0 * tokens * 3 * self.inner_size * self.hidden

    def inner(self, h, ctx: StepContext, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        if self.alpha == 1.702 and self.offset == 1.0:
            # the product's own epilogue clamps and gates (its constants are these two)
            return self.ops.linear(h, self.w_gate_up, None, self.ops.GEMM_GLU_CLAMPED, out=out, alpha=self.limit)
        complete = getattr(h, "complete", None)
        rows = self.ops.linear(h if complete is None else complete(), self.w_gate_up, None, self.ops.GEMM_STORE_F32)
        return self.ops.gated_clamp_act(rows, self.limit, self.alpha, self.offset, self.env.dtype, out=out)

    def output_projection(self):
        return self.w_down, None

    def forward(self, h: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        return self.ops.linear(self.inner(h, ctx), self.w_down, None, self.ops.GEMM_STORE)

    def forward_f32(self, h: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        return self.ops.linear(self.inner(h, ctx), self.w_down, None, self.ops.GEMM_STORE_F32)

    def forward_add(self, h: torch.Tensor, x: torch.Tensor, ctx: StepContext, next_norm=None, defer: bool = False):
        a = self.inner(h, ctx)
        fused = next_norm.fusable() if next_norm is not None else None
        if fused is not None:
            return self.ops.linear_add_norm(a, self.w_down, None, x, fused[0], fused[1], self.env.dtype, defer=defer)
        self.ops.linear(a, self.w_down, None, self.ops.GEMM_ADD_F32, out=x)
        return None
