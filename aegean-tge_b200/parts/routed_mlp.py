"""A routed feed-forward: a mixture of small experts, of which each token uses a few.

With h the input, R = experts + identity router outputs:

    z = Wr h (float32)          s = softmax(z) over all R outputs
    choice = s + correction     the ``top`` largest choice values are taken, looking only inside the ``keep`` of
                                ``count`` groups of neighbouring outputs whose best choice value is largest
    w_k = s_k / (sum of the chosen s + 1e-20)
    out = sum_k w_k E_k(h)      E_e(h) = Wdown_e relu(Wup_e h)^2 for an expert, h itself for an identity output

The correction steers the choice only; the weights use the plain scores.  Identity outputs are the last ``identity``
router outputs and have no tensors.  The sum over a token's choices is formed in float32 in the order of the choice
and added into the float32 stream.

Three ways through the experts.  A step of very few tokens lets each (token, choice) pair read its expert's rows
directly (``experts_direct``: two kernels).  A step of some tokens whose choices between them reach most experts
anyway (a decode batch, a short portion: at least twice as many pairs as experts, at most ``DENSE_MAX_TOKENS``
tokens) goes through ALL experts: one product of the tokens with every up matrix, ``experts_dense_weigh`` (the
chosen experts' activated rows times their weights, zeros elsewhere), one product with the down matrices side by
side along k that adds into the stream; every expert's weights cross the memory bus once, on the tensor cores, and
the work wasted on zeros is free while the step is bound by those bytes.  Neither reads anything from the host, so
both can be captured into a CUDA graph.  A step of many tokens groups the pairs by expert and runs one ordinary product per
expert and projection over that expert's block of rows (``experts_group`` -> products ->
``experts_combine_add``); the host reads the group sizes, which a step with prompt portions may do.

The down matrices are kept side by side, [hidden, experts, inner]: expert e's matrix is the strided view [:, e, :].
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .base import FEED_FORWARDS, FeedForward, ParamSpec, StepContext, build_part

DIRECT_MAX_TOKENS = 32      # steps of up to this many tokens (and every step of single tokens) avoid the grouped path
DENSE_MAX_TOKENS = 256      # beyond this many tokens the wasted products of the dense path would cost more than its bytes


@FEED_FORWARDS.register("routed_experts")
class RoutedExperts(FeedForward):
    """params: ``hidden_size``, ``intermediate_size`` (an expert's inner width), ``experts``, ``top``, optional
    ``identity`` (default 0), ``group_count`` / ``group_keep`` (default 1 / 1: no groups), ``correction`` (bool,
    default True: the checkpoint holds a correction of the choice), ``activation`` (``"relu_squared"``, the only one
    the expert kernels apply so far), ``router_bias`` (bool, default False: a bias added to the router's logits, so it
    steers the choice and the weights alike), ``shared`` (None, or the PartSpec of a feed-forward that every token
    uses and whose output is added; its parameters are this part's under ``shared.<local name>``).
    With no correction and no groups the weights are the softmax over the chosen logits alone: a chosen output's share
    of the softmax over all, divided by the chosen ones' sum, is the same number.
    weights: ``router.weight`` [experts + identity, hidden], ``router.bias`` and ``correction`` (float32 [experts +
    identity]), ``experts.<e>.up.weight`` [inner, hidden], ``experts.<e>.down.weight`` [hidden, inner]."""
    graph_safe = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.inner_size = int(p["intermediate_size"])
        self.experts = int(p["experts"])
        self.identity = int(p.get("identity", 0))
        self.top = int(p["top"])
        self.group_count = int(p.get("group_count", 1))
        self.group_keep = int(p.get("group_keep", 1))
        self.has_correction = bool(p.get("correction", True))
        self.has_router_bias = bool(p.get("router_bias", False))
        shared = p.get("shared")
        self.shared: Optional[FeedForward] = build_part(FEED_FORWARDS, shared, env) if shared is not None else None
        if self.shared is not None:
            self.graph_safe = bool(self.shared.graph_safe)
        self.router_bias: Optional[torch.Tensor] = None
        self.outputs = self.experts + self.identity
        if str(p.get("activation", "relu_squared")) != "relu_squared":
            raise ValueError(f"routed_experts: unknown activation '{p.get('activation')}'")
        if min(self.hidden, self.inner_size, self.top, self.group_count, self.group_keep) <= 0 or self.experts < 0 \
                or self.identity < 0 or self.outputs <= 0:
            raise ValueError("routed_experts: sizes must be positive")
        if self.outputs % self.group_count or self.group_keep > self.group_count:
            raise ValueError(f"routed_experts: {self.group_count} groups ({self.group_keep} kept) of {self.outputs} router outputs")
        if self.top > (self.outputs // self.group_count) * self.group_keep:
            raise ValueError(f"routed_experts: {self.top} choices do not fit the kept groups")
        if self.outputs > 1024:
            raise ValueError("routed_experts: the router kernel takes up to 1024 outputs")
        self.w_router: Optional[torch.Tensor] = None
        self.correction: Optional[torch.Tensor] = None
        self.w_up: Optional[torch.Tensor] = None         # [experts, inner, hidden]
        self.w_down: Optional[torch.Tensor] = None       # [hidden, experts, inner]

    def param_specs(self) -> Dict[str, ParamSpec]:
        specs = {"router.weight": ParamSpec((self.outputs, self.hidden))}
        if self.has_correction:
            specs["correction"] = ParamSpec((self.outputs,), role="vector")
        if self.has_router_bias:
            specs["router.bias"] = ParamSpec((self.outputs,), role="vector")
        if self.shared is not None:
            specs.update({f"shared.{local}": param for local, param in self.shared.param_specs().items()})
        for e in range(self.experts):
            specs[f"experts.{e}.up.weight"] = ParamSpec((self.inner_size, self.hidden))
            specs[f"experts.{e}.down.weight"] = ParamSpec((self.hidden, self.inner_size))
        return specs

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.w_router = tensors["router.weight"].contiguous()
        self.correction = tensors["correction"].contiguous() if self.has_correction else None
        self.router_bias = tensors["router.bias"].contiguous() if self.has_router_bias else None
        if self.shared is not None:
            self.shared.load({name[len("shared."):]: t for name, t in tensors.items() if name.startswith("shared.")})
        if self.experts:
            self.w_up = torch.stack([tensors[f"experts.{e}.up.weight"] for e in range(self.experts)]).contiguous()
            self.w_down = torch.stack([tensors[f"experts.{e}.down.weight"] for e in range(self.experts)], dim=1).contiguous()
        else:
            self.w_up = torch.empty((0, self.inner_size, self.hidden), dtype=self.w_router.dtype, device=self.w_router.device)
            self.w_down = torch.empty((self.hidden, 0, self.inner_size), dtype=self.w_router.dtype, device=self.w_router.device)

    def param_bytes(self) -> int:
        """What one token's step reads: the router and the chosen experts (a large batch touches more of them)."""
        item = self.env.dtype.itemsize
        extra = self.shared.param_bytes() if self.shared is not None else 0
        return (self.outputs * self.hidden + min(self.top, self.experts) * 2 * self.inner_size * self.hidden) * item + 4 * self.outputs + extra

    def dense(self, tokens: int) -> bool:
        """Whether a step of this many tokens runs all experts (its choices reach most of them anyway)."""
        return bool(self.experts) and 2 * self.experts <= tokens * self.top and tokens <= DENSE_MAX_TOKENS

    def step_param_bytes(self, tokens: int) -> int:
        """What a step of ``tokens`` tokens reads: the router, and all experts on the dense path, else as many as
        uniform choices would reach on average."""
        item = self.env.dtype.itemsize
        reached = self.experts if self.dense(tokens) else self.experts * (1.0 - (1.0 - min(self.top / self.outputs, 1.0)) ** tokens)
        extra = self.shared.param_bytes() if self.shared is not None else 0
        return int((self.outputs * self.hidden + reached * 2 * self.inner_size * self.hidden) * item) + 4 * self.outputs + extra

    def flops(self, tokens: int, pairs: float) -> float:
        extra = self.shared.flops(tokens, pairs) if self.shared is not None else 0.0
        return 2.0 * tokens * (self.outputs * self.hidden + self.top * 2 * self.inner_size * self.hidden) + extra

    def route(self, h: torch.Tensor):
        """(ids int32 [T, top], weights float32 [T, top]); the logits are a float32 product of the rows as given."""
        complete = getattr(h, "complete", None)
        if complete is not None:
            h = complete()
        logits = self.ops.linear(h, self.w_router, self.router_bias, self.ops.GEMM_STORE_F32)
        ids, weights = self.ops.router_topk(logits, self.correction, self.top, self.group_count, self.group_keep)
        return h, ids, weights

    def forward_add(self, h: torch.Tensor, x: torch.Tensor, ctx: StepContext, next_norm=None):
        h = self.add_routed(h, x, ctx)
        if self.shared is not None:
            # the feed-forward every token uses adds last, and with it whatever it can do for the next norm
            return self.shared.forward_add(h, x, ctx, next_norm=next_norm)
        return None

    def add_routed(self, h: torch.Tensor, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        """Adds the chosen experts' weighted outputs into ``x``; returns the rows as the experts read them."""
        ops = self.ops
        h, ids, weights = self.route(h)
        tokens = h.shape[0]
        few = ctx.max_q_len <= 1 or tokens <= DIRECT_MAX_TOKENS
        if self.dense(tokens):
            z = ops.linear(h, self.w_up.view(self.experts * self.inner_size, self.hidden), None, ops.GEMM_STORE)
            ops.experts_dense_weigh(z, ids, weights, h, x, self.experts)
            ops.linear(z, self.w_down.view(self.hidden, self.experts * self.inner_size), None, ops.GEMM_ADD_F32, out=x)
            return h
        if few or self.experts == 0:
            ops.experts_direct(h, self.w_up, self.w_down, ids, weights, x)
            return h
        place, offsets, grouped = ops.experts_group(h, ids, self.experts)
        bounds: List[int] = offsets.tolist()             # the host learns the group sizes: not a captured step
        rows = bounds[-1]
        inner = torch.empty((max(rows, 1), self.inner_size), dtype=h.dtype, device=h.device)
        outputs = torch.empty((max(rows, 1), self.hidden), dtype=torch.float32, device=h.device)
        for e in range(self.experts):
            lo, hi = bounds[e], bounds[e + 1]
            if hi > lo:
                ops.linear(grouped[lo:hi], self.w_up[e], None, ops.GEMM_STORE, out=inner[lo:hi])
        if rows:
            ops.activation(inner[:rows], ops.ACT_RELU_SQUARED)
        for e in range(self.experts):
            lo, hi = bounds[e], bounds[e + 1]
            if hi > lo:
                ops.linear(inner[lo:hi], self.w_down[:, e, :], None, ops.GEMM_STORE_F32, out=outputs[lo:hi])
        ops.experts_combine_add(outputs, place, weights, h, x)
        return h

    def forward_f32(self, h: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        out = torch.zeros((h.shape[0], self.hidden), dtype=torch.float32, device=h.device)
        self.forward_add(h, out, ctx)
        return out

    def forward(self, h: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        return self.ops.to_run_dtype(self.forward_f32(h, ctx), self.env.dtype)
