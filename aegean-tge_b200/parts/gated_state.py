"""Mixers that keep a matrix per head which every token decays, writes to and reads.

``gated_delta_rule``: with h the input, q = Wq h and k = Wk h (``kv_heads`` heads of ``head_dim``), v = Wv h (``heads``
heads of ``value_dim``; head n uses q/k head n // (heads / kv_heads)); each of q, k, v passes a short causal
convolution over time per channel and SiLU; q and k become unit vectors per head, q times head_dim^-1/2; per head

    b = sigmoid(Wb h)                               how much of the new value is written
    a = exp(-exp(A_log) softplus(Wa h + dt_bias))   how much of the state is kept
    S <- a S;  u = b (v - S^T k);  S <- S + k u^T;  o = S^T q

(the readout sees the token's own write); each head's o over its root mean square, times a weight of ``value_dim``
shared by the heads, times silu(Wg h); then Wo.

``state_space``: one product gives [z | x | B | C | dt] (x and z of heads x value_dim, B and C of ``groups`` x ``state``,
one dt per head); x, B and C pass the convolution (with a bias) and SiLU; dt <- softplus(dt + dt_bias); per head

    S <- exp(-exp(A_log) dt) S + dt B x^T;   y = S^T C + D x

y times silu(z), normalised in ``norm_groups`` equal parts (the gate comes before the norm), times a weight; then Wo.

Both keep, per request, the state S in float32 and the convolution's last taps-1 inputs.  They share their kernels:
``ops.gated_prepare`` readies what the recurrence takes, ``ops.gated_rule_scan`` walks the tokens (the state-space
recurrence is the delta rule without its correction, with k = B, q = C, b = dt), ``ops.gated_norm`` normalises and gates.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .base import MIXERS, LayerCache, Mixer, ParamSpec, StateSpec, StepContext


class _MatrixStateMixer(Mixer):
    """What the two have in common: one input product stored in float32, the prepared rows, the scan, the last product."""
    graph_safe = True

    hidden: int
    heads: int
    groups: int
    key_dim: int
    value_dim: int
    taps: int
    eps: float
    w_in: Optional[torch.Tensor]
    w_o: Optional[torch.Tensor]

    def channels(self) -> int:
        return 2 * self.groups * self.key_dim + self.heads * self.value_dim

    def state_spec(self) -> Optional[StateSpec]:
        entries = [("state", (self.heads, self.key_dim, self.value_dim))]
        if self.taps > 1:
            entries.append(("conv", (self.taps - 1, self.channels())))
        return StateSpec(entries=tuple(entries))

    def output_projection(self):
        return self.w_o, None

    def forward(self, h: torch.Tensor, ctx: StepContext, cache: LayerCache) -> torch.Tensor:
        return self.ops.linear(self.inner(h, ctx, cache), self.w_o, None, self.ops.GEMM_STORE)

    def forward_f32(self, h, ctx: StepContext, cache: LayerCache, out=None, alpha: float = 1.0, accumulate: bool = False):
        epilogue = self.ops.GEMM_ADD_F32 if accumulate else self.ops.GEMM_STORE_F32
        return self.ops.linear(self.inner(h, ctx, cache), self.w_o, None, epilogue, out=out, alpha=alpha)

    def forward_add(self, h: torch.Tensor, x: torch.Tensor, ctx: StepContext, cache: LayerCache, next_norm=None):
        a = self.inner(h, ctx, cache)
        fused = next_norm.fusable() if next_norm is not None else None
        if fused is not None:
            return self.ops.linear_add_norm(a, self.w_o, None, x, fused[0], fused[1], self.env.dtype)
        self.ops.linear(a, self.w_o, None, self.ops.GEMM_ADD_F32, out=x)
        return None


@MIXERS.register("gated_delta_rule")
class GatedDeltaRule(_MatrixStateMixer):
    """params: ``hidden_size``, ``heads``, ``kv_heads``, ``head_dim``, ``value_dim``, ``taps`` (of the convolution, 1: none),
    ``eps`` (of the readout's norm), optional ``unit_eps`` (inside the unit norm's root, default 1e-6).
    weights: ``q|k|v|g|b|a|o.weight``, ``q|k|v.conv.weight`` (float32 [channels, taps], the last tap the current token's),
    ``A_log``, ``dt_bias`` (float32 [heads]), ``norm.weight`` (float32 [value_dim])."""

    def __init__(self, spec, env):
        super().__init__(spec, env)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.heads = int(p["heads"])
        self.groups = int(p["kv_heads"])
        self.key_dim = int(p["head_dim"])
        self.value_dim = int(p["value_dim"])
        self.taps = int(p.get("taps", 1))
        self.eps = float(p["eps"])
        self.unit_eps = float(p.get("unit_eps", 1e-6))
        if min(self.hidden, self.heads, self.groups, self.key_dim, self.value_dim) <= 0 or self.heads % self.groups:
            raise ValueError(f"gated_delta_rule: {self.heads} heads on {self.groups} q/k heads; sizes must be positive")
        if not 1 <= self.taps <= 16 or self.key_dim > 256:
            raise ValueError(f"gated_delta_rule: {self.taps} taps (1 to 16), keys of {self.key_dim} (up to 256)")
        self.qk_dim = self.groups * self.key_dim
        self.o_dim = self.heads * self.value_dim
        self.w_in = self.w_o = self.conv_w = self.a_log = self.dt_bias = self.norm_w = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        specs = {"q.weight": ParamSpec((self.qk_dim, self.hidden)), "k.weight": ParamSpec((self.qk_dim, self.hidden)),
                 "v.weight": ParamSpec((self.o_dim, self.hidden)), "g.weight": ParamSpec((self.o_dim, self.hidden)),
                 "b.weight": ParamSpec((self.heads, self.hidden)), "a.weight": ParamSpec((self.heads, self.hidden)),
                 "o.weight": ParamSpec((self.hidden, self.o_dim)),
                 "q.conv.weight": ParamSpec((self.qk_dim, self.taps), role="vector"),
                 "k.conv.weight": ParamSpec((self.qk_dim, self.taps), role="vector"),
                 "v.conv.weight": ParamSpec((self.o_dim, self.taps), role="vector"),
                 "A_log": ParamSpec((self.heads,), role="vector"), "dt_bias": ParamSpec((self.heads,), role="vector"),
                 "norm.weight": ParamSpec((self.value_dim,), role="vector")}
        return specs

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        # rows of q, k, v (the convolved run), then the gate, b and a: one product
        self.w_in = torch.cat([tensors[f"{t}.weight"] for t in ("q", "k", "v", "g", "b", "a")], dim=0).contiguous()
        self.conv_w = torch.cat([tensors[f"{t}.conv.weight"] for t in ("q", "k", "v")], dim=0).contiguous()
        self.w_o = tensors["o.weight"].contiguous()
        self.a_log = tensors["A_log"].contiguous()
        self.dt_bias = tensors["dt_bias"].contiguous()
        self.norm_w = tensors["norm.weight"].repeat(self.heads).contiguous()      # one weight for all heads

    def flops(self, tokens: int, pairs: float) -> float:
        products = 2.0 * tokens * (2 * self.qk_dim + 3 * self.o_dim + 2 * self.heads) * self.hidden
        return products + 6.0 * tokens * self.heads * self.key_dim * self.value_dim     # correction, write, readout

    def inner(self, h: torch.Tensor, ctx: StepContext, cache: LayerCache, out: Optional[torch.Tensor] = None):
        ops = self.ops
        raw = ops.linear(h, self.w_in, None, ops.GEMM_STORE_F32)
        qk, v, gates = ops.gated_prepare(raw, ops.GATED_DELTA, self.groups, self.heads, self.key_dim, self.value_dim,
                                         self.taps, self.conv_w, None, cache.state.get("conv"), ctx.slots, ctx.q_start,
                                         ctx.seq_of_token, ctx.num_seqs, self.a_log, self.dt_bias, unit_eps=self.unit_eps,
                                         q_scale=self.key_dim ** -0.5)
        o = ops.gated_rule_scan(qk, v, gates, cache.state["state"], ctx.slots, ctx.q_start, ctx.num_seqs, delta=True)
        gate = raw[:, self.channels():self.channels() + self.o_dim]
        return ops.gated_norm(o, gate, self.norm_w, self.heads, self.eps, sigmoid=False, out=out, out_dtype=self.env.dtype)


@MIXERS.register("state_space")
class StateSpace(_MatrixStateMixer):
    """params: ``hidden_size``, ``heads``, ``value_dim``, ``state`` (rows of a head's state), ``groups`` (of B and C; head n
    uses group n // (heads / groups)), ``norm_groups``, ``taps``, ``eps``.
    weights: ``in.weight`` [2 heads value_dim + 2 groups state + heads, hidden], ``conv.weight`` (float32 [channels, taps]),
    ``conv.bias``, ``dt_bias``, ``A_log``, ``D`` (float32 [heads]), ``norm.weight`` (float32 [heads value_dim]), ``o.weight``."""

    def __init__(self, spec, env):
        super().__init__(spec, env)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.heads = int(p["heads"])
        self.groups = int(p.get("groups", 1))
        self.key_dim = int(p["state"])
        self.value_dim = int(p["value_dim"])
        self.norm_groups = int(p.get("norm_groups", 1))
        self.taps = int(p.get("taps", 1))
        self.eps = float(p["eps"])
        self.o_dim = self.heads * self.value_dim
        if min(self.hidden, self.heads, self.groups, self.key_dim, self.value_dim, self.norm_groups) <= 0 \
                or self.heads % self.groups or self.o_dim % self.norm_groups:
            raise ValueError(f"state_space: {self.heads} heads on {self.groups} groups, {self.norm_groups} norm groups over "
                             f"{self.o_dim}; sizes must be positive and divide")
        if not 1 <= self.taps <= 16 or self.key_dim > 256:
            raise ValueError(f"state_space: {self.taps} taps (1 to 16), states of {self.key_dim} rows (up to 256)")
        self.w_in = self.w_o = self.conv_w = self.conv_b = self.a_log = self.dt_bias = self.skip = self.norm_w = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        rows = self.o_dim + self.channels() + self.heads
        return {"in.weight": ParamSpec((rows, self.hidden)), "conv.weight": ParamSpec((self.channels(), self.taps), role="vector"),
                "conv.bias": ParamSpec((self.channels(),), role="vector"), "dt_bias": ParamSpec((self.heads,), role="vector"),
                "A_log": ParamSpec((self.heads,), role="vector"), "D": ParamSpec((self.heads,), role="vector"),
                "norm.weight": ParamSpec((self.o_dim,), role="vector"), "o.weight": ParamSpec((self.hidden, self.o_dim))}

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.w_in = tensors["in.weight"].contiguous()
        self.conv_w = tensors["conv.weight"].contiguous()
        self.conv_b = tensors["conv.bias"].contiguous()
        self.dt_bias = tensors["dt_bias"].contiguous()
        self.a_log = tensors["A_log"].contiguous()
        self.skip = tensors["D"].contiguous()
        self.norm_w = tensors["norm.weight"].contiguous()
        self.w_o = tensors["o.weight"].contiguous()

    def flops(self, tokens: int, pairs: float) -> float:
        products = 2.0 * tokens * (3 * self.o_dim + 2 * self.groups * self.key_dim + self.heads) * self.hidden
        return products + 4.0 * tokens * self.heads * self.key_dim * self.value_dim      # write and readout

    def inner(self, h: torch.Tensor, ctx: StepContext, cache: LayerCache, out: Optional[torch.Tensor] = None):
        ops = self.ops
        raw = ops.linear(h, self.w_in, None, ops.GEMM_STORE_F32)
        qk, v, gates = ops.gated_prepare(raw, ops.GATED_STATE_SPACE, self.groups, self.heads, self.key_dim, self.value_dim,
                                         self.taps, self.conv_w, self.conv_b, cache.state.get("conv"), ctx.slots, ctx.q_start,
                                         ctx.seq_of_token, ctx.num_seqs, self.a_log, self.dt_bias)
        y = ops.gated_rule_scan(qk, v, gates, cache.state["state"], ctx.slots, ctx.q_start, ctx.num_seqs, delta=False,
                                skip=self.skip)
        return ops.gated_norm(y, raw[:, :self.o_dim], self.norm_w, self.norm_groups, self.eps, sigmoid=False, out=out,
                              gate_first=True, out_dtype=self.env.dtype)
