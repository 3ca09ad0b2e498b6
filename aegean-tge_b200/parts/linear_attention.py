"""Linear attention with a fixed decay per head, and the sum of several mixers.

``decay_linear_attention`` keeps, per request and head, a matrix S [dim, vdim] in float32 instead of keys and
values: S_t = c_h S_(t-1) + k_t v_t^T and o_t = S_t^T q_t, with no softmax and no denominator.  What surrounds the
recurrence is chosen by parameters, so that the variants in use are one part: an activation on q, k and v; a
rotation of q and k; a factor on k; a root-mean-square norm of the readout per head or over all heads, with or
without a learned weight; a gate, SiLU or logistic, computed from the same input; then the output product.  One
product yields q, k, v and the gate; one kernel walks the tokens (it activates, rotates and scales on the way in, and
carries the state in the request's slot); one kernel normalises and gates.

``mixer_sum`` runs several mixers on the same input and adds their outputs with fixed factors, in float32.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from ..config.model_spec import PartSpec
from .base import (MIXERS, POSITIONS, LayerCache, Mixer, PagedCacheSpec, ParamSpec, StateSpec, StepContext, build_part)


@MIXERS.register("decay_linear_attention")
class DecayLinearAttention(Mixer):
    """params: ``hidden_size``, ``heads``, ``head_dim``, ``value_dim``, ``decay`` (one factor in (0, 1] per head),
    ``eps``; optional ``position`` (a PartSpec, default none), ``k_scale`` (default 1), ``activation`` (``"none"``
    or ``"silu"``, on q, k and v), ``out_norm`` (``"head"``: each head's readout over its own root mean square, or
    ``"all"``: all heads together), ``out_norm_weight`` (bool: a learned weight of the readout's size), ``gate``
    (``"silu"`` or ``"sigmoid"``).
    weights: ``q|k|v|g|o.weight`` and, with ``out_norm_weight``, ``norm.weight``.
    """
    graph_safe = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.heads = int(p["heads"])
        self.head_dim = int(p["head_dim"])
        self.value_dim = int(p["value_dim"])
        self.eps = float(p["eps"])
        decay = [float(c) for c in p["decay"]]
        if self.heads <= 0 or self.head_dim <= 0 or self.value_dim <= 0:
            raise ValueError("decay_linear_attention: sizes must be positive")
        if len(decay) != self.heads or not all(0.0 < c <= 1.0 for c in decay):
            raise ValueError(f"decay_linear_attention: {self.heads} heads need as many decays in (0, 1], got {decay}")
        self.decay_values = decay
        self.k_scale = float(p.get("k_scale", 1.0))
        self.activation = str(p.get("activation", "none"))
        self.out_norm = str(p.get("out_norm", "head"))
        self.out_norm_weight = bool(p.get("out_norm_weight", False))
        self.gate = str(p.get("gate", "silu"))
        if self.activation not in ("none", "silu") or self.out_norm not in ("head", "all") or self.gate not in ("silu", "sigmoid"):
            raise ValueError(f"decay_linear_attention: activation {self.activation!r}, out_norm {self.out_norm!r} or "
                             f"gate {self.gate!r} is not known")
        self.position = build_part(POSITIONS, p.get("position", PartSpec("none")), env)
        tables = self.position.rotary_tables()
        if tables is None:
            raise ValueError("decay_linear_attention: the position encoding must be a rotation with tables, or none")
        self.cos, self.sin, self.rotary = tables
        if self.rotary > self.head_dim:
            raise ValueError("decay_linear_attention: more rotated elements than the head has")
        self.graph_safe = bool(self.position.graph_safe)
        self.q_dim = self.heads * self.head_dim
        self.o_dim = self.heads * self.value_dim
        self.decay = torch.tensor(decay, dtype=torch.float32, device=env.device)
        self.w_in: Optional[torch.Tensor] = None       # rows of q, k, v and the gate: one product
        self.w_o: Optional[torch.Tensor] = None
        self.norm_w: Optional[torch.Tensor] = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        specs = {"q.weight": ParamSpec((self.q_dim, self.hidden)), "k.weight": ParamSpec((self.q_dim, self.hidden)),
                 "v.weight": ParamSpec((self.o_dim, self.hidden)), "g.weight": ParamSpec((self.o_dim, self.hidden)),
                 "o.weight": ParamSpec((self.hidden, self.o_dim))}
        if self.out_norm_weight:
            specs["norm.weight"] = ParamSpec((self.o_dim,), role="vector")
        return specs

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.w_in = torch.cat([tensors["q.weight"], tensors["k.weight"], tensors["v.weight"], tensors["g.weight"]],
                              dim=0).contiguous()
        self.w_o = tensors["o.weight"].contiguous()
        if self.out_norm_weight:
            self.norm_w = tensors["norm.weight"].contiguous()

    def state_spec(self) -> Optional[StateSpec]:
        return StateSpec(entries=(("state", (self.heads, self.head_dim, self.value_dim)),))

    def flops(self, tokens: int, pairs: float) -> float:
        products = 2.0 * tokens * (2 * self.q_dim + 3 * self.o_dim) * self.hidden
        return products + 4.0 * tokens * self.heads * self.head_dim * self.value_dim     # state update and readout

    def inner(self, h: torch.Tensor, ctx: StepContext, cache: LayerCache, out: Optional[torch.Tensor] = None):
        ops = self.ops
        rows = ops.linear(h, self.w_in, None, ops.GEMM_STORE)
        o = ops.decay_scan(rows, 0, self.q_dim, 2 * self.q_dim, self.heads, self.head_dim, self.value_dim, self.decay,
                           cache.state["state"], ctx.slots, ctx.q_start, ctx.positions, ctx.num_seqs,
                           activation=self.activation == "silu", cos=self.cos, sin=self.sin, rotary=self.rotary,
                           k_scale=self.k_scale, max_q_len=ctx.max_q_len)
        gate = rows[:, 2 * self.q_dim + self.o_dim:]
        return ops.gated_norm(o, gate, self.norm_w, self.heads if self.out_norm == "head" else 1, self.eps,
                              sigmoid=self.gate == "sigmoid", out=out)

    def output_projection(self):
        return self.w_o, None

    def forward(self, h: torch.Tensor, ctx: StepContext, cache: LayerCache) -> torch.Tensor:
        return self.ops.linear(self.inner(h, ctx, cache), self.w_o, None, self.ops.GEMM_STORE)

    def forward_f32(self, h, ctx: StepContext, cache: LayerCache, out=None, alpha: float = 1.0, accumulate: bool = False):
        ops = self.ops
        a = self.inner(h, ctx, cache)
        if accumulate:
            return ops.linear(a, self.w_o, None, ops.GEMM_ADD_F32, out=out, alpha=alpha)
        return ops.linear(a, self.w_o, None, ops.GEMM_STORE_F32, out=out, alpha=alpha)


@MIXERS.register("mixer_sum")
class MixerSum(Mixer):
    """Several mixers side by side on the same input: out = sum_b scale_b * mixer_b(h), added up in float32.

    params: ``branches``: a list of ``(name, PartSpec, scale)``.  A branch's parameters are this part's under
    ``<name>.<local name>``, its state entries likewise; at most one branch keeps pages (they become this part's).
    Optional ``normalize`` (``{"eps": e, "hidden_size": H}``): each branch's output is first divided by its root mean
    square over the width and multiplied by a weight of its own, out = sum_b scale_b * rms(mixer_b(h)) w_b; weights
    ``<name>.out_norm.weight`` (float32 [H]).
    """

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.branches: List[Tuple[str, Mixer, float]] = []
        for name, part, scale in spec.params["branches"]:
            self.branches.append((str(name), build_part(MIXERS, part, env), float(scale)))
        if not self.branches:
            raise ValueError("mixer_sum: no branches")
        if len({name for name, _, _ in self.branches}) != len(self.branches):
            raise ValueError("mixer_sum: two branches of one name")
        paged = [name for name, mixer, _ in self.branches if mixer.cache_spec() is not None]
        if len(paged) > 1:
            raise ValueError(f"mixer_sum: branches {paged} all keep pages; one may")
        self.paged_branch = paged[0] if paged else None
        self.graph_safe = all(mixer.graph_safe for _, mixer, _ in self.branches)
        normalize = spec.params.get("normalize")
        self.normalize = None if normalize is None else (float(normalize["eps"]), int(normalize["hidden_size"]))
        self.out_norms: Dict[str, torch.Tensor] = {}

    def param_specs(self) -> Dict[str, ParamSpec]:
        specs = {f"{name}.{local}": param for name, mixer, _ in self.branches
                 for local, param in mixer.param_specs().items()}
        if self.normalize is not None:
            for name, _, _ in self.branches:
                specs[f"{name}.out_norm.weight"] = ParamSpec((self.normalize[1],), role="vector")
        return specs

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        for name, mixer, _ in self.branches:
            prefix = name + "."
            if self.normalize is not None:
                self.out_norms[name] = tensors[prefix + "out_norm.weight"].contiguous()
            mixer.load({key[len(prefix):]: t for key, t in tensors.items()
                        if key.startswith(prefix) and key != prefix + "out_norm.weight"})

    def param_bytes(self) -> int:
        return sum(mixer.param_bytes() for _, mixer, _ in self.branches)

    def flops(self, tokens: int, pairs: float) -> float:
        return sum(mixer.flops(tokens, pairs) for _, mixer, _ in self.branches)

    def cache_spec(self) -> Optional[PagedCacheSpec]:
        for _, mixer, _ in self.branches:
            if mixer.cache_spec() is not None:
                return mixer.cache_spec()
        return None

    def extra_cache_specs(self) -> Dict[str, PagedCacheSpec]:
        for name, mixer, _ in self.branches:
            if name == self.paged_branch:
                return mixer.extra_cache_specs()
        return {}

    def state_spec(self) -> Optional[StateSpec]:
        entries = []
        for name, mixer, _ in self.branches:
            state = mixer.state_spec()
            if state is not None:
                entries += [(f"{name}.{local}", shape) for local, shape in state.entries]
        return StateSpec(entries=tuple(entries)) if entries else None

    def _branch_cache(self, name: str, cache: LayerCache) -> LayerCache:
        prefix = name + "."
        view = LayerCache(owner=cache.owner)
        if name == self.paged_branch:
            view.paged, view.group, view.more = cache.paged, cache.group, cache.more
        view.state = {key[len(prefix):]: t for key, t in cache.state.items() if key.startswith(prefix)}
        return view

    def forward_f32(self, h, ctx: StepContext, cache: LayerCache, out=None, alpha: float = 1.0, accumulate: bool = False):
        if self.normalize is not None:
            if out is None or not accumulate:
                if out is None:
                    out = torch.empty((h.shape[0], self.env.hidden_size), dtype=torch.float32, device=h.device)
                out.zero_()
            self.add_normalized(h, out, ctx, cache, alpha)
            return out
        for index, (name, mixer, scale) in enumerate(self.branches):
            out = mixer.forward_f32(h, ctx, self._branch_cache(name, cache), out=out, alpha=alpha * scale,
                                    accumulate=accumulate or index > 0)
        return out

    def add_normalized(self, h, x: torch.Tensor, ctx: StepContext, cache: LayerCache, alpha: float = 1.0) -> None:
        """x += alpha * sum_b scale_b * rms(mixer_b(h)) w_b: every branch's float32 output is normalised over the width
        and added by one kernel."""
        eps = self.normalize[0]
        for name, mixer, scale in self.branches:
            y = mixer.forward_f32(h, ctx, self._branch_cache(name, cache))
            self.ops.norm_scale_add(x, y, self.out_norms[name], eps, alpha=alpha * scale)

    def forward_add(self, h: torch.Tensor, x: torch.Tensor, ctx: StepContext, cache: LayerCache, next_norm=None):
        if self.normalize is None:
            return super().forward_add(h, x, ctx, cache, next_norm=next_norm)
        self.add_normalized(h, x, ctx, cache)
        return None

    def forward(self, h: torch.Tensor, ctx: StepContext, cache: LayerCache) -> torch.Tensor:
        return self.ops.to_run_dtype(self.forward_f32(h, ctx, cache), self.env.dtype)
