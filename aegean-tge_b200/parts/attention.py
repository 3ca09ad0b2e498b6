"""Grouped-query attention over the paged cache.

In the reference's order (src/models/qwen2.cpp:2059-2103): three projections
of the normed input, then the biases, then the rotation of q and k, then the
cache write of rotated k and plain v, then for every query head ``h`` causal
softmax attention against kv head ``h // group`` with scores
``dot(q, k) * head_dim**-0.5`` (src/cpu/scalar/attention_scalar.cpp:48-115),
then the output projection added to the stream.  Here q, k and v are one
product over row-concatenated weights with the bias in its epilogue, the
rotation and the cache write are one kernel, and the output projection adds
into the float32 stream in its epilogue.

Options that other designs add, all off by default: values of a size of
their own (``value_dim``); an RMS norm of q and of k before the scores,
over each head or over a token's whole projection (``qk_norm``); a sink, one
learned score per head that joins the softmax's denominator with no key or
value behind it (``sinks``); and a blend of the values with those that an
earlier layer computed for the same token (``value_mix``).  With a norm or a
blend, one kernel normalises, blends and stores after the q/k/v product.

Two more, for designs that bound what a request keeps: a short causal
convolution over time on every channel of q, k and v right after the
projection (``short_conv``; its last inputs are per-request state), and,
with a window, pooled blocks (``pool``): beside the window's tokens a query
sees the mean key and mean value of every block of that many positions that
lies wholly before the window.  The pooled entries live in pages of their
own, one entry per block, so the tokens' pages can be given back once the
window and the block in the making have passed them.  Either option, or a
rotation with values of another size than the keys, takes the general path:
product, then one kernel that convolves, normalises, rotates and stores,
one that pools, and the attention.

Three more, which go together (the *keyed* path): the values are the keys as
projected (``values: "keys"``: no value weight; with a q/k norm the values are
the keys from before it, so both are stored); a temperature on the queries
that grows with the position (``q_temp``: q times 1 + coef ln(floor((p + 1) /
every) + 1)); and a learned bias by distance (``distance_bias``), a table
[rows, heads] added unscaled to the scaled scores: distances below rows/2
have a row each, beyond that the rows are spaced evenly in the logarithm up
to ``far``, where the last row is reached and kept.  Product of q and k with
the biases, one kernel that stores the values, normalises, applies the
temperature and stores the keys, then the attention with the bias expanded
to one entry per distance.
"""
from __future__ import annotations

import math
from typing import Dict, Optional

import torch

from ..config.model_spec import PartSpec
from .base import (MIXERS, POSITIONS, LayerCache, Mixer, PagedCacheSpec, ParamSpec, StateSpec, StepContext, build_part)


@MIXERS.register("gqa_attention")
class GQAttention(Mixer):
    """params: ``hidden_size``, ``heads``, ``kv_heads``, ``head_dim``,
    ``qkv_bias`` (bool), ``o_bias`` (bool), ``window`` (None or tokens),
    ``position`` (a PartSpec), optional ``scale``; optional ``value_dim`` (default ``head_dim``),
    ``qk_norm`` (None, or ``{"scope": "projection" | "head", "eps": e}``), ``sinks`` (bool),
    ``value_mix`` (None, ``"first"``: this layer's values are kept for the step under ``value_mix_key``, or
    ``"blend"``: v <- (1 - w) v + w v_first with the learned scalar w); ``short_conv`` (None or the number of taps),
    ``pool`` (None or the pooled blocks' size; needs a window), ``prepare_in_one_kernel`` (bool: take the general path,
    one kernel between the product and the attention, whatever the options).
    weights: ``q|k|v|o.weight`` and, with the bias flags, ``q|k|v|o.bias``; ``q_norm.weight`` / ``k_norm.weight``
    (float32, the projection's or one head's size); ``sink`` [heads]; ``value_mix.weight`` (a scalar);
    ``q|k|v.conv.weight`` (float32 [channels, taps]).
    The keyed path: ``values`` (``"own"``, the default, or ``"keys"``: no ``v.weight`` / ``v.bias``), ``q_temp`` (None
    or ``{"coef": c, "every": n}``), ``distance_bias`` (None or ``{"far": D}``; weight ``rel`` float32 [rows, heads], the
    rows taken from the tensor).
    """
    graph_safe = True
    can_defer_norm = True
    takes_deferred_rows = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.heads = int(p["heads"])
        self.kv_heads = int(p["kv_heads"])
        self.head_dim = int(p["head_dim"])
        self.qkv_bias = bool(p.get("qkv_bias", False))
        self.o_bias = bool(p.get("o_bias", False))
        self.window = p.get("window")
        if self.heads <= 0 or self.kv_heads <= 0 or self.heads % self.kv_heads:
            raise ValueError(f"attention: {self.heads} heads are not a multiple of {self.kv_heads} kv heads")
        if self.window is not None and int(self.window) <= 0:
            raise ValueError("attention: a window must be positive")
        self.scale = float(p.get("scale", self.head_dim ** -0.5))
        self.value_dim = int(p.get("value_dim", self.head_dim))
        norm = p.get("qk_norm")
        self.qk_norm = None if norm is None else (str(norm["scope"]), float(norm["eps"]))
        if self.qk_norm is not None and (self.qk_norm[0] not in ("projection", "head") or not self.qk_norm[1] > 0.0):
            raise ValueError(f"attention: qk_norm {norm!r} needs scope 'projection' or 'head' and a positive eps")
        self.sinks = bool(p.get("sinks", False))
        self.value_mix = p.get("value_mix")
        if self.value_mix not in (None, "first", "blend"):
            raise ValueError(f"attention: value_mix {self.value_mix!r} is none of None, 'first', 'blend'")
        self.value_mix_key = ("value_mix", str(p.get("value_mix_key", "values")))
        if self.value_dim <= 0:
            raise ValueError("attention: value_dim must be positive")
        self.values_are_keys = str(p.get("values", "own")) == "keys"
        if str(p.get("values", "own")) not in ("own", "keys"):
            raise ValueError(f"attention: values {p.get('values')!r} are 'own' or 'keys'")
        temp, dist = p.get("q_temp"), p.get("distance_bias")
        self.q_temp = None if temp is None else (float(temp["coef"]), int(temp["every"]))
        self.dist_far = None if dist is None else float(dist["far"])
        if self.q_temp is not None and self.q_temp[1] <= 0:
            raise ValueError("attention: q_temp.every must be positive")
        if (self.q_temp is not None or self.dist_far is not None) and not self.values_are_keys:
            raise ValueError("attention: a query temperature and a bias by distance are built for values that are the keys")
        self.dist_table: Optional[torch.Tensor] = None
        self.taps = int(p.get("short_conv") or 0)
        self.pool = int(p.get("pool") or 0)
        if self.taps < 0 or self.taps > 16:
            raise ValueError(f"attention: a short convolution has 1 to 16 taps, not {self.taps}")
        if self.pool < 0 or (self.pool and self.window is None):
            raise ValueError("attention: pooled blocks need a positive size and a window")
        position: PartSpec = p.get("position", PartSpec("none"))
        self.position = build_part(POSITIONS, position, env)
        self.graph_safe = bool(self.position.graph_safe)
        self.q_dim = self.heads * self.head_dim
        self.kv_dim = self.kv_heads * self.head_dim
        self.v_dim = self.kv_heads * self.value_dim
        self.o_dim = self.heads * self.value_dim
        # the plain layer: rotation, store and attention as the fused kernels know them
        self.plain = (self.qk_norm is None and self.value_mix is None and self.value_dim == self.head_dim
                      and not self.values_are_keys)
        tables = self.position.rotary_tables()
        self.rotates = tables is None or tables[2] > 0
        if self.values_are_keys:
            if (self.value_dim != self.head_dim or self.rotates or self.value_mix is not None or self.taps or self.pool
                    or p.get("prepare_in_one_kernel") or (self.qk_norm is not None and self.qk_norm[0] != "head")):
                raise ValueError("attention: values that are the keys go with equal sizes, no rotation, a per-head q/k norm "
                                 "or none, and neither convolution, pooled blocks nor value mixing")
            self.v_dim = 0
        # the general path: convolution, per-head norm, rotation and store in one kernel, pooled blocks
        self.general = bool(p.get("prepare_in_one_kernel") or self.taps or self.pool
                            or (self.value_dim != self.head_dim and self.rotates))
        if self.general:
            if self.value_mix is not None or self.qkv_bias or (self.qk_norm is not None and self.qk_norm[0] != "head"):
                raise ValueError("attention: a short convolution, pooled blocks, or a rotation with values of their own "
                                 "size go with a per-head q/k norm or none, without biases on q, k, v or value mixing")
            if tables is None:
                raise ValueError("attention: the general path rotates by tables, or not at all")
        self.conv_w: Optional[torch.Tensor] = None
        self.q_norm_w: Optional[torch.Tensor] = None
        self.k_norm_w: Optional[torch.Tensor] = None
        self.sink: Optional[torch.Tensor] = None
        self.mix_w: Optional[torch.Tensor] = None
        # q/k/v rows and, below them, rows that a block placed there (a feed-forward's up rows), in one tensor
        self.w_shared: Optional[torch.Tensor] = None
        self.w_qkv: Optional[torch.Tensor] = None
        self.b_qkv: Optional[torch.Tensor] = None
        self.w_o: Optional[torch.Tensor] = None
        self.b_o: Optional[torch.Tensor] = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        specs = {
            "q.weight": ParamSpec((self.q_dim, self.hidden)),
            "k.weight": ParamSpec((self.kv_dim, self.hidden)),
            "v.weight": ParamSpec((self.v_dim, self.hidden)),
            "o.weight": ParamSpec((self.hidden, self.o_dim)),
        }
        if self.values_are_keys:
            del specs["v.weight"]
        if self.dist_far is not None:
            specs["rel"] = ParamSpec((-1, self.heads), role="vector")
        if self.qk_norm is not None:
            per_head = self.qk_norm[0] == "head"
            specs["q_norm.weight"] = ParamSpec((self.head_dim if per_head else self.q_dim,), role="vector")
            specs["k_norm.weight"] = ParamSpec((self.head_dim if per_head else self.kv_dim,), role="vector")
        if self.sinks:
            specs["sink"] = ParamSpec((self.heads,), role="vector")
        if self.value_mix is not None or "value_mix.weight" in self.spec.weights:
            # only a blending layer uses the scalar; a checkpoint may hold one for the other layers too (the first
            # of a chain, layers that do not mix), so a model spec may name it for them and it is then optional
            specs["value_mix.weight"] = ParamSpec((), role="vector", optional=self.value_mix != "blend")
        if self.taps:
            specs["q.conv.weight"] = ParamSpec((self.q_dim, self.taps), role="vector")
            specs["k.conv.weight"] = ParamSpec((self.kv_dim, self.taps), role="vector")
            specs["v.conv.weight"] = ParamSpec((self.v_dim, self.taps), role="vector")
        if self.qkv_bias:
            specs["q.bias"] = ParamSpec((self.q_dim,), role="vector")
            specs["k.bias"] = ParamSpec((self.kv_dim,), role="vector")
            if not self.values_are_keys:
                specs["v.bias"] = ParamSpec((self.v_dim,), role="vector")
        if self.o_bias:
            specs["o.bias"] = ParamSpec((self.hidden,), role="vector")
        return specs

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        # rows of q, then k, then v: one product serves all three
        rows = ("q", "k") if self.values_are_keys else ("q", "k", "v")
        self.w_qkv = torch.cat([tensors[f"{t}.weight"] for t in rows], dim=0).contiguous()
        if self.qkv_bias:
            self.b_qkv = torch.cat([tensors[f"{t}.bias"] for t in rows]).contiguous()
        if self.dist_far is not None:
            self.dist_table = self.expand_distance_bias(tensors["rel"], self.dist_far)
        self.w_o = tensors["o.weight"].contiguous()
        self.b_o = tensors["o.bias"].contiguous() if self.o_bias else None
        if self.qk_norm is not None:
            self.q_norm_w = tensors["q_norm.weight"].contiguous()
            self.k_norm_w = tensors["k_norm.weight"].contiguous()
        if self.sinks:
            self.sink = tensors["sink"].contiguous()
        if self.taps:
            self.conv_w = torch.cat([tensors["q.conv.weight"], tensors["k.conv.weight"], tensors["v.conv.weight"]],
                                    dim=0).contiguous()
        if self.value_mix == "blend":
            self.mix_w = tensors["value_mix.weight"].reshape(1).contiguous()

    @staticmethod
    def distance_row(n: int, rows: int, far: float) -> int:
        """The table row of distance n: n itself below rows/2; beyond, rows/2 + floor(ln(n / (rows/2)) / ln(far /
        (rows/2)) * (rows - rows/2)), and never past the last row (rows/2 a whole number, rounded down)."""
        half = rows // 2
        if n < half:
            return n
        return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))

    @classmethod
    def expand_distance_bias(cls, rel: torch.Tensor, far: float) -> torch.Tensor:
        """``rel`` [rows, heads] -> float32 [heads, span], one entry per distance up to the first that reaches the last
        row (every larger distance shares it): what the attention kernels index by min(distance, span - 1)."""
        rows = rel.shape[0]
        if rows < 2 or not far > rows // 2:
            raise ValueError(f"attention: a bias by distance needs two rows or more (got {rows}) and far > rows/2 (got {far})")
        picks = []
        n = 0
        while True:
            picks.append(cls.distance_row(n, rows, far))
            if picks[-1] == rows - 1:
                break
            n += 1
        index = torch.tensor(picks, dtype=torch.long, device=rel.device)
        return rel.float()[index].t().contiguous()

    def flops(self, tokens: int, pairs: float) -> float:
        products = 2.0 * tokens * (self.q_dim + self.kv_dim + self.v_dim + self.o_dim) * self.hidden
        return products + 2.0 * self.heads * (self.head_dim + self.value_dim) * pairs     # scores and weighted values

    def attend_keyed(self, h, ctx: StepContext, cache: LayerCache, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Product of q and k; values stored, q and k normalised, temperature, keys stored; attention."""
        ops = self.ops
        complete = getattr(h, "complete", None)
        if complete is not None:
            h = complete()
        k_pages, v_pages = cache.paged["k"], cache.paged["v"]
        table = ctx.block_tables[cache.group]
        qk = ops.linear(h, self.w_qkv, self.b_qkv, ops.GEMM_STORE)
        coef, every = self.q_temp if self.q_temp is not None else (0.0, 0)
        ops.qk_temp_store(qk, self.q_norm_w, self.k_norm_w, self.qk_norm[1] if self.qk_norm else 1.0, coef, every,
                          ctx.positions, ctx.seq_of_token, table if cache.owner else None, k_pages if cache.owner else None,
                          v_pages if cache.owner else None, self.heads, self.kv_heads, self.head_dim)
        return ops.attention(qk[:, :self.q_dim], k_pages, v_pages, table, ctx.q_start, ctx.start_pos, ctx.positions,
                             ctx.seq_of_token, ctx.num_seqs, ctx.max_q_len, ctx.max_ctx_len, self.heads, self.kv_heads,
                             self.head_dim, self.scale, window=int(self.window or 0), split_tokens=ctx.attn_split_tokens,
                             typical_ctx_len=ctx.typical_ctx_len, decode_prefix=ctx.decode_prefix, sink=self.sink, out=out,
                             dist_bias=self.dist_table)

    def cache_spec(self) -> Optional[PagedCacheSpec]:
        # with pooled blocks a token is also read when its block is averaged, which is when the block's last token
        # arrives: the pages keep whichever reaches further back, the window or a block
        window = None if self.window is None else max(int(self.window), self.pool)
        return PagedCacheSpec(entries=(("k", (self.kv_heads, self.head_dim)), ("v", (self.kv_heads, self.value_dim))),
                              window=window)

    def extra_cache_specs(self) -> Dict[str, PagedCacheSpec]:
        if not self.pool:
            return {}
        return {"pooled": PagedCacheSpec(entries=(("k", (self.kv_heads, self.head_dim)), ("v", (self.kv_heads, self.value_dim))),
                                         window=None, stride=self.pool)}

    def state_spec(self) -> Optional[StateSpec]:
        if self.taps > 1:
            return StateSpec(entries=(("conv", (self.taps - 1, self.q_dim + self.kv_dim + self.v_dim)),))
        return None

    def attend_general(self, h, ctx: StepContext, cache: LayerCache, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Product; convolution, per-head norm, rotation and store; pooled blocks; attention."""
        ops = self.ops
        k_pages, v_pages = cache.paged["k"], cache.paged["v"]
        table = ctx.block_tables[cache.group]
        cos, sin, rotary = self.position.rotary_tables()
        raw = ops.linear(h, self.w_qkv, None, ops.GEMM_STORE)
        q = ops.conv_norm_rope_store(raw, self.conv_w, self.taps, cache.state.get("conv"), ctx.slots, ctx.q_start,
                                     ctx.num_seqs, self.q_norm_w, self.k_norm_w, self.qk_norm[1] if self.qk_norm else 1.0,
                                     cos, sin, rotary, ctx.positions, ctx.seq_of_token, table,
                                     k_pages if cache.owner else None, v_pages if cache.owner else None,
                                     self.heads, self.kv_heads, self.head_dim, self.value_dim)
        pooled = {}
        if self.pool:
            more = cache.more["pooled"]
            pool_table = ctx.block_tables[more.group]
            if cache.owner:
                ops.pool_kv(k_pages, v_pages, table, more.paged["k"], more.paged["v"], pool_table, ctx.positions,
                            ctx.seq_of_token, self.pool)
            pooled = {"pool": self.pool, "pooled_k": more.paged["k"], "pooled_v": more.paged["v"], "pool_table": pool_table}
        return ops.attention(q, k_pages, v_pages, table, ctx.q_start, ctx.start_pos, ctx.positions, ctx.seq_of_token,
                             ctx.num_seqs, ctx.max_q_len, ctx.max_ctx_len, self.heads, self.kv_heads, self.head_dim,
                             self.scale, window=int(self.window or 0), split_tokens=ctx.attn_split_tokens,
                             typical_ctx_len=ctx.typical_ctx_len, decode_prefix=ctx.decode_prefix, sink=self.sink,
                             out=out, **pooled)

    def share_input_projection(self, rows: torch.Tensor) -> Optional[torch.Tensor]:
        """A block offers the rows of another product over the same input (a feed-forward's up weight) to be
        multiplied together with q, k and v.  A mixer whose small-batch kernel can carry them (whole-projection
        q/k norm, no rotation, no biases) puts them below its own rows in one tensor and returns the view that now
        holds them (the caller uses it in place of its copy); None: it cannot."""
        if (self.plain or self.general or self.values_are_keys or self.rotates or self.qkv_bias
                or (self.qk_norm is not None and self.qk_norm[0] != "projection")):
            return None
        if self.w_qkv is None or rows.dtype != self.w_qkv.dtype or rows.shape[1] != self.hidden:
            return None
        count = self.w_qkv.shape[0]
        self.w_shared = torch.cat([self.w_qkv, rows], dim=0).contiguous()
        self.w_qkv = self.w_shared[:count]
        return self.w_shared[count:]

    def attend(self, h: torch.Tensor, ctx: StepContext, cache: LayerCache,
               out: Optional[torch.Tensor] = None, beside=None):
        """Everything up to, not including, the output projection: [T, heads*value_dim] (into ``out`` if given).

        ``beside``: (output view, epilogue) for the rows that :meth:`share_input_projection` took in; the result is
        then a pair (rows, whether the shared rows were multiplied and activated here)."""
        if self.general or self.values_are_keys:
            a = (self.attend_keyed if self.values_are_keys else self.attend_general)(h, ctx, cache, out=out)
            return a if beside is None else (a, False)
        ops = self.ops
        k_pages, v_pages = cache.paged["k"], cache.paged["v"]
        table = ctx.block_tables[cache.group]
        tables = self.position.rotary_tables()
        did_beside = False
        if not self.plain:
            other = blend = None
            if self.value_mix == "blend":
                if self.value_mix_key not in ctx.scratch:
                    raise RuntimeError("attention: no earlier layer of this step left values to blend with")
                other, blend = ctx.scratch[self.value_mix_key], self.mix_w
            store_here = cache.owner and not self.rotates     # a rotated layer stores after its rotation
            q_w, k_w, eps, per_head = self.q_norm_w, self.k_norm_w, 1.0, False
            if self.qk_norm is not None:
                per_head, eps = self.qk_norm[0] == "head", self.qk_norm[1]
            qkv = None
            if not per_head and not self.rotates and self.b_qkv is None:
                # small batches: the product's partial sums are added, normalised, blended and stored by one kernel
                shared = beside is not None and self.w_shared is not None
                qkv = ops.linear_qkv_norm_act_store(
                    h, self.w_shared if shared else self.w_qkv, self.heads, self.kv_heads, self.head_dim, self.value_dim,
                    q_w, k_w, eps, ctx.positions, ctx.seq_of_token, table if store_here else None,
                    k_pages if store_here else None, v_pages if store_here else None, v_other=other, blend=blend,
                    act_out=beside[0] if shared else None, activation=beside[1] if shared else ops.GEMM_GELU)
                did_beside = shared and qkv is not None
            if qkv is None:
                qkv = ops.linear(h, self.w_qkv, self.b_qkv, ops.GEMM_STORE)
                ops.qk_norm_kv_store(qkv, q_w, k_w, eps, per_head, ctx.positions, ctx.seq_of_token,
                                     table if store_here else None, k_pages if store_here else None,
                                     v_pages if store_here else None, self.heads, self.kv_heads, self.head_dim,
                                     self.value_dim, v_other=other, blend=blend)
            if self.value_mix == "first":
                ctx.scratch[self.value_mix_key] = qkv[:, self.q_dim + self.kv_dim:self.q_dim + self.kv_dim + self.v_dim]
            if self.rotates:
                if tables is None:
                    q = qkv[:, :self.q_dim].view(-1, self.heads, self.head_dim)
                    k = qkv[:, self.q_dim:self.q_dim + self.kv_dim].view(-1, self.kv_heads, self.head_dim)
                    self.position.apply(q, k, ctx.positions)
                    cos = sin = None
                    rotary = 0
                else:
                    cos, sin, rotary = tables
                ops.rope_kv_store(qkv, cos, sin, rotary, ctx.positions, ctx.seq_of_token, table,
                                  k_pages if cache.owner else None, v_pages if cache.owner else None,
                                  self.heads, self.kv_heads, self.head_dim)
        elif tables is not None and cache.owner:
            # product, bias, rotation and cache store together (one or two kernels, chosen by batch size)
            cos, sin, rotary = tables
            qkv = ops.linear_qkv_rope_store(h, self.w_qkv, self.b_qkv, cos, sin, rotary, ctx.positions,
                                            ctx.seq_of_token, table, k_pages, v_pages, self.heads, self.kv_heads,
                                            self.head_dim)
        else:
            qkv = ops.linear(h, self.w_qkv, self.b_qkv, ops.GEMM_STORE)
            if tables is None:
                q = qkv[:, :self.q_dim].view(-1, self.heads, self.head_dim)
                k = qkv[:, self.q_dim:self.q_dim + self.kv_dim].view(-1, self.kv_heads, self.head_dim)
                self.position.apply(q, k, ctx.positions)
                cos = sin = None
                rotary = 0
            else:
                cos, sin, rotary = tables
            ops.rope_kv_store(qkv, cos, sin, rotary, ctx.positions, ctx.seq_of_token, table,
                              k_pages if cache.owner else None, v_pages if cache.owner else None,
                              self.heads, self.kv_heads, self.head_dim)
        a = ops.attention(qkv[:, :self.q_dim], k_pages, v_pages, table, ctx.q_start, ctx.start_pos, ctx.positions,
                          ctx.seq_of_token, ctx.num_seqs, ctx.max_q_len, ctx.max_ctx_len, self.heads,
                          self.kv_heads, self.head_dim, self.scale, window=int(self.window or 0),
                          split_tokens=ctx.attn_split_tokens, typical_ctx_len=ctx.typical_ctx_len,
                          decode_prefix=ctx.decode_prefix, sink=self.sink, out=out)
        return a if beside is None else (a, did_beside)

    def inner(self, h, ctx: StepContext, cache: LayerCache, out: Optional[torch.Tensor] = None, beside=None):
        return self.attend(h, ctx, cache, out=out, beside=beside)

    def output_projection(self):
        return self.w_o, self.b_o

    def forward(self, h: torch.Tensor, ctx: StepContext, cache: LayerCache) -> torch.Tensor:
        return self.ops.linear(self.attend(h, ctx, cache), self.w_o, self.b_o, self.ops.GEMM_STORE)

    def forward_f32(self, h, ctx: StepContext, cache: LayerCache, out=None, alpha: float = 1.0, accumulate: bool = False):
        a = self.attend(h, ctx, cache)
        epilogue = self.ops.GEMM_ADD_F32 if accumulate else self.ops.GEMM_STORE_F32
        return self.ops.linear(a, self.w_o, self.b_o, epilogue, out=out, alpha=alpha)

    def forward_add(self, h: torch.Tensor, x: torch.Tensor, ctx: StepContext, cache: LayerCache, next_norm=None,
                    defer: bool = False):
        a = self.attend(h, ctx, cache)
        fused = next_norm.fusable() if next_norm is not None else None
        if fused is not None:
            return self.ops.linear_add_norm(a, self.w_o, self.b_o, x, fused[0], fused[1], self.env.dtype, defer=defer)
        self.ops.linear(a, self.w_o, self.b_o, self.ops.GEMM_ADD_F32, out=x)
        return None
