"""Attention over a latent cache, and the token-shift wrapper of a mixer.

**Latent attention.**  Queries and keys/values both pass through a narrow latent.  With h the mixer's input:

    cq = rms(Wdq h) gq                     q = Wuq cq              per head [dim plain | rot rotated]
    [c_raw | kr] = Wdkv h                  c = rms(c_raw) gkv      kr: one rotated key part for all heads
    k_n = [Wuk_n c | kr]                   v_n = Wuv_n c
    s_ij = scale (q_i . k_j),  j <= i      softmax, o = sum_j p_ij v_j
    out = Wo (gate * o)                    gate = sigmoid(Wg h), one per head or one per element, or none

A token keeps only ``[c | kr]`` (kv_rank + rot numbers, one cache entry, whatever the head count).  The keys and
values are never materialised: the query's plain part is carried into the latent space, q~_n = Wuk_n^T q_n, so that
s_ij = scale (q~_n . c_j + qr_n . kr_j), the paged attention kernels run with ONE key/value head whose keys are the
entries and whose values are the entries' first kv_rank numbers, and the attended latent returns through Wuv_n.  The
kernels between the products: ``latent_prepare`` (both norms, rotation and store of the shared key part, gate),
``head_linear`` (the two per-head products, the second with the gate), ``rotate_interleaved`` (the queries'
rotated part).

Long prompt portions go another way (``expand_keys``): there many queries meet every key, and attention with one
key/value head of kv_rank + rot numbers costs more per pair than attention with every head's own keys of dim + rot
and values of vdim.  So the latents of all positions the step's requests hold are gathered from the cache
(``latent_gather``), one product with [Wuk; Wuv] gives every head's plain key parts and values, ``latent_scatter`` puts
them into pages of the step's own beside the shared key part, and the ordinary paged attention runs with as many
key/value heads as heads; the queries then need no Wuk and the attended rows no Wuv, only the gate (``gate_rows``).
Both ways compute the same sums in another order.  A layer may read another layer's entries (``LayerSpec.cache_from``; param ``shared_kv``): it then has
no Wdkv and stores nothing.

**Token shift.**  ``shifted_mixer`` wraps any mixer: what the inner mixer reads is h_t + (h_(t-1) - h_t) * mu, element
by element, with h_(t-1) the previous token's input as it arrived (zeros before the first token).  The last input
of a request is per-request state, so portions and single tokens continue where the step before stopped.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..config.model_spec import PartSpec
from .base import (MIXERS, POSITIONS, LayerCache, Mixer, PagedCacheSpec, ParamSpec, StateSpec, StepContext, build_part)


_EXPANDED: Dict[tuple, tuple] = {}      # the steps' own key and value pages, per device and geometry
_SMS: Dict[int, int] = {}


def _sm_count(device) -> int:
    index = device.index if device.index is not None else torch.cuda.current_device()
    if index not in _SMS:
        _SMS[index] = int(torch.cuda.get_device_properties(index).multi_processor_count)
    return _SMS[index]


@MIXERS.register("latent_attention")
class LatentAttention(Mixer):
    """params: ``hidden_size``, ``heads``, ``head_dim`` (plain query/key numbers per head), ``rope_dim`` (rotated
    ones), ``value_dim``, ``q_rank``, ``kv_rank``, ``scale``, ``eps`` (of the two latent norms), ``gate`` (``"none"``,
    ``"head"`` or ``"element"``), ``position`` (a PartSpec that offers ``pair_tables()``: the rotation of the rope_dim
    part), ``shared_kv`` (bool: the entries are another layer's), ``expand_keys`` (``"auto"``: every head's own keys
    and values for steps with long portions, where the tensor-core attention takes the sizes; ``"never"``;
    ``"always"``).
    weights: ``dq|uq|dkv|uk|uv|g|o.weight``, ``dq_norm.weight``, ``dkv_norm.weight`` (float32)."""
    graph_safe = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.heads = int(p["heads"])
        self.dim = int(p["head_dim"])
        self.rot = int(p["rope_dim"])
        self.vdim = int(p["value_dim"])
        self.q_rank = int(p["q_rank"])
        self.kv_rank = int(p["kv_rank"])
        self.scale = float(p["scale"])
        self.eps = float(p["eps"])
        self.gate = str(p.get("gate", "none"))
        self.shared_kv = bool(p.get("shared_kv", False))
        self.expand_keys = str(p.get("expand_keys", "auto"))
        if self.expand_keys not in ("auto", "never", "always"):
            raise ValueError(f"latent_attention: expand_keys {self.expand_keys!r} is none of 'auto', 'never', 'always'")
        if min(self.hidden, self.heads, self.dim, self.vdim, self.q_rank, self.kv_rank) <= 0 or self.rot < 0:
            raise ValueError("latent_attention: sizes must be positive")
        if self.gate not in ("none", "head", "element"):
            raise ValueError(f"latent_attention: gate {self.gate!r} is none of 'none', 'head', 'element'")
        if not self.eps > 0.0:
            raise ValueError("latent_attention: eps must be positive")
        if self.kv_rank + self.rot > 256:
            raise ValueError(f"latent_attention: entries of {self.kv_rank} + {self.rot} numbers exceed the 256 the "
                             f"attention kernels take")
        position: PartSpec = p.get("position", PartSpec("none"))
        self.position = build_part(POSITIONS, position, env)
        tables = getattr(self.position, "pair_tables", None)
        if self.rot and tables is None and position.kind != "none":
            raise ValueError(f"latent_attention: position encoding '{position.kind}' offers no tables of neighbouring pairs")
        self.cos, self.sin, self.rot_dims = tables() if (tables is not None and self.rot) else (None, None, 0)
        if self.rot_dims > self.rot:
            raise ValueError("latent_attention: more rotated numbers than the rotated part holds")
        self.graph_safe = bool(self.position.graph_safe)
        self.gate_n = {"none": 0, "head": self.heads, "element": self.heads * self.vdim}[self.gate]
        self.entry = self.kv_rank + self.rot
        self.w_in: Optional[torch.Tensor] = None        # rows [Wdq; Wdkv; Wg]: one product over the input
        self.w_uq: Optional[torch.Tensor] = None
        self.w_uk_t: Optional[torch.Tensor] = None      # [heads, kv_rank, dim]: queries into the latent space
        self.w_uv: Optional[torch.Tensor] = None        # [heads, vdim, kv_rank]: attended latents to values
        self.w_ukv: Optional[torch.Tensor] = None       # rows [Wuk; Wuv]: latents to every head's keys and values
        self.w_o: Optional[torch.Tensor] = None
        self.q_norm_w: Optional[torch.Tensor] = None
        self.kv_norm_w: Optional[torch.Tensor] = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        specs = {
            "dq.weight": ParamSpec((self.q_rank, self.hidden)),
            "dq_norm.weight": ParamSpec((self.q_rank,), role="vector"),
            "uq.weight": ParamSpec((self.heads * (self.dim + self.rot), self.q_rank)),
            "uk.weight": ParamSpec((self.heads * self.dim, self.kv_rank)),
            "uv.weight": ParamSpec((self.heads * self.vdim, self.kv_rank)),
            "o.weight": ParamSpec((self.hidden, self.heads * self.vdim)),
        }
        if not self.shared_kv:
            specs["dkv.weight"] = ParamSpec((self.kv_rank + self.rot, self.hidden))
            specs["dkv_norm.weight"] = ParamSpec((self.kv_rank,), role="vector")
        if self.gate_n:
            specs["g.weight"] = ParamSpec((self.gate_n, self.hidden))
        return specs

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        rows = [tensors["dq.weight"]]
        if not self.shared_kv:
            rows.append(tensors["dkv.weight"])
            self.kv_norm_w = tensors["dkv_norm.weight"].contiguous()
        if self.gate_n:
            rows.append(tensors["g.weight"])
        self.w_in = torch.cat(rows, dim=0).contiguous()
        self.q_norm_w = tensors["dq_norm.weight"].contiguous()
        self.w_uq = tensors["uq.weight"].contiguous()
        self.w_uk_t = tensors["uk.weight"].view(self.heads, self.dim, self.kv_rank).transpose(1, 2).contiguous()
        self.w_uv = tensors["uv.weight"].view(self.heads, self.vdim, self.kv_rank).contiguous()
        self.w_ukv = torch.cat([tensors["uk.weight"], tensors["uv.weight"]], dim=0).contiguous()
        self.w_o = tensors["o.weight"].contiguous()

    def flops(self, tokens: int, pairs: float) -> float:
        in_rows = self.q_rank + (0 if self.shared_kv else self.entry) + self.gate_n
        products = 2.0 * tokens * (in_rows * self.hidden + self.heads * (self.dim + self.rot) * self.q_rank
                                   + self.heads * self.kv_rank * (self.dim + self.vdim) + self.heads * self.vdim * self.hidden)
        # per query-key pair: every head's own keys and values (what long portions run) or the entries as one head
        return products + 2.0 * self.heads * min(self.entry + self.kv_rank, self.dim + self.rot + self.vdim) * pairs

    def cache_spec(self) -> Optional[PagedCacheSpec]:
        return PagedCacheSpec(entries=(("kv", (1, self.entry)),), window=None)

    def attend(self, h: torch.Tensor, ctx: StepContext, cache: LayerCache, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Everything up to, not including, the output projection: the gated heads [T, heads * value_dim]."""
        ops = self.ops
        tokens = h.shape[0]
        pages = cache.paged["kv"]
        table = ctx.block_tables[cache.group]
        dtype = self.env.dtype
        own = not self.shared_kv
        raw = ops.linear(h, self.w_in, None, ops.GEMM_STORE_F32)
        q_latent, gate = ops.latent_prepare(raw, self.q_rank, self.kv_rank, self.rot, self.gate_n, own, self.q_norm_w,
                                            self.kv_norm_w, self.eps, self.cos, self.sin, self.rot_dims, ctx.positions,
                                            ctx.seq_of_token, table, pages if (own and cache.owner) else None, dtype)
        q = ops.linear(q_latent, self.w_uq, None, ops.GEMM_STORE)
        per_head = self.dim + self.rot
        if self.expands(ctx, pages):
            return self.attend_expanded(q, gate, ctx, pages, table, out)
        queries = torch.empty((tokens, self.heads * self.entry), dtype=dtype, device=h.device)
        ops.head_linear(q, per_head, self.w_uk_t, queries, self.entry)
        if self.rot:
            ops.rotate_interleaved(q[:, self.dim:], per_head, queries[:, self.kv_rank:], self.entry, self.heads, self.rot,
                                   self.cos, self.sin, self.rot_dims, ctx.positions)
        # single tokens: the decode kernels take the heads that share a key/value head as the rows of one tile of 16,
        # so more heads than that go in equal runs of up to 16 (the entries are few bytes; reading them twice is cheap)
        single = ctx.max_q_len <= 1 and dtype == torch.bfloat16
        runs = -(-self.heads // 16) if single else 1
        size = -(-self.heads // runs)
        split = ctx.attn_split_tokens
        if single and split == 0 and self.entry > 128:
            # entries this wide leave room for one block of the decode kernel per SM, so the keys are cut into just
            # enough runs to give every SM a block, not into the many short ones that suit narrow heads
            bound = max(ctx.typical_ctx_len or ctx.max_ctx_len, 1)
            want = max(_sm_count(h.device) // max(ctx.num_seqs, 1), 1)
            split = max(64 * -(-(-(-bound // want)) // 64), 128)
        attended = torch.empty((tokens, self.heads * self.kv_rank), dtype=dtype, device=h.device)
        for lo in range(0, self.heads, size):
            n = min(size, self.heads - lo)
            ops.attention(queries[:, lo * self.entry:(lo + n) * self.entry], pages, None, table, ctx.q_start, ctx.start_pos,
                          ctx.positions, ctx.seq_of_token, ctx.num_seqs, ctx.max_q_len, ctx.max_ctx_len, n, 1, self.entry,
                          self.scale, split_tokens=split, typical_ctx_len=ctx.typical_ctx_len,
                          decode_prefix=ctx.decode_prefix, values_in_keys=self.kv_rank,
                          out=attended[:, lo * self.kv_rank:(lo + n) * self.kv_rank])
        if out is None:
            out = torch.empty((tokens, self.heads * self.vdim), dtype=dtype, device=h.device)
        mode = {"none": 0, "head": 1, "element": 2}[self.gate]
        return ops.head_linear(attended, self.kv_rank, self.w_uv, out, self.vdim, gate if mode else None, mode)

    def expands(self, ctx: StepContext, pages: torch.Tensor) -> bool:
        """Whether this step gives every head its own keys and values: long portions that between them bring a fair
        share of the positions whose keys they read (each position's keys cost a product row; each query-key pair
        saves a little)."""
        if self.expand_keys == "never" or not ctx.host_q_lens or len(ctx.host_start_pos) != len(ctx.host_q_lens):
            return False
        if self.expand_keys == "always":
            return True
        held = sum(s + n for s, n in zip(ctx.host_start_pos, ctx.host_q_lens))
        return (self.env.dtype == torch.bfloat16 and ctx.max_q_len >= 32 and held <= 16 * ctx.num_tokens
                and self.ops.mma_attention_supports(self.dim + self.rot, self.heads, self.heads, pages.shape[2], self.vdim))

    def own_pages(self, ctx: StepContext, page_size: int, device):
        """The step's own pages, one run per request: (page owners, page indices, block table [S, most], count); made
        once per step and shared by the model's layers of this kind."""
        key = ("latent_own_pages", page_size)
        if key not in ctx.scratch:
            counts = [-(-(s + n) // page_size) for s, n in zip(ctx.host_start_pos, ctx.host_q_lens)]
            most = max(counts)
            owners, indices, rows, first = [], [], [], 0
            for seq, count in enumerate(counts):
                owners += [seq] * count
                indices += list(range(count))
                rows.append(list(range(first, first + count)) + [-1] * (most - count))
                first += count
            make = lambda values: torch.tensor(values, dtype=torch.int32).to(device, non_blocking=True)
            ctx.scratch[key] = (make(owners), make(indices), make(rows), first)
        return ctx.scratch[key]

    def attend_expanded(self, q: torch.Tensor, gate, ctx: StepContext, pages: torch.Tensor, table: torch.Tensor,
                        out: Optional[torch.Tensor]) -> torch.Tensor:
        ops = self.ops
        dtype, device = self.env.dtype, q.device
        page_size = pages.shape[2]
        per = self.dim + self.rot
        owners, indices, own_table, count = self.own_pages(ctx, page_size, device)
        # buffers that only grow, shared by all layers of these sizes: the attention kernels keep one descriptor per
        # (address, geometry) of a page pool
        held = _EXPANDED.get((device, self.heads, page_size, per, self.vdim, dtype))
        if held is None or held[0].shape[0] < count:
            room = max(count, 2 * held[0].shape[0] if held is not None else 0)
            held = (torch.zeros((room, self.heads, page_size, per), dtype=dtype, device=device),
                    torch.zeros((room, self.heads, page_size, self.vdim), dtype=dtype, device=device))
            _EXPANDED[(device, self.heads, page_size, per, self.vdim, dtype)] = held
        keys, values = held
        latents = torch.empty((count * page_size, self.kv_rank), dtype=dtype, device=device)
        ops.latent_gather(pages, table, owners, indices, ctx.ctx_len, self.kv_rank, self.heads, latents, keys)
        expanded = ops.linear(latents, self.w_ukv, None, ops.GEMM_STORE)
        ops.latent_scatter(expanded, count, self.dim, keys, values)
        queries = torch.empty_like(q)
        ops.rotate_interleaved(q, per, queries, per, self.heads, per, self.cos, self.sin, self.rot_dims, ctx.positions,
                               first=self.dim)
        attended = ops.attention(queries, keys, values, own_table, ctx.q_start, ctx.start_pos, ctx.positions, ctx.seq_of_token,
                                 ctx.num_seqs, ctx.max_q_len, ctx.max_ctx_len, self.heads, self.heads, per, self.scale,
                                 split_tokens=ctx.attn_split_tokens, typical_ctx_len=ctx.typical_ctx_len,
                                 decode_prefix=ctx.decode_prefix, out=out)
        mode = {"none": 0, "head": 1, "element": 2}[self.gate]
        return ops.gate_rows(attended, gate, self.heads, mode) if mode else attended

    def inner(self, h, ctx: StepContext, cache: LayerCache, out: Optional[torch.Tensor] = None):
        return self.attend(h, ctx, cache, out=out)

    def output_projection(self):
        return self.w_o, None

    def forward(self, h: torch.Tensor, ctx: StepContext, cache: LayerCache) -> torch.Tensor:
        return self.ops.linear(self.attend(h, ctx, cache), self.w_o, None, self.ops.GEMM_STORE)

    def forward_f32(self, h, ctx: StepContext, cache: LayerCache, out=None, alpha: float = 1.0, accumulate: bool = False):
        epilogue = self.ops.GEMM_ADD_F32 if accumulate else self.ops.GEMM_STORE_F32
        return self.ops.linear(self.attend(h, ctx, cache), self.w_o, None, epilogue, out=out, alpha=alpha)

    def forward_add(self, h: torch.Tensor, x: torch.Tensor, ctx: StepContext, cache: LayerCache, next_norm=None):
        self.ops.linear(self.attend(h, ctx, cache), self.w_o, None, self.ops.GEMM_ADD_F32, out=x)
        return None


@MIXERS.register("shifted_mixer")
class ShiftedMixer(Mixer):
    """params: ``hidden_size``, ``inner`` (the wrapped mixer's PartSpec).  weights: ``shift`` (float32 [hidden]) and the
    wrapped mixer's under ``inner.<name>``.  State: the request's last input row (``shift``), beside the wrapped
    mixer's own entries."""

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.hidden = int(spec.params["hidden_size"])
        inner: PartSpec = spec.params["inner"]
        self.mixer: Mixer = build_part(MIXERS, inner, env)
        self.graph_safe = bool(self.mixer.graph_safe)
        self.mu: Optional[torch.Tensor] = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        specs = {"shift": ParamSpec((self.hidden,), role="vector")}
        specs.update({f"inner.{name}": param for name, param in self.mixer.param_specs().items()})
        return specs

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.mu = tensors["shift"].contiguous()
        self.mixer.load({name[len("inner."):]: t for name, t in tensors.items() if name.startswith("inner.")})

    def param_bytes(self) -> int:
        return 4 * self.hidden + self.mixer.param_bytes()

    def flops(self, tokens: int, pairs: float) -> float:
        return self.mixer.flops(tokens, pairs)

    def cache_spec(self):
        return self.mixer.cache_spec()

    def extra_cache_specs(self):
        return self.mixer.extra_cache_specs()

    def state_spec(self) -> Optional[StateSpec]:
        inner = self.mixer.state_spec()
        entries = (("shift", (self.hidden,)),) + (tuple(inner.entries) if inner is not None else ())
        return StateSpec(entries=entries)

    def shifted(self, h, ctx: StepContext, cache: LayerCache) -> torch.Tensor:
        complete = getattr(h, "complete", None)       # rows that travel without their norm factor
        if complete is not None:
            h = complete()
        return self.ops.token_shift(h, self.mu, cache.state["shift"], ctx.slots, ctx.seq_of_token, ctx.q_start,
                                    ctx.start_pos, ctx.num_seqs)

    def inner(self, h, ctx: StepContext, cache: LayerCache, out: Optional[torch.Tensor] = None):
        return self.mixer.inner(self.shifted(h, ctx, cache), ctx, cache, out=out)

    def output_projection(self):
        return self.mixer.output_projection()

    def forward(self, h, ctx: StepContext, cache: LayerCache) -> torch.Tensor:
        return self.mixer.forward(self.shifted(h, ctx, cache), ctx, cache)

    def forward_f32(self, h, ctx: StepContext, cache: LayerCache, out=None, alpha: float = 1.0, accumulate: bool = False):
        return self.mixer.forward_f32(self.shifted(h, ctx, cache), ctx, cache, out=out, alpha=alpha, accumulate=accumulate)

    def forward_add(self, h, x, ctx: StepContext, cache: LayerCache, next_norm=None):
        return self.mixer.forward_add(self.shifted(h, ctx, cache), x, ctx, cache, next_norm=next_norm)
