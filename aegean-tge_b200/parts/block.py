"""Arrangements of a mixer and a feed-forward around the residual stream."""
from __future__ import annotations

from typing import Optional

import torch

from .base import BLOCKS, Block, LayerCache, StepContext


@BLOCKS.register("pre_norm")
class PreNormBlock(Block):
    """x += mixer(norm1(x)); x += ffn(norm2(x)).

    The stream ``x`` is float32 and is never itself normalised: each norm's
    output feeds the part and the part's output is added back
    (src/models/qwen2.cpp:2055, :2099-2105, :2118).  A layer without feed-forward (and then without second norm)
    is x += mixer(norm1(x)) alone.
    """

    passes_deferred_rows = True

    def forward(self, x, ctx: StepContext, cache: LayerCache, h=None, next_norm=None, next_takes_deferred=False):
        if h is None:
            h = self.mixer_norm.forward(x)
        if self.feed_forward is None:
            if isinstance(h, self.env.ops.DeferredRows) and not self.mixer.takes_deferred_rows:
                h = h.complete()
            return self.mixer.forward_add(h, x, ctx, cache, next_norm=next_norm)
        # a part is only asked to leave the norm's factor to its successor if both sides say they can
        defer = {"defer": True} if self.mixer.can_defer_norm and self.feed_forward.takes_deferred_rows else {}
        h = self.mixer.forward_add(h, x, ctx, cache, next_norm=self.ffn_norm, **defer)
        if h is None:
            h = self.ffn_norm.forward(x)
        defer = {"defer": True} if self.feed_forward.can_defer_norm and next_takes_deferred else {}
        return self.feed_forward.forward_add(h, x, ctx, next_norm=next_norm, **defer)


@BLOCKS.register("parallel")
class ParallelBlock(Block):
    """h = norm(x); x += m * (mixer(h) + ffn(h)): one norm, both sublayers read its output.  With a second norm
    the feed-forward reads its own, x += m * (mixer(norm1(x)) + ffn(norm2(x))), both norms taken of the same x.

    params: ``residual_mult`` (m, default 1).  The feed-forward may be absent (x += m * mixer(h)).

    When both sublayers end in a plain product (``inner`` / ``output_projection``), the two products are one:
    the mixer's inner rows and the feed-forward's activated rows are written side by side into one buffer
    [T, a | g] and multiplied by the column-concatenated weights [Wo | Wdown], so the stream is read and written
    once, with m applied in that product's epilogue, and the sum of the two sublayers is formed in float32 inside
    the accumulator.  For small batches the same kernel that adds the product into the stream also applies the
    next layer's norm.  Sublayers that cannot hand out their last product are run whole and added one by one.
    """

    passes_deferred_rows = True

    def __init__(self, mixer, feed_forward, mixer_norm, ffn_norm, env, params=None):
        super().__init__(mixer, feed_forward, mixer_norm, ffn_norm, env, params)
        if ffn_norm is not None and feed_forward is None:
            if not getattr(ffn_norm, "optional", False):
                raise ValueError("parallel block: a second norm without a feed-forward to read it")
            # else: a norm that a checkpoint may hold for a layer without feed-forward: loaded if present, read by
            # nothing
        self.mult = float(self.params.get("residual_mult", 1.0))
        self.w_out: Optional[torch.Tensor] = None
        self.b_out: Optional[torch.Tensor] = None
        self.split = 0
        self.shared_input = False      # the feed-forward's up rows lie below the mixer's q/k/v rows

    def loaded(self) -> None:
        """Concatenates the two output weights along their columns, once the parts have theirs."""
        mixer_out = self.mixer.output_projection()
        if mixer_out is None:
            return
        if self.feed_forward is None:
            self.w_out, self.b_out = mixer_out
            self.split = mixer_out[0].shape[1]
            return
        ffn_out = self.feed_forward.output_projection()
        if ffn_out is None:
            return
        (w_a, b_a), (w_f, b_f) = mixer_out, ffn_out
        self.split = w_a.shape[1]
        self.w_out = torch.cat([w_a, w_f], dim=1).contiguous()
        # the parts' own copies are not needed again: this block runs their last products
        self.mixer.w_o = None
        self.feed_forward.w_down = None
        # the two first products read the same rows too: a mixer that can carry the up rows through its own
        # small-batch kernel takes them in (they stay one tensor; both parts keep views of it)
        share = getattr(self.mixer, "share_input_projection", None)
        adopt = getattr(self.feed_forward, "adopt_input_projection", None)
        if share is not None and adopt is not None and self.ffn_norm is None:
            view = share(self.feed_forward.input_projection())
            if view is not None:
                adopt(view)
                self.shared_input = True
        if b_a is not None or b_f is not None:
            zero = torch.zeros(w_a.shape[0], dtype=torch.float32, device=w_a.device)
            self.b_out = ((b_a if b_a is not None else zero) + (b_f if b_f is not None else zero)).contiguous()

    def forward(self, x, ctx: StepContext, cache: LayerCache, h=None, next_norm=None, next_takes_deferred=False):
        ops = self.env.ops
        # the feed-forward's rows: its own norm of the same x (taken before anything is added), else the mixer's
        own_rows = self.ffn_norm is not None and self.feed_forward is not None
        both = getattr(self.mixer_norm, "forward_with", None) if (h is None and own_rows) else None
        pair = both(self.ffn_norm, x) if both is not None else None       # two norms that share their statistics
        if pair is not None:
            h, b = pair
        else:
            if h is None:
                h = self.mixer_norm.forward(x)
            b = self.ffn_norm.forward(x) if own_rows else h
        if self.w_out is None:
            # whole sublayers, added one by one
            if isinstance(h, ops.DeferredRows):
                h = h.complete()
                b = b if own_rows else h
            if self.mult == 1.0:
                # each sublayer adds its last product (or its weighted sum) into the float32 stream itself
                self.mixer.forward_add(h, x, ctx, cache)
                if self.feed_forward is not None:
                    self.feed_forward.forward_add(b, x, ctx)
                return None
            ops.add_to_stream(x, self.mixer.forward(h, ctx, cache), alpha=self.mult)
            if self.feed_forward is not None:
                ops.add_to_stream(x, self.feed_forward.forward(b, ctx), alpha=self.mult)
            return None
        tokens = x.shape[0]
        inner = torch.empty((tokens, self.w_out.shape[1]), dtype=self.env.dtype, device=x.device)
        if self.shared_input:
            beside = (inner[:, self.split:], self.feed_forward.epilogue())
            _rows, done = self.mixer.inner(h, ctx, cache, out=inner[:, :self.split], beside=beside)
            if not done:
                self.feed_forward.inner(h, ctx, out=inner[:, self.split:])
        else:
            if self.feed_forward is not None:
                self.feed_forward.inner(b, ctx, out=inner[:, self.split:])
            self.mixer.inner(h, ctx, cache, out=inner[:, :self.split])
        fused = next_norm.fusable() if next_norm is not None else None
        if fused is not None:
            return ops.linear_add_norm(inner, self.w_out, self.b_out, x, fused[0], fused[1], self.env.dtype,
                                       defer=bool(next_takes_deferred), alpha=self.mult)
        ops.linear(inner, self.w_out, self.b_out, ops.GEMM_ADD_F32, out=x, alpha=self.mult)
        return None


@BLOCKS.register("post_norm")
class PostNormBlock(Block):
    """x <- norm1(a x + mixer(x)); x <- norm2(a x + ffn(x)): the norm comes after the sum, and the sublayers
    read the stream itself.

    params: ``alpha`` (a, default 1).  The feed-forward and its norm may be absent; a second norm without a feed-forward
    (a checkpoint that holds one for such a layer) normalises ``a x`` alone.  The stream stays float32; the
    kernel that normalises it also writes the rows the next product reads, so a sublayer's input is never normed
    on its own.  ``forward`` returns those rows for the next layer.
    """

    def __init__(self, mixer, feed_forward, mixer_norm, ffn_norm, env, params=None):
        super().__init__(mixer, feed_forward, mixer_norm, ffn_norm, env, params)
        if feed_forward is not None and ffn_norm is None:
            raise ValueError("post-norm block: a feed-forward needs the norm that follows its sum")
        self.alpha = float(self.params.get("alpha", 1.0))

    def forward(self, x, ctx: StepContext, cache: LayerCache, h=None, next_norm=None):
        ops = self.env.ops
        if h is None:
            h = ops.to_run_dtype(x, self.env.dtype)
        weight, eps = self.mixer_norm.fusable()
        h = ops.scale_add_norm(x, self.mixer.forward_f32(h, ctx, cache), self.alpha, weight, eps, self.env.dtype)
        second = self.ffn_norm.fusable() if self.ffn_norm is not None else None
        if self.feed_forward is not None:
            weight, eps = second
            h = ops.scale_add_norm(x, self.feed_forward.forward_f32(h, ctx), self.alpha, weight, eps, self.env.dtype)
        elif second is not None:
            h = ops.scale_add_norm(x, torch.zeros_like(x), self.alpha, second[0], second[1], self.env.dtype)
        return h
