"""The arrangement of parts in a layer."""

from __future__ import annotations

import torch

from ..tracing import scope
from .base import Block, FeedForward, LayerCache, Mixer, Norm, StepContext, register_part


class PreNormBlock(Block):
    """x += mixer(norm1(x)); x += feed_forward(norm2(x))  (llama4/llama4_jax/model.py:1156-1183).

    The residual sums are done in float32 inside the following norm's kernel: a block returns its
    last delta unadded, and the next block's first norm (or the model's final norm) adds it.
    The feed-forward (with norm2) may be missing: the block is then its first sublayer alone."""

    def __init__(self, norm1: Norm, mixer: Mixer, norm2: Norm | None = None, feed_forward: FeedForward | None = None):
        if (feed_forward is None) != (norm2 is None):
            raise ValueError("a feed-forward comes with its norm, or not at all")
        self.norm1, self.mixer, self.norm2, self.feed_forward = norm1, mixer, norm2, feed_forward

    def sub_parts(self):
        return tuple(p for p in (self.norm1, self.mixer, self.norm2, self.feed_forward) if p is not None)

    def forward(self, ctx: StepContext, x: torch.Tensor, delta, cache: LayerCache) -> torch.Tensor:
        dt = ctx.runtime.dtype
        with scope("attn_pre_norm"):  # the reference's names (model.py:1169-1180); each norm also adds the residual
            h = self.norm1.forward(ctx, x, delta, out_dtype=dt)[0]
        a = self.mixer.forward(ctx, h, cache)
        if self.feed_forward is None:
            return a
        want32 = self.feed_forward.needs_f32_input
        router = self.feed_forward.router_request() if self.norm2.fuses_router else None
        with scope("attn_post_norm"):
            h, h32, routing = self.norm2.forward(ctx, x, a, out_dtype=dt, want_f32=want32, router=router)
        with scope("ffn"):
            return self.feed_forward.forward(ctx, h, h32, routing)


register_part("block", "pre_norm", PreNormBlock)


class ScaledPreNormBlock(Block):
    """A pre-norm block whose sublayers' outputs are multiplied channel by channel by a vector each before they are
    added:  x += scale1 * mixer(norm1(x));  x += scale2 * feed_forward(norm2(x)).  The feed-forward (with norm2 and
    scale2) may be missing.  A sublayer's output goes on as a :class:`Scaled` delta: the scale, the residual sum and
    the next norm are one kernel."""

    def __init__(self, norm1: Norm, mixer: Mixer, scale1: torch.Tensor, norm2: Norm | None = None,
                 feed_forward: FeedForward | None = None, scale2: torch.Tensor | None = None):
        if (feed_forward is None) != (norm2 is None) or (feed_forward is None) != (scale2 is None):
            raise ValueError("a feed-forward comes with its norm and its scale, or not at all")
        self.norm1, self.mixer, self.norm2, self.feed_forward = norm1, mixer, norm2, feed_forward
        self.scale1 = scale1.to(torch.float32).contiguous()
        self.scale2 = None if scale2 is None else scale2.to(torch.float32).contiguous()

    def sub_parts(self):
        return tuple(p for p in (self.norm1, self.mixer, self.norm2, self.feed_forward) if p is not None)

    def forward(self, ctx: StepContext, x: torch.Tensor, delta, cache: LayerCache):
        from .base import Scaled, as_rows

        dt = ctx.runtime.dtype
        with scope("attn_pre_norm"):
            if self.mixer.needs_f32_input:
                _, h32, _ = self.norm1.forward(ctx, x, delta, out_dtype=None, want_f32=True)
                y = self.mixer.forward(ctx, None, cache, h32=h32)
            else:
                h = self.norm1.forward(ctx, x, delta, out_dtype=dt)[0]
                y = self.mixer.forward(ctx, h, cache)
        pending = Scaled(as_rows(y), self.scale1)
        if self.feed_forward is None:
            return pending
        with scope("attn_post_norm"):
            h, h32, _ = self.norm2.forward(ctx, x, pending, out_dtype=dt, want_f32=self.feed_forward.needs_f32_input)
        with scope("ffn"):
            y = self.feed_forward.forward(ctx, h, h32, None)
        return Scaled(as_rows(y), self.scale2)


register_part("block", "scaled_pre_norm", ScaledPreNormBlock)


class SandwichNormBlock(Block):
    """A block that norms each sublayer's input and its output, and scales what it adds:

        x += mult * norm1b(mixer(norm1(x)));   x += mult * norm2b(feed_forward(norm2(x)))

    ``feed_forward`` (with its two norms) may be None: the block then has the first sublayer only.
    A sublayer's output goes on as a :class:`PostNormed` delta: the closing norm, the scaled residual sum and the
    next opening norm are one kernel.  ``feed_forward.bias_out`` (the bias of its last product), if it has one, is
    added inside that kernel too."""

    def __init__(self, norm1: Norm, mixer: Mixer, norm1b: Norm, norm2: Norm | None = None,
                 feed_forward: FeedForward | None = None, norm2b: Norm | None = None, mult: float = 1.0):
        if (feed_forward is None) != (norm2 is None) or (feed_forward is None) != (norm2b is None):
            raise ValueError("a feed-forward comes with both of its norms, or not at all")
        self.norm1, self.mixer, self.norm1b = norm1, mixer, norm1b
        self.norm2, self.feed_forward, self.norm2b = norm2, feed_forward, norm2b
        self.mult = float(mult)

    def sub_parts(self):
        return tuple(p for p in (self.norm1, self.mixer, self.norm1b, self.norm2, self.feed_forward, self.norm2b) if p is not None)

    def _closing(self, norm: Norm, y, bias=None):
        from .base import PostNormed, as_rows

        return PostNormed(as_rows(y), norm.weight, norm.eps, norm.groups, self.mult, bias)

    def forward(self, ctx: StepContext, x: torch.Tensor, delta, cache: LayerCache):
        dt = ctx.runtime.dtype
        with scope("attn_pre_norm"):
            if self.mixer.needs_f32_input:
                _, h32, _ = self.norm1.forward(ctx, x, delta, out_dtype=None, want_f32=True)
                y = self.mixer.forward(ctx, None, cache, h32=h32)
            else:
                h = self.norm1.forward(ctx, x, delta, out_dtype=dt)[0]
                y = self.mixer.forward(ctx, h, cache)
        pending = self._closing(self.norm1b, y)
        if self.feed_forward is None:
            return pending
        with scope("attn_post_norm"):
            h = self.norm2.forward(ctx, x, pending, out_dtype=dt)[0]
        with scope("ffn"):
            y = self.feed_forward.forward(ctx, h, None, None)
        return self._closing(self.norm2b, y, getattr(self.feed_forward, "bias_out", None))


class ReinjectionBlock(Block):
    """Feeds the embedding's output into the stream again:  x <- W [x; x0] + step,  x0 = what the embedding put out
    for the token, W: [D, 2D] (x's half first), ``step``: a vector of this entry (one per pass of a loop over layers).
    It mixes nothing across tokens and keeps no cache or state.  The product of W's second half with x0 is the same
    for every such block of a step that shares W: it is made once and kept in the step's scratch."""

    mixer = None
    wants_embedding_output = True
    kernel_libraries = ("group_norm",)

    def __init__(self, w_in: torch.Tensor, step: torch.Tensor):
        D = w_in.shape[0]
        if w_in.shape[1] != 2 * D or step.shape != (D,):
            raise ValueError(f"re-injection weights do not fit: {tuple(w_in.shape)}, step {tuple(step.shape)}")
        self.w_x, self.w_x0 = w_in[:, :D].contiguous(), w_in[:, D:].contiguous()
        self.step = step.to(torch.float32).contiguous()

    def share_weights(self, other: "ReinjectionBlock") -> None:
        """Another pass over the same W: keep one copy of its halves."""
        self.w_x, self.w_x0 = other.w_x, other.w_x0

    def forward(self, ctx: StepContext, x: torch.Tensor, delta, cache: LayerCache):
        from ..kernels import api as K
        from .base import as_rows
        from .linear import linear
        from .norms import add_to_residual

        dt = ctx.runtime.dtype
        n, D = x.shape
        key = ("reinjection", self.w_x0.data_ptr())
        u0 = ctx.scratch.get(key)
        if u0 is None:
            x0 = torch.empty((n, D), dtype=dt, device=x.device)
            K.bias_act(ctx.scratch["embedding_output"], x0)
            u = as_rows(linear(ctx, x0, self.w_x0, torch.float32, partials=True))
            u0 = torch.empty((n, D), dtype=torch.float32, device=x.device)
            K.bias_act(u.data, u0, splits=u.splits)
            ctx.scratch[key] = u0
        xa = torch.empty((n, D), dtype=dt, device=x.device)
        add_to_residual(x, delta, pre_norm=False, out=xa)  # x += pending; xa = x in the activations' type
        y = as_rows(linear(ctx, xa, self.w_x, torch.float32, partials=True))
        K.bias_act(y.data, x, self.step, u0, splits=y.splits)  # x = W_x x + W_x0 x0 + step
        return None


class EmbeddingReentryBlock(Block):
    """Adds the embedding's output to the stream once more:  x <- x + x0,  x0 = what the embedding put out for the token
    (scaled as the embedding scales it).  It stands in front of every pass but the first of a stretch of layers that
    runs several times.  It has no weights, mixes nothing across tokens and keeps no cache or state, and it launches
    nothing: x0 joins the pending delta as one more term of the sum that the next norm's kernel adds to x."""

    mixer = None
    wants_embedding_output = True

    def forward(self, ctx: StepContext, x: torch.Tensor, delta, cache: LayerCache):
        from ..kernels import api as K
        from .base import Rows, RowSum, as_rows

        x0 = ctx.scratch["embedding_output"]
        if isinstance(delta, RowSum):
            terms, before = list(delta.terms), delta.materialize
        else:
            d = as_rows(delta)
            terms, before = ([] if d is None else [d]), None

        def materialize() -> torch.Tensor:
            if before is not None:
                return before() + x0
            if not terms:
                return x0
            out = torch.empty_like(x0)
            K.bias_act(terms[0].data, out, None, x0, "none", terms[0].splits)  # the partials in order, then x0
            return out

        return RowSum(terms + [Rows(x0, 1)], materialize)


class HyperConnectionBlock(Block):
    """A pre-norm block over several residual streams per token.  Each sublayer q (mixer, then feed-forward) has read
    weights in_q [S], write weights out_q [S] and a mix matrix mix_q [S, S] (indexed [from, to]):

        u = sum_s in_q[s] x_s;   y = sublayer(norm_q(u));   x_t <- sum_s mix_q[s, t] x_s + out_q[t] y   (all t at once).

    The read weights live in the norms (``StreamRMSNorm``); a sublayer's output goes on as a :class:`StreamMixed`, so
    that its write-back, the next sublayer's read and that sublayer's norm are one kernel.  The feed-forward (with its
    norm and weights) may be missing."""

    def __init__(self, norm1: Norm, mixer: Mixer, mix1: torch.Tensor, write1: torch.Tensor, norm2: Norm | None = None,
                 feed_forward: FeedForward | None = None, mix2: torch.Tensor | None = None, write2: torch.Tensor | None = None):
        if len({feed_forward is None, norm2 is None, mix2 is None, write2 is None}) != 1:
            raise ValueError("a feed-forward comes with its norm, its mix matrix and its write weights, or not at all")
        self.norm1, self.mixer, self.norm2, self.feed_forward = norm1, mixer, norm2, feed_forward
        f32 = lambda t: None if t is None else t.to(torch.float32).contiguous()  # noqa: E731
        self.mix1, self.write1, self.mix2, self.write2 = f32(mix1), f32(write1), f32(mix2), f32(write2)
        S = self.write1.numel()
        if self.mix1.shape != (S, S) or (self.mix2 is not None and (self.mix2.shape != (S, S) or self.write2.numel() != S)):
            raise ValueError(f"{S} streams take mix matrices of {S} x {S} and {S} write weights")

    def sub_parts(self):
        return tuple(p for p in (self.norm1, self.mixer, self.norm2, self.feed_forward) if p is not None)

    def forward(self, ctx: StepContext, x: torch.Tensor, delta, cache: LayerCache):
        from .base import StreamMixed, as_rows

        dt = ctx.runtime.dtype
        with scope("attn_pre_norm"):
            h = self.norm1.forward(ctx, x, delta, out_dtype=dt)[0]
        y = self.mixer.forward(ctx, h, cache)
        pending = StreamMixed(as_rows(y), self.mix1, self.write1)
        if self.feed_forward is None:
            return pending
        with scope("attn_post_norm"):
            h, h32, _ = self.norm2.forward(ctx, x, pending, out_dtype=dt, want_f32=self.feed_forward.needs_f32_input)
        with scope("ffn"):
            y = self.feed_forward.forward(ctx, h, h32, None)
        return StreamMixed(as_rows(y), self.mix2, self.write2)


register_part("block", "hyper_connection", HyperConnectionBlock)
register_part("block", "sandwich_norm", SandwichNormBlock)
register_part("block", "reinjection", ReinjectionBlock)
register_part("block", "embedding_reentry", EmbeddingReentryBlock)
