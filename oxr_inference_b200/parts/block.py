"""How a mixer and a feed-forward are arranged into one block."""

from __future__ import annotations

import torch

from oxr_inference_b200.parts.base import ARRANGEMENTS, DeferredLinear, FeedForward, LayerCache, Mixer, Norm, StepContext


@ARRANGEMENTS.register("pre_norm")
class PreNormBlock:
    """``x += mixer(norm1(x)); x += feed_forward(norm2(x))`` (the second sublayer only when the block has a feed-forward), carried as
    (last output not yet added, residual):
    each norm first adds the pending output into the fp32 residual stream (oxr_runtime/language.py:184-187,
    253-257,266-269). Returns the feed-forward's output and the residual; whoever comes next adds them.

    Two optional hand-overs take the norm kernels out of a decode step; each happens only when both sides say that they can.
    A norm that ``accepts_deferred`` gets the part before it with its last projection still to do (:class:`DeferredLinear`;
    with ``defer_output`` the block's own output is left like that for the next block's norm, which the decoder asks for only
    when the next block ``accepts_deferred_input``), so that the product can add itself into the residual stream. And when
    the part behind such a norm ``accepts_lazy_input``, the norm may hand it a not yet normalised ``h`` that its first
    projection normalises itself."""

    supports_deferred = True

    def __init__(self, mixer: Mixer, mixer_norm: Norm, feed_forward: FeedForward | None, feed_forward_norm: Norm | None):
        if (feed_forward is None) != (feed_forward_norm is None):
            raise ValueError("a feed-forward comes with its norm or not at all")
        self.mixer, self.mixer_norm = mixer, mixer_norm
        self.feed_forward, self.feed_forward_norm = feed_forward, feed_forward_norm

    def parts(self) -> dict[str, object]:
        out = {"mixer": self.mixer, "mixer_norm": self.mixer_norm}
        if self.feed_forward is not None:
            out.update(feed_forward=self.feed_forward, feed_forward_norm=self.feed_forward_norm)
        return out

    @property
    def accepts_deferred_input(self) -> bool:
        return bool(self.mixer_norm.accepts_deferred)

    @staticmethod
    def _norm(norm: Norm, x, residual, behind) -> tuple:
        if norm.accepts_deferred:
            return norm.forward(x, residual, lazy=bool(getattr(behind, "accepts_lazy_input", False)))
        if isinstance(x, DeferredLinear):
            x = x.materialize()
        return norm.forward(x, residual)

    def forward(self, x, residual: torch.Tensor | None, ctx: StepContext, cache: LayerCache, defer_output: bool = False):
        if residual is None and torch.is_tensor(x) and x.dtype == torch.float32 and getattr(self.mixer_norm, "runtime", None) is not None \
                and self.mixer_norm.runtime.dtype != torch.float32 and hasattr(self.mixer_norm, "stream_norm"):
            # the embedding handed over the fp32 stream itself (not 16-bit activations): it is the residual, nothing is pending
            h, residual = self.mixer_norm.stream_norm(x), x
        elif x is None:
            # the block before kept the stream whole
            h = self.mixer_norm.stream_norm(residual)
        else:
            h, residual = self._norm(self.mixer_norm, x, residual, self.mixer)
        if self.feed_forward is None:   # the mixer's sublayer only: its output stays pending for whoever comes next
            return self.mixer.forward(h, ctx, cache), residual
        if self.feed_forward_norm.accepts_deferred:
            a = self.mixer.forward_deferred(h, ctx, cache)
        else:
            a = self.mixer.forward(h, ctx, cache)
        h, residual = self._norm(self.feed_forward_norm, a, residual, self.feed_forward)
        return (self.feed_forward.forward_deferred(h) if defer_output else self.feed_forward.forward(h)), residual


@ARRANGEMENTS.register("sandwich_norm")
class SandwichNormBlock:
    """``x += post_norm(mixer(pre_norm(x)))`` and, when the block has a feed-forward, ``x += post_norm(ff(pre_norm(x)))``: a norm on
    both sides of each sublayer. Nothing can stay pending between sublayers (the output is normalised before it is added), so the
    fp32 stream is kept whole: ``forward`` takes it in ``residual`` (or, for the first block, in ``x``), updates it in place and
    returns ``(None, stream)``. The post-norm, the add and the pre-norm that follows inside the block are one kernel."""

    supports_deferred = False
    accepts_deferred_input = False

    def __init__(self, mixer: Mixer, mixer_norm: Norm, feed_forward: FeedForward | None, feed_forward_norm: Norm | None, *,
                 mixer_post_norm: Norm, feed_forward_post_norm: Norm | None = None):
        if (feed_forward is None) != (feed_forward_norm is None) or (feed_forward is None) != (feed_forward_post_norm is None):
            raise ValueError("a feed-forward comes with both of its norms or not at all")
        self.mixer, self.mixer_norm, self.mixer_post_norm = mixer, mixer_norm, mixer_post_norm
        self.feed_forward, self.feed_forward_norm, self.feed_forward_post_norm = feed_forward, feed_forward_norm, feed_forward_post_norm

    def parts(self) -> dict[str, object]:
        out = {"mixer": self.mixer, "mixer_norm": self.mixer_norm, "mixer_post_norm": self.mixer_post_norm}
        if self.feed_forward is not None:
            out.update(feed_forward=self.feed_forward, feed_forward_norm=self.feed_forward_norm, feed_forward_post_norm=self.feed_forward_post_norm)
        return out

    def forward(self, x, residual: torch.Tensor | None, ctx: StepContext, cache: LayerCache, defer_output: bool = False):
        if residual is None:
            if isinstance(x, DeferredLinear):
                x = x.materialize()
            if x.dtype != torch.float32:
                raise ValueError("this arrangement keeps the stream in fp32: the embedding must hand it over whole")
            stream = x
        elif x is not None:
            raise ValueError("this arrangement takes the stream whole; the block before it left an output that is not yet added")
        else:
            stream = residual
        a = self.mixer.forward(self.mixer_norm.stream_norm(stream), ctx, cache)
        if self.feed_forward is None:
            self.mixer_post_norm.add_normed(stream, a)
            return None, stream
        h = self.mixer_post_norm.add_normed(stream, a, then=self.feed_forward_norm)
        self.feed_forward_post_norm.add_normed(stream, self.feed_forward.forward(h))
        return None, stream
