"""How a layer's parts are arranged: the pre-norm residual block, and the block with both branches side by side.

``h += mixer(norm1(h)); h += feed_forward(norm2(h))`` as in
``src/turboserve/engine/model/layers.py:469-487``. The residual stream ``h`` is fp32; a part's
output is not added at once but handed on as ``pending`` and added by the next norm's kernel
(the fused residual-add + norm), so each sum is computed in 32-bit and read once.
"""

from __future__ import annotations

import torch

from .base import FeedForward, Mixer, Norm, register_block


class PreNormBlock:
    def __init__(self, mixer: Mixer, feed_forward: FeedForward, mixer_norm: Norm, feed_forward_norm: Norm) -> None:
        self.mixer = mixer
        self.feed_forward = feed_forward
        self.mixer_norm = mixer_norm
        self.feed_forward_norm = feed_forward_norm

    def forward(self, residual: torch.Tensor, pending: torch.Tensor | None, ctx, cache) -> torch.Tensor:
        """Run the layer; returns the new pending update (the feed-forward's output)."""
        n, hidden = ctx.batch.num_tokens, residual.shape[-1]
        normed = ctx.buffer("block.normed", (n, hidden))
        self.mixer_norm.forward(residual, pending, normed, ctx)
        mixed = self.mixer.forward(normed, ctx, cache)
        self.feed_forward_norm.forward(residual, mixed, normed, ctx)
        return self.feed_forward.forward(normed, ctx)


class ParallelBlock:
    """Mixer and feed-forward side by side on the same input: ``h += mixer(norm1(h)) + ff(norm2(h))``.

    Both branches' outputs are handed on as a pair of pending updates; the next norm's kernel adds
    both into the fp32 residual (and a stream shift, if the next run brings one) and, when both
    norms are RMS norms with one ``eps``, writes both normed inputs in the same pass. A layer
    without a feed-forward has one branch.
    """

    takes_shift = True

    def __init__(self, mixer: Mixer, feed_forward: FeedForward | None, mixer_norm: Norm, feed_forward_norm: Norm | None) -> None:
        self.mixer = mixer
        self.feed_forward = feed_forward
        self.mixer_norm = mixer_norm
        self.feed_forward_norm = feed_forward_norm
        if (feed_forward is None) != (feed_forward_norm is None):
            raise ValueError("a feed-forward and its norm go together")

    def forward(self, residual: torch.Tensor, pending, ctx, cache, shift: torch.Tensor | None = None):
        n, hidden = ctx.batch.num_tokens, residual.shape[-1]
        for_mixer = ctx.buffer("block.normed", (n, hidden))
        if self.feed_forward is None:
            self.mixer_norm.forward(residual, pending, for_mixer, ctx, shift=shift)
            return self.mixer.forward(for_mixer, ctx, cache)
        for_ff = ctx.buffer("block.normed_ff", (n, hidden))
        pair = getattr(self.mixer_norm, "forward_pair", None)
        if pair is not None and getattr(self.feed_forward_norm, "eps", None) == getattr(self.mixer_norm, "eps", 0):
            pair(residual, pending, self.feed_forward_norm, for_mixer, for_ff, ctx, shift=shift)
        else:
            self.mixer_norm.forward(residual, pending, for_mixer, ctx, shift=shift)
            self.feed_forward_norm.forward(residual, None, for_ff, ctx)
        mixed = self.mixer.forward(for_mixer, ctx, cache)
        return mixed, self.feed_forward.forward(for_ff, ctx)


register_block("pre_norm", PreNormBlock)
register_block("parallel", ParallelBlock)
