"""Arrangements of norms, mixer and feed-forward inside a layer."""

from __future__ import annotations

from pagedserve_b200.parts.base import Block, register_part


@register_part("block", "pre_norm")
class PreNormBlock(Block):
    """h += mixer(norm(h)); h += feed_forward(norm(h))
    (reference: src/model/paged_decoder.py:181-189, 210-228).  The residual stream ``h``
    is float32 and is updated in place; the adds happen in the epilogues of the
    mixer's and the feed-forward's last matrix products."""

    graph_safe = True

    required_norms = ("pre_mixer", "pre_feed_forward")

    @staticmethod
    def _normed(norm, consumer, hidden):
        # a consumer whose first operation is a matrix product may take the norm unevaluated
        if getattr(consumer, "accepts_deferred_norm", False) and hasattr(norm, "defer"):
            return norm.defer(hidden)
        return norm.forward(hidden)

    def forward(self, hidden, ctx, layer):
        self.mixer.forward(self._normed(self.norms["pre_mixer"], self.mixer, hidden), hidden, ctx, layer)
        self.feed_forward.forward(self._normed(self.norms["pre_feed_forward"], self.feed_forward, hidden),
                                  hidden, ctx)
