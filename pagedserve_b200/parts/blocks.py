"""Arrangements of norms, mixer and feed-forward inside a layer."""

from __future__ import annotations

from pagedserve_b200.parts.base import Block, register_part


@register_part("block", "pre_norm")
class PreNormBlock(Block):
    """h += mixer(norm(h)); h += feed_forward(norm(h))
    (reference: src/model/paged_decoder.py:181-189, 210-228).  The residual stream ``h``
    is float32 and is updated in place; the adds happen in the epilogues of the
    mixer's and the feed-forward's last matrix products.  A layer whose feed-forward is the ``none`` part has
    the first sublayer only, and no second norm."""

    graph_safe = True

    @property
    def required_norms(self):
        if getattr(self.feed_forward, "is_empty", False):
            return ("pre_mixer",)
        return ("pre_mixer", "pre_feed_forward")

    @staticmethod
    def _normed(norm, consumer, hidden):
        # a consumer whose first operation is a matrix product may take the norm unevaluated
        if getattr(consumer, "accepts_deferred_norm", False) and hasattr(norm, "defer"):
            return norm.defer(hidden)
        return norm.forward(hidden)

    def forward(self, hidden, ctx, layer):
        self.mixer.forward(self._normed(self.norms["pre_mixer"], self.mixer, hidden), hidden, ctx, layer)
        if getattr(self.feed_forward, "is_empty", False):
            return
        self.feed_forward.forward(self._normed(self.norms["pre_feed_forward"], self.feed_forward, hidden),
                                  hidden, ctx)
