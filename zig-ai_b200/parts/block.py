"""Arrangement of a layer's parts: pre-norm residual block.

    r  = norm_a(h);  h = h + mixer(r);  r2 = norm_b(h);  h = h + feed_forward(r2)

(src/transformer/hybrid_layer.zig:364-365, 370-377, 409-422, 488-491; LFM2 uses `ffn_norm` as the
second norm, :302-305).  Both kinds of LFM2 layer use it; the reference's device path leaves out
the residual on ShortConv layers (:627), which is not followed.  Each addition is carried as a
pending term into the next norm's kernel, which adds it into the 32-bit residual stream.
"""
from __future__ import annotations

from .base import Block, NormedTerm, register_part


class PreNormResidual(Block):
    graph_safe = True      # forward launches kernels only; nothing is read back to the host

    def __init__(self, mixer, mixer_norm, feed_forward=None, ff_norm=None):
        super().__init__()
        self.mixer_norm = self.sub("mixer_norm", "norm", mixer_norm)
        self.mixer = self.sub("mixer", "mixer", mixer)
        self.feed_forward = None                   # a layer may have no feed-forward (and then no second norm)
        if feed_forward is not None:
            self.ff_norm = self.sub("ff_norm", "norm", ff_norm)
            self.feed_forward = self.sub("feed_forward", "feed_forward", feed_forward)

    def params(self):
        return {}

    def forward(self, h, pending, step, cache, write_cache=True):
        r = self.mixer_norm.forward(h, pending, step, lazy=self.mixer.accepts_lazy_input)
        m = self.mixer.forward(r, step, self.cache_for(self.mixer, cache), write_cache)
        if self.feed_forward is None:
            return h, m
        r2 = self.ff_norm.forward(h, m, step, lazy=self.feed_forward.accepts_lazy_input)
        f = self.feed_forward.forward(r2, step)
        return h, f


class SandwichResidual(Block):
    """A norm before and a norm after each sublayer; the feed-forward is optional:

        h = h + post_mixer(mixer(pre_mixer(h)));   h = h + post_ff(feed_forward(pre_ff(h)))

    The norm after a sublayer, the addition and the norm before the next sublayer run as one kernel: a
    sublayer's output travels as a `NormedTerm` into the next norm (of this block, of the next block, or
    the model's final norm)."""
    graph_safe = True      # forward launches kernels only; nothing is read back to the host

    def __init__(self, mixer, mixer_norm, mixer_post_norm, feed_forward=None, ff_norm=None, ff_post_norm=None):
        super().__init__()
        self.mixer_norm = self.sub("mixer_norm", "norm", mixer_norm)
        self.mixer = self.sub("mixer", "mixer", mixer)
        self.mixer_post_norm = self.sub("mixer_post_norm", "norm", mixer_post_norm)
        self.feed_forward = None
        if feed_forward is not None:
            self.ff_norm = self.sub("ff_norm", "norm", ff_norm)
            self.feed_forward = self.sub("feed_forward", "feed_forward", feed_forward)
            self.ff_post_norm = self.sub("ff_post_norm", "norm", ff_post_norm)

    def params(self):
        return {}

    def forward(self, h, pending, step, cache, write_cache=True):
        r = self.mixer_norm.forward(h, pending, step, lazy=self.mixer.accepts_lazy_input)
        m = self.mixer.forward(r, step, self.cache_for(self.mixer, cache), write_cache)
        term = NormedTerm(m, self.mixer_post_norm.weight, self.mixer_post_norm.eps)
        if self.feed_forward is None:
            return h, term
        r2 = self.ff_norm.forward(h, term, step, lazy=self.feed_forward.accepts_lazy_input)
        f = self.feed_forward.forward(r2, step)
        return h, NormedTerm(f, self.ff_post_norm.weight, self.ff_post_norm.eps)


class PostNormResidual(Block):
    """A norm on each sublayer's output only, and a factor on the normed term; the sublayers read the residual stream itself:

        h = h + mult * norm_a(mixer(h));   h = h + mult * norm_b(feed_forward(h))

    A sublayer's output travels as a `NormedTerm` (the factor folded into the norm's weight, once, in 32-bit) into whatever
    comes next: this block's next sublayer, the next block, or the model's final norm.  The kernel that adds it to the
    32-bit stream also rounds the stream to the activations' dtype for the sublayer that reads it."""
    graph_safe = True      # forward launches kernels only; nothing is read back to the host

    def __init__(self, mixer, mixer_norm, feed_forward=None, ff_norm=None, mult: float = 1.0):
        super().__init__()
        self.mult = float(mult)
        self.mixer = self.sub("mixer", "mixer", mixer)
        self.mixer_norm = self.sub("mixer_norm", "norm", mixer_norm)
        self.feed_forward = None
        if feed_forward is not None:
            self.feed_forward = self.sub("feed_forward", "feed_forward", feed_forward)
            self.ff_norm = self.sub("ff_norm", "norm", ff_norm)
        self._gammas = {}

    def params(self):
        return {}

    def _term(self, data, norm):
        g = self._gammas.get(id(norm))
        if g is None or g[0] is not norm.weight:
            g = self._gammas[id(norm)] = (norm.weight, (norm.weight.float() * self.mult).contiguous())
        return NormedTerm(data, g[1], norm.eps)

    @staticmethod
    def _read(h, pending, step):
        """Add what is pending and return the stream in the activations' dtype."""
        if isinstance(pending, NormedTerm):
            return step.ops.add_cast(h.data, pending.data, step.dtype, pending.gamma, pending.eps)
        return step.ops.add_cast(h.data, pending, step.dtype)

    def forward(self, h, pending, step, cache, write_cache=True):
        m = self.mixer.forward(self._read(h, pending, step), step, self.cache_for(self.mixer, cache), write_cache)
        term = self._term(m, self.mixer_norm)
        if self.feed_forward is None:
            return h, term
        f = self.feed_forward.forward(self._read(h, term, step), step)
        return h, self._term(f, self.ff_norm)


register_part("block", "prenorm_residual", PreNormResidual)
register_part("block", "postnorm_residual", PostNormResidual)
register_part("block", "sandwich_residual", SandwichResidual)
