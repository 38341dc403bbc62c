"""Arrangements of norm, mixer and feed-forward around the residual stream."""
from __future__ import annotations

import torch

from ..registry import BLOCKS
from .base import Block, CacheBundle


@BLOCKS.register("pre_norm")
class PreNormBlock(Block):
    """``h += mixer(norm(h)); h += ffn(norm(h))`` (crates/leone/src/runtime.rs:9103-9317).  A layer
    without a feed-forward (and without its norm) is the first half only."""

    chains_norms = True       # forward takes pre= and after= (see below)

    def __init__(self, mixer, feed_forward, mixer_norm, ffn_norm, **extra):
        if mixer_norm is None or (feed_forward is None) != (ffn_norm is None) or extra:
            raise ValueError("the pre_norm arrangement is norm, mixer and, optionally, norm, feed-forward: "
                             "it takes exactly those parts")
        super().__init__(mixer, feed_forward, mixer_norm, ffn_norm)

    def entry_norm(self, ctx, hidden):
        """The norm before the mixer as a DeferredNorm for the block before this one to fill,
        or None if it has to run as a kernel."""
        if getattr(self.mixer, "accepts_deferred_norm", False):
            return self.mixer_norm.defer(ctx, hidden, "mixer")
        return None

    def forward(self, ctx, cache, hidden, pre=None, after=None):
        """``pre``: this block's entry norm, already folded into the previous block's last
        product (or None); ``after``: the next block's entry norm for this block's last product
        to fold in.  Returns ``after`` if it was filled, else None."""
        x = pre if pre is not None and pre.ready else self.mixer_norm.forward(ctx, hidden)
        if self.feed_forward is None:
            if after is not None and getattr(self.mixer, "fuses_following_norm", False):
                self.mixer.forward(ctx, cache, x, hidden, then=after)
            else:
                self.mixer.forward(ctx, cache, x, hidden)
            return after if after is not None and after.ready else None
        mid = None
        if getattr(self.mixer, "fuses_following_norm", False) and \
                getattr(self.feed_forward, "accepts_deferred_norm", False):
            mid = self.ffn_norm.defer(ctx, hidden, "ffn")
        if mid is not None:
            self.mixer.forward(ctx, cache, x, hidden, then=mid)
        else:
            self.mixer.forward(ctx, cache, x, hidden)
        x = mid if mid is not None and mid.ready else self.ffn_norm.forward(ctx, hidden)
        if after is not None and getattr(self.feed_forward, "fuses_following_norm", False):
            self.feed_forward.forward(ctx, x, hidden, then=after)
        else:
            self.feed_forward.forward(ctx, x, hidden)
        return after if after is not None and after.ready else None


@BLOCKS.register("pre_norm_conv")
class PreNormConvBlock(Block):
    """``h += mixer(c1(norm(h))); h += ffn(c2(norm(h)))`` where ``c1`` and ``c2`` are convolution parts
    with state of their own (extra parts ``mixer_conv`` and ``ffn_conv``; either may be missing):
    what a sublayer reads passes through a short causal convolution over time first.  The norm's
    rows go to the convolution in fp32 where the norm offers that.  The arrangement keeps the
    convolutions' state beside the mixer's cache.  A layer without a feed-forward is the first half
    only."""

    def __init__(self, mixer, feed_forward, mixer_norm, ffn_norm, mixer_conv=None, ffn_conv=None, **extra):
        if mixer_norm is None or (feed_forward is None) != (ffn_norm is None) or extra or \
                (feed_forward is None and ffn_conv is not None):
            raise ValueError("the pre_norm_conv arrangement is norm, convolution, mixer and, optionally, norm, "
                             "convolution, feed-forward: it takes exactly those parts")
        super().__init__(mixer, feed_forward, mixer_norm, ffn_norm)
        self.mixer_conv, self.ffn_conv = mixer_conv, ffn_conv

    def cache_request(self):
        return CacheBundle({"mixer": self.mixer.cache_request(),
                            "mixer_conv": None if self.mixer_conv is None else self.mixer_conv.cache_request(),
                            "ffn_conv": None if self.ffn_conv is None else self.ffn_conv.cache_request()})

    @staticmethod
    def _read(ctx, hidden, norm, conv, cache, tag):
        if conv is None:
            return norm.forward(ctx, hidden)
        try:
            wide = norm.forward(ctx, hidden, out_name="normed_wide", dtype=torch.float32)
        except TypeError:                      # a norm that gives the run dtype only
            wide = norm.forward(ctx, hidden)
        return conv.forward(ctx, cache, wide, out_name="normed_conv_" + tag)

    def forward(self, ctx, cache, hidden):
        x = self._read(ctx, hidden, self.mixer_norm, self.mixer_conv, cache["mixer_conv"], "a")
        self.mixer.forward(ctx, cache["mixer"], x, hidden)
        if self.feed_forward is not None:
            x = self._read(ctx, hidden, self.ffn_norm, self.ffn_conv, cache["ffn_conv"], "b")
            self.feed_forward.forward(ctx, x, hidden)


@BLOCKS.register("parallel")
class ParallelBlock(Block):
    """``h <- h + mixer(norm_a(h)) + ffn(norm_b(h))``: both branches read the same ``h``, each
    through a norm of its own.  Both norms are made before either branch adds to the residual
    stream (in one pass over the rows where the kernels offer it: the two share the rows' mean
    square when they are RMS norms with one eps).  A layer without a feed-forward has the mixer
    branch only."""

    def __init__(self, mixer, feed_forward, mixer_norm, ffn_norm, **extra):
        if mixer_norm is None or (feed_forward is None) != (ffn_norm is None) or extra:
            raise ValueError("the parallel arrangement is a mixer with its norm and, optionally, a feed-forward with its")
        super().__init__(mixer, feed_forward, mixer_norm, ffn_norm)

    def forward(self, ctx, cache, hidden):
        a, b = self.mixer_norm, self.ffn_norm
        if b is None:
            self.mixer.forward(ctx, cache, a.forward(ctx, hidden), hidden)
            return
        pair = getattr(a, "forward_pair", None)
        if pair is not None and type(a) is type(b) and getattr(a, "eps", None) == getattr(b, "eps", 0):
            xa, xb = pair(ctx, hidden, b)
        else:
            xa = a.forward(ctx, hidden)
            xb = b.forward(ctx, hidden, out_name="normed_b")
        self.mixer.forward(ctx, cache, xa, hidden)
        self.feed_forward.forward(ctx, xb, hidden)


@BLOCKS.register("post_norm")
class PostNormBlock(Block):
    """``h += norm_a(mixer(h)); h += norm_b(ffn(h))``: a sublayer reads the residual stream itself, and the
    norm is on what it gives back.  Then, if the layer has one, a further part ``after`` (registry
    ``feed_forward``) that reads the stream and adds to it on its own terms.  A layer without a
    feed-forward (and without its norm) is the mixer's half only.

    The sublayer writes into a branch buffer: a part that declares ``writes_fresh`` is told so
    (``fresh=True``) and stores its result there; any other part adds into the zeroed buffer.  In a
    bfloat16 run the sublayers read the stream rounded to bfloat16; the kernel that adds a normed branch
    leaves that rounded copy for the next reader (``ctx.stream_copy``), so it is formed by a kernel of
    its own only where a block of another kind ran before."""

    keeps_stream_copy = True

    def __init__(self, mixer, feed_forward, mixer_norm, ffn_norm, after=None, **extra):
        if mixer_norm is None or (feed_forward is None) != (ffn_norm is None) or extra:
            raise ValueError("the post_norm arrangement is mixer, norm and, optionally, feed-forward, norm and a part "
                             "after them: it takes exactly those parts")
        for norm in (mixer_norm, ffn_norm):
            if norm is not None and not hasattr(norm, "add_normed"):
                raise ValueError("the post_norm arrangement needs norms that can add a normed branch to the stream")
        super().__init__(mixer, feed_forward, mixer_norm, ffn_norm)
        self.after = after

    @staticmethod
    def _read(ctx, rt, hidden):
        """The stream as the sublayers' products read it: itself in a 32-bit run, else its rounded copy."""
        if rt.dtype == torch.float32:
            return hidden, None
        copy = rt.buffer("stream_rounded", hidden.shape[0], hidden.shape[1], rt.dtype)
        if getattr(ctx, "stream_copy", None) is not copy:
            rt.ops.convert(hidden, copy)
            ctx.stream_copy = copy
        return copy, copy

    @staticmethod
    def _run(part, rt, branch, *args):
        if getattr(part, "writes_fresh", False):
            part.forward(*args, branch, fresh=True)
        else:
            rt.ops.zero(branch)
            part.forward(*args, branch)

    def forward(self, ctx, cache, hidden):
        rt = self.mixer.rt
        branch = rt.buffer("sublayer_out", hidden.shape[0], hidden.shape[1], torch.float32)
        x, copy = self._read(ctx, rt, hidden)
        folds = getattr(self.mixer, "adds_normed", None)
        if folds is not None and folds(self.mixer_norm):
            # the mixer adds its normed result itself (the norm folded into its last kernel)
            self.mixer.forward(ctx, cache, x, hidden, normed_by=self.mixer_norm, rounded=copy)
        else:
            self._run(self.mixer, rt, branch, ctx, cache, x)
            self.mixer_norm.add_normed(ctx, branch, hidden, rounded=copy)
        if self.feed_forward is not None:
            x, copy = self._read(ctx, rt, hidden)
            self._run(self.feed_forward, rt, branch, ctx, x)
            self.ffn_norm.add_normed(ctx, branch, hidden, rounded=copy)
        if self.after is not None:
            x, copy = self._read(ctx, rt, hidden)
            if getattr(self.after, "keeps_stream_copy", False):
                self.after.forward(ctx, x, hidden, rounded=copy)
            else:
                self.after.forward(ctx, x, hidden)
                ctx.stream_copy = None
