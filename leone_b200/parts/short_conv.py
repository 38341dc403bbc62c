"""A short causal convolution over time on every channel, with state.

``y_t = sum_j w[:, j] x_(t - taps + 1 + j)`` (``w`` stored ``[channels, taps]``, no bias; inputs
before a sequence's start are zero), optionally plus ``x_t`` itself (``add_input``).  The last
``taps - 1`` inputs of every sequence are fixed-size state (fp32, one record per request slot), so a
sequence may be cut anywhere.  Used where an arrangement or a mixer puts such a convolution in front
of something: the part turns rows ``x`` into rows ``y`` and advances its state.
"""
from __future__ import annotations

import torch

from ..registry import CONVS
from .base import FixedState, Part, WeightSpec


@CONVS.register("short_conv")
class ShortConv(Part):
    def __init__(self, params, rt):
        super().__init__(params, rt)
        self.channels = int(params["channels"])
        self.taps = int(params["taps"])
        if not 1 <= self.taps <= 16:
            raise ValueError(f"short_conv: taps {self.taps} (1 to 16)")
        self.add_input = bool(params.get("add_input", False))
        self.name = params.get("name", "conv")
        self.weight = None

    def weight_specs(self):
        return [WeightSpec(self.name, (self.channels, self.taps), std=0.2)]

    def load(self, tensors):
        self.weight = tensors[self.name].float().contiguous()

    def weight_bytes(self):
        return self.channels * self.taps * 4

    def scratch_bytes(self, max_tokens):
        return max_tokens * self.channels * self.rt.dtype.itemsize

    def cache_request(self):
        return FixedState((self.taps - 1, self.channels)) if self.taps > 1 else None

    def forward(self, ctx, cache, x, out_name="conv_out", out_dtype=None):
        """``x``: ``[N, channels]`` fp32 or the run dtype; returns ``[N, channels]`` in the run dtype
        (or ``out_dtype``) and leaves the state as it is after the step's tokens."""
        rt, ops = self.rt, self.rt.ops
        out = rt.buffer(out_name, x.shape[0], self.channels, out_dtype or rt.dtype)
        state = cache.state if cache is not None else None
        # a step of one token a sequence: the convolution's kernel moves the state on itself
        fused = state is not None and cache.writes and bool(ctx.decode_only)
        ops.short_conv(ctx, x, self.weight, state, out, add_input=self.add_input, update_state=fused)
        if state is not None and cache.writes and not fused:
            ops.short_conv_state(ctx, x, state)
        return out
