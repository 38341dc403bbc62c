"""Parts that rewrite the residual stream between layers.

``concat_linear``: ``x <- W [x; x0]`` with ``W`` stored ``[hidden, 2 hidden]`` (the stream's columns
first), ``x0`` being what the embedding left.  The two halves of ``W`` are kept apart, so that the
product over ``x0``, which is the same at every place the part runs in a step, is formed once per
step (fp32) and the product over ``x`` adds it in its epilogue.

``add_origin``: ``x <- x + scale * x0``, no weights: the embedding's rows added to the stream again.
"""
from __future__ import annotations

import torch

from ..registry import INJECTIONS
from .base import Injection, WeightSpec


@INJECTIONS.register("concat_linear")
class ConcatLinear(Injection):
    def __init__(self, params, rt):
        super().__init__(params, rt)
        self.hidden = int(params["hidden_size"])
        self.name = params["name"]
        self.w_stream = self.w_origin = None
        self._origin_done = False     # whether this step's product over x0 sits in the buffer

    def weight_specs(self):
        return [WeightSpec(self.name, (self.hidden, 2 * self.hidden))]

    def load(self, tensors):
        w = tensors[self.name]
        self.w_stream = self.rt.ops.prepare_matrix(w[:, :self.hidden].contiguous())
        self.w_origin = self.rt.ops.prepare_matrix(w[:, self.hidden:].contiguous())

    def weight_bytes(self):
        return 2 * self.hidden * self.hidden * self.rt.dtype.itemsize

    def scratch_bytes(self, max_tokens):
        return max_tokens * self.hidden * (4 + self.rt.dtype.itemsize)

    def load_transient_bytes(self):
        return 2 * self.hidden * self.hidden * self.rt.dtype.itemsize

    def begin_step(self, ctx):
        self._origin_done = False

    def forward(self, ctx, hidden, origin):
        rt, ops = self.rt, self.rt.ops
        n = hidden.shape[0]
        operand = rt.buffer("inject_operand", n, self.hidden, rt.dtype)
        const = rt.buffer("inject_origin_part", n, self.hidden, torch.float32)
        if not self._origin_done:
            ops.convert(origin, operand)
            ops.linear(operand, self.w_origin, const)
            self._origin_done = True
        ops.convert(hidden, operand)
        ops.linear(operand, self.w_stream, hidden, residual=const)


@INJECTIONS.register("add_origin")
class AddOrigin(Injection):
    def __init__(self, params, rt):
        super().__init__(params, rt)
        self.scale = float(params.get("scale", 1.0))

    def forward(self, ctx, hidden, origin):
        self.rt.ops.add_scaled(hidden, origin, self.scale)
