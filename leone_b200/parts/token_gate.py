"""A per-layer token input: a slice of a second token table, gated by the stream, added to the stream.

``e`` = columns ``offset .. offset + dim`` of the token's row of the table ``table`` (which the model's
embedding part gathers once per step for all layers, ``ctx.token_rows[table]``); ``g = gelu_tanh(W_gate
x) * e``; ``y = W_proj g``; ``hidden += y / sqrt(mean(y^2) + eps) * w`` with a plain weight.  Tensors:
``gate`` ``[dim, hidden]``, ``proj`` ``[hidden, dim]``, ``norm`` ``[hidden]`` (names are parameters).
The gate's product has fp32 results, the activation and the norm are fp32.
"""
from __future__ import annotations

import torch

from ..registry import FEED_FORWARDS
from .base import FeedForward, WeightSpec


@FEED_FORWARDS.register("token_gate")
class TokenGate(FeedForward):
    keeps_stream_copy = True      # forward(..., rounded=) also leaves the new stream in the run dtype

    def __init__(self, params, rt):
        super().__init__(params, rt)
        self.hidden = int(params["hidden_size"])
        self.dim = int(params["dim"])
        self.offset = int(params.get("offset", 0))
        self.table = params["table"]
        self.eps = float(params["norm_eps"])
        self.names = {k: params.get(f"{k}_name", k) for k in ("gate", "proj", "norm")}
        self.w_gate = self.w_proj = self.norm_w = None

    def weight_specs(self):
        n = self.names
        return [WeightSpec(n["gate"], (self.dim, self.hidden)), WeightSpec(n["proj"], (self.hidden, self.dim)),
                WeightSpec(n["norm"], (self.hidden,), role="norm", std=0.1)]

    def load(self, tensors):
        n = self.names
        self.w_gate = self.rt.ops.prepare_matrix(tensors[n["gate"]])
        self.w_proj = self.rt.ops.prepare_matrix(tensors[n["proj"]])
        self.norm_w = tensors[n["norm"]]

    def weight_bytes(self):
        return 2 * self.dim * self.hidden * self.rt.dtype.itemsize

    def scratch_bytes(self, max_tokens):
        return max_tokens * (self.dim * (4 + self.rt.dtype.itemsize) + self.hidden * 4)

    def forward(self, ctx, x, hidden, rounded=None):
        rt, ops = self.rt, self.rt.ops
        n = hidden.shape[0]
        rows = ctx.token_rows.get(self.table)
        if rows is None:
            raise ValueError(f"token_gate: the embedding part gathers no rows of table '{self.table}'")
        z = rt.buffer("token_gate_z", n, self.dim, torch.float32)
        ops.linear(x, self.w_gate, z)
        g = rt.buffer("token_gate_g", n, self.dim, rt.dtype)
        ops.gelu_gate(z, rows, self.offset, g)
        y = rt.buffer("token_gate_y", n, self.hidden, torch.float32)
        ops.linear(g, self.w_proj, y)
        ops.rms_norm_add(hidden, y, self.norm_w, self.eps, rounded=rounded)
