"""minGRU: a gated recurrence whose gates read only the current token.

``z = sigmoid(W_z x + b_z)``, ``u = W_x x + b_x``, candidate ``c = u + 1/2`` where ``u >= 0`` and
``sigmoid(u)`` where ``u < 0``; element by element ``S_t = (1 - z_t) S_(t-1) + z_t c_t``; the mixer's
output is ``out_scale * W_o (S_t * silu(W_g x))`` added to the residual stream.  The state
``[width]`` is fp32, starts at zero and lives in the request's state slot between steps.  The three
input projections are one product with fp32 results; gates, candidate and state are fp32.  The
recurrence is linear in ``S``, so prompt portions longer than ``2 chunk`` tokens are cut into chunks
that run side by side (per-chunk sums, a pass over the chunks, then the outputs).  Chunks are short:
a thread walks a chunk's tokens one after the other, and a prompt of a few thousand tokens should
still give every SM several blocks.

(Feng et al., "Were RNNs All We Needed?" describes minGRU and this candidate function.)
"""
from __future__ import annotations

import torch

from ..registry import MIXERS
from .base import FixedState, Mixer, WeightSpec


DEFAULT_CHUNK = 16


@MIXERS.register("min_gru")
class MinGRU(Mixer):
    def __init__(self, params, rt):
        super().__init__(params, rt)
        self.hidden = int(params["hidden_size"])
        self.width = int(params["width"])
        self.out_scale = float(params.get("out_scale", 1.0))
        self.chunk = int(params.get("chunk", DEFAULT_CHUNK))
        self.names = {k: params.get(f"{k}_name", k) for k in ("z", "x", "g", "o")}
        self.bias_names = {k: params.get(f"{k}_bias_name", f"{k}.b") for k in ("z", "x")}
        self.w_in = self.w_o = self.z_bias = self.x_bias = None

    def weight_specs(self):
        n, b = self.names, self.bias_names
        return [WeightSpec(n["z"], (self.width, self.hidden)), WeightSpec(b["z"], (self.width,), role="vector", std=0.5),
                WeightSpec(n["x"], (self.width, self.hidden)), WeightSpec(b["x"], (self.width,), role="vector", std=0.5),
                WeightSpec(n["g"], (self.width, self.hidden)), WeightSpec(n["o"], (self.hidden, self.width))]

    def load(self, tensors):
        n, b = self.names, self.bias_names
        stacked = torch.cat([tensors[n["z"]], tensors[n["x"]], tensors[n["g"]]], dim=0).contiguous()
        self.w_in = self.rt.ops.prepare_matrix(stacked)
        self.w_o = self.rt.ops.prepare_matrix(tensors[n["o"]])
        self.z_bias = tensors[b["z"]].float().contiguous()
        self.x_bias = tensors[b["x"]].float().contiguous()

    def weight_bytes(self):
        return 4 * self.width * self.hidden * self.rt.dtype.itemsize

    def scratch_bytes(self, max_tokens):
        chunks = max_tokens // max(self.chunk, 1) + 1
        return max_tokens * self.width * (12 + self.rt.dtype.itemsize) + 2 * chunks * self.width * 4

    def load_transient_bytes(self):
        return 3 * self.width * self.hidden * self.rt.dtype.itemsize

    def cache_request(self):
        return FixedState((self.width,))

    def forward(self, ctx, cache, x, hidden):
        rt, ops = self.rt, self.rt.ops
        n = hidden.shape[0]
        proj = rt.buffer("min_gru_proj", n, 3 * self.width, torch.float32)
        ops.linear(x, self.w_in, proj)
        gated = rt.buffer("min_gru_out", n, self.width, rt.dtype)
        chunk = 0
        if not ctx.decode_only and self.chunk > 0 and ctx.max_q_len > 2 * self.chunk:
            chunk = self.chunk
        ops.min_gru(ctx, proj, self.z_bias, self.x_bias, cache.state, gated, out_scale=self.out_scale, chunk=chunk)
        ops.linear(gated, self.w_o, hidden, residual=hidden)
