"""Attention through a cached latent, with a sliding window, a softmax sink and an output gate.

Per head ``dim`` unrotated and ``rot_dim`` rotated query/key dimensions, values of ``vdim``, a latent
of ``kv_rank``.  ``q = W_q x`` laid out head by head as [dim | rot_dim].  ``W_dkv x`` has ``kv_rank +
rot_dim`` rows: the first ``kv_rank``, RMS-normed with a weight, are the latent ``c``; the last
``rot_dim`` are one key part shared by all heads, rotated by the position encoding like the queries'
rotated parts.  A head's unrotated key is ``W_uk c`` and its value ``W_uv c``, so only ``c`` and the
rotated part are cached (one row of ``kv_rank + rot_dim`` per token, no value pool), and the two
products are moved to the query side: ``q_lat = W_uk^T q_plain`` and ``out = W_uv sum_j w_j c_j``.
``score = (q_plain . k_plain + q_rot . k_rot) * scale`` over the keys of the window (``None`` = all),
softmax in fp32 whose denominator also holds ``exp(sink_h)`` if the mixer has sinks, each head's
result multiplied by ``sigmoid(W_g x)_h`` if it has an output gate, then ``W_o``.

Every size and constant is a parameter: the window, the scale, whether there are sinks and a gate,
and which position encoding rotates (one that offers ``frequencies()``).

``q_rank``: the queries go through a latent too: ``c_q = rms_norm(W_dq x) * w`` (``q_rank`` wide, the
layer's eps), ``q = W_uq c_q`` (tensors ``dq``, ``dq_norm``, ``uq`` instead of ``q``).  ``gate =
"elementwise"``: ``W_g`` has ``heads * vdim`` rows and the concatenated heads are multiplied element by
element with ``sigmoid(W_g x)`` (``gate = True``: one number per head).
"""
from __future__ import annotations

import torch

from ..registry import MIXERS
from .base import Mixer, PagedKV, WeightSpec


@MIXERS.register("latent_attention")
class LatentAttention(Mixer):
    writes_fresh = True           # forward(..., fresh=True) stores its result instead of adding it

    def __init__(self, params, rt, position_encodings=None):
        super().__init__(params, rt)
        self.hidden = int(params["hidden_size"])
        self.heads = int(params["heads"])
        self.dim = int(params["dim"])
        self.rot_dim = int(params["rot_dim"])
        self.vdim = int(params["vdim"])
        self.rank = int(params["kv_rank"])
        self.scale = float(params["scale"])
        self.window = params.get("window")
        self.eps = float(params["eps"])
        self.has_sink = bool(params.get("sink", False))
        self.gate_elementwise = params.get("gate") == "elementwise"
        self.has_gate = bool(params.get("gate", False)) and not self.gate_elementwise
        self.q_rank = int(params.get("q_rank") or 0)
        pe_name = params.get("position_encoding")
        self.pos = (position_encodings or {}).get(pe_name) if pe_name else None
        if pe_name and self.pos is None:
            raise ValueError(f"latent attention names position encoding '{pe_name}' that the model lacks")
        if self.pos is not None and not hasattr(self.pos, "frequencies"):
            raise ValueError("latent attention rotates with an encoding that offers frequencies()")
        self.names = {k: params.get(f"{k}_name", k)
                      for k in ("q", "dkv", "dkv_norm", "uk", "uv", "sink", "g", "o", "dq", "dq_norm", "uq")}
        self.q_cols = self.heads * (self.dim + self.rot_dim)
        self.dk = self.rank + self.rot_dim
        self.gate_rows = self.heads if self.has_gate else (self.heads * self.vdim if self.gate_elementwise else 0)
        # q, dkv and the gate rows are one product; its rows are padded to a multiple of 16.  With a query
        # latent the queries come from a product of their own and start a padded row apart from the rest.
        self.rest_off = -(-self.q_cols // 16) * 16 if self.q_rank else self.q_cols
        self.cols = -(-(self.rest_off + self.dk + self.gate_rows) // 16) * 16
        self.w_in = self.w_ukt = self.w_uv = self.w_o = self.norm_w = self.sink = None
        self.w_dq = self.w_uq = self.dq_norm_w = None

    def weight_specs(self):
        n = self.names
        if self.q_rank:
            first = [WeightSpec(n["dq"], (self.q_rank, self.hidden)), WeightSpec(n["dq_norm"], (self.q_rank,), role="norm", std=0.1),
                     WeightSpec(n["uq"], (self.q_cols, self.q_rank))]
        else:
            first = [WeightSpec(n["q"], (self.q_cols, self.hidden))]
        specs = first + [WeightSpec(n["dkv"], (self.dk, self.hidden)),
                 WeightSpec(n["dkv_norm"], (self.rank,), role="norm", std=0.1),
                 WeightSpec(n["uk"], (self.heads * self.dim, self.rank)),
                 WeightSpec(n["uv"], (self.heads * self.vdim, self.rank))]
        if self.has_sink:
            specs.append(WeightSpec(n["sink"], (self.heads,), role="vector", std=1.0))
        if self.gate_rows:
            specs.append(WeightSpec(n["g"], (self.gate_rows, self.hidden)))
        specs.append(WeightSpec(n["o"], (self.hidden, self.heads * self.vdim)))
        return specs

    def load(self, tensors):
        n = self.names
        rows = [tensors[n["dkv"]]] if self.q_rank else [tensors[n["q"]], tensors[n["dkv"]]]
        if self.gate_rows:
            rows.append(tensors[n["g"]])
        used = sum(r.shape[0] for r in rows)
        want = self.cols - self.rest_off if self.q_rank else self.cols
        if used < want:
            rows.append(torch.zeros((want - used, self.hidden), dtype=rows[0].dtype, device=rows[0].device))
        if self.q_rank:
            self.w_dq = self.rt.ops.prepare_matrix(tensors[n["dq"]])
            self.w_uq = self.rt.ops.prepare_matrix(tensors[n["uq"]])
            self.dq_norm_w = tensors[n["dq_norm"]]
        self.w_in = self.rt.ops.prepare_matrix(torch.cat(rows, dim=0).contiguous())
        # W_uk [heads * dim, rank] as [heads, rank, dim]: the product that moves it to the query side
        self.w_ukt = tensors[n["uk"]].view(self.heads, self.dim, self.rank).transpose(1, 2).contiguous()
        self.w_uv = tensors[n["uv"]].contiguous()             # [heads * vdim, rank]
        self.w_o = self.rt.ops.prepare_matrix(tensors[n["o"]])
        self.norm_w = tensors[n["dkv_norm"]]
        self.sink = tensors[n["sink"]] if self.has_sink else None

    def weight_bytes(self):
        q_side = self.q_rank * (self.hidden + self.q_cols) - self.q_cols * self.hidden if self.q_rank else 0
        return (self.cols * self.hidden + q_side + self.heads * (self.dim + self.vdim) * self.rank
                + self.hidden * self.heads * self.vdim) * self.rt.dtype.itemsize

    def scratch_bytes(self, max_tokens):
        return max_tokens * (self.cols + self.heads * (self.dk + self.rank + self.vdim)) * self.rt.dtype.itemsize

    def load_transient_bytes(self):
        return (self.cols * self.hidden + self.heads * self.dim * self.rank) * self.rt.dtype.itemsize

    def cache_request(self):
        # one row per token: the normed latent and the shared rotated key part; no values
        return PagedKV(1, self.dk, self.window, value_head_dim=0, tag="latent")

    def forward(self, ctx, cache, x, hidden, fresh=False):
        rt, ops = self.rt, self.rt.ops
        n = hidden.shape[0]
        proj = rt.buffer("latent_proj", n, self.cols, rt.dtype)
        if self.q_rank:
            cq_wide = rt.buffer("latent_cq_wide", n, self.q_rank, torch.float32)
            ops.linear(x, self.w_dq, cq_wide)
            cq = rt.buffer("latent_cq", n, self.q_rank, rt.dtype)
            ops.rms_norm(cq_wide, self.dq_norm_w, cq, self.eps)
            ops.linear(cq, self.w_uq, proj[:, :self.q_cols])
            ops.linear(x, self.w_in, proj[:, self.rest_off:])
        else:
            ops.linear(x, self.w_in, proj)
        q_abs = rt.buffer("latent_q", n, self.heads * self.dk, rt.dtype)
        freqs, magnitude, pairing = None, 1.0, "adjacent"
        if self.pos is not None:
            freqs, magnitude, pairing = self.pos.frequencies(), self.pos.magnitude, self.pos.pairing
        ops.latent_prepare(ctx, proj, q_abs, self.heads, self.dim, self.rot_dim, self.rank, self.norm_w, self.eps,
                           freqs, magnitude, pairing, cache if cache.writes else None,
                           q_off=0, dkv_off=self.rest_off)
        # q_lat[t, h, :] = W_uk[h]^T q_plain[t, h, :]
        ops.linear_per_head(proj, self.dim + self.rot_dim, self.w_ukt, q_abs, self.dk, self.heads, self.dim, self.rank)
        o_lat = rt.buffer("latent_o", n, self.heads * self.rank, rt.dtype)
        gate = proj[:, self.rest_off + self.dk:] if self.has_gate else None
        ops.attention_latent(ctx, q_abs, o_lat, cache, self.heads, self.dk, self.rank, self.scale, self.window,
                             self.sink, gate)
        # out[t, h, :] = W_uv[h] o_lat[t, h, :]
        out = rt.buffer("latent_out", n, self.heads * self.vdim, rt.dtype)
        ops.linear_per_head(o_lat, self.rank, self.w_uv.view(self.heads, self.vdim, self.rank), out, self.vdim,
                            self.heads, self.rank, self.vdim)
        if self.gate_elementwise:
            g0 = self.rest_off + self.dk
            ops.gate_rows(out, proj[:, g0:g0 + self.heads * self.vdim], "sigmoid")
        ops.linear(out, self.w_o, hidden, residual=None if fresh else hidden)
