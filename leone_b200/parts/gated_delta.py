"""The gated delta rule: a recurrence whose state is corrected towards each new value.

``q = W_q x`` and ``k = W_k x`` (``kv_heads x dim``), ``v = W_v x`` (``heads x vdim``); each passes a short
causal convolution over time per channel (``conv_taps``; tensors ``<name>.conv`` ``[channels, taps]``, the
last ``taps - 1`` projected rows are state) and silu; q and k become unit vectors per head (``x /
sqrt(sum x^2 + 1e-6)``), q times ``dim^(-1/2)``; head ``h`` reads q/k head ``h // (heads / kv_heads)``.
Per head, with ``beta = sigmoid(W_b x)`` and ``g = exp(-exp(A_log) softplus(W_a x + dt_bias))``:

    S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q

so the read-out sees the token's own write.  Every head's ``o`` is divided by its root mean square over
``vdim``, multiplied by a weight ``[vdim]`` shared by the heads and by ``silu(W_g x)``, then ``W_o``.
The state ``[heads, dim, vdim]`` is fp32, starts at zero and lives in the request's state slot between
steps, beside the convolution's.  The input projections are one product with fp32 results; the
convolution, its activation, the unit norms, the gates, the decay and the recurrence are fp32.

(Yang et al., "Gated Delta Networks: Improving Mamba2 with Delta Rule" describes this recurrence.)
"""
from __future__ import annotations

import torch

from ..registry import MIXERS
from .base import CacheBundle, FixedState, Mixer, WeightSpec


@MIXERS.register("gated_delta_rule")
class GatedDeltaRule(Mixer):
    writes_fresh = True           # forward(..., fresh=True) stores its result instead of adding it

    def __init__(self, params, rt):
        super().__init__(params, rt)
        self.hidden = int(params["hidden_size"])
        self.heads = int(params["heads"])
        self.kv_heads = int(params.get("kv_heads") or self.heads)
        if self.heads % self.kv_heads:
            raise ValueError(f"gated_delta_rule: heads {self.heads} is not a multiple of kv_heads {self.kv_heads}")
        self.dim = int(params["dim"])
        self.vdim = int(params["vdim"])
        self.taps = int(params.get("conv_taps") or 0)
        self.eps = float(params["norm_eps"])
        self.q_scale = float(params.get("q_scale", self.dim ** -0.5))
        self.names = {k: params.get(f"{k}_name", k) for k in ("q", "k", "v", "g", "a", "b", "o", "norm", "A_log", "dt_bias")}
        self.conv_names = {k: params.get(f"{k}_conv_name", f"{self.names[k]}.conv") for k in ("q", "k", "v")}
        self.qk = self.kv_heads * self.dim
        self.hv = self.heads * self.vdim
        self.conv_cols = 2 * self.qk + self.hv
        # rows of the one input product: q, k, v (the convolution's channels), the gate, then a and b
        self.g_off = self.conv_cols
        self.a_off = self.g_off + self.hv
        self.b_off = self.a_off + self.heads
        self.cols = -(-(self.b_off + self.heads) // 16) * 16
        self.w_in = self.w_o = self.conv_w = self.norm_w = self.a_log = self.dt_bias = None

    def weight_specs(self):
        n = self.names
        rows = {"q": self.qk, "k": self.qk, "v": self.hv}
        specs = []
        for k in ("q", "k", "v"):
            specs.append(WeightSpec(n[k], (rows[k], self.hidden)))
            if self.taps:
                specs.append(WeightSpec(self.conv_names[k], (rows[k], self.taps), std=0.3))
        specs += [WeightSpec(n["b"], (self.heads, self.hidden)), WeightSpec(n["A_log"], (self.heads,), role="vector", std=0.5),
                  WeightSpec(n["norm"], (self.vdim,), role="norm", std=0.1), WeightSpec(n["a"], (self.heads, self.hidden)),
                  WeightSpec(n["dt_bias"], (self.heads,), role="vector", std=0.5),
                  WeightSpec(n["g"], (self.hv, self.hidden)), WeightSpec(n["o"], (self.hidden, self.hv))]
        return specs

    def load(self, tensors):
        n = self.names
        rows = [tensors[n[k]] for k in ("q", "k", "v", "g", "a", "b")]
        used = sum(r.shape[0] for r in rows)
        if used < self.cols:
            rows.append(torch.zeros((self.cols - used, self.hidden), dtype=rows[0].dtype, device=rows[0].device))
        self.w_in = self.rt.ops.prepare_matrix(torch.cat(rows, dim=0).contiguous())
        self.w_o = self.rt.ops.prepare_matrix(tensors[n["o"]])
        if self.taps:
            self.conv_w = torch.cat([tensors[self.conv_names[k]].float() for k in ("q", "k", "v")], dim=0).contiguous()
        else:       # no convolution: one tap of weight one, so that the same kernel applies the activation
            self.conv_w = torch.ones((self.conv_cols, 1), dtype=torch.float32, device=rows[0].device)
        self.norm_w = tensors[n["norm"]]
        self.a_log = tensors[n["A_log"]].float().contiguous()
        self.dt_bias = tensors[n["dt_bias"]].float().contiguous()

    def weight_bytes(self):
        return (self.cols * self.hidden + self.hidden * self.hv) * self.rt.dtype.itemsize

    def scratch_bytes(self, max_tokens):
        return max_tokens * ((self.cols + self.conv_cols + self.hv) * 4 + self.hv * self.rt.dtype.itemsize)

    def load_transient_bytes(self):
        return self.cols * self.hidden * self.rt.dtype.itemsize

    def cache_request(self):
        return CacheBundle({"state": FixedState((self.heads, self.dim, self.vdim)),
                            "conv": FixedState((self.taps - 1, self.conv_cols)) if self.taps > 1 else None})

    def forward(self, ctx, cache, x, hidden, fresh=False):
        rt, ops = self.rt, self.rt.ops
        n = hidden.shape[0]
        state, conv = cache["state"], cache["conv"]
        proj = rt.buffer("delta_proj", n, self.cols, torch.float32)
        ops.linear(x, self.w_in, proj)
        act = rt.buffer("delta_act", n, self.conv_cols, torch.float32)
        conv_state = conv.state if conv is not None else None
        raw = proj[:, :self.conv_cols]
        # a step of one token a sequence: the convolution's kernel moves its state on itself
        fused = conv_state is not None and conv.writes and bool(ctx.decode_only)
        ops.short_conv(ctx, raw, self.conv_w, conv_state, act, activation="silu", update_state=fused)
        if conv_state is not None and conv.writes and not fused:
            ops.short_conv_state(ctx, raw, conv_state)
        o = rt.buffer("delta_o", n, self.hv, torch.float32)
        ops.gated_delta(ctx, act, proj, o, state.state, self.a_log, self.dt_bias, self.heads, self.kv_heads, self.dim,
                        self.vdim, q_off=0, k_off=self.qk, v_off=2 * self.qk, a_off=self.a_off, b_off=self.b_off,
                        q_scale=self.q_scale)
        gated = rt.buffer("delta_gated", n, self.hv, rt.dtype)
        ops.group_gate_norm(o, self.norm_w, proj[:, self.g_off:self.g_off + self.hv], gated, self.eps, self.heads,
                            self.vdim, act="silu")
        ops.linear(gated, self.w_o, hidden, residual=None if fresh else hidden)
