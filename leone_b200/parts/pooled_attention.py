"""Attention over a sliding window of tokens and, before the window, pooled blocks.

``q, k, v = W_qkv x`` (``heads`` query heads on ``kv_heads`` key/value heads, key width ``head_dim``,
value width ``value_head_dim``); optionally a short causal convolution over time on every channel of
q, k and v (``conv_taps``; the last ``taps - 1`` projected rows are state); a rotation of q and k (a
position encoding that offers its frequencies: partial, half-split or adjacent pairs, YaRN with its
magnitude on cos and sin); optionally q and k divided by their root mean square per head after the
rotation (``unit_norm``, no weight).  The query at position ``p`` sees the keys ``j`` with ``0 <= p -
j < window`` and one mean key and value for every block of ``pool`` positions that lies wholly before
the window (block ``b`` holds positions ``b pool .. b pool + pool - 1`` and is seen when ``b pool +
pool - 1 <= p - window``); tokens that left the window and whose block is not yet complete are not
seen.  One softmax over ``(q . k) * scale`` for all of them; ``hidden += out_scale * W_o out``.

Three caches: the token rows (pages go back once ``window + pool`` positions lie behind them), the
block means (one row per ``pool`` positions, kept for the request's life; a block's means are formed
from the token rows as the cache holds them, in the step that brings the block's last token), and the
convolution's state.
"""
from __future__ import annotations

import torch

from ..registry import MIXERS
from .base import CacheBundle, FixedState, Mixer, PagedKV, WeightSpec


@MIXERS.register("pooled_window_attention")
class PooledWindowAttention(Mixer):
    def __init__(self, params, rt, position_encodings=None):
        super().__init__(params, rt)
        self.hidden = int(params["hidden_size"])
        self.n_q = int(params["num_heads"])
        self.n_kv = int(params["num_kv_heads"])
        self.d = int(params["head_dim"])
        self.dv = int(params.get("value_head_dim") or self.d)
        if self.n_q % self.n_kv:
            raise ValueError(f"num_heads {self.n_q} is not a multiple of num_kv_heads {self.n_kv}")
        self.scale = float(params["scale"])
        self.window = int(params["window"])
        self.pool = int(params["pool"])
        if self.window <= 0 or self.pool <= 0:
            raise ValueError(f"pooled_window_attention: window {self.window}, pool {self.pool}")
        self.taps = int(params.get("conv_taps") or 0)
        self.unit_norm = bool(params.get("unit_norm", False))
        self.eps = float(params.get("norm_eps", 1e-6))
        self.out_scale = float(params.get("out_scale", 1.0))
        pe_name = params.get("position_encoding")
        self.pos = (position_encodings or {}).get(pe_name) if pe_name else None
        if pe_name and (self.pos is None or not hasattr(self.pos, "frequencies")):
            raise ValueError(f"pooled_window_attention needs position encoding '{pe_name}' to offer its frequencies")
        self.names = {k: params.get(f"{k}_name", k) for k in ("q", "k", "v", "o")}
        self.conv_names = {k: params.get(f"{k}_conv_name", f"{self.names[k]}.conv") for k in ("q", "k", "v")}
        self.cols = (self.n_q + self.n_kv) * self.d + self.n_kv * self.dv
        self.w_qkv = self.w_o = self.conv_w = None

    def weight_specs(self):
        n = self.names
        rows = {"q": self.n_q * self.d, "k": self.n_kv * self.d, "v": self.n_kv * self.dv}
        specs = [WeightSpec(n[k], (rows[k], self.hidden)) for k in ("q", "k", "v")]
        if self.taps:
            specs += [WeightSpec(self.conv_names[k], (rows[k], self.taps), std=0.3) for k in ("q", "k", "v")]
        specs.append(WeightSpec(n["o"], (self.hidden, self.n_q * self.dv)))
        return specs

    def load(self, tensors):
        n = self.names
        stacked = torch.cat([tensors[n["q"]], tensors[n["k"]], tensors[n["v"]]], dim=0).contiguous()
        self.w_qkv = self.rt.ops.prepare_matrix(stacked)
        self.w_o = self.rt.ops.prepare_matrix(tensors[n["o"]])
        if self.taps:
            self.conv_w = torch.cat([tensors[self.conv_names[k]].float() for k in ("q", "k", "v")], dim=0).contiguous()

    def weight_bytes(self):
        return (self.cols * self.hidden + self.hidden * self.n_q * self.dv) * self.rt.dtype.itemsize

    def scratch_bytes(self, max_tokens):
        return max_tokens * (self.cols * 4 + self.n_q * (self.d + self.dv) * self.rt.dtype.itemsize)

    def load_transient_bytes(self):
        return self.cols * self.hidden * self.rt.dtype.itemsize

    def cache_request(self):
        members = {
            # a token row is read as a key for `window` positions and once more when its block's means are formed
            "tokens": PagedKV(self.n_kv, self.d, self.window + self.pool, value_head_dim=self.dv, tag="window+pool"),
            "blocks": PagedKV(self.n_kv, self.d, None, value_head_dim=self.dv, tag="block means",
                              tokens_per_row=self.pool),
            "conv": FixedState((self.taps - 1, self.cols)) if self.taps > 1 else None,
        }
        return CacheBundle(members)

    def forward(self, ctx, cache, x, hidden):
        rt, ops = self.rt, self.rt.ops
        n = hidden.shape[0]
        tokens, blocks, conv = cache["tokens"], cache["blocks"], cache["conv"]
        proj = rt.buffer("pooled_attn_proj", n, self.cols, torch.float32)
        ops.linear(x, self.w_qkv, proj)
        q = rt.buffer("pooled_attn_q", n, self.n_q * self.d, rt.dtype)
        freqs, pairing, magnitude = None, "half_split", 1.0
        if self.pos is not None:
            freqs, pairing, magnitude = self.pos.frequencies(), self.pos.pairing, float(getattr(self.pos, "magnitude", 1.0))
        state = conv.state if conv is not None else None
        # a step of one token a sequence: the preparation kernel moves the convolution's state on itself
        fused = state is not None and conv.writes and bool(ctx.decode_only)
        ops.attention_pooled_prepare(ctx, proj, q, self.n_q, self.n_kv, self.d, self.dv, self.conv_w, state, freqs,
                                     pairing, magnitude, self.unit_norm, self.eps, tokens, update_state=fused)
        if state is not None and conv.writes and not fused:
            ops.short_conv_state(ctx, proj, state)
        if tokens.writes:
            ops.attention_pool_blocks(ctx, tokens, blocks, self.n_kv, self.d, self.dv, self.pool)
        out = rt.buffer("attn_out", n, self.n_q * self.dv, rt.dtype)
        ops.attention_pooled(ctx, q, out, tokens, blocks, self.n_q, self.n_kv, self.d, self.dv, self.scale, self.window,
                             self.pool, out_scale=self.out_scale)
        ops.linear(out, self.w_o, hidden, residual=hidden)
