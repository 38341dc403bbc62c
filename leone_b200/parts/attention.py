"""Causal grouped-query attention over a paged cache.

One step of the reference's layer (crates/leone/src/runtime.rs:9111-9157):
``q, k, v = W_qkv x``; per-head RMSNorm of q and k with one weight ``[head_dim]``
shared by all heads and the layer's eps, v untouched
(crates/leone/src/model.rs:601-631, crates/leone/src/cpu.rs:802-820); rotary
on q and k; k and v written at their positions; for a query at absolute
position ``p`` the keys ``max(0, p-window+1) .. p`` are read with
``kv_head = q_head // (n_q / n_kv)``, ``score = (q.k) / sqrt(head_dim)``,
softmax and weighted sum in fp32 (crates/leone/src/cpu.rs:2299-2421); then
``hidden += W_o attn``.  The window is this part's own parameter (``None`` =
all keys); the reference has no windowed layer.

Every size is a parameter: number of heads, groups, head size (independent of
the hidden size), presence of the q/k norm, the position encoding and the
window.

Further parameters, this part's own (the reference has none of them); with any of them the layer
runs on the kernels of ``csrc/attention_masked.cu``:

``value_head_dim``: values of another width than queries and keys.
``mask``: what the query at position ``p`` sees besides ``j <= p``: ``"causal"`` (everything),
``"window"`` (``p - j < window``) or ``"chunk"`` (``floor(j / chunk) == floor(p / chunk)``, chunks
counted from position 0 of the sequence).
``weights``: how scores become weights: ``"softmax"``; ``"softmax_plus_one"`` (``exp(s_j) / (1 +
sum exp(s_j))``: one more member of score 0 without a value); ``"sigmoid"`` (``sigmoid(s_j +
b_head)`` for every seen key on its own, nothing normalised; ``b`` is the tensor ``bias_name``).
``qk_norm = "whole"``: one RMS norm over all of a token's query heads together (weight
``[heads * head_dim]``, multiplied directly) and one over its key heads, before rotation.
A position encoding that offers ``frequencies()`` instead of a table (``rotary_computed``): the
kernel forms the angles in fp32, on the first ``rotary_dim`` elements of a head.

Scores mixed across heads (``csrc/attention_mixed_heads.cu``; softmax weights only), each part of it
present when its parameter is: ``head_temp_name`` (a tensor ``[heads]``: the head's score is multiplied
by its number), ``score_cap`` (``cap * tanh(score / cap)``), ``head_mix_name`` (a tensor ``[heads,
heads]``: after scale, temperature and cap, head ``h``'s score becomes ``sum_g M[h, g] score_g``, before
the mask and the softmax), ``sink_name`` (a tensor ``[heads]``: the softmax's denominator also holds
``exp(sink_h)``, a member without key or value that is neither scaled nor capped nor mixed).
"""
from __future__ import annotations

import math

import torch

from ..registry import MIXERS
from .base import DeferredNorm, Mixer, PagedKV, WeightSpec


@MIXERS.register("attention")
class Attention(Mixer):
    accepts_deferred_norm = True
    fuses_following_norm = True
    writes_fresh = True           # forward(..., fresh=True) stores its result instead of adding it

    def __init__(self, params, rt, position_encodings=None):
        super().__init__(params, rt)
        self.hidden = int(params["hidden_size"])
        self.n_q = int(params["num_heads"])
        self.n_kv = int(params["num_kv_heads"])
        self.d = int(params["head_dim"])
        if self.n_q % self.n_kv:
            raise ValueError(f"num_heads {self.n_q} is not a multiple of num_kv_heads {self.n_kv}")
        self.dv = int(params.get("value_head_dim") or self.d)
        norm = params.get("qk_norm", False)
        self.qk_norm = bool(norm)
        self.norm_whole = norm == "whole"
        self.eps = float(params.get("qk_norm_eps", 1e-6))
        self.window = params.get("window")
        self.chunk = params.get("chunk")
        self.mask = params.get("mask") or ("window" if self.window else "causal")
        self.weights = params.get("weights", "softmax")
        if self.mask not in ("causal", "window", "chunk") or self.weights not in ("softmax", "softmax_plus_one", "sigmoid"):
            raise ValueError(f"attention: mask '{self.mask}' / weights '{self.weights}'")
        if (self.mask == "window") != bool(self.window) or (self.mask == "chunk") != bool(self.chunk):
            raise ValueError(f"attention: mask '{self.mask}' with window {self.window} and chunk {self.chunk}")
        self.bias_name = params.get("bias_name", "bias")
        self.bias = None
        self.temp_name, self.mix_name = params.get("head_temp_name"), params.get("head_mix_name")
        self.sink_name = params.get("sink_name")
        cap = params.get("score_cap")
        self.score_cap = float(cap) if cap else None
        self.temp = self.mix = self.sink = None
        self.mixed = bool(self.temp_name or self.mix_name or self.sink_name or self.score_cap)
        if self.mixed and self.weights != "softmax":
            raise ValueError("attention: temperature, cap, mixing and sink go with softmax weights")
        self.scale = float(params.get("scale", 1.0 / math.sqrt(self.d)))
        pe_name = params.get("position_encoding")
        self.pos = (position_encodings or {}).get(pe_name) if pe_name else None
        if pe_name and self.pos is None:
            raise ValueError(f"attention names position encoding '{pe_name}' that the model lacks")
        self.names = {k: params.get(f"{k}_name", f"{k}_proj.weight") for k in ("q", "k", "v", "o")}
        self.q_norm_name = params.get("q_norm_name", "q_norm.weight")
        self.k_norm_name = params.get("k_norm_name", "k_norm.weight")
        self.w_qkv = self.w_o = self.q_norm_w = self.k_norm_w = None
        self.qkv_cols = (self.n_q + self.n_kv) * self.d + self.n_kv * self.dv
        # the layer as the reference has it runs on the kernels tuned for it; anything else on the general ones
        self.general = (self.dv != self.d or self.mask == "chunk" or self.weights != "softmax" or self.norm_whole
                        or self.mixed or (self.pos is not None and hasattr(self.pos, "frequencies")))
        if self.general and self.pos is not None and not hasattr(self.pos, "frequencies"):
            raise ValueError("attention: the general kernels take a position encoding that offers its frequencies")

    def weight_specs(self):
        specs = [WeightSpec(self.names["q"], (self.n_q * self.d, self.hidden)),
                 WeightSpec(self.names["k"], (self.n_kv * self.d, self.hidden)),
                 WeightSpec(self.names["v"], (self.n_kv * self.dv, self.hidden)),
                 WeightSpec(self.names["o"], (self.hidden, self.n_q * self.dv))]
        if self.qk_norm:
            nq, nk = (self.n_q * self.d, self.n_kv * self.d) if self.norm_whole else (self.d, self.d)
            specs += [WeightSpec(self.q_norm_name, (nq,), role="norm", std=0.1),
                      WeightSpec(self.k_norm_name, (nk,), role="norm", std=0.1)]
        if self.weights == "sigmoid":
            specs.append(WeightSpec(self.bias_name, (self.n_q,), role="vector", std=0.5))
        if self.temp_name:
            specs.append(WeightSpec(self.temp_name, (self.n_q,), role="norm", std=0.2))
        if self.mix_name:
            specs.append(WeightSpec(self.mix_name, (self.n_q, self.n_q), role="vector", std=0.3))
        if self.sink_name:
            specs.append(WeightSpec(self.sink_name, (self.n_q,), role="vector", std=1.0))
        return specs

    def load(self, tensors):
        stacked = torch.cat([tensors[self.names["q"]], tensors[self.names["k"]],
                             tensors[self.names["v"]]], dim=0).contiguous()
        self.w_qkv = self.rt.ops.prepare_matrix(stacked)
        self.w_o = self.rt.ops.prepare_matrix(tensors[self.names["o"]])
        self.q_norm_f32 = self.k_norm_f32 = None
        if self.qk_norm:
            self.q_norm_w = tensors[self.q_norm_name]
            self.k_norm_w = tensors[self.k_norm_name]
            # fp32 copies for the decode kernel that does the norm itself
            self.q_norm_f32 = self.q_norm_w.float().contiguous()
            self.k_norm_f32 = self.k_norm_w.float().contiguous()
        if self.weights == "sigmoid":
            self.bias = tensors[self.bias_name].float().contiguous()
        self.temp = tensors[self.temp_name].float().contiguous() if self.temp_name else None
        self.mix = tensors[self.mix_name].float().contiguous() if self.mix_name else None
        self.sink = tensors[self.sink_name].float().contiguous() if self.sink_name else None

    def weight_bytes(self):
        return (self.qkv_cols * self.hidden + self.hidden * self.n_q * self.dv) * self.rt.dtype.itemsize

    def scratch_bytes(self, max_tokens):
        return max_tokens * (self.qkv_cols + self.n_q * self.dv) * self.rt.dtype.itemsize

    def load_transient_bytes(self):
        return self.qkv_cols * self.hidden * self.rt.dtype.itemsize       # q, k, v beside their stacked copy

    def cache_request(self):
        return PagedKV(self.n_kv, self.d, self.window, value_head_dim=self.dv)

    def _out_proj(self, attn, hidden, then, fresh=False):
        """``hidden += W_o attn`` (``fresh``: ``hidden = W_o attn``); folds the norm that follows (``then``)
        into the product if it can."""
        ops = self.rt.ops
        n = hidden.shape[0]
        if fresh:
            ops.linear(attn, self.w_o, hidden)
        elif then is not None and hasattr(ops, "linear_fuses_norm") and ops.linear_fuses_norm(n, self.w_o):
            then.prepare(self.rt, ops.norm_parts(n, self.hidden))
            ops.linear(attn, self.w_o, hidden, residual=hidden, norm_out=then)
            then.ready = True
        else:
            ops.linear(attn, self.w_o, hidden, residual=hidden)

    def forward(self, ctx, cache, x, hidden, then=None, fresh=False):
        rt = self.rt
        n = hidden.shape[0]
        qkv = rt.buffer("qkv", n, self.qkv_cols, rt.dtype)
        if isinstance(x, DeferredNorm):
            if x.ready and rt.ops.linear_fuses_norm(n, self.w_qkv):
                rt.ops.linear(x.xn, self.w_qkv, qkv, norm_in=x)          # the norm's factor in the epilogue
            else:
                rt.ops.linear(x.materialize(), self.w_qkv, qkv)
        else:
            rt.ops.linear(x, self.w_qkv, qkv)
        if self.general:
            self._forward_general(ctx, cache, qkv, hidden, then, fresh)
            return
        table, rotary_dim, pairing = None, 0, None
        if self.pos is not None:
            table = self.pos.rotary_table()
            if table is not None:
                rotary_dim, pairing = table.shape[1] * 2, self.pos.pairing
                if pairing not in ("half_split", "adjacent"):
                    raise ValueError(f"attention kernels rotate half-split or adjacent pairs, not '{pairing}'")
        attn = rt.buffer("attn_out", n, self.n_q * self.d, rt.dtype)
        # A decode step whose new key goes to this layer's own cache: the attention kernel may norm
        # and rotate q and the new k and write the cache itself.  (A layer that reads another
        # layer's cache takes every key from there, the newest too, so it is not fused.)
        fusable = cache.writes and (self.pos is None or (table is not None and rotary_dim == self.d))
        if fusable and hasattr(rt.ops, "can_fuse_decode") and \
                rt.ops.can_fuse_decode(ctx, qkv, self.n_q, self.n_kv, self.d):
            rt.ops.attention(ctx, qkv, attn, self.n_q, self.n_kv, self.d, self.scale, self.window, cache,
                             fuse=dict(q_w=self.q_norm_f32, k_w=self.k_norm_f32, eps=self.eps, rope=table,
                                       write_cache=True, pairing=pairing or "half_split"))
            self._out_proj(attn, hidden, then, fresh)
            return
        # q/k norm, rotation and the cache write are one kernel; an encoding without a
        # rotary table is applied by the encoding itself between norm and cache write.
        if self.pos is not None and table is None:
            rt.ops.qk_norm_rope_write(ctx, qkv, self.n_q, self.n_kv, self.d, self.q_norm_w,
                                      self.k_norm_w, self.eps, None, 0, None)
            q = qkv[:, :self.n_q * self.d].unflatten(1, (self.n_q, self.d))
            k = qkv[:, self.n_q * self.d:(self.n_q + self.n_kv) * self.d].unflatten(1, (self.n_kv, self.d))
            self.pos.apply(ctx, q, k)
            rt.ops.qk_norm_rope_write(ctx, qkv, self.n_q, self.n_kv, self.d, None, None,
                                      self.eps, None, 0, cache if cache.writes else None)
        else:
            extra = {} if pairing in (None, "half_split") else dict(pairing=pairing)
            rt.ops.qk_norm_rope_write(ctx, qkv, self.n_q, self.n_kv, self.d, self.q_norm_w,
                                      self.k_norm_w, self.eps, table, rotary_dim,
                                      cache if cache.writes else None, **extra)
        rt.ops.attention(ctx, qkv, attn, self.n_q, self.n_kv, self.d, self.scale,
                         self.window, cache)
        self._out_proj(attn, hidden, then, fresh)

    def _forward_general(self, ctx, cache, qkv, hidden, then, fresh=False):
        """Masks, weight rules, norms and widths beyond the reference's layer: one kernel norms and
        rotates q and k in fp32 and writes the new keys and values into their pages, one does the
        attention over the pages.  A layer that is causal softmax attention with equal key and
        value widths goes on to the framework's tuned attention kernels from there."""
        rt, ops = self.rt, self.rt.ops
        n = hidden.shape[0]
        freqs, pairing = (None, "half_split") if self.pos is None else (self.pos.frequencies(), self.pos.pairing)
        if self.pos is not None and getattr(self.pos, "magnitude", 1.0) != 1.0:
            raise ValueError("attention: a scaled rotation is not among this kernel's forms")
        ops.attention_prepare(ctx, qkv, self.n_q, self.n_kv, self.d, self.dv,
                              "whole" if self.norm_whole else ("per_head" if self.qk_norm else None),
                              self.q_norm_f32 if self.qk_norm else None, self.k_norm_f32 if self.qk_norm else None,
                              self.eps, freqs, pairing, cache if cache.writes else None)
        attn = rt.buffer("attn_out", n, self.n_q * self.dv, rt.dtype)
        size = self.window if self.mask == "window" else (self.chunk if self.mask == "chunk" else 0)
        if self.mixed:
            ops.attention_mixed_heads(ctx, qkv, attn, cache, self.n_q, self.n_kv, self.d, self.dv, self.scale, self.temp,
                                      self.score_cap, self.mix, self.sink, self.mask, int(size or 0))
        elif self.weights == "softmax" and self.mask != "chunk" and self.dv == self.d:
            ops.attention(ctx, qkv, attn, self.n_q, self.n_kv, self.d, self.scale, self.window, cache)
        else:
            ops.attention_masked(ctx, qkv, attn, self.n_q, self.n_kv, self.d, self.dv, self.scale, self.mask,
                                 int(size or 0), self.weights, self.bias, cache)
        self._out_proj(attn, hidden, then, fresh)
