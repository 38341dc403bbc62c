"""Token embedding: ``h[t, :] = scale * E[id_t, :]`` into the fp32 residual stream.

The reference gathers the row without a factor and treats an id outside the table as an error
(crates/leone/src/runtime.rs:7380-7386, 6686-6692; crates/leone/src/cpu.rs:1243-1265); ``scale``
(default 1) is this part's own parameter for models that multiply their embeddings.  ``norm``
(a mapping with ``name``, ``eps`` and optionally ``weight_offset``; default none) adds an RMS norm
of the gathered rows, in fp32, with a weight of the part's own: ``h = rms_norm(scale * E[id])``.
``side_tables`` (a list of ``{"name", "width"}``; default none): further tables ``[vocab, width]`` whose
rows of the step's tokens are gathered too (fp32) and offered to the layers as ``ctx.token_rows[name]``.
"""
from __future__ import annotations

from ..registry import EMBEDDINGS
from .base import Embedding, WeightSpec


@EMBEDDINGS.register("token_embedding")
class TokenEmbedding(Embedding):
    def __init__(self, params, rt):
        super().__init__(params, rt)
        self.vocab = int(params["vocab_size"])
        self.hidden = int(params["hidden_size"])
        self.name = params["name"]
        self.scale = float(params.get("scale", 1.0))
        self.weight = None
        norm = params.get("norm")
        self.norm_name = norm["name"] if norm else None
        self.norm_eps = float(norm["eps"]) if norm else 0.0
        self.norm_offset = float(norm.get("weight_offset", 0.0)) if norm else 0.0
        self.norm_weight = None
        self.side_tables = [(t["name"], int(t["width"])) for t in params.get("side_tables") or ()]
        self.side_weights = {}

    def weight_specs(self):
        specs = [WeightSpec(self.name, (self.vocab, self.hidden), role="embedding")]
        specs += [WeightSpec(name, (self.vocab, width), role="embedding") for name, width in self.side_tables]
        if self.norm_name:
            specs.append(WeightSpec(self.norm_name, (self.hidden,), role="vector" if self.norm_offset else "norm", std=0.1))
        return specs

    def load(self, tensors):
        self.weight = tensors[self.name]
        self.side_weights = {name: tensors[name] for name, _ in self.side_tables}
        if self.norm_name:
            self.norm_weight = (tensors[self.norm_name].float() + self.norm_offset).contiguous()

    def scratch_bytes(self, max_tokens):
        return max_tokens * 4 * ((self.hidden if self.norm_name else 0) + sum(w for _, w in self.side_tables))

    def table(self):
        return self.weight

    def forward(self, ctx, hidden):
        rows = hidden
        if self.norm_name:
            rows = self.rt.buffer("embedding_rows", hidden.shape[0], self.hidden, hidden.dtype)
        if self.scale == 1.0:
            self.rt.ops.embedding(self.weight, ctx.token_ids, rows, ctx.status)
        else:
            self.rt.ops.embedding(self.weight, ctx.token_ids, rows, ctx.status, self.scale)
        if self.norm_name:
            self.rt.ops.rms_norm(rows, self.norm_weight, hidden, self.norm_eps)
        for name, width in self.side_tables:
            side = self.rt.buffer(f"token_rows_{name}", hidden.shape[0], width, hidden.dtype)
            self.rt.ops.embedding(self.side_weights[name], ctx.token_ids, side, ctx.status)
            ctx.token_rows[name] = side
