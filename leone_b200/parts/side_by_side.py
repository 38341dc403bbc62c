"""Several mixers side by side on the same input.

``hidden += sum_b mixer_b(x)``: every branch is a mixer of a registered kind with its own parameters
(tensor names, sizes, an output scale if it has one), reads the same normed rows and adds its own
output to the residual stream; each owns the cache it asks for.  ``branches`` is a list of ``{"name",
"kind", "params"}``; the caches arrive under the branches' names.

``combine = "normed_mean"``: ``hidden += (1 / branches) sum_b rms_norm(mixer_b(x)) * w_b`` instead: every
branch's output is RMS-normed over the model width (``norm_eps``) with a weight of its own (the branch's
``norm_name``) before the mean is taken.
"""
from __future__ import annotations

import inspect

import torch

from ..registry import MIXERS
from .base import CacheBundle, Mixer, WeightSpec


@MIXERS.register("side_by_side")
class SideBySide(Mixer):
    writes_fresh = True           # forward(..., fresh=True) stores its result instead of adding it

    def adds_normed(self, norm) -> bool:
        """True if ``forward(..., normed_by=norm)`` can fold the arrangement's norm on this mixer's output into
        its own combining kernel."""
        return (self.combine == "normed_mean" and len(self.branches) == 2 and getattr(norm, "eps", None) == self.eps
                and getattr(norm, "weight", None) is not None and norm.weight.dtype == self.norm_weights[0].dtype
                and self.hidden <= 12000)

    def __init__(self, params, rt, position_encodings=None):
        super().__init__(params, rt)
        self.combine = params.get("combine", "sum")
        if self.combine not in ("sum", "normed_mean"):
            raise ValueError(f"side_by_side: combine '{self.combine}'")
        self.norm_names = [b.get("norm_name") for b in params["branches"]]
        self.norm_weights = []
        if self.combine == "normed_mean":
            self.hidden = int(params["hidden_size"])
            self.eps = float(params["norm_eps"])
            if not all(self.norm_names):
                raise ValueError("side_by_side: the normed mean needs a norm_name for every branch")
        self.branches = []
        for b in params["branches"]:
            cls = MIXERS.get(b["kind"])
            if "position_encodings" in inspect.signature(cls.__init__).parameters:
                part = cls(dict(b["params"]), rt, position_encodings=position_encodings)
            else:
                part = cls(dict(b["params"]), rt)
            self.branches.append((b["name"], part))
        if len({name for name, _ in self.branches}) != len(self.branches) or not self.branches:
            raise ValueError("side_by_side: branches need distinct names")

    def weight_specs(self):
        specs = [s for _, part in self.branches for s in part.weight_specs()]
        if self.combine == "normed_mean":
            specs += [WeightSpec(name, (self.hidden,), role="norm", std=0.1) for name in self.norm_names]
        return specs

    def load(self, tensors):
        for _, part in self.branches:
            part.load({s.name: tensors[s.name] for s in part.weight_specs()})
        if self.combine == "normed_mean":
            self.norm_weights = [tensors[name] for name in self.norm_names]

    def weight_bytes(self):
        return sum(part.weight_bytes() for _, part in self.branches if hasattr(part, "weight_bytes"))

    def scratch_bytes(self, max_tokens):
        return sum(part.scratch_bytes(max_tokens) for _, part in self.branches)

    def load_transient_bytes(self):
        return max(part.load_transient_bytes() for _, part in self.branches)

    def cache_request(self):
        return CacheBundle({name: part.cache_request() for name, part in self.branches})

    def forward(self, ctx, cache, x, hidden, fresh=False, normed_by=None, rounded=None):
        """``normed_by``: a norm part whose ``weight`` and ``eps`` norm this mixer's whole result before it is
        added to ``hidden`` (the arrangement's norm on the mixer's output, folded into the combining kernel:
        only offered to a mixer that declares ``adds_normed``, and only taken with two branches of the normed
        mean and the same eps); ``rounded``: also the new ``hidden`` in the run dtype."""
        if self.combine == "sum":
            if fresh:
                self.rt.ops.zero(hidden)
            for name, part in self.branches:
                part.forward(ctx, cache[name], x, hidden)
            return
        rt, ops = self.rt, self.rt.ops
        outs = []
        for i, (name, part) in enumerate(self.branches):
            out = rt.buffer(f"side_by_side_{i}", hidden.shape[0], hidden.shape[1], torch.float32)
            if getattr(part, "writes_fresh", False):
                part.forward(ctx, cache[name], x, out, fresh=True)
            else:
                ops.zero(out)
                part.forward(ctx, cache[name], x, out)
            outs.append(out)
        coef, w = 1.0 / len(outs), self.norm_weights
        if normed_by is not None:
            # hidden += norm(mean of the normed branches): the two norms after one another in one kernel
            ops.rms_norm_add(hidden, outs[0], w[0], self.eps, b=outs[1], w_b=w[1], coef=coef, accumulate=True,
                             rounded=rounded, then=normed_by.weight)
            return
        # the normed outputs two at a time: one pass over the rows for a pair of branches
        for i in range(0, len(outs), 2):
            pair = i + 1 < len(outs)
            ops.rms_norm_add(hidden, outs[i], w[i], self.eps, b=outs[i + 1] if pair else None,
                             w_b=w[i + 1] if pair else None, coef=coef, accumulate=not (fresh and i == 0))
