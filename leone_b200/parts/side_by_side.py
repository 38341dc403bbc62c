"""Several mixers side by side on the same input.

``hidden += sum_b mixer_b(x)``: every branch is a mixer of a registered kind with its own parameters
(tensor names, sizes, an output scale if it has one), reads the same normed rows and adds its own
output to the residual stream; each owns the cache it asks for.  ``branches`` is a list of ``{"name",
"kind", "params"}``; the caches arrive under the branches' names.
"""
from __future__ import annotations

import inspect

from ..registry import MIXERS
from .base import CacheBundle, Mixer


@MIXERS.register("side_by_side")
class SideBySide(Mixer):
    def __init__(self, params, rt, position_encodings=None):
        super().__init__(params, rt)
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
        return [s for _, part in self.branches for s in part.weight_specs()]

    def load(self, tensors):
        for _, part in self.branches:
            part.load({s.name: tensors[s.name] for s in part.weight_specs()})

    def weight_bytes(self):
        return sum(part.weight_bytes() for _, part in self.branches if hasattr(part, "weight_bytes"))

    def scratch_bytes(self, max_tokens):
        return sum(part.scratch_bytes(max_tokens) for _, part in self.branches)

    def load_transient_bytes(self):
        return max(part.load_transient_bytes() for _, part in self.branches)

    def cache_request(self):
        return CacheBundle({name: part.cache_request() for name, part in self.branches})

    def forward(self, ctx, cache, x, hidden):
        for name, part in self.branches:
            part.forward(ctx, cache[name], x, hidden)
