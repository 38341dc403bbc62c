"""RMSNorm over the residual stream.

``y_c = x_c * w_c / sqrt(mean_c(x_c^2) + eps)`` with the sum of squares in
fp32; the weight multiplies directly, not as ``1 + w``
(crates/leone/src/cpu.rs:1642-1663; CUDA counterpart
crates/leone-cuda/cuda/ie_cuda.cu:2357-2380).  ``weight_offset`` (default 0) is this part's own
parameter for models that store the gain as its distance from a constant: the gain is
``weight_offset + w``, formed once at load time in fp32.
"""
from __future__ import annotations

from ..registry import NORMS
from .base import DeferredNorm, Norm, WeightSpec


@NORMS.register("rms_norm")
class RMSNorm(Norm):
    def __init__(self, params, rt):
        super().__init__(params, rt)
        self.size = int(params["size"])
        self.eps = float(params["eps"])
        self.name = params.get("name", "weight")
        self.offset = float(params.get("weight_offset", 0.0))
        self.weight = self.weight_f32 = None

    def weight_specs(self):
        # a gain stored around zero is drawn around zero
        return [WeightSpec(self.name, (self.size,), role="vector" if self.offset else "norm", std=0.1)]

    def load(self, tensors):
        self.weight = tensors[self.name]
        if self.offset:
            self.weight = (self.weight.float() + self.offset).contiguous()
        self.weight_f32 = self.weight.float().contiguous()    # for a product that applies the norm itself

    def defer(self, ctx, hidden, tag="a"):
        return DeferredNorm(self, ctx, hidden, self.weight_f32, self.eps, tag)

    def forward(self, ctx, hidden, rows=None, out_name="normed", dtype=None):
        """``dtype``: of the result (default: the run dtype; fp32 for a consumer that goes on in fp32)."""
        n = hidden.shape[0] if rows is None else rows.shape[0]
        out = self.rt.buffer(out_name, n, self.size, dtype or self.rt.dtype)
        self.rt.ops.rms_norm(hidden, self.weight, out, self.eps, rows)
        return out

    def add_normed(self, ctx, branch, hidden, rounded=None):
        """``hidden += rms_norm(branch) * weight``: this norm on a sublayer's output ``branch`` (fp32), added
        to the residual stream; ``rounded``: also the new stream in another dtype."""
        self.rt.ops.rms_norm_add(hidden, branch, self.weight, self.eps, rounded=rounded)

    def forward_pair(self, ctx, hidden, other: "RMSNorm"):
        """This norm and ``other`` (same size and eps) of the same rows in one pass."""
        n = hidden.shape[0]
        out_a = self.rt.buffer("normed", n, self.size, self.rt.dtype)
        out_b = self.rt.buffer("normed_b", n, self.size, self.rt.dtype)
        self.rt.ops.rms_norm_pair(hidden, self.weight, other.weight, out_a, out_b, self.eps)
        return out_a, out_b
