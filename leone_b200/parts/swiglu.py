"""Dense SwiGLU feed-forward: ``hidden += W_down (silu(W_gate x) * W_up x)``.

``silu(g) = g / (1 + exp(-g))`` in fp32 (crates/leone/src/cpu.rs:903-905);
order of operations crates/leone/src/runtime.rs:9298-9317.  Gate and up
matrices are stacked row-wise at load time so one product feeds both
(the reference pairs them in one launch too, ie_cuda.cu:1896-1931).

The gate's shape is this part's own parameters, for gated layers of the same family:
``y = g' * sigmoid(gate_slope * g') * (u' + up_shift)`` with ``g' = min(g, limit)`` and
``u' = clamp(u, -limit, limit)``.  The defaults (``gate_slope = 1``, no ``limit``, ``up_shift = 0``)
are SwiGLU.
"""
from __future__ import annotations

from ..registry import FEED_FORWARDS
from .base import DeferredNorm, FeedForward, WeightSpec


@FEED_FORWARDS.register("swiglu")
class SwiGLU(FeedForward):
    accepts_deferred_norm = True
    fuses_following_norm = True
    writes_fresh = True           # forward(..., fresh=True) stores its result instead of adding it

    def __init__(self, params, rt):
        super().__init__(params, rt)
        self.hidden = int(params["hidden_size"])
        self.inter = int(params["intermediate_size"])
        self.gate_name = params.get("gate_name", "gate_proj.weight")
        self.up_name = params.get("up_name", "up_proj.weight")
        self.down_name = params.get("down_name", "down_proj.weight")
        self.w_gate_up = None
        self.w_down = None
        slope, limit, shift = float(params.get("gate_slope", 1.0)), params.get("limit"), float(params.get("up_shift", 0.0))
        if limit is not None and not float(limit) > 0.0:
            raise ValueError(f"a gated layer's limit must be positive, got {limit}")
        # None: plain SwiGLU (the kernels' default); else (slope, limit, shift) with limit = inf for none
        self.gate_shape = None if (slope == 1.0 and limit is None and shift == 0.0) else \
            (slope, float("inf") if limit is None else float(limit), shift)

    def weight_specs(self):
        return [WeightSpec(self.gate_name, (self.inter, self.hidden)),
                WeightSpec(self.up_name, (self.inter, self.hidden)),
                WeightSpec(self.down_name, (self.hidden, self.inter))]

    def load(self, tensors):
        self.w_gate_up = self.rt.ops.prepare_gate_up(tensors[self.gate_name], tensors[self.up_name])
        self.w_down = self.rt.ops.prepare_matrix(tensors[self.down_name])

    def weight_bytes(self):
        return (2 * self.inter * self.hidden + self.hidden * self.inter) * self.rt.dtype.itemsize

    def scratch_bytes(self, max_tokens):
        # the activation; a path without the fused epilogue also holds gate and up side by side
        return max_tokens * 3 * self.inter * self.rt.dtype.itemsize

    def load_transient_bytes(self):
        return 2 * self.inter * self.hidden * self.rt.dtype.itemsize       # gate and up beside their interleaved copy

    def forward(self, ctx, x, hidden, then=None, fresh=False):
        n = hidden.shape[0]
        ops = self.rt.ops
        act = self.rt.buffer("ffn_act", n, self.inter, self.rt.dtype)
        kw = {} if self.gate_shape is None else {"gate_shape": self.gate_shape}
        if isinstance(x, DeferredNorm):
            if x.ready and ops.linear_fuses_norm(n, self.w_gate_up):
                ops.linear_swiglu(x.xn, self.w_gate_up, act, norm_in=x, **kw)      # the norm's factor in the epilogue
            else:
                ops.linear_swiglu(x.materialize(), self.w_gate_up, act, **kw)
        else:
            ops.linear_swiglu(x, self.w_gate_up, act, **kw)
        if then is not None and hasattr(ops, "linear_fuses_norm") and ops.linear_fuses_norm(n, self.w_down):
            then.prepare(self.rt, ops.norm_parts(n, self.hidden))
            ops.linear(act, self.w_down, hidden, residual=hidden, norm_out=then)
            then.ready = True
        else:
            ops.linear(act, self.w_down, hidden, residual=None if fresh else hidden)
