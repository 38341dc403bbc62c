"""Mixture of experts: each token runs through its ``top`` best-scoring small gated layers.

Router logits ``z = W_router x`` and scores in fp32: ``score = "sigmoid"`` (each expert's own
``sigmoid(z_e)``) or ``"softmax"``; the ``top`` largest are chosen (the lowest index among equal
scores) and weigh their experts, as they are or divided by their sum (``renormalize``).  The weight
multiplies the expert's input (``scale = "input"``: ``sum expert_e(w_e x)``) or its output
(``"output"``).  An expert is ``W_down (silu(W_gate a) * (W_up a))`` without biases.  An optional
shared expert of the same form (size ``shared_size``) runs on every token and is added.

``score = "softmax_chosen"``: the logits themselves are ranked and the chosen experts' weights are
the softmax over the chosen logits only.  ``router_bias_name``: a bias ``[experts]`` added to the
router logits (fp32).  ``shared_gate_name``: a matrix ``[1, hidden]``; the shared expert's output is
multiplied by ``sigmoid(w_sg . x)``, one number per token (its logit rides in the router's fp32
product).  ``out_scale`` multiplies everything the part adds to the residual stream.

Further parameters, each off by default: ``expert_form = "relu_squared"`` makes an expert the
ungated ``W_down max(W_up a, 0)^2`` (tensors ``up`` and ``down`` only); ``groups`` and
``groups_kept`` restrict the choice to the experts of the best groups (the experts form ``groups``
equal runs of neighbours, a run is worth its largest score, the ``groups_kept`` best runs stay, the
lowest index among equal ones); ``weight_scale`` multiplies the chosen weights (after an optional
renormalisation).

``correction_name``: a tensor ``[experts]`` added to the scores for the choice (and for a group's worth)
only; the weights stay the scores without it.  ``identity``: the router has that many outputs past the
experts whose "expert" has no tensors and gives back its input (times the weight); they take part in
the scores, the groups and the choice like any other.

Experts' matrices are stacked at load time (``[experts, ff, hidden]`` twice and ``[experts, hidden,
ff]``); the pairs (token, choice) are grouped by expert on the device and the grouped products run
over them, so nothing is read back by the host and a captured decode step can replay it.
"""
from __future__ import annotations

import torch

from ..registry import FEED_FORWARDS
from .base import FeedForward, WeightSpec


@FEED_FORWARDS.register("routed_experts")
class RoutedExperts(FeedForward):
    writes_fresh = True           # forward(..., fresh=True) stores its result instead of adding it

    def __init__(self, params, rt):
        super().__init__(params, rt)
        self.hidden = int(params["hidden_size"])
        self.ff = int(params["expert_size"])
        self.experts = int(params["num_experts"])
        self.top = int(params["top"])
        self.score = params.get("score", "sigmoid")
        self.renormalize = bool(params.get("renormalize", False))
        self.scale = params.get("scale", "input")
        shared = params.get("shared_size")
        self.shared_ff = int(shared) if shared else None
        self.form = params.get("expert_form", "gated_silu")
        self.groups = int(params.get("groups", 1))
        self.groups_kept = int(params.get("groups_kept", self.groups))
        self.weight_scale = float(params.get("weight_scale", 1.0))
        self.out_scale = float(params.get("out_scale", 1.0))
        self.router_bias_name = params.get("router_bias_name")
        self.shared_gate_name = params.get("shared_gate_name") if self.shared_ff else None
        self.router_bias = None
        self.correction_name = params.get("correction_name")
        self.correction = None
        self.identity = int(params.get("identity", 0))
        self.outputs = self.experts + self.identity          # what the router chooses among
        if self.identity and (self.scale == "input" or shared):
            raise ValueError("routed experts: identity experts are weighted at their output and go without a shared expert")
        if self.score not in ("sigmoid", "softmax", "softmax_chosen") or self.scale not in ("input", "output"):
            raise ValueError(f"routed experts: score '{self.score}' / scale '{self.scale}'")
        if self.form not in ("gated_silu", "relu_squared"):
            raise ValueError(f"routed experts: expert form '{self.form}'")
        if self.groups < 1 or self.outputs % self.groups or not 0 < self.groups_kept <= self.groups or \
                self.top > self.outputs // self.groups * self.groups_kept:
            raise ValueError(f"routed experts: {self.experts} experts in {self.groups} groups, {self.groups_kept} kept, "
                             f"{self.top} chosen")
        if self.form == "relu_squared" and self.scale == "input":
            raise ValueError("routed experts: ungated experts are weighted at their output")
        if not 0 < self.top <= self.outputs:
            raise ValueError(f"routed experts: top {self.top} of {self.experts}")
        self.router_name = params.get("router_name", "router")
        self.expert_pattern = params.get("expert_pattern", "e{}.{}")      # (index, gate|up|down)
        self.shared_pattern = params.get("shared_pattern", "shared.{}")
        self.w_router = self.w_gate = self.w_up = self.w_down = self.w_shared_gate_up = self.w_shared_down = None

    def _expert(self, e, which):
        return self.expert_pattern.format(e, which)

    @property
    def gated(self):
        return self.form == "gated_silu"

    def weight_specs(self):
        specs = []
        for e in range(self.experts):
            if self.gated:
                specs.append(WeightSpec(self._expert(e, "gate"), (self.ff, self.hidden)))
            specs += [WeightSpec(self._expert(e, "up"), (self.ff, self.hidden)),
                      WeightSpec(self._expert(e, "down"), (self.hidden, self.ff))]
        specs.append(WeightSpec(self.router_name, (self.outputs, self.hidden)))
        if self.router_bias_name:
            specs.append(WeightSpec(self.router_bias_name, (self.outputs,), role="vector", std=0.5))
        if self.correction_name:
            specs.append(WeightSpec(self.correction_name, (self.outputs,), role="vector", std=0.05))
        if self.shared_gate_name:
            specs.append(WeightSpec(self.shared_gate_name, (1, self.hidden)))
        if self.shared_ff:
            specs += [WeightSpec(self.shared_pattern.format("gate"), (self.shared_ff, self.hidden)),
                      WeightSpec(self.shared_pattern.format("up"), (self.shared_ff, self.hidden)),
                      WeightSpec(self.shared_pattern.format("down"), (self.hidden, self.shared_ff))]
        return specs

    def load(self, tensors):
        def stack(which):
            return torch.stack([tensors[self._expert(e, which)] for e in range(self.experts)]).contiguous()
        self.w_gate, self.w_up, self.w_down = stack("gate") if self.gated else None, stack("up"), stack("down")
        router = tensors[self.router_name]
        if self.shared_gate_name:           # the gate's logit is one more row of the router's product
            router = torch.cat([router, tensors[self.shared_gate_name].to(router.dtype)], dim=0)
        self.w_router = self.rt.ops.prepare_matrix(router.contiguous())
        if self.router_bias_name:
            self.router_bias = tensors[self.router_bias_name].float().contiguous()
        if self.correction_name:
            self.correction = tensors[self.correction_name].float().contiguous()
        if self.shared_ff:
            ops = self.rt.ops
            self.w_shared_gate_up = ops.prepare_gate_up(tensors[self.shared_pattern.format("gate")],
                                                        tensors[self.shared_pattern.format("up")])
            self.w_shared_down = ops.prepare_matrix(tensors[self.shared_pattern.format("down")])

    def weight_bytes(self):
        # a decode step reads the router, the shared expert and `top` experts per token (at most all)
        per_expert = (3 if self.gated else 2) * self.ff * self.hidden
        return (self.outputs * self.hidden + 3 * (self.shared_ff or 0) * self.hidden
                + self.top * per_expert) * self.rt.dtype.itemsize

    def scratch_bytes(self, max_tokens):
        pairs = max_tokens * self.top
        item = self.rt.dtype.itemsize
        return pairs * (8 + self.ff * item + self.hidden * 4) + 4 * (self.experts + 1 + pairs) \
            + max_tokens * 3 * (self.shared_ff or 0) * item

    def load_transient_bytes(self):
        return (3 if self.gated else 2) * self.experts * self.ff * self.hidden * self.rt.dtype.itemsize

    def forward(self, ctx, x, hidden, fresh=False):
        rt, ops = self.rt, self.rt.ops
        n = hidden.shape[0]
        pairs = n * self.top
        chosen = rt.flat_buffer("experts_chosen", pairs, torch.int32, reserve=rt.max_tokens * self.top)[:pairs]
        weight = rt.flat_buffer("experts_weight", pairs, torch.float32, reserve=rt.max_tokens * self.top)[:pairs]
        extra = {}
        scale = self.weight_scale * self.out_scale
        if self.groups > 1 or scale != 1.0:
            extra = dict(groups=self.groups, groups_kept=self.groups_kept, weight_scale=scale)
        if self.router_bias is not None or self.shared_gate_name:
            extra.update(bias=self.router_bias, experts=self.outputs)
        if self.correction is not None:
            extra.update(correction=self.correction)
        softmax = "chosen" if self.score == "softmax_chosen" else self.score == "softmax"
        logits = ops.experts_route(x, self.w_router, chosen, weight, self.top, softmax, self.renormalize, **extra)
        more = {}
        if self.identity or fresh:
            more = dict(identity=self.identity, fresh=fresh)
        ops.experts_forward(x, self.w_gate, self.w_up, self.w_down, chosen, weight, self.top,
                            self.scale == "input", hidden, rt, **more)
        if self.shared_ff:
            act = rt.buffer("experts_shared_act", n, self.shared_ff, rt.dtype)
            ops.linear_swiglu(x, self.w_shared_gate_up, act)
            if self.shared_gate_name or self.out_scale != 1.0:
                gate = logits[:, self.experts:self.experts + 1] if self.shared_gate_name else None
                ops.scale_rows(act, gate, self.out_scale)
            ops.linear(act, self.w_shared_down, hidden, residual=hidden)
