"""A feed-forward of many small gated experts of which every token uses a few, plus an optional shared expert.

    z       = W_r x                         router logits, float32
    s       = sigmoid(z)                    scores (``score="softmax"``: softmax of z over all experts)
    c       = s + correction                choice scores (the weights below use s)
    groups  : the experts form ``groups`` equal runs of neighbours; a group's score is the sum of its ``group_top``
              largest c; only experts of the ``keep_groups`` best groups can be chosen
    chosen  = the ``top`` allowed experts with the largest c
    w_e     = s_e / (sum of the chosen s + weight_eps) * route_scale
    expert  : g = min(W_gate x, limit); u = clamp(W_up x, -limit, limit); W_down (g * sigmoid(slope * g) * (u + 1))
              (``activation="silu"``: plain W_down (silu(W_gate x) * W_up x), no clamp)
    y       = sum_e w_e expert_e(x)  +  shared(x)

Everything runs on the device from the batch layout alone (no host read of the routing), so a decode step through it
can be replayed as a CUDA graph: the router's product (``ops.moe_router_logits``), one kernel that scores and chooses (``ops.moe_route``), a
counting sort of the (token, choice) pairs by expert (``ops.moe_sort``), two grouped products over the sorted rows
(``ops.moe_gate_up`` with the activation on its output, ``ops.moe_down`` with the token's weight), and a sum in a
fixed order (``ops.moe_combine``).  The experts' matrices are stacked [experts, rows, columns] at load.
"""

from __future__ import annotations

import torch

from ..kernels import ops
from .base import FeedForward, ParamSpec, register_feed_forward


@register_feed_forward("routed_experts")
class RoutedExperts(FeedForward):
    """params: ``experts``, ``top``, ``groups`` and ``keep_groups`` (default 1 / 1: no groups), ``group_top``
    (default 2; 1: a group is scored by its best expert), ``route_scale``, ``weight_eps``, ``score`` (``"sigmoid"`` or
    ``"softmax"``), ``correction`` (bool, default True: a learned per-expert offset of the choice scores),
    ``activation`` (``"clamped_swish"``, the default, with ``limit`` and ``swish_slope``; or ``"silu"``),
    ``intermediate_size`` of an expert, ``shared`` (None, or ``{"intermediate_size", "limit"}``), ``names`` (``expert`` with ``{}`` for
    the index, ``gate``, ``up``, ``down``, ``router``, ``correction``, ``shared``)."""

    graph_safe = True
    #: ``forward(..., defer_sum=True)`` hands back an ``ops.ExpertParts`` for a norm that adds the rows up itself
    defers_sum = True

    NAMES = {"expert": "experts.{}", "gate": "gate_proj.weight", "up": "up_proj.weight", "down": "down_proj.weight",
             "router": "router.weight", "correction": "router.correction", "shared": "shared_expert"}

    def __init__(self, spec, **kw):
        super().__init__(spec, **kw)
        p = spec.params
        self.experts, self.top = int(p["experts"]), int(p["top"])
        self.groups, self.keep_groups = int(p.get("groups") or 1), int(p.get("keep_groups") or 1)
        self.group_top = int(p.get("group_top", 2))
        if self.experts <= 0 or self.experts % self.groups or not 0 < self.keep_groups <= self.groups:
            raise ValueError(f"routed_experts: {self.experts} experts do not form {self.groups} equal groups of which "
                             f"{self.keep_groups} are kept")
        if not 0 < self.top <= self.keep_groups * (self.experts // self.groups):
            raise ValueError(f"routed_experts: top {self.top} is more than the kept groups hold")
        if self.experts > ops.MOE_MAX_EXPERTS or self.top > ops.MOE_MAX_TOP:
            raise ValueError(f"routed_experts: the kernels take up to {ops.MOE_MAX_EXPERTS} experts and a top of "
                             f"{ops.MOE_MAX_TOP}")
        self.score = str(p.get("score", "sigmoid"))
        if self.score not in ops.MOE_SCORES:
            raise ValueError(f"routed_experts: score must be one of {sorted(ops.MOE_SCORES)}, got {self.score!r}")
        self.activation = str(p.get("activation", "clamped_swish"))
        if self.activation not in ("clamped_swish", "silu"):
            raise ValueError(f"routed_experts: activation must be 'clamped_swish' or 'silu', got {self.activation!r}")
        self.route_scale = float(p.get("route_scale", 1.0))
        self.weight_eps = float(p.get("weight_eps", 1e-20))
        self.has_correction = bool(p.get("correction", True))
        self.intermediate_size = int(p["intermediate_size"])
        shared = p.get("shared")
        self.shared_size = int(shared["intermediate_size"]) if shared else 0
        if self.activation == "silu":
            # the clamped form with nothing to clamp, a slope of one and no offset on the up half is SiLU times up
            self.limit, self.swish_slope, self.up_offset, self.shared_limit = float("inf"), 1.0, 0.0, float("inf")
        else:
            self.limit, self.swish_slope, self.up_offset = float(p["limit"]), float(p.get("swish_slope", 1.702)), 1.0
            self.shared_limit = float(shared["limit"]) if shared else 0.0
        self.names = dict(self.NAMES, **(p.get("names") or {}))
        self.w_router = self.correction = self.w_gate_up = self.w_down = self.shared_gate_up = self.shared_down = None

    def _expert(self, index: int, which: str) -> str:
        return f"{self.names['expert'].format(index)}.{self.names[which]}"

    def param_specs(self):
        f, h, n = self.intermediate_size, self.hidden_size, self.names
        specs = {}
        for e in range(self.experts):
            specs[self._expert(e, "gate")] = ParamSpec((f, h))
            specs[self._expert(e, "up")] = ParamSpec((f, h))
            specs[self._expert(e, "down")] = ParamSpec((h, f))
        specs[n["router"]] = ParamSpec((self.experts, h))
        if self.has_correction:
            specs[n["correction"]] = ParamSpec((self.experts,), kind="vector", init="around_zero")
        if self.shared_size:
            specs[f"{n['shared']}.{n['gate']}"] = ParamSpec((self.shared_size, h))
            specs[f"{n['shared']}.{n['up']}"] = ParamSpec((self.shared_size, h))
            specs[f"{n['shared']}.{n['down']}"] = ParamSpec((h, self.shared_size))
        return specs

    def load(self, tensors):
        n = self.names
        # [experts, gate rows then up rows, hidden] and [experts, hidden, intermediate]
        self.w_gate_up = torch.stack([torch.cat((tensors[self._expert(e, "gate")], tensors[self._expert(e, "up")]), dim=0)
                                      for e in range(self.experts)]).contiguous()
        self.w_down = torch.stack([tensors[self._expert(e, "down")] for e in range(self.experts)]).contiguous()
        self.w_router = tensors[n["router"]].contiguous()
        self.correction = tensors[n["correction"]].float().contiguous() if self.has_correction else None
        if self.shared_size:
            self.shared_gate_up = torch.cat((tensors[f"{n['shared']}.{n['gate']}"], tensors[f"{n['shared']}.{n['up']}"]),
                                            dim=0).contiguous()
            self.shared_down = tensors[f"{n['shared']}.{n['down']}"].contiguous()

    def forward(self, x, ctx, defer_sum: bool = False):
        status = getattr(ctx, "status", None)
        logits = ops.moe_router_logits(x, self.w_router, status=status)
        chosen, weights = ops.moe_route(logits, self.correction, top=self.top, groups=self.groups,
                                        keep_groups=self.keep_groups, group_top=self.group_top,
                                        scale=self.route_scale, weight_eps=self.weight_eps, score=self.score)
        order, offsets = ops.moe_sort(chosen, self.experts)
        act = ops.moe_gate_up(x, self.w_gate_up, order, offsets, top=self.top, limit=self.limit,
                              slope=self.swish_slope, up_offset=self.up_offset)
        parts = ops.moe_down(act, self.w_down, order, offsets, weights)
        shared = None
        if self.shared_size:
            if self.activation == "silu":
                shared = ops.linear(ops.gated_linear(x, self.shared_gate_up, 0, status=status), self.shared_down,
                                    status=status)
            else:
                both = ops.linear(x, self.shared_gate_up, status=status)
                shared = ops.linear(ops.glu(both, "clamped_swish", 0, self.shared_limit, self.swish_slope),
                                    self.shared_down, status=status)
        result = ops.ExpertParts(parts, shared, self.top)
        return result if defer_sum else result.materialize()
