"""Mixture-of-experts feed-forwards: ``grouped_moe`` (below) and ``glu_moe`` (experts that are
clamped gated units, sigmoid or softmax scores, the weight on the expert's input or output, an
optional shared expert; at the end of this file).

``grouped_moe``:

Scores s = softmax(W_router h) over all experts, in 32-bit (the router matrix stays float32 in
every mode).  The experts form ``num_groups`` equal runs of neighbours; a group's score is its
largest score, and only experts of the ``keep_groups`` best groups can be chosen; of those the
``top`` largest scores are the token's experts, with their scores as weights (not renormalised).
Expert e: W_down_e act(W_up_e h), act the square of relu, no biases.  The output is the weighted
sum.  Everything runs on the device (``ops.moe``): no count ever visits the host."""
from __future__ import annotations

import torch

from dispec_b200.ops import moe as moe_ops
from dispec_b200.parts.base import FeedForward, TensorSpec
from dispec_b200.registry import register_part


@register_part("feed_forward", "grouped_moe")
class GroupedMoE(FeedForward):
    def __init__(self, hidden_size: int, intermediate_size: int, num_experts: int, top: int,
                 num_groups: int = 1, keep_groups: int = 1):
        if num_experts <= 0 or num_groups <= 0 or num_experts % num_groups:
            raise ValueError(f"grouped_moe: {num_experts} experts do not form {num_groups} equal groups")
        if not 0 < keep_groups <= num_groups:
            raise ValueError(f"grouped_moe: keep_groups={keep_groups} outside 1..{num_groups}")
        if not 0 < top <= keep_groups * (num_experts // num_groups):
            raise ValueError(f"grouped_moe: top={top} experts cannot come from {keep_groups} groups of "
                             f"{num_experts // num_groups}")
        self.hidden_size, self.intermediate_size = hidden_size, intermediate_size
        self.num_experts, self.top, self.num_groups, self.keep_groups = num_experts, top, num_groups, keep_groups

    def tensor_specs(self):
        h, i = self.hidden_size, self.intermediate_size
        specs = {"router.weight": TensorSpec((self.num_experts, h), dtype="float32")}
        for e in range(self.num_experts):
            specs[f"experts.{e}.up.weight"] = TensorSpec((i, h))
            specs[f"experts.{e}.down.weight"] = TensorSpec((h, i))
        return specs

    def load(self, tensors):
        E = self.num_experts
        self.w_router = tensors["router.weight"]
        self.w_up = torch.stack([tensors[f"experts.{e}.up.weight"] for e in range(E)]).contiguous()
        self.w_down = torch.stack([tensors[f"experts.{e}.down.weight"] for e in range(E)]).contiguous()

    def forward(self, ctx, x):
        ids, wts = moe_ops.route(x, self.w_router, self.num_groups, self.keep_groups, self.top)
        plan = moe_ops.plan(ids, self.num_experts, moe_ops.tensor_cores_supported(x.dtype, self.hidden_size,
                                                                                   self.intermediate_size))
        a = moe_ops.expert_product(plan, x, self.w_up, x.dtype, rows_are_tokens=True, scatter=False, square_relu=True)
        y = moe_ops.expert_product(plan, a, self.w_down, torch.float32, rows_are_tokens=False, scatter=True)
        return moe_ops.combine(y, wts, ids)


@register_part("feed_forward", "glu_moe")
class GatedMoE(FeedForward):
    """Mixture of experts whose experts are clamped gated units without biases:

        expert_e(a) = W_down_e y,  y = g * sigmoid(alpha * g) * (u + 1),
        g = min(W_gate_e a, limit),  u = clamp(W_up_e a, -limit, limit).

    Router logits z = W_router h in 32-bit (the router matrix stays float32 in every mode);
    scores s = sigmoid(z) (``score`` "sigmoid") or softmax(z); groups of experts as in
    ``grouped_moe``; the ``top`` largest scores name the token's experts and are their weights w,
    not renormalised.  ``weight_on`` "input": the output is the sum of expert_e(w h) (the factor is
    applied to the 32-bit sums W_gate_e h and W_up_e h, which is the same product, before the
    clamps); "output": the sum of w expert_e(h).  ``shared``: a feed-forward part that runs for
    every token and is added.  Everything runs on the device (``ops.moe``).

    Further switches: ``limit`` None: no clamps; ``up_shift``: the unit is g * sigmoid(alpha * g) *
    (u + up_shift) (no limit, alpha 1 and up_shift 0: silu(W_gate a) * (W_up a)).  ``group_score``
    "top2_sum": a group's score is the sum of its two largest scores (default: its largest).
    ``normalize``: the weights are the chosen scores divided by their sum (+ 1e-20), times
    ``weight_scale``.  ``shared_gate``: the shared part's result is multiplied by sigmoid(w_sg . h),
    one number per token (tensor ``shared_gate.weight`` [1, hidden_size], float32: its row rides in
    the router's product)."""

    def __init__(self, hidden_size: int, intermediate_size: int, num_experts: int, top: int, limit: float | None,
                 alpha: float = 1.702, score: str = "sigmoid", weight_on: str = "input", num_groups: int = 1,
                 keep_groups: int = 1, shared=None, up_shift: float = 1.0, group_score: str = "max",
                 normalize: bool = False, weight_scale: float = 1.0, shared_gate: bool = False):
        if num_experts <= 0 or num_groups <= 0 or num_experts % num_groups:
            raise ValueError(f"glu_moe: {num_experts} experts do not form {num_groups} equal groups")
        if not 0 < keep_groups <= num_groups:
            raise ValueError(f"glu_moe: keep_groups={keep_groups} outside 1..{num_groups}")
        if not 0 < top <= keep_groups * (num_experts // num_groups):
            raise ValueError(f"glu_moe: top={top} experts cannot come from {keep_groups} groups of "
                             f"{num_experts // num_groups}")
        if score not in ("sigmoid", "softmax") or weight_on not in ("input", "output"):
            raise ValueError(f"glu_moe: score={score!r} / weight_on={weight_on!r} are not known")
        limit = float("inf") if limit is None else limit
        if not limit > 0:
            raise ValueError(f"glu_moe: the limit must be positive, got {limit}")
        if group_score not in ("max", "top2_sum"):
            raise ValueError(f"glu_moe: group_score={group_score!r} is not known")
        if shared_gate and shared is None:
            raise ValueError("glu_moe: a gate on the shared part but no shared part")
        self.up_shift, self.group_score = float(up_shift), group_score
        self.normalize, self.weight_scale, self.shared_gate = bool(normalize), float(weight_scale), bool(shared_gate)
        self.hidden_size, self.intermediate_size = hidden_size, intermediate_size
        self.num_experts, self.top, self.num_groups, self.keep_groups = num_experts, top, num_groups, keep_groups
        self.limit, self.alpha, self.score, self.weight_on = float(limit), float(alpha), score, weight_on
        self.shared = shared

    def tensor_specs(self):
        h, i = self.hidden_size, self.intermediate_size
        specs = {"router.weight": TensorSpec((self.num_experts, h), dtype="float32")}
        for e in range(self.num_experts):
            specs[f"experts.{e}.gate.weight"] = TensorSpec((i, h))
            specs[f"experts.{e}.up.weight"] = TensorSpec((i, h))
            specs[f"experts.{e}.down.weight"] = TensorSpec((h, i))
        if self.shared_gate:
            specs["shared_gate.weight"] = TensorSpec((1, h), dtype="float32")
        return specs

    def load(self, tensors):
        E, h, i = self.num_experts, self.hidden_size, self.intermediate_size
        self.w_router = tensors["router.weight"]
        if self.shared_gate:
            self.w_router = torch.cat([self.w_router, tensors["shared_gate.weight"]], dim=0).contiguous()
        # rows of the gate and up matrices in turn: the product's epilogue holds a gate and its up
        # value in one thread and writes the unit's result
        self.w_gate_up = torch.stack(
            [torch.stack([tensors[f"experts.{e}.gate.weight"], tensors[f"experts.{e}.up.weight"]], dim=1).reshape(2 * i, h)
             for e in range(E)]).contiguous()
        self.w_down = torch.stack([tensors[f"experts.{e}.down.weight"] for e in range(E)]).contiguous()

    def forward(self, ctx, x):
        routed = moe_ops.route(x, self.w_router, self.num_groups, self.keep_groups, self.top, score=self.score,
                               group_score=self.group_score, normalize=self.normalize, weight_scale=self.weight_scale,
                               extra_rows=1 if self.shared_gate else 0)
        ids, wts = routed[0], routed[1]
        plan = moe_ops.plan(ids, self.num_experts, moe_ops.tensor_cores_supported(x.dtype, self.hidden_size,
                                                                                   self.intermediate_size))
        on_input = self.weight_on == "input"
        a = moe_ops.expert_product(plan, x, self.w_gate_up, x.dtype, rows_are_tokens=True, scatter=False,
                                   clamped_glu=(self.limit, self.alpha), row_scale=wts.view(-1) if on_input else None,
                                   up_shift=self.up_shift)
        y = moe_ops.expert_product(plan, a, self.w_down, torch.float32, rows_are_tokens=False, scatter=True)
        base = self.shared.forward(ctx, x) if self.shared is not None else None
        return moe_ops.combine(y, None if on_input else wts, ids, base=base,
                               base_scale=routed[2] if self.shared_gate else None)
