"""Mixture of experts as a feed-forward: every token runs ``top`` of ``num_experts`` small gated
feed-forward layers and adds their outputs, weighted.

Routing, ``routing="top_logits"``: logits ``W_router x + bias`` in 32-bit; the ``top`` largest choose (ties: the lower
index); the weights are the softmax over the chosen logits only.  ``routing="scores"``: s = softmax over all router
outputs; the choice runs on s + a stored ``correction`` within the ``groups_keep`` best of ``groups`` equal groups of
neighbouring outputs (a group's value is its largest s + correction); the weights are s * ``route_scale``, not
renormalised.  The last ``num_identity`` router outputs are identity experts: no tensors, their output is the token's
row itself (``num_experts`` counts the experts with weights).

An expert is ``W_down(a * sigmoid(alpha a) * (b + shift))`` with ``a = min(W_gate x, limit)`` and
``b = clamp(W_up x, -limit, limit)``; ``limit=None``, ``alpha=1``, ``shift=0`` give ``silu(W_gate x) * (W_up x)``.

A step's (token, expert) pairs are sorted by expert on the device (``csrc/moe.cu``).  In bfloat16
with rows of whole 16 bytes a step of up to 16 tokens runs the weight-streaming kernel for few pairs
an expert (gate and up with the activation in the epilogue, then down), and a larger step hands
the two products of the experts to the library's grouped product,
which reads the group sizes on the device, with a gather before, the experts' activation between
and the rows left in sorted order; float32 and other sizes run this package's own grouped kernels
(gate and up with the activation in the epilogue, then down).  Nothing comes back to the host, so
the work can sit in a captured graph.  Either way there is one row per pair at the end;
``forward(..., combine=False)`` hands those, the router's weights and where each row lies on
(``kernels.WeightedRows``) for a kernel that adds them on its way, otherwise they are added here.
"""

from __future__ import annotations

from typing import Mapping, Optional

import torch

from kairyu_b200 import kernels
from kairyu_b200.parts.base import FEED_FORWARDS, FeedForward, StepContext, TensorSpec


@FEED_FORWARDS.register("moe")
class MixtureOfExperts(FeedForward):
    graph_safe = True
    weighted_rows = True  # forward takes combine=False

    def __init__(
        self,
        *,
        prefix: str,
        hidden_size: int,
        intermediate_size: int,
        num_experts: int,
        top: int,
        limit: Optional[float],
        alpha: float = 1.702,
        shift: float = 1.0,
        router_bias: bool = True,
        routing: str = "top_logits",
        num_identity: int = 0,
        groups: int = 1,
        groups_keep: int = 1,
        route_scale: float = 1.0,
        dtype: torch.dtype,
        device: str,
        **_: object,
    ) -> None:
        outputs = num_experts + num_identity
        if not 1 <= top <= outputs:
            raise ValueError(f"a token cannot use {top} of {outputs} experts")
        if routing not in ("top_logits", "scores"):
            raise ValueError(f"unknown routing {routing!r} (top_logits, scores)")
        if routing == "top_logits" and (num_identity or groups != 1):
            raise ValueError("identity experts and groups come with routing by scores")
        if routing == "scores" and (groups < 1 or outputs % groups or not 1 <= groups_keep <= groups or top > groups_keep * (outputs // groups)):
            raise ValueError(f"{outputs} router outputs in {groups} groups of which {groups_keep} stay cannot give {top} experts a token")
        self.routing = routing
        self.num_identity = num_identity
        self.num_outputs = outputs
        self.groups = groups
        self.groups_keep = groups_keep
        self.route_scale = float(route_scale)
        self.shift = float(shift)
        # a kernel that adds the rows itself (kernels.WeightedRows) knows nothing of identity experts
        self.weighted_rows = num_identity == 0
        self.prefix = prefix
        self.hidden_size = hidden_size
        self.intermediate_size = intermediate_size
        self.num_experts = num_experts
        self.top = top
        self.limit = float("inf") if limit is None else float(limit)
        self.alpha = float(alpha)
        self.router_bias = router_bias and routing == "top_logits"
        self.dtype = dtype
        self.correction: Optional[torch.Tensor] = None
        self.w_router: Optional[torch.Tensor] = None
        self.b_router: Optional[torch.Tensor] = None
        self.w_gate_up: Optional[torch.Tensor] = None  # [experts, 2 * intermediate, hidden]: gate rows, then up rows
        self.w_down: Optional[torch.Tensor] = None     # [experts, hidden, intermediate]

    def tensor_specs(self) -> list[TensorSpec]:
        p, h, f = self.prefix, self.hidden_size, self.intermediate_size
        specs = []
        for e in range(self.num_experts):
            specs += [
                TensorSpec(f"{p}.e{e}.gate", (f, h)),
                TensorSpec(f"{p}.e{e}.up", (f, h)),
                TensorSpec(f"{p}.e{e}.down", (h, f)),
            ]
        specs.append(TensorSpec(f"{p}.router", (self.num_outputs, h)))
        if self.routing == "scores":
            specs.append(TensorSpec(f"{p}.correction", (self.num_outputs,), role="vector", init="normal"))
        if self.router_bias:
            specs.append(TensorSpec(f"{p}.router.b", (self.num_experts,), role="vector", init="normal"))
        return specs

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        p = self.prefix
        experts = range(self.num_experts)
        self.w_gate_up = torch.stack(
            [torch.cat([tensors[f"{p}.e{e}.gate"], tensors[f"{p}.e{e}.up"]], dim=0) for e in experts], dim=0
        ).contiguous()
        self.w_down = torch.stack([tensors[f"{p}.e{e}.down"] for e in experts], dim=0).contiguous()
        self.w_router = tensors[f"{p}.router"].contiguous()
        self.b_router = tensors[f"{p}.router.b"].contiguous() if self.router_bias else None
        self.correction = tensors[f"{p}.correction"].contiguous() if self.routing == "scores" else None

    def bytes_streamed(self) -> int:
        """What a single token reads: the router and ``top`` experts."""
        per_expert = (self.w_gate_up[0].numel() + self.w_down[0].numel()) * self.w_down.element_size()
        return self.w_router.numel() * self.w_router.element_size() + self.top * per_expert

    def forward(self, x: torch.Tensor, ctx: StepContext, combine: bool = True):
        tokens = x.shape[0]
        ws = ctx.workspace
        experts, top = self.num_outputs, self.top  # identity experts have runs in the plan too; the products skip them
        logits = ws.buffer("moe.logits", tokens, experts, torch.float32)
        kernels.linear(x, self.w_router, None, logits)
        ids = ws.buffer("moe.ids", tokens, top, torch.int32)
        weights = ws.buffer("moe.weights", tokens, top, torch.float32)
        if self.routing == "scores":
            kernels.moe_route_scores(logits, self.correction, top, ids, weights, groups=self.groups, keep=self.groups_keep, scale=self.route_scale)
        else:
            kernels.moe_route(logits, self.b_router, top, ids, weights)
        pairs = tokens * top
        plan = kernels.moe_plan(ids, experts, ws.flat("moe.plan", kernels.moe_plan_size(pairs, experts), torch.int32))
        unit = dict(limit=self.limit, alpha=self.alpha, shift=self.shift)
        if kernels.moe_skinny_ok(tokens, self.hidden_size, self.intermediate_size, self.dtype):
            # a decode-sized step: an expert has a handful of pairs and its weights stream once (gate and up with the
            # activation in the epilogue, then down)
            hidden = ws.buffer("moe.hidden", pairs, self.intermediate_size, self.dtype)
            kernels.moe_skinny(x, self.w_gate_up, hidden, plan, top=top, gated=True, **unit)
            rows, at = ws.buffer("moe.rows", pairs, self.hidden_size, torch.float32), None
            kernels.moe_skinny(hidden, self.w_down, rows, plan, top=top, gated=False)
        elif kernels.moe_library_products_ok(self.hidden_size, self.intermediate_size, self.dtype):
            # bfloat16, aligned sizes: the tokens' rows are laid out run by run and the library's grouped
            # product (group sizes read on the device) runs both products; the rows stay in that order
            ends = plan["ends"][: self.num_experts]  # where the runs of the experts with weights end
            gathered = ws.buffer("moe.gathered", pairs, self.hidden_size, self.dtype)
            kernels.gather_rows(x, plan["token_of"], gathered)
            gate_up = kernels.moe_library_product(gathered, self.w_gate_up, ends)
            hidden = ws.buffer("moe.hidden", pairs, self.intermediate_size, self.dtype)
            kernels.moe_activation(gate_up, hidden, **unit)
            rows, at = kernels.moe_library_product(hidden, self.w_down, ends), plan["place_of"]
        else:
            hidden = ws.buffer("moe.hidden", pairs, self.intermediate_size, self.dtype)
            kernels.moe_grouped(x, self.w_gate_up, hidden, plan, top=top, gated=True, **unit)
            rows, at = ws.buffer("moe.rows", pairs, self.hidden_size, torch.float32), None
            kernels.moe_grouped(hidden, self.w_down, rows, plan, top=top, gated=False)
        if not combine:
            if self.num_identity:
                raise ValueError("a mixture with identity experts adds its rows itself")
            return kernels.WeightedRows(rows, weights, at)
        out = ws.buffer("moe.out", tokens, self.hidden_size, self.dtype)
        if self.num_identity:
            kernels.moe_combine(rows, weights, out, at, ids=ids, x=x, experts=self.num_experts)
        else:
            kernels.moe_combine(rows, weights, out, at)
        return out
