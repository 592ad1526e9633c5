"""Mixture of experts as a feed-forward: every token runs ``top`` of ``num_experts`` small gated
feed-forward layers and adds their outputs, weighted.

Routing, ``routing="top_logits"``: logits ``W_router x + bias`` in 32-bit; the ``top`` largest choose (ties: the lower
index); the weights are the softmax over the chosen logits only.  ``routing="scores"``: s = softmax over all router
outputs; the choice runs on s + a stored ``correction`` within the ``groups_keep`` best of ``groups`` equal groups of
neighbouring outputs (a group's value is its largest s + correction); the weights are s * ``route_scale``, not
renormalised.  ``score_function="sigmoid"`` takes s = sigmoid(logit), each output by itself, in place of the softmax;
``correction=False`` means the file stores none.  The last ``num_identity`` router outputs are identity experts: no
tensors, their output is the token's row itself (``num_experts`` counts the experts with weights).

``weight_on="input"``: the router's weight multiplies the expert's input, ``sum_k expert_k(w_k x)``, instead of its output
(the experts are not linear, so the two differ); the pairs' rows are then scaled on their way to the first product and
added up unweighted.

``shared_expert`` (a dict: ``intermediate_size``, optional ``limit`` / ``alpha`` / ``shift``, ``gate``): one more expert of the same
form that every token runs (tensors ``<prefix>.shared.gate`` / ``.up`` / ``.down``); with ``gate`` its output is multiplied
by ``sigmoid(w_sg . x)``, one number a token (tensor ``<prefix>.shared.sg``, [1, hidden]), which is computed with the router's
logits, in 32-bit, as one more row of that product.

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
from kairyu_b200.parts.base import FEED_FORWARDS, FeedForward, PartSpec, StepContext, TensorSpec


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
        score_function: str = "softmax",
        correction: bool = True,
        weight_on: str = "output",
        shared_expert: Optional[Mapping[str, object]] = None,
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
        if score_function not in ("softmax", "sigmoid"):
            raise ValueError(f"unknown score function {score_function!r} (softmax, sigmoid)")
        if weight_on not in ("output", "input"):
            raise ValueError(f"a router's weight multiplies an expert's output or its input, not {weight_on!r}")
        if routing == "top_logits" and score_function != "softmax":
            raise ValueError("a score function other than the softmax comes with routing by scores")
        if routing == "top_logits" and shared_expert is not None and dict(shared_expert).get("gate"):
            raise ValueError("a gated shared expert comes with routing by scores")
        if weight_on == "input" and num_identity:
            raise ValueError("identity experts take the router's weight on their output")
        self.score_function = score_function
        self.has_correction = correction and routing == "scores"
        self.weight_on_input = weight_on == "input"
        self.shared = None
        self.shared_gate = False
        if shared_expert is not None:
            options = dict(shared_expert)
            self.shared_gate = bool(options.pop("gate", False))
            self.shared = FEED_FORWARDS.build(
                PartSpec("gated_unit", prefix=f"{prefix}.shared", hidden_size=hidden_size, tag="moe.shared", **options), dtype=dtype, device=device
            )
        self.w_shared_gate: Optional[torch.Tensor] = None
        self.routing = routing
        self.num_identity = num_identity
        self.num_outputs = outputs
        self.groups = groups
        self.groups_keep = groups_keep
        self.route_scale = float(route_scale)
        self.shift = float(shift)
        # a kernel that adds the rows itself (kernels.WeightedRows) knows nothing of identity experts
        self.weighted_rows = num_identity == 0 and not self.weight_on_input and self.shared is None
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
        if self.has_correction:
            specs.append(TensorSpec(f"{p}.correction", (self.num_outputs,), role="vector", init="normal"))
        if self.router_bias:
            specs.append(TensorSpec(f"{p}.router.b", (self.num_experts,), role="vector", init="normal"))
        if self.shared is not None:
            specs += self.shared.tensor_specs()
            if self.shared_gate:
                specs.append(TensorSpec(f"{p}.shared.sg", (1, h)))
        return specs

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        p = self.prefix
        experts = range(self.num_experts)
        self.w_gate_up = torch.stack(
            [torch.cat([tensors[f"{p}.e{e}.gate"], tensors[f"{p}.e{e}.up"]], dim=0) for e in experts], dim=0
        ).contiguous()
        self.w_down = torch.stack([tensors[f"{p}.e{e}.down"] for e in experts], dim=0).contiguous()
        self.w_router = tensors[f"{p}.router"].contiguous()
        if self.shared is not None:
            self.shared.load(tensors)
            if self.shared_gate:  # the gate's row rides behind the router's rows: one product, 32-bit output
                self.w_router = torch.cat([self.w_router, tensors[f"{p}.shared.sg"].view(1, -1)], dim=0).contiguous()
        self.b_router = tensors[f"{p}.router.b"].contiguous() if self.router_bias else None
        self.correction = tensors[f"{p}.correction"].contiguous() if self.has_correction else None

    def bytes_streamed(self) -> int:
        """What a single token reads: the router and ``top`` experts."""
        per_expert = (self.w_gate_up[0].numel() + self.w_down[0].numel()) * self.w_down.element_size()
        shared = self.shared.bytes_streamed() if self.shared is not None else 0
        return self.w_router.numel() * self.w_router.element_size() + self.top * per_expert + shared

    def forward(self, x: torch.Tensor, ctx: StepContext, combine: bool = True):
        tokens = x.shape[0]
        tokens_rows = x  # the step's rows as they came (x may become the pairs' scaled rows below)
        ws = ctx.workspace
        experts, top = self.num_outputs, self.top  # identity experts have runs in the plan too; the products skip them
        columns = self.w_router.shape[0]  # the router's outputs, and the shared expert's gate behind them if it has one
        logits = ws.buffer("moe.logits", tokens, columns, torch.float32)
        kernels.linear(x, self.w_router, None, logits)
        ids = ws.buffer("moe.ids", tokens, top, torch.int32)
        weights = ws.buffer("moe.weights", tokens, top, torch.float32)
        if self.routing == "scores":
            kernels.moe_route_scores(logits[:, :experts], self.correction, top, ids, weights, groups=self.groups, keep=self.groups_keep,
                                     scale=self.route_scale, score=self.score_function)
        else:
            kernels.moe_route(logits, self.b_router, top, ids, weights)
        pairs = tokens * top
        plan = kernels.moe_plan(ids, experts, ws.flat("moe.plan", kernels.moe_plan_size(pairs, experts), torch.int32))
        unit = dict(limit=self.limit, alpha=self.alpha, shift=self.shift)
        library = not kernels.moe_skinny_ok(tokens, self.hidden_size, self.intermediate_size, self.dtype) \
            and kernels.moe_library_products_ok(self.hidden_size, self.intermediate_size, self.dtype)
        if self.weight_on_input and not library:
            # a row a pair, w * x, in the order of the pairs: the products then see `pairs` tokens of one expert each
            scaled = ws.buffer("moe.scaled", pairs, self.hidden_size, self.dtype)
            kernels.moe_scale_rows(x, weights.view(-1), scaled, per=top)
            x, top = scaled, 1
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
            if self.weight_on_input:
                kernels.moe_scale_rows(x, weights.view(-1), gathered, rows=plan["token_of"], index=plan["sorted"])
            else:
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
            if not self.weighted_rows:
                raise ValueError("a mixture with identity experts, weights on the experts' inputs or a shared expert adds its rows itself")
            return kernels.WeightedRows(rows, weights, at)
        out = ws.buffer("moe.out", tokens, self.hidden_size, self.dtype)
        extras = {}
        if self.shared is not None:
            extras = dict(extra=self.shared.forward(tokens_rows, ctx), extra_gate=logits[:, experts:] if self.shared_gate else None)
        if self.num_identity:
            kernels.moe_combine(rows, weights, out, at, ids=ids, x=x, experts=self.num_experts, **extras)
        elif self.weight_on_input:
            kernels.moe_combine(rows, None, out, at, top=self.top, **extras)
        else:
            kernels.moe_combine(rows, weights, out, at, **extras)
        return out
