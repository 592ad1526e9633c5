"""SiLU-gated feed-forward (kairyu/models/layers.py:193-244):
``down(silu(gate(x)) * up(x))``.  gate and up are one matrix product over the
row-concatenated weight (the reference runs them as two).  ``names``: the three tensors'
names under ``prefix`` (gate, up, down) where a file calls them otherwise."""

from __future__ import annotations

from typing import Mapping, Optional

import torch

from kairyu_b200 import kernels
from kairyu_b200.parts.base import FEED_FORWARDS, FeedForward, StepContext, TensorSpec


@FEED_FORWARDS.register("swiglu")
class SwiGLU(FeedForward):
    graph_safe = True

    def __init__(
        self,
        *,
        prefix: str,
        hidden_size: int,
        intermediate_size: int,
        activation: str,
        dtype: torch.dtype,
        device: str,
        names: tuple = ("gate_proj.weight", "up_proj.weight", "down_proj.weight"),
        **_: object,
    ) -> None:
        if activation != "silu":
            raise ValueError(f"gated feed-forward activation {activation!r} is not implemented (silu)")
        self.names = tuple(names)
        self.prefix = prefix
        self.hidden_size = hidden_size
        self.intermediate_size = intermediate_size
        self.dtype = dtype
        self.w_gate_up: Optional[torch.Tensor] = None
        self.w_down: Optional[torch.Tensor] = None

    def tensor_specs(self) -> list[TensorSpec]:
        p = self.prefix
        gate, up, down = self.names
        return [
            TensorSpec(f"{p}.{gate}", (self.intermediate_size, self.hidden_size)),
            TensorSpec(f"{p}.{up}", (self.intermediate_size, self.hidden_size)),
            TensorSpec(f"{p}.{down}", (self.hidden_size, self.intermediate_size)),
        ]

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        p = self.prefix
        gate, up, down = self.names
        self.w_gate_up = torch.cat([tensors[f"{p}.{gate}"], tensors[f"{p}.{up}"]], dim=0).contiguous()
        self.w_down = tensors[f"{p}.{down}"].contiguous()

    def bytes_streamed(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.w_gate_up, self.w_down))

    def fusable_norm(self, tokens: int) -> bool:
        """Whether both products can take the norms around them into their epilogues."""
        return kernels.fused_norm_shapes_ok(tokens, self.hidden_size, self.intermediate_size)

    def forward(self, x, ctx: StepContext, fold=None):
        """``x``: rows, or a ``kernels.PreNormed``; ``fold`` (a ``kernels.ResidualNorm``): the down
        product adds its result to the residual and returns the ``PreNormed`` for the next norm."""
        tokens = x.shape[0]
        ws = ctx.workspace
        hidden = ws.buffer("ffn.hidden", tokens, self.intermediate_size, self.dtype)
        kernels.linear_swiglu(x, self.w_gate_up, hidden, ws)
        if fold is not None:
            kernels.linear(hidden, self.w_down, None, None, fold=fold)
            return fold.result()
        out = ws.buffer("ffn.out", tokens, self.hidden_size, self.dtype)
        kernels.linear(hidden, self.w_down, None, out)
        return out


@FEED_FORWARDS.register("mlp")
class UngatedMLP(FeedForward):
    """``down(act(up(x)))`` without a gate and without biases.  ``activation``: ``relu2`` (the square of
    relu), ``gelu_tanh`` or ``silu``; it runs in 32-bit on the up product's rows, with one rounding at
    the store.  ``up_name`` / ``down_name``: the two tensors' names under ``prefix``."""

    graph_safe = True

    def __init__(
        self,
        *,
        prefix: str,
        hidden_size: int,
        intermediate_size: int,
        activation: str,
        up_name: str = "up",
        down_name: str = "down",
        dtype: torch.dtype,
        device: str,
        **_: object,
    ) -> None:
        if activation not in kernels.ACTIVATIONS:
            raise ValueError(f"feed-forward activation {activation!r} is not implemented ({', '.join(kernels.ACTIVATIONS)})")
        self.prefix = prefix
        self.hidden_size = hidden_size
        self.intermediate_size = intermediate_size
        self.activation = activation
        self.up_name = f"{prefix}.{up_name}"
        self.down_name = f"{prefix}.{down_name}"
        self.dtype = dtype
        self.w_up: Optional[torch.Tensor] = None
        self.w_down: Optional[torch.Tensor] = None

    def tensor_specs(self) -> list[TensorSpec]:
        return [
            TensorSpec(self.up_name, (self.intermediate_size, self.hidden_size)),
            TensorSpec(self.down_name, (self.hidden_size, self.intermediate_size)),
        ]

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.w_up = tensors[self.up_name].contiguous()
        self.w_down = tensors[self.down_name].contiguous()

    def bytes_streamed(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.w_up, self.w_down))

    def fusable_norm(self, tokens: int) -> bool:
        """Whether both products can take the norms around them into their epilogues."""
        return kernels.fused_norm_shapes_ok(tokens, self.hidden_size, self.intermediate_size)

    def forward(self, x, ctx: StepContext, fold=None):
        """``x``: rows, or a ``kernels.PreNormed``; ``fold`` (a ``kernels.ResidualNorm``): the down product
        adds its result to the residual and returns the ``PreNormed`` for the next norm."""
        tokens = x.shape[0]
        ws = ctx.workspace
        hidden = ws.buffer("mlp.hidden", tokens, self.intermediate_size, self.dtype)
        kernels.linear(x, self.w_up, None, hidden)
        kernels.activation(hidden, hidden, self.activation)
        if fold is not None:
            kernels.linear(hidden, self.w_down, None, None, fold=fold)
            return fold.result()
        out = ws.buffer("mlp.out", tokens, self.hidden_size, self.dtype)
        kernels.linear(hidden, self.w_down, None, out)
        return out


@FEED_FORWARDS.register("gated_unit")
class GatedUnit(FeedForward):
    """``down(a * sigmoid(alpha a) * (b + shift))`` with ``a = min(gate(x), limit)`` and ``b = clamp(up(x), -limit, limit)``, no
    biases: the unit the experts of ``moe`` are made of, as a dense feed-forward.  ``limit=None``, ``alpha=1``, ``shift=0`` is
    ``silu(gate(x)) * up(x)``.  gate and up are one product over the row-concatenated weight; the unit's arithmetic is
    32-bit with one rounding at the store.  ``gate_name`` / ``up_name`` / ``down_name``: the tensors' names under ``prefix``."""

    graph_safe = True

    def __init__(
        self,
        *,
        prefix: str,
        hidden_size: int,
        intermediate_size: int,
        limit: Optional[float] = None,
        alpha: float = 1.0,
        shift: float = 0.0,
        gate_name: str = "gate",
        up_name: str = "up",
        down_name: str = "down",
        tag: str = "glu",
        dtype: torch.dtype,
        device: str,
        **_: object,
    ) -> None:
        self.prefix = prefix
        self.hidden_size = hidden_size
        self.intermediate_size = intermediate_size
        self.limit = float("inf") if limit is None else float(limit)
        self.alpha = float(alpha)
        self.shift = float(shift)
        self.names = tuple(f"{prefix}.{name}" for name in (gate_name, up_name, down_name))
        self.tag = tag  # workspace buffers are named by it: two units that are alive at once take different tags
        self.dtype = dtype
        self.w_gate_up: Optional[torch.Tensor] = None
        self.w_down: Optional[torch.Tensor] = None

    @property
    def plain(self) -> bool:
        return self.limit == float("inf") and self.alpha == 1.0 and self.shift == 0.0

    def tensor_specs(self) -> list[TensorSpec]:
        gate, up, down = self.names
        return [
            TensorSpec(gate, (self.intermediate_size, self.hidden_size)),
            TensorSpec(up, (self.intermediate_size, self.hidden_size)),
            TensorSpec(down, (self.hidden_size, self.intermediate_size)),
        ]

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        gate, up, down = self.names
        self.w_gate_up = torch.cat([tensors[gate], tensors[up]], dim=0).contiguous()
        self.w_down = tensors[down].contiguous()

    def bytes_streamed(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.w_gate_up, self.w_down))

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        tokens = x.shape[0]
        ws = ctx.workspace
        hidden = ws.buffer(f"{self.tag}.hidden", tokens, self.intermediate_size, self.dtype)
        if self.plain:
            kernels.linear_swiglu(x, self.w_gate_up, hidden, ws)  # a few rows: the gate rides in the product's epilogue
        else:
            gate_up = ws.buffer(f"{self.tag}.gate_up", tokens, 2 * self.intermediate_size, self.dtype)
            kernels.linear(x, self.w_gate_up, None, gate_up)
            kernels.moe_activation(gate_up, hidden, limit=self.limit, alpha=self.alpha, shift=self.shift)
        out = ws.buffer(f"{self.tag}.out", tokens, self.hidden_size, self.dtype)
        kernels.linear(hidden, self.w_down, None, out)
        return out
