"""Norms with the residual sum fused in: RMSNorm (kairyu/models/layers.py:21-46) and layer norm with weight and bias."""

from __future__ import annotations

from typing import Mapping, Optional

import torch

from kairyu_b200 import kernels
from kairyu_b200.parts.base import NORMS, Norm, StepContext, TensorSpec


@NORMS.register("rmsnorm")
class RMSNorm(Norm):
    """``y = x * rsqrt(mean(x^2) + eps) * (offset + weight)`` with fp32 statistics.  ``offset`` is 0 unless
    given; a file that stores its norm weights around zero names 1, and the sum is then formed once,
    at loading, in 32-bit, and held so.  ``scalar``: the weight is ONE number for all coordinates (a tensor
    without dimensions); it is spread over the width once, at loading, in 32-bit."""

    graph_safe = True

    def __init__(self, *, name: str, size: int, eps: float, dtype: torch.dtype, device: str, offset: float = 0.0, scalar: bool = False,
                 **_: object) -> None:
        self.name = name  # full tensor name of the weight
        self.size = size
        self.eps = float(eps)
        self.offset = float(offset)
        self.scalar = bool(scalar)
        self.dtype = dtype
        self.device = device
        self.weight: Optional[torch.Tensor] = None

    def tensor_specs(self) -> list[TensorSpec]:
        shape = () if self.scalar else (self.size,)
        return [TensorSpec(self.name, shape, role="vector", init="norm" if self.offset == 0.0 else "normal")]

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.weight = tensors[self.name].contiguous()
        if self.scalar:
            self.weight = self.weight.float().reshape(1).expand(self.size).contiguous()
        if self.offset != 0.0:
            self.weight = (self.weight.float() + self.offset).contiguous()

    def bytes_streamed(self) -> int:
        return self.weight.numel() * self.weight.element_size()

    def apply(
        self,
        residual: torch.Tensor,
        delta: Optional[torch.Tensor],
        ctx: StepContext,
        *,
        rows: Optional[torch.Tensor] = None,
    ) -> torch.Tensor:
        count = rows.numel() if rows is not None else residual.shape[0]
        # a subset of rows (the model's last norm, at the wanted places) has a buffer of its own
        out = ctx.workspace.buffer("norm.out" if rows is None else "norm.rows.out", count, self.size, self.dtype)
        if isinstance(delta, kernels.PendingNormed):  # a normed sub-layer output still to be added: one kernel for both norms
            kernels.sandwich_norm(residual, delta, self.weight, self.eps, out, rows=rows)
            return out
        kernels.rmsnorm(residual, self.weight, self.eps, out, delta=delta, rows=rows)
        return out

    def pending(self, y: torch.Tensor) -> "kernels.PendingNormed":
        """For an arrangement that norms a sub-layer's OUTPUT: ``residual += norm(y)`` handed on undone, for the
        norm that reads the stream next to do in its own kernel (``apply`` of this class takes it as ``delta``)."""
        return kernels.PendingNormed(y, self.weight, self.eps)

    def add_normed(self, residual: torch.Tensor, y, ctx: StepContext) -> torch.Tensor:
        """For an arrangement that norms a sub-layer's OUTPUT: ``residual += norm(y)``.  Returns the
        residual's rows as the next sub-layer's products read them: the fp32 residual itself in
        32-bit mode, else a copy in the activation dtype that the same kernel writes.  ``y`` may be a
        ``kernels.WeightedRows`` (a mixture's rows before their weighted sum)."""
        copy = None
        if self.dtype != torch.float32:
            copy = ctx.workspace.buffer("residual.copy", residual.shape[0], self.size, self.dtype)
        kernels.output_norm_add(residual, y, self.weight, self.eps, copy)
        return residual if copy is None else copy

    def fold_target(self, residual: torch.Tensor, ctx: StepContext, tag: str) -> "kernels.ResidualNorm":
        """For a product that takes this norm's first half into its epilogue: it adds its result
        to ``residual`` and leaves the rows weighted and their sums of squares; the product that
        reads them scales by the root mean square (kernels.ResidualNorm / kernels.PreNormed)."""
        rows = residual.shape[0]
        values = ctx.workspace.buffer(f"norm.fold.{tag}.values", rows, self.size, torch.bfloat16)
        sumsq = ctx.workspace.flat(f"norm.fold.{tag}.sumsq", 16 * kernels.skinny_blocks(rows, self.size), torch.float32).view(-1, 16)
        return kernels.ResidualNorm(residual, self.weight, self.eps, values, sumsq)


@NORMS.register("layernorm")
class LayerNorm(Norm):
    """``y = (x - mean(x)) * rsqrt(mean((x - mean(x))^2) + eps) * weight + bias`` with fp32 statistics.  The bias is the tensor
    ``bias_name`` (default: the weight's name + ``.b``).  ``apply`` takes one pending sum or two (``kernels.PendingSums``:
    a layer whose mixer and feed-forward ran side by side) and adds them in the same kernel."""

    graph_safe = True

    def __init__(self, *, name: str, size: int, eps: float, dtype: torch.dtype, device: str, bias_name: Optional[str] = None, **_: object) -> None:
        self.name = name
        self.bias_name = bias_name or f"{name}.b"
        self.size = size
        self.eps = float(eps)
        self.dtype = dtype
        self.device = device
        self.weight: Optional[torch.Tensor] = None
        self.bias: Optional[torch.Tensor] = None

    def tensor_specs(self) -> list[TensorSpec]:
        return [
            TensorSpec(self.name, (self.size,), role="vector", init="norm"),
            TensorSpec(self.bias_name, (self.size,), role="vector", init="normal"),
        ]

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.weight = tensors[self.name].contiguous()
        self.bias = tensors[self.bias_name].contiguous()
        if self.weight.dtype != self.bias.dtype:  # one of them stored in 32-bit: both are held so
            self.weight, self.bias = self.weight.float(), self.bias.float()

    def bytes_streamed(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.weight, self.bias))

    def apply(
        self,
        residual: torch.Tensor,
        delta,
        ctx: StepContext,
        *,
        rows: Optional[torch.Tensor] = None,
    ) -> torch.Tensor:
        count = rows.numel() if rows is not None else residual.shape[0]
        out = ctx.workspace.buffer("norm.out" if rows is None else "norm.rows.out", count, self.size, self.dtype)
        first, second = (delta.first, delta.second) if isinstance(delta, kernels.PendingSums) else (delta, None)
        kernels.layernorm(residual, self.weight, self.bias, self.eps, out, delta=first, delta2=second, rows=rows)
        return out
