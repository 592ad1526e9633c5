"""Arrangements of norms, mixer and feed-forward around the residual stream."""

from __future__ import annotations

from typing import Mapping, Optional

import torch

from kairyu_b200 import kernels
from kairyu_b200.parts.base import (
    BLOCKS,
    FEED_FORWARDS,
    MIXERS,
    NORMS,
    Block,
    CacheView,
    LayerSpec,
    Norm,
    StepContext,
    TensorSpec,
)


@BLOCKS.register("pre_norm")
class PreNormBlock(Block):
    """``x += mixer(norm(x)); x += ffn(norm(x))`` (kairyu/models/llama.py:88-101).

    The residual is fp32.  Each sub-layer's output is handed on as a pending
    delta and added by the next norm's kernel.

    For a few bf16 rows (decode) the norms have no kernel of their own: the product before a
    norm adds its result to the residual and leaves the rows weighted and their sums of squares
    (``kernels.ResidualNorm``), the product after it scales by the root mean square
    (``kernels.PreNormed``).  That needs norms that offer ``fold_target`` (RMSNorm does) and a
    mixer and feed-forward that offer ``fusable_norm``; any other part gets the plain flow.
    """

    graph_safe = True

    takes_next_norm = True  # forward accepts the norm of the block that runs next

    def __init__(self, *, layer: LayerSpec, dtype: torch.dtype, device: str, shared: dict, **_: object) -> None:
        context = dict(dtype=dtype, device=device, shared=shared)
        self.mixer_norm = NORMS.build(layer.mixer_norm, **context)
        self.mixer = MIXERS.build(layer.mixer, **context)
        # a layer may have no feed-forward: the block is then x += mixer(norm(x)) alone
        self.ffn_norm = NORMS.build(layer.ffn_norm, **context) if layer.ffn is not None else None
        self.ffn = FEED_FORWARDS.build(layer.ffn, **context) if layer.ffn is not None else None
        self._parts = tuple(part for part in (self.mixer_norm, self.mixer, self.ffn_norm, self.ffn) if part is not None)

    def tensor_specs(self) -> list[TensorSpec]:
        return [spec for part in self._parts for spec in part.tensor_specs()]

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        for part in self._parts:
            part.load(tensors)

    def bytes_streamed(self) -> int:
        return sum(part.bytes_streamed() for part in self._parts)

    def _fused(self, ctx: StepContext) -> bool:
        if ctx.dtype != torch.bfloat16 or self.ffn is None or not kernels.fused_norm_available():
            return False
        if not (hasattr(self.mixer_norm, "fold_target") and hasattr(self.ffn_norm, "fold_target")):
            return False  # a norm offers ``fold_target`` when the products around it can take its two halves
        mixer_ok = getattr(self.mixer, "fusable_norm", None)
        ffn_ok = getattr(self.ffn, "fusable_norm", None)
        return bool(mixer_ok and ffn_ok and mixer_ok(ctx.num_tokens) and ffn_ok(ctx.num_tokens))

    def prenorm_target(self, ctx: StepContext) -> Optional[Norm]:
        """The norm the block before this one may fold into its last product, or None."""
        return self.mixer_norm if self._fused(ctx) else None

    def forward(
        self,
        residual: torch.Tensor,
        delta,
        ctx: StepContext,
        cache: CacheView,
        next_norm: Optional[Norm] = None,
    ):
        if isinstance(delta, kernels.PreNormed):  # the block before has added its output and begun our norm
            normed = delta
        else:
            normed = self.mixer_norm.apply(residual, delta, ctx)
        if self.ffn is None:
            return residual, self.mixer.forward(normed, ctx, cache)
        if not self._fused(ctx):
            mixed = self.mixer.forward(normed, ctx, cache)
            normed = self.ffn_norm.apply(residual, mixed, ctx)
            return residual, self.ffn.forward(normed, ctx)
        mixed = self.mixer.forward(normed, ctx, cache, fold=self.ffn_norm.fold_target(residual, ctx, "ffn"))
        fold = next_norm.fold_target(residual, ctx, "mixer") if next_norm is not None else None
        return residual, self.ffn.forward(mixed, ctx, fold=fold)


@BLOCKS.register("output_norm")
class OutputNormBlock(Block):
    """``x += norm1(mixer(x)); x += norm2(ffn(x))``: the norms sit on the sub-layers' outputs, and the
    sub-layers read the stream itself.  A layer may have no feed-forward.

    The residual is fp32; one kernel per sub-layer norms the output, adds it to the residual and
    leaves the residual's rows in the activation dtype for the next products (``Norm.add_normed``).
    That copy travels to the next block in place of a pending delta (``kernels.ResidualCopy``).  A
    feed-forward that can hand over its rows before their weighted sum (a mixture of experts) does,
    and the same kernel adds them.
    """

    graph_safe = True

    def __init__(self, *, layer: LayerSpec, dtype: torch.dtype, device: str, shared: dict, **_: object) -> None:
        context = dict(dtype=dtype, device=device, shared=shared)
        self.dtype = dtype
        self.mixer = MIXERS.build(layer.mixer, **context)
        self.mixer_norm = NORMS.build(layer.mixer_norm, **context)
        self.ffn = FEED_FORWARDS.build(layer.ffn, **context) if layer.ffn is not None else None
        self.ffn_norm = NORMS.build(layer.ffn_norm, **context) if layer.ffn is not None else None
        self._parts = tuple(part for part in (self.mixer, self.mixer_norm, self.ffn, self.ffn_norm) if part is not None)
        for norm in (self.mixer_norm, self.ffn_norm):
            if norm is not None and not hasattr(norm, "add_normed"):
                raise ValueError("this arrangement needs norms that offer add_normed (rmsnorm does)")

    def tensor_specs(self) -> list[TensorSpec]:
        return [spec for part in self._parts for spec in part.tensor_specs()]

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        for part in self._parts:
            part.load(tensors)

    def bytes_streamed(self) -> int:
        return sum(part.bytes_streamed() for part in self._parts)

    def forward(self, residual: torch.Tensor, delta, ctx: StepContext, cache: CacheView):
        if isinstance(delta, kernels.ResidualCopy):
            rows = delta.values
        elif delta is not None:
            raise ValueError("an output-norm block cannot follow a block that leaves a sum to be added")
        elif self.dtype == torch.float32:
            rows = residual
        else:  # the model's first block: the embedding's rows
            rows = ctx.workspace.buffer("residual.copy", residual.shape[0], residual.shape[1], self.dtype)
            kernels.residual_copy(residual, rows)
        rows = self.mixer_norm.add_normed(residual, self.mixer.forward(rows, ctx, cache), ctx)
        if self.ffn is not None:
            if getattr(self.ffn, "weighted_rows", False):
                output = self.ffn.forward(rows, ctx, combine=False)
            else:
                output = self.ffn.forward(rows, ctx)
            rows = self.ffn_norm.add_normed(residual, output, ctx)
        return residual, (None if rows is residual else kernels.ResidualCopy(rows))


@BLOCKS.register("parallel")
class ParallelBlock(Block):
    """``h = norm(x); x += mixer(h) + ffn(h)``: one norm a layer, and both sub-layers read its output.  A layer may have no
    feed-forward.

    The residual is fp32.  The two outputs are handed on unsummed (``kernels.PendingSums``) and the next norm's kernel adds
    them to the residual, in 32-bit, on its way, so the layer's sum costs no kernel of its own; the norm must be one that
    takes two pending sums (``layernorm`` does)."""

    graph_safe = True

    def __init__(self, *, layer: LayerSpec, dtype: torch.dtype, device: str, shared: dict, **_: object) -> None:
        context = dict(dtype=dtype, device=device, shared=shared)
        self.mixer_norm = NORMS.build(layer.mixer_norm, **context)
        self.mixer = MIXERS.build(layer.mixer, **context)
        self.ffn = FEED_FORWARDS.build(layer.ffn, **context) if layer.ffn is not None else None
        if layer.ffn_norm is not None:
            raise ValueError("a parallel layer has one norm; its feed-forward reads the mixer's input")
        self._parts = tuple(part for part in (self.mixer_norm, self.mixer, self.ffn) if part is not None)

    def tensor_specs(self) -> list[TensorSpec]:
        return [spec for part in self._parts for spec in part.tensor_specs()]

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        for part in self._parts:
            part.load(tensors)

    def bytes_streamed(self) -> int:
        return sum(part.bytes_streamed() for part in self._parts)

    def forward(self, residual: torch.Tensor, delta, ctx: StepContext, cache: CacheView):
        normed = self.mixer_norm.apply(residual, delta, ctx)
        mixed = self.mixer.forward(normed, ctx, cache)
        if self.ffn is None:
            return residual, mixed
        return residual, kernels.PendingSums(mixed, self.ffn.forward(normed, ctx))


@BLOCKS.register("sandwich_norm")
class SandwichNormBlock(Block):
    """``x += post1(mixer(pre1(x))); x += post2(ffn(pre2(x)))``: a norm before and a norm after each sub-layer.  A layer
    may have no feed-forward.

    The residual is fp32.  A sub-layer's output is handed on with its post-norm still to be applied
    (``kernels.PendingNormed``), and the kernel of the norm that reads the stream next norms it, adds it to the
    residual and norms the sum, so a sub-layer costs one norm kernel although it has two norms.  The norms must
    offer ``pending`` and take what it returns as ``delta`` (``rmsnorm`` does)."""

    graph_safe = True

    def __init__(self, *, layer: LayerSpec, dtype: torch.dtype, device: str, shared: dict, **_: object) -> None:
        context = dict(dtype=dtype, device=device, shared=shared)
        if layer.mixer_post_norm is None or (layer.ffn is not None and (layer.ffn_norm is None or layer.ffn_post_norm is None)):
            raise ValueError("this arrangement needs a norm before and a norm after each sub-layer")
        self.mixer_norm = NORMS.build(layer.mixer_norm, **context)
        self.mixer = MIXERS.build(layer.mixer, **context)
        self.mixer_post_norm = NORMS.build(layer.mixer_post_norm, **context)
        self.ffn_norm = NORMS.build(layer.ffn_norm, **context) if layer.ffn is not None else None
        self.ffn = FEED_FORWARDS.build(layer.ffn, **context) if layer.ffn is not None else None
        self.ffn_post_norm = NORMS.build(layer.ffn_post_norm, **context) if layer.ffn is not None else None
        self._parts = tuple(part for part in (self.mixer_norm, self.mixer, self.mixer_post_norm, self.ffn_norm, self.ffn, self.ffn_post_norm)
                            if part is not None)
        for norm in (self.mixer_post_norm, self.ffn_post_norm):
            if norm is not None and not hasattr(norm, "pending"):
                raise ValueError("this arrangement needs output norms that offer pending (rmsnorm does)")

    def tensor_specs(self) -> list[TensorSpec]:
        return [spec for part in self._parts for spec in part.tensor_specs()]

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        for part in self._parts:
            part.load(tensors)

    def bytes_streamed(self) -> int:
        return sum(part.bytes_streamed() for part in self._parts)

    def forward(self, residual: torch.Tensor, delta, ctx: StepContext, cache: CacheView):
        normed = self.mixer_norm.apply(residual, delta, ctx)
        pending = self.mixer_post_norm.pending(self.mixer.forward(normed, ctx, cache))
        if self.ffn is None:
            return residual, pending
        normed = self.ffn_norm.apply(residual, pending, ctx)
        return residual, self.ffn_post_norm.pending(self.ffn.forward(normed, ctx))
