"""Two mixers side by side on one input: ``left_scale * left(x) + right_scale * right(x)``.

Both read the same rows; each keeps what it keeps (pages, per-request state), and the cache slot of the layer holds
both: the paged cache is the side's that asks for one (at most one side may), the state tensors are the left's followed
by the right's.  Tensors: the left mixer's under ``<prefix>.left``, the right's under ``<prefix>.right`` (the two specs
carry those prefixes).  The sum is formed in 32-bit with one rounding.
"""

from __future__ import annotations

import dataclasses
from typing import Any, Mapping

import torch

from kairyu_b200 import kernels
from kairyu_b200.parts.base import MIXERS, CacheView, Mixer, PagedKVSpec, PartSpec, StateSpec, StepContext, TensorSpec


@MIXERS.register("side_by_side")
class SideBySide(Mixer):
    graph_safe = True

    def __init__(self, *, left: PartSpec, right: PartSpec, left_scale: float, right_scale: float, hidden_size: int, dtype: torch.dtype,
                 device: str, shared: dict, **_: object) -> None:
        context = dict(dtype=dtype, device=device, shared=shared)
        self.left = MIXERS.build(left, **context)
        self.right = MIXERS.build(right, **context)
        self.left_scale = float(left_scale)
        self.right_scale = float(right_scale)
        self.hidden_size = hidden_size
        self.dtype = dtype
        self._parts = (self.left, self.right)
        specs = [spec for side in self._parts for spec in side.cache_specs()]
        if sum(isinstance(spec, PagedKVSpec) for spec in specs) > 1:
            raise ValueError("two mixers side by side: at most one of them may keep pages")
        self._left_states = sum(isinstance(spec, StateSpec) for spec in self.left.cache_specs())

    def tensor_specs(self) -> list[TensorSpec]:
        return [spec for side in self._parts for spec in side.tensor_specs()]

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        for side in self._parts:
            side.load(tensors)

    def bytes_streamed(self) -> int:
        return sum(side.bytes_streamed() for side in self._parts)

    def cache_specs(self) -> tuple[Any, ...]:
        return tuple(spec for side in self._parts for spec in side.cache_specs())

    def query_tile_sizes(self) -> tuple[int, ...]:
        return tuple(size for side in self._parts for size in side.query_tile_sizes())

    def _views(self, cache: CacheView) -> tuple[CacheView, CacheView]:
        states = cache.state if isinstance(cache.state, (list, tuple)) else ([] if cache.state is None else [cache.state])
        views = []
        for side, mine in ((self.left, states[: self._left_states]), (self.right, states[self._left_states :])):
            paged = any(isinstance(spec, PagedKVSpec) for spec in side.cache_specs())
            view = dataclasses.replace(cache, state=None if not mine else (mine[0] if len(mine) == 1 else list(mine)))
            if not paged:
                view.k = view.v = None
                view.group = -1
            views.append(view)
        return views[0], views[1]

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: CacheView) -> torch.Tensor:
        left_view, right_view = self._views(cache)
        left = self.left.forward(x, ctx, left_view)
        right = self.right.forward(x, ctx, right_view)
        out = ctx.workspace.buffer("side_by_side.out", x.shape[0], self.hidden_size, self.dtype)
        kernels.scaled_sum(left, self.left_scale, right, self.right_scale, out)
        return out
