"""Grouped-query attention with an output gate over the paged cache, keys and values of different widths.

One product gives ``q | k | v | g`` (``g``: the gate's rows, ``num_heads * value_dim``).  Then, per token::

    q <- q * rsqrt(mean(q^2) + eps) * wq     over ALL num_heads * head_dim columns at once  (``qk_norm="projection"``)
    k <- k * rsqrt(mean(k^2) + eps) * wk     over all num_kv_heads * head_dim columns       (``qk_norm=None``: neither)
    the first ``rotary_dim`` columns of every head of q and k turn by the token's position: pairs
    (i, i + rotary_dim/2), or (2i, 2i + 1) with ``rotary_interleaved``; columns behind them keep their values
    s(i, j) = q(i) . k(j) * scale            over the keys i sees (itself and the ``window - 1`` before it; None: all)
    p(i, j) = exp(s(i, j)) / (exp(sink_h) + sum_j' exp(s(i, j')))
    o = (sum_j p(i, j) v(j)) * sigmoid(g)    (``gate=False``: no gate, and no gate rows in the product)

``qk_norm="head"``: the norm runs over each head's ``head_dim`` columns, with weights of ``head_dim`` entries that the
heads share.  ``value_position``: a rotary encoding of the VALUES: the value at position j is turned by j over the columns
that encoding covers before it is cached, and each head's result at position i is turned back by -i before the gate, so that
what a query sees of a value depends on their distance alone.  ``own_kv=False``: the mixer has no key and value projections
(nor their norm); it attends over a cache that another layer's call wrote in the same step, with queries, sink and gate of
its own (the run order names that slot with ``writes_cache=False``).

``sink``: ``None`` (a plain softmax), ``"zero"`` (a sink of logit 0: one added to the denominator, no tensor) or
``"learned"`` (tensor ``<prefix>.sink``, one logit a query head).  A sink is a term exp(sink) of the denominator alone, taken as stored.
The gate reads the mixer's input, as the projections do.  Query head h uses key/value head
``h // (num_heads / num_kv_heads)``.  Cached per token and key/value head: the normed, rotated key (``head_dim``) and the
value (``value_dim``).  Norm statistics, the rotation, scores, softmax and the gate are 32-bit in both modes.
bfloat16 with ``head_dim == value_dim`` of a size the paged tensor-core kernels take runs on them (prompt portions in query
tiles, single tokens split over the keys), the sink in their last step and the gate at their store; everything else runs the
32-bit-arithmetic kernel.

Tensors under ``prefix``: ``q``, ``k``, ``v``, ``o``, and ``g``, ``q.norm``, ``k.norm``, ``sink`` as the options ask.
"""

from __future__ import annotations

from typing import Any, Mapping, Optional

import torch

from kairyu_b200 import kernels
from kairyu_b200.parts.attention import run_paged_attention
from kairyu_b200.parts.base import MIXERS, POSITION_ENCODINGS, CacheView, Mixer, PagedKVSpec, PartSpec, StepContext, TensorSpec


@MIXERS.register("gated_attention")
class GatedAttention(Mixer):
    graph_safe = True

    def __init__(
        self,
        *,
        prefix: str,
        hidden_size: int,
        num_heads: int,
        num_kv_heads: int,
        head_dim: int,
        value_dim: int,
        scale: float,
        norm_eps: float,
        qk_norm: Optional[str] = "projection",
        position: Optional[PartSpec] = None,
        rotary_interleaved: bool = False,
        sink: Optional[str] = "zero",
        gate: bool = True,
        window: Optional[int] = None,
        value_position: Optional[PartSpec] = None,
        own_kv: bool = True,
        dtype: torch.dtype,
        device: str,
        shared: Optional[dict] = None,
        **_: object,
    ) -> None:
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} query heads are not a multiple of {num_kv_heads} KV heads")
        if qk_norm not in (None, "projection", "head"):
            raise ValueError(f"unknown query/key norm {qk_norm!r} (None, 'projection', 'head')")
        if sink not in (None, "zero", "learned"):
            raise ValueError(f"unknown sink {sink!r} (None, 'zero', 'learned')")
        self.prefix = prefix
        self.hidden_size = hidden_size
        self.num_heads = num_heads
        self.num_kv_heads = num_kv_heads
        self.head_dim = head_dim
        self.value_dim = value_dim
        self.scale = float(scale)
        self.norm_eps = float(norm_eps)
        self.qk_norm = qk_norm
        self.rotary_interleaved = rotary_interleaved
        self.sink = sink
        self.gate = gate
        self.window = window
        self.dtype = dtype
        self.device = device
        self.own_kv = bool(own_kv)
        table = shared if shared is not None else {}

        def encoding(spec: Optional[PartSpec], width: int):
            if spec is None:
                return None
            key = ("position", spec)
            if key not in table:  # one table for all layers that ask for the same encoding
                table[key] = POSITION_ENCODINGS.build(spec, device=device, dtype=dtype)
            if table[key].rotary_dim > width:
                raise ValueError(f"{table[key].rotary_dim} rotated columns in a head of {width}")
            return table[key]

        self.position = encoding(position, head_dim)
        self.value_position = encoding(value_position, value_dim)
        self.q_size = num_heads * head_dim
        self.k_size = num_kv_heads * head_dim if self.own_kv else 0
        self.v_size = num_kv_heads * value_dim if self.own_kv else 0
        self.out_size = num_heads * value_dim
        self.k_offset = self.q_size
        self.v_offset = self.q_size + self.k_size
        self.g_offset = self.v_offset + self.v_size
        self.packed_width = self.g_offset + (self.out_size if gate else 0)
        self.w_in: Optional[torch.Tensor] = None  # [q | k | v | g rows, hidden]
        self.w_o: Optional[torch.Tensor] = None
        self.q_norm_weight: Optional[torch.Tensor] = None
        self.k_norm_weight: Optional[torch.Tensor] = None
        self.sinks: Optional[torch.Tensor] = None

    # -- weights
    def tensor_specs(self) -> list[TensorSpec]:
        p = self.prefix
        specs = [TensorSpec(f"{p}.q", (self.q_size, self.hidden_size))]
        if self.own_kv:
            specs += [TensorSpec(f"{p}.k", (self.k_size, self.hidden_size)), TensorSpec(f"{p}.v", (self.v_size, self.hidden_size))]
        if self.qk_norm:
            per_head = self.qk_norm == "head"
            specs.append(TensorSpec(f"{p}.q.norm", (self.head_dim if per_head else self.q_size,), role="vector", init="norm"))
            if self.own_kv:
                specs.append(TensorSpec(f"{p}.k.norm", (self.head_dim if per_head else self.k_size,), role="vector", init="norm"))
        if self.gate:
            specs.append(TensorSpec(f"{p}.g", (self.out_size, self.hidden_size)))
        if self.sink == "learned":
            specs.append(TensorSpec(f"{p}.sink", (self.num_heads,), role="vector", init="normal"))
        specs.append(TensorSpec(f"{p}.o", (self.hidden_size, self.out_size)))
        return specs

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        p = self.prefix
        rows = [tensors[f"{p}.q"]] + ([tensors[f"{p}.k"], tensors[f"{p}.v"]] if self.own_kv else []) + ([tensors[f"{p}.g"]] if self.gate else [])
        self.w_in = torch.cat(rows, dim=0).contiguous()
        self.w_o = tensors[f"{p}.o"].contiguous()
        if self.qk_norm:
            self.q_norm_weight = tensors[f"{p}.q.norm"].contiguous()
            # without keys of its own the kernel norms no key; it still wants the two weights as a pair
            self.k_norm_weight = tensors[f"{p}.k.norm"].contiguous() if self.own_kv else self.q_norm_weight
            if self.q_norm_weight.dtype != self.k_norm_weight.dtype:
                self.q_norm_weight, self.k_norm_weight = self.q_norm_weight.float(), self.k_norm_weight.float()
        if self.sink == "learned":
            self.sinks = tensors[f"{p}.sink"].float().contiguous()  # they enter the softmax, which is 32-bit
        elif self.sink == "zero":
            self.sinks = torch.zeros(self.num_heads, dtype=torch.float32, device=self.w_o.device)

    def bytes_streamed(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.w_in, self.w_o, self.q_norm_weight, self.k_norm_weight) if t is not None)

    # -- cache
    def cache_specs(self) -> tuple[Any, ...]:
        if not self.own_kv:
            return ()  # it reads a slot another call wrote
        return (PagedKVSpec(self.num_kv_heads, self.head_dim, self.window, v_head_dim=self.value_dim),)

    def _tensor_cores(self) -> bool:
        """bfloat16 with keys and values of one width: the paged tensor-core kernels (sink and gate in their last
        steps).  Other widths and float32 take the 32-bit-arithmetic kernel."""
        return (self.dtype == torch.bfloat16 and self.head_dim == self.value_dim
                and kernels.attention_mma_supported(self.head_dim, self.num_heads, self.num_kv_heads)
                and (self.sink is None or kernels.ATTENTION_MMA_SINKS))

    def query_tile_sizes(self) -> tuple[int, ...]:
        if not self._tensor_cores():
            return ()
        wide = kernels.attention_prefill_wide_tile_rows(self.head_dim)
        return (kernels.attention_prefill_tile_rows(self.head_dim),) + ((wide,) if wide else ())

    # -- compute
    def forward(self, x: torch.Tensor, ctx: StepContext, cache: CacheView) -> torch.Tensor:
        tokens = x.shape[0]
        ws = ctx.workspace
        packed = ws.buffer("gattn.packed", tokens, self.packed_width, self.dtype)
        kernels.linear(x, self.w_in, None, packed)
        block_table = ctx.block_tables[cache.group]
        cos, sin = self.position.rotary_tables() if self.position is not None else (None, None)
        v_cos, v_sin = self.value_position.rotary_tables() if self.value_position is not None else (None, None)
        writes = cache.writes and self.own_kv
        if cache.writes and not self.own_kv:
            raise ValueError("a mixer without key and value projections cannot be the writer of a cache slot")
        kernels.projection_norm_rope_write(
            packed, num_q_heads=self.num_heads, num_kv_heads=self.num_kv_heads if self.own_kv else 0, head_dim=self.head_dim,
            value_dim=self.value_dim, k_offset=self.k_offset, v_offset=self.v_offset, positions=ctx.positions, row_ids=ctx.row_ids,
            q_norm_weight=self.q_norm_weight, k_norm_weight=self.k_norm_weight, eps=self.norm_eps, cos=cos, sin=sin,
            interleaved=self.rotary_interleaved, block_table=block_table if writes else None,
            write_from=ctx.write_from if writes else None, k_cache=cache.k if writes else None, v_cache=cache.v if writes else None,
            flag=ctx.error_flag, per_head_norm=self.qk_norm == "head", v_cos=v_cos if writes else None, v_sin=v_sin if writes else None,
        )
        mixed = ws.buffer("gattn.mixed", tokens, self.out_size, self.dtype)
        gate = packed[:, self.g_offset :] if self.gate else None
        if self._tensor_cores() and not ctx.extras.get("force_generic_attention", False):
            run_paged_attention(packed, mixed, cache, ctx, num_q_heads=self.num_heads, num_kv_heads=self.num_kv_heads, head_dim=self.head_dim,
                                scale=self.scale, window=self.window or 0, sinks=self.sinks, gate=gate)
        else:
            kernels.diff_attention_generic(
                packed, mixed, cache.k, cache.v, positions=ctx.positions, row_ids=ctx.row_ids, block_table=block_table,
                num_q_heads=self.num_heads, maps=1, scale=self.scale, window=self.window or 0, sinks=self.sinks, gate=gate, flag=ctx.error_flag,
            )
        if v_cos is not None:  # the values were cached turned by their positions: turn each head's sum back by the query's
            if self.gate:
                raise ValueError("turned values with an output gate: the gate would have to follow the turning back")
            kernels.rotate_heads(mixed, heads=self.num_heads, head_dim=self.value_dim, cos=v_cos, sin=v_sin, positions=ctx.positions,
                                 interleaved=self.rotary_interleaved, inverse=True, flag=ctx.error_flag)
        out = ws.buffer("gattn.out", tokens, self.hidden_size, self.dtype)
        kernels.linear(mixed, self.w_o, None, out)
        return out
