"""Latent attention: attention whose keys and values are all products of one compressed row a token.

A token's row ``c = rmsnorm(W_dkv x)`` (``kv_rank`` wide) is all that is cached.  Head h has
``k = W_uk[h] c`` and ``v = W_uv[h] c``; since ``q.k = (W_uk[h]^T q).c`` and
``sum_j p_j v_j = W_uv[h] (sum_j p_j c_j)``, the up-projections move to the query and to the
output, and what runs over the cache is multi-query attention with ONE key/value head of width
``kv_rank`` whose keys and values are the same rows.  So the paged attention kernels of this
package serve it unchanged (the cached rows are passed as keys and as values), and a token costs
``kv_rank`` cached numbers whatever the number of heads.  ``window`` (a token sees itself and the
``window - 1`` before it) and ``scale`` are parameters.

Positions (``rot_dim`` > 0, ``position`` a rotary encoding of that many dimensions): every head's query
has ``rot_dim`` further columns behind its ``head_dim`` (the query product's rows are laid out head by
head as [head_dim | rot_dim]) and the down-projection ``rot_dim`` further rows, one key part that all
heads share.  Both are rotated (pairs (2i, 2i + 1) with ``rotary_interleaved``, else (i, i + rot_dim/2));
the key part is not normed.  The score is ``(q.k + q_rot.k_rot) * scale``.  The rotated key part is cached
behind the latent row, the rotated query part stands behind the query carried into the latent space, and
the attention kernels see one key/value head of width ``kv_rank + rot_dim`` whose values are the first
``kv_rank`` columns of its rows.

``sink``: a learned logit a head (tensor ``<prefix>.sink``) that joins the softmax's denominator and
nothing else (exp(sink) is one more term of the sum, taken as stored: no row of the cache stands behind it).
"""

from __future__ import annotations

from typing import Any, Mapping, Optional

import torch

from kairyu_b200 import kernels
from kairyu_b200.parts.attention import run_paged_attention
from kairyu_b200.parts.base import MIXERS, POSITION_ENCODINGS, CacheView, Mixer, PagedKVSpec, PartSpec, StepContext, TensorSpec


@MIXERS.register("latent_attention")
class LatentAttention(Mixer):
    graph_safe = True

    def __init__(
        self,
        *,
        prefix: str,
        hidden_size: int,
        num_heads: int,
        head_dim: int,
        value_dim: int,
        kv_rank: int,
        scale: float,
        norm_eps: float,
        window: Optional[int] = None,
        rot_dim: int = 0,
        position: Optional[PartSpec] = None,
        rotary_interleaved: bool = True,
        sink: bool = False,
        dtype: torch.dtype,
        device: str,
        shared: Optional[dict] = None,
        **_: object,
    ) -> None:
        if (rot_dim > 0) != (position is not None) or rot_dim % 2:
            raise ValueError("a rotated part of the keys comes with a rotary encoding of its (even) width")
        self.rot_dim = rot_dim
        self.rotary_interleaved = rotary_interleaved
        self.position = None
        if position is not None:
            key = ("position", position)
            table = shared if shared is not None else {}
            if key not in table:  # one table for all layers that ask for the same encoding
                table[key] = POSITION_ENCODINGS.build(position, device=device, dtype=dtype)
            self.position = table[key]
            if self.position.rotary_dim != rot_dim:
                raise ValueError(f"the rotary encoding turns {self.position.rotary_dim} dimensions, the rotated part has {rot_dim}")
        self.has_sink = sink
        self.sinks: Optional[torch.Tensor] = None
        self.prefix = prefix
        self.hidden_size = hidden_size
        self.num_heads = num_heads
        self.head_dim = head_dim
        self.value_dim = value_dim
        self.kv_rank = kv_rank
        self.scale = float(scale)
        self.norm_eps = float(norm_eps)
        self.window = window
        self.dtype = dtype
        self.q_head_width = head_dim + rot_dim
        self.q_size = num_heads * self.q_head_width
        self.row_width = kv_rank + rot_dim  # a cached row: the latent, then the rotated key part
        self.w_in: Optional[torch.Tensor] = None      # [q_size + kv_rank, hidden]: q rows, then the down-projection's
        self.latent_norm: Optional[torch.Tensor] = None
        self.w_absorb: Optional[torch.Tensor] = None  # [heads, kv_rank, head_dim]: W_uk[h]^T
        self.w_up_v: Optional[torch.Tensor] = None    # [heads, value_dim, kv_rank]
        self.w_o: Optional[torch.Tensor] = None

    def tensor_specs(self) -> list[TensorSpec]:
        p = self.prefix
        return [
            TensorSpec(f"{p}.q", (self.q_size, self.hidden_size)),
            TensorSpec(f"{p}.dkv", (self.row_width, self.hidden_size)),
            TensorSpec(f"{p}.dkv.norm", (self.kv_rank,), role="vector", init="norm"),
            TensorSpec(f"{p}.uk", (self.num_heads * self.head_dim, self.kv_rank)),
            TensorSpec(f"{p}.uv", (self.num_heads * self.value_dim, self.kv_rank)),
            TensorSpec(f"{p}.o", (self.hidden_size, self.num_heads * self.value_dim)),
        ] + ([TensorSpec(f"{p}.sink", (self.num_heads,), role="vector", init="normal")] if self.has_sink else [])

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        p = self.prefix
        self.w_in = torch.cat([tensors[f"{p}.q"], tensors[f"{p}.dkv"]], dim=0).contiguous()
        self.latent_norm = tensors[f"{p}.dkv.norm"].contiguous()
        self.w_absorb = tensors[f"{p}.uk"].view(self.num_heads, self.head_dim, self.kv_rank).transpose(1, 2).contiguous()
        self.w_up_v = tensors[f"{p}.uv"].view(self.num_heads, self.value_dim, self.kv_rank).contiguous()
        self.w_o = tensors[f"{p}.o"].contiguous()
        if self.has_sink:
            self.sinks = tensors[f"{p}.sink"].float().contiguous()  # they enter the softmax, which is 32-bit

    def bytes_streamed(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.w_in, self.latent_norm, self.w_absorb, self.w_up_v, self.w_o))

    def cache_specs(self) -> tuple[Any, ...]:
        # one "head" of kv_rank columns a position and no value rows of their own
        return (PagedKVSpec(1, self.row_width, self.window, v_head_dim=0),)

    HEADS_PER_CALL = 16  # the tensor-core attention kernels take up to 16 query heads a key/value head

    def _tensor_cores(self) -> bool:
        return (self.dtype == torch.bfloat16 and kernels.attention_mma_supported(self.row_width, min(self.num_heads, self.HEADS_PER_CALL), 1)
                and (not self.has_sink or kernels.ATTENTION_MMA_SINKS))

    def query_tile_sizes(self) -> tuple[int, ...]:
        if not self._tensor_cores():
            return ()
        wide = kernels.attention_prefill_wide_tile_rows(self.row_width)
        return (kernels.attention_prefill_tile_rows(self.row_width),) + ((wide,) if wide else ())

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: CacheView) -> torch.Tensor:
        tokens = x.shape[0]
        ws = ctx.workspace
        heads, rank, width = self.num_heads, self.kv_rank, self.row_width
        packed = ws.buffer("latent.packed", tokens, self.q_size + width, self.dtype)
        kernels.linear(x, self.w_in, None, packed)
        # a query row a head: [the query carried into the latent space | its rotated part], as wide as a cached row
        q_latent = ws.buffer("latent.q", tokens, heads * width, self.dtype)
        if cache.writes or self.rot_dim:
            rotary = {}
            if self.rot_dim:
                cos, sin = self.position.rotary_tables()
                rotary = dict(rot_dim=self.rot_dim, cos=cos, sin=sin, interleaved=self.rotary_interleaved, q_out=q_latent,
                              num_heads=heads, q_head_width=self.q_head_width)
            kernels.latent_norm_write(
                packed, self.q_size, rank, self.latent_norm, self.norm_eps, cache.k if cache.writes else None,
                positions=ctx.positions, row_ids=ctx.row_ids, block_table=ctx.block_tables[cache.group] if cache.writes else None,
                write_from=ctx.write_from, flag=ctx.error_flag, **rotary,
            )
        queries = packed[:, : self.q_size].unflatten(1, (heads, self.q_head_width))[:, :, : self.head_dim]
        kernels.heads_linear(queries, self.w_absorb, q_latent.view(tokens, heads, width)[:, :, :rank])
        mixed = ws.buffer("latent.mixed", tokens, heads * width, self.dtype)
        rows = CacheView(k=cache.k, v=cache.k, page_size=cache.page_size, group=cache.group, writes=False)
        # all heads read the same rows; more heads than a kernel takes go in several calls over column ranges
        per_call = self.HEADS_PER_CALL if self._tensor_cores() else heads
        for first in range(0, heads, per_call):
            count = min(per_call, heads - first)
            columns = slice(first * width, (first + count) * width)
            run_paged_attention(q_latent[:, columns], mixed[:, columns], rows, ctx, num_q_heads=count, num_kv_heads=1, head_dim=width,
                                scale=self.scale, window=self.window or 0, value_dim=rank,
                                sinks=self.sinks[first : first + count] if self.sinks is not None else None)
        values = ws.buffer("latent.values", tokens, heads * self.value_dim, self.dtype)
        kernels.heads_linear(mixed.view(tokens, heads, width)[:, :, :rank], self.w_up_v, values.view(tokens, heads, self.value_dim))
        out = ws.buffer("latent.out", tokens, self.hidden_size, self.dtype)
        kernels.linear(values, self.w_o, None, out)
        return out
