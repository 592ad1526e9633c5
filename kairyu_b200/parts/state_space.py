"""A selective state-space mixer in its state-space-duality form (the layer usually called Mamba-2).

One product gives ``z | x | B | C`` and a second, with 32-bit output, the step sizes ``dt`` (one a head);
``inner = num_heads * value_dim``, ``B`` and ``C`` are ``groups`` rows of ``state_size`` each, and head h uses group
``h // (num_heads / groups)``.  ``x | B | C`` pass a causal convolution over time per channel (``conv_taps`` taps, the
last one the current token's, zeros before the start, with a bias) and silu.  Per head a state ``S`` [state_size,
value_dim] (fp32) is carried from token to token::

    dt <- softplus(dt + dt_bias)
    S  <- exp(-exp(A_log_h) dt) S + dt B x^T
    y   = S^T C + D_h x

``y`` (heads side by side) is multiplied by ``silu(z)``, then RMS-normed in ``norm_groups`` equal parts (each by its own
root mean square), times a weight a column, and projected.  What a request keeps between steps is S and the
convolution's last ``conv_taps - 1`` inputs: two per-request state tensors, no pages.  Everything between the
projections and the output product is 32-bit.  The kernels are in ``csrc/ssm.cu``; the recurrence is the one the
delta rule uses, without the delta (``csrc/linear_recurrence.cuh``).

Tensors under ``prefix``: ``in`` [2 inner + 2 groups state_size + heads, hidden], ``conv`` [inner + 2 groups state_size,
taps], ``conv.b``, ``dt_bias``, ``A_log``, ``D`` [heads], ``norm`` [inner], ``o`` [hidden, inner].
"""

from __future__ import annotations

from typing import Any, Mapping, Optional

import torch

from kairyu_b200 import kernels
from kairyu_b200.parts.base import MIXERS, CacheView, Mixer, StateSpec, StepContext, TensorSpec


@MIXERS.register("state_space_dual")
class StateSpaceDual(Mixer):
    graph_safe = True

    def __init__(
        self,
        *,
        prefix: str,
        hidden_size: int,
        num_heads: int,
        value_dim: int,
        state_size: int,
        groups: int,
        norm_groups: int,
        conv_taps: int,
        norm_eps: float,
        dtype: torch.dtype,
        device: str,
        **_: object,
    ) -> None:
        if num_heads % groups:
            raise ValueError(f"{num_heads} heads are not a multiple of {groups} groups")
        if (num_heads * value_dim) % norm_groups:
            raise ValueError(f"{num_heads * value_dim} columns do not split into {norm_groups} equal parts")
        self.prefix = prefix
        self.hidden_size = hidden_size
        self.num_heads = num_heads
        self.value_dim = value_dim
        self.state_size = state_size
        self.groups = groups
        self.norm_groups = norm_groups
        self.conv_taps = conv_taps
        self.norm_eps = float(norm_eps)
        self.dtype = dtype
        self.inner = num_heads * value_dim
        self.channels = self.inner + 2 * groups * state_size  # what the convolution runs over
        self.w_in: Optional[torch.Tensor] = None   # [z | x | B | C rows, hidden]
        self.w_dt: Optional[torch.Tensor] = None   # [heads, hidden]
        self.taps: Optional[torch.Tensor] = None
        self.conv_bias: Optional[torch.Tensor] = None
        self.a_log: Optional[torch.Tensor] = None
        self.dt_bias: Optional[torch.Tensor] = None
        self.skip: Optional[torch.Tensor] = None
        self.out_norm: Optional[torch.Tensor] = None
        self.w_o: Optional[torch.Tensor] = None

    def tensor_specs(self) -> list[TensorSpec]:
        p, h = self.prefix, self.hidden_size
        return [
            TensorSpec(f"{p}.in", (self.inner + self.channels + self.num_heads, h)),
            TensorSpec(f"{p}.conv", (self.channels, self.conv_taps), role="vector", init="taps"),
            TensorSpec(f"{p}.conv.b", (self.channels,), role="vector", init="normal"),
            TensorSpec(f"{p}.dt_bias", (self.num_heads,), role="vector", init="normal"),
            TensorSpec(f"{p}.A_log", (self.num_heads,), role="vector", init="normal"),
            TensorSpec(f"{p}.D", (self.num_heads,), role="vector", init="norm"),
            TensorSpec(f"{p}.norm", (self.inner,), role="vector", init="norm"),
            TensorSpec(f"{p}.o", (h, self.inner)),
        ]

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        p = self.prefix
        w = tensors[f"{p}.in"]
        self.w_in = w[: self.inner + self.channels].contiguous()
        self.w_dt = w[self.inner + self.channels :].contiguous()
        # what enters the recurrence is 32-bit whatever the compute dtype
        self.taps = tensors[f"{p}.conv"].float().contiguous()
        self.conv_bias = tensors[f"{p}.conv.b"].float().contiguous()
        self.a_log = tensors[f"{p}.A_log"].float().contiguous()
        self.dt_bias = tensors[f"{p}.dt_bias"].float().contiguous()
        self.skip = tensors[f"{p}.D"].float().contiguous()
        self.out_norm = tensors[f"{p}.norm"].float().contiguous()
        self.w_o = tensors[f"{p}.o"].contiguous()

    def bytes_streamed(self) -> int:
        held = (self.w_in, self.w_dt, self.taps, self.conv_bias, self.a_log, self.dt_bias, self.skip, self.out_norm, self.w_o)
        return sum(t.numel() * t.element_size() for t in held)

    def cache_specs(self) -> tuple[Any, ...]:
        specs = [StateSpec((self.num_heads, self.value_dim, self.state_size), "float32")]  # S column by column
        if self.conv_taps > 1:
            specs.append(StateSpec((self.conv_taps - 1, self.channels), "float32"))
        return tuple(specs)

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: CacheView) -> torch.Tensor:
        tokens = x.shape[0]
        ws = ctx.workspace
        f32 = torch.float32
        states = cache.state if isinstance(cache.state, (list, tuple)) else [cache.state]
        memory = states[0]
        kept_inputs = states[1] if self.conv_taps > 1 else None
        packed = ws.buffer("ssm.packed", tokens, self.inner + self.channels, self.dtype)
        kernels.linear(x, self.w_in, None, packed)
        dt_raw = ws.buffer("ssm.dt_raw", tokens, self.num_heads, f32)
        kernels.linear(x, self.w_dt, None, dt_raw)
        xs = ws.buffer("ssm.x", tokens, self.inner, f32)
        b = ws.buffer("ssm.b", tokens, self.groups * self.state_size, f32)
        c = ws.buffer("ssm.c", tokens, self.groups * self.state_size, f32)
        dt = ws.buffer("ssm.dt", tokens, self.num_heads, f32)
        decay = ws.buffer("ssm.decay", tokens, self.num_heads, f32)
        sizes = dict(groups=self.groups, state=self.state_size, heads=self.num_heads, vdim=self.value_dim)
        kernels.ssm_prepare(
            packed[:, self.inner :], dt_raw, self.taps, self.conv_bias, kept_inputs, row_ids=ctx.row_ids, qo_indptr=ctx.qo_indptr,
            state_slots=ctx.state_slots, a_log=self.a_log, dt_bias=self.dt_bias, x=xs, b=b, c=c, dt=dt, decay=decay, flag=ctx.error_flag, **sizes,
        )
        read_out = ws.buffer("ssm.y", tokens, self.inner, f32)
        kernels.ssm_recurrence(c, b, xs, dt, decay, memory, read_out, qo_indptr=ctx.qo_indptr, state_slots=ctx.state_slots, **sizes)
        normed = ws.buffer("ssm.normed", tokens, self.inner, self.dtype)
        kernels.ssm_gated_norm(read_out, xs, self.skip, packed[:, : self.inner], self.out_norm, self.norm_eps, normed,
                               heads=self.num_heads, vdim=self.value_dim, norm_groups=self.norm_groups)
        out = ws.buffer("ssm.out", tokens, self.hidden_size, self.dtype)
        kernels.linear(normed, self.w_o, None, out)
        return out
