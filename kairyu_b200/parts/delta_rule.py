"""The gated delta rule as a mixer: linear attention whose memory is a matrix per head.

Per head and request a state ``S`` [dim, vdim] (fp32) is carried from token to token::

    S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q

``q, k`` (``num_kv_heads`` heads of ``head_dim``) and ``v`` (``num_heads`` heads of ``value_dim``) are
projections followed by a causal convolution over time per channel (``conv_taps`` taps) and silu;
q and k are unit vectors per head, q also times ``head_dim^-1/2``; ``beta = sigmoid(W_b x)`` and
``g = exp(-exp(A_log) * softplus(W_a x + dt_bias))`` per head.  The read-out is normed per head
(RMS over ``value_dim``, one weight shared by the heads), gated by ``silu(W_g x)`` and projected.
What a request keeps between steps is S and the convolution's last ``conv_taps - 1`` inputs: two
per-request state tensors, no pages.  The kernels are in ``csrc/delta_rule.cu``.

Options.  ``decay="channel"`` with ``decay_rank``: one decay a head AND key channel,
``g = exp(-exp(A_log_h) * softplus(W_a2 (W_a1 x) + dt_bias))`` laid out heads x head_dim (tensors ``a1`` [rank, hidden],
``a2`` [heads * head_dim, rank], ``dt_bias`` [heads * head_dim]); g then scales the rows of S that belong to key
channels.  ``gate_rank``: the output gate's projection in two steps, ``W_g2 (W_g1 x)`` (tensors ``g1``, ``g2``) in place
of ``g``.  ``gate_activation``: ``silu`` or ``sigmoid``.
"""

from __future__ import annotations

from typing import Any, Mapping, Optional

import torch

from kairyu_b200 import kernels
from kairyu_b200.parts.base import MIXERS, CacheView, Mixer, StateSpec, StepContext, TensorSpec


@MIXERS.register("gated_delta")
class GatedDeltaRule(Mixer):
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
        conv_taps: int,
        norm_eps: float,
        dtype: torch.dtype,
        device: str,
        decay: str = "head",
        decay_rank: Optional[int] = None,
        gate_rank: Optional[int] = None,
        gate_activation: str = "silu",
        **_: object,
    ) -> None:
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} heads are not a multiple of {num_kv_heads} query/key heads")
        if decay not in ("head", "channel") or (decay == "channel") != (decay_rank is not None):
            raise ValueError("decay is 'head', or 'channel' with a decay_rank")
        if gate_activation not in ("silu", "sigmoid"):
            raise ValueError(f"unknown gate activation {gate_activation!r} (silu, sigmoid)")
        self.channel_decay = decay == "channel"
        self.decay_rank = decay_rank or 0
        self.gate_rank = gate_rank or 0
        self.gate_activation = gate_activation
        self.prefix = prefix
        self.hidden_size = hidden_size
        self.num_heads = num_heads
        self.num_kv_heads = num_kv_heads
        self.head_dim = head_dim
        self.value_dim = value_dim
        self.conv_taps = conv_taps
        self.norm_eps = float(norm_eps)
        self.dtype = dtype
        self.qk_size = num_kv_heads * head_dim
        self.v_size = num_heads * value_dim
        self.channels = 2 * self.qk_size + self.v_size  # what the convolution runs over
        # the packed product's columns: q | k | v, then the gate's rows (full rank) or the first steps of the two-step products
        self.a1_offset = self.channels + (0 if self.gate_rank else self.v_size)
        self.g1_offset = self.a1_offset + self.decay_rank
        self.packed_width = self.g1_offset + self.gate_rank
        self.w_in: Optional[torch.Tensor] = None     # [q | k | v | gate or (a1 | g1) rows, hidden]
        self.w_gates: Optional[torch.Tensor] = None  # [b | a rows, hidden]; b alone with a decay a channel
        self.w_a2: Optional[torch.Tensor] = None
        self.w_g2: Optional[torch.Tensor] = None
        self.taps: Optional[torch.Tensor] = None     # [channels, taps] fp32
        self.a_log: Optional[torch.Tensor] = None
        self.dt_bias: Optional[torch.Tensor] = None
        self.out_norm: Optional[torch.Tensor] = None
        self.w_o: Optional[torch.Tensor] = None

    def tensor_specs(self) -> list[TensorSpec]:
        p, h = self.prefix, self.hidden_size
        specs = [
            TensorSpec(f"{p}.q", (self.qk_size, h)),
            TensorSpec(f"{p}.q.conv", (self.qk_size, self.conv_taps), role="vector", init="taps"),
            TensorSpec(f"{p}.k", (self.qk_size, h)),
            TensorSpec(f"{p}.k.conv", (self.qk_size, self.conv_taps), role="vector", init="taps"),
            TensorSpec(f"{p}.v", (self.v_size, h)),
            TensorSpec(f"{p}.v.conv", (self.v_size, self.conv_taps), role="vector", init="taps"),
            TensorSpec(f"{p}.b", (self.num_heads, h)),
            TensorSpec(f"{p}.A_log", (self.num_heads,), role="vector", init="normal"),
            TensorSpec(f"{p}.norm", (self.value_dim,), role="vector", init="norm"),
        ]
        if self.channel_decay:
            specs += [
                TensorSpec(f"{p}.a1", (self.decay_rank, h)),
                TensorSpec(f"{p}.a2", (self.num_heads * self.head_dim, self.decay_rank)),
                TensorSpec(f"{p}.dt_bias", (self.num_heads * self.head_dim,), role="vector", init="normal"),
            ]
        else:
            specs += [TensorSpec(f"{p}.a", (self.num_heads, h)), TensorSpec(f"{p}.dt_bias", (self.num_heads,), role="vector", init="normal")]
        if self.gate_rank:
            specs += [TensorSpec(f"{p}.g1", (self.gate_rank, h)), TensorSpec(f"{p}.g2", (self.v_size, self.gate_rank))]
        else:
            specs.append(TensorSpec(f"{p}.g", (self.v_size, h)))
        specs.append(TensorSpec(f"{p}.o", (h, self.v_size)))
        return specs

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        p = self.prefix
        names = ["q", "k", "v"] + ([] if self.gate_rank else ["g"]) + (["a1"] if self.channel_decay else []) + (["g1"] if self.gate_rank else [])
        self.w_in = torch.cat([tensors[f"{p}.{name}"] for name in names], dim=0).contiguous()
        self.w_gates = (tensors[f"{p}.b"] if self.channel_decay else torch.cat([tensors[f"{p}.b"], tensors[f"{p}.a"]], dim=0)).contiguous()
        self.w_a2 = tensors[f"{p}.a2"].contiguous() if self.channel_decay else None
        self.w_g2 = tensors[f"{p}.g2"].contiguous() if self.gate_rank else None
        # what enters the recurrence is 32-bit whatever the compute dtype
        self.taps = torch.cat([tensors[f"{p}.{name}.conv"] for name in ("q", "k", "v")], dim=0).float().contiguous()
        self.a_log = tensors[f"{p}.A_log"].float().contiguous()
        self.dt_bias = tensors[f"{p}.dt_bias"].float().contiguous()
        self.out_norm = tensors[f"{p}.norm"].float().contiguous()
        self.w_o = tensors[f"{p}.o"].contiguous()

    def bytes_streamed(self) -> int:
        held = (self.w_in, self.w_gates, self.w_a2, self.w_g2, self.taps, self.a_log, self.dt_bias, self.out_norm, self.w_o)
        return sum(t.numel() * t.element_size() for t in held if t is not None)

    def cache_specs(self) -> tuple[Any, ...]:
        specs = [StateSpec((self.num_heads, self.value_dim, self.head_dim), "float32")]  # S column by column
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
        packed = ws.buffer("delta.packed", tokens, self.packed_width, self.dtype)
        kernels.linear(x, self.w_in, None, packed)
        gates = ws.buffer("delta.gates", tokens, self.w_gates.shape[0], f32)
        kernels.linear(x, self.w_gates, None, gates)
        decays = self.num_heads * (self.head_dim if self.channel_decay else 1)
        channel_a = None
        if self.channel_decay:  # the decay's second step, to 32-bit: it enters the recurrence
            channel_a = ws.buffer("delta.channel_a", tokens, decays, f32)
            kernels.linear(packed[:, self.a1_offset : self.a1_offset + self.decay_rank], self.w_a2, None, channel_a)
        q = ws.buffer("delta.q", tokens, self.qk_size, f32)
        k = ws.buffer("delta.k", tokens, self.qk_size, f32)
        v = ws.buffer("delta.v", tokens, self.v_size, f32)
        beta = ws.buffer("delta.beta", tokens, self.num_heads, f32)
        decay = ws.buffer("delta.decay", tokens, decays, f32)
        sizes = dict(kv_heads=self.num_kv_heads, dim=self.head_dim, heads=self.num_heads, vdim=self.value_dim)
        kernels.delta_prepare(
            packed, gates, self.taps, kept_inputs, row_ids=ctx.row_ids, qo_indptr=ctx.qo_indptr, state_slots=ctx.state_slots,
            a_log=self.a_log, dt_bias=self.dt_bias, q=q, k=k, v=v, beta=beta, decay=decay, flag=ctx.error_flag, channel_a=channel_a, **sizes,
        )
        read_out = ws.buffer("delta.o", tokens, self.v_size, f32)
        kernels.delta_recurrence(q, k, v, beta, decay, memory, read_out, qo_indptr=ctx.qo_indptr, state_slots=ctx.state_slots,
                                 channel_decay=self.channel_decay, **sizes)
        normed = ws.buffer("delta.normed", tokens, self.v_size, self.dtype)
        if self.gate_rank:
            gate = ws.buffer("delta.gate", tokens, self.v_size, self.dtype)
            kernels.linear(packed[:, self.g1_offset : self.g1_offset + self.gate_rank], self.w_g2, None, gate)
            gate_offset = 0
        else:
            gate, gate_offset = packed, self.channels
        kernels.delta_gated_norm(read_out, gate, gate_offset, self.out_norm, self.norm_eps, normed, heads=self.num_heads, vdim=self.value_dim,
                                 gate_activation=self.gate_activation)
        out = ws.buffer("delta.out", tokens, self.hidden_size, self.dtype)
        kernels.linear(normed, self.w_o, None, out)
        return out
