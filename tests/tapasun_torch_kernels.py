"""Plain torch statements of the kernels that Tapasun's parts call beyond those of ``torch_kernels``,
``makilorn_torch_kernels``, ``karesun_torch_kernels`` and ``mapalorn_torch_kernels``, with the signatures of
``kairyu_b200.kernels``, for CPU runs of the cache manager, the step function, the scheduler and the command line
(32-bit only).  ``install`` puts them all in place of the kernels for one test.  They are test code: the package has no
implementation but its kernels."""

from __future__ import annotations

import torch

import mapalorn_torch_kernels
from mapalorn_torch_kernels import _place, _turn


def sandwich_norm(residual, pending, weight, eps, out, *, rows=None):
    picked = rows.long() if rows is not None else slice(None)
    total = residual[picked]
    if pending is not None:
        y = pending.values[picked].float()
        total = total + y * torch.rsqrt(y.pow(2).mean(-1, keepdim=True) + pending.eps) * pending.weight.float()
        if rows is None:
            residual.copy_(total)
    if out is not None:
        normed = total * torch.rsqrt(total.pow(2).mean(-1, keepdim=True) + eps) * weight.float()
        out[: normed.shape[0]].copy_(normed.to(out.dtype))


def projection_norm_rope_write(packed, *, num_q_heads, num_kv_heads, head_dim, value_dim, k_offset, v_offset, positions, row_ids,
                               q_norm_weight=None, k_norm_weight=None, eps=0.0, cos=None, sin=None, interleaved=False, block_table=None,
                               write_from=None, k_cache=None, v_cache=None, flag=None, per_head_norm=False, v_cos=None, v_sin=None):
    q_size, k_size, v_size = num_q_heads * head_dim, num_kv_heads * head_dim, num_kv_heads * value_dim
    for t in range(packed.shape[0]):
        position, row = int(positions[t]), int(row_ids[t])
        q = packed[t, :q_size].float().view(num_q_heads, head_dim).clone()
        k = packed[t, k_offset : k_offset + k_size].float().view(num_kv_heads, head_dim).clone()
        if q_norm_weight is not None and per_head_norm:
            q = q * torch.rsqrt(q.pow(2).mean(-1, keepdim=True) + eps) * q_norm_weight.float()
            k = k * torch.rsqrt(k.pow(2).mean(-1, keepdim=True) + eps) * k_norm_weight.float()
        elif q_norm_weight is not None:
            q = (q.reshape(-1) * torch.rsqrt(q.pow(2).mean() + eps) * q_norm_weight.float()).view(num_q_heads, head_dim)
            k = (k.reshape(-1) * torch.rsqrt(k.pow(2).mean() + eps) * k_norm_weight.float()).view(num_kv_heads, head_dim)
        if cos is not None:
            for h in range(num_q_heads):
                q[h] = _turn(q[h], cos[position], sin[position], interleaved)
            for h in range(num_kv_heads):
                k[h] = _turn(k[h], cos[position], sin[position], interleaved)
        packed[t, :q_size] = q.reshape(-1).to(packed.dtype)
        if k_cache is not None:
            place = _place(k_cache, block_table, write_from, row, position)
            if place is not None:
                v = packed[t, v_offset : v_offset + v_size].float().view(num_kv_heads, value_dim).clone()
                if v_cos is not None:
                    for h in range(num_kv_heads):
                        v[h] = _turn(v[h], v_cos[position], v_sin[position], interleaved)
                k_cache[place[0], place[1]] = k.to(k_cache.dtype)
                v_cache[place[0], place[1]] = v.to(v_cache.dtype)


def rotate_heads(x, *, heads, head_dim, cos, sin, positions, interleaved=False, inverse=False, flag=None):
    for t in range(x.shape[0]):
        position = int(positions[t])
        for h in range(heads):
            head = x[t, h * head_dim : (h + 1) * head_dim].float()
            x[t, h * head_dim : (h + 1) * head_dim] = _turn(head, cos[position], -sin[position] if inverse else sin[position], interleaved).to(x.dtype)


def scaled_sum(a, scale_a, b, scale_b, out):
    out.copy_((scale_a * a.float() + scale_b * b.float()).to(out.dtype))


def _convolve(inputs_of_row, taps, conv_state, qo_indptr, state_slots, tokens, bias=None):
    """Causal convolution of each row's portion, reaching into its kept inputs, which are then replaced."""
    n = taps.shape[1]
    conv = torch.zeros(tokens, taps.shape[0])
    for row in range(qo_indptr.numel() - 1):
        t0, t1 = int(qo_indptr[row]), int(qo_indptr[row + 1])
        slot = int(state_slots[row])
        inputs = inputs_of_row(t0, t1)
        if n > 1:
            history = torch.cat([conv_state[slot], inputs], dim=0)
            conv_state[slot] = history[-(n - 1) :]
        else:
            history = inputs
        for index in range(t1 - t0):
            conv[t0 + index] = (history[index : index + n] * taps.t()).sum(0)
    if bias is not None:
        conv = conv + bias
    return conv / (1.0 + torch.exp(-conv))


def delta_prepare(packed, gates, taps, conv_state, *, row_ids, qo_indptr, state_slots, a_log, dt_bias, kv_heads, dim, heads, vdim,
                  q, k, v, beta, decay, flag=None, channel_a=None):
    channels = 2 * kv_heads * dim + heads * vdim
    tokens = packed.shape[0]
    act = _convolve(lambda t0, t1: packed[t0:t1, :channels].float(), taps, conv_state, qo_indptr, state_slots, tokens)
    qk = kv_heads * dim
    qh = act[:, :qk].view(tokens, kv_heads, dim)
    kh = act[:, qk : 2 * qk].view(tokens, kv_heads, dim)
    q.view(tokens, kv_heads, dim).copy_(qh * torch.rsqrt(qh.pow(2).sum(-1, keepdim=True) + 1e-6) * dim ** -0.5)
    k.view(tokens, kv_heads, dim).copy_(kh * torch.rsqrt(kh.pow(2).sum(-1, keepdim=True) + 1e-6))
    v.view(tokens, heads * vdim).copy_(act[:, 2 * qk :])
    beta.copy_(torch.sigmoid(gates[:, :heads]))
    if channel_a is None:
        decay.copy_(torch.exp(-torch.exp(a_log) * torch.nn.functional.softplus(gates[:, heads:] + dt_bias)))
    else:
        rate = torch.exp(a_log).repeat_interleave(dim)
        decay.copy_(torch.exp(-rate * torch.nn.functional.softplus(channel_a + dt_bias)))


def _recurrence(q, k, v, beta, decay, states, out, qo_indptr, state_slots, kv_heads, dim, heads, vdim, channel, delta):
    tokens = q.shape[0]
    q, k = q.view(tokens, kv_heads, dim), k.view(tokens, kv_heads, dim)
    v, out = v.view(tokens, heads, vdim), out.view(tokens, heads, vdim)
    decay = decay.view(tokens, heads, dim) if channel else decay.view(tokens, heads)
    for row in range(qo_indptr.numel() - 1):
        slot = int(state_slots[row])
        for h in range(heads):
            S = states[slot, h].t().clone()  # stored column by column: [vdim, dim]
            for t in range(int(qo_indptr[row]), int(qo_indptr[row + 1])):
                kt, qt = k[t, h // (heads // kv_heads)], q[t, h // (heads // kv_heads)]
                S = decay[t, h][:, None] * S if channel else decay[t, h] * S
                u = beta[t, h] * (v[t, h] - S.t() @ kt) if delta else beta[t, h] * v[t, h]
                S = S + torch.outer(kt, u)
                out[t, h] = S.t() @ qt
            states[slot, h] = S.t()


def delta_recurrence(q, k, v, beta, decay, states, out, *, qo_indptr, state_slots, kv_heads, dim, heads, vdim, channel_decay=False):
    _recurrence(q, k, v, beta, decay, states, out, qo_indptr, state_slots, kv_heads, dim, heads, vdim, channel_decay, True)


def delta_gated_norm(o, packed, gate_offset, weight, eps, out, *, heads, vdim, gate_activation="silu"):
    tokens = packed.shape[0]
    o = o.view(tokens, heads, vdim)
    gate = packed[:, gate_offset : gate_offset + heads * vdim].float().view(tokens, heads, vdim)
    factor = torch.sigmoid(gate) if gate_activation == "sigmoid" else gate * torch.sigmoid(gate)
    normed = o * torch.rsqrt(o.pow(2).mean(-1, keepdim=True) + eps) * weight * factor
    out.copy_(normed.reshape(tokens, heads * vdim).to(out.dtype))


def ssm_prepare(packed, dt_raw, taps, conv_bias, conv_state, *, row_ids, qo_indptr, state_slots, a_log, dt_bias, groups, state, heads, vdim,
                x, b, c, dt, decay, flag=None):
    inner, gn = heads * vdim, groups * state
    tokens = packed.shape[0]
    act = _convolve(lambda t0, t1: packed[t0:t1, : inner + 2 * gn].float(), taps, conv_state, qo_indptr, state_slots, tokens, conv_bias)
    x.view(tokens, inner).copy_(act[:, :inner])
    b.view(tokens, gn).copy_(act[:, inner : inner + gn])
    c.view(tokens, gn).copy_(act[:, inner + gn :])
    dt.copy_(torch.nn.functional.softplus(dt_raw + dt_bias))
    decay.copy_(torch.exp(-torch.exp(a_log) * dt))


def ssm_recurrence(c, b, x, dt, decay, states, out, *, qo_indptr, state_slots, groups, state, heads, vdim):
    _recurrence(c, b, x, dt, decay, states, out, qo_indptr, state_slots, groups, state, heads, vdim, False, False)


def ssm_gated_norm(y, x, skip, z, weight, eps, out, *, heads, vdim, norm_groups):
    tokens, inner = out.shape
    value = (y.view(tokens, heads, vdim) + skip[None, :, None] * x.view(tokens, heads, vdim)).reshape(tokens, inner)
    zf = z.float()
    value = (value * zf * torch.sigmoid(zf)).view(tokens, norm_groups, inner // norm_groups)
    normed = value * torch.rsqrt(value.pow(2).mean(-1, keepdim=True) + eps)
    out.copy_((normed.reshape(tokens, inner) * weight).to(out.dtype))


_NAMES = [
    "sandwich_norm", "projection_norm_rope_write", "rotate_heads", "scaled_sum", "delta_prepare", "delta_recurrence", "delta_gated_norm",
    "ssm_prepare", "ssm_recurrence", "ssm_gated_norm",
]


def install(monkeypatch) -> None:
    import kairyu_b200.kernels as kernels

    mapalorn_torch_kernels.install(monkeypatch)
    for name in _NAMES:
        monkeypatch.setattr(kernels, name, globals()[name])
