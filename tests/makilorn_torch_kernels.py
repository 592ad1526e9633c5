"""Plain torch statements of the kernels that Makilorn's parts call, with the signatures of
``kairyu_b200.kernels``, for CPU runs of the cache manager, the step function, the scheduler and
the command line (32-bit only).  ``install`` puts them, and those of ``torch_kernels``, in place of
the kernels for one test.  They are test code: the package has no implementation but its kernels."""

from __future__ import annotations

import torch

import torch_kernels


def output_norm_add(residual, y, weight, eps, copy):
    import kairyu_b200.kernels as kernels

    if isinstance(y, kernels.WeightedRows):
        tokens, top = y.weights.shape
        rows = y.rows.float() if y.at is None else y.rows.float()[y.at.long()]
        y = (rows.view(tokens, top, -1) * y.weights.unsqueeze(-1)).sum(1)
    y = y.float()
    residual.add_(y * torch.rsqrt(y.pow(2).mean(-1, keepdim=True) + eps) * weight.float())
    if copy is not None:
        copy.copy_(residual.to(copy.dtype))


def residual_copy(residual, copy):
    copy.copy_(residual.to(copy.dtype))


def latent_norm_write(packed, offset, rank, weight, eps, cache, *, positions, row_ids, block_table, write_from, flag=None):
    z = packed[:, offset : offset + rank].float()
    c = z * torch.rsqrt(z.pow(2).mean(-1, keepdim=True) + eps) * weight.float()
    page_size = cache.shape[1]
    for t in range(packed.shape[0]):
        position, row = int(positions[t]), int(row_ids[t])
        if write_from is not None and position < int(write_from[row]):
            continue
        page = int(block_table[row, position // page_size])
        assert 0 <= page < cache.shape[0]
        cache[page, position % page_size, 0] = c[t].to(cache.dtype)


def heads_linear(x, weight, out):
    out.copy_(torch.einsum("thk,hnk->thn", x.float(), weight.float()).to(out.dtype))


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


def moe_route(logits, bias, top, ids, weights):
    z = logits + (bias.float() if bias is not None else 0.0)
    for t in range(z.shape[0]):
        chosen = sorted(range(z.shape[1]), key=lambda e: (-float(z[t, e]), e))[:top]
        ids[t] = torch.tensor(chosen, dtype=torch.int32)
        weights[t] = torch.softmax(z[t, chosen], dim=0)


def moe_plan(ids, experts, plan):
    top = ids.shape[1]
    flat = ids.reshape(-1).tolist()
    order = sorted(range(len(flat)), key=lambda p: (flat[p], p))
    return {"sorted": order, "experts": flat, "top": top}


def moe_grouped(a, weight, out, plan, *, top, gated, limit=0.0, alpha=1.702, shift=1.0):
    for place, pair in enumerate(plan["sorted"]):
        w = weight[plan["experts"][pair]].float()
        if gated:
            both = w @ a[pair // top].float()
            half = both.shape[0] // 2
            g = both[:half].clamp(max=limit)
            u = both[half:].clamp(min=-limit, max=limit)
            out[place] = (g * torch.sigmoid(alpha * g) * (u + shift)).to(out.dtype)
        else:
            out[pair] = w @ a[place].float()


def moe_combine(rows, weights, out, at=None):
    tokens, top = weights.shape
    picked = rows.float() if at is None else rows.float()[at.long()]
    out.copy_((picked.view(tokens, top, -1) * weights.unsqueeze(-1)).sum(1).to(out.dtype))


_NAMES = [
    "output_norm_add", "residual_copy", "latent_norm_write", "heads_linear", "delta_prepare", "delta_recurrence", "delta_gated_norm",
    "moe_route", "moe_plan", "moe_grouped", "moe_combine",
]


def install(monkeypatch) -> None:
    import kairyu_b200.kernels as kernels

    torch_kernels.install(monkeypatch)
    for name in _NAMES:
        monkeypatch.setattr(kernels, name, globals()[name])
