"""Plain torch statements of the kernels that Karesun's parts call beyond those of ``torch_kernels``
and ``makilorn_torch_kernels``, with the signatures of ``kairyu_b200.kernels``, for CPU runs of the cache
manager, the step function, the scheduler and the command line (32-bit only).  ``install`` puts them all in
place of the kernels for one test.  They are test code: the package has no implementation but its kernels."""

from __future__ import annotations

import math

import torch

import makilorn_torch_kernels


def add_positions(table, positions, x, flag=None):
    x.add_(table[positions.long()].float())


def activation(x, out, kind):
    v = x.float()
    if kind == "relu2":
        y = torch.relu(v) ** 2
    elif kind == "gelu_tanh":
        y = 0.5 * v * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (v + 0.044715 * v ** 3)))
    else:
        y = v / (1.0 + torch.exp(-v))
    out.copy_(y.to(out.dtype))


def paged_kv_write(packed, k_offset, v_offset, k_cache, v_cache, *, positions, row_ids, block_table, write_from=None, flag=None):
    page_size = k_cache.shape[1]
    k_width, v_width = k_cache.shape[2] * k_cache.shape[3], v_cache.shape[2] * v_cache.shape[3]
    for t in range(packed.shape[0]):
        position, row = int(positions[t]), int(row_ids[t])
        if write_from is not None and position < int(write_from[row]):
            continue
        page = int(block_table[row, position // page_size])
        assert 0 <= page < k_cache.shape[0]
        k_cache[page, position % page_size] = packed[t, k_offset : k_offset + k_width].view(k_cache.shape[2:])
        v_cache[page, position % page_size] = packed[t, v_offset : v_offset + v_width].view(v_cache.shape[2:])


def diff_attention_generic(q, out, k_cache, v_cache, *, positions, row_ids, block_table, num_q_heads, maps, scale, softcap=0.0, window=0,
                           lam=0.0, head_norm_eps=None, out_scale=1.0, flag=None):
    page_size, kv_heads = k_cache.shape[1], k_cache.shape[2]
    dim, vdim = k_cache.shape[3] // maps, v_cache.shape[3]
    group = num_q_heads // kv_heads
    for t in range(q.shape[0]):
        position, row = int(positions[t]), int(row_ids[t])
        first = max(0, position + 1 - window) if window > 0 else 0
        places = [(int(block_table[row, j // page_size]), j % page_size) for j in range(first, position + 1)]
        assert all(0 <= page < k_cache.shape[0] for page, _ in places)
        keys = torch.stack([k_cache[page, at] for page, at in places]).float()      # [keys, kv_heads, maps * dim]
        values = torch.stack([v_cache[page, at] for page, at in places]).float()    # [keys, kv_heads, vdim]
        for h in range(num_q_heads):
            o = None
            for m in range(maps):
                query = q[t, (h * maps + m) * dim : (h * maps + m + 1) * dim].float()
                s = keys[:, h // group, m * dim : (m + 1) * dim] @ query * scale
                if softcap > 0:
                    s = softcap * torch.tanh(s / softcap)
                a = torch.softmax(s, dim=0) @ values[:, h // group]
                o = a if m == 0 else o - lam * a
            if head_norm_eps is not None:
                o = o * torch.rsqrt((o * o).mean() + head_norm_eps) * out_scale
            out[t, h * vdim : (h + 1) * vdim] = o.to(out.dtype)


def moe_route_scores(logits, correction, top, ids, weights, *, groups=1, keep=1, scale=1.0, score="softmax"):
    outputs = logits.shape[1]
    per = outputs // groups
    for t in range(logits.shape[0]):
        z = logits[t].float()
        s = torch.sigmoid(z) if score == "sigmoid" else torch.softmax(z, dim=0)
        c = s + (correction.float() if correction is not None else 0.0)
        values = [float(c[g * per : (g + 1) * per].max()) for g in range(groups)]
        kept = sorted(range(groups), key=lambda g: (-values[g], g))[:keep]
        allowed = [e for e in range(outputs) if e // per in kept]
        chosen = sorted(allowed, key=lambda e: (-float(c[e]), e))[:top]
        ids[t] = torch.tensor(chosen, dtype=torch.int32)
        weights[t] = s[chosen] * scale


def moe_grouped(a, weight, out, plan, *, top, gated, limit=0.0, alpha=1.702, shift=1.0):
    for place, pair in enumerate(plan["sorted"]):
        expert = plan["experts"][pair]
        if expert >= weight.shape[0]:
            continue  # an identity expert: no weights, the sum takes the token's row
        w = weight[expert].float()
        if gated:
            both = w @ a[pair // top].float()
            half = both.shape[0] // 2
            g = both[:half].clamp(max=limit)
            u = both[half:].clamp(min=-limit, max=limit)
            out[place] = (g * torch.sigmoid(alpha * g) * (u + shift)).to(out.dtype)
        else:
            out[pair] = w @ a[place].float()


def moe_combine(rows, weights, out, at=None, *, ids=None, x=None, experts=0, top=None, extra=None, extra_gate=None):
    tokens = out.shape[0]
    top = weights.shape[1] if weights is not None else top
    picked = rows.float() if at is None else rows.float()[at.long()]
    picked = picked.view(tokens, top, -1).clone()
    if ids is not None:
        for t in range(tokens):
            for k in range(top):
                if int(ids[t, k]) >= experts:
                    picked[t, k] = x[t].float()
    total = (picked * weights.unsqueeze(-1)).sum(1) if weights is not None else picked.sum(1)
    if extra is not None:
        total = total + extra.float() * (torch.sigmoid(extra_gate.float().reshape(tokens, 1)) if extra_gate is not None else 1.0)
    out.copy_(total.to(out.dtype))


_NAMES = ["add_positions", "activation", "paged_kv_write", "diff_attention_generic", "moe_route_scores", "moe_grouped", "moe_combine"]


def install(monkeypatch) -> None:
    import kairyu_b200.kernels as kernels

    makilorn_torch_kernels.install(monkeypatch)
    for name in _NAMES:
        monkeypatch.setattr(kernels, name, globals()[name])
