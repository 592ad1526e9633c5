"""Plain torch statements of the kernels that Mapalorn's parts call beyond those of ``torch_kernels``,
``makilorn_torch_kernels`` and ``karesun_torch_kernels``, with the signatures of ``kairyu_b200.kernels``, for CPU runs of
the cache manager, the step function, the scheduler and the command line (32-bit only).  ``install`` puts them all in
place of the kernels for one test.  They are test code: the package has no implementation but its kernels."""

from __future__ import annotations

import torch

import karesun_torch_kernels


def layernorm(x, weight, bias, eps, out, *, delta=None, delta2=None, rows=None):
    total = x
    if rows is None:
        for pending in (delta, delta2):
            if pending is not None:
                x.add_(pending.float())
    else:
        picked = rows.long()
        total = x[picked]
        for pending in (delta, delta2):
            if pending is not None:
                total = total + pending[picked].float()
    mean = total.mean(-1, keepdim=True)
    centred = total - mean
    y = centred * torch.rsqrt(centred.pow(2).mean(-1, keepdim=True) + eps) * weight.float() + bias.float()
    out[: y.shape[0]].copy_(y.to(out.dtype))


def _turn(vector, cos, sin, interleaved):
    """The first 2 * len(cos) entries of ``vector`` turned; the rest as they are."""
    half = cos.numel()
    out = vector.clone()
    if interleaved:
        u, v = vector[0 : 2 * half : 2], vector[1 : 2 * half : 2]
        out[0 : 2 * half : 2] = u * cos - v * sin
        out[1 : 2 * half : 2] = v * cos + u * sin
    else:
        u, v = vector[:half], vector[half : 2 * half]
        out[:half] = u * cos - v * sin
        out[half : 2 * half] = v * cos + u * sin
    return out


def _place(cache, block_table, write_from, row, position):
    """(page, offset) the token's row goes to, or None when its position lies in pages the request only reads."""
    if write_from is not None and position < int(write_from[row]):
        return None
    page_size = cache.shape[1]
    page = int(block_table[row, position // page_size])
    assert 0 <= page < cache.shape[0]
    return page, position % page_size


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


def latent_norm_write(packed, offset, rank, weight, eps, cache, *, positions, row_ids, block_table, write_from, flag=None, rot_dim=0,
                      cos=None, sin=None, interleaved=True, q_out=None, num_heads=0, q_head_width=0):
    z = packed[:, offset : offset + rank].float()
    c = z * torch.rsqrt(z.pow(2).mean(-1, keepdim=True) + eps) * weight.float()
    width = rank + rot_dim
    for t in range(packed.shape[0]):
        position, row = int(positions[t]), int(row_ids[t])
        stored = c[t]
        if rot_dim:
            key_part = _turn(packed[t, offset + rank : offset + width].float(), cos[position], sin[position], interleaved)
            stored = torch.cat([c[t], key_part])
            if q_out is not None:
                for h in range(num_heads):
                    first = h * q_head_width + q_head_width - rot_dim
                    q_out[t, h * width + rank : (h + 1) * width] = _turn(
                        packed[t, first : first + rot_dim].float(), cos[position], sin[position], interleaved
                    ).to(q_out.dtype)
        if cache is not None:
            place = _place(cache, block_table, write_from, row, position)
            if place is not None:
                cache[place[0], place[1], 0] = stored.to(cache.dtype)


def _visible(cache, block_table, row, position, window):
    page_size = cache.shape[1]
    first = max(0, position + 1 - window) if window > 0 else 0
    places = [(int(block_table[row, j // page_size]), j % page_size) for j in range(first, position + 1)]
    assert all(0 <= page < cache.shape[0] for page, _ in places)
    return places


def _softmax_with_sink(scores, sink):
    if sink is None:
        return torch.softmax(scores, dim=0)
    top = torch.maximum(scores.max(), sink)
    e = torch.exp(scores - top)
    return e / (e.sum() + torch.exp(sink - top))


def paged_attention_generic(q, out, k_cache, v_cache, *, positions, row_ids, block_table, num_q_heads, scale, window=0, flag=None, sinks=None,
                            value_dim=None, out_head_stride=None):
    kv_heads, dim = k_cache.shape[2], k_cache.shape[3]
    value_dim = dim if value_dim is None else value_dim
    stride = value_dim if out_head_stride is None else out_head_stride
    group = num_q_heads // kv_heads
    for t in range(q.shape[0]):
        places = _visible(k_cache, block_table, int(row_ids[t]), int(positions[t]), window)
        keys = torch.stack([k_cache[page, at] for page, at in places]).float()
        values = torch.stack([v_cache[page, at] for page, at in places]).float()[..., :value_dim]
        for h in range(num_q_heads):
            s = keys[:, h // group] @ q[t, h * dim : (h + 1) * dim].float() * scale
            p = _softmax_with_sink(s, sinks[h] if sinks is not None else None)
            out[t, h * stride : h * stride + value_dim] = (p @ values[:, h // group]).to(out.dtype)


def diff_attention_generic(q, out, k_cache, v_cache, *, positions, row_ids, block_table, num_q_heads, maps, scale, softcap=0.0, window=0,
                           lam=0.0, head_norm_eps=None, out_scale=1.0, flag=None, sinks=None, gate=None):
    kv_heads = k_cache.shape[2]
    dim, vdim = k_cache.shape[3] // maps, v_cache.shape[3]
    group = num_q_heads // kv_heads
    for t in range(q.shape[0]):
        places = _visible(k_cache, block_table, int(row_ids[t]), int(positions[t]), window)
        keys = torch.stack([k_cache[page, at] for page, at in places]).float()
        values = torch.stack([v_cache[page, at] for page, at in places]).float()
        for h in range(num_q_heads):
            o = None
            for m in range(maps):
                query = q[t, (h * maps + m) * dim : (h * maps + m + 1) * dim].float()
                s = keys[:, h // group, m * dim : (m + 1) * dim] @ query * scale
                if softcap > 0:
                    s = softcap * torch.tanh(s / softcap)
                a = _softmax_with_sink(s, sinks[h] if sinks is not None else None) @ values[:, h // group]
                o = a if m == 0 else o - lam * a
            if head_norm_eps is not None:
                o = o * torch.rsqrt((o * o).mean() + head_norm_eps) * out_scale
            if gate is not None:
                o = o * torch.sigmoid(gate[t, h * vdim : (h + 1) * vdim].float())
            out[t, h * vdim : (h + 1) * vdim] = o.to(out.dtype)


def moe_scale_rows(src, scale, out, *, rows=None, per=1, index=None):
    for i in range(out.shape[0]):
        source = int(rows[i]) if rows is not None else i // per
        weight = scale[int(index[i])] if index is not None else scale[i]
        out[i] = (src[source].float() * weight).to(out.dtype)


def moe_activation(gate_up, out, *, limit, alpha=1.702, shift=1.0):
    half = gate_up.shape[1] // 2
    g = gate_up[:, :half].float().clamp(max=limit)
    u = gate_up[:, half:].float().clamp(min=-limit, max=limit)
    out.copy_((g * torch.sigmoid(alpha * g) * (u + shift)).to(out.dtype))


_NAMES = [
    "layernorm", "projection_norm_rope_write", "latent_norm_write", "paged_attention_generic", "diff_attention_generic", "moe_scale_rows", "moe_activation",
]


def install(monkeypatch) -> None:
    import kairyu_b200.kernels as kernels

    karesun_torch_kernels.install(monkeypatch)
    for name in _NAMES:
        monkeypatch.setattr(kernels, name, globals()[name])
