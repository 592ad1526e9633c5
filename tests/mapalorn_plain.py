"""Mapalorn written out slowly: one function per mechanism, whole sequences, no cache, no batch,
64-bit unless told otherwise.  It shares nothing with the engine; the tests compare the engine with it.

A model is ``(config, tensors)``: the dict of ``config.json`` and a dict name -> tensor.

    layer:   h = LN(x);  x <- x + (mixer(h) + ff(h))          LN(x) = (x - mean) / sqrt(var + eps) * w + b
    loop:    layers start .. stop-1 run `times` times, then the rest
    logits:  head . LN_final(x)
"""

from __future__ import annotations

import math

import torch


def layer_norm(x, w, b, eps):
    mean = x.mean(-1, keepdim=True)
    var = ((x - mean) ** 2).mean(-1, keepdim=True)
    return (x - mean) / torch.sqrt(var + eps) * w + b


def rms_norm(x, w, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


def angles(positions, dims, base):
    """[tokens, dims/2]: position p times base^(-2i/dims)."""
    i = torch.arange(dims // 2, dtype=torch.float64)
    return positions.to(torch.float64)[:, None] * base ** (-2.0 * i / dims)[None, :]


def rotate_interleaved(x, positions, dims, base):
    """x [tokens, heads, d]: the pairs (2i, 2i+1) of the first `dims` columns turn by the angle i."""
    a = angles(positions, dims, base).to(x.dtype)
    cos, sin = a.cos()[:, None, :], a.sin()[:, None, :]
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = u * cos - v * sin
    out[..., 1:dims:2] = v * cos + u * sin
    return out


def rotate_halves(x, positions, dims, base):
    """x [tokens, heads, d]: the pairs (i, i + dims/2) of the first `dims` columns turn by the angle i."""
    a = angles(positions, dims, base).to(x.dtype)
    cos, sin = a.cos()[:, None, :], a.sin()[:, None, :]
    half = dims // 2
    u, v = x[..., :half], x[..., half:dims]
    out = x.clone()
    out[..., :half] = u * cos - v * sin
    out[..., half:dims] = v * cos + u * sin
    return out


def causal_softmax_with_sink(scores, sink):
    """scores [heads, n, n]; sink [heads]: a logit a head that joins the denominator and nothing else."""
    n = scores.shape[-1]
    mask = torch.ones(n, n, dtype=torch.bool).tril()
    scores = scores.masked_fill(~mask, -math.inf)
    top = torch.maximum(scores.max(-1, keepdim=True).values, sink[:, None, None])
    e = torch.exp(scores - top)
    return e / (e.sum(-1, keepdim=True) + torch.exp(sink[:, None, None] - top))


def latent_attention(h, w, m, eps):
    """w: the mixer's tensors by their short names; m: the mixer's entry of the config."""
    n = h.shape[0]
    H, d, r, dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    positions = torch.arange(n)
    q = (h @ w["q"].T).view(n, H, d + r)
    down = h @ w["dkv"].T
    c = rms_norm(down[:, :rank], w["dkv.norm"], eps)
    k_rot = rotate_interleaved(down[:, None, rank:], positions, m["rot"]["dims"], m["rot"]["base"])  # [n, 1, r]
    q_rot = rotate_interleaved(q[..., d:], positions, m["rot"]["dims"], m["rot"]["base"])
    k = (c @ w["uk"].T).view(n, H, d)
    v = (c @ w["uv"].T).view(n, H, dv)
    scores = (torch.einsum("ihd,jhd->hij", q[..., :d], k) + torch.einsum("ihd,jd->hij", q_rot, k_rot[:, 0])) * m["scale"]
    p = causal_softmax_with_sink(scores, w["sink"].to(h.dtype))
    mixed = torch.einsum("hij,jhd->ihd", p, v).reshape(n, H * dv)
    return mixed @ w["o"].T


def gated_attention(h, w, m, eps):
    n = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    positions = torch.arange(n)
    q = rms_norm(h @ w["q"].T, w["q.norm"], eps).view(n, H, d)
    k = rms_norm(h @ w["k"].T, w["k.norm"], eps).view(n, G, d)
    v = (h @ w["v"].T).view(n, G, dv)
    q = rotate_halves(q, positions, m["rot"]["dims"], m["rot"]["base"])
    k = rotate_halves(k, positions, m["rot"]["dims"], m["rot"]["base"])
    k = k.repeat_interleave(H // G, dim=1)
    v = v.repeat_interleave(H // G, dim=1)
    scores = torch.einsum("ihd,jhd->hij", q, k) * m["scale"]
    p = causal_softmax_with_sink(scores, torch.zeros(H, dtype=h.dtype))
    mixed = torch.einsum("hij,jhd->ihd", p, v).reshape(n, H * dv)
    mixed = mixed * torch.sigmoid(h @ w["g"].T)
    return mixed @ w["o"].T


def dense_ff(h, w, limit):
    g = (h @ w["gate"].T).clamp(max=limit)
    u = (h @ w["up"].T).clamp(-limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1)) @ w["down"].T


def silu_expert(h, gate, up, down):
    a = h @ gate.T
    return (a * torch.sigmoid(a) * (h @ up.T)) @ down.T


def expert_mixture(h, w, f):
    """Every token: its `top` experts by sigmoid score (ties to the lower index), each fed w * h; a shared
    expert times one sigmoid gate a token on top, when the layer has one."""
    n = h.shape[0]
    scores = torch.sigmoid(h @ w["router"].T)
    out = torch.zeros_like(h)
    for t in range(n):
        chosen = sorted(range(scores.shape[1]), key=lambda e: (-float(scores[t, e]), e))[: f["router"]["top"]]
        for e in chosen:
            out[t] += silu_expert(scores[t, e] * h[t], w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"])
    if f.get("shared"):
        shared = silu_expert(h, w["shared.gate"], w["shared.up"], w["shared.down"])
        out = out + shared * torch.sigmoid(h @ w["shared.sg"].T)
    return out


def sub(tensors, prefix, dtype):
    cut = len(prefix) + 1
    return {name[cut:]: t.to(dtype) for name, t in tensors.items() if name.startswith(prefix + ".")}


def run_order(config):
    """Layer indices in the order they run."""
    count = len(config["layers"])
    loop = config.get("loop")
    if not loop:
        return list(range(count))
    start, stop, times = loop["start"], loop["stop"], loop["times"]
    return list(range(start)) + list(range(start, stop)) * times + list(range(stop, count))


def forward(config, tensors, tokens, dtype=torch.float64, streams=None):
    """Logits [len(tokens), vocab]; ``streams``, a list, receives the residual stream after every layer run."""
    eps = config["norm"]["eps"]
    x = tensors["embed"].to(dtype)[torch.as_tensor(tokens, dtype=torch.long)]
    for index in run_order(config):
        layer = config["layers"][index]
        p = f"l{index}"
        h = layer_norm(x, tensors[f"{p}.norm1"].to(dtype), tensors[f"{p}.norm1.b"].to(dtype), eps)
        w = sub(tensors, f"{p}.mix", dtype)
        if layer["type"] == "latent_attention":
            y = latent_attention(h, w, layer["mixer"], eps)
        else:
            y = gated_attention(h, w, layer["mixer"], eps)
        f = layer.get("mlp")
        if f is not None:
            w = sub(tensors, f"{p}.mlp", dtype)
            y = y + (dense_ff(h, w, f["limit"]) if f["kind"] == "dense" else expert_mixture(h, w, f))
        x = x + y
        if streams is not None:
            streams.append(x.clone())
    x = layer_norm(x, tensors["final.norm"].to(dtype), tensors["final.norm.b"].to(dtype), eps)
    return x @ tensors["head"].to(dtype).T
