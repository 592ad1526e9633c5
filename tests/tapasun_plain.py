"""Tapasun written out slowly: 64-bit, whole sequences, no cache, no batch, one function a mechanism.

It shares nothing with the engine: the tests compare the engine's logits with these.  Notation: T tokens, positions
0 .. T - 1; a matrix W is stored [out, in] and applied as x @ W.T.
"""

from __future__ import annotations

import math
from typing import Any, Mapping, Optional

import torch

F = torch.float64


def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x divided by its root mean square over the last axis, eps inside the root."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def scalar_norm(x: torch.Tensor, g: torch.Tensor, eps: float) -> torch.Tensor:
    return unit_rms(x, eps) * g.reshape(())


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def softplus(z: torch.Tensor) -> torch.Tensor:
    return torch.where(z > 40.0, z, torch.log1p(torch.exp(torch.clamp(z, max=40.0))))


def frequencies(rot: Mapping[str, Any]) -> torch.Tensor:
    """f_i = base^(-2i/dims), then the scaling the table names."""
    dims = rot["dims"]
    plain = [rot["base"] ** (-2.0 * i / dims) for i in range(dims // 2)]
    scaling = rot.get("scaling")
    if not scaling:
        return torch.tensor(plain, dtype=F)
    if "original" not in scaling:
        return torch.tensor([f / scaling["factor"] for f in plain], dtype=F)
    out = []
    for f in plain:
        wavelength = 2.0 * math.pi / f
        if wavelength < scaling["original"] / scaling["high"]:
            out.append(f)
        elif wavelength > scaling["original"] / scaling["low"]:
            out.append(f / scaling["factor"])
        else:
            s = (scaling["original"] / wavelength - scaling["low"]) / (scaling["high"] - scaling["low"])
            out.append((1.0 - s) * f / scaling["factor"] + s * f)
    return torch.tensor(out, dtype=F)


def turn(x: torch.Tensor, positions: torch.Tensor, freqs: torch.Tensor, sign: float = 1.0) -> torch.Tensor:
    """x [T, heads, width]: columns (2i, 2i + 1), i < len(freqs), turn by sign * position * f_i; the rest stay."""
    n = freqs.numel()
    angle = sign * positions.to(F)[:, None, None] * freqs[None, None, :]
    c, s = angle.cos(), angle.sin()
    u, v = x[..., 0 : 2 * n : 2], x[..., 1 : 2 * n : 2]
    out = x.clone()
    out[..., 0 : 2 * n : 2] = u * c - v * s
    out[..., 1 : 2 * n : 2] = v * c + u * s
    return out


def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, sink: torch.Tensor) -> torch.Tensor:
    """q [T, H, D], k [T, G, D], v [T, G, V]; p_ij = exp(s_ij) / (exp(sink_h) + sum_j' exp(s_ij')), j <= i."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[-1], dtype=F)
    for h in range(H):
        g = h // (H // G)
        for i in range(T):
            s = (k[: i + 1, g] @ q[i, h]) * scale
            top = torch.maximum(s.max(), sink[h])
            e = torch.exp(s - top)
            out[i, h] = (e @ v[: i + 1, g]) / (e.sum() + torch.exp(sink[h] - top))
    return out


def attention_keys_values(h: torch.Tensor, w: Mapping[str, torch.Tensor], p: str, m: Mapping[str, Any], eps: float):
    """The keys (normed a head, turned) and values a layer with projections of its own caches."""
    T = h.shape[0]
    positions = torch.arange(T)
    k = (h @ w[f"{p}.k"].T).view(T, m["kv_heads"], m["dim"])
    v = (h @ w[f"{p}.v"].T).view(T, m["kv_heads"], m["vdim"])
    k = turn(unit_rms(k, eps) * w[f"{p}.k.norm"], positions, frequencies(m["rot"]))
    return k, v


def attention(h: torch.Tensor, w: Mapping[str, torch.Tensor], p: str, m: Mapping[str, Any], eps: float, keys_values) -> torch.Tensor:
    T = h.shape[0]
    q = (h @ w[f"{p}.q"].T).view(T, m["heads"], m["dim"])
    q = turn(unit_rms(q, eps) * w[f"{p}.q.norm"], torch.arange(T), frequencies(m["rot"]))
    k, v = keys_values
    o = causal_attention(q, k, v, m["scale"], torch.zeros(m["heads"], dtype=F))  # a sink of score 0: one in the denominator
    return o.reshape(T, -1) @ w[f"{p}.o"].T


def sink_attention_turned_values(h: torch.Tensor, w: Mapping[str, torch.Tensor], p: str, m: Mapping[str, Any]) -> torch.Tensor:
    T = h.shape[0]
    positions = torch.arange(T)
    f = frequencies(m["rot"])
    q = turn((h @ w[f"{p}.q"].T).view(T, m["heads"], m["dim"]), positions, f)
    k = turn((h @ w[f"{p}.k"].T).view(T, m["kv_heads"], m["dim"]), positions, f)
    v = (h @ w[f"{p}.v"].T).view(T, m["kv_heads"], m["vdim"])
    value_freqs = frequencies({"base": m["rot"]["base"], "dims": m["vdim"]})  # over all of vdim, never scaled
    o = causal_attention(q, k, turn(v, positions, value_freqs), m["scale"], w[f"{p}.sink"])
    return turn(o, positions, value_freqs, sign=-1.0).reshape(T, -1) @ w[f"{p}.o"].T


def short_convolution(x: torch.Tensor, taps: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x [T, C], taps [C, n]: y_t = sum_j taps[:, n - 1 - j] x_(t - j), zeros before the start."""
    T, C = x.shape
    n = taps.shape[1]
    y = torch.zeros_like(x)
    for t in range(T):
        for j in range(n):
            if t - j >= 0:
                y[t] += taps[:, n - 1 - j] * x[t - j]
    return y if bias is None else y + bias


def gated_delta(h: torch.Tensor, w: Mapping[str, torch.Tensor], p: str, m: Mapping[str, Any], eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(short_convolution(h @ w[f"{p}.q"].T, w[f"{p}.q.conv"])).view(T, G, D)
    k = silu(short_convolution(h @ w[f"{p}.k"].T, w[f"{p}.k.conv"])).view(T, G, D)
    v = silu(short_convolution(h @ w[f"{p}.v"].T, w[f"{p}.v.conv"])).view(T, H, V)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * D ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ w[f"{p}.b"].T)
    a = (h @ w[f"{p}.a1"].T) @ w[f"{p}.a2"].T + w[f"{p}.dt_bias"]
    decay = torch.exp(-torch.exp(w[f"{p}.A_log"])[None, :, None] * softplus(a).view(T, H, D))
    gate = torch.sigmoid((h @ w[f"{p}.g1"].T) @ w[f"{p}.g2"].T).view(T, H, V)
    o = torch.zeros(T, H, V, dtype=F)
    for head in range(H):
        g = head // (H // G)
        S = torch.zeros(D, V, dtype=F)
        for t in range(T):
            S = decay[t, head][:, None] * S
            u = beta[t, head] * (v[t, head] - S.T @ k[t, g])
            S = S + torch.outer(k[t, g], u)
            o[t, head] = S.T @ q[t, g]
    o = unit_rms(o, eps) * w[f"{p}.norm"] * gate
    return o.reshape(T, -1) @ w[f"{p}.o"].T


def state_space(h: torch.Tensor, w: Mapping[str, torch.Tensor], p: str, m: Mapping[str, Any], eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, V, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * V
    packed = h @ w[f"{p}.in"].T
    z, xbc, dt = packed[:, :inner], packed[:, inner : 2 * inner + 2 * G * N], packed[:, 2 * inner + 2 * G * N :]
    xbc = silu(short_convolution(xbc, w[f"{p}.conv"], w[f"{p}.conv.b"]))
    x = xbc[:, :inner].view(T, H, V)
    B = xbc[:, inner : inner + G * N].view(T, G, N)
    C = xbc[:, inner + G * N :].view(T, G, N)
    dt = softplus(dt + w[f"{p}.dt_bias"])
    rate = torch.exp(w[f"{p}.A_log"])
    y = torch.zeros(T, H, V, dtype=F)
    for head in range(H):
        g = head // (H // G)
        S = torch.zeros(N, V, dtype=F)
        for t in range(T):
            S = torch.exp(-rate[head] * dt[t, head]) * S + dt[t, head] * torch.outer(B[t, g], x[t, head])
            y[t, head] = S.T @ C[t, g] + w[f"{p}.D"][head] * x[t, head]
    y = y.reshape(T, inner) * silu(z)
    parts = m["norm_groups"]
    y = unit_rms(y.view(T, parts, inner // parts), eps).reshape(T, inner) * w[f"{p}.norm"]
    return y @ w[f"{p}.o"].T


def feed_forward(h: torch.Tensor, w: Mapping[str, torch.Tensor], p: str) -> torch.Tensor:
    return (silu(h @ w[f"{p}.gate"].T) * (h @ w[f"{p}.up"].T)) @ w[f"{p}.down"].T


def forward(cfg: Mapping[str, Any], weights: Mapping[str, torch.Tensor], tokens, *, layers_out: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] of one sequence."""
    w = {name: t.to(F) for name, t in weights.items()}
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.as_tensor(tokens)] * cfg.get("embedding", {}).get("scale", 1.0)
    kept: dict[int, Any] = {}
    for index, entry in enumerate(cfg["layers"]):
        p, m = f"l{index}", entry["mixer"]
        h = scalar_norm(x, w[f"{p}.norm1"], eps)
        if entry["type"] == "attention":
            if m.get("kv_from") is None:
                kept[index] = attention_keys_values(h, w, f"{p}.mix", m, eps)
            y = attention(h, w, f"{p}.mix", m, eps, kept[index if m.get("kv_from") is None else m["kv_from"]])
        elif entry["type"] == "parallel":
            y = m["left_scale"] * sink_attention_turned_values(h, w, f"{p}.mix.left", m["left"]) \
                + m["right_scale"] * gated_delta(h, w, f"{p}.mix.right", m["right"], eps)
        else:
            y = state_space(h, w, f"{p}.mix", m, eps)
        x = x + scalar_norm(y, w[f"{p}.norm1b"], eps)
        if entry.get("mlp") is not None:
            y = feed_forward(scalar_norm(x, w[f"{p}.norm2"], eps), w, f"{p}.mlp")
            x = x + scalar_norm(y, w[f"{p}.norm2b"], eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    return scalar_norm(x, w["final.norm"], eps) @ w["head"].T
