"""Small Tapasun configurations and weights for the tests.

The weights are drawn so that a fault shows: query and key gains large enough for the softmax to pick single keys (a
wrong rotation, key/value head or lost key moves the result by far more than rounding), sinks of the size of the
scores, scalar norm weights away from one, decays that differ from channel to channel and are neither 0 nor 1, step
sizes of the order of one, convolutions whose every tap matters.  The configurations differ in every size, also in
those a model may happen to make equal or 1: key and value widths, heads and key/value heads (one, some, all), the
delta rule's heads against its query/key heads, groups against norm groups, 1 to 5 taps, layers without feed-forward,
several layers reading one layer's keys, rotated parts narrower than a head and as wide, the three kinds of frequency
scaling.
"""

from __future__ import annotations

import json
from pathlib import Path
from typing import Any, Mapping, Optional

import torch
from safetensors.torch import save_file

LLAMA3 = {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 64}  # wavelengths of 16 to 64 positions are blended


def rot(base, dims, scaling=None):
    table = {"base": base, "dims": dims}
    if scaling is not None:
        table["scaling"] = scaling
    return table


def attention(heads, kv_heads, dim, vdim, scale, rot_dims, base=10000.0, scaling=None, kv_from=None):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "rot": rot(base, rot_dims, scaling)}
    if kv_from is not None:
        mixer["kv_from"] = kv_from
    return {"type": "attention", "mixer": mixer}


def left(heads, kv_heads, dim, vdim, scale, rot_dims, base=10000.0, scaling=None):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "rot": rot(base, rot_dims, scaling)}


def right(heads, kv_heads, dim, vdim, conv):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}


def parallel(left_mixer, right_mixer, left_scale=0.7, right_scale=0.4):
    return {"type": "parallel", "mixer": {"left": left_mixer, "right": right_mixer, "left_scale": left_scale, "right_scale": right_scale}}


def mamba2(heads, vdim, state, groups, norm_groups, conv):
    return {"type": "mamba2", "mixer": {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "norm_groups": norm_groups, "conv": conv}}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def layer(mixer, mlp):
    return dict(mixer, mlp=mlp)


def config(width, vocab, layers, eps=1e-5, embedding_scale=None):
    cfg = {"architecture": "Tapasun", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if embedding_scale is not None:
        cfg["embedding"] = {"scale": embedding_scale}
    return cfg


# name -> (config, seed, page size, ranks of the delta rule's two-step projections (decay, gate))
CASES: dict[str, tuple[dict, int, int, tuple[int, int]]] = {
    # heads of 32 and 16 with equal key and value widths: the tensor-core kernels in bfloat16; two layers read layer 0's keys
    "shared_keys": (config(48, 97, [
        layer(attention(4, 2, 32, 32, 0.2, 16, base=500.0, scaling=LLAMA3), dense(40)),
        layer(parallel(left(4, 2, 16, 16, 0.3, 8, base=300.0, scaling={"factor": 2.0}), right(4, 2, 16, 8, 3)), dense(24)),
        layer(attention(2, 2, 32, 32, 0.25, 32, kv_from=0), None),
        layer(mamba2(4, 8, 16, 2, 1, 4), dense(32)),
        layer(attention(4, 2, 32, 32, 0.2, 8, base=50.0, kv_from=0), dense(16)),
    ], embedding_scale=6.9), 51, 8, (6, 5)),
    # nothing a multiple of 8: the 32-bit-arithmetic kernels in both modes; one key/value head; one tap; one group
    "odd": (config(50, 77, [
        layer(mamba2(3, 6, 5, 1, 3, 1), None),
        layer(attention(3, 1, 10, 14, 0.35, 6), dense(30)),
        layer(parallel(left(3, 3, 6, 10, 0.5, 2, base=50.0), right(3, 1, 5, 7, 1), left_scale=1.0, right_scale=1.0), dense(18)),
        layer(attention(6, 1, 10, 14, 0.3, 10, base=100.0, scaling={"factor": 3.0}, kv_from=1), dense(22)),
    ], eps=1e-6), 52, 16, (3, 7)),
    # heads of 128 and 64: the tcgen05 and TMA-fed kernels in bfloat16; wide recurrent states; five taps
    "wide": (config(64, 131, [
        layer(parallel(left(2, 1, 64, 64, 0.12, 32, scaling={"factor": 8.0}), right(2, 2, 64, 48, 5), left_scale=0.5, right_scale=0.9), dense(96)),
        layer(attention(4, 1, 128, 128, 0.09, 64, base=40000.0, scaling=LLAMA3), dense(64)),
        layer(mamba2(4, 32, 64, 4, 2, 2), dense(48)),
        layer(attention(2, 1, 128, 128, 0.09, 64, base=40000.0, scaling=LLAMA3, kv_from=1), None),
    ], embedding_scale=8.0), 53, 16, (8, 16)),
    # pages of four; values wider and narrower than keys; more groups than norm groups and the reverse
    "small_pages": (config(32, 61, [
        layer(attention(6, 2, 16, 24, 0.25, 8), dense(24)),
        layer(mamba2(4, 4, 8, 4, 2, 3), None),
        layer(parallel(left(2, 1, 24, 8, 0.2, 24), right(6, 3, 8, 4, 2)), dense(16)),
        layer(mamba2(2, 16, 12, 1, 4, 4), dense(8)),
    ]), 54, 4, (4, 4)),
}


def _normal(generator, shape, std):
    return torch.randn(shape, generator=generator, dtype=torch.float32) * std


def _scalar(generator, around=1.0, spread=0.25):
    return (around + _normal(generator, (), spread)).abs() + 0.25


def make_weights(cfg: Mapping[str, Any], seed: int, ranks: tuple[int, int] = (4, 4)) -> dict[str, torch.Tensor]:
    """fp32 tensors whose values are exact in bfloat16 (a model folder written in either dtype holds the same numbers)."""
    g = torch.Generator().manual_seed(seed)
    width, vocab = cfg["width"], cfg["vocab"]
    w: dict[str, torch.Tensor] = {"embed": _normal(g, (vocab, width), 1.0), "final.norm": _scalar(g), "head": _normal(g, (vocab, width), width ** -0.5)}

    def attention_weights(p: str, m: Mapping[str, Any], *, normed: bool, own_kv: bool) -> None:
        heads, kvh, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        gain = (3.0 / m["scale"]) ** 0.5  # scores of a few units: the softmax picks single keys
        part = 1.0 if normed else gain * dim ** -0.25  # normed rows have unit mean square: the norm weights carry the scores' size
        w[f"{p}.q"] = _normal(g, (heads * dim, width), part * width ** -0.5)
        if own_kv:
            w[f"{p}.k"] = _normal(g, (kvh * dim, width), part * width ** -0.5)
            w[f"{p}.v"] = _normal(g, (kvh * vdim, width), width ** -0.5)
        if normed:
            w[f"{p}.q.norm"] = (1.0 + _normal(g, (dim,), 0.2)) * gain * dim ** -0.25
            if own_kv:
                w[f"{p}.k.norm"] = (1.0 + _normal(g, (dim,), 0.2)) * gain * dim ** -0.25
        w[f"{p}.o"] = _normal(g, (width, heads * vdim), (heads * vdim) ** -0.5)

    for index, entry in enumerate(cfg["layers"]):
        p, m = f"l{index}", entry["mixer"]
        for name in ("norm1", "norm1b"):
            w[f"{p}.{name}"] = _scalar(g)
        if entry["type"] == "attention":
            attention_weights(f"{p}.mix", m, normed=True, own_kv=m.get("kv_from") is None)
        elif entry["type"] == "parallel":
            attention_weights(f"{p}.mix.left", m["left"], normed=False, own_kv=True)
            w[f"{p}.mix.left.sink"] = _normal(g, (m["left"]["heads"],), 1.5)
            r, q = m["right"], f"{p}.mix.right"
            heads, kvh, dim, vdim, taps = r["heads"], r["kv_heads"], r["dim"], r["vdim"], r["conv"]
            for name, rows in (("q", kvh * dim), ("k", kvh * dim), ("v", heads * vdim)):
                w[f"{q}.{name}"] = _normal(g, (rows, width), 1.5 * width ** -0.5)
                w[f"{q}.{name}.conv"] = _normal(g, (rows, taps), 0.6)
            w[f"{q}.b"] = _normal(g, (heads, width), 1.5 * width ** -0.5)
            w[f"{q}.A_log"] = _normal(g, (heads,), 0.5) - 0.5
            w[f"{q}.norm"] = 1.0 + _normal(g, (vdim,), 0.2)
            w[f"{q}.a1"] = _normal(g, (ranks[0], width), width ** -0.5)
            w[f"{q}.a2"] = _normal(g, (heads * dim, ranks[0]), 1.5 * ranks[0] ** -0.5)
            w[f"{q}.dt_bias"] = _normal(g, (heads * dim,), 1.0)
            w[f"{q}.g1"] = _normal(g, (ranks[1], width), width ** -0.5)
            w[f"{q}.g2"] = _normal(g, (heads * vdim, ranks[1]), 1.5 * ranks[1] ** -0.5)
            w[f"{q}.o"] = _normal(g, (width, heads * vdim), (heads * vdim) ** -0.5)
        else:
            q = f"{p}.mix"
            heads, vdim, state, groups, taps = m["heads"], m["vdim"], m["state"], m["groups"], m["conv"]
            inner, channels = heads * vdim, heads * vdim + 2 * groups * state
            w[f"{q}.in"] = _normal(g, (inner + channels + heads, width), 1.5 * width ** -0.5)
            w[f"{q}.conv"] = _normal(g, (channels, taps), 0.6)
            w[f"{q}.conv.b"] = _normal(g, (channels,), 0.3)
            w[f"{q}.dt_bias"] = _normal(g, (heads,), 1.0)
            w[f"{q}.A_log"] = _normal(g, (heads,), 0.5) - 0.5
            w[f"{q}.D"] = 1.0 + _normal(g, (heads,), 0.3)
            w[f"{q}.norm"] = 1.0 + _normal(g, (inner,), 0.2)
            w[f"{q}.o"] = _normal(g, (width, inner), inner ** -0.5)
        mlp = entry["mlp"]
        if mlp is None:
            continue
        for name in ("norm2", "norm2b"):
            w[f"{p}.{name}"] = _scalar(g)
        w[f"{p}.mlp.gate"] = _normal(g, (mlp["ff"], width), 1.5 * width ** -0.5)
        w[f"{p}.mlp.up"] = _normal(g, (mlp["ff"], width), 1.5 * width ** -0.5)
        w[f"{p}.mlp.down"] = _normal(g, (width, mlp["ff"]), mlp["ff"] ** -0.5)
    return {name: t.to(torch.bfloat16).to(torch.float32) for name, t in w.items()}


def write_model(cfg: Mapping[str, Any], weights: Mapping[str, torch.Tensor], folder: Path, dtype: torch.dtype = torch.bfloat16) -> Path:
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(cfg))
    save_file({name: t.to(dtype).contiguous() for name, t in weights.items()}, str(folder / "model.safetensors"))
    return folder


def relative_error(got, want) -> float:
    """Largest over the rows of rms(difference, its mean taken off) / rms(wanted row, its mean taken off)."""
    import numpy as np

    got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    d = got - want
    d = d - d.mean(-1, keepdims=True)
    ref = want - want.mean(-1, keepdims=True)
    return float((np.sqrt((d * d).mean(-1)) / np.sqrt((ref * ref).mean(-1) + 1e-30)).max())
