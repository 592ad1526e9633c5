"""Small Mapalorn configurations and weights for the tests.

The weights are drawn so that a fault shows: queries and keys are large enough for the softmax to pick single keys
(a wrong rotation, a wrong key/value head or a lost key then moves the result by far more than rounding), the sinks are
of the size of the scores (leaving one out, scaling it or counting it twice changes every weight), the layer norms have
biases, the norm weights differ from one, the dense feed-forward's products reach beyond its limit on both sides, the
routers spread their logits and the shared expert's gate is neither open nor shut.  The configurations differ in every
size: heads and key/value heads (one, several, as many as heads), key and value widths (equal, wider, narrower, no
multiple of 8), rotated parts narrower than a head and as wide, latent ranks, one expert a token and several and all of
them, mixtures with and without a shared expert, layers without a feed-forward, loops at the start, in the middle, of one
layer, of one pass, and none.
"""

from __future__ import annotations

import json
from pathlib import Path
from typing import Any, Mapping

import torch
from safetensors.torch import save_file


def latent(heads, dim, rot_dim, vdim, kv_rank, scale, base=10000.0):
    return {"type": "latent_attention",
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale, "rot": {"base": base, "dims": rot_dim}}}


def gated(heads, kv_heads, dim, vdim, scale, rot_dims, base=10000.0):
    return {"type": "attention",
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "rot": {"base": base, "dims": rot_dims}}}


def dense(ff, limit):
    return {"kind": "dense", "ff": ff, "limit": limit}


def moe(experts, top, ff, shared=None):
    mlp = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}
    if shared is not None:
        mlp["shared"] = {"ff": shared}
    return mlp


def layer(mixer, mlp):
    return dict(mixer, mlp=mlp)


def config(width, vocab, layers, loop=None, eps=1e-5):
    cfg = {"architecture": "Mapalorn", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if loop is not None:
        cfg["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return cfg


# name -> (config, seed, page size)
CASES: dict[str, tuple[dict, int, int]] = {
    # cached rows of 48 and heads of 32 and 16: the tensor-core kernels in bfloat16; a loop in the middle; two and three
    # experts a token; a rotated part narrower than the head; a layer without feed-forward
    "looped": (config(48, 97, [
        layer(gated(4, 2, 32, 16, 0.2, 16, base=500.0), dense(40, 1.5)),
        layer(latent(3, 16, 16, 24, 32, 0.25), moe(6, 2, 24, shared=16)),
        layer(gated(2, 2, 16, 32, 0.3, 16), moe(4, 3, 16)),
        layer(latent(2, 24, 8, 16, 40, 0.2, base=300.0), None),
    ], loop=(1, 3, 2)), 41, 8),
    # nothing a multiple of 8: the 32-bit-arithmetic kernels in both modes; every expert chosen; a loop of one layer at the start
    "odd": (config(50, 77, [
        layer(latent(3, 10, 6, 14, 18, 0.4, base=100.0), moe(3, 3, 18, shared=10)),
        layer(gated(3, 1, 10, 14, 0.35, 6), dense(30, 0.8)),
        layer(gated(3, 3, 6, 20, 0.5, 2, base=50.0), None),
    ], loop=(0, 1, 3), eps=1e-6), 42, 16),
    # no loop; the widest rows; one expert of one; four query heads a key/value head; the whole head rotated
    "wide": (config(64, 131, [
        layer(latent(5, 32, 64, 48, 128, 0.12, base=40000.0), moe(1, 1, 32)),
        layer(gated(4, 1, 128, 64, 0.09, 128), moe(5, 1, 24, shared=40)),
        layer(gated(2, 2, 64, 128, 0.12, 32), dense(96, 3.0)),
    ]), 43, 16),
    # pages of four; a loop of one pass (which is no loop) over the end; more heads than one attention call takes
    "small_pages": (config(32, 61, [
        layer(latent(18, 8, 8, 8, 24, 0.35), dense(24, 1.0)),
        layer(gated(6, 2, 16, 16, 0.25, 8), moe(4, 2, 8, shared=8)),
    ], loop=(1, 2, 1)), 44, 4),
}


def _normal(generator, shape, std):
    return torch.randn(shape, generator=generator, dtype=torch.float32) * std


def make_weights(cfg: Mapping[str, Any], seed: int) -> dict[str, torch.Tensor]:
    """fp32 tensors whose values are exact in bfloat16 (a model folder written in either dtype holds the same numbers)."""
    g = torch.Generator().manual_seed(seed)
    width, vocab = cfg["width"], cfg["vocab"]
    w: dict[str, torch.Tensor] = {
        "embed": _normal(g, (vocab, width), 1.0), "final.norm": 1.0 + _normal(g, (width,), 0.1), "final.norm.b": _normal(g, (width,), 0.1),
        "head": _normal(g, (vocab, width), width ** -0.5),
    }
    for index, entry in enumerate(cfg["layers"]):
        p, m = f"l{index}", entry["mixer"]
        heads, dim, vdim = m["heads"], m["dim"], m["vdim"]
        w[f"{p}.norm1"] = 1.0 + _normal(g, (width,), 0.1)
        w[f"{p}.norm1.b"] = _normal(g, (width,), 0.2)
        gain = (3.0 / m["scale"]) ** 0.5  # scores of a few units: the softmax picks single keys
        if entry["type"] == "latent_attention":
            rot, rank = m["rot_dim"], m["kv_rank"]
            part = gain * (dim + rot) ** -0.25
            w[f"{p}.mix.q"] = _normal(g, (heads * (dim + rot), width), part * width ** -0.5)
            w[f"{p}.mix.dkv"] = _normal(g, (rank + rot, width), width ** -0.5)
            w[f"{p}.mix.dkv"][rank:] *= part
            w[f"{p}.mix.dkv.norm"] = 1.0 + _normal(g, (rank,), 0.2)
            w[f"{p}.mix.uk"] = _normal(g, (heads * dim, rank), part * rank ** -0.5)
            w[f"{p}.mix.uv"] = _normal(g, (heads * vdim, rank), rank ** -0.5)
            w[f"{p}.mix.sink"] = _normal(g, (heads,), 1.5)
        else:
            kvh = m["kv_heads"]
            w[f"{p}.mix.q"] = _normal(g, (heads * dim, width), width ** -0.5)
            w[f"{p}.mix.k"] = _normal(g, (kvh * dim, width), width ** -0.5)
            w[f"{p}.mix.v"] = _normal(g, (kvh * vdim, width), width ** -0.5)
            # the normed rows have unit mean square, so the norm weights carry the scores' size
            w[f"{p}.mix.q.norm"] = (1.0 + _normal(g, (heads * dim,), 0.2)) * gain * dim ** -0.25
            w[f"{p}.mix.k.norm"] = (1.0 + _normal(g, (kvh * dim,), 0.2)) * gain * dim ** -0.25
            w[f"{p}.mix.g"] = _normal(g, (heads * vdim, width), 1.5 * width ** -0.5)
        w[f"{p}.mix.o"] = _normal(g, (width, heads * vdim), (heads * vdim) ** -0.5)
        mlp = entry["mlp"]
        if mlp is None:
            continue
        if mlp["kind"] == "dense":
            # products of about twice the limit at one standard deviation: both clamps and the one-sided one act
            w[f"{p}.mlp.gate"] = _normal(g, (mlp["ff"], width), 1.2 * mlp["limit"] * width ** -0.5)
            w[f"{p}.mlp.up"] = _normal(g, (mlp["ff"], width), 1.2 * mlp["limit"] * width ** -0.5)
            w[f"{p}.mlp.down"] = _normal(g, (width, mlp["ff"]), mlp["ff"] ** -0.5 / mlp["limit"])
            continue
        ff = mlp["expert"]["ff"]
        for e in range(mlp["router"]["experts"]):
            w[f"{p}.mlp.e{e}.gate"] = _normal(g, (ff, width), 1.5 * width ** -0.5)
            w[f"{p}.mlp.e{e}.up"] = _normal(g, (ff, width), 1.5 * width ** -0.5)
            w[f"{p}.mlp.e{e}.down"] = _normal(g, (width, ff), ff ** -0.5)
        w[f"{p}.mlp.router"] = _normal(g, (mlp["router"]["experts"], width), 2 * width ** -0.5)
        if mlp.get("shared"):
            sff = mlp["shared"]["ff"]
            w[f"{p}.mlp.shared.gate"] = _normal(g, (sff, width), 1.5 * width ** -0.5)
            w[f"{p}.mlp.shared.up"] = _normal(g, (sff, width), 1.5 * width ** -0.5)
            w[f"{p}.mlp.shared.down"] = _normal(g, (width, sff), sff ** -0.5)
            w[f"{p}.mlp.shared.sg"] = _normal(g, (1, width), 1.5 * width ** -0.5)
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
