"""``bench.py --design mapalorn``: prefill and decode throughput of the Mapalorn design at a few layer
sizes, beside the closest design this package has, Makilorn (latent attention and a mixture of experts
too), at the same width, layer count, cached row width and expert sizes (random bf16 weights, synthetic
tokens).  One JSON line; the default workload of bench.py and its line are untouched by this option.

Eight layers: (latent attention, latent attention, latent attention, gated attention) twice; the first
layer's feed-forward is dense, the others' a mixture with a shared expert.  Latent rows of 192 + 64
rotated columns beside Makilorn's rows of 256; the gated attention's heads of 128 with a quarter as many
key/value heads stand where Makilorn has its recurrent layers.  Makilorn's windows are set beyond the
lengths used here, so that both attend over everything.  Measured as ``bench_makilorn.py`` measures: a
2,048-token prompt in one step (median of 5 after 3 warm-up steps) and decode steps at batch 8 and 64
over 2,048-token prompts (CUDA events around ``steps`` replayed steps after ``warmup``; every step reads
its layers' weights and the requests' caches, several times the 126 MB L2).
"""

from __future__ import annotations

import json
import sys

from bench_makilorn import LAYERS, PAGE_SIZE, PROMPT, VOCAB, _decode_ms, _engine, _prefill_ms

# width, heads, experts, experts a token, expert rows, shared expert's rows
SIZES = {
    "w2048": dict(width=2048, heads=16, experts=32, top=4, ff=1024, shared=1024),
    "w4096": dict(width=4096, heads=32, experts=32, top=4, ff=2048, shared=2048),
}
RANK, ROTATED = 192, 64


def mapalorn_config(size: dict) -> dict:
    heads = size["heads"]
    latent = {"heads": heads, "dim": 128, "rot_dim": ROTATED, "vdim": 128, "kv_rank": RANK, "scale": (128 + ROTATED) ** -0.5,
              "rot": {"base": 10000.0, "dims": ROTATED}}
    gated = {"heads": heads, "kv_heads": max(heads // 4, 1), "dim": 128, "vdim": 128, "scale": 128 ** -0.5, "rot": {"base": 10000.0, "dims": 64}}
    mixture = {"kind": "moe", "router": {"experts": size["experts"], "top": size["top"]}, "expert": {"ff": size["ff"]}, "shared": {"ff": size["shared"]}}
    dense = {"kind": "dense", "ff": size["top"] * size["ff"] + size["shared"], "limit": 7.0}
    layers = []
    for index in range(LAYERS):
        mixer = {"type": "attention", "mixer": gated} if index % 4 == 3 else {"type": "latent_attention", "mixer": latent}
        layers.append(dict(mixer, mlp=dense if index == 0 else mixture))
    return {"architecture": "Mapalorn", "vocab": VOCAB, "width": size["width"], "norm": {"eps": 1e-5}, "max_positions": 4096, "layers": layers}


def makilorn_config(size: dict) -> dict:
    heads = size["heads"]
    mlp = {"kind": "moe", "router": {"experts": size["experts"], "top": size["top"]}, "expert": {"ff": size["ff"], "limit": 7.0}}
    attention = {"type": "latent_attention", "mlp": mlp,
                 "mixer": {"heads": heads, "dim": 128, "vdim": 128, "kv_rank": RANK + ROTATED, "scale": 128 ** -0.5, "mask": {"size": 2 * PROMPT}}}
    recurrent = {"type": "delta", "mlp": mlp, "mixer": {"heads": heads, "kv_heads": heads // 2, "dim": 128, "vdim": 128, "conv": 4}}
    return {"architecture": "Makilorn", "vocab": VOCAB, "width": size["width"], "norm": {"eps": 1e-5},
            "layers": [recurrent if index % 4 == 3 else attention for index in range(LAYERS)]}


def run(args) -> int:
    import torch

    if not torch.cuda.is_available():
        print("bench.py: no CUDA device; kairyu_b200 has no CPU path", file=sys.stderr)
        return 1
    torch.cuda.set_device(0)
    steps, warmup = min(args.steps, 64), max(args.warmup, 3)
    sizes = {}
    launches = 0
    for name, size in SIZES.items():
        entry = {}
        for model, config in (("mapalorn", mapalorn_config(size)), ("makilorn", makilorn_config(size))):
            engine = _engine(config, 64)
            prefill = _prefill_ms(engine)
            result = {"prefill_ms": prefill, "prefill_tokens_per_s": PROMPT / (prefill / 1e3),
                      "weight_bytes_per_decode_token": engine.model.bytes_streamed_per_step()}
            for batch in (8, 64):
                ms, count = _decode_ms(engine, batch, steps, warmup)
                launches += count
                result[f"decode_b{batch}_ms"] = ms
                result[f"decode_b{batch}_tokens_per_s"] = batch / (ms / 1e3)
            entry[model] = result
            del engine
            torch.cuda.empty_cache()
        for what in ("prefill", "decode_b8", "decode_b64"):
            entry[f"{what}_ratio"] = entry["mapalorn"][f"{what}_tokens_per_s"] / entry["makilorn"][f"{what}_tokens_per_s"]
        sizes[name] = dict(size, layers=LAYERS, kv_rank=RANK, rot_dim=ROTATED, **entry)
    print(json.dumps({
        "metric": "mapalorn_vs_makilorn_tokens_per_s", "design": "Mapalorn", "n_gpus": 1, "steps": steps, "warmup": warmup, "dtype": "bf16",
        "data": "synthetic", "gpu_launches": launches,
        "config": {"prompt_len": PROMPT, "page_size": PAGE_SIZE, "layers": LAYERS, "inputs": "weights and caches larger than L2"},
        "sizes": sizes,
    }))
    return 0
