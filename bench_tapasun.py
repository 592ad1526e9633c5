"""``bench.py --design tapasun``: prefill and decode throughput of the Tapasun design at a few layer sizes, beside the
closest model this package has at equal size: the dense Qwen3 decoder (grouped-query attention with a norm a head on
queries and keys, a silu-gated feed-forward) of the same width, layer count, heads, key/value heads and feed-forward
rows (random bf16 weights, synthetic tokens).  One JSON line; the default workload of bench.py and its line are
untouched by this option.

Eight layers: attention, attention, attention beside the delta rule, state space, two attention layers that read
layer 1's keys, attention beside the delta rule, state space; heads of 128 with a quarter as many key/value heads,
half of every head rotated; the delta rule with as many heads of 128 and two-step projections of rank 64; the state
space layer with heads of 64, 128 state channels and 8 groups.  Measured as ``bench_makilorn.py`` measures: a
2,048-token prompt in one step (median of 5 after 3 warm-up steps) and decode steps at batch 8 and 64 over 2,048-token
prompts (CUDA events around ``steps`` replayed steps after ``warmup``; every step reads its layers' weights and the
requests' caches, several times the 126 MB L2).
"""

from __future__ import annotations

import json
import sys

from bench_makilorn import LAYERS, PAGE_SIZE, PROMPT, VOCAB, _decode_ms, _engine, _prefill_ms

SIZES = {
    "w2048": dict(width=2048, heads=16, ff=8192),
    "w4096": dict(width=4096, heads=32, ff=14336),
}
LOW_RANK = 64


def tapasun_config(size: dict) -> dict:
    width, heads = size["width"], size["heads"]
    kv_heads = max(heads // 4, 1)
    rot = {"base": 500000.0, "dims": 64, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}}
    plain = {"heads": heads, "kv_heads": kv_heads, "dim": 128, "vdim": 128, "scale": 128 ** -0.5, "rot": rot}
    side = {"left": {"heads": heads, "kv_heads": kv_heads, "dim": 128, "vdim": 128, "scale": 128 ** -0.5,
                     "rot": {"base": 500000.0, "dims": 64, "scaling": {"factor": 2.0}}},
            "right": {"heads": heads, "kv_heads": heads // 2, "dim": 128, "vdim": 128, "conv": 4, "decay_rank": LOW_RANK, "gate_rank": LOW_RANK},
            "left_scale": 0.7, "right_scale": 0.4}
    space = {"heads": 2 * width // 64, "vdim": 64, "state": 128, "groups": 8, "norm_groups": 8, "conv": 4}
    mlp = {"kind": "dense", "ff": size["ff"]}
    mixers = [("attention", plain), ("attention", plain), ("parallel", side), ("mamba2", space),
              ("attention", dict(plain, kv_from=1)), ("attention", dict(plain, kv_from=1)), ("parallel", side), ("mamba2", space)]
    assert len(mixers) == LAYERS
    return {"architecture": "Tapasun", "vocab": VOCAB, "width": width, "norm": {"eps": 1e-6}, "embedding": {"scale": width ** 0.5},
            "max_positions": 4096, "layers": [{"type": kind, "mixer": mixer, "mlp": mlp} for kind, mixer in mixers]}


def dense_config(size: dict) -> dict:
    return {
        "architectures": ["Qwen3ForCausalLM"], "hidden_size": size["width"], "num_hidden_layers": LAYERS,
        "num_attention_heads": size["heads"], "num_key_value_heads": max(size["heads"] // 4, 1), "head_dim": 128,
        "intermediate_size": size["ff"], "vocab_size": VOCAB, "rope_theta": 500000.0,
        "max_position_embeddings": 8192, "rms_norm_eps": 1e-6, "tie_word_embeddings": False, "hidden_act": "silu",
    }


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
        for model, config in (("tapasun", tapasun_config(size)), ("dense", dense_config(size))):
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
            entry[f"{what}_ratio"] = entry["tapasun"][f"{what}_tokens_per_s"] / entry["dense"][f"{what}_tokens_per_s"]
        sizes[name] = dict(size, layers=LAYERS, **entry)
    print(json.dumps({
        "metric": "tapasun_vs_dense_tokens_per_s", "design": "Tapasun", "n_gpus": 1, "steps": steps, "warmup": warmup, "dtype": "bf16",
        "data": "synthetic", "gpu_launches": launches,
        "config": {"prompt_len": PROMPT, "page_size": PAGE_SIZE, "layers": LAYERS, "inputs": "weights and caches larger than L2"},
        "sizes": sizes,
    }))
    return 0
