"""Tapasun without a GPU: the config reader, the spec it builds (a layer that reads another layer's keys names that
layer's cache slot and keeps nothing itself; what every slot keeps), model folders written and read back (scalar norm
weights, ranks read from the tensors' shapes), what the GPU tests' bounds can see, the plain implementation's own
pieces, and, with the kernels replaced by their torch statements, every cut through the step function and greedy
generation through the scheduler and the command line."""

import json

import numpy as np
import pytest
import torch

import tapasun_plain as plain
import traces
from tapasun_cases import CASES, attention, config, dense, layer, left, make_weights, mamba2, parallel, relative_error, right, write_model

from kairyu_b200.cache import CacheLayout
from kairyu_b200.config.model_config import ConfigError
from kairyu_b200.engine.engine import build_model, load_model
from kairyu_b200.parts import PagedKVSpec, StateSpec
from kairyu_b200.registry import architecture_of, supported_architectures
from kairyu_b200.weights.loading import WeightError, load_into, read_config_with_shapes


def test_registered_by_its_config_key():
    assert "Tapasun" in supported_architectures()
    assert architecture_of({"architecture": "Tapasun"}).name == "Tapasun"


def _with_ranks(cfg, ranks):
    """The config with the delta rule's ranks named (what a folder's tensor shapes would say)."""
    cfg = json.loads(json.dumps(cfg))
    for entry in cfg["layers"]:
        if entry["type"] == "parallel":
            entry["mixer"]["right"].update(decay_rank=ranks[0], gate_rank=ranks[1])
    return cfg


@pytest.mark.parametrize("name", list(CASES))
def test_spec_run_order_and_cache_needs(name):
    cfg, _, _, ranks = CASES[name]
    model, parsed = build_model(_with_ranks(cfg, ranks), dtype="float32", device="meta")
    entries = cfg["layers"]
    assert len(model.blocks) == len(entries) == len(model.schedule)
    assert [call.layer for call in model.schedule] == list(range(len(entries)))
    needs = model.cache_slot_specs()
    for index, (entry, call) in enumerate(zip(entries, model.schedule)):
        m = entry["mixer"]
        source = m.get("kv_from") if entry["type"] == "attention" else None
        if source is not None:
            # it reads the slot of the layer it names and keeps nothing itself
            assert (call.cache_slot, call.writes_cache) == (source, False) and index not in needs
            assert not model.blocks[index].mixer.cache_specs()
            continue
        assert (call.cache_slot, call.writes_cache) == (index, True)
        if entry["type"] == "attention":
            assert needs[index] == (PagedKVSpec(m["kv_heads"], m["dim"], None, v_head_dim=m["vdim"]),)
        elif entry["type"] == "parallel":
            l, r = m["left"], m["right"]
            channels = 2 * r["kv_heads"] * r["dim"] + r["heads"] * r["vdim"]
            kept = (StateSpec((r["conv"] - 1, channels), "float32"),) if r["conv"] > 1 else ()
            assert needs[index] == (PagedKVSpec(l["kv_heads"], l["dim"], None, v_head_dim=l["vdim"]),
                                    StateSpec((r["heads"], r["vdim"], r["dim"]), "float32")) + kept
        else:
            channels = m["heads"] * m["vdim"] + 2 * m["groups"] * m["state"]
            kept = (StateSpec((m["conv"] - 1, channels), "float32"),) if m["conv"] > 1 else ()
            assert needs[index] == (StateSpec((m["heads"], m["vdim"], m["state"]), "float32"),) + kept
    for entry, block in zip(entries, model.blocks):
        assert (block.ffn is None) == (entry["mlp"] is None)
    assert {spec.name for spec in model.tensor_specs()} == set(make_weights(cfg, 0, ranks))
    assert {spec.name: tuple(spec.shape) for spec in model.tensor_specs()} == {n: tuple(t.shape) for n, t in make_weights(cfg, 0, ranks).items()}
    assert parsed.vocab_size == cfg["vocab"] and parsed.hidden_size == cfg["width"]
    assert parsed.embedding_scale == cfg.get("embedding", {}).get("scale", 1.0)
    assert model.graph_safe()


@pytest.mark.parametrize("damage, message", [
    (lambda c: c.pop("vocab"), "vocab"),
    (lambda c: c.pop("width"), "width"),
    (lambda c: c["norm"].pop("eps"), "eps"),
    (lambda c: c["embedding"].pop("scale"), "scale"),
    (lambda c: c["layers"][0]["mixer"].pop("vdim"), "vdim"),
    (lambda c: c["layers"][0].update(type="conv"), "unknown layer type"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "multiple"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), "even"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=64), "at most dim"),
    (lambda c: c["layers"][0]["mixer"]["rot"]["scaling"].pop("high"), "high"),
    (lambda c: c["layers"][0]["mixer"]["rot"]["scaling"].update(factor=0), "factor"),
    (lambda c: c["layers"][1]["mixer"]["left"].pop("scale"), "scale"),
    (lambda c: c["layers"][1]["mixer"]["left"].update(vdim=15), "even"),
    (lambda c: c["layers"][1]["mixer"]["right"].update(kv_heads=3), "multiple"),
    (lambda c: c["layers"][1]["mixer"].pop("right_scale"), "right_scale"),
    (lambda c: c["layers"][2]["mixer"].update(kv_from=3), "earlier layer"),
    (lambda c: c["layers"][4]["mixer"].update(kv_from=2), "keys and values of its own"),
    (lambda c: c["layers"][4]["mixer"].update(kv_from=1), "keys and values of its own"),
    (lambda c: c["layers"][4]["mixer"].update(dim=16), "differ in dim"),
    (lambda c: c["layers"][3]["mixer"].update(groups=3), "multiple"),
    (lambda c: c["layers"][3]["mixer"].update(norm_groups=5), "equal parts"),
    (lambda c: c["layers"][3]["mixer"].pop("state"), "state"),
    (lambda c: c["layers"][0]["mlp"].update(kind="gated"), "unknown feed-forward"),
    (lambda c: c["layers"][0]["mlp"].pop("ff"), "ff"),
])
def test_config_errors_name_the_key(damage, message):
    cfg = json.loads(json.dumps(CASES["shared_keys"][0]))
    damage(cfg)
    with pytest.raises(ConfigError, match=message):
        build_model(cfg, dtype="float32", device="meta")


def test_model_folder_round_trip(tmp_path):
    cfg, seed, _, ranks = CASES["shared_keys"]
    weights = make_weights(cfg, seed, ranks)
    folder = write_model(cfg, weights, tmp_path / "m")
    # the ranks of the two-step projections are in no config key: the tensors' shapes give them
    shapes = read_config_with_shapes(folder)["tensor_shapes"]
    assert shapes["l1.mix.right.a1"] == [ranks[0], cfg["width"]] and shapes["l1.norm1"] == []
    model, _ = load_model(folder, dtype="float32", device="cpu")
    first, side, borrowed = model.blocks[0].mixer, model.blocks[1].mixer, model.blocks[2].mixer
    assert torch.equal(first.w_in[first.k_offset : first.v_offset], weights["l0.mix.k"])
    assert torch.equal(first.q_norm_weight, weights["l0.mix.q.norm"]) and first.q_norm_weight.numel() == cfg["layers"][0]["mixer"]["dim"]
    assert torch.equal(side.left.sinks, weights["l1.mix.left.sink"])
    assert (side.right.decay_rank, side.right.gate_rank) == ranks and torch.equal(side.right.w_a2, weights["l1.mix.right.a2"])
    assert borrowed.w_in.shape[0] == borrowed.q_size and not borrowed.own_kv  # queries alone
    norm = model.blocks[0].mixer_norm.weight  # one number, spread over the width
    assert norm.shape == (cfg["width"],) and torch.equal(norm, weights["l0.norm1"].expand(cfg["width"]))
    assert torch.equal(model.blocks[3].mixer.w_dt, weights["l3.mix.in"][-4:])
    broken = dict(weights)
    del broken["l1.mix.left.sink"]
    broken["l2.mix.q.norm"] = torch.zeros(5)
    with pytest.raises(WeightError) as error:
        load_model(write_model(cfg, broken, tmp_path / "b"), dtype="float32", device="cpu")
    assert error.value.missing == ["l1.mix.left.sink"] and error.value.wrong_shape[0][0] == "l2.mix.q.norm"
    extra = dict(weights)
    extra["l2.mix.k"] = torch.zeros(64, 48)  # a layer that borrows keys has none of its own
    with pytest.raises(WeightError):
        load_into(load_model(folder, dtype="float32", device="cpu")[0], write_model(cfg, extra, tmp_path / "e"), strict_unexpected=True)


def test_random_weights_through_the_registry(tmp_path):
    from kairyu_b200.weights import write_random_model

    cfg, _, _, ranks = CASES["small_pages"]
    folder = write_random_model(_with_ranks(cfg, ranks), tmp_path / "r", seed=4, dtype="bfloat16")
    model, _ = load_model(folder, dtype="float32", device="cpu")
    assert (model.blocks[2].mixer.right.decay_rank, model.blocks[2].mixer.right.gate_rank) == ranks


def _faults():
    """Ways to get one mechanism wrong, each a (name, patch) where ``patch(mp)`` replaces one piece of the plain model."""
    def replace(name, function):
        return lambda mp: mp.setattr(plain, name, function)

    original = {name: getattr(plain, name) for name in ("turn", "causal_attention", "frequencies", "short_convolution", "unit_rms", "softplus")}

    def halves(x, positions, freqs, sign=1.0):  # pairs (i, i + n) in place of (2i, 2i + 1)
        n = freqs.numel()
        angle = sign * positions.to(plain.F)[:, None, None] * freqs[None, None, :]
        c, s = angle.cos(), angle.sin()
        out = x.clone()
        out[..., :n] = x[..., :n] * c - x[..., n : 2 * n] * s
        out[..., n : 2 * n] = x[..., n : 2 * n] * c + x[..., :n] * s
        return out

    def no_sink(q, k, v, scale, sink):
        return original["causal_attention"](q, k, v, scale, torch.full_like(sink, -1e9))

    def scaled_sink(q, k, v, scale, sink):
        return original["causal_attention"](q, k, v, scale, sink * scale + 0.7)

    def unscaled(rot):
        return original["frequencies"]({"base": rot["base"], "dims": rot["dims"]})

    def one_tap_late(x, taps, bias=None):  # the last column taken for the oldest token's
        return original["short_convolution"](x, taps.flip(1), bias)

    def eps_outside(x, eps):
        return x / (torch.sqrt((x * x).mean(-1, keepdim=True)) + 0.3)  # eps outside the root, and large

    return [("halves", replace("turn", halves)), ("no sink", replace("causal_attention", no_sink)), ("sink scaled", replace("causal_attention", scaled_sink)),
            ("no frequency scaling", replace("frequencies", unscaled)), ("taps reversed", replace("short_convolution", one_tap_late)),
            ("another norm", replace("unit_rms", eps_outside)), ("softplus clamped", replace("softplus", lambda z: original["softplus"](z).clamp(max=1.0)))]


@pytest.mark.parametrize("name", ["shared_keys", "small_pages"])
def test_the_bounds_see_each_fault(name, monkeypatch):
    """Each mechanism got wrong moves the median position by more than the bfloat16 bound of the GPU tests."""
    cfg, seed, _, ranks = CASES[name]
    weights = make_weights(cfg, seed, ranks)
    tokens = traces.make_requests(cfg["vocab"], [60], seed=1)["r0"]
    right_logits = plain.forward(cfg, weights, tokens).numpy()
    for what, patch in _faults():
        if name == "small_pages" and what in ("no frequency scaling", "no sink", "sink scaled"):
            continue  # that case has no scaled frequencies, and its only learned sinks sit beside a strong right side
        with monkeypatch.context() as mp:
            patch(mp)
            wrong = plain.forward(cfg, weights, tokens).numpy()
        errors = [relative_error(wrong[t], right_logits[t]) for t in range(len(tokens))]
        if "sink" in what:
            # The norm on the mixer's output takes a common factor off again, so a sink shows where it weighs differently from
            # head to head: at a sequence's first tokens, where it stands beside one key or a few (hundreds of times the
            # float32 bound there, and of the order of the bfloat16 bound).
            assert max(errors[:6]) > 0.02, (what, errors[:6])
        else:
            assert np.median(errors[8:]) > 0.05, (what, np.median(errors[8:]))


def test_plain_model_pieces():
    """The oracle's own pieces against facts that need no second implementation."""
    f = plain.frequencies({"base": 100.0, "dims": 8})
    assert torch.allclose(f, torch.tensor([1.0, 100 ** -0.25, 100 ** -0.5, 100 ** -0.75], dtype=plain.F))
    scaled = plain.frequencies({"base": 100.0, "dims": 8, "scaling": {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 64}})
    # wavelengths 6.3, 19.9, 62.8, 198.7 against the edges 16 and 64: kept, blended, blended, divided
    assert scaled[0] == f[0] and scaled[3] == f[3] / 4.0 and f[1] / 4.0 < scaled[1] < f[1] and f[2] / 4.0 < scaled[2] < f[2]
    s = (64 / (2 * np.pi / f[1].item()) - 1.0) / 3.0
    assert abs(scaled[1].item() - ((1 - s) * f[1].item() / 4.0 + s * f[1].item())) < 1e-12
    assert torch.allclose(plain.frequencies({"base": 100.0, "dims": 8, "scaling": {"factor": 2.0}}), f / 2.0)
    # a turn keeps lengths, turns pair (2i, 2i + 1), leaves the columns behind alone, and is undone by the opposite sign
    x = torch.randn(5, 2, 10, dtype=plain.F)
    positions = torch.arange(5)
    y = plain.turn(x, positions, f[:3])
    assert torch.allclose(y[..., 6:], x[..., 6:]) and torch.allclose(y.norm(dim=-1), x.norm(dim=-1)) and torch.equal(y[0], x[0])
    assert torch.allclose(plain.turn(y, positions, f[:3], sign=-1.0), x)
    assert torch.allclose(y[1, 0, 0], x[1, 0, 0] * np.cos(1.0) - x[1, 0, 1] * np.sin(1.0))
    # scores depend on the distance alone
    q, k = torch.randn(1, 1, 8, dtype=plain.F), torch.randn(1, 1, 8, dtype=plain.F)
    at = lambda i, j: (plain.turn(q, torch.tensor([i]), f) * plain.turn(k, torch.tensor([j]), f)).sum()
    assert torch.allclose(at(9, 4), at(105, 100))
    # one key: the sink takes its share; a sink far below takes none
    v = torch.randn(1, 1, 3, dtype=plain.F)
    o = plain.causal_attention(q, k, v, 0.5, torch.zeros(1, dtype=plain.F))
    score = (q * k).sum() * 0.5
    assert torch.allclose(o[0, 0], v[0, 0] * torch.exp(score) / (1.0 + torch.exp(score)))
    assert torch.allclose(plain.causal_attention(q, k, v, 0.5, torch.full((1,), -1e9, dtype=plain.F))[0, 0], v[0, 0])
    # the convolution: the last column is the current token's, zeros before the start
    taps = torch.tensor([[1.0, 10.0, 100.0]], dtype=plain.F)
    signal = torch.tensor([[1.0], [2.0], [3.0]], dtype=plain.F)
    assert plain.short_convolution(signal, taps).flatten().tolist() == [100.0, 210.0, 321.0]
    assert plain.short_convolution(signal, taps, torch.tensor([0.5], dtype=plain.F)).flatten().tolist() == [100.5, 210.5, 321.5]
    # the delta rule writes what the memory lacks: after a token with beta 1 and no decay, reading with its key gives its value
    assert abs(plain.softplus(torch.tensor(0.0, dtype=plain.F)).item() - np.log(2.0)) < 1e-12
    assert plain.softplus(torch.tensor(100.0, dtype=plain.F)).item() == 100.0


SHORT = [33, 12, 40, 9, 2, 1, 27]


def cpu_runner(folder, *, page_size, num_pages, max_requests=4):
    from kairyu_b200.cache import CacheManager, CacheStorage
    from kairyu_b200.engine.runner import ModelRunner

    model, _ = load_model(folder, dtype="float32", device="cpu")
    layout = CacheLayout.from_slot_specs(model.cache_slot_specs())
    cache = CacheManager(layout, num_pages=num_pages, page_size=page_size, max_requests=max_requests)
    storage = CacheStorage(layout, num_pages=num_pages, page_size=page_size, max_requests=max_requests, dtype=model.dtype, device="cpu")
    return ModelRunner(model, cache, storage, max_model_len=512, decode_mode="eager", check_tables=True, debug_poison=True)


@pytest.mark.parametrize("name", ["shared_keys", "odd", "small_pages"])
def test_every_cut_on_the_cpu(name, tmp_path, monkeypatch):
    """Three state slots for seven requests, a pool for the cut's peak: pages and slots change hands."""
    import tapasun_torch_kernels

    tapasun_torch_kernels.install(monkeypatch)
    cfg, seed, page_size, ranks = CASES[name]
    weights = make_weights(cfg, seed, ranks)
    folder = write_model(cfg, weights, tmp_path / "m")
    requests = traces.make_requests(cfg["vocab"], SHORT, seed=3)
    expected = {n: plain.forward(cfg, weights, t).numpy() for n, t in requests.items()}
    cuts = {
        "whole": traces.trace_whole(requests),
        "tail": traces.trace_decode_tail(requests, 6),
        "chunks": traces.trace_chunks(requests, sizes=(5, 2, 11, 3)),
        "mixed": traces.trace_mixed(requests, seed=4, max_live=3),
    }
    pool = max(traces.peak_tokens(steps, round_to=page_size) for steps in cuts.values()) // page_size + 1
    runner = cpu_runner(folder, page_size=page_size, num_pages=pool, max_requests=3)
    for cut, steps in cuts.items():
        result = traces.run_in_process(runner, steps)
        assert len(result) == sum(SHORT)
        worst = max(relative_error(row, expected[n][p]) for (n, p), row in result.items())
        assert worst < 1e-4, (cut, worst)
        assert runner.cache.live_requests == 0


def test_generation_and_the_command_line_on_the_cpu(tmp_path, capsys, monkeypatch):
    """make-random, validate, generate: greedy tokens through the scheduler (a token budget that cuts the
    prompts) equal the plain model's own continuation."""
    import tapasun_torch_kernels
    from safetensors.torch import load_file

    from kairyu_b200.entrypoints import cli

    tapasun_torch_kernels.install(monkeypatch)
    cfg, _, _, ranks = CASES["shared_keys"]
    cfg = _with_ranks(cfg, ranks)
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    folder = tmp_path / "model"
    cli.main(["make-random", str(tmp_path / "config.json"), str(folder), "--seed", "5", "--dtype", "float32"])
    cli.main(["validate", str(folder)])
    assert "valid: Tapasun, 5 layers" in capsys.readouterr().out
    prompts = [[5, 17, 3, 9], [1], list(range(20, 60))]
    cli.main(["generate", str(folder), "--dtype", "float32", "--device", "cpu", "--temperature", "0", "--max-tokens", "6", "--num-pages", "24",
              "--page-size", "8", "--max-num-seqs", "2", "--max-num-batched-tokens", "16"]
             + [arg for p in prompts for arg in ("--prompt-token-ids", ",".join(map(str, p)))])
    lines = [json.loads(line) for line in capsys.readouterr().out.splitlines() if line.startswith("{")]
    weights = {n: t.float() for n, t in load_file(str(folder / "model.safetensors")).items()}
    for prompt, line in zip(prompts, lines):
        tokens = list(prompt)
        for _ in range(6):
            tokens.append(int(plain.forward(cfg, weights, tokens)[-1].argmax()))
        assert line["outputs"][0]["token_ids"] == tokens[len(prompt):]


def test_bench_configurations_build():
    """The sizes ``bench.py --design tapasun`` runs parse and build, and the dense decoder beside them is of equal size
    (weights within a sixth of each other)."""
    import math
    import sys
    from pathlib import Path

    sys.path.insert(0, str(Path(__file__).resolve().parent.parent))
    import bench_tapasun

    for size in bench_tapasun.SIZES.values():
        ours, _ = build_model(bench_tapasun.tapasun_config(size), dtype="bfloat16", device="meta")
        dense_model, _ = build_model(bench_tapasun.dense_config(size), dtype="bfloat16", device="meta")
        count = lambda model: sum(math.prod(spec.shape) for spec in model.tensor_specs())
        assert 1.0 <= count(ours) / count(dense_model) < 7 / 6
        assert ours.graph_safe() and len(ours.schedule) == bench_tapasun.LAYERS
