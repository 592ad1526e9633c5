"""Mapalorn on the GPU against the plain implementation in ``mapalorn_plain.py``: every mechanism alone, whole
prompts against token-by-token decoding, portions down to two tokens, unequal requests in one batch over a pool
so small that pages are used again, keys and sinks made to stand out (far away, at page borders, beside the
first tokens), long decoding, and greedy generation through ``LLM.generate``."""

import types

import numpy as np
import pytest
import torch

import mapalorn_plain as plain
import traces
from mapalorn_cases import CASES, config, dense, gated, latent, layer, make_weights, moe, relative_error, write_model

pytestmark = pytest.mark.gpu

# rms of the logits' error over rms of the logits, per position
FP32_BOUND = 1e-4
BF16_BOUND = 5e-2
LENGTHS = [70, 45, 101, 38, 64, 83, 9, 55, 2, 1]


def expected_rows(cfg, weights, requests):
    return {name: plain.forward(cfg, weights, tokens).numpy() for name, tokens in requests.items()}


def make_runner(folder, dtype, *, page_size, num_pages, max_requests=4, decode_mode="eager", max_model_len=512):
    from kairyu_b200.cache import CacheLayout, CacheManager, CacheStorage
    from kairyu_b200.engine.engine import load_model
    from kairyu_b200.engine.runner import ModelRunner

    model, _ = load_model(folder, dtype=dtype, device="cuda")
    layout = CacheLayout.from_slot_specs(model.cache_slot_specs())
    cache = CacheManager(layout, num_pages=num_pages, page_size=page_size, max_requests=max_requests)
    storage = CacheStorage(layout, num_pages=num_pages, page_size=page_size, max_requests=max_requests, dtype=model.dtype, device="cuda")
    return ModelRunner(model, cache, storage, max_model_len=max_model_len, decode_mode=decode_mode, max_graph_batch=max_requests,
                       check_tables=True, debug_poison=True)


def beyond(result, expected, bound):
    errors = [(name, position, relative_error(row, expected[name][position])) for (name, position), row in result.items()]
    return [entry for entry in errors if not entry[2] < bound][:12]


def judge(result, expected, dtype, what=""):
    """float32: every position within the bound.  bfloat16: the weights make the softmax pick single keys and the
    routers choose among close scores, so that faults show; rounding to bfloat16 then costs a few per cent at a
    typical position and much more where a close call turns.  A fault moves the median position beyond the bound or
    many positions far beyond it (test_mapalorn_cpu.py: test_the_bounds_see_each_fault), so the median is held to
    BF16_BOUND and few positions may be far off."""
    errors = np.array([relative_error(row, expected[name][position]) for (name, position), row in result.items()])
    if str(dtype).endswith("float32"):
        print(f"[mapalorn] {what} float32: worst {errors.max():.3e} bound {FP32_BOUND:.1e}")
        assert errors.max() < FP32_BOUND, (what, errors.max(), beyond(result, expected, FP32_BOUND))
    else:
        far = float((errors >= 3 * BF16_BOUND).mean())
        print(f"[mapalorn] {what} bfloat16: median {np.median(errors):.3e} worst {errors.max():.3e} far off {far:.3f} bound {BF16_BOUND:.1e}")
        assert np.median(errors) < BF16_BOUND and far <= 0.10, (what, np.median(errors), far, beyond(result, expected, 3 * BF16_BOUND))


@pytest.fixture(scope="module", params=list(CASES))
def case(request, tmp_path_factory):
    cfg, seed, page_size = CASES[request.param]
    weights = make_weights(cfg, seed)
    folder = write_model(cfg, weights, tmp_path_factory.mktemp(request.param))
    requests = traces.make_requests(cfg["vocab"], LENGTHS, seed=seed + 100)
    return dict(name=request.param, cfg=cfg, page_size=page_size, weights=weights, folder=folder, requests=requests,
                expected=expected_rows(cfg, weights, requests))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("decode_mode", ["eager", "cuda_graph"])
def test_every_cut_matches_plain(case, dtype, decode_mode):
    """Whole prompts, tails decoded token by token, portions of changing size and mixed batches, one after the
    other on one engine whose pool holds far less than all requests (pages change hands; pages that went back
    are overwritten before the next step)."""
    requests = case["requests"]
    cuts = {
        "whole": traces.trace_whole(requests),
        "tail": traces.trace_decode_tail(requests, 32),
        "chunks": traces.trace_chunks(requests),
        "twos": traces.trace_chunks(requests, sizes=(2,)),
        "mixed": traces.trace_mixed(requests, seed=5),
    }
    pool = max(traces.peak_tokens(steps) for steps in cuts.values()) // case["page_size"] + 1
    total = sum(len(t) for t in requests.values())
    assert pool * case["page_size"] < total
    runner = make_runner(case["folder"], dtype, page_size=case["page_size"], num_pages=pool, decode_mode=decode_mode)
    results = {}
    for cut, steps in cuts.items():
        results[cut] = traces.run_in_process(runner, steps)
        assert len(results[cut]) == total
        judge(results[cut], case["expected"], dtype, f"{case['name']} {decode_mode} {cut}")
        assert runner.cache.live_requests == 0
    if decode_mode == "cuda_graph":
        assert runner.counters["graph_replays"] > 0
    if dtype == "float32":
        # no 32-bit sum depends on the batch or on where a prompt was cut
        for cut in ("tail", "chunks", "twos", "mixed"):
            different = [key for key, row in results["whole"].items() if not np.array_equal(row, results[cut][key])]
            assert not different, (cut, different[:12])


MIXERS = {
    "latent narrow": latent(2, 16, 16, 16, 16, 0.3),                 # rows of 32: tensor cores in bfloat16
    "latent rows of 128": latent(5, 32, 48, 24, 80, 0.2, base=5000.0),
    "latent rows of 256": latent(3, 64, 64, 128, 192, 0.12),
    "latent many heads": latent(20, 16, 8, 16, 40, 0.3),             # more heads than one attention call takes
    "latent odd": latent(3, 10, 6, 14, 26, 0.4, base=77.0),          # rows that are no multiple of 16: 32-bit arithmetic in both modes
    "latent one head": latent(1, 24, 2, 8, 30, 0.3),
    "latent rows of 64": latent(4, 16, 16, 16, 48, 0.3),             # the tcgen05 and TMA-fed kernels over rows that are keys and values at once
    "latent rows of 192": latent(2, 32, 32, 32, 160, 0.2, base=3000.0),
    "latent rows of 96": latent(3, 48, 32, 16, 64, 0.2),             # padded to 128 in shared memory
    "gated equal widths": gated(4, 2, 32, 32, 0.25, 16),             # tensor cores in bfloat16
    "gated heads of 128": gated(2, 1, 128, 128, 0.1, 128),
    "gated heads of 64": gated(4, 1, 64, 64, 0.2, 32, base=2000.0),
    "gated heads of 96": gated(6, 3, 96, 96, 0.15, 48),
    "gated heads of 256": gated(2, 2, 256, 256, 0.08, 64),
    "gated sixteen a group": gated(16, 1, 16, 16, 0.3, 8, base=300.0),
    "gated wider values": gated(3, 3, 16, 40, 0.4, 16),              # 32-bit arithmetic in both modes
    "gated narrower values": gated(6, 2, 48, 16, 0.2, 24),
    "gated two columns turn": gated(2, 1, 10, 10, 0.5, 2),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("kind", list(MIXERS))
def test_one_mixer_alone(kind, dtype, tmp_path):
    """A model of one layer without feed-forward, so that the mixer is all that mixes: a prompt of 230 tokens in one
    step, then 90 tokens decoded one by one through a graph."""
    cfg = config(40, 53, [layer(MIXERS[kind], None)])
    weights = make_weights(cfg, 7)
    folder = write_model(cfg, weights, tmp_path / "m")
    tokens = traces.make_requests(53, [320], seed=3)["r0"]
    expected = {"r0": plain.forward(cfg, weights, tokens).numpy()}
    steps = traces.trace_decode_tail({"r0": tokens}, 90)
    runner = make_runner(folder, dtype, page_size=16, num_pages=24, decode_mode="cuda_graph")
    result = traces.run_in_process(runner, steps)
    judge(result, expected, dtype, f"{kind} alone")


def _attention_reference(q, k, v, scale, sinks, positions):
    """o [len(positions), heads * dv] from whole-sequence q [L, H, D], k [L, G, D], v [L, G, DV], sinks [H] (64-bit)."""
    heads, group = q.shape[1], q.shape[1] // k.shape[1]
    kk, vv = k.repeat_interleave(group, dim=1), v.repeat_interleave(group, dim=1)
    scores = torch.einsum("ihd,jhd->hij", q, kk) * scale
    p = plain.causal_softmax_with_sink(scores, sinks)
    return torch.einsum("hij,jhd->ihd", p, vv).reshape(q.shape[0], heads * v.shape[2])[positions]


@pytest.mark.parametrize("variant", ["float32 generic", "bfloat16 generic", "bfloat16 tensor cores", "bfloat16 tensor cores, keys split",
                                     "bfloat16 tensor cores, two tiles a block"])
@pytest.mark.parametrize("sizes", [(4, 2, 32, 16), (16, 1, 128, 64), (3, 3, 64, 128), (8, 2, 128, 16), (2, 1, 256, 16), (4, 1, 192, 32), (6, 2, 96, 8)])
def test_keys_and_sinks_that_stand_out(variant, sizes):
    """The attention kernels alone over a 900-token sequence in shuffled pages.  Among keys whose scores are near
    zero, one key a query is given a score of 18: at distances 0 and 1, at a page's last and first place, at the
    sequence's first tokens and hundreds of tokens away; leaving it out moves the result by half its size.  The sinks
    are as large as those scores (some heads) or far below (others), so that a sink that is left out, scaled or counted
    twice changes every weight.  With a gate.  The same queries run as one prompt, as a portion that starts in the middle
    of a page beside single tokens of other lengths, and as single tokens alone.  Heads of 64 and 128 take the tcgen05
    kernels for prompt portions: one query tile a block, a tile's keys split over three blocks whose parts a second kernel
    joins, and two query tiles a block; the other sizes and single tokens the mma.sync kernels."""
    from kairyu_b200 import kernels
    from kairyu_b200.engine.workspace import Workspace

    dtype = torch.float32 if variant.startswith("float32") else torch.bfloat16
    H, G, D, page = sizes[0], sizes[1], sizes[2], sizes[3]
    L, scale = 900, 0.5
    gen = torch.Generator().manual_seed(11)
    q = torch.randn(L, H, D, generator=gen) * 0.1
    k = torch.randn(L, G, D, generator=gen) * 0.1
    v = torch.randn(L, G, D, generator=gen)
    gate = torch.randn(L, H * D, generator=gen) * 2
    sinks = torch.tensor([18.0 if h % 2 == 0 else -3.0 for h in range(H)]) + torch.randn(H, generator=gen) * 0.3
    wanted = []
    for index, distance in enumerate([0, 1, page - 1, page, page + 1, 600, None, None]):
        at = 880 - 9 * index  # positions that are no multiple of anything
        key = at - distance if distance is not None else index - 6  # None: the sequence's first and second token
        u = torch.nn.functional.normalize(torch.randn(D, generator=gen), dim=0) * 6.0
        q[at] = u
        k[key] = u
        wanted.append(at)
    wanted += [0, 1, 2, page - 1, page]  # the first tokens: few keys beside the sink
    q, k, v, gate = (t.to(dtype).double() for t in (q, k, v, gate))  # what the kernels are given, exactly
    want = _attention_reference(q, k, v, scale, sinks.double(), wanted) * torch.sigmoid(gate[wanted])
    for wrong in (sinks * scale, sinks + float(np.log(2.0)), torch.full_like(sinks, -1e9)):  # the sinks matter
        assert (_attention_reference(q, k, v, scale, wrong.double(), wanted) * torch.sigmoid(gate[wanted]) - want).abs().max() > 0.2

    pages = torch.randperm(L // page + 1, generator=gen) + 1
    k_cache = torch.zeros(len(pages) + 1, page, G, D, dtype=dtype, device="cuda")
    v_cache = torch.zeros(len(pages) + 1, page, G, D, dtype=dtype, device="cuda")
    for position in range(L):
        k_cache[pages[position // page], position % page] = k[position].to(dtype)
        v_cache[pages[position // page], position % page] = v[position].to(dtype)
    i32 = dict(dtype=torch.int32, device="cuda")
    sinks_gpu = sinks.cuda()
    bound = 2e-5 if dtype == torch.float32 else 3e-2
    tile = kernels.attention_prefill_tile_rows(D)

    def run(q_rows, gate_rows, positions, row_ids, table, seq_lens, qo_indptr):
        out = torch.zeros(q_rows.shape[0], H * D, dtype=dtype, device="cuda")
        if variant.endswith("generic"):
            # the kernel of the gated mixer (one map, sinks, gate) and the kernel of the latent mixer (sinks; the gate applied here)
            kernels.diff_attention_generic(q_rows, out, k_cache, v_cache, positions=positions, row_ids=row_ids, block_table=table, num_q_heads=H,
                                           maps=1, scale=scale, window=0, sinks=sinks_gpu, gate=gate_rows)
            other = torch.zeros_like(out)
            kernels.paged_attention_generic(q_rows, other, k_cache, v_cache, positions=positions, row_ids=row_ids, block_table=table,
                                            num_q_heads=H, scale=scale, window=0, sinks=sinks_gpu)
            other = other.float() * torch.sigmoid(gate_rows.float())
            assert (other - out.float()).abs().max() < bound
            return out
        rows = len(seq_lens)
        counts = [qo_indptr[r + 1] - qo_indptr[r] for r in range(rows)]
        tile_rows = [r for r in range(rows) if counts[r] > 1 for _ in range(0, counts[r], tile)]
        tile_starts = [s for r in range(rows) if counts[r] > 1 for s in range(0, counts[r], tile)]
        single = [r for r in range(rows) if counts[r] == 1]
        common = dict(seq_lens=torch.tensor(seq_lens, **i32), block_table=table, num_q_heads=H, scale=scale, sinks=sinks_gpu, gate=gate_rows)
        if tile_rows:
            extra = {}
            if variant.endswith("keys split"):
                extra = dict(workspace=Workspace("cuda"), num_splits=3, max_seq_len=max(seq_lens))
            wide = kernels.attention_prefill_wide_tile_rows(D)
            if variant.endswith("two tiles a block") and wide:
                wide_rows = [r for r in range(rows) if counts[r] > 1 for _ in range(0, counts[r], wide)]
                wide_starts = [s for r in range(rows) if counts[r] > 1 for s in range(0, counts[r], wide)]
                extra = dict(wide_tiles=(len(wide_rows), torch.tensor(wide_rows, **i32), torch.tensor(wide_starts, **i32)), two_tiles=True,
                             max_seq_len=max(seq_lens))
            kernels.attention_prefill_mma(q_rows, out, k_cache, v_cache, qo_indptr=torch.tensor(qo_indptr, **i32), tile_rows=torch.tensor(tile_rows, **i32),
                                          tile_starts=torch.tensor(tile_starts, **i32), num_tiles=len(tile_rows), **extra, **common)
        if single:
            # the TMA-fed kernel (heads of 64 and up): as many splits as it chooses, three (a merge kernel divides), or one (it divides itself)
            splits = 3 if variant.endswith("keys split") else 1 if variant.endswith("two tiles a block") else None
            kernels.attention_decode_mma(q_rows, out, k_cache, v_cache, decode_rows=torch.tensor(single, **i32), num_splits=splits,
                                         decode_tokens=torch.tensor([qo_indptr[r] for r in single], **i32), num_rows=len(single),
                                         max_seq_len=max(seq_lens), workspace=Workspace("cuda"), **common)
        return out

    flat_q = q.reshape(L, H * D).to(dtype).cuda()
    flat_gate = gate.to(dtype).cuda()
    table = pages.to(torch.int32).cuda()[None, :].contiguous()
    got = run(flat_q, flat_gate, torch.arange(L, **i32), torch.zeros(L, **i32), table, [L], [0, L])
    assert (got[wanted].double().cpu() - want).abs().max() < bound
    start = 613
    rows_q = torch.cat([flat_q[start:], flat_q[wanted]])
    rows_gate = torch.cat([flat_gate[start:], flat_gate[wanted]])
    positions = torch.tensor(list(range(start, L)) + wanted, **i32)
    row_ids = torch.tensor([0] * (L - start) + list(range(1, len(wanted) + 1)), **i32)
    tables = table.repeat(len(wanted) + 1, 1).contiguous()
    indptr = [0, L - start] + [L - start + n + 1 for n in range(len(wanted))]
    got = run(rows_q, rows_gate, positions, row_ids, tables, [L] + [at + 1 for at in wanted], indptr)
    in_portion = [at - start for at in wanted if at >= start]
    assert (got[in_portion].double().cpu() - want[[n for n, at in enumerate(wanted) if at >= start]]).abs().max() < bound
    assert (got[L - start :].double().cpu() - want).abs().max() < bound


def _step_context(tokens, dtype):
    from kairyu_b200.engine.workspace import Workspace
    from kairyu_b200.parts import StepContext

    return StepContext(num_tokens=tokens, num_rows=1, dtype=dtype, token_ids=None, positions=None, row_ids=None, qo_indptr=None, seq_lens=None,
                       write_from=None, state_slots=None, block_tables={}, host_qo_indptr=(), host_seq_lens=(), workspace=Workspace("cuda"))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("sizes", [
    # width, experts, top, ff, shared ff (None: no shared expert), tokens
    (40, 5, 3, 24, 16, 33), (64, 6, 1, 16, 64, 3), (72, 4, 4, 40, None, 16), (136, 3, 2, 200, 8, 11), (24, 1, 1, 70, 70, 130),
    (96, 16, 1, 96, 96, 700), (50, 2, 2, 18, 10, 300),
])
def test_feed_forwards_alone(sizes, dtype):
    """The mixture part by itself against the plain mixture (the chosen experts' scores multiply their INPUTS; the shared
    expert behind its gate), the router's choices one by one, and the dense part with products far beyond its limit on
    both sides (a gate branch clamped from below, an up branch not clamped, a missing one in (u + 1) each move it by
    tenths)."""
    from kairyu_b200.parts import FEED_FORWARDS, PartSpec

    width, experts, top, ff, shared, tokens = sizes
    mlp = moe(experts, top, ff, shared=shared)
    cfg = config(width, 11, [layer(gated(1, 1, 8, 8, 1.0, 4), mlp), layer(gated(1, 1, 8, 8, 1.0, 4), dense(ff, 0.75))])
    weights = make_weights(cfg, 3)
    g = torch.Generator().manual_seed(9)
    x = torch.randn(tokens, width, generator=g).to(torch.bfloat16).float()
    ctx = _step_context(tokens, dtype)
    bound = 1e-5 if dtype == torch.float32 else 3e-2

    part = FEED_FORWARDS.build(PartSpec(
        "moe", prefix="l0.mlp", hidden_size=width, intermediate_size=ff, num_experts=experts, top=top, routing="scores", score_function="sigmoid",
        correction=False, weight_on="input", limit=None, alpha=1.0, shift=0.0, router_bias=False,
        shared_expert=dict(intermediate_size=shared, gate=True) if shared is not None else None), dtype=dtype, device="cuda")
    part.load({n: t.to(dtype).cuda() for n, t in weights.items() if n.startswith("l0.mlp")})
    w = plain.sub(weights, "l0.mlp", torch.float64)
    want = plain.expert_mixture(x.double(), w, mlp)
    got = part.forward(x.to(device="cuda", dtype=dtype), ctx).float().cpu().double()
    scores = torch.sigmoid(x.double() @ w["router"].T)
    if dtype == torch.float32 or top == experts:
        assert (got - want).abs().max() < bound * want.abs().max()
    else:  # bfloat16 may turn a close call between two experts: those tokens aside
        ranked = scores.sort(dim=1, descending=True).values
        clear = (ranked[:, top - 1] - ranked[:, top]) > 0.02
        assert clear.float().mean() > 0.5
        assert (got - want)[clear].abs().max() < bound * want.abs().max()

    unit = FEED_FORWARDS.build(PartSpec("gated_unit", prefix="l1.mlp", hidden_size=width, intermediate_size=ff, limit=0.75, alpha=1.702, shift=1.0),
                               dtype=dtype, device="cuda")
    unit.load({n: t.to(dtype).cuda() for n, t in weights.items() if n.startswith("l1.mlp")})
    w = plain.sub(weights, "l1.mlp", torch.float64)
    big = x * 3.0
    assert ((big.double() @ w["gate"].T) < -0.75).float().mean() > 0.2 and ((big.double() @ w["up"].T).abs() > 0.75).float().mean() > 0.4
    want = plain.dense_ff(big.double(), w, 0.75)
    got = unit.forward(big.to(device="cuda", dtype=dtype), ctx).float().cpu().double()
    assert (got - want).abs().max() < bound * want.abs().max()
    both_sides = ((big.double() @ w["gate"].T).clamp(-0.75, 0.75))
    other = (both_sides * torch.sigmoid(1.702 * both_sides) * ((big.double() @ w["up"].T).clamp(-0.75, 0.75) + 1)) @ w["down"].T
    assert (other - want).abs().max() > 5 * bound * want.abs().max()


def _projection_case(kernels, plain, g, dtype, tokens, page, heads, kvh, dim, vdim, rot, spare, block_table, row_ids, where, write_from):
    k_off, v_off = heads * dim, heads * dim + kvh * dim
    angles = plain.angles(torch.arange(64), rot, 100.0)
    cos, sin = angles.cos().float().cuda(), angles.sin().float().cuda()
    qw = (1 + 0.2 * torch.randn(heads * dim, generator=g)).to(torch.bfloat16)
    kw = (1 + 0.2 * torch.randn(kvh * dim, generator=g)).to(torch.bfloat16)
    for interleaved, turn in ((False, plain.rotate_halves), (True, plain.rotate_interleaved)):
        source = torch.randn(tokens, v_off + kvh * vdim + spare, generator=g).to(dtype)
        packed = source.clone().cuda()
        k_cache = torch.zeros(9, page, kvh, dim, dtype=dtype, device="cuda")
        v_cache = torch.zeros(9, page, kvh, vdim, dtype=dtype, device="cuda")
        kernels.projection_norm_rope_write(
            packed, num_q_heads=heads, num_kv_heads=kvh, head_dim=dim, value_dim=vdim, k_offset=k_off, v_offset=v_off, positions=where, row_ids=row_ids,
            q_norm_weight=qw.to(dtype).cuda(), k_norm_weight=kw.to(dtype).cuda(), eps=1e-5, cos=cos, sin=sin, interleaved=interleaved,
            block_table=block_table, write_from=write_from, k_cache=k_cache, v_cache=v_cache)
        s = source.double()
        q_want = turn(plain.rms_norm(s[:, :k_off], qw.double(), 1e-5).view(tokens, heads, dim), where.cpu(), rot, 100.0).reshape(tokens, -1)
        k_want = turn(plain.rms_norm(s[:, k_off:v_off], kw.double(), 1e-5).view(tokens, kvh, dim), where.cpu(), rot, 100.0).reshape(tokens, -1)
        tolerance = 1e-5 if dtype == torch.float32 else 0.03
        assert (packed[:, :k_off].cpu().double() - q_want).abs().max() < tolerance
        assert torch.equal(packed[:, v_off:].cpu(), source[:, v_off:])
        for t in range(tokens):
            position, row = int(where[t]), int(row_ids[t])
            slot = (int(block_table[row, position // page]), position % page)
            if position >= int(write_from[row]):
                assert (k_cache[slot].flatten().cpu().double() - k_want[t]).abs().max() < tolerance
                assert torch.equal(v_cache[slot].flatten().cpu(), source[t, v_off : v_off + kvh * vdim])
            else:
                assert not k_cache[slot].any() and not v_cache[slot].any()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_small_kernels(dtype):
    """The layer norm with two pending sums and on listed rows, the norm over a whole projection with both rotary layouts
    and the page write of keys and values of different widths, and the latent row's norm, rotation and page write."""
    from kairyu_b200 import kernels

    g = torch.Generator().manual_seed(4)
    tokens, width = 37, 72
    weight = (1 + 0.1 * torch.randn(width, generator=g)).to(torch.bfloat16)
    bias = (0.3 * torch.randn(width, generator=g)).to(torch.bfloat16)
    x = torch.randn(tokens, width, generator=g) * 3 + 1.5  # a mean that is not zero: the variance is of the deviations
    d1 = torch.randn(tokens, width, generator=g).to(dtype)
    d2 = torch.randn(tokens, width, generator=g).to(dtype)
    residual = x.clone().cuda()
    out = torch.empty(tokens, width, dtype=dtype, device="cuda")
    kernels.layernorm(residual, weight.to(dtype).cuda(), bias.to(dtype).cuda(), 1e-5, out, delta=d1.cuda(), delta2=d2.cuda())
    total = x.double() + d1.double() + d2.double()
    assert (residual.cpu().double() - total).abs().max() < 1e-5  # the sums are kept in 32-bit
    want = plain.layer_norm(total, weight.double(), bias.double(), 1e-5)
    assert (out.cpu().double() - want).abs().max() < (1e-5 if dtype == torch.float32 else 0.03)
    rows = torch.tensor([5, 0, 36], dtype=torch.int32, device="cuda")
    few = torch.empty(3, width, dtype=dtype, device="cuda")
    kernels.layernorm(residual, weight.to(dtype).cuda(), bias.to(dtype).cuda(), 1e-5, few, rows=rows)
    assert torch.equal(few, out[rows.long()])

    page = 8
    block_table = torch.tensor([[3, 1, 7, 5, 2, -1], [4, 6, 8, -1, -1, -1]], dtype=torch.int32, device="cuda")
    row_ids = torch.tensor([0] * 30 + [1] * 7, dtype=torch.int32, device="cuda")
    where = torch.tensor(list(range(5, 35)) + list(range(11, 18)), dtype=torch.int32, device="cuda")
    write_from = torch.tensor([8, 0], dtype=torch.int32, device="cuda")  # row 0 only reads its first page
    # widths that are no whole 16 bytes (an element a thread), and rows of whole 16-byte groups (eight a thread in bfloat16):
    # part of a head rotated, and all of it
    for heads, kvh, dim, vdim, rot, spare in ((3, 1, 20, 12, 8, 5), (3, 2, 32, 16, 16, 8), (2, 1, 64, 24, 64, 0), (4, 4, 16, 8, 8, 16)):
        _projection_case(kernels, plain, g, dtype, tokens, page, heads, kvh, dim, vdim, rot, spare, block_table, row_ids, where, write_from)

    # the latent row: [heads * (dim + rot) query | rank latent | rot key part]
    heads, dim, rot, rank = 3, 10, 6, 18
    q_size, row_width = heads * (dim + rot), rank + rot
    source = torch.randn(tokens, q_size + row_width, generator=g).to(dtype)
    packed = source.clone().cuda()
    norm_w = (1 + 0.2 * torch.randn(rank, generator=g)).to(torch.bfloat16)
    angles = plain.angles(torch.arange(64), rot, 1000.0)
    cos, sin = angles.cos().float().cuda(), angles.sin().float().cuda()
    cache = torch.zeros(9, page, 1, row_width, dtype=dtype, device="cuda")
    q_out = torch.zeros(tokens, heads * row_width, dtype=dtype, device="cuda")
    kernels.latent_norm_write(packed, q_size, rank, norm_w.to(dtype).cuda(), 1e-5, cache, positions=where, row_ids=row_ids, block_table=block_table,
                              write_from=write_from, rot_dim=rot, cos=cos, sin=sin, interleaved=True, q_out=q_out, num_heads=heads, q_head_width=dim + rot)
    s = source.double()
    latent_want = plain.rms_norm(s[:, q_size : q_size + rank], norm_w.double(), 1e-5)
    key_want = plain.rotate_interleaved(s[:, None, q_size + rank :], where.cpu(), rot, 1000.0)[:, 0]
    q_rot_want = plain.rotate_interleaved(s[:, :q_size].view(tokens, heads, dim + rot)[..., dim:], where.cpu(), rot, 1000.0)
    tolerance = 1e-5 if dtype == torch.float32 else 0.03
    assert (q_out.view(tokens, heads, row_width)[..., rank:].cpu().double() - q_rot_want).abs().max() < tolerance
    for t in range(tokens):
        position, row = int(where[t]), int(row_ids[t])
        slot = (int(block_table[row, position // page]), position % page)
        if position >= int(write_from[row]):
            assert (cache[slot].flatten().cpu().double() - torch.cat([latent_want[t], key_want[t]])).abs().max() < tolerance
        else:
            assert not cache[slot].any()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_engine(case, dtype):
    """``LLM.generate`` with a token budget that cuts the prompts into portions and batches them with decoding
    requests; greedy tokens against the plain model's own greedy continuation."""
    from kairyu_b200.entrypoints.llm import LLM
    from kairyu_b200.entrypoints.prompt import TokensPrompt
    from kairyu_b200.sampling.params import SamplingParams

    cfg, weights = case["cfg"], case["weights"]
    prompts = [tokens for tokens in list(case["requests"].values())[:6]]
    new = 12
    llm = LLM(model=str(case["folder"]), dtype=dtype, num_pages=64 * 16 // case["page_size"], page_size=case["page_size"], max_num_batched_tokens=24,
              max_num_seqs=4, max_model_len=256)
    outputs = llm.generate([TokensPrompt(prompt_token_ids=tokens) for tokens in prompts],
                           SamplingParams(temperature=0.0, max_tokens=new, ignore_eos=True), use_tqdm=False)
    for tokens, output in zip(prompts, outputs):
        got = list(output.outputs[0].token_ids)
        assert len(got) == new
        # teacher-forced: at every step the engine's choice is (nearly) the plain model's best given the engine's own history
        logits = plain.forward(cfg, weights, list(tokens) + got).numpy()
        close = []
        for step, token in enumerate(got):
            row = logits[len(tokens) - 1 + step]
            close.append((row.max() - row[token]) / row.std())
        if dtype == "float32":
            assert max(close) <= 1e-4, close
        else:  # bfloat16 may turn a close call: most steps agree
            assert np.mean(np.array(close) <= 0.15) >= 0.8, close


def test_trace_program(case, tmp_path):
    """The same through ``bin/trace_run``: a pool for the trace's peak."""
    steps = traces.trace_mixed(case["requests"], seed=9)
    result = traces.run_program(case["folder"], tmp_path / "out", steps, dtype="float32", max_tokens=traces.peak_tokens(steps), vocab=case["cfg"]["vocab"],
                                extra=["--page-size", str(case["page_size"])])
    worst = max(relative_error(row, case["expected"][name][position]) for (name, position), row in result.items())
    assert worst < FP32_BOUND
