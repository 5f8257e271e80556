"""Rizovik in the engine against the plain implementation (tests/plain_rizovik.py): whole models under every
way of cutting the work, in 32-bit and in bfloat16: whole prompts, long decoding one token at a time, portions
down to two tokens (and single first tokens), mixed batches of unequal requests with so few pages and slots
that they are used again (pages given back are filled with NaN), the stream after every layer, and greedy
generation through the engine's own entry point and scheduler.  The kernels of its mechanisms alone, with
inputs made so that a fault shows, are in test_rizovik_kernels_gpu.py."""

import functools
import json

import numpy as np
import pytest
import torch

from plain_rizovik import F64, MIXERS, forward, rms_norm, routed_feed_forward
from replay_util import (collect, peak_tokens, random_tokens, tolerance, trace_batched_tail, trace_mixed,
                         trace_portions, trace_tail, trace_whole)
from rizovik_models import CONFIGS, PAGE_SIZE, delta, kept, model, moe, pooled, read_model, rot, without_choice, write_model

pytestmark = pytest.mark.gpu

DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}
# A routed layer's choice is a step function of its input: where two logits lie closer than the input's
# rounding moves them, another expert runs and the logits are another computation's.  The plain side
# reports every token's margin, and a request is compared up to its first close call only.  In float32
# that is rare.  In bfloat16 it would be every few tokens, so the bfloat16 models take every expert
# (``without_choice``: the weights stay each token's own); the choice itself is float32's to test, and
# one bfloat16 model keeps it and is compared as far as its margins allow.
CLOSE_CALL = {"float32": 2e-4, "bfloat16": 0.05}

ONE_LAYER = {
    # single layers: the mechanism alone, through the engine
    "pooled": model(50, 48, 0.8, 1e-6, [pooled(3, 1, 16, 24, 11, 4, rot(40.0, 12), 0.3, None)]),
    "kept": model(50, 40, 1.3, 1e-6, [kept(4, 2, 12, 20, 13, 5, rot(90.0, 12, factor=3.0), 0.4, None)]),
    "delta": model(50, 56, 0.6, 1e-5, [delta(2, 1, 40, 36, 4, None)]),
    "routed": model(50, 40, 0.9, 1e-6, [delta(1, 1, 8, 8, 2, moe(10, 2, 24)), kept(2, 1, 8, 8, 4, 2, rot(10.0, 8), 0.5, moe(3, 1, 13))]),
}
ALL = {**CONFIGS, **ONE_LAYER}


def config_for(name: str, dtype: str, keep_choice: bool = False) -> dict:
    return ALL[name] if dtype == "float32" or keep_choice else without_choice(ALL[name])


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    made = {}

    def get(name: str, dtype: str, keep_choice: bool = False):
        key = (name, dtype, keep_choice)
        if key not in made:
            made[key] = write_model(tmp_path_factory.mktemp(f"rizovik_{name}_{dtype}"), config_for(name, dtype, keep_choice),
                                    seed=23 + sum(map(ord, name)), dtype=DTYPES[dtype])
        return made[key]

    return get


@functools.lru_cache(maxsize=256)
def _plain(folder: str, tokens: tuple):
    """(logits [T, vocab], every position's smallest routing margin over the routed layers; inf without any)."""
    config, weights = read_model(folder)
    margins: list = []
    logits = forward(config, weights, list(tokens), margins=margins).numpy()
    smallest = np.min(np.array([m.numpy() for m in margins]), axis=0) if margins else np.full(len(tokens), np.inf)
    return logits, smallest


@functools.lru_cache(maxsize=256)
def _plain_with_roundings(folder: str, tokens: tuple):
    """The plain model with what every part reads and puts out rounded to bfloat16, and nothing else: how far
    rounding alone moves the logits of this model and these tokens.  Behind every part stands a norm, which
    magnifies a rounding where the part's output is small against its rounding step, so for some drawn sizes
    this is many times the usual bound."""
    config, weights = read_model(folder)
    w = {name: t.to(F64) for name, t in weights.items()}
    eps, mult = float(config["norm"]["eps"]), float(config["residual_mult"])
    rounded = lambda t: t.to(torch.bfloat16).to(F64)
    x = w["embed"][torch.tensor(list(tokens), dtype=torch.long)]
    for index, layer in enumerate(config["layers"]):
        prefix = f"l{layer.get('weights_of', index)}"
        mixed = rounded(MIXERS[layer["type"]](rounded(x), w, f"{prefix}.mix", layer["mixer"], eps))
        x = x + mult * rms_norm(mixed, w[f"{prefix}.norm1"], eps)
        if layer.get("mlp") is not None:
            y = rounded(routed_feed_forward(rounded(x), w, f"{prefix}.mlp", layer["mlp"]))
            x = x + mult * rms_norm(y, w[f"{prefix}.norm2"], eps)
    return (rms_norm(x, w["final.norm"], eps) @ w["embed"].T).numpy()


def replay(folder, dtype, steps, page_size, max_requests=4, graphs=True):
    from zephyr_b200.engine.replay import TraceReplayer

    replayer = TraceReplayer(folder, dtype, peak_tokens(steps, max(64, page_size)), page_size=page_size,
                             max_requests=max_requests)
    replayer.runner.poison_freed_pages = True
    replayer.runner.use_cuda_graphs = graphs
    outputs = {}
    for step in steps:
        result = replayer.step(step)
        if result is not None:
            outputs[step["step"]] = result
        replayer.runner.manager.check_invariants()
    return outputs


def assert_rows_match(rows, requests, folder, dtype, what, least=0.5, close_call=None, roundings=False):
    """Every compared row of logits within its bound (``replay_util.tolerance``) in float32; in bfloat16 no
    row beyond four bounds and at most one in ten beyond one (every part's output passes a norm, which
    magnifies roundings where the output's spread is small).  A fault of a mask, a page, a state or a routed
    token moves logits by tens to hundreds of bounds.  ``roundings`` (bfloat16, sizes drawn at random, which
    the same test also runs in float32 within one bound): no row beyond six bounds and at most one in six
    beyond one, or three and five times what rounding the parts' inputs and outputs alone does to the plain
    model on the same rows if that is more (``_plain_with_roundings``; the engine rounds in more places:
    queries, cached keys and values, what an expert keeps between its two products; with a large score scale
    the rounding of queries and keys outweighs the rest)."""
    ratios, skipped, alone = {}, 0, {}
    for (rid, position), got in sorted(rows.items()):
        expected, margins = _plain(str(folder), tuple(requests[rid]))
        close = np.nonzero(margins < (close_call or CLOSE_CALL[dtype]))[0]
        if close.size and position >= close[0]:
            skipped += 1
            continue
        assert np.isfinite(got).all(), f"{what}: non-finite logits for {rid} at {position}"
        ratios[(rid, position)] = float(np.abs(got.astype(np.float64) - expected[position]).max()) / tolerance(dtype, expected[position])
        if roundings and dtype == "bfloat16":
            moved = _plain_with_roundings(str(folder), tuple(requests[rid]))[position]
            alone[(rid, position)] = float(np.abs(moved - expected[position]).max()) / tolerance(dtype, expected[position])
    assert len(ratios) >= least * len(rows), f"{what}: {skipped} of {len(rows)} rows lie behind a close routing call"
    over = [key for key, ratio in ratios.items() if ratio > 1.0]
    worst = max(ratios, key=ratios.get)
    print(f"[rizovik] {what} {dtype}: worst error {ratios[worst]:.2f} of its bound at {worst}, {len(over)} of {len(ratios)} "
          f"beyond it, {skipped} rows behind a close routing call")
    limit, allowed = (1.0, 0) if dtype == "float32" else (4.0, max(1, len(ratios) // 10))
    if alone:
        limit = max(6.0, 3.0 * max(alone.values()))
        allowed = max(len(ratios) // 6, 5 * sum(ratio > 1.0 for ratio in alone.values()))
        print(f"[rizovik] {what}: rounding alone moves the plain model by up to {max(alone.values()):.2f} bounds")
    assert ratios[worst] <= limit and len(over) <= allowed, \
        f"{what}: first wrong logits at request {over[0][0]} position {over[0][1]}: {ratios[over[0]]:.2f} bounds"


LENGTHS = {"A": [70, 128, 45, 33, 100, 5, 17, 64], "B": [1, 9, 133, 70, 41, 196, 23, 2], "C": [150, 40, 66, 129, 31, 200],
           "pooled": [90, 3, 47, 130], "kept": [60, 17, 1, 133], "delta": [77, 2, 31, 120], "routed": [60, 17, 1, 33]}
TRACES = {"whole": trace_whole, "tail": functools.partial(trace_tail, tail=60),
          "portions": functools.partial(trace_portions, sizes=(1, 1, 2, 7, 2, 5, 3, 2, 11, 2, 4, 1, 6, 23)),
          "mixed": trace_mixed, "batched": trace_batched_tail}


def make_requests(name):
    return {f"r{i}": random_tokens(ALL[name]["vocab"], n, seed=100 * sum(map(ord, name)) + i)
            for i, n in enumerate(LENGTHS[name])}


@pytest.mark.parametrize("mode", list(TRACES))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(ALL))
def test_replay_matches_plain(folders, cuda_device, name, dtype, mode):
    folder, requests = folders(name, dtype), make_requests(name)
    steps = TRACES[mode](requests)
    rows = collect(steps, replay(folder, dtype, steps, PAGE_SIZE.get(name, 16)))
    assert_rows_match(rows, requests, folder, dtype, f"{name} {mode}")


@pytest.mark.parametrize("name", ["A", "B"])
def test_the_residual_stream_after_every_layer(folders, cuda_device, name):
    """Layer run by layer run in float32 (a layer that runs another's tensors counts each time): the stream
    after each, its last summand added, against the plain one's."""
    from zephyr_b200.engine.replay import TraceReplayer

    folder = folders(name, "float32")
    config, weights = read_model(folder)
    tokens = random_tokens(config["vocab"], 90, seed=4)
    plain_streams: list = []
    forward(config, weights, tokens, layers_out=plain_streams)
    replayer = TraceReplayer(folder, "float32", 128, page_size=PAGE_SIZE[name])
    replayer.runner.use_cuda_graphs = False
    seen = []
    for block in replayer.runner.model.layers:
        def wrapped(stream, ctx, call, inner=block.forward):
            out = inner(stream, ctx, call)
            total = out.hidden.clone()
            if out.deferred is not None:
                out.deferred.apply(total)
            seen.append(total.cpu().double())
            return out
        block.forward = wrapped
    replayer.step({"step": 0, "entries": [{"id": "a", "tokens": tokens, "want": []}], "end": ["a"]})
    assert len(seen) == len(plain_streams) == len(config["layers"])
    for index, (got, expected) in enumerate(zip(seen, plain_streams)):
        assert (got - expected).abs().max() < 3e-5 * float(expected.abs().max()), index


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_two_requests_at_a_time_through_few_pages_and_slots(folders, cuda_device, dtype):
    """Eight requests, two live at a time, two state slots: every page and both slots (the delta rule's
    state and its convolutions' last inputs) are used again and again."""
    folder, requests = folders("A", dtype), make_requests("A")
    steps = trace_mixed(requests, max_live=2, seed=5)
    rows = collect(steps, replay(folder, dtype, steps, PAGE_SIZE["A"], max_requests=2))
    assert_rows_match(rows, requests, folder, dtype, "A two live")


def test_a_kept_choice_in_bfloat16(folders, cuda_device):
    """The routed model with its real choice in bfloat16, each request compared up to its first close call."""
    folder, requests = folders("routed", "bfloat16", True), make_requests("routed")
    steps = trace_portions(requests)
    rows = collect(steps, replay(folder, "bfloat16", steps, 16))
    assert_rows_match(rows, requests, folder, "bfloat16", "routed, choice kept", least=0.1, close_call=0.05)


def test_captured_steps_equal_launched_ones(folders, cuda_device):
    """Steps replayed from CUDA graphs give the logits of steps launched kernel by kernel: the pooling of
    blocks, the delta rule's state and the routing stay on the device."""
    folder, requests = folders("A", "float32"), make_requests("A")
    steps = trace_batched_tail(requests, tail=20)
    with_graphs = collect(steps, replay(folder, "float32", steps, 16, graphs=True))
    without = collect(steps, replay(folder, "float32", steps, 16, graphs=False))
    assert with_graphs.keys() == without.keys()
    for key in with_graphs:
        assert np.array_equal(with_graphs[key], without[key]), key


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(folders, cuda_device, dtype):
    """A short prompt and 190 tokens decoded one by one: the windows pass over decoded tokens, blocks become
    whole and seen one after the other, pages behind the windows are given back while the kept ones stay."""
    for name in ("A", "B", "C", "delta"):
        folder = folders(name, dtype)
        requests = {"long": random_tokens(ALL[name]["vocab"], 200, seed=9)}
        steps = trace_tail(requests, tail=190)
        assert_rows_match(collect(steps, replay(folder, dtype, steps, PAGE_SIZE.get(name, 16))), requests, folder, dtype,
                          f"{name} long decoding")


LONG = model(90, 128, 0.8, 1e-6, [
    pooled(8, 2, 32, 48, 100, 24, rot(1000.0, 16), 0.15, moe(8, 2, 64)),
    delta(4, 2, 64, 32, 4, moe(6, 3, 40)),
    kept(6, 3, 64, 64, 200, 50, rot(5000.0, 64, factor=2.0), 0.12, moe(4, 1, 96))])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prompts_of_many_hundred_tokens(tmp_path, cuda_device, dtype):
    """Portions of more than 512 tokens (from where the products with many rows and the grouped products of a
    routed layer run on the tensor cores' own kernels in bfloat16) beside short ones: a prompt of 1100 tokens
    whole, one of 700 in portions of 530, 2 and 168, and a third of 600 that comes in beside decoded tokens of
    the first; keys many hundred positions behind every window."""
    config = LONG if dtype == "float32" else without_choice(LONG)
    folder = write_model(tmp_path / "long", config, seed=77, dtype=DTYPES[dtype])
    requests = {"a": random_tokens(90, 1112, seed=1), "b": random_tokens(90, 712, seed=2), "c": random_tokens(90, 606, seed=3)}
    every = lambda lo, hi: list(range(0, hi - lo, 37)) + [hi - lo - 1]
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": requests["a"][:1100], "want": every(0, 1100)}], "end": []},
             {"step": 1, "entries": [{"id": "b", "tokens": requests["b"][:530], "want": every(0, 530)}], "end": []},
             {"step": 2, "entries": [{"id": "b", "tokens": requests["b"][530:532], "want": [0, 1]},
                                     {"id": "a", "tokens": requests["a"][1100:1101], "want": [0]}], "end": []},
             {"step": 3, "entries": [{"id": "a", "tokens": requests["a"][1101:1102], "want": [0]},
                                     {"id": "c", "tokens": requests["c"][:600], "want": every(0, 600)},
                                     {"id": "b", "tokens": requests["b"][532:700], "want": every(532, 700)}], "end": []}]
    for i in range(6):
        steps.append({"step": 4 + i, "entries": [{"id": "a", "tokens": [requests["a"][1102 + i]], "want": [0]},
                                                 {"id": "c", "tokens": [requests["c"][600 + i]], "want": [0]},
                                                 {"id": "b", "tokens": [requests["b"][700 + i]], "want": [0]}],
                      "end": ["a", "b", "c"] if i == 5 else []})
    requests = {"a": requests["a"][:1108], "b": requests["b"][:706], "c": requests["c"][:606]}
    rows = collect(steps, replay(folder, dtype, steps, 32))
    assert len(rows) > 60
    assert_rows_match(rows, requests, folder, dtype, "long prompts", least=0.3)


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("C", "bfloat16"), ("B", "float32"), ("delta", "bfloat16")])
def test_greedy_generation_through_the_engine(folders, cuda_device, name, dtype):
    from zephyr_b200 import Engine
    from zephyr_b200.engine import KvCacheOptions, PagedSchedulerConfig

    folder = folders(name, dtype)
    config, weights = read_model(folder)
    engine = Engine(folder, dtype=dtype, max_seq_len=256,
                    scheduler=PagedSchedulerConfig(max_num_seqs=3, max_num_batched_tokens=16, max_prefill_chunk_tokens=7),
                    kv_cache=KvCacheOptions(block_size=PAGE_SIZE.get(name, 16), num_blocks=40))
    prompts = [random_tokens(config["vocab"], n, seed=n) for n in (5, 11, 17, 40, 3)]
    outputs = engine.generate(prompts, max_tokens=10, temperature=0.0, ignore_eos=True)
    for prompt, output in zip(prompts, outputs):
        tokens = list(prompt)
        for index, got in enumerate(output.token_ids):
            margins: list = []
            logits = forward(config, weights, tokens, margins=margins)[-1]
            if margins and min(float(m.min()) for m in margins) < CLOSE_CALL[dtype]:
                break           # a close routing call somewhere in the sequence: the engine may take another expert
            top = torch.topk(logits, 2).values
            if got != int(logits.argmax()):
                # a first difference is forgiven where the two best lie closer than twice the engine's bound
                assert float(top[0] - top[1]) <= 2 * tolerance(dtype, logits.numpy()), (prompt, index)
                break
            tokens.append(got)
        assert output.usage.completion_tokens == 10
    assert engine.runner.manager.num_requests == 0
    engine.runner.manager.check_invariants()


def test_the_replay_program_on_rizovik(folders, cuda_device, tmp_path):
    """bin/trace_run picks the architecture from config.json and writes the logits of a mixed trace."""
    import subprocess
    import sys
    from pathlib import Path

    folder, requests = folders("B", "float32"), make_requests("B")
    steps = trace_mixed(requests, seed=3)
    root = Path(__file__).resolve().parent.parent
    out = tmp_path / "out"
    done = subprocess.run([sys.executable, str(root / "bin" / "trace_run"), "--model", str(folder), "--dtype", "float32",
                           "--out", str(out), "--max-tokens", str(peak_tokens(steps))],
                          input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600)
    assert done.returncode == 0, done.stderr[-2000:]
    assert [line for line in done.stdout.splitlines() if line.startswith("done ")] == [f"done {s['step']}" for s in steps]
    outputs = {s["step"]: np.fromfile(out / f"{s['step']}.f32", dtype="<f4").reshape(-1, CONFIGS["B"]["vocab"])
               for s in steps if any(e["want"] for e in s["entries"])}
    assert_rows_match(collect(steps, outputs), requests, folder, "float32", "B through the program")
