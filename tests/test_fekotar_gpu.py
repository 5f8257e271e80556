"""Fekotar in the engine against the plain implementation (tests/plain_fekotar.py): each kernel of its
mechanisms alone, then whole models under every way of cutting the work, in 32-bit and in bfloat16: whole
prompts, long decoding one token at a time, portions down to two tokens (and single first tokens), mixed
batches of unequal requests with so few pages and slots that they are used again (pages given back are
filled with NaN), and greedy generation through the engine's own entry point and scheduler.  Where random
weights would hide a fault (a key far back among hundreds, the rotated part of a score, the token a request
remembers between steps), inputs are made so that it shows."""

import functools
import json
import math

import numpy as np
import pytest
import torch

from fekotar_models import CONFIGS, PAGE_SIZE, dense, latent, moe, read_model, without_choice, write_model, yarn
from plain_fekotar import (F64, GATE_SLOPE, forward, group_routing, pair_rows, rms_norm, rotate_halves,
                           rotation_frequencies)
from replay_util import (collect, peak_tokens, random_tokens, tolerance, trace_batched_tail, trace_mixed,
                         trace_portions, trace_tail, trace_whole)

pytestmark = pytest.mark.gpu

DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}
# A routed layer's choice is a step function of its input: where two scores lie closer than the input's
# rounding moves them, another expert runs and the logits are another computation's.  The plain side
# reports every token's margin, and a request is compared up to its first close call only.  In float32
# that is rare.  In bfloat16 it would be every few tokens, so the bfloat16 models take every expert
# (``without_choice``: the weights stay each token's own); the choice itself is float32's to test, and
# one bfloat16 model keeps it and is compared as far as its margins allow.
CLOSE_CALL = {"float32": 1e-5, "bfloat16": 0.03}

ONE_LAYER = {
    # single layers: the mechanism alone, through the engine
    "mixer": {"architecture": "Fekotar", "vocab": 50, "width": 48, "logit_scale": 1.5, "norm": {"eps": 1e-6},
              "layers": [latent(3, 8, 12, 12, 20, 10, 0.4, None, base=40.0, scaling=yarn(2.5, 24, 3.0, 0.5))]},
    "routed": {"architecture": "Fekotar", "vocab": 50, "width": 40, "logit_scale": 1.0, "norm": {"eps": 1e-6},
               "embedding": {"bigram": {"buckets": 11, "mul_prev": 5, "mul_cur": 3}},
               "layers": [latent(1, 8, 8, 8, 24, 8, 0.5, moe(10, 2, 24, scale=3.0, groups=(5, 3)), base=10.0),
                          latent(2, 8, 8, 8, 8, 8, 0.5, dense(24, 1.0), base=10.0)]},
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
            made[key] = write_model(tmp_path_factory.mktemp(f"fekotar_{name}_{dtype}"), config_for(name, dtype, keep_choice),
                                    seed=17 + sum(map(ord, name)), dtype=DTYPES[dtype])
        return made[key]

    return get


@functools.lru_cache(maxsize=256)
def _plain(folder: str, tokens: tuple):
    """(logits [T, vocab], every position's smallest routing margin over the routed layers; inf without any)."""
    config, weights = read_model(folder)
    margins: list = []
    logits = forward(config, weights, list(tokens), margins=margins).numpy()
    smallest = np.min(np.array(margins), axis=0) if margins else np.full(len(tokens), np.inf)
    return logits, smallest


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


def assert_rows_match(rows, requests, folder, dtype, what, least=0.5, close_call=None):
    """Every compared row of logits within its bound (``replay_util.tolerance``) in float32; in bfloat16 no
    row beyond four bounds and at most one in ten beyond one.  A fault of a mask, a page, a remembered
    token or a routed token moves logits by tens to hundreds of bounds."""
    ratios, skipped = {}, 0
    for (rid, position), got in sorted(rows.items()):
        expected, margins = _plain(str(folder), tuple(requests[rid]))
        close = np.nonzero(margins < (close_call or CLOSE_CALL[dtype]))[0]
        if close.size and position >= close[0]:
            skipped += 1
            continue
        assert np.isfinite(got).all(), f"{what}: non-finite logits for {rid} at {position}"
        ratios[(rid, position)] = float(np.abs(got.astype(np.float64) - expected[position]).max()) / tolerance(dtype, expected[position])
    assert len(ratios) >= least * len(rows), f"{what}: {skipped} of {len(rows)} rows lie behind a close routing call"
    over = [key for key, ratio in ratios.items() if ratio > 1.0]
    worst = max(ratios, key=ratios.get)
    print(f"[fekotar] {what} {dtype}: worst error {ratios[worst]:.2f} of its bound at {worst}, {len(over)} of {len(ratios)} "
          f"beyond it, {skipped} rows behind a close routing call")
    limit, allowed = (1.0, 0) if dtype == "float32" else (4.0, max(1, len(ratios) // 10))
    assert ratios[worst] <= limit and len(over) <= allowed, \
        f"{what}: first wrong logits at request {over[0][0]} position {over[0][1]}: {ratios[over[0]]:.2f} bounds"


LENGTHS = {"A": [70, 128, 45, 33, 100, 5, 17, 64], "B": [1, 9, 33, 70, 41, 96, 23, 2], "C": [150, 40, 66, 129, 31, 200],
           "mixer": [90, 3, 47, 130], "routed": [60, 17, 1, 33]}
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


def test_the_residual_stream_after_every_layer(folders, cuda_device):
    """Layer by layer in float32: the stream after each layer (its pending summands added) against the
    plain one's."""
    from zephyr_b200.engine.replay import TraceReplayer

    folder = folders("A", "float32")
    config, weights = read_model(folder)
    tokens = random_tokens(config["vocab"], 37, seed=4)
    plain_streams: list = []
    forward(config, weights, tokens, streams=plain_streams)
    replayer = TraceReplayer(folder, "float32", 64)
    replayer.runner.use_cuda_graphs = False
    seen = []
    for block in replayer.runner.model.layers:
        def wrapped(stream, ctx, call, inner=block.forward):
            out = inner(stream, ctx, call)
            total = out.hidden.clone()
            for part in (out.pending if isinstance(out.pending, tuple) else ()):
                total += part.float()
            seen.append(total.cpu().double())
            return out
        block.forward = wrapped
    replayer.step({"step": 0, "entries": [{"id": "a", "tokens": tokens, "want": []}], "end": ["a"]})
    assert len(seen) == len(plain_streams)
    for index, (got, expected) in enumerate(zip(seen, plain_streams)):
        assert (got - expected).abs().max() < 2e-5 * float(expected.abs().max()), index


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_two_requests_at_a_time_through_few_pages_and_slots(folders, cuda_device, dtype):
    """Eight requests, two live at a time, two state slots: every page and both slots (which hold each
    request's last token) are used again and again."""
    folder, requests = folders("A", dtype), make_requests("A")
    steps = trace_mixed(requests, max_live=2, seed=5)
    rows = collect(steps, replay(folder, dtype, steps, PAGE_SIZE["A"], max_requests=2))
    assert_rows_match(rows, requests, folder, dtype, "A two live")


def test_a_kept_choice_in_bfloat16(folders, cuda_device):
    """The routed model with its real choice in bfloat16, each request compared up to its first close call.
    The routed layer is the first one: its input differs from the plain one's by one rounding only, so a
    call is close at a margin of 0.004 already."""
    folder, requests = folders("routed", "bfloat16", True), make_requests("routed")
    steps = trace_portions(requests)
    rows = collect(steps, replay(folder, "bfloat16", steps, 16))
    assert_rows_match(rows, requests, folder, "bfloat16", "routed, choice kept", least=0.15, close_call=0.004)


def test_captured_steps_equal_launched_ones(folders, cuda_device):
    """Steps replayed from CUDA graphs give the logits of steps launched kernel by kernel: the remembered
    token and the routing stay on the device."""
    folder, requests = folders("A", "float32"), make_requests("A")
    steps = trace_batched_tail(requests, tail=20)
    with_graphs = collect(steps, replay(folder, "float32", steps, 16, graphs=True))
    without = collect(steps, replay(folder, "float32", steps, 16, graphs=False))
    assert with_graphs.keys() == without.keys()
    for key in with_graphs:
        assert np.array_equal(with_graphs[key], without[key]), key


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(folders, cuda_device, dtype):
    """A short prompt and 190 tokens decoded one by one: the context crosses a dozen pages, and positions
    run far past the YaRN scaling's original context."""
    for name in ("A", "C", "mixer"):
        folder = folders(name, dtype)
        requests = {"long": random_tokens(ALL[name]["vocab"], 200, seed=9)}
        steps = trace_tail(requests, tail=190)
        assert_rows_match(collect(steps, replay(folder, dtype, steps, PAGE_SIZE.get(name, 16))), requests, folder, dtype,
                          f"{name} long decoding")


LONG = {"architecture": "Fekotar", "vocab": 90, "width": 128, "logit_scale": 0.5, "norm": {"eps": 1e-6},
        "embedding": {"bigram": {"buckets": 61, "mul_prev": 13, "mul_cur": 5}},
        "layers": [latent(8, 32, 32, 24, 96, 40, 0.12, dense(192, 1.0), base=1000.0, scaling=yarn(2.0, 128, 16.0, 1.0)),
                   latent(4, 16, 16, 32, 144, 24, 0.1, moe(8, 2, 64, scale=1.5, groups=(4, 2)), base=5000.0),
                   latent(16, 24, 64, 16, 64, 64, 0.1, moe(6, 3, 40, scale=0.7), base=300.0, scaling=yarn(4.0, 64, 8.0, 2.0))]}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prompts_of_many_hundred_tokens(tmp_path, cuda_device, dtype):
    """Portions of more than 512 tokens (from where the products with many rows and the grouped products of a
    routed layer run on the tensor cores' own kernels in bfloat16) and of more than 1024 (from where the
    products per head stage all of K at once) beside short ones: a prompt of 1100 tokens whole, one of 700 in
    portions of 530, 2 and 168, and a third of 600 that comes in beside decoded tokens of the first."""
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
    assert_rows_match(rows, requests, folder, dtype, "long prompts")


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("C", "bfloat16"), ("B", "float32"), ("mixer", "bfloat16")])
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
            if margins and float(np.min(np.array(margins))) < CLOSE_CALL[dtype]:
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


def test_the_replay_program_on_fekotar(folders, cuda_device, tmp_path):
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


# ------------------------------------------------------------------------------------- kernels alone
def _i32(values, device):
    return torch.tensor(list(values), dtype=torch.int32, device=device)


def _rows(n, ctx, device):
    """(row_q_start, row_q_len, row_ctx) of a step with one row of n new tokens behind ctx cached ones."""
    return _i32([0], device), _i32([n], device), _i32([ctx], device)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_hashed_pair_embedding_remembers_the_last_token(cuda_device, dtype):
    """Three requests in portions that share steps, over two slots' worth of reuse: every token's row of the
    second table is the hash with the token before it, across step borders, and the table's last row at
    position 0 whatever the slot held before."""
    from zephyr_b200.kernels import ops

    torch_dtype = DTYPES[dtype]
    g = torch.Generator().manual_seed(3)
    vocab, width, buckets, mul_prev, mul_cur = 41, 24, 13, 1000003, 29
    table = torch.randn(vocab, width, generator=g).to(torch_dtype)
    pairs = torch.randn(buckets + 1, width, generator=g).to(torch_dtype)
    sequences = {"a": random_tokens(vocab, 23, 1), "b": random_tokens(vocab, 9, 2), "c": random_tokens(vocab, 14, 3)}
    slot_of = {"a": 1, "b": 0, "c": 1}                       # c takes a's slot after a has ended
    last_token = torch.full((2,), 7, dtype=torch.int32, device=cuda_device)        # stale values
    status = ops.new_status(cuda_device)
    steps = [{"a": 5, "b": 2}, {"a": 1, "b": 1}, {"b": 6, "a": 17}, {"c": 1}, {"c": 2}, {"c": 11}]
    fed = {name: 0 for name in sequences}
    got = {name: [] for name in sequences}
    for step in steps:
        ids, positions, token_row, q_start, q_len, slots = [], [], [], [], [], []
        for row, (name, n) in enumerate(step.items()):
            q_start.append(len(ids)); q_len.append(n); slots.append(slot_of[name])
            ids += sequences[name][fed[name]:fed[name] + n]
            positions += range(fed[name], fed[name] + n)
            token_row += [row] * n
        out = ops.pair_embedding(table.to(cuda_device), pairs.to(cuda_device), _i32(ids, cuda_device), _i32(positions, cuda_device),
                                 _i32(token_row, cuda_device), _i32(q_start, cuda_device), _i32(q_len, cuda_device),
                                 _i32(slots, cuda_device), last_token, mul_prev, mul_cur, status)
        assert out.dtype == torch.float32
        for row, (name, n) in enumerate(step.items()):
            got[name].append(out[q_start[row]:q_start[row] + n].cpu())
            fed[name] += n
    ops.check_status(status)
    for name, tokens in sequences.items():
        rows = pair_rows(tokens, buckets, mul_prev, mul_cur)
        expected = table.double()[torch.tensor(tokens)] + pairs.double()[torch.tensor(rows)]
        assert (torch.cat(got[name]).double() - expected).abs().max() < 1e-6, name
    assert pair_rows([3, 5], buckets, mul_prev, mul_cur) != pair_rows([5, 5], buckets, mul_prev, mul_cur)


@pytest.mark.parametrize("a_dtype,b_dtype,out_dtype", [("float32", "float32", "float32"), ("bfloat16", "float32", "bfloat16"),
                                                       ("bfloat16", "bfloat16", "bfloat16"), (None, "bfloat16", "bfloat16"),
                                                       (None, None, "bfloat16")])
@pytest.mark.parametrize("width", [48, 257, 1024, 5000])
def test_sum_and_rms_norm_on_a_float32_stream(cuda_device, width, a_dtype, b_dtype, out_dtype):
    from zephyr_b200.kernels import ops

    g = torch.Generator().manual_seed(width)
    rows, eps = 7, 1e-5
    wide = torch.randn(rows, width + 5, generator=g).to(cuda_device)
    x = wide[:, 3:3 + width]                                  # rows that are slices of wider rows
    before, wide_before = x.clone(), wide.clone()
    a = torch.randn(rows, width, generator=g).to(DTYPES[a_dtype]).to(cuda_device) if a_dtype else None
    b = torch.randn(rows, width, generator=g).to(DTYPES[b_dtype]).to(cuda_device) if b_dtype else None
    w = (torch.randn(width, generator=g) * 0.2 + 1.0).to(cuda_device)
    out = ops.sum_rms_norm(x, a, b, w, eps, out_dtype=DTYPES[out_dtype])
    summed = before.double() + ((a.double() if a is not None else 0) + (b.double() if b is not None else 0))
    assert (x.double() - summed).abs().max() < 1e-6
    expected = rms_norm(x.double(), eps, w.double())
    bound = 1e-5 if out_dtype == "float32" else 2.0 ** -8
    assert out.dtype == DTYPES[out_dtype] and (out.double() - expected).abs().max() < bound * float(expected.abs().max())
    assert torch.equal(wide[:, :3], wide_before[:, :3]) and torch.equal(wide[:, 3 + width:], wide_before[:, 3 + width:])
    assert ops.sum_rms_norm(x, a, None, None, eps) is None


@pytest.mark.parametrize("in_dtype,out_dtype", [("float32", "float32"), ("float32", "bfloat16"), ("bfloat16", "bfloat16")])
@pytest.mark.parametrize("tokens,inner,blocked,biased,limit", [(5, 24, True, True, 1.0), (300, 50, False, True, 0.5),
                                                               (17, 160, True, False, 2.5), (1, 7, False, False, 4.0)])
def test_bounded_gate(cuda_device, in_dtype, out_dtype, tokens, inner, blocked, biased, limit):
    from zephyr_b200.kernels import ops

    g = torch.Generator().manual_seed(tokens + inner)
    gate = (torch.randn(tokens, inner, generator=g) * 2.0).to(DTYPES[in_dtype])
    up = (torch.randn(tokens, inner, generator=g) * 2.0).to(DTYPES[in_dtype])
    b_gate, b_up = torch.randn(inner, generator=g), torch.randn(inner, generator=g)
    if blocked:
        packed = torch.stack([gate.view(tokens, -1, 8), up.view(tokens, -1, 8)], dim=2).reshape(tokens, 2 * inner)
        bias = torch.stack([b_gate.view(-1, 8), b_up.view(-1, 8)], dim=1).reshape(-1)
    else:
        packed, bias = torch.cat([gate, up], dim=1), torch.cat([b_gate, b_up])
    out = ops.clamped_gate(packed.contiguous().to(cuda_device), bias.to(cuda_device) if biased else None, limit, GATE_SLOPE, 1.0,
                           DTYPES[out_dtype], blocked=blocked)
    gd = gate.double() + (b_gate.double() if biased else 0.0)
    ud = up.double() + (b_up.double() if biased else 0.0)
    gd, ud = gd.clamp(max=limit), ud.clamp(min=-limit, max=limit)
    expected = gd * torch.sigmoid(GATE_SLOPE * gd) * (ud + 1.0)
    if tokens * inner >= 100:
        assert float((gd == limit).double().mean()) > 0.02 and float((ud.abs() == limit).double().mean()) > 0.02      # the bounds bite
    bound = 1e-5 if out_dtype == "float32" else 2.0 ** -8
    assert (out.cpu().double() - expected).abs().max() < bound * max(1.0, float(expected.abs().max()))


def _bounded_feed_forward_case(tokens, width, inner, biased, limit, seed):
    """x, gate and up weights (bfloat16 values), biases, and y = g * sigmoid(slope * g) * (u + 1) in float64."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(tokens, width, generator=g).bfloat16()
    w_gate = (torch.randn(inner, width, generator=g) * 1.5 * width ** -0.5).bfloat16()
    w_up = (torch.randn(inner, width, generator=g) * 1.5 * width ** -0.5).bfloat16()
    b_gate, b_up = (torch.randn(inner, generator=g) * 0.5, torch.randn(inner, generator=g) * 0.5) if biased else (None, None)
    gd = x.double() @ w_gate.double().T + (b_gate.double() if biased else 0.0)
    ud = x.double() @ w_up.double().T + (b_up.double() if biased else 0.0)
    gd, ud = gd.clamp(max=limit), ud.clamp(min=-limit, max=limit)
    assert float((gd == limit).double().mean()) > 0.02 and float((ud.abs() == limit).double().mean()) > 0.02      # the bounds bite
    return x, w_gate, w_up, b_gate, b_up, gd * torch.sigmoid(GATE_SLOPE * gd) * (ud + 1.0)


@pytest.mark.parametrize("kernel,tokens,width,inner,biased,limit", [
    ("few", 1, 64, 24, True, 1.0), ("few", 7, 200, 136, False, 0.7), ("few", 16, 1024, 512, True, 1.5),
    ("many", 130, 64, 24, True, 1.0), ("many", 600, 200, 136, True, 0.7), ("many", 300, 96, 1000, False, 1.2),
    ("many", 257, 512, 328, True, 2.0)])
def test_bounded_gate_where_the_product_ends(cuda_device, kernel, tokens, width, inner, biased, limit):
    """Biases, bounds and the gate inside the product's kernel: the weight streamer for few rows, tcgen05 for many,
    with inner sizes that end inside a tile of columns and row counts that end inside a tile of rows."""
    from zephyr_b200.kernels import ops

    x, w_gate, w_up, b_gate, b_up, expected = _bounded_feed_forward_case(tokens, width, inner, biased, limit, tokens + inner)
    packed = torch.stack([w_gate.view(-1, 8, width), w_up.view(-1, 8, width)], dim=1).reshape(-1, width).contiguous().to(cuda_device)
    bias = torch.stack([b_gate.view(-1, 8), b_up.view(-1, 8)], dim=1).reshape(-1).contiguous().to(cuda_device) if biased else None
    form = ops.BoundedGate(bias, limit, GATE_SLOPE, 1.0)
    product = ops.gemm_small if kernel == "few" else ops.gemm_tc
    out = product(x.to(cuda_device), packed, swiglu=True, bounded=form)
    ops.check_status(ops.device_status(cuda_device))
    assert out.shape == (tokens, inner) and out.dtype == torch.bfloat16
    assert (out.cpu().double() - expected).abs().max() < 2.0 ** -7 * max(1.0, float(expected.abs().max()))


@pytest.mark.parametrize("tokens", [3, 40, 520])
@pytest.mark.parametrize("inner,biased", [(48, True), (50, True), (136, False)])
def test_the_bounded_feed_forward_part_at_every_count_of_rows(cuda_device, tokens, inner, biased):
    """The part picks a kernel by the number of rows; every choice computes the same function."""
    from zephyr_b200.config.spec import FeedForwardSpec
    from zephyr_b200.parts.base import FEED_FORWARDS

    width, limit = 72, 0.9
    x, w_gate, w_up, b_gate, b_up, hidden = _bounded_feed_forward_case(tokens, width, inner, biased, limit, 5 * tokens + inner)
    g = torch.Generator().manual_seed(inner)
    w_down = (torch.randn(width, inner, generator=g) * inner ** -0.5).bfloat16()
    b_down = torch.randn(width, generator=g) * 0.5
    names = {"gate_proj": "gate", "up_proj": "up", "down_proj": "down"}
    weights = {"gate": w_gate, "up": w_up, "down": w_down}
    if biased:
        names.update({"gate_bias": "gate.b", "up_bias": "up.b", "down_bias": "down.b"})
        weights.update({"gate.b": b_gate, "up.b": b_up, "down.b": b_down})
    spec = FeedForwardSpec("gated", {"hidden_size": width, "intermediate_size": inner, "activation": "clamped_swish", "limit": limit,
                                     "alpha": GATE_SLOPE, "up_shift": 1.0, **names})
    part = FEED_FORWARDS["gated"](spec, {k: v.to(cuda_device) for k, v in weights.items()}, torch.bfloat16)
    out = part.forward(x.to(cuda_device)).float().cpu().double()
    expected = hidden @ w_down.double().T + (b_down.double() if biased else 0.0)
    assert (out - expected).abs().max() < 2.0 ** -6 * max(1.0, float(expected.abs().max()))


@pytest.mark.parametrize("experts,top,groups,scale", [(15, 2, (3, 2), 1.75), (8, 3, (4, 2), 1.5), (10, 2, (5, 3), 3.0), (12, 4, (2, 1), 0.8),
                                                      (9, 2, (3, 3), 1.0), (6, 1, None, 0.5), (4, 4, None, 2.5), (200, 8, (25, 4), 1.0),
                                                      (7, 7, (7, 7), 1.0), (16, 1, (16, 1), 1.0), (6, 3, (2, 1), 1.0)])
def test_sigmoid_routing_limited_to_groups(cuda_device, experts, top, groups, scale):
    """Scores of each logit on its own, the best groups by the sum of their two largest scores, the largest
    allowed scores, weights = score * scale.  One token is given two groups whose single best scores are in
    the other order than their marks, so a choice by the single best would show."""
    from zephyr_b200.kernels import ops

    g = torch.Generator().manual_seed(experts * 10 + top)
    tokens = 257
    z = torch.randn(tokens, experts, generator=g) * 2.0
    router = {"experts": experts, "top": top, "scale": scale}
    if groups is not None:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
        per = experts // groups[0]
        if per >= 2 and groups[0] >= 2 and groups[1] < groups[0]:
            z[0] = -6.0
            z[0, 0] = 3.0                       # group 0: one very large score and nothing else
            z[0, per], z[0, per + 1] = 1.5, 1.4       # group 1: two good ones, whose sum is larger
    ids, weights, margin = group_routing(z.double(), router)
    got_ids, got_weights = ops.route(z.to(cuda_device), None, top, "sigmoid",
                                     (groups[0], groups[1], 2) if groups is not None else None, scale)
    sure = margin > 1e-6
    assert int(sure.sum()) > tokens // 2
    assert torch.equal(got_ids.cpu().long()[sure], ids[sure])
    assert (got_weights.cpu().double()[sure] - weights[sure]).abs().max() < 1e-6 * max(1.0, scale)
    if groups is not None and groups[1] == 1 and experts // groups[0] >= 2 and groups[0] >= 2:
        assert int(got_ids[0, 0]) == experts // groups[0]          # the group with the larger sum wins


@pytest.mark.parametrize("gate_kind", ["none", "head", "value"])
@pytest.mark.parametrize("x_dtype,w_dtype", [("float32", "float32"), ("bfloat16", "bfloat16"), ("float32", "bfloat16")])
@pytest.mark.parametrize("tokens,heads,n,k,x_head,y_head", [(1, 3, 48, 16, 24, 60), (70, 2, 20, 8, 8, 20), (200, 5, 130, 24, 29, 131),
                                                            (33, 8, 16, 128, 160, 16), (200, 5, 130, 160, 192, 131),
                                                            (150, 3, 96, 512, 512, 128), (65, 2, 128, 32, 40, 128),
                                                            (300, 4, 250, 48, 48, 250), (1030, 3, 96, 128, 160, 128),
                                                            (1100, 2, 130, 48, 48, 131), (1024, 5, 250, 16, 24, 250)])
def test_products_per_head_on_slices_of_wider_heads(cuda_device, x_dtype, w_dtype, tokens, heads, n, k, x_head, y_head, gate_kind):
    from zephyr_b200.kernels import ops

    g = torch.Generator().manual_seed(tokens + heads + n)
    x = torch.randn(tokens, heads * x_head, generator=g).to(DTYPES[x_dtype])
    w = (torch.randn(heads, n, k, generator=g) * k ** -0.5).to(DTYPES[w_dtype])
    gate = {"none": None, "head": torch.randn(tokens, heads, generator=g), "value": torch.randn(tokens, heads * n, generator=g)}[gate_kind]
    out = torch.full((tokens, heads * y_head), 7.0, dtype=DTYPES[w_dtype], device=cuda_device)
    ops.head_linear(x.to(cuda_device), w.to(cuda_device), gate=gate.to(cuda_device) if gate is not None else None,
                    x_head_stride=x_head, out=out, out_head_stride=y_head)
    xs = x.double().view(tokens, heads, x_head)[:, :, :k]
    if x_dtype == "float32" and w_dtype == "bfloat16":
        xs = xs.to(torch.bfloat16).double()                   # rounded as it is staged for the tensor cores
    expected = torch.einsum("thk,hnk->thn", xs, w.double())
    if gate_kind == "head":
        expected = expected * torch.sigmoid(gate.double()).view(tokens, heads, 1)
    elif gate_kind == "value":
        expected = expected * torch.sigmoid(gate.double()).view(tokens, heads, n)
    got = out.cpu().double().view(tokens, heads, y_head)
    bound = 1e-5 if w_dtype == "float32" else 2.0 ** -7
    assert (got[:, :, :n] - expected).abs().max() < bound * max(1.0, float(expected.abs().max()))
    assert (got[:, :, n:] == 7.0).all()                       # what lies between the heads' outputs is left alone
    if w_dtype == "bfloat16":
        # rows on 16-byte boundaries with a K that is a multiple of 16 may take a kernel that stages all of K at
        # once, with 32 or 64 rows a CTA by the row count: the sums are those of the walk along k, to the bit
        for form in (1, 2, 3):
            other = torch.full_like(out, 7.0)
            ops.head_linear(x.to(cuda_device), w.to(cuda_device), gate=gate.to(cuda_device) if gate is not None else None,
                            x_head_stride=x_head, out=other, out_head_stride=y_head, walk=form)
            assert torch.equal(out, other), form


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("rank,rot,heads,page,scaling", [(40, 8, 3, 16, yarn(4.0, 64, 8.0, 2.0)), (96, 32, 8, 16, yarn(8.0, 128, 16.0, 1.0)),
                                                         (28, 4, 6, 16, None), (64, 64, 16, 32, yarn(2.0, 16, 2.0, 0.25)),
                                                         (128, 32, 4, 32, None), (30, 2, 1, 16, None), (48, 16, 20, 16, yarn(3.0, 50, 5.0, 1.0)),
                                                         (512, 64, 2, 16, yarn(4.0, 64, 8.0, 1.0)), (700, 68, 1, 32, None),
                                                         (160, 32, 18, 16, None), (200, 24, 3, 32, yarn(2.0, 64, 8.0, 1.0)),
                                                         (192, 64, 5, 16, None)])
def test_attention_over_a_latent_with_a_rotated_part(cuda_device, dtype, rank, rot, heads, page, scaling):
    """The cached row is the normed latent followed by the rotated key part; queries carry the same two
    pieces.  Queries of head 0 point at one row each THROUGH THE ROTATED PART ONLY (the latent part of those
    queries is zero): a row hundreds of positions back, the first row, the row just before; so a rotation
    by a wrong position, a wrong pairing or a missing multiplier shows.  A portion, then tokens alone, over
    pages out of order; the general kernel and, where they take the shape, the fast ones."""
    from zephyr_b200.kernels import ops

    torch_dtype = DTYPES[dtype]
    g = torch.Generator().manual_seed(rank + rot + heads)
    T, eps, width = 333, 1e-6, rank + rot
    scale = 1.0 / math.sqrt(width)
    freqs, mult = rotation_frequencies({"dims": rot, "base": 300.0, "scaling": scaling})
    kv = torch.randn(T, width, generator=g)
    norm_w = torch.randn(rank, generator=g) * 0.2 + 1.0
    head_stride = 5 + rot                                     # a head of the query projection: 5 unrotated values, then the rotated ones
    q_proj = torch.randn(T, heads, head_stride, generator=g)
    q_lat = torch.randn(T, heads, rank, generator=g)          # the unrotated part, as already carried into the latent space
    positions = torch.arange(T)
    targets = {p: (p - 300, 0, p - 1)[p % 3] for p in range(T - 30, T)}
    for p, target in targets.items():
        # the query's rotated part, turned back by its own position and forth by the target's, equals the target's key part
        aimed = rotate_halves(kv[target, rank:].double().view(1, 1, rot), torch.tensor([target - p]), freqs, 1.0)[0, 0]
        q_proj[p, 0, 5:] = (aimed * (16.0 * math.sqrt(width) / rot)).float()        # a score of about 16 at the target
        q_lat[p, 0] = 0.0
    rows_kept = torch.cat([rms_norm(kv[:, :rank].double(), eps, norm_w.double()),
                           rotate_halves(kv[:, rank:].double().view(T, 1, rot), positions, freqs, mult)[:, 0]], dim=1)
    rows_kept = rows_kept.to(torch_dtype).double()            # what the cache holds
    q_rot = rotate_halves(q_proj[..., 5:].double(), positions, freqs, mult)
    q_full = torch.cat([q_lat.to(torch_dtype).double(), q_rot.to(torch_dtype).double()], dim=-1)
    scores = torch.einsum("ihd,jd->hij", q_full, rows_kept) * scale
    visible = torch.ones(T, T, dtype=torch.bool).tril()
    probs = torch.softmax(scores.masked_fill(~visible, -math.inf), dim=-1)
    expected = torch.einsum("hij,jd->ihd", probs, rows_kept).reshape(T, heads * width)

    blocks = -(-T // page)
    order = torch.randperm(blocks, generator=g) + 1
    table = order.to(torch.int32).view(1, -1).to(cuda_device)
    cache = torch.full((blocks + 1, page * width), float("nan"), dtype=torch_dtype, device=cuda_device)
    status = ops.new_status(cuda_device)
    tile = ops.attention_tile_tokens(heads)
    fast_ok = ops.paged_decode_supported(heads, 1, width, torch_dtype)
    prompt_ok = ops.paged_prefill_supported(heads, 1, width, torch_dtype)     # single tokens too, as tiles of one token
    outs, fast_outs, at = [], [], 0
    for n in [T - 12] + [1] * 12:
        rows = _rows(n, at, cuda_device)
        pos = torch.arange(at, at + n, dtype=torch.int32, device=cuda_device)
        qs = torch.empty(n, heads * width, dtype=torch_dtype, device=cuda_device)
        qs.view(n, heads, width)[:, :, :rank] = q_lat[at:at + n].to(torch_dtype).to(cuda_device)
        ops.latent_rope(q_proj[at:at + n].reshape(n, -1).to(cuda_device), heads, head_stride, 5, qs, kv[at:at + n].to(cuda_device),
                        rank, rot, norm_w.to(cuda_device), eps, freqs.float().to(cuda_device), mult, pos,
                        torch.zeros(n, dtype=torch.int32, device=cuda_device), cache, table, status, torch_dtype)
        tile_q0 = torch.arange(0, n, tile, dtype=torch.int32, device=cuda_device)
        outs.append(ops.paged_attention(qs, cache, table, torch.zeros_like(tile_q0), tile_q0, tile, *rows, heads, 1, width, 0,
                                        scale, status, shared_kv=True))
        if prompt_ok:
            fast = torch.full_like(outs[-1], float("nan"))
            if n == 1 and fast_ok:
                ops.paged_decode(qs, cache, table, rows[0], rows[0], rows[2], at + 1, heads, 1, width, 0, scale, status, fast,
                                 keys_only=True)
            else:
                wide = ops.paged_prefill_tile_tokens()
                wide_q0 = torch.arange(0, n, wide, dtype=torch.int32, device=cuda_device)
                ops.paged_prefill(qs, cache, table, torch.zeros_like(wide_q0), wide_q0, *rows, heads, 1, width, 0, scale,
                                  status, fast, keys_only=True)
            fast_outs.append(fast)
        at += n
    ops.check_status(status)
    bound = (3e-5 if dtype == "float32" else 0.04) * max(1.0, float(expected.abs().max()))
    for got in [torch.cat(outs)] + ([torch.cat(fast_outs)] if prompt_ok else []):
        got = got.cpu().double()
        assert torch.isfinite(got).all()
        assert (got - expected).abs().max() < bound
    assert fast_ok == (dtype == "bfloat16" and width in (32, 64, 96, 128) and heads <= 16)
    assert prompt_ok == (dtype == "bfloat16" and width % 32 == 0 and width <= 256)
    if dtype == "float32" and rot >= 32:      # (fewer rotated values: other rows lie as close by chance)
        for p, target in targets.items():       # the pointed-at row decides head 0's output
            if target >= 0:
                direction = torch.cat(outs).cpu().double()[p, :width]
                cosine = float(direction @ rows_kept[target] / (direction.norm() * rows_kept[target].norm()))
                assert cosine > 0.9, (p, target, cosine)
