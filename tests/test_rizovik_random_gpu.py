"""Rizovik configurations drawn at random (sizes that are no multiples of anything in particular, layers in any
number and order whose sizes differ from one another, windows, blocks and kept starts in every relation to one
another and to the page, layers that run another layer's tensors), each replayed in a mixed trace, in portions
and with a decoded tail against the plain implementation: what a particular choice of sizes would hide, another
one shows."""

import functools
import random

import pytest

from replay_util import collect, random_tokens, trace_mixed, trace_portions, trace_tail
from rizovik_models import again, delta, kept, model, moe, pooled, rot, without_choice, write_model
from test_rizovik_gpu import DTYPES, assert_rows_match, replay

pytestmark = pytest.mark.gpu


def draw_config(seed: int) -> dict:
    rng = random.Random(seed)
    width = rng.choice([40, 72, 100, 136, 50, 256, 33, 320])

    def feed_forward():
        if rng.random() < 0.15:
            return None
        experts = rng.choice([1, 2, 3, 5, 8, 12, 17])
        return moe(experts, rng.randint(1, min(experts, 6)), rng.choice([8, 24, 30, 64, 13, 128]))

    def rotation(dim):
        dims = rng.choice([d for d in (2, 4, 6, 8, 16, 20, 32, 64, 128, dim) if d <= dim and d % 2 == 0])
        return rot(rng.choice([20.0, 500.0, 10000.0, 300000.0]), dims, rng.choice([None, None, 1.0, 2.0, 16.0]))

    def heads():
        groups = rng.choice([1, 1, 2, 3, 4])
        return groups * rng.choice([1, 2, 3, 4, 6, 8, 17]), groups

    def layer():
        kind = rng.random()
        H, G = heads()
        if kind < 0.36:
            dim = rng.choice([8, 16, 24, 32, 64, 128, 20, 96])
            return pooled(H, G, dim, rng.choice([8, 16, 20, 32, 64, 128, 40]), rng.choice([1, 3, 8, 17, 40, 64, 100]),
                          rng.choice([1, 2, 5, 8, 16, 24, 50]), rotation(dim), rng.uniform(0.05, 0.4), feed_forward())
        if kind < 0.72:
            dim = rng.choice([8, 16, 24, 32, 64, 128, 20, 96])
            return kept(H, G, dim, rng.choice([8, 16, 20, 32, 64, 128, 40]), rng.choice([1, 3, 8, 17, 40, 64, 100]),
                        rng.choice([0, 1, 4, 16, 20, 33, 70]), rotation(dim), rng.uniform(0.05, 0.4), feed_forward())
        H = min(H, 8)
        H -= H % G
        return delta(max(H, G), G, rng.choice([4, 8, 16, 32, 48, 64, 96, 128, 200]), rng.choice([4, 8, 20, 32, 64, 128, 9]),
                     rng.randint(1, 5), feed_forward())

    layers = [layer() for _ in range(rng.randint(1, 5))]
    for _ in range(rng.choice([0, 0, 1, 2])):
        layers.append(again(layers, rng.randrange(len([l for l in layers if "weights_of" not in l]))))
    return model(rng.randint(50, 700), width, rng.choice([0.5, 0.8, 1.0, 1.4]), rng.choice([1e-5, 1e-6]), layers)


@pytest.mark.parametrize("seed,dtype", [(s, "float32") for s in list(range(12)) + list(range(100, 108))] + [(s, "bfloat16") for s in range(100, 108)])
def test_a_configuration_drawn_at_random(tmp_path, cuda_device, seed, dtype):
    drawn = draw_config(seed)
    # bfloat16 models take every expert: a choice between close logits is float32's to test
    config = drawn if dtype == "float32" else without_choice(drawn)
    folder = write_model(tmp_path / "model", config, seed=seed, dtype=DTYPES[dtype])
    rng = random.Random(seed + 1)
    requests = {f"r{i}": random_tokens(config["vocab"], rng.randint(1, 170), seed=seed * 10 + i) for i in range(6)}
    for build in (trace_mixed, trace_portions, functools.partial(trace_tail, tail=40)):
        steps = build(requests)
        rows = collect(steps, replay(folder, dtype, steps, page_size=rng.choice([16, 32, 64])))
        assert_rows_match(rows, requests, folder, dtype, f"seed {seed} {getattr(build, '__name__', 'trace_tail')}", least=0.3,
                          roundings=True)
