"""Fekotar configurations drawn at random (sizes that are no multiples of anything in particular, layers in
any number whose sizes differ from one another, every optional piece present or absent, cached rows that the
tensor-core attention kernels take and rows that they do not), each replayed in a mixed trace, in portions
and with a decoded tail against the plain implementation: what a particular choice of sizes would hide,
another one shows."""

import functools
import random

import pytest

from fekotar_models import dense, latent, moe, without_choice, write_model, yarn
from replay_util import collect, random_tokens, trace_mixed, trace_portions, trace_tail
from test_fekotar_gpu import DTYPES, assert_rows_match, replay

pytestmark = pytest.mark.gpu


def draw_config(seed: int) -> dict:
    rng = random.Random(seed)
    width = rng.choice([40, 72, 100, 136, 50, 256, 33, 320])

    def feed_forward():
        kind = rng.random()
        if kind < 0.15:
            return None
        if kind < 0.5:
            return dense(rng.choice([48, 100, 36, 44, 256, 27]), rng.choice([0.5, 1.0, 2.0, 7.0]))
        count = rng.choice([1, 2, 3, 4, 5])
        per_group = rng.choice([1, 2, 3, 4])             # a group's mark adds its two largest scores (or its one)
        experts = count * per_group
        keep = rng.randint(1, count)
        top = rng.randint(1, min(keep * per_group, 6))
        groups = (count, keep) if rng.random() < 0.8 else None
        return moe(experts, top, rng.choice([8, 24, 30, 64, 13]), scale=rng.choice([0.5, 1.0, 2.0, 2.5]), groups=groups)

    def rotated():
        # the cached row is kv_rank + rot_dim values: 32, 64, 96 and 128 go to the tensor-core kernels in bfloat16
        rank, rot = rng.choice([(96, 32), (48, 16), (24, 8), (64, 64), (112, 16), (20, 12), (130, 30), (56, 0), (27, 6),
                                (256, 64), (128, 32), (36, 28)])
        scaling = None
        if rot and rng.random() < 0.7:
            original = rng.choice([16, 32, 64, 512])
            scaling = yarn(rng.choice([1.5, 2.0, 4.0, 8.0]), original, rng.choice([32.0, 8.0, 4.0]), rng.choice([1.0, 0.5, 2.0]))
        return rank, rot, scaling, rng.choice([20.0, 500.0, 10000.0, 80000.0])

    layers = []
    for _ in range(rng.randint(1, 6)):
        rank, rot, scaling, base = rotated()
        layers.append(latent(rng.choice([1, 2, 3, 5, 8, 12, 18]), rng.choice([4, 8, 16, 24, 32, 7, 64]), rot,
                             rng.choice([4, 8, 20, 32, 48, 64, 9]), rank, rng.choice([8, 12, 40, 80, 17]),
                             rng.uniform(0.05, 0.4), feed_forward(), base=base, scaling=scaling))
    config = {"architecture": "Fekotar", "vocab": rng.randint(50, 700), "width": width,
              "logit_scale": rng.choice([0.25, 0.5, 1.0, 3.0]), "norm": {"eps": rng.choice([1e-5, 1e-6])}, "layers": layers}
    if rng.random() < 0.75:
        config["embedding"] = {"bigram": {"buckets": rng.choice([7, 53, 1019, 4099]), "mul_prev": rng.choice([1, 31, 131, 100003]),
                                          "mul_cur": rng.choice([1, 19, 7, 99991])}}
    return config


@pytest.mark.parametrize("seed,dtype", [(s, "float32") for s in range(10)] + [(s, "bfloat16") for s in range(100, 106)])
def test_a_configuration_drawn_at_random(tmp_path, cuda_device, seed, dtype):
    drawn = draw_config(seed)
    # bfloat16 models take every expert: a choice between close scores is float32's to test
    config = drawn if dtype == "float32" else without_choice(drawn)
    folder = write_model(tmp_path / "model", config, seed=seed, dtype=DTYPES[dtype])
    rng = random.Random(seed + 1)
    requests = {f"r{i}": random_tokens(config["vocab"], rng.randint(1, 170), seed=seed * 10 + i) for i in range(6)}
    for build in (trace_mixed, trace_portions, functools.partial(trace_tail, tail=40)):
        steps = build(requests)
        rows = collect(steps, replay(folder, dtype, steps, page_size=rng.choice([16, 32, 64])))
        assert_rows_match(rows, requests, folder, dtype, f"seed {seed} {getattr(build, '__name__', 'trace_tail')}")
