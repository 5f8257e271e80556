"""Fekotar on the CPU: its configuration, registry entry, declared tensors and stores, the frequencies of
its rotation, the plain routing rule, refused configurations, and the random-weights mode."""

import copy
import json
import math

import pytest
import torch

from fekotar_models import CONFIGS, make_weights, without_choice
from plain_fekotar import group_routing, pair_rows, rotation_frequencies
from zephyr_b200.cache import PagedCacheSpec, StateCacheSpec
from zephyr_b200.config import ConfigError, FekotarConfig
from zephyr_b200.config.registry import resolve_architecture
from zephyr_b200.parts import expected_weights
from zephyr_b200.parts.model import cache_specs
from zephyr_b200.parts.position import yarn_frequencies


@pytest.mark.parametrize("name", list(CONFIGS))
def test_configuration_to_spec_and_back(name):
    config = FekotarConfig.from_dict(CONFIGS[name])
    assert resolve_architecture(CONFIGS[name]).config_class is FekotarConfig
    assert FekotarConfig.from_dict(config.to_dict()).to_dict() == config.to_dict()
    spec = config.to_model_spec()
    assert spec.architecture == "Fekotar" and len(spec.layers) == len(CONFIGS[name]["layers"])
    assert all(layer.block == "parallel_residual" and set(layer.norms) == {"input"} for layer in spec.layers)
    assert spec.output.params["logit_scale"] == CONFIGS[name]["logit_scale"]
    pair = (CONFIGS[name].get("embedding") or {}).get("bigram")
    assert spec.input.kind == ("pair_embedding" if pair else "embedding")


@pytest.mark.parametrize("name", list(CONFIGS))
def test_declared_tensors_are_the_test_weights(name):
    spec = FekotarConfig.from_dict(CONFIGS[name]).to_model_spec()
    declared = expected_weights(spec)
    made = make_weights(CONFIGS[name], seed=1)
    assert set(declared) == set(made)
    for tensor_name, decl in declared.items():
        assert tuple(decl.shape) == tuple(made[tensor_name].shape), tensor_name


def test_stores():
    """A layer keeps one row of kv_rank + rot_dim values a position, keys only; the pair table adds one
    int32 per request behind the layers' stores, and a model without it keeps no state."""
    spec = FekotarConfig.from_dict(CONFIGS["A"]).to_model_spec()
    stores = cache_specs(spec)
    mixers = [layer["mixer"] for layer in CONFIGS["A"]["layers"]]
    assert stores[:-1] == [PagedCacheSpec(1, key_dim=m["kv_rank"] + m["rot_dim"], keys_only=True) for m in mixers]
    assert stores[-1] == StateCacheSpec((1,), "int32")
    assert all(isinstance(s, PagedCacheSpec) for s in cache_specs(FekotarConfig.from_dict(CONFIGS["B"]).to_model_spec()))


def test_frequencies():
    rot = {"dims": 16, "base": 300.0, "scaling": {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 0.5}}
    plain, mult = rotation_frequencies(rot)
    base = [300.0 ** (-2.0 * i / 16) for i in range(8)]
    ours, our_mult = yarn_frequencies(base, 16, 300.0, 4.0, 64, 8.0, 0.5)
    assert mult == our_mult == pytest.approx(0.1 * math.log(4.0) + 1.0)
    assert ours == pytest.approx(plain.tolist(), rel=1e-14)
    assert ours[0] == base[0] and ours[-1] == pytest.approx(base[-1] / 4.0)       # fast ones stay, slow ones are divided
    assert any(b / 4.0 < o < b for o, b in zip(ours, base))                        # and some lie on the ramp
    unscaled, one = rotation_frequencies({"dims": 16, "base": 300.0, "scaling": None})
    assert one == 1.0 and unscaled.tolist() == pytest.approx(base)


def test_the_plain_rules():
    assert pair_rows([4, 9, 9], 7, 3, 5) == [7, (4 * 3 + 9 * 5) % 7, (9 * 3 + 9 * 5) % 7]
    z = torch.tensor([[3.0, -9.0, 1.5, 1.4, 0.0, -1.0]], dtype=torch.float64)
    ids, weights, margin = group_routing(z, {"experts": 6, "top": 2, "scale": 2.0, "groups": {"count": 3, "keep": 1}})
    assert ids.tolist() == [[2, 3]]             # the group whose two best add up to most, not the group of the best
    assert weights[0].tolist() == pytest.approx([2.0 / (1 + math.exp(-1.5)), 2.0 / (1 + math.exp(-1.4))])
    ids, _, _ = group_routing(z, {"experts": 6, "top": 2, "scale": 1.0})
    assert ids.tolist() == [[0, 2]]
    assert float(margin) > 0


@pytest.mark.parametrize("change,words", [
    (lambda c: c["layers"][0].update(type="attention"), "unknown layer type"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=4), "rot.dims must equal rot_dim"),
    (lambda c: c["layers"][0]["mixer"].update(rot_dim=7), "even"),
    (lambda c: c["layers"][0]["mlp"].update(limit=0.0), "limit"),
    (lambda c: c["layers"][1]["mlp"]["router"]["groups"].update(count=3), "groups"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=9), "top"),
    (lambda c: c["embedding"]["bigram"].update(buckets=0), "buckets"),
    (lambda c: c.update(architecture="Other"), "not a Fekotar"),
])
def test_refused_configurations(change, words):
    config = copy.deepcopy(CONFIGS["A"])
    change(config)
    with pytest.raises(ConfigError, match=words):
        FekotarConfig.from_dict(config)


def test_a_model_without_choice_is_the_same_model():
    changed = without_choice(CONFIGS["A"])
    assert changed["layers"][1]["mlp"]["router"]["top"] == 8 and CONFIGS["A"]["layers"][1]["mlp"]["router"]["top"] == 3
    FekotarConfig.from_dict(changed).to_model_spec()


def test_random_model(tmp_path):
    from zephyr_b200.cli import main
    from zephyr_b200.weights import Checkpoint

    path = tmp_path / "config.json"
    path.write_text(json.dumps(CONFIGS["C"]))
    assert main(["random-model", "--config", str(path), "--seed", "3", "--out", str(tmp_path / "model")]) == 0
    store = Checkpoint(tmp_path / "model")
    assert set(store.names()) == set(expected_weights(FekotarConfig.from_dict(CONFIGS["C"]).to_model_spec()))
    assert json.loads((tmp_path / "model" / "config.json").read_text())["architecture"] == "Fekotar"
