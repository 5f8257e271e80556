"""Rizovik on the host: reading config.json, the model spec it turns into, the tensors it declares, the stores of
its layers (a pooled layer keeps a second store of one entry per block; a layer that runs another layer's tensors
has stores of its own), pages that a window gives back while a kept start stays, the rotation's frequencies, the
plain rules, and ``random-model``."""

import copy
import json

import pytest
import torch

from plain_rizovik import F64, kept_window_mask, pooled_window_mask, rotation_frequencies, route, short_convolution
from rizovik_models import CONFIGS, make_weights


def test_the_registry_finds_the_design_by_its_own_key():
    from zephyr_b200.config import RizovikConfig, resolve_architecture

    assert resolve_architecture(CONFIGS["A"]).config_class is RizovikConfig
    config = RizovikConfig.from_dict(CONFIGS["B"])
    assert RizovikConfig.from_dict(config.to_dict()) == config
    assert json.loads(json.dumps(config.to_dict())) == CONFIGS["B"]


@pytest.mark.parametrize("name", list(CONFIGS))
def test_declared_tensors_are_the_checkpoints(name):
    from zephyr_b200.config import RizovikConfig
    from zephyr_b200.parts import expected_weights

    weights = make_weights(CONFIGS[name], seed=1)
    declared = expected_weights(RizovikConfig.from_dict(CONFIGS[name]).to_model_spec())
    assert set(declared) == set(weights)
    for tensor_name, decl in declared.items():
        assert tuple(weights[tensor_name].shape) == decl.shape, tensor_name


def test_the_spec_names_every_mechanism_with_its_constants():
    from zephyr_b200.cache import PagedCacheSpec, StateCacheSpec
    from zephyr_b200.config import RizovikConfig
    from zephyr_b200.parts import cache_specs

    spec = RizovikConfig.from_dict(CONFIGS["A"]).to_model_spec()
    # six entries, four with tensors of their own: the run order names two layers twice, each time with new stores
    assert len(spec.layers) == 4 and [call.layer for call in spec.run_order] == [0, 1, 2, 3, 0, 2]
    assert [call.caches for call in spec.run_order] == [(0, 1), (2,), (3,), (4,), (5, 6), (7,)]
    stores = cache_specs(spec)
    # the tokens of a pooled layer stay until window and block have both passed them; the blocks' store holds
    # one entry per block and keeps them all
    assert stores[0] == stores[5] == PagedCacheSpec(2, key_dim=24, value_dim=40, window=19)
    assert stores[1] == stores[6] == PagedCacheSpec(2, key_dim=24, value_dim=40, every=5)
    assert stores[2] == PagedCacheSpec(3, key_dim=20, value_dim=12, window=23, keep_first=7)
    assert stores[4] == PagedCacheSpec(2, key_dim=48, window=9)
    assert stores[3] == stores[7] == StateCacheSpec((4 * 24 * 20 + 2 * (2 * 2 * 24 + 4 * 20),), "float32")
    wide = RizovikConfig.from_dict(CONFIGS["B"]).to_model_spec()
    assert cache_specs(wide)[1].window == 64 and wide.layers[1].mixer.params["window"] == 36     # a block longer than the window
    assert [layer.block for layer in spec.layers] == ["outnorm_residual"] * 4
    assert all(layer.block_params == {"residual_mult": 0.6} for layer in spec.layers)
    assert all(norm.kind == "rmsnorm" for layer in spec.layers for norm in layer.norms.values())
    assert spec.output.params["weight"] == "embed"                              # the head is the table itself
    first, second, third = (spec.layers[i].mixer for i in range(3))
    assert first.kind == second.kind == "attention" and third.kind == "gated_delta"
    assert first.params["qk_norm"] == "whole" and first.params["value_unit_norm"] and first.params["pool"] == 5
    assert first.params["out_gate"] == "l0.mix.g" and "head_mix" not in first.params and first.params["scale"] == 0.25
    assert second.params["qk_norm"] == "per_head" and second.params["keep_first"] == 7 and second.params["head_mix"] == "l1.mix.talk"
    assert first.position.kind == "rope_halves" and first.position.params["dims"] == 16 and first.position.params["scaling"] is None
    assert second.position.params["scaling"] == {"kind": "linear", "factor": 4.0}
    assert (third.params["heads"], third.params["qk_heads"], third.params["key_dim"], third.params["value_dim"], third.params["conv"]) == (4, 2, 24, 20, 3)
    routed = spec.layers[0].feed_forward
    assert routed.kind == "routed" and routed.params["scores"] == "top_softmax" and routed.params["router_bias"] == "l0.mlp.router.b"
    assert spec.layers[2].feed_forward is None and set(spec.layers[2].norms) == {"mixer_out"}


def test_an_entry_with_constants_of_its_own_over_another_layers_tensors():
    from zephyr_b200.config import RizovikConfig
    from zephyr_b200.parts import expected_weights

    config = copy.deepcopy(CONFIGS["A"])
    config["layers"][4]["mixer"]["mask"]["size"] = 31
    spec = RizovikConfig.from_dict(config).to_model_spec()
    assert len(spec.layers) == 5 and [call.layer for call in spec.run_order] == [0, 1, 2, 3, 4, 2]
    assert spec.layers[4].mixer.params["window"] == 31 and spec.layers[4].mixer.params["q_proj"] == "l0.mix.q"
    assert set(expected_weights(spec)) == set(make_weights(CONFIGS["A"], seed=1))


@pytest.mark.parametrize("change,message", [
    (lambda c: c["layers"][0].update(type="conv"), "unknown layer type"),
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=4), "multiple of kv_heads"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=26), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"]["mask"].pop("pool"), "pool"),
    (lambda c: c["layers"][1]["mixer"]["mask"].update(keep_first=-1), "keep_first"),
    (lambda c: c["layers"][2]["mixer"].pop("conv"), "conv"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=8), "router.top"),
    (lambda c: c["layers"][0].update(mlp={"kind": "dense", "ff": 8}), "moe"),
    (lambda c: c["layers"][4].update(weights_of=4), "weights_of"),
    (lambda c: c["layers"][4].update(weights_of=9), "weights_of"),
    (lambda c: c.update(vocab=0), "vocab"),
    (lambda c: c.pop("norm"), "norm"),
])
def test_bad_configurations_are_refused(change, message):
    from zephyr_b200.config import ConfigError, RizovikConfig

    config = copy.deepcopy(CONFIGS["A"])
    change(config)
    with pytest.raises(ConfigError, match=message):
        RizovikConfig.from_dict(config)


def test_a_window_gives_pages_back_but_for_the_kept_start():
    """Pages of 4 positions, a window of 6 that keeps the first 5 tokens: the first two pages stay for good, the
    ones behind them go as the window passes; a store of one entry per 8 positions grows an eighth as fast."""
    from zephyr_b200.cache import CacheManager, PagedCacheSpec

    manager = CacheManager([PagedCacheSpec(1, key_dim=8, window=6, keep_first=5), PagedCacheSpec(1, key_dim=8, every=8),
                            PagedCacheSpec(1, key_dim=8, window=6)], page_size=4, num_pages=40, max_requests=3)
    assert len(manager.groups) == 3 and manager.groups[1].pool.num_pages < 40
    assert manager.add_request("a")
    for length in range(1, 60):
        assert manager.ensure_capacity("a", length)
        manager.commit("a", length)
        manager.check_invariants()
        kept, pooled, plain = (manager.block_table("a", g) for g in range(3))
        dead = max(0, (length - 6 + 1) // 4)
        assert [page != 0 for page in plain] == [block >= dead for block in range(len(plain))]
        assert [page != 0 for page in kept] == [block >= dead or block < 2 for block in range(len(kept))]
        assert len(pooled) == -(-(-(-length // 8)) // 4) and all(page != 0 for page in pooled)
    free_before = [manager.num_free_pages(g) for g in range(3)]
    manager.free_request("a")
    manager.check_invariants()
    assert [manager.num_free_pages(g) for g in range(3)] == [group.pool.num_usable for group in manager.groups]
    assert free_before[0] == manager.groups[0].pool.num_usable - 2 - len([b for b in range(15) if b >= (59 - 5) // 4])
    with pytest.raises(Exception):
        CacheManager([PagedCacheSpec(1, key_dim=8, window=6, every=2)], page_size=4, num_pages=8, max_requests=1)


def test_a_store_of_blocks_has_room_for_every_request():
    """As many requests as slots, each a little more than whole pages of blocks: the smaller pool still holds them."""
    from zephyr_b200.cache import CacheManager, PagedCacheSpec

    manager = CacheManager([PagedCacheSpec(1, key_dim=8), PagedCacheSpec(1, key_dim=8, every=3)], page_size=4, num_pages=26,
                           max_requests=4)
    for name, length in (("a", 13), ("b", 25), ("c", 37), ("d", 25)):         # 4 + 7 + 10 + 7 = 28 > 25 pages: d must wait
        assert manager.add_request(name)
        assert manager.ensure_capacity(name, length) == (name != "d")
    manager.free_request("a")
    assert manager.ensure_capacity("d", 25)
    manager.check_invariants()


def test_frequencies_masks_and_the_plain_rules():
    f = rotation_frequencies({"base": 100.0, "dims": 8})
    assert torch.allclose(f, torch.tensor([1.0, 100.0 ** -0.25, 0.1, 100.0 ** -0.75], dtype=F64))
    assert torch.allclose(rotation_frequencies({"base": 100.0, "dims": 8, "scaling": {"factor": 4.0}}), f / 4.0)
    from zephyr_b200.config.spec import PositionSpec
    from zephyr_b200.parts.position import RopeHalves
    part = RopeHalves(PositionSpec("rope_halves", 16, 64, {"base": 100.0, "dims": 8, "scaling": {"kind": "linear", "factor": 4.0}}),
                      torch.float32, "cpu")
    freqs, dims, mult = part.as_half_frequencies()
    assert dims == 8 and mult == 1.0 and torch.allclose(freqs.double(), f / 4.0, rtol=1e-7)
    # a window of 3 with blocks of 2: query 6 sees tokens 4, 5, 6 and the blocks that end at or before position 3
    tokens, blocks = pooled_window_mask(8, 3, 2)
    assert tokens[6].nonzero().flatten().tolist() == [4, 5, 6] and blocks[6].tolist() == [True, True, False, False]
    assert blocks[4].tolist() == [True, False, False, False] and not blocks[3].any()     # block 0 ends at 1 = 4 - 3
    # a window of 3 that keeps 2 tokens
    assert kept_window_mask(8, 3, 2)[6].nonzero().flatten().tolist() == [0, 1, 4, 5, 6]
    # the largest logits with their bias, weighted among themselves; equal logits go to the lower index
    w = {"r.router": torch.eye(4, dtype=F64), "r.router.b": torch.tensor([0.0, 0.0, 0.0, 3.0], dtype=F64)}
    ids, weights, margin = route(torch.tensor([[2.0, 1.0, 0.0, 0.0], [0.0, 0.0, 0.0, -3.0]], dtype=F64), w, "r", 2)
    assert ids.tolist() == [[3, 0], [0, 1]] and margin.tolist() == [1.0, 0.0]
    assert torch.allclose(weights[0], torch.softmax(torch.tensor([3.0, 2.0], dtype=F64), 0)) and weights[1].tolist() == [0.5, 0.5]
    # the last column of the taps weighs the current token; nothing comes before the start
    y = short_convolution(torch.tensor([[1.0], [2.0], [3.0]], dtype=F64), torch.tensor([[100.0, 10.0, 1.0]], dtype=F64))
    assert y.flatten().tolist() == [1.0, 12.0, 123.0]


def test_random_model_from_the_command_line(tmp_path):
    from zephyr_b200.cli import main
    from zephyr_b200.config import load_model_config
    from zephyr_b200.parts import expected_weights
    from zephyr_b200.weights import Checkpoint
    from zephyr_b200.weights.loader import check_store

    source = tmp_path / "config.json"
    source.write_text(json.dumps(CONFIGS["C"]))
    assert main(["random-model", "--config", str(source), "--out", str(tmp_path / "model"), "--seed", "3"]) == 0
    config = load_model_config(tmp_path / "model")
    assert config.to_dict() == CONFIGS["C"]
    store = Checkpoint(tmp_path / "model")
    check_store(store, expected_weights(config.to_model_spec()))
    assert tuple(store.shape("l0.mix.q.norm")) == (16 * 64,) and tuple(store.shape("l2.mix.talk")) == (8, 8)
