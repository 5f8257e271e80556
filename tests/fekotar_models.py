"""Small Fekotar configurations and weights for the tests: sizes that differ from one another in every way the
design allows (head counts, unrotated and rotated and value sizes unlike each other, cached rows of 32, 64
and 128 values, which the tensor-core attention kernels take, and of 36, 48 and 160, which they do not, with
and without YaRN, with and without the hashed pair table, a logit multiplier of one and others, bounds
that cut a large and a small share, routers with and without groups, that keep all groups or one, that take
one expert or all, a layer without a feed-forward, a layer without a rotated part, widths and inner sizes
that are no multiples of eight)."""

from __future__ import annotations

import copy
import json
from pathlib import Path

import torch


def latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, mlp, base=10000.0, scaling=None):
    mixer = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank, "scale": scale}
    if rot_dim:
        mixer["rot"] = {"base": base, "dims": rot_dim, "scaling": scaling}
    return {"type": "latent_attention", "mixer": mixer, "mlp": mlp}


def yarn(factor, original, fast, slow):
    return {"factor": factor, "original": original, "fast": fast, "slow": slow}


def dense(ff, limit):
    return {"kind": "dense", "ff": ff, "limit": limit}


def moe(experts, top, ff, scale=1.0, groups=None):
    router = {"experts": experts, "top": top, "scale": scale}
    if groups is not None:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    return {"kind": "moe", "expert": {"ff": ff}, "router": router}


CONFIGS = {
    # A: cached rows that only the general attention kernel takes beside one of 32 values; a pair table; a
    # layer without a feed-forward; a layer without a rotated part; groups of two experts
    "A": {"architecture": "Fekotar", "vocab": 97, "width": 64, "logit_scale": 0.7, "norm": {"eps": 1e-5},
          "embedding": {"bigram": {"buckets": 53, "mul_prev": 31, "mul_cur": 7}}, "layers": [
        latent(3, 16, 8, 24, 40, 20, 0.3, dense(80, 2.0), base=500.0, scaling=yarn(4.0, 64, 8.0, 2.0)),
        latent(2, 8, 16, 40, 20, 12, 0.5, moe(8, 3, 40, scale=1.5, groups=(4, 2)), base=10000.0),
        latent(4, 12, 0, 6, 36, 30, 0.4, None),
        latent(6, 16, 4, 8, 28, 16, 0.25, moe(6, 1, 56, scale=0.5), base=100.0, scaling=yarn(1.5, 32, 4.0, 0.5))]},
    # B: no pair table, a logit multiplier of one, a width that is no power of two, cached rows of 128 and 64
    # values (the tensor-core kernels in bfloat16), a router whose groups are all kept, an inner size that is
    # no multiple of eight, a bound that cuts most values
    "B": {"architecture": "Fekotar", "vocab": 131, "width": 96, "logit_scale": 1.0, "norm": {"eps": 1e-6}, "layers": [
        latent(8, 24, 32, 16, 96, 40, 0.2, moe(9, 2, 36, scale=1.0, groups=(3, 3)), base=2000.0, scaling=yarn(8.0, 128, 16.0, 1.0)),
        latent(5, 32, 16, 32, 48, 64, 0.15, dense(50, 0.5), base=70000.0),
        latent(2, 40, 8, 20, 56, 8, 0.3, moe(4, 4, 20, scale=2.5))]},
    # C: pages of 32, sixteen heads on a cached row of 128, a row of 160, one group kept of two, one value a head
    "C": {"architecture": "Fekotar", "vocab": 64, "width": 128, "logit_scale": 2.0, "norm": {"eps": 1e-6},
          "embedding": {"bigram": {"buckets": 200, "mul_prev": 3, "mul_cur": 1001}}, "layers": [
        latent(16, 16, 64, 8, 64, 48, 0.2, moe(12, 4, 24, scale=0.8, groups=(2, 1)), base=300.0, scaling=yarn(2.0, 16, 2.0, 0.25)),
        latent(4, 32, 32, 1, 128, 32, 0.1, dense(160, 1.5), base=1000.0, scaling=yarn(3.0, 100, 10.0, 3.0)),
        latent(1, 64, 2, 64, 30, 16, 0.4, dense(24, 4.0), base=20.0)]},
}
PAGE_SIZE = {"A": 16, "B": 16, "C": 32}


def without_choice(config: dict) -> dict:
    """The same model with routers that take every expert (all groups kept): the weights stay each token's
    own, and no rounding of a layer's input can change which experts run."""
    out = copy.deepcopy(config)
    for layer in out["layers"]:
        mlp = layer.get("mlp")
        if mlp is not None and mlp["kind"] == "moe":
            router = mlp["router"]
            router["top"] = router["experts"]
            if router.get("groups") is not None:
                router["groups"]["keep"] = router["groups"]["count"]
    return out


def make_weights(config: dict, seed: int) -> dict[str, torch.Tensor]:
    """Float32 tensors by name, from distributions that keep every mechanism alive: scales around one, gates
    on both sides of one half, biases that matter, products whose values reach the bounds, router logits
    spread wide enough that scores are told apart."""
    g = torch.Generator().manual_seed(seed)
    width = config["width"]

    def normal(*shape, std=1.0, mean=0.0):
        return torch.randn(*shape, generator=g) * std + mean

    def linear(out, inp, gain=1.0):
        return normal(out, inp, std=gain * inp ** -0.5)

    W = {"embed": normal(config["vocab"], width), "final.norm": normal(width, std=0.1, mean=1.0),
         "head": linear(config["vocab"], width)}
    pair = (config.get("embedding") or {}).get("bigram")
    if pair:
        W["bigram"] = normal(pair["buckets"] + 1, width, std=0.7)
    for index, layer in enumerate(config["layers"]):
        L, m = f"l{index}", layer["mixer"]
        heads, dim, rot, vdim, rank, q_rank = (m[k] for k in ("heads", "dim", "rot_dim", "vdim", "kv_rank", "q_rank"))
        W[f"{L}.norm1"] = normal(width, std=0.1, mean=1.0)
        W.update({f"{L}.mix.dq": linear(q_rank, width), f"{L}.mix.dq.norm": normal(q_rank, std=0.2, mean=1.0),
                  f"{L}.mix.uq": linear(heads * (dim + rot), q_rank, 1.5), f"{L}.mix.dkv": linear(rank + rot, width, 1.5),
                  f"{L}.mix.dkv.norm": normal(rank, std=0.2, mean=1.0), f"{L}.mix.uk": linear(heads * dim, rank, 2.0),
                  f"{L}.mix.uv": linear(heads * vdim, rank), f"{L}.mix.g": linear(heads * vdim, width, 1.5),
                  f"{L}.mix.o": linear(width, heads * vdim)})
        mlp = layer["mlp"]
        if mlp is None:
            continue
        if mlp["kind"] == "dense":
            ff = mlp["ff"]
            W.update({f"{L}.mlp.gate": linear(ff, width, 1.5), f"{L}.mlp.gate.b": normal(ff, std=0.3),
                      f"{L}.mlp.up": linear(ff, width, 1.5), f"{L}.mlp.up.b": normal(ff, std=0.3),
                      f"{L}.mlp.down": linear(width, ff), f"{L}.mlp.down.b": normal(width, std=0.3)})
        else:
            ff, experts = mlp["expert"]["ff"], mlp["router"]["experts"]
            W[f"{L}.mlp.router"] = linear(experts, width, 2.0)
            for e in range(experts):
                W.update({f"{L}.mlp.e{e}.gate": linear(ff, width), f"{L}.mlp.e{e}.up": linear(ff, width),
                          f"{L}.mlp.e{e}.down": linear(width, ff)})
    return W


def write_model(folder: Path, config: dict, seed: int, dtype: torch.dtype) -> Path:
    """config.json and model.safetensors in ``dtype``.  The plain implementation reads the stored
    (rounded) values back, so both sides start from the same numbers."""
    from zephyr_b200.weights.safetensors_io import save_safetensors

    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(config, indent=1))
    save_safetensors(folder / "model.safetensors",
                     {name: t.to(dtype).contiguous() for name, t in make_weights(config, seed).items()})
    return folder


def read_model(folder: Path) -> tuple[dict, dict[str, torch.Tensor]]:
    from zephyr_b200.weights import Checkpoint

    store = Checkpoint(folder)
    return json.loads((Path(folder) / "config.json").read_text()), {name: store.read(name) for name in store.names()}
