"""Small Rizovik configurations and weights for the tests: sizes that differ from one another in every way the
design allows (head counts and ratios, key and value sizes unlike each other and no multiples of 16, rotation
on part of a head and on all of it, with and without a divisor of the frequencies, windows smaller and larger
than a page, pooled blocks smaller and larger than the window and than a page, kept first tokens from none to
more than a page, one to eight taps, delta heads with few and many key channels, routers that take one expert
or all, a layer without a feed-forward, layers that run another layer's tensors, a multiplier of one)."""

from __future__ import annotations

import copy
import json
from pathlib import Path

import torch


def rot(base, dims, factor=None):
    out = {"base": base, "dims": dims}
    if factor is not None:
        out["scaling"] = {"factor": factor}
    return out


def pooled(heads, kv_heads, dim, vdim, size, pool, rotation, scale, mlp):
    return {"type": "attention", "mlp": mlp,
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "rot": rotation,
                      "mask": {"size": size, "pool": pool}}}


def kept(heads, kv_heads, dim, vdim, size, keep_first, rotation, scale, mlp):
    return {"type": "attention_2", "mlp": mlp,
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "rot": rotation,
                      "mask": {"size": size, "keep_first": keep_first}}}


def delta(heads, kv_heads, dim, vdim, conv, mlp):
    return {"type": "delta", "mlp": mlp,
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}}


def again(layers, source):
    """A layer that runs layer ``source``'s tensors: the same entry with ``weights_of``."""
    return {**copy.deepcopy(layers[source]), "weights_of": source}


def moe(experts, top, ff):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def model(vocab, width, mult, eps, layers):
    return {"architecture": "Rizovik", "vocab": vocab, "width": width, "residual_mult": mult, "norm": {"eps": eps},
            "layers": layers}


def _a_layers():
    layers = [pooled(4, 2, 24, 40, 19, 5, rot(300.0, 16), 0.25, moe(6, 2, 40)),
              kept(6, 3, 20, 12, 23, 7, rot(10000.0, 20, factor=4.0), 0.3, moe(5, 1, 24)),
              delta(4, 2, 24, 20, 3, None),
              kept(2, 2, 48, 48, 9, 0, rot(50.0, 8), 0.2, moe(4, 4, 36))]
    return layers + [again(layers, 0), again(layers, 2)]


def _b_layers():
    layers = [delta(3, 1, 96, 70, 4, moe(7, 3, 50)),
              pooled(8, 1, 32, 32, 36, 64, rot(300000.0, 32), 0.18, moe(9, 2, 72)),
              kept(5, 5, 16, 24, 70, 33, rot(1000.0, 6), 0.35, None),
              pooled(3, 3, 40, 8, 12, 12, rot(20.0, 40, factor=2.0), 0.22, moe(3, 2, 27))]
    return layers + [again(layers, 1)]


CONFIGS = {
    # A: a block smaller than its window and than a page, kept tokens fewer than a page and none, groups of
    # two, value heads wider and narrower than the keys, delta heads of few channels, layers run twice
    "A": model(97, 64, 0.6, 1e-5, _a_layers()),
    # B: a block larger than its window and than a page (tokens leave the window before their block is whole),
    # a block as long as the window, more kept tokens than a page holds, a multiplier of one, delta heads of 96
    # channels with one q/k head for three value heads, pages of 32
    "B": model(131, 96, 1.0, 1e-6, _b_layers()),
    # C: head sizes that the tensor-core kernels would take, 16 heads on 2, a window of one token, a block of
    # one token, eight taps and one tap
    "C": model(64, 128, 0.5, 1e-6, [
        pooled(16, 2, 64, 64, 1, 1, rot(1000.0, 64), 0.125, moe(11, 2, 24)),
        delta(2, 2, 16, 128, 8, moe(2, 1, 48)),
        kept(8, 4, 128, 128, 33, 40, rot(500000.0, 32, factor=16.0), 0.09, moe(4, 2, 16)),
        delta(6, 3, 128, 32, 1, None),
        pooled(2, 1, 128, 128, 50, 14, rot(100.0, 2), 0.1, moe(8, 3, 40))]),
}
PAGE_SIZE = {"A": 16, "B": 32, "C": 16}


def without_choice(config: dict) -> dict:
    """The same model with routers that take every expert: the weights stay each token's own, and no
    rounding of a layer's input can change which experts run."""
    out = copy.deepcopy(config)
    for layer in out["layers"]:
        if layer.get("mlp") is not None:
            layer["mlp"]["router"]["top"] = layer["mlp"]["router"]["experts"]
    return out


def make_weights(config: dict, seed: int) -> dict[str, torch.Tensor]:
    """Float32 tensors by name, from distributions that keep every mechanism alive: scales around one, gates
    on both sides of one half, a mixing matrix with entries of both signs beside its diagonal, decays between
    a half and one, router logits spread wide enough that they are told apart."""
    g = torch.Generator().manual_seed(seed)
    width = config["width"]

    def normal(*shape, std=1.0, mean=0.0):
        return torch.randn(*shape, generator=g) * std + mean

    def linear(out, inp, gain=1.0):
        return normal(out, inp, std=gain * inp ** -0.5)

    W = {"embed": normal(config["vocab"], width), "final.norm": normal(width, std=0.1, mean=1.0)}
    for index, layer in enumerate(config["layers"]):
        if "weights_of" in layer:
            continue
        L, m = f"l{index}", layer["mixer"]
        H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        W[f"{L}.norm1"] = normal(width, std=0.1, mean=1.0)
        if layer["type"] == "delta":
            taps = m["conv"]
            W.update({f"{L}.mix.q": linear(G * d, width, 2.0), f"{L}.mix.k": linear(G * d, width, 2.0),
                      f"{L}.mix.v": linear(H * dv, width, 2.0), f"{L}.mix.g": linear(H * dv, width, 1.5),
                      f"{L}.mix.q.conv": normal(G * d, taps, std=0.6), f"{L}.mix.k.conv": normal(G * d, taps, std=0.6),
                      f"{L}.mix.v.conv": normal(H * dv, taps, std=0.6),
                      f"{L}.mix.b": linear(H, width, 1.5), f"{L}.mix.a": linear(H, width, 1.5),
                      f"{L}.mix.A_log": normal(H, std=0.5, mean=-1.0), f"{L}.mix.dt_bias": normal(H, std=0.7),
                      f"{L}.mix.norm": normal(dv, std=0.2, mean=1.0), f"{L}.mix.o": linear(width, H * dv)})
        else:
            whole = layer["type"] == "attention"
            W.update({f"{L}.mix.q": linear(H * d, width, 1.5), f"{L}.mix.k": linear(G * d, width, 1.5),
                      f"{L}.mix.v": linear(G * dv, width, 1.5), f"{L}.mix.o": linear(width, H * dv),
                      f"{L}.mix.q.norm": normal(H * d if whole else d, std=0.3, mean=1.0),
                      f"{L}.mix.k.norm": normal(G * d if whole else d, std=0.3, mean=1.0)})
            if whole:
                W[f"{L}.mix.g"] = linear(H * dv, width, 1.5)
            else:
                W[f"{L}.mix.talk"] = torch.eye(H) * 0.8 + normal(H, H, std=0.3)
        mlp = layer.get("mlp")
        if mlp is None:
            continue
        ff, experts = mlp["expert"]["ff"], mlp["router"]["experts"]
        W[f"{L}.norm2"] = normal(width, std=0.1, mean=1.0)
        W[f"{L}.mlp.router"] = linear(experts, width, 2.0)
        W[f"{L}.mlp.router.b"] = normal(experts, std=0.5)
        for e in range(experts):
            W.update({f"{L}.mlp.e{e}.gate": linear(ff, width, 1.5), f"{L}.mlp.e{e}.up": linear(ff, width, 1.5),
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
