"""Fekotar, plainly: float64 on the CPU, one function per mechanism, written from the design's equations.
It shares no code with the package; the tests compare the engine with it.

A layer:  h = rmsnorm(x) w;  x <- x + (mixer(h) + ff(h)).
"""

from __future__ import annotations

import math

import torch

F64 = torch.float64
GATE_SLOPE = 1.702


def rms_norm(x: torch.Tensor, eps: float, w: torch.Tensor | None = None) -> torch.Tensor:
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if w is None else y * w


# ------------------------------------------------------------------------------------------ embedding
def pair_rows(tokens: list[int], buckets: int, mul_prev: int, mul_cur: int) -> list[int]:
    """The row of the second table for every token: a hash of the token and the one before it; the table's
    last row (number ``buckets``) for a sequence's first token."""
    rows = [buckets]
    for prev, cur in zip(tokens[:-1], tokens[1:]):
        rows.append((prev * mul_prev + cur * mul_cur) % buckets)
    return rows


def embed(config: dict, W: dict, tokens: list[int]) -> torch.Tensor:
    x = W["embed"].to(F64)[torch.tensor(tokens)]
    pair = (config.get("embedding") or {}).get("bigram")
    if pair:
        rows = pair_rows(tokens, pair["buckets"], pair["mul_prev"], pair["mul_cur"])
        x = x + W["bigram"].to(F64)[torch.tensor(rows)]
    return x


# ------------------------------------------------------------------------------------------- rotation
def rotation_frequencies(rot: dict) -> tuple[torch.Tensor, float]:
    """f_i = base^(-2i/dims), with YaRN: the ramp over the dimension index between the dimensions that make
    ``fast`` and ``slow`` turns over ``original`` positions; returns (frequencies, multiplier on cos and sin)."""
    dims, base = rot["dims"], rot["base"]
    freqs = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    scaling = rot.get("scaling")
    if not scaling:
        return torch.tensor(freqs, dtype=F64), 1.0
    factor, original = scaling["factor"], scaling["original"]

    def dim_of(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(dim_of(scaling["fast"])), 0)
    hi = min(math.ceil(dim_of(scaling["slow"])), dims - 1)
    scaled = []
    for i, f in enumerate(freqs):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        scaled.append(f / factor * ramp + f * (1.0 - ramp))
    return torch.tensor(scaled, dtype=F64), 0.1 * math.log(factor) + 1.0


def rotate_halves(x: torch.Tensor, positions: torch.Tensor, freqs: torch.Tensor, mult: float) -> torch.Tensor:
    """x [T, heads, dims]: dimension i pairs with i + dims/2; (u, v) -> (u c - v s, v c + u s)."""
    half = x.shape[-1] // 2
    angle = positions.to(F64)[:, None] * freqs[None, :]
    c, s = (torch.cos(angle) * mult)[:, None, :], (torch.sin(angle) * mult)[:, None, :]
    u, v = x[..., :half], x[..., half:]
    return torch.cat([u * c - v * s, v * c + u * s], dim=-1)


# ------------------------------------------------------------------------------------ latent attention
def latent_attention(W: dict, prefix: str, m: dict, h: torch.Tensor, eps: float) -> torch.Tensor:
    T = h.shape[0]
    heads, dim, rot, vdim, rank = m["heads"], m["dim"], m.get("rot_dim", 0), m["vdim"], m["kv_rank"]
    w = lambda name: W[f"{prefix}.{name}"].to(F64)
    q_latent = rms_norm(h @ w("dq").T, eps, w("dq.norm"))
    q = (q_latent @ w("uq").T).view(T, heads, dim + rot)
    down = h @ w("dkv").T
    c = rms_norm(down[:, :rank], eps, w("dkv.norm"))
    k = (c @ w("uk").T).view(T, heads, dim)
    v = (c @ w("uv").T).view(T, heads, vdim)
    scores = torch.einsum("ihd,jhd->hij", q[..., :dim], k)
    if rot:
        freqs, mult = rotation_frequencies(m["rot"])
        positions = torch.arange(T)
        q_rot = rotate_halves(q[..., dim:], positions, freqs, mult)
        k_rot = rotate_halves(down[:, rank:].view(T, 1, rot), positions, freqs, mult)[:, 0]
        scores = scores + torch.einsum("ihd,jd->hij", q_rot, k_rot)
    scores = scores * m["scale"]
    visible = torch.ones(T, T, dtype=torch.bool).tril()
    probs = torch.softmax(scores.masked_fill(~visible, -math.inf), dim=-1)
    out = torch.einsum("hij,jhd->ihd", probs, v).reshape(T, heads * vdim)
    out = out * torch.sigmoid(h @ w("g").T)
    return out @ w("o").T


# --------------------------------------------------------------------------------------- feed-forwards
def bounded_feed_forward(W: dict, prefix: str, mlp: dict, h: torch.Tensor) -> torch.Tensor:
    w = lambda name: W[f"{prefix}.{name}"].to(F64)
    limit = mlp["limit"]
    g = torch.clamp(h @ w("gate").T + w("gate.b"), max=limit)
    u = torch.clamp(h @ w("up").T + w("up.b"), min=-limit, max=limit)
    return (g * torch.sigmoid(GATE_SLOPE * g) * (u + 1.0)) @ w("down").T + w("down.b")


def group_routing(z: torch.Tensor, router: dict) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Router logits [T, experts] -> (ids [T, top], weights [T, top], margin [T]).  Scores are sigmoid(z); only
    experts of the ``keep`` groups whose two largest scores add up to most can be taken; the ``top`` largest
    allowed scores are taken, weighted by score * scale.  The margin is the smallest gap a rounding would
    have to bridge to change the choice: between the last kept and the first dropped group, and between the
    last taken and the first untaken allowed expert."""
    T, experts = z.shape
    top = router["top"]
    s = torch.sigmoid(z)
    margin = torch.full((T,), math.inf, dtype=F64)
    allowed = torch.ones(T, experts, dtype=torch.bool)
    groups = router.get("groups")
    if groups and groups["count"] > 1 and groups["keep"] < groups["count"]:
        count, keep = groups["count"], groups["keep"]
        per = experts // count
        marks = s.view(T, count, per).topk(min(2, per), dim=-1).values.sum(-1)
        ordered = marks.sort(dim=-1, descending=True)
        margin = torch.minimum(margin, ordered.values[:, keep - 1] - ordered.values[:, keep])
        kept = torch.zeros(T, count, dtype=torch.bool)
        kept.scatter_(1, ordered.indices[:, :keep], True)
        allowed = kept[:, :, None].expand(T, count, per).reshape(T, experts)
    masked = torch.where(allowed, s, torch.full_like(s, -1.0))
    ordered = masked.sort(dim=-1, descending=True)
    ids = ordered.indices[:, :top]
    if top < experts:
        gap = ordered.values[:, top - 1] - ordered.values[:, top]
        gap = torch.where(ordered.values[:, top] < 0, torch.full_like(gap, math.inf), gap)    # nothing left to take instead
        margin = torch.minimum(margin, gap)
    weights = torch.gather(s, 1, ids) * float(router.get("scale", 1.0))
    return ids, weights, margin


def routed_feed_forward(W: dict, prefix: str, mlp: dict, h: torch.Tensor, margins: list | None = None) -> torch.Tensor:
    ids, weights, margin = group_routing(h @ W[f"{prefix}.router"].to(F64).T, mlp["router"])
    if margins is not None:
        margins.append(margin.numpy())
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, weight in zip(ids[t].tolist(), weights[t]):
            gate = h[t] @ W[f"{prefix}.e{e}.gate"].to(F64).T
            up = h[t] @ W[f"{prefix}.e{e}.up"].to(F64).T
            out[t] += weight * ((gate * torch.sigmoid(gate) * up) @ W[f"{prefix}.e{e}.down"].to(F64).T)
    return out


# ---------------------------------------------------------------------------------------------- model
def forward(config: dict, W: dict, tokens: list[int], margins: list | None = None, streams: list | None = None) -> torch.Tensor:
    """Logits [T, vocab] of one sequence.  ``margins`` collects every routed layer's per-position margin,
    ``streams`` the residual stream after every layer."""
    eps = config["norm"]["eps"]
    x = embed(config, W, tokens)
    for index, layer in enumerate(config["layers"]):
        h = rms_norm(x, eps, W[f"l{index}.norm1"].to(F64))
        total = latent_attention(W, f"l{index}.mix", layer["mixer"], h, eps)
        mlp = layer.get("mlp")
        if mlp is not None and mlp["kind"] == "dense":
            total = total + bounded_feed_forward(W, f"l{index}.mlp", mlp, h)
        elif mlp is not None:
            total = total + routed_feed_forward(W, f"l{index}.mlp", mlp, h, margins)
        x = x + total
        if streams is not None:
            streams.append(x.clone())
    h = rms_norm(x, eps, W["final.norm"].to(F64))
    return (h @ W["head"].to(F64).T) * float(config.get("logit_scale", 1.0))
