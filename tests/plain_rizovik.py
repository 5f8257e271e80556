"""A plain, slow Rizovik in float64: one function per mechanism, written from the design's equations
and sharing nothing with the package.  Weights come as a dict of torch tensors by checkpoint name; the
configuration is the design's own ``config.json`` dictionary.

The layer: x <- x + m N1(mixer(x)); x <- x + m N2(ff(x)), N being an RMS norm with a scale, m the model's
``residual_mult``; the parts read x itself.  A layer with ``weights_of``: j runs layer j's tensors on a
store of its own.  Mixers: ``attention`` (grouped heads, RMS norm over the whole q and the whole k,
rotation of halves on part of a head, unit-RMS values, a window of tokens and behind it the means of
whole blocks of keys and values, a sigmoid gate per output value); ``attention_2`` (per-head RMS norm of
q and k, rotation with frequencies divided by a factor, a window that also keeps the first tokens, the
heads' softmax weights mixed by a matrix); ``delta`` (the gated delta rule behind short causal
convolutions).  Feed-forward: routed SiLU experts chosen by the largest biased logits and weighted by
the softmax over the chosen logits.
"""

from __future__ import annotations

import math

import torch

F64 = torch.float64


def rms_unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return rms_unit(x, eps) * w


def rotation_frequencies(rot: dict) -> torch.Tensor:
    """f_i = base^(-2 i / dims), i < dims / 2, each divided by scaling.factor where there is one."""
    dims = int(rot["dims"])
    f = torch.tensor([float(rot["base"]) ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=F64)
    if rot.get("scaling"):
        f = f / float(rot["scaling"]["factor"])
    return f


def rotate_halves(x: torch.Tensor, positions: torch.Tensor, rot: dict) -> torch.Tensor:
    """x [T, heads, dim]: value i < dims / 2 of every head is turned together with value i + dims / 2 by
    the angle position * f_i; the values from dims on stay."""
    dims = int(rot["dims"])
    half = dims // 2
    angle = positions.to(F64).view(-1, 1, 1) * rotation_frequencies(rot).view(1, 1, half)
    c, s = torch.cos(angle), torch.sin(angle)
    a, b = x[..., :half], x[..., half:dims]
    return torch.cat([a * c - b * s, b * c + a * s, x[..., dims:]], dim=-1)


def softmax_over(scores: torch.Tensor, visible: torch.Tensor) -> torch.Tensor:
    scores = scores.masked_fill(~visible, -math.inf)
    e = torch.exp(scores - scores.max(-1, keepdim=True).values)
    return e / e.sum(-1, keepdim=True)


def pooled_window_mask(T: int, size: int, pool: int) -> tuple[torch.Tensor, torch.Tensor]:
    """(tokens [T, T], blocks [T, T // pool]): query i sees token j if 0 <= i - j < size, and block b (the
    positions b pool .. b pool + pool - 1) if its last position is at most i - size."""
    i = torch.arange(T).view(T, 1)
    j = torch.arange(T).view(1, T)
    tokens = (i - j >= 0) & (i - j < size)
    b = torch.arange(T // pool).view(1, -1)
    blocks = b * pool + pool - 1 <= i - size
    return tokens, blocks


def pooled_attention(h: torch.Tensor, w: dict, prefix: str, m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rms_norm(h @ w[f"{prefix}.q"].T, w[f"{prefix}.q.norm"], eps).view(T, H, d)
    k = rms_norm(h @ w[f"{prefix}.k"].T, w[f"{prefix}.k.norm"], eps).view(T, G, d)
    v = rms_unit((h @ w[f"{prefix}.v"].T).view(T, G, dv), eps)
    positions = torch.arange(T)
    q, k = rotate_halves(q, positions, m["rot"]), rotate_halves(k, positions, m["rot"])
    size, pool = int(m["mask"]["size"]), int(m["mask"]["pool"])
    nb = T // pool
    k_blocks = k[: nb * pool].view(nb, pool, G, d).mean(1)
    v_blocks = v[: nb * pool].view(nb, pool, G, dv).mean(1)
    tokens, blocks = pooled_window_mask(T, size, pool)
    visible = torch.cat([tokens, blocks], dim=1)
    per = H // G
    out = torch.zeros(T, H, dv, dtype=F64)
    for head in range(H):
        g = head // per
        keys = torch.cat([k[:, g], k_blocks[:, g]], dim=0)
        values = torch.cat([v[:, g], v_blocks[:, g]], dim=0)
        p = softmax_over(q[:, head] @ keys.T * m["scale"], visible)
        out[:, head] = p @ values
    gate = torch.sigmoid(h @ w[f"{prefix}.g"].T)
    return (out.reshape(T, H * dv) * gate) @ w[f"{prefix}.o"].T


def kept_window_mask(T: int, size: int, keep_first: int) -> torch.Tensor:
    i = torch.arange(T).view(T, 1)
    j = torch.arange(T).view(1, T)
    return (j <= i) & ((i - j < size) | (j < keep_first))


def mixed_heads_attention(h: torch.Tensor, w: dict, prefix: str, m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rms_norm((h @ w[f"{prefix}.q"].T).view(T, H, d), w[f"{prefix}.q.norm"], eps)
    k = rms_norm((h @ w[f"{prefix}.k"].T).view(T, G, d), w[f"{prefix}.k.norm"], eps)
    v = (h @ w[f"{prefix}.v"].T).view(T, G, dv)
    positions = torch.arange(T)
    q, k = rotate_halves(q, positions, m["rot"]), rotate_halves(k, positions, m["rot"])
    visible = kept_window_mask(T, int(m["mask"]["size"]), int(m["mask"].get("keep_first", 0)))
    per = H // G
    p = torch.stack([softmax_over(q[:, head] @ k[:, head // per].T * m["scale"], visible) for head in range(H)])
    mixed = torch.einsum("hg,gij->hij", w[f"{prefix}.talk"], p)
    out = torch.stack([mixed[head] @ v[:, head // per] for head in range(H)], dim=1)
    return out.reshape(T, H * dv) @ w[f"{prefix}.o"].T


def short_convolution(x: torch.Tensor, taps: torch.Tensor) -> torch.Tensor:
    """x [T, C], taps [C, n]: y_t = sum_j taps[:, n - 1 - j] x_{t - j}, zeros before the start."""
    T, n = x.shape[0], taps.shape[1]
    padded = torch.cat([torch.zeros(n - 1, x.shape[1], dtype=x.dtype), x], dim=0)
    y = torch.zeros_like(x)
    for j in range(n):
        y = y + padded[n - 1 - j: n - 1 - j + T] * taps[:, n - 1 - j]
    return y


def silu(x: torch.Tensor) -> torch.Tensor:
    return x * torch.sigmoid(x)


def delta_rule(q, k, v, beta, decay):
    """q, k [T, H, d], v [T, H, dv], beta and decay [T, H] -> [T, H, dv]; the state starts at zero."""
    T, H, d = q.shape
    S = torch.zeros(H, d, v.shape[-1], dtype=F64)
    out = torch.zeros_like(v)
    for t in range(T):
        S = S * decay[t].view(H, 1, 1)
        read = torch.einsum("hdv,hd->hv", S, k[t])
        u = beta[t].view(H, 1) * (v[t] - read)
        S = S + torch.einsum("hd,hv->hdv", k[t], u)
        out[t] = torch.einsum("hdv,hd->hv", S, q[t])
    return out


def delta_mixer(h: torch.Tensor, w: dict, prefix: str, m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(short_convolution(h @ w[f"{prefix}.q"].T, w[f"{prefix}.q.conv"])).view(T, G, d)
    k = silu(short_convolution(h @ w[f"{prefix}.k"].T, w[f"{prefix}.k.conv"])).view(T, G, d)
    v = silu(short_convolution(h @ w[f"{prefix}.v"].T, w[f"{prefix}.v.conv"])).view(T, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * d ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    per = H // G
    q, k = q.repeat_interleave(per, dim=1), k.repeat_interleave(per, dim=1)
    beta = torch.sigmoid(h @ w[f"{prefix}.b"].T)
    step = torch.nn.functional.softplus(h @ w[f"{prefix}.a"].T + w[f"{prefix}.dt_bias"])
    decay = torch.exp(-torch.exp(w[f"{prefix}.A_log"]) * step)
    o = delta_rule(q, k, v, beta, decay)
    o = rms_unit(o, eps) * w[f"{prefix}.norm"]
    o = o.reshape(T, H * dv) * silu(h @ w[f"{prefix}.g"].T)
    return o @ w[f"{prefix}.o"].T


def route(h: torch.Tensor, w: dict, prefix: str, top: int):
    """(ids [T, top], weights [T, top], margin [T]): the ``top`` largest logits z = Wr h + b, their softmax
    among themselves, and how far the last taken logit lies above the first one left out."""
    z = h @ w[f"{prefix}.router"].T + w[f"{prefix}.router.b"]
    ordered, ids = torch.sort(z, dim=-1, descending=True, stable=True)
    margin = ordered[:, top - 1] - ordered[:, top] if z.shape[1] > top else torch.full((h.shape[0],), math.inf, dtype=F64)
    chosen = ordered[:, :top]
    e = torch.exp(chosen - chosen[:, :1])
    return ids[:, :top], e / e.sum(-1, keepdim=True), margin


def routed_feed_forward(h: torch.Tensor, w: dict, prefix: str, mlp: dict, margins: list | None = None) -> torch.Tensor:
    ids, weights, margin = route(h, w, prefix, int(mlp["router"]["top"]))
    if margins is not None:
        margins.append(margin)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, weight in zip(ids[t].tolist(), weights[t]):
            x = h[t]
            y = silu(w[f"{prefix}.e{e}.gate"] @ x) * (w[f"{prefix}.e{e}.up"] @ x)
            out[t] += weight * (w[f"{prefix}.e{e}.down"] @ y)
    return out


MIXERS = {"attention": pooled_attention, "attention_2": mixed_heads_attention, "delta": delta_mixer}


def forward(config: dict, weights: dict, tokens: list[int], layers_out: list | None = None,
            margins: list | None = None) -> torch.Tensor:
    """Logits [T, vocab] of one sequence.  ``layers_out`` collects the stream after every layer run,
    ``margins`` every routed layer's per-token margin of its choice."""
    w = {name: t.to(F64) for name, t in weights.items()}
    eps, mult = float(config["norm"]["eps"]), float(config["residual_mult"])
    x = w["embed"][torch.tensor(tokens, dtype=torch.long)]
    for index, layer in enumerate(config["layers"]):
        source = layer.get("weights_of", index)
        prefix = f"l{source}"
        mixed = MIXERS[layer["type"]](x, w, f"{prefix}.mix", layer["mixer"], eps)
        x = x + mult * rms_norm(mixed, w[f"{prefix}.norm1"], eps)
        if layer.get("mlp") is not None:
            y = routed_feed_forward(x, w, f"{prefix}.mlp", layer["mlp"], margins)
            x = x + mult * rms_norm(y, w[f"{prefix}.norm2"], eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    return rms_norm(x, w["final.norm"], eps) @ w["embed"].T
