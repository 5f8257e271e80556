"""The kernels of Rizovik's mechanisms alone, each against a plain float64 restatement (tests/plain_rizovik.py),
with inputs made so that a fault shows: queries that point at ONE key each (just inside a window and just
outside it, the last kept token and the first one that is not kept, a block of pooled keys that has just come
into sight and one that has not yet, keys hundreds of positions back), over pages out of order, as a portion of
a prompt and decoded alone; the delta rule in portions of every size over slots that are used again; routing
with ties and a bias that decides; the sum of a normed output into the stream."""

import math

import pytest
import torch

from plain_rizovik import (F64, delta_rule, kept_window_mask, pooled_window_mask, rms_norm, rms_unit, rotate_halves, route,
                           softmax_over)

pytestmark = pytest.mark.gpu

DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def _i32(values, device):
    return torch.tensor(list(values), dtype=torch.int32, device=device)


def _attention_case(seed, T, H, G, d, dv, targets, sharp=24.0):
    """Projections q [T, H, d], k [T, G, d], v [T, G, dv] of unit-size values in which query head 0 at position
    p points at key ``targets[p]`` of its key/value head with a score of about ``sharp`` before scaling."""
    g = torch.Generator().manual_seed(seed)
    q, k, v = torch.randn(T, H, d, generator=g), torch.randn(T, G, d, generator=g), torch.randn(T, G, dv, generator=g)
    for p, target in targets.items():
        q[p, 0] = k[target, 0] * (sharp / float(k[target, 0].pow(2).sum()))
    return q, k, v


def _run_attention(cuda_device, dtype, q, k, v, H, G, page, portions, *, window, pool=0, keep_first=0, mix=None,
                   norm="none", q_w=None, k_w=None, rot=None, value_norm=False, scale=1.0, eps=1e-6, fast=False):
    """The engine's kernels on one request cut into ``portions``: projection -> norms, rotation, cache write ->
    pooling of the blocks that became whole -> the general attention kernel, or with ``fast`` the tensor-core
    prompt kernel, single tokens included (-> the mixing of heads)."""
    from zephyr_b200.kernels import ops

    torch_dtype = DTYPES[dtype]
    T, d, dv = q.shape[0], q.shape[2], v.shape[2]
    g = torch.Generator().manual_seed(T + page)
    blocks = -(-T // page)
    table = (torch.randperm(blocks, generator=g) + 1).to(torch.int32).view(1, -1).to(cuda_device)
    cache = torch.full((blocks + 1, page * G * (d + dv)), float("nan"), dtype=torch_dtype, device=cuda_device)
    if d == dv:
        cache = cache.view(blocks + 1, 2, G, page, d)
    pool_blocks = -(-(T // max(pool, 1) + 1) // page)
    pool_table = (torch.randperm(pool_blocks, generator=g) + 1).to(torch.int32).view(1, -1).to(cuda_device)
    pool_cache = torch.full((pool_blocks + 1, *cache.shape[1:]), float("nan"), dtype=torch_dtype, device=cuda_device)
    status = ops.new_status(cuda_device)
    tile = ops.attention_tile_tokens(H // G)
    projected = torch.cat([q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1)], dim=1).float().to(cuda_device)
    freqs, dims = (None, 0)
    if rot is not None:
        from plain_rizovik import rotation_frequencies
        freqs, dims = rotation_frequencies(rot).float().to(cuda_device), rot["dims"]
    outs, at = [], 0
    for n in portions:
        pos = torch.arange(at, at + n, dtype=torch.int32, device=cuda_device)
        rows = (_i32([0], cuda_device), _i32([n], cuda_device), _i32([at], cuda_device))
        zeros = torch.zeros(n, dtype=torch.int32, device=cuda_device)
        qs = ops.qkv_halves(projected[at:at + n], H, G, d, dv, norm, q_w.to(cuda_device) if q_w is not None else None,
                            k_w.to(cuda_device) if k_w is not None else None, eps, freqs, dims, 1.0, value_norm, pos, zeros,
                            cache, table, status, torch_dtype)
        extra = {}
        if pool:
            ops.pool_blocks(cache, table, pool_cache, pool_table, pos, zeros, G, d, dv, pool, status)
            extra = dict(pool=pool, pool_cache=pool_cache, pool_table=pool_table)
        tile_q0 = torch.arange(0, n, tile, dtype=torch.int32, device=cuda_device)
        args = (qs, cache, table, torch.zeros_like(tile_q0), tile_q0, tile, *rows, H, G, d, window, scale, status)
        if fast:
            wide_q0 = torch.arange(0, n, ops.paged_prefill_tile_tokens(), dtype=torch.int32, device=cuda_device)
            out = torch.full((n, H * dv * (G if mix is not None else 1)), float("nan"), device=cuda_device,
                             dtype=torch.float32 if mix is not None else torch_dtype)
            # (a single token's query rows are the heads of a group, where a group has at most 16)
            ops.paged_prefill(qs, cache, table, torch.zeros_like(wide_q0), wide_q0, *rows, H, G, d, window, scale, status, out,
                              keep_first=keep_first, cross_values=mix is not None, by_group=n == 1 and H // G <= 16, **extra)
            outs.append(ops.head_mix(out, mix.float().to(cuda_device), H, G, dv, torch_dtype) if mix is not None else out)
        elif mix is not None:
            crossed = ops.paged_attention(*args, value_dim=dv, keep_first=keep_first, cross_values=True,
                                          out_dtype=torch.float32, **extra)
            outs.append(ops.head_mix(crossed, mix.float().to(cuda_device), H, G, dv, torch_dtype))
        else:
            outs.append(ops.paged_attention(*args, value_dim=dv, keep_first=keep_first, **extra))
        at += n
    ops.check_status(status)
    return torch.cat(outs).cpu().double()


def _prompt_kernel_takes(H, G, d, dv, dtype):
    from zephyr_b200.kernels import ops

    return d == dv and ops.paged_prefill_supported(H, G, d, DTYPES[dtype])


def _expected_attention(dtype, q, k, v, H, G, visible_tokens, visible_blocks=None, pool=0, mix=None, scale=1.0):
    """float64, from keys and values as the cache holds them (rounded to the engine's type)."""
    T, d, dv = q.shape[0], q.shape[2], v.shape[2]
    held = lambda t: t.to(DTYPES[dtype]).double()
    q, k, v = held(q), held(k), held(v)
    keys, values, visible = k, v, visible_tokens
    if pool:
        nb = T // pool
        keys = torch.cat([k, held(k[: nb * pool].view(nb, pool, G, d).mean(1))])
        values = torch.cat([v, held(v[: nb * pool].view(nb, pool, G, dv).mean(1))])
        visible = torch.cat([visible_tokens, visible_blocks], dim=1)
    per = H // G
    weights = torch.stack([softmax_over(q[:, h] @ keys[:, h // per].T * scale, visible) for h in range(H)])
    if mix is not None:
        weights = torch.einsum("hg,gij->hij", mix.double(), weights)
    return torch.stack([weights[h] @ values[:, h // per] for h in range(H)], dim=1).reshape(T, H * dv)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,d,dv,size,pool,page", [(4, 2, 32, 32, 44, 12, 16), (3, 1, 24, 40, 19, 5, 16), (8, 1, 64, 16, 12, 12, 32),
                                                    (2, 2, 16, 48, 36, 64, 16), (6, 3, 128, 128, 70, 8, 64), (5, 1, 20, 20, 1, 1, 16),
                                                    (17, 1, 16, 16, 33, 3, 16), (4, 2, 64, 64, 19, 5, 16), (6, 1, 96, 96, 100, 2, 32),
                                                    (2, 1, 256, 256, 64, 64, 16), (34, 2, 32, 32, 21, 3, 16)])
def test_a_window_followed_by_pooled_blocks(cuda_device, dtype, H, G, d, dv, size, pool, page):
    """Queries of head 0 point at the last key inside the window, at the first one outside it (which may be
    seen only through its block's mean, or not at all), at a key of the block that has just come into sight, at
    one of the block that has not yet, and at keys far back."""
    T = 333
    targets = {}
    for p in range(T - 60, T):
        newest = (p - size + 1) // pool - 1                     # the newest block in sight
        choice = [p - size + 1, p - size, newest * pool + pool - 1, (newest + 1) * pool, 3, p][p % 6]
        targets[p] = min(max(choice, 0), p)
    q, k, v = _attention_case(H * 100 + size, T, H, G, d, dv, targets)
    tokens, blocks = pooled_window_mask(T, size, pool)
    expected = _expected_attention(dtype, q, k, v, H, G, tokens, blocks, pool)
    bound = (3e-5 if dtype == "float32" else 0.03) * max(1.0, float(expected.abs().max()))
    for portions in ([T - 40] + [1] * 40, [7, 2, 150, 1, 1, 90, 2] + [1] * 20 + [T - 273]):
        got = _run_attention(cuda_device, dtype, q, k, v, H, G, page, portions, window=size, pool=pool)
        assert torch.isfinite(got).all()
        assert (got - expected).abs().max() < bound, portions[:3]
        if _prompt_kernel_takes(H, G, d, dv, dtype):
            got = _run_attention(cuda_device, dtype, q, k, v, H, G, page, portions, window=size, pool=pool, fast=True)
            assert torch.isfinite(got).all()
            assert (got - expected).abs().max() < bound, ("tensor cores", portions[:3])
    # what is pointed at decides: leaving the blocks out, or seeing a block one token early, would not pass
    no_blocks = _expected_attention(dtype, q, k, v, H, G, tokens, torch.zeros_like(blocks), pool)
    early = _expected_attention(dtype, q, k, v, H, G, tokens, pooled_window_mask(T + 1, size, pool)[1][1:, : T // pool], pool)
    if 1 < pool <= 5:          # (a larger block's mean answers a pointed query only weakly)
        assert (no_blocks - expected).abs().max() > 0.3
        assert (early - expected).abs().max() > 0.3


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,d,dv,size,keep,page", [(4, 2, 32, 32, 90, 22, 16), (6, 3, 20, 12, 23, 7, 16), (2, 2, 48, 48, 9, 0, 16),
                                                    (5, 5, 16, 24, 70, 33, 32), (8, 4, 128, 128, 33, 40, 16), (3, 1, 64, 64, 5, 1, 64),
                                                    (4, 1, 16, 16, 300, 4, 16), (6, 2, 32, 32, 70, 65, 16), (4, 4, 160, 160, 64, 64, 32),
                                                    (17, 1, 64, 64, 30, 9, 16)])
def test_a_window_that_keeps_the_first_tokens_with_mixed_heads(cuda_device, dtype, H, G, d, dv, size, keep, page):
    """Queries of head 0 point at the last kept token, the first one that is not kept, the edges of the window
    and the first token; the heads' weights are mixed by a matrix with entries of both signs, so every head's
    output carries every other head's weights on its OWN key/value head's values."""
    T = 333
    targets = {p: min(max([keep - 1, keep, p - size + 1, p - size, 0, p - 1][p % 6], 0), p) for p in range(T - 60, T)}
    q, k, v = _attention_case(H * 100 + size + keep, T, H, G, d, dv, targets)
    g = torch.Generator().manual_seed(keep)
    mix = torch.eye(H) * 0.7 + torch.randn(H, H, generator=g) * 0.4
    visible = kept_window_mask(T, size, keep)
    expected = _expected_attention(dtype, q, k, v, H, G, visible, mix=mix)
    plain_heads = _expected_attention(dtype, q, k, v, H, G, visible)
    bound = (3e-5 if dtype == "float32" else 0.03) * max(1.0, float(expected.abs().max()))
    for portions in ([T - 40] + [1] * 40, [7, 2, 150, 1, 1, 90, 2] + [1] * 20 + [T - 273]):
        got = _run_attention(cuda_device, dtype, q, k, v, H, G, page, portions, window=size, keep_first=keep, mix=mix)
        assert torch.isfinite(got).all()
        assert (got - expected).abs().max() < bound, portions[:3]
        unmixed = _run_attention(cuda_device, dtype, q, k, v, H, G, page, portions, window=size, keep_first=keep)
        assert (unmixed - plain_heads).abs().max() < bound
        if _prompt_kernel_takes(H, G, d, dv, dtype):
            got = _run_attention(cuda_device, dtype, q, k, v, H, G, page, portions, window=size, keep_first=keep, mix=mix, fast=True)
            assert torch.isfinite(got).all()
            assert (got - expected).abs().max() < bound, ("tensor cores", portions[:3])
            unmixed = _run_attention(cuda_device, dtype, q, k, v, H, G, page, portions, window=size, keep_first=keep, fast=True)
            assert (unmixed - plain_heads).abs().max() < bound
    if keep and size + keep < T - 60:
        assert (_expected_attention(dtype, q, k, v, H, G, kept_window_mask(T, size, keep - 1), mix=mix) - expected).abs().max() > 0.3
        assert (_expected_attention(dtype, q, k, v, H, G, kept_window_mask(T, size, keep + 1), mix=mix) - expected).abs().max() > 0.3


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,d,dv,norm,scales,dims,factor,value_norm", [
    (4, 2, 32, 32, "whole", True, 16, None, True), (3, 1, 24, 40, "per_head", True, 24, 4.0, False),
    (6, 6, 20, 12, "whole", False, 2, None, False), (2, 1, 128, 64, "per_head", False, 64, 16.0, True),
    (5, 1, 16, 16, "none", False, 16, None, True), (8, 2, 64, 64, "whole", True, 0, None, True)])
def test_norms_rotation_of_halves_and_the_cache_write(cuda_device, dtype, H, G, d, dv, norm, scales, dims, factor, value_norm):
    """Queries that come out of the kernel and, through an attention over one key per query (a window of one
    token), the values it wrote; the keys through the scores of a window of two."""
    T, eps = 150, 1e-5
    g = torch.Generator().manual_seed(H * d + dims)
    q, k, v = (torch.randn(T, H, d, generator=g) * 2.0, torch.randn(T, G, d, generator=g) * 0.5, torch.randn(T, G, dv, generator=g) * 3.0)
    size = {"whole": (H * d, G * d), "per_head": (d, d), "none": (0, 0)}[norm]
    q_w = torch.randn(size[0], generator=g) * 0.3 + 1.0 if scales else None
    k_w = torch.randn(size[1], generator=g) * 0.3 + 1.0 if scales else None
    rot = {"base": 300.0, "dims": dims, **({"scaling": {"factor": factor}} if factor else {})} if dims else None
    one = lambda w, n: w.double() if w is not None else torch.ones(n, dtype=F64)
    if norm == "whole":
        qn = (rms_unit(q.double().reshape(T, -1), eps) * one(q_w, H * d)).view(T, H, d)
        kn = (rms_unit(k.double().reshape(T, -1), eps) * one(k_w, G * d)).view(T, G, d)
    elif norm == "per_head":
        qn, kn = rms_unit(q.double(), eps) * one(q_w, d), rms_unit(k.double(), eps) * one(k_w, d)
    else:
        qn, kn = q.double(), k.double()
    positions = torch.arange(T)
    if rot is not None:
        qn, kn = rotate_halves(qn, positions, rot), rotate_halves(kn, positions, rot)
    vn = rms_unit(v.double(), eps) if value_norm else v.double()
    common = dict(norm=norm, q_w=q_w, k_w=k_w, rot=rot, value_norm=value_norm, eps=eps)
    # a window of one token: the output is the value the kernel wrote for the query's own position
    own = _run_attention(cuda_device, dtype, q, k, v, H, G, 16, [100, 1, 1, 48], window=1, **common)
    expected_own = vn.to(DTYPES[dtype]).double().repeat_interleave(H // G, dim=1).reshape(T, H * dv)
    assert (own - expected_own).abs().max() < (1e-5 if dtype == "float32" else 2.0 ** -8) * max(1.0, float(expected_own.abs().max()))
    # a window of two: the weights of the two keys carry q . k of the rotated, normed vectors
    two = _run_attention(cuda_device, dtype, q, k, v, H, G, 16, [100, 1, 1, 48], window=2, scale=0.2, **common)
    expected_two = _expected_attention(dtype, qn.float(), kn.float(), vn.float(), H, G, kept_window_mask(T, 2, 0), scale=0.2)
    assert (two - expected_two).abs().max() < (5e-5 if dtype == "float32" else 0.04) * max(1.0, float(expected_two.abs().max()))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads,groups,dim,vdim", [(2, 1, 32, 48), (4, 2, 24, 20), (3, 1, 96, 70), (6, 3, 128, 32), (2, 2, 16, 128),
                                                   (1, 1, 200, 9), (8, 2, 8, 20), (2, 1, 64, 64), (3, 3, 40, 36)])
def test_the_delta_rule_in_portions_over_slots_used_again(cuda_device, dtype, heads, groups, dim, vdim):
    """Two requests side by side in portions of unequal sizes (down to one and two tokens), then a third in the
    first one's slot, which is zeroed as the engine zeroes it: outputs against the plain recurrence run over
    each request whole."""
    from zephyr_b200.kernels import ops

    torch_dtype = DTYPES[dtype]
    g = torch.Generator().manual_seed(heads * dim + vdim)
    lengths = {"a": 150, "b": 77, "c": 40}
    data = {}
    for name, T in lengths.items():
        q, k, v = (torch.randn(T, groups, dim, generator=g), torch.randn(T, groups, dim, generator=g) * 3.0,
                   torch.randn(T, heads, vdim, generator=g))
        b, a = torch.randn(T, heads, generator=g) * 1.5, torch.randn(T, heads, generator=g) * 2.0
        data[name] = tuple(t.to(torch_dtype) for t in (q, k, v)) + (b, a)
    a_log, dt_bias = torch.randn(heads, generator=g) * 0.5 - 1.0, torch.randn(heads, generator=g) * 0.7

    def plain(name):
        q, k, v, b, a = (t.double() for t in data[name])
        qn = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * dim ** -0.5
        kn = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
        per = heads // groups
        decay = torch.exp(-torch.exp(a_log.double()) * torch.nn.functional.softplus(a + dt_bias.double()))
        return delta_rule(qn.repeat_interleave(per, 1), kn.repeat_interleave(per, 1), v, torch.sigmoid(b), decay).reshape(len(q), -1)

    state = torch.full((3, heads * dim * vdim + 5), float("nan"), dtype=torch.float32, device=cuda_device)[:, :heads * dim * vdim]
    status = ops.new_status(cuda_device)
    got = {name: [] for name in lengths}

    def step(entries):
        """entries: (name, slot, first, count) rows of one batch."""
        parts = [[data[name][i][first:first + count] for name, _, first, count in entries] for i in range(5)]
        q, k, v, b, a = (torch.cat(p).to(cuda_device) for p in parts)
        T = q.shape[0]
        ba = torch.cat([b, a], dim=1).contiguous()
        counts = [count for *_, count in entries]
        starts = [sum(counts[:i]) for i in range(len(counts))]
        out = ops.delta_rule(q.view(T, -1), k.view(T, -1), v.view(T, -1), ba[:, :heads], ba[:, heads:], a_log.to(cuda_device),
                             dt_bias.to(cuda_device), heads, groups, dim, vdim, state, _i32([slot for _, slot, _, _ in entries], cuda_device),
                             _i32(starts, cuda_device), _i32(counts, cuda_device), status, q_scale=dim ** -0.5)
        for (name, *_), start, count in zip(entries, starts, counts):
            got[name].append(out[start:start + count].cpu().double())

    state[0].zero_(); state[2].zero_()
    cuts_a, cuts_b = [33, 1, 1, 2, 60, 7, 46], [2, 20, 1, 17, 1, 30, 6]
    at_a = at_b = 0
    for ca, cb in zip(cuts_a, cuts_b):
        step([("a", 2, at_a, ca), ("b", 0, at_b, cb)])
        at_a, at_b = at_a + ca, at_b + cb
    state[2].zero_()                       # request c takes a's slot
    step([("c", 2, 0, 39)])
    step([("c", 2, 39, 1)])
    ops.check_status(status)
    for name in lengths:
        expected, out = plain(name), torch.cat(got[name])
        assert torch.isfinite(out).all()
        assert (out - expected).abs().max() < 2e-5 * max(1.0, float(expected.abs().max())), name


@pytest.mark.parametrize("experts,top", [(12, 2), (5, 1), (4, 4), (17, 6), (200, 8), (1, 1), (33, 3)])
def test_routing_by_the_largest_biased_logits(cuda_device, experts, top):
    """The ``top`` largest of logits + bias, weighted by the softmax over the taken ones only; a bias that decides
    the choice for one token, and equal logits, which go to the lower index."""
    from zephyr_b200.kernels import ops

    g = torch.Generator().manual_seed(experts * 10 + top)
    tokens = 257
    z = torch.randn(tokens, experts, generator=g) * 2.0
    bias = torch.randn(experts, generator=g)
    if experts > top:
        z[0] = 0.0
        bias[experts - 1] = 10.0           # without the bias the last output would not be taken for token 0
    w = {"r.router": torch.eye(experts, dtype=F64), "r.router.b": bias.double()}
    ids, weights, margin = route(z.double(), w, "r", top)
    got_ids, got_weights = ops.route(z.to(cuda_device), None, top, "top_softmax", logit_bias=bias.to(cuda_device))
    sure = margin > 1e-5
    sure[0] = False
    assert int(sure.sum()) > tokens // 2
    assert torch.equal(got_ids.cpu().long()[sure], ids[sure])
    assert (got_weights.cpu().double()[sure] - weights[sure]).abs().max() < 1e-6
    assert (got_weights.cpu().double().sum(-1) - 1.0).abs().max() < 1e-6
    if experts > top:
        assert int(got_ids[0, 0]) == experts - 1
        if top > 1:                        # the other logits of token 0 tie but for their biases
            order = torch.sort(bias[:-1], descending=True, stable=True).indices[: top - 1]
            assert got_ids[0, 1:].cpu().tolist() == order.tolist()
    same = torch.zeros(3, experts)
    tied, _ = ops.route(same.to(cuda_device), None, top, "top_softmax")
    assert tied.cpu().tolist() == [list(range(top))] * 3


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("width", [48, 257, 1024, 5000])
def test_the_sum_of_a_normed_output_into_the_stream(cuda_device, dtype, width):
    """stream += m * rmsnorm(delta) w, alone, with the sum rounded for the part that reads it next, and with
    the next norm in the same pass."""
    from zephyr_b200.kernels import ops

    g = torch.Generator().manual_seed(width)
    rows, mult, eps = 37, 0.6, 1e-5
    stream = torch.randn(rows, width, generator=g) * 3.0
    delta_rows = (torch.randn(rows, width, generator=g) * 0.01).to(DTYPES[dtype])
    w1, w2 = torch.randn(width, generator=g) * 0.2 + 1.0, torch.randn(width, generator=g) * 0.2 + 1.0
    total = stream.double() + mult * rms_norm(delta_rows.double(), w1.double(), eps)
    bound = 1e-5 if dtype == "float32" else 2.0 ** -8
    for form in ("alone", "rounded", "then"):
        residual = stream.clone().to(cuda_device)
        out = ops.residual_rms_norm(residual, delta_rows.to(cuda_device), w1.to(cuda_device), eps, mult,
                                    w2.to(cuda_device) if form == "then" else None, eps, rounded_sum=form == "rounded")
        assert (residual.cpu().double() - total).abs().max() < 1e-5 * float(total.abs().max())
        if form == "alone":
            assert out is None
        elif form == "rounded":
            assert out.dtype == DTYPES[dtype] and (out.cpu().double() - total).abs().max() < bound * float(total.abs().max())
        else:
            expected = rms_norm(total, w2.double(), eps)
            assert (out.cpu().double() - expected).abs().max() < bound * max(1.0, float(expected.abs().max()))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_sigmoid_gate_value_by_value(cuda_device, dtype):
    from zephyr_b200.kernels import ops

    g = torch.Generator().manual_seed(3)
    x = torch.randn(70, 200, generator=g).to(DTYPES[dtype])
    wide = torch.randn(70, 333, generator=g) * 3.0
    got = ops.sigmoid_gate(x.clone().to(cuda_device), wide.to(cuda_device)[:, 100:300])
    expected = x.double() * torch.sigmoid(wide[:, 100:300].double())
    assert (got.cpu().double() - expected).abs().max() < (1e-6 if dtype == "float32" else 2.0 ** -8) * float(expected.abs().max())
