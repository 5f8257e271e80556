"""Times one kernel of this package alone, on synthetic inputs, and prints what it achieves.

    python -m zephyr_b200.kernels.timing decode_attention --batch 8 --context 4096
    python -m zephyr_b200.kernels.timing prefill_attention --tokens 2048
    python -m zephyr_b200.kernels.timing gemm_small --rows 8 --n 6144 --k 1024 [--swiglu]
    python -m zephyr_b200.kernels.timing fused_chain --rows 8 --hidden 1024 --ffn 3072
    python -m zephyr_b200.kernels.timing sample --rows 8 --vocab 151936
    python -m zephyr_b200.kernels.timing products --tokens 2048 --hidden 1024 --ffn 3072
    python -m zephyr_b200.kernels.timing gemm_tc --tokens 2048 --n 6144 --k 1024 [--swiglu] [--library]
    python -m zephyr_b200.kernels.timing state_scan --mode gated|state_space --heads 8 --head-dim 128 --value-dim 256 [--tokens 0 --rows 8]
    python -m zephyr_b200.kernels.timing conv_silu --n 2560 [--tokens 0 --rows 8]
    python -m zephyr_b200.kernels.timing norms --hidden 2048 --n 2048
    python -m zephyr_b200.kernels.timing decode_attention --context 1024 --chunk 1024
    python -m zephyr_b200.kernels.timing decode_attention --softcap 30 | --keys-only --kv-heads 1
    python -m zephyr_b200.kernels.timing experts --tokens 2048 --hidden 2048 --ffn 1536 --experts 16 --top 4
    python -m zephyr_b200.kernels.timing head_linear --tokens 2048 --heads 16 --n 128 --k 128
    python -m zephyr_b200.kernels.timing stream_parts --tokens 2048 --hidden 2048 --ffn 6144

Each case rotates over several copies of its large operands, together larger than the L2 cache, so
that a kernel bound by memory is timed against memory and not against L2.  Time is taken with CUDA
events around a CUDA graph of ``--iters`` launches, after ``--warmup`` plain launches.  The line printed is JSON: the
kernel, its sizes, microseconds per launch, and GB/s over the bytes the kernel has to read, or
TFLOP/s over the products it has to form.  This is also the small program that a profiler is
pointed at when one kernel is to be looked at by itself.
"""
from __future__ import annotations

import argparse
import json
import math
import sys

import torch

from . import ops

L2_BYTES = 126 << 20


def _time(run, warmup: int, iters: int) -> float:
    """Microseconds per call of ``run(i)``.  The timed calls are captured in one CUDA graph, so that
    a kernel of a few microseconds is not timed against the host's launch rate."""
    for i in range(warmup):
        run(i)
    torch.cuda.synchronize()
    stream = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(stream):
        with ops.capture(graph, stream=stream):
            for i in range(iters):
                run(warmup + i)
        graph.replay()
        torch.cuda.synchronize()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record(stream)
        graph.replay()
        end.record(stream)
        torch.cuda.synchronize()
    return begin.elapsed_time(end) / iters * 1e3


RESIDENT = False      # --resident: one copy of every operand, so that a small one stays in L2


def _copies(bytes_each: int) -> int:
    if RESIDENT:
        return 1
    return max(2, min(16, math.ceil(2 * L2_BYTES / max(bytes_each, 1))))


SEQUENTIAL_PAGES = False      # --sequential-pages: a request's pages lie behind one another in the pool


def _paged_inputs(batch: int, context: int, nkv: int, hd: int, page: int, device, keys_only: bool = False):
    pages_per = math.ceil(context / page)
    num_pages = batch * pages_per + 1
    shape = (num_pages, nkv * page * hd) if keys_only else (num_pages, 2, nkv, page, hd)
    cache_bytes = num_pages * (1 if keys_only else 2) * nkv * page * hd * 2
    caches = [torch.randn(shape, device=device, dtype=torch.bfloat16) for _ in range(_copies(cache_bytes))]
    order = torch.arange(num_pages - 1, device=device) if SEQUENTIAL_PAGES else torch.randperm(num_pages - 1, device=device)
    table = (order[: batch * pages_per] + 1).int().view(batch, pages_per)
    return caches, table.contiguous()


def decode_attention(args) -> dict:
    device = torch.device("cuda")
    nh, nkv, hd, B, ctx = args.heads, args.kv_heads, args.head_dim, args.batch, args.context
    caches, table = _paged_inputs(B, ctx, nkv, hd, args.page_size, device, args.keys_only)
    q = torch.randn((B, nh * hd), device=device, dtype=torch.bfloat16)
    rows = torch.arange(B, dtype=torch.int32, device=device)
    row_ctx = torch.full((B,), ctx - 1, dtype=torch.int32, device=device)
    status, out = ops.new_status(device), torch.empty_like(q)
    split = args.split or None
    chunk = getattr(args, "chunk", 0)
    masks = dict(chunk=chunk, sinks=torch.zeros(nh, device=device)) if chunk else {}
    masks.update(softcap=args.softcap, keys_only=args.keys_only)

    def run(i):
        ops.paged_decode(q, caches[i % len(caches)], table, rows, rows, row_ctx, ctx, nh, nkv, hd, args.window,
                         1 / math.sqrt(hd), status, out=out, split_size=split, **masks)
    us = _time(run, args.warmup, args.iters)
    trace = torch.zeros((1024, 8), dtype=torch.int32, device=device)
    ops.paged_decode_trace(trace)
    for i in range(3):          # the last launch's timeline stays
        run(i)
    ops.paged_decode_trace(None)
    ops.check_status(status, "decode_attention")
    live = min(ctx, args.window) if args.window else ctx
    if chunk:
        live = min(live, (ctx - 1) % chunk + 1)
    read = B * live * nkv * hd * 2 * (1 if args.keys_only else 2)
    return {"kernel": "paged_decode_kernel", "softcap": args.softcap, "keys_only": args.keys_only, "batch": B, "context": ctx, "heads": nh, "kv_heads": nkv, "head_dim": hd,
            "page_size": args.page_size, "window": args.window, "chunk": chunk, "split_size": split or "balanced", "us": round(us, 2),
            "bytes_read": read, "gbs": round(read / us / 1e3, 1), "timeline_ns": _decode_timeline(trace)}


def _decode_timeline(trace: torch.Tensor) -> dict:
    """The last launch over all its CTAs: when the first and the last CTA reached each mark,
    nanoseconds from the earliest start; and the fewest and most items and tiles of a CTA."""
    t = trace.cpu().to(torch.int64)
    t = t[t[:, 4] != 0]
    if t.shape[0] == 0:
        return {}
    marks = ("start", "earlier_kernels_done", "first_tile_landed", "last_tile_done", "end")
    rel = (t[:, :5] - t[:, 0].min()) & 0xFFFFFFFF
    out = {m: [int(rel[:, i].min()), int(rel[:, i].max())] for i, m in enumerate(marks)}
    counted = t[t[:, 7] != 0]
    if counted.shape[0]:
        arrival = (counted[:, 7] - t[:, 0].min()) & 0xFFFFFFFF
        out["last_arrival_counted"] = [int(arrival.min()), int(arrival.max())]
    out.update(ctas=int(t.shape[0]), items=[int(t[:, 5].min()), int(t[:, 5].max())],
               tiles=[int(t[:, 6].min()), int(t[:, 6].max())])
    return out


def prefill_attention(args) -> dict:
    device = torch.device("cuda")
    nh, nkv, hd, T = args.heads, args.kv_heads, args.head_dim, args.tokens
    caches, table = _paged_inputs(1, T, nkv, hd, args.page_size, device, args.keys_only)
    q = torch.randn((T, nh * hd), device=device, dtype=torch.bfloat16)
    tile = ops.paged_prefill_tile_tokens()
    n_tiles = math.ceil(T / tile)
    tile_row = torch.zeros(n_tiles, dtype=torch.int32, device=device)
    tile_q0 = (torch.arange(n_tiles, dtype=torch.int32, device=device) * tile).contiguous()
    zero = torch.zeros(1, dtype=torch.int32, device=device)
    q_len = torch.full((1,), T, dtype=torch.int32, device=device)
    status, out = ops.new_status(device), torch.empty_like(q)
    chunk = getattr(args, "chunk", 0)
    masks = dict(chunk=chunk, sinks=torch.zeros(nh, device=device)) if chunk else {}
    masks.update(softcap=args.softcap, keys_only=args.keys_only)

    def run(i):
        ops.paged_prefill(q, caches[i % len(caches)], table, tile_row, tile_q0, zero, q_len, zero, nh, nkv, hd,
                          args.window, 1 / math.sqrt(hd), status, out=out, **masks)
    us = _time(run, args.warmup, args.iters)
    trace = torch.zeros((2, 64, 4), dtype=torch.int32, device=device)
    ops.paged_prefill_trace(trace)
    for i in range(2):
        run(i)
    ops.paged_prefill_trace(None)
    ops.check_status(status, "prefill_attention")
    # Two products of 2 * hd flops per (query, visible key) pair and head.
    pairs = sum(min(t + 1, args.window) if args.window else (t % chunk + 1 if chunk else t + 1) for t in range(T))
    flops = 4 * hd * pairs * nh
    return {"kernel": "paged_prefill_kernel", "chunk": chunk, "softcap": args.softcap, "keys_only": args.keys_only, "tokens": T, "heads": nh, "kv_heads": nkv, "head_dim": hd,
            "page_size": args.page_size, "window": args.window, "us": round(us, 2), "flops": flops,
            "tflops": round(flops / us / 1e6, 1), "longest_cta_ns": _prefill_timeline(trace)}


def _prefill_timeline(trace: torch.Tensor) -> list:
    """The launch's longest CTA, tile by tile: [S issued, softmax began, probabilities written,
    O += P V issued, keys asked for, values asked for], ns from the first mark.  Empty if the kernel
    that ran keeps no timeline."""
    t = trace.cpu().to(torch.int64)
    n = int((t[0, :, 3] != 0).sum())
    if n == 0:
        return []
    base = min(int(t[0, 0, 0]), int(t[1, 0, 0]))
    both = torch.cat([t[0, :n], t[1, :n, :2]], dim=1)
    return ((both - base) & 0xFFFFFFFF).tolist()


def gemm_small(args) -> dict:
    device = torch.device("cuda")
    M, N, K = args.rows, args.n, args.k
    weights = [torch.randn((N, K), device=device, dtype=torch.bfloat16) for _ in range(_copies(N * K * 2))]
    x = torch.randn((M, K), device=device, dtype=torch.bfloat16)
    out_dtype = torch.float32 if args.float_out else torch.bfloat16

    def run(i):
        ops.gemm_small(x, weights[i % len(weights)], out_dtype=out_dtype, swiglu=args.swiglu)
    us = _time(run, args.warmup, args.iters)
    read = N * K * 2
    return {"kernel": "gemm_small_kernel", "rows": M, "n": N, "k": K, "swiglu": bool(args.swiglu),
            "out": str(out_dtype).replace("torch.", ""), "us": round(us, 2), "bytes_read": read,
            "gbs": round(read / us / 1e3, 1)}


def sample(args) -> dict:
    device = torch.device("cuda")
    R, V = args.rows, args.vocab
    logits = [torch.randn((R, V), device=device, dtype=torch.float32) * args.logit_scale for _ in range(_copies(R * V * 4))]
    rows = None
    if args.temperature >= 1e-7 or args.top_logprobs >= 0:
        rows = [ops.SampleRow(temperature=args.temperature, uniform=0.1 + 0.8 * r / R, top_k=args.top_k,
                              top_p=args.top_p, min_p=args.min_p, num_logprobs=args.top_logprobs) for r in range(R)]
    status = ops.new_status(device)

    def run(i):
        ops.sample_rows(logits[i % len(logits)], rows, status)
    us = _time(run, args.warmup, args.iters)
    ops.check_status(status, "sample")
    state = ops.last_sample_job_state()
    return {"kernel": "sample kernels", "rows": R, "vocab": V, "temperature": args.temperature, "top_k": args.top_k,
            "top_p": args.top_p, "min_p": args.min_p, "top_logprobs": args.top_logprobs, "logit_scale": args.logit_scale,
            "rankings": len(state), "rankings_decided_in_the_head": sum(done for _, done in state), "us": round(us, 2)}


def _chain_timeline(trace: torch.Tensor) -> dict:
    """The last launch's stages over all CTAs: when the first and the last CTA reached each mark
    (start, input in place, products done, barrier passed), nanoseconds from the earliest start."""
    t = trace.cpu().to(torch.int64)
    t = (t - t[:, 0, 0].min()) & 0xFFFFFFFF
    marks = ("start", "input", "products", "barrier")
    return {f"stage{s}": {m: [int(t[:, s, i].min()), int(t[:, s, i].max())] for i, m in enumerate(marks)}
            for s in range(t.shape[1])}


def fused_chain(args) -> dict:
    """A layer's tail as one chain: output projection, add + norm + gate/up + silu * up, down
    projection, add + norm + the next layer's input projection."""
    device = torch.device("cuda")
    M, d, q, ffn, qkv = args.rows, args.hidden, args.heads * args.head_dim, args.ffn, (args.heads + 2 * args.kv_heads) * args.head_dim
    layer_bytes = 2 * (d * q + 2 * ffn * d + d * ffn + qkv * d)
    rnd = lambda *shape: torch.randn(shape, device=device, dtype=torch.bfloat16) * 0.05
    layers = [(rnd(d, q), rnd(2 * ffn, d), rnd(d, ffn), rnd(qkv, d)) for _ in range(_copies(layer_bytes))]
    norm = torch.ones(d, device=device, dtype=torch.bfloat16)
    attn, residual = rnd(M, q), rnd(M, d)
    buf = lambda n: torch.empty((M, n), device=device, dtype=torch.bfloat16)
    o, act, down, out, r1, r2 = buf(d), buf(ffn), buf(d), buf(qkv), buf(d), buf(d)
    status = ops.new_status(device)
    trace = torch.zeros((ops.fused_chain_grid(), 4, 4), dtype=torch.int32, device=device)

    def stages(i):
        w_o, w_gu, w_down, w_qkv = layers[i % len(layers)]
        return [ops.ChainStage(w=w_o, y=o, x=attn),
                ops.ChainStage(w=w_gu, y=act, residual_in=residual, residual_out=r1, delta=o, norm_w=norm, eps=1e-6, swiglu=True),
                ops.ChainStage(w=w_down, y=down, x=act),
                ops.ChainStage(w=w_qkv, y=out, residual_in=r1, residual_out=r2, delta=down, norm_w=norm, eps=1e-6)]

    whole = all(ops.fused_chain_stage_supported(M, st.w, st.norm_w is not None, st.swiglu) for st in stages(0))
    if whole:
        def run(i):
            ops.fused_chain(stages(i), M, status, trace=trace)
    else:
        # A stage whose input does not fit in shared memory (the down projection of a wide model) runs as
        # kernels of its own between two shorter chains, as in a model's step.
        from ..parts.fused import run_stages

        def run(i):
            run_stages(stages(i), M, status)
    us = _time(run, args.warmup, args.iters)
    ops.check_status(status, "fused_chain")
    return {"kernel": "fused_chain_kernel" if whole else "fused_chain_kernel + gemm_small_kernel", "rows": M, "hidden": d,
            "q": q, "ffn": ffn, "qkv": qkv, "us": round(us, 2), "bytes_read": layer_bytes,
            "gbs": round(layer_bytes / us / 1e3, 1), "timeline_ns": _chain_timeline(trace) if whole else {}}


def products(args) -> dict:
    """A layer's four matrix products for a prompt portion of ``--tokens`` tokens, as the engine runs
    them: the vendor library's tensor-core product for bfloat16 beyond 16 rows, and for gate/up, from
    ``ops.GEMM_TC_MIN_ROWS`` rows on, this package's tcgen05 product with the activation in its epilogue."""
    device = torch.device("cuda")
    T, d, q, ffn, qkv = args.tokens, args.hidden, args.heads * args.head_dim, args.ffn, (args.heads + 2 * args.kv_heads) * args.head_dim
    layer_bytes = 2 * (d * q + 2 * ffn * d + d * ffn + qkv * d)
    rnd = lambda *shape: torch.randn(shape, device=device, dtype=torch.bfloat16) * 0.05
    layers = [(rnd(qkv, d), rnd(d, q), rnd(2 * ffn, d), rnd(d, ffn)) for _ in range(_copies(layer_bytes))]
    x, attn, act = rnd(T, d), rnd(T, q), rnd(T, ffn)

    def run(i):
        w_qkv, w_o, w_gu, w_down = layers[i % len(layers)]
        ops.linear(x, w_qkv)
        ops.linear(attn, w_o)
        if (T >= ops.GEMM_TC_MIN_ROWS or not ops.USE_LIBRARY_PRODUCTS) and ops.gemm_tc_supported(x, w_gu, swiglu=True):
            ops.gemm_tc(x, w_gu, swiglu=True)
        else:
            ops.silu_mul(ops.linear(x, w_gu), blocked=True)
        ops.linear(act, w_down)
    us = _time(run, args.warmup, args.iters)
    flops = 2.0 * T * (qkv * d + d * q + 2 * ffn * d + d * ffn)
    return {"kernel": "a layer's prompt products (cuBLASLt; gate/up + activation on tcgen05)", "tokens": T, "hidden": d, "q": q, "ffn": ffn, "qkv": qkv,
            "us": round(us, 2), "flops": flops, "tflops": round(flops / us / 1e6, 1)}


def gemm_tc(args) -> dict:
    """One product x [tokens, k] w[n, k]^T on this package's tcgen05 kernel (``--swiglu``: with the
    activation in its epilogue; ``--library``: the vendor library's product, and the activation
    kernel after it, on the same operands)."""
    device = torch.device("cuda")
    T, N, K = args.tokens, args.n, args.k
    rnd = lambda *shape: torch.randn(shape, device=device, dtype=torch.bfloat16) * 0.05
    weights = [rnd(N, K) for _ in range(_copies(2 * N * K))]
    x = rnd(T, K)
    status = torch.zeros(4, dtype=torch.int32, device=device)

    def run(i):
        w = weights[i % len(weights)]
        if args.library:
            y = ops.linear(x, w)
            if args.swiglu:
                ops.silu_mul(y, blocked=True)
        else:
            ops.gemm_tc(x, w, swiglu=args.swiglu, block_n=args.block_n, status=status)
    us = _time(run, args.warmup, args.iters)
    flops = 2.0 * T * N * K
    return {"kernel": "library product" if args.library else "gemm_tc_kernel", "tokens": T, "n": N, "k": K,
            "swiglu": args.swiglu, "block_n": args.block_n, "us": round(us, 2), "flops": flops,
            "tflops": round(flops / us / 1e6, 1), "status": status.tolist()}


CASES = {"gemm_tc": gemm_tc, "fused_chain": fused_chain, "products": products, "decode_attention": decode_attention, "prefill_attention": prefill_attention, "gemm_small": gemm_small,
         "sample": sample}


# ---- the kernels of recurrent layers and of layer norms (csrc/recurrent.cu, csrc/qkv_pairs.cu) ----
def _row_shape(args, device):
    """(tokens, slots, row starts, row lengths): ``--rows`` requests of one token each, or one of ``--tokens``."""
    if args.tokens > 0:
        counts = [args.tokens]
    else:
        counts = [1] * args.rows
    starts = torch.tensor([sum(counts[:i]) for i in range(len(counts))], dtype=torch.int32, device=device)
    return sum(counts), torch.arange(len(counts), dtype=torch.int32, device=device), starts, \
        torch.tensor(counts, dtype=torch.int32, device=device)


def state_scan(args) -> dict:
    """The decayed outer-product recurrence: ``--mode gated|state_space``, ``--heads``, ``--head-dim`` key
    channels, ``--value-dim`` value channels; ``--tokens 0`` decodes ``--rows`` requests by one token."""
    device = torch.device("cuda")
    H, D, V = args.heads, args.head_dim, args.value_dim
    T, slots, starts, lens = _row_shape(args, device)
    R = slots.numel()
    state_bytes = R * H * D * V * 4
    states = [torch.zeros((R, H * D * V), device=device) for _ in range(_copies(state_bytes) if args.tokens == 0 else 1)]
    bf = torch.bfloat16
    status = ops.new_status(device)
    segment = None if args.segment < 0 else args.segment
    if args.mode == "gated":
        q, k, v = (torch.randn((T, H * n), device=device, dtype=bf) for n in (D, D, V))
        z, bias = torch.randn((T, H * D), device=device) + 3.0, torch.zeros(H * D, device=device)

        def run(i):
            ops.decayed_state_scan("gated", q, k, v, H, D, V, states[i % len(states)], slots, starts, lens, status,
                                   decay_logits=z, decay_bias=bias, inv_tau=1 / 16, q_scale=D ** -0.5, segment=segment)
        read = T * (2 * H * D * 2 + H * V * 2 + H * D * 4)
    else:
        G = max(1, args.kv_heads)
        q, k = (torch.randn((T, G * D), device=device, dtype=bf) for _ in range(2))
        v, dt = torch.randn((T, H * V), device=device, dtype=bf), torch.randn((T, H), device=device, dtype=bf)
        consts = [torch.zeros(H, device=device) for _ in range(3)]

        def run(i):
            ops.decayed_state_scan("state_space", q, k, v, H, D, V, states[i % len(states)], slots, starts, lens, status,
                                   dt=dt, dt_bias=consts[0], a_log=consts[1], skip=consts[2], heads_per_group=H // G,
                                   segment=segment)
        read = T * (2 * G * D * 2 + H * V * 2 + H * 2)
    us = _time(run, args.warmup, args.iters)
    ops.check_status(status, "state_scan")
    moved = 2 * state_bytes + read + T * H * V * 4
    flops = 4 * T * H * D * V          # two multiply-adds per state element and token
    return {"kernel": "decayed_state_scan_kernel", "mode": args.mode, "segment": args.segment, "rows": R, "tokens": T, "heads": H, "key_dim": D,
            "value_dim": V, "us": round(us, 2), "bytes": moved, "gbs": round(moved / us / 1e3, 1),
            "tflops_fp32": round(flops / us / 1e6, 2)}


def conv_silu(args) -> dict:
    device = torch.device("cuda")
    C, taps = args.n, 4
    T, slots, starts, lens = _row_shape(args, device)
    xs = [torch.randn((T, C), device=device, dtype=torch.bfloat16) for _ in range(_copies(T * C * 2))]
    w, b = torch.randn((C, taps), device=device), torch.zeros(C, device=device)
    state = torch.zeros((slots.numel(), (taps - 1) * C), device=device)
    status = ops.new_status(device)
    token_row = torch.repeat_interleave(torch.arange(slots.numel(), device=device), lens.long()).int()
    us = _time(lambda i: ops.causal_conv_silu(xs[i % len(xs)], C, w, b, state, slots, starts, lens, token_row, status),
               args.warmup, args.iters)
    moved = T * C * 4 + 2 * state.numel() * 4
    return {"kernel": "causal_conv_silu_kernel", "tokens": T, "rows": slots.numel(), "channels": C, "us": round(us, 2),
            "bytes": moved, "gbs": round(moved / us / 1e3, 1)}


def norms(args) -> dict:
    """The fused residual sum + layer norm + next layer norm beside the other architecture's residual sum +
    RMS norm, the gated group norm, and the two kernels between a q/k/v projection and the attention."""
    device = torch.device("cuda")
    T, H = (args.tokens or args.rows), args.hidden
    bf = torch.bfloat16
    n = _copies(T * H * 12)
    residual32 = [torch.randn((T, H), device=device) for _ in range(n)]
    residual16 = [torch.randn((T, H), device=device, dtype=bf) for _ in range(n)]
    delta = [torch.randn((T, H), device=device, dtype=bf) for _ in range(n)]
    w = [torch.ones(H, device=device) for _ in range(4)]
    out = {"tokens": T, "hidden": H}
    us = _time(lambda i: ops.residual_layer_norm(residual32[i % n], delta[i % n], w[0], w[1], 1e-6, 0.5, w[2], w[3], 1e-6),
               args.warmup, args.iters)
    out["residual_layer_norm"] = {"us": round(us, 2), "gbs": round(T * H * 12 / us / 1e3, 1)}
    # the form of a block that norms its parts' outputs only: one norm without a shift, and the sum rounded for the next part
    us = _time(lambda i: ops.residual_layer_norm(residual32[i % n], delta[i % n], w[0], None, 1e-6, 1.0, rounded_sum=True),
               args.warmup, args.iters)
    out["residual_layer_norm_rounded_sum"] = {"us": round(us, 2), "gbs": round(T * H * 12 / us / 1e3, 1)}
    us = _time(lambda i: ops.add_rmsnorm(residual16[i % n], delta[i % n], w[0], 1e-6), args.warmup, args.iters)
    out["add_rmsnorm"] = {"us": round(us, 2), "gbs": round(T * H * 8 / us / 1e3, 1)}
    W = args.n
    o = [torch.randn((T, W), device=device) for _ in range(_copies(T * W * 8))]
    gate = torch.randn((T, W), device=device, dtype=bf)
    scale = torch.ones(W, device=device)
    us = _time(lambda i: ops.gated_group_rms_norm(o[i % len(o)], gate, scale, W // 2, 1e-6, True), args.warmup, args.iters)
    out["gated_group_rms_norm"] = {"width": W, "us": round(us, 2), "gbs": round(T * W * 8 / us / 1e3, 1)}
    nh, nkv, hd = args.heads, args.kv_heads, args.head_dim
    width = (nh + 2 * nkv) * hd
    pages = math.ceil(T / args.page_size) + 1
    cache = torch.zeros((pages, 2, nkv, args.page_size, hd), device=device, dtype=bf)
    table = torch.arange(1, pages, dtype=torch.int32, device=device).view(1, -1)
    positions = torch.arange(T, dtype=torch.int32, device=device)
    token_row = torch.zeros(T, dtype=torch.int32, device=device)
    status = ops.new_status(device)
    qkv32 = [torch.randn((T, width), device=device) for _ in range(_copies(T * width * 6))]
    qkv16 = [t.to(bf) for t in qkv32]
    ones, freqs = torch.ones(hd, device=device), torch.rand(hd // 2, device=device)
    bias = torch.zeros(width, device=device)
    us = _time(lambda i: ops.qkv_pairs(qkv32[i % len(qkv32)], nh, nkv, hd, hd, bias, ones, ones, 1e-6, freqs, hd, positions,
                                       token_row, cache, table, status, bf), args.warmup, args.iters)
    out["qkv_pairs"] = {"width": width, "us": round(us, 2), "gbs": round(T * width * 6 / us / 1e3, 1)}
    # the same kernel for keys that are the values: unit norms without scales, a multiplier by position, no value columns
    narrow = (nh + nkv) * hd
    us = _time(lambda i: ops.qkv_pairs(qkv32[i % len(qkv32)][:, :narrow], nh, nkv, hd, hd, None, None, None, 1e-6, None, 0,
                                       positions, token_row, cache, table, status, bf, unit_norm=True, values_from_keys=True,
                                       q_temp=(0.2, 128)), args.warmup, args.iters)
    moved = T * (narrow * 4 + (nh + 2 * nkv) * hd * 2)
    out["qkv_pairs_keys_as_values"] = {"width": narrow, "us": round(us, 2), "gbs": round(moved / us / 1e3, 1)}
    cos, sin = torch.ones((T, hd // 2), device=device), torch.zeros((T, hd // 2), device=device)
    ones16 = ones.to(bf)
    us = _time(lambda i: ops.qk_norm_rope_cache(qkv16[i % len(qkv16)], nh, nkv, hd, ones16, ones16, 1e-6, cos, sin, positions,
                                                token_row, cache, table, status), args.warmup, args.iters)
    out["qk_norm_rope_cache"] = {"width": width, "us": round(us, 2), "gbs": round(T * width * 4 / us / 1e3, 1)}
    ops.check_status(status, "norms")
    return out


CASES.update({"state_scan": state_scan, "conv_silu": conv_silu, "norms": norms})


def stream_parts(args) -> dict:
    """The small kernels of a design whose layers run mixer and feed-forward side by side on a float32 stream,
    each beside its like: the sum of two summands + RMS norm beside sum + layer norm with a rounded sum and
    beside the bfloat16 stream's sum + RMS norm; the bounded gate with biases on a float32 product beside
    SiLU * up on a bfloat16 one; the latent's norm + rotation + cache write beside the latent's norm + cache
    write alone; the hashed pair embedding beside the plain float32 one; routing by sigmoid scores limited
    to groups beside softmax routing."""
    device = torch.device("cuda")
    T, H, I = (args.tokens or args.rows), args.hidden, args.ffn
    bf = torch.bfloat16
    out = {"tokens": T, "hidden": H, "ffn": I}
    n = _copies(T * H * 14)
    stream = [torch.randn((T, H), device=device) for _ in range(n)]
    stream16 = [torch.randn((T, H), device=device, dtype=bf) for _ in range(n)]
    a16 = [torch.randn((T, H), device=device, dtype=bf) for _ in range(n)]
    b32 = [torch.randn((T, H), device=device) for _ in range(n)]
    w = torch.ones(H, device=device, dtype=bf)
    w32 = torch.ones(H, device=device)
    us = _time(lambda i: ops.sum_rms_norm(stream[i % n], a16[i % n], a16[(i + 1) % n], w, 1e-6, bf), args.warmup, args.iters)
    out["sum_rms_norm_two_bf16"] = {"us": round(us, 2), "gbs": round(T * H * 14 / us / 1e3, 1)}
    us = _time(lambda i: ops.sum_rms_norm(stream[i % n], a16[i % n], b32[i % n], w, 1e-6, bf), args.warmup, args.iters)
    out["sum_rms_norm_bf16_f32"] = {"us": round(us, 2), "gbs": round(T * H * 16 / us / 1e3, 1)}
    us = _time(lambda i: ops.residual_layer_norm(stream[i % n], a16[i % n], w32, None, 1e-6, 1.0, rounded_sum=True),
               args.warmup, args.iters)
    out["like: residual_layer_norm_rounded_sum"] = {"us": round(us, 2), "gbs": round(T * H * 12 / us / 1e3, 1)}
    us = _time(lambda i: ops.add_rmsnorm(stream16[i % n], a16[i % n], w, 1e-6), args.warmup, args.iters)
    out["like: add_rmsnorm"] = {"us": round(us, 2), "gbs": round(T * H * 8 / us / 1e3, 1)}
    m = _copies(T * I * 10)
    gu32 = [torch.randn((T, 2 * I), device=device) for _ in range(m)]
    gu16 = [torch.randn((T, 2 * I), device=device, dtype=bf) for _ in range(m)]
    bias = torch.zeros(2 * I, device=device)
    us = _time(lambda i: ops.clamped_gate(gu32[i % m], bias, 7.0, 1.702, 1.0, bf, blocked=True), args.warmup, args.iters)
    out["clamped_gate_f32_in"] = {"us": round(us, 2), "gbs": round(T * I * 10 / us / 1e3, 1)}
    us = _time(lambda i: ops.silu_mul(gu16[i % m], blocked=True), args.warmup, args.iters)
    out["like: silu_mul_bf16_in"] = {"us": round(us, 2), "gbs": round(T * I * 6 / us / 1e3, 1)}
    # The same gate where the gate/up product ends: the weight streamer for a step's few rows (bound by the
    # weight's bytes), tcgen05 for a prompt's many (bound by the products), each beside SiLU * up in that place.
    form = ops.BoundedGate(bias, 7.0, 1.702, 1.0)
    c = _copies(2 * I * H * 2)
    packed = [torch.randn((2 * I, H), device=device, dtype=bf) * H ** -0.5 for _ in range(c)]
    few = torch.randn((8, H), device=device, dtype=bf)
    for name, extra in (("bounded", {"bounded": form}), ("like: silu", {})):
        us = _time(lambda i: ops.gemm_small(few, packed[i % c], swiglu=True, **extra), args.warmup, args.iters)
        out[f"gate_up_8_rows, {name}"] = {"us": round(us, 2), "gbs": round(2 * I * H * 2 / us / 1e3, 1)}
    if T >= 128 and ops.gemm_tc_supported(stream16[0], packed[0], swiglu=True):
        for name, extra in (("bounded", {"bounded": form}), ("like: silu", {})):
            us = _time(lambda i: ops.gemm_tc(stream16[i % n], packed[i % c], swiglu=True, **extra), args.warmup, args.iters)
            out[f"gate_up_{T}_rows, {name}"] = {"us": round(us, 2), "tflops": round(2 * T * 2 * I * H / us / 1e6, 1)}
    nh, rank, rot, dim = args.heads, args.head_dim - 32, 32, 128
    width = rank + rot
    pages = math.ceil(T / args.page_size) + 1
    cache = torch.zeros((pages, args.page_size * width), device=device, dtype=bf)
    table = torch.arange(1, pages, dtype=torch.int32, device=device).view(1, -1)
    positions = torch.arange(T, dtype=torch.int32, device=device)
    token_row = torch.zeros(T, dtype=torch.int32, device=device)
    status = ops.new_status(device)
    k = _copies(T * nh * (dim + rot) * 4)
    q = [torch.randn((T, nh * (dim + rot)), device=device) for _ in range(k)]
    kv = torch.randn((T, width), device=device)
    q_out = torch.empty((T, nh * width), device=device, dtype=bf)
    ones, freqs = torch.ones(rank, device=device), torch.rand(rot // 2, device=device)
    us = _time(lambda i: ops.latent_rope(q[i % k], nh, dim + rot, dim, q_out, kv, rank, rot, ones, 1e-6, freqs, 1.2, positions,
                                         token_row, cache, table, status, bf), args.warmup, args.iters)
    moved = T * (nh * rot * 6 + width * 6)
    out["latent_rope"] = {"heads": nh, "rank": rank, "rot": rot, "us": round(us, 2), "gbs": round(moved / us / 1e3, 1)}
    ones_w = torch.ones(width, device=device)
    us = _time(lambda i: ops.qkv_pairs(kv, 0, 1, width, 0, None, None, ones_w, 1e-6, None, 0, positions, token_row, cache, table,
                                       status, bf), args.warmup, args.iters)
    out["like: latent norm + cache write"] = {"us": round(us, 2), "gbs": round(T * width * 6 / us / 1e3, 1)}
    V = 32768
    table_e = torch.randn((V, H), device=device, dtype=bf)
    pairs = torch.randn((65522, H), device=device, dtype=bf)
    ids = torch.randint(0, V, (T,), dtype=torch.int32, device=device)
    one = torch.zeros(1, dtype=torch.int32, device=device)
    rows_len = torch.full((1,), T, dtype=torch.int32, device=device)
    last = torch.zeros(4, dtype=torch.int32, device=device)
    us = _time(lambda i: ops.pair_embedding(table_e, pairs, ids, positions, token_row, one, rows_len, one, last, 36313, 27191, status),
               args.warmup, args.iters)
    out["pair_embedding (two launches)"] = {"us": round(us, 2), "gbs": round(T * H * 8 / us / 1e3, 1)}
    us = _time(lambda i: ops.embedding_f32(table_e, ids, status), args.warmup, args.iters)
    out["like: embedding_f32"] = {"us": round(us, 2), "gbs": round(T * H * 6 / us / 1e3, 1)}
    logits = torch.randn((T, args.experts), device=device)
    us = _time(lambda i: ops.route(logits, None, args.top, "sigmoid", (4, 2, 2), 2.5), args.warmup, args.iters)
    out["route_sigmoid_groups"] = {"experts": args.experts, "top": args.top, "us": round(us, 2)}
    us = _time(lambda i: ops.route(logits, None, args.top), args.warmup, args.iters)
    out["like: route_softmax"] = {"us": round(us, 2)}
    ops.check_status(status, "stream_parts")
    return out


def experts(args) -> dict:
    """A routed feed-forward's products: ``--tokens`` tokens of width ``--hidden``, each taking ``--top`` of
    ``--experts`` experts of inner size ``--ffn`` (uniform random choices), routing excluded.  With few
    tokens the bound is the bytes of the experts that were hit, with many the products."""
    device, bf = torch.device("cuda"), torch.bfloat16
    T, H, F, E, top = args.tokens, args.hidden, args.ffn, args.experts, args.top
    copies = _copies(3 * E * F * H * 2)
    # gate and up rows in alternating blocks of 8, as the routed part keeps them
    gate_up = [torch.randn((E, 2 * F, H), device=device, dtype=bf) * H ** -0.5 for _ in range(copies)]
    down = [torch.randn((E, H, F), device=device, dtype=bf) * F ** -0.5 for _ in range(copies)]
    x = torch.randn((T, H), device=device, dtype=bf)
    ids = torch.stack([torch.randperm(E, device=device)[:top] for _ in range(T)]).int().contiguous()
    weights = torch.rand((T, top), device=device)
    ops.USE_GROUPED_TCGEN05 = not args.legacy_prefill        # --legacy-prefill: the mma.sync tiles whatever the token count
    us = _time(lambda i: ops.routed_experts(x, ids, weights, gate_up[i % copies], None, down[i % copies]),
               args.warmup, args.iters)
    hit = int(torch.unique(ids).numel())
    flops = 2.0 * T * top * 3 * F * H
    read = hit * 3 * F * H * 2
    ops.check_status(ops.device_status(device), "experts")
    return {"kernel": "route_align + expert products + combine", "tokens": T, "hidden": H, "ffn": F, "experts": E, "top": top,
            "experts_hit": hit, "us": round(us, 2), "tflops": round(flops / us / 1e6, 1), "weights_gbs": round(read / us / 1e3, 1)}


def head_linear(args) -> dict:
    """The product per head: ``--tokens`` rows of ``--heads`` heads, [n, k] per head; all of K staged at once
    beside the walk along k in steps; bfloat16 rows, then bfloat16 rows with a float32 gate per output value,
    then float32 rows that are slices of wider heads (queries on their way into a latent space)."""
    device, bf = torch.device("cuda"), torch.bfloat16
    T, heads, N, K = args.tokens, args.heads, args.n, args.k
    copies = _copies(T * heads * (N + K) * 2)
    w = torch.randn((heads, N, K), device=device, dtype=bf)
    flops = 2.0 * T * heads * N * K
    out = {"kernel": "head_linear_whole_k_kernel", "tokens": T, "heads": heads, "n": N, "k": K}

    def both(name, moved, call):
        for label, walk in (("", 0), (", walk", 1), (", 32 rows a CTA", 2), (", 64 rows a CTA", 3)):
            us = _time(lambda i: call(i, walk), args.warmup, args.iters)
            out[name + label] = {"us": round(us, 2), "tflops": round(flops / us / 1e6, 1), "gbs": round(moved / us / 1e3, 1)}

    x = [torch.randn((T, heads * K), device=device, dtype=bf) for _ in range(copies)]
    both("bf16 rows", T * heads * (N + K) * 2 + heads * N * K * 2, lambda i, walk: ops.head_linear(x[i % copies], w, walk=walk))
    gates = [torch.randn((T, heads * N), device=device) for _ in range(copies)]
    both("bf16 rows, a gate per value", T * heads * (N * 6 + K * 2) + heads * N * K * 2,
         lambda i, walk: ops.head_linear(x[i % copies], w, gate=gates[i % copies], walk=walk))
    del x, gates
    wide = K + 32
    xf = [torch.randn((T, heads * wide), device=device) for _ in range(copies)]
    y = torch.empty((T, heads * (N + 32)), device=device, dtype=bf)
    both("float32 rows, slices of wider heads", T * heads * (N * 2 + K * 4) + heads * N * K * 2,
         lambda i, walk: ops.head_linear(xf[i % copies], w, x_head_stride=wide, out=y, out_head_stride=N + 32, walk=walk))
    return out


CASES.update({"experts": experts, "head_linear": head_linear, "stream_parts": stream_parts})


def delta_rule(args) -> dict:
    """The gated delta rule (unit norms, steps and decays, then the scan): one request of ``--tokens`` tokens, or
    ``--rows`` requests of one token each with ``--tokens 0``; ``--heads`` value heads on ``--kv-heads`` q/k heads of
    ``--head-dim`` key channels and ``--value-dim`` value channels."""
    device = torch.device("cuda")
    heads, groups, D, V = args.heads, args.kv_heads, args.head_dim, args.value_dim
    T, slots, starts, lens = _row_shape(args, device)
    n = _copies(T * (2 * groups * D + heads * V) * 4)
    q = [torch.randn((T, groups * D), device=device) for _ in range(n)]
    k = [torch.randn((T, groups * D), device=device) for _ in range(n)]
    v = [torch.randn((T, heads * V), device=device) for _ in range(n)]
    steps = torch.randn((T, 2 * heads), device=device)
    a_log, dt_bias = torch.zeros(heads, device=device) - 1.0, torch.zeros(heads, device=device)
    state = torch.zeros((slots.numel(), heads * D * V), device=device)
    status = ops.new_status(device)
    us = _time(lambda i: ops.delta_rule(q[i % n], k[i % n], v[i % n], steps[:, :heads], steps[:, heads:], a_log, dt_bias, heads,
                                        groups, D, V, state, slots, starts, lens, status, q_scale=D ** -0.5),
               args.warmup, args.iters)
    ops.check_status(status, "delta_rule")
    per_token = 7.0 * heads * D * V          # three sums of D x V multiply-adds and the write, as operations
    return {"tokens": T, "requests": slots.numel(), "heads": heads, "key_channels": D, "value_channels": V, "us": round(us, 2),
            "tflops_f32": round(T * per_token / us / 1e6, 2),
            "state_gbs": round(2 * slots.numel() * heads * D * V * 4 / us / 1e3, 1)}


def windowed_attention(args) -> dict:
    """Attention over a window of ``--window`` (default 1024) with the masks that come in runs of key tiles: pooled
    blocks of 16 positions, 64 kept first tokens, and every head's weights on every key/value head's values; a
    prompt of ``--tokens`` tokens as tiles of tokens, and ``--batch`` single tokens at ``--context`` as tiles of a
    group's heads, on the mma.sync prompt kernel; beside them the window alone."""
    device = torch.device("cuda")
    H, G, d, page = args.heads, args.kv_heads, args.head_dim, args.page_size
    window = args.window or 1024
    status = ops.new_status(device)
    out = {"heads": H, "kv_heads": G, "head_dim": d, "window": window}

    def run(new_tokens: int, before: int, requests: int, pool=0, keep_first=0, cross=False) -> float:
        T = new_tokens * requests
        q = torch.randn((T, H * d), device=device, dtype=torch.bfloat16)
        caches, table = _paged_inputs(requests, before + new_tokens, G, d, page, device)
        pooled = torch.randn_like(caches[0])
        start = torch.arange(0, T, new_tokens, dtype=torch.int32, device=device)
        lens = torch.full((requests,), new_tokens, dtype=torch.int32, device=device)
        ctx = torch.full((requests,), before, dtype=torch.int32, device=device)
        single = new_tokens == 1
        tile = 1 if single else ops.paged_prefill_tile_tokens()
        per = -(-new_tokens // tile)
        tile_row = torch.arange(requests, dtype=torch.int32, device=device).repeat_interleave(per)
        tile_q0 = (torch.arange(per, dtype=torch.int32, device=device) * tile).repeat(requests)
        result = torch.empty((T, H * d * (G if cross else 1)), device=device, dtype=torch.float32 if cross else torch.bfloat16)
        extra = dict(pool=pool, pool_cache=pooled, pool_table=table) if pool else {}
        masked = bool(pool or keep_first or cross)
        return _time(lambda i: ops.paged_prefill(q, caches[i % len(caches)], table, tile_row, tile_q0, start, lens, ctx, H, G, d,
                                                 window, d ** -0.5, status, result, keep_first=keep_first, cross_values=cross,
                                                 by_group=single and masked and H // G <= 16, **extra),
                     args.warmup, args.iters)

    for name, masks in (("window alone", {}), ("blocks of 16", {"pool": 16}), ("64 kept", {"keep_first": 64}),
                        ("64 kept, pairs of heads", {"keep_first": 64, "cross": True})):
        out[name] = {"prompt_us": round(run(args.tokens, 0, 1, **masks), 1),
                     "single_tokens_us": round(run(1, args.context - 1, args.batch, **masks), 1)}
    ops.check_status(status, "windowed_attention")
    return out


def window_parts(args) -> dict:
    """The small kernels around windowed attention, each beside its like where there is one: norms + rotation of
    halves + cache write beside unit norms + cache write with keys as values; the means of blocks; the mixing of
    heads; the sigmoid gate; the sum of an RMS-normed output into a float32 stream beside the layer-norm form;
    routing by the largest biased logits beside softmax routing."""
    device = torch.device("cuda")
    T, W, H, G, d, page = args.tokens, args.hidden, args.heads, args.kv_heads, args.head_dim, args.page_size
    bf = torch.bfloat16
    status = ops.new_status(device)
    out = {"tokens": T, "hidden": W}
    n = _copies(T * W * 12)
    stream = [torch.randn((T, W), device=device) for _ in range(n)]
    delta = [torch.randn((T, W), device=device, dtype=bf) for _ in range(n)]
    w = torch.ones(W, device=device)
    us = _time(lambda i: ops.residual_rms_norm(stream[i % n], delta[i % n], w, 1e-6, 0.5, rounded_sum=True), args.warmup, args.iters)
    out["residual_rms_norm_rounded_sum"] = {"us": round(us, 2), "gbs": round(T * W * 12 / us / 1e3, 1)}
    us = _time(lambda i: ops.residual_layer_norm(stream[i % n], delta[i % n], w, None, 1e-6, 1.0, rounded_sum=True), args.warmup, args.iters)
    out["like: residual_layer_norm_rounded_sum"] = {"us": round(us, 2), "gbs": round(T * W * 12 / us / 1e3, 1)}
    blocks = -(-T // page)
    table = torch.arange(1, blocks + 1, dtype=torch.int32, device=device).view(1, -1)
    cache = torch.zeros((blocks + 1, 2, G, page, d), dtype=bf, device=device)
    pooled = torch.zeros_like(cache)
    positions = torch.arange(T, dtype=torch.int32, device=device)
    rows = torch.zeros(T, dtype=torch.int32, device=device)
    width = (H + 2 * G) * d
    m = _copies(T * width * 4)
    projected = [torch.randn((T, width), device=device) for _ in range(m)]
    q_w, k_w, freqs = torch.ones(H * d, device=device), torch.ones(G * d, device=device), torch.rand(d // 4, device=device)
    us = _time(lambda i: ops.qkv_halves(projected[i % m], H, G, d, d, "whole", q_w, k_w, 1e-6, freqs, d // 2, 1.0, True, positions,
                                        rows, cache, table, status, bf), args.warmup, args.iters)
    out["qkv_halves"] = {"us": round(us, 2), "gbs": round(T * width * 6 / us / 1e3, 1)}
    narrow = (H + G) * d
    us = _time(lambda i: ops.qkv_pairs(projected[i % m][:, :narrow], H, G, d, d, None, None, None, 1e-6, None, 0, positions, rows,
                                       cache, table, status, bf, unit_norm=True, values_from_keys=True, q_temp=(0.2, 128)),
               args.warmup, args.iters)
    out["like: qkv_pairs_keys_as_values"] = {"us": round(us, 2), "gbs": round(T * (narrow * 4 + width * 2) / us / 1e3, 1)}
    us = _time(lambda i: ops.pool_blocks(cache, table, pooled, table, positions, rows, G, d, d, 16, status), args.warmup, args.iters)
    out["pool_blocks_of_16"] = {"us": round(us, 2), "read_mb": round(T * 2 * G * d * 2 / 1e6, 1)}
    crossed = torch.randn((T, H * G * d), device=device)
    mix = torch.randn((H, H), device=device)
    us = _time(lambda i: ops.head_mix(crossed, mix, H, G, d, bf), args.warmup, args.iters)
    out["head_mix"] = {"us": round(us, 2), "gbs": round((crossed.numel() * 4 + T * H * d * 2) / us / 1e3, 1)}
    attended = torch.randn((T, H * d), device=device, dtype=bf)
    gate = torch.randn((T, H * d), device=device)
    us = _time(lambda i: ops.sigmoid_gate(attended, gate), args.warmup, args.iters)
    out["sigmoid_gate"] = {"us": round(us, 2), "gbs": round(T * H * d * 8 / us / 1e3, 1)}
    logits, bias = torch.randn((T, args.experts), device=device), torch.randn(args.experts, device=device)
    us = _time(lambda i: ops.route(logits, None, args.top, "top_softmax", logit_bias=bias), args.warmup, args.iters)
    out["route_top_softmax"] = {"us": round(us, 2)}
    us = _time(lambda i: ops.route(logits, None, args.top, "softmax"), args.warmup, args.iters)
    out["like: route_softmax"] = {"us": round(us, 2)}
    ops.check_status(status, "window_parts")
    return out


CASES.update({"delta_rule": delta_rule, "windowed_attention": windowed_attention, "window_parts": window_parts})


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(prog="python -m zephyr_b200.kernels.timing", description=__doc__.split("\n")[0])
    parser.add_argument("case", choices=sorted(CASES))
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--iters", type=int, default=40)
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--context", type=int, default=4096)
    parser.add_argument("--tokens", type=int, default=2048)
    parser.add_argument("--heads", type=int, default=16)
    parser.add_argument("--kv-heads", type=int, default=8)
    parser.add_argument("--head-dim", type=int, default=128)
    parser.add_argument("--page-size", type=int, default=16)
    parser.add_argument("--window", type=int, default=0)
    parser.add_argument("--chunk", type=int, default=0, help="attention: a chunked mask of this size, with sinks")
    parser.add_argument("--softcap", type=float, default=0.0, help="attention: scores bounded by softcap * tanh(s / softcap)")
    parser.add_argument("--keys-only", action="store_true", help="attention: a cache of keys that are the values too")
    parser.add_argument("--experts", type=int, default=16)
    parser.add_argument("--top", type=int, default=4)
    parser.add_argument("--value-dim", type=int, default=128, help="state_scan: value channels per head")
    parser.add_argument("--mode", choices=("gated", "state_space"), default="gated")
    parser.add_argument("--segment", type=int, default=-1, help="state_scan: tokens of a segment (0: one piece; -1: chosen)")
    parser.add_argument("--split", type=int, default=0, help="fixed splits of this many positions in the decode kernel (0: balanced items)")
    parser.add_argument("--rows", type=int, default=8)
    parser.add_argument("--n", type=int, default=6144)
    parser.add_argument("--k", type=int, default=1024)
    parser.add_argument("--hidden", type=int, default=1024)
    parser.add_argument("--ffn", type=int, default=3072)
    parser.add_argument("--swiglu", action="store_true")
    parser.add_argument("--float-out", action="store_true")
    parser.add_argument("--vocab", type=int, default=151936)
    parser.add_argument("--temperature", type=float, default=0.0)
    parser.add_argument("--top-k", type=int, default=0)
    parser.add_argument("--top-p", type=float, default=0.0)
    parser.add_argument("--min-p", type=float, default=0.0)
    parser.add_argument("--top-logprobs", type=int, default=-1)
    parser.add_argument("--logit-scale", type=float, default=1.0, help="the logits are normal draws times this")
    parser.add_argument("--sequential-pages", action="store_true",
                        help="block tables that walk the pool in order instead of a random permutation")
    parser.add_argument("--legacy-prefill", action="store_true", help="prompt attention on mma.sync even where tcgen05 applies")
    parser.add_argument("--library", action="store_true", help="gemm_tc: time the vendor library's product instead")
    parser.add_argument("--own-products", action="store_true", help="products: none of them on the vendor library")
    parser.add_argument("--block-n", type=int, default=0, help="gemm_tc: width of an output tile (256, 128; 0: chosen)")
    parser.add_argument("--resident", action="store_true",
                        help="do not rotate operands: what fits in L2 is read from L2")
    args = parser.parse_args(argv)
    global RESIDENT, SEQUENTIAL_PAGES
    RESIDENT, SEQUENTIAL_PAGES = args.resident, args.sequential_pages
    ops.USE_TCGEN05_PREFILL = not args.legacy_prefill
    ops.USE_LIBRARY_PRODUCTS = not args.own_products
    if not torch.cuda.is_available():
        print("a CUDA device is needed", file=sys.stderr)
        return 2
    print(json.dumps(CASES[args.case](args)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
