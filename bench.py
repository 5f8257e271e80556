"""Decode and prefill throughput of the engine on one B200, with the fraction of the roofline.

    python bench.py [--steps K] [--warmup W] [--gpus 1] [--impl ours|reference]
                    [--shape 0.6b|8b|32b] [--batch 8] [--context 4096] [--layers L]

One JSON line on standard output.  A "step" is one decode step of ``--batch`` sequences whose
contexts end at ``--context`` tokens.  ``value`` is decoded tokens a second timed on the device;
``e2e`` is the same through the Python entry point (``Engine.add_request`` / ``Engine.step``), with
the step's inputs copied from pinned host memory and the sampled tokens read back every step.
Weights are seeded random values of the named shape; token ids are seeded uniform random numbers.
Every decode step reads all weights and the whole cache of the live requests, several GB, far more
than the 126 MB L2, so no L2 flush is needed between timed steps (``config.l2`` says so).
"""

from __future__ import annotations

import argparse
import json
import os
import random
import statistics
import subprocess
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

SHAPES = {      # the layer sizes of the Qwen3 family members the benchmark names
    "0.6b": dict(num_hidden_layers=28, hidden_size=1024, num_attention_heads=16, num_key_value_heads=8, head_dim=128,
                 intermediate_size=3072, vocab_size=151936, tie_word_embeddings=True),
    "8b": dict(num_hidden_layers=36, hidden_size=4096, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
               intermediate_size=12288, vocab_size=151936, tie_word_embeddings=False),
    "32b": dict(num_hidden_layers=64, hidden_size=5120, num_attention_heads=64, num_key_value_heads=8, head_dim=128,
                intermediate_size=25600, vocab_size=151936, tie_word_embeddings=False),
}
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}

# ``--arch legelix``: layer sizes of the kind a model of a few billion parameters has, for the design whose
# layers alternate gated linear attention with attention and Mamba-2 side by side, each beside the Qwen3
# decoder of the same width, feed-forward, head counts and number of layers.
LEGELIX_SIZES = {
    "w2048": dict(width=2048, ff=6144, layers=8, heads=16, kv_heads=8, head_dim=128, chunk=1024,
                  gla=dict(heads=8, dim=128, vdim=256), ssm=dict(heads=32, vdim=64, state=128, groups=2)),
    "w4096": dict(width=4096, ff=12288, layers=8, heads=32, kv_heads=8, head_dim=128, chunk=2048,
                  gla=dict(heads=16, dim=128, vdim=256), ssm=dict(heads=64, vdim=64, state=128, groups=4)),
}

# ``--arch gefovik``: the same for the design whose layers norm their parts' outputs: one latent-attention
# layer in four, the others attention with keys as values, a bound on the scores and a query multiplier;
# feed-forwards dense (ReLU) and routed (16 experts and 2 identity experts, a token takes 4) in turn.  A
# routed layer's four experts together are as wide as the dense feed-forward.
GEFOVIK_SIZES = {
    "w2048": dict(width=2048, ff=6144, layers=8, heads=16, kv_heads=8, head_dim=128, rank=128, experts=16, identity=2, top=4),
    "w4096": dict(width=4096, ff=12288, layers=8, heads=32, kv_heads=8, head_dim=128, rank=128, latent_heads=16, experts=16,
                  identity=2, top=4),
}

# ``--arch fekotar``: the same for the design whose layers run latent attention (queries through a latent of
# their own, a rotated part, a gate per value) and a feed-forward side by side on one norm's output;
# feed-forwards bounded dense and routed (16 experts in 4 groups of which 2 are kept, a token takes 4) in
# turn.  A position keeps kv_rank + rot_dim = 128 values (160 in the last entry).  Beside it runs Gefovik, the closest
# design the engine has, with latent attention over a latent as wide in every layer and the same feed-forward sizes.
FEKOTAR_SIZES = {
    "w1024": dict(width=1024, ff=3072, layers=8, heads=8, dim=128, rot_dim=32, vdim=128, kv_rank=96, q_rank=384, experts=16, top=4,
                  groups=(4, 2)),
    "w2048": dict(width=2048, ff=6144, layers=8, heads=16, dim=128, rot_dim=32, vdim=128, kv_rank=96, q_rank=768, experts=16, top=4,
                  groups=(4, 2)),
    "w4096": dict(width=4096, ff=12288, layers=8, heads=16, dim=128, rot_dim=32, vdim=128, kv_rank=96, q_rank=1536, experts=16, top=4,
                  groups=(4, 2)),
    # a position keeps 128 + 32 = 160 values: prompts and decoded tokens on the mma.sync prompt kernel
    "w2048r160": dict(width=2048, ff=6144, layers=8, heads=16, dim=128, rot_dim=32, vdim=128, kv_rank=128, q_rank=768, experts=16,
                      top=4, groups=(4, 2)),
}


# ``--arch rizovik``: the same for the design whose layers mix attention over a window followed by pooled blocks
# (whole-projection norms, a gate per value), attention over a window that keeps the first tokens (the heads'
# weights mixed), and the gated delta rule, each with a routed feed-forward (16 experts, a token takes 4: a
# layer's active width is ``ff``); two of eight layers run an earlier layer's tensors.  Beside it runs Gefovik,
# the closest design the engine has (norms behind the parts, routed feed-forwards), with capped attention of the
# same head counts in every layer and the same routed sizes.
RIZOVIK_SIZES = {
    "w1024": dict(width=1024, ff=3072, layers=8, heads=8, kv_heads=4, head_dim=128, window=1024, pool=16, keep_first=64,
                  delta=dict(heads=8, kv_heads=4, dim=128, vdim=128), experts=16, top=4),
    "w2048": dict(width=2048, ff=6144, layers=8, heads=16, kv_heads=8, head_dim=128, window=1024, pool=16, keep_first=64,
                  delta=dict(heads=16, kv_heads=8, dim=128, vdim=128), experts=16, top=4),
    "w4096": dict(width=4096, ff=12288, layers=8, heads=32, kv_heads=8, head_dim=128, window=1024, pool=16, keep_first=64,
                  delta=dict(heads=32, kv_heads=8, dim=128, vdim=128), experts=16, top=4),
}


def metric_name(args) -> str:
    """One string for both arms: the driver divides their values only if the strings are equal."""
    return f"decode tok/s @ batch {args.batch}, context {args.context} (Qwen3-{args.shape.upper()} shape)"


def kernel_fractions(config, batch: int, context: int, peak: dict) -> tuple[dict, dict]:
    """The step's dominant kernels alone, timed with CUDA events over rotating operands larger than L2
    (``zephyr_b200.kernels.timing``): achieved bytes/s over the copy rate for the decode kernels,
    FLOP/s over the library's burst rate for the prompt kernels.  A layer's share of the decode step
    is its products (one fused chain) and its attention; the head comes once."""
    from types import SimpleNamespace

    from zephyr_b200.kernels import timing

    base = dict(warmup=3, iters=20, heads=config.num_attention_heads, kv_heads=config.num_key_value_heads,
                head_dim=config.head_dim, page_size=PAGE_SIZE, window=0, split=0, softcap=0.0, keys_only=False,
                hidden=config.hidden_size, ffn=config.intermediate_size)
    chain = timing.fused_chain(SimpleNamespace(rows=batch, **base))
    attention = timing.decode_attention(SimpleNamespace(batch=batch, context=context, **base))
    head = timing.gemm_small(SimpleNamespace(rows=batch, n=config.vocab_size, k=config.hidden_size, swiglu=False,
                                             float_out=True, **base))
    hbm, tflops = peak["hbm_gbs"], peak["bf16_tflops"]
    decode = {"layer_products": {"us": chain["us"], "frac": round(chain["gbs"] / hbm, 3)},
              "decode_attention": {"us": attention["us"], "frac": round(attention["gbs"] / hbm, 3)},
              "lm_head": {"us": head["us"], "frac": round(head["gbs"] / hbm, 3)}}
    prompt_attention = timing.prefill_attention(SimpleNamespace(tokens=PREFILL_TOKENS, **base))
    prompt_products = timing.products(SimpleNamespace(tokens=PREFILL_TOKENS, **base))
    prefill = {"attention": {"us": prompt_attention["us"], "frac": round(prompt_attention["tflops"] / tflops, 3)},
               "layer_products": {"us": prompt_products["us"], "frac": round(prompt_products["tflops"] / tflops, 3)}}
    return decode, prefill
PREFILL_TOKENS = 2048
PAGE_SIZE = 16


def peaks() -> tuple[dict, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            data = json.loads(path.read_text())
            if "hbm_gbs" in data and "bf16_tflops" in data:
                return data, "measured"
        except (OSError, ValueError):
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons every 200 ms while a timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.process = None

    def start(self):
        try:
            self.process = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "50"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.process = None

    def stop(self) -> dict:
        if self.process is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.process.terminate()
        try:
            out, _ = self.process.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.process.kill()
            out, _ = self.process.communicate()
        clocks, maxima, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                clocks.append(float(parts[0]))
                maxima.append(float(parts[1]))
            except ValueError:
                continue
            for name, value in zip(names, parts[3:7]):
                if value.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(clocks) if clocks else None,
                "sm_max_mhz": max(maxima) if maxima else None, "reasons": sorted(reasons), "samples": len(clocks)}


def build_engine(shape: str, layers: int | None, batch: int, context: int, dtype: str = "bfloat16",
                 prefill_together: int = 1):
    import torch

    from zephyr_b200 import Engine, Qwen3Config
    from zephyr_b200.engine import KvCacheOptions, PagedSchedulerConfig
    from zephyr_b200.parts import expected_weights
    from zephyr_b200.weights import RandomWeights

    sizes = dict(SHAPES[shape])
    full_layers = sizes["num_hidden_layers"]
    if layers:
        sizes["num_hidden_layers"] = layers
    config = Qwen3Config(max_position_embeddings=max(context, 4096), rms_norm_eps=1e-6, rope_theta=1000000.0, **sizes)
    spec = config.to_model_spec()
    store = RandomWeights(expected_weights(spec), seed=0, dtype=getattr(torch, dtype), device="cuda")
    # The pool is sized by the engine from the memory that is left after the weights and a profiled
    # step; it never holds more than ``batch`` sequences of the model's length need.
    engine = Engine(None, dtype=dtype, model_config=config, weights=store, max_seq_len=context,
                    kv_cache=KvCacheOptions(block_size=PAGE_SIZE),
                    # The token budget lets `prefill_together` whole prompts share one step, so that the
                    # sequences of the end-to-end run start decoding together and the batch stays whole.
                    scheduler=PagedSchedulerConfig(max_num_seqs=batch,
                                                   max_num_batched_tokens=max(PREFILL_TOKENS, batch,
                                                                              prefill_together * context),
                                                   max_prefill_chunk_tokens=max(PREFILL_TOKENS, context)))
    needed = batch * -(-context // PAGE_SIZE)
    if engine.runner.manager.groups[0].pool.num_usable < needed:
        raise SystemExit(f"bench.py: the cache pool got {engine.runner.manager.groups[0].pool.num_usable} pages, "
                         f"{needed} are needed for batch {batch} at context {context}")
    return engine, config, full_layers


def build_pair(size: str, batch: int, context: int):
    """(Legelix engine, Qwen3 engine builder) of one entry of ``LEGELIX_SIZES``; random weights, bfloat16."""
    import torch

    from zephyr_b200 import Engine
    from zephyr_b200.config import LegelixConfig, Qwen3Config
    from zephyr_b200.engine import KvCacheOptions, PagedSchedulerConfig
    from zephyr_b200.parts import expected_weights
    from zephyr_b200.weights import RandomWeights

    z = LEGELIX_SIZES[size]
    mlp = {"kind": "dense", "ff": z["ff"]}
    gla = {"type": "gla", "mixer": dict(tau=16.0, **z["gla"]), "mlp": mlp}
    left = dict(heads=z["heads"], kv_heads=z["kv_heads"], dim=z["head_dim"], vdim=z["head_dim"], scale=z["head_dim"] ** -0.5,
                mask={"size": z["chunk"]}, rot={"base": 500000.0, "dims": z["head_dim"],
                                                "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}})
    both = {"type": "parallel", "mlp": mlp, "mixer": {"left": left, "right": dict(conv=4, norm_groups=2, **z["ssm"]),
                                                      "left_scale": 1.0, "right_scale": 1.0}}
    legelix = LegelixConfig(vocab=32768, width=z["width"], layers=tuple([gla, both] * (z["layers"] // 2)), norm_eps=1e-6,
                            residual_mult=0.5, decay_rank=16)
    qwen = Qwen3Config(max_position_embeddings=max(context, 4096), rms_norm_eps=1e-6, rope_theta=1000000.0,
                       num_hidden_layers=z["layers"], hidden_size=z["width"], num_attention_heads=z["heads"],
                       num_key_value_heads=z["kv_heads"], head_dim=z["head_dim"], intermediate_size=z["ff"],
                       vocab_size=32768, tie_word_embeddings=False)

    def make(config):
        store = RandomWeights(expected_weights(config.to_model_spec()), seed=0, dtype=torch.bfloat16, device="cuda")
        return Engine(None, dtype="bfloat16", model_config=config, weights=store, max_seq_len=context,
                      kv_cache=KvCacheOptions(block_size=PAGE_SIZE, num_blocks=(batch + 1) * -(-context // PAGE_SIZE) + 1),
                      scheduler=PagedSchedulerConfig(max_num_seqs=batch + 1, max_num_batched_tokens=max(PREFILL_TOKENS, batch),
                                                     max_prefill_chunk_tokens=PREFILL_TOKENS))
    return legelix, qwen, make


def build_gefovik_pair(size: str, batch: int, context: int):
    """(Gefovik configuration, Qwen3 configuration, engine builder) of one entry of ``GEFOVIK_SIZES``."""
    from zephyr_b200.config import GefovikConfig

    z = GEFOVIK_SIZES[size]
    dense = {"kind": "dense", "ff": z["ff"]}
    routed = {"kind": "moe", "expert": {"ff": z["ff"] // z["top"]},
              "router": {"experts": z["experts"], "identity": z["identity"], "top": z["top"]}}
    hd = z["head_dim"]
    latent = {"type": "latent_attention", "mlp": dense,
              "mixer": dict(heads=z.get("latent_heads", z["heads"]), dim=hd, vdim=hd, kv_rank=z["rank"], scale=hd ** -0.5)}
    capped = dict(heads=z["heads"], kv_heads=z["kv_heads"], dim=hd, vdim=hd, scale=hd ** -0.5, softcap=50.0,
                  q_temp={"coef": 0.2, "every": 128})
    four = [latent, {"type": "attention", "mixer": capped, "mlp": routed}, {"type": "attention", "mixer": capped, "mlp": dense},
            {"type": "attention", "mixer": capped, "mlp": routed}]
    gefovik = GefovikConfig(vocab=32768, width=z["width"], layers=tuple(four * (z["layers"] // 4)), norm_eps=1e-6,
                            embedding_scale=1.0)
    _, qwen, make = build_pair(size, batch, context)
    return gefovik, qwen, make


def build_fekotar_pair(size: str, batch: int, context: int):
    """(Fekotar configuration, Gefovik configuration of equal sizes, engine builder) of one entry of ``FEKOTAR_SIZES``."""
    from zephyr_b200.config import FekotarConfig, GefovikConfig

    z = FEKOTAR_SIZES[size]
    scale = (z["dim"] + z["rot_dim"]) ** -0.5
    mixer = dict(heads=z["heads"], dim=z["dim"], rot_dim=z["rot_dim"], vdim=z["vdim"], kv_rank=z["kv_rank"], q_rank=z["q_rank"],
                 scale=scale, rot={"base": 10000.0, "dims": z["rot_dim"],
                                   "scaling": {"factor": 40.0, "original": 4096, "fast": 32.0, "slow": 1.0}})
    router = {"experts": z["experts"], "top": z["top"], "scale": 2.5, "groups": {"count": z["groups"][0], "keep": z["groups"][1]}}
    dense = {"kind": "dense", "ff": z["ff"], "limit": 7.0}
    routed = {"kind": "moe", "expert": {"ff": z["ff"] // z["top"]}, "router": router}
    fekotar = FekotarConfig(vocab=32768, width=z["width"], norm_eps=1e-6, logit_scale=0.25,
                            bigram={"buckets": 65521, "mul_prev": 36313, "mul_cur": 27191},
                            layers=tuple({"type": "latent_attention", "mixer": mixer, "mlp": mlp}
                                         for mlp in [dense, routed] * (z["layers"] // 2)))
    latent = dict(heads=z["heads"], dim=z["dim"], vdim=z["vdim"], kv_rank=z["kv_rank"] + z["rot_dim"], scale=z["dim"] ** -0.5)
    old_dense = {"kind": "dense", "ff": z["ff"]}
    old_routed = {"kind": "moe", "expert": {"ff": z["ff"] // z["top"]}, "router": {"experts": z["experts"], "identity": 0, "top": z["top"]}}
    gefovik = GefovikConfig(vocab=32768, width=z["width"], norm_eps=1e-6, embedding_scale=1.0,
                            layers=tuple({"type": "latent_attention", "mixer": latent, "mlp": mlp}
                                         for mlp in [old_dense, old_routed] * (z["layers"] // 2)))
    _, _, make = build_pair("w2048", batch, context)
    return fekotar, gefovik, make


def build_rizovik_pair(size: str, batch: int, context: int):
    """(Rizovik configuration, Gefovik configuration of equal sizes, engine builder) of one entry of ``RIZOVIK_SIZES``."""
    from zephyr_b200.config import GefovikConfig, RizovikConfig

    z = RIZOVIK_SIZES[size]
    hd = z["head_dim"]
    routed = {"kind": "moe", "expert": {"ff": z["ff"] // z["top"]}, "router": {"experts": z["experts"], "top": z["top"]}}
    sizes = dict(heads=z["heads"], kv_heads=z["kv_heads"], dim=hd, vdim=hd, scale=hd ** -0.5)
    pooled = {"type": "attention", "mlp": routed,
              "mixer": dict(sizes, rot={"base": 300000.0, "dims": hd // 2}, mask={"size": z["window"], "pool": z["pool"]})}
    kept = {"type": "attention_2", "mlp": routed,
            "mixer": dict(sizes, rot={"base": 40000.0, "dims": hd // 4, "scaling": {"factor": 4.0}},
                          mask={"size": z["window"], "keep_first": z["keep_first"]})}
    delta = {"type": "delta", "mlp": routed, "mixer": dict(conv=4, **z["delta"])}
    six = [pooled, kept, delta, pooled, kept, delta]
    layers = six + [dict(six[0], weights_of=0), dict(six[1], weights_of=1)]
    rizovik = RizovikConfig(vocab=32768, width=z["width"], norm_eps=1e-6, residual_mult=0.6, layers=tuple(layers[:z["layers"]]))
    old_routed = {"kind": "moe", "expert": {"ff": z["ff"] // z["top"]}, "router": {"experts": z["experts"], "identity": 0, "top": z["top"]}}
    capped = dict(heads=z["heads"], kv_heads=z["kv_heads"], dim=hd, vdim=hd, scale=hd ** -0.5, softcap=50.0,
                  q_temp={"coef": 0.2, "every": 128})
    gefovik = GefovikConfig(vocab=32768, width=z["width"], norm_eps=1e-6, embedding_scale=1.0,
                            layers=tuple({"type": "attention", "mixer": capped, "mlp": old_routed} for _ in range(z["layers"])))
    _, _, make = build_pair("w2048", batch, context)
    return rizovik, gefovik, make


def run_legelix(args) -> dict:
    """Prefill of 2048 tokens and a decode step of ``--batch`` requests at ``--context``, device-timed, for
    every entry of ``LEGELIX_SIZES`` (or ``GEFOVIK_SIZES``) and for the Qwen3 decoder of equal size beside it."""
    import gc

    import torch

    out = {"arch": args.arch, "batch": args.batch, "context": args.context, "prefill_tokens": PREFILL_TOKENS, "dtype": "bf16",
           "data": "synthetic: seeded random weights and token ids", "sizes": {}}
    table, pair, beside = {"legelix": (LEGELIX_SIZES, build_pair, "qwen3"), "gefovik": (GEFOVIK_SIZES, build_gefovik_pair, "qwen3"),
                           "fekotar": (FEKOTAR_SIZES, build_fekotar_pair, "gefovik"),
                           "rizovik": (RIZOVIK_SIZES, build_rizovik_pair, "gefovik")}[args.arch]
    for size in (args.sizes.split(",") if args.sizes else table):
        legelix, qwen, make = pair(size, args.batch, args.context)
        row = {}
        for name, config in ((args.arch, legelix), (beside, qwen)):
            engine = make(config)
            prefill_ms = device_prefill(engine, PREFILL_TOKENS, 3, 5)
            decode_ms, launches, _ = device_decode(engine, args.batch, args.context, args.warmup, args.steps, None)
            row[name] = {"prefill_ms": round(prefill_ms, 3), "prefill_tok_s": round(PREFILL_TOKENS / prefill_ms * 1e3),
                         "decode_ms_per_step": round(decode_ms, 4), "decode_tok_s": round(args.batch / decode_ms * 1e3),
                         "gpu_launches": launches, "weights_gb": round(engine.model.weight_bytes_read_per_step() / 1e9, 3)}
            del engine
            gc.collect()
            torch.cuda.empty_cache()
        out["sizes"][size] = row
    return out


def model_flops_per_token(config) -> float:
    """Matrix-product FLOPs per token of the layers (the head runs on the wanted rows only)."""
    h, i = config.hidden_size, config.intermediate_size
    qkv = (config.num_attention_heads + 2 * config.num_key_value_heads) * config.head_dim
    per_layer = 2 * (qkv * h + config.num_attention_heads * config.head_dim * h + 2 * i * h + i * h)
    return per_layer * config.num_hidden_layers


def prefill_flops(config, tokens: int) -> float:
    attention = config.num_hidden_layers * config.num_attention_heads * 2.0 * tokens * tokens * config.head_dim
    return model_flops_per_token(config) * tokens + attention + 2.0 * config.vocab_size * config.hidden_size


def device_decode(engine, batch: int, context: int, warmup: int, steps: int, sampler_clock: ClockSampler | None):
    """Device-timed decode: ``steps`` steps of ``batch`` sequences whose contexts end at ``context``."""
    import torch

    from zephyr_b200.engine import StepEntry
    from zephyr_b200.kernels import ops
    from zephyr_b200.sampling import SamplingParams

    runner, vocab = engine.runner, engine.vocab_size
    rng = random.Random(1234)
    start = context - (warmup + steps)
    ids = [("bench", i) for i in range(batch)]
    for rid in ids:
        assert runner.add_request(rid)
        done = 0
        while done < start:
            count = min(PREFILL_TOKENS, start - done)
            runner.step([StepEntry(rid, [rng.randrange(vocab) for _ in range(count)], ())])
            done += count
    runner.check()
    greedy = [SamplingParams(temperature=0.0)] * batch

    def one_step():
        logits = runner.step([StepEntry(rid, [rng.randrange(vocab)], (0,)) for rid in ids])
        return engine.sampler.sample_async(logits, greedy, [None] * batch)

    if sampler_clock:
        sampler_clock.start()        # nvidia-smi takes a moment to start: the warm-up gives it that
    for _ in range(warmup):
        one_step()
    torch.cuda.synchronize()
    launches_before = ops.LAUNCHES
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    begin.record()
    for _ in range(steps):
        one_step()
    end.record()
    torch.cuda.synchronize()
    clocks = sampler_clock.stop() if sampler_clock else None
    launches = ops.LAUNCHES - launches_before
    runner.check()
    ms = begin.elapsed_time(end) / steps
    for rid in ids:
        runner.free_request(rid)
    return ms, launches, clocks


def e2e_decode(engine, batch: int, context: int, warmup: int, steps: int):
    """The same through the entry point: every step copies its inputs from pinned host memory and
    reads the sampled tokens back."""
    import torch

    from zephyr_b200 import GenerationParams

    rng = random.Random(4321)
    start = context - (warmup + steps) - 1
    params = GenerationParams(max_tokens=warmup + steps + 1, temperature=0.0, ignore_eos=True)
    requests = [engine.add_request([rng.randrange(engine.vocab_size) for _ in range(start)], params)
                for _ in range(batch)]
    while any(engine.sequences[(r, 0)].state.value != "decode" for r in requests):
        engine.step()
    assert len({len(engine.sequences[(r, 0)].token_ids) for r in requests}) == 1, "the batch must decode in step"
    for _ in range(warmup):
        engine.step()
    torch.cuda.synchronize()
    # Bytes per step: the packed int32 step description up (taken from the last warm-up step; it
    # grows by a page id per sequence every 16 steps), the sampled ids and two status words down.
    h2d = engine.runner.last_step_h2d_bytes + 8 * 0
    d2h = 4 * batch + 2 * 16
    began = time.perf_counter()
    for _ in range(steps):
        engine.step()
    torch.cuda.synchronize()
    seconds = time.perf_counter() - began
    for r in requests:
        engine.cancel(r)
        engine.take_output(r)
    return batch * steps / seconds, h2d, d2h


def device_prefill(engine, tokens: int, warmup: int, reps: int):
    import torch

    from zephyr_b200.engine import StepEntry

    runner, vocab = engine.runner, engine.vocab_size
    rng = random.Random(99)
    times = []
    for rep in range(warmup + reps):
        rid = ("prefill", rep)
        assert runner.add_request(rid)
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        entry = [StepEntry(rid, [rng.randrange(vocab) for _ in range(tokens)], (tokens - 1,))]
        torch.cuda.synchronize()
        begin.record()
        runner.step(entry)
        end.record()
        torch.cuda.synchronize()
        if rep >= warmup:
            times.append(begin.elapsed_time(end))
        runner.free_request(rid)
    runner.check()
    return statistics.median(times)


def run_ours(args) -> dict:
    import torch

    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device")
    peak, peak_source = peaks()
    engine, config, full_layers = build_engine(args.shape, args.layers, max(args.batch, 64) if args.points else args.batch,
                                               args.context, prefill_together=args.batch)
    runner = engine.runner
    clock = ClockSampler()
    ms, launches, clocks = device_decode(engine, args.batch, args.context, args.warmup, args.steps, clock)
    value = args.batch * 1000.0 / ms
    weight_bytes = engine.model.weight_bytes_read_per_step()
    cache_bytes = args.batch * (args.context - args.steps / 2.0) * runner.cache_bytes_per_token()
    achieved = (weight_bytes + cache_bytes) / (ms * 1e-3) / 1e9
    e2e_value, h2d, d2h = e2e_decode(engine, args.batch, args.context, args.warmup, args.steps)
    prefill_ms = device_prefill(engine, PREFILL_TOKENS, 3, 5)
    flops = prefill_flops(config, PREFILL_TOKENS)
    points = {}
    if args.points:
        for batch in (1, 64):
            p_ms, _, _ = device_decode(engine, batch, args.context, 3, max(8, args.steps // 2), None)
            points[f"decode_b{batch}"] = round(batch * 1000.0 / p_ms, 1)
    decode_kernels, prefill_kernels = kernel_fractions(config, args.batch, args.context, peak)
    result = {
        "metric": metric_name(args),
        "value": round(value, 1), "unit": "tok/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic (seeded random weights and token ids)", "impl": "ours",
        "config": {
            "model": f"Qwen3-{args.shape.upper()} shape", "global_batch": args.batch, "seq_len": args.context,
            "parallelism": "single GPU", "layers": config.num_hidden_layers, "layers_full": full_layers,
            "hidden_size": config.hidden_size, "heads": config.num_attention_heads,
            "kv_heads": config.num_key_value_heads, "head_dim": config.head_dim,
            "intermediate_size": config.intermediate_size, "vocab_size": config.vocab_size,
            "tied_head": config.tie_word_embeddings, "kv_page_size": PAGE_SIZE, "prefill_tokens": PREFILL_TOKENS,
            "l2": "inputs (weights + cache, GBs per step) larger than L2; no flush",
            "peaks": f"{peak_source}: copy rate for decode, burst bf16 product rate for prefill",
            "cache_pages": runner.manager.groups[0].pool.num_usable,
        },
        "e2e": {"value": round(e2e_value, 1), "unit": "tok/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": launches,
        "clocks": clocks,
        "prefill": {"value": round(PREFILL_TOKENS * 1000.0 / prefill_ms, 1), "tokens": PREFILL_TOKENS,
                    "ms": round(prefill_ms, 3),
                    "frac": round(flops / (prefill_ms * 1e-3) / (peak["bf16_tflops"] * 1e12), 4),
                    "kernels": prefill_kernels},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / peak["hbm_gbs"], 4), "kernels": decode_kernels},
        "points": points,
    }
    return result


def run_reference(args) -> dict:
    """The unmodified reference, installed under baseline/_ref, through its own public Python API
    (``zephyr._C.Engine``: ``submit`` / ``wait_for_outputs``) on the same shape: seeded random weights
    written to a model folder, seeded random prompts (fresh ids for every run, so that its prefix
    cache cannot help).  Decode throughput is counted over the token increments it publishes, from
    the moment every sequence has produced its first token to the end of the run."""
    ref = ROOT / "baseline" / "_ref"
    if not (ref / "zephyr").is_dir():
        return {"impl": "reference", "unavailable": "baseline/_ref holds no installed reference (zephyr) package"}
    import tempfile

    import torch

    if not torch.cuda.is_available():
        return {"impl": "reference", "unavailable": "no CUDA device"}
    sys.path.insert(0, str(ref))
    try:
        from zephyr import _C
    except Exception as error:      # the reference's own import chain (tokenizer front end, native module)
        return {"impl": "reference", "unavailable": f"cannot import the installed reference: {type(error).__name__}: {error}"[:300]}

    from zephyr_b200 import Qwen3Config, write_random_model

    sizes = dict(SHAPES[args.shape])
    full_layers = sizes["num_hidden_layers"]
    if args.layers:
        sizes["num_hidden_layers"] = args.layers
    config = Qwen3Config(max_position_embeddings=max(args.context, 4096), rms_norm_eps=1e-6, rope_theta=1000000.0, **sizes)
    rng = random.Random(77)
    steps, batch = args.steps, args.batch
    start = args.context - steps - 1
    with tempfile.TemporaryDirectory() as folder:
        write_random_model(config, 0, folder, dtype=torch.bfloat16)
        try:
            options = _C.EngineOptions(folder, devices=[0], dtype="bfloat16", max_seq_len=args.context,
                                       scheduler=_C.PagedSchedulerConfig(max_num_seqs=batch,
                                                                         max_num_batched_tokens=PREFILL_TOKENS,
                                                                         max_prefill_chunk_tokens=PREFILL_TOKENS),
                                       eos_token_ids=[])
        except Exception as error:
            return {"impl": "reference", "unavailable": f"the reference engine did not start: {type(error).__name__}: {error}"[:300]}

        native = _C.Engine(options, kv_cache=_C.KvCacheOptions(block_size=PAGE_SIZE))

        def run(new_tokens: int, count: int, length: int):
            """Submit ``count`` requests and follow the token increments as they come out.  Returns
            (seconds in all, seconds from the moment every sequence has its first token to the end,
            tokens produced in that second stretch)."""
            requests = [_C.GenerationRequest([rng.randrange(config.vocab_size) for _ in range(length)],
                                             sampling=_C.SamplingParams(temperature=0.0), max_new_tokens=new_tokens,
                                             ignore_eos=True) for _ in range(count)]
            torch.cuda.synchronize()
            began = time.perf_counter()
            produced = {native.submit(request): 0 for request in requests}
            finished, all_started, tokens_at_start = 0, None, 0
            while finished < count:
                for output in native.wait_for_outputs():
                    produced[output.request_id] += sum(len(choice.tokens) for choice in output.result)
                    if output.status is not None:
                        if output.status != _C.RequestStatus.COMPLETED:
                            raise RuntimeError(f"request ended with {output.status}: {output.error_message}")
                        finished += 1
                if all_started is None and all(n >= 1 for n in produced.values()):
                    all_started, tokens_at_start = time.perf_counter(), sum(produced.values())
            ended = time.perf_counter()
            assert all(n == new_tokens for n in produced.values())
            return ended - began, ended - (all_started or ended), sum(produced.values()) - tokens_at_start

        clock = ClockSampler()
        try:
            run(2, batch, start)
            clock.start()
            _, decode_seconds, decode_tokens = run(steps + 1, batch, start)
            clocks = clock.stop()
            prefill_runs = [run(1, 1, PREFILL_TOKENS)[0] for _ in range(3)]
        except Exception as error:
            clock.stop()
            return {"impl": "reference", "unavailable": f"the reference failed while generating: {type(error).__name__}: {error}"[:300]}
        finally:
            native.close()
    value = decode_tokens / max(decode_seconds, 1e-9)
    steps_timed = max(decode_tokens / batch, 1e-9)
    prefill_ms = statistics.median(prefill_runs[1:]) * 1e3
    return {
        "metric": metric_name(args), "value": round(value, 1),
        "unit": "tok/s", "n_gpus": 1, "steps": steps, "warmup": args.warmup,
        "ms_per_step": round(decode_seconds / steps_timed * 1e3, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic (seeded random weights and token ids)",
        "impl": "reference",
        "config": {"model": f"Qwen3-{args.shape.upper()} shape", "global_batch": batch, "seq_len": args.context,
                   "parallelism": "single GPU", "layers": config.num_hidden_layers, "layers_full": full_layers,
                   "kv_page_size": PAGE_SIZE, "prefill_tokens": PREFILL_TOKENS,
                   "timing": "wall clock over _C.Engine token increments, from every sequence's first token to the end"},
        "e2e": {"value": round(value, 1), "unit": "tok/s", "h2d_bytes_per_step": None, "d2h_bytes_per_step": None},
        "clocks": clocks,
        "prefill": {"value": round(PREFILL_TOKENS * 1e3 / prefill_ms, 1), "tokens": PREFILL_TOKENS, "ms": round(prefill_ms, 3)},
    }


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=64)
    parser.add_argument("--warmup", type=int, default=8)
    parser.add_argument("--impl", choices=("ours", "reference"), default="ours")
    parser.add_argument("--shape", choices=sorted(SHAPES), default="0.6b")
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--context", type=int, default=4096)
    parser.add_argument("--layers", type=int, default=None, help="fewer layers than the shape has (both are reported)")
    parser.add_argument("--no-points", dest="points", action="store_false", help="skip decode at batch 1 and 64")
    parser.add_argument("--own-products", action="store_true",
                        help="with --only: no product on the vendor library (all on this package's tcgen05 kernel)")
    parser.add_argument("--arch", choices=("qwen3", "legelix", "gefovik", "fekotar", "rizovik"), default="qwen3",
                        help="legelix, gefovik: prefill and decode of that design at a few layer sizes, beside Qwen3 of equal "
                             "size; fekotar, rizovik: the same beside Gefovik of equal size")
    parser.add_argument("--sizes", default="", help="--arch legelix|gefovik|fekotar|rizovik: entries of that design's table of sizes, with commas (default: all)")
    parser.add_argument("--only", choices=("prefill", "decode"), default=None,
                        help="time only the 2048-token prefill, or only the decode step, and print a short line "
                             "(the program a profiler is pointed at)")
    args = parser.parse_args()
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not measured")
        return 2
    if args.warmup < 3:
        args.warmup = 3
    if args.arch in ("legelix", "gefovik", "fekotar", "rizovik"):
        print(json.dumps(run_legelix(args)))
        return 0
    if args.only is not None and args.impl == "ours":
        if args.own_products:
            from zephyr_b200.kernels import ops
            ops.USE_LIBRARY_PRODUCTS = False
        engine, config, _ = build_engine(args.shape, args.layers, args.batch, args.context, prefill_together=1)
        if args.only == "prefill":
            ms = device_prefill(engine, PREFILL_TOKENS, 3, args.steps)
            print(json.dumps({"only": "prefill", "tokens": PREFILL_TOKENS, "layers": config.num_hidden_layers, "ms": round(ms, 4)}))
        else:
            ms, launches, _ = device_decode(engine, args.batch, args.context, args.warmup, args.steps, None)
            print(json.dumps({"only": "decode", "batch": args.batch, "layers": config.num_hidden_layers, "ms_per_step": round(ms, 4),
                              "gpu_launches": launches}))
        return 0
    result = run_reference(args) if args.impl == "reference" else run_ours(args)
    print(json.dumps(result))
    return 0


if __name__ == "__main__":
    sys.exit(main())
