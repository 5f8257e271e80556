"""Grouped-query causal attention over the paged cache, as a mixer.

q = x Wq^T, k = x Wk^T, v = x Wv^T without bias; q and k are RMS-normalised per head (one scale
vector each, shared by the heads) before the position encoding; query head j reads key/value head
j // (heads / kv_heads); scale 1/sqrt(head_dim); causal, with an optional window; the heads are
concatenated in order and projected by Wo (reference: src/model/causal_lm/qwen3.cpp:17-69).

The three projections run as one product over the row-concatenated weight.  Per-head norm, rotation
and the cache write are one kernel when the position encoding offers rotation tables
(``PositionEncoding.as_rotation_tables``: the NeoX rotation, or no encoding at all); any other
encoding goes through its own ``apply`` and separate norm and write kernels.

Beyond that form the part takes, as parameters: biases on the four projections (``q_bias`` ...), values
of another width than the keys (``value_dim``), a score scale of its own (``scale``), a chunked mask
(``chunk`` = n: position i sees j <= i only if i // n == j // n, chunks counted from position 0), a
learned sink per query head (``sinks``: exp(sink_h) joins the softmax's denominator, with no key, no
value and no scaling), and the rotation of adjacent pairs on part of the head (position kind
``rope_pairs``), values that are the keys as projected, before their norm (``values_from_keys``: there is
no value projection), a per-head norm of q and k without scales (``unit_qk_norm``), a multiplier on the
normed queries that grows with the position, 1 + coef * ln(floor((p + 1) / every) + 1) (``q_temp`` =
{"coef", "every"}), and a smooth bound on the scaled scores, s <- softcap * tanh(s / softcap)
(``softcap``).  Any of these sends the layer down the general path: the projection's float32 output
goes through one kernel (bias, norms, rotation, cache write: ``ops.qkv_pairs``) and the general
attention kernel, which takes all of them, for prompts and single tokens alike.

A second family of parameters runs through ``ops.qkv_halves`` instead: the rotation of halves on part of a
head (position kind ``rope_halves``: value i of the first ``dims`` pairs with value i + dims / 2), an RMS norm
over ALL heads of q and of k at once with a scale per column (``qk_norm`` "whole"; "per_head" is the default),
values divided by their root mean square per head (``value_unit_norm``), first tokens that a window never
lets go (``keep_first`` = n: key j < n stays visible, at its true position), pooled blocks behind the window
(``pool`` = P: the means of the keys and of the values of every whole block of P positions are kept in a
second store, one entry a block, and a query at position i sees, beside its window, the blocks that end at
or before i - window, in the same softmax), a mixing of the heads' softmax weights (``head_mix``: a matrix M
[heads, heads]; head h applies sum_g M[h, g] weights_g to the values of its own key/value head), and a
sigmoid gate on the joined heads before the output projection (``out_gate``: sigmoid(Wg x), value by value).
"""

from __future__ import annotations

import math
from typing import Mapping

import torch

from ..cache import PagedCacheSpec
from ..config.errors import ConfigError
from ..config.spec import LayerCall, MixerSpec
from ..kernels import ops
from ..weights.loader import ROLE_LINEAR, ROLE_NORM, ROLE_ZERO, WeightDecl
from .base import POSITION_ENCODINGS, Mixer, StepContext, lookup, register_mixer


class Attention(Mixer):
    graph_safe = True

    def __init__(self, spec: MixerSpec, weights: Mapping[str, torch.Tensor], dtype: torch.dtype,
                 device: torch.device | str):
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.nh = int(p["num_heads"])
        self.nkv = int(p["num_kv_heads"])
        self.hd = int(p["head_dim"])
        self.window = int(p.get("window", 0))
        self.unit_norm = bool(p.get("unit_qk_norm", False))
        self.eps = float(p["qk_norm_eps"]) if (p.get("q_norm") or self.unit_norm or p.get("value_unit_norm")) else 0.0
        self.values_from_keys = bool(p.get("values_from_keys", False))
        self.softcap = float(p.get("softcap") or 0.0)
        temp = p.get("q_temp")
        self.q_temp = (float(temp["coef"]), int(temp["every"])) if temp else None
        if self.unit_norm and p.get("q_norm"):
            raise ConfigError("a norm of q and k has scales or has none")
        if self.softcap < 0.0 or (self.q_temp is not None and self.q_temp[1] <= 0):
            raise ConfigError("softcap is not negative and q_temp.every is positive")
        self.dtype = dtype
        if self.nh <= 0 or self.nkv <= 0 or self.nh % self.nkv != 0:
            raise ConfigError("attention needs positive head counts with heads divisible by kv_heads")
        if self.hd <= 0 or self.hd > 512:
            raise ConfigError(f"attention kernels take head sizes up to 512, not {self.hd}")
        self.vd = int(p.get("value_dim") or self.hd)
        self.chunk = int(p.get("chunk") or 0)
        if self.vd <= 0 or self.vd > 512 or self.chunk < 0:
            raise ConfigError("attention takes value widths up to 512 and a chunk size that is not negative")
        self.scale = float(p["scale"]) if p.get("scale") is not None else 1.0 / math.sqrt(float(self.hd))
        if self.values_from_keys and self.vd != self.hd:
            raise ConfigError("values that are the keys have the keys' width")
        projections = ("q_proj", "k_proj") if self.values_from_keys else ("q_proj", "k_proj", "v_proj")
        self.w_qkv = torch.cat([weights[p[name]] for name in projections], dim=0).contiguous()
        self.w_q = self.w_qkv[: self.nh * self.hd]
        self.w_o = weights[p["o_proj"]]
        self.q_norm = weights[p["q_norm"]] if p.get("q_norm") else None
        self.k_norm = weights[p["k_norm"]] if p.get("k_norm") else None
        if (self.q_norm is None) != (self.k_norm is None):
            raise ConfigError("q_norm and k_norm come together")
        if spec.position is not None:
            self.position = lookup(POSITION_ENCODINGS, "position encoding", spec.position.kind)(
                spec.position, dtype, device)
        else:
            self.position = None
        biases = [weights[p[name]] if p.get(name) else None
                  for name in (("q_bias", "k_bias") if self.values_from_keys else ("q_bias", "k_bias", "v_bias"))]
        if any(b is not None for b in biases) and any(b is None for b in biases):
            raise ConfigError("q, k and v biases come together")
        self.qkv_bias = torch.cat([b.float() for b in biases]).contiguous() if biases[0] is not None else None
        self.o_bias = weights[p["o_bias"]].float().contiguous() if p.get("o_bias") else None
        self.sinks = weights[p["sinks"]].float().contiguous() if p.get("sinks") else None
        pairs = getattr(self.position, "as_pair_frequencies", None)
        self.pair_freqs, self.pair_dims = pairs() if pairs is not None else (None, 0)
        halves = getattr(self.position, "as_half_frequencies", None)
        self.half_freqs, self.half_dims, self.half_mult = halves() if halves is not None else (None, 0, 1.0)
        self.qk_norm = str(p.get("qk_norm") or "per_head")
        self.value_unit_norm = bool(p.get("value_unit_norm", False))
        self.keep_first = int(p.get("keep_first") or 0)
        self.pool = int(p.get("pool") or 0)
        self.head_mix = weights[p["head_mix"]].float().contiguous() if p.get("head_mix") else None
        self.w_gate = weights[p["out_gate"]] if p.get("out_gate") else None
        if self.qk_norm not in ("per_head", "whole") or self.keep_first < 0 or self.pool < 0:
            raise ConfigError("qk_norm is 'per_head' or 'whole'; keep_first and pool are not negative")
        if (self.keep_first or self.pool) and self.window <= 0:
            raise ConfigError("kept first tokens and pooled blocks come with a window")
        # What runs through the kernel that rotates halves.
        self.halves = (halves is not None or self.qk_norm == "whole" or self.value_unit_norm or self.keep_first > 0
                       or self.pool > 0 or self.head_mix is not None or self.w_gate is not None)
        if self.halves and (pairs is not None or self.qkv_bias is not None or self.values_from_keys or self.unit_norm
                            or self.q_temp is not None):
            raise ConfigError("the rotation of halves and its companions do not combine with biases, a rotation of "
                              "adjacent pairs, keys as values, unit norms or a query multiplier")
        # What only the general path takes.
        self.general = (pairs is not None or self.vd != self.hd or self.chunk > 0 or self.sinks is not None
                        or self.qkv_bias is not None or self.o_bias is not None or p.get("scale") is not None
                        or self.values_from_keys or self.unit_norm or self.softcap > 0.0 or self.q_temp is not None
                        or self.halves)
        if self.general:
            self._init_general(p)
            return
        if self.hd % 16 != 0 or self.hd < 16:
            raise ConfigError(f"attention kernels take head sizes 16..256 in steps of 16, not {self.hd}")
        # The fused kernels (norm + rotation + cache write, and the decode attention that does all of it
        # itself) rotate NeoX pairs by per-position angles from float32 tables; an encoding says whether
        # it is one of those, and any other goes through its own ``apply``.
        tables = self.position.as_rotation_tables() if self.position is not None else (None, None)
        self.fused_position = tables is not None
        self.cos, self.sin = tables if tables is not None else (None, None)
        # An encoding that is a bias on the scores: only the general kernel adds one.
        self.score_slopes = self.position.as_score_slopes() if self.position is not None else None
        self.group = self.nh // self.nkv
        self.tile_tokens = ops.attention_tile_tokens(self.group)
        self.fast_decode = self.score_slopes is None and ops.paged_decode_supported(self.nh, self.nkv, self.hd, dtype)
        # Decode-only steps of this many requests or more: position encoding inside the attention kernel.
        # With few requests the kernel's own chain (the projection's arrival, a head's loads, its norm
        # and rotation, then the first tile) is as long as the separate kernel's: 4467 against 4620
        # tokens a second at 8 requests, 11305 against 11143 at 64.
        self.fuse_decode_rows = 32
        self.fast_prefill = self.score_slopes is None and ops.paged_prefill_supported(self.nh, self.nkv, self.hd, dtype)
        self.prefill_tile_tokens = ops.paged_prefill_tile_tokens()

    def _init_general(self, p) -> None:
        if self.hd % 2 != 0 and self.pair_freqs is not None:
            raise ConfigError("a rotation of adjacent pairs takes even key widths")
        if self.score_slopes_wanted():
            raise ConfigError("a bias on the scores and the general path's extras do not combine")
        if (self.position is not None and self.pair_freqs is None and self.half_freqs is None
                and self.position.as_rotation_tables() != (None, None)):
            raise ConfigError("the general attention path rotates adjacent pairs, halves of part of a head, or nothing")
        if self.halves and self.w_gate is not None:
            self.w_qkv = torch.cat([self.w_qkv, self.w_gate], dim=0).contiguous()
            self.w_q = self.w_qkv[: self.nh * self.hd]
        self.q_norm = self.q_norm.float().contiguous() if self.q_norm is not None else None
        self.k_norm = self.k_norm.float().contiguous() if self.k_norm is not None else None
        self.score_slopes = None
        self.group = self.nh // self.nkv
        self.tile_tokens = ops.attention_tile_tokens(self.group)
        self.fused_position = False
        # The split-context decode kernel and the tensor-core prompt kernel take a chunked mask, sinks and
        # a bound on the scores too, for keys and values of one width in bfloat16; everything else stays
        # with the general kernel.
        equal = self.vd == self.hd
        # Kept first tokens, pooled blocks and mixed heads are masks and outputs of the mma.sync prompt kernel
        # (and of the general one); it then serves single tokens too, as tiles of one token.
        self.windowed = bool(self.keep_first or self.pool or self.head_mix is not None)
        self.fast_decode = equal and not self.windowed and ops.paged_decode_supported(self.nh, self.nkv, self.hd, self.dtype)
        self.fast_prefill = equal and ops.paged_prefill_supported(self.nh, self.nkv, self.hd, self.dtype)
        self.prefill_tile_tokens = ops.paged_prefill_tile_tokens()

    def score_slopes_wanted(self) -> bool:
        return self.position is not None and self.position.as_score_slopes() is not None

    @staticmethod
    def weight_decls(spec: MixerSpec) -> dict[str, WeightDecl]:
        p = spec.params
        hidden, nh, nkv, hd = int(p["hidden_size"]), int(p["num_heads"]), int(p["num_kv_heads"]), int(p["head_dim"])
        vd = int(p.get("value_dim") or hd)
        decls = {
            p["q_proj"]: WeightDecl((nh * hd, hidden), ROLE_LINEAR),
            p["k_proj"]: WeightDecl((nkv * hd, hidden), ROLE_LINEAR),
            p["o_proj"]: WeightDecl((hidden, nh * vd), ROLE_LINEAR),
        }
        if not p.get("values_from_keys"):
            decls[p["v_proj"]] = WeightDecl((nkv * vd, hidden), ROLE_LINEAR)
        if p.get("q_norm"):
            whole = p.get("qk_norm") == "whole"
            decls[p["q_norm"]] = WeightDecl((nh * hd if whole else hd,), ROLE_NORM)
            decls[p["k_norm"]] = WeightDecl((nkv * hd if whole else hd,), ROLE_NORM)
        if p.get("head_mix"):
            decls[p["head_mix"]] = WeightDecl((nh, nh), ROLE_LINEAR)
        if p.get("out_gate"):
            decls[p["out_gate"]] = WeightDecl((nh * vd, hidden), ROLE_LINEAR)
        for name, size in (("q_bias", nh * hd), ("k_bias", nkv * hd), ("v_bias", nkv * vd), ("o_bias", hidden),
                           ("sinks", nh)):
            if p.get(name) and not (name == "v_bias" and p.get("values_from_keys")):
                decls[p[name]] = WeightDecl((size,), ROLE_ZERO)
        return decls

    def weights_read(self) -> list[torch.Tensor]:
        return [t for t in (self.w_qkv, self.w_o, self.q_norm, self.k_norm, self.head_mix) if t is not None]

    @staticmethod
    def cache_spec(spec: MixerSpec) -> "PagedCacheSpec | tuple":
        """The tokens' pages; with pooled blocks a second store of one entry per block beside them.  The
        tokens of a block must outlive the window until their block is whole, so the pages of a pooled
        layer are given back by the larger of the two."""
        p = spec.params
        window, pool = int(p.get("window", 0)), int(p.get("pool") or 0)
        sizes = dict(key_dim=int(p["head_dim"]), value_dim=int(p.get("value_dim") or p["head_dim"]))
        tokens = PagedCacheSpec(int(p["num_kv_heads"]), window=max(window, pool) if window > 0 else 0,
                                chunk=int(p.get("chunk") or 0), keep_first=int(p.get("keep_first") or 0), **sizes)
        if pool <= 0:
            return tokens
        return tokens, PagedCacheSpec(int(p["num_kv_heads"]), every=pool, **sizes)

    @staticmethod
    def tile_requests(spec: MixerSpec) -> list[tuple[int, str]]:
        p = spec.params
        tokens = ops.attention_tile_tokens(int(p["num_heads"]) // int(p["num_kv_heads"]))
        wide = ops.paged_prefill_tile_tokens()
        return [(tokens, "all"), (tokens, "multi"), (tokens, "single"), (wide, "multi"), (wide, "all")]

    # ------------------------------------------------------------------ forward
    def _store_projected(self, projected: torch.Tensor, ctx: StepContext, call: LayerCall) -> torch.Tensor:
        """Per-head norm, rotation and cache write in one kernel; returns the queries."""
        nh, nkv, hd = self.nh, self.nkv, self.hd
        table = ctx.block_table(call.cache)
        cos, sin = self.cos, self.sin
        if call.writes_cache:
            return ops.qk_norm_rope_cache(projected, nh, nkv, hd, self.q_norm, self.k_norm, self.eps, cos, sin,
                                          ctx.positions, ctx.token_row, ctx.caches[call.cache], table, ctx.status)
        return ops.qk_norm_rope_cache(projected, nh, 1, hd, self.q_norm, self.k_norm, self.eps, cos, sin,
                                      ctx.positions, ctx.token_row, None, table, ctx.status)

    def _project_and_store(self, x: torch.Tensor, ctx: StepContext, call: LayerCall) -> torch.Tensor:
        nh, nkv, hd = self.nh, self.nkv, self.hd
        cache = ctx.caches[call.cache]
        table = ctx.block_table(call.cache)
        if self.fused_position:
            # A layer that reads another layer's cache needs no k and v.
            return self._store_projected(ops.linear(x, self.w_qkv if call.writes_cache else self.w_q), ctx, call)
        # Any other position encoding: the parts one after the other.
        T = x.shape[0]
        if not call.writes_cache:
            q = ops.linear(x, self.w_q)
            if self.q_norm is not None:
                q = ops.rmsnorm(q.view(T, nh, hd), self.q_norm, self.eps).view(T, nh * hd)
            return self.position.apply(q, nh, ctx.positions, ctx.status)
        qkv = ops.linear(x, self.w_qkv)
        q = qkv[:, : nh * hd].contiguous()
        k = qkv[:, nh * hd: (nh + nkv) * hd].contiguous()
        v = qkv[:, (nh + nkv) * hd:]
        if self.q_norm is not None:
            q = ops.rmsnorm(q.view(T, nh, hd), self.q_norm, self.eps).view(T, nh * hd)
            k = ops.rmsnorm(k.view(T, nkv, hd), self.k_norm, self.eps).view(T, nkv * hd)
        q = self.position.apply(q, nh, ctx.positions, ctx.status)
        k = self.position.apply(k, nkv, ctx.positions, ctx.status)
        ops.kv_write(k, v, nkv, hd, ctx.positions, ctx.token_row, cache, table, ctx.status)
        return q

    def attend(self, q: torch.Tensor, ctx: StepContext, call: LayerCall) -> torch.Tensor:
        """Rows with one new token go to the split-context decode kernel, rows with several to the
        tensor-core prompt kernel, where those kernels take this shape and type; whatever is left
        goes to the general kernel."""
        cache = ctx.caches[call.cache]
        table = ctx.block_table(call.cache)
        if self.general and self.windowed:
            return self._attend_windowed(q, ctx, call, cache, table)
        out = torch.empty((q.shape[0], self.nh * self.vd), dtype=q.dtype, device=q.device)
        common = (self.nh, self.nkv, self.hd, self.window, self.scale, ctx.status)
        masks = {"chunk": self.chunk, "sinks": self.sinks} if (self.chunk or self.sinks is not None) else {}
        if self.softcap > 0.0:
            masks["softcap"] = self.softcap
        decode_done = self.fast_decode and ctx.num_decode_rows > 0
        if decode_done:
            ops.paged_decode(q, cache, table, ctx.decode_rows, ctx.row_q_start, ctx.row_ctx, ctx.max_decode_context,
                             *common, out=out, **masks)
        prefill_done = False
        if self.fast_prefill:
            tile_row, tile_q0 = ctx.tiles[(self.prefill_tile_tokens, "multi")]
            prefill_done = True
            if tile_row.numel() > 0:
                ops.paged_prefill(q, cache, table, tile_row, tile_q0, ctx.row_q_start, ctx.row_q_len, ctx.row_ctx,
                                  *common, out=out, **masks)
        if decode_done and prefill_done:
            return out
        which = "multi" if decode_done else ("single" if prefill_done else "all")
        tile_row, tile_q0 = ctx.tiles[(self.tile_tokens, which)]
        if tile_row.numel() > 0:
            ops.paged_attention(q, cache, table, tile_row, tile_q0, self.tile_tokens, ctx.row_q_start, ctx.row_q_len,
                                ctx.row_ctx, *common, out=out, head_slopes=self.score_slopes, value_dim=self.vd, **masks)
        return out

    def _attend_windowed(self, q: torch.Tensor, ctx: StepContext, call: LayerCall, cache, table) -> torch.Tensor:
        """Attention with kept first tokens, pooled blocks or mixed heads: every row, prompts and single
        tokens alike, on the mma.sync prompt kernel where it takes the shape (bfloat16, one width for keys
        and values that is a multiple of 32 up to 256; a single token's query rows are the heads of a group, so
        its keys and values stream once a group), on the general kernel elsewhere.  With mixed heads
        the kernel hands out every head's weights on every key/value head's values, unrounded, and a second
        kernel mixes them."""
        masks = {"chunk": self.chunk, "sinks": self.sinks, "keep_first": self.keep_first}
        if self.softcap > 0.0:
            masks["softcap"] = self.softcap
        if self.pool:
            masks.update(pool=self.pool, pool_cache=ctx.caches[call.extra_caches[0]],
                         pool_table=ctx.block_table(call.extra_caches[0]))
        mixed = self.head_mix is not None
        width = self.nh * self.vd * (self.nkv if mixed else 1)
        out = torch.empty((q.shape[0], width), dtype=torch.float32 if mixed else q.dtype, device=q.device)
        common = (self.nh, self.nkv, self.hd, self.window, self.scale, ctx.status)
        if self.fast_prefill:
            # Rows with several tokens as tiles of tokens; single tokens as tiles of the heads of a group.
            # (The kernel takes groups of up to 16 heads that way; larger ones run as tiles of one token.)
            for which, by_group in (((self.prefill_tile_tokens, "multi"), False),
                                    ((self.tile_tokens, "single"), self.group <= 16)):
                tile_row, tile_q0 = ctx.tiles[which]
                if tile_row.numel() > 0:
                    ops.paged_prefill(q, cache, table, tile_row, tile_q0, ctx.row_q_start, ctx.row_q_len, ctx.row_ctx,
                                      *common, out=out, cross_values=mixed, by_group=by_group, **masks)
        else:
            tile_row, tile_q0 = ctx.tiles[(self.tile_tokens, "all")]
            ops.paged_attention(q, cache, table, tile_row, tile_q0, self.tile_tokens, ctx.row_q_start, ctx.row_q_len,
                                ctx.row_ctx, *common, out=out, value_dim=self.vd, cross_values=mixed,
                                out_dtype=out.dtype, **masks)
        return ops.head_mix(out, self.head_mix, self.nh, self.nkv, self.vd, q.dtype) if mixed else out

    takes_out_dtype = True

    def _forward_general(self, x: torch.Tensor, ctx: StepContext, call: LayerCall,
                         out_dtype: torch.dtype | None) -> torch.Tensor:
        """Projection in float32 -> bias, norms, rotation, cache write -> the general kernel -> output
        projection (its bias added to the float32 or rounded product as ``out_dtype`` says)."""
        table = ctx.block_table(call.cache)
        # A layer that reads another layer's cache needs no k and v.
        weight, bias, cache = self.w_qkv, self.qkv_bias, ctx.caches[call.cache]
        if not call.writes_cache:
            weight, cache = self.w_q, None
            bias = bias[: self.nh * self.hd] if bias is not None else None
        projected = ops.linear(x, weight, out_dtype=torch.float32)
        if self.halves:
            return self._forward_halves(projected, ctx, call, cache, table, out_dtype)
        q = ops.qkv_pairs(projected, self.nh, self.nkv, self.hd, self.vd, bias, self.q_norm, self.k_norm, self.eps,
                          self.pair_freqs, self.pair_dims, ctx.positions, ctx.token_row, cache, table, ctx.status,
                          self.dtype, unit_norm=self.unit_norm, values_from_keys=self.values_from_keys,
                          q_temp=self.q_temp)
        attended = self.attend(q, ctx, call)
        return ops.linear(attended, self.w_o, out_dtype=out_dtype, bias=self.o_bias)

    def _forward_halves(self, projected: torch.Tensor, ctx: StepContext, call: LayerCall, cache, table,
                        out_dtype: torch.dtype | None) -> torch.Tensor:
        """Norms, rotation of halves and cache write in one kernel; the blocks that this step's tokens
        complete are pooled; attention; the gate; the output projection."""
        if not call.writes_cache and self.w_gate is not None:
            raise ConfigError("a gated layer that reads another layer's cache is not built")
        q = ops.qkv_halves(projected, self.nh, self.nkv, self.hd, self.vd, self.qk_norm if self.q_norm is not None else "none",
                           self.q_norm, self.k_norm, self.eps, self.half_freqs, self.half_dims, self.half_mult,
                           self.value_unit_norm, ctx.positions, ctx.token_row, cache, table, ctx.status, self.dtype)
        if self.pool and call.writes_cache:
            ops.pool_blocks(cache, table, ctx.caches[call.extra_caches[0]], ctx.block_table(call.extra_caches[0]),
                            ctx.positions, ctx.token_row, self.nkv, self.hd, self.vd, self.pool, ctx.status)
        attended = self.attend(q, ctx, call)
        if self.w_gate is not None:
            at = (self.nh + 2 * self.nkv) * self.hd if self.vd == self.hd else self.nh * self.hd + self.nkv * (self.hd + self.vd)
            ops.sigmoid_gate(attended, projected[:, at:at + self.nh * self.vd])
        return ops.linear(attended, self.w_o, out_dtype=out_dtype, bias=self.o_bias)

    def forward(self, x: torch.Tensor, ctx: StepContext, call: LayerCall,
                out_dtype: torch.dtype | None = None) -> torch.Tensor:
        if self.general:
            return self._forward_general(x, ctx, call, out_dtype)
        if out_dtype not in (None, x.dtype):
            return self.forward(x, ctx, call).to(out_dtype)
        if self.fused_position and call.writes_cache:
            return ops.linear(self.core(ops.linear(x, self.w_qkv), ctx, call), self.w_o)
        q = self._project_and_store(x, ctx, call)
        return ops.linear(self.attend(q, ctx, call), self.w_o)

    def projections(self, call: LayerCall) -> tuple[torch.Tensor, torch.Tensor] | None:
        if not self.fused_position or self.general:
            return None
        return (self.w_qkv if call.writes_cache else self.w_q), self.w_o

    def core(self, projected: torch.Tensor, ctx: StepContext, call: LayerCall) -> torch.Tensor:
        if self._decodes_in_one(projected, ctx, call):
            # Every request brings one token: norms, rotation, the cache write of the new key and value
            # and the attention are one kernel, and nothing stands between the projection and it.
            out = torch.empty((projected.shape[0], self.nh * self.hd), dtype=projected.dtype, device=projected.device)
            return ops.paged_decode_fused(
                projected, ctx.caches[call.cache], ctx.block_table(call.cache), ctx.decode_rows, ctx.row_q_start,
                ctx.row_ctx, ctx.max_decode_context, self.nh, self.nkv, self.hd, self.window, self.scale, self.q_norm,
                self.k_norm, self.eps, self.cos, self.sin, ctx.status, out)
        return self.attend(self._store_projected(projected, ctx, call), ctx, call)

    def _decodes_in_one(self, projected: torch.Tensor, ctx: StepContext, call: LayerCall) -> bool:
        return (self.fast_decode and self.fused_position and call.writes_cache and projected.dtype == torch.bfloat16
                and ctx.num_decode_rows == ctx.num_rows == ctx.num_tokens and ctx.num_rows >= self.fuse_decode_rows)


register_mixer("attention", Attention)
