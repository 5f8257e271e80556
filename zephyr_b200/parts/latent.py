"""Latent attention as a mixer: keys and values of all heads are two linear maps of one small latent per
position, and only the latent is cached.

    q = Wq h                                   [heads, dim]
    c = rmsnorm(Wc h) * w_c                    [rank]        (the latent; the one thing a position keeps)
    k_j = Wuk c_j,  v_j = Wuv c_j              per head: [dim], [vdim]
    score_ij = scale * (q_i . k_j),  causal;   softmax, with exp(sink_h) in the denominator where the
                                               spec names sinks (a term without key or value)
    o_i = sum_j p_ij v_j,  times sigmoid(Wg h)_h where the spec names a gate;  out = Wo concat(o)

Optional pieces, each named by the spec: queries through a latent of their own (c_q = rmsnorm(Wdq h) w_q,
q = Wuq c_q); a rotated part (``rot_dim`` > 0 with a position encoding that offers ``as_half_frequencies``:
every query head carries ``rot_dim`` more values behind its ``dim`` unrotated ones, the latent projection
``rot_dim`` more rows that form ONE rotated key part shared by all heads, and the score is
q_unrotated . k_unrotated + q_rotated . k_rotated; the cached row is then the normed latent followed by
the rotated key part, and the values are maps of its first ``rank`` entries); a gate per output value
instead of one per head (a gate matrix of heads * vdim rows).

Without a rotated part there is no position encoding.  The part works in the latent space, which is what makes caching c alone
enough: q_i . (Wuk_h c_j) = (Wuk_h^T q_i) . c_j and sum_j p_ij Wuv_h c_j = Wuv_h (sum_j p_ij c_j).  So the
queries are carried into the latent space head by head (``ops.head_linear`` with the transposed key
maps), the attention runs with ONE key/value head of width ``rank`` whose keys are its values (a cache
that keeps keys only), and the result is carried out by the value maps, with the gate in the same
kernel.  Scores, softmax and the latent's norm are float32.
"""

from __future__ import annotations

from typing import Mapping

import torch

from ..cache import PagedCacheSpec
from ..config.errors import ConfigError
from ..config.spec import LayerCall, MixerSpec
from ..kernels import ops
from ..weights.loader import ROLE_LINEAR, ROLE_NORM, ROLE_ZERO, WeightDecl
from .base import POSITION_ENCODINGS, Mixer, StepContext, lookup, register_mixer


class LatentAttention(Mixer):
    graph_safe = True
    takes_out_dtype = True

    def __init__(self, spec: MixerSpec, weights: Mapping[str, torch.Tensor], dtype: torch.dtype,
                 device: torch.device | str):
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.nh, self.hd, self.vd, self.rank = int(p["num_heads"]), int(p["head_dim"]), int(p["value_dim"]), int(p["rank"])
        self.scale = float(p["scale"])
        self.eps = float(p["norm_eps"])
        self.dtype = dtype
        if min(self.nh, self.hd, self.vd, self.rank) <= 0:
            raise ConfigError("latent attention needs positive head count, head sizes and rank")
        self.rot = int(p.get("rot_dim", 0))
        self.kw = self.rank + self.rot            # what a position keeps: the latent and the rotated key part
        if self.kw > 768:
            raise ConfigError(f"latent attention keeps at most 768 values a position, not {self.kw}")
        self.position = None
        self.freqs, self.rope_mult = None, 1.0
        if self.rot > 0:
            if spec.position is None:
                raise ConfigError("a rotated part needs a position encoding")
            self.position = lookup(POSITION_ENCODINGS, "position encoding", spec.position.kind)(spec.position, dtype, device)
            halves = getattr(self.position, "as_half_frequencies", None)
            if halves is None or halves()[1] != self.rot:
                raise ConfigError("latent attention rotates the halves of its whole rotated part (dims = rot_dim)")
            self.freqs, _, self.rope_mult = halves()
        nh, hd, vd, rank = self.nh, self.hd, self.vd, self.rank
        gate = weights[p["gate"]] if p.get("gate") else None
        # One product for everything that reads the layer's input: queries (or their latent), the latent, the gates.
        self.q_rank = int(p["q_rank"]) if p.get("q_down") else 0
        first = weights[p["q_down"]] if self.q_rank else weights[p["q_proj"]]
        rows = [first, weights[p["latent_proj"]]] + ([gate] if gate is not None else [])
        self.w_in = torch.cat(rows, dim=0).contiguous()
        self.q_cols = first.shape[0]
        self.w_q_up = weights[p["q_proj"]] if self.q_rank else None
        self.q_norm = weights[p["q_down_norm"]].float().contiguous() if self.q_rank else None
        self.has_gate = gate is not None
        self.latent_norm = weights[p["latent_norm"]].float().contiguous()
        # Per head [rank, dim]: the key map transposed, so that it carries a query into the latent space.
        self.w_q_to_latent = weights[p["k_up"]].view(nh, hd, rank).transpose(1, 2).contiguous()
        if gate is not None and gate.shape[0] not in (nh, nh * vd):
            raise ConfigError("a gate has one row per head or one per output value")
        self.w_latent_to_v = weights[p["v_up"]].view(nh, vd, rank).contiguous()
        self.w_o = weights[p["o_proj"]]
        self.sinks = weights[p["sinks"]].float().contiguous() if p.get("sinks") else None
        self.tile_tokens = ops.attention_tile_tokens(nh)
        # In bfloat16 the split-context decode kernel and the tensor-core prompt kernel take the latent
        # as one key/value head whose keys are its values, where they take its width and head count.
        self.fast_decode = ops.paged_decode_supported(nh, 1, self.kw, dtype)
        self.fast_prefill = ops.paged_prefill_supported(nh, 1, self.kw, dtype)
        self.prefill_tile_tokens = ops.paged_prefill_tile_tokens()

    @staticmethod
    def weight_decls(spec: MixerSpec) -> dict[str, WeightDecl]:
        p = spec.params
        hidden, nh, hd, vd, rank = (int(p[k]) for k in ("hidden_size", "num_heads", "head_dim", "value_dim", "rank"))
        rot = int(p.get("rot_dim", 0))
        decls = {
            p["q_proj"]: WeightDecl((nh * (hd + rot), int(p["q_rank"]) if p.get("q_down") else hidden), ROLE_LINEAR),
            p["latent_proj"]: WeightDecl((rank + rot, hidden), ROLE_LINEAR),
            p["latent_norm"]: WeightDecl((rank,), ROLE_NORM),
            p["k_up"]: WeightDecl((nh * hd, rank), ROLE_LINEAR),
            p["v_up"]: WeightDecl((nh * vd, rank), ROLE_LINEAR),
            p["o_proj"]: WeightDecl((hidden, nh * vd), ROLE_LINEAR),
        }
        if p.get("q_down"):
            decls[p["q_down"]] = WeightDecl((int(p["q_rank"]), hidden), ROLE_LINEAR)
            decls[p["q_down_norm"]] = WeightDecl((int(p["q_rank"]),), ROLE_NORM)
        if p.get("gate"):
            decls[p["gate"]] = WeightDecl((nh * vd if p.get("gate_per_element") else nh, hidden), ROLE_LINEAR)
        if p.get("sinks"):
            decls[p["sinks"]] = WeightDecl((nh,), ROLE_ZERO)
        return decls

    def weights_read(self) -> list[torch.Tensor]:
        return [w for w in (self.w_in, self.w_q_up, self.q_norm, self.w_q_to_latent, self.w_latent_to_v, self.w_o,
                            self.latent_norm) if w is not None]

    @staticmethod
    def cache_spec(spec: MixerSpec) -> PagedCacheSpec:
        return PagedCacheSpec(1, key_dim=int(spec.params["rank"]) + int(spec.params.get("rot_dim", 0)), keys_only=True)

    @staticmethod
    def tile_requests(spec: MixerSpec) -> list[tuple[int, str]]:
        tokens = ops.attention_tile_tokens(int(spec.params["num_heads"]))
        wide = ops.paged_prefill_tile_tokens()
        return [(tokens, "all"), (tokens, "multi"), (tokens, "single"), (wide, "multi"), (wide, "all")]

    def forward(self, x: torch.Tensor, ctx: StepContext, call: LayerCall,
                out_dtype: torch.dtype | None = None) -> torch.Tensor:
        nh, hd, rank, rot, kw = self.nh, self.hd, self.rank, self.rot, self.kw
        table = ctx.block_table(call.cache)
        cache = ctx.caches[call.cache]
        projected = ops.linear(x, self.w_in, out_dtype=torch.float32)          # [T, queries | latent (+ rotated key) | gates]
        at = self.q_cols
        if self.q_rank:
            # The queries' own latent: its norm in float32, then the map to the heads (kept unrounded).
            q_latent_in = ops.sum_rms_norm(projected[:, :at], None, None, self.q_norm, self.eps, out_dtype=self.dtype)
            queries = ops.linear(q_latent_in, self.w_q_up, out_dtype=torch.float32)
        else:
            queries = projected[:, :at]
        if rot == 0:
            if call.writes_cache:
                # The latent's norm and its place in the pages, one kernel; nothing else is kept of a position.
                ops.qkv_pairs(projected[:, at: at + rank], 0, 1, rank, 0, None, None, self.latent_norm, self.eps,
                              None, 0, ctx.positions, ctx.token_row, cache, table, ctx.status, self.dtype)
            q_latent = ops.head_linear(queries, self.w_q_to_latent)             # [T, nh * rank], the model's type
        else:
            # Every head's unrotated part is carried into the latent space; its rotated part follows it as it
            # is (turned by the position), so that one dot product with the cached row gives both terms.
            q_latent = torch.empty((x.shape[0], nh * kw), dtype=self.dtype, device=x.device)
            ops.head_linear(queries, self.w_q_to_latent, x_head_stride=hd + rot, out=q_latent, out_head_stride=kw)
            ops.latent_rope(queries, nh, hd + rot, hd, q_latent, projected[:, at: at + kw], rank, rot, self.latent_norm,
                            self.eps, self.freqs, self.rope_mult, ctx.positions, ctx.token_row,
                            cache if call.writes_cache else None, table, ctx.status, self.dtype)
        attended = self.attend(q_latent, ctx, cache, table)
        gate = projected[:, at + kw:] if self.has_gate else None
        heads_out = ops.head_linear(attended, self.w_latent_to_v, gate=gate, x_head_stride=kw)     # [T, nh * vd]
        return ops.linear(heads_out, self.w_o, out_dtype=out_dtype)

    def attend(self, q: torch.Tensor, ctx: StepContext, cache: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
        """Attention of the latent-space queries [T, heads * (rank + rot)] over the cached rows: rows with one
        new token on the split-context kernel, rows with several on a tensor-core prompt kernel, where
        those take this shape and type (the prompt kernels take more widths than the split-context one, and
        then serve single tokens as well); whatever is left on the general kernel."""
        out = torch.empty_like(q)
        common = (self.nh, 1, self.kw, 0, self.scale, ctx.status)
        decode_done = self.fast_decode and ctx.num_decode_rows > 0
        if decode_done:
            ops.paged_decode(q, cache, table, ctx.decode_rows, ctx.row_q_start, ctx.row_ctx, ctx.max_decode_context,
                             *common, out=out, sinks=self.sinks, keys_only=True)
        prefill_done = False
        if self.fast_prefill and not self.fast_decode:
            # A row that the split-context kernel does not take (its width, or more than 16 heads): single tokens
            # go through the tensor-core prompt kernel too, as tiles of one token; two orders of magnitude
            # above the general kernel at contexts of thousands.
            tile_row, tile_q0 = ctx.tiles[(self.prefill_tile_tokens, "all")]
            if tile_row.numel() > 0:
                ops.paged_prefill(q, cache, table, tile_row, tile_q0, ctx.row_q_start, ctx.row_q_len, ctx.row_ctx,
                                  *common, out=out, sinks=self.sinks, keys_only=True)
            return out
        if self.fast_prefill:
            tile_row, tile_q0 = ctx.tiles[(self.prefill_tile_tokens, "multi")]
            prefill_done = True
            if tile_row.numel() > 0:
                ops.paged_prefill(q, cache, table, tile_row, tile_q0, ctx.row_q_start, ctx.row_q_len, ctx.row_ctx,
                                  *common, out=out, sinks=self.sinks, keys_only=True)
        if decode_done and prefill_done:
            return out
        which = "multi" if decode_done else ("single" if prefill_done else "all")
        tile_row, tile_q0 = ctx.tiles[(self.tile_tokens, which)]
        if tile_row.numel() > 0:
            ops.paged_attention(q, cache, table, tile_row, tile_q0, self.tile_tokens, ctx.row_q_start, ctx.row_q_len,
                                ctx.row_ctx, *common, out=out, sinks=self.sinks, shared_kv=True)
        return out


register_mixer("latent_attention", LatentAttention)
