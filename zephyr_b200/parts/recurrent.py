"""Mixers that carry a state of fixed size per request instead of a growing cache, and a mixer that
runs several mixers side by side.

Both recurrent mixers are the same recurrence per head,

    S_t = diag(a_t) S_{t-1} + k_t v_t^T        (S: key channels x value channels, float32)
    o_t = S_t^T q_t

with different ways to the decay a_t, and live in the request's state slot
(``StateCacheSpec``): the slot is zeroed when a request is admitted, read at the start of a step's
portion and written back at its end, so prompts may be cut anywhere.

``gla`` (gated linear attention): q = Wq h / sqrt(dim), k = Wk h, v = Wv h; a decay per key channel
a = sigmoid(z)^(1/tau) with z = Wa2 (Wa1 h) + b, a low-rank projection whose inner size is the
checkpoint's; each head's o is RMS-normed over its value channels with one scale vector shared by the
heads, the heads are joined, multiplied by silu(Wg h) and projected by Wo.

``mamba2`` (the state-space form of Mamba-2): Win h = [z | x | B | C | dt]; x, B and C pass a causal
convolution over a few taps per channel and SiLU (its last taps - 1 inputs belong to the state too);
dt = softplus(dt + dt_bias) without a clamp; per head a = exp(-exp(A_log) dt), k = dt B, q = C of the
head's group, v = x, and o += D x; o joined over heads times silu(z), then RMS-normed in
``norm_groups`` equal parts (the gate comes before the norm), times a scale per column, then Wo.

``gated_delta`` (the gated delta rule): q = Wq h and k = Wk h with ``qk_heads`` heads of ``key_dim``, v = Wv h
with ``heads`` heads of ``value_dim``; each passes a causal convolution over a few taps per channel (no bias)
and SiLU; q and k are made unit vectors per head, x / sqrt(sum(x^2) + 1e-6), q also times key_dim^(-1/2);
beta = sigmoid(Wb h) and g = exp(-exp(A_log) softplus(Wa h + dt_bias)) per head; per head
S <- g S, u = beta (v - S^T k), S <- S + k u^T, o = S^T q; each head's o is RMS-normed over its value
channels with one scale vector shared by the heads, the heads are joined, multiplied by silu(Wg h) and
projected by Wo.  The state and the convolution's last taps - 1 inputs live in the request's slot.

``parallel``: the sum of several mixers over the same input, each with a weight.  Every branch keeps
its own store; the call's first cache id goes to the first branch and its ``extra_caches`` to the
others.

Decays, their logarithms, softplus, step sizes, the state and the unit norms are float32 inside the
kernels (csrc/recurrent.cu); projections and the convolution's output have the model's type.
"""

from __future__ import annotations

import dataclasses
from typing import Mapping

import torch

from ..cache import StateCacheSpec
from ..config.errors import ConfigError
from ..config.spec import LayerCall, MixerSpec
from ..kernels import ops
from ..weights.loader import ROLE_LINEAR, ROLE_NORM, ROLE_ZERO, WeightDecl
from .base import MIXERS, Mixer, StepContext, lookup, register_mixer

MAX_KEY_CHANNELS = 256        # what the scan kernel takes per head (csrc/recurrent.cu: 16 warps of 16 channels)


def _vector(weights: Mapping[str, torch.Tensor], name: str) -> torch.Tensor:
    return weights[name].float().contiguous()


class GatedLinearAttention(Mixer):
    graph_safe = True
    takes_out_dtype = True

    def __init__(self, spec: MixerSpec, weights: Mapping[str, torch.Tensor], dtype: torch.dtype,
                 device: torch.device | str):
        p = spec.params
        self.hidden, self.heads = int(p["hidden_size"]), int(p["heads"])
        self.dim, self.vdim = int(p["key_dim"]), int(p["value_dim"])
        self.tau, self.eps = float(p["tau"]), float(p["norm_eps"])
        _check_sizes(self.heads, self.dim, self.vdim)
        if not self.tau > 0.0:
            raise ConfigError("the decay's temperature must be positive")
        hd, hv = self.heads * self.dim, self.heads * self.vdim
        self.rank = weights[p["a1"]].shape[0]
        if weights[p["a2"]].shape != (hd, self.rank):
            raise ConfigError("the two factors of the decay projection do not fit each other")
        # One product for everything that reads the input: q | k | v | gate | the decay's inner factor.
        self.w_in = torch.cat([weights[p[n]] for n in ("q", "k", "v", "g", "a1")], dim=0).contiguous()
        self.cuts = (0, hd, 2 * hd, 2 * hd + hv, 2 * hd + 2 * hv, 2 * hd + 2 * hv + self.rank)
        self.w_a2 = weights[p["a2"]]
        self.a2_bias = _vector(weights, p["a2_bias"])
        self.norm = _vector(weights, p["norm"])
        self.w_o = weights[p["o"]]

    @staticmethod
    def weight_decls(spec: MixerSpec) -> dict[str, WeightDecl]:
        p = spec.params
        hidden, hd, hv = int(p["hidden_size"]), int(p["heads"]) * int(p["key_dim"]), int(p["heads"]) * int(p["value_dim"])
        rank = int(p["decay_rank"]) if p.get("decay_rank") else -1      # -1: the checkpoint gives it
        return {
            p["q"]: WeightDecl((hd, hidden), ROLE_LINEAR), p["k"]: WeightDecl((hd, hidden), ROLE_LINEAR),
            p["v"]: WeightDecl((hv, hidden), ROLE_LINEAR), p["g"]: WeightDecl((hv, hidden), ROLE_LINEAR),
            p["o"]: WeightDecl((hidden, hv), ROLE_LINEAR), p["norm"]: WeightDecl((int(p["value_dim"]),), ROLE_NORM),
            p["a1"]: WeightDecl((rank, hidden), ROLE_LINEAR), p["a2"]: WeightDecl((hd, rank), ROLE_LINEAR),
            p["a2_bias"]: WeightDecl((hd,), ROLE_ZERO),
        }

    def weights_read(self) -> list[torch.Tensor]:
        return [self.w_in, self.w_a2, self.w_o, self.a2_bias, self.norm]

    @staticmethod
    def cache_spec(spec: MixerSpec) -> StateCacheSpec:
        p = spec.params
        return StateCacheSpec(shape=(int(p["heads"]) * int(p["key_dim"]) * int(p["value_dim"]),), dtype="float32")

    def forward(self, x: torch.Tensor, ctx: StepContext, call: LayerCall,
                out_dtype: torch.dtype | None = None) -> torch.Tensor:
        c = self.cuts
        projected = ops.linear(x, self.w_in)
        q, k, v, gate, inner = (projected[:, c[i]:c[i + 1]] for i in range(5))
        logits = ops.linear(inner, self.w_a2, out_dtype=torch.float32)
        o = ops.decayed_state_scan("gated", q, k, v, self.heads, self.dim, self.vdim, ctx.caches[call.cache],
                                   ctx.state_slots, ctx.row_q_start, ctx.row_q_len, ctx.status, decay_logits=logits,
                                   decay_bias=self.a2_bias, inv_tau=1.0 / self.tau, q_scale=self.dim ** -0.5,
                                   write_state=call.writes_cache)
        normed = ops.gated_group_rms_norm(o, gate, self.norm, self.vdim, self.eps, gate_first=False)
        return ops.linear(normed, self.w_o, out_dtype=out_dtype)


class Mamba2(Mixer):
    graph_safe = True
    takes_out_dtype = True

    def __init__(self, spec: MixerSpec, weights: Mapping[str, torch.Tensor], dtype: torch.dtype,
                 device: torch.device | str):
        p = spec.params
        self.hidden, self.heads, self.vdim = int(p["hidden_size"]), int(p["heads"]), int(p["value_dim"])
        self.state, self.groups, self.taps = int(p["state"]), int(p["groups"]), int(p["conv"])
        self.norm_groups, self.eps = int(p["norm_groups"]), float(p["norm_eps"])
        _check_sizes(self.heads, self.state, self.vdim)
        self.inner = self.heads * self.vdim
        if self.groups <= 0 or self.heads % self.groups != 0:
            raise ConfigError("the heads must divide evenly over the groups of B and C")
        if self.norm_groups <= 0 or self.inner % self.norm_groups != 0:
            raise ConfigError("the gated norm's parts must divide the inner width evenly")
        if not 1 <= self.taps <= ops.CONV_MAX_TAPS:
            raise ConfigError(f"the convolution takes 1 to {ops.CONV_MAX_TAPS} taps")
        self.channels = self.inner + 2 * self.groups * self.state
        self.w_in = weights[p["in"]]
        self.conv_w = weights[p["conv_weight"]].float().contiguous()
        self.conv_b = _vector(weights, p["conv_bias"])
        self.dt_bias, self.a_log, self.skip = (_vector(weights, p[n]) for n in ("dt_bias", "a_log", "skip"))
        self.norm = _vector(weights, p["norm"])
        self.w_o = weights[p["o"]]
        self.scan_floats = self.heads * self.state * self.vdim

    @staticmethod
    def _sizes(p) -> tuple[int, int, int]:
        inner = int(p["heads"]) * int(p["value_dim"])
        channels = inner + 2 * int(p["groups"]) * int(p["state"])
        return inner, channels, inner + channels + int(p["heads"])

    @staticmethod
    def weight_decls(spec: MixerSpec) -> dict[str, WeightDecl]:
        p = spec.params
        hidden, heads = int(p["hidden_size"]), int(p["heads"])
        inner, channels, projected = Mamba2._sizes(p)
        return {
            p["in"]: WeightDecl((projected, hidden), ROLE_LINEAR),
            p["conv_weight"]: WeightDecl((channels, int(p["conv"])), ROLE_LINEAR),
            p["conv_bias"]: WeightDecl((channels,), ROLE_ZERO),
            p["dt_bias"]: WeightDecl((heads,), ROLE_ZERO), p["a_log"]: WeightDecl((heads,), ROLE_ZERO),
            p["skip"]: WeightDecl((heads,), ROLE_NORM), p["norm"]: WeightDecl((inner,), ROLE_NORM),
            p["o"]: WeightDecl((hidden, inner), ROLE_LINEAR),
        }

    def weights_read(self) -> list[torch.Tensor]:
        return [self.w_in, self.w_o, self.conv_w, self.conv_b, self.norm]

    @staticmethod
    def cache_spec(spec: MixerSpec) -> StateCacheSpec:
        """The recurrence's state [heads, state, value_dim] and behind it the convolution's last
        taps - 1 inputs [taps - 1, channels], as one float32 vector."""
        p = spec.params
        _, channels, _ = Mamba2._sizes(p)
        scan = int(p["heads"]) * int(p["state"]) * int(p["value_dim"])
        return StateCacheSpec(shape=(scan + (int(p["conv"]) - 1) * channels,), dtype="float32")

    def forward(self, x: torch.Tensor, ctx: StepContext, call: LayerCall,
                out_dtype: torch.dtype | None = None) -> torch.Tensor:
        inner, gn = self.inner, self.groups * self.state
        store = ctx.caches[call.cache]
        projected = ops.linear(x, self.w_in)             # z | x | B | C | dt
        mixed = ops.causal_conv_silu(projected[:, inner:], self.channels, self.conv_w, self.conv_b,
                                     store[:, self.scan_floats:], ctx.state_slots, ctx.row_q_start, ctx.row_q_len,
                                     ctx.token_row, ctx.status, write_state=call.writes_cache)
        o = ops.decayed_state_scan("state_space", mixed[:, inner + gn:], mixed[:, inner:inner + gn], mixed[:, :inner],
                                   self.heads, self.state, self.vdim, store[:, :self.scan_floats], ctx.state_slots,
                                   ctx.row_q_start, ctx.row_q_len, ctx.status, dt=projected[:, inner + self.channels:],
                                   dt_bias=self.dt_bias, a_log=self.a_log, skip=self.skip,
                                   heads_per_group=self.heads // self.groups, write_state=call.writes_cache)
        normed = ops.gated_group_rms_norm(o, projected[:, :inner], self.norm, inner // self.norm_groups, self.eps,
                                          gate_first=True)
        return ops.linear(normed, self.w_o, out_dtype=out_dtype)


class GatedDeltaRule(Mixer):
    graph_safe = True
    takes_out_dtype = True

    UNIT_EPS = 1e-6      # inside the root of the unit norms of q and k: the design fixes it

    def __init__(self, spec: MixerSpec, weights: Mapping[str, torch.Tensor], dtype: torch.dtype,
                 device: torch.device | str):
        p = spec.params
        self.hidden, self.heads, self.qk_heads = int(p["hidden_size"]), int(p["heads"]), int(p["qk_heads"])
        self.dim, self.vdim, self.taps = int(p["key_dim"]), int(p["value_dim"]), int(p["conv"])
        self.eps = float(p["norm_eps"])
        if min(self.heads, self.qk_heads, self.dim, self.vdim) <= 0 or self.heads % self.qk_heads != 0:
            raise ConfigError("the delta rule needs positive sizes and heads that are a multiple of the q/k heads")
        if self.dim > ops.delta_max_channels():
            raise ConfigError(f"the delta rule takes up to {ops.delta_max_channels()} key channels per head, not {self.dim}")
        if not 1 <= self.taps <= ops.CONV_MAX_TAPS:
            raise ConfigError(f"the convolution takes 1 to {ops.CONV_MAX_TAPS} taps")
        qk, hv = self.qk_heads * self.dim, self.heads * self.vdim
        self.channels = 2 * qk + hv
        # One product with float32 sums out for everything on the way into the recurrence: q | k | v | b | a
        # (a unit norm of q and k divides by their length, so where q . k is small a rounding of the
        # projection or of the convolution's output to bfloat16 would turn the normed read-out by a large
        # angle); the output gate comes out of a second product, in the model's type.
        self.w_in = torch.cat([weights[p[n]] for n in ("q", "k", "v", "b", "a")], dim=0).contiguous()
        self.w_g = weights[p["g"]]
        self.conv_w = torch.cat([weights[p[n]] for n in ("q_conv", "k_conv", "v_conv")], dim=0).float().contiguous()
        self.conv_b = torch.zeros(self.channels, dtype=torch.float32, device=self.conv_w.device)
        self.a_log, self.dt_bias = _vector(weights, p["a_log"]), _vector(weights, p["dt_bias"])
        self.norm = _vector(weights, p["norm"])
        self.w_o = weights[p["o"]]
        self.cuts = (0, qk, 2 * qk, 2 * qk + hv)
        self.scan_floats = self.heads * self.dim * self.vdim

    @staticmethod
    def weight_decls(spec: MixerSpec) -> dict[str, WeightDecl]:
        p = spec.params
        hidden, heads, taps = int(p["hidden_size"]), int(p["heads"]), int(p["conv"])
        qk, hv = int(p["qk_heads"]) * int(p["key_dim"]), heads * int(p["value_dim"])
        return {
            p["q"]: WeightDecl((qk, hidden), ROLE_LINEAR), p["k"]: WeightDecl((qk, hidden), ROLE_LINEAR),
            p["v"]: WeightDecl((hv, hidden), ROLE_LINEAR), p["g"]: WeightDecl((hv, hidden), ROLE_LINEAR),
            p["q_conv"]: WeightDecl((qk, taps), ROLE_LINEAR), p["k_conv"]: WeightDecl((qk, taps), ROLE_LINEAR),
            p["v_conv"]: WeightDecl((hv, taps), ROLE_LINEAR),
            p["b"]: WeightDecl((heads, hidden), ROLE_LINEAR), p["a"]: WeightDecl((heads, hidden), ROLE_LINEAR),
            p["a_log"]: WeightDecl((heads,), ROLE_ZERO), p["dt_bias"]: WeightDecl((heads,), ROLE_ZERO),
            p["norm"]: WeightDecl((int(p["value_dim"]),), ROLE_NORM), p["o"]: WeightDecl((hidden, hv), ROLE_LINEAR),
        }

    def weights_read(self) -> list[torch.Tensor]:
        return [self.w_in, self.w_g, self.w_o, self.conv_w, self.norm]

    @staticmethod
    def cache_spec(spec: MixerSpec) -> StateCacheSpec:
        """The rule's state [heads, value_dim, key_dim] and behind it the convolution's last taps - 1 inputs
        [taps - 1, channels], as one float32 vector."""
        p = spec.params
        channels = 2 * int(p["qk_heads"]) * int(p["key_dim"]) + int(p["heads"]) * int(p["value_dim"])
        scan = int(p["heads"]) * int(p["key_dim"]) * int(p["value_dim"])
        return StateCacheSpec(shape=(scan + (int(p["conv"]) - 1) * channels,), dtype="float32")

    def forward(self, x: torch.Tensor, ctx: StepContext, call: LayerCall,
                out_dtype: torch.dtype | None = None) -> torch.Tensor:
        c, store = self.cuts, ctx.caches[call.cache]
        projected = ops.linear(x, self.w_in, out_dtype=torch.float32)      # q | k | v | b | a
        steps = projected[:, c[3]:]
        mixed = ops.causal_conv_silu(projected, self.channels, self.conv_w, self.conv_b, store[:, self.scan_floats:],
                                     ctx.state_slots, ctx.row_q_start, ctx.row_q_len, ctx.token_row, ctx.status,
                                     write_state=call.writes_cache)
        o = ops.delta_rule(mixed[:, c[0]:c[1]], mixed[:, c[1]:c[2]], mixed[:, c[2]:c[3]], steps[:, :self.heads],
                           steps[:, self.heads:], self.a_log, self.dt_bias, self.heads, self.qk_heads, self.dim,
                           self.vdim, store[:, :self.scan_floats], ctx.state_slots, ctx.row_q_start, ctx.row_q_len,
                           ctx.status, q_scale=self.dim ** -0.5, unit_eps=self.UNIT_EPS, write_state=call.writes_cache)
        normed = ops.gated_group_rms_norm(o, ops.linear(x, self.w_g), self.norm, self.vdim, self.eps, gate_first=False)
        return ops.linear(normed, self.w_o, out_dtype=out_dtype)


def _check_sizes(heads: int, key_channels: int, value_channels: int) -> None:
    if heads <= 0 or key_channels <= 0 or value_channels <= 0:
        raise ConfigError("a recurrent mixer needs positive head counts and widths")
    if key_channels > MAX_KEY_CHANNELS:
        raise ConfigError(f"the recurrence takes up to {MAX_KEY_CHANNELS} key channels per head, not {key_channels}")


class ParallelMixers(Mixer):
    """y = sum_i scale_i * mixer_i(x): ``params["branches"]`` lists (MixerSpec, scale) pairs.  The sum is
    formed from the branches' float32 outputs with one rounding."""

    takes_out_dtype = True

    def __init__(self, spec: MixerSpec, weights: Mapping[str, torch.Tensor], dtype: torch.dtype,
                 device: torch.device | str):
        branches = spec.params["branches"]
        if len(branches) != 2:
            raise ConfigError("mixers run side by side in pairs")
        self.dtype = dtype
        self.branches = [lookup(MIXERS, "mixer", sub.kind)(sub, weights, dtype, device) for sub, _ in branches]
        self.scales = [float(scale) for _, scale in branches]
        self.graph_safe = all(getattr(branch, "graph_safe", False) for branch in self.branches)
        positions = [getattr(branch, "position", None) for branch in self.branches]
        self.position = next((p for p in positions if p is not None), None)
        self.stores = [_store_count(sub) for sub, _ in branches]

    @staticmethod
    def weight_decls(spec: MixerSpec) -> dict[str, WeightDecl]:
        decls: dict[str, WeightDecl] = {}
        for sub, _ in spec.params["branches"]:
            decls.update(lookup(MIXERS, "mixer", sub.kind).weight_decls(sub))
        return decls

    def weights_read(self) -> list[torch.Tensor]:
        return [tensor for branch in self.branches for tensor in branch.weights_read()]

    @staticmethod
    def cache_spec(spec: MixerSpec) -> tuple:
        needs = []
        for sub, _ in spec.params["branches"]:
            need = lookup(MIXERS, "mixer", sub.kind).cache_spec(sub)
            needs += list(need) if isinstance(need, tuple) else [need]
        return tuple(needs)

    @staticmethod
    def tile_requests(spec: MixerSpec) -> list[tuple[int, str]]:
        wanted: list[tuple[int, str]] = []
        for sub, _ in spec.params["branches"]:
            for request in lookup(MIXERS, "mixer", sub.kind).tile_requests(sub):
                if request not in wanted:
                    wanted.append(request)
        return wanted

    def forward(self, x: torch.Tensor, ctx: StepContext, call: LayerCall,
                out_dtype: torch.dtype | None = None) -> torch.Tensor:
        outputs, at = [], 0
        for branch, count in zip(self.branches, self.stores):
            ids = call.caches[at:at + count]
            at += count
            own = dataclasses.replace(call, cache=ids[0], extra_caches=tuple(ids[1:]))
            if getattr(branch, "takes_out_dtype", False):
                outputs.append(branch.forward(x, ctx, own, out_dtype=torch.float32))
            else:
                outputs.append(branch.forward(x, ctx, own))
        if outputs[0].dtype != outputs[1].dtype:
            outputs = [o.float() for o in outputs]
        return ops.scaled_sum(outputs[0], outputs[1], self.scales[0], self.scales[1], out_dtype=out_dtype or self.dtype)


def _store_count(sub: MixerSpec) -> int:
    need = lookup(MIXERS, "mixer", sub.kind).cache_spec(sub)
    return len(need) if isinstance(need, tuple) else 1


register_mixer("gated_delta", GatedDeltaRule)
register_mixer("gla", GatedLinearAttention)
register_mixer("mamba2", Mamba2)
register_mixer("parallel", ParallelMixers)
