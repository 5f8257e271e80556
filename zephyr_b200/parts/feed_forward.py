"""The dense gated feed-forward: down(act(gate(x)) * up(x)), no biases; act is SiLU (SwiGLU) unless
the spec's ``activation`` says "relu".

``activation`` "clamped_swish" is the bounded form, with biases on all three products where the spec names
them: g = min(gate(x), limit), u = clamp(up(x), -limit, limit), y = g * sigmoid(alpha * g) * (u + up_shift),
out = down(y).  Biases, bounds and the activation act on the product's unrounded float32 sums, inside the
product's kernel for few rows and for many (one pass over the float32 product otherwise); the down product's
bias joins the float32 sum into the stream.

Gate and up run as one product over one packed weight [2I, H], as the reference packs them at
load (src/layer/mlp.cpp:16-36); the reference puts all gate rows first, this part alternates blocks
of 8 gate rows and 8 up rows (see ``__init__``).  silu and the product are one float32
pass with a single rounding; the reference rounds between them (src/layer/activation.cu:31-33).
"""

from __future__ import annotations

from typing import Mapping

import torch

from ..config.errors import ConfigError
from ..config.spec import FeedForwardSpec
from ..kernels import ops
from ..weights.loader import ROLE_LINEAR, ROLE_ZERO, WeightDecl
from .base import FeedForward, register_feed_forward


class SwiGLU(FeedForward):
    graph_safe = True

    def __init__(self, spec: FeedForwardSpec, weights: Mapping[str, torch.Tensor], dtype: torch.dtype):
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.intermediate = int(p["intermediate_size"])
        self.activation = str(p.get("activation", "silu"))
        self.clamped = self.activation == "clamped_swish"
        if self.activation not in ops.ACTIVATIONS and not self.clamped:
            raise ConfigError(f"a gated feed-forward's activation is one of {sorted(ops.ACTIVATIONS) + ['clamped_swish']}")
        self.dtype = dtype
        self.limit = float(p.get("limit", 0.0))
        self.alpha = float(p.get("alpha", 1.0))
        self.up_shift = float(p.get("up_shift", 0.0))
        if self.clamped and not self.limit > 0.0:
            raise ConfigError("the bounded activation needs a positive limit")
        has_bias = [bool(p.get(k)) for k in ("gate_bias", "up_bias", "down_bias")]
        if any(has_bias) and not self.clamped:
            raise ConfigError("biases come with the bounded activation only")
        if has_bias[0] != has_bias[1]:
            raise ConfigError("gate and up carry biases together or not at all")
        gate, up = weights[p["gate_proj"]], weights[p["up_proj"]]
        # With I a multiple of 8 the rows alternate in blocks of 8 gate rows and their 8 up rows, the
        # order in which the decode kernel applies silu(gate) * up inside the product's epilogue.
        self.blocked = self.intermediate % 8 == 0
        if self.blocked:
            k = gate.shape[1]
            self.w_gate_up = torch.stack([gate.view(-1, 8, k), up.view(-1, 8, k)], dim=1).reshape(-1, k).contiguous()
        else:
            self.w_gate_up = torch.cat([gate, up], dim=0).contiguous()
        self.w_down = weights[p["down_proj"]]
        self.b_gate_up = self.b_down = None
        if has_bias[0]:
            b_gate, b_up = weights[p["gate_bias"]].float(), weights[p["up_bias"]].float()
            if self.blocked:
                self.b_gate_up = torch.stack([b_gate.view(-1, 8), b_up.view(-1, 8)], dim=1).reshape(-1).contiguous()
            else:
                self.b_gate_up = torch.cat([b_gate, b_up]).contiguous()
        if has_bias[2]:
            self.b_down = weights[p["down_bias"]].float().contiguous()

    @staticmethod
    def weight_decls(spec: FeedForwardSpec) -> dict[str, WeightDecl]:
        p = spec.params
        hidden, inter = int(p["hidden_size"]), int(p["intermediate_size"])
        decls = {
            p["gate_proj"]: WeightDecl((inter, hidden), ROLE_LINEAR),
            p["up_proj"]: WeightDecl((inter, hidden), ROLE_LINEAR),
            p["down_proj"]: WeightDecl((hidden, inter), ROLE_LINEAR),
        }
        for key, size in (("gate_bias", inter), ("up_bias", inter), ("down_bias", hidden)):
            if p.get(key):
                decls[p[key]] = WeightDecl((size,), ROLE_ZERO)
        return decls

    def as_gated_products(self) -> tuple[torch.Tensor, torch.Tensor] | None:
        # The chain of small products has SiLU in its epilogue; another activation keeps the layer off it.
        return (self.w_gate_up, self.w_down) if self.blocked and self.activation == "silu" else None

    def _bounded_hidden(self, x: torch.Tensor) -> torch.Tensor:
        # Biases, bounds and the gate where the products' float32 sums leave the tensor cores: a decode step's
        # few rows on the weight streamer, a prompt's many on tcgen05; what lies between, and float32, takes
        # the library's product and one pass over its unrounded result.
        if self.blocked and x.dtype == torch.bfloat16:
            bounded = ops.BoundedGate(self.b_gate_up, self.limit, self.alpha, self.up_shift)
            if x.shape[0] <= ops.SMALL_GEMM_ROWS and ops.gemm_small_supported(x, self.w_gate_up):
                return ops.gemm_small(x, self.w_gate_up, swiglu=True, bounded=bounded)
            if ((x.shape[0] >= ops.GEMM_TC_MIN_ROWS or not ops.USE_LIBRARY_PRODUCTS)
                    and ops.gemm_tc_supported(x, self.w_gate_up, swiglu=True)):
                return ops.gemm_tc(x, self.w_gate_up, swiglu=True, bounded=bounded)
        product = ops.linear(x, self.w_gate_up, out_dtype=torch.float32)
        return ops.clamped_gate(product, self.b_gate_up, self.limit, self.alpha, self.up_shift, self.dtype, blocked=self.blocked)

    def forward_summands(self, x: torch.Tensor) -> tuple[torch.Tensor, ...]:
        if self.clamped and self.b_down is not None:      # the last bias joins the sum into the stream, in float32
            return ops.linear(self._bounded_hidden(x), self.w_down), self.b_down
        return (self.forward(x),)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.clamped:
            hidden = self._bounded_hidden(x)
            if self.b_down is None:
                return ops.linear(hidden, self.w_down)
            return ops.add_bias(ops.linear(hidden, self.w_down, out_dtype=torch.float32), self.b_down)
        act = self.activation
        if self.blocked and x.shape[0] <= ops.SMALL_GEMM_ROWS and ops.gemm_small_supported(x, self.w_gate_up):
            hidden = ops.gemm_small(x, self.w_gate_up, swiglu=True, act=act)       # product and activation in one kernel
        elif (self.blocked and (x.shape[0] >= ops.GEMM_TC_MIN_ROWS or not ops.USE_LIBRARY_PRODUCTS)
              and ops.gemm_tc_supported(x, self.w_gate_up, swiglu=True)):
            hidden = ops.gemm_tc(x, self.w_gate_up, swiglu=True, act=act)          # the same for a prompt's many rows, on tcgen05
        else:
            hidden = ops.silu_mul(ops.linear(x, self.w_gate_up), blocked=self.blocked, act=act)
        return ops.linear(hidden, self.w_down)


register_feed_forward("swiglu", SwiGLU)
register_feed_forward("gated", SwiGLU)        # the same part under the name that fits any activation
