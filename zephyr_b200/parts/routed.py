"""A routed feed-forward (mixture of experts) with token choice.

    z = Wr x                                   router logits, float32
    s = softmax(z)                             over ALL router outputs
    choice = s + correction                    a learned shift that moves the choice and nothing else
    the ``top`` outputs with the largest choice are taken; each counts with its s (not renormalised)
    out = sum over the taken outputs e of  s_e * expert_e(x)

Further forms, each named by the spec: ``scores`` "sigmoid" (s = sigmoid(z), every output on its own);
``groups`` = {count, keep, top}: the outputs form ``count`` equal runs of neighbours, a run's mark is the sum of
its ``top`` largest choice values, and only outputs of the ``keep`` runs with the largest marks can be taken;
``weight_scale``: a multiplier on every weight; ``router_bias``: a bias b on the logits, z = Wr x + b;
``scores`` "top_softmax": the ``top`` largest logits are taken, and their outputs count with the softmax over
the taken logits only.

The first ``experts`` router outputs are gated feed-forwards, expert_e(x) = down_e(act(gate_e x) * (up_e x)),
without biases; the last ``identity`` outputs are identity experts, expert(x) = x, which have no tensors.
Every expert's matrices are stacked at load ([experts, ff, hidden] and [experts, hidden, ff]) so that
one launch serves all experts (``ops.routed_experts``: the tokens sorted by expert on the device, two
products over that order, one weighted sum in float32).  Nothing of the routing comes back to the host,
so a step with this part can be captured and replayed.
"""

from __future__ import annotations

from typing import Mapping

import torch

from ..config.errors import ConfigError
from ..config.spec import FeedForwardSpec
from ..kernels import ops
from ..weights.loader import ROLE_LINEAR, ROLE_ZERO, WeightDecl
from .base import FeedForward, register_feed_forward


class RoutedFeedForward(FeedForward):
    graph_safe = True

    def __init__(self, spec: FeedForwardSpec, weights: Mapping[str, torch.Tensor], dtype: torch.dtype):
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.intermediate = int(p["intermediate_size"])
        self.experts, self.identity, self.top = int(p["experts"]), int(p.get("identity", 0)), int(p["top"])
        self.activation = str(p.get("activation", "silu"))
        outputs = self.experts + self.identity
        if self.experts <= 0 or self.identity < 0 or not 0 < self.top <= outputs:
            raise ConfigError("a routed feed-forward needs experts, and takes between one and all of its outputs")
        if self.activation not in ops.ACTIVATIONS:
            raise ConfigError(f"an expert's activation is one of {sorted(ops.ACTIVATIONS)}")
        self.scores = str(p.get("scores", "softmax"))
        if self.scores not in ops.ROUTE_SCORES:
            raise ConfigError(f"router scores are one of {sorted(ops.ROUTE_SCORES)}")
        self.weight_scale = float(p.get("weight_scale", 1.0))
        self.groups = None
        if p.get("groups"):
            g = p["groups"]
            count, keep, group_top = int(g["count"]), int(g["keep"]), int(g.get("top", 2))
            if (count <= 0 or outputs % count != 0 or not 0 < keep <= count or group_top <= 0
                    or keep * (outputs // count) < self.top):
                raise ConfigError("router groups must divide the outputs evenly, and the kept groups must hold the choices")
            if count > 1:
                self.groups = (count, keep, group_top)
        self.w_router = weights[p["router"]]
        self.correction = weights[p["correction"]].float().contiguous() if p.get("correction") else None
        self.router_bias = weights[p["router_bias"]].float().contiguous() if p.get("router_bias") else None
        if outputs > ops.route_max_outputs():
            raise ConfigError(f"the routing kernel takes up to {ops.route_max_outputs()} router outputs, not {outputs}")
        names = p["expert_names"]
        self.w_gate = torch.stack([weights[gate] for gate, _, _ in names]).contiguous()
        self.w_up = torch.stack([weights[up] for _, up, _ in names]).contiguous()
        self.w_down = torch.stack([weights[down] for _, _, down in names]).contiguous()
        if self.intermediate % 8 == 0:
            # Blocks of 8 gate rows and their 8 up rows: the layout whose product applies the activation
            # where the sums leave the tensor cores.  The separate matrices are not kept beside it.
            self.w_gate, self.w_up = ops.interleave_gate_up(self.w_gate, self.w_up), None

    @staticmethod
    def weight_decls(spec: FeedForwardSpec) -> dict[str, WeightDecl]:
        p = spec.params
        hidden, inter = int(p["hidden_size"]), int(p["intermediate_size"])
        outputs = int(p["experts"]) + int(p.get("identity", 0))
        if len(p["expert_names"]) != int(p["experts"]):
            raise ConfigError("one (gate, up, down) name triple per expert")
        decls = {p["router"]: WeightDecl((outputs, hidden), ROLE_LINEAR)}
        if p.get("correction"):
            decls[p["correction"]] = WeightDecl((outputs,), ROLE_ZERO)
        if p.get("router_bias"):
            decls[p["router_bias"]] = WeightDecl((outputs,), ROLE_ZERO)
        for gate, up, down in p["expert_names"]:
            decls[gate] = WeightDecl((inter, hidden), ROLE_LINEAR)
            decls[up] = WeightDecl((inter, hidden), ROLE_LINEAR)
            decls[down] = WeightDecl((hidden, inter), ROLE_LINEAR)
        return decls

    def weights_read(self) -> list[torch.Tensor]:
        return [w for w in (self.w_router, self.w_gate, self.w_up, self.w_down) if w is not None]

    def route(self, x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        logits = ops.linear(x, self.w_router, out_dtype=torch.float32)
        return ops.route(logits, self.correction, self.top, self.scores, self.groups, self.weight_scale,
                         logit_bias=self.router_bias)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        ids, weights = self.route(x)
        return ops.routed_experts(x, ids, weights, self.w_gate, self.w_up, self.w_down, act=self.activation)


register_feed_forward("routed", RoutedFeedForward)
