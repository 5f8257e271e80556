"""What lies before the first layer and after the last one, as parts.

``embedding``: h[t, :] = E[id[t], :] (reference: src/layer/embedding.cpp:17-31,
src/model/causal_lm/qwen3.cpp:122-123,169), times ``scale`` where the spec gives one (float32 streams).

``pair_embedding``: h[t, :] = E[id[t], :] + B[r[t], :] on a float32 stream, where B is a second table of
``buckets`` + 1 rows and r[t] = (id[t-1] * mul_prev + id[t] * mul_cur) mod buckets hashes the token with the
one before it; a sequence's first token takes B's last row.  The token before a step's first one is kept
per request in a state slot (one int32), so a prompt may be cut anywhere.

``norm_head``: the final norm and the vocabulary projection without bias, for the wanted tokens only
(reference: src/model/causal_lm/qwen3.cpp:133-136,173-180).  The norm is row-wise, so it runs on
the wanted rows alone (the reference norms every token and selects after); the logits come out in
float32 whatever the model's type (the reference stores them in the model's type).  A tied head
names the embedding's tensor and so reads the very same memory.  ``logit_scale``: a multiplier on the
float32 logits.
"""

from __future__ import annotations

from typing import Mapping

import torch

from ..config.errors import ConfigError
from ..cache import StateCacheSpec
from ..config.spec import InputSpec, OutputSpec
from ..kernels import ops
from ..weights.loader import ROLE_EMBEDDING, ROLE_LINEAR, WeightDecl
from .base import NORMS, InputPart, OutputPart, ResidualStream, StepContext, lookup, register_input, register_output


class Embedding(InputPart):
    graph_safe = True

    def __init__(self, spec: InputSpec, weights: Mapping[str, torch.Tensor], dtype: torch.dtype):
        self.table = weights[spec.params["weight"]]
        # A model whose residual stream is float32 takes the table's rows as float32 from the start.
        self.float32_stream = bool(spec.params.get("float32_stream", False))
        self.scale = float(spec.params.get("scale", 1.0))
        # For models whose first part reads the stream itself: hand on its rounding with it.
        self.rounded_copy = bool(spec.params.get("rounded_copy", False))
        if self.scale != 1.0 and not self.float32_stream:
            raise ConfigError("an embedding multiplier comes with a float32 stream")

    @staticmethod
    def weight_decls(spec: InputSpec) -> dict[str, WeightDecl]:
        p = spec.params
        return {p["weight"]: WeightDecl((int(p["vocab_size"]), int(p["hidden_size"])), ROLE_EMBEDDING)}

    def weights_read(self) -> list[torch.Tensor]:
        return []          # a step gathers a few rows of the table; it does not stream it

    def forward(self, ctx: StepContext) -> torch.Tensor:
        if self.float32_stream and (self.scale != 1.0 or self.rounded_copy):
            # The stream, and its rounding for the first part that reads the stream itself.
            if self.table.dtype == torch.float32:
                return ops.embedding_f32(self.table, ctx.token_ids, ctx.status, self.scale)
            hidden, rounded = ops.embedding_f32(self.table, ctx.token_ids, ctx.status, self.scale, rounded=True)
            return ResidualStream(hidden, rounded=rounded)
        if self.float32_stream:
            return ops.embedding_f32(self.table, ctx.token_ids, ctx.status)
        return ops.embedding(self.table, ctx.token_ids, ctx.status)


class PairEmbedding(InputPart):
    graph_safe = True

    def __init__(self, spec: InputSpec, weights: Mapping[str, torch.Tensor], dtype: torch.dtype):
        p = spec.params
        self.table = weights[p["weight"]]
        self.pair_table = weights[p["pair_weight"]]
        self.buckets = int(p["buckets"])
        self.mul_prev, self.mul_cur = int(p["mul_prev"]), int(p["mul_cur"])
        if self.buckets <= 0 or self.mul_prev < 0 or self.mul_cur < 0:
            raise ConfigError("the pair hash needs a positive number of buckets and non-negative multipliers")
        if (self.mul_prev + self.mul_cur) * int(p["vocab_size"]) >= 2 ** 62:
            raise ConfigError("the pair hash's multipliers are too large for 64-bit arithmetic")

    @staticmethod
    def weight_decls(spec: InputSpec) -> dict[str, WeightDecl]:
        p = spec.params
        return {p["weight"]: WeightDecl((int(p["vocab_size"]), int(p["hidden_size"])), ROLE_EMBEDDING),
                p["pair_weight"]: WeightDecl((int(p["buckets"]) + 1, int(p["hidden_size"])), ROLE_EMBEDDING)}

    @staticmethod
    def cache_spec(spec: InputSpec) -> StateCacheSpec:
        return StateCacheSpec((1,), "int32")          # the request's last token

    def weights_read(self) -> list[torch.Tensor]:
        return []          # a step gathers a few rows of the tables

    def forward(self, ctx: StepContext) -> ResidualStream:
        last_token = ctx.caches[self.cache_id].view(-1)
        return ResidualStream(ops.pair_embedding(self.table, self.pair_table, ctx.token_ids, ctx.positions,
                                                 ctx.token_row, ctx.row_q_start, ctx.row_q_len, ctx.state_slots,
                                                 last_token, self.mul_prev, self.mul_cur, ctx.status))


class NormHead(OutputPart):
    graph_safe = True

    def __init__(self, spec: OutputSpec, weights: Mapping[str, torch.Tensor], dtype: torch.dtype):
        p = spec.params
        self.vocab_size = int(p["vocab_size"])
        self.logit_scale = float(p.get("logit_scale", 1.0))
        self.norm = lookup(NORMS, "norm", p["norm"].kind)(p["norm"], weights, dtype)
        self.weight = weights[p["weight"]]

    @staticmethod
    def weight_decls(spec: OutputSpec) -> dict[str, WeightDecl]:
        p = spec.params
        decls = dict(lookup(NORMS, "norm", p["norm"].kind).weight_decls(p["norm"]))
        # A name the input part declares too (a tied head) keeps the role it was given first.
        decls[p["weight"]] = WeightDecl((int(p["vocab_size"]), int(p["hidden_size"])), ROLE_LINEAR)
        return decls

    def weights_read(self) -> list[torch.Tensor]:
        return [self.weight, *self.norm.weights_read()]

    def forward(self, stream: ResidualStream, ctx: StepContext) -> torch.Tensor:
        wanted = ctx.logit_tokens
        if wanted.numel() == 0:
            return torch.empty((0, self.vocab_size), dtype=torch.float32, device=stream.hidden.device)
        if stream.deferred is not None:
            stream.flush()
        rows = ops.gather_rows(stream.hidden, wanted, ctx.status)
        if isinstance(stream.pending, tuple):       # summands that are added to each other first, then to the stream
            normed = self.norm.sum_forward(rows, tuple(ops.gather_rows(part, wanted, ctx.status) if part.dim() == 2 else part
                                                       for part in stream.pending))
        elif stream.pending is not None:
            normed = self.norm.add_forward(rows, ops.gather_rows(stream.pending, wanted, ctx.status))
        else:
            normed = self.norm.forward(rows)
        logits = ops.linear(normed, self.weight, out_dtype=torch.float32)
        return ops.scale_rows(logits, self.logit_scale) if self.logit_scale != 1.0 else logits


register_input("embedding", Embedding)
register_input("pair_embedding", PairEmbedding)
register_output("norm_head", NormHead)
