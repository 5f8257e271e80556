"""Arrangements of a layer's parts around the residual stream.

``prenorm_residual``: r = x + mixer(norm1(x)); x' = r + ffn(norm2(r)), the sums in float32
(reference: src/model/causal_lm/qwen3.cpp:79-88).  Each sum is folded into the norm that follows
it, so the block hands its last summand on as ``pending``.

``sandwich_residual``: a norm before and one behind each part, and a multiplier m on what joins the
stream: r = x + m * mixer_out(mixer(mixer_norm(x))); x' = r + m * ffn_out(ffn(ffn_norm(r))).  The
stream is float32.  The feed-forward may be missing; the layer is then its first half.  Each sum
runs in the same kernel as the norm that follows it where the norms offer that (``Norm.add_scaled``),
the last one as a ``DeferredSum`` that the next block or the output part takes up.

``outnorm_residual``: a norm on each part's output only; the parts read the stream itself:
r = x + m * mixer_out(mixer(x)); x' = r + m * ffn_out(ffn(r)), m = ``residual_mult`` (1 unless given).  The stream is float32; in a bfloat16 model the
parts get its rounding, which the kernel that does a sum writes in the same pass.

``parallel_residual``: one norm, whose output both parts read: h = norm(x); x' = x + (mixer(h) + ffn(h)).
The stream is float32.  The two summands travel as a pair in ``pending`` and join the stream in the same
kernel as the next layer's norm (``Norm.sum_forward``).
"""

from __future__ import annotations

from typing import Mapping

import torch

from ..config.spec import LayerCall
from .base import Block, DeferredSum, FeedForward, Mixer, Norm, ResidualStream, StepContext, register_block
from .fused import BlockPlan


class PreNormResidual(Block):
    graph_safe = True

    norm_names = ("mixer", "feed_forward")

    def __init__(self, mixer: Mixer, feed_forward: FeedForward, norms: Mapping[str, Norm]):
        self.mixer = mixer
        self.feed_forward = feed_forward
        self.norms = dict(norms)
        self.mixer_norm = norms["mixer"]
        self.feed_forward_norm = norms["feed_forward"]

    def forward(self, stream: ResidualStream, ctx: StepContext, call: LayerCall) -> ResidualStream:
        if stream.pending is None:
            normed = self.mixer_norm.forward(stream.hidden)
        else:
            normed = self.mixer_norm.add_forward(stream.hidden, stream.pending)
        mixed = self.mixer.forward(normed, ctx, call)
        normed = self.feed_forward_norm.add_forward(stream.hidden, mixed)
        stream.pending = self.feed_forward.forward(normed)
        return stream


    def chain_plan(self) -> BlockPlan | None:
        mixer_norm, ffn_norm = self.mixer_norm.as_rms_scale(), self.feed_forward_norm.as_rms_scale()
        gated = self.feed_forward.as_gated_products()
        if mixer_norm is None or ffn_norm is None or gated is None:
            return None
        return BlockPlan(self.mixer, mixer_norm, ffn_norm, gated[0], gated[1])


class SandwichResidual(Block):
    graph_safe = True
    feed_forward_optional = True

    norm_names = ("mixer", "mixer_out", "feed_forward", "feed_forward_out")

    def __init__(self, mixer: Mixer, feed_forward: FeedForward | None, norms: Mapping[str, Norm], params=None):
        self.mixer = mixer
        self.feed_forward = feed_forward
        self.norms = dict(norms)
        self.mult = float((params or {}).get("residual_mult", 1.0))

    def forward(self, stream: ResidualStream, ctx: StepContext, call: LayerCall) -> ResidualStream:
        if stream.pending is not None or stream.hidden.dtype != torch.float32:
            stream.hidden = stream.flush().float()
        norms, hidden = self.norms, stream.hidden
        if stream.deferred is not None:
            normed = stream.deferred.apply(hidden, then=norms["mixer"])
            stream.deferred = None
        else:
            normed = norms["mixer"].forward(hidden)
        mixed = self.mixer.forward(normed, ctx, call)
        summand = DeferredSum(mixed, norms["mixer_out"], self.mult)
        if self.feed_forward is not None:
            normed = summand.apply(hidden, then=norms["feed_forward"])
            summand = DeferredSum(self.feed_forward.forward(normed), norms["feed_forward_out"], self.mult)
        stream.deferred = summand
        return stream


class OutputNormResidual(Block):
    graph_safe = True
    feed_forward_optional = True

    norm_names = ("mixer_out", "feed_forward_out")

    def __init__(self, mixer: Mixer, feed_forward: FeedForward | None, norms: Mapping[str, Norm], params=None):
        self.mixer = mixer
        self.feed_forward = feed_forward
        self.norms = dict(norms)
        self.dtype = norms["mixer_out"].dtype
        self.mult = float((params or {}).get("residual_mult", 1.0))

    def forward(self, stream: ResidualStream, ctx: StepContext, call: LayerCall) -> ResidualStream:
        if stream.pending is not None or stream.hidden.dtype != torch.float32:
            stream.hidden, stream.rounded = stream.flush().float(), None
        hidden = stream.hidden
        if stream.deferred is not None:
            x = stream.deferred.apply(hidden, rounded=self.dtype)
            stream.deferred = None
        elif stream.rounded is not None:
            x = stream.rounded
        else:
            x = hidden if self.dtype == torch.float32 else hidden.to(self.dtype)
        stream.rounded = None
        summand = DeferredSum(self.mixer.forward(x, ctx, call), self.norms["mixer_out"], self.mult)
        if self.feed_forward is not None:
            x = summand.apply(hidden, rounded=self.dtype)
            summand = DeferredSum(self.feed_forward.forward(x), self.norms["feed_forward_out"], self.mult)
        stream.deferred = summand
        return stream


class ParallelResidual(Block):
    graph_safe = True
    feed_forward_optional = True

    norm_names = ("input",)

    def __init__(self, mixer: Mixer, feed_forward: FeedForward | None, norms: Mapping[str, Norm], params=None):
        self.mixer = mixer
        self.feed_forward = feed_forward
        self.norms = dict(norms)
        self.norm = norms["input"]
        if not hasattr(self.norm, "sum_forward"):
            raise TypeError("the parallel block needs a norm that adds a pair of summands as it norms (sum_forward)")

    def forward(self, stream: ResidualStream, ctx: StepContext, call: LayerCall) -> ResidualStream:
        if stream.deferred is not None or stream.hidden.dtype != torch.float32:
            stream.hidden = stream.flush().float()
        pending = stream.pending if stream.pending is not None else ()
        if not isinstance(pending, tuple):
            pending = (pending,)
        normed = self.norm.sum_forward(stream.hidden, pending)
        stream.rounded = None
        mixed = self.mixer.forward(normed, ctx, call)
        if self.feed_forward is None:
            stream.pending = (mixed,)
        else:
            stream.pending = (mixed, *self.feed_forward.forward_summands(normed))
        return stream


register_block("prenorm_residual", PreNormResidual)
register_block("parallel_residual", ParallelResidual)
register_block("outnorm_residual", OutputNormResidual)
register_block("sandwich_residual", SandwichResidual)
