"""Typed configuration of Fekotar, a decoder whose layers run their mixer and their feed-forward side by
side on one norm's output.

config.json names the design under ``architecture`` and lists its layers under ``layers``; each entry
gives ``type`` (which mixer), ``mixer`` (its sizes and constants) and ``mlp`` (the feed-forward, or null
for a layer without one).  Model-wide keys: ``vocab``, ``width``, ``norm.eps``, ``logit_scale`` (a
multiplier on the logits, default 1) and ``embedding.bigram`` = {``buckets``, ``mul_prev``, ``mul_cur``}
(a second embedding table of buckets + 1 rows, looked up by a hash of the token and the token before it;
absent: a plain embedding).

Mixer type ``latent_attention``: ``heads``, ``dim`` (unrotated query/key size per head), ``rot_dim``
(rotated size per head; one rotated key part is shared by all heads), ``vdim``, ``kv_rank`` (the latent a
position keeps), ``q_rank`` (the queries' own latent), ``scale`` (on the scores, as given), ``rot`` =
{``base``, ``dims`` (= ``rot_dim``), ``scaling`` = null or {``factor``, ``original``, ``fast``, ``slow``}
(YaRN)}.  Rotation of halves; causal softmax; a sigmoid gate per output value; no sinks.

Feed-forwards (``mlp.kind``): ``dense`` (``ff``, ``limit``: bounded gate and up with biases on all three
products, y = g sigmoid(1.702 g) (u + 1)) and ``moe`` (``expert.ff``; ``router.experts`` gated SiLU experts
without biases of which a token takes ``router.top``; scores are the logistic function of float32 router
logits; ``router.groups`` = {``count``, ``keep``}: only experts of the ``keep`` groups whose two largest
scores add up to most can be taken; weights are the scores times ``router.scale``, not renormalised).

Every layer is h = rmsnorm(x) w; x <- x + (mixer(h) + ff(h)) on a float32 residual stream (the
``parallel_residual`` block).  Tensor names: ``embed``, ``bigram``, ``l<i>.norm1``,
``l<i>.mix.dq|dq.norm|uq|dkv|dkv.norm|uk|uv|g|o``, ``l<i>.mlp.gate|up|down`` each with ``.b``, or
``l<i>.mlp.router|e<j>.gate|up|down``, ``final.norm``, ``head``.
"""

from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Mapping

from .errors import ConfigError
from .legelix import MAX_POSITIONS, _int, _number, _table
from .spec import FeedForwardSpec, InputSpec, LayerSpec, MixerSpec, ModelSpec, NormSpec, OutputSpec, PositionSpec

# Constants the design fixes.
GATE_ALPHA = 1.702        # the slope inside the dense feed-forward's sigmoid
UP_SHIFT = 1.0            # what is added to the bounded up projection
GROUP_TOP = 2             # a group's mark is the sum of this many of its largest scores


@dataclass
class FekotarConfig:
    vocab: int
    width: int
    layers: tuple[Mapping[str, Any], ...]
    norm_eps: float
    logit_scale: float
    bigram: Mapping[str, int] | None

    architecture = "Fekotar"
    model_type = "fekotar"

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, config: Mapping[str, Any], where: str = "config.json") -> "FekotarConfig":
        if not isinstance(config, Mapping):
            raise ConfigError(f"{where}: the configuration must be a JSON object")
        if config.get("architecture", cls.architecture) != cls.architecture:
            raise ConfigError(f"{where}: not a {cls.architecture} configuration")
        layers = config.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError(f"{where}: 'layers' must be a non-empty list")
        bigram = None
        embedding = config.get("embedding")
        if embedding is not None and _table(config, "embedding", where).get("bigram") is not None:
            table = _table(embedding, "bigram", where)
            bigram = {"buckets": _int(table, "buckets", where)}
            for key in ("mul_prev", "mul_cur"):
                value = table.get(key)
                if isinstance(value, bool) or not isinstance(value, int) or value < 0:
                    raise ConfigError(f"{where}: embedding.bigram.{key} must be a non-negative integer")
                bigram[key] = value
        scale = _number(config, "logit_scale", where) if config.get("logit_scale") is not None else 1.0
        result = cls(vocab=_int(config, "vocab", where), width=_int(config, "width", where),
                     layers=tuple(copy.deepcopy(layers)), norm_eps=_number(_table(config, "norm", where), "eps", where),
                     logit_scale=scale, bigram=bigram)
        result.validate(where)
        return result

    def validate(self, where: str = "config") -> None:
        if not self.norm_eps > 0.0:
            raise ConfigError(f"{where}: norm.eps must be positive")
        for index, layer in enumerate(self.layers):
            at = f"{where}: layers[{index}]"
            if not isinstance(layer, Mapping):
                raise ConfigError(f"{at} must be a JSON object")
            kind, mixer = layer.get("type"), _table(layer, "mixer", at)
            if kind != "latent_attention":
                raise ConfigError(f"{at}: unknown layer type {kind!r}; known: latent_attention")
            for key in ("heads", "dim", "vdim", "kv_rank", "q_rank"):
                _int(mixer, key, at)
            _number(mixer, "scale", at)
            rot_dim = mixer.get("rot_dim", 0)
            if isinstance(rot_dim, bool) or not isinstance(rot_dim, int) or rot_dim < 0 or rot_dim % 2 != 0:
                raise ConfigError(f"{at}: rot_dim must be an even non-negative integer")
            if rot_dim > 0:
                rot = _table(mixer, "rot", at)
                if not _number(rot, "base", at) > 1.0:
                    raise ConfigError(f"{at}: rot.base must be greater than one")
                if _int(rot, "dims", at) != rot_dim:
                    raise ConfigError(f"{at}: the rotated part is rotated as a whole, so rot.dims must equal rot_dim")
                if rot.get("scaling") is not None:
                    scaling = _table(rot, "scaling", at)
                    for key in ("factor", "original", "fast", "slow"):
                        if not _number(scaling, key, at) > 0.0:
                            raise ConfigError(f"{at}: rot.scaling.{key} must be positive")
            mlp = layer.get("mlp")
            if mlp is None:
                continue
            if not isinstance(mlp, Mapping) or mlp.get("kind") not in ("dense", "moe"):
                raise ConfigError(f"{at}: 'mlp' must be null, a dense or a moe feed-forward")
            if mlp["kind"] == "dense":
                _int(mlp, "ff", at)
                if not _number(mlp, "limit", at) > 0.0:
                    raise ConfigError(f"{at}: mlp.limit must be positive")
            else:
                _int(_table(mlp, "expert", at), "ff", at)
                router = _table(mlp, "router", at)
                experts, top = _int(router, "experts", at), _int(router, "top", at)
                if top > experts:
                    raise ConfigError(f"{at}: router.top exceeds the number of experts")
                if router.get("scale") is not None:
                    _number(router, "scale", at)
                if router.get("groups") is not None:
                    groups = _table(router, "groups", at)
                    count, keep = _int(groups, "count", at), _int(groups, "keep", at)
                    if experts % count != 0 or keep > count or keep * (experts // count) < top:
                        raise ConfigError(f"{at}: router.groups must divide the experts evenly, keep <= count, and the "
                                          "kept groups must hold router.top experts")

    # ------------------------------------------------------------------ writing
    def to_dict(self) -> dict[str, Any]:
        out: dict[str, Any] = {"architecture": self.architecture, "layers": copy.deepcopy(list(self.layers)),
                               "logit_scale": self.logit_scale, "norm": {"eps": self.norm_eps}, "vocab": self.vocab,
                               "width": self.width}
        if self.bigram is not None:
            out["embedding"] = {"bigram": dict(self.bigram)}
        return out

    # --------------------------------------------------------------- model spec
    def _latent_attention(self, prefix: str, m: Mapping[str, Any]) -> MixerSpec:
        rot_dim = int(m.get("rot_dim", 0))
        position = None
        if rot_dim > 0:
            rot = m["rot"]
            position = PositionSpec("rope_halves", head_dim=rot_dim, max_positions=MAX_POSITIONS, params={
                "base": float(rot["base"]), "dims": rot_dim,
                "scaling": dict(rot["scaling"]) if rot.get("scaling") is not None else None})
        return MixerSpec("latent_attention", {
            "hidden_size": self.width, "num_heads": m["heads"], "head_dim": m["dim"], "value_dim": m["vdim"],
            "rank": m["kv_rank"], "rot_dim": rot_dim, "scale": float(m["scale"]), "norm_eps": self.norm_eps,
            "q_rank": m["q_rank"], "q_down": f"{prefix}.dq", "q_down_norm": f"{prefix}.dq.norm", "q_proj": f"{prefix}.uq",
            "latent_proj": f"{prefix}.dkv", "latent_norm": f"{prefix}.dkv.norm", "k_up": f"{prefix}.uk",
            "v_up": f"{prefix}.uv", "gate": f"{prefix}.g", "gate_per_element": True, "o_proj": f"{prefix}.o"}, position)

    def _feed_forward(self, prefix: str, mlp: Mapping[str, Any]) -> FeedForwardSpec:
        if mlp["kind"] == "dense":
            return FeedForwardSpec("gated", {
                "hidden_size": self.width, "intermediate_size": mlp["ff"], "activation": "clamped_swish",
                "limit": float(mlp["limit"]), "alpha": GATE_ALPHA, "up_shift": UP_SHIFT,
                "gate_proj": f"{prefix}.gate", "up_proj": f"{prefix}.up", "down_proj": f"{prefix}.down",
                "gate_bias": f"{prefix}.gate.b", "up_bias": f"{prefix}.up.b", "down_bias": f"{prefix}.down.b"})
        router = mlp["router"]
        groups = router.get("groups")
        return FeedForwardSpec("routed", {
            "hidden_size": self.width, "intermediate_size": mlp["expert"]["ff"], "activation": "silu",
            "experts": router["experts"], "identity": 0, "top": router["top"], "scores": "sigmoid",
            "weight_scale": float(router.get("scale", 1.0) if router.get("scale") is not None else 1.0),
            "groups": {"count": groups["count"], "keep": groups["keep"], "top": GROUP_TOP} if groups is not None else None,
            "router": f"{prefix}.router",
            "expert_names": tuple((f"{prefix}.e{j}.gate", f"{prefix}.e{j}.up", f"{prefix}.e{j}.down")
                                  for j in range(router["experts"]))})

    def _norm(self, name: str) -> NormSpec:
        return NormSpec("rmsnorm", self.width, self.norm_eps, name)

    def to_model_spec(self) -> ModelSpec:
        from ..parts.model import run_order_for

        layers = []
        for index, layer in enumerate(self.layers):
            prefix = f"l{index}"
            mixer = self._latent_attention(f"{prefix}.mix", layer["mixer"])
            feed_forward = self._feed_forward(f"{prefix}.mlp", layer["mlp"]) if layer.get("mlp") is not None else None
            layers.append(LayerSpec("parallel_residual", mixer, feed_forward, {"input": self._norm(f"{prefix}.norm1")}))
        if self.bigram is not None:
            source = InputSpec("pair_embedding", {"weight": "embed", "pair_weight": "bigram", "vocab_size": self.vocab,
                                                  "hidden_size": self.width, **self.bigram})
        else:
            source = InputSpec("embedding", {"weight": "embed", "vocab_size": self.vocab, "hidden_size": self.width,
                                             "float32_stream": True})
        spec = ModelSpec(
            architecture=self.architecture, vocab_size=self.vocab, hidden_size=self.width, max_seq_len=MAX_POSITIONS,
            input=source, layers=tuple(layers), run_order=run_order_for(layers),
            output=OutputSpec("norm_head", {"norm": self._norm("final.norm"), "weight": "head", "vocab_size": self.vocab,
                                            "hidden_size": self.width, "logit_scale": self.logit_scale}))
        spec.validate()
        return spec
