"""Typed configuration of Rizovik, a decoder that norms what its parts put out and whose layers mix
two kinds of windowed attention with the gated delta rule.

config.json names the design under ``architecture`` and lists its layers under ``layers``; each entry
gives ``type`` (which mixer), ``mixer`` (its sizes and constants) and ``mlp`` (the feed-forward, or null
for a layer without one).  An entry with ``weights_of``: j has no tensors of its own: it runs layer j's
(mixer, feed-forward and norms) on a cache or state of its own.  Model-wide keys: ``vocab``, ``width``,
``norm.eps``, ``residual_mult``.

Mixer types:

  * ``attention``: ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``, ``rot`` = {``base``, ``dims``, and
    optionally ``scaling.factor``}, ``mask`` = {``size``, ``pool``}.  RMS norm over the whole of q and the
    whole of k (scales per column), rotation of halves on the first ``dims`` values of a head, values
    divided by their root mean square per head, a window of ``size`` tokens followed by the means of whole
    blocks of ``pool`` tokens, a sigmoid gate per output value.
  * ``attention_2``: the same sizes; ``mask`` = {``size``, ``keep_first``}.  RMS norm of q and k per head with
    one scale vector shared by the heads, the same rotation (``rot.scaling.factor`` divides every
    frequency), a window that keeps the first ``keep_first`` tokens, the heads' softmax weights mixed by a
    matrix.
  * ``delta``: ``heads`` value heads of ``vdim``, ``kv_heads`` query/key heads of ``dim``, ``conv`` taps.  The
    gated delta rule behind short causal convolutions.

Feed-forward (``mlp.kind`` "moe"): ``router.experts`` gated SiLU experts of ``expert.ff``, of which a token
takes the ``router.top`` with the largest logits (router weight and bias), weighted by the softmax over the
taken logits.

Every layer is x <- x + m N(mixer(x)), x <- x + m N(ff(x)) on a float32 residual stream (the
``outnorm_residual`` block with ``residual_mult`` m), N an RMS norm with a scale.  The head is the embedding
table.  Tensor names: ``embed``, ``l<i>.norm1|norm2``, ``l<i>.mix.q|k|v|o`` with ``q.norm|k.norm`` and ``g`` or
``talk``, or ``l<i>.mix.q|k|v|q.conv|k.conv|v.conv|b|a|A_log|dt_bias|norm|g|o``,
``l<i>.mlp.router|router.b|e<j>.gate|up|down``, ``final.norm``.
"""

from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Mapping

from .errors import ConfigError
from .legelix import MAX_POSITIONS, _int, _number, _table
from .spec import FeedForwardSpec, InputSpec, LayerCall, LayerSpec, MixerSpec, ModelSpec, NormSpec, OutputSpec, PositionSpec


@dataclass
class RizovikConfig:
    vocab: int
    width: int
    layers: tuple[Mapping[str, Any], ...]
    norm_eps: float
    residual_mult: float

    architecture = "Rizovik"
    model_type = "rizovik"

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, config: Mapping[str, Any], where: str = "config.json") -> "RizovikConfig":
        if not isinstance(config, Mapping):
            raise ConfigError(f"{where}: the configuration must be a JSON object")
        if config.get("architecture", cls.architecture) != cls.architecture:
            raise ConfigError(f"{where}: not a {cls.architecture} configuration")
        layers = config.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError(f"{where}: 'layers' must be a non-empty list")
        result = cls(vocab=_int(config, "vocab", where), width=_int(config, "width", where),
                     layers=tuple(copy.deepcopy(layers)), norm_eps=_number(_table(config, "norm", where), "eps", where),
                     residual_mult=_number(config, "residual_mult", where) if config.get("residual_mult") is not None else 1.0)
        result.validate(where)
        return result

    def source_of(self, index: int) -> int:
        """The layer whose tensors layer ``index`` runs: itself, or the one its ``weights_of`` names."""
        seen = {index}
        while "weights_of" in self.layers[index]:
            index = int(self.layers[index]["weights_of"])
            if index in seen:
                raise ConfigError(f"layers[{index}]: weights_of runs in a circle")
            seen.add(index)
        return index

    def validate(self, where: str = "config") -> None:
        if not self.norm_eps > 0.0:
            raise ConfigError(f"{where}: norm.eps must be positive")
        for index, layer in enumerate(self.layers):
            at = f"{where}: layers[{index}]"
            if not isinstance(layer, Mapping):
                raise ConfigError(f"{at} must be a JSON object")
            if "weights_of" in layer:
                source = layer["weights_of"]
                if (isinstance(source, bool) or not isinstance(source, int) or not 0 <= source < len(self.layers)
                        or source == index):
                    raise ConfigError(f"{at}: weights_of must name another layer")
                self.source_of(index)
            kind, mixer = layer.get("type"), _table(layer, "mixer", at)
            if kind in ("attention", "attention_2"):
                for key in ("heads", "kv_heads", "dim", "vdim"):
                    _int(mixer, key, at)
                if mixer["heads"] % mixer["kv_heads"] != 0:
                    raise ConfigError(f"{at}: heads must be a multiple of kv_heads")
                _number(mixer, "scale", at)
                rot = _table(mixer, "rot", at)
                if not _number(rot, "base", at) > 1.0:
                    raise ConfigError(f"{at}: rot.base must be greater than one")
                if _int(rot, "dims", at) % 2 != 0 or rot["dims"] > mixer["dim"]:
                    raise ConfigError(f"{at}: rot.dims must be even and no more than dim")
                if rot.get("scaling") is not None and not _number(_table(rot, "scaling", at), "factor", at) > 0.0:
                    raise ConfigError(f"{at}: rot.scaling.factor must be positive")
                mask = _table(mixer, "mask", at)
                _int(mask, "size", at)
                if kind == "attention":
                    _int(mask, "pool", at)
                elif mask.get("keep_first") is not None:
                    keep = mask["keep_first"]
                    if isinstance(keep, bool) or not isinstance(keep, int) or keep < 0:
                        raise ConfigError(f"{at}: mask.keep_first must be a non-negative integer")
            elif kind == "delta":
                for key in ("heads", "kv_heads", "dim", "vdim", "conv"):
                    _int(mixer, key, at)
                if mixer["heads"] % mixer["kv_heads"] != 0:
                    raise ConfigError(f"{at}: heads must be a multiple of kv_heads")
            else:
                raise ConfigError(f"{at}: unknown layer type {kind!r}; known: attention, attention_2, delta")
            mlp = layer.get("mlp")
            if mlp is None:
                continue
            if not isinstance(mlp, Mapping) or mlp.get("kind") != "moe":
                raise ConfigError(f"{at}: 'mlp' must be null or a moe feed-forward")
            _int(_table(mlp, "expert", at), "ff", at)
            router = _table(mlp, "router", at)
            if _int(router, "top", at) > _int(router, "experts", at):
                raise ConfigError(f"{at}: router.top exceeds the number of experts")

    # ------------------------------------------------------------------ writing
    def to_dict(self) -> dict[str, Any]:
        return {"architecture": self.architecture, "layers": copy.deepcopy(list(self.layers)),
                "norm": {"eps": self.norm_eps}, "residual_mult": self.residual_mult, "vocab": self.vocab,
                "width": self.width}

    # --------------------------------------------------------------- model spec
    def _attention(self, prefix: str, m: Mapping[str, Any], pooled: bool) -> MixerSpec:
        rot, mask = m["rot"], m["mask"]
        scaling = None
        if rot.get("scaling") is not None and float(rot["scaling"]["factor"]) != 1.0:
            scaling = {"kind": "linear", "factor": float(rot["scaling"]["factor"])}
        position = PositionSpec("rope_halves", head_dim=m["dim"], max_positions=MAX_POSITIONS,
                                params={"base": float(rot["base"]), "dims": rot["dims"], "scaling": scaling})
        params = {
            "hidden_size": self.width, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "head_dim": m["dim"],
            "value_dim": m["vdim"], "window": mask["size"], "scale": float(m["scale"]), "qk_norm_eps": self.norm_eps,
            "q_proj": f"{prefix}.q", "k_proj": f"{prefix}.k", "v_proj": f"{prefix}.v", "o_proj": f"{prefix}.o",
            "q_norm": f"{prefix}.q.norm", "k_norm": f"{prefix}.k.norm"}
        if pooled:
            params.update(qk_norm="whole", value_unit_norm=True, pool=mask["pool"], out_gate=f"{prefix}.g")
        else:
            params.update(qk_norm="per_head", keep_first=int(mask.get("keep_first") or 0), head_mix=f"{prefix}.talk")
        return MixerSpec("attention", params, position)

    def _delta(self, prefix: str, m: Mapping[str, Any]) -> MixerSpec:
        return MixerSpec("gated_delta", {
            "hidden_size": self.width, "heads": m["heads"], "qk_heads": m["kv_heads"], "key_dim": m["dim"],
            "value_dim": m["vdim"], "conv": m["conv"], "norm_eps": self.norm_eps,
            "q": f"{prefix}.q", "k": f"{prefix}.k", "v": f"{prefix}.v", "g": f"{prefix}.g", "o": f"{prefix}.o",
            "q_conv": f"{prefix}.q.conv", "k_conv": f"{prefix}.k.conv", "v_conv": f"{prefix}.v.conv",
            "b": f"{prefix}.b", "a": f"{prefix}.a", "a_log": f"{prefix}.A_log", "dt_bias": f"{prefix}.dt_bias",
            "norm": f"{prefix}.norm"})

    def _feed_forward(self, prefix: str, mlp: Mapping[str, Any]) -> FeedForwardSpec:
        router = mlp["router"]
        return FeedForwardSpec("routed", {
            "hidden_size": self.width, "intermediate_size": mlp["expert"]["ff"], "activation": "silu",
            "experts": router["experts"], "top": router["top"], "scores": "top_softmax",
            "router": f"{prefix}.router", "router_bias": f"{prefix}.router.b",
            "expert_names": tuple((f"{prefix}.e{j}.gate", f"{prefix}.e{j}.up", f"{prefix}.e{j}.down")
                                  for j in range(router["experts"]))})

    def _norm(self, name: str) -> NormSpec:
        return NormSpec("rmsnorm", self.width, self.norm_eps, name)

    def to_model_spec(self) -> ModelSpec:
        from ..parts.base import MIXERS, lookup

        layers, spec_index = [], {}
        for index, layer in enumerate(self.layers):
            source = self.source_of(index)
            if source != index and {k: v for k, v in layer.items() if k != "weights_of"} == dict(self.layers[source]):
                continue          # the same parts run again: the run order names them twice
            # (An entry that names another layer's tensors but brings constants of its own gets parts of
            # its own over those tensors.)
            prefix, m = f"l{source}", layer["mixer"]
            if layer["type"] == "delta":
                mixer = self._delta(f"{prefix}.mix", m)
            else:
                mixer = self._attention(f"{prefix}.mix", m, pooled=layer["type"] == "attention")
            norms = {"mixer_out": self._norm(f"{prefix}.norm1")}
            feed_forward = None
            if layer.get("mlp") is not None:
                feed_forward = self._feed_forward(f"{prefix}.mlp", layer["mlp"])
                norms["feed_forward_out"] = self._norm(f"{prefix}.norm2")
            spec_index[index] = len(layers)
            layers.append(LayerSpec("outnorm_residual", mixer, feed_forward, norms,
                                    block_params={"residual_mult": self.residual_mult}))
        # The run order names a layer once for itself and once more for every layer that runs its tensors,
        # each time with stores of its own.
        calls, next_id = [], 0
        for index in range(len(self.layers)):
            which = spec_index[index] if index in spec_index else spec_index[self.source_of(index)]
            needs = lookup(MIXERS, "mixer", layers[which].mixer.kind).cache_spec(layers[which].mixer)
            count = len(needs) if isinstance(needs, tuple) else 1
            calls.append(LayerCall(layer=which, cache=next_id, extra_caches=tuple(range(next_id + 1, next_id + count))))
            next_id += count
        spec = ModelSpec(
            architecture=self.architecture, vocab_size=self.vocab, hidden_size=self.width, max_seq_len=MAX_POSITIONS,
            input=InputSpec("embedding", {"weight": "embed", "vocab_size": self.vocab, "hidden_size": self.width,
                                          "float32_stream": True, "rounded_copy": True}),
            layers=tuple(layers), run_order=tuple(calls),
            output=OutputSpec("norm_head", {"norm": self._norm("final.norm"), "weight": "embed",
                                            "vocab_size": self.vocab, "hidden_size": self.width}))
        spec.validate()
        return spec
