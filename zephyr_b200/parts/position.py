"""Position encodings applied to queries and keys.

``rope_neox``: inv_freq[i] = 1 / theta^(2i/hd) for i < hd/2, angle[p, i] = p * inv_freq[i], all in
float32; cos and sin of the float32 angle; rotation of the pairs (i, i + hd/2)
(reference: src/layer/rotary_embedding.cpp:36-55, src/layer/rotary_embedding.cu:24-47).  The
tables stay float32 on the device (the reference rounds them to the model's type).

``rope_pairs``: rotation of adjacent pairs (2i, 2i + 1) on the first ``dims`` dimensions of a head, with
optional scaling of the frequencies by wavelength.

``rope_halves``: rotation of the pairs (i, i + dims/2) on the first ``dims`` dimensions of a head, angles
formed on the device as float32 products, with optional YaRN scaling of the frequencies and its
multiplier on cosine and sine.

``none``: no encoding.
"""

from __future__ import annotations

import math

import torch

from ..config.errors import ConfigError
from ..config.spec import PositionSpec
from ..kernels import ops
from .base import PositionEncoding, register_position_encoding


def rope_tables(head_dim: int, max_positions: int, theta: float) -> tuple[torch.Tensor, torch.Tensor]:
    """cos and sin, float32 [max_positions, head_dim/2], computed on the host in float32."""
    index = torch.arange(0, head_dim // 2, dtype=torch.float32)
    exponent = (2.0 * index) / torch.tensor(float(head_dim), dtype=torch.float32)
    inv_freq = 1.0 / torch.pow(torch.tensor(float(theta), dtype=torch.float32), exponent)
    angles = torch.arange(max_positions, dtype=torch.float32)[:, None] * inv_freq[None, :]
    return torch.cos(angles).contiguous(), torch.sin(angles).contiguous()


class RopeNeox(PositionEncoding):
    graph_safe = True

    kind = "rope_neox"

    def __init__(self, spec: PositionSpec, dtype: torch.dtype, device: torch.device | str):
        if spec.head_dim <= 0 or spec.head_dim % 2 != 0:
            raise ConfigError("a rotary head size must be positive and even")
        theta = float(spec.params.get("theta", 10000.0))
        if not theta > 0.0 or theta == float("inf"):
            raise ConfigError("the rotary base must be finite and positive")
        self.head_dim = spec.head_dim
        self.max_positions = spec.max_positions
        cos, sin = rope_tables(spec.head_dim, spec.max_positions, theta)
        self.cos = cos.to(device)
        self.sin = sin.to(device)

    def apply(self, x: torch.Tensor, heads: int, positions: torch.Tensor, status: torch.Tensor) -> torch.Tensor:
        return ops.rope(x, heads, self.head_dim, self.cos, self.sin, positions, status)

    def as_rotation_tables(self) -> tuple[torch.Tensor, torch.Tensor]:
        return self.cos, self.sin


class NoPosition(PositionEncoding):
    graph_safe = True

    kind = "none"

    def __init__(self, spec: PositionSpec, dtype: torch.dtype, device: torch.device | str):
        self.head_dim = spec.head_dim
        self.max_positions = spec.max_positions

    def apply(self, x: torch.Tensor, heads: int, positions: torch.Tensor, status: torch.Tensor) -> torch.Tensor:
        return x

    def as_rotation_tables(self) -> tuple[None, None]:
        return None, None


def scaled_frequencies(freqs: list[float], factor: float, low: float, high: float, original: float) -> list[float]:
    """Frequency scaling by wavelength (the scheme Llama 3.1 uses to stretch a context of ``original``
    positions): with wavelength l = 2 pi / f, a frequency is kept where l < original / high, divided by
    ``factor`` where l > original / low, and in between blended with s = (original / l - low) /
    (high - low) as (1 - s) f / factor + s f."""
    out = []
    for f in freqs:
        wavelength = 2.0 * math.pi / f
        if wavelength < original / high:
            out.append(f)
        elif wavelength > original / low:
            out.append(f / factor)
        else:
            s = (original / wavelength - low) / (high - low)
            out.append((1.0 - s) * f / factor + s * f)
    return out


class RopePairs(PositionEncoding):
    """Rotation of adjacent pairs: dimensions 2i and 2i + 1 of every head, for i < dims / 2, turn by the
    angle position * f_i with f_i = base^(-2i / dims); dimensions from ``dims`` on pass unchanged.
    (u, v) -> (u cos a - v sin a, v cos a + u sin a).  ``params``: base, dims (default: the head size),
    scaling (None, or factor / low / high / original as in ``scaled_frequencies``).  Frequencies are
    worked out in double precision on the host and kept as float32; angles are float32 products on the
    device.  The attention part hands the frequencies to the kernel that also norms and stores
    (``as_pair_frequencies``); ``apply`` is not offered apart from it."""

    graph_safe = True

    kind = "rope_pairs"

    def __init__(self, spec: PositionSpec, dtype: torch.dtype, device: torch.device | str):
        dims = int(spec.params.get("dims", spec.head_dim))
        base = float(spec.params.get("base", 10000.0))
        if dims <= 0 or dims % 2 != 0 or dims > spec.head_dim:
            raise ConfigError("rotated dimensions must be even, positive and no more than the head size")
        if not base > 0.0 or base == float("inf"):
            raise ConfigError("the rotary base must be finite and positive")
        freqs = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
        scaling = spec.params.get("scaling")
        if scaling:
            factor, low, high, original = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
            if factor <= 0.0 or original <= 0.0 or high == low or low <= 0.0 or high <= 0.0:
                raise ConfigError("frequency scaling needs positive factor, low, high and original, and low != high")
            freqs = scaled_frequencies(freqs, factor, low, high, original)
        self.head_dim = spec.head_dim
        self.dims = dims
        self.max_positions = spec.max_positions
        self.freqs = torch.tensor(freqs, dtype=torch.float64).to(torch.float32).to(device)

    def as_pair_frequencies(self) -> tuple[torch.Tensor, int]:
        return self.freqs, self.dims

    def apply(self, x: torch.Tensor, heads: int, positions: torch.Tensor, status: torch.Tensor) -> torch.Tensor:
        raise ConfigError("the rotation of adjacent pairs runs inside the attention's own kernel only")


def yarn_frequencies(freqs: list[float], dims: int, base: float, factor: float, original: float, fast: float,
                     slow: float) -> tuple[list[float], float]:
    """YaRN: frequencies that turn often within the ``original`` context stay, those that turn seldom are
    divided by ``factor``, with a linear ramp over the dimension index in between.  The dimension whose
    frequency makes t turns over ``original`` positions is d(t) = dims ln(original / (2 pi t)) / (2 ln base);
    the ramp runs from lo = max(floor(d(fast)), 0) to hi = min(ceil(d(slow)), dims - 1):
    r_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1), f_i' = r_i f_i / factor + (1 - r_i) f_i.
    Returns the frequencies and the multiplier 0.1 ln(factor) + 1 that goes on cosine and sine."""
    def turns_to_dim(turns: float) -> float:
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(turns_to_dim(fast)), 0)
    hi = min(math.ceil(turns_to_dim(slow)), dims - 1)
    out = []
    for i, f in enumerate(freqs):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(f / factor * ramp + f * (1.0 - ramp))
    return out, 0.1 * math.log(factor) + 1.0


class RopeHalves(PositionEncoding):
    """Rotation of halves: dimension i of the rotated part pairs with dimension i + dims / 2, i < dims / 2;
    (u, v) -> (u c - v s, v c + u s) with c = m cos(p f_i), s = m sin(p f_i), f_i = base^(-2i / dims).
    ``params``: base, dims (default: the head size), scaling (None; or factor / original / fast / slow as in
    ``yarn_frequencies``, which also sets m; or kind "linear" with a factor: every frequency divided by it;
    m = 1 without YaRN).  Frequencies are worked out in double
    precision on the host and kept as float32; angles are float32 products on the device.  Mixers hand
    frequencies and multiplier to their own kernels (``as_half_frequencies``); ``apply`` is not offered."""

    graph_safe = True

    kind = "rope_halves"

    def __init__(self, spec: PositionSpec, dtype: torch.dtype, device: torch.device | str):
        dims = int(spec.params.get("dims", spec.head_dim))
        base = float(spec.params.get("base", 10000.0))
        if dims <= 0 or dims % 2 != 0 or dims > spec.head_dim:
            raise ConfigError("rotated dimensions must be even, positive and no more than the head size")
        if not base > 1.0 or base == float("inf"):
            raise ConfigError("the rotary base must be finite and greater than one")
        freqs = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
        self.mult = 1.0
        scaling = spec.params.get("scaling")
        if scaling and scaling.get("kind") == "linear":
            factor = float(scaling["factor"])
            if not factor > 0.0 or factor == float("inf"):
                raise ConfigError("linear scaling needs a finite positive factor")
            freqs = [f / factor for f in freqs]
        elif scaling:
            factor, original, fast, slow = (float(scaling[k]) for k in ("factor", "original", "fast", "slow"))
            if factor <= 0.0 or original <= 0.0 or fast <= 0.0 or slow <= 0.0:
                raise ConfigError("YaRN scaling needs positive factor, original, fast and slow")
            freqs, self.mult = yarn_frequencies(freqs, dims, base, factor, original, fast, slow)
        self.head_dim = spec.head_dim
        self.dims = dims
        self.max_positions = spec.max_positions
        self.freqs = torch.tensor(freqs, dtype=torch.float64).to(torch.float32).to(device)

    def as_half_frequencies(self) -> tuple[torch.Tensor, int, float]:
        return self.freqs, self.dims, self.mult

    def apply(self, x: torch.Tensor, heads: int, positions: torch.Tensor, status: torch.Tensor) -> torch.Tensor:
        raise ConfigError("the rotation of halves with scaled frequencies runs inside a mixer's own kernel only")


register_position_encoding("rope_neox", RopeNeox)
register_position_encoding("rope_halves", RopeHalves)
register_position_encoding("rope_pairs", RopePairs)
register_position_encoding("none", NoPosition)
