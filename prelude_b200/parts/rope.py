"""Position encodings.  A position part owns its tables; the mixer hands them
to its kernel together with each token's absolute position.

Rotary tables follow the reference (crates/prelude-core/src/models/commons/attn_utils.rs:32-50):
inv_freq_j = float32(1 / theta^(2j / rotary_dim)) with the power in float64,
angle[p, j] = float32(p) * inv_freq_j, cos and sin taken in float32.  The
tables stay float32 in every mode (the reference rounds them to the model's
type); they are computed once on the host.
"""
from __future__ import annotations

import math
from typing import Dict, Optional, Tuple

import torch

from ..config.spec import NoPositionSpec, RopeSpec, RotaryBandScaling, RotaryRampScaling, RotaryRatesSpec
from ..weights.loader import TensorReq
from .registry import RunContext, register_part

_TABLE_CACHE: Dict[tuple, Tuple[torch.Tensor, torch.Tensor]] = {}


@register_part("position", "rope_half")
class RotaryHalf:
    """Pairs element j with j + rotary_dim/2 (attn_utils.rs:52-59)."""

    def __init__(self, spec: RopeSpec, prefix: str = ""):
        if spec.rotary_dim % 2 or not 0 < spec.rotary_dim <= spec.head_dim:
            raise ValueError(f"rotary_dim={spec.rotary_dim} must be even and in (0, head_dim={spec.head_dim}]")
        self.spec = spec
        self.cos: Optional[torch.Tensor] = None
        self.sin: Optional[torch.Tensor] = None

    def tensors(self) -> Dict[str, TensorReq]:
        return {}

    def load(self, get, ctx: RunContext) -> None:
        s = self.spec
        key = (s.rotary_dim, s.theta, s.max_positions, str(ctx.device))
        if key not in _TABLE_CACHE:       # the layers of a model share one pair of tables
            inv = [1.0 / math.pow(float(s.theta), i / float(s.rotary_dim)) for i in range(0, s.rotary_dim, 2)]
            inv_freq = torch.tensor(inv, dtype=torch.float64).to(torch.float32)
            pos = torch.arange(s.max_positions, dtype=torch.float32).reshape(-1, 1)
            ang = pos * inv_freq.reshape(1, -1)
            _TABLE_CACHE[key] = (ang.cos().contiguous().to(ctx.device), ang.sin().contiguous().to(ctx.device))
        self.cos, self.sin = _TABLE_CACHE[key]

    @property
    def rotary_dim(self) -> int:
        return self.spec.rotary_dim


@register_part("position", "none")
class NoPosition:
    def __init__(self, spec: NoPositionSpec, prefix: str = ""):
        self.spec = spec
        self.cos = self.sin = None
        self.rotary_dim = 0

    def tensors(self) -> Dict[str, TensorReq]:
        return {}

    def load(self, get, ctx: RunContext) -> None:
        pass


def rotary_rates(spec: RotaryRatesSpec):
    """(rates, amplitude) of a ``RotaryRatesSpec`` in 64-bit: rate_i = base^(-2i/dims), rescaled as the spec's
    ``scaling`` says; the amplitude multiplies cosine and sine alike."""
    dims, base, sc = spec.dims, float(spec.base), spec.scaling
    plain = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    if sc is None:
        return plain, 1.0
    if isinstance(sc, RotaryBandScaling):
        out = []
        for f in plain:
            wavelength = 2.0 * math.pi / f
            if wavelength < sc.original / sc.high:
                out.append(f)
            elif wavelength > sc.original / sc.low:
                out.append(f / sc.factor)
            else:
                s = (sc.original / wavelength - sc.low) / (sc.high - sc.low)
                out.append((1.0 - s) * f / sc.factor + s * f)
        return out, 1.0
    if isinstance(sc, RotaryRampScaling):
        def turn(t: float) -> float:
            return dims * math.log(sc.original / (2.0 * math.pi * t)) / (2.0 * math.log(base))

        lo = max(math.floor(turn(sc.fast)), 0)
        hi = min(math.ceil(turn(sc.slow)), dims - 1)
        out = []
        for i, f in enumerate(plain):
            ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
            out.append(f / sc.factor * ramp + f * (1.0 - ramp))
        return out, sc.amplitude_slope * math.log(sc.factor) + 1.0
    raise ValueError(f"unknown rotary scaling {sc!r}")


@register_part("position", "rotary_rates")
class RotaryRates:
    """Rotation given by its rates: the kernel takes angle = position * rate in 32-bit and the cosine and sine of it,
    so no table and no longest sequence exist.  ``rates`` is float32 [dims / 2] (made in 64-bit, rounded once)."""

    def __init__(self, spec: RotaryRatesSpec, prefix: str = ""):
        if spec.dims % 2 or spec.dims <= 0:
            raise ValueError(f"a rotation turns pairs: dims={spec.dims} must be even and positive")
        self.spec = spec
        self.rates_host, self.amplitude = rotary_rates(spec)
        self.rates: Optional[torch.Tensor] = None
        self.cos = self.sin = None

    def tensors(self) -> Dict[str, TensorReq]:
        return {}

    def load(self, get, ctx: RunContext) -> None:
        self.rates = torch.tensor(self.rates_host, dtype=torch.float64).to(torch.float32).to(ctx.device)

    @property
    def rotary_dim(self) -> int:
        return self.spec.dims

    @property
    def adjacent(self) -> bool:
        return bool(self.spec.adjacent)
