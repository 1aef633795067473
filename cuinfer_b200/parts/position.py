"""Position encodings.

``rope_neox``: rotate-half rotary encoding over the first ``rotary_dim`` elements of a head
(csrc/model/rope_cache.cpp:15-24, :47-58; csrc/ops/qk_norm_rope_fused.cu:114-139): for i < r/2,
``f_i = 1 / theta^(2i / r)``, angle ``p · f_i``, both in 32 bits; pairs are (i, i + r/2).  The table
``[positions, r/2, (cos, sin)]`` is computed once in 32 bits on the host, as the reference does, and
handed to the kernel that applies it.  ``none``: no encoding.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from .base import PositionEncoding
from .registry import POSITION_ENCODINGS
from .spec import PartSpec


_TABLES: dict = {}


@POSITION_ENCODINGS.register("rope_neox")
class RotaryNeox(PositionEncoding):
    def __init__(self, spec: PartSpec, *, hidden_size: int, prefix: str, dtype: torch.dtype) -> None:
        super().__init__(spec, hidden_size=hidden_size, prefix=prefix, dtype=dtype)
        self.theta = float(spec.theta)
        self.rotary_dim = int(spec.rotary_dim)
        self.max_positions = int(spec.max_positions)
        if self.rotary_dim <= 0 or self.rotary_dim % 2:
            raise ValueError(f"rope_neox: rotary_dim must be positive and even, got {self.rotary_dim}")
        self._table: Optional[torch.Tensor] = None
        self._device: Optional[torch.device] = None

    def host_table(self) -> torch.Tensor:
        half = self.rotary_dim // 2
        exponent = torch.arange(0, half, dtype=torch.float32) * 2.0 / float(self.rotary_dim)
        inv_freq = 1.0 / torch.pow(torch.tensor(self.theta, dtype=torch.float32), exponent)
        pos = torch.arange(self.max_positions, dtype=torch.float32)
        angle = pos[:, None] * inv_freq[None, :]
        return torch.stack((torch.cos(angle), torch.sin(angle)), dim=-1).contiguous()

    def load(self, store) -> None:
        self._device = store.device

    def table(self) -> Optional[torch.Tensor]:
        if self._table is None:
            # layers with the same constants share one table on the device
            device = torch.device(self._device or "cuda")
            key = (self.theta, self.rotary_dim, self.max_positions, str(device))
            if key not in _TABLES:
                _TABLES[key] = self.host_table().to(device)
            self._table = _TABLES[key]
        return self._table


@POSITION_ENCODINGS.register("none")
class NoPosition(PositionEncoding):
    rotary_dim = 0

    def table(self) -> Optional[torch.Tensor]:
        return None


@POSITION_ENCODINGS.register("rope_interleaved")
class RotaryInterleaved(PositionEncoding):
    """Rotary encoding with neighbouring pairs: over the first ``rotary_dim`` elements of the vector it is applied to,
    element 2i pairs with 2i+1 and the pair (u, v) at position p becomes ``(u cos a - v sin a, v cos a + u sin a)`` with
    ``a = p * f_i``, ``f_i = theta ** (-2i / rotary_dim)``.  There is no table and hence no largest position: the
    kernels that apply it take the frequencies (32-bit, rounded once from double precision) and compute the angle and
    its full-range sine and cosine in 32 bits.  Spec: ``PartSpec("rope_interleaved", theta=..., rotary_dim=...,
    scaling=None)``.  ``scaling = (factor, low, high, original)`` rescales the frequencies by wavelength
    ``l = 2 pi / f`` against a context of ``original`` tokens: kept where ``l < original / high``, divided by ``factor``
    where ``l > original / low``, and in between ``(1 - s) f / factor + s f`` with ``s = (original / l - low) / (high - low)``.

    ``scaling`` may also be a mapping that names another law:

    * ``{"kind": "linear", "factor": c}``: every frequency is divided by ``c``;
    * ``{"kind": "ramp", "factor": c, "original": n, "fast": a, "slow": b}``: with
      ``index(t) = rotary_dim * ln(n / (2 pi t)) / (2 ln theta)`` (the pair whose wave makes ``t`` turns over ``n``
      positions), ``lo = max(floor(index(a)), 0)``, ``hi = min(ceil(index(b)), rotary_dim - 1)`` and
      ``r_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1)``, pair i turns at ``f_i / c * r_i + f_i * (1 - r_i)``, and both
      cosine and sine are multiplied by ``magnitude = 0.1 ln(c) + 1`` (the kernels take it beside the frequencies)."""

    def __init__(self, spec: PartSpec, *, hidden_size: int, prefix: str, dtype: torch.dtype) -> None:
        super().__init__(spec, hidden_size=hidden_size, prefix=prefix, dtype=dtype)
        self.theta = float(spec.theta)
        self.rotary_dim = int(spec.rotary_dim)
        if self.rotary_dim < 0 or self.rotary_dim % 2 or not self.theta > 0:
            raise ValueError(f"rope_interleaved: rotary_dim must be even and theta positive, got {self.rotary_dim}, {self.theta}")
        scaling = spec.get("scaling")
        self.law: Optional[tuple] = None            # ("linear", factor) or ("ramp", factor, original, fast, slow)
        self.magnitude = 1.0                        # what cosine and sine are multiplied by
        if isinstance(scaling, dict):
            kind = scaling.get("kind")
            if kind == "linear":
                self.law = ("linear", float(scaling["factor"]))
            elif kind == "ramp":
                self.law = ("ramp",) + tuple(float(scaling[k]) for k in ("factor", "original", "fast", "slow"))
                if self.law[2] <= 0 or self.law[3] <= 0 or self.law[4] <= 0 or self.theta == 1.0:
                    raise ValueError(f"rope: a ramp needs positive original, fast and slow and theta != 1, got {scaling}")
                self.magnitude = 0.1 * math.log(self.law[1]) + 1.0
            else:
                raise ValueError(f"rope: scaling kind {kind!r} is not linear or ramp")
            if not self.law[1] > 0:
                raise ValueError(f"rope: the scaling factor must be positive, got {scaling}")
            scaling = None
        self.scaling = tuple(float(v) for v in scaling) if scaling else None
        if self.scaling is not None and (len(self.scaling) != 4 or self.scaling[0] <= 0 or self.scaling[2] == self.scaling[1]
                                         or self.scaling[1] <= 0 or self.scaling[2] <= 0 or self.scaling[3] <= 0):
            raise ValueError(f"rope_interleaved: scaling must be (factor, low, high, original) with low != high, got {scaling}")
        self._freq: Optional[torch.Tensor] = None
        self._device: Optional[torch.device] = None

    # which elements form a pair: "interleaved" (2i, 2i+1) or "half" (i, i + rotary_dim / 2); the kernels that take the
    # frequencies ask for it
    layout = "interleaved"

    def host_frequencies(self) -> torch.Tensor:
        i = torch.arange(self.rotary_dim // 2, dtype=torch.float64)
        f = torch.pow(torch.tensor(self.theta, dtype=torch.float64), -2.0 * i / max(self.rotary_dim, 1))
        if self.scaling is not None:
            factor, low, high, original = self.scaling
            wavelength = 2.0 * math.pi / f
            s = (original / wavelength - low) / (high - low)
            blended = (1.0 - s) * f / factor + s * f
            f = torch.where(wavelength < original / high, f, torch.where(wavelength > original / low, f / factor, blended))
        if self.law is not None and self.law[0] == "linear":
            f = f / self.law[1]
        elif self.law is not None:
            _, factor, original, fast, slow = self.law
            dims = self.rotary_dim

            def index_of(turns: float) -> float:
                return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(self.theta))

            lo = max(math.floor(index_of(fast)), 0)
            hi = min(math.ceil(index_of(slow)), dims - 1)
            ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
            f = f / factor * ramp + f * (1.0 - ramp)
        return f.float()

    def load(self, store) -> None:
        self._device = store.device

    def frequencies(self) -> Optional[torch.Tensor]:
        """float32 [rotary_dim / 2] on the device, or None when nothing is rotated."""
        if self.rotary_dim == 0:
            return None
        if self._freq is None:
            device = torch.device(self._device or "cuda")
            key = ("interleaved", self.theta, self.rotary_dim, self.scaling, self.law, str(device))
            if key not in _TABLES:
                _TABLES[key] = self.host_frequencies().to(device)
            self._freq = _TABLES[key]
        return self._freq


@POSITION_ENCODINGS.register("rope_half")
class RotaryHalf(RotaryInterleaved):
    """The same rotation with another pairing: over the first ``rotary_dim`` elements, element i pairs with
    ``i + rotary_dim / 2`` (i < rotary_dim / 2), angle ``p * theta ** (-2i / rotary_dim)``; the elements from
    ``rotary_dim`` on pass unchanged.  No table and no largest position, as for ``rope_interleaved``, whose spec it
    shares: ``PartSpec("rope_half", theta=..., rotary_dim=..., scaling=None)``."""

    layout = "half"
