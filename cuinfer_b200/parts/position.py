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
    where ``l > original / low``, and in between ``(1 - s) f / factor + s f`` with ``s = (original / l - low) / (high - low)``."""

    def __init__(self, spec: PartSpec, *, hidden_size: int, prefix: str, dtype: torch.dtype) -> None:
        super().__init__(spec, hidden_size=hidden_size, prefix=prefix, dtype=dtype)
        self.theta = float(spec.theta)
        self.rotary_dim = int(spec.rotary_dim)
        if self.rotary_dim < 0 or self.rotary_dim % 2 or not self.theta > 0:
            raise ValueError(f"rope_interleaved: rotary_dim must be even and theta positive, got {self.rotary_dim}, {self.theta}")
        scaling = spec.get("scaling")
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
        return f.float()

    def load(self, store) -> None:
        self._device = store.device

    def frequencies(self) -> Optional[torch.Tensor]:
        """float32 [rotary_dim / 2] on the device, or None when nothing is rotated."""
        if self.rotary_dim == 0:
            return None
        if self._freq is None:
            device = torch.device(self._device or "cuda")
            key = ("interleaved", self.theta, self.rotary_dim, self.scaling, str(device))
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
