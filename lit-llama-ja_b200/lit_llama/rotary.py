"""Rotary positions in the "rotate half" layout on the first ``dims`` dimensions of a head: dimension ``i`` is paired with
``i + dims/2`` and the pair turns by ``position * f_i``, ``f_i = base^(-2i/dims)``.  The frequencies may be rescaled for
longer contexts:

* ``linear``: every ``f_i`` divided by ``factor``;
* ``bands`` (the Llama-3.1 rule): by wavelength ``l = 2 pi / f`` - kept where ``l < original/high``, divided by ``factor``
  where ``l > original/low``, and between the two ``(1 - s) f/factor + s f`` with ``s = (original/l - low) / (high - low)``;
* ``yarn``: by pair index - with ``d(t) = dims ln(original / (2 pi t)) / (2 ln base)`` the index of the pair that makes ``t``
  turns over ``original`` positions, ``lo = max(floor(d(fast)), 0)``, ``hi = min(ceil(d(slow)), dims - 1)`` and
  ``ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1)``, the frequency is ``f_i / factor * ramp_i + f_i (1 - ramp_i)``, and
  every cosine and sine is multiplied by ``magnitude = 0.1 ln(factor) + 1``.

The table is made once on the host in float64 and kept as fp32; the kernels form ``angle = float(position) * f_i`` and its
sine and cosine in fp32 (csrc/rotary_attn.cu).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional

import torch


@dataclass
class RotarySpec:
    dims: int                          # rotated dimensions of every head (even, <= the head's size); 0: no rotation
    base: float = 10000.0
    scaling: Optional[str] = None      # None | "linear" | "bands" | "yarn"
    factor: float = 1.0
    low: float = 1.0
    high: float = 1.0
    original: float = 0.0
    fast: float = 32.0                 # yarn: turns over ``original`` positions above which a pair keeps its frequency
    slow: float = 1.0                  # yarn: turns below which a pair's frequency is divided by ``factor``

    def __post_init__(self):
        if self.dims < 0 or self.dims % 2:
            raise ValueError(f"{self.dims} rotated dimensions (an even number)")
        if self.scaling not in (None, "linear", "bands", "yarn"):
            raise ValueError(f"unknown frequency scaling {self.scaling!r}")

    @classmethod
    def from_dict(cls, rot: Optional[dict], head_dim: Optional[int] = None) -> "RotarySpec":
        """``{"dims", "base", "scaling": {"factor"[, "low", "high", "original"] | [, "fast", "slow", "original"]}}``; None: no
        rotation.  ``dims`` left out: the whole head (``head_dim``)."""
        if not rot:
            return cls(dims=0)
        dims = int(rot["dims"]) if rot.get("dims") is not None else int(head_dim)
        sc = rot.get("scaling") or None
        if sc is None:
            return cls(dims=dims, base=float(rot["base"]))
        if sc.get("fast") is not None or sc.get("slow") is not None:
            return cls(dims=dims, base=float(rot["base"]), scaling="yarn", factor=float(sc["factor"]), original=float(sc["original"]),
                       fast=float(sc.get("fast", 32.0)), slow=float(sc.get("slow", 1.0)))
        if sc.get("original") is None:
            return cls(dims=dims, base=float(rot["base"]), scaling="linear", factor=float(sc["factor"]))
        return cls(dims=dims, base=float(rot["base"]), scaling="bands", factor=float(sc["factor"]),
                   low=float(sc["low"]), high=float(sc["high"]), original=float(sc["original"]))

    @property
    def magnitude(self) -> float:
        """What every cosine and sine is multiplied by (1 except under ``yarn``)."""
        return 0.1 * math.log(self.factor) + 1.0 if self.scaling == "yarn" else 1.0

    def _pair_index(self, turns: float) -> float:
        return self.dims * math.log(self.original / (2.0 * math.pi * turns)) / (2.0 * math.log(self.base))

    def frequencies(self, device=None) -> torch.Tensor:
        """fp32 ``[dims / 2]`` (one entry, unused, when nothing is rotated)."""
        out = []
        if self.scaling == "yarn" and self.dims:
            lo = max(math.floor(self._pair_index(self.fast)), 0)
            hi = min(math.ceil(self._pair_index(self.slow)), self.dims - 1)
        for i in range(self.dims // 2):
            f = self.base ** (-2.0 * i / self.dims)
            if self.scaling == "yarn":
                ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
                f = f / self.factor * ramp + f * (1.0 - ramp)
            elif self.scaling == "linear":
                f /= self.factor
            elif self.scaling == "bands":
                wave = 2.0 * math.pi / f
                if wave > self.original / self.low:
                    f /= self.factor
                elif wave >= self.original / self.high:
                    s = (self.original / wave - self.low) / (self.high - self.low)
                    f = (1.0 - s) * f / self.factor + s * f
            out.append(f)
        return torch.tensor(out or [0.0], dtype=torch.float64).to(torch.float32).to(device)

    def table(self, n_pos: int, device=None) -> torch.Tensor:
        """``[n_pos, dims / 2, 2]`` fp32 (cos, sin) * magnitude of ``position * f_i`` for kernels that look the turn up instead
        of forming it; the fp32 frequencies are those of ``frequencies()``, the angles are exact products of them."""
        if self.dims == 0:
            return torch.zeros((n_pos, 1, 2), dtype=torch.float32, device=device)
        ang = torch.arange(n_pos, dtype=torch.float64)[:, None] * self.frequencies().double()[None]
        return (torch.stack((ang.cos(), ang.sin()), dim=-1) * self.magnitude).float().contiguous().to(device)
