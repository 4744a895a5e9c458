"""Rotary positions in the "rotate half" layout on the first ``dims`` dimensions of a head: dimension ``i`` is paired with
``i + dims/2`` and the pair turns by ``position * f_i``, ``f_i = base^(-2i/dims)``.  The frequencies may be rescaled for
longer contexts:

* ``linear``: every ``f_i`` divided by ``factor``;
* ``bands`` (the Llama-3.1 rule): by wavelength ``l = 2 pi / f`` - kept where ``l < original/high``, divided by ``factor``
  where ``l > original/low``, and between the two ``(1 - s) f/factor + s f`` with ``s = (original/l - low) / (high - low)``.

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
    scaling: Optional[str] = None      # None | "linear" | "bands"
    factor: float = 1.0
    low: float = 1.0
    high: float = 1.0
    original: float = 0.0

    def __post_init__(self):
        if self.dims < 0 or self.dims % 2:
            raise ValueError(f"{self.dims} rotated dimensions (an even number)")
        if self.scaling not in (None, "linear", "bands"):
            raise ValueError(f"unknown frequency scaling {self.scaling!r}")

    @classmethod
    def from_dict(cls, rot: Optional[dict], head_dim: Optional[int] = None) -> "RotarySpec":
        """``{"dims", "base", "scaling": {"factor"[, "low", "high", "original"]}}``; None: no rotation.  ``dims`` left out:
        the whole head (``head_dim``)."""
        if not rot:
            return cls(dims=0)
        dims = int(rot["dims"]) if rot.get("dims") is not None else int(head_dim)
        sc = rot.get("scaling") or None
        if sc is None:
            return cls(dims=dims, base=float(rot["base"]))
        if sc.get("original") is None:
            return cls(dims=dims, base=float(rot["base"]), scaling="linear", factor=float(sc["factor"]))
        return cls(dims=dims, base=float(rot["base"]), scaling="bands", factor=float(sc["factor"]),
                   low=float(sc["low"]), high=float(sc["high"]), original=float(sc["original"]))

    def frequencies(self, device=None) -> torch.Tensor:
        """fp32 ``[dims / 2]`` (one entry, unused, when nothing is rotated)."""
        out = []
        for i in range(self.dims // 2):
            f = self.base ** (-2.0 * i / self.dims)
            if self.scaling == "linear":
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
