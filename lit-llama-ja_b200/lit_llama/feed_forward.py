"""Dense feed-forward layers of the folder-loaded models: ``W_down act(W_up h)`` with the activation as a parameter."""
from __future__ import annotations

import torch
import torch.nn as nn
from torch.nn import functional as F

from . import _native as N


class DenseFF(nn.Module):
    """``act``: "relu2" (the square of relu), "gelu" (the erf form) or "gelu_tanh"."""

    def __init__(self, width: int, ff: int, act: str, dtype: torch.dtype, device) -> None:
        super().__init__()
        if act not in ("relu2", "gelu", "gelu_tanh"):
            raise ValueError(f"unknown feed-forward activation {act!r}")
        self.act = act
        kw = dict(dtype=dtype, device=device)
        self.w_up = nn.Parameter(torch.zeros((ff, width), **kw), requires_grad=False)
        self.w_down = nn.Parameter(torch.zeros((width, ff), **kw), requires_grad=False)

    def load(self, get) -> None:
        self.w_up.copy_(get("up"))
        self.w_down.copy_(get("down"))

    def forward(self, x_act: torch.Tensor) -> torch.Tensor:
        h = F.linear(x_act, self.w_up)
        if self.act == "relu2":
            N.call("ll_relu_squared", N.ptr(h), N.dtype_code(h.dtype), h.numel(), N.stream())
        else:
            N.call("ll_gelu", N.ptr(h), N.dtype_code(h.dtype), 1 if self.act == "gelu_tanh" else 0, h.numel(), N.stream())
        return F.linear(h, self.w_down)
