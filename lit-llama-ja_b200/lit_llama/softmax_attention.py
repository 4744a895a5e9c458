"""Softmax attention with rotary positions over a ring of key / value rows, grouped key/value heads and an element-wise
sigmoid gate on the heads' outputs, with the variations models differ in as parameters of the spec:

    q, k <- [shortconv]( W h )                       a short causal filter per channel, its last inputs kept as state
    q, k <- rmsnorm_row(.) * w                       one norm over the WHOLE projection, before the heads are split
    q, k <- rotate(., position)                      rotary.RotarySpec (partial dimensions, rescaled frequencies)
    v     = W_v h,  or the keys as they are before the rotation (``own_values`` False)
    s_h(i, j) = scale * q_h(i).k_g(j)  [-> cap * tanh(s / cap)]
    visible:    j <= i  [and i - j < window]  [and j // chunk == i // chunk]
    w = exp(s) / (sum_visible exp(s) [+ exp(sink_h)])         the sink is a learned number per head without key or value
    out = W_o( concat_h( sum_j w v_g(j) ) * sigmoid(W_g h) )

With ``maps`` = 2 every head carries two score maps (differential attention): the q and k projections hold ``[map 0 | map 1]``
per head, both maps attend over the same values, and the head's output is

    o = a_0 - lam * a_1,   lam = exp(lq1 . lk1) - exp(lq2 . lk2) + diff,       o <- o / sqrt(mean(o^2) + eps) * (1 - diff)

(``lq1`` ... ``lk2`` learned vectors of the layer, ``diff`` a constant of the spec).  ``gate`` False: no sigmoid gate.

A layer with ``kv_from`` set has no key / value tensors: it appends nothing and reads the ring of the layer it names
(whose keys are stored after norm and rotation), with its own queries, mask, sink and gate.

Cache: ``[B, R, G * maps * dim]`` keys and ``[B, R, G * vdim]`` values, position j at slot ``j % R`` (csrc/rotary_attn.cu).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Tuple

import torch
import torch.nn as nn
from torch.nn import functional as F

from . import _native as N
from .rotary import RotarySpec
from .short_conv import ShortConv


def pad8(n: int) -> int:
    return (n + 7) // 8 * 8


@dataclass
class SoftmaxAttentionSpec:
    width: int
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    eps: float
    rotary: RotarySpec = field(default_factory=lambda: RotarySpec(0))
    softcap: float = 0.0                 # 0: scores are not capped
    window: Optional[int] = None         # sliding window (None: none)
    chunk: Optional[int] = None          # chunk-local mask (None: none)
    sink: bool = False
    qk_norm: bool = False
    conv_taps: int = 0                   # 0: no short convolution on q and k
    own_values: bool = True              # False: the values are the un-rotated keys
    kv_from: Optional[int] = None        # index of the layer whose ring this layer reads
    maps: int = 1                        # score maps per head; 2: the difference of two softmax maps with a unit norm per head
    diff: float = 0.0                    # the constant of the two-map combination
    gate: bool = True                    # sigmoid(W_g h) on the heads' outputs

    def __post_init__(self):
        if self.heads % self.kv_heads:
            raise ValueError(f"{self.heads} query heads over {self.kv_heads} key/value heads")
        if not self.own_values and self.vdim != self.dim:
            raise ValueError("values taken from the keys have the keys' size")
        if self.maps not in (1, 2):
            raise ValueError(f"{self.maps} score maps per head (1 or 2)")
        if self.maps > 1 and not self.own_values:
            raise ValueError("values taken from the keys need one score map per head")
        if self.rotary.dims > self.dim:
            raise ValueError(f"{self.rotary.dims} rotated dimensions in heads of {self.dim}")

    @property
    def reach(self) -> Optional[int]:
        """A query at position i reads no key before ``i - reach + 1`` (None: unbounded)."""
        bounds = [b for b in (self.window, self.chunk) if b is not None]
        return min(bounds) if bounds else None


class SoftmaxAttention(nn.Module):
    def __init__(self, spec: SoftmaxAttentionSpec, dtype: torch.dtype, device) -> None:
        super().__init__()
        s = self.spec = spec
        kw = dict(dtype=dtype, device=device)
        f32 = dict(dtype=torch.float32, device=device)
        hd, gd, gv, hv = s.heads * s.maps * s.dim, s.kv_heads * s.maps * s.dim, s.kv_heads * s.vdim, s.heads * s.vdim
        self.owner = s.kv_from is None
        names, at = [("q", hd)] + ([("k", gd)] if self.owner else []) + ([("v", gv)] if self.owner and s.own_values else []) \
            + ([("g", hv)] if s.gate else []), 0
        self.cols = {}
        for name, n in names:
            self.cols[name] = at
            at += n
        self.n_in = at
        self.w_in = nn.Parameter(torch.zeros((pad8(self.n_in), s.width), **kw), requires_grad=False)
        self.conv_channels = hd + (gd if self.owner else 0)
        self.conv = ShortConv(self.conv_channels, s.conv_taps, False, device) if s.conv_taps > 0 else None
        self.q_norm = nn.Parameter(torch.ones(hd, **f32), requires_grad=False) if s.qk_norm else None
        self.k_norm = nn.Parameter(torch.ones(gd, **f32), requires_grad=False) if s.qk_norm and self.owner else None
        self.sink = nn.Parameter(torch.zeros(s.heads * s.maps, **f32), requires_grad=False) if s.sink else None
        self.register_buffer("freq", s.rotary.frequencies(device), persistent=False)
        self.diff_lambda = 0.0                         # lam of the two-map combination, formed at load time
        # queries that are neither filtered, normed nor turned are read where the input projection left them
        self.plain_q = self.conv is None and not s.qk_norm and s.rotary.dims == 0
        self.w_o = nn.Parameter(torch.zeros((s.width, hv), **kw), requires_grad=False)

    def state_shapes(self, B: int) -> List[Tuple[int, ...]]:
        return [self.conv.state_shape(B)] if self.conv is not None else []

    def cache_shapes(self, B: int, ring: int) -> List[Tuple[int, ...]]:
        s = self.spec
        return [(B, ring, s.kv_heads * s.maps * s.dim), (B, ring, s.kv_heads * s.vdim)] if self.owner else []

    def load(self, get) -> None:
        """``get(suffix)`` returns the tensor '<layer>.mix.<suffix>'."""
        s = self.spec
        self.w_in.zero_()
        self.w_in[: self.n_in].copy_(torch.cat([get(n).to(self.w_in.dtype) for n in self.cols], dim=0))
        if self.conv is not None:
            self.conv.load(torch.cat([get("q.conv").float()] + ([get("k.conv").float()] if self.owner else []), dim=0))
        if self.q_norm is not None:
            self.q_norm.copy_(get("q.norm").float())
        if self.k_norm is not None:
            self.k_norm.copy_(get("k.norm").float())
        if self.sink is not None:
            self.sink.copy_(get("sink").float())
        if s.maps == 2:
            l = [get(n).double() for n in ("lq1", "lk1", "lq2", "lk2")]
            self.diff_lambda = float(torch.exp((l[0] * l[1]).sum()) - torch.exp((l[2] * l[3]).sum()) + s.diff)
        self.w_o.copy_(get("o"))

    def forward(self, u: torch.Tensor, B: int, T: int, pos_ids: torch.Tensor, caches, conv_state=None, splits: int = 1,
                form: int = 0) -> torch.Tensor:
        return F.linear(self.attend(F.linear(u, self.w_in), B, T, pos_ids, caches, conv_state, splits, form), self.w_o)

    def attend(self, proj: torch.Tensor, B: int, T: int, pos_ids: torch.Tensor, caches, conv_state=None, splits: int = 1,
               form: int = 0) -> torch.Tensor:
        """``proj``: the stacked input projection's output; ``caches`` = (keys, values) of this layer or of the one it reads.
        Returns the gated heads ``[B*T, heads * vdim]`` (before the output projection)."""
        s = self.spec
        c = self.cols
        kc, vc = caches
        M = B * T
        dtc = N.dtype_code(proj.dtype)
        ring = kc.shape[1]
        st = N.stream()
        hd = s.heads * s.maps * s.dim
        if self.conv is not None:
            src = self.conv(proj, 0, conv_state, pos_ids, B, T, proj.dtype)
            q_at, k_at = N.ptr(src), N.ptr_at(src, hd)
        else:
            src = proj
            q_at, k_at = N.ptr_at(proj, c["q"]), (N.ptr_at(proj, c["k"]) if self.owner else None)
        v_at = N.ptr_at(proj, c["v"]) if "v" in c else None
        if self.plain_q:
            q, q_ptr, q_stride = None, q_at, src.stride(0)
        else:
            q = torch.empty((M, hd), dtype=proj.dtype, device=proj.device)
            q_ptr, q_stride = N.ptr(q), hd
        if self.owner or not self.plain_q:
            N.call("ll_qk_rotary_append_maps", None if self.plain_q else q_at, src.stride(0), k_at if self.owner else None, src.stride(0),
                   v_at, proj.stride(0), dtc, N.ptr(self.q_norm), N.ptr(self.k_norm), float(s.eps), N.ptr(self.freq), s.rotary.dims,
                   N.ptr(pos_ids), N.ptr(q), N.ptr(kc), N.ptr(vc), B, T, s.heads, s.kv_heads, s.dim, s.vdim, ring, s.maps, st)
        gate_at, gate_stride = (N.ptr_at(proj, c["g"]), proj.stride(0)) if s.gate else (None, 0)
        scratch = None
        if splits > 1 or (s.maps > 1 and (form != 0 or not N.call_ret("ll_softmax_attn_tensor_form", dtc, T, s.dim, s.vdim, q_stride,
                                                                       gate_stride, splits))):
            scratch = torch.empty(N.call_ret("ll_softmax_attn_scratch_bytes", M, s.heads * s.maps, s.vdim, splits) // 4,
                                  dtype=torch.float32, device=proj.device)
        y = torch.empty((M, s.heads * s.vdim), dtype=proj.dtype, device=proj.device)
        N.call("ll_softmax_attn_maps", q_ptr, q_stride, gate_at, gate_stride, N.ptr(kc), N.ptr(vc), dtc, N.ptr(pos_ids),
               N.ptr(self.sink), float(s.scale), float(s.softcap), B, T, s.heads, s.kv_heads, s.dim, s.vdim, s.window or 0, s.chunk or 0,
               ring, splits, form, s.maps, float(self.diff_lambda), float(1.0 - s.diff), float(s.eps), N.ptr(scratch), N.ptr(y), st)
        return y
