"""Mixers built on a linear recurrence with a diagonal decay (csrc/decay_scan.cu), whose fp32 state replaces a cache:

* ``StateSpaceMixer`` - selective state space with a scalar decay per head and token ("Mamba-2" form):
      [z | x | B | C | dt] = W_in h;  (x, B, C) <- silu(shortconv(x, B, C));  dt <- softplus(dt + dt_bias)
      S_t = exp(-exp(A_log) dt_t) S_(t-1) + dt_t B_t x_t^T;   y_t = S_t^T C_t + D x_t
      out = W_o ( groupnorm( y * silu(z) ) * w )
* ``GatedLinearAttention`` - a decay per key channel:
      alpha = sigmoid(W_a2 W_a1 h + b)^(1/tau);  S_t = diag(alpha_t) S_(t-1) + k_t v_t^T;  o_t = S_t^T q_t * dim^(-1/2)
      out = W_o ( headnorm(o) * w * silu(W_g h) )
* ``MatrixMemoryMixer`` - matrix memory with exponential gates ("mLSTM" form): log gates li = cap(W_i h + b_i),
  lf = logsigmoid(cap(W_f h + b_f)), cap(z) = c tanh(z / c), and a running stabiliser mx (0 at the start):
      mx_t = max(lf_t + mx_(t-1), li_t);  S_t = e^(lf_t + mx_(t-1) - mx_t) S_(t-1) + e^(li_t - mx_t) k_t v_t^T;  n_t alike with k_t alone
      o_t = S_t^T q_t / (max(|n_t . q_t|, e^(-mx_t)) + 1e-6),  q_t = W_q h * dim^(-1/2)
      out = W_o ( headnorm(o) * w * sigmoid(W_g h) )
  The normaliser n rides in the same walk as one more value column that is constantly 1.

Decays, step sizes, the state, the read-out and the norms are fp32; the projections, the short convolution's output and
the gates are in the activation dtype.  A sequence at position 0 starts from a zero state whatever its slot holds.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Tuple

import torch
import torch.nn as nn
from torch.nn import functional as F

from . import _native as N
from .short_conv import ShortConv


def pad8(n: int) -> int:
    return (n + 7) // 8 * 8


def decay_scan(q, q_col, k, k_col, v, v_col, decay, per_channel, kscale, skip, qscale, state, pos_ids, B, T, H, qk_heads, n, p,
               unit_col=False):
    """fp32 ``[B*T, H*p]``: the read-out of the recurrence (see csrc/decay_scan.cu); ``state`` is advanced in place.
    ``unit_col``: the last of the ``p`` columns of every head is the constant 1 (``v`` holds ``p - 1`` per head)."""
    y = torch.empty((B * T, H * p), dtype=torch.float32, device=v.device)
    N.call("ll_decay_scan", N.ptr_at(q, q_col), q.stride(0), N.ptr_at(k, k_col), k.stride(0), N.ptr_at(v, v_col), v.stride(0),
           N.dtype_code(v.dtype), N.ptr(decay), 1 if per_channel else 0, N.ptr(kscale), N.ptr(skip), float(qscale), N.ptr(state),
           N.ptr(pos_ids), N.ptr(y), B, T, H, qk_heads, n, p, 1 if unit_col else 0, N.stream())
    return y


def gated_group_norm(y, gate, gate_col, weight, shared, eps, groups, gate_first, out_dtype, sigmoid=False, part=None, stab=None):
    """``y`` fp32 ``[rows, groups * part]`` (``part`` None: the parts are what is normed, nothing between them); see
    csrc/residual_ops.cu for ``stab``."""
    C = y.shape[1] if part is None else groups * part
    out = torch.empty((y.shape[0], C), dtype=out_dtype, device=y.device)
    N.call("ll_gated_group_norm", N.ptr(y), y.shape[1] // groups, N.ptr(stab), N.ptr_at(gate, gate_col), gate.stride(0), N.ptr(weight),
           1 if shared else 0, float(eps), groups, 1 if gate_first else 0, 1 if sigmoid else 0, N.ptr(out), N.dtype_code(out_dtype),
           y.shape[0], C, N.stream())
    return out


@dataclass
class StateSpaceSpec:
    width: int
    heads: int
    vdim: int               # channels per head
    state: int              # state rows per head (N)
    groups: int             # B and C are shared by heads / groups consecutive heads
    norm_groups: int
    taps: int
    eps: float

    def __post_init__(self):
        if self.heads % self.groups or (self.heads * self.vdim) % self.norm_groups:
            raise ValueError(f"{self.heads} heads in {self.groups} groups, inner size in {self.norm_groups} norm parts")

    @property
    def inner(self) -> int:
        return self.heads * self.vdim

    @property
    def conv_channels(self) -> int:
        return self.inner + 2 * self.groups * self.state


class StateSpaceMixer(nn.Module):
    def __init__(self, spec: StateSpaceSpec, dtype: torch.dtype, device) -> None:
        super().__init__()
        s = self.spec = spec
        kw = dict(dtype=dtype, device=device)
        f32 = dict(dtype=torch.float32, device=device)
        self.n_in = 2 * s.inner + 2 * s.groups * s.state + s.heads
        self.w_in = nn.Parameter(torch.zeros((pad8(self.n_in), s.width), **kw), requires_grad=False)
        self.conv = ShortConv(s.conv_channels, s.taps, True, device)
        self.dt_bias = nn.Parameter(torch.zeros(s.heads, **f32), requires_grad=False)
        self.a_log = nn.Parameter(torch.zeros(s.heads, **f32), requires_grad=False)
        self.skip = nn.Parameter(torch.zeros(s.heads, **f32), requires_grad=False)
        self.norm = nn.Parameter(torch.ones(s.inner, **f32), requires_grad=False)
        self.w_o = nn.Parameter(torch.zeros((s.width, s.inner), **kw), requires_grad=False)

    def state_shapes(self, B: int) -> List[Tuple[int, ...]]:
        """fp32 tensors a sequence batch carries: the convolution's inputs, the recurrence's state."""
        s = self.spec
        return [self.conv.state_shape(B), (B, s.heads, s.state, s.vdim)]

    def load(self, get) -> None:
        """``get(suffix)`` returns the tensor '<layer>.mix.<suffix>'."""
        self.w_in.zero_()
        self.w_in[: self.n_in].copy_(get("in"))
        self.conv.load(get("conv"), get("conv.b"))
        self.dt_bias.copy_(get("dt_bias").float())
        self.a_log.copy_(get("A_log").float())
        self.skip.copy_(get("D").float())
        self.norm.copy_(get("norm").float())
        self.w_o.copy_(get("o"))

    def forward(self, u: torch.Tensor, B: int, T: int, pos_ids: torch.Tensor, states) -> List[Tuple[torch.Tensor, float]]:
        s = self.spec
        conv_state, ssm_state = states
        M = B * T
        proj = F.linear(u, self.w_in)
        xbc = self.conv(proj, s.inner, conv_state, pos_ids, B, T, u.dtype, silu=True)
        dt = torch.empty((M, s.heads), dtype=torch.float32, device=u.device)
        decay = torch.empty_like(dt)
        N.call("ll_ssm_gates", N.ptr_at(proj, 2 * s.inner + 2 * s.groups * s.state), N.dtype_code(proj.dtype), proj.stride(0),
               N.ptr(self.dt_bias), N.ptr(self.a_log), N.ptr(dt), N.ptr(decay), M, s.heads, N.stream())
        gn = s.groups * s.state
        y = decay_scan(xbc, s.inner + gn, xbc, s.inner, xbc, 0, decay, False, dt, self.skip, 1.0, ssm_state, pos_ids, B, T,
                       s.heads, s.groups, s.state, s.vdim)
        out = gated_group_norm(y, proj, 0, self.norm, False, s.eps, s.norm_groups, True, u.dtype)
        return [(F.linear(out, self.w_o), 1.0)]


@dataclass
class LinearAttentionSpec:
    width: int
    heads: int
    dim: int                # query / key channels per head
    vdim: int
    tau: float
    decay_rank: int         # inner size of the low-rank decay projection
    eps: float


class GatedLinearAttention(nn.Module):
    def __init__(self, spec: LinearAttentionSpec, dtype: torch.dtype, device) -> None:
        super().__init__()
        s = self.spec = spec
        kw = dict(dtype=dtype, device=device)
        f32 = dict(dtype=torch.float32, device=device)
        hd, hv = s.heads * s.dim, s.heads * s.vdim
        self.cols = dict(q=0, k=hd, v=2 * hd, g=2 * hd + hv, a1=2 * hd + 2 * hv)
        self.n_in = 2 * hd + 2 * hv + s.decay_rank
        self.w_a2 = nn.Parameter(torch.zeros((pad8(hd), s.decay_rank), **kw), requires_grad=False)
        self.b_a2 = nn.Parameter(torch.zeros(hd, **f32), requires_grad=False)
        self.norm = nn.Parameter(torch.ones(s.vdim, **f32), requires_grad=False)
        self.w_o = nn.Parameter(torch.zeros((s.width, hv), **kw), requires_grad=False)

    def state_shapes(self, B: int) -> List[Tuple[int, ...]]:
        s = self.spec
        return [(B, s.heads, s.dim, s.vdim)]

    def in_weight(self, get) -> torch.Tensor:
        """The rows this mixer adds to a stacked input projection: [q; k; v; g; a1]."""
        return torch.cat([get("q"), get("k"), get("v"), get("g"), get("a1")], dim=0)

    def load(self, get) -> None:
        s = self.spec
        self.w_a2.zero_()
        self.w_a2[: s.heads * s.dim].copy_(get("a2"))
        self.b_a2.copy_(get("a2.b").float())
        self.norm.copy_(get("norm").float())
        self.w_o.copy_(get("o"))

    def forward(self, proj: torch.Tensor, col0: int, B: int, T: int, pos_ids: torch.Tensor, states) -> torch.Tensor:
        """``proj``: the stacked input projection's output, this mixer's columns starting at ``col0``."""
        s = self.spec
        c = self.cols
        M = B * T
        hd = s.heads * s.dim
        za = F.linear(proj[:, col0 + c["a1"]: col0 + c["a1"] + s.decay_rank], self.w_a2)
        alpha = torch.empty((M, hd), dtype=torch.float32, device=proj.device)
        N.call("ll_channel_decay", N.ptr(za), N.dtype_code(za.dtype), za.stride(0), N.ptr(self.b_a2), float(s.tau), N.ptr(alpha), M, hd,
               N.stream())
        y = decay_scan(proj, col0 + c["q"], proj, col0 + c["k"], proj, col0 + c["v"], alpha, True, None, None, s.dim ** -0.5,
                       states[0], pos_ids, B, T, s.heads, s.heads, s.dim, s.vdim)
        out = gated_group_norm(y, proj, col0 + c["g"], self.norm, True, s.eps, s.heads, False, proj.dtype)
        return F.linear(out, self.w_o)


@dataclass
class MatrixMemorySpec:
    width: int
    heads: int
    dim: int                # query / key channels per head
    vdim: int
    gate_cap: float         # 0: the gates' pre-activations are not capped
    eps: float


class MatrixMemoryMixer(nn.Module):
    def __init__(self, spec: MatrixMemorySpec, dtype: torch.dtype, device) -> None:
        super().__init__()
        s = self.spec = spec
        kw = dict(dtype=dtype, device=device)
        f32 = dict(dtype=torch.float32, device=device)
        hd, hv = s.heads * s.dim, s.heads * s.vdim
        self.cols = dict(q=0, k=hd, v=2 * hd, g=2 * hd + hv, i=2 * hd + 2 * hv, f=2 * hd + 2 * hv + s.heads)
        self.n_in = 2 * hd + 2 * hv + 2 * s.heads
        self.w_in = nn.Parameter(torch.zeros((pad8(self.n_in), s.width), **kw), requires_grad=False)
        self.bias_i = nn.Parameter(torch.zeros(s.heads, **f32), requires_grad=False)
        self.bias_f = nn.Parameter(torch.zeros(s.heads, **f32), requires_grad=False)
        self.norm = nn.Parameter(torch.ones(hv, **f32), requires_grad=False)
        self.w_o = nn.Parameter(torch.zeros((s.width, hv), **kw), requires_grad=False)

    def state_shapes(self, B: int) -> List[Tuple[int, ...]]:
        """fp32: the memory with its normaliser as the last column, the stabiliser."""
        s = self.spec
        return [(B, s.heads, s.dim, s.vdim + 1), (B, s.heads)]

    def load(self, get) -> None:
        """``get(suffix)`` returns the tensor '<layer>.mix.<suffix>'."""
        self.w_in.zero_()
        self.w_in[: self.n_in].copy_(torch.cat([get(n).to(self.w_in.dtype) for n in self.cols], dim=0))
        self.bias_i.copy_(get("i.b").float())
        self.bias_f.copy_(get("f.b").float())
        self.norm.copy_(get("norm").float())
        self.w_o.copy_(get("o"))

    def forward(self, u: torch.Tensor, B: int, T: int, pos_ids: torch.Tensor, states) -> torch.Tensor:
        s = self.spec
        c = self.cols
        memory, stabiliser = states
        M = B * T
        proj = F.linear(u, self.w_in)
        keep = torch.empty((M, s.heads), dtype=torch.float32, device=u.device)
        take, stab = torch.empty_like(keep), torch.empty_like(keep)
        N.call("ll_matrix_memory_gates", N.ptr_at(proj, c["i"]), N.ptr_at(proj, c["f"]), N.dtype_code(proj.dtype), proj.stride(0),
               N.ptr(self.bias_i), N.ptr(self.bias_f), float(s.gate_cap), N.ptr(stabiliser), N.ptr(pos_ids), N.ptr(keep), N.ptr(take),
               N.ptr(stab), B, T, s.heads, N.stream())
        y = decay_scan(proj, c["q"], proj, c["k"], proj, c["v"], keep, False, take, None, s.dim ** -0.5, memory, pos_ids, B, T,
                       s.heads, s.heads, s.dim, s.vdim + 1, unit_col=True)
        out = gated_group_norm(y, proj, c["g"], self.norm, False, s.eps, s.heads, False, proj.dtype, sigmoid=True, part=s.vdim, stab=stab)
        return F.linear(out, self.w_o)
