"""Latent attention: keys and values are up-projections of one low-rank row per token, plus one rotated key part that all
heads share; only that row is cached.

With h the mixer's input, per token
    [q | g | d] = W_in h            q: heads x [nope_dim | rot_dim];  g: one gate logit per head;  d: [kv_rank | rot_dim]
    c = rmsnorm(d[:kv_rank]) * w    k_rot = rope(d[kv_rank:])          -> the cache row [c | k_rot]
    score(i, j, head) = (q_nope . (W_uk c_j) + rope(q_rot) . k_rot_j) * scale,   j in the sliding window of i
    out = W_o concat_heads( sigmoid(g) * sum_j softmax_j(score) (W_uv c_j) )
The kernels work in latent space: W_uk is absorbed into the query (q_lat = W_uk^T q_nope, a batched GEMM over heads) and
W_uv is applied to the weighted sum of the c_j, so every head reads the same cache row once, in prefill and in decoding
alike.  A layer built with ``kv_from`` has no down-projection: it reads another layer's rows with its own W_uk, W_uv,
queries and window.

Variations, all parameters of the spec:
* ``q_rank``: the queries pass a latent of their own, ``q = W_uq (rmsnorm(W_dq h) * w_q)``; the input projection is then
  ``[dq | g | d]``.
* ``gate``: "head" (one logit per head, as above), "element" (``sigmoid(W_g h)`` holds heads * v_dim numbers, one for every
  number the heads put out; applied after W_uv) or "none".
* ``rot_layout``: "interleaved" pairs dimension 2i with 2i+1; "half" pairs i with i + rot_dims/2.  The kernels turn
  interleaved pairs; a "half" checkpoint has the rows of its rotated query and key parts reordered once at load time (the
  same reordering on both sides of the dot product leaves the scores as they are).
* ``rotary``: a ``rotary.RotarySpec`` whose ``table()`` (rescaled frequencies, magnitude) replaces the plain table.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn as nn
from torch.nn import functional as F

from . import _native as N
from .rotary import RotarySpec


@dataclass
class LatentAttentionSpec:
    width: int
    heads: int
    nope_dim: int                 # un-rotated query / key dimensions per head
    rot_dim: int                  # rotated dimensions per head (one key part for all heads)
    v_dim: int
    kv_rank: int
    window: Optional[int]         # position i sees i - window + 1 .. i; None: everything before it
    scale: float
    rot_base: float = 10000.0
    rot_dims: Optional[int] = None   # the first rot_dims of the rotated part turn, the rest pass; default all
    eps: float = 1e-5
    kv_from: Optional[int] = None    # index of the layer whose cache rows this layer reads
    q_rank: Optional[int] = None     # queries through a normed latent of this size; None: q = W_q h
    gate: str = "head"               # "head" | "element" | "none"
    rot_layout: str = "interleaved"  # "interleaved" | "half"
    rotary: Optional[RotarySpec] = None   # rescaled frequencies and magnitude; None: base^(-2i/rot_dims)

    def __post_init__(self):
        if self.rotary is not None:
            self.rot_dims, self.rot_base = self.rotary.dims, self.rotary.base
        if self.gate not in ("head", "element", "none") or self.rot_layout not in ("interleaved", "half"):
            raise ValueError(f"latent attention: gate {self.gate!r}, rotary layout {self.rot_layout!r}")
        if self.rot_dims is None:
            self.rot_dims = self.rot_dim
        if self.rot_dims % 2 or not 0 <= self.rot_dims <= self.rot_dim:
            raise ValueError(f"rot_dims {self.rot_dims} must be even and at most rot_dim {self.rot_dim}")

    @property
    def row(self) -> int:
        return self.kv_rank + self.rot_dim

    @property
    def q_head(self) -> int:
        return self.nope_dim + self.rot_dim

    @property
    def gate_cols(self) -> int:
        return {"head": self.heads, "element": self.heads * self.v_dim, "none": 0}[self.gate]

    def rope_table(self, n_pos: int, device) -> torch.Tensor:
        if self.rotary is not None:
            return self.rotary.table(n_pos, device)
        return build_rope_table(n_pos, self.rot_dims, self.rot_base, device)

    def rot_order(self) -> torch.Tensor:
        """Where every dimension of the stored rotated part sits in the checkpoint's: the identity, or for the "half" layout
        (i paired with i + rot_dims/2) the order that puts the two of a pair side by side."""
        order = list(range(self.rot_dim))
        if self.rot_layout == "half":
            half = self.rot_dims // 2
            for i in range(half):
                order[2 * i], order[2 * i + 1] = i, i + half
        return torch.tensor(order, dtype=torch.long)


def build_rope_table(n_pos: int, rot_dims: int, base: float, device) -> torch.Tensor:
    """``[n_pos, rot_dims / 2, 2]`` fp32 (cos, sin) of ``pos * base^(-2i / rot_dims)``; angles formed in float64 so that the
    table is exact to fp32 rounding at any position."""
    i = torch.arange(rot_dims // 2, dtype=torch.float64)
    freq = torch.pow(torch.tensor(float(base), dtype=torch.float64), -2.0 * i / max(rot_dims, 1))
    ang = torch.arange(n_pos, dtype=torch.float64)[:, None] * freq[None]
    if rot_dims == 0:                       # nothing turns: a table the kernels never index, but a valid address
        return torch.zeros((n_pos, 1, 2), dtype=torch.float32, device=device)
    return torch.stack((ang.cos(), ang.sin()), dim=-1).float().contiguous().to(device)


class LatentAttention(nn.Module):
    def __init__(self, spec: LatentAttentionSpec, dtype: torch.dtype, device) -> None:
        super().__init__()
        s = self.spec = spec
        self.owns_cache = s.kv_from is None
        self.q_cols = s.heads * s.q_head
        self.q_in = s.q_rank if s.q_rank is not None else self.q_cols       # what the input projection holds for the queries
        self.gate_col0 = self.q_in
        self.kv_col0 = self.q_in + s.gate_cols
        n_in = self.kv_col0 + (s.row if self.owns_cache else 0)
        self.n_in = n_in
        n_in = (n_in + 7) // 8 * 8          # rows of zeros up to a multiple of 8: the library's fast GEMMs want aligned outputs
        kw = dict(dtype=dtype, device=device)
        self.w_in = nn.Parameter(torch.empty((n_in, s.width), **kw), requires_grad=False)          # [W_q | W_dq; W_g; W_dkv]
        self.q_norm = nn.Parameter(torch.ones(s.q_rank, dtype=torch.float32, device=device), requires_grad=False) \
            if s.q_rank is not None else None
        self.w_uq = nn.Parameter(torch.empty((self.q_cols, s.q_rank), **kw), requires_grad=False) if s.q_rank is not None else None
        self.w_uk = nn.Parameter(torch.empty((s.heads, s.nope_dim, s.kv_rank), **kw), requires_grad=False)
        self.w_uv_t = nn.Parameter(torch.empty((s.heads, s.kv_rank, s.v_dim), **kw), requires_grad=False)
        self.w_o = nn.Parameter(torch.empty((s.width, s.heads * s.v_dim), **kw), requires_grad=False)
        self.kv_norm = nn.Parameter(torch.ones(s.kv_rank, dtype=torch.float32, device=device), requires_grad=False) \
            if self.owns_cache else None

    def load(self, get) -> None:
        """``get(suffix)`` returns the tensor '<layer>.mix.<suffix>' ([out, in] for the Linears)."""
        s = self.spec
        order = s.rot_order()

        def q_rows(w):                      # the rotated part of every head's query rows in the stored order
            w = w.reshape(s.heads, s.q_head, -1)
            return torch.cat([w[:, : s.nope_dim], w[:, s.nope_dim:][:, order]], dim=1).reshape(self.q_cols, -1)

        parts = [get("dq")] if s.q_rank is not None else [q_rows(get("q"))]
        if s.gate != "none":
            parts.append(get("g"))
        if self.owns_cache:
            dkv = get("dkv")
            parts.append(torch.cat([dkv[: s.kv_rank], dkv[s.kv_rank:][order]], dim=0))
        self.w_in.zero_()
        self.w_in[: self.n_in].copy_(torch.cat([p.to(self.w_in.dtype) for p in parts], dim=0))
        if s.q_rank is not None:
            self.q_norm.copy_(get("dq.norm").float())
            self.w_uq.copy_(q_rows(get("uq")))
        self.w_uk.copy_(get("uk").reshape(s.heads, s.nope_dim, s.kv_rank))
        self.w_uv_t.copy_(get("uv").reshape(s.heads, s.v_dim, s.kv_rank).transpose(1, 2))
        self.w_o.copy_(get("o"))
        if self.owns_cache:
            self.kv_norm.copy_(get("dkv.norm").float())

    def forward(self, x_act: torch.Tensor, B: int, T: int, pos_ids: torch.Tensor, rope: torch.Tensor, cache: torch.Tensor,
                splits: int = 1) -> torch.Tensor:
        """x_act ``[B*T, width]`` -> ``[B*T, width]``; ``cache`` ``[B, S, row]`` is this layer's or its source's (already
        appended to by the source in this step)."""
        s = self.spec
        M = B * T
        dt = N.dtype_code(x_act.dtype)
        st = N.stream()
        proj = F.linear(x_act, self.w_in)                                     # [M, n_in]
        S = cache.shape[1]
        if self.owns_cache:
            N.call("ll_latent_kv_append", N.ptr(proj), dt, proj.shape[1], self.kv_col0, N.ptr(self.kv_norm), float(s.eps),
                   N.ptr(rope), N.ptr(pos_ids), N.ptr(cache), B, T, s.kv_rank, s.rot_dim, s.rot_dims, S, st)
        if s.q_rank is not None:
            cq = torch.empty((M, s.q_rank), dtype=x_act.dtype, device=x_act.device)
            N.call("ll_row_norm", N.ptr(proj), proj.shape[1], N.ptr(self.q_norm), float(s.eps), N.ptr(cq), s.q_rank, dt, M, s.q_rank, st)
            q = F.linear(cq, self.w_uq)                                       # [M, heads * q_head]
        else:
            q = proj
        q_nope = q[:, : self.q_cols].view(M, s.heads, s.q_head)[:, :, : s.nope_dim].transpose(0, 1)   # [H, M, nope] view
        q_lat = torch.bmm(q_nope, self.w_uk)                                  # [H, M, kv_rank]
        o_lat = torch.empty_like(q_lat)
        scratch = None
        if splits > 1:
            scratch = torch.empty(N.call_ret("ll_latent_attn_scratch_bytes", M, s.heads, s.kv_rank, splits) // 4,
                                  dtype=torch.float32, device=x_act.device)
        head_gate = self.gate_col0 if (s.gate == "head" and s.q_rank is None) else -1
        N.call("ll_latent_attn", N.ptr(q_lat), M * s.kv_rank, s.kv_rank, N.ptr(q), q.shape[1], s.nope_dim, s.q_head,
               head_gate, N.ptr(rope), N.ptr(pos_ids), N.ptr(cache), N.ptr(o_lat), M * s.kv_rank, s.kv_rank, dt, B, T,
               s.heads, s.kv_rank, s.rot_dim, s.rot_dims, S, s.window if s.window is not None else 0, float(s.scale), splits,
               N.ptr(scratch), st)
        o = torch.bmm(o_lat, self.w_uv_t).transpose(0, 1).reshape(M, s.heads * s.v_dim)     # [M, heads * v_dim]
        if s.gate == "element":
            N.call("ll_sigmoid_gate_mul", N.ptr(o), o.shape[1], N.ptr_at(proj, self.gate_col0), proj.shape[1], N.ptr(o), o.shape[1], dt,
                   M, s.heads * s.v_dim, st)
        elif s.gate == "head" and s.q_rank is not None:
            raise NotImplementedError("a gate per head beside latent queries")
        return F.linear(o, self.w_o)
