"""Bededra: a decoder-only model whose layers add two branches to an fp32 stream, both reading the same stream through
their own norm,

    x <- x + mixer( h1 + shortconv(h1) ) + ff( h2 ),        h1 = rmsnorm(x) * w1,   h2 = rmsnorm(x) * w2

with mixers of two kinds in any order - ``mamba2`` (selective state space, recurrence.StateSpaceMixer) and ``parallel``
(window attention with kept first tokens beside gated linear attention, their outputs added with fixed scales) - and
feed-forwards that are dense (squared relu) or a mixture of silu-gated experts chosen among the best groups of experts.

Per-sequence memory: every layer keeps the last ``taps - 1`` normed inputs of its short convolution; a ``mamba2`` layer the
inputs of its inner convolution and its state; a ``parallel`` layer key / value rows (kept tokens + ring) and the state of
the linear attention.  All of it lives in tensors from the package's ``TensorPool`` with stable addresses, written in
place; nothing is cleared between requests: the kernels start a sequence from nothing when its first position is 0.
``forward`` is the package's common step function (stepping.PortionedDecoder).
"""
from __future__ import annotations

import json
from dataclasses import dataclass, field
from pathlib import Path
from typing import Dict, List, Optional, Tuple, Union

import torch
import torch.nn as nn
from torch.nn import functional as F

from . import _native as N
from .cache import TensorPool
from .feed_forward import DenseFF
from .moe import MoE, MoESpec
from .recurrence import GatedLinearAttention, LinearAttentionSpec, StateSpaceMixer, StateSpaceSpec, pad8
from .short_conv import ShortConv
from .stepping import PortionedDecoder, add_norm_pair, head_logits
from .window_attention import WindowAttention, WindowAttentionSpec

ARCHITECTURE = "Bededra"


@dataclass
class ParallelSpec:
    left: WindowAttentionSpec
    right: LinearAttentionSpec
    left_scale: float
    right_scale: float


@dataclass
class DenseSpec:
    ff: int
    act: str = "relu2"


@dataclass
class BededraLayer:
    kind: str                                          # "mamba2" | "parallel"
    mixer: Union[StateSpaceSpec, ParallelSpec]
    mlp: Union[None, DenseSpec, MoESpec]


@dataclass
class BededraConfig:
    vocab: int
    width: int
    eps: float
    canon_taps: int                                    # 0: layers read their normed input as it is
    layers: List[BededraLayer] = field(default_factory=list)

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def n_layer(self) -> int:
        return len(self.layers)

    @property
    def block_size(self) -> int:
        """No position table: any length the memory is sized for."""
        return 1 << 30

    @classmethod
    def from_dict(cls, cfg: dict, shapes: Optional[Dict[str, Tuple[int, ...]]] = None) -> "BededraConfig":
        """From the dictionary of a ``config.json``; sizes it leaves out are taken from the tensors' shapes."""
        shapes = shapes or {}

        def pick(value, name, axis, div=1):
            if value is not None:
                return int(value)
            if name in shapes:
                return shapes[name][axis] // div
            raise KeyError(f"config.json gives no size that tensor {name!r} would determine, and the tensor is absent")

        width = pick(cfg.get("width"), "embed", 1)
        vocab = pick(cfg.get("vocab"), "embed", 0)
        eps = float(cfg["norm"]["eps"])
        canon = cfg.get("canon") or {}
        taps = int(canon["taps"]) if canon.get("taps") is not None else (shapes["l0.canon1"][1] if "l0.canon1" in shapes else 0)
        layers = []
        for i, lc in enumerate(cfg["layers"]):
            kind, m, p = lc.get("type"), lc["mixer"], f"l{i}.mix."
            if kind == "mamba2":
                heads = pick(m.get("heads"), p + "A_log", 0)
                mixer = StateSpaceSpec(width=width, heads=heads, vdim=pick(m.get("vdim"), p + "o", 1, heads), state=int(m["state"]),
                                       groups=int(m.get("groups", 1)), norm_groups=int(m.get("norm_groups", 1)),
                                       taps=pick(m.get("conv"), p + "conv", 1), eps=eps)
            elif kind == "parallel":
                l, r = m["left"], m["right"]
                lh = pick(l.get("heads"), p + "left.r1", 0)
                lg = int(l["kv_heads"]) if l.get("kv_heads") is not None else lh
                mask = l.get("mask") or {}
                left = WindowAttentionSpec(
                    width=width, heads=lh, kv_heads=lg, dim=pick(l.get("dim"), p + "left.q", 0, lh),
                    vdim=pick(l.get("vdim"), p + "left.v", 0, lg), scale=float(l["scale"]), softcap=float(l.get("softcap") or 0.0),
                    window=int(mask["size"]) if mask.get("size") is not None else None, keep_first=int(mask.get("keep_first") or 0))
                rh = int(r["heads"])
                right = LinearAttentionSpec(width=width, heads=rh, dim=pick(r.get("dim"), p + "right.q", 0, rh),
                                            vdim=pick(r.get("vdim"), p + "right.v", 0, rh), tau=float(r["tau"]),
                                            decay_rank=pick(r.get("decay_rank"), p + "right.a1", 0), eps=eps)
                mixer = ParallelSpec(left, right, float(m.get("left_scale", 1.0)), float(m.get("right_scale", 1.0)))
            else:
                raise ValueError(f"layer {i}: unknown mixer type {kind!r}")
            f, q = lc.get("mlp"), f"l{i}.mlp."
            if f is None:
                mlp = None
            elif f.get("kind") == "dense":
                mlp = DenseSpec(ff=pick(f.get("ff"), q + "up", 0))
            elif f.get("kind") == "moe":
                r = f["router"]
                g = r.get("groups") or {}
                count = int(g.get("count", 1))
                mlp = MoESpec(width=width, experts=pick(r.get("experts"), q + "router", 0), top=int(r["top"]),
                              ff=pick((f.get("expert") or {}).get("ff"), q + "e0.gate", 0), limit=float("inf"), alpha=1.0,
                              up_shift=0.0, score="all", groups=count, keep_groups=int(g.get("keep", count)), router_bias=False)
            else:
                raise ValueError(f"layer {i}: unknown feed-forward kind {f.get('kind')!r}")
            layers.append(BededraLayer(kind, mixer, mlp))
        return cls(vocab=vocab, width=width, eps=eps, canon_taps=taps, layers=layers)


class ParallelMixer(nn.Module):
    """Window attention and gated linear attention side by side on one stacked input projection."""

    def __init__(self, spec: ParallelSpec, dtype, device) -> None:
        super().__init__()
        self.spec = spec
        self.left = WindowAttention(spec.left, dtype, device)
        self.right = GatedLinearAttention(spec.right, dtype, device)
        self.right_col0 = self.left.n_in
        self.n_in = self.left.n_in + self.right.n_in
        self.w_in = nn.Parameter(torch.zeros((pad8(self.n_in), spec.left.width), dtype=dtype, device=device), requires_grad=False)

    def load(self, get) -> None:
        lget, rget = (lambda s: get("left." + s)), (lambda s: get("right." + s))
        self.w_in.zero_()
        self.w_in[: self.n_in].copy_(torch.cat([self.left.in_weight(lget).to(self.w_in.dtype),
                                                self.right.in_weight(rget).to(self.w_in.dtype)], dim=0))
        self.left.load(lget)
        self.right.load(rget)

    def forward(self, u, B, T, pos_ids, caches, states, splits):
        proj = F.linear(u, self.w_in)
        return [(self.left(proj, 0, B, T, pos_ids, caches, splits), self.spec.left_scale),
                (self.right(proj, self.right_col0, B, T, pos_ids, states), self.spec.right_scale)]


class BededraBlock(nn.Module):
    def __init__(self, index: int, layer: BededraLayer, cfg: BededraConfig, dtype, device) -> None:
        super().__init__()
        f32 = dict(dtype=torch.float32, device=device)
        self.index, self.kind = index, layer.kind
        self.norm1 = nn.Parameter(torch.ones(cfg.width, **f32), requires_grad=False)
        self.canon = ShortConv(cfg.width, cfg.canon_taps, False, device) if cfg.canon_taps > 0 else None
        self.mix = StateSpaceMixer(layer.mixer, dtype, device) if layer.kind == "mamba2" else ParallelMixer(layer.mixer, dtype, device)
        self.mlp = None
        if isinstance(layer.mlp, DenseSpec):
            self.mlp = DenseFF(cfg.width, layer.mlp.ff, layer.mlp.act, dtype, device)
        elif isinstance(layer.mlp, MoESpec):
            self.mlp = MoE(layer.mlp, dtype, device)
        self.norm2 = nn.Parameter(torch.ones(cfg.width, **f32), requires_grad=False) if self.mlp is not None else None

    def load(self, get) -> None:
        p = f"l{self.index}."
        self.norm1.copy_(get(p + "norm1").float())
        if self.canon is not None:
            self.canon.load(get(p + "canon1"))
        self.mix.load(lambda s: get(p + "mix." + s))
        if self.mlp is not None:
            self.norm2.copy_(get(p + "norm2").float())
            self.mlp.load(lambda s: get(p + "mlp." + s))

    def state_shapes(self, B: int) -> List[Tuple[int, ...]]:
        """fp32 state: [canon inputs] + the mixer's."""
        shapes = [self.canon.state_shape(B)] if self.canon is not None else []
        if self.kind == "mamba2":
            return shapes + self.mix.state_shapes(B)
        return shapes + self.mix.right.state_shapes(B)


class Bededra(PortionedDecoder):
    architecture = ARCHITECTURE

    def __init__(self, config: BededraConfig, dtype: torch.dtype = torch.bfloat16, device="cuda") -> None:
        super().__init__()
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError("Bededra runs in bfloat16 or float32")
        self.config = config
        self.dtype, self.device = dtype, torch.device(device)
        kw = dict(dtype=dtype, device=self.device)
        self.embed = nn.Parameter(torch.empty((config.vocab, config.width), **kw), requires_grad=False)
        self.blocks = nn.ModuleList(BededraBlock(i, l, config, dtype, self.device) for i, l in enumerate(config.layers))
        self.final_norm = nn.Parameter(torch.ones(config.width, dtype=torch.float32, device=self.device), requires_grad=False)
        self.head = nn.Parameter(torch.zeros((pad8(config.vocab), config.width), **kw), requires_grad=False)
        self._pool = TensorPool(max_sets=4, on_evict=self._drop_graphs)
        self._attn = [b.mix.left.spec for b in self.blocks if b.kind == "parallel"]
        self.states: List[torch.Tensor] = []          # fp32, every layer's in order (see BededraBlock.state_shapes)
        self.kv_caches: List[torch.Tensor] = []       # (keys, values) of every parallel layer in order
        self._rings: Tuple[int, ...] = ()
        self._batch = 0

    # ------------------------------------------------------------------ weights
    @torch.no_grad()
    def load_tensors(self, get) -> None:
        """``get(name)`` returns the checkpoint tensor of that name (any float dtype, CPU or GPU)."""
        self.embed.copy_(get("embed"))
        self.head.zero_()
        self.head[: self.config.vocab].copy_(get("head"))
        self.final_norm.copy_(get("final.norm").float())
        for b in self.blocks:
            b.load(get)

    @classmethod
    def from_dir(cls, path, dtype: torch.dtype = torch.bfloat16, device="cuda") -> "Bededra":
        """A folder with ``config.json`` and ``model.safetensors``."""
        from .safetensors_io import SafetensorsFile

        path = Path(path)
        with open(path / "config.json") as f:
            cfg = json.load(f)
        with SafetensorsFile(path / "model.safetensors") as st:
            model = cls(BededraConfig.from_dict(cfg, st.shapes()), dtype=dtype, device=device)
            model.load_tensors(st.get)
        return model.eval()

    # ------------------------------------------------------------------ memory
    def reset_cache(self) -> None:
        """The sequences end: their slots are given back (the tensors stay allocated; the next sequence starts at position
        0, where the kernels take nothing from them)."""
        self.states, self.kv_caches, self._rings, self._batch = [], [], (), 0

    def _ring_plan(self, max_seq_length: int) -> Tuple[int, ...]:
        portion = min(self.prefill_portion, max_seq_length)
        return tuple(s.ring(max_seq_length, portion) for s in self._attn)

    def _begin(self, B: int, max_seq_length: int, keep: bool) -> None:
        rings = self._ring_plan(max_seq_length)
        if self.states and self._batch == B and self._rings == rings:
            return
        st_shapes = [s for b in self.blocks for s in b.state_shapes(B)]
        kv_shapes = []
        n = 0
        for b in self.blocks:
            if b.kind == "parallel":
                kv_shapes += b.mix.left.cache_shapes(B, rings[n])
                n += 1
        if keep:
            self.states = self._pool.get(st_shapes, torch.float32, self.device, zero=False)
            self.kv_caches = self._pool.get(kv_shapes, self.dtype, self.device, zero=False) if kv_shapes else []
        else:                      # a forward that keeps nothing: scratch memory, the pool's sets stay as they are
            self.states = [torch.empty(s, dtype=torch.float32, device=self.device) for s in st_shapes]
            self.kv_caches = [torch.empty(s, dtype=self.dtype, device=self.device) for s in kv_shapes]
        self._rings, self._batch = rings, B

    def _piece(self, max_seq_length: int) -> int:
        return min([max_seq_length] + [s.portion(r, max_seq_length) for s, r in zip(self._attn, self._rings)])

    def _graph_key(self, B: int) -> tuple:
        return (B, self._rings, self.states[0].data_ptr(), self.kv_caches[0].data_ptr() if self.kv_caches else 0)

    def _save_memory(self):
        saved = (self.states, self.kv_caches, self._rings, self._batch)
        self.states, self.kv_caches, self._rings, self._batch = [], [], (), 0
        return saved

    def _restore_memory(self, saved) -> None:
        self.states, self.kv_caches, self._rings, self._batch = saved

    def _warm_step(self, s_idx, s_pos) -> None:
        """The eager runs before a capture advance the recurrent state; put it back afterwards (the cache row they write is
        the one the real step writes again)."""
        kept = [t.clone() for t in self.states]
        super()._warm_step(s_idx, s_pos)
        for t, k in zip(self.states, kept):
            t.copy_(k)

    # ------------------------------------------------------------------ forward
    def _forward_portion(self, idx: torch.Tensor, pos_ids: torch.Tensor, sel) -> torch.Tensor:
        cfg = self.config
        B, T = idx.shape
        M, E = B * T, cfg.width
        dev = idx.device
        act = N.dtype_code(self.dtype)
        x = torch.empty((M, E), dtype=torch.float32, device=dev)
        N.call("ll_embed_scaled", N.ptr(self.embed), act, N.ptr(idx.reshape(-1).contiguous()), 1.0, N.ptr(x), None, act, M, E, N.stream())
        sms = N.call_ret("ll_sm_count")
        pending: List[Tuple[torch.Tensor, float]] = []
        si = ci = 0
        for i, blk in enumerate(self.blocks):
            h1 = torch.empty((M, E), dtype=torch.float32 if blk.canon is not None else self.dtype, device=dev)
            h2 = torch.empty((M, E), dtype=self.dtype, device=dev) if blk.mlp is not None else None
            add_norm_pair(x, pending, blk.norm1, blk.norm2, cfg.eps, h1, h2, self.dtype)
            if self.layer_probe is not None and i > 0:
                self.layer_probe(i - 1, x)
            if blk.canon is not None:
                u = blk.canon(h1, 0, self.states[si], pos_ids, B, T, self.dtype, residual=True)
                si += 1
            else:
                u = h1
            if blk.kind == "mamba2":
                pending = blk.mix(u, B, T, pos_ids, self.states[si:si + 2])
                si += 2
            else:
                spec = blk.mix.left.spec
                span = min(spec.window if spec.window is not None else (1 << 30), self._rings[ci // 2]) + spec.keep_first
                splits = max(1, min(64, (2 * sms) // max(1, M), (span + 63) // 64))     # few queries: share a long window among blocks
                pending = blk.mix(u, B, T, pos_ids, self.kv_caches[ci:ci + 2], self.states[si:si + 1], splits)
                ci += 2
                si += 1
            if blk.mlp is not None:
                pending = pending + [(blk.mlp(h2), 1.0)]
        if sel is not None and len(sel) == 0:      # the step only fills the memory
            return torch.empty((B, 0, cfg.vocab), dtype=torch.float32, device=dev)
        add_norm_pair(x, pending, None, None, cfg.eps, None, None, self.dtype)
        if self.layer_probe is not None:
            self.layer_probe(cfg.n_layer - 1, x)
        if sel is not None:
            ridx = (torch.arange(B, device=dev)[:, None] * T + torch.tensor(sel, device=dev, dtype=torch.long)[None]).reshape(-1)
            x = x.index_select(0, ridx).contiguous()
        xn = torch.empty((x.shape[0], E), dtype=self.dtype, device=dev)
        add_norm_pair(x, [], self.final_norm, None, cfg.eps, xn, None, self.dtype)
        return head_logits(xn, self.head, cfg.vocab).reshape(B, -1, cfg.vocab)
