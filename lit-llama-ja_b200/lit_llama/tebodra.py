"""Tebodra: a decoder-only model of pre-norm sublayers on an fp32 stream, both scaled by one residual multiplier r,

    x <- x + r * mixer( rmsnorm(x) * (1 + w1) );      x <- x + r * ff( rmsnorm(x) * (1 + w2) )     (ff may be absent)

with mixers of three kinds in whatever order ``config.json`` lists them:

* ``attention``   - softmax attention (softmax_attention.SoftmaxAttention) whose q and k pass a short causal filter, whose
  values are the filtered keys before the rotation, with capped scores and band-wise rescaled rotary frequencies;
* ``attention_2`` - the same module with a norm over the whole q / k projections, a chunk-local mask, a sink in the softmax
  denominator and linearly rescaled frequencies; with ``kv_from`` it reads the ring of an earlier layer instead of its own;
* ``mlstm``       - matrix memory with exponential gates (recurrence.MatrixMemoryMixer).

Feed-forward: ``W_down gelu(W_up h)`` (erf form).  Output: ``head . (rmsnorm(x) * (1 + w_f))``.  The norm weights are
stored around zero; ``1 + w`` is formed once at load time in fp32.

Per-sequence memory: key / value rings of the attention layers that own them (a borrowing layer holds none), the inputs of
the short filters, the matrix memories with their normalisers and stabilisers.  All of it lives in tensors from the package's
``TensorPool`` with stable addresses, written in place; nothing is cleared between requests: the kernels start a sequence
from nothing when its first position is 0.  ``forward`` is the package's common step function (stepping.PortionedDecoder).
"""
from __future__ import annotations

import json
from dataclasses import dataclass, field
from pathlib import Path
from typing import Dict, List, Optional, Tuple, Union

import torch
import torch.nn as nn

from . import _native as N
from .cache import TensorPool, max_portion, ring_length
from .feed_forward import DenseFF
from .recurrence import MatrixMemoryMixer, MatrixMemorySpec, pad8
from .rotary import RotarySpec
from .softmax_attention import SoftmaxAttention, SoftmaxAttentionSpec
from .stepping import PortionedDecoder, add_norm_pair, head_logits

ARCHITECTURE = "Tebodra"


@dataclass
class TebodraLayer:
    kind: str                                          # "attention" | "attention_2" | "mlstm"
    mixer: Union[SoftmaxAttentionSpec, MatrixMemorySpec]
    ff: Optional[int]                                  # inner size of the dense feed-forward; None: the layer has none
    act: str = "gelu"


@dataclass
class TebodraConfig:
    vocab: int
    width: int
    eps: float
    residual_mult: float
    layers: List[TebodraLayer] = field(default_factory=list)

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
    def from_dict(cls, cfg: dict, shapes: Optional[Dict[str, Tuple[int, ...]]] = None) -> "TebodraConfig":
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
        layers: List[TebodraLayer] = []
        for i, lc in enumerate(cfg["layers"]):
            kind, m, p = lc.get("type"), lc["mixer"], f"l{i}.mix."
            if kind in ("attention", "attention_2"):
                second = kind == "attention_2"
                src = m.get("kv_from")
                if src is not None:
                    src = int(src)
                    if not 0 <= src < i or not isinstance(layers[src].mixer, SoftmaxAttentionSpec) or layers[src].mixer.kv_from is not None:
                        raise ValueError(f"layer {i}: kv_from {src} does not name an earlier attention layer with keys of its own")
                dim = int(m["dim"])
                heads = pick(m.get("heads"), p + "q", 0, dim)
                kv_heads = int(m["kv_heads"]) if m.get("kv_heads") is not None else (layers[src].mixer.kv_heads if src is not None
                                                                                       else pick(None, p + "k", 0, dim))
                mask = m.get("mask") or {}
                taps = m.get("conv")
                if taps is None:
                    taps = shapes[p + "q.conv"][1] if p + "q.conv" in shapes else 0
                # the kind fixes which parts a layer has; where the tensors are known, their presence has the last word
                has = (lambda name, default: (p + name in shapes) if shapes else default)
                sink, qk_norm = has("sink", second), has("q.norm", second)
                own_values = has("v", second) if src is None else layers[src].mixer.own_values
                mixer = SoftmaxAttentionSpec(
                    width=width, heads=heads, kv_heads=kv_heads, dim=dim, vdim=int(m["vdim"]) if m.get("vdim") is not None else dim,
                    scale=float(m["scale"]) if m.get("scale") is not None else dim ** -0.5, eps=eps,
                    rotary=RotarySpec.from_dict(m.get("rot"), dim), softcap=float(m.get("softcap") or 0.0),
                    window=None, chunk=int(mask["size"]) if mask.get("size") is not None else None, sink=sink, qk_norm=qk_norm,
                    conv_taps=int(taps), own_values=own_values, kv_from=src)
                if src is not None:
                    o = layers[src].mixer
                    if (o.kv_heads, o.dim, o.vdim) != (mixer.kv_heads, mixer.dim, mixer.vdim):
                        raise ValueError(f"layer {i}: its key/value heads differ from those of layer {src}, whose ring it reads")
            elif kind == "mlstm":
                heads = int(m["heads"])
                mixer = MatrixMemorySpec(width=width, heads=heads, dim=pick(m.get("dim"), p + "q", 0, heads),
                                         vdim=pick(m.get("vdim"), p + "v", 0, heads), gate_cap=float(m.get("gate_cap") or 0.0), eps=eps)
            else:
                raise ValueError(f"layer {i}: unknown mixer type {kind!r}")
            f = lc.get("mlp")
            if f is None:
                ff = None
            elif f.get("kind", "dense") == "dense":
                ff = pick(f.get("ff"), f"l{i}.mlp.up", 0)
            else:
                raise ValueError(f"layer {i}: unknown feed-forward kind {f.get('kind')!r}")
            layers.append(TebodraLayer(kind, mixer, ff))
        return cls(vocab=vocab, width=width, eps=eps, residual_mult=float(cfg.get("residual_mult", 1.0)), layers=layers)


class TebodraBlock(nn.Module):
    def __init__(self, index: int, layer: TebodraLayer, cfg: TebodraConfig, dtype, device) -> None:
        super().__init__()
        f32 = dict(dtype=torch.float32, device=device)
        self.index, self.kind = index, layer.kind
        self.norm1 = nn.Parameter(torch.ones(cfg.width, **f32), requires_grad=False)          # holds 1 + w
        self.mix = MatrixMemoryMixer(layer.mixer, dtype, device) if layer.kind == "mlstm" else SoftmaxAttention(layer.mixer, dtype, device)
        self.mlp = DenseFF(cfg.width, layer.ff, layer.act, dtype, device) if layer.ff is not None else None
        self.norm2 = nn.Parameter(torch.ones(cfg.width, **f32), requires_grad=False) if self.mlp is not None else None

    def load(self, get) -> None:
        p = f"l{self.index}."
        self.norm1.copy_(1.0 + get(p + "norm1").float())
        self.mix.load(lambda s: get(p + "mix." + s))
        if self.mlp is not None:
            self.norm2.copy_(1.0 + get(p + "norm2").float())
            self.mlp.load(lambda s: get(p + "mlp." + s))


class Tebodra(PortionedDecoder):
    architecture = ARCHITECTURE

    def __init__(self, config: TebodraConfig, dtype: torch.dtype = torch.bfloat16, device="cuda") -> None:
        super().__init__()
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError("Tebodra runs in bfloat16 or float32")
        self.config = config
        self.dtype, self.device = dtype, torch.device(device)
        kw = dict(dtype=dtype, device=self.device)
        self.embed = nn.Parameter(torch.empty((config.vocab, config.width), **kw), requires_grad=False)
        self.blocks = nn.ModuleList(TebodraBlock(i, l, config, dtype, self.device) for i, l in enumerate(config.layers))
        self.final_norm = nn.Parameter(torch.ones(config.width, dtype=torch.float32, device=self.device), requires_grad=False)
        self.head = nn.Parameter(torch.zeros((pad8(config.vocab), config.width), **kw), requires_grad=False)
        self._pool = TensorPool(max_sets=4, on_evict=self._drop_graphs)
        # rings: one per attention layer with keys of its own, long enough for the furthest look-back among its readers
        self._owners = [i for i, l in enumerate(config.layers) if l.kind != "mlstm" and l.mixer.kv_from is None]
        self._reach: List[Optional[int]] = []
        for i in self._owners:
            readers = [config.layers[i].mixer] + [l.mixer for l in config.layers if l.kind != "mlstm" and l.mixer.kv_from == i]
            reaches = [s.reach for s in readers]
            self._reach.append(None if any(r is None for r in reaches) else max(reaches))
        self._cache_of = {}                            # layer index -> index of its ring among the owners
        for n, i in enumerate(self._owners):
            self._cache_of[i] = n
        for i, l in enumerate(config.layers):
            if l.kind != "mlstm" and l.mixer.kv_from is not None:
                self._cache_of[i] = self._cache_of[l.mixer.kv_from]
        self.states: List[torch.Tensor] = []          # fp32, every layer's in order (filter inputs; memory, stabiliser)
        self.kv_caches: List[torch.Tensor] = []       # (keys, values) of every owner in order
        self._rings: Tuple[int, ...] = ()
        self._batch = 0

    # ------------------------------------------------------------------ weights
    @torch.no_grad()
    def load_tensors(self, get) -> None:
        """``get(name)`` returns the checkpoint tensor of that name (any float dtype, CPU or GPU)."""
        self.embed.copy_(get("embed"))
        self.head.zero_()
        self.head[: self.config.vocab].copy_(get("head"))
        self.final_norm.copy_(1.0 + get("final.norm").float())
        for b in self.blocks:
            b.load(get)

    @classmethod
    def from_dir(cls, path, dtype: torch.dtype = torch.bfloat16, device="cuda") -> "Tebodra":
        """A folder with ``config.json`` and ``model.safetensors``."""
        from .safetensors_io import SafetensorsFile

        path = Path(path)
        with open(path / "config.json") as f:
            cfg = json.load(f)
        with SafetensorsFile(path / "model.safetensors") as st:
            model = cls(TebodraConfig.from_dict(cfg, st.shapes()), dtype=dtype, device=device)
            model.load_tensors(st.get)
        return model.eval()

    # ------------------------------------------------------------------ memory
    def reset_cache(self) -> None:
        """The sequences end: their slots are given back (the tensors stay allocated; the next sequence starts at position
        0, where the kernels take nothing from them)."""
        self.states, self.kv_caches, self._rings, self._batch = [], [], (), 0

    def _ring_plan(self, max_seq_length: int) -> Tuple[int, ...]:
        portion = min(self.prefill_portion, max_seq_length)
        return tuple(max(1, ring_length(max_seq_length, r, portion)) for r in self._reach)

    def _state_shapes(self, B: int) -> List[Tuple[int, ...]]:
        return [s for b in self.blocks for s in b.mix.state_shapes(B)]

    def _begin(self, B: int, max_seq_length: int, keep: bool) -> None:
        rings = self._ring_plan(max_seq_length)
        if (self.states or self.kv_caches) and self._batch == B and self._rings == rings:
            return
        st_shapes = self._state_shapes(B)
        kv_shapes = [s for n, i in enumerate(self._owners) for s in self.blocks[i].mix.cache_shapes(B, rings[n])]
        if keep:
            self.states = self._pool.get(st_shapes, torch.float32, self.device, zero=False) if st_shapes else []
            self.kv_caches = self._pool.get(kv_shapes, self.dtype, self.device, zero=False) if kv_shapes else []
        else:                      # a forward that keeps nothing: scratch memory, the pool's sets stay as they are
            self.states = [torch.empty(s, dtype=torch.float32, device=self.device) for s in st_shapes]
            self.kv_caches = [torch.empty(s, dtype=self.dtype, device=self.device) for s in kv_shapes]
        self._rings, self._batch = rings, B

    def _piece(self, max_seq_length: int) -> int:
        return min([max_seq_length] + [max_portion(ring, max_seq_length, r) for r, ring in zip(self._reach, self._rings)])

    def _graph_key(self, B: int) -> tuple:
        return (B, self._rings, self.states[0].data_ptr() if self.states else 0, self.kv_caches[0].data_ptr() if self.kv_caches else 0)

    def _save_memory(self):
        saved = (self.states, self.kv_caches, self._rings, self._batch)
        self.states, self.kv_caches, self._rings, self._batch = [], [], (), 0
        return saved

    def _restore_memory(self, saved) -> None:
        self.states, self.kv_caches, self._rings, self._batch = saved

    def _warm_step(self, s_idx, s_pos) -> None:
        """The eager runs before a capture advance the recurrent state; put it back afterwards (the ring row they write is
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
        r = cfg.residual_mult
        x = torch.empty((M, E), dtype=torch.float32, device=dev)
        N.call("ll_embed_scaled", N.ptr(self.embed), act, N.ptr(idx.reshape(-1).contiguous()), 1.0, N.ptr(x), None, act, M, E, N.stream())
        sms = N.call_ret("ll_sm_count")
        pending: List[Tuple[torch.Tensor, float]] = []
        si = 0
        for i, blk in enumerate(self.blocks):
            h = torch.empty((M, E), dtype=self.dtype, device=dev)
            add_norm_pair(x, pending, blk.norm1, None, cfg.eps, h, None, self.dtype)
            if self.layer_probe is not None and i > 0:
                self.layer_probe(i - 1, x)
            if blk.kind == "mlstm":
                y = blk.mix(h, B, T, pos_ids, self.states[si:si + 2])
                si += 2
            else:
                n = self._cache_of[i]
                spec = blk.mix.spec
                ring = self._rings[n]
                span = min(spec.reach if spec.reach is not None else (1 << 30), ring)
                # few queries: share a long look-back among blocks
                splits = max(1, min(64, (2 * sms) // max(1, (M * spec.heads + 3) // 4), (span + 127) // 128))
                conv_state = None
                if blk.mix.conv is not None:
                    conv_state = self.states[si]
                    si += 1
                y = blk.mix(h, B, T, pos_ids, self.kv_caches[2 * n:2 * n + 2], conv_state, splits)
            pending = [(y, r)]
            if blk.mlp is not None:
                h2 = torch.empty((M, E), dtype=self.dtype, device=dev)
                add_norm_pair(x, pending, blk.norm2, None, cfg.eps, h2, None, self.dtype)
                pending = [(blk.mlp(h2), r)]
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
