"""Bumulix: a decoder-only model whose residual stream is kept as ``S`` copies (hyper-connections).  Sublayer q of a layer
(1: the mixer, 2: the feed-forward, absent when the layer has none) reads one learned mix of the copies and writes into all:

    u = sum_s in_q[s] X[s];      y = ls_q * sublayer( rmsnorm(u) * (1 + w_q) );
    X'[t] = sum_s mix_q[s, t] X[s] + r * out_q[t] * y                  (all copies at once from the old ones)

``r`` is the model's residual multiplier, ``ls_q`` a per-channel scale of the sublayer's result (absent when the checkpoint
has no such tensor); a config without ``streams`` keeps one copy and ``x <- x + r * y``.  After the last layer x is the sum of
the copies; logits = cap * tanh( embed . (rmsnorm(x) * (1 + w_f)) / cap ) with the embedding table as the head.

Mixers, in whatever order ``config.json`` lists them:

* ``attention``        - softmax attention over a sliding window without positional rotation, two score maps per head combined
  as a difference with a unit norm per head (softmax_attention.SoftmaxAttention with ``maps`` = 2), no gate;
* ``latent_attention`` - latent attention (latent_attention.LatentAttention) with queries through a normed latent, the
  "rotate half" pairing, YaRN-rescaled frequencies, an element-wise sigmoid gate, causal over the whole past.

Feed-forward: ``W_down gelu_tanh(W_up h)``.  A layer with ``weights_of: j`` computes with layer j's modules (mixer,
feed-forward, norms, scales, stream coefficients) and keeps rings of its own.

Per-sequence memory: per layer one key ring and one value ring (attention; as long as the window and a step need) or one
ring of latent rows (latent attention; the whole sequence).  All of it lives in tensors from the package's ``TensorPool`` with
stable addresses, written in place; ``forward`` is the package's common step function (stepping.PortionedDecoder).
"""
from __future__ import annotations

import json
from dataclasses import astuple, dataclass, field
from pathlib import Path
from typing import Dict, List, Optional, Tuple, Union

import torch
import torch.nn as nn

from . import _native as N
from .cache import TensorPool, max_portion, ring_length
from .feed_forward import DenseFF
from .latent_attention import LatentAttention, LatentAttentionSpec
from .rotary import RotarySpec
from .softmax_attention import SoftmaxAttention, SoftmaxAttentionSpec, pad8
from .stepping import PortionedDecoder, head_logits, hyper_mix_norm

ARCHITECTURE = "Bumulix"


@dataclass
class BumulixLayer:
    kind: str                                          # "attention" | "latent_attention"
    mixer: Union[SoftmaxAttentionSpec, LatentAttentionSpec]
    ff: Optional[int]                                  # inner size of the dense feed-forward; None: the layer has none
    weights_of: Optional[int] = None                   # index of the layer whose modules this layer computes with
    layer_scale: bool = True                           # per-channel scales ls1 / ls2 on the sublayers' results


@dataclass
class BumulixConfig:
    vocab: int
    width: int
    eps: float
    residual_mult: float
    streams: Optional[int]                             # copies of the stream; None: one plain residual stream
    logit_softcap: float                               # 0: the logits are not capped
    layers: List[BumulixLayer] = field(default_factory=list)

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def n_layer(self) -> int:
        return len(self.layers)

    @property
    def block_size(self) -> int:
        """No position table bounds the length: any the memory is sized for."""
        return 1 << 30

    @property
    def copies(self) -> int:
        return self.streams if self.streams else 1

    @classmethod
    def from_dict(cls, cfg: dict, shapes: Optional[Dict[str, Tuple[int, ...]]] = None) -> "BumulixConfig":
        """From the dictionary of a ``config.json``; sizes it leaves out are taken from the tensors' shapes, and where the
        tensors' names are known their presence decides which optional parts a layer has."""
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
        entries = cfg["layers"]
        layers: List[BumulixLayer] = []
        for i, lc in enumerate(entries):
            src = lc.get("weights_of")
            if src is not None:
                src = int(src)
                if not 0 <= src < len(entries) or src == i or entries[src].get("weights_of") is not None:
                    raise ValueError(f"layer {i}: weights_of {src} does not name a layer with tensors of its own")
            kind, m, p = lc.get("type"), lc["mixer"], f"l{i if src is None else src}.mix."
            if kind == "attention":
                dim = int(m["dim"])
                kv_heads = pick(m.get("kv_heads"), p + "v", 0, int(m["vdim"]) if m.get("vdim") is not None else dim)
                maps = (2 if "diff" in m else 1) if p + "k" not in shapes else shapes[p + "k"][0] // (kv_heads * dim)
                heads = pick(m.get("heads"), p + "q", 0, dim * maps)
                mask = m.get("mask") or {}
                mixer = SoftmaxAttentionSpec(
                    width=width, heads=heads, kv_heads=kv_heads, dim=dim, vdim=int(m["vdim"]) if m.get("vdim") is not None else dim,
                    scale=float(m["scale"]) if m.get("scale") is not None else dim ** -0.5, eps=eps, rotary=RotarySpec(0),
                    window=int(mask["size"]) if mask.get("size") is not None else None, maps=maps, diff=float(m.get("diff", 0.0)),
                    gate=False)
            elif kind == "latent_attention":
                dim, rot_dim = int(m["dim"]), int(m.get("rot_dim") or 0)
                heads = pick(m.get("heads"), p + "uk", 0, dim)
                rot = m.get("rot") if rot_dim else None
                rotary = RotarySpec.from_dict(rot, rot_dim) if rot else RotarySpec(0)
                q_rank = m.get("q_rank")
                if q_rank is None and p + "dq" in shapes:
                    q_rank = shapes[p + "dq"][0]
                if shapes and p + "dq" not in shapes:
                    q_rank = None
                gate = "element" if (not shapes or p + "g" in shapes) else "none"
                mixer = LatentAttentionSpec(
                    width=width, heads=heads, nope_dim=dim, rot_dim=rot_dim, v_dim=int(m["vdim"]) if m.get("vdim") is not None else dim,
                    kv_rank=pick(m.get("kv_rank"), p + "uk", 1), window=None,
                    scale=float(m["scale"]) if m.get("scale") is not None else (dim + rot_dim) ** -0.5, eps=eps,
                    q_rank=int(q_rank) if q_rank is not None else None, gate=gate, rot_layout="half", rotary=rotary)
            else:
                raise ValueError(f"layer {i}: unknown mixer type {kind!r}")
            f = lc.get("mlp")
            if f is None:
                ff = None
            elif f.get("kind", "dense") == "dense":
                ff = pick(f.get("ff"), f"l{i if src is None else src}.mlp.up", 0)
            else:
                raise ValueError(f"layer {i}: unknown feed-forward kind {f.get('kind')!r}")
            scaled = (f"l{i if src is None else src}.ls1" in shapes) if shapes else True
            layers.append(BumulixLayer(kind, mixer, ff, src, scaled))
        for i, l in enumerate(layers):
            if l.weights_of is not None:
                o = layers[l.weights_of]
                if (o.kind, o.mixer, o.ff) != (l.kind, l.mixer, l.ff):
                    raise ValueError(f"layer {i}: its entry differs from that of layer {l.weights_of}, whose tensors it uses")
        streams = cfg.get("streams")
        if streams is not None and not 1 <= int(streams) <= 8:
            raise ValueError(f"{streams} copies of the stream (1 to 8)")
        return cls(vocab=vocab, width=width, eps=eps, residual_mult=float(cfg.get("residual_mult", 1.0)),
                   streams=int(streams) if streams is not None else None, logit_softcap=float(cfg.get("logit_softcap") or 0.0),
                   layers=layers)


class HyperConnection(nn.Module):
    """The stream coefficients of one sublayer: ``w_in [S]`` (read), ``mix [S, S]`` (row: the copy read, column: the copy written) and ``w_out [S]``
    (write), fp32.  A model with one plain stream has ``mix`` = None and ``w_out`` = [1]."""

    def __init__(self, streams: Optional[int], device) -> None:
        super().__init__()
        f32 = dict(dtype=torch.float32, device=device)
        S = streams if streams else 1
        self.w_out = nn.Parameter(torch.ones(S, **f32), requires_grad=False)
        self.w_in = nn.Parameter(torch.ones(S, **f32), requires_grad=False) if streams else None
        self.mix = nn.Parameter(torch.eye(S, **f32), requires_grad=False) if streams else None

    def load(self, get) -> None:
        if self.mix is not None:
            self.w_in.copy_(get("in").float())
            self.w_out.copy_(get("out").float())
            self.mix.copy_(get("mix").float())


class BumulixBlock(nn.Module):
    def __init__(self, index: int, layer: BumulixLayer, cfg: BumulixConfig, dtype, device) -> None:
        super().__init__()
        f32 = dict(dtype=torch.float32, device=device)
        self.index, self.kind = index, layer.kind
        self.norm1 = nn.Parameter(torch.ones(cfg.width, **f32), requires_grad=False)          # holds 1 + w
        self.hc1 = HyperConnection(cfg.streams, device)
        self.ls1 = nn.Parameter(torch.ones(cfg.width, **f32), requires_grad=False) if layer.layer_scale else None
        self.mix = SoftmaxAttention(layer.mixer, dtype, device) if layer.kind == "attention" else LatentAttention(layer.mixer, dtype, device)
        self.mlp = DenseFF(cfg.width, layer.ff, "gelu_tanh", dtype, device) if layer.ff is not None else None
        has2 = self.mlp is not None
        self.norm2 = nn.Parameter(torch.ones(cfg.width, **f32), requires_grad=False) if has2 else None
        self.hc2 = HyperConnection(cfg.streams, device) if has2 else None
        self.ls2 = nn.Parameter(torch.ones(cfg.width, **f32), requires_grad=False) if has2 and layer.layer_scale else None

    def load(self, get) -> None:
        p = f"l{self.index}."
        self.norm1.copy_(1.0 + get(p + "norm1").float())
        self.hc1.load(lambda s: get(p + "hc1." + s))
        if self.ls1 is not None:
            self.ls1.copy_(get(p + "ls1").float())
        self.mix.load(lambda s: get(p + "mix." + s))
        if self.mlp is not None:
            self.norm2.copy_(1.0 + get(p + "norm2").float())
            self.hc2.load(lambda s: get(p + "hc2." + s))
            if self.ls2 is not None:
                self.ls2.copy_(get(p + "ls2").float())
            self.mlp.load(lambda s: get(p + "mlp." + s))


class Bumulix(PortionedDecoder):
    architecture = ARCHITECTURE

    def __init__(self, config: BumulixConfig, dtype: torch.dtype = torch.bfloat16, device="cuda") -> None:
        super().__init__()
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError("Bumulix runs in bfloat16 or float32")
        self.config = config
        self.dtype, self.device = dtype, torch.device(device)
        kw = dict(dtype=dtype, device=self.device)
        # the table is the head as well; the library's fast GEMMs want a multiple of 8 output rows (zero rows at the end)
        self.embed = nn.Parameter(torch.zeros((pad8(config.vocab), config.width), **kw), requires_grad=False)
        own = {i: BumulixBlock(i, l, config, dtype, self.device) for i, l in enumerate(config.layers) if l.weights_of is None}
        self.blocks = nn.ModuleList(own.values())
        self._block_of = [own[i if l.weights_of is None else l.weights_of] for i, l in enumerate(config.layers)]
        self.final_norm = nn.Parameter(torch.ones(config.width, dtype=torch.float32, device=self.device), requires_grad=False)
        self._pool = TensorPool(max_sets=4, on_evict=self._drop_graphs)
        self._reach: List[Optional[int]] = [l.mixer.reach if l.kind == "attention" else l.mixer.window for l in config.layers]
        self._cache_at: List[int] = []                 # where every layer's rings start in kv_caches
        n = 0
        for l in config.layers:
            self._cache_at.append(n)
            n += 2 if l.kind == "attention" else 1
        self.kv_caches: List[torch.Tensor] = []
        self._rings: Tuple[int, ...] = ()
        self._batch = 0
        self._rope: Dict[tuple, torch.Tensor] = {}
        self._rope_len = 0

    # ------------------------------------------------------------------ weights
    @torch.no_grad()
    def load_tensors(self, get) -> None:
        """``get(name)`` returns the checkpoint tensor of that name (any float dtype, CPU or GPU)."""
        self.embed.zero_()
        self.embed[: self.config.vocab].copy_(get("embed"))
        self.final_norm.copy_(1.0 + get("final.norm").float())
        for b in self.blocks:
            b.load(get)

    @classmethod
    def from_dir(cls, path, dtype: torch.dtype = torch.bfloat16, device="cuda") -> "Bumulix":
        """A folder with ``config.json`` and ``model.safetensors``."""
        from .safetensors_io import SafetensorsFile

        path = Path(path)
        with open(path / "config.json") as f:
            cfg = json.load(f)
        with SafetensorsFile(path / "model.safetensors") as st:
            model = cls(BumulixConfig.from_dict(cfg, st.shapes()), dtype=dtype, device=device)
            model.load_tensors(st.get)
        return model.eval()

    # ------------------------------------------------------------------ memory
    def reset_cache(self) -> None:
        """The sequences end: their slots are given back (the tensors stay allocated; the next sequence writes over them from
        position 0 and no kernel reads a slot its sequence has not written)."""
        self.kv_caches, self._rings, self._batch = [], (), 0

    def _ring_plan(self, max_seq_length: int) -> Tuple[int, ...]:
        portion = min(self.prefill_portion, max_seq_length)
        return tuple(max(1, ring_length(max_seq_length, r, portion)) for r in self._reach)

    def _ensure_rope(self, n_pos: int) -> None:
        if n_pos <= self._rope_len:
            return
        n = max(n_pos, 2 * self._rope_len, 1024)
        for l in self.config.layers:
            if l.kind == "latent_attention":
                self._rope[astuple(l.mixer.rotary)] = l.mixer.rope_table(n, self.device)
        self._rope_len = n
        self._drop_graphs()

    def _begin(self, B: int, max_seq_length: int, keep: bool) -> None:
        self._ensure_rope(max_seq_length)
        rings = self._ring_plan(max_seq_length)
        if self.kv_caches and self._batch == B and self._rings == rings:
            return
        shapes: List[Tuple[int, ...]] = []
        for l, blk, ring in zip(self.config.layers, self._block_of, rings):
            shapes += blk.mix.cache_shapes(B, ring) if l.kind == "attention" else [(B, ring, l.mixer.row)]
        if keep:
            self.kv_caches = self._pool.get(shapes, self.dtype, self.device, zero=False)
        else:                      # a forward that keeps nothing: scratch memory, the pool's sets stay as they are
            self.kv_caches = [torch.empty(s, dtype=self.dtype, device=self.device) for s in shapes]
        self._rings, self._batch = rings, B

    def _piece(self, max_seq_length: int) -> int:
        return min([max_seq_length] + [max_portion(ring, max_seq_length, r) for r, ring in zip(self._reach, self._rings)])

    def _graph_key(self, B: int) -> tuple:
        return (B, self._rings, self.kv_caches[0].data_ptr() if self.kv_caches else 0)

    def _save_memory(self):
        saved = (self.kv_caches, self._rings, self._batch)
        self.kv_caches, self._rings, self._batch = [], (), 0
        return saved

    def _restore_memory(self, saved) -> None:
        self.kv_caches, self._rings, self._batch = saved

    # ------------------------------------------------------------------ forward
    def _forward_portion(self, idx: torch.Tensor, pos_ids: torch.Tensor, sel) -> torch.Tensor:
        cfg = self.config
        B, T = idx.shape
        M, E, S = B * T, cfg.width, cfg.copies
        dev = idx.device
        act = N.dtype_code(self.dtype)
        r = cfg.residual_mult
        x0 = torch.empty((M, E), dtype=torch.float32, device=dev)
        N.call("ll_embed_scaled", N.ptr(self.embed), act, N.ptr(idx.reshape(-1).contiguous()), 1.0, N.ptr(x0), None, act, M, E, N.stream())
        X = torch.empty((M, S, E), dtype=torch.float32, device=dev)
        sms = N.call_ret("ll_sm_count")
        src = x0                           # the first read spreads the embedding output over the copies
        pending = None                     # (y, ls, hc) of the sublayer whose result is not in the copies yet
        total = torch.empty((M, E), dtype=torch.float32, device=dev) if self.layer_probe is not None else None
        for i, (layer, blk) in enumerate(zip(cfg.layers, self._block_of)):
            h = torch.empty((M, E), dtype=self.dtype, device=dev)
            hyper_mix_norm(src, X, pending, r, blk.hc1.w_in, blk.norm1, cfg.eps, h, total if i > 0 else None, self.dtype)
            src = X
            if self.layer_probe is not None and i > 0:
                self.layer_probe(i - 1, total)
            ring = self._rings[i]
            at = self._cache_at[i]
            spec = blk.mix.spec
            if layer.kind == "attention":
                span = min(spec.reach if spec.reach is not None else (1 << 30), ring)
                # few queries: share the look-back among blocks, down to 32 keys each (a group of lanes walks its keys one
                # after the other, every step a round trip to memory)
                splits = max(1, min(64, (2 * sms) // max(1, (M * spec.heads * spec.maps + 3) // 4), (span + 31) // 32))
                y = blk.mix(h, B, T, pos_ids, self.kv_caches[at:at + 2], None, splits)
            else:
                splits = max(1, min(16, (2 * sms) // max(1, M * ((spec.heads + 31) // 32)), (ring + 63) // 64))
                y = blk.mix(h, B, T, pos_ids, self._rope[astuple(spec.rotary)], self.kv_caches[at], splits)
            pending = (y, blk.ls1, blk.hc1)
            if blk.mlp is not None:
                h2 = torch.empty((M, E), dtype=self.dtype, device=dev)
                hyper_mix_norm(X, X, pending, r, blk.hc2.w_in, blk.norm2, cfg.eps, h2, None, self.dtype)
                pending = (blk.mlp(h2), blk.ls2, blk.hc2)
        if sel is not None and len(sel) == 0 and self.layer_probe is None:      # the step only fills the memory
            return torch.empty((B, 0, cfg.vocab), dtype=torch.float32, device=dev)
        xn = torch.empty((M, E), dtype=self.dtype, device=dev)
        hyper_mix_norm(src, X, pending, r, None, self.final_norm, cfg.eps, xn, total, self.dtype)
        if self.layer_probe is not None:
            self.layer_probe(cfg.n_layer - 1, total)
        if sel is not None:
            if len(sel) == 0:
                return torch.empty((B, 0, cfg.vocab), dtype=torch.float32, device=dev)
            ridx = (torch.arange(B, device=dev)[:, None] * T + torch.tensor(sel, device=dev, dtype=torch.long)[None]).reshape(-1)
            xn = xn.index_select(0, ridx).contiguous()
        logits = head_logits(xn, self.embed, cfg.vocab)
        if cfg.logit_softcap > 0.0:
            logits = logits.contiguous()
            N.call("ll_tanh_cap", N.ptr(logits), float(cfg.logit_softcap), logits.numel(), N.stream())
        return logits.reshape(B, -1, cfg.vocab)
