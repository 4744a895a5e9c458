"""The step function the folder-loaded models share: ``forward(idx, max_seq_length, input_pos, out_rows)`` with LLaMA's
signature (model.py), so that ``generate()``, its sampler and the trace session drive every model alike.

A call appends ``T`` tokens at consecutive positions to the model's per-sequence memory (rings, recurrent state) and
returns fp32 logits.  Long inputs run as several passes of at most ``_piece()`` tokens (a ring must not overwrite a slot
one of the pass's own queries still reads); a single token replays one CUDA graph per (batch, cache identity), with the
token and its position in device tensors the graph reads.  A model supplies the hooks below.
"""
from __future__ import annotations

import contextlib
import gc
import os
from typing import Dict, Optional

import torch
import torch.nn as nn

from . import _native as N


@contextlib.contextmanager
def graph_capture(g: "torch.cuda.CUDAGraph"):
    """``with torch.cuda.graph(g)`` that no garbage collection can break.  A model that was dropped while it still held
    captured steps is a dead reference cycle; when the collector finds it, the graphs inside are destroyed, and destroying a
    graph while ANY stream of the process captures invalidates that capture (its next launch then fails).  So the dead
    cycles are collected before the capture begins and the collector rests until it has ended."""
    gc.collect()
    was_enabled = gc.isenabled()
    gc.disable()
    try:
        with torch.cuda.graph(g):
            yield
    finally:
        if was_enabled:
            gc.enable()


class PortionedDecoder(nn.Module):
    use_fused_decode = False       # generate(): the per-op sampling loop drives these models
    use_step_graph = True          # single-token steps replay one CUDA graph
    prefill_portion = 4096         # most tokens one pass appends; longer prompts run as several passes
    layer_probe = None             # callable(layer index, fp32 stream [B*T, width]) after every layer, for inspection

    def __init__(self) -> None:
        super().__init__()
        self._step_graphs: Dict[tuple, dict] = {}
        self._sized_for = 0

    # ------------------------------------------------------------------ hooks
    def _begin(self, B: int, max_seq_length: int, keep: bool) -> None:
        """Make the memory for ``B`` sequences of up to ``max_seq_length`` tokens current (``keep`` False: scratch memory
        for a forward that keeps nothing)."""
        raise NotImplementedError

    def _piece(self, max_seq_length: int) -> int:
        """Most tokens one pass may append."""
        raise NotImplementedError

    def _graph_key(self, B: int) -> tuple:
        """Identity of the memory a captured step reads and writes."""
        raise NotImplementedError

    def _save_memory(self):
        raise NotImplementedError

    def _restore_memory(self, saved) -> None:
        raise NotImplementedError

    def _forward_portion(self, idx: torch.Tensor, pos_ids: torch.Tensor, sel) -> torch.Tensor:
        raise NotImplementedError

    def _drop_graphs(self) -> None:
        self._step_graphs.clear()

    # ------------------------------------------------------------------ forward
    @torch.no_grad()
    def forward(self, idx: torch.Tensor, max_seq_length: Optional[int] = None, input_pos: Optional[torch.Tensor] = None,
                out_rows=None) -> torch.Tensor:
        """``idx [B, T]`` at positions ``input_pos [T]`` (consecutive; None: a forward without kept memory from position 0).
        Returns fp32 logits ``[B, T, vocab]``, or ``[B, len(out_rows), vocab]`` for the token indices in ``out_rows``."""
        N.require_cuda(idx)
        B, T = idx.shape
        keep = input_pos is not None
        saved = None
        if not keep:
            saved = self._save_memory()
            pos0, max_seq_length = 0, T
        else:
            pos0 = int(input_pos[0])
            if max_seq_length is None:         # the length the memory was last sized for, unless the sequence outgrows it
                max_seq_length = max(pos0 + T, self._sized_for)
            self._sized_for = max_seq_length
        assert pos0 + T <= max_seq_length, f"positions up to {pos0 + T} but the cache holds {max_seq_length}"
        self._begin(B, max_seq_length, keep)
        piece = max(1, min(self.prefill_portion, self._piece(max_seq_length)))
        rows = None if out_rows is None else [int(r) for r in out_rows]
        outs = []
        for t0 in range(0, T, piece):
            t1 = min(T, t0 + piece)
            sel = None
            if rows is not None:
                sel = [r - t0 for r in rows if t0 <= r < t1]
            part = idx[:, t0:t1]
            if t1 - t0 == 1 and keep and self.use_step_graph and os.environ.get("LLB200_STEP_GRAPH", "1") != "0" \
                    and not torch.cuda.is_current_stream_capturing():
                lg = self._graphed_step(part, pos0 + t0)
                if sel is not None:
                    lg = lg[:, sel]
            else:
                pos_ids = torch.arange(pos0 + t0, pos0 + t1, dtype=torch.int32, device=idx.device)
                lg = self._forward_portion(part.contiguous(), pos_ids, sel)
            outs.append(lg)
        if not keep:
            self._restore_memory(saved)
        return outs[0] if len(outs) == 1 else torch.cat(outs, dim=1)

    def _graphed_step(self, idx: torch.Tensor, pos: int) -> torch.Tensor:
        key = self._graph_key(idx.shape[0])
        ent = self._step_graphs.get(key)
        if ent is None:
            s_idx = idx.clone()
            s_pos = torch.full((1,), pos, dtype=torch.int32, device=idx.device)
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):          # warm-up: library handles and workspaces
                self._warm_step(s_idx, s_pos)
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with graph_capture(g):
                out = self._forward_portion(s_idx, s_pos, None)
            ent = self._step_graphs[key] = dict(graph=g, idx=s_idx, pos=s_pos, out=out)
        ent["idx"].copy_(idx)
        ent["pos"].fill_(pos)
        ent["graph"].replay()
        return ent["out"].clone()

    def _warm_step(self, s_idx: torch.Tensor, s_pos: torch.Tensor) -> None:
        """Run the step eagerly before it is captured.  A model whose step only rewrites its own cache row runs it as it
        is; one with recurrent state must leave that state as it found it."""
        for _ in range(2):
            self._forward_portion(s_idx, s_pos, None)


def head_logits(xn: torch.Tensor, head: torch.Tensor, vocab: int) -> torch.Tensor:
    """fp32 logits ``[rows, vocab]`` of normed rows ``xn`` against ``head`` (``[vocab rounded up to 8, width]``, zero rows
    at the end: the library's fast GEMMs want aligned outputs)."""
    if xn.dtype == torch.float32:
        logits = xn @ head.t()
    else:
        try:
            logits = torch.mm(xn, head.t(), out_dtype=torch.float32)
        except RuntimeError:           # a width the library's mixed-output GEMM does not take: fp32 product of the same operands
            logits = xn.float() @ head.float().t()
    return logits[:, :vocab]


def add_norm_pair(x, branches, w1, w2, eps, out1, out2, act_dtype) -> None:
    """``x += sum scale * branch`` in place (fp32); then ``out1 = rmsnorm(x) * w1`` and ``out2 = rmsnorm(x) * w2`` (either
    may be None).  ``out1`` may be fp32 or the activation dtype."""
    assert len(branches) <= 3
    b = list(branches) + [(None, 0.0)] * (3 - len(branches))
    N.call("ll_add_norm_pair", N.ptr(x), N.ptr(b[0][0]), float(b[0][1]), N.ptr(b[1][0]), float(b[1][1]), N.ptr(b[2][0]), float(b[2][1]),
           N.ptr(w1), N.ptr(w2), float(eps), N.ptr(out1), 1 if (out1 is not None and out1.dtype == torch.float32) else 0, N.ptr(out2),
           N.dtype_code(act_dtype), x.shape[0], x.shape[1], N.stream())


def hyper_mix_norm(src, X, pending, r, w_in, w, eps, h, total, act_dtype) -> None:
    """One launch between two sublayers of a model whose stream is kept as copies ``X [rows, S, width]`` (fp32, updated in
    place): the result of the sublayer before (``pending`` = (y, per-channel scale or None, its HyperConnection); None: there
    is none) goes into all copies, ``X'[t] = sum_s mix[s, t] X[s] + r * out[t] * scale * y``; then ``h = rmsnorm(sum_t
    w_in[t] X'[t]) * w`` (``w_in`` None: the plain sum) and, if asked for, ``total`` = the plain sum of the copies.  ``src``
    is ``X``, or the embedding output ``[rows, width]`` that every copy starts as."""
    M, S, E = X.shape
    y, ls, hc = pending if pending is not None else (None, None, None)
    spread = src is not X
    N.call("ll_hyper_mix_norm", N.ptr(src), E if spread else S * E, 0 if spread else E, N.ptr(X), N.ptr(y), N.ptr(ls), float(r),
           N.ptr(hc.mix) if hc is not None else None, N.ptr(hc.w_out) if hc is not None else None, N.ptr(w_in), N.ptr(w), float(eps),
           N.ptr(h), 1 if (h is not None and h.dtype == torch.float32) else 0, N.ptr(total), N.dtype_code(act_dtype), M, S, E, N.stream())
