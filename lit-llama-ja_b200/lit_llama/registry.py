"""Which model class serves which checkpoint.

A model folder holds ``config.json`` (its ``"architecture"`` names the design) and ``model.safetensors``; the reference's
LLaMA checkpoints are single ``.pth`` files whose embedding width names the size (``utils.llama_model_lookup``).
``load_model`` takes either and returns a model with the package's common surface: ``forward(idx, max_seq_length,
input_pos)``, ``reset_cache()``, ``config.vocab_size``.
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Callable, Dict, Optional

import torch

_FROM_DIR: Dict[str, Callable] = {}


def register_architecture(name: str, from_dir: Callable) -> None:
    """``from_dir(path, dtype=, device=)`` builds and loads the model of a folder whose config names ``name``."""
    _FROM_DIR[name] = from_dir


def architectures():
    _builtin()
    return sorted(_FROM_DIR)


def _builtin() -> None:
    if "Lepalorn" not in _FROM_DIR:
        from .lepalorn import ARCHITECTURE, Lepalorn

        register_architecture(ARCHITECTURE, Lepalorn.from_dir)
    if "Bededra" not in _FROM_DIR:
        from .bededra import ARCHITECTURE, Bededra

        register_architecture(ARCHITECTURE, Bededra.from_dir)
    if "Tebodra" not in _FROM_DIR:
        from .tebodra import ARCHITECTURE, Tebodra

        register_architecture(ARCHITECTURE, Tebodra.from_dir)
    if "Bumulix" not in _FROM_DIR:
        from .bumulix import ARCHITECTURE, Bumulix

        register_architecture(ARCHITECTURE, Bumulix.from_dir)


def load_model_dir(path, dtype: torch.dtype = torch.bfloat16, device="cuda"):
    _builtin()
    path = Path(path)
    with open(path / "config.json") as f:
        arch = json.load(f).get("architecture")
    if arch not in _FROM_DIR:
        raise ValueError(f"{path}: architecture {arch!r} is not one of {sorted(_FROM_DIR)}")
    return _FROM_DIR[arch](path, dtype=dtype, device=device)


def load_model(path, quantize: Optional[str] = None, device="cuda", dtype: torch.dtype = torch.bfloat16):
    """A model folder (any registered architecture) or a LLaMA ``.pth`` checkpoint (optionally quantized)."""
    path = Path(path)
    if path.is_dir():
        if quantize is not None:
            raise ValueError("--quantize applies to LLaMA checkpoints")
        return load_model_dir(path, dtype=dtype, device=device)
    from .utils import EmptyInitOnDevice, lazy_load, llama_model_lookup, stream_load_state_dict
    from .model import LLaMA

    with lazy_load(path) as checkpoint:
        name = llama_model_lookup(checkpoint)
        with EmptyInitOnDevice(device=device, dtype=dtype, quantization_mode=quantize):
            model = LLaMA.from_name(name)
        if torch.device(device).type == "cuda" and quantize is not None and quantize.startswith("gptq"):
            stream_load_state_dict(model, path, strict=True)
        else:
            model.load_state_dict(checkpoint)
    return model.eval()
