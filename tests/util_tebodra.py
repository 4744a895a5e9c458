"""Builders shared by the Tebodra tests: small random models written as model folders (config.json + safetensors) and
loaded back through the package's registry, and comparisons against the float64 oracle (oracle/tebodra.py)."""
import json

import numpy as np
import torch

from tests.util_bededra import bf16, load, rel_err, run_schedule      # noqa: F401  (model-agnostic helpers)

TOL32 = 2e-4


def attn(heads, kv_heads, dim, conv=3, rot_dims=None, base=1000.0, bands=(4.0, 1.0, 4.0, 32), softcap=20.0, scale=None):
    """Mixer ``attention``: filters on q and k, values = un-rotated keys, capped scores, band-wise rescaled frequencies."""
    rot = {"base": base, "dims": dim if rot_dims is None else rot_dims}
    if bands is not None:
        rot["scaling"] = dict(zip(("factor", "low", "high", "original"), bands))
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "conv": conv, "rot": rot,
         "scale": dim ** -0.5 if scale is None else scale}
    if softcap:
        m["softcap"] = softcap
    return {"type": "attention", "mixer": m}


def attn2(heads, kv_heads, dim, vdim, chunk, rot_dims=None, base=500.0, factor=2.0, scale=None, kv_from=None):
    """Mixer ``attention_2``: whole-projection norms, chunk mask, sink, linearly rescaled frequencies, maybe a borrowed ring."""
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "mask": {"size": chunk},
         "rot": {"base": base, "dims": dim if rot_dims is None else rot_dims, "scaling": {"factor": factor}},
         "scale": dim ** -0.5 if scale is None else scale}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "attention_2", "mixer": m}


def mlstm(heads, dim, vdim, cap=10.0):
    return {"type": "mlstm", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def model_cfg(vocab, width, layers, eps=1e-5, mult=0.7):
    """``layers``: (mixer entry from attn() / attn2() / mlstm(), feed-forward entry or None)."""
    return {"architecture": "Tebodra", "vocab": vocab, "width": width, "norm": {"eps": eps}, "residual_mult": mult,
            "layers": [dict(m, mlp=f) for m, f in layers]}


def random_weights(cfg, seed=0, qk_gain=2.0):
    """Every tensor of the design with values that keep activations of order one; already rounded to bfloat16."""
    r = np.random.RandomState(seed)
    E, W = cfg["width"], {}

    def lin(o, i, gain=1.0):
        return r.randn(o, i) * gain / np.sqrt(i)

    W["embed"] = r.randn(cfg["vocab"], E)
    W["head"] = lin(cfg["vocab"], E)
    W["final.norm"] = 0.2 * r.randn(E)
    for i, lc in enumerate(cfg["layers"]):
        p, m = f"l{i}.", lc["mixer"]
        W[p + "norm1"] = 0.2 * r.randn(E)
        if lc["type"] == "mlstm":
            H, D, V = m["heads"], m["dim"], m["vdim"]
            W[p + "mix.q"], W[p + "mix.k"], W[p + "mix.v"] = lin(H * D, E, qk_gain), lin(H * D, E, qk_gain), lin(H * V, E)
            W[p + "mix.g"], W[p + "mix.o"] = lin(H * V, E), lin(E, H * V)
            W[p + "mix.norm"] = 1 + 0.1 * r.randn(H * V)
            W[p + "mix.i"], W[p + "mix.f"] = lin(H, E, 2.0), lin(H, E, 2.0)
            W[p + "mix.i.b"], W[p + "mix.f.b"] = r.randn(H), r.uniform(0.5, 4.0, H)
        else:
            H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            W[p + "mix.q"] = lin(H * D, E, qk_gain)
            W[p + "mix.g"], W[p + "mix.o"] = lin(H * V, E), lin(E, H * V)
            own = m.get("kv_from") is None
            if own:
                W[p + "mix.k"] = lin(G * D, E, qk_gain)
            if lc["type"] == "attention":
                if m.get("conv"):
                    W[p + "mix.q.conv"] = 0.6 * r.randn(H * D, m["conv"])
                    W[p + "mix.k.conv"] = 0.6 * r.randn(G * D, m["conv"])
            else:
                W[p + "mix.q.norm"] = 1 + 0.2 * r.randn(H * D)
                W[p + "mix.sink"] = r.randn(H)
                if own:
                    W[p + "mix.k.norm"] = 1 + 0.2 * r.randn(G * D)
                    W[p + "mix.v"] = lin(G * V, E)
        if lc.get("mlp") is not None:
            W[p + "norm2"] = 0.2 * r.randn(E)
            W[p + "mlp.up"], W[p + "mlp.down"] = lin(lc["mlp"]["ff"], E), lin(E, lc["mlp"]["ff"])
    return {k: bf16(v) for k, v in W.items()}


def case_mixed(seed=0):
    """Sizes that share nothing with each other; every kind of mixer in an order of its own, a ring read by two layers with
    different chunks, feed-forwards present and absent, partial and full rotation."""
    layers = [
        (mlstm(3, 10, 12, cap=8.0), dense(24)),
        (attn2(6, 2, 8, 12, chunk=7, rot_dims=8, scale=0.6), None),
        (attn(4, 4, 12, conv=2, rot_dims=6, base=50.0, bands=(4.0, 1.0, 4.0, 16), softcap=5.0, scale=0.5), dense(32)),
        (attn2(6, 2, 8, 12, chunk=11, rot_dims=8, scale=0.4, kv_from=1), dense(16)),
        (attn2(2, 1, 16, 8, chunk=5, rot_dims=4, base=20.0, factor=3.0), dense(20)),
        (mlstm(2, 6, 4, cap=3.0), None),
    ]
    cfg = model_cfg(61, 40, layers, eps=1e-4, mult=0.7)
    return cfg, random_weights(cfg, seed)


def case_ones(seed=1):
    """Sizes that are 1 or equal where a real model's differ: one head, as many key/value heads as query heads, one tap, a
    chunk of one position (a query sees itself and the sink), a chunk longer than any test sequence, no cap, no scaling,
    multiplier 1."""
    a = attn(1, 1, 8, conv=1, rot_dims=2, bands=None, softcap=0.0)
    layers = [
        (attn2(1, 1, 4, 4, chunk=1), dense(8)),
        (mlstm(1, 1, 1, cap=0.0), dense(8)),
        (a, None),
        (attn2(2, 2, 4, 4, chunk=1000, rot_dims=4, factor=1.0), dense(4)),
        (attn2(2, 2, 4, 4, chunk=2, rot_dims=4, factor=1.0, kv_from=3), None),
    ]
    cfg = model_cfg(19, 8, layers, eps=1e-6, mult=1.0)
    return cfg, random_weights(cfg, seed)


def case_odd(seed=2):
    """Nothing is a multiple of 4: every kernel takes its unaligned path."""
    layers = [
        (attn(3, 3, 6, conv=5, rot_dims=2, softcap=7.0), dense(13)),
        (mlstm(5, 7, 5, cap=6.0), dense(11)),
        (attn2(6, 3, 10, 6, chunk=9, rot_dims=6), None),
    ]
    cfg = model_cfg(37, 30, layers, eps=1e-6, mult=0.5)
    return cfg, random_weights(cfg, seed)


def case_wide(seed=3):
    """Head sizes in multiples of 8 (the tensor-core form in bf16), different key and value sizes, prompts longer than a
    query tile with chunk edges inside tiles."""
    layers = [
        (attn2(4, 2, 32, 16, chunk=40, rot_dims=16), dense(48)),
        (attn(4, 1, 72, conv=3, rot_dims=24, softcap=30.0), None),
        (attn2(4, 2, 32, 16, chunk=23, rot_dims=16, kv_from=0), dense(48)),
        (mlstm(2, 16, 24), None),
    ]
    cfg = model_cfg(83, 64, layers, eps=1e-5, mult=0.6)
    return cfg, random_weights(cfg, seed, qk_gain=1.5)


def write_model(folder, cfg, W):
    from lit_llama.safetensors_io import save_safetensors

    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(cfg))
    save_safetensors({k: torch.from_numpy(np.asarray(v, dtype=np.float32)).to(torch.bfloat16) for k, v in W.items()},
                     folder / "model.safetensors")
    return folder


def agrees(got, want, dtype):
    """fp32: summation order only.  bf16: GEMM operands, ring rows and activations are rounded through every layer."""
    if dtype == torch.float32:
        return rel_err(got, want) < TOL32
    per_token = np.abs(got - want).reshape(-1, got.shape[-1]).max(-1) / np.abs(want).max()
    return bool(np.median(per_token) < 0.04 and per_token.max() < 0.25)
