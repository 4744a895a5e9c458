"""Builders shared by the Bumulix tests: small random models written as model folders (config.json + safetensors) and
loaded back through the package's registry, and comparisons against the float64 oracle (oracle/bumulix.py)."""
import json

import numpy as np
import torch

from tests.util_bededra import bf16, load, rel_err, run_schedule      # noqa: F401  (model-agnostic helpers)

TOL32 = 2e-4


def agrees(got, want, dtype):
    """fp32: summation order only.  bf16: GEMM operands, ring rows and activations are rounded through every layer, and the
    unit norm of a difference of two maps magnifies that where the difference is small (with one value per head it is a
    sign): the typical token must be close and only a few may be far."""
    if dtype == torch.float32:
        return rel_err(got, want) < TOL32
    per_token = np.abs(got - want).reshape(-1, got.shape[-1]).max(-1) / np.abs(want).max()
    return bool(np.median(per_token) < 0.04 and np.mean(per_token > 0.25) <= 0.1)


def diff_attn(heads, kv_heads, dim, vdim, window=None, diff=0.4, scale=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "diff": diff, "scale": dim ** -0.5 if scale is None else scale}
    if window is not None:
        m["mask"] = {"size": window}
    return {"type": "attention", "mixer": m}


def latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, base=300.0, yarn=(4.0, 64, 8.0, 1.0), scale=None):
    """``yarn``: (factor, original, fast, slow) or None for plain frequencies."""
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank,
         "scale": (dim + rot_dim) ** -0.5 if scale is None else scale}
    if rot_dim:
        m["rot"] = {"base": base, "dims": rot_dim}
        if yarn is not None:
            m["rot"]["scaling"] = dict(zip(("factor", "original", "fast", "slow"), yarn))
    return {"type": "latent_attention", "mixer": m}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def model_cfg(vocab, width, layers, streams=2, eps=1e-5, mult=0.6, cap=12.0):
    """``layers``: (mixer entry, feed-forward entry or None) or an int j: the layer computes with layer j's tensors."""
    out = [None if isinstance(l, int) else dict(l[0], mlp=l[1]) for l in layers]
    for i, l in enumerate(layers):
        if isinstance(l, int):                 # earlier or later in the list
            out[i] = dict(out[l], weights_of=l)
    cfg = {"architecture": "Bumulix", "vocab": vocab, "width": width, "norm": {"eps": eps}, "residual_mult": mult, "layers": out}
    if streams is not None:
        cfg["streams"] = streams
    if cap:
        cfg["logit_softcap"] = cap
    return cfg


def random_weights(cfg, seed=0, qk_gain=2.0, layer_scale=True):
    """Every tensor of the design with values that keep activations of order one; already rounded to bfloat16."""
    r = np.random.RandomState(seed)
    E, S, W = cfg["width"], cfg.get("streams"), {}

    def lin(o, i, gain=1.0):
        return r.randn(o, i) * gain / np.sqrt(i)

    W["embed"] = r.randn(cfg["vocab"], E)
    W["final.norm"] = 0.2 * r.randn(E)
    for i, lc in enumerate(cfg["layers"]):
        if lc.get("weights_of") is not None:
            continue
        p, m = f"l{i}.", lc["mixer"]
        subs = ["1"] + (["2"] if lc.get("mlp") is not None else [])
        for q in subs:
            W[p + "norm" + q] = 0.2 * r.randn(E)
            if layer_scale:
                W[p + "ls" + q] = r.uniform(0.5, 1.5, E)
            if S:
                W[p + f"hc{q}.in"] = r.uniform(0.3, 1.0, S) * r.choice([-1.0, 1.0], S)
                W[p + f"hc{q}.out"] = r.uniform(0.5, 1.2, S)
                W[p + f"hc{q}.mix"] = np.eye(S) * 0.8 + 0.3 * r.randn(S, S)
        if lc["type"] == "attention":
            H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            W[p + "mix.q"], W[p + "mix.k"] = lin(H * 2 * D, E, qk_gain), lin(G * 2 * D, E, qk_gain)
            W[p + "mix.v"], W[p + "mix.o"] = lin(G * V, E), lin(E, H * V)
            for n in ("lq1", "lk1", "lq2", "lk2"):
                W[p + "mix." + n] = 0.5 * r.randn(D) / np.sqrt(D)
        else:
            H, D, R, V, KR, QR = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["q_rank"]
            W[p + "mix.dq"], W[p + "mix.dq.norm"] = lin(QR, E), 1 + 0.2 * r.randn(QR)
            W[p + "mix.uq"] = lin(H * (D + R), QR, qk_gain)
            W[p + "mix.dkv"], W[p + "mix.dkv.norm"] = lin(KR + R, E, qk_gain), 1 + 0.2 * r.randn(KR)
            W[p + "mix.uk"], W[p + "mix.uv"] = lin(H * D, KR, qk_gain), lin(H * V, KR)
            W[p + "mix.g"], W[p + "mix.o"] = lin(H * V, E), lin(E, H * V)
        if lc.get("mlp") is not None:
            W[p + "mlp.up"], W[p + "mlp.down"] = lin(lc["mlp"]["ff"], E), lin(E, lc["mlp"]["ff"])
    return {k: bf16(v) for k, v in W.items()}


def case_mixed(seed=0):
    """Sizes that share nothing with each other; both mixers in an order of its own, three copies of the stream, grouped
    key/value heads, two windows, layers with and without feed-forward, layers that compute with another layer's tensors
    (one of them names a LATER layer)."""
    layers = [
        (latent(3, 6, 4, 10, 12, 7, base=50.0, yarn=(4.0, 32, 8.0, 1.0)), dense(24)),
        (diff_attn(6, 2, 8, 12, window=5, diff=0.3, scale=0.5), None),
        1,
        5,
        0,
        (diff_attn(2, 1, 16, 8, window=9, diff=0.6), dense(20)),
        (latent(2, 8, 8, 4, 5, 9, base=20.0, yarn=None), None),
    ]
    cfg = model_cfg(61, 40, layers, streams=3, eps=1e-4, mult=0.7, cap=9.0)
    return cfg, random_weights(cfg, seed, qk_gain=1.2)


def case_ones(seed=1):
    """Sizes that are 1 or equal where a real model's differ: one copy of the stream (with coefficients), one head, one
    value dimension, a window of one position (a query sees itself), a window longer than any test sequence, latents of one
    number, one rotated pair, multiplier 1."""
    layers = [
        (diff_attn(1, 1, 4, 1, window=1), dense(8)),
        (latent(1, 1, 2, 1, 1, 1, yarn=(2.0, 8, 4.0, 1.0)), dense(8)),
        (diff_attn(2, 2, 4, 4, window=1000, diff=0.5), None),
        (diff_attn(2, 1, 2, 2, window=2, diff=0.1), dense(4)),
        0,
    ]
    cfg = model_cfg(19, 8, layers, streams=1, eps=1e-6, mult=1.0, cap=30.0)
    return cfg, random_weights(cfg, seed)


def case_plain(seed=2):
    """What a config may leave out: no copies of the stream (a plain residual sum), no per-channel scales, no cap on the
    logits, no window (every earlier token is visible), no frequency scaling."""
    layers = [
        (diff_attn(2, 2, 8, 8, window=None), dense(16)),
        (latent(2, 8, 4, 8, 8, 8, yarn=None), dense(16)),
        (diff_attn(4, 1, 4, 8, window=6), None),
    ]
    cfg = model_cfg(29, 24, layers, streams=None, eps=1e-5, mult=0.8, cap=None)
    return cfg, random_weights(cfg, seed, layer_scale=False)


def case_odd(seed=3):
    """Nothing is a multiple of 4: every kernel takes its unaligned path; five copies of the stream."""
    layers = [
        (diff_attn(3, 3, 6, 5, window=7), dense(13)),
        (latent(5, 7, 6, 5, 9, 11, base=33.0, yarn=(3.0, 16, 6.0, 2.0)), dense(11)),
        (diff_attn(6, 3, 10, 6, window=3, diff=0.7), None),
    ]
    cfg = model_cfg(37, 30, layers, streams=5, eps=1e-6, mult=0.5, cap=7.0)
    return cfg, random_weights(cfg, seed)


def case_wide(seed=4):
    """Head sizes in multiples of 8 (the tensor-core forms in bf16), key and value sizes that differ, prompts longer than a
    query tile with window edges inside tiles."""
    layers = [
        (diff_attn(4, 2, 32, 16, window=40), dense(48)),
        (latent(4, 16, 16, 24, 32, 24, base=1000.0, yarn=(8.0, 64, 16.0, 1.0)), None),
        (diff_attn(2, 1, 72, 88, window=70, diff=0.2), dense(48)),
        0,
    ]
    cfg = model_cfg(83, 64, layers, streams=2, eps=1e-5, mult=0.6, cap=15.0)
    return cfg, random_weights(cfg, seed, qk_gain=1.5)


def write_model(folder, cfg, W):
    from lit_llama.safetensors_io import save_safetensors

    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(cfg))
    save_safetensors({k: torch.from_numpy(np.asarray(v, dtype=np.float32)).to(torch.bfloat16) for k, v in W.items()},
                     folder / "model.safetensors")
    return folder
