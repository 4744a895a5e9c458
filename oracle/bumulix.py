"""Plain, slow float64 statement of the Bumulix design, one function per mechanism (numpy only; test infrastructure,
never imported by the product).  It works on a whole sequence at once and keeps no cache: whatever schedule the product
runs (portions, single tokens, rings), its logits must equal these.

The stream is ``S`` copies X[0..S-1] of the embedding output (hyper-connections).  Sublayer q of a layer (1: mixer,
2: feed-forward; the second is absent when the layer has none) reads one mix of the copies and writes into all of them:

    u = sum_s in_q[s] X[s];    y = ls_q * sublayer(rms(u) * (1 + w_q));
    X'[t] = sum_s mix_q[s, t] X[s] + r * out_q[t] * y            (all t from the old copies)

with r the model's residual multiplier and ``ls_q`` a per-channel scale of the sublayer's result.  A model without
``streams`` keeps one x and ``x <- x + r * y``; a layer without ``ls`` tensors has no per-channel scale.  After the last
layer x is the sum of the copies, logits = cap * tanh(embed . (rms(x) * (1 + w_f)) / cap).

Mixers: ``attention`` (two softmax maps per head over a sliding window without positions, combined as a difference with a
learned weight and a unit norm per head) and ``latent_attention`` (queries through a low-rank latent, keys and values as
up-projections of one normed latent row per token plus one rotary key part for all heads, YaRN-rescaled frequencies, a
sigmoid gate element by element).  Feed-forward: W_down gelu_tanh(W_up h).  A layer with ``weights_of: j`` computes with
layer j's tensors.

Checkpoint names: ``embed``, ``final.norm``; per layer i ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.ls1``, ``l<i>.ls2``,
``l<i>.hc<q>.in / .out / .mix``, ``l<i>.mix.*``, ``l<i>.mlp.*``; Linear weights are [out, in].
"""
import math

import numpy as np


def unit_rms(x, eps):
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def norm_one_plus(x, w, eps):
    return unit_rms(x, eps) * (1.0 + w)


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def softmax_rows(s, visible):
    """Softmax of every row of ``s`` over the entries where ``visible`` holds (every row sees at least itself)."""
    s = np.where(visible, s, -np.inf)
    e = np.exp(s - s.max(axis=-1, keepdims=True))
    return e / e.sum(axis=-1, keepdims=True)


def causal_mask(T, window=None):
    i, j = np.arange(T)[:, None], np.arange(T)[None, :]
    vis = j <= i
    if window is not None:
        vis &= (i - j) < window
    return vis


# ------------------------------------------------------------------------------------------------ rotary positions
def yarn_frequencies(rot):
    """(frequencies [dims/2], magnitude) of a rotation entry ``{"base", "dims"[, "scaling"]}``.  Without scaling the
    frequencies are base^(-2i/dims) and the magnitude is 1.  With it, the pair index at which a wave makes ``t`` turns over
    ``original`` positions is d(t) = dims ln(original / (2 pi t)) / (2 ln base); pairs below d(fast) keep their frequency,
    pairs above d(slow) have it divided by ``factor``, with a linear ramp between; cosines and sines are scaled by
    0.1 ln(factor) + 1."""
    dims = int(rot["dims"])
    base = float(rot["base"])
    f = np.array([base ** (-2.0 * i / dims) for i in range(dims // 2)])
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor, orig = float(sc["factor"]), float(sc["original"])

    def d(t):
        return dims * math.log(orig / (2.0 * math.pi * t)) / (2.0 * math.log(base))

    lo = max(math.floor(d(float(sc["fast"]))), 0)
    hi = min(math.ceil(d(float(sc["slow"]))), dims - 1)
    ramp = np.clip((np.arange(dims // 2) - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_half(x, rot, positions):
    """x [T, ..., d]: the first ``dims`` of the last axis turn, dimension i paired with i + dims/2; the rest pass."""
    dims = int(rot["dims"])
    f, mag = yarn_frequencies(rot)
    half = dims // 2
    shape = (len(positions),) + (1,) * (x.ndim - 2) + (half,)
    a = (np.asarray(positions, dtype=np.float64)[:, None] * f[None, :]).reshape(shape)
    c, s = np.cos(a) * mag, np.sin(a) * mag
    u, v = x[..., :half], x[..., half:dims]
    return np.concatenate([u * c - v * s, v * c + u * s, x[..., dims:]], axis=-1)


# ------------------------------------------------------------------------------------------------ mixers
def differential_attention(h, W, m, eps):
    """h [T, E] -> [T, E].  Every head scores its keys twice: a head's q rows (a key/value head's k rows) hold map 0, then map 1, and
    both maps weigh the same values; o = a1 - lam * a2, divided by its root mean square over the head's values, times (1 - diff)."""
    T = h.shape[0]
    H, G, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    diff = float(m["diff"])
    window = (m.get("mask") or {}).get("size")
    q = (h @ W["q"].T).reshape(T, H, 2, d)
    k = (h @ W["k"].T).reshape(T, G, 2, d)
    v = (h @ W["v"].T).reshape(T, G, dv)
    lam = math.exp(float(np.sum(W["lq1"] * W["lk1"]))) - math.exp(float(np.sum(W["lq2"] * W["lk2"]))) + diff
    vis = causal_mask(T, window)
    out = np.zeros((T, H, dv))
    for hh in range(H):
        g = hh // (H // G)
        a = [softmax_rows(q[:, hh, mp] @ k[:, g, mp].T * float(m["scale"]), vis) @ v[:, g] for mp in range(2)]
        out[:, hh] = unit_rms(a[0] - lam * a[1], eps) * (1.0 - diff)
    return out.reshape(T, H * dv) @ W["o"].T


def latent_attention(h, W, m, eps, positions=None):
    """h [T, E] -> [T, E].  Queries: W_uq rms(W_dq h) * w; keys and values: up-projections of c = rms(first kv_rank rows
    of W_dkv h) * w, plus the last rot_dim rows as one rotary key part for all heads; causal softmax; heads times
    sigmoid(W_g h) element by element."""
    T = h.shape[0]
    H, d, r, dv, kr = int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"]), int(m["kv_rank"])
    positions = np.arange(T) if positions is None else positions
    rot = dict(m["rot"], dims=m["rot"].get("dims", r)) if m.get("rot") else {"dims": 0, "base": 1.0}
    cq = unit_rms(h @ W["dq"].T, eps) * W["dq.norm"]
    q = (cq @ W["uq"].T).reshape(T, H, d + r)
    kv = h @ W["dkv"].T
    c = unit_rms(kv[:, :kr], eps) * W["dkv.norm"]
    k_rot = rotate_half(kv[:, kr:], rot, positions) if r else kv[:, kr:]
    q_rot = rotate_half(q[:, :, d:], rot, positions) if r else q[:, :, d:]
    k_nope = (c @ W["uk"].T).reshape(T, H, d)
    val = (c @ W["uv"].T).reshape(T, H, dv)
    vis = causal_mask(T)
    out = np.zeros((T, H, dv))
    for hh in range(H):
        s = (q[:, hh, :d] @ k_nope[:, hh].T + q_rot[:, hh] @ k_rot.T) * float(m["scale"])
        out[:, hh] = softmax_rows(s, vis) @ val[:, hh]
    return (out.reshape(T, H * dv) * sigmoid(h @ W["g"].T)) @ W["o"].T


def dense_ff(h, W):
    return gelu_tanh(h @ W["up"].T) @ W["down"].T


# ------------------------------------------------------------------------------------------------ stream
def hyper_read(X, w_in):
    """X [S, T, E] -> the sublayer's input mix [T, E]."""
    return np.tensordot(w_in, X, axes=(0, 0))


def hyper_write(X, y, mix, w_out, r):
    """All copies at once from the old ones: X'[t] = sum_s mix[s, t] X[s] + r * out[t] * y."""
    return np.tensordot(mix.T, X, axes=(1, 0)) + r * w_out[:, None, None] * y[None]


def sub(weights, prefix):
    n = len(prefix)
    return {k[n:]: v for k, v in weights.items() if k.startswith(prefix)}


def forward(cfg, weights, tokens, layer_streams=None):
    """fp64 logits [T, vocab] of one sequence.  ``weights``: name -> array; ``layer_streams`` (a list) receives the summed
    stream [T, E] after every layer."""
    Wt = {k: np.asarray(v, dtype=np.float64) for k, v in weights.items()}
    eps, r = float(cfg["norm"]["eps"]), float(cfg.get("residual_mult", 1.0))
    S = cfg.get("streams")
    x0 = Wt["embed"][np.asarray(tokens)]
    X = np.stack([x0] * int(S)) if S else x0[None]
    for i, lc in enumerate(cfg["layers"]):
        p = f"l{int(lc.get('weights_of', i))}."
        kinds = [("1", "mix.")] + ([("2", "mlp.")] if lc.get("mlp") is not None else [])
        for q, part in kinds:
            u = hyper_read(X, Wt[p + f"hc{q}.in"]) if S else X[0]
            h = norm_one_plus(u, Wt[p + "norm" + q], eps)
            W = sub(Wt, p + part)
            if part == "mlp.":
                y = dense_ff(h, W)
            elif lc["type"] == "attention":
                y = differential_attention(h, W, lc["mixer"], eps)
            elif lc["type"] == "latent_attention":
                y = latent_attention(h, W, lc["mixer"], eps)
            else:
                raise ValueError(lc["type"])
            if p + "ls" + q in Wt:
                y = y * Wt[p + "ls" + q]
            X = hyper_write(X, y, Wt[p + f"hc{q}.mix"], Wt[p + f"hc{q}.out"], r) if S else X + r * y[None]
        if layer_streams is not None:
            layer_streams.append(X.sum(axis=0))
    x = norm_one_plus(X.sum(axis=0), Wt["final.norm"], eps)
    logits = x @ Wt["embed"].T
    cap = cfg.get("logit_softcap")
    return float(cap) * np.tanh(logits / float(cap)) if cap else logits
