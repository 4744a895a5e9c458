"""Plain, slow float64 statement of the Tebodra design, one function per mechanism (numpy only; test infrastructure,
never imported by the product).  It works on a whole sequence at once and keeps no cache: whatever schedule the product
runs (portions, single tokens, rings, recurrent state handed from step to step), its logits must equal these.

A layer is two pre-norm sublayers on one stream, both scaled by the model's residual multiplier r:

    x <- x + r * mixer(norm1(x));     x <- x + r * ff(norm2(x))        (the second is absent when the layer has no ff)

with norm(x) = x / sqrt(mean(x^2) + eps) * (1 + w).  Mixers: ``attention`` (softmax attention whose values are the
un-rotated keys, short convolutions on q and k, capped scores), ``attention_2`` (norm over the whole q and k projections,
chunk-local mask, a sink in the softmax denominator, optionally the keys and values of an earlier layer) and ``mlstm``
(matrix memory with exponential gates and a running stabiliser).  Feed-forward: W_down gelu(W_up h), the erf form.

Checkpoint names: ``embed``, ``head``, ``final.norm``; per layer i ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.mix.*``,
``l<i>.mlp.*``; Linear weights are [out, in].
"""
import math

import numpy as np


def unit_rms(x, eps):
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def norm_one_plus(x, w, eps):
    return unit_rms(x, eps) * (1.0 + w)


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def log_sigmoid(z):
    return -np.logaddexp(0.0, -z)


def gelu_erf(z):
    return 0.5 * z * (1.0 + np.vectorize(math.erf)(z / math.sqrt(2.0)))


def causal_filter(u, w):
    """u [T, C], w [C, taps]: y_t = sum_j w[:, j] u_(t - taps + 1 + j), nothing before the first token."""
    T, taps = u.shape[0], w.shape[1]
    y = np.zeros_like(u)
    for t in range(T):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                y[t] += w[:, j] * u[s]
    return y


def rotary_frequencies(rot):
    """One frequency per rotated pair: base^(-2i/dims), then the scaling the config asks for.  A scaling with ``original``
    bends by wavelength (short waves kept, long ones divided by ``factor``, a linear blend between); one with a factor
    alone divides every frequency."""
    dims = int(rot["dims"])
    f = np.array([float(rot["base"]) ** (-2.0 * i / dims) for i in range(dims // 2)])
    sc = rot.get("scaling")
    if not sc:
        return f
    factor = float(sc["factor"])
    if "original" not in sc:
        return f / factor
    orig, low, high = float(sc["original"]), float(sc["low"]), float(sc["high"])
    out = np.empty_like(f)
    for i, fi in enumerate(f):
        wave = 2.0 * math.pi / fi
        if wave < orig / high:
            out[i] = fi
        elif wave > orig / low:
            out[i] = fi / factor
        else:
            s = (orig / wave - low) / (high - low)
            out[i] = (1.0 - s) * fi / factor + s * fi
    return out


def rotate(x, rot, positions):
    """x [T, heads, dim]: the first rot.dims dimensions of every head turn, dimension i paired with i + dims/2."""
    dims = int(rot["dims"])
    half = dims // 2
    ang = np.asarray(positions, dtype=np.float64)[:, None] * rotary_frequencies(rot)[None, :]       # [T, half]
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    out = x.copy()
    a, b = x[..., :half], x[..., half:dims]
    out[..., :half] = a * c - b * s
    out[..., half:dims] = b * c + a * s
    return out


def softmax_attention(q, k, v, scale, softcap=None, chunk=None, sink=None):
    """q [T, H, d], k [T, G, d], v [T, G, e] -> [T, H, e].  Query i sees keys j <= i (within its chunk of ``chunk``
    positions, when given); scores are capped by cap * tanh(s / cap) when ``softcap`` is given; ``sink`` [H] adds exp(sink_h)
    to the denominator only."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = np.zeros((T, H, v.shape[2]))
    for h in range(H):
        g = h // (H // G)
        for i in range(T):
            lo = 0 if chunk is None else (i // chunk) * chunk
            s = (k[lo:i + 1, g] @ q[i, h]) * scale
            if softcap:
                s = softcap * np.tanh(s / softcap)
            top = max(s.max(), sink[h]) if sink is not None else s.max()
            w = np.exp(s - top)
            den = w.sum() + (math.exp(sink[h] - top) if sink is not None else 0.0)
            out[i, h] = (w[:, None] * v[lo:i + 1, g]).sum(0) / den
    return out


def attention(h, W, p, m, positions):
    """Mixer ``attention``: q and k pass a short causal filter, the values are the filtered keys before they turn."""
    T = h.shape[0]
    H, G, d = m["heads"], m["kv_heads"], m["dim"]
    q, k = h @ W[p + "q"].T, h @ W[p + "k"].T
    if p + "q.conv" in W:
        q, k = causal_filter(q, W[p + "q.conv"]), causal_filter(k, W[p + "k.conv"])
    v = k.reshape(T, G, d).copy()
    q, k = rotate(q.reshape(T, H, d), m["rot"], positions), rotate(k.reshape(T, G, d), m["rot"], positions)
    o = softmax_attention(q, k, v, m["scale"], softcap=m.get("softcap"))
    return (o.reshape(T, -1) * sigmoid(h @ W[p + "g"].T)) @ W[p + "o"].T, (k, v)


def attention_2(h, W, p, m, positions, eps, borrowed=None):
    """Mixer ``attention_2``: one RMS norm over the whole query projection (and one over the key projection) with plain
    weights, chunk-local mask, sink.  ``borrowed``: (keys, values) of the layer named by ``kv_from``."""
    T = h.shape[0]
    H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = unit_rms(h @ W[p + "q"].T, eps) * W[p + "q.norm"]
    q = rotate(q.reshape(T, H, d), m["rot"], positions)
    if borrowed is None:
        k = unit_rms(h @ W[p + "k"].T, eps) * W[p + "k.norm"]
        k = rotate(k.reshape(T, G, d), m["rot"], positions)
        v = (h @ W[p + "v"].T).reshape(T, G, e)
    else:
        k, v = borrowed
    chunk = (m.get("mask") or {}).get("size")
    o = softmax_attention(q, k, v, m["scale"], chunk=chunk, sink=W.get(p + "sink"))
    return (o.reshape(T, -1) * sigmoid(h @ W[p + "g"].T)) @ W[p + "o"].T, (k, v)


def mlstm(h, W, p, m, eps):
    """Matrix memory with a log input gate i and a log forget gate f, both capped, and a running maximum mx that starts at 0:
        mx_t = max(f_t + mx_(t-1), i_t);  S_t = e^(f_t + mx_(t-1) - mx_t) S_(t-1) + e^(i_t - mx_t) k_t v_t^T;  n_t alike with k_t
        o_t = S_t^T q_t / (max(|n_t . q_t|, e^(-mx_t)) + 1e-6)
    then every head divided by its root mean square, a weight over all heads, a sigmoid gate, the output projection."""
    T = h.shape[0]
    H, d, e, cap = m["heads"], m["dim"], m["vdim"], float(m.get("gate_cap") or 0.0)

    def capped(z):                      # a cap of 0 (or none) leaves the pre-activation as it is
        return cap * np.tanh(z / cap) if cap > 0 else z
    q = (h @ W[p + "q"].T).reshape(T, H, d) * d ** -0.5
    k = (h @ W[p + "k"].T).reshape(T, H, d)
    v = (h @ W[p + "v"].T).reshape(T, H, e)
    gi = capped(h @ W[p + "i"].T + W[p + "i.b"])
    gf = log_sigmoid(capped(h @ W[p + "f"].T + W[p + "f.b"]))
    out = np.zeros((T, H, e))
    for a in range(H):
        S, n, mx = np.zeros((d, e)), np.zeros(d), 0.0
        for t in range(T):
            new = max(gf[t, a] + mx, gi[t, a])
            keep, take = math.exp(gf[t, a] + mx - new), math.exp(gi[t, a] - new)
            S = keep * S + take * np.outer(k[t, a], v[t, a])
            n = keep * n + take * k[t, a]
            mx = new
            out[t, a] = (S.T @ q[t, a]) / (max(abs(n @ q[t, a]), math.exp(-mx)) + 1e-6)
    out = unit_rms(out, eps).reshape(T, H * e) * W[p + "norm"]
    return (out * sigmoid(h @ W[p + "g"].T)) @ W[p + "o"].T


def dense_ff(h, W, p):
    return gelu_erf(h @ W[p + "up"].T) @ W[p + "down"].T


def forward(cfg, W, tokens, return_layers=False):
    """cfg: the dictionary of config.json; W: name -> float64 array; tokens: ids of ONE sequence from position 0.
    Returns logits [T, vocab] (and the stream after every layer, [layers, T, width])."""
    tokens = np.asarray(tokens)
    eps, r = float(cfg["norm"]["eps"]), float(cfg.get("residual_mult", 1.0))
    positions = np.arange(len(tokens))
    x = W["embed"][tokens]
    kept, streams = {}, []
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.mix.", layer["mixer"]
        h = norm_one_plus(x, W[f"l{i}.norm1"], eps)
        if layer["type"] == "attention":
            y, kept[i] = attention(h, W, p, m, positions)
        elif layer["type"] == "attention_2":
            src = m.get("kv_from")
            y, kept[i] = attention_2(h, W, p, m, positions, eps, borrowed=None if src is None else kept[src])
        elif layer["type"] == "mlstm":
            y = mlstm(h, W, p, m, eps)
        else:
            raise ValueError(layer["type"])
        x = x + r * y
        if layer.get("mlp") is not None:
            x = x + r * dense_ff(norm_one_plus(x, W[f"l{i}.norm2"], eps), W, f"l{i}.mlp.")
        streams.append(x.copy())
    logits = norm_one_plus(x, W["final.norm"], eps) @ W["head"].T
    return (logits, np.stack(streams)) if return_layers else logits
