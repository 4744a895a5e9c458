"""The mechanisms Bededra brought, each alone on the GPU against its float64 statement (oracle/bededra.py): short
convolution with state, the diagonal-decay recurrence in both uses, window attention with kept tokens / soft cap /
distance penalty / mixed heads on a ring that wraps, the group-limited router, the plain gated experts, the norms.
Inputs are made so that a fault shows: one key that takes nearly all the weight just inside or just outside a window, a
far key among hundreds, a kept token, decays close to one over a long sequence."""
import numpy as np
import pytest
import torch

from oracle import bededra as O

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]
TOL = {torch.float32: 2e-5, torch.bfloat16: 2e-2}


def dev(a, dtype=torch.float32):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to("cuda", dtype)


def rounded(a, dtype):
    """What the kernel sees of ``a`` in ``dtype``, as float64."""
    return dev(a, dtype).double().cpu().numpy()


def close(got, want, tol):
    got = got.double().cpu().numpy() if torch.is_tensor(got) else got
    err = np.abs(got - want).max() / max(np.abs(want).max(), 1e-9)
    assert err < tol, err


def pos(lo, hi):
    return torch.arange(lo, hi, dtype=torch.int32, device="cuda")


# ------------------------------------------------------------------ short convolution
@pytest.mark.parametrize("taps,portions", [(4, [1] * 9), (4, [9]), (4, [2, 1, 3, 3]), (1, [4, 5]), (8, [3, 2, 4]), (3, [1, 8])])
@pytest.mark.parametrize("dtype", DTYPES)
def test_short_conv_in_portions(taps, portions, dtype):
    from lit_llama.short_conv import ShortConv

    r = np.random.RandomState(taps)
    B, T, C, stride, col0 = 2, sum(portions), 37, 50, 5
    x = r.randn(B, T, stride)
    w, b = r.randn(C, taps), r.randn(C)
    conv = ShortConv(C, taps, True, "cuda")
    conv.load(dev(w), dev(b))
    state = torch.full(conv.state_shape(B), float("nan"), device="cuda")      # a slot nobody cleared
    xr = rounded(x, dtype)
    for residual, silu in ((False, True), (True, False)):
        want = np.stack([O.short_conv(xr[i, :, col0:col0 + C], w, b) for i in range(B)])
        if residual:
            want = want + xr[:, :, col0:col0 + C]
        if silu:
            want = O.silu(want)
        got, at = [], 0
        for n in portions:
            part = dev(x[:, at:at + n].reshape(B * n, stride), dtype)
            got.append(conv(part, col0, state, pos(at, at + n), B, n, dtype, residual=residual, silu=silu).reshape(B, n, C))
            at += n
        close(torch.cat(got, 1), want, TOL[dtype])


def test_short_conv_long_prompt_many_time_tiles():
    from lit_llama.short_conv import ShortConv

    r = np.random.RandomState(0)
    T, C = 700, 16
    x, w = r.randn(T, C), r.randn(C, 4)
    conv = ShortConv(C, 4, False, "cuda")
    conv.load(dev(w))
    state = torch.zeros(conv.state_shape(1), device="cuda")
    a = conv(dev(x[:650]), 0, state, pos(0, 650), 1, 650, torch.float32)
    b = conv(dev(x[650:]), 0, state, pos(650, 700), 1, 50, torch.float32)
    close(torch.cat([a, b]), O.short_conv(x, w), 2e-5)


# ------------------------------------------------------------------ recurrence
@pytest.mark.parametrize("H,G,n,p", [(3, 1, 10, 8), (4, 2, 48, 32), (2, 2, 16, 5), (1, 1, 1, 1), (2, 1, 130, 3), (6, 6, 32, 64), (2, 1, 300, 3), (2, 2, 128, 16)])
@pytest.mark.parametrize("per_channel", [False, True])
def test_decay_scan_in_portions(H, G, n, p, per_channel):
    from lit_llama.recurrence import decay_scan

    r = np.random.RandomState(n + p)
    T = 41
    q, k, v = r.randn(T, G * n), r.randn(T, G * n), r.randn(T, H * p)
    a = r.uniform(0.7, 1.0, (T, H, n) if per_channel else (T, H))
    ks, skip = r.uniform(0.1, 1.5, (T, H)), r.randn(H)
    want = np.zeros((T, H * p))
    for h in range(H):
        g = h // (H // G)
        want[:, h * p:(h + 1) * p] = O.linear_recurrence(q[:, g * n:(g + 1) * n], k[:, g * n:(g + 1) * n], v[:, h * p:(h + 1) * p],
                                                         a[:, h], ks[:, h], skip[h], 0.5)
    state = torch.full((1, H, n, p), float("nan"), device="cuda")
    for portions in ([T], [1] * T, [17, 2, 1, 21]):
        got, at = [], 0
        for m in portions:
            sl = slice(at, at + m)
            got.append(decay_scan(dev(q[sl]), 0, dev(k[sl]), 0, dev(v[sl]), 0, dev(a[sl]), per_channel, dev(ks[sl]), dev(skip), 0.5,
                                  state, pos(at, at + m), 1, m, H, G, n, p))
            at += m
        close(torch.cat(got), want, 2e-5)


def test_decay_scan_remembers_over_a_long_sequence():
    """Decay one: what the first token wrote is read back unchanged 600 tokens later, across portions."""
    from lit_llama.recurrence import decay_scan

    T, n, p = 600, 8, 4
    q, k, v = np.zeros((T, n)), np.zeros((T, n)), np.zeros((T, p))
    k[0, 3], v[0] = 1.0, [1.0, 2.0, 3.0, 4.0]
    q[-1, 3] = 1.0
    a = np.ones((T, 1))
    state = torch.zeros((1, 1, n, p), device="cuda")
    y1 = decay_scan(dev(q[:333]), 0, dev(k[:333]), 0, dev(v[:333]), 0, dev(a[:333]), False, None, None, 1.0, state, pos(0, 333), 1, 333,
                    1, 1, n, p)
    y2 = decay_scan(dev(q[333:]), 0, dev(k[333:]), 0, dev(v[333:]), 0, dev(a[333:]), False, None, None, 1.0, state, pos(333, T), 1,
                    T - 333, 1, 1, n, p)
    assert float(y1.abs().max()) == 0.0
    close(y2[-1], np.array([1.0, 2.0, 3.0, 4.0]), 1e-6)


def test_gates_of_the_recurrences():
    from lit_llama import _native as N

    r = np.random.RandomState(3)
    M, H = 9, 5
    raw, bias, a_log = r.randn(M, H + 3) * 4, r.randn(H), r.randn(H)
    dt, decay = torch.empty((M, H), device="cuda"), torch.empty((M, H), device="cuda")
    x, bd, ad = dev(raw), dev(bias), dev(a_log)
    N.call("ll_ssm_gates", N.ptr_at(x, 3), N.LL_F32, H + 3, N.ptr(bd), N.ptr(ad), N.ptr(dt), N.ptr(decay), M, H, N.stream())
    want = O.softplus(raw[:, 3:] + bias)
    close(dt, want, 1e-5)
    close(decay, np.exp(-np.exp(a_log) * want), 1e-5)
    z, b = r.randn(M, H) * 5, r.randn(H)
    out = torch.empty((M, H), device="cuda")
    zd, bd = dev(z), dev(b)
    N.call("ll_channel_decay", N.ptr(zd), N.LL_F32, H, N.ptr(bd), 7.0, N.ptr(out), M, H, N.stream())
    close(out, O.sigmoid(z + b) ** (1 / 7.0), 1e-5)


@pytest.mark.parametrize("gate_first,shared,groups", [(True, False, 1), (True, False, 3), (False, True, 4), (False, True, 1)])
@pytest.mark.parametrize("dtype", DTYPES)
def test_gated_group_norm(gate_first, shared, groups, dtype):
    from lit_llama.recurrence import gated_group_norm

    r = np.random.RandomState(groups)
    M, gs = 7, 10
    C = groups * gs
    y, g = r.randn(M, C), r.randn(M, C + 6)
    w = r.randn(gs if shared else C)
    gr = rounded(g, dtype)[:, 6:]
    wf = np.tile(w, groups) if shared else w
    if gate_first:
        want = O.rms((y * O.silu(gr)).reshape(M, groups, gs), 1e-5).reshape(M, C) * wf
    else:
        want = O.rms(y.reshape(M, groups, gs), 1e-5).reshape(M, C) * wf * O.silu(gr)
    got = gated_group_norm(dev(y), dev(g, dtype), 6, dev(w), shared, 1e-5, groups, gate_first, dtype)
    close(got, want, TOL[dtype])


# ------------------------------------------------------------------ window attention
def attention_setup(H, G, D, V, window, keep, ring, dtype, cap=30.0, seed=0):
    from lit_llama.window_attention import WindowAttention, WindowAttentionSpec

    r = np.random.RandomState(seed)
    spec = WindowAttentionSpec(width=H * V, heads=H, kv_heads=G, dim=D, vdim=V, scale=D ** -0.5, softcap=cap, window=window,
                               keep_first=keep)
    att = WindowAttention(spec, dtype, "cuda")
    r1, r2, talk = r.uniform(0, 0.5, H), r.uniform(0.1, 2, H), np.eye(H) + 0.3 * r.randn(H, H)
    att.r1.copy_(dev(r1)); att.r2.copy_(dev(r2)); att.talk.copy_(dev(talk))
    att.w_o.copy_(torch.eye(H * V, device="cuda", dtype=dtype))
    caches = [torch.full(s, float("nan"), device="cuda", dtype=dtype) for s in att.cache_shapes(1, ring)]
    return att, caches, (r1, r2, talk)


def run_attention(att, caches, proj, portions, dtype, splits=1):
    out, at = [], 0
    for n in portions:
        out.append(att(dev(proj[at:at + n], dtype), 0, 1, n, pos(at, at + n), caches, splits))
        at += n
    return torch.cat(out)


def attention_want(att, proj, params, dtype):
    s = att.spec
    c = att.cols
    pr = rounded(proj, dtype)
    T = pr.shape[0]
    q = pr[:, :c["k"]].reshape(T, s.heads, s.dim)
    k = pr[:, c["k"]:c["v"]].reshape(T, s.kv_heads, s.dim)
    v = pr[:, c["v"]:c["g"]].reshape(T, s.kv_heads, s.vdim)
    r1, r2, talk = params
    return O.attention_core(q, k, v, pr[:, c["g"]:], r1, r2, talk, s.scale, s.softcap, s.window, s.keep_first).reshape(T, -1)


@pytest.mark.parametrize("H,G,D,V,window,keep", [(4, 2, 8, 8, 6, 2), (3, 3, 5, 7, 4, 0), (6, 1, 16, 4, 9, 3), (1, 1, 4, 4, 1, 0),
                                                 (2, 2, 8, 12, None, 0), (8, 4, 64, 64, 12, 5), (2, 1, 8, 8, 3, 7),
                                                 # sizes the tensor-core form takes in bfloat16 (heads padded to 16; two heads
                                                 # per warp and two rounds of output heads; one head)
                                                 (3, 1, 16, 16, 5, 1), (16, 4, 32, 16, 20, 3), (32, 8, 16, 32, 9, 2),
                                                 (1, 1, 128, 128, None, 0), (40, 40, 16, 16, 7, 0)])
@pytest.mark.parametrize("dtype", DTYPES)
def test_window_attention_on_a_wrapping_ring(H, G, D, V, window, keep, dtype):
    T = 40
    for ring_portion, portions in ((T, [T]), (1, [1] * T), (3, [3, 2, 1, 3, 3, 3, 1, 2, 3, 3, 3, 3, 3, 3, 3, 1]), (8, [8, 5, 8, 8, 8, 3])):
        ring = T - keep if window is None else min(T, window - 1 + ring_portion)
        att, caches, params = attention_setup(H, G, D, V, window, keep, ring, dtype, seed=H + D)
        proj = np.random.RandomState(1).randn(T, att.n_in)
        got = run_attention(att, caches, proj, portions, dtype)
        close(got, attention_want(att, proj, params, dtype), TOL[dtype] * 2)


@pytest.mark.parametrize("dtype", DTYPES)
def test_window_attention_over_many_chunks(dtype):
    """A window of 100 keys beside 7 kept tokens over 300 tokens: every query tile walks several staged chunks, the ring
    (window - 1 + 64 slots) wraps twice, and the last tokens are decoded alone with the window split over blocks."""
    H, G, D, V, window, keep, T = 8, 2, 32, 32, 100, 7, 300
    att, caches, params = attention_setup(H, G, D, V, window, keep, window - 1 + 64, dtype, cap=25.0, seed=3)
    proj = np.random.RandomState(4).randn(T, att.n_in)
    want = attention_want(att, proj, params, dtype)
    for portions, splits in (([64] * 4 + [44], 1), ([50, 64, 64, 64, 40] + [1] * 18, 4)):
        out, at = [], 0
        for n in portions:
            out.append(att(dev(proj[at:at + n], dtype), 0, 1, n, pos(at, at + n), caches, splits if n == 1 else 1))
            at += n
        close(torch.cat(out), want, TOL[dtype] * 2)


@pytest.mark.parametrize("splits", [1, 3, 16])
def test_one_key_that_takes_the_weight_at_every_edge(splits):
    """Query i and one key j* share a large component, so j* takes nearly all of the weight when it is visible: j* just
    inside the window (i - j* = window - 1), just outside (= window), a kept token far back, the first token after the
    kept ones (not kept, out of the window), in a prompt's portion and decoded alone, on a ring that has wrapped."""
    H, G, D, V, window, keep, T = 2, 1, 8, 4, 16, 3, 120
    dtype = torch.float32
    for i, jstar in ((100, 85), (100, 84), (100, 2), (100, 3), (60, 45), (60, 44), (119, 0), (18, 3), (19, 3)):
        att, caches, params = attention_setup(H, G, D, V, window, keep, window - 1 + 20, dtype, cap=40.0)
        proj = 0.1 * np.random.RandomState(i).randn(T, att.n_in)
        c = att.cols
        proj[i, 0:D] += 6.0; proj[i, D:2 * D] += 6.0                    # both heads' queries
        proj[jstar, c["k"]:c["k"] + D] += 6.0
        proj[jstar, c["v"]:c["v"] + V] = [9.0, -9.0, 9.0, -9.0]
        want = attention_want(att, proj, params, dtype)
        seen = O.visible(i, jstar, window, keep)
        assert (np.abs(want[i]).max() > 1.0) == seen                     # the case shows what it is meant to show
        for portions in ([20] * 6, [20] * (i // 20) + [1] * (T - 20 * (i // 20))):
            got = run_attention(att, caches, proj, portions, dtype, splits)
            close(got, want, 2e-5)


def test_a_far_key_among_hundreds():
    H, G, D, V, T = 4, 2, 16, 8, 700
    att, caches, params = attention_setup(H, G, D, V, None, 0, T, torch.float32, cap=60.0)
    proj = 0.1 * np.random.RandomState(5).randn(T, att.n_in)
    c = att.cols
    att.r1.zero_()
    params = (np.zeros(H), params[1], params[2])
    proj[T - 1, :H * D] += 5.0
    proj[11, c["k"]:c["k"] + G * D] += 5.0
    proj[11, c["v"]:c["v"] + G * V] = 7.0
    want = attention_want(att, proj, params, torch.float32)
    assert np.abs(want[T - 1]).max() > 1.0
    got = run_attention(att, caches, proj, [650] + [1] * 50, torch.float32, splits=7)
    close(got, want, 2e-5)


# ------------------------------------------------------------------ router and experts
@pytest.mark.parametrize("X,top,count,keep", [(16, 4, 4, 3), (6, 2, 3, 2), (9, 2, 3, 1), (4, 4, 2, 2), (8, 3, 1, 1), (1, 1, 1, 1), (40, 5, 8, 2)])
@pytest.mark.parametrize("dtype", DTYPES)
def test_group_limited_router(X, top, count, keep, dtype):
    from lit_llama.moe import MoE, MoESpec

    r = np.random.RandomState(X)
    M, E = 33, 24
    spec = MoESpec(width=E, experts=X, top=top, ff=8, limit=float("inf"), alpha=1.0, up_shift=0.0, score="all", groups=count,
                   keep_groups=keep, router_bias=False)
    moe = MoE(spec, dtype, "cuda")
    w = r.randn(X, E)
    moe.w_router.copy_(dev(w))
    x = r.randn(M, E)
    idx, wts, offsets, perm = moe.route(dev(x, dtype))
    widx, wwts = O.route(rounded(x, dtype), rounded(w, torch.float32), top, count, keep)
    assert np.array_equal(np.sort(idx.cpu().numpy(), 1), np.sort(widx, 1))
    order = np.argsort(idx.cpu().numpy(), 1)
    close(np.take_along_axis(wts.double().cpu().numpy(), order, 1), np.take_along_axis(wwts, np.argsort(widx, 1), 1), 1e-5)
    off, pm, flat = offsets.cpu().numpy(), perm.cpu().numpy(), idx.cpu().numpy().reshape(-1)
    assert off[-1] == M * top and sorted(pm.tolist()) == list(range(M * top))
    for e in range(X):
        assert (flat[pm[off[e]:off[e + 1]]] == e).all()


@pytest.mark.parametrize("M,E,ff", [(5, 32, 16), (600, 64, 64)])
@pytest.mark.parametrize("dtype", DTYPES)
def test_plain_gated_experts(M, E, ff, dtype):
    """silu(gate) * up without clamp or shift, through the router and both grouped products (M = 600 in bfloat16 takes the
    tcgen05 kernels)."""
    from lit_llama.moe import MoE, MoESpec

    r = np.random.RandomState(M)
    X, top = 4, 2
    cfgf = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": X, "top": top, "groups": {"count": 2, "keep": 2}}}
    spec = MoESpec(width=E, experts=X, top=top, ff=ff, limit=float("inf"), alpha=1.0, up_shift=0.0, score="all", groups=2, keep_groups=2,
                   router_bias=False)
    moe = MoE(spec, dtype, "cuda")
    W = {"router": r.randn(X, E)}
    for e in range(X):
        W[f"e{e}.gate"], W[f"e{e}.up"], W[f"e{e}.down"] = r.randn(ff, E) * 3 / np.sqrt(E), r.randn(ff, E) / np.sqrt(E), r.randn(E, ff) / 4
    W = {k: rounded(v, dtype if k != "router" else torch.float32) for k, v in W.items()}
    moe.load(lambda s: dev(W[s]))
    x = r.randn(M, E)
    want = O.moe_ff(rounded(x, dtype), W, "", cfgf)
    close(moe(dev(x, dtype)), want, TOL[dtype] * 2)


@pytest.mark.parametrize("dtype", DTYPES)
def test_residual_update_and_both_norms(dtype):
    from lit_llama.stepping import add_norm_pair

    r = np.random.RandomState(0)
    M, E = 6, 50
    x, a, b, c = r.randn(M, E), r.randn(M, E), r.randn(M, E), r.randn(M, E)
    w1, w2 = r.randn(E), r.randn(E)
    xs = dev(x)
    h1 = torch.empty((M, E), device="cuda")
    h2 = torch.empty((M, E), device="cuda", dtype=dtype)
    add_norm_pair(xs, [(dev(a, dtype), 0.75), (dev(b, dtype), 1.25), (dev(c, dtype), 1.0)], dev(w1), dev(w2), 1e-6, h1, h2, dtype)
    nx = x + 0.75 * rounded(a, dtype) + 1.25 * rounded(b, dtype) + rounded(c, dtype)
    close(xs, nx, 1e-6)
    close(h1, O.rms(nx, 1e-6) * w1, 1e-5)
    close(h2, O.rms(nx, 1e-6) * w2, TOL[dtype])


@pytest.mark.parametrize("dtype", DTYPES)
def test_dense_feed_forward(dtype):
    from lit_llama.feed_forward import DenseFF

    r = np.random.RandomState(1)
    M, E, ff = 9, 24, 40
    W = {"up": rounded(r.randn(ff, E) / 5, dtype), "down": rounded(r.randn(E, ff) / 6, dtype)}
    f = DenseFF(E, ff, "relu2", dtype, "cuda")
    f.load(lambda s: dev(W[s]))
    x = r.randn(M, E)
    close(f(dev(x, dtype)), O.dense_ff(rounded(x, dtype), W, ""), TOL[dtype] * 2)
