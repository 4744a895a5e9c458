"""The mechanisms Tebodra adds, each alone against its float64 statement (oracle/tebodra.py): rotation with norm and ring
append, softmax attention in its fp32 and tensor-core forms (chunk edges, far keys, the sink, the first tokens, rings that
wrap, key ranges split over blocks), the exponential gates with their stabiliser, the recurrence with a normaliser column,
the read-out norm, gelu.  Inputs are made so that a fault shows: one key takes the whole weight just inside or just outside
a chunk, far back among hundreds, or nothing but the sink does."""
import math

import numpy as np
import pytest
import torch

from oracle import tebodra as O
from tests.util_tebodra import bf16

pytestmark = pytest.mark.gpu


def dev(a, dtype=torch.float32):
    return None if a is None else torch.tensor(np.asarray(a, dtype=np.float64), dtype=dtype, device="cuda")


def host(t):
    return t.double().cpu().numpy()


def pos(a, b):
    return torch.arange(a, b, dtype=torch.int32, device="cuda")


def run_attention(q, k, v, first, ring, scale, dtype, cap=0.0, chunk=0, window=0, sink=None, gate=None, splits=1, form=0):
    """q [L, H, d], k [L, G, d], v [L, G, e] for positions 0..L-1; the queries at ``first``..L-1 run in ONE step against a ring
    of ``ring`` slots that holds every position written so far (position j in slot j % ring).  Returns [L - first, H, e]."""
    import lit_llama._native as N

    L, H, d = q.shape
    G, e = k.shape[1], v.shape[2]
    T = L - first
    kh, vh = np.full((1, ring, G * d), np.nan), np.full((1, ring, G * e), np.nan)
    for j in range(L):
        kh[0, j % ring], vh[0, j % ring] = k[j].reshape(-1), v[j].reshape(-1)
    kc, vc = dev(kh, dtype), dev(vh, dtype)
    qd = dev(q[first:].reshape(T, H * d), dtype)
    gd = dev(gate[first:].reshape(T, H * e), dtype) if gate is not None else None
    sd, pd = dev(sink), pos(first, L)                           # operands stay alive until the kernel has run
    y = torch.empty((T, H * e), dtype=dtype, device="cuda")
    scratch = torch.empty(max(4, N.call_ret("ll_softmax_attn_scratch_bytes", T, H, e, splits) // 4), dtype=torch.float32, device="cuda")
    N.call("ll_softmax_attn", N.ptr(qd), H * d, N.ptr(gd), H * e, N.ptr(kc), N.ptr(vc), N.dtype_code(dtype), N.ptr(pd),
           N.ptr(sd), float(scale), float(cap), 1, T, H, G, d, e, window, chunk, ring, splits, form, N.ptr(scratch), N.ptr(y),
           N.stream())
    torch.cuda.synchronize()
    return host(y).reshape(T, H, e)


def want_attention(q, k, v, first, scale, cap=0.0, chunk=0, sink=None, gate=None):
    o = O.softmax_attention(q, k, v, scale, softcap=cap or None, chunk=chunk or None, sink=sink)
    if gate is not None:
        o = o * O.sigmoid(gate)
    return o[first:]


def rand_qkv(r, L, H, G, d, e, gain=1.0):
    return bf16(r.randn(L, H, d) * gain), bf16(r.randn(L, G, d) * gain), bf16(r.randn(L, G, e))


@pytest.mark.parametrize("H,G,d,e", [(4, 2, 16, 16), (3, 3, 6, 10), (6, 1, 40, 24), (2, 2, 72, 136), (1, 1, 1, 1), (8, 2, 200, 8)])
@pytest.mark.parametrize("chunk,cap,with_sink", [(0, 0.0, False), (9, 0.0, True), (0, 4.0, False), (16, 2.5, True)])
def test_attention_against_oracle_fp32(H, G, d, e, chunk, cap, with_sink):
    r = np.random.RandomState(H * 100 + d + chunk)
    L = 50
    q, k, v = rand_qkv(r, L, H, G, d, e)
    sink = bf16(r.randn(H)) if with_sink else None
    gate = bf16(r.randn(L, H, e))
    scale = 1.7 / math.sqrt(d)
    for first, splits in ((0, 1), (30, 1), (49, 1), (49, 3), (47, 16)):
        ring = L if not chunk else chunk - 1 + (L - first)       # as short as the look-back allows: it wraps
        got = run_attention(q, k, v, first, ring, scale, torch.float32, cap, chunk, 0, sink, gate, splits)
        want = want_attention(q, k, v, first, scale, cap, chunk, sink, gate)
        assert np.abs(got - want).max() < 2e-5 * max(1.0, np.abs(want).max()), (first, splits)


@pytest.mark.parametrize("d,e", [(16, 16), (32, 8), (8, 64), (72, 40), (96, 96), (128, 128), (64, 128)])
@pytest.mark.parametrize("chunk,cap,with_sink", [(0, 0.0, False), (40, 0.0, True), (23, 3.0, True)])
def test_tensor_core_form_against_oracle(d, e, chunk, cap, with_sink):
    """bf16 steps of 16 tokens or more: tiles of 64 queries, chunk edges inside tiles, a last tile that is not full, heads
    narrower than the padded tile, a ring that wraps."""
    r = np.random.RandomState(d + e + chunk)
    L, H, G = 171, 4, 2
    q, k, v = rand_qkv(r, L, H, G, d, e)
    sink = bf16(r.randn(H)) if with_sink else None
    gate = bf16(r.randn(L, H, e))
    scale = 1.7 / math.sqrt(d)
    for first in (0, 41, 155):
        ring = L if not chunk else chunk - 1 + (L - first)
        want = want_attention(q, k, v, first, scale, cap, chunk, sink, gate)
        got = run_attention(q, k, v, first, ring, scale, torch.bfloat16, cap, chunk, 0, sink, gate)
        plain = run_attention(q, k, v, first, ring, scale, torch.bfloat16, cap, chunk, 0, sink, gate, form=1)
        tol = 1.5e-2 * max(1.0, np.abs(want).max())             # the outputs are bf16
        assert np.abs(got - want).max() < tol and np.abs(plain - want).max() < tol, first


def _spike(L, H, G, d, e, at, query, r):
    """Small random keys, except that key ``at`` and query ``query`` point the same way with a large product."""
    q, k, v = rand_qkv(r, L, H, G, d, e, gain=0.05)
    u = np.zeros(d)
    u[0] = 6.0
    k[at, :] = u
    q[query, :] = u
    return q, k, v


@pytest.mark.parametrize("dtype,first,splits", [(torch.float32, 0, 1), (torch.float32, 60, 1), (torch.float32, 69, 1), (torch.float32, 69, 3),
                                                (torch.float32, 69, 16), (torch.bfloat16, 0, 1), (torch.bfloat16, 50, 1)])
def test_a_key_just_inside_and_just_outside_a_chunk(dtype, first, splits):
    """Query 69 lies in the chunk 64..79.  A key at 64 that matches it takes nearly all the weight; the same key at 63 is not
    seen at all.  In a prompt's portion and decoded alone, whatever the split of the keys."""
    r = np.random.RandomState(5)
    L, H, G, d, e, chunk = 70, 4, 2, 16, 16, 16
    for at, seen in ((64, True), (63, False)):
        q, k, v = _spike(L, H, G, d, e, at, 69, r)
        got = run_attention(q, k, v, first, L, 1.0, dtype, chunk=chunk, splits=splits)[-1]
        want = want_attention(q, k, v, first, 1.0, chunk=chunk)[-1]
        assert np.abs(got - want).max() < (2e-5 if dtype == torch.float32 else 2e-2)
        near = np.abs(got - v[at][np.arange(H) // (H // G)]).max()
        assert (near < 0.05) == seen, (at, near)


@pytest.mark.parametrize("dtype,first,splits", [(torch.float32, 0, 1), (torch.float32, 699, 1), (torch.float32, 699, 16), (torch.bfloat16, 600, 1)])
def test_a_far_key_among_hundreds(dtype, first, splits):
    r = np.random.RandomState(6)
    L, H, G, d, e = 700, 2, 1, 32, 32
    q, k, v = _spike(L, H, G, d, e, 3, 699, r)
    got = run_attention(q, k, v, first, L, 1.0, dtype, splits=splits)[-1]
    want = want_attention(q, k, v, first, 1.0)[-1]
    assert np.abs(got - want).max() < (2e-5 if dtype == torch.float32 else 2e-2)
    assert np.abs(got - v[3][[0, 0]]).max() < 0.05


@pytest.mark.parametrize("dtype,first", [(torch.float32, 0), (torch.float32, 39), (torch.bfloat16, 0)])
def test_the_sink_takes_weight_without_a_value(dtype, first):
    """Scores near zero and a sink of 8: almost nothing is left for the values.  Without the sink the output is their mean."""
    r = np.random.RandomState(7)
    L, H, G, d, e = 40, 2, 2, 8, 8
    q, k, v = rand_qkv(r, L, H, G, d, e, gain=0.01)
    v = v + 3.0
    sink = np.array([8.0, -30.0])
    got = run_attention(q, k, v, first, L, 1.0, dtype, sink=sink)
    want = want_attention(q, k, v, first, 1.0, sink=sink)
    assert np.abs(got - want).max() < (2e-5 if dtype == torch.float32 else 3e-2)
    assert np.abs(got[-1, 0]).max() < 0.1 and np.abs(got[-1, 1] - 3.0).max() < 1.0


def test_rotation_norm_and_ring_append_far_from_zero():
    """Positions 5000.., a partial rotation with band-wise rescaled frequencies, whole-row norms, values that are the keys
    before they turn, and rows landing in their ring slots; a second call with queries only leaves the ring alone."""
    import lit_llama._native as N
    from lit_llama.rotary import RotarySpec

    r = np.random.RandomState(8)
    T, H, G, d, ring, p0 = 9, 3, 1, 10, 11, 5000       # a step never brings more tokens than the ring has slots
    rot = {"base": 300.0, "dims": 6, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 24}}
    q, k = bf16(r.randn(T, H * d)), bf16(r.randn(T, G * d))
    wq, wk = bf16(1 + 0.3 * r.randn(H * d)), bf16(1 + 0.3 * r.randn(G * d))
    eps = 1e-3
    spec = RotarySpec.from_dict(rot)
    freq = spec.frequencies("cuda")
    assert np.abs(host(freq) - O.rotary_frequencies(rot)).max() < 1e-7
    positions = np.arange(p0, p0 + T)
    for normed in (True, False):
        qn = O.unit_rms(q, eps) * wq if normed else q
        kn = O.unit_rms(k, eps) * wk if normed else k
        want_q = O.rotate(qn.reshape(T, H, d), rot, positions).reshape(T, -1)
        want_k = O.rotate(kn.reshape(T, G, d), rot, positions).reshape(T, -1)
        qd, kd = dev(q), dev(k)
        wqd, wkd = (dev(wq), dev(wk)) if normed else (None, None)
        pd = pos(p0, p0 + T)
        q_out = torch.empty((T, H * d), device="cuda")
        kc = torch.zeros((1, ring, G * d), device="cuda")
        vc = torch.zeros((1, ring, G * d), device="cuda")
        N.call("ll_qk_rotary_append", N.ptr(qd), H * d, N.ptr(kd), G * d, None, 0, N.LL_F32, N.ptr(wqd),
               N.ptr(wkd), eps, N.ptr(freq), spec.dims, N.ptr(pd), N.ptr(q_out), N.ptr(kc),
               N.ptr(vc), 1, T, H, G, d, d, ring, N.stream())
        # fp32 angles of about 5000 radians carry an error of a few 1e-4
        assert np.abs(host(q_out) - want_q).max() < 3e-3
        for t in range(T):
            assert np.abs(host(kc[0, (p0 + t) % ring]) - want_k[t]).max() < 3e-3
            assert np.abs(host(vc[0, (p0 + t) % ring]) - kn[t]).max() < 1e-6
        before = kc.clone()
        N.call("ll_qk_rotary_append", N.ptr(qd), H * d, None, 0, None, 0, N.LL_F32, N.ptr(wqd), None, eps,
               N.ptr(freq), spec.dims, N.ptr(pd), N.ptr(q_out), None, None, 1, T, H, G, d, d, ring, N.stream())
        assert torch.equal(before, kc)
    near = O.rotate(q.reshape(T, H, d), rot, np.arange(T)).reshape(T, -1)                  # near zero the angles are exact
    qd, pd = dev(q), pos(0, T)
    N.call("ll_qk_rotary_append", N.ptr(qd), H * d, None, 0, None, 0, N.LL_F32, None, None, eps, N.ptr(freq), spec.dims,
           N.ptr(pd), N.ptr(q_out), None, None, 1, T, H, G, d, d, ring, N.stream())
    assert np.abs(host(q_out) - near).max() < 2e-6


def _gates(zi, zf, cap):
    T, H = zi.shape
    c = (lambda z: cap * np.tanh(z / cap)) if cap > 0 else (lambda z: z)
    li, lf = c(zi), O.log_sigmoid(c(zf))
    keep, take, stab = np.zeros((T, H)), np.zeros((T, H)), np.zeros((T, H))
    mx = np.zeros(H)
    for t in range(T):
        new = np.maximum(lf[t] + mx, li[t])
        keep[t], take[t], stab[t] = np.exp(lf[t] + mx - new), np.exp(li[t] - new), new
        mx = new
    return keep, take, stab, li, lf


@pytest.mark.parametrize("cap", [0.0, 4.0])
@pytest.mark.parametrize("portions", [[75], [1] * 75, [31, 1, 33, 2, 8]])
def test_exponential_gates_and_their_stabiliser(cap, portions):
    import lit_llama._native as N

    r = np.random.RandomState(9)
    T, H = 75, 5
    zi, zf = r.randn(T, H) * 3 + np.array([-9, -2, 0, 2, 9.0]), r.randn(T, H) * 3 + 1
    bi, bf = r.randn(H), r.randn(H)
    want = _gates(zi + bi, zf + bf, cap)
    raw = dev(np.concatenate([zi, zf], 1))
    bid, bfd = dev(bi), dev(bf)
    mstate = torch.full((1, H), float("nan"), device="cuda")
    outs, at = [], 0
    for n in portions:
        k, t, s = (torch.empty((n, H), device="cuda") for _ in range(3))
        part, pd = raw[at:at + n].contiguous(), pos(at, at + n)
        N.call("ll_matrix_memory_gates", N.ptr(part), N.ptr_at(part, H), N.LL_F32, 2 * H, N.ptr(bid), N.ptr(bfd), cap, N.ptr(mstate),
               N.ptr(pd), N.ptr(k), N.ptr(t), N.ptr(s), 1, n, H, N.stream())
        outs.append([host(k), host(t), host(s)])
        at += n
    keep, take, stab = (np.concatenate([o[j] for o in outs]) for j in range(3))
    # the stabiliser may be rounded in another order than the token-by-token walk (its sums run over up to 32 tokens) ...
    assert np.abs(stab - want[2]).max() < 2e-4 and np.abs(keep - want[0]).max() < 2e-4 and np.abs(take / want[1] - 1).max() < 2e-4
    # ... but the gates must be exactly those of the stabiliser that is reported: the memory then does not depend on it
    li, lf = want[3], want[4]
    prev = np.concatenate([np.zeros((1, H)), stab[:-1]])
    assert np.abs(keep - np.exp(lf + prev - stab)).max() < 2e-6 and np.abs(take / np.exp(li - stab) - 1).max() < 1e-5


@pytest.mark.parametrize("n,p", [(1, 1), (7, 5), (16, 64), (48, 65), (130, 3)])
def test_recurrence_with_a_normaliser_column(n, p):
    """The unit column: S's last column sums the scaled keys alone, y's last column is its product with the query."""
    from lit_llama.recurrence import decay_scan

    r = np.random.RandomState(n + p)
    T, H = 41, 3
    q, k, v = r.randn(T, H * n), r.randn(T, H * n), r.randn(T, H * p)
    a, ks = r.uniform(0.5, 1.0, (T, H)), r.uniform(0.1, 2.0, (T, H))
    want = np.zeros((T, H, p + 1))
    for h in range(H):
        S = np.zeros((n, p + 1))
        for t in range(T):
            vv = np.concatenate([v[t, h * p:(h + 1) * p], [1.0]])
            S = a[t, h] * S + ks[t, h] * np.outer(k[t, h * n:(h + 1) * n], vv)
            want[t, h] = 0.5 * S.T @ q[t, h * n:(h + 1) * n]
    state = torch.full((1, H, n, p + 1), float("nan"), device="cuda")
    got = []
    for lo, hi in ((0, 17), (17, 18), (18, 41)):
        got.append(host(decay_scan(dev(q[lo:hi]), 0, dev(k[lo:hi]), 0, dev(v[lo:hi]), 0, dev(a[lo:hi]), False, dev(ks[lo:hi]), None, 0.5,
                                   state, pos(lo, hi), 1, hi - lo, H, H, n, p + 1, unit_col=True)))
    got = np.concatenate(got).reshape(T, H, p + 1)
    assert np.abs(got - want).max() < 2e-5 * np.abs(want).max()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_read_out_norm_with_normaliser_and_sigmoid_gate(dtype):
    from lit_llama.recurrence import gated_group_norm

    r = np.random.RandomState(11)
    M, H, p, eps = 13, 3, 10, 1e-3
    y = r.randn(M, H, p + 1)
    y[:, 0, p] = 1e-4                                           # a tiny normaliser: the stabiliser's exp(-mx) takes over
    stab = r.randn(M, H) * 3
    gate, w = bf16(r.randn(M, H * p + 5)), 1 + 0.2 * r.randn(H * p)
    den = np.maximum(np.abs(y[:, :, p]), np.exp(-stab)) + 1e-6
    want = (O.unit_rms(y[:, :, :p] / den[:, :, None], eps).reshape(M, H * p) * w) * O.sigmoid(gate[:, 3:3 + H * p])
    got = gated_group_norm(dev(y.reshape(M, -1)), dev(gate, dtype), 3, dev(w), False, eps, H, False, dtype, sigmoid=True, part=p, stab=dev(stab))
    assert np.abs(host(got) - want).max() < (1e-5 if dtype == torch.float32 else 2e-2) * np.abs(want).max()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("portions", [[60], [1] * 60, [2, 29, 1, 28]])
def test_matrix_memory_mixer(dtype, portions):
    """The whole mixer against the oracle; input gates far above and far below the forget path, so that the stabiliser moves
    and both branches of the read-out's maximum are taken."""
    from lit_llama.recurrence import MatrixMemoryMixer, MatrixMemorySpec

    r = np.random.RandomState(12)
    T, E, H, d, e = 60, 24, 3, 6, 10
    m = {"heads": H, "dim": d, "vdim": e, "gate_cap": 12.0}
    W = {n: bf16(r.randn(o, E) / math.sqrt(E)) for n, o in (("q", H * d), ("k", H * d), ("v", H * e), ("g", H * e), ("o", 0))}
    W["o"] = bf16(r.randn(E, H * e) / math.sqrt(H * e))
    W["i"], W["f"] = bf16(r.randn(H, E)), bf16(r.randn(H, E))
    W["i.b"], W["f.b"], W["norm"] = bf16([-8.0, 0.0, 8.0]), bf16([3.0, 0.0, -3.0]), bf16(1 + 0.1 * r.randn(H * e))
    h = bf16(r.randn(T, E))
    want = O.mlstm(h, W, "", m, 1e-5)
    mix = MatrixMemoryMixer(MatrixMemorySpec(E, H, d, e, 12.0, 1e-5), dtype, "cuda")
    mix.load(lambda s: torch.tensor(W[s]))
    states = [torch.full(s, float("nan"), device="cuda") for s in mix.state_shapes(1)]
    got, at = [], 0
    for n in portions:
        got.append(host(mix(dev(h[at:at + n], dtype), 1, n, pos(at, at + n), states)))
        at += n
    err = np.abs(np.concatenate(got) - want).max() / np.abs(want).max()
    # bf16: the gates' pre-activations (up to 8 in size here) are GEMM outputs rounded to 8 bits before they are exponentiated
    assert err < (2e-4 if dtype == torch.float32 else 1e-1), err


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gelu_both_forms(dtype):
    from lit_llama.feed_forward import DenseFF

    z = bf16(np.linspace(-6, 6, 301))
    want = {"gelu": O.gelu_erf(z), "gelu_tanh": 0.5 * z * (1 + np.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3)))}
    for act, w in want.items():
        ff = DenseFF(301, 301, act, dtype, "cuda")
        ff.load(lambda s: torch.eye(301))
        got = host(ff(dev(z[None], dtype)))[0]
        assert np.abs(got - w).max() < (1e-6 if dtype == torch.float32 else 3e-2)
    assert np.abs(want["gelu"] - want["gelu_tanh"]).max() > 1e-4          # the two forms are told apart
