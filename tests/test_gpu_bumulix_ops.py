"""The mechanisms Bumulix brought, each alone against its float64 statement (oracle/bumulix.py): the stream kept as copies,
softmax attention with two score maps per head in both forms (keys at a window's edge, rings that wrap, split key ranges),
latent attention with latent queries, the rotate-half pairing, YaRN frequencies and an element-wise gate (a far key found
only through the right angle), and the small kernels between them."""
import math

import numpy as np
import pytest
import torch

from oracle import bumulix as O
from tests.util_bumulix import bf16

pytestmark = pytest.mark.gpu


def dev(a, dtype=torch.float32):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float64)).to(dtype).cuda()


def close(got, want, dtype):
    tol = 3e-5 if dtype == torch.float32 else 1.5e-2
    err = float(np.abs(got - want).max() / max(np.abs(want).max(), 1e-30))
    assert err < tol, err


# ------------------------------------------------------------------------------------------------ copies of the stream
class Coeff:
    def __init__(self, mix, w_out):
        self.mix, self.w_out = mix, w_out


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("S,dim", [(1, 7), (2, 40), (3, 33), (4, 600), (5, 16), (8, 130)])
def test_stream_copies_write_then_read(S, dim, dtype):
    from lit_llama.stepping import hyper_mix_norm

    r = np.random.RandomState(S * 100 + dim)
    M, eps, mult = 5, 1e-4, 0.7
    x0 = r.randn(M, dim)
    w_in, w_out, mix = r.randn(S), r.randn(S), np.eye(S) + 0.4 * r.randn(S, S)
    ls, w = r.uniform(0.5, 1.5, dim), 1 + 0.2 * r.randn(dim)
    y = bf16(r.randn(M, dim)) if dtype == torch.bfloat16 else r.randn(M, dim)
    X = torch.full((M, S, dim), float("nan"), device="cuda")
    h = torch.empty((M, dim), dtype=dtype, device="cuda")
    # every copy starts as the embedding output; the first read
    hyper_mix_norm(dev(x0), X, None, mult, dev(w_in), dev(w), eps, h, None, dtype)
    Xo = np.stack([x0] * S)
    close(X.double().cpu().numpy(), Xo.transpose(1, 0, 2), torch.float32)
    close(h.double().cpu().numpy(), O.unit_rms(O.hyper_read(Xo, w_in), eps) * w, dtype)
    # a sublayer's result goes into all copies at once from the old ones, then the next read
    w_in2 = r.randn(S)
    total = torch.empty((M, dim), device="cuda")
    hyper_mix_norm(X, X, (dev(y, dtype), dev(ls), Coeff(dev(mix), dev(w_out))), mult, dev(w_in2), dev(w), eps, h, total, dtype)
    Xo = O.hyper_write(Xo, y * ls, mix, w_out, mult)
    close(X.double().cpu().numpy(), Xo.transpose(1, 0, 2), torch.float32)
    close(total.double().cpu().numpy(), Xo.sum(0), torch.float32)
    close(h.double().cpu().numpy(), O.unit_rms(O.hyper_read(Xo, w_in2), eps) * w, dtype)
    # no mix matrix, no scale: every copy keeps itself; the read is the plain sum
    hyper_mix_norm(X, X, (dev(y, dtype), None, Coeff(None, dev(w_out))), mult, None, dev(w), eps, h, None, dtype)
    Xo = O.hyper_write(Xo, y, np.eye(S), w_out, mult)
    close(X.double().cpu().numpy(), Xo.transpose(1, 0, 2), torch.float32)
    close(h.double().cpu().numpy(), O.unit_rms(Xo.sum(0), eps) * w, dtype)


# ------------------------------------------------------------------------------------------------ two score maps per head
def two_map_module(H, G, d, dv, window, diff, lam_vecs, scale, eps, dtype):
    from lit_llama.rotary import RotarySpec
    from lit_llama.softmax_attention import SoftmaxAttention, SoftmaxAttentionSpec

    spec = SoftmaxAttentionSpec(width=8, heads=H, kv_heads=G, dim=d, vdim=dv, scale=scale, eps=eps, rotary=RotarySpec(0), window=window,
                                maps=2, diff=diff, gate=False)
    mod = SoftmaxAttention(spec, dtype, "cuda")
    mod.diff_lambda = math.exp(float(lam_vecs[0] @ lam_vecs[1])) - math.exp(float(lam_vecs[2] @ lam_vecs[3])) + diff
    return mod


def oracle_two_maps(q, k, v, H, G, d, dv, window, diff, lam_vecs, scale, eps):
    """The oracle's mixer on projections that are given: the input is [q | k | v] and the weights select its parts."""
    h = np.concatenate([q, k, v], axis=1)
    n, I = h.shape[1], np.eye(h.shape[1])
    W = {"q": I[: q.shape[1]], "k": I[q.shape[1]: q.shape[1] + k.shape[1]], "v": I[n - v.shape[1]:], "o": np.eye(H * dv),
         "lq1": lam_vecs[0], "lk1": lam_vecs[1], "lq2": lam_vecs[2], "lk2": lam_vecs[3]}
    m = {"heads": H, "kv_heads": G, "dim": d, "vdim": dv, "diff": diff, "scale": scale}
    if window is not None:
        m["mask"] = {"size": window}
    return O.differential_attention(h, W, m, eps)


def attend(mod, q, k, v, portions, ring, dtype, splits=1, form=0, expect_tensor_form=None):
    from lit_llama import _native as N

    proj = dev(np.concatenate([q, k, v], axis=1), dtype)
    kc = torch.full((1, ring, k.shape[1]), float("nan"), dtype=dtype, device="cuda")
    vc = torch.full((1, ring, v.shape[1]), float("nan"), dtype=dtype, device="cuda")
    out, at = [], 0
    for n in portions:
        pos = torch.arange(at, at + n, dtype=torch.int32, device="cuda")
        part = proj[at:at + n].contiguous()
        if expect_tensor_form is not None and n >= 16:
            s = mod.spec
            assert N.call_ret("ll_softmax_attn_tensor_form", N.dtype_code(dtype), n, s.dim, s.vdim, part.stride(0), 0, splits) == \
                (1 if expect_tensor_form else 0)
        out.append(mod.attend(part, 1, n, pos, (kc, vc), None, splits, form))
        at += n
    return torch.cat(out).double().cpu().numpy()


SHAPES = [(1, 1, 1, 1), (3, 3, 6, 5), (6, 2, 8, 12), (4, 2, 32, 16), (2, 1, 72, 88), (2, 2, 128, 128), (1, 1, 200, 130)]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window", [None, 1, 5, 70])
@pytest.mark.parametrize("shape", SHAPES)
def test_two_maps_against_the_oracle(shape, window, dtype):
    H, G, d, dv = shape
    r = np.random.RandomState(hash((shape, window)) % 1000)
    T, eps, diff, scale = 150, 1e-5, 0.35, 1.3 * d ** -0.5
    q, k, v = bf16(r.randn(T, H * 2 * d)), bf16(r.randn(T, G * 2 * d)), bf16(r.randn(T, G * dv))
    lam = [0.4 * r.randn(d) / math.sqrt(d) for _ in range(4)]
    want = oracle_two_maps(q, k, v, H, G, d, dv, window, diff, lam, scale, eps)
    mod = two_map_module(H, G, d, dv, window, diff, lam, scale, eps, dtype)
    reach = window if window is not None else T
    # whole prompt (bf16 heads in multiples of 8: the tensor-core form), portions, single tokens with split key ranges,
    # and the shortest ring the look-back allows, which wraps many times
    close(attend(mod, q, k, v, [T], T, dtype), want, dtype)
    close(attend(mod, q, k, v, [T], T, dtype, form=1), want, dtype)
    close(attend(mod, q, k, v, [70, 17, 2, 61], T, dtype), want, dtype)
    close(attend(mod, q, k, v, [100] + [1] * 50, T, dtype, splits=3), want, dtype)
    if window is not None:
        close(attend(mod, q, k, v, [24] * 6 + [6], reach - 1 + 24, dtype), want, dtype)
        close(attend(mod, q, k, v, [1] * T, reach, dtype), want, dtype)


@pytest.mark.parametrize("dtype,form", [(torch.float32, 0), (torch.bfloat16, 0), (torch.bfloat16, 1)])
@pytest.mark.parametrize("inside", [True, False])
@pytest.mark.parametrize("window", [2, 33, 64, 65])
def test_a_key_at_the_windows_edge(window, inside, dtype, form):
    """ONE key takes nearly all the weight of the first map of a query exactly ``window - 1`` positions later (seen) or
    ``window`` positions later (not seen); its value row is unlike the others, so a window that is one position off moves
    the result by much more than the tolerance.  Queries in a prompt, at the start of a portion, and decoded alone."""
    H, G, d, dv = 2, 1, 16, 8
    r = np.random.RandomState(window)
    T, eps, diff, scale = 140, 1e-5, 0.4, 0.5
    q, k, v = 0.3 * r.randn(T, H * 2 * d), 0.3 * r.randn(T, G * 2 * d), r.randn(T, G * dv)
    lam = [0.4 * r.randn(d) / math.sqrt(d) for _ in range(4)]
    for i in (70, 100, 120, 139):
        j = i - window + 1 if inside else i - window
        k[j, :d] = 6.0 * q[i, :d] / np.linalg.norm(q[i, :d])           # map 0 of the one key head, seen by head 0
        q[i, :d] *= 6.0 / np.linalg.norm(q[i, :d])
        v[j] = 10.0 * np.sign(r.randn(G * dv))
    q, k, v = bf16(q), bf16(k), bf16(v)
    want = oracle_two_maps(q, k, v, H, G, d, dv, window, diff, lam, scale, eps)
    other = oracle_two_maps(q, k, v, H, G, d, dv, window + (-1 if inside else 1), diff, lam, scale, eps)
    assert np.abs(want - other)[[70, 100, 120, 139]].max() > 0.3          # the test's inputs do show the edge
    mod = two_map_module(H, G, d, dv, window, diff, lam, scale, eps, dtype)
    ring = window - 1 + 40
    close(attend(mod, q, k, v, [T], T, dtype, form=form), want, dtype)
    close(attend(mod, q, k, v, [40, 30, 30, 20, 19, 1], ring, dtype, form=form), want, dtype)       # 70, 100, 120 open a portion
    close(attend(mod, q, k, v, [40, 20] + [1] * 80, ring, dtype, form=form), want, dtype)   # a pass appends at most ring - (window - 1)
    close(attend(mod, q, k, v, [60] + [1] * 80, T, dtype, splits=3, form=form), want, dtype)


def test_the_tensor_core_form_is_the_one_that_runs():
    """bf16 heads in multiples of 8 with 16 tokens or more go to the tensor-core kernel; anything else to the fp32 form."""
    r = np.random.RandomState(0)
    H, G, d, dv, T = 2, 2, 24, 40, 64
    q, k, v = bf16(r.randn(T, H * 2 * d)), bf16(r.randn(T, G * 2 * d)), bf16(r.randn(T, G * dv))
    lam = [0.1 * r.randn(d) for _ in range(4)]
    mod = two_map_module(H, G, d, dv, 9, 0.3, lam, 0.2, 1e-5, torch.bfloat16)
    want = oracle_two_maps(q, k, v, H, G, d, dv, 9, 0.3, lam, 0.2, 1e-5)
    close(attend(mod, q, k, v, [T], T, torch.bfloat16, expect_tensor_form=True), want, torch.bfloat16)
    mod32 = two_map_module(H, G, d, dv, 9, 0.3, lam, 0.2, 1e-5, torch.float32)
    close(attend(mod32, q, k, v, [T], T, torch.float32, expect_tensor_form=False), want, torch.float32)


# ------------------------------------------------------------------------------------------------ latent attention
def latent_module(m, W, width, eps, dtype):
    from lit_llama.latent_attention import LatentAttention, LatentAttentionSpec
    from lit_llama.rotary import RotarySpec

    rotary = RotarySpec.from_dict(m.get("rot"), m["rot_dim"]) if m.get("rot") else RotarySpec(0)
    spec = LatentAttentionSpec(width=width, heads=m["heads"], nope_dim=m["dim"], rot_dim=m["rot_dim"], v_dim=m["vdim"],
                               kv_rank=m["kv_rank"], window=None, scale=m["scale"], eps=eps, q_rank=m["q_rank"], gate="element",
                               rot_layout="half", rotary=rotary)
    mod = LatentAttention(spec, dtype, "cuda")
    with torch.no_grad():
        mod.load(lambda s: dev(W[s], dtype))
    return mod


def run_latent(mod, h, portions, dtype, splits=1):
    T = h.shape[0]
    x = dev(h, dtype)
    cache = torch.full((1, T, mod.spec.row), float("nan"), dtype=dtype, device="cuda")
    rope = mod.spec.rope_table(T, "cuda")
    out, at = [], 0
    for n in portions:
        pos = torch.arange(at, at + n, dtype=torch.int32, device="cuda")
        out.append(mod(x[at:at + n].contiguous(), 1, n, pos, rope, cache, splits))
        at += n
    return torch.cat(out).double().cpu().numpy()


def latent_weights(r, E, m, gain=1.5):
    H, D, R, V, KR, QR = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["q_rank"]

    def lin(o, i, g=1.0):
        return r.randn(o, i) * g / np.sqrt(i)

    W = {"dq": lin(QR, E), "dq.norm": 1 + 0.2 * r.randn(QR), "uq": lin(H * (D + R), QR, gain), "dkv": lin(KR + R, E, gain),
         "dkv.norm": 1 + 0.2 * r.randn(KR), "uk": lin(H * D, KR, gain), "uv": lin(H * V, KR), "g": lin(H * V, E), "o": lin(E, H * V)}
    return {k: bf16(v) for k, v in W.items()}


LATENTS = [
    dict(heads=1, dim=1, rot_dim=2, vdim=1, kv_rank=1, q_rank=1, scale=0.7, rot={"base": 10.0, "dims": 2}),
    dict(heads=3, dim=6, rot_dim=4, vdim=10, kv_rank=12, q_rank=7, scale=0.4,
         rot={"base": 50.0, "dims": 4, "scaling": {"factor": 4.0, "original": 32, "fast": 8.0, "slow": 1.0}}),
    dict(heads=5, dim=7, rot_dim=6, vdim=5, kv_rank=9, q_rank=11, scale=0.3,
         rot={"base": 33.0, "dims": 6, "scaling": {"factor": 3.0, "original": 16, "fast": 6.0, "slow": 2.0}}),
    dict(heads=4, dim=16, rot_dim=16, vdim=24, kv_rank=32, q_rank=24, scale=0.2,
         rot={"base": 1000.0, "dims": 16, "scaling": {"factor": 8.0, "original": 64, "fast": 16.0, "slow": 1.0}}),
    dict(heads=8, dim=32, rot_dim=8, vdim=16, kv_rank=64, q_rank=40, scale=0.15, rot={"base": 10000.0, "dims": 8}),
]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("m", LATENTS)
def test_latent_attention_against_the_oracle(m, dtype):
    r = np.random.RandomState(m["heads"])
    E, T, eps = 40, 90, 1e-5
    W = latent_weights(r, E, m)
    h = bf16(r.randn(T, E))
    want = O.latent_attention(h, W, m, eps)
    mod = latent_module(m, W, E, eps, dtype)

    def ok(got):
        if dtype == torch.float32:
            close(got, want, dtype)
        else:          # bf16: the latents, the absorbed queries and two more products are rounded on the way
            assert np.abs(got - want).max() / np.abs(want).max() < 0.06

    ok(run_latent(mod, h, [T], dtype))
    ok(run_latent(mod, h, [40, 17, 2, 31], dtype))
    ok(run_latent(mod, h, [50] + [1] * 40, dtype, splits=2))
    ok(run_latent(mod, h, [1] * T, dtype))


def test_a_far_key_found_only_through_the_right_angle():
    """Among 600 keys ONE, near the start, points along the last query's rotated part once both are turned by their own
    positions - with YaRN's blended frequencies and in the rotate-half pairing.  A wrong frequency, pairing or position
    leaves the score among the others and the output elsewhere."""
    m = dict(heads=2, dim=4, rot_dim=16, vdim=6, kv_rank=8, q_rank=16, scale=0.5,
             rot={"base": 100.0, "dims": 16, "scaling": {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}})
    r = np.random.RandomState(5)
    R, T, far, eps = 16, 600, 3, 1e-5
    E = 2 * R + 8
    W = latent_weights(r, E, m, gain=0.3)
    # the rotary key part is columns 0..R-1 of the input, the query latent columns R..2R-1, and every head's rotated query
    # part is the latent itself
    W["dkv"][m["kv_rank"]:] = 0.0
    W["dkv"][m["kv_rank"]:, :R] = np.eye(R)
    W["dq"][:] = 0.0
    W["dq"][:, R:2 * R] = np.eye(R)
    W["dq.norm"][:] = 1.0
    uq = W["uq"].reshape(2, 4 + R, 16)
    uq[:, 4:, :] = 4.0 * np.eye(R)
    h = 0.2 * r.randn(T, E)
    a = r.randn(R)
    a *= 3.0 / np.linalg.norm(a)
    h[far, :R] = a
    rot = m["rot"]
    # the query that, turned by the last position, meets the key turned by its own: q = turn(a, far - last)
    back = O.rotate_half(a[None], rot, [far])
    f, mag = O.yarn_frequencies(rot)
    ang = -(T - 1) * f
    u, v = back[0, : R // 2], back[0, R // 2:]
    h[T - 1, R:2 * R] = np.concatenate([u * np.cos(ang) - v * np.sin(ang), v * np.cos(ang) + u * np.sin(ang)])
    h, W = bf16(h), {k: bf16(x) for k, x in W.items()}
    want = O.latent_attention(h, W, m, eps)
    # the inputs do show it: without that key, or with other frequencies, the last output is somewhere else
    gone = h.copy()
    gone[far, :R] = 0.0
    assert np.abs(want[-1] - O.latent_attention(gone, W, m, eps)[-1]).max() > 0.2 * np.abs(want[-1]).max()
    for other in (dict(rot, base=400.0), {"base": 100.0, "dims": 16}):
        assert np.abs(want[-1] - O.latent_attention(h, W, dict(m, rot=other), eps)[-1]).max() > 0.05 * np.abs(want[-1]).max()
    mod = latent_module(m, W, E, eps, torch.float32)
    close(run_latent(mod, h, [T], torch.float32), want, torch.float32)
    close(run_latent(mod, h, [T - 1, 1], torch.float32, splits=4)[-1:], want[-1:], torch.float32)
    mod16 = latent_module(m, W, E, eps, torch.bfloat16)
    got = run_latent(mod16, h, [T], torch.bfloat16)
    assert np.abs(got[-1] - want[-1]).max() < 0.06 * np.abs(want[-1]).max()


# ------------------------------------------------------------------------------------------------ small kernels
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_row_norm_gate_and_cap(dtype):
    from lit_llama import _native as N

    r = np.random.RandomState(1)
    rows, dim, stride = 7, 37, 50
    x = bf16(r.randn(rows, stride))
    w = 1 + 0.3 * r.randn(dim)
    xd, out = dev(x, dtype), torch.empty((rows, dim), dtype=dtype, device="cuda")
    N.call("ll_row_norm", N.ptr(xd), stride, N.ptr(dev(w)), 1e-3, N.ptr(out), dim, N.dtype_code(dtype), rows, dim, N.stream())
    close(out.double().cpu().numpy(), O.unit_rms(x[:, :dim], 1e-3) * w, dtype)
    a, g = bf16(r.randn(rows, dim)), bf16(3 * r.randn(rows, stride))
    ad, gd = dev(a, dtype), dev(g, dtype)
    N.call("ll_sigmoid_gate_mul", N.ptr(ad), dim, N.ptr_at(gd, 5), stride, N.ptr(ad), dim, N.dtype_code(dtype), rows, dim, N.stream())
    close(ad.double().cpu().numpy(), a * O.sigmoid(g[:, 5:5 + dim]), dtype)
    z = 40 * r.randn(rows, dim)
    zd = dev(z)
    N.call("ll_tanh_cap", N.ptr(zd), 12.5, zd.numel(), N.stream())
    close(zd.double().cpu().numpy(), 12.5 * np.tanh(z / 12.5), torch.float32)
