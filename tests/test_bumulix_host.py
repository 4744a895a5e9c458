"""Host-side logic of the Bumulix family (no GPU): configuration from file and from tensor shapes, the frequency table
against the oracle, the reordering of rotated dimensions, ring arithmetic, oracle identities, the family's kernel list."""
import importlib.util
import math

import numpy as np
import pytest

from oracle import bumulix as O
from tests.conftest import PKG
from tests.util_bumulix import case_mixed, case_ones, case_plain, random_weights

pytest.importorskip("lit_llama._native", reason="the CUDA library is not built")

from lit_llama.bumulix import BumulixConfig            # noqa: E402
from lit_llama.cache import max_portion, ring_length   # noqa: E402
from lit_llama.rotary import RotarySpec                # noqa: E402


def shapes_of(W):
    return {k: tuple(np.shape(v)) for k, v in W.items()}


def test_config_from_file_and_shapes():
    cfg, W = case_mixed()
    c = BumulixConfig.from_dict(cfg, shapes_of(W))
    assert (c.vocab, c.width, c.streams, c.copies, c.logit_softcap, c.residual_mult) == (61, 40, 3, 3, 9.0, 0.7)
    assert [l.kind for l in c.layers] == ["latent_attention", "attention", "attention", "attention", "latent_attention",
                                          "attention", "latent_attention"]
    assert [l.weights_of for l in c.layers] == [None, None, 1, 5, 0, None, None]
    a = c.layers[1].mixer
    assert (a.heads, a.kv_heads, a.dim, a.vdim, a.window, a.maps, a.diff, a.gate, a.reach) == (6, 2, 8, 12, 5, 2, 0.3, False, 5)
    l = c.layers[0].mixer
    assert (l.heads, l.nope_dim, l.rot_dim, l.v_dim, l.kv_rank, l.q_rank, l.gate, l.rot_layout, l.window) == \
        (3, 6, 4, 10, 12, 7, "element", "half", None)
    assert l.rotary.scaling == "yarn" and c.layers[6].mixer.rotary.scaling is None
    assert c.layers[1].ff is None and c.layers[3].ff == 20
    # sizes the file leaves out come from the tensors
    gone = ("heads", "kv_heads", "kv_rank", "q_rank")
    slim = dict(cfg, layers=[dict(x, mixer={k: v for k, v in x["mixer"].items() if k not in gone},
                                  mlp=(None if x["mlp"] is None else {"kind": "dense"})) for x in cfg["layers"]])
    del slim["vocab"], slim["width"]
    assert BumulixConfig.from_dict(slim, shapes_of(W)) == c


def test_config_branches_and_refusals():
    cfg, W = case_plain()
    c = BumulixConfig.from_dict(cfg, shapes_of(W))
    assert c.streams is None and c.copies == 1 and c.logit_softcap == 0.0
    assert not c.layers[0].layer_scale and c.layers[0].mixer.window is None and c.layers[0].mixer.reach is None
    assert c.layers[1].mixer.rotary.scaling is None and c.layers[1].mixer.rotary.magnitude == 1.0
    cfg1, W1 = case_ones()
    assert BumulixConfig.from_dict(cfg1, shapes_of(W1)).streams == 1
    bad = dict(cfg, layers=cfg["layers"] + [dict(cfg["layers"][0], weights_of=7)])
    with pytest.raises(ValueError):
        BumulixConfig.from_dict(bad)
    chain = dict(cfg, layers=cfg["layers"] + [dict(cfg["layers"][0], weights_of=0), dict(cfg["layers"][0], weights_of=3)])
    with pytest.raises(ValueError):
        BumulixConfig.from_dict(chain)
    unlike = dict(cfg, layers=cfg["layers"] + [dict(cfg["layers"][0], weights_of=1)])
    with pytest.raises(ValueError):
        BumulixConfig.from_dict(unlike)
    with pytest.raises(ValueError):
        BumulixConfig.from_dict(dict(cfg, layers=[dict(cfg["layers"][0], type="conv")]))
    with pytest.raises(ValueError):
        BumulixConfig.from_dict(dict(cfg, streams=9))


@pytest.mark.parametrize("rot", [
    {"base": 20.0, "dims": 8},
    {"base": 50.0, "dims": 4, "scaling": {"factor": 4.0, "original": 32, "fast": 8.0, "slow": 1.0}},
    {"base": 10000.0, "dims": 64, "scaling": {"factor": 16.0, "original": 4096, "fast": 32.0, "slow": 1.0}},
    {"base": 33.0, "dims": 6, "scaling": {"factor": 3.0, "original": 16, "fast": 6.0, "slow": 2.0}},
    {"base": 500.0, "dims": 12, "scaling": {"factor": 2.0, "original": 8, "fast": 1000.0, "slow": 900.0}},     # lo == hi: a step
])
def test_yarn_frequencies_and_table(rot):
    spec = RotarySpec.from_dict(rot)
    f, mag = O.yarn_frequencies(rot)
    assert np.allclose(spec.frequencies().double().numpy(), f, rtol=1e-6)
    assert math.isclose(spec.magnitude, mag)
    if "scaling" in rot:
        plain = np.array([rot["base"] ** (-2.0 * i / rot["dims"]) for i in range(rot["dims"] // 2)])
        assert np.all(f <= plain * (1 + 1e-12)) and np.all(f >= plain / rot["scaling"]["factor"] * (1 - 1e-12))
    tab = spec.table(70).double().numpy()
    x = np.random.RandomState(0).randn(70, rot["dims"])
    want = O.rotate_half(x, rot, np.arange(70))
    half = rot["dims"] // 2
    got = np.concatenate([x[:, :half] * tab[:, :, 0] - x[:, half:] * tab[:, :, 1], x[:, half:] * tab[:, :, 0] + x[:, :half] * tab[:, :, 1]], 1)
    assert np.abs(got - want).max() < 5e-5


def test_reordering_of_the_rotated_dimensions_keeps_the_scores():
    """Pairs (i, i + dims/2) stored side by side and turned as neighbours give the same dot products."""
    from lit_llama.latent_attention import LatentAttentionSpec

    spec = LatentAttentionSpec(width=8, heads=1, nope_dim=2, rot_dim=10, v_dim=2, kv_rank=2, window=None, scale=1.0,
                               rot_layout="half", rotary=RotarySpec(6, base=30.0))
    order = spec.rot_order().numpy()
    assert sorted(order.tolist()) == list(range(10)) and order[:6].tolist() == [0, 3, 1, 4, 2, 5] and order[6:].tolist() == [6, 7, 8, 9]
    rot = {"base": 30.0, "dims": 6}
    r = np.random.RandomState(0)
    q, k = r.randn(5, 10), r.randn(5, 10)
    want = O.rotate_half(q, rot, np.arange(5)) @ O.rotate_half(k, rot, np.arange(5) + 3).T
    tab = spec.rope_table(9, None).double().numpy()

    def turn(x, pos):
        x = x[:, order].copy()
        for n, p in enumerate(pos):
            u, v = x[n, 0:6:2].copy(), x[n, 1:6:2].copy()
            x[n, 0:6:2], x[n, 1:6:2] = u * tab[p, :, 0] - v * tab[p, :, 1], v * tab[p, :, 0] + u * tab[p, :, 1]
        return x

    assert np.abs(turn(q, np.arange(5)) @ turn(k, np.arange(5) + 3).T - want).max() < 1e-5


def test_rings_hold_what_a_step_reads():
    for window in (1, 2, 5, 72):
        for portion in (1, 2, 7, 64):
            ring = ring_length(1000, window, portion)
            piece = max_portion(ring, 1000, window)
            assert piece >= 1 and (window - 1) + piece <= ring          # no pass writes a slot one of its queries reads
    assert ring_length(50, None, 8) == 50 and max_portion(50, 50, None) == 50


def test_oracle_identities():
    cfg, W = case_mixed()
    toks = np.random.RandomState(0).randint(0, cfg["vocab"], size=20).tolist()
    full = O.forward(cfg, W, toks)
    assert np.abs(O.forward(cfg, W, toks[:11]) - full[:11]).max() < 1e-9          # causal
    assert np.abs(full).max() <= cfg["logit_softcap"]
    # one copy with unit coefficients is the plain residual stream
    pcfg, PW = case_plain()
    one = dict(pcfg, streams=1)
    W1 = dict(PW)
    for i, lc in enumerate(pcfg["layers"]):
        for q in ("1", "2"):
            W1[f"l{i}.hc{q}.in"], W1[f"l{i}.hc{q}.out"], W1[f"l{i}.hc{q}.mix"] = np.ones(1), np.ones(1), np.ones((1, 1))
    t2 = toks[:15]
    t2 = [t % pcfg["vocab"] for t in t2]
    assert np.abs(O.forward(one, W1, t2) - O.forward(pcfg, PW, t2)).max() < 1e-9
    # a key outside the window does not matter
    m = {"heads": 1, "kv_heads": 1, "dim": 4, "vdim": 3, "diff": 0.3, "scale": 0.5, "mask": {"size": 3}}
    r = np.random.RandomState(1)
    Wm = {"q": r.randn(8, 6), "k": r.randn(8, 6), "v": r.randn(3, 6), "o": np.eye(3), "lq1": r.randn(4), "lk1": r.randn(4),
          "lq2": r.randn(4), "lk2": r.randn(4)}
    h = r.randn(9, 6)
    h2 = h.copy()
    h2[2] += 5.0
    a, b = O.differential_attention(h, Wm, m, 1e-5), O.differential_attention(h2, Wm, m, 1e-5)
    assert np.abs(a[5:] - b[5:]).max() < 1e-12 and np.abs(a[4] - b[4]).max() > 1e-3


def test_family_kernel_list():
    spec = importlib.util.spec_from_file_location("llb200_build", PKG / "build.py")
    build = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(build)
    assert build.FAMILY_SOURCES["Bumulix"] == ["quant_pack", "residual_ops", "rotary_attn", "latent_attn"]
    for s in build.FAMILY_SOURCES["Bumulix"]:
        assert (build.CSRC / f"{s}.cu").exists()
    from lit_llama.registry import architectures

    assert "Bumulix" in architectures()
