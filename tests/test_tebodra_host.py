"""Host-side parts of the Tebodra family (no GPU): configuration from a file's dictionary and from tensor shapes, rotary
frequency tables against the oracle, which ring a layer reads and how long it is, oracle identities, kernel lists."""
import importlib.util
import math

import numpy as np
import pytest

from oracle import tebodra as O
from tests.util_tebodra import case_mixed


def need_package():
    """The package's modules load the kernels' library when imported; where it is not built these tests are skipped."""
    pytest.importorskip("torch")
    try:
        import lit_llama._native  # noqa: F401
    except ImportError as e:
        pytest.skip(str(e))


def test_configuration_from_file_and_from_shapes():
    need_package()
    from lit_llama.tebodra import TebodraConfig

    cfg, W = case_mixed()
    c = TebodraConfig.from_dict(cfg)
    assert [l.kind for l in c.layers] == ["mlstm", "attention_2", "attention", "attention_2", "attention_2", "mlstm"]
    a2, a1, b = c.layers[1].mixer, c.layers[2].mixer, c.layers[3].mixer
    assert (a2.chunk, a2.sink, a2.qk_norm, a2.own_values, a2.conv_taps, a2.softcap) == (7, True, True, True, 0, 0.0)
    assert (a1.chunk, a1.sink, a1.qk_norm, a1.own_values, a1.conv_taps, a1.softcap) == (None, False, False, False, 2, 5.0)
    assert a1.rotary.scaling == "bands" and a2.rotary.scaling == "linear" and a1.rotary.dims == 6
    assert b.kv_from == 1 and b.chunk == 11 and c.layers[5].ff is None and c.layers[0].ff == 24
    assert c.residual_mult == 0.7 and c.eps == 1e-4
    lean = {k: v for k, v in cfg.items() if k not in ("vocab", "width")}          # sizes the file leaves out come from shapes
    lean["layers"] = [dict(l, mlp=(None if l["mlp"] is None else {"kind": "dense"})) for l in cfg["layers"]]
    c2 = TebodraConfig.from_dict(lean, {k: v.shape for k, v in W.items()})
    assert (c2.vocab, c2.width, [l.ff for l in c2.layers]) == (c.vocab, c.width, [l.ff for l in c.layers])
    assert [(l.mixer.sink, l.mixer.qk_norm, l.mixer.own_values) for l in c2.layers if l.kind != "mlstm"] == \
        [(l.mixer.sink, l.mixer.qk_norm, l.mixer.own_values) for l in c.layers if l.kind != "mlstm"]
    bad = dict(cfg, layers=[dict(cfg["layers"][3])] + cfg["layers"][1:])
    with pytest.raises(ValueError):
        TebodraConfig.from_dict(bad)                                             # kv_from must name an earlier owner
    with pytest.raises(ValueError):
        TebodraConfig.from_dict(dict(cfg, layers=[dict(cfg["layers"][0], type="other")]))


@pytest.mark.parametrize("rot", [
    {"base": 250.0, "dims": 12},
    {"base": 1e4, "dims": 32, "scaling": {"factor": 3.0}},
    {"base": 5e5, "dims": 48, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 512}},
    {"base": 100.0, "dims": 8, "scaling": {"factor": 2.0, "low": 2.0, "high": 16.0, "original": 64}},
])
def test_rotary_frequency_tables(rot):
    need_package()
    from lit_llama.rotary import RotarySpec

    got = RotarySpec.from_dict(rot).frequencies().double().numpy()
    want = O.rotary_frequencies(rot)
    assert got.shape == want.shape and np.abs(got / want - 1).max() < 1e-7
    if "original" in rot.get("scaling", {}):
        sc = rot["scaling"]
        plain = O.rotary_frequencies({"base": rot["base"], "dims": rot["dims"]})
        wave = 2 * math.pi / plain
        assert np.allclose(want[wave < sc["original"] / sc["high"]], plain[wave < sc["original"] / sc["high"]])
        assert np.allclose(want[wave > sc["original"] / sc["low"]], plain[wave > sc["original"] / sc["low"]] / sc["factor"])
        assert len({tuple(np.round(want / plain, 6))}) == 1 and (want <= plain + 1e-12).all()


def test_rings_and_their_readers():
    """Arithmetic of the model's memory plan, on the spec alone: the look-back of a chunk mask, and a ring sized for the
    furthest-looking reader never has a step overwrite a slot one of its own queries reads."""
    need_package()
    from lit_llama.cache import max_portion, ring_length
    from lit_llama.softmax_attention import SoftmaxAttentionSpec

    s = SoftmaxAttentionSpec(width=8, heads=2, kv_heads=1, dim=4, vdim=4, scale=1.0, eps=1e-5, chunk=11)
    assert s.reach == 11 and SoftmaxAttentionSpec(width=8, heads=2, kv_heads=1, dim=4, vdim=4, scale=1.0, eps=1e-5).reach is None
    for chunk in (1, 5, 11):
        for portion in (1, 2, 8):
            ring = ring_length(1000, chunk, portion)
            assert max_portion(ring, 1000, chunk) == portion
            for first in range(0, 40):                                           # a step of `portion` tokens from `first`
                written = {(first + t) % ring for t in range(portion)}
                for t in range(portion):
                    i = first + t
                    reads = {j % ring for j in range((i // chunk) * chunk, first)}        # keys of earlier steps it sees
                    assert not (reads & written)


def test_oracle_identities():
    """A chunk longer than the sequence is the causal mask; a sink of minus infinity is no sink; the matrix memory's
    output does not depend on where its stabiliser starts, as long as the read-out's floor is not reached."""
    r = np.random.RandomState(0)
    q, k, v = r.randn(12, 4, 6), r.randn(12, 2, 6), r.randn(12, 2, 5)
    a = O.softmax_attention(q, k, v, 0.4)
    assert np.allclose(a, O.softmax_attention(q, k, v, 0.4, chunk=100))
    assert np.allclose(a, O.softmax_attention(q, k, v, 0.4, sink=np.full(4, -1e9)))
    c = O.softmax_attention(q, k, v, 0.4, chunk=5)
    assert np.allclose(c[5:10], O.softmax_attention(q[5:10], k[5:10], v[5:10], 0.4))
    assert np.abs(O.softmax_attention(q, k, v, 0.4, sink=np.full(4, 30.0))).max() < 1e-8
    assert np.allclose(O.gelu_erf(np.array([0.0, 1.0, -1.0])), [0.0, 0.8413447460685429, -0.15865525393145707])


def test_family_kernel_list():
    spec = importlib.util.spec_from_file_location("llb200_build", str(__import__("tests.conftest", fromlist=["PKG"]).PKG / "build.py"))
    build = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(build)
    assert "Tebodra" in build.FAMILY_SOURCES
    for stem in build.FAMILY_SOURCES["Tebodra"]:
        assert (build.CSRC / f"{stem}.cu").exists()
    assert "rotary_attn" in build.FAMILY_SOURCES["Tebodra"] and "window_attn" not in build.FAMILY_SOURCES["Tebodra"]
