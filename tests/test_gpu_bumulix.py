"""Bumulix on the GPU against the float64 oracle (oracle/bumulix.py): whole prompts and every layer's summed stream,
token-by-token decoding, portions down to two tokens, rings that wrap, memory that another request used before, batch rows
against each alone, sizes that are 1, parts a config may leave out, sizes that are odd, long decoding, greedy generation
through ``generate()`` and the trace session.  Every comparison is against the oracle run on the WHOLE sequence without any
memory."""
import numpy as np
import pytest
import torch

from oracle import bumulix as O
from tests.util_bumulix import (TOL32, agrees, case_mixed, case_odd, case_ones, case_plain, case_wide, load, rel_err, run_schedule,
                                write_model)

pytestmark = pytest.mark.gpu

T_LONG = 45


def fixture_of(case, name, n_tokens, seed):
    @pytest.fixture(scope="module")
    def fx(tmp_path_factory):
        cfg, W = case()
        folder = write_model(tmp_path_factory.mktemp(name), cfg, W)
        toks = np.random.RandomState(seed).randint(0, cfg["vocab"], size=n_tokens).tolist()
        return cfg, W, folder, toks, O.forward(cfg, W, toks)
    return fx


mixed = fixture_of(case_mixed, "mixed", T_LONG, 7)
ones = fixture_of(case_ones, "ones", 23, 8)
plain = fixture_of(case_plain, "plain", 31, 9)
odd = fixture_of(case_odd, "odd", 31, 10)
wide = fixture_of(case_wide, "wide", 150, 11)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_whole_prompt_and_every_layer(mixed, dtype):
    cfg, W, folder, toks, want = mixed
    m = load(folder, dtype)
    streams = []
    m.layer_probe = lambda i, x: streams.append(x.double().cpu().numpy().copy())
    got = run_schedule(m, toks, [len(toks)], 64)[0]
    want_streams = []
    O.forward(cfg, W, toks, want_streams)
    assert len(streams) == len(want_streams) == len(cfg["layers"])
    for i, (g, w) in enumerate(zip(streams, want_streams)):
        assert agrees(g, w, dtype), f"summed stream after layer {i}: {rel_err(g, w)}"
    assert agrees(got, want, dtype), rel_err(got, want)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_token_by_token_equals_prefill(mixed, dtype):
    cfg, W, folder, toks, want = mixed
    m = load(folder, dtype)
    got = run_schedule(m, toks, [1] * len(toks), 64)[0]        # the first tokens of a sequence included
    assert agrees(got, want, dtype), rel_err(got, want)
    got = run_schedule(m, toks, [len(toks) - 20] + [1] * 20, 64)[0]
    assert agrees(got, want, dtype), rel_err(got, want)


@pytest.mark.parametrize("portions", [[2] * 22 + [1], [3, 2, 7, 1, 1, 11, 2, 5, 13], [44, 1], [1, 44], [5, 40], [1, 1, 1, 2, 40]])
def test_portions_of_any_size(mixed, portions):
    cfg, W, folder, toks, want = mixed
    m = load(folder, torch.float32)
    assert rel_err(run_schedule(m, toks, portions, 64)[0], want) < TOL32


@pytest.mark.parametrize("portion", [1, 2, 3, 8])
def test_ring_wraps_and_slots_are_reused(mixed, portion):
    """Key / value rings of (window - 1 + portion) slots: every slot is overwritten several times within one sequence, in
    prompts (cut into passes by the model itself) and in decoding.  Layers that compute with the same tensors keep rings of
    their own; the latent rows keep every position."""
    cfg, W, folder, toks, want = mixed
    m = load(folder, torch.float32, prefill_portion=portion)
    got = run_schedule(m, toks, [30] + [1] * 15, 64)[0]
    assert m._rings == (64, 5 - 1 + portion, 5 - 1 + portion, 9 - 1 + portion, 64, 9 - 1 + portion, 64)
    assert len({t.data_ptr() for t in m.kv_caches}) == 4 * 2 + 3
    assert rel_err(got, want) < TOL32
    got = run_schedule(m, toks, [7, 2, 21, 15], 64)[0]
    assert rel_err(got, want) < TOL32


def test_a_new_request_reuses_the_memory_of_an_ended_one(mixed):
    """Nothing is cleared between requests: the rows of the ended request are still there when the next one starts."""
    cfg, W, folder, toks, want = mixed
    m = load(folder, torch.float32)
    other = np.random.RandomState(9).randint(0, cfg["vocab"], size=40).tolist()
    run_schedule(m, other, [33] + [1] * 7, 64)                       # fills the memory and captures the step graph
    ptr = m.kv_caches[0].data_ptr()
    for portions in ([T_LONG], [1] * T_LONG, [20] + [1] * 25):
        got = run_schedule(m, toks, portions, 64)[0]
        assert m.kv_caches[0].data_ptr() == ptr
        assert rel_err(got, want) < TOL32


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_batch_rows_equal_each_alone(mixed, dtype):
    cfg, W, folder, toks, want = mixed
    m = load(folder, dtype)
    other = np.random.RandomState(10).randint(0, cfg["vocab"], size=T_LONG).tolist()
    want_other = O.forward(cfg, W, other)
    got = run_schedule(m, [toks, other], [17, 2, 1, 1, 24], 64)
    assert agrees(got[0], want, dtype) and agrees(got[1], want_other, dtype), (rel_err(got[0], want), rel_err(got[1], want_other))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_sizes_that_are_one(ones, dtype):
    cfg, W, folder, toks, want = ones
    m = load(folder, dtype)
    for portions in ([len(toks)], [1] * len(toks), [2] * 11 + [1]):
        got = run_schedule(m, toks, portions, 32)[0]
        assert agrees(got, want, dtype), rel_err(got, want)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_parts_a_config_may_leave_out(plain, dtype):
    cfg, W, folder, toks, want = plain
    m = load(folder, dtype)
    assert m.config.streams is None and m.config.logit_softcap == 0.0 and m.blocks[0].ls1 is None
    assert m.config.layers[0].mixer.window is None
    for portions in ([len(toks)], [1] * len(toks), [9, 2, 20]):
        got = run_schedule(m, toks, portions, 32)[0]
        assert agrees(got, want, dtype), rel_err(got, want)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_sizes_that_are_odd(odd, dtype):
    cfg, W, folder, toks, want = odd
    m = load(folder, dtype)
    for portions in ([len(toks)], [9] + [1] * 22, [2, 3, 5, 7, 11, 3]):
        got = run_schedule(m, toks, portions, 32)[0]
        assert agrees(got, want, dtype), rel_err(got, want)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_wide_heads_and_prompts_longer_than_a_query_tile(wide, dtype):
    """bf16 prompts of 16 tokens or more take the tensor-core attention kernels; shorter portions and single tokens the
    fp32 forms."""
    cfg, W, folder, toks, want = wide
    m = load(folder, dtype)
    for portions in ([150], [70, 17, 63], [100] + [1] * 50, [16, 3, 64, 65, 2]):
        got = run_schedule(m, toks, portions, 160)[0]
        assert agrees(got, want, dtype), rel_err(got, want)
    m = load(folder, dtype, prefill_portion=24)               # rings of 39 + 24 and 69 + 24 slots wrap inside the prompt
    got = run_schedule(m, toks, [150], 160)[0]
    assert m._rings[0] == 40 - 1 + 24 and m._rings[2] == 70 - 1 + 24
    assert agrees(got, want, dtype), rel_err(got, want)


def test_long_decoding_through_small_rings(mixed):
    cfg, W, folder, _, _ = mixed
    toks = np.random.RandomState(11).randint(0, cfg["vocab"], size=130).tolist()
    want = O.forward(cfg, W, toks)
    m = load(folder, torch.float32, prefill_portion=2)
    got = run_schedule(m, toks, [20] + [1] * 110, 256)[0]
    assert rel_err(got, want) < TOL32


def test_forward_without_kept_memory_leaves_the_memory_alone(mixed):
    cfg, W, folder, toks, want = mixed
    m = load(folder, torch.float32)
    idx = torch.tensor([toks], device="cuda")
    m.reset_cache()
    a = m(idx[:, :30], 64, torch.arange(30))
    probe = m(idx[:, :12]).double().cpu().numpy()[0]             # no positions: scratch memory
    b = m(idx[:, 30:], 64, torch.arange(30, T_LONG))
    assert rel_err(probe, want[:12]) < TOL32
    assert rel_err(torch.cat([a, b], 1).double().cpu().numpy()[0], want) < TOL32


def test_greedy_generation_through_generate(mixed):
    import generate as G

    cfg, W, folder, toks, _ = mixed
    m = G.load_model(folder, None, torch.device("cuda"), torch.float32)
    prompt = torch.tensor(toks[:9], device="cuda")
    out = G.generate(m, prompt, 12, temperature=1.0, top_k=1).tolist()
    m.reset_cache()
    seq = list(toks[:9])
    for _ in range(12):
        seq.append(int(np.argmax(O.forward(cfg, W, seq)[-1])))
    assert out == seq


def test_trace_session_frees_and_reuses(mixed):
    from lit_llama.trace import TraceSession

    cfg, W, folder, toks, want = mixed
    m = load(folder, torch.float32)
    s = TraceSession(m, 64)
    other = np.random.RandomState(12).randint(0, cfg["vocab"], size=21).tolist()
    assert s.step([{"id": "a", "tokens": other[:20], "want": []}]) is None
    s.step([{"id": "a", "tokens": other[20:], "want": [0]}], end=["a"])
    rows = [s.step([{"id": "b", "tokens": toks[:10], "want": [0, 9]}]),
            s.step([{"id": "b", "tokens": toks[10:12], "want": [1]}]),
            s.step([{"id": "b", "tokens": toks[12:13], "want": [0]}]),
            s.step([{"id": "b", "tokens": toks[13:], "want": [T_LONG - 14]}], end=["b"])]
    got = torch.cat(rows).double().cpu().numpy()
    assert rel_err(got, want[[0, 9, 11, 12, T_LONG - 1]]) < TOL32
