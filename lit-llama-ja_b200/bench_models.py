"""Throughput of a model family beside its closest relative at equal size: prefill tokens/s, batch-1 decode tokens/s, and
the hot kernels of each timed alone against the measured roofline.  ``bench.py --family lepalorn``: Lepalorn beside LLaMA;
``bench.py --family bededra``: Bededra beside Lepalorn; ``bench.py --family tebodra``: Tebodra beside Bededra.  Random weights, layer shapes of real
models, a few layers each (every layer costs the same).  Timing: CUDA events, warm-up, an L2 flush (a 256 MB write)
between timed iterations."""
from __future__ import annotations

import json
import math
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent.parent

# width, layers, heads, nope, rot, v, kv_rank, window, experts, top, ff, shared_ff  (top * ff + shared_ff = LLaMA's n_hidden)
SIZES = {
    "w1024": dict(width=1024, layers=4, heads=8, nope=64, rot=32, v=64, kv_rank=256, window=512, experts=16, top=2, ff=768, shared=1280),
    "w2048": dict(width=2048, layers=4, heads=16, nope=128, rot=64, v=128, kv_rank=512, window=1024, experts=32, top=4, ff=1024, shared=1536),
    "w4096": dict(width=4096, layers=2, heads=32, nope=128, rot=64, v=128, kv_rank=512, window=2048, experts=32, top=4, ff=2048, shared=2816),
}
VOCAB = 32000


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return d["hbm_gbs"] * 1e9, d["bf16_tflops"] * 1e12, "measured"
    return 6.65e12, 1.59e15, "fallback"


class Timer:
    def __init__(self, device):
        self.flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)

    def __call__(self, fn, iters=5, warmup=3, graph=False):
        """Median device time of ``fn()`` with a cold L2.  ``graph``: ``fn`` is captured once and the timed region is one
        graph launch, so that a sequence of short kernels is not timed at the pace the host issues it."""
        for _ in range(warmup):
            fn()
        if graph:
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                fn()
            fn = g.replay
            fn()
        ts = []
        for _ in range(iters):
            self.flush.fill_(1)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b) * 1e-3)
        ts.sort()
        return ts[len(ts) // 2]


def lepalorn_model(s, device, dtype=torch.bfloat16):
    from lit_llama.latent_attention import LatentAttentionSpec
    from lit_llama.lepalorn import Lepalorn, LepalornConfig, LepalornLayer
    from lit_llama.moe import MoESpec

    layers = []
    for i in range(s["layers"]):
        mx = LatentAttentionSpec(width=s["width"], heads=s["heads"], nope_dim=s["nope"], rot_dim=s["rot"], v_dim=s["v"],
                                 kv_rank=s["kv_rank"], window=s["window"], scale=(s["nope"] + s["rot"]) ** -0.5,
                                 kv_from=(i - 1) if i % 2 == 1 else None)
        layers.append(LepalornLayer(mx, MoESpec(s["width"], s["experts"], s["top"], s["ff"], 7.0, s["shared"], 7.0)))
    m = Lepalorn(LepalornConfig(VOCAB, s["width"], 1e-5, 1.0, layers), dtype=dtype, device=device)
    g = torch.Generator(device=device).manual_seed(0)
    for n, p in m.named_parameters():
        if p.dim() >= 2:
            p.copy_((torch.randn(p.shape, generator=g, device=device) / math.sqrt(p.shape[-1])).to(p.dtype))
        elif n.endswith("dwa"):
            p.zero_()
            p[-1] = 1.0
    return m.eval()


def llama_model(s, device):
    from lit_llama.model import LLaMA, LLaMAConfig

    cfg = LLaMAConfig(block_size=8192, vocab_size=VOCAB, n_layer=s["layers"], n_head=s["heads"], n_embd=s["width"])
    with torch.device(device):
        m = LLaMA(cfg).to(torch.bfloat16)
    m.apply(m._init_weights)
    m.use_fused_decode = False          # unquantized: the per-module path, single-token steps as one graph replay
    m.graph_every_batch = True
    return m.eval()


def end_to_end(model, timer, prompt_len, device, max_seq):
    idx = torch.randint(0, VOCAB, (1, prompt_len), device=device)
    pos = torch.arange(prompt_len, device=device)

    def prefill():
        model.reset_cache()
        model(idx, max_seq, pos)

    t_prefill = timer(prefill, iters=3, warmup=2)
    one, p1 = idx[:, :1].contiguous(), torch.arange(prompt_len, prompt_len + 1, device=device)
    n = 16

    def decode():
        for _ in range(n):
            model(one, max_seq, p1)

    t_decode = timer(decode, iters=3, warmup=2) / n
    return prompt_len / t_prefill, 1.0 / t_decode


def kernel_table(s, lep, device, timer, prompt_len):
    """The hot kernels of one layer alone.  Roofline time = max(flops / tensor peak, bytes / copy bandwidth)."""
    from torch.nn import functional as F

    from lit_llama import _native as N

    hbm, tflops, which = peaks()
    bf = torch.bfloat16
    E, H, KR, R, W = s["width"], s["heads"], s["kv_rank"], s["rot"], s["window"]
    rows = []

    def add(name, t, flops, nbytes):
        roof = max(flops / tflops, nbytes / hbm)
        rows.append(dict(kernel=name, us=round(t * 1e6, 1), roofline_us=round(roof * 1e6, 2), fraction=round(roof / t, 4)))

    blk = lep.blocks[0]
    for T, tag in ((prompt_len, "prefill"), (1, "decode")):
        x = torch.randn((T, E), device=device, dtype=bf)
        pos0 = 0 if T > 1 else prompt_len
        pos_ids = torch.arange(pos0, pos0 + T, dtype=torch.int32, device=device)
        lep.reset_cache()
        lep._ensure_cache(1, prompt_len + 64)
        lep._ensure_rope(prompt_len + 64)
        cache = lep.kv_caches[0]
        cache.normal_()
        rope = lep._rope[(blk.mix.spec.rot_base, blk.mix.spec.rot_dims)]
        proj = F.linear(x, blk.mix.w_in)
        q_lat = torch.randn((H, T, KR), device=device, dtype=bf)
        o_lat = torch.empty_like(q_lat)
        splits = 1 if T > 1 else max(1, min(16, (W + 63) // 64))
        scratch = torch.empty(max(1, N.call_ret("ll_latent_attn_scratch_bytes", T, H, KR, splits) // 4), device=device)

        def attn():
            N.call("ll_latent_attn", N.ptr(q_lat), T * KR, KR, N.ptr(proj), proj.shape[1], s["nope"], s["nope"] + R, blk.mix.gate_col0,
                   N.ptr(rope), N.ptr(pos_ids), N.ptr(cache), N.ptr(o_lat), T * KR, KR, N.LL_BF16, 1, T, H, KR, R, R, cache.shape[1], W,
                   0.1, splits, N.ptr(scratch), N.stream())

        keys = sum(min(W, p + 1) for p in range(pos0, pos0 + T))
        add(f"latent_attn {tag}", timer(attn, graph=True), 2.0 * keys * H * (2 * KR + R), 2.0 * (min(W + T, pos0 + T) * (KR + R) + 2 * H * T * KR))
        # LLaMA's attention at equal heads and head size = nope + rot
        hs = s["width"] // H
        q = torch.randn((1, H, T, hs), device=device, dtype=bf)
        if T > 1:
            k, v = torch.randn_like(q), torch.randn_like(q)
            add("llama sdpa prefill (library, full causal)", timer(lambda: F.scaled_dot_product_attention(q, k, v, is_causal=True), graph=True),
                2.0 * (T * (T + 1) / 2) * H * 2 * hs, 2.0 * 4 * T * H * hs)
        elif hs in (32, 64, 128):
            S = prompt_len + 64
            kc, vc = torch.randn((1, H, S, hs), device=device, dtype=bf), torch.randn((1, H, S, hs), device=device, dtype=bf)
            y = torch.empty((1, 1, H * hs), device=device, dtype=bf)
            p3 = torch.tensor([prompt_len, prompt_len, prompt_len + 1], dtype=torch.int32, device=device)
            sp = max(1, min(8, (2 * N._fn["ll_sm_count"]()) // H, (S + 63) // 64))
            ws = N.Workspace.get(device).ensure(attn_bytes=N.attn_scratch_bytes(1, H, hs, sp), attn_counters=H)
            add("llama decode_attn", timer(lambda: N.call("ll_decode_attn", N.ptr(q), N.ptr(kc), N.ptr(vc), N.ptr(p3), N.ptr(y), N.LL_BF16, 1,
                                                          H, hs, S, sp, N.ptr(ws.attn_scratch), N.ptr(ws.attn_counters), 0, N.stream()), graph=True),
                4.0 * (prompt_len + 1) * H * hs, 2.0 * 2 * (prompt_len + 1) * H * hs)
        # experts: both grouped GEMMs of the layer / LLaMA's three MLP GEMMs
        moe = blk.mlp
        _, w, offsets, perm = moe.route(x)
        n = T * s["top"]
        h = torch.empty((n, s["ff"]), dtype=bf, device=device)
        yy = torch.empty((n, E), dtype=bf, device=device)

        tc = moe.takes_tensor_cores(n, x)         # the path the module takes for a step of this size
        xs = torch.empty((n, E), dtype=bf, device=device) if tc else None

        def experts():
            if tc:
                N.call("ll_moe_gather_rows", N.ptr(x), E, N.ptr(perm), s["top"], n, E, N.ptr(xs), N.stream())
                N.call("ll_moe_grouped_gemm_tc", N.ptr(xs), N.ptr(moe.w_gu), N.ptr(offsets), N.ptr(perm), 1, n, s["experts"], s["ff"], E,
                       7.0, 1.702, N.ptr(h), s["ff"], N.stream())
                N.call("ll_moe_grouped_gemm_tc", N.ptr(h), N.ptr(moe.w_down), N.ptr(offsets), N.ptr(perm), 0, n, s["experts"], E, s["ff"],
                       0.0, 0.0, N.ptr(yy), E, N.stream())
                return
            N.call("ll_moe_grouped_gemm", N.ptr(x), E, N.ptr(moe.w_gu), N.ptr(offsets), N.ptr(perm), 1, N.LL_BF16, n, s["top"], s["experts"],
                   s["ff"], E, 7.0, 1.702, N.ptr(h), s["ff"], N.stream())
            N.call("ll_moe_grouped_gemm", N.ptr(h), s["ff"], N.ptr(moe.w_down), N.ptr(offsets), N.ptr(perm), 0, N.LL_BF16, n, s["top"],
                   s["experts"], E, s["ff"], 0.0, 0.0, N.ptr(yy), E, N.stream())

        used = min(s["experts"], n)
        add(f"moe grouped GEMMs {tag}" + (" (tcgen05, with the row gather)" if tc else ""), timer(experts, graph=True), 2.0 * n * 3 * s["ff"] * E, 2.0 * used * 3 * s["ff"] * E)
        nh = s["top"] * s["ff"] + s["shared"]
        w1, w2 = torch.randn((2 * nh, E), device=device, dtype=bf), torch.randn((E, nh), device=device, dtype=bf)
        hh = torch.empty((T, nh), device=device, dtype=bf)

        def mlp():
            F.linear(x, w1)
            F.linear(hh, w2)

        add(f"llama MLP GEMMs {tag} (library)", timer(mlp, graph=True), 2.0 * T * 3 * nh * E, 2.0 * 3 * nh * E)
    return rows, which


# Bededra at the widths of SIZES: layers alternate parallel / mamba2; left = window attention (kv heads = heads / 4), right =
# gated linear attention, state space with inner size 2 * width; experts as Lepalorn's at that width (no shared expert)
BEDEDRA_SIZES = {
    "w1024": dict(width=1024, layers=4, heads=8, kv=2, dim=64, window=512, keep=16, r_heads=4, r_dim=64, r_vdim=128, rank=16,
                  m_heads=32, m_vdim=64, state=128, experts=16, top=2, ff=768, groups=4, keep_groups=2),
    "w2048": dict(width=2048, layers=4, heads=16, kv=4, dim=128, window=1024, keep=16, r_heads=8, r_dim=64, r_vdim=128, rank=16,
                  m_heads=64, m_vdim=64, state=128, experts=32, top=4, ff=1024, groups=8, keep_groups=4),
    "w4096": dict(width=4096, layers=2, heads=32, kv=8, dim=128, window=2048, keep=16, r_heads=16, r_dim=64, r_vdim=128, rank=16,
                  m_heads=128, m_vdim=64, state=128, experts=32, top=4, ff=2048, groups=8, keep_groups=4),
}


def bededra_model(s, device, dtype=torch.bfloat16):
    from lit_llama.bededra import Bededra, BededraConfig

    ff = {"kind": "moe", "expert": {"ff": s["ff"]},
          "router": {"experts": s["experts"], "top": s["top"], "groups": {"count": s["groups"], "keep": s["keep_groups"]}}}
    par = {"type": "parallel", "mlp": ff, "mixer": {
        "left": {"heads": s["heads"], "kv_heads": s["kv"], "dim": s["dim"], "vdim": s["dim"], "scale": s["dim"] ** -0.5, "softcap": 30.0,
                 "mask": {"size": s["window"], "keep_first": s["keep"]}},
        "right": {"heads": s["r_heads"], "dim": s["r_dim"], "vdim": s["r_vdim"], "tau": 8.0, "decay_rank": s["rank"]},
        "left_scale": 0.7, "right_scale": 1.2}}
    mam = {"type": "mamba2", "mlp": ff, "mixer": {"heads": s["m_heads"], "vdim": s["m_vdim"], "state": s["state"], "groups": 1,
                                                  "norm_groups": 1, "conv": 4}}
    cfg = {"vocab": VOCAB, "width": s["width"], "norm": {"eps": 1e-5}, "canon": {"taps": 4},
           "layers": [par if i % 2 == 0 else mam for i in range(s["layers"])]}
    m = Bededra(BededraConfig.from_dict(cfg), dtype=dtype, device=device)
    g = torch.Generator(device=device).manual_seed(0)
    fixed = {"r1": 0.1, "r2": 1.0, "dt_bias": -1.0, "a_log": 0.0, "skip": 1.0, "b_a2": 2.0}
    for n, p in m.named_parameters():
        leaf = n.rsplit(".", 1)[-1]
        if leaf == "talk":
            p.copy_(torch.eye(p.shape[0], device=device) + 0.05 * torch.randn(p.shape, generator=g, device=device))
        elif p.dim() >= 2 and "conv" not in n and "canon" not in n:
            p.copy_((torch.randn(p.shape, generator=g, device=device) / math.sqrt(p.shape[-1])).to(p.dtype))
        elif p.dim() >= 2:
            p.copy_(0.3 * torch.randn(p.shape, generator=g, device=device))
        elif leaf in fixed:
            p.fill_(fixed[leaf])
    return m.eval()


def bededra_kernel_table(s, model, device, timer, prompt_len):
    """The mixers' kernels of one parallel and one mamba2 layer alone.  Roofline time = max(flops / tensor peak, bytes /
    copy bandwidth), flops and bytes counted for the mechanism (one sweep over the visible keys; one update and one
    read-out of the state per token), not for what the kernel happens to do."""
    from torch.nn import functional as F

    from lit_llama import _native as N
    from lit_llama.recurrence import decay_scan

    hbm, tflops, which = peaks()
    bf = torch.bfloat16
    rows = []

    def add(name, t, flops, nbytes):
        roof = max(flops / tflops, nbytes / hbm)
        rows.append(dict(kernel=name, us=round(t * 1e6, 1), roofline_us=round(roof * 1e6, 2), fraction=round(roof / t, 4)))

    par = next(b for b in model.blocks if b.kind == "parallel")
    mam = next(b for b in model.blocks if b.kind == "mamba2")
    E, H, G, D, W, K = s["width"], s["heads"], s["kv"], s["dim"], s["window"], s["keep"]
    for T, tag in ((prompt_len, "prefill"), (1, "decode")):
        pos0 = 0 if T > 1 else prompt_len
        pos_ids = torch.arange(pos0, pos0 + T, dtype=torch.int32, device=device)
        model.reset_cache()
        model._begin(1, prompt_len + 64, True)
        for t in model.kv_caches:
            t.normal_()
        for t in model.states:
            t.zero_()
        x = torch.randn((T, E), device=device, dtype=bf)
        proj = F.linear(x, par.mix.w_in)
        att = par.mix.left
        caches = model.kv_caches[:2]
        span = min(W, caches[0].shape[1] - K) + K
        splits = 1 if T > 1 else max(1, min(64, (span + 63) // 64))
        keys = sum(min(W, p + 1) + max(0, min(K, p + 1 - W)) for p in range(pos0, pos0 + T))

        def attn():
            att.attend(proj, 0, 1, T, pos_ids, caches, splits)

        add(f"window_attn {tag} (append + two sweeps + gate)", timer(attn, graph=True), 2.0 * keys * H * 2 * D,
            2.0 * (min(W + K + T, pos0 + T) * G * 2 * D + 2 * T * H * D))
        # gated linear attention: the recurrence alone
        r = par.mix.right
        rs = r.spec
        alpha = torch.rand((T, rs.heads * rs.dim), device=device) * 0.1 + 0.9
        st_r = model.states[1:2]
        c0 = par.mix.right_col0

        def gla():
            decay_scan(proj, c0 + r.cols["q"], proj, c0 + r.cols["k"], proj, c0 + r.cols["v"], alpha, True, None, None, 0.125, st_r[0],
                       pos_ids, 1, T, rs.heads, rs.heads, rs.dim, rs.vdim)

        nst = rs.heads * rs.dim * rs.vdim
        add(f"decay_scan {tag} (gated linear attention)", timer(gla, graph=True), 4.0 * T * nst,
            2.0 * T * rs.heads * (2 * rs.dim + rs.vdim) + 4.0 * T * rs.heads * (rs.dim + rs.vdim) + 8.0 * nst)
        # state space: the recurrence alone
        ms = mam.mix.spec
        xbc = torch.randn((T, ms.conv_channels), device=device, dtype=bf)
        dtv = torch.rand((T, ms.heads), device=device) * 0.5
        dec = torch.rand((T, ms.heads), device=device) * 0.1 + 0.9
        st_m = torch.zeros((1, ms.heads, ms.state, ms.vdim), device=device)
        gn = ms.groups * ms.state

        def ssm():
            decay_scan(xbc, ms.inner + gn, xbc, ms.inner, xbc, 0, dec, False, dtv, mam.mix.skip, 1.0, st_m, pos_ids, 1, T, ms.heads,
                       ms.groups, ms.state, ms.vdim)

        nst = ms.heads * ms.state * ms.vdim
        add(f"decay_scan {tag} (state space)", timer(ssm, graph=True), 4.0 * T * nst,
            2.0 * T * ms.conv_channels + 4.0 * T * (2 * ms.heads + ms.inner) + 8.0 * nst)
        # the layer's short convolution and its two norms (bandwidth)
        xs = torch.randn((T, E), device=device)
        h1, h2 = torch.empty((T, E), device=device), torch.empty((T, E), device=device, dtype=bf)
        from lit_llama.stepping import add_norm_pair

        a0 = torch.randn((T, E), device=device, dtype=bf)
        add(f"add + two norms {tag}", timer(lambda: add_norm_pair(xs, [(a0, 1.0), (a0, 0.5)], par.norm1, par.norm2, 1e-5, h1, h2, bf),
                                           graph=True), 0.0, T * E * (4 + 4 + 2 + 2 + 4 + 2))
        cst = model.states[0]
        add(f"short_conv {tag}", timer(lambda: par.canon(h1, 0, cst, pos_ids, 1, T, bf, residual=True), graph=True), 0.0, T * E * (4 + 2))
    return rows, which


def run_bededra(args):
    import sys

    sys.path.insert(0, str(ROOT))
    from __graft_entry__ import build

    build()
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    timer = Timer(device)
    prompt_len = 2048
    out = {"family": "bededra", "beside": "lepalorn", "dtype": "bf16", "data": "synthetic (random weights)", "prompt_len": prompt_len,
           "batch": 1, "l2": "256 MB written between timed iterations", "sizes": {}}
    names = [n for n in BEDEDRA_SIZES if not getattr(args, "size", None) or n == args.size]
    for name in names:
        s = BEDEDRA_SIZES[name]
        with torch.no_grad():
            m = bededra_model(s, device)
            pre, dec = end_to_end(m, timer, prompt_len, device, prompt_len + 64)
            rows, which = bededra_kernel_table(s, m, device, timer, prompt_len)
            del m
            torch.cuda.empty_cache()
            lep = lepalorn_model(SIZES[name], device)
            lpre, ldec = end_to_end(lep, timer, prompt_len, device, prompt_len + 64)
            lrows, _ = kernel_table(SIZES[name], lep, device, timer, prompt_len)
            del lep
            torch.cuda.empty_cache()
        out["sizes"][name] = {"config": s, "bededra": {"prefill_tokens_per_s": round(pre), "decode_tokens_per_s": round(dec, 1)},
                              "lepalorn_same_width": {"prefill_tokens_per_s": round(lpre), "decode_tokens_per_s": round(ldec, 1)},
                              "kernels": rows, "lepalorn_kernels": [r for r in lrows if not r["kernel"].startswith("llama")],
                              "roofline": f"of {which}"}
    print(json.dumps(out))
    return 0


# Tebodra at the widths of SIZES, as deep as Bededra there.  Layers cycle through: attention_2 with a chunk mask (the size of
# Bededra's window), matrix memory, attention over the whole past (filters of 4 taps, half of every head rotated), attention_2
# reading the first layer's ring.  Attention heads as Bededra's; the matrix memory's values span the width, its keys half of
# that; a dense feed-forward of 4 x width.
TEBODRA_SIZES = {
    "w1024": dict(width=1024, layers=4, heads=8, kv=2, dim=64, chunk=512, m_heads=4, m_dim=128, m_vdim=256, ff=4096),
    "w2048": dict(width=2048, layers=4, heads=16, kv=4, dim=128, chunk=1024, m_heads=8, m_dim=128, m_vdim=256, ff=8192),
    "w4096": dict(width=4096, layers=2, heads=32, kv=8, dim=128, chunk=2048, m_heads=16, m_dim=128, m_vdim=256, ff=16384),
}


def tebodra_model(s, device, dtype=torch.bfloat16):
    from lit_llama.tebodra import Tebodra, TebodraConfig

    ff = {"kind": "dense", "ff": s["ff"]}
    D = s["dim"]
    chunked = {"type": "attention_2", "mlp": ff, "mixer": {
        "heads": s["heads"], "kv_heads": s["kv"], "dim": D, "vdim": D, "scale": D ** -0.5, "mask": {"size": s["chunk"]},
        "rot": {"base": 10000.0, "dims": D, "scaling": {"factor": 4.0}}}}
    memory = {"type": "mlstm", "mlp": None, "mixer": {"heads": s["m_heads"], "dim": s["m_dim"], "vdim": s["m_vdim"], "gate_cap": 15.0}}
    full = {"type": "attention", "mlp": ff, "mixer": {
        "heads": s["heads"], "kv_heads": s["kv"], "dim": D, "vdim": D, "scale": D ** -0.5, "conv": 4, "softcap": 50.0,
        "rot": {"base": 500000.0, "dims": D // 2, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}}}}
    borrow = {"type": "attention_2", "mlp": ff, "mixer": dict(chunked["mixer"], kv_from=0)}
    cycle = [chunked, memory, full, borrow] if s["layers"] >= 4 else [full, memory]
    cfg = {"vocab": VOCAB, "width": s["width"], "norm": {"eps": 1e-5}, "residual_mult": 0.5,
           "layers": [cycle[i % len(cycle)] for i in range(s["layers"])]}
    m = Tebodra(TebodraConfig.from_dict(cfg), dtype=dtype, device=device)
    g = torch.Generator(device=device).manual_seed(0)
    for n, p in m.named_parameters():
        leaf = n.rsplit(".", 1)[-1]
        if p.dim() >= 2 and "conv" not in n:
            p.copy_((torch.randn(p.shape, generator=g, device=device) / math.sqrt(p.shape[-1])).to(p.dtype))
        elif p.dim() >= 2:
            p.copy_(0.3 * torch.randn(p.shape, generator=g, device=device))
        elif leaf == "bias_f":
            p.fill_(3.0)
    return m.eval()


def tebodra_kernel_table(s, model, device, timer, prompt_len):
    """The mixers' kernels alone, one layer of each kind.  Roofline time = max(flops / tensor peak, bytes / copy bandwidth),
    flops and bytes counted for the mechanism (one sweep over the visible keys; one update and one read-out of the memory
    per token), not for what the kernel happens to do."""
    from torch.nn import functional as F

    from lit_llama.stepping import add_norm_pair
    from lit_llama.recurrence import decay_scan, gated_group_norm

    hbm, tflops, which = peaks()
    bf = torch.bfloat16
    rows = []

    def add(name, t, flops, nbytes):
        roof = max(flops / tflops, nbytes / hbm)
        rows.append(dict(kernel=name, us=round(t * 1e6, 1), roofline_us=round(roof * 1e6, 2), fraction=round(roof / t, 4)))

    E, H, G, D = s["width"], s["heads"], s["kv"], s["dim"]
    blocks = {}
    for i, b in enumerate(model.blocks):
        key = b.kind if b.kind == "mlstm" or b.mix.owner else "borrow"
        blocks.setdefault(key, (i, b))
    for T, tag in ((prompt_len, "prefill"), (1, "decode")):
        pos0 = 0 if T > 1 else prompt_len
        pos_ids = torch.arange(pos0, pos0 + T, dtype=torch.int32, device=device)
        model.reset_cache()
        model._begin(1, prompt_len + 64, True)
        for t in model.kv_caches:
            t.normal_()
        for t in model.states:
            t.zero_()
        x = torch.randn((T, E), device=device, dtype=bf)
        sms = torch.cuda.get_device_properties(device).multi_processor_count
        for kind, label in (("attention", "whole past, filters, cap"), ("attention_2", "chunk, norms, sink")):
            if kind not in blocks:
                continue
            i, blk = blocks[kind]
            att, spec = blk.mix, blk.mix.spec
            n = model._cache_of[i]
            caches = model.kv_caches[2 * n:2 * n + 2]
            proj = F.linear(x, att.w_in)
            conv_state = torch.zeros(att.conv.state_shape(1), device=device) if att.conv is not None else None
            reach = spec.reach or (1 << 30)
            span = min(reach, caches[0].shape[1])
            splits = 1 if T > 1 else max(1, min(64, (2 * sms) // max(1, (H + 3) // 4), (span + 127) // 128))
            keys = sum(p - (0 if spec.chunk is None else (p // spec.chunk) * spec.chunk) + 1 for p in range(pos0, pos0 + T))
            rows_read = min(pos0 + T, (reach if T == 1 else pos0 + T))

            def attn():
                att.attend(proj, 1, T, pos_ids, caches, conv_state, splits)

            add(f"rotary_attn {tag} ({label}: filter + norm/rotation/append + attention + gate)", timer(attn, graph=True),
                2.0 * keys * H * 2 * D, 2.0 * (rows_read * G * 2 * D + 3 * T * H * D))
        # matrix memory: gates, the walk with its normaliser column, the read-out norm
        _, mem = blocks["mlstm"]
        mm, ms = mem.mix, mem.mix.spec
        proj = F.linear(x, mm.w_in)
        c = mm.cols
        keep = torch.rand((T, ms.heads), device=device) * 0.1 + 0.9
        take = torch.rand((T, ms.heads), device=device)
        stab = torch.zeros((T, ms.heads), device=device)
        memory = torch.zeros((1, ms.heads, ms.dim, ms.vdim + 1), device=device)
        mstate = torch.zeros((1, ms.heads), device=device)
        from lit_llama import _native as N

        def gates():
            N.call("ll_matrix_memory_gates", N.ptr_at(proj, c["i"]), N.ptr_at(proj, c["f"]), N.dtype_code(bf), proj.stride(0),
                   N.ptr(mm.bias_i), N.ptr(mm.bias_f), float(ms.gate_cap), N.ptr(mstate), N.ptr(pos_ids), N.ptr(keep), N.ptr(take),
                   N.ptr(stab), 1, T, ms.heads, N.stream())

        add(f"matrix_memory_gates {tag}", timer(gates, graph=True), 0.0, T * ms.heads * (4 + 12))
        keep.uniform_(0.9, 1.0)
        take.uniform_(0.0, 1.0)

        def walk():
            decay_scan(proj, c["q"], proj, c["k"], proj, c["v"], keep, False, take, None, ms.dim ** -0.5, memory, pos_ids, 1, T, ms.heads,
                       ms.heads, ms.dim, ms.vdim + 1, unit_col=True)

        nst = ms.heads * ms.dim * (ms.vdim + 1)
        add(f"decay_scan {tag} (matrix memory + normaliser)", timer(walk, graph=True), 4.0 * T * nst,
            2.0 * T * ms.heads * (2 * ms.dim + ms.vdim) + 4.0 * T * ms.heads * (2 + ms.vdim + 1) + 8.0 * nst)
        yv = torch.randn((T, ms.heads * (ms.vdim + 1)), device=device)
        add(f"read-out norm + gate {tag}", timer(lambda: gated_group_norm(yv, proj, c["g"], mm.norm, False, 1e-5, ms.heads, False, bf,
                                                                          sigmoid=True, part=ms.vdim, stab=stab), graph=True),
            0.0, T * ms.heads * ms.vdim * (4 + 2 + 2))
        xs = torch.randn((T, E), device=device)
        h1 = torch.empty((T, E), device=device, dtype=bf)
        a0 = torch.randn((T, E), device=device, dtype=bf)
        add(f"add + norm {tag}", timer(lambda: add_norm_pair(xs, [(a0, 0.5)], mem.norm1, None, 1e-5, h1, None, bf), graph=True), 0.0,
            T * E * (4 + 4 + 2 + 4 + 2))
        hh = torch.randn((T, s["ff"]), device=device, dtype=bf)
        add(f"gelu {tag}", timer(lambda: N.call("ll_gelu", N.ptr(hh), N.dtype_code(bf), 0, hh.numel(), N.stream()), graph=True), 0.0,
            T * s["ff"] * 4)
    return rows, which


def run_tebodra(args):
    import sys

    sys.path.insert(0, str(ROOT))
    from __graft_entry__ import build

    build()
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    timer = Timer(device)
    prompt_len = 2048
    out = {"family": "tebodra", "beside": "bededra", "dtype": "bf16", "data": "synthetic (random weights)", "prompt_len": prompt_len,
           "batch": 1, "l2": "256 MB written between timed iterations", "sizes": {}}
    names = [n for n in TEBODRA_SIZES if not getattr(args, "size", None) or n == args.size]
    for name in names:
        s = TEBODRA_SIZES[name]
        with torch.no_grad():
            m = tebodra_model(s, device)
            pre, dec = end_to_end(m, timer, prompt_len, device, prompt_len + 64)
            rows, which = tebodra_kernel_table(s, m, device, timer, prompt_len)
            del m
            torch.cuda.empty_cache()
            bed = bededra_model(BEDEDRA_SIZES[name], device)
            bpre, bdec = end_to_end(bed, timer, prompt_len, device, prompt_len + 64)
            brows, _ = bededra_kernel_table(BEDEDRA_SIZES[name], bed, device, timer, prompt_len)
            del bed
            torch.cuda.empty_cache()
        out["sizes"][name] = {"config": s, "tebodra": {"prefill_tokens_per_s": round(pre), "decode_tokens_per_s": round(dec, 1)},
                              "bededra_same_width": {"prefill_tokens_per_s": round(bpre), "decode_tokens_per_s": round(bdec, 1)},
                              "kernels": rows, "bededra_kernels": brows, "roofline": f"of {which}"}
    print(json.dumps(out))
    return 0


# two-map attention: maps of dim (together Tebodra's head size), values of 2 * dim; latent attention as in the Lepalorn sizes
BUMULIX_SIZES = {
    "w1024": dict(width=1024, layers=4, heads=8, kv=2, dim=32, vdim=64, window=512, l_heads=8, nope=64, rot=32, v=64, kv_rank=256,
                  q_rank=384, ff=4096, streams=2),
    "w2048": dict(width=2048, layers=4, heads=16, kv=4, dim=64, vdim=128, window=1024, l_heads=16, nope=128, rot=64, v=128, kv_rank=512,
                  q_rank=768, ff=8192, streams=2),
    "w4096": dict(width=4096, layers=2, heads=32, kv=8, dim=64, vdim=128, window=2048, l_heads=32, nope=128, rot=64, v=128, kv_rank=512,
                  q_rank=1536, ff=16384, streams=2),
}


def bumulix_model(s, device, dtype=torch.bfloat16):
    from lit_llama.bumulix import Bumulix, BumulixConfig

    ff = {"kind": "dense", "ff": s["ff"]}
    window = {"type": "attention", "mlp": ff, "mixer": {
        "heads": s["heads"], "kv_heads": s["kv"], "dim": s["dim"], "vdim": s["vdim"], "diff": 0.5, "scale": s["dim"] ** -0.5,
        "mask": {"size": s["window"]}}}
    lat = {"type": "latent_attention", "mlp": ff, "mixer": {
        "heads": s["l_heads"], "dim": s["nope"], "rot_dim": s["rot"], "vdim": s["v"], "kv_rank": s["kv_rank"], "q_rank": s["q_rank"],
        "scale": (s["nope"] + s["rot"]) ** -0.5,
        "rot": {"base": 10000.0, "dims": s["rot"], "scaling": {"factor": 8.0, "original": 4096, "fast": 32.0, "slow": 1.0}}}}
    cycle = [window, lat, dict(window, weights_of=0), dict(lat, weights_of=1)] if s["layers"] >= 4 else [window, lat]
    cfg = {"vocab": VOCAB, "width": s["width"], "norm": {"eps": 1e-5}, "residual_mult": 0.5, "streams": s["streams"], "logit_softcap": 30.0,
           "layers": [cycle[i % len(cycle)] for i in range(s["layers"])]}
    m = Bumulix(BumulixConfig.from_dict(cfg), dtype=dtype, device=device)
    g = torch.Generator(device=device).manual_seed(0)
    for n, p in m.named_parameters():
        if p.dim() >= 2 and ".hc" not in n:
            p.copy_((torch.randn(p.shape, generator=g, device=device) / math.sqrt(p.shape[-1])).to(p.dtype))
    for b in m.blocks:
        if b.kind == "attention":
            b.mix.diff_lambda = 0.6
    return m.eval()


def bumulix_kernel_table(s, model, device, timer, prompt_len):
    """The mixers' kernels alone, one layer of each kind, and the stream update.  Roofline time = max(flops / tensor peak,
    bytes / copy bandwidth), flops and bytes counted for the mechanism (one sweep over the visible keys per score map; every
    copy of the stream read and written once), not for what the kernel happens to do."""
    from torch.nn import functional as F

    from lit_llama import _native as N
    from lit_llama.stepping import hyper_mix_norm

    hbm, tflops, which = peaks()
    bf = torch.bfloat16
    rows = []

    def add(name, t, flops, nbytes):
        roof = max(flops / tflops, nbytes / hbm)
        rows.append(dict(kernel=name, us=round(t * 1e6, 1), roofline_us=round(roof * 1e6, 2), fraction=round(roof / t, 4)))

    E, S = s["width"], s["streams"]
    first = {}
    for i, (l, b) in enumerate(zip(model.config.layers, model._block_of)):
        first.setdefault(l.kind, (i, b))
    sms = torch.cuda.get_device_properties(device).multi_processor_count
    for T, tag in ((prompt_len, "prefill"), (1, "decode")):
        pos0 = 0 if T > 1 else prompt_len
        pos_ids = torch.arange(pos0, pos0 + T, dtype=torch.int32, device=device)
        model.reset_cache()
        model._begin(1, prompt_len + 64, True)
        for t in model.kv_caches:
            t.normal_()
        x = torch.randn((T, E), device=device, dtype=bf)
        # two score maps over a window
        i, blk = first["attention"]
        att, spec = blk.mix, blk.mix.spec
        at = model._cache_at[i]
        caches = model.kv_caches[at:at + 2]
        proj = F.linear(x, att.w_in)
        H, G, D, V, W = spec.heads, spec.kv_heads, spec.dim, spec.vdim, spec.window
        span = min(W, caches[0].shape[1])
        splits = 1 if T > 1 else max(1, min(64, (2 * sms) // max(1, (H * 2 + 3) // 4), (span + 31) // 32))
        keys = sum(min(p + 1, W) for p in range(pos0, pos0 + T))
        rows_read = min(pos0 + T, W + T - 1)
        add(f"two-map attention {tag} (append + attention + difference + unit norm)",
            timer(lambda: att.attend(proj, 1, T, pos_ids, caches, None, splits), graph=True),
            2.0 * keys * H * 2 * (D + V), 2.0 * (rows_read * G * (2 * D + V) + T * (H * 2 * D + G * (2 * D + V) + H * V)))
        # latent attention over the whole past
        i, blk = first["latent_attention"]
        lat, ls = blk.mix, blk.mix.spec
        cache = model.kv_caches[model._cache_at[i]]
        rope = model._rope[next(iter(model._rope))]
        lsplits = 1 if T > 1 else max(1, min(16, (2 * sms) // max(1, (ls.heads + 31) // 32), (cache.shape[1] + 63) // 64))
        lkeys = sum(p + 1 for p in range(pos0, pos0 + T))
        proj_l = F.linear(x, lat.w_in)
        cq = torch.empty((T, ls.q_rank), dtype=bf, device=device)
        q = F.linear(cq, lat.w_uq)
        q_lat = torch.randn((ls.heads, T, ls.kv_rank), dtype=bf, device=device)
        o_lat = torch.empty_like(q_lat)
        o = torch.randn((T, ls.heads * ls.v_dim), dtype=bf, device=device)
        scratch = torch.empty(N.call_ret("ll_latent_attn_scratch_bytes", T, ls.heads, ls.kv_rank, lsplits) // 4 + 4, device=device)
        dt = N.dtype_code(bf)

        def latent_kernels():
            st = N.stream()
            N.call("ll_latent_kv_append", N.ptr(proj_l), dt, proj_l.shape[1], lat.kv_col0, N.ptr(lat.kv_norm), 1e-5, N.ptr(rope),
                   N.ptr(pos_ids), N.ptr(cache), 1, T, ls.kv_rank, ls.rot_dim, ls.rot_dims, cache.shape[1], st)
            N.call("ll_row_norm", N.ptr(proj_l), proj_l.shape[1], N.ptr(lat.q_norm), 1e-5, N.ptr(cq), ls.q_rank, dt, T, ls.q_rank, st)
            N.call("ll_latent_attn", N.ptr(q_lat), T * ls.kv_rank, ls.kv_rank, N.ptr(q), q.shape[1], ls.nope_dim, ls.q_head, -1,
                   N.ptr(rope), N.ptr(pos_ids), N.ptr(cache), N.ptr(o_lat), T * ls.kv_rank, ls.kv_rank, dt, 1, T, ls.heads, ls.kv_rank,
                   ls.rot_dim, ls.rot_dims, cache.shape[1], 0, float(ls.scale), lsplits, N.ptr(scratch), st)
            N.call("ll_sigmoid_gate_mul", N.ptr(o), o.shape[1], N.ptr_at(proj_l, lat.gate_col0), proj_l.shape[1], N.ptr(o), o.shape[1], dt,
                   T, ls.heads * ls.v_dim, st)

        add(f"latent attention {tag} (latent norms + append + attention in latent space + element-wise gate)",
            timer(latent_kernels, graph=True), 2.0 * lkeys * ls.heads * (2 * ls.kv_rank + ls.rot_dim),
            2.0 * ((pos0 + T) * ls.row + T * ls.heads * (2 * ls.kv_rank + ls.rot_dim + 2 * ls.v_dim)))
        # the stream: one sublayer's result into all copies, the next sublayer's input out
        X = torch.randn((T, S, E), device=device)
        y = torch.randn((T, E), device=device, dtype=bf)
        h = torch.empty((T, E), device=device, dtype=bf)
        add(f"stream copies: write + read + norm {tag}",
            timer(lambda: hyper_mix_norm(X, X, (y, blk.ls1, blk.hc1), 0.5, blk.hc2.w_in, blk.norm2, 1e-5, h, None, bf), graph=True), 0.0,
            T * E * (8 * S + 2 + 2))
        hh = torch.randn((T, s["ff"]), device=device, dtype=bf)
        add(f"gelu (tanh form) {tag}", timer(lambda: N.call("ll_gelu", N.ptr(hh), dt, 1, hh.numel(), N.stream()), graph=True), 0.0,
            T * s["ff"] * 4)
    return rows, which


def run_bumulix(args):
    import sys

    sys.path.insert(0, str(ROOT))
    from __graft_entry__ import build

    build()
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    timer = Timer(device)
    prompt_len = 2048
    out = {"family": "bumulix", "beside": "tebodra", "dtype": "bf16", "data": "synthetic (random weights)", "prompt_len": prompt_len,
           "batch": 1, "l2": "256 MB written between timed iterations", "sizes": {}}
    names = [n for n in BUMULIX_SIZES if not getattr(args, "size", None) or n == args.size]
    for name in names:
        s = BUMULIX_SIZES[name]
        with torch.no_grad():
            m = bumulix_model(s, device)
            pre, dec = end_to_end(m, timer, prompt_len, device, prompt_len + 64)
            rows, which = bumulix_kernel_table(s, m, device, timer, prompt_len)
            del m
            torch.cuda.empty_cache()
            teb = tebodra_model(TEBODRA_SIZES[name], device)
            tpre, tdec = end_to_end(teb, timer, prompt_len, device, prompt_len + 64)
            trows, _ = tebodra_kernel_table(TEBODRA_SIZES[name], teb, device, timer, prompt_len)
            del teb
            torch.cuda.empty_cache()
        out["sizes"][name] = {"config": s, "bumulix": {"prefill_tokens_per_s": round(pre), "decode_tokens_per_s": round(dec, 1)},
                              "tebodra_same_width": {"prefill_tokens_per_s": round(tpre), "decode_tokens_per_s": round(tdec, 1)},
                              "kernels": rows, "tebodra_kernels": trows, "roofline": f"of {which}"}
    print(json.dumps(out))
    return 0


def run(args):
    import sys

    if args.family == "bededra":
        return run_bededra(args)
    if args.family == "tebodra":
        return run_tebodra(args)
    if args.family == "bumulix":
        return run_bumulix(args)
    sys.path.insert(0, str(ROOT))
    from __graft_entry__ import build

    build()
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    timer = Timer(device)
    prompt_len = 2048
    out = {"family": "lepalorn", "dtype": "bf16", "data": "synthetic (random weights)", "prompt_len": prompt_len, "batch": 1,
           "l2": "256 MB written between timed iterations", "sizes": {}}
    names = [n for n in SIZES if not getattr(args, "size", None) or n == args.size]
    for name in names:
        s = SIZES[name]
        with torch.no_grad():
            lep = lepalorn_model(s, device)
            pre, dec = end_to_end(lep, timer, prompt_len, device, prompt_len + 64)
            rows, which = kernel_table(s, lep, device, timer, prompt_len)
            del lep
            torch.cuda.empty_cache()
            ll = llama_model(s, device)
            lpre, ldec = end_to_end(ll, timer, prompt_len, device, prompt_len + 64)
            del ll
            torch.cuda.empty_cache()
        out["sizes"][name] = {"config": s, "lepalorn": {"prefill_tokens_per_s": round(pre), "decode_tokens_per_s": round(dec, 1)},
                              "llama_bf16_same_width": {"prefill_tokens_per_s": round(lpre), "decode_tokens_per_s": round(ldec, 1)},
                              "kernels": rows, "roofline": f"of {which}"}
    print(json.dumps(out))
    return 0
