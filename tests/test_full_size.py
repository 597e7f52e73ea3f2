"""Parity at the full sizes of the benchmark configurations, with the CPU oracle on the other side every time. Needs a B200.

  config 0 / 1  one token, 256 + 1 experts, 40 layers: symmetric int4 (fp16 group scales) and GGUF Q4_K (zero-point blobs);
                the cooperative one-token kernel and the graph of per-layer kernels, every layer teacher-forced
  config 2      4 tokens x 40 layers, every layer teacher-forced, plus the chained graph end to end
  config 3      all 2048 tokens of the prefill chunk (tcgen05 grouped GEMM) against the oracle
  config 4      64 tokens x 40 layers, every layer teacher-forced, plus the chained graph end to end

Teacher-forced: layer l of the GPU gets the ORACLE's input to layer l, so a routing flip cannot cascade; the selected
experts must be identical and the outputs inside the bars of tests/parity.py. End to end: the GPU chains its own outputs
through all 40 layers; the drift against the oracle chain is measured on the tokens whose routing stayed identical in
every layer (a near-tie that flips changes the function being computed, not its accuracy) and those are counted.
The host side builds only the experts a batch selected (the generator is keyed by (seed, layer, expert)).
"""
import numpy as np
import pytest
import torch

import moe_b200 as m
from oracle import oracle as o
from parity import check_ffn, record

pytestmark = [pytest.mark.gpu, pytest.mark.usefixtures("lib_built")]
DEV = "cuda:0"
E, K, NL, SEED = 256, 8, 40, 0


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


def router(layer):
    return (np.random.default_rng([77, layer]).standard_normal((E + 1, 2048)) * 0.02).astype(np.float32)


_host_cache = {}


def host_expert(fmt, layer, e):
    key = (fmt, layer, e)
    if key not in _host_cache:
        if len(_host_cache) > 600:
            _host_cache.clear()
        _host_cache[key] = m.synth_expert_host(fmt, SEED, layer, e)
    return _host_cache[key]


def oracle_block(fmt, layer, W, x):
    """x_{l+1} = x + moe(rmsnorm(x)) by the oracle, building only the selected experts. Returns (x_next, ids)."""
    xn = o.rmsnorm(x)
    ids, _ = o.router_topk(o.router_logits(W, xn, x.shape[0]), E, K, True, x.shape[0], E + 1)
    need = set(np.unique(ids).tolist()) | {E}
    blobs = [host_expert(fmt, layer, e) if e in need else None for e in range(E + 1)]
    moe, ri, _, _ = o.layer_forward(fmt, blobs, W, xn, K)
    assert np.array_equal(ri, ids)
    return x + moe, ri


def make_layers(ctx, fmt):
    layers, Ws = [], []
    for l in range(NL):
        L = m.Layer(ctx, fmt, E)
        L.fill_synth(SEED, l)
        W = router(l)
        L.set_router(W)
        layers.append(L); Ws.append(W)
    torch.cuda.synchronize()
    return layers, Ws


@pytest.fixture(scope="module")
def sym40():
    ctx = m.Context(0, max_tokens=64, max_experts=E, top_k=K)
    layers, Ws = make_layers(ctx, m.FMT_SYM_F16)
    yield ctx, layers, Ws
    for L in layers:
        L.close()
    ctx.close()


def forced_and_chained(ctx, layers, Ws, fmt, T, name):
    """Every layer teacher-forced against the oracle, then the chained graph; returns the oracle's per-layer inputs."""
    rng = np.random.default_rng(1000 + T)
    x0 = rng.standard_normal((T, 2048)).astype(np.float32)
    xs, ids_ref = [x0], []
    worst = (0.0, 0.0, 0.0)
    for l in range(NL):
        x_next, ri = oracle_block(fmt, l, Ws[l], xs[l])
        idx = torch.empty(T, K, dtype=torch.int32, device=DEV)
        got = layers[l].forward(dev(xs[l]), T, K, idx=idx, flags=2).cpu().numpy()
        assert np.array_equal(idx.cpu().numpy(), ri), f"{name}: layer {l} selected other experts than the oracle"
        r = check_ffn(got, x_next, fmt, f"{name} layer {l} teacher-forced", quiet=True)
        worst = tuple(max(a, b) for a, b in zip(worst, r))
        xs.append(x_next); ids_ref.append(ri)
    assert ctx.status() == 0
    record(f"{name}: worst of {NL} teacher-forced layers", *worst, float(np.abs(xs[-1]).max()))
    return x0, xs, ids_ref


def chained_drift(ctx, layers, x0, xs, ids_ref, T, name, fmt):
    """The stack as one replay (graph, or the cooperative kernel for one token) against the oracle chain."""
    stack = m.Stack(ctx, layers, T, K, m.F32)
    y = stack.run(dev(x0)).cpu().numpy().copy()
    y2 = stack.run(dev(x0)).cpu().numpy()
    kernels = stack.kernel_count
    stack.close()
    assert ctx.status() == 0 and np.isfinite(y).all() and np.array_equal(y, y2)
    # which tokens kept the oracle's routing in every layer: chain the per-layer calls and compare the ids
    x = dev(x0)
    same = np.ones(T, bool)
    bufs = [torch.empty(T, 2048, device=DEV), torch.empty(T, 2048, device=DEV)]
    for l, L in enumerate(layers):
        idx = torch.empty(T, K, dtype=torch.int32, device=DEV)
        x = L.forward(x, T, K, out=bufs[l & 1], idx=idx, flags=2)
        same &= (idx.cpu().numpy() == ids_ref[l]).all(axis=1)
    assert same.sum() >= max(1, int(0.75 * T)), f"{name}: only {same.sum()} of {T} tokens kept the oracle's routing through {NL} layers"
    r = check_ffn(y[same], xs[-1][same], fmt, f"{name} end to end over {NL} layers ({int(same.sum())} of {T} tokens with identical routing)")
    return y, kernels


@pytest.mark.parametrize("T", [64, 4])
def test_config_2_and_4_every_layer_against_the_oracle(sym40, T):
    ctx, layers, Ws = sym40
    name = f"config {4 if T == 64 else 2}: {T} tokens x {NL} layers x {E + 1} experts"
    x0, xs, ids_ref = forced_and_chained(ctx, layers, Ws, m.FMT_SYM_F16, T, name)
    y, kernels = chained_drift(ctx, layers, x0, xs, ids_ref, T, name, m.FMT_SYM_F16)
    assert kernels > NL   # a graph of per-layer kernels
    # the graph replays exactly what the chained layer calls compute
    x = dev(x0)
    bufs = [torch.empty(T, 2048, device=DEV), torch.empty(T, 2048, device=DEV)]
    for l, L in enumerate(layers):
        x = L.forward(x, T, K, out=bufs[l & 1], flags=2)
    assert np.array_equal(y, x.cpu().numpy())


def one_token_checks(ctx, layers, Ws, fmt, name):
    """One token: per layer (teacher-forced) the per-layer kernels AND the cooperative kernel run on that single layer;
    then the cooperative kernel over all 40 layers against the oracle chain."""
    x0, xs, ids_ref = forced_and_chained(ctx, layers, Ws, fmt, 1, name + ", per-layer kernels")
    worst = (0.0, 0.0, 0.0)
    for l in range(NL):
        one = m.Stack(ctx, [layers[l]], 1, K, m.F32)
        assert one.kernel_count == 1
        got = one.run(dev(xs[l])).cpu().numpy()
        one.close()
        r = check_ffn(got, xs[l + 1], fmt, f"{name} layer {l}, cooperative kernel teacher-forced", quiet=True)
        worst = tuple(max(a, b) for a, b in zip(worst, r))
    assert ctx.status() == 0
    record(f"{name}: cooperative kernel, worst of {NL} teacher-forced layers", *worst, float(np.abs(xs[-1]).max()))
    y, kernels = chained_drift(ctx, layers, x0, xs, ids_ref, 1, name + ", cooperative kernel", fmt)
    assert kernels == 1
    ctx.set_fused_decode(False)
    try:
        yg, kernels = chained_drift(ctx, layers, x0, xs, ids_ref, 1, name + ", graph of per-layer kernels", fmt)
    finally:
        ctx.set_fused_decode(True)
    assert kernels > NL


def test_config_0_one_token_symmetric(sym40):
    ctx, layers, Ws = sym40
    one_token_checks(ctx, layers, Ws, m.FMT_SYM_F16, f"config 0: 1 token x {NL} layers x {E + 1} experts (i4_gs64)")


def test_config_1_one_token_q4k():
    ctx = m.Context(0, max_tokens=4, max_experts=E, top_k=K)
    layers, Ws = make_layers(ctx, m.FMT_ZP)
    try:
        one_token_checks(ctx, layers, Ws, m.FMT_ZP, f"config 1: 1 token x {NL} layers x {E + 1} experts (Q4_K as zero point)")
        # the single layer of the configuration as the plain layer call (no norm, no residual), like config 0's
        rng = np.random.default_rng(5)
        X = rng.standard_normal((1, 2048)).astype(np.float32)
        ids, _ = o.router_topk(o.router_logits(Ws[0], X, 1), E, K, True, 1, E + 1)
        blobs = [host_expert(m.FMT_ZP, 0, e) if (e in ids or e == E) else None for e in range(E + 1)]
        ref, ri, rw, _ = o.layer_forward(m.FMT_ZP, blobs, Ws[0], X, K)
        idx = torch.empty(1, K, dtype=torch.int32, device=DEV); w = torch.empty(1, K, device=DEV)
        out = layers[0].forward(dev(X), 1, K, idx=idx, w=w).cpu().numpy()
        assert np.array_equal(idx.cpu().numpy(), ri) and np.allclose(w.cpu().numpy(), rw, rtol=2e-6, atol=0)
        check_ffn(out, ref, m.FMT_ZP, "config 1: one Q4_K layer, one token")
    finally:
        for L in layers:
            L.close()
        ctx.close()


def test_config_3_all_2048_tokens_against_the_oracle():
    """The full prefill chunk on the tcgen05 grouped GEMM: every one of the 2048 tokens against the oracle, and the streaming
    kernels on the same batch (an independent implementation) against the oracle as well."""
    T = 2048
    rng = np.random.default_rng(2048)
    c = m.Context(0, max_tokens=T, max_experts=E, top_k=K)
    L = m.Layer(c, m.FMT_SYM_F16, E)
    L.fill_synth(SEED, 0)
    W = router(0)
    L.set_router(W)
    X = torch.from_numpy(rng.standard_normal((T, 2048)).astype(np.float32)).to(torch.bfloat16)
    host = [host_expert(m.FMT_SYM_F16, 0, e) for e in range(E + 1)]
    ref, ri, rw, _ = o.layer_forward(m.FMT_SYM_F16, host, W, X.float().numpy(), K)
    try:
        for fam, min_tokens in (("tcgen05 grouped GEMM", 256), ("streaming kernels", 1 << 20)):
            c.set_prefill_min_tokens(min_tokens)
            idx = torch.empty(T, K, dtype=torch.int32, device=DEV); w = torch.empty(T, K, device=DEV)
            out = L.forward(X.to(DEV), T, K, idx=idx, w=w).cpu().numpy()
            assert c.status() == 0
            assert np.array_equal(idx.cpu().numpy(), ri), fam
            assert np.allclose(w.cpu().numpy(), rw, rtol=2e-6, atol=0)
            check_ffn(out, ref, m.FMT_SYM_F16, f"config 3: 2048 tokens x {E + 1} experts, {fam}")
    finally:
        L.close(); c.close()
