"""The expert-parallel path (token all-to-all over peer memory) with all ranks emulated on ONE GPU: R contexts, R sets of
layers holding a slice of the experts each, R exchange buffers that are simply each other's "peers" in the same address
space. The phases of a step are enqueued rank after rank (all dispatches of a layer, then all expert phases), so every flag
a kernel waits for has already been raised and no kernel ever waits on a kernel that has not run. What is checked is the
whole of the device code - token ownership, selective row pushes, planning of the held experts only, partial sums, the
owner's sum in rank order - against the oracle chain. Needs a B200."""
import numpy as np
import pytest
import torch

import moe_b200 as m
from moe_b200 import ep as eph
from oracle import oracle as o
from parity import check_ffn

pytestmark = [pytest.mark.gpu, pytest.mark.usefixtures("lib_built")]
DEV = "cuda:0"


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


class Ranks:
    def __init__(self, world, E, T, K, NL, fmt, seed, max_tokens=None, prefill_min=None):
        self.world, self.T, self.K, self.NL = world, T, K, NL
        rng = np.random.default_rng(seed)
        self.Ws = [(rng.standard_normal((E + 1, 2048)) * 0.02).astype(np.float32) for _ in range(NL)]
        self.hosts = [[m.synth_expert_host(fmt, seed, l, e) for e in range(E + 1)] for l in range(NL)]
        self.ctxs, self.layers, self.bufs, self.eps = [], [], [], []
        for r in range(world):
            c = m.Context(0, max_tokens=max_tokens or max(T, 8), max_experts=E, top_k=K)
            if prefill_min:
                c.set_prefill_min_tokens(prefill_min)
            first, cnt = eph.expert_range(E, r, world)
            ls = []
            for l in range(NL):
                L = m.Layer(c, fmt, E, first_local=first, n_local=cnt)
                L.fill_synth(seed, l); L.set_router(self.Ws[l])
                ls.append(L)
            self.ctxs.append(c); self.layers.append(ls)
            self.bufs.append(m.ExchangeBuffer(T, K, world))
        ptrs = [b.ptr for b in self.bufs]
        for r in range(world):
            self.eps.append(m.EP(self.ctxs[r], r, world, T, K, E, ptrs))

    def step(self, X, residual=True):
        """One step, phase by phase over the ranks; returns the [T][H] output assembled from the owners' rows."""
        for e in self.eps:
            e.begin_step()
        for l in range(self.NL):
            for r, e in enumerate(self.eps):
                e.dispatch(self.layers[r][l], l, X if l == 0 else None, residual)
            for r, e in enumerate(self.eps):
                e.experts(self.layers[r][l], l)
        out = torch.zeros(self.T, 2048, device=DEV)
        for e in self.eps:
            e.finish(self.NL, out[e.first_token:e.first_token + e.n_own], residual)
        torch.cuda.synchronize()
        for c in self.ctxs:
            assert c.status() == 0
        return out.cpu().numpy()

    def close(self):
        for e in self.eps:
            e.close()
        for b in self.bufs:
            b.close()
        for ls in self.layers:
            for L in ls:
                L.close()
        for c in self.ctxs:
            c.close()


def oracle_chain(R, fmt, X, K):
    x = X.copy()
    for l in range(R.NL):
        moe, _, _, _ = o.layer_forward(fmt, R.hosts[l], R.Ws[l], o.rmsnorm(x), K)
        x = x + moe
    return x


@pytest.mark.parametrize("world,T,fmt", [(2, 16, m.FMT_SYM_F16), (3, 5, m.FMT_SYM_F16), (4, 64, m.FMT_SYM_F16), (8, 64, m.FMT_SYM_F16),
                                         (2, 7, m.FMT_ZP), (3, 20, m.FMT_SYM_F32)])
def test_residual_blocks_match_the_oracle_chain(world, T, fmt):
    E, K, NL = 32, 8, 3
    R = Ranks(world, E, T, K, NL, fmt, seed=10 + world)
    try:
        assert sum(e.n_own for e in R.eps) == T and [e.first_token for e in R.eps] == [eph.token_range(T, r, world)[0] for r in range(world)]
        rng = np.random.default_rng(T)
        for rep in range(2):   # the second step re-uses every buffer and flag with the next step number
            X = rng.standard_normal((T, 2048)).astype(np.float32)
            got = R.step(dev(X))
            check_ffn(got, oracle_chain(R, fmt, X, K), fmt, f"expert parallel, {world} emulated ranks, {T} tokens, format {fmt}, step {rep}")
    finally:
        R.close()


def test_plain_layer_and_bf16_input():
    E, K, T, world = 32, 8, 24, 2
    R = Ranks(world, E, T, K, 1, m.FMT_SYM_F16, seed=3)
    try:
        X = torch.randn(T, 2048, generator=torch.Generator().manual_seed(1)).to(torch.bfloat16)
        got = R.step(X.to(DEV), residual=False)
        ref, _, _, _ = o.layer_forward(m.FMT_SYM_F16, R.hosts[0], R.Ws[0], X.float().numpy(), K)
        check_ffn(got, ref, m.FMT_SYM_F16, "expert parallel, plain layer, bf16 input")
    finally:
        R.close()


@pytest.mark.parametrize("residual,bf16", [(False, True), (True, False)])
def test_prefill_size_batch_on_the_grouped_gemm(residual, bf16):
    """A batch large enough for the tcgen05 grouped GEMM: the owners make the fp16 columns (one per token for exact bf16
    input of a plain layer, hi + lo otherwise) and the ranks' tiles read what the peers stored."""
    E, K, T, world, NL = 64, 8, 300, 2, (2 if residual else 1)
    R = Ranks(world, E, T, K, NL, m.FMT_SYM_F16, seed=8, max_tokens=T, prefill_min=256)
    try:
        Xf = np.random.default_rng(5).standard_normal((T, 2048)).astype(np.float32)
        X = torch.from_numpy(Xf).to(torch.bfloat16) if bf16 else torch.from_numpy(Xf)
        got = R.step(X.to(DEV), residual=residual)
        Xv = X.float().numpy()
        if residual:
            ref = oracle_chain(R, m.FMT_SYM_F16, Xv, K)
        else:
            ref, _, _, _ = o.layer_forward(m.FMT_SYM_F16, R.hosts[0], R.Ws[0], Xv, K)
        check_ffn(got, ref, m.FMT_SYM_F16, f"expert parallel prefill, residual={residual}, bf16={bf16}")
    finally:
        R.close()


def test_a_rank_whose_peer_never_answers_gives_up_and_reports(lib_built):
    """Rank 0 of 2 runs a whole step alone: the flags rank 1 would raise never come. Its planner and its combine kernel run
    out of polls (about two seconds each), record 7 and 8 in the error word and finish; nothing hangs, nothing faults, and
    the same context then computes a correct layer."""
    E, K, T = 32, 8, 8
    R = Ranks(2, E, T, K, 1, m.FMT_SYM_F16, seed=4)
    try:
        X = np.random.default_rng(0).standard_normal((T, 2048)).astype(np.float32)
        e = R.eps[0]
        out = torch.zeros(e.n_own, 2048, device=DEV)
        e.step(R.layers[0], dev(X), out)
        torch.cuda.synchronize()
        assert R.ctxs[0].status() in (7, 8)
        assert R.ctxs[0].status() == 0
        assert bool(torch.isfinite(out).all())
        assert R.ctxs[0].selftest_timeout(2, 4096) == 8
    finally:
        R.close()
