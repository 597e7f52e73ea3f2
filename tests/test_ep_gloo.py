"""Expert parallelism on CPU ranks (gloo, world size 2 and 3): the sharding arithmetic and the per-layer exchange of
moe_b200/ep.py, with the oracle as each rank's compute. The sum of the ranks' partial outputs must equal the
single-process layer."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _rank_main(rank, world, port, E, T, q):
    sys.path.insert(0, ROOT)
    import moe_b200 as m
    from moe_b200 import ep
    from oracle import oracle as o
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    rng = np.random.default_rng(3)
    W = (rng.standard_normal((E + 1, 2048)) * 0.02).astype(np.float32)
    X = rng.standard_normal((T, 2048)).astype(np.float32)
    first, cnt = ep.expert_range(E, rank, world)
    t0, t1 = ep.shared_token_range(T, rank, world)
    blobs = [m.synth_expert_host(m.FMT_SYM_F16, 4, 0, e) if first <= e < first + cnt else None for e in range(E)]
    shared = m.synth_expert_host(m.FMT_SYM_F16, 4, 0, E)

    def partial(x):
        xn = o.rmsnorm(x.numpy())
        out, idx, w, logits = o.layer_forward(m.FMT_SYM_F16, blobs + [None], W, xn, 8)   # this rank's routed experts only
        if t1 > t0:                                                                       # + the shared expert for its token slice
            sh = o.run_pairs(m.FMT_SYM_F16, [(shared, list(range(t0, t1)), list(range(t1 - t0)), [1.0] * (t1 - t0))], xn, t1 - t0)
            out[t0:t1] += sh / (1.0 + np.exp(-logits[t0:t1, E:E + 1]))
        return torch.from_numpy(out)

    y = ep.ep_block(torch.from_numpy(X), partial)
    if rank == 0:
        blobs_all = [m.synth_expert_host(m.FMT_SYM_F16, 4, 0, e) for e in range(E + 1)]
        ref, _, _, _ = o.layer_forward(m.FMT_SYM_F16, blobs_all, W, o.rmsnorm(X), 8)
        ref = X + ref
        err = float(np.abs(y.numpy() - ref).max()); rel = float(np.linalg.norm(y.numpy() - ref) / np.linalg.norm(ref))
        q.put((err, rel))
    dist.destroy_process_group()


def _exchange_main(rank, world, port, E, T, q):
    """The token all-to-all protocol of the peer-memory path (moe_b200.ep.exchange_block) with the oracle as every rank's
    compute: own tokens routed by their owner, rows only where needed, partial rows summed by the owner in rank order."""
    sys.path.insert(0, ROOT)
    import moe_b200 as m
    from moe_b200 import ep
    from oracle import oracle as o
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    rng = np.random.default_rng(5)
    W = (rng.standard_normal((E + 1, 2048)) * 0.02).astype(np.float32)
    X = rng.standard_normal((T, 2048)).astype(np.float32)
    first, cnt = ep.expert_range(E, rank, world)
    t0, t1 = ep.token_range(T, rank, world)
    held = [m.synth_expert_host(m.FMT_SYM_F16, 4, 0, e) if first <= e < first + cnt else None for e in range(E)]
    shared = m.synth_expert_host(m.FMT_SYM_F16, 4, 0, E)
    gate = {}

    def route(x_own):
        xn = o.rmsnorm(x_own)
        logits = o.router_logits(W, xn, xn.shape[0])
        idx, w = o.router_topk(logits, E, 8, True, xn.shape[0], E + 1)
        gate["logit"] = logits[:, E:E + 1]
        return xn, idx, w

    def partial(xn, idx, w, toks):
        out, ri, _, _ = o.layer_forward(m.FMT_SYM_F16, held + [None], W, xn[toks], 8, flags=1)   # this rank's experts only
        assert np.array_equal(ri, idx[toks])                                                       # the same routing everywhere
        return out

    def shared_fn(xn_own, idx, w):
        n = xn_own.shape[0]
        sh = o.run_pairs(m.FMT_SYM_F16, [(shared, list(range(n)), list(range(n)), [1.0] * n)], xn_own, n)
        return (sh / (1.0 + np.exp(-gate["logit"]))).astype(np.float32)

    y = ep.exchange_block(X[t0:t1], T, E, route, partial, shared_fn)
    blobs_all = [m.synth_expert_host(m.FMT_SYM_F16, 4, 0, e) for e in range(E + 1)]
    ref, _, _, _ = o.layer_forward(m.FMT_SYM_F16, blobs_all, W, o.rmsnorm(X), 8)
    ref = (X + ref)[t0:t1]
    q.put((rank, float(np.abs(y - ref).max()), float(np.linalg.norm(y - ref) / np.linalg.norm(ref))))
    dist.destroy_process_group()


@pytest.mark.parametrize("world,T", [(2, 5), (3, 7)])
def test_token_all_to_all_protocol_on_cpu_ranks(lib_built, world, T):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29650 + world + os.getpid() % 200
    procs = [ctx.Process(target=_exchange_main, args=(r, world, port, 32, T, q)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(180)
        assert p.exitcode == 0
    for _ in range(world):
        rank, err, rel = q.get(timeout=10)
        assert rel <= 1e-6 and err <= 1e-4, (rank, err, rel)   # fp32 sums in another order, nothing else


@pytest.mark.parametrize("world", [2, 3])
def test_expert_parallel_block_on_cpu_ranks(lib_built, world):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29600 + world + os.getpid() % 200
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, 32, 5, q)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(180)
        assert p.exitcode == 0
    err, rel = q.get(timeout=10)
    assert rel <= 1e-6 and err <= 1e-4, (err, rel)   # fp32 sums in another order, nothing else


def test_partition_arithmetic():
    from moe_b200 import ep
    for n, world in ((256, 8), (256, 3), (64, 4), (5, 8), (1, 2)):
        seen = []
        for r in range(world):
            f, c = ep.expert_range(n, r, world)
            seen += list(range(f, f + c))
            t0, t1 = ep.shared_token_range(n, r, world)
            assert 0 <= t0 <= t1 <= n and (t0, t1) == ep.token_range(n, r, world)
        assert seen == list(range(n))
        assert sum(ep.shared_token_range(n, r, world)[1] - ep.shared_token_range(n, r, world)[0] for r in range(world)) == n


def test_which_ranks_a_token_needs():
    from moe_b200 import ep
    idx = np.array([[0, 1, 2, 3, 4, 5, 6, 7], [0, 40, 80, 120, 160, 200, 240, 255], [250, 251, 252, 253, 254, 255, 249, 248]])
    need = ep.ranks_of(idx, 256, 8)
    assert need[0].tolist() == [True] + [False] * 7 and need[2].tolist() == [False] * 7 + [True]
    assert need[1].tolist() == [True, True, True, True, False, True, True, True]   # 160 belongs to rank 5: nobody picked 128..159
    need3 = ep.ranks_of(idx, 256, 3)   # 86 + 85 + 85 experts
    assert need3[0].tolist() == [True, False, False] and need3[1].tolist() == [True, True, True] and need3[2].tolist() == [False, False, True]
