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
            assert 0 <= t0 <= t1 <= n
        assert seen == list(range(n))
        assert sum(ep.shared_token_range(n, r, world)[1] - ep.shared_token_range(n, r, world)[0] for r in range(world)) == n
