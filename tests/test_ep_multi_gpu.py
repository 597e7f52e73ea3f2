"""The expert-parallel path on real peers: one process per GPU, exchange buffers mapped through CUDA IPC, each rank replaying
its own CUDA graph. Skipped with fewer than two GPUs. The ranks' outputs (their own tokens' rows) are checked against the
oracle chain; torch.distributed (gloo) only carries the IPC handles and the barriers."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
pytestmark = [pytest.mark.gpu, pytest.mark.usefixtures("lib_built")]


def _rank_main(rank, world, port, T, NL, q):
    sys.path.insert(0, ROOT); sys.path.insert(0, os.path.join(ROOT, "tests"))
    import torch.distributed as dist
    import moe_b200 as m
    from moe_b200 import ep
    from oracle import oracle as o
    from parity import check_ffn
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.cuda.set_device(rank)
    E, K, fmt = 32, 8, m.FMT_SYM_F16
    rng = np.random.default_rng(21)
    Ws = [(rng.standard_normal((E + 1, 2048)) * 0.02).astype(np.float32) for _ in range(NL)]
    ctx = m.Context(rank, max_tokens=T, max_experts=E, top_k=K)
    first, cnt = ep.expert_range(E, rank, world)
    layers = []
    for l in range(NL):
        L = m.Layer(ctx, fmt, E, first_local=first, n_local=cnt)
        L.fill_synth(9, l); L.set_router(Ws[l])
        layers.append(L)
    stack = ep.EPStack(ctx, layers, T, K, torch.float32)
    worst = 0.0
    for rep in range(3):
        X = np.random.default_rng(100 + rep).standard_normal((T, 2048)).astype(np.float32)
        got = stack.run(torch.from_numpy(X).to(f"cuda:{rank}")).cpu().numpy()
        x = X.copy()
        for l in range(NL):
            hosts = [m.synth_expert_host(fmt, 9, l, e) for e in range(E + 1)]
            moe, _, _, _ = o.layer_forward(fmt, hosts, Ws[l], o.rmsnorm(x), K)
            x = x + moe
        r = check_ffn(got, x[stack.t0:stack.t0 + stack.n_own], fmt, f"rank {rank} of {world}, replay {rep}", quiet=True)
        worst = max(worst, r[0])
    assert ctx.status() == 0
    q.put((rank, worst))
    stack.close()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_ranks_on_their_own_gpus_match_the_oracle(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29700 + world + os.getpid() % 200
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, 16, 3, q)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(300)
        assert p.exitcode == 0
    got = sorted(q.get(timeout=10) for _ in range(world))
    assert [g[0] for g in got] == list(range(world)) and all(g[1] <= 1e-3 for g in got)
