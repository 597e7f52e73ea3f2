"""Expert parallelism over the GPUs of one node: experts sharded across ranks, tokens owned by ranks, token all-to-all.

Rank r of R holds routed experts [r*E/R, (r+1)*E/R) of every layer plus the (replicated) router and shared expert, and owns
the tokens [r*T/R, (r+1)*T/R): it keeps their residual rows, normalises and routes them, runs the shared expert for them
and returns their outputs. Per layer two exchanges: dispatch (ids and weights of every token to every rank, the normalised
activation row to the ranks that hold one of the token's selected experts) and combine (one partial output row per token
and rank that ran one of its experts, back to the token's owner, who adds them in rank order).

`EPStack` is the product path: the exchanges are done by the library's own kernels through peer-mapped exchange buffers
(moexb_ep_*, no collective call); this module only passes the buffers' IPC handles between the processes.
`exchange_block` is the same protocol written out on host arrays over any torch.distributed backend, with the per-rank
compute injected - the CPU tests drive it with the oracle over gloo to pin the partitioning arithmetic.
`EPStackAllReduce` is the earlier form (every rank routes all tokens, one NCCL all-reduce of the partial outputs per layer),
kept as the fallback where peer mapping is unavailable and as the baseline the peer-memory exchange is measured against.
"""
import numpy as np
import torch
import torch.distributed as dist


def expert_range(n_experts, rank, world):
    """[first, first + count) of the routed experts rank holds (even split, remainder to the first ranks)."""
    base, rem = divmod(n_experts, world)
    first = rank * base + min(rank, rem)
    return first, base + (1 if rank < rem else 0)


def token_range(n_tokens, rank, world):
    """[t0, t1) of the tokens rank owns."""
    base, rem = divmod(n_tokens, world)
    t0 = rank * base + min(rank, rem)
    return t0, t0 + base + (1 if rank < rem else 0)


shared_token_range = token_range   # the owner of a token is also the rank that runs the shared expert for it


def ranks_of(idx, n_experts, world):
    """[T][world] bool: which ranks hold one of each token's selected experts."""
    idx = np.asarray(idx)
    out = np.zeros((idx.shape[0], world), bool)
    for r in range(world):
        f, c = expert_range(n_experts, r, world)
        out[:, r] = ((idx >= f) & (idx < f + c)).any(axis=1)
    return out


def exchange_block(x_own, T, n_experts, route_fn, partial_fn, shared_fn, group=None):
    """One residual block x_next = x + moe(norm(x)) for the tokens this rank owns, with the protocol of the peer-memory path
    on host arrays (numpy float32) and torch.distributed collectives.
      route_fn(x_own)            -> (xn_own [n][H], idx [n][K], w [n][K]): normalise and route the own tokens
      partial_fn(xn, idx, w, t)  -> [len(t)][H]: for the tokens t (absolute ids, rows of xn / idx / w [T]) the sum, in
                                    router-rank order, of the weighted outputs of the experts THIS rank holds
      shared_fn(xn_own, idx, w)  -> [n][H]: the gated shared expert for the own tokens
    Returns x_next for the own tokens."""
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    t0, t1 = token_range(T, rank, world)
    xn_own, idx_own, w_own = route_fn(x_own)
    H, K = xn_own.shape[1], idx_own.shape[1]
    # dispatch: every rank learns every token's ids and weights; activation rows go to the ranks that need them (here: all
    # rows are gathered and the ones a rank does not need are blanked, so that a wrong read shows up)
    parts = [None] * world
    dist.all_gather_object(parts, (xn_own, idx_own, w_own), group=group)
    xn = np.concatenate([p[0] for p in parts]); idx = np.concatenate([p[1] for p in parts]); w = np.concatenate([p[2] for p in parts])
    need = ranks_of(idx, n_experts, world)
    xn = np.where(need[:, rank:rank + 1], xn, np.nan).astype(np.float32)
    xn[t0:t1] = xn_own
    # experts: partial rows for the tokens that selected one of this rank's experts
    mine = np.nonzero(need[:, rank])[0]
    partial = partial_fn(xn, idx, w, mine) if len(mine) else np.zeros((0, H), np.float32)
    # combine: each partial row goes to the token's owner
    send = [None] * world
    for r in range(world):
        a, b = token_range(T, r, world)
        sel = (mine >= a) & (mine < b)
        send[r] = (mine[sel], partial[sel])
    recv = [None] * world
    for r in range(world):   # gather-to-owner, one owner at a time (gloo has no all-to-all)
        got = [None] * world if rank == r else None
        dist.gather_object(send[r], got, dst=r, group=group)
        if rank == r:
            recv = got
    acc = np.zeros((t1 - t0, H), np.float32)
    for s in range(world):   # fixed rank order
        toks, rows = recv[s]
        for t, row in zip(toks, rows):
            acc[t - t0] += row
    acc += shared_fn(xn_own, idx_own, w_own)
    return x_own + acc


class EPStack:
    """The layers of one rank as residual blocks (or one plain layer) with the token all-to-all done by the library's kernels
    over peer memory, captured as one CUDA graph per rank. run(X) takes the whole batch [T][H] on every rank and returns
    this rank's own rows."""

    def __init__(self, ctx, layers, T, K=8, x_dtype=torch.float32, group=None, residual=True):
        from . import api, _lib
        self.ctx, self.layers, self.T, self.K, self.group = ctx, layers, T, K, group
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        self.buf = api.ExchangeBuffer(T, K, world)
        handles = [None] * world
        dist.all_gather_object(handles, self.buf.handle, group=group)
        # every rank maps every other rank's buffer; if that fails anywhere (no peer access, IPC closed to this process) all
        # ranks learn of it and raise together, so that the caller can fall back as one
        err, ptrs = None, None
        try:
            ptrs = [self.buf.ptr if r == rank else self.buf.open_peer(handles[r]) for r in range(world)]
        except Exception as e:   # noqa: BLE001 - reported to every rank below
            err = f"rank {rank}: {e}"
        errs = [None] * world
        dist.all_gather_object(errs, err, group=group)
        if any(errs):
            self.buf.close()
            raise RuntimeError("peer mapping of the exchange buffers failed: " + "; ".join(e for e in errs if e))
        self.ep = api.EP(ctx, rank, world, T, K, layers[0].n_routed, ptrs)
        self.t0, self.n_own = self.ep.first_token, self.ep.n_own
        dist.barrier(group=group)   # every rank's buffer is mapped everywhere before the first store
        self.stack = self.ep.stack(layers, _lib.BF16 if x_dtype == torch.bfloat16 else _lib.F32, residual)
        self.out = torch.empty(self.n_own, 2048, device=torch.device("cuda", ctx.device), dtype=torch.float32)

    @property
    def kernel_count(self):
        return self.stack.kernel_count

    def run(self, X):
        return self.stack.run(X, self.out)

    def run_host(self, X_host, out_host):
        return self.stack.run_host(X_host, out_host)

    def close(self):
        torch.cuda.synchronize()
        dist.barrier(group=self.group)   # nobody unmaps a buffer a peer may still write
        self.stack.close(); self.ep.close(); self.buf.close()


def ep_block(x, partial_fn, group=None):
    """One residual block in the all-reduce form: x_next = x + all_reduce_sum(partial_fn(x)).
    partial_fn(x) -> this rank's partial MoE output [T][H] for the normalised, routed tokens."""
    part = partial_fn(x)
    dist.all_reduce(part, op=dist.ReduceOp.SUM, group=group)
    return x + part


class EPStackAllReduce:
    """The all-reduce form: every rank routes all T tokens, runs the pairs of its own experts, and one NCCL all-reduce per
    layer sums the partial outputs; kernels and all-reduces captured in one CUDA graph."""

    def __init__(self, ctx, layers, T, K=8, x_dtype=torch.float32, group=None, use_graph=True):
        self.ctx, self.layers, self.T, self.K, self.group = ctx, layers, T, K, group
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        self.sh0, self.sh1 = token_range(T, rank, world)
        dev = torch.device("cuda", ctx.device)
        self.x_in = torch.zeros(T, 2048, device=dev, dtype=x_dtype)
        self.x = torch.zeros(T, 2048, device=dev, dtype=torch.float32)
        self.part = torch.zeros(T, 2048, device=dev, dtype=torch.float32)
        self.graph = None
        if use_graph:
            # warm up (NCCL connections, lazy kernel attributes) on a side stream, then capture
            s = torch.cuda.Stream(device=dev)
            s.wait_stream(torch.cuda.current_stream(dev))
            with torch.cuda.stream(s):
                for _ in range(2):
                    self._step()
            torch.cuda.current_stream(dev).wait_stream(s)
            torch.cuda.synchronize(dev)
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph):
                self._step()

    def _step(self):
        from .api import ep_residual_norm
        n = len(self.layers)
        for l, L in enumerate(self.layers):
            # layer 0 reads the step's input (f32 or bf16) and normalises it; later layers find their normalised input in
            # the context, left there by the residual kernel of the layer before
            L.forward_ep(self.x_in if l == 0 else self.x, self.T, self.K, self.part, self.sh0, self.sh1, pre_normed=l > 0)
            dist.all_reduce(self.part, op=dist.ReduceOp.SUM, group=self.group)
            if l == 0:
                self.x.copy_(self.x_in)
            ep_residual_norm(self.ctx, self.layers[l + 1] if l + 1 < n else None, self.x, self.part, self.x, self.T)

    def run(self, X):
        self.x_in.copy_(X, non_blocking=True)
        if self.graph is not None:
            self.graph.replay()
        else:
            self._step()
        return self.x
