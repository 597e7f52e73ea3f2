"""Expert parallelism over the GPUs of one node: experts sharded across ranks, one all-reduce per layer.

Rank r of R holds routed experts [r*E/R, (r+1)*E/R) of every layer plus the (replicated) router and shared expert.
Every rank carries the whole residual stream x [T][H]: it normalises and routes all T tokens itself (router logits are
bit-identical everywhere, so all ranks agree on the routing without exchanging it), runs the (token, expert) pairs of
its own experts and the shared expert for its slice of the tokens, and the partial outputs are summed with one NCCL
all-reduce - the only exchange on the path. At decode sizes (64 tokens = 512 KB per layer) this costs one collective
launch per layer instead of the two of a dispatch/combine all-to-all.

The host logic here (which experts and which shared-expert tokens a rank owns, the per-layer exchange and residual)
is device-independent: `ep_block` takes the rank's partial-compute function, so the CPU tests drive it with the oracle
over gloo and the benchmark with the CUDA library over NCCL.
"""
import torch
import torch.distributed as dist


def expert_range(n_experts, rank, world):
    """[first, first + count) of the routed experts rank holds (even split, remainder to the first ranks)."""
    base, rem = divmod(n_experts, world)
    first = rank * base + min(rank, rem)
    return first, base + (1 if rank < rem else 0)


def shared_token_range(n_tokens, rank, world):
    """[t0, t1) of the tokens whose shared-expert output rank computes."""
    base, rem = divmod(n_tokens, world)
    t0 = rank * base + min(rank, rem)
    return t0, t0 + base + (1 if rank < rem else 0)


def ep_block(x, partial_fn, group=None):
    """One residual block under expert parallelism: x_next = x + all_reduce_sum(partial_fn(x)).
    partial_fn(x) -> this rank's partial MoE output [T][H] for the normalised, routed tokens."""
    part = partial_fn(x)
    dist.all_reduce(part, op=dist.ReduceOp.SUM, group=group)
    return x + part


class EPStack:
    """The layers of one rank chained as residual blocks, captured (kernels and all-reduces) in one CUDA graph."""

    def __init__(self, ctx, layers, T, K=8, x_dtype=torch.float32, group=None, use_graph=True):
        self.ctx, self.layers, self.T, self.K, self.group = ctx, layers, T, K, group
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        self.sh0, self.sh1 = shared_token_range(T, rank, world)
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
