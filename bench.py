"""Benchmark of the MoE expert-FFN path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--only] [--impl ours|reference]

A step is one pass of a batch of synthetic tokens through the workload's MoE layers (router -> top-8 -> int4 experts ->
combine + shared expert), chained as residual blocks. One JSON line is printed by rank 0: the headline workload at the top
level and every other workload under "workloads", each with its own device-timed value, end-to-end value, roofline and
CPU baseline.

Workloads (shapes of the reference model: hidden 2048, 256 routed + 1 shared expert, intermediate 512, top-8):
  serve64      64 tokens (bf16) through 40 layers of i4_gs64 experts - batched decode serving (headline)
  decode1      1 token (f32) through 40 layers of i4_gs64 experts
  decode1_q4k  1 token (f32) through 40 layers of GGUF Q4_K experts (zero-point blobs)
  mtp4         4 tokens (f32) through 40 layers - speculative-verify batch
  prefill2048  2048 tokens (bf16) through 1 layer (the plain layer, no norm or residual around it)
Weights are seeded synthetic tensors generated on the device (17 GB for 40 layers, larger than L2, so every step streams
them from HBM); inputs are seeded normal tokens. With more than one GPU the same tokens are spread over the ranks (strong
scaling): serve64 is the headline and prefill2048 rides along under "workloads"; the one-token workloads stay on one GPU.

--impl reference times the reference's own CPU expert code (oracle/_ref, built from the reference tree; the C port in
oracle/ where that is absent) on the host cores, on a bounded sample of the same workload, without loading the CUDA library.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time
from concurrent.futures import ThreadPoolExecutor

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

EH, EI, E, K = 2048, 512, 256, 8
Q_BYTES = 3 * EH * EI // 2
WORKLOADS = {
    # name: (tokens, layers, expert format, input dtype, BASELINE config)
    "serve64": (64, 40, "sym_f16", "bf16", 4),
    "decode1": (1, 40, "sym_f16", "f32", 0),
    "decode1_q4k": (1, 40, "zp", "f32", 1),
    "mtp4": (4, 40, "sym_f16", "f32", 2),
    "prefill2048": (2048, 1, "sym_f16", "bf16", 3),
}
SEED = 0
# dram__bytes_read.sum + dram__bytes_write.sum over the algorithmic bytes of the roofline kernel, from the ncu captures
# summarised under profiles/ (gate/up kernel on a 2-layer case of serve64; the one-token stack kernel; the grouped GEMM)
TRAFFIC_RATIO = {"serve64": 1.01, "decode1": 1.015, "prefill2048": 1.105}


def router_weights(layer):
    """[E+1][H] f32 N(0, 0.02); row E is the shared expert's gate vector."""
    return (np.random.default_rng([SEED, layer, 1]).standard_normal((E + 1, EH)) * 0.02).astype(np.float32)


def tokens(T, step):
    return np.random.default_rng([SEED, step, 2]).standard_normal((T, EH)).astype(np.float32)


def to_bf16_values(x):
    """x rounded to bfloat16 (nearest even), as float32 - the values a bf16 input tensor holds."""
    u = np.ascontiguousarray(x, np.float32).view(np.uint32)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000).astype(np.uint32)
    return r.view(np.float32)


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        j = json.load(open(p))
        return float(j["hbm_gbs"]), float(j["bf16_tflops"]), "measured"
    return 6650.0, 1590.0, "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons of one GPU, sampled while the timed regions run."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.lines, self.proc = [], None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(index), "--query-gpu=" + self.Q, "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            pass

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 7 or not f[0].isdigit():
                continue
            sm.append(int(f[0])); mx.append(int(f[1]))
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons),
                "samples": len(sm)}


# ---- CPU arm: the reference's CPU expert path on the host cores ----------------------------------------------------------

def cpu_block(o, blobs, W, X, threads, use_ref, fmt):
    """One residual MoE block on the CPU. Router / top-k / grouping / combine from the C port (the reference has no CPU code
    for them); expert math by the compiled reference when oracle/_ref exists, with the entry point the reference's engine
    uses at that size: CpuExperts::run (decode, int8 activations) for one token, CpuExperts::run_pairs_small (int8
    activations, at most 9 tokens per expert) for a speculative-verify batch, CpuExperts::run_pairs (fp32) beyond."""
    T = X.shape[0]
    xn = o.rmsnorm(X)
    logits = o.router_logits(W, xn, T)
    idx, w = o.router_topk(logits, E, K, True, T, E + 1)
    if use_ref and T == 1:
        gate1 = 1.0 / (1.0 + np.exp(-logits[0, E]))
        # run() takes at most 8 experts per call (its member scratch, cpu_expert.h:266): the routed 8, then the shared one
        y = o.ref_run([blobs[e] for e in idx[0]], w[0], xn[0], zp=(fmt == o.FMT_ZP), threads=threads)
        y = y + o.ref_run([blobs[E]], np.array([gate1], np.float32), xn[0], zp=(fmt == o.FMT_ZP), threads=threads)
        return X + y[None, :]
    items, pt, pp, pw = o.group_pairs(idx, w, E)
    jobs = [(blobs[e], pt[s:s + c], pp[s:s + c], pw[s:s + c]) for e, s, c in items]
    gate = 1.0 / (1.0 + np.exp(-logits[:, E]))
    jobs.append((blobs[E], np.arange(T, dtype=np.int32), np.arange(T * K, T * K + T, dtype=np.int32), gate.astype(np.float32)))
    if use_ref and T <= 9:
        yp = o.ref_run_pairs_small(jobs, xn, T * (K + 1), zp=(fmt == o.FMT_ZP), threads=threads)
    elif use_ref:
        yp = o.ref_run_pairs(jobs, xn, T * (K + 1), zp=(fmt == o.FMT_ZP), threads=threads)
    else:
        yp = o.run_pairs(fmt, jobs, xn, T * (K + 1))
    return X + o.pairs_reduce(yp[:T * K], K, T) + yp[T * K:]


def reference_default_threads(cores):
    """The reference engine's own default for its CPU expert pool: clamp(hardware_concurrency / 2, 2, 8) (moex.cu:173)."""
    return max(2, min(8, cores // 2))


class CpuArm:
    """The CPU path of one workload on a bounded sample (sample_layers of its layers), blobs built by the checker library."""

    def __init__(self, workload, sample_layers):
        from oracle import oracle as o
        self.o = o
        self.T, self.NL, fmtname, xdt, _ = WORKLOADS[workload]
        self.use_ref = o.ref() is not None
        # the reference's CPU code reads f32 group scales: the same values, widened
        self.fmt = o.FMT_ZP if fmtname == "zp" else (o.FMT_SYM_F32 if self.use_ref else o.FMT_SYM_F16)
        self.cores = os.cpu_count() or 1
        self.nl = min(sample_layers, self.NL)
        with ThreadPoolExecutor(self.cores) as ex:
            self.blobs = [list(ex.map(lambda e, l=l: o.synth_expert(self.fmt, SEED, l, e), range(E + 1))) for l in range(self.nl)]
        self.Ws = [router_weights(l) for l in range(self.nl)]
        X = tokens(self.T, 0)
        self.X = to_bf16_values(X) if xdt == "bf16" else X

    def one_pass(self, threads):
        self.o.set_threads(threads)
        t0 = time.perf_counter()
        x = self.X
        for l in range(self.nl):
            x = cpu_block(self.o, self.blobs[l], self.Ws[l], x, threads, self.use_ref, self.fmt)
        return time.perf_counter() - t0

    def timed(self, threads, warmup, reps):
        for _ in range(max(1, warmup)):   # the first pass warms the thread pools and page tables
            self.one_pass(threads)
        times = [self.one_pass(threads) for _ in range(reps)]
        return float(np.median(times))

    def experts_by(self):
        if not self.use_ref:
            return "the C port"
        fn = ("CpuExperts::run (int8 activations, the decode path)" if self.T == 1 else
              "CpuExperts::run_pairs_small (int8 activations, the speculative-verify path)" if self.T <= 9 else "CpuExperts::run_pairs (fp32)")
        return fn + " of the compiled reference"

    def report(self, sample_s, threads, reps):
        per_layer = sample_s / self.nl
        return {"value": self.T / (per_layer * self.NL), "unit": "tokens/s", "cores": threads, "kind": "reference" if self.use_ref else "port",
                "sample": f"{self.nl} of {self.NL} layers x {self.T} tokens, median of {reps} passes, {per_layer * 1e3:.2f} ms/layer, "
                          f"experts by {self.experts_by()}, router/top-k/combine by the C port; weights "
                          f"{self.nl * (E + 1) * self.o.expert_bytes(self.fmt) / 1e6:.0f} MB > L3"}


def cpu_baseline(workload, reps):
    """cpu_baseline object of a workload: all host cores, and the reference's own default thread count beside it. Timed in a
    process of its own - the reference arm of this file - because the reference's thread pool spin-waits on every core it
    was given, and this process's CUDA and torch threads would share those cores with it."""
    cmd = [sys.executable, os.path.abspath(__file__), "--impl", "reference", "--workload", workload, "--steps", str(reps), "--warmup", "3"]
    env = {k: v for k, v in os.environ.items() if k not in ("RANK", "WORLD_SIZE", "LOCAL_RANK", "OMP_NUM_THREADS")}
    r = subprocess.run(cmd, capture_output=True, text=True, env=env, timeout=600)
    lines = [ln for ln in r.stdout.splitlines() if ln.startswith("{")]
    if r.returncode or not lines:
        return {"value": None, "unit": "tokens/s", "cores": os.cpu_count(), "kind": "unavailable", "sample": (r.stderr or r.stdout)[-300:]}
    return json.loads(lines[-1])["cpu_baseline"]


def run_reference(args):
    if int(os.environ.get("RANK", "0")) != 0:
        return
    # idle OpenMP workers of the C port (router, top-k) must not spin on the cores the reference's own pool is about to use
    os.environ.setdefault("OMP_WAIT_POLICY", "passive")
    T, NL, fmtname, xdt, _ = WORKLOADS[args.workload]
    arm = CpuArm(args.workload, 2 if T <= 64 else 1)
    # each step of this arm is one pass over the bounded sample, on every host core (the thread count is set explicitly: a
    # launcher's OMP_NUM_THREADS does not apply)
    sample_s = arm.timed(arm.cores, args.warmup, max(1, args.steps))
    base = arm.report(sample_s, arm.cores, max(1, args.steps))
    dflt = reference_default_threads(arm.cores)
    if dflt != arm.cores:
        d = arm.report(arm.timed(dflt, 1, max(3, min(args.steps, 7))), dflt, max(3, min(args.steps, 7)))
        base["reference_default_threads"] = {"threads": dflt, "value": d["value"], "unit": "tokens/s", "rule": "clamp(cores / 2, 2, 8), moex.cu:173"}
    line = {"impl": "reference", "metric": "MoE int4 expert-FFN tokens/s", "value": base["value"], "unit": "tokens/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": sample_s * 1e3, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "step_is": f"one pass over the sample: {arm.nl} of {NL} layers; value = tokens / (ms_per_step / {arm.nl} * {NL})",
            "full_stack_ms_extrapolated": sample_s / arm.nl * NL * 1e3,
            "config": config_of(args.workload, args.gpus), "cpu_baseline": base,
            "e2e": {"value": base["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


def config_of(workload, n_gpus):
    T, NL, fmtname, xdt, cfg = WORKLOADS[workload]
    return {"workload": workload, "baseline_config": cfg, "tokens": T, "layers": NL, "experts": f"{E} routed + 1 shared, top-{K}", "hidden": EH,
            "intermediate": EI, "expert_format": {"sym_f16": "i4_gs64 (fp16 group scales)", "zp": "GGUF Q4_K as zero-point blobs"}[fmtname],
            "input_dtype": xdt, "router": "fp32",
            # expert weights a step reads: the experts its tokens select (at least K + 1 per layer), far more than the 126 MB of L2
            "l2": ("a step reads at least %.0f MB of expert weights from %.1f GB resident, more than L2; no flush needed"
                   % (NL * (K + 1) * 1.671168, NL * (E + 1) * 1.671168e-3)) if NL > 1 else "429 MB of layer weights exceed L2",
            "parallelism": "single GPU" if n_gpus == 1 else PARALLELISM.format(n=n_gpus, e=E // n_gpus)}


PARALLELISM = ("expert parallel over {n} GPUs: {e} routed experts and 1/{n} of the tokens per rank, router and shared expert "
               "replicated; per layer a token all-to-all each way (dispatch of activation rows, combine of partial rows) done by "
               "the library's kernels over peer-mapped memory, no collective call")


# ---- GPU arm -----------------------------------------------------------------------------------------------------------------

class Env:
    """What every workload of one process shares: torch, the library, the rank layout, the clock sampler."""

    def __init__(self, args):
        import torch
        import moe_b200 as m
        from moe_b200 import ep
        self.torch, self.m, self.ep, self.args = torch, m, ep, args
        self.rank, self.world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        self.dist = None
        if self.world > 1:
            import torch.distributed as dist
            dist.init_process_group("nccl", device_id=torch.device("cuda", self.local))
            self.dist = dist
        torch.cuda.set_device(self.local)
        self.dev = torch.device("cuda", self.local)
        self.first, self.count = ep.expert_range(E, self.rank, self.world)
        self.layer_sets = {}
        self.fallback = None   # set when the peer-memory exchange could not be set up and the all-reduce form ran instead

    def barrier(self):
        if self.dist:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def max_over_ranks(self, v):
        t = self.torch.tensor([v], device=self.dev, dtype=self.torch.float64)
        if self.dist:
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def layers(self, ctx_key, fmt, NL, max_tokens):
        """Layers (and their context) of one (format, token capacity): built once, shared by the workloads that fit."""
        key = (ctx_key, fmt, NL)
        if key not in self.layer_sets:
            m = self.m
            ctx = m.Context(self.local, max_tokens=max_tokens, max_experts=E, top_k=K)
            ctx.set_pairs_per_pass(self.args.pairs_per_pass)
            ls = []
            for l in range(NL):
                L = m.Layer(ctx, fmt, E, first_local=self.first, n_local=self.count)
                L.fill_synth(SEED, l)
                L.set_router(router_weights(l))
                ls.append(L)
            self.torch.cuda.synchronize()
            self.layer_sets[key] = (ctx, ls)
        return self.layer_sets[key]


def measure(env, workload, allreduce=False):
    """One workload on this process's GPU(s): device-timed throughput, end-to-end throughput, per-kernel roofline.
    allreduce: at more than one GPU take the all-reduce form of expert parallelism instead of the peer-memory exchange."""
    torch, m, args = env.torch, env.m, env.args
    T, NL, fmtname, xdt, _ = WORKLOADS[workload]
    world, rank, dev = env.world, env.rank, env.dev
    fmt = m.FMT_ZP if fmtname == "zp" else m.FMT_SYM_F16
    ctx, layers = env.layers("big" if T > 64 else "small", fmt, NL, max(T, 64))
    x_torch_dtype = torch.bfloat16 if xdt == "bf16" else torch.float32
    eps = None
    if world == 1:
        stack = m.Stack(ctx, layers, T, K, m.BF16 if xdt == "bf16" else m.F32, residual=NL > 1)
        kernel_count, out_rows = stack.kernel_count, T
    else:
        # expert parallel: every rank gets the whole batch, owns 1/world of the tokens and returns their rows; the step of a
        # rank (kernels, pushes into the peers' buffers, bounded waits on their flags) is one graph
        try:
            eps = None if allreduce else env.ep.EPStack(ctx, layers, T, K, x_torch_dtype, residual=NL > 1)
        except RuntimeError as e:   # raised on every rank together: peer mapping is not available here
            env.fallback = f"all-reduce form ({e})"
            eps = None
        if eps is not None:
            kernel_count, out_rows = eps.kernel_count, eps.n_own

            class _S:  # the Stack interface on top of the expert-parallel step
                def run(self, X, out):
                    eps.stack.run(X, out)

                def run_host(self, Xh_, out_h_):
                    eps.stack.run_host(Xh_, out_h_)

                def close(self):
                    eps.close()
        else:
            old = env.ep.EPStackAllReduce(ctx, layers, T, K, x_torch_dtype)
            kernel_count, out_rows = 0, T

            class _S:  # every rank carries all T rows; one NCCL all-reduce per layer
                def run(self, X, out):
                    out.copy_(old.run(X))

                def run_host(self, Xh_, out_h_):
                    out_h_.copy_(old.run(Xh_), non_blocking=True)
                    torch.cuda.current_stream().synchronize()

                def close(self):
                    pass
        stack = _S()
    Xh = [torch.from_numpy(tokens(T, s % 8)).to(x_torch_dtype).pin_memory() for s in range(8)]
    Xd = [x.to(dev) for x in Xh]
    out = torch.empty(out_rows, EH, device=dev)
    out_h = torch.empty(out_rows, EH).pin_memory()

    # ---- device-resident throughput: inputs already in HBM ----
    env.barrier()   # the ranks start their first exchange together: a peer's flag wait is bounded to a second or two
    for s in range(args.warmup):
        stack.run(Xd[s % 8], out)
    env.barrier()
    l0 = m.launch_count()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for s in range(args.steps):
        stack.run(Xd[s % 8], out)
    ev1.record()
    env.barrier()
    launches = m.launch_count() - l0
    ms_step = env.max_over_ranks(ev0.elapsed_time(ev1)) / args.steps
    assert bool(torch.isfinite(out).all()), "non-finite output"
    status = ctx.status()
    if eps is not None and env.max_over_ranks(float(status != 0)) > 0:
        # a rank gave up waiting for a peer's flag: all ranks leave the peer-memory form together and measure the all-reduce form
        env.fallback = f"all-reduce form (peer exchange wait timed out, status {status} on rank {rank})"
        stack.close()
        return measure(env, workload, allreduce=True)
    assert status == 0, "a device-side wait timed out"

    # ---- end to end: host buffers through the C ABI, copies inside the timed region ----
    for s in range(args.warmup):
        stack.run_host(Xh[s % 8], out_h)
    env.barrier()
    t0 = time.perf_counter()
    for s in range(args.steps):
        stack.run_host(Xh[s % 8], out_h)
    env.barrier()
    e2e_ms = env.max_over_ranks((time.perf_counter() - t0) * 1e3 / args.steps)

    # ---- per-kernel durations (CUDA events around each kernel, direct launches) and the distinct experts per layer ----
    ctx.profile(True)
    idx = torch.empty(NL, T, K, dtype=torch.int32, device=dev)
    reps = 3
    bufs = [torch.empty(T, EH, device=dev), torch.empty(T, EH, device=dev)]
    sh0, sh1 = env.ep.shared_token_range(T, rank, world)
    for r in range(reps + 1):
        x = Xd[r % 8]
        for l, L in enumerate(layers):
            if world == 1:
                x = L.forward(x, T, K, out=bufs[l & 1], idx=idx[l], flags=2 if NL > 1 else 0)
            elif eps is None:
                part = L.forward_ep(x, T, K, bufs[l & 1], sh0, sh1, idx=idx[l])
                env.dist.all_reduce(part)
                x = x.float() + part
            else:
                if l == 0:
                    eps.ep.begin_step()
                eps.ep.dispatch(L, l, x if l == 0 else None, NL > 1)
                eps.ep.experts(L, l)
                eps.ep.read_routing(idx[l])
                if l == NL - 1:
                    eps.ep.finish(NL, out, NL > 1)
        if r == 0:
            ctx.profile_read()  # discard the first pass
    prof_ms, prof_n = ctx.profile_read()
    ctx.profile(False)
    first, count = env.first, env.count

    def local(ix):  # the routed experts this rank holds
        return ix[(ix >= first) & (ix < first + count)]
    distinct = float(np.mean([len(torch.unique(local(idx[l]))) for l in range(NL)])) + 1  # + the shared expert
    # passes over expert weights: an expert with n tokens is streamed ceil(n / maxp) times (maxp pairs per sub-item)
    maxp = 128 if T >= 256 else args.pairs_per_pass if (T >= 8 and fmt != m.FMT_ZP) else 4
    passes = float(np.mean([int(torch.ceil(torch.bincount(local(idx[l].flatten()).long(), minlength=E) / maxp).sum()) for l in range(NL)])) + (sh1 - sh0 + maxp - 1) // maxp
    eb = m.expert_bytes(fmt)
    qb_gu, qb_dn = 2 * EI * EH // 2, EH * EI // 2
    sc_total = eb - m.Q_BYTES
    bytes_gu = distinct * (qb_gu + sc_total * 2 / 3) + T * EH * 4
    bytes_dn = distinct * (qb_dn + sc_total / 3)
    names = ["router", "topk", "group", "gate_up", "down", "combine", "other"]
    per_launch_us = {n: float(prof_ms[i] / max(1, prof_n[i]) * 1e3) for i, n in enumerate(names)}
    share = {n: float(prof_ms[i] / max(1e-9, prof_ms.sum())) for i, n in enumerate(names)}
    hbm_peak, tensor_peak, peak_kind = peaks()
    achieved = bytes_gu / (per_launch_us["gate_up"] * 1e-6) / 1e9
    ratio = TRAFFIC_RATIO.get(workload)
    layer_bytes = distinct * eb + (E + 1) * EH * 4 + 2 * T * EH * 4
    res = {
        "config": config_of(workload, world), "value": T / (ms_step * 1e-3), "unit": "tokens/s", "ms_per_step": ms_step,
        "e2e": {"value": T / (e2e_ms * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": Xh[0].numel() * Xh[0].element_size(),
                "d2h_bytes_per_step": T * EH * 4, "ms_per_step": e2e_ms},
        "gpu_launches": int(launches), "kernels_per_step": kernel_count,
        "roofline": {"bound": "hbm", "kernel": "gate_up (expert gate/up projection + SwiGLU)", "achieved": achieved, "peak": hbm_peak, "unit": "GB/s",
                     "frac": achieved / hbm_peak, "peak_kind": peak_kind, "traffic": ratio * bytes_gu if ratio and T > 1 else None,
                     "algorithmic_bytes_per_launch": bytes_gu,
                     "us_per_launch": per_launch_us["gate_up"], "distinct_experts_per_layer": distinct, "expert_passes_per_layer": passes,
                     "down": {"achieved": bytes_dn / (per_launch_us["down"] * 1e-6) / 1e9, "us_per_launch": per_launch_us["down"],
                              "algorithmic_bytes_per_launch": bytes_dn},
                     "whole_layer": {"algorithmic_bytes": layer_bytes, "us": ms_step * 1e3 / NL, "achieved": layer_bytes / (ms_step * 1e-3 / NL) / 1e9,
                                     "frac": layer_bytes / (ms_step * 1e-3 / NL) / 1e9 / hbm_peak},
                     "kernel_us_per_launch": per_launch_us, "kernel_time_share": share},
        "per_layer": {"us": ms_step * 1e3 / NL, "tokens_per_s": T / (ms_step * 1e-3 / NL)},
        "per_stack": {"layers": NL, "ms": ms_step, "tokens_per_s": T / (ms_step * 1e-3)},
    }
    r = res["roofline"]
    if T == 1 and world == 1 and kernel_count == 1:
        # the one-token stack is ONE cooperative kernel: its roofline is the whole step
        step_bytes = layer_bytes * NL
        r.update({"kernel": "decode_stack_k (all layers of the stack in one cooperative launch)", "achieved": step_bytes / (ms_step * 1e-3) / 1e9,
                  "algorithmic_bytes_per_launch": step_bytes, "us_per_launch": ms_step * 1e3,
                  "traffic": TRAFFIC_RATIO["decode1"] * step_bytes if workload == "decode1" else None,
                  "note": "kernel_us_per_launch below are the per-layer kernels of the multi-launch path, timed separately"})
        r["frac"] = r["achieved"] / r["peak"]
    if T >= 256:
        # the prefill chunk is a dense contraction: gate/up grouped GEMM against the measured cuBLAS bf16 burst figure
        npairs = int(sum(int(((idx[l] >= first) & (idx[l] < first + count)).sum()) for l in range(NL)) / NL) + (sh1 - sh0)
        flops_gu, flops_dn = 2.0 * npairs * EH * 2 * EI, 2.0 * npairs * EH * EI
        r.update({"bound": "tensor", "unit": "TFLOP/s", "achieved": flops_gu / (per_launch_us["gate_up"] * 1e-6) / 1e12, "peak": tensor_peak,
                  "algorithmic_flops_per_launch": flops_gu, "pairs_per_layer": npairs, "hbm_achieved_gbs": achieved, "hbm_frac": achieved / hbm_peak,
                  "note": "weights enter the tensor core as an exact fp16 hi + lo pair: 2 MMAs per weight tile (gate/up), 4 (down), so the "
                          "nominal-flop fraction cannot exceed 0.50 / 0.25 at full tensor-pipe activity"})
        r["frac"] = r["achieved"] / r["peak"]
        r["down"].update({"achieved": flops_dn / (per_launch_us["down"] * 1e-6) / 1e12, "algorithmic_flops_per_launch": flops_dn})
        r["whole_layer"].update({"flops": 1.5 * flops_gu + 2.0 * T * (E + 1) * EH,
                                 "tflops": (1.5 * flops_gu + 2.0 * T * (E + 1) * EH) / (ms_step * 1e-3 / NL) / 1e12})
    # the same fraction against the nominal figures (HBM3e 8 TB/s, dense bf16 2,250 TFLOP/s), for context
    r["nominal_peak"] = 2250.0 if r["unit"] == "TFLOP/s" else 8000.0
    r["frac_of_nominal"] = r["achieved"] / r["nominal_peak"]
    if workload == "serve64" and world == 1:
        res["independent_inputs"] = independent_inputs(env, ctx, layers, T, eb)
    stack.close()
    return res


def independent_inputs(env, ctx, layers, T, eb):
    """The chained synthetic stack routes less diversely than a real model would (its residual stream becomes dominated by
    the large synthetic expert outputs, so tokens pick similar experts). Beside it: the same 40 layers, each fed its own
    independent N(0, 1) batch - the per-layer calls captured in one graph - which routes like independent tokens do."""
    torch, args = env.torch, env.args
    NL = len(layers)
    xs = [torch.from_numpy(tokens(T, 100 + l)).to(env.dev) for l in range(NL)]
    bufs = [torch.empty(T, EH, device=env.dev), torch.empty(T, EH, device=env.dev)]
    idx = torch.empty(NL, T, K, dtype=torch.int32, device=env.dev)

    def step(with_idx):
        for l, L in enumerate(layers):
            L.forward(xs[l], T, K, out=bufs[l & 1], idx=idx[l] if with_idx else None, flags=2)
    step(True)
    torch.cuda.synchronize()
    distinct = float(np.mean([len(torch.unique(idx[l])) for l in range(NL)])) + 1
    s = torch.cuda.Stream(device=env.dev)
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        step(False)
    torch.cuda.current_stream().wait_stream(s)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        step(False)
    for _ in range(args.warmup):
        g.replay()
    torch.cuda.synchronize()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for _ in range(args.steps):
        g.replay()
    ev1.record()
    torch.cuda.synchronize()
    ms = ev0.elapsed_time(ev1) / args.steps
    layer_bytes = distinct * eb + (E + 1) * EH * 4 + 2 * T * EH * 4
    hbm_peak, _, _ = peaks()
    return {"what": "40 layers, each on its own independent N(0,1) batch of 64 tokens (no chaining), one graph", "ms_per_step": ms,
            "tokens_per_s": T / (ms * 1e-3), "distinct_experts_per_layer": distinct, "whole_layer_gbs": layer_bytes / (ms * 1e-3 / NL) / 1e9,
            "whole_layer_frac": layer_bytes / (ms * 1e-3 / NL) / 1e9 / hbm_peak}


def emulate_ranks(args):
    """The expert-parallel step with all ranks on ONE GPU (for profiling its kernels with a single-GPU tool): R contexts whose
    exchange buffers are each other's peers; the phases of a step are enqueued rank after rank, so that every flag a kernel
    waits for has been raised. Prints one JSON line with the step time of that serialised execution (not a throughput)."""
    import torch
    import moe_b200 as m
    from moe_b200 import ep
    R = args.emulate_ranks
    T, NL, fmtname, xdt, _ = WORKLOADS[args.workload]
    fmt = m.FMT_ZP if fmtname == "zp" else m.FMT_SYM_F16
    ctxs, layers, bufs, eps = [], [], [], []
    for r in range(R):
        c = m.Context(0, max_tokens=max(T, 64), max_experts=E, top_k=K)
        first, count = ep.expert_range(E, r, R)
        ls = []
        for l in range(NL):
            L = m.Layer(c, fmt, E, first_local=first, n_local=count)
            L.fill_synth(SEED, l); L.set_router(router_weights(l))
            ls.append(L)
        ctxs.append(c); layers.append(ls); bufs.append(m.ExchangeBuffer(T, K, R))
    for r in range(R):
        eps.append(m.EP(ctxs[r], r, R, T, K, E, [b.ptr for b in bufs]))
    X = torch.from_numpy(tokens(T, 0)).to(torch.bfloat16 if xdt == "bf16" else torch.float32).cuda()
    outs = [torch.zeros(e.n_own, EH, device="cuda") for e in eps]
    residual = NL > 1

    def step():
        for e in eps:
            e.begin_step()
        for l in range(NL):
            for r, e in enumerate(eps):
                e.dispatch(layers[r][l], l, X if l == 0 else None, residual)
            for r, e in enumerate(eps):
                e.experts(layers[r][l], l)
        for r, e in enumerate(eps):
            e.finish(NL, outs[r], residual)
    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    torch.cuda.synchronize()
    ms = (time.perf_counter() - t0) * 1e3 / args.steps
    print(json.dumps({"emulated_ranks": R, "workload": args.workload, "layers": NL, "ms_per_serialised_step": ms,
                      "status": [c.status() for c in ctxs], "finite": bool(all(torch.isfinite(o).all() for o in outs))}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="serve64", choices=sorted(WORKLOADS), help="the headline workload of the JSON line")
    ap.add_argument("--only", action="store_true", help="measure the headline workload alone (no \"workloads\" object)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--pairs-per-pass", type=int, default=8, choices=[4, 8], help="sub-item width of the streaming kernels")
    ap.add_argument("--layers", type=int, default=0, help="override the workload's layer count (small profiling cases)")
    ap.add_argument("--emulate-ranks", type=int, default=0, help="run the expert-parallel step with this many ranks emulated on one GPU (profiling aid)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.layers > 0:
        T_, _, f_, x_, c_ = WORKLOADS[args.workload]
        WORKLOADS[args.workload] = (T_, args.layers, f_, x_, c_)
    if args.impl == "reference":
        return run_reference(args)
    if args.emulate_ranks > 1:
        return emulate_ranks(args)

    env = Env(args)
    torch = env.torch
    sampler = ClockSampler(env.local) if env.rank == 0 else None
    head = measure(env, args.workload)
    others = {}
    if not args.only and not args.layers:
        names = [w for w in ("decode1", "decode1_q4k", "mtp4", "prefill2048", "serve64") if w != args.workload]
        if env.world > 1:
            names = [w for w in names if WORKLOADS[w][0] >= 64]   # the one-token and 4-token workloads stay on one GPU
        for w in names:
            others[w] = measure(env, w)
    clocks = sampler.stop() if sampler else None
    cpu_on = env.rank == 0 and env.world == 1 and not args.no_cpu_baseline
    if cpu_on:
        head["cpu_baseline"] = cpu_baseline(args.workload, 11)
        for w in others:
            others[w]["cpu_baseline"] = cpu_baseline(w, 11 if WORKLOADS[w][0] <= 64 else 5)
    line = {"metric": "MoE int4 expert-FFN tokens/s", "value": head["value"], "unit": "tokens/s", "n_gpus": env.world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": head["ms_per_step"], "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32 accumulate on int4 weights", "data": "synthetic", "config": head["config"],
            "e2e": head["e2e"], "gpu_launches": head["gpu_launches"], "roofline": head["roofline"], "clocks": clocks,
            "per_layer": head["per_layer"], "per_stack": head["per_stack"]}
    for k in ("cpu_baseline", "independent_inputs"):
        if k in head:
            line[k] = head[k]
    if env.fallback:
        line["config"]["parallelism"] += " - NOT USED in this run: " + env.fallback
    if others:
        line["workloads"] = others
    if env.rank == 0:
        print(json.dumps(line))
    if env.dist:
        # leave without tearing NCCL down under a live CUDA graph: everything has been measured and printed
        sys.stdout.flush()
        env.dist.barrier()
        torch.cuda.synchronize()
        os._exit(0)
    for ctx, layers in env.layer_sets.values():
        for L in layers:
            L.close()
        ctx.close()


if __name__ == "__main__":
    main()
