"""Benchmark of the MoE expert-FFN path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl ours|reference]

A step is one pass of a batch of synthetic tokens through the workload's MoE layers (router -> top-8 -> int4 experts ->
combine + shared expert), chained as residual blocks. One JSON line is printed by rank 0.

Workloads (shapes of the reference model: hidden 2048, 256 routed + 1 shared expert, intermediate 512, top-8):
  serve64      64 tokens (bf16) through 40 layers of i4_gs64 experts - batched decode serving (default)
  decode1      1 token (f32) through 40 layers of i4_gs64 experts
  decode1_q4k  1 token (f32) through 40 layers of GGUF Q4_K experts (zero-point blobs)
  mtp4         4 tokens (f32) through 40 layers - speculative-verify batch
  prefill2048  2048 tokens (bf16) through 1 layer (the plain layer, no norm or residual around it)
Weights are seeded synthetic tensors generated on the device (17 GB for 40 layers, larger than L2, so every step streams
them from HBM); inputs are seeded normal tokens.

--impl reference times the reference's own CPU expert code (oracle/_ref, built from the reference tree; the C port in
oracle/ where that is absent) on the host cores, on a bounded sample of the same workload.
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
WORKLOADS = {
    # name: (tokens, layers, expert format, input dtype)
    "serve64": (64, 40, "sym_f16", "bf16"),
    "decode1": (1, 40, "sym_f16", "f32"),
    "decode1_q4k": (1, 40, "zp", "f32"),
    "mtp4": (4, 40, "sym_f16", "f32"),
    "prefill2048": (2048, 1, "sym_f16", "bf16"),
}
SEED = 0


def router_weights(layer):
    """[E+1][H] f32 N(0, 0.02); row E is the shared expert's gate vector."""
    return (np.random.default_rng([SEED, layer, 1]).standard_normal((E + 1, EH)) * 0.02).astype(np.float32)


def tokens(T, step):
    return np.random.default_rng([SEED, step, 2]).standard_normal((T, EH)).astype(np.float32)


def measured_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        return float(json.load(open(p))["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def tensor_peak():
    """Dense bf16 TFLOP/s (the cuBLAS burst figure: the grouped GEMM is timed alone, kernel by kernel)."""
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        return float(json.load(open(p))["bf16_tflops"]), "measured"
    return 1590.0, "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons of one GPU, sampled while the timed region runs."""
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
    """One residual MoE block on the CPU: router / top-k / grouping / combine from the C port (the reference has no CPU
    code for them), expert math by the compiled reference when oracle/_ref exists: CpuExperts::run (its decode path, int8
    activations) for one token, CpuExperts::run_pairs (fp32) for a batch."""
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
    if use_ref:
        yp = o.ref_run_pairs(jobs, xn, T * (K + 1), zp=(fmt == o.FMT_ZP), threads=threads)
    else:
        yp = o.run_pairs(fmt, jobs, xn, T * (K + 1))
    return X + o.pairs_reduce(yp[:T * K], K, T) + yp[T * K:]


def cpu_arm(workload, sample_layers, reps):
    """tokens/s of the CPU path on a bounded sample (sample_layers layers of the stack, extrapolated to all layers)."""
    import moe_b200 as m
    from oracle import oracle as o
    T, NL, fmtname, _ = WORKLOADS[workload]
    use_ref = o.ref() is not None
    fmt = o.FMT_ZP if fmtname == "zp" else (o.FMT_SYM_F32 if use_ref else o.FMT_SYM_F16)  # the reference reads f32 scales
    cores = os.cpu_count() or 1
    nl = min(sample_layers, NL)
    with ThreadPoolExecutor(cores) as ex:
        blobs = [list(ex.map(lambda e, l=l: m.synth_expert_host(fmt, SEED, l, e), range(E + 1))) for l in range(nl)]
    Ws = [router_weights(l) for l in range(nl)]
    X = tokens(T, 0)
    if WORKLOADS[workload][3] == "bf16":
        import torch
        X = torch.from_numpy(X).to(torch.bfloat16).float().numpy()
    times = []
    for r in range(reps + 1):  # the first pass warms the thread pool and page tables
        t0 = time.perf_counter()
        x = X
        for l in range(nl):
            x = cpu_block(o, blobs[l], Ws[l], x, cores, use_ref, fmt)
        times.append(time.perf_counter() - t0)
    per_layer = float(np.median(times[1:])) / nl
    return {"value": T / (per_layer * NL), "unit": "tokens/s", "cores": cores, "kind": "reference" if use_ref else "port",
            "sample": f"{nl} of {NL} layers x {T} tokens, median of {reps} passes, {per_layer * 1e3:.2f} ms/layer, "
                      f"experts by {('CpuExperts::run (int8 activations, the decode path)' if T == 1 else 'CpuExperts::run_pairs (fp32)') + ' of the compiled reference' if use_ref else 'the C port'}, "
                      f"router/top-k/combine by the C port; weights {nl * (E + 1) * o.expert_bytes(fmt) / 1e6:.0f} MB > L3"}, per_layer


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    T, NL, fmtname, xdt = WORKLOADS[args.workload]
    sample_layers = 2 if T <= 64 else 1
    reps = max(1, args.steps)
    # each "step" of this arm is one pass over the bounded sample; warm-up passes are the first ones of cpu_arm
    base, per_layer = cpu_arm(args.workload, sample_layers, reps)
    line = {"impl": "reference", "metric": "MoE int4 expert-FFN tokens/s", "value": base["value"], "unit": "tokens/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": per_layer * NL * 1e3, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": config_of(args.workload, 1), "cpu_baseline": base,
            "e2e": {"value": base["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


def config_of(workload, n_gpus):
    T, NL, fmtname, xdt = WORKLOADS[workload]
    return {"workload": workload, "tokens": T, "layers": NL, "experts": f"{E} routed + 1 shared, top-{K}", "hidden": EH, "intermediate": EI,
            "expert_format": {"sym_f16": "i4_gs64 (fp16 group scales)", "zp": "GGUF Q4_K as zero-point blobs"}[fmtname],
            "input_dtype": xdt, "router": "fp32",
            # expert weights a step reads: the experts its tokens select (at least K + 1 per layer), far more than the 126 MB of L2
            "l2": ("a step reads at least %.0f MB of expert weights from %.1f GB resident, more than L2; no flush needed"
                   % (NL * (K + 1) * 1.671168, NL * (E + 1) * 1.671168e-3)) if NL > 1 else "429 MB of layer weights exceed L2",
            "parallelism": "single GPU" if n_gpus == 1 else f"expert parallel over {n_gpus} GPUs: {E // n_gpus} routed experts per rank, router and "
                           "shared expert replicated, one NCCL all-reduce of the partial outputs per layer"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="serve64", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--pairs-per-pass", type=int, default=8, choices=[4, 8], help="sub-item width of the streaming kernels")
    ap.add_argument("--layers", type=int, default=0, help="override the workload's layer count (small profiling cases)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.layers > 0:
        T_, _, f_, x_ = WORKLOADS[args.workload]
        WORKLOADS[args.workload] = (T_, args.layers, f_, x_)
    if args.impl == "reference":
        return run_reference(args)

    import torch
    import moe_b200 as m
    rank, world, local = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("LOCAL_RANK", "0"))
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    T, NL, fmtname, xdt = WORKLOADS[args.workload]
    fmt = m.FMT_ZP if fmtname == "zp" else m.FMT_SYM_F16
    ctx = m.Context(local, max_tokens=T, max_experts=E, top_k=K)
    ctx.set_pairs_per_pass(args.pairs_per_pass)
    from moe_b200 import ep
    first, count = ep.expert_range(E, rank, world)
    layers = []
    for l in range(NL):
        L = m.Layer(ctx, fmt, E, first_local=first, n_local=count)
        L.fill_synth(SEED, l)
        L.set_router(router_weights(l))
        layers.append(L)
    torch.cuda.synchronize()
    x_torch_dtype = torch.bfloat16 if xdt == "bf16" else torch.float32
    if world == 1:
        stack = m.Stack(ctx, layers, T, K, m.BF16 if xdt == "bf16" else m.F32, residual=NL > 1)
    else:
        # expert parallel: every rank sees the same tokens; the step is captured with its all-reduces in one graph
        eps = ep.EPStack(ctx, layers, T, K, x_torch_dtype)

        class _S:  # the Stack interface on top of the expert-parallel step
            kernel_count = 0

            def run(self, X, out):
                out.copy_(eps.run(X))

            def run_host(self, Xh_, out_h_):
                out_h_.copy_(eps.run(Xh_), non_blocking=True)
                torch.cuda.current_stream().synchronize()

            def close(self):
                pass
        stack = _S()
    Xh = [torch.from_numpy(tokens(T, s % 8)).to(x_torch_dtype).pin_memory() for s in range(8)]
    Xd = [x.to(dev) for x in Xh]
    out = torch.empty(T, EH, device=dev)
    out_h = torch.empty(T, EH).pin_memory()

    def barrier():
        if dist:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident throughput: inputs already in HBM ----
    for s in range(args.warmup):
        stack.run(Xd[s % 8], out)
    barrier()
    sampler = ClockSampler(local) if rank == 0 else None
    l0 = m.launch_count()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for s in range(args.steps):
        stack.run(Xd[s % 8], out)
    ev1.record()
    barrier()
    launches = m.launch_count() - l0
    ms = torch.tensor([ev0.elapsed_time(ev1)], device=dev)
    if dist:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms_step = float(ms.item()) / args.steps
    assert bool(torch.isfinite(out).all()), "non-finite output"

    # ---- end to end: host buffers through the C ABI, copies inside the timed region ----
    for s in range(args.warmup):
        stack.run_host(Xh[s % 8], out_h)
    barrier()
    t0 = time.perf_counter()
    for s in range(args.steps):
        stack.run_host(Xh[s % 8], out_h)
    barrier()
    e2e_ms = torch.tensor([(time.perf_counter() - t0) * 1e3 / args.steps], device=dev)
    if dist:
        dist.all_reduce(e2e_ms, op=dist.ReduceOp.MAX)
    clocks = sampler.stop() if sampler else None

    # ---- per-kernel durations (CUDA events around each kernel, direct launches) and the distinct experts per layer ----
    ctx.profile(True)
    idx = torch.empty(NL, T, K, dtype=torch.int32, device=dev)
    reps = 3
    bufs = [torch.empty(T, EH, device=dev), torch.empty(T, EH, device=dev)]
    sh0, sh1 = ep.shared_token_range(T, rank, world)
    for r in range(reps + 1):
        x = Xd[r % 8]
        for l, L in enumerate(layers):
            if world == 1:
                x = L.forward(x, T, K, out=bufs[l & 1], idx=idx[l], flags=2 if NL > 1 else 0)
            else:
                part = L.forward_ep(x, T, K, bufs[l & 1], sh0, sh1, idx=idx[l])
                dist.all_reduce(part)
                x = x.float() + part
        if r == 0:
            ctx.profile_read()  # discard the first pass
    prof_ms, prof_n = ctx.profile_read()
    ctx.profile(False)
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
    peak, peak_kind = measured_peak()
    achieved = bytes_gu / (per_launch_us["gate_up"] * 1e-6) / 1e9
    # DRAM traffic of the gate/up kernel: dram__bytes_read + dram__bytes_write of one ncu capture of this kernel on a
    # 2-layer case of the 64-token workload came to 1.015 x its algorithmic bytes; scaled here by the units processed
    traffic = 1.015 * bytes_gu if T <= 64 else None
    layer_bytes = distinct * eb + (E + 1) * EH * 4 + 2 * T * EH * 4
    tokens_total = T  # the same 64 tokens at every N: strong scaling
    line = {
        "metric": "MoE int4 expert-FFN tokens/s", "value": tokens_total / (ms_step * 1e-3), "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32 accumulate on int4 weights", "data": "synthetic",
        "config": config_of(args.workload, world),
        "e2e": {"value": tokens_total / (float(e2e_ms.item()) * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": Xh[0].numel() * Xh[0].element_size(),
                "d2h_bytes_per_step": out_h.numel() * 4, "ms_per_step": float(e2e_ms.item())},
        "gpu_launches": int(launches),
        "roofline": {"bound": "hbm", "kernel": "gate_up (expert gate/up projection + SwiGLU)", "achieved": achieved, "peak": peak, "unit": "GB/s",
                     "frac": achieved / peak, "peak_kind": peak_kind, "traffic": traffic, "algorithmic_bytes_per_launch": bytes_gu,
                     "us_per_launch": per_launch_us["gate_up"], "distinct_experts_per_layer": distinct, "expert_passes_per_layer": passes,
                     "down": {"achieved": bytes_dn / (per_launch_us["down"] * 1e-6) / 1e9, "us_per_launch": per_launch_us["down"],
                              "algorithmic_bytes_per_launch": bytes_dn},
                     "whole_layer": {"algorithmic_bytes": layer_bytes, "us": ms_step * 1e3 / NL, "achieved": layer_bytes / (ms_step * 1e-3 / NL) / 1e9,
                                     "frac": layer_bytes / (ms_step * 1e-3 / NL) / 1e9 / peak},
                     "kernel_us_per_launch": per_launch_us, "kernel_time_share": share},
        "clocks": clocks,
        "per_layer": {"us": ms_step * 1e3 / NL, "tokens_per_s": tokens_total / (ms_step * 1e-3 / NL)},
    }
    if T == 1 and world == 1 and stack.kernel_count == 1:
        # the one-token stack is ONE cooperative kernel: its roofline is the whole step
        r = line["roofline"]
        step_bytes = layer_bytes * NL
        r.update({"kernel": "decode_stack_k (all layers of the stack in one cooperative launch)", "achieved": step_bytes / (ms_step * 1e-3) / 1e9,
                  "algorithmic_bytes_per_launch": step_bytes, "us_per_launch": ms_step * 1e3,
                  # dram__bytes_read + dram__bytes_write of an ncu capture of this kernel on this workload: 1.003 x algorithmic
                  "traffic": 1.003 * step_bytes,
                  "note": "kernel_us_per_launch below are the per-layer kernels of the multi-launch path, timed separately"})
        r["frac"] = r["achieved"] / r["peak"]
    if T >= 256:
        # the prefill chunk is a dense contraction: gate/up grouped GEMM against the measured cuBLAS bf16 burst figure
        npairs = int(sum(int(((idx[l] >= first) & (idx[l] < first + count)).sum()) for l in range(NL)) / NL) + (sh1 - sh0)
        flops_gu, flops_dn = 2.0 * npairs * EH * 2 * EI, 2.0 * npairs * EH * EI
        tpeak = tensor_peak()
        r = line["roofline"]
        r.update({"bound": "tensor", "unit": "TFLOP/s", "achieved": flops_gu / (per_launch_us["gate_up"] * 1e-6) / 1e12, "peak": tpeak[0],
                  "peak_kind": tpeak[1], "algorithmic_flops_per_launch": flops_gu, "pairs_per_layer": npairs,
                  "hbm_achieved_gbs": achieved, "hbm_frac": achieved / peak})
        r["frac"] = r["achieved"] / r["peak"]
        r["down"].update({"achieved": flops_dn / (per_launch_us["down"] * 1e-6) / 1e12, "algorithmic_flops_per_launch": flops_dn})
        r["whole_layer"].update({"flops": 1.5 * flops_gu + 2.0 * T * (E + 1) * EH,
                                 "tflops": (1.5 * flops_gu + 2.0 * T * (E + 1) * EH) / (ms_step * 1e-3 / NL) / 1e12})
    # the same fraction against the nominal figures (HBM3e 8 TB/s, dense bf16 2,250 TFLOP/s), for context
    r_ = line["roofline"]
    r_["nominal_peak"] = 2250.0 if r_["unit"] == "TFLOP/s" else 8000.0
    r_["frac_of_nominal"] = r_["achieved"] / r_["nominal_peak"]
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"], _ = cpu_arm(args.workload, 2 if T <= 64 else 1, 3)
    if rank == 0:
        print(json.dumps(line))
    if dist:
        # leave without tearing NCCL down under a live CUDA graph: everything has been measured and printed
        sys.stdout.flush()
        dist.barrier()
        torch.cuda.synchronize()
        os._exit(0)
    stack.close()
    for L in layers:
        L.close()
    ctx.close()


if __name__ == "__main__":
    main()
