"""Generates the golden vectors under tests/golden/ from the reference itself. Run in a container that has the
reference tree (default /root/reference) and oracle/_ref built (make -C oracle):

    python tests/golden/make_golden.py

Outputs (all small, committed):
  q4k_fixture.bin      the Q4_K record of the reference's tests/gguf_blocks.bin (16 real super-blocks + the 4096 fp32
                       values the gguf Python package gives for them), same record framing: u32 type, u32 n, raw, f32
  gguf_blocks_subset.bin  the records of the same fixture for the block formats the loader reads (F32, F16, BF16, Q8_0, Q4_0,
                       Q4_1, Q5_0, Q5_1, Q4_K, Q5_K, Q6_K, IQ4_NL, IQ4_XS), same framing
  gguf_zp_ref.npz      gg_zp_row of the compiled reference on each of those records whose length is a multiple of 256
  q4k_zp_ref.npz       gg_zp_row(GG_Q4_K) of the compiled reference on that record: nibble bytes, [sc, mn], (d, dmin)
  run_pairs_ref.npz    CpuExperts::run_pairs / run_pairs_small / run of the compiled reference on seeded synthetic
                       experts (symmetric and zero-point), inputs included (X) or identified by CRC (blobs)
  dequant_ref.npz      dequant_expert() of the reference's ref/qwen36_ref.py on one synthetic expert (sampled values
                       and per-matrix sums)
  moe_ref.npz          Qwen36Ref.moe() of ref/qwen36_ref.py (fp32 torch, CPU) on a synthetic 32-expert layer: router
                       logits, selected ids, weights, layer output
"""
import os
import struct
import sys
import zlib

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
REF = os.environ.get("MOEX_REF", "/root/reference")
sys.path.insert(0, ROOT)

import moe_b200 as m  # noqa: E402  (host-side synthetic generator only; no GPU is used here)
from oracle import oracle as o  # noqa: E402

GG_Q4_K = 12


def q4k_record():
    with open(os.path.join(REF, "tests", "gguf_blocks.bin"), "rb") as f:
        data = f.read()
    sizes = {0: (1, 4), 1: (1, 2), 30: (1, 2), 8: (32, 34), 2: (32, 18), 20: (32, 18), 3: (32, 20), 6: (32, 22), 7: (32, 24),
             39: (32, 17), 10: (256, 84), 11: (256, 110), 23: (256, 136), 18: (256, 98), 21: (256, 110), 12: (256, 144),
             13: (256, 176), 14: (256, 210)}
    off = 0
    while off < len(data):
        t, n = struct.unpack_from("<II", data, off)
        bn, bb = sizes[t]
        raw_len = n // bn * bb
        if t == GG_Q4_K:
            return data[off:off + 8 + raw_len + 4 * n], n, raw_len
        off += 8 + raw_len + 4 * n
    raise SystemExit("no Q4_K record in the fixture")


READ_TYPES = (0, 1, 30, 8, 2, 3, 6, 7, 20, 12, 13, 14, 23)


def block_subset():
    """The fixture's records of READ_TYPES, and the reference's zero-point refit of each."""
    with open(os.path.join(REF, "tests", "gguf_blocks.bin"), "rb") as f:
        data = f.read()
    sizes = {0: (1, 4), 1: (1, 2), 30: (1, 2), 8: (32, 34), 2: (32, 18), 20: (32, 18), 3: (32, 20), 6: (32, 22), 7: (32, 24),
             39: (32, 17), 10: (256, 84), 11: (256, 110), 23: (256, 136), 18: (256, 98), 21: (256, 110), 12: (256, 144),
             13: (256, 176), 14: (256, 210)}
    off, out, zp = 0, b"", {}
    while off < len(data):
        t, n = struct.unpack_from("<II", data, off)
        bn, bb = sizes[t]
        raw_len = n // bn * bb
        if t in READ_TYPES:
            out += data[off:off + 8 + raw_len + 4 * n]
            if n % 256 == 0:
                raw = np.frombuffer(data, np.uint8, raw_len, off + 8).copy()
                qb, cs, sup = o.ref_gg_zp_row(t, raw, n)
                zp[f"qb{t}"], zp[f"cs{t}"], zp[f"sup{t}"] = qb, cs, sup
        off += 8 + raw_len + 4 * n
    open(os.path.join(HERE, "gguf_blocks_subset.bin"), "wb").write(out)
    np.savez_compressed(os.path.join(HERE, "gguf_zp_ref.npz"), **zp)


def main():
    assert o.ref() is not None, "oracle/_ref is not built: make -C oracle"
    block_subset()
    rec, n, raw_len = q4k_record()
    open(os.path.join(HERE, "q4k_fixture.bin"), "wb").write(rec)
    raw = np.frombuffer(rec, np.uint8, raw_len, 8).copy()
    qb, cs, sup = o.ref_gg_zp_row(GG_Q4_K, raw, n)
    np.savez_compressed(os.path.join(HERE, "q4k_zp_ref.npz"), qb=qb, cs=cs, sup=sup)

    # expert pairs through the compiled reference
    rng = np.random.default_rng(20240607)
    X = rng.standard_normal((3, 2048)).astype(np.float32)
    spec = [(0, [0, 2], [0, 4], [0.3, 0.2]), (1, [1, 2], [3, 5], [0.5, 0.25])]  # (expert, toks, pids, ws)
    out = {"X": X, "spec_expert": np.array([s[0] for s in spec]), "seed": 11, "layer": 2}
    for name, fmt, zp in (("sym", m.FMT_SYM_F32, False), ("zp", m.FMT_ZP, True)):
        blobs = [m.synth_expert_host(fmt, 11, 2, s[0]) for s in spec]
        jobs = [(b, s[1], s[2], s[3]) for b, s in zip(blobs, spec)]
        out[name + "_crc"] = np.array([zlib.crc32(b.tobytes()) for b in blobs], np.uint64)
        out[name + "_run_pairs"] = o.ref_run_pairs(jobs, X, 6, zp=zp)
        out[name + "_run_pairs_small"] = o.ref_run_pairs_small(jobs, X, 6, zp=zp)
        out[name + "_run"] = o.ref_run(blobs, [0.6, 0.4], X[0], zp=zp)
    np.savez_compressed(os.path.join(HERE, "run_pairs_ref.npz"), **out)

    # the Python reference: dequant_expert and moe()
    sys.path.insert(0, os.path.join(REF, "ref"))
    import torch
    import qwen36_ref as R
    H, I = 2048, 512
    blob = m.synth_expert_host(m.FMT_SYM_F32, 7, 1, 5)
    g, u, d = R.dequant_expert(torch.from_numpy(blob[:m.Q_BYTES].copy()), torch.from_numpy(blob[m.Q_BYTES:].view(np.float32).copy()), H, I, 64)
    full = torch.cat([g.reshape(-1), u.reshape(-1), d.reshape(-1)]).numpy()
    pos = rng.integers(0, full.size, 16384)
    np.savez_compressed(os.path.join(HERE, "dequant_ref.npz"), seed=7, layer=1, expert=5, crc=np.uint64(zlib.crc32(blob.tobytes())), pos=pos,
                        val=full[pos], sums=np.array([g.double().sum().item(), u.double().sum().item(), d.double().sum().item()]),
                        abs_sums=np.array([g.double().abs().sum().item(), u.double().abs().sum().item(), d.double().abs().sum().item()]))

    E, K, T = 32, 8, 3
    blobs = [m.synth_expert_host(m.FMT_SYM_F32, 5, 0, e) for e in range(E + 1)]
    Wr = (rng.standard_normal((E + 1, H)) * 0.02).astype(np.float32)  # row E = the shared expert's gate vector
    Xm = rng.standard_normal((T, H)).astype(np.float32)

    def deq(b):
        return R.dequant_expert(torch.from_numpy(b[:m.Q_BYTES].copy()), torch.from_numpy(b[m.Q_BYTES:].view(np.float32).copy()), H, I, 64)

    sg, su, sd = deq(blobs[E])

    class Shim:  # the attributes Qwen36Ref.moe() reads
        c = {"topk": K}
        W = [{"mlp.gate.weight": torch.from_numpy(Wr[:E]), "mlp.shared_expert.gate_proj.weight": sg,
              "mlp.shared_expert.up_proj.weight": su, "mlp.shared_expert.down_proj.weight": sd,
              "mlp.shared_expert_gate.weight": torch.from_numpy(Wr[E:E + 1])}]
        routes = []
        mv = staticmethod(R.Qwen36Ref.mv)

        def expert(self, i, e):
            return deq(blobs[e])

    dumped = {}
    shim = Shim()
    outs = []
    with torch.no_grad():
        for t in range(T):
            d = {}
            outs.append(R.Qwen36Ref.moe(shim, 0, torch.from_numpy(Xm[t]), lambda k, v, d=d: d.__setitem__(k, v.clone())).numpy())
            for k, v in d.items():
                dumped.setdefault(k, []).append(v.numpy())
    np.savez_compressed(os.path.join(HERE, "moe_ref.npz"), seed=5, layer=0, E=E, K=K, Wr=Wr, X=Xm,
                        crc=np.array([zlib.crc32(b.tobytes()) for b in blobs], np.uint64),
                        router_logits=np.stack(dumped["router_logits"]), route_idx=np.stack(dumped["route_idx"]),
                        route_w=np.stack(dumped["route_w"]), moe_out=np.stack(outs))
    for f in sorted(os.listdir(HERE)):
        print(f, os.path.getsize(os.path.join(HERE, f)))


if __name__ == "__main__":
    main()
