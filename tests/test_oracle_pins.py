"""The CPU oracle (oracle/oracle.c) against the reference's own vectors: its GGUF fixture, outputs of its compiled CPU
code (oracle/_ref, committed as tests/golden/*.npz by tests/golden/make_golden.py) and outputs of its Python model."""
import os
import struct
import zlib

import numpy as np
import pytest

import moe_b200 as m
from oracle import oracle as o

pytestmark = pytest.mark.usefixtures("lib_built")


def relmax(got, ref):  # the reference's own metric: max abs error over the largest reference magnitude (test_kernels.cu:49-56)
    return float(np.abs(got.astype(np.float64) - ref).max() / (np.abs(ref).max() + 1e-30))


def load_q4k(golden_dir):
    rec = open(os.path.join(golden_dir, "q4k_fixture.bin"), "rb").read()
    t, n = struct.unpack_from("<II", rec, 0)
    assert t == 12 and n == 4096
    raw = np.frombuffer(rec, np.uint8, n // 256 * 144, 8).copy()
    want = np.frombuffer(rec, np.float32, n, 8 + raw.size).copy()
    return raw, want, n


def test_q4k_dequant_matches_reference_fixture(golden_dir):
    raw, want, n = load_q4k(golden_dir)
    got = o.q4k_dequant(raw, n)
    assert np.array_equal(got, want)  # the reference's own test allows 1e-6 of max (test_gguf.cpp:26); these agree bit for bit


def test_q4k_to_zero_point_matches_compiled_reference(golden_dir):
    raw, want, n = load_q4k(golden_dir)
    g = np.load(os.path.join(golden_dir, "q4k_zp_ref.npz"))
    qb, cs, sup = o.q4k_to_zp_row(raw, n)
    assert np.array_equal(qb, g["qb"]) and np.array_equal(cs, g["cs"]) and np.array_equal(sup, g["sup"])
    back = np.array([o.zp_at(qb, cs, sup, i) for i in range(n)], np.float32)
    assert np.array_equal(back, want)  # "Q4_K experts carried over exactly" (test_gguf.cpp:107)


def test_run_pairs_matches_compiled_reference(golden_dir):
    g = np.load(os.path.join(golden_dir, "run_pairs_ref.npz"))
    X = g["X"]
    spec = [(0, [0, 2], [0, 4], [0.3, 0.2]), (1, [1, 2], [3, 5], [0.5, 0.25])]
    for name, fmt in (("sym", m.FMT_SYM_F32), ("zp", m.FMT_ZP)):
        blobs = [m.synth_expert_host(fmt, int(g["seed"]), int(g["layer"]), s[0]) for s in spec]
        assert [zlib.crc32(b.tobytes()) for b in blobs] == list(g[name + "_crc"]), "synthetic inputs differ from the golden run"
        y = o.run_pairs(fmt, [(b, s[1], s[2], s[3]) for b, s in zip(blobs, spec)], X, 6)
        ref = g[name + "_run_pairs"]
        if name == "sym":
            assert np.array_equal(y, ref)
        else:
            assert relmax(y, ref) < 1e-6
        # the reference's int8-activation paths stay within its own 2e-2 bound of the fp32 path (test_kernels.cu:225, 336)
        assert relmax(g[name + "_run_pairs_small"], ref) < 2e-2
    # fp16 scales hold the same values as the widened f32 scales
    b16 = [m.synth_expert_host(m.FMT_SYM_F16, int(g["seed"]), int(g["layer"]), s[0]) for s in spec]
    y16 = o.run_pairs(m.FMT_SYM_F16, [(b, s[1], s[2], s[3]) for b, s in zip(b16, spec)], X, 6)
    assert np.array_equal(y16, g["sym_run_pairs"])


def test_dequant_matches_python_reference(golden_dir):
    g = np.load(os.path.join(golden_dir, "dequant_ref.npz"))
    blob = m.synth_expert_host(m.FMT_SYM_F32, int(g["seed"]), int(g["layer"]), int(g["expert"]))
    assert zlib.crc32(blob.tobytes()) == int(g["crc"])
    w = o.dequant(m.FMT_SYM_F32, blob)
    assert np.array_equal(w[g["pos"]], g["val"])
    n = m.EH * m.EI
    sums = [w[i * n:(i + 1) * n].astype(np.float64).sum() for i in range(3)]
    assert np.allclose(sums, g["sums"], rtol=0, atol=1e-6 * g["abs_sums"].max())
    # the fp16-scale blob dequantises to the same values
    assert np.array_equal(o.dequant(m.FMT_SYM_F16, m.synth_expert_host(m.FMT_SYM_F16, int(g["seed"]), int(g["layer"]), int(g["expert"]))), w)


def test_layer_matches_python_reference_moe(golden_dir):
    g = np.load(os.path.join(golden_dir, "moe_ref.npz"))
    E, K = int(g["E"]), int(g["K"])
    blobs = [m.synth_expert_host(m.FMT_SYM_F32, int(g["seed"]), int(g["layer"]), e) for e in range(E + 1)]
    assert [zlib.crc32(b.tobytes()) for b in blobs] == list(g["crc"])
    out, idx, w, logits = o.layer_forward(m.FMT_SYM_F32, blobs, g["Wr"], g["X"], K)
    assert np.array_equal(idx, g["route_idx"])                       # "top-8 ids" must be identical (test_kernels.cu:146)
    assert relmax(logits[:, :E], g["router_logits"]) < 1e-5          # the reference's bounds (test_kernels.cu:141, 148, 171)
    assert relmax(w, g["route_w"]) < 1e-5
    assert relmax(out, g["moe_out"]) < 1e-5


def test_zero_point_blob_of_synthetic_q4k(golden_dir):
    gate, up, down = m.synth_q4k_host(3, 1, 2)
    blob = o.q4k_to_zp(gate, up, down)
    assert np.array_equal(blob, m.synth_expert_host(m.FMT_ZP, 3, 1, 2))  # the product's converter, bit for bit
    w = o.dequant(m.FMT_ZP, blob)
    n = m.EH * m.EI
    assert np.array_equal(w[:n], o.q4k_dequant(gate, n))       # zero-point weights == GGUF dequantisation, bit for bit
    assert np.array_equal(w[2 * n:], o.q4k_dequant(down, n))


@pytest.mark.skipif(o.ref() is None, reason="oracle/_ref not built (reference tree absent)")
def test_live_against_compiled_reference():
    rng = np.random.default_rng(5)
    T = 5
    X = rng.standard_normal((T, 2048)).astype(np.float32)
    for fmt, zp in ((m.FMT_SYM_F32, False), (m.FMT_ZP, True)):
        blobs = [m.synth_expert_host(fmt, 9, 3, e) for e in range(3)]
        jobs, p = [], 0
        for b in blobs:
            toks = sorted(rng.choice(T, size=int(rng.integers(1, T + 1)), replace=False).tolist())
            jobs.append((b, toks, list(range(p, p + len(toks))), rng.uniform(0.05, 0.5, len(toks)).astype(np.float32)))
            p += len(toks)
        y, yr = o.run_pairs(fmt, jobs, X, p), o.ref_run_pairs(jobs, X, p, zp=zp)
        assert np.array_equal(y, yr) if not zp else relmax(y, yr) < 1e-6
    raw = rng.integers(0, 256, 144 * 8, dtype=np.uint8)
    raw.reshape(8, 144)[:, :4] = rng.uniform(1e-4, 1e-2, (8, 2)).astype(np.float16).view(np.uint8)
    assert np.array_equal(o.q4k_dequant(raw, 2048), o.ref_gg_dequant(12, raw, 2048))
    for a, b in zip(o.q4k_to_zp_row(raw, 2048), o.ref_gg_zp_row(12, raw, 2048)):
        assert np.array_equal(a, b)


def test_layer_against_float64_statement():
    """orc_layer_forward against a direct float64 statement of ref/qwen36_ref.py:201-220 on dequantised weights."""
    rng = np.random.default_rng(1)
    E, K, T = 32, 8, 2
    blobs = [m.synth_expert_host(m.FMT_SYM_F16, 2, 0, e) for e in range(E + 1)]
    W = (rng.standard_normal((E + 1, 2048)) * 0.02).astype(np.float32)
    X = rng.standard_normal((T, 2048)).astype(np.float32)
    out, idx, w, logits = o.layer_forward(m.FMT_SYM_F16, blobs, W, X, K)
    n = m.EH * m.EI
    for t in range(T):
        x = X[t].astype(np.float64)
        lg = W[:E].astype(np.float64) @ x
        p = np.exp(lg - lg.max()); p /= p.sum()
        top = np.argsort(-p, kind="stable")[:K]
        assert list(top) == list(idx[t])
        wt = p[top] / p[top].sum()
        assert np.allclose(wt, w[t], rtol=1e-5)
        acc = np.zeros(2048)

        def ffn(b):
            q = o.dequant(m.FMT_SYM_F16, b).astype(np.float64)
            gt, up, dn = q[:n].reshape(512, 2048), q[n:2 * n].reshape(512, 2048), q[2 * n:].reshape(2048, 512)
            a = gt @ x
            return dn @ (a / (1 + np.exp(-a)) * (up @ x))

        for e, ww in zip(top, wt):
            acc += ww * ffn(blobs[e])
        acc += ffn(blobs[E]) / (1 + np.exp(-(W[E].astype(np.float64) @ x)))
        assert relmax(out[t], acc) < 1e-5


def test_host_generator_of_the_checker_matches_the_product_generator(lib_built):
    """The benchmark's CPU arm builds its experts with the checker library alone; the bytes are the product's (whose device
    generator the GPU tests compare with its host generator)."""
    import moe_b200 as m
    for fmt in (o.FMT_SYM_F32, o.FMT_SYM_F16, o.FMT_ZP):
        for layer, e in ((0, 0), (39, 256), (7, 131)):
            assert np.array_equal(o.synth_expert(fmt, 5, layer, e), m.synth_expert_host(fmt, 5, layer, e)), (fmt, layer, e)
