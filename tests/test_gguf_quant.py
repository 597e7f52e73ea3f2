"""The GGUF block formats other than Q4_K on the host (moexb_gguf_dequant_host, moexb_gguf_row_to_zp): de-quantisation
against the reference's own fixture records (the values the gguf Python package gives for real blocks), and the 4-bit
zero-point refit byte for byte against gg_zp_row of the compiled reference (golden file, and live where oracle/_ref exists).
No GPU is used."""
import os
import struct

import numpy as np
import pytest

import moe_b200 as m
from oracle import oracle as o

BLOCK = {0: (1, 4), 1: (1, 2), 30: (1, 2), 8: (32, 34), 2: (32, 18), 20: (32, 18), 3: (32, 20), 6: (32, 22), 7: (32, 24),
         12: (256, 144), 13: (256, 176), 14: (256, 210), 23: (256, 136)}


def records(golden_dir):
    data = open(os.path.join(golden_dir, "gguf_blocks_subset.bin"), "rb").read()
    off = 0
    while off < len(data):
        t, n = struct.unpack_from("<II", data, off)
        bn, bb = BLOCK[t]
        raw = np.frombuffer(data, np.uint8, n // bn * bb, off + 8).copy()
        want = np.frombuffer(data, np.float32, n, off + 8 + raw.size).copy()
        off += 8 + raw.size + 4 * n
        yield t, n, raw, want


def test_dequantisation_matches_the_reference_fixture(lib_built, golden_dir):
    seen = set()
    for t, n, raw, want in records(golden_dir):
        assert np.array_equal(m.gguf_dequant_host(t, raw, n), want), f"ggml type {t}"
        if o.ref() is not None:
            assert np.array_equal(o.ref_gg_dequant(t, raw, n), want)
        seen.add(t)
    assert seen == set(BLOCK)
    with pytest.raises(m.MoexbError, match="not readable"):
        m.gguf_dequant_host(10, np.zeros(84, np.uint8), 256)      # Q2_K
    with pytest.raises(m.MoexbError, match="not readable"):
        m.gguf_dequant_host(14, np.zeros(210, np.uint8), 100)     # not a multiple of the block size


def test_zero_point_refit_is_byte_identical_to_the_reference(lib_built, golden_dir):
    gold = np.load(os.path.join(golden_dir, "gguf_zp_ref.npz"))
    for t, n, raw, want in records(golden_dir):
        if n % 256:
            continue
        qb, cs, sup = m.gguf_row_to_zp(t, raw, n)
        assert np.array_equal(qb, gold[f"qb{t}"]) and np.array_equal(cs, gold[f"cs{t}"]) and np.array_equal(sup, gold[f"sup{t}"]), f"ggml type {t}"
        # decoded back (gg_zp_at, gguf.h:332-335): Q4_K exactly, the others within the reference's own bound (relative RMS < 0.1)
        dec = np.array([o.zp_at(qb, cs, sup, i) for i in range(n)], np.float32)
        if t == 12:
            assert np.abs(dec - want).max() <= 1e-6 * np.abs(want).max()
        else:
            assert np.sqrt(((dec - want) ** 2).sum() / (want ** 2).sum()) < 0.1, f"ggml type {t}"


def test_refit_on_random_blocks_against_the_compiled_reference(lib_built):
    if o.ref() is None:
        pytest.skip("oracle/_ref is not built")
    rng = np.random.default_rng(6)
    for t, d_offsets in ((14, [208]), (13, [0, 2]), (23, [0]), (8, [0]), (20, [0])):
        bn, bb = BLOCK[t]
        cols = 2048
        b = rng.integers(0, 256, (cols // bn, bb), dtype=np.uint8)
        for off in d_offsets:
            b[:, off:off + 2] = rng.uniform(1e-3, 1e-2, cols // bn).astype(np.float16).view(np.uint8).reshape(-1, 2)
        raw = b.reshape(-1)
        qb, cs, sup = m.gguf_row_to_zp(t, raw, cols)
        rq, rc, rs = o.ref_gg_zp_row(t, raw, cols)
        assert np.array_equal(qb, rq) and np.array_equal(cs, rc) and np.array_equal(sup, rs), f"ggml type {t}"
