"""CPU-side checks of the product: the library loads and exports the whole C ABI, argument errors are reported as
status codes with a message, and the host half of the synthetic generator is deterministic."""
import ctypes as C
import os
import re

import numpy as np
import pytest

import moe_b200 as m
from moe_b200 import _lib

pytestmark = pytest.mark.usefixtures("lib_built")
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    header = open(os.path.join(ROOT, "include", "moexb.h")).read()
    declared = set(re.findall(r"\b(moexb_[a-z0-9_]+)\s*\(", header))
    declared -= {"moexb_pair_item", "moexb_pair"}
    assert len(declared) >= 25
    L = m.lib()
    for name in sorted(declared):
        assert hasattr(L, name), f"{name} is declared in include/moexb.h but not exported"
    assert declared == set(_lib.SIGNATURES), "the ctypes table and the header disagree"
    assert L.moexb_version() >= 1


def test_expert_bytes_match_reference_constants():
    assert m.expert_bytes(m.FMT_SYM_F32) == 1769472   # EXPERT_BYTES_SYM, kernels.cuh:424
    assert m.expert_bytes(m.FMT_ZP) == 1818624        # EXPERT_BYTES_ZP, kernels.cuh:426
    assert m.expert_bytes(m.FMT_SYM_F16) == 1671168
    assert m.expert_bytes(7) == 0
    assert C.sizeof(m.PairItem) == 16 and C.sizeof(m.Pair) == 12   # kernels.cuh:688-689


def test_argument_errors_are_status_codes():
    L = m.lib()
    assert L.moexb_router_topk(None, 256, 8, 1, None, None, None, 1, 256) == -1
    assert b"null pointer" in L.moexb_last_error()
    buf = np.zeros(16, np.float32).ctypes.data
    assert L.moexb_router_topk(buf, 250, 8, 1, buf, buf, None, 1, 256) == -1   # E not a multiple of 32
    assert b"E=250" in L.moexb_last_error()
    assert L.moexb_gemv_f32(buf, buf, buf, 100, 4, None, 1) == -1              # I not a multiple of 128
    assert L.moexb_experts_forward(9, buf, buf, 8, buf, buf, buf, None, None) == -1
    assert b"format" in L.moexb_last_error()
    assert L.moexb_experts_forward(0, buf, buf, 17, buf, buf, buf, None, None) == -1
    assert L.moexb_q4k_dequant(buf, 100, buf, None) == -1
    with pytest.raises(m.MoexbError):
        _lib.check(-1)


def test_synthetic_experts_are_deterministic_and_distributed_as_specified():
    a = m.synth_expert_host(m.FMT_SYM_F16, 0, 0, 3)
    assert np.array_equal(a, m.synth_expert_host(m.FMT_SYM_F16, 0, 0, 3))
    assert not np.array_equal(a, m.synth_expert_host(m.FMT_SYM_F16, 0, 0, 4))
    assert not np.array_equal(a[:4096], m.synth_expert_host(m.FMT_SYM_F16, 0, 1, 3)[:4096])
    assert not np.array_equal(a[:4096], m.synth_expert_host(m.FMT_SYM_F16, 1, 0, 3)[:4096])
    nib = np.concatenate([a[:m.Q_BYTES] & 15, a[:m.Q_BYTES] >> 4])
    hist = np.bincount(nib, minlength=16) / nib.size
    assert np.abs(hist - 1 / 16).max() < 2e-3                    # uniform over [-8, 7]
    s = a[m.Q_BYTES:].view(np.float16).astype(np.float64)
    assert abs(s.mean() - 0.02 * np.sqrt(2 / np.pi)) < 2e-4      # |N(0, 0.02)|
    assert abs(np.sqrt((s ** 2).mean()) - 0.02) < 3e-4
    b = m.synth_expert_host(m.FMT_SYM_F32, 0, 0, 3)
    assert np.array_equal(b[:m.Q_BYTES], a[:m.Q_BYTES])
    assert np.array_equal(b[m.Q_BYTES:].view(np.float32), a[m.Q_BYTES:].view(np.float16).astype(np.float32))
    g, u, d = m.synth_q4k_host(0, 0, 3)
    dd = g.reshape(-1, 144)[:, :4].copy().view(np.float16).astype(np.float64)
    assert abs(dd.mean() - 0.01 * np.sqrt(2 / np.pi)) < 2e-4     # d, dmin = |N(0, 0.01)|


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "libmoexb.so"))
    with pytest.raises(m.MoexbError, match="no fallback"):
        _lib.lib()
