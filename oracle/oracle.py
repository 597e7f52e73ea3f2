"""ctypes wrappers of the CPU checker libraries - TEST INFRASTRUCTURE, not part of the product.

liboracle.so (oracle/_build, the plain-C restatement in oracle.c) and, when it was built, libmoex_ref.so (oracle/_ref,
the reference's own cpu_expert.h / gguf.h compiled from the reference tree). Only tests/, __graft_entry__.smoke() and
bench.py's CPU-baseline legs import this module.
"""
import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(HERE, "_build", "liboracle.so")
REF_SO = os.path.join(HERE, "_ref", "libmoex_ref.so")

EH, EI = 2048, 512
Q_BYTES = 3 * EH * EI // 2
CHUNKS = 3 * EH * EI // 32
FMT_SYM_F32, FMT_SYM_F16, FMT_ZP = 0, 1, 2


def build():
    """Compile oracle.c (always) and the reference driver (when the reference tree is present)."""
    r = subprocess.run(["make", "-C", HERE], capture_output=True, text=True)
    if r.returncode:
        raise RuntimeError("oracle build failed:\n" + r.stdout + r.stderr)


_orc = None
_ref = None


def _p(a):
    return a.ctypes.data_as(C.c_void_p) if a is not None else None


def orc():
    global _orc
    if _orc is None:
        if not os.path.exists(ORACLE_SO):
            build()
        _orc = C.CDLL(ORACLE_SO)
        _orc.orc_expert_bytes.restype = C.c_size_t
        _orc.orc_zp_at.restype = C.c_float
        _orc.orc_half.restype = C.c_float
        _orc.orc_group_pairs.restype = C.c_int
    return _orc


def ref():
    """The compiled reference, or None where it was not built."""
    global _ref
    if _ref is None and os.path.exists(REF_SO):
        _ref = C.CDLL(REF_SO)
        _ref.ref_gg_zp_at.restype = C.c_float
    return _ref


def expert_bytes(fmt):
    return orc().orc_expert_bytes(fmt)


def set_threads(n):
    """Threads of the OpenMP loops in liboracle.so (router logits, expert pairs), whatever OMP_NUM_THREADS says."""
    orc().orc_set_threads(int(n))


def synth_expert(fmt, seed, layer, expert):
    """The seeded synthetic expert (layer, expert) as a numpy uint8 blob: the same bytes as the product's generator."""
    out = np.empty(expert_bytes(fmt), np.uint8)
    assert orc().orc_synth_expert(fmt, C.c_uint(seed), layer, expert, _p(out)) == 0
    return out


def dequant(fmt, blob):
    out = np.empty(3 * EH * EI, np.float32)
    orc().orc_dequant(fmt, _p(blob), _p(out))
    return out


def q4k_dequant(blocks, n):
    y = np.empty(n, np.float32)
    orc().orc_q4k_dequant(_p(blocks), C.c_longlong(n), _p(y))
    return y


def q4k_to_zp_row(src, cols):
    qb = np.empty(cols // 2, np.uint8); cs = np.empty(cols // 32 * 2, np.uint8); sup = np.empty(cols // 256 * 2, np.uint16)
    orc().orc_q4k_to_zp_row(_p(src), cols, _p(qb), _p(cs), _p(sup))
    return qb, cs, sup


def q4k_to_zp(gate, up, down):
    blob = np.zeros(expert_bytes(FMT_ZP), np.uint8)
    orc().orc_q4k_to_zp(_p(gate), _p(up), _p(down), _p(blob))
    return blob


def zp_at(qb, cs, sup, i):
    return orc().orc_zp_at(_p(qb), _p(cs), _p(sup), i)


def router_logits(W, x, rows=1):
    """W [O][I] float32 or float16; x [rows][I] float32."""
    O, I = W.shape
    y = np.empty((rows, O), np.float32)
    x = np.ascontiguousarray(x, np.float32)
    orc().orc_router_logits(_p(np.ascontiguousarray(W)), int(W.dtype == np.float16), _p(x), _p(y), I, O, rows)
    return y


def router_topk(logits, E, K, norm=True, T=1, ld=None):
    ld = E if ld is None else ld
    idx = np.empty((T, K), np.int32); w = np.empty((T, K), np.float32)
    orc().orc_router_topk(_p(np.ascontiguousarray(logits, np.float32)), E, K, int(norm), _p(idx), _p(w), T, ld)
    return idx, w


def _jobs(jobs):
    """jobs: list of (blob, toks, pids, ws) -> flat arrays."""
    blobs = (C.c_void_p * len(jobs))(*[j[0].ctypes.data for j in jobs])
    start = np.zeros(len(jobs) + 1, np.int32)
    for i, j in enumerate(jobs):
        start[i + 1] = start[i] + len(j[1])
    toks = np.concatenate([np.asarray(j[1], np.int32) for j in jobs]) if jobs else np.zeros(0, np.int32)
    pids = np.concatenate([np.asarray(j[2], np.int32) for j in jobs]) if jobs else np.zeros(0, np.int32)
    ws = np.concatenate([np.asarray(j[3], np.float32) for j in jobs]) if jobs else np.zeros(0, np.float32)
    return blobs, start, toks, pids, ws


def run_pairs(fmt, jobs, X, npairs, want_act=False):
    """fp32 expert pairs (CpuExperts::run_pairs restated). Returns ypair [npairs][H] (and act [npairs][I])."""
    X = np.ascontiguousarray(X, np.float32)
    T = X.shape[0]
    blobs, start, toks, pids, ws = _jobs(jobs)
    ypair = np.zeros((npairs, EH), np.float32)
    act = np.zeros((npairs, EI), np.float32) if want_act else None
    orc().orc_run_pairs(fmt, len(jobs), blobs, _p(start), _p(toks), _p(pids), _p(ws), _p(X), T, npairs, _p(ypair), _p(act))
    return (ypair, act) if want_act else ypair


def pairs_reduce(ypair, K, T):
    moe = np.empty((T, EH), np.float32)
    orc().orc_pairs_reduce(_p(ypair), _p(moe), K, EH, T)
    return moe


def group_pairs(idx, w, E, held=None):
    """Returns (items [(e, start, count)], pair_t, pair_p, pair_w)."""
    T, K = idx.shape
    ie = np.empty(E, np.int32); st = np.empty(E, np.int32); ct = np.empty(E, np.int32)
    pt = np.empty(T * K, np.int32); pp = np.empty(T * K, np.int32); pw = np.empty(T * K, np.float32)
    h = None if held is None else np.ascontiguousarray(held, np.uint8)
    ni = orc().orc_group_pairs(_p(np.ascontiguousarray(idx, np.int32)), _p(np.ascontiguousarray(w, np.float32)), T, K, E,
                               _p(h), _p(ie), _p(st), _p(ct), _p(pt), _p(pp), _p(pw))
    n = int(st[ni - 1] + ct[ni - 1]) if ni else 0
    return [(int(ie[i]), int(st[i]), int(ct[i])) for i in range(ni)], pt[:n], pp[:n], pw[:n]


def rmsnorm(x, eps=1e-6):
    x = np.ascontiguousarray(x, np.float32)
    y = np.empty_like(x)
    orc().orc_rmsnorm(_p(x), _p(y), x.shape[-1], x.shape[0], C.c_float(eps))
    return y


def layer_forward(fmt, blobs, W, X, K=8, flags=0):
    """blobs: list of E+1 numpy blobs (None = not held). Returns (out [T][H], idx, w, logits [T][E+1])."""
    X = np.ascontiguousarray(X, np.float32)
    T, E = X.shape[0], len(blobs) - 1
    bp = (C.c_void_p * (E + 1))(*[(b.ctypes.data if b is not None else None) for b in blobs])
    out = np.empty((T, EH), np.float32); idx = np.empty((T, K), np.int32); w = np.empty((T, K), np.float32)
    logits = np.empty((T, E + 1), np.float32)
    W = np.ascontiguousarray(W)
    orc().orc_layer_forward(fmt, bp, _p(W), int(W.dtype == np.float16), _p(X), T, E, K, _p(out), _p(idx), _p(w), _p(logits), flags)
    return out, idx, w, logits


# ---- the compiled reference (oracle/_ref) ----------------------------------------------------------------------------

def ref_run_pairs(jobs, X, npairs, zp=False, threads=4):
    """CpuExperts::run_pairs of the reference; blobs in the reference layouts (FMT_SYM_F32 or FMT_ZP)."""
    X = np.ascontiguousarray(X, np.float32)
    blobs, start, toks, pids, ws = _jobs(jobs)
    ypair = np.zeros((npairs, EH), np.float32)
    ref().ref_run_pairs(threads, int(zp), len(jobs), blobs, _p(start), _p(toks), _p(pids), _p(ws), _p(X), X.shape[0], npairs, _p(ypair))
    return ypair


def ref_run_pairs_small(jobs, X, npairs, zp=False, threads=4):
    X = np.ascontiguousarray(X, np.float32)
    blobs, start, toks, pids, ws = _jobs(jobs)
    ypair = np.zeros((npairs, EH), np.float32)
    ref().ref_run_pairs_small(threads, int(zp), len(jobs), blobs, _p(start), _p(toks), _p(pids), _p(ws), _p(X), X.shape[0], _p(ypair))
    return ypair


def ref_run(blobs, w, x, zp=False, threads=4):
    """CpuExperts::run (int8 activations): out [H]."""
    bp = (C.c_void_p * len(blobs))(*[b.ctypes.data for b in blobs])
    out = np.empty(EH, np.float32)
    ref().ref_run(threads, int(zp), len(blobs), bp, _p(np.ascontiguousarray(w, np.float32)), _p(np.ascontiguousarray(x, np.float32)), _p(out))
    return out


def ref_gg_dequant(gg_type, raw, n):
    y = np.empty(n, np.float32)
    rc = ref().ref_gg_dequant(gg_type, _p(raw), C.c_longlong(n), _p(y))
    assert rc == 0
    return y


def ref_gg_zp_row(gg_type, src, cols):
    qb = np.empty(cols // 2, np.uint8); cs = np.empty(cols // 32 * 2, np.uint8); sup = np.empty(cols // 256 * 2, np.uint16)
    tmp = np.empty(cols, np.float32)
    ref().ref_gg_zp_row(gg_type, _p(src), cols, _p(qb), _p(cs), _p(sup), _p(tmp))
    return qb, cs, sup


def ref_gguf_tensor(path, name):
    """The reference's own GGUF reader (struct Gguf, gguf.h:345-462) on `path`: (shape, ggml type, file offset of the
    data or -1, bytes per row) of one tensor; None if absent; raises ValueError with the reader's message if it throws."""
    ne = (C.c_longlong * 4)(); ty = C.c_uint(0); off = C.c_longlong(0); rb = C.c_longlong(0)
    err = C.create_string_buffer(256)
    nd = ref().ref_gguf_tensor(os.fsencode(path), name.encode(), ne, C.byref(ty), C.byref(off), C.byref(rb), err, 256)
    if nd == -2:
        return None
    if nd < 0:
        raise ValueError(err.value.decode())
    return tuple(ne[:nd]), ty.value, off.value, rb.value


def sym_f16_to_f32(blob):
    """An FMT_SYM_F16 blob re-encoded as FMT_SYM_F32 (same values): the layout the reference's CPU code reads."""
    out = np.empty(Q_BYTES + CHUNKS // 2 * 4, np.uint8)
    out[:Q_BYTES] = blob[:Q_BYTES]
    out[Q_BYTES:] = blob[Q_BYTES:].view(np.float16).astype(np.float32).view(np.uint8)
    return out
