"""GGUF ingest: the file reader behind moexb_gguf_* (no GPU) against files written by tests/gguf_file.py and against the
reference's own reader compiled into oracle/_ref (struct Gguf, gguf.h:345-462; its test: tests/test_gguf.cpp:37-78 writes
a tiny file, reads it back, then cuts it short), and the load of a block's Q4_K expert tensors into a resident layer
(GPU), which must give the very bytes moexb_q4k_to_zp / the reference's gg_zp_row give."""
import numpy as np
import pytest

import moe_b200 as m
from oracle import oracle as o
from tests import gguf_file as gf

pytestmark = pytest.mark.usefixtures("lib_built")
EH, EI = m.EH, m.EI


def small_file(path, version=3, alignment=None, nested=False):
    rng = np.random.default_rng(5)
    a = rng.standard_normal((3, 64)).astype(np.float32)
    b = rng.standard_normal((2, 32)).astype(np.float16)
    q = rng.integers(0, 256, 2 * 512 // 256 * 144, dtype=np.uint8)  # 2 rows of 512 Q4_K values
    kv = [("general.architecture", gf.STR, "qwen35moe"), ("general.name", gf.STR, "tiny"),
          ("qwen35moe.block_count", gf.U32, 2), ("some.f32", gf.F32, 1.5), ("some.bool", gf.BOOL, 1),
          ("some.i64", gf.I64, -7), ("some.f64", gf.F64, 2.25),
          ("tokenizer.ggml.tokens", gf.ARR, (gf.STR, ["a", "bc", "", "def"])),
          ("tokenizer.ggml.token_type", gf.ARR, (gf.I32, [1, 2, 3, 4]))]
    if nested:  # an array of arrays: allowed by the format, not read by the reference's reader
        kv.append(("nested", gf.ARR, (gf.ARR, [(gf.U8, [1, 2]), (gf.STR, ["x"])])))
    tensors = [("blk.0.a.weight", (64, 3), gf.GGML_F32, a.tobytes()), ("blk.0.b.weight", (32, 2), gf.GGML_F16, b.tobytes()),
               ("blk.1.q.weight", (512, 2), gf.GGML_Q4_K, q.tobytes()), ("odd.type", (8,), 99, b"\1" * 8)]
    where = gf.write_gguf(path, kv, tensors, version=version, alignment=alignment)
    return tensors, where


@pytest.mark.parametrize("version,alignment", [(3, None), (2, None), (3, 64), (3, 4096)])
def test_reader_lists_every_tensor_with_its_bytes(tmp_path, version, alignment):
    path = str(tmp_path / "tiny.gguf")
    tensors, where = small_file(path, version, alignment, nested=True)
    g = m.Gguf(path)
    assert g.names() == [t[0] for t in tensors]
    whole = np.fromfile(path, np.uint8)
    for name, ne, ty, data in tensors:
        got_ty, got_ne, raw = g.tensor(name)
        assert (got_ty, got_ne) == (ty, tuple(ne))
        if ty == 99:
            assert raw is None  # listed, but a type whose block size is unknown has no data pointer
            continue
        assert raw.tobytes() == data
        assert where[name] % (alignment or 32) == 0
        assert whole[where[name]: where[name] + len(data)].tobytes() == data
    with pytest.raises(m.MoexbError, match="missing from the GGUF"):
        g.tensor("blk.9.nothing")
    g.close()


@pytest.mark.skipif(o.ref() is None, reason="oracle/_ref not built (reference tree absent)")
@pytest.mark.parametrize("alignment", [None, 256])
def test_reader_agrees_with_the_reference_reader(tmp_path, alignment):
    path = str(tmp_path / "tiny.gguf")
    tensors, where = small_file(path, 3, alignment)
    g = m.Gguf(path)
    base = None
    for name, ne, ty, data in tensors:
        ref = o.ref_gguf_tensor(path, name)
        got_ty, got_ne, raw = g.tensor(name)
        assert ref[0] == got_ne and ref[1] == got_ty
        if raw is None:
            assert ref[2] == -1
            continue
        assert ref[2] == where[name]
        # our pointer sits at the same offset of our own mapping
        base = raw.ctypes.data - where[name] if base is None else base
        assert raw.ctypes.data - base == ref[2]
        assert ref[3] * int(np.prod(ne[1:])) == len(data)
    assert o.ref_gguf_tensor(path, "blk.9.nothing") is None
    g.close()


def test_bad_files_are_refused_with_a_reason(tmp_path):
    path = str(tmp_path / "tiny.gguf")
    tensors, where = small_file(path)
    whole = open(path, "rb").read()

    def refused(data, match):
        p = str(tmp_path / "bad.gguf")
        open(p, "wb").write(data)
        with pytest.raises(m.MoexbError, match=match):
            m.Gguf(p)
        if o.ref() is not None:  # the reference reader refuses the same files
            with pytest.raises(ValueError):
                o.ref_gguf_tensor(p, "blk.0.a.weight")

    refused(b"GGUX" + whole[4:], "no GGUF magic")
    refused(whole[:4] + (1).to_bytes(4, "little") + whole[8:], "version 1")
    refused(whole[:60], "truncated")                      # inside the metadata
    first = min(where.values())
    refused(whole[: first - 40], "truncated|past the end")  # inside the tensor directory or its padding
    refused(whole[: where["blk.1.q.weight"] + 100], "past the end of the file")  # inside a tensor's data
    with pytest.raises(m.MoexbError, match="cannot open"):
        m.Gguf(str(tmp_path / "absent.gguf"))
    p = str(tmp_path / "align.gguf")
    gf.write_gguf(p, [("general.alignment", gf.U32, 48)], [("t", (4,), gf.GGML_F32, b"\0" * 16)])
    with pytest.raises(m.MoexbError, match="alignment 48"):
        m.Gguf(p)
    p = str(tmp_path / "rows.gguf")
    gf.write_gguf(p, [], [("t", (100,), gf.GGML_Q4_K, b"\0" * 144)])
    with pytest.raises(m.MoexbError, match="whole number of blocks"):
        m.Gguf(p)


# ---- a block's expert tensors into a resident layer (GPU) -------------------------------------------------------------

E_SMALL, SEED, BLOCK = 32, 21, 3


def random_blocks(rng, n_blocks, block_bytes, d_offsets, scale_range=None):
    """n_blocks blocks of random bytes with small positive fp16 values at the byte offsets of the block's d / dmin."""
    b = rng.integers(0, 256, (n_blocks, block_bytes), dtype=np.uint8)
    for off in d_offsets:
        b[:, off:off + 2] = (rng.uniform(1e-3, 1e-2, n_blocks).astype(np.float16)).view(np.uint8).reshape(n_blocks, 2)
    return b.reshape(-1)


def other_format_experts(rng):
    """Expert tensors of two distinct experts repeated to E_SMALL: gate as Q6_K (210-byte blocks, d at byte 208), up as Q5_K
    (176 bytes, d and dmin at 0 and 2), down as IQ4_XS (136 bytes, d at 0); and an F16 shared expert."""
    nb = EH * EI // 256
    reps = E_SMALL // 2
    gate = np.tile(random_blocks(rng, 2 * nb, 210, [208]), reps)
    up = np.tile(random_blocks(rng, 2 * nb, 176, [0, 2]), reps)
    down = np.tile(random_blocks(rng, 2 * nb, 136, [0]), reps)
    sh = [(rng.standard_normal(EH * EI) * 0.05).astype(np.float16).view(np.uint8) for _ in range(3)]
    return gate, up, down, sh[0], sh[1], sh[2]


@pytest.fixture(scope="module")
def expert_file(tmp_path_factory):
    """Block 3 of a GGUF with 32 routed Q4_K experts + a Q4_K shared expert, an F16 router and a BF16 shared gate vector;
    block 4 with the same experts but an F32 router and no shared tensors; block 5 with Q2_K-typed expert tensors (a type the
    loader does not read); block 6 with 32 experts in three other block formats - gate Q6_K, up Q5_K, down IQ4_XS - and an
    F16 shared expert, which the loader re-quantises to 4 bits."""
    path = str(tmp_path_factory.mktemp("gguf") / "experts.gguf")
    parts = [m.synth_q4k_host(SEED, BLOCK, e) for e in range(E_SMALL + 1)]
    stack = [np.concatenate([p[k] for p in parts[:E_SMALL]]) for k in range(3)]
    rng = np.random.default_rng(9)
    W = (rng.standard_normal((E_SMALL + 1, EH)) * 0.02).astype(np.float32)
    w16 = W[:E_SMALL].astype(np.float16)
    gate_bf16 = (W[E_SMALL].view(np.uint32) >> 16).astype(np.uint16)  # truncation: exact in bf16 by construction below
    W[E_SMALL] = (gate_bf16.astype(np.uint32) << 16).view(np.float32)
    tensors = []
    for blk, router, shared in ((BLOCK, w16, True), (BLOCK + 1, W[:E_SMALL], False)):
        p = f"blk.{blk}."
        tensors += [(p + "ffn_gate_exps.weight", (EH, EI, E_SMALL), gf.GGML_Q4_K, stack[0]),
                    (p + "ffn_up_exps.weight", (EH, EI, E_SMALL), gf.GGML_Q4_K, stack[1]),
                    (p + "ffn_down_exps.weight", (EI, EH, E_SMALL), gf.GGML_Q4_K, stack[2]),
                    (p + "ffn_gate_inp.weight", (EH, E_SMALL), gf.GGML_F16 if router.dtype == np.float16 else gf.GGML_F32, router.tobytes())]
        if shared:
            tensors += [(p + "ffn_gate_shexp.weight", (EH, EI), gf.GGML_Q4_K, parts[E_SMALL][0]),
                        (p + "ffn_up_shexp.weight", (EH, EI), gf.GGML_Q4_K, parts[E_SMALL][1]),
                        (p + "ffn_down_shexp.weight", (EI, EH), gf.GGML_Q4_K, parts[E_SMALL][2]),
                        (p + "ffn_gate_inp_shexp.weight", (EH,), gf.GGML_BF16, gate_bf16.tobytes())]
    p = f"blk.{BLOCK + 2}."
    q2 = np.zeros(EH * EI // 256 * 84 * E_SMALL, np.uint8)  # Q2_K blocks
    tensors += [(p + "ffn_gate_exps.weight", (EH, EI, E_SMALL), 10, q2), (p + "ffn_up_exps.weight", (EH, EI, E_SMALL), 10, q2),
                (p + "ffn_down_exps.weight", (EI, EH, E_SMALL), 10, q2)]
    p = f"blk.{BLOCK + 3}."
    mixed = other_format_experts(rng)
    tensors += [(p + "ffn_gate_exps.weight", (EH, EI, E_SMALL), 14, mixed[0]), (p + "ffn_up_exps.weight", (EH, EI, E_SMALL), 13, mixed[1]),
                (p + "ffn_down_exps.weight", (EI, EH, E_SMALL), 23, mixed[2]),
                (p + "ffn_gate_shexp.weight", (EH, EI), gf.GGML_F16, mixed[3]), (p + "ffn_up_shexp.weight", (EH, EI), gf.GGML_F16, mixed[4]),
                (p + "ffn_down_shexp.weight", (EI, EH), gf.GGML_F16, mixed[5]),
                (p + "ffn_gate_inp.weight", (EH, E_SMALL), gf.GGML_F32, W[:E_SMALL].tobytes()),
                (p + "ffn_gate_inp_shexp.weight", (EH,), gf.GGML_F32, W[E_SMALL].tobytes())]
    gf.write_gguf(path, [("general.architecture", gf.STR, "qwen35moe")], tensors)
    Wr = np.concatenate([w16.astype(np.float32), W[E_SMALL:]])  # what a layer holds after loading block 3
    return path, Wr, W


@pytest.fixture(scope="module")
def gctx():
    c = m.Context(0, max_tokens=64, max_experts=256, top_k=8)
    yield c
    c.close()


@pytest.mark.gpu
@pytest.mark.parametrize("layout", [m.LAYOUT_TILED, m.LAYOUT_REFERENCE])
def test_layer_loaded_from_a_gguf_block_holds_the_converted_bytes(gctx, expert_file, layout):
    import torch
    path, Wr, _ = expert_file
    g = m.Gguf(path)
    L = m.Layer(gctx, m.FMT_ZP, E_SMALL, router_dtype=m.F32, layout=layout)
    assert L.load_gguf(g, BLOCK) == 15
    for e in range(E_SMALL + 1):
        want = m.synth_expert_host(m.FMT_ZP, SEED, BLOCK, e)  # = moexb_q4k_to_zp of the same raw tensors
        assert np.array_equal(L.export_blob(e), want), f"expert {e}"
    # ... which is what the reference's importer makes of those rows (gg_zp_row, gguf.h:302-330)
    if o.ref() is not None:
        gate = m.synth_q4k_host(SEED, BLOCK, 7)[0]
        qb, cs, sup = o.ref_gg_zp_row(12, gate[: EH // 256 * 144], EH)
        assert np.array_equal(L.export_blob(7)[: EH // 2], qb)
    # the router rows arrive converted to the layer's dtype, the shared gate vector as the last row
    class Mem:
        __cuda_array_interface__ = {"shape": ((E_SMALL + 1) * EH,), "typestr": "<f4", "version": 2,
                                    "data": (m.lib().moexb_layer_router(L.h), False)}
    assert np.array_equal(torch.as_tensor(Mem(), device="cuda:0").cpu().numpy().reshape(E_SMALL + 1, EH), Wr)
    # and the layer computes what a layer filled by upload does
    X = torch.randn(5, EH, device="cuda:0")
    L2 = m.Layer(gctx, m.FMT_ZP, E_SMALL, router_dtype=m.F32, layout=layout)
    for e in range(E_SMALL + 1):
        L2.upload_blob(e, m.synth_expert_host(m.FMT_ZP, SEED, BLOCK, e))
    L2.set_router(Wr)
    assert torch.equal(L.forward(X, 5), L2.forward(X, 5))
    L.close(); L2.close(); g.close()


@pytest.mark.gpu
def test_gguf_load_of_a_slice_of_experts_and_refusals(gctx, expert_file):
    path, _, W = expert_file
    g = m.Gguf(path)
    # expert parallelism: a layer that holds experts 8..15 takes only those; block 4 has no shared tensors
    L = m.Layer(gctx, m.FMT_ZP, E_SMALL, first_local=8, n_local=8, router_dtype=m.F16)
    L.upload_blob(E_SMALL, m.synth_expert_host(m.FMT_ZP, 1, 1, 1))
    assert L.load_gguf(g, BLOCK + 1) == 1 | 4
    for e in (8, 15):
        assert np.array_equal(L.export_blob(e), m.synth_expert_host(m.FMT_ZP, SEED, BLOCK, e))
    assert np.array_equal(L.export_blob(E_SMALL), m.synth_expert_host(m.FMT_ZP, 1, 1, 1))  # shared expert left as it was
    with pytest.raises(m.MoexbError, match="not held"):
        L.export_blob(7)
    with pytest.raises(m.MoexbError, match="missing from the GGUF"):
        L.load_gguf(g, 9)
    with pytest.raises(m.MoexbError, match="cannot re-quantise"):
        L.load_gguf(g, BLOCK + 2)
    L.close()
    L = m.Layer(gctx, m.FMT_ZP, 64)
    with pytest.raises(m.MoexbError, match="not the one this layer needs"):
        L.load_gguf(g, BLOCK)
    L.close()
    L = m.Layer(gctx, m.FMT_SYM_F16, E_SMALL)
    with pytest.raises(m.MoexbError, match="MOEXB_FMT_ZP"):
        L.load_gguf(g, BLOCK)
    L.close(); g.close()


@pytest.mark.gpu
def test_gguf_block_in_other_formats_is_requantised_as_the_reference_does(gctx, expert_file):
    """Expert tensors that are not Q4_K (here Q6_K, Q5_K, IQ4_XS and an F16 shared expert) are re-quantised to 4 bits at load
    time by the per-32 least-squares refit: the loaded blobs hold, row for row, what moexb_gguf_row_to_zp gives - which is byte
    for byte what the reference's gg_zp_row gives - and the layer computes on them what the oracle computes on the same blobs."""
    import torch
    path, _, W = expert_file
    g = m.Gguf(path)
    L = m.Layer(gctx, m.FMT_ZP, E_SMALL, router_dtype=m.F32)
    assert L.load_gguf(g, BLOCK + 3) == 15
    blobs = [L.export_blob(e) for e in range(E_SMALL + 1)]
    assert np.array_equal(blobs[0], blobs[2]) and not np.array_equal(blobs[0], blobs[1])   # the file repeats two experts
    names = ("ffn_gate_exps.weight", "ffn_up_exps.weight", "ffn_down_exps.weight")
    for k, (name, cols, rows) in enumerate(zip(names, (EH, EH, EI), (EI, EI, EH))):
        ty, ne, raw = g.tensor(f"blk.{BLOCK + 3}.{name}")
        row_bytes = raw.size // (E_SMALL * rows)
        for e, r in ((0, 0), (1, rows - 1), (5, 17)):
            src = raw[(e * rows + r) * row_bytes:(e * rows + r + 1) * row_bytes]
            qb, cs, sup = m.gguf_row_to_zp(ty, src, cols)
            row = (0 if k == 0 else EI if k == 1 else 0) + r
            qoff = row * (EH // 2) if k < 2 else 2 * EI * (EH // 2) + row * (EI // 2)
            assert np.array_equal(blobs[e][qoff:qoff + cols // 2], qb), (name, e, r)
            if o.ref() is not None:
                rq, rc, rs = o.ref_gg_zp_row(ty, src, cols)
                assert np.array_equal(qb, rq) and np.array_equal(cs, rc) and np.array_equal(sup, rs), (name, e, r)
    X = np.random.default_rng(3).standard_normal((5, EH)).astype(np.float32)
    idx = torch.empty(5, 8, dtype=torch.int32, device="cuda:0")
    out = L.forward(torch.from_numpy(X).to("cuda:0"), 5, idx=idx).cpu().numpy()
    ref, ri, _, _ = o.layer_forward(m.FMT_ZP, blobs, W, X, 8)
    assert np.array_equal(idx.cpu().numpy(), ri)
    assert np.linalg.norm(out - ref) <= 1e-3 * np.linalg.norm(ref)
    L.close(); g.close()
