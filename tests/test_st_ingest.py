"""Safetensors container ingest: the reader behind moexb_st_* (no GPU) on files shaped like the reference engine's model
container (st.h:19-111: one file per layer, a flat JSON directory; moex.cu:933-939: an expert = `merged_weight` + `qs`),
and the load of a layer's experts and router from such a file into a resident layer (GPU)."""
import json
import struct

import numpy as np
import pytest

import moe_b200 as m

pytestmark = pytest.mark.usefixtures("lib_built")
EH, EI, Q_BYTES = m.EH, m.EI, m.Q_BYTES


def write_st(path, tensors, metadata=None, pad_to=8):
    """tensors = [(name, dtype, shape, bytes)] -> a safetensors file; returns {name: absolute offset}."""
    head, pos = {}, 0
    if metadata is not None:
        head["__metadata__"] = metadata
    for name, dtype, shape, data in tensors:
        head[name] = {"dtype": dtype, "shape": list(shape), "data_offsets": [pos, pos + len(data)]}
        pos += len(data)
    h = json.dumps(head, separators=(",", ":")).encode()
    h += b" " * (-len(h) % pad_to)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(h)) + h)
        for _, _, _, data in tensors:
            f.write(bytes(data))
    return {name: 8 + len(h) + head[name]["data_offsets"][0] for name, _, _, _ in tensors}


def test_reader_lists_every_tensor_with_its_bytes(tmp_path):
    rng = np.random.default_rng(2)
    a = rng.standard_normal((3, 5)).astype(np.float32)
    b = rng.integers(0, 256, 77, dtype=np.uint8)
    tensors = [("model.layers.0.a", "F32", (3, 5), a.tobytes()), ("model.layers.0.b", "U8", (77,), b.tobytes()),
               ("empty", "F16", (0, 4), b""), ("scalar", "I64", (), struct.pack("<q", 5))]
    path = str(tmp_path / "layer.safetensors")
    where = write_st(path, tensors, metadata={"format": "pt", "note": "{not a tensor}"})
    s = m.SafeTensors(path)
    assert s.names() == [t[0] for t in tensors]
    whole = open(path, "rb").read()
    for name, dtype, shape, data in tensors:
        got_dtype, got_shape, raw = s.tensor(name)
        assert (got_dtype, got_shape) == (dtype, tuple(shape))
        assert raw.tobytes() == data == whole[where[name]: where[name] + len(data)]
    with pytest.raises(m.MoexbError, match="missing tensor nothing"):
        s.tensor("nothing")
    s.close()


def test_bad_files_are_refused_with_a_reason(tmp_path):
    path = str(tmp_path / "ok.safetensors")
    write_st(path, [("t", "F32", (2,), b"\0" * 8)])
    whole = open(path, "rb").read()

    def refused(data, match):
        p = str(tmp_path / "bad.safetensors")
        open(p, "wb").write(data)
        with pytest.raises(m.MoexbError, match=match):
            m.SafeTensors(p)

    refused(whole[:5], "shorter than its header length")
    refused(struct.pack("<Q", 1 << 40) + whole[8:], "exceeds the file")
    refused(whole[:-4], "data offsets outside the file")                      # the tensor's bytes are cut short
    refused(whole[:8] + b"[" + whole[9:], "not a JSON object")
    refused(whole.replace(b'"data_offsets"', b'"data_offsetz"'), "data offsets outside the file")  # no offsets at all
    refused(whole.replace(b'"shape":[2]', b'"shape":[x]'), "not the JSON directory")
    refused(whole.replace(b"[0,8]", b"[8,0]"), "data offsets outside the file")
    with pytest.raises(m.MoexbError, match="cannot open"):
        m.SafeTensors(str(tmp_path / "absent.safetensors"))


# ---- a layer's experts into a resident layer (GPU) -------------------------------------------------------------------------

E_SMALL, SEED, LAYER = 32, 33, 2


def layer_file(path, fmt, scales_f16_exact=True):
    """A container file of layer 2: 32 experts as merged_weight + qs (the reference's names), the F16 router and the shared
    gate vector. fmt: the layout of the blobs the file's tensors are cut from (SYM_F32 or ZP)."""
    rng = np.random.default_rng(4)
    tensors, blobs = [], []
    for e in range(E_SMALL):
        if fmt == m.FMT_ZP:
            blob = m.synth_expert_host(m.FMT_ZP, SEED, LAYER, e)
            qs_dtype = "U8"
        else:
            b16 = m.synth_expert_host(m.FMT_SYM_F16, SEED, LAYER, e)
            scales = b16[Q_BYTES:].view(np.float16).astype(np.float32)
            if not scales_f16_exact and e == 5:
                scales[100] = np.float32(0.01)  # not an fp16 value
            blob = np.concatenate([b16[:Q_BYTES], scales.view(np.uint8)])
            qs_dtype = "F32"
        blobs.append(blob)
        p = f"model.layers.{LAYER}.mlp.experts.{e}."
        tensors += [(p + "merged_weight", "U8", (Q_BYTES,), blob[:Q_BYTES].tobytes()),
                    (p + "qs", qs_dtype, ((len(blob) - Q_BYTES) // (1 if qs_dtype == "U8" else 4),), blob[Q_BYTES:].tobytes())]
    W = (rng.standard_normal((E_SMALL + 1, EH)) * 0.02).astype(np.float16)
    tensors += [(f"model.layers.{LAYER}.mlp.gate.weight", "F16", (E_SMALL, EH), W[:E_SMALL].tobytes()),
                (f"model.layers.{LAYER}.mlp.shared_expert_gate.weight", "F16", (1, EH), W[E_SMALL:].tobytes())]
    write_st(path, tensors, metadata={"format": "pt"})
    return blobs, W


@pytest.fixture(scope="module")
def gctx():
    c = m.Context(0, max_tokens=64, max_experts=256, top_k=8)
    yield c
    c.close()


@pytest.mark.gpu
@pytest.mark.parametrize("file_fmt,layer_fmt", [(m.FMT_SYM_F32, m.FMT_SYM_F32), (m.FMT_SYM_F32, m.FMT_SYM_F16), (m.FMT_ZP, m.FMT_ZP)])
def test_layer_loaded_from_a_container_file_holds_its_bytes(gctx, tmp_path, file_fmt, layer_fmt):
    import torch
    path = str(tmp_path / "layer.safetensors")
    blobs, W = layer_file(path, file_fmt)
    s = m.SafeTensors(path)
    L = m.Layer(gctx, layer_fmt, E_SMALL, router_dtype=m.F16)
    shared = m.synth_expert_host(layer_fmt, SEED, LAYER, E_SMALL)
    L.upload_blob(E_SMALL, shared)
    assert L.load_st(s, f"model.layers.{LAYER}.") == 1 | 4 | 8
    for e in range(E_SMALL):
        want = blobs[e] if layer_fmt == file_fmt else m.synth_expert_host(m.FMT_SYM_F16, SEED, LAYER, e)
        assert np.array_equal(L.export_blob(e), want), f"expert {e}"
    assert np.array_equal(L.export_blob(E_SMALL), shared)  # the container holds the shared expert dense: left as it was
    # the same layer filled through the upload entry points computes the same
    L2 = m.Layer(gctx, layer_fmt, E_SMALL, router_dtype=m.F16)
    for e in range(E_SMALL + 1):
        L2.upload_blob(e, L.export_blob(e))
    L2.set_router(W)
    X = torch.randn(5, EH, device="cuda:0")
    assert torch.equal(L.forward(X, 5), L2.forward(X, 5))
    L.close(); L2.close(); s.close()


@pytest.mark.gpu
def test_container_load_refusals_and_a_slice_of_experts(gctx, tmp_path):
    path = str(tmp_path / "layer.safetensors")
    blobs, _ = layer_file(path, m.FMT_SYM_F32, scales_f16_exact=False)
    s = m.SafeTensors(path)
    L = m.Layer(gctx, m.FMT_SYM_F16, E_SMALL)
    with pytest.raises(m.MoexbError, match="is not an fp16 value"):
        L.load_st(s, f"model.layers.{LAYER}.")
    L.close()
    L = m.Layer(gctx, m.FMT_ZP, E_SMALL)
    with pytest.raises(m.MoexbError, match="not the scale part of this layer's expert format"):
        L.load_st(s, f"model.layers.{LAYER}.")
    L.close()
    L = m.Layer(gctx, m.FMT_SYM_F32, E_SMALL, first_local=16, n_local=16)  # one rank's experts of two
    assert L.load_st(s, f"model.layers.{LAYER}.") & 1
    assert np.array_equal(L.export_blob(16), blobs[16]) and np.array_equal(L.export_blob(31), blobs[31])
    with pytest.raises(m.MoexbError, match="missing tensor model.layers.7.mlp.experts.16.merged_weight"):
        L.load_st(s, "model.layers.7.")
    L.close(); s.close()
