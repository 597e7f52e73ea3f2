"""A minimal writer of GGUF files (the published container layout, versions 2 and 3) for the ingest tests.

write_gguf(path, kv, tensors): kv = [(key, type_id, value)], tensors = [(name, ne, ggml_type, bytes)] with ne[0] the row
length. Returns {name: absolute file offset of the tensor's data}.
"""
import struct

U8, I8, U16, I16, U32, I32, F32, BOOL, STR, ARR, U64, I64, F64 = range(13)
_FMT = {U8: "<B", I8: "<b", U16: "<H", I16: "<h", U32: "<I", I32: "<i", F32: "<f", BOOL: "<B", U64: "<Q", I64: "<q", F64: "<d"}
GGML_F32, GGML_F16, GGML_Q4_K, GGML_BF16 = 0, 1, 12, 30


def _str(s):
    b = s.encode() if isinstance(s, str) else s
    return struct.pack("<Q", len(b)) + b


def _value(ty, v):
    if ty == STR:
        return _str(v)
    if ty == ARR:
        et, items = v
        return struct.pack("<IQ", et, len(items)) + b"".join(_value(et, x) for x in items)
    return struct.pack(_FMT[ty], v)


def write_gguf(path, kv, tensors, version=3, alignment=None):
    kv = list(kv)
    if alignment is not None:
        kv.append(("general.alignment", U32, alignment))
    align = alignment or 32
    head = b"GGUF" + struct.pack("<IQQ", version, len(tensors), len(kv))
    for k, ty, v in kv:
        head += _str(k) + struct.pack("<I", ty) + _value(ty, v)
    offs, pos = [], 0
    for _, _, _, data in tensors:
        offs.append(pos)
        pos = (pos + len(data) + align - 1) // align * align
    for (name, ne, ty, _), off in zip(tensors, offs):
        head += _str(name) + struct.pack("<I", len(ne)) + b"".join(struct.pack("<Q", d) for d in ne) + struct.pack("<IQ", ty, off)
    start = (len(head) + align - 1) // align * align
    where = {}
    with open(path, "wb") as f:
        f.write(head + b"\0" * (start - len(head)))
        for (name, _, _, data), off in zip(tensors, offs):
            f.seek(start + off)
            f.write(bytes(data))
            where[name] = start + off
        end = start + (offs[-1] + len(tensors[-1][3]) if tensors else 0)
        f.truncate(end)
    return where
