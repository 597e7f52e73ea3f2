"""Host-side mirror of the reference's expert-layer entry points (src/kernels.cuh of the reference) on torch tensors.

Every function forwards to the C ABI with raw device pointers on torch's current stream; argument names and order
follow the reference functions named in include/moexb.h. Nothing here computes: without the CUDA library these raise.
"""
import ctypes as C
import os

import numpy as np
import torch

from . import _lib
from ._lib import EH, EI, F32, BF16, F16, check, lib


def _ptr(t):
    if t is None:
        return None
    if isinstance(t, torch.Tensor):
        assert t.is_cuda and t.is_contiguous(), "device-resident contiguous tensor expected"
        return t.data_ptr()
    return int(t)


def _stream():
    return torch.cuda.current_stream().cuda_stream


def expert_bytes(fmt):
    return lib().moexb_expert_bytes(fmt)


def gemv_f16(W, x, y=None, rows=1):
    """y[r] = W . x[r]; W [O][I] float16 (reference gemv_f16, kernels.cuh:93)."""
    O, I = W.shape
    y = torch.empty(rows, O, device=x.device, dtype=torch.float32) if y is None else y
    check(lib().moexb_gemv_f16(_ptr(W), _ptr(x), _ptr(y), I, O, _stream(), rows))
    return y


def gemv_f32(W, x, y=None, rows=1):
    O, I = W.shape
    y = torch.empty(rows, O, device=x.device, dtype=torch.float32) if y is None else y
    check(lib().moexb_gemv_f32(_ptr(W), _ptr(x), _ptr(y), I, O, _stream(), rows))
    return y


def router_topk(logits, E, K, norm=True, T=1, ld=None):
    """(idx [T][K] int32, w [T][K] f32) (reference router_topk, kernels.cuh:409)."""
    ld = E if ld is None else ld
    idx = torch.empty(T, K, device=logits.device, dtype=torch.int32)
    w = torch.empty(T, K, device=logits.device, dtype=torch.float32)
    check(lib().moexb_router_topk(_ptr(logits), E, K, int(norm), _ptr(idx), _ptr(w), _stream(), T, ld))
    return idx, w


def experts_forward(fmt, slots, w, K, x, act=None, out=None, nh=None):
    """One token through K experts (reference experts_forward, kernels.cuh:662). slots: int64 tensor of blob pointers."""
    act = torch.empty(K * EI, device=x.device, dtype=torch.float32) if act is None else act
    out = torch.empty(EH, device=x.device, dtype=torch.float32) if out is None else out
    check(lib().moexb_experts_forward(fmt, _ptr(slots), _ptr(w), K, _ptr(x), _ptr(act), _ptr(out), _stream(), _ptr(nh)))
    return out


def pairs_forward(fmt, items, n_items, pairs, X, act, ypair):
    """reference pairs_forward (kernels.cuh:767). items / pairs: uint8 tensors holding PairItem / Pair records."""
    check(lib().moexb_pairs_forward(fmt, _ptr(items), n_items, _ptr(pairs), _ptr(X), _ptr(act), _ptr(ypair), _stream()))
    return ypair


def pairs_forward_dev(fmt, items, nitems, max_items, pairs, X, act, ypair):
    check(lib().moexb_pairs_forward_dev(fmt, _ptr(items), _ptr(nitems), max_items, _ptr(pairs), _ptr(X), _ptr(act),
                                        _ptr(ypair), _stream()))
    return ypair


def pairs_reduce(ypair, ycpu, moe, K, D, T, use_cpu=None):
    check(lib().moexb_pairs_reduce(_ptr(ypair), _ptr(ycpu), _ptr(moe), K, D, T, _ptr(use_cpu), _stream()))
    return moe


def gated_add_rows(out, sh, gl, gl_stride, D, T):
    check(lib().moexb_gated_add_rows(_ptr(out), _ptr(sh), _ptr(gl), gl_stride, D, T, _stream()))
    return out


def shared_expert_add(fmt, blob, gl, gl_stride, X, T, out, scratch=None):
    if scratch is None:
        scratch = torch.empty(T * (EI + EH + 3) + 4, device=X.device, dtype=torch.float32)
    check(lib().moexb_shared_expert_add(fmt, _ptr(blob), _ptr(gl), gl_stride, _ptr(X), T, _ptr(out), _ptr(scratch), _stream()))
    return out


def group_pairs(idx, w, T, K, E, slot_table):
    """Device pair grouping; returns (items uint8 [E*16], pairs uint8 [T*K*12], nitems int32 [1])."""
    dev = idx.device
    items = torch.zeros(E * C.sizeof(_lib.PairItem), device=dev, dtype=torch.uint8)
    pairs = torch.zeros(T * K * C.sizeof(_lib.Pair), device=dev, dtype=torch.uint8)
    nitems = torch.zeros(1, device=dev, dtype=torch.int32)
    counts = torch.zeros(E, device=dev, dtype=torch.int32)
    check(lib().moexb_group_pairs(_ptr(idx), _ptr(w), T, K, E, _ptr(slot_table), _ptr(items), _ptr(pairs), _ptr(nitems),
                                  _ptr(counts), _stream()))
    return items, pairs, nitems


def dequant(fmt, blob):
    out = torch.empty(3 * EH * EI, device=blob.device, dtype=torch.float32)
    check(lib().moexb_dequant(fmt, _ptr(blob), _ptr(out), _stream()))
    return out


def q4k_dequant(blocks, n):
    y = torch.empty(n, device=blocks.device, dtype=torch.float32)
    check(lib().moexb_q4k_dequant(_ptr(blocks), n, _ptr(y), _stream()))
    return y


def q4k_to_zp(gate, up, down):
    blob = torch.empty(expert_bytes(_lib.FMT_ZP), device=gate.device, dtype=torch.uint8)
    check(lib().moexb_q4k_to_zp(_ptr(gate), _ptr(up), _ptr(down), _ptr(blob), _stream()))
    return blob


def gguf_dequant_host(ggml_type, raw, n):
    """moexb_gguf_dequant_host: n values of ggml-typed blocks (numpy uint8) as float32, on the CPU."""
    raw = np.ascontiguousarray(raw, np.uint8)
    y = np.empty(n, np.float32)
    check(lib().moexb_gguf_dequant_host(ggml_type, raw.ctypes.data, n, y.ctypes.data))
    return y


def gguf_row_to_zp(ggml_type, raw, cols):
    """moexb_gguf_row_to_zp: (nibble bytes, [sc, mn] bytes, (d, dm) fp16 bits) of one row, on the CPU."""
    raw = np.ascontiguousarray(raw, np.uint8)
    qb = np.empty(cols // 2, np.uint8); cs = np.empty(cols // 32 * 2, np.uint8); sup = np.empty(cols // 256 * 2, np.uint16)
    check(lib().moexb_gguf_row_to_zp(ggml_type, raw.ctypes.data, cols, qb.ctypes.data, cs.ctypes.data, sup.ctypes.data))
    return qb, cs, sup


def synth_expert_host(fmt, seed, layer, expert):
    """The synthetic expert (layer, expert) as a numpy uint8 blob; runs on the CPU."""
    out = np.empty(expert_bytes(fmt), dtype=np.uint8)
    check(lib().moexb_synth_expert_host(fmt, seed, layer, expert, out.ctypes.data))
    return out


def synth_q4k_host(seed, layer, expert):
    nb = EH * EI // 256 * 144
    g, u, d = (np.empty(nb, dtype=np.uint8) for _ in range(3))
    check(lib().moexb_synth_q4k_host(seed, layer, expert, g.ctypes.data, u.ctypes.data, d.ctypes.data))
    return g, u, d


class Context:
    """moexb_ctx: workspace of the layer-level calls on one device."""

    def __init__(self, device=0, max_tokens=64, max_experts=256, top_k=8):
        h = C.c_void_p()
        check(lib().moexb_ctx_create(device, max_tokens, max_experts, top_k, C.byref(h)))
        self.h, self.device, self.max_tokens, self.top_k = h, device, max_tokens, top_k

    def synth_experts(self, fmt, seed, layer, e0, n, dst):
        check(lib().moexb_synth_experts(self.h, fmt, seed, layer, e0, n, _ptr(dst), _stream()))

    def make_default(self, on=True):
        """moexb_set_default_ctx: the pointer-level one-token entry point (experts_forward) uses this context's workspace and
        runs the streaming kernels."""
        check(lib().moexb_set_default_ctx(self.h if on else None, self.device))

    def set_path(self, path):
        """0 = streaming tensor-core kernels (default), 1 = fp32 SIMT kernels."""
        check(lib().moexb_ctx_set_path(self.h, path))

    def set_prefill_min_tokens(self, tokens):
        check(lib().moexb_ctx_set_prefill_min_tokens(self.h, tokens))

    def set_fused_decode(self, on):
        check(lib().moexb_ctx_set_fused_decode(self.h, int(on)))

    def set_pairs_per_pass(self, pairs):
        check(lib().moexb_ctx_set_pairs_per_pass(self.h, pairs))

    def status(self):
        """Synchronises and returns the streaming kernels' error word (0 = fine)."""
        st = C.c_int(0)
        check(lib().moexb_ctx_status(self.h, C.byref(st)))
        return st.value

    def selftest_timeout(self, which, polls=4096):
        """moexb_ctx_selftest_timeout: lets one bounded device-side wait run out (0 = pipeline barrier, 1 = grid barrier)
        and returns the error word it leaves."""
        st = C.c_int(0)
        check(lib().moexb_ctx_selftest_timeout(self.h, which, polls, C.byref(st)))
        return st.value

    def pairs_forward_tc(self, fmt, items, n_items, pairs, X, T, npairs, act, ypair):
        """reference pairs_forward_tc (kernels.cuh:955) on the streaming kernels."""
        check(lib().moexb_pairs_forward_tc(self.h, fmt, _ptr(items), n_items, _ptr(pairs), _ptr(X), T, npairs, _ptr(act), _ptr(ypair), _stream()))
        return ypair

    def profile(self, on):
        check(lib().moexb_ctx_profile(self.h, int(on)))

    def profile_read(self):
        """(ms per tag, launches per tag) since the last read; tags as MOEXB_PROF_* in include/moexb.h."""
        ms = np.zeros(7, np.float32); n = np.zeros(7, np.int32)
        check(lib().moexb_ctx_profile_read(self.h, ms.ctypes.data, n.ctypes.data))
        return ms, n

    def close(self):
        if self.h:
            lib().moexb_ctx_destroy(self.h)
            self.h = None


class Gguf:
    """moexb_gguf: a GGUF model file mapped read-only, with its tensor directory (the reference's struct Gguf,
    gguf.h:345-462). Needs no GPU."""

    def __init__(self, path):
        h = C.c_void_p()
        check(lib().moexb_gguf_open(os.fsencode(path), C.byref(h)))
        self.h = h

    def names(self):
        return [lib().moexb_gguf_tensor_name(self.h, i).decode() for i in range(lib().moexb_gguf_tensor_count(self.h))]

    def tensor(self, name):
        """(ggml type, shape ne[0..n_dims-1] with ne[0] the row length, bytes as a numpy uint8 view of the mapping or
        None when the type's block size is unknown). The view is valid until close()."""
        ty, nd, nb, data = C.c_int(0), C.c_int(0), C.c_longlong(0), C.c_void_p()
        ne = (C.c_longlong * 4)()
        check(lib().moexb_gguf_tensor(self.h, name.encode(), C.byref(ty), C.byref(nd), ne, C.byref(data), C.byref(nb)))
        raw = None
        if data.value:
            raw = np.ctypeslib.as_array(C.cast(data, C.POINTER(C.c_uint8)), shape=(nb.value,))
        return ty.value, tuple(ne[: nd.value]), raw

    def close(self):
        if self.h:
            lib().moexb_gguf_close(self.h)
            self.h = None


class SafeTensors:
    """moexb_st: one safetensors file of the reference engine's model container, mapped read-only (the reference's
    struct Container, st.h:19-111). Needs no GPU."""

    def __init__(self, path):
        h = C.c_void_p()
        check(lib().moexb_st_open(os.fsencode(path), C.byref(h)))
        self.h = h

    def names(self):
        return [lib().moexb_st_tensor_name(self.h, i).decode() for i in range(lib().moexb_st_tensor_count(self.h))]

    def tensor(self, name):
        """(dtype string, shape, bytes as a numpy uint8 view of the mapping, valid until close())."""
        dt = C.create_string_buffer(8)
        nd, nb, data = C.c_int(0), C.c_longlong(0), C.c_void_p()
        shape = (C.c_longlong * 8)()
        check(lib().moexb_st_tensor(self.h, name.encode(), dt, C.byref(nd), shape, C.byref(data), C.byref(nb)))
        raw = np.empty(0, np.uint8)
        if nb.value:
            raw = np.ctypeslib.as_array(C.cast(data, C.POINTER(C.c_uint8)), shape=(nb.value,))
        return dt.value.decode(), tuple(shape[: nd.value]), raw

    def close(self):
        if self.h:
            lib().moexb_st_close(self.h)
            self.h = None


class Layer:
    """moexb_layer: one MoE layer resident in HBM (routed experts [first_local, first_local+n_local), shared expert,
    router with the shared gate vector as its last row)."""

    def __init__(self, ctx, fmt, n_routed=256, first_local=0, n_local=None, router_dtype=F32, layout=_lib.LAYOUT_TILED):
        n_local = n_routed - first_local if n_local is None else n_local
        h = C.c_void_p()
        check(lib().moexb_layer_create(ctx.h, fmt, n_routed, first_local, n_local, router_dtype, layout, C.byref(h)))
        self.layout = layout
        self.h, self.ctx, self.fmt, self.n_routed, self.router_dtype = h, ctx, fmt, n_routed, router_dtype
        self.first_local, self.n_local = first_local, n_local

    def blob_ptr(self, e):
        return lib().moexb_layer_blob(self.h, e)

    def slot_table(self):
        return lib().moexb_layer_slot_table(self.h)

    def set_router(self, W):
        """W: numpy [n_routed+1][H], float32 or float16 matching router_dtype."""
        W = np.ascontiguousarray(W, dtype=np.float32 if self.router_dtype == F32 else np.float16)
        assert W.shape == (self.n_routed + 1, EH)
        check(lib().moexb_layer_set_router(self.h, W.ctypes.data))

    def fill_synth(self, seed, layer_index):
        check(lib().moexb_layer_fill_synth(self.h, seed, layer_index, _stream()))

    def load_gguf(self, gguf, block):
        """moexb_layer_load_gguf: block `block` of an open Gguf into this MOEXB_FMT_ZP layer. Returns the bit set of
        what the file provided (1 routed experts, 2 shared expert, 4 router rows, 8 shared gate vector)."""
        got = C.c_int(0)
        check(lib().moexb_layer_load_gguf(self.h, gguf.h, block, C.byref(got)))
        return got.value

    def load_st(self, st, prefix):
        """moexb_layer_load_st: the experts and router of `prefix` ("model.layers.<l>.") from an open SafeTensors file.
        Returns the bit set of what the file provided (1 routed experts, 4 router rows, 8 shared gate vector)."""
        got = C.c_int(0)
        check(lib().moexb_layer_load_st(self.h, st.h, prefix.encode(), C.byref(got)))
        return got.value

    def upload_blob(self, e, blob):
        """Copy a host blob (numpy uint8 of expert_bytes(fmt)) into expert e's place."""
        blob = np.ascontiguousarray(blob, dtype=np.uint8)
        assert blob.size == expert_bytes(self.fmt)
        check(lib().moexb_layer_upload_expert(self.h, e, blob.ctypes.data))

    def export_blob(self, e):
        """Expert e's blob in the reference layout, as numpy uint8."""
        out = np.empty(expert_bytes(self.fmt), dtype=np.uint8)
        check(lib().moexb_layer_export_expert(self.h, e, out.ctypes.data))
        return out

    def forward(self, X, T, K=8, out=None, idx=None, w=None, flags=0):
        """moexb_layer_forward. X: [T][H] float32 or bfloat16 device tensor."""
        x_dtype = BF16 if X.dtype == torch.bfloat16 else F32
        out = torch.empty(T, EH, device=X.device, dtype=torch.float32) if out is None else out
        check(lib().moexb_layer_forward(self.ctx.h, self.h, _ptr(X), x_dtype, T, K, _ptr(out), _ptr(idx), _ptr(w), flags, _stream()))
        return out

    def forward_ep(self, X, T, K, out, shared_t0, shared_t1, idx=None, w=None, pre_normed=False):
        """moexb_layer_forward_ep: this rank's partial of one residual block (no residual added)."""
        x_dtype = BF16 if X.dtype == torch.bfloat16 else F32
        check(lib().moexb_layer_forward_ep(self.ctx.h, self.h, _ptr(X), x_dtype, T, K, _ptr(out), _ptr(idx), _ptr(w), shared_t0, shared_t1,
                                           int(pre_normed), _stream()))
        return out

    def close(self):
        if self.h:
            lib().moexb_layer_destroy(self.h)
            self.h = None


def ep_residual_norm(ctx, next_layer, x, total, out, T):
    """moexb_ep_residual_norm: out = x + total, plus the next layer's normalised input when next_layer is given."""
    check(lib().moexb_ep_residual_norm(ctx.h, next_layer.h if next_layer is not None else None, _ptr(x), _ptr(total), _ptr(out), T, _stream()))
    return out


class ExchangeBuffer:
    """One rank's exchange buffer of the expert-parallel path: device memory that the peers map (moexb_ep_buffer_*)."""

    def __init__(self, max_tokens, top_k, world):
        self.bytes = lib().moexb_ep_buffer_bytes(max_tokens, top_k, world)
        p = C.c_void_p()
        self._handle = (C.c_ubyte * 64)()
        check(lib().moexb_ep_buffer_alloc(self.bytes, C.byref(p), self._handle))
        self.ptr, self._opened = p.value, []

    @property
    def handle(self):
        """The 64 bytes another process of this node passes to open_peer()."""
        return bytes(self._handle)

    def open_peer(self, handle):
        """Maps a peer's buffer from its handle; returns the device pointer (valid until close())."""
        h = (C.c_ubyte * 64).from_buffer_copy(handle)
        p = C.c_void_p()
        check(lib().moexb_ep_buffer_open(h, C.byref(p)))
        self._opened.append(p.value)
        return p.value

    def close(self):
        for p in self._opened:
            lib().moexb_ep_buffer_close(p)
        self._opened = []
        if self.ptr:
            lib().moexb_ep_buffer_free(self.ptr)
            self.ptr = None


class EP:
    """moexb_ep: this rank's part of the expert-parallel path. bufs: the exchange buffer of every rank as a device pointer
    valid here (index = rank). While it exists the context serves this path only."""

    def __init__(self, ctx, rank, world, T, K, n_routed, bufs):
        arr = (C.c_void_p * world)(*bufs)
        h = C.c_void_p()
        check(lib().moexb_ep_create(ctx.h, rank, world, T, K, n_routed, arr, C.byref(h)))
        self.h, self.ctx, self.rank, self.world, self.T, self.K = h, ctx, rank, world, T, K
        f, n = C.c_int(0), C.c_int(0)
        check(lib().moexb_ep_own_tokens(h, C.byref(f), C.byref(n)))
        self.first_token, self.n_own = f.value, n.value

    def begin_step(self):
        check(lib().moexb_ep_begin_step(self.h, _stream()))

    def read_routing(self, idx=None, w=None):
        """moexb_ep_read_routing: ids / weights [T][K] of all tokens as this rank holds them after experts() of a layer."""
        check(lib().moexb_ep_read_routing(self.h, _ptr(idx), _ptr(w), _stream()))

    def dispatch(self, layer, l, X=None, residual=True):
        x_dtype = BF16 if (X is not None and X.dtype == torch.bfloat16) else F32
        check(lib().moexb_ep_dispatch(self.h, layer.h, l, _ptr(X), x_dtype, int(residual), _stream()))

    def experts(self, layer, l):
        check(lib().moexb_ep_experts(self.h, layer.h, l, _stream()))

    def finish(self, n_layers, out_own, residual=True):
        check(lib().moexb_ep_finish(self.h, n_layers, int(residual), _ptr(out_own), _stream()))
        return out_own

    def step(self, layers, X, out_own, residual=True):
        """moexb_ep_step: the whole step enqueued on the current stream."""
        arr = (C.c_void_p * len(layers))(*[l.h for l in layers])
        x_dtype = BF16 if X.dtype == torch.bfloat16 else F32
        check(lib().moexb_ep_step(self.h, arr, len(layers), _ptr(X), x_dtype, int(residual), _ptr(out_own), _stream()))
        return out_own

    def stack(self, layers, x_dtype=F32, residual=True):
        """moexb_ep_stack_create: the step captured as one CUDA graph; run / run_host take the whole batch [T][H] and
        return this rank's own rows [n_own][H]."""
        arr = (C.c_void_p * len(layers))(*[l.h for l in layers])
        h = C.c_void_p()
        check(lib().moexb_ep_stack_create(self.h, arr, len(layers), x_dtype, int(residual), C.byref(h)))
        s = Stack.__new__(Stack)
        s.h, s.T, s.layers, s.x_dtype, s.out_rows = h, self.T, layers, x_dtype, self.n_own
        return s

    def close(self):
        if self.h:
            lib().moexb_ep_destroy(self.h)
            self.h = None


class Stack:
    """moexb_stack: n layers chained as residual blocks for a fixed token count, replayed as one CUDA graph."""

    def __init__(self, ctx, layers, T, K=8, x_dtype=F32, residual=True):
        arr = (C.c_void_p * len(layers))(*[l.h for l in layers])
        h = C.c_void_p()
        check(lib().moexb_stack_create(ctx.h, arr, len(layers), T, K, x_dtype, int(residual), C.byref(h)))
        self.h, self.T, self.layers, self.x_dtype, self.out_rows = h, T, layers, x_dtype, T

    @property
    def kernel_count(self):
        return lib().moexb_stack_kernel_count(self.h)

    def run(self, X, out=None):
        out = torch.empty(self.out_rows, EH, device=X.device, dtype=torch.float32) if out is None else out
        check(lib().moexb_stack_run(self.h, _ptr(X), _ptr(out), _stream()))
        return out

    def run_host(self, X_host, out_host):
        """X_host / out_host: CPU tensors (pinned for full speed). Returns after the result has landed."""
        assert not X_host.is_cuda and not out_host.is_cuda and X_host.is_contiguous() and out_host.is_contiguous()
        check(lib().moexb_stack_run_host(self.h, X_host.data_ptr(), out_host.data_ptr(), _stream()))
        return out_host

    def close(self):
        if self.h:
            lib().moexb_stack_destroy(self.h)
            self.h = None


def launch_count():
    return lib().moexb_launch_count()
