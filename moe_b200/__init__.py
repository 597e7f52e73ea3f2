"""moe_b200: the MoE expert-FFN hot path of the moex engine, hand-written for NVIDIA B200 (sm_100a).

The product is libmoexb.so (CUDA kernels behind the C ABI of include/moexb.h). This package is the thin host-side
mirror of the reference's expert-layer entry points (same names and argument meaning as src/kernels.cuh of the
reference) on torch tensors, used by the tests and the benchmark.
"""
from ._lib import (FMT_SYM_F32, FMT_SYM_F16, FMT_ZP, F32, BF16, F16, LAYOUT_TILED, LAYOUT_REFERENCE, EH, EI, EGS, Q_BYTES, CHUNKS, MoexbError,
                   PairItem, Pair, lib)
from .api import (expert_bytes, gemv_f16, gemv_f32, router_topk, experts_forward, pairs_forward, pairs_forward_dev,
                  pairs_reduce, gated_add_rows, shared_expert_add, group_pairs, dequant, q4k_dequant, q4k_to_zp,
                  synth_expert_host, synth_q4k_host, gguf_dequant_host, gguf_row_to_zp, Context, Layer, Stack, Gguf, SafeTensors, launch_count, ep_residual_norm,
                  ExchangeBuffer, EP)
