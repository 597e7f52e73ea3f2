"""The allocation-free decode entry point, moexb_experts_forward_static, against moexb_experts_forward.

Some hosts of this library cannot allocate device memory once they are running - they committed all of it at start-up,
or they call from a thread that must not block in the allocator - so this entry point keeps its scratch in a fixed
array inside the library. The test calls it through the C ABI twice in a row (the second call with other inputs and
fewer experts, so values left behind by the first call would show) and compares each result with the ordinary entry
point, within the tolerance of the other FFN tests (relative L2 1e-3, max-abs 2e-3). Collected last on purpose.
"""
import numpy as np
import pytest
import torch

import moe_b200 as m

pytestmark = [pytest.mark.gpu, pytest.mark.usefixtures("lib_built")]
DEV = "cuda:0"


def test_static_scratch_entry_point_matches_experts_forward_twice():
    L = m.lib()
    fmt = m.FMT_SYM_F16
    blobs = [torch.from_numpy(m.synth_expert_host(fmt, 21, 0, e)).to(DEV) for e in range(9)]
    slots = torch.tensor([b.data_ptr() for b in blobs], dtype=torch.int64, device=DEV)
    rng = np.random.default_rng(77)
    stream = torch.cuda.current_stream().cuda_stream
    for call, K in enumerate((9, 5)):
        x = torch.from_numpy(rng.standard_normal(2048).astype(np.float32)).to(DEV)
        w = torch.from_numpy(rng.uniform(0.05, 0.3, K).astype(np.float32)).to(DEV)
        ref = m.experts_forward(fmt, slots, w, K, x)
        out = torch.full((2048,), float("nan"), device=DEV)
        rc = L.moexb_experts_forward_static(fmt, slots.data_ptr(), w.data_ptr(), K, x.data_ptr(), out.data_ptr(), stream, None)
        assert rc == 0, L.moexb_last_error().decode()
        got, want = out.cpu().numpy().astype(np.float64), ref.cpu().numpy().astype(np.float64)
        assert np.isfinite(got).all()
        rel = np.linalg.norm(got - want) / np.linalg.norm(want)
        assert rel <= 1e-3 and np.abs(got - want).max() <= 2e-3, f"call {call}: rel-L2 {rel:.3e}, max-abs {np.abs(got - want).max():.3e}"
    # more experts than the built-in scratch holds: refused with a message, nothing launched
    assert L.moexb_experts_forward_static(fmt, slots.data_ptr(), w.data_ptr(), 17, x.data_ptr(), out.data_ptr(), stream, None) == -1
    assert b"at most 16" in L.moexb_last_error()
