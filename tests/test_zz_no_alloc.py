"""The allocation-free matvec entry point, `qmm_gemv_f32_static`.

Some callers of this library cannot call cudaMalloc while they run (a serving loop
that must not hit the allocator's device-wide synchronization, a process whose HBM
is fully committed).  For them the library keeps the packed activations in a fixed
device array inside its own image.  This test calls that entry point through the
C ABI twice in a row — the second call finds the first call's bytes in the shared
array — and compares each result with the ordinary `qmm_gemv_f32`.  It lives in a
file of its own that sorts last so that a failure here cannot hide another test.
"""
import numpy as np
import pytest

from litenn_b200 import capi, synth
from helpers import REL_TOL, max_rel_err

pytestmark = pytest.mark.gpu


def test_static_scratch_matvec_matches_allocating_matvec(qmm_lib):
    import torch
    assert torch.cuda.is_available()
    torch.cuda.set_device(0)
    n, k = 272, 2048
    payload = synth.make_weight(capi.Q4_0, n, k, seed=21, name="noalloc.w")
    w = capi.Weight.from_host(capi.Q4_0, payload, n, k)
    # two calls in a row with different batch sizes and data: the second overwrites the first's scratch
    for call, m in enumerate((5, 1)):
        x = torch.from_numpy(synth.make_activation(m, k, seed=21 + call, name="noalloc.x")).cuda()
        y_ref = torch.empty((m, n), dtype=torch.float32, device="cuda")
        y_new = torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda")
        w.gemv_f32(x.data_ptr(), y_ref.data_ptr(), m)
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        w.gemv_f32_static(x.data_ptr(), y_new.data_ptr(), m)
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        assert capi.kernel_status(0) == 0
        got, ref = y_new.cpu().numpy(), y_ref.cpu().numpy()
        assert np.isfinite(got).all()
        assert max_rel_err(got, ref) <= REL_TOL, f"call {call}"


def test_static_scratch_rejects_oversized_requests(qmm_lib):
    import torch
    torch.cuda.set_device(0)
    n, k = 16, 32768  # m = 16 needs ~1.2 MB of packed activations: beyond the fixed 640 KiB
    payload = synth.make_weight(capi.Q8_0, n, k, seed=3, name="noalloc.big")
    w = capi.Weight.from_host(capi.Q8_0, payload, n, k)
    x = torch.zeros((16, k), device="cuda")
    y = torch.zeros((16, n), device="cuda")
    with pytest.raises(capi.QmmError) as e:
        w.gemv_f32_static(x.data_ptr(), y.data_ptr(), 16)
    assert e.value.code == capi.E_INVALID and "fixed scratch" in str(e.value)
    w.gemv_f32_static(x.data_ptr(), y.data_ptr(), 1)  # m = 1 fits
    torch.cuda.synchronize()
