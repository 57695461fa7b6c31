"""The workspace-free dense backward (snntc_fc_backward_noalloc) against the regular entry point.

Collected last on purpose (file name): a run that stops at the first failure has then already been
through every other test. The entry point exists for callers that cannot allocate device memory at
the time of the call; its scratch is a fixed array inside the library, shared by all calls, so the
test calls it twice in a row with different inputs and checks each result against
snntc_fc_backward, which gets a fresh caller-owned workspace. Both paths run the same kernels with
the same launch plan, so the results must be identical bit for bit.
"""
import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _problem(seed, B, I, J, bv):
    import torch
    rng = np.random.default_rng(seed)
    x = torch.from_numpy(np.exp(np.abs(rng.standard_normal((B, I)))).astype(np.float32)).cuda()
    w = torch.from_numpy(rng.standard_normal((I + (bv > 1e-8), J)).astype(np.float32)).cuda()
    g = torch.from_numpy(rng.standard_normal((2 * B, J)).astype(np.float32)).cuda()
    params = np.array([1e5, 1e-10, 1.0, 0, 0, bv], np.float32)
    return x, w, g, params


def _stream():
    import torch
    return torch.cuda.current_stream().cuda_stream


def _forward(lib, x, w, params):
    import torch
    B, I = x.shape
    rows, J = w.shape
    out = torch.empty((2 * B, J), dtype=torch.float32, device="cuda")
    nb = lib.snntc_fc_forward_workspace_bytes(B, I, J)
    ws = torch.empty(max(nb, 4) // 4 + 1, dtype=torch.float32, device="cuda")
    rc = lib.snntc_fc_forward(x.data_ptr(), w.data_ptr(), params.ctypes.data, out.data_ptr(), B, I, rows, J,
                              ws.data_ptr(), ws.numel() * 4, _stream())
    assert rc == 0
    return out


def _backward_regular(lib, g, x, w, params, out):
    import torch
    B, I = x.shape
    rows, J = w.shape
    dx = torch.empty_like(x); dw = torch.empty_like(w); dp = torch.full((6,), 7.0, device="cuda")
    nb = lib.snntc_fc_backward_workspace_bytes(B, I, rows, J)
    ws = torch.empty(max(nb, 4) // 4 + 1, dtype=torch.float32, device="cuda")
    rc = lib.snntc_fc_backward(g.data_ptr(), x.data_ptr(), w.data_ptr(), params.ctypes.data, out.data_ptr(),
                               dx.data_ptr(), dw.data_ptr(), dp.data_ptr(), B, I, rows, J,
                               ws.data_ptr(), ws.numel() * 4, _stream())
    assert rc == 0
    return dx, dw, dp, nb


def _backward_noalloc(lib, g, x, w, params, out):
    import torch
    B, I = x.shape
    rows, J = w.shape
    dx = torch.empty_like(x); dw = torch.empty_like(w); dp = torch.full((6,), 7.0, device="cuda")
    rc = lib.snntc_fc_backward_noalloc(g.data_ptr(), x.data_ptr(), w.data_ptr(), params.ctypes.data, out.data_ptr(),
                                       dx.data_ptr(), dw.data_ptr(), dp.data_ptr(), B, I, rows, J, _stream())
    return rc, dx, dw, dp


def test_noalloc_matches_regular_entry_point_twice_in_a_row():
    import torch
    from snntc_2023_b200 import _lib
    lib = _lib.load()
    assert lib.snntc_noalloc_scratch_bytes() == 8 << 20
    # two different problems back to back: the second must not see anything of the first in the shared array
    for seed, B, I, J, bv in ((101, 512, 300, 200, 1.0), (102, 384, 257, 130, 0.0)):
        x, w, g, params = _problem(seed, B, I, J, bv)
        out = _forward(lib, x, w, params)
        dx0, dw0, dp0, need = _backward_regular(lib, g, x, w, params, out)
        assert 0 < need <= lib.snntc_noalloc_scratch_bytes(), "the case must really use the scratch"
        rc, dx1, dw1, dp1 = _backward_noalloc(lib, g, x, w, params, out)
        assert rc == 0, lib.snntc_status_string(rc)
        torch.cuda.synchronize()
        assert torch.equal(dx0, dx1)
        assert torch.equal(dw0, dw1)
        assert torch.equal(dp0, dp1) and float(dp1.abs().sum()) == 0.0
        assert torch.isfinite(dw1).all()


def test_noalloc_refuses_problems_larger_than_its_scratch():
    import torch
    from snntc_2023_b200 import _lib
    lib = _lib.load()
    B, I, J, bv = 128, 28352, 64, 0.0
    need = lib.snntc_fc_backward_workspace_bytes(B, I, I, J)
    if need <= lib.snntc_noalloc_scratch_bytes():
        pytest.skip("this device's launch plan keeps the problem inside the scratch")
    x, w, g, params = _problem(103, B, I, J, bv)
    out = torch.zeros((2 * B, J), device="cuda")
    sentinel = torch.full_like(w, 3.0)
    rc = lib.snntc_fc_backward_noalloc(g.data_ptr(), x.data_ptr(), w.data_ptr(), params.ctypes.data, out.data_ptr(),
                                       0, sentinel.data_ptr(), 0, B, I, I, J, _stream())
    assert rc == -5 and b"workspace" in lib.snntc_status_string(rc)
    torch.cuda.synchronize()
    assert float((sentinel - 3.0).abs().max()) == 0.0  # nothing was launched
