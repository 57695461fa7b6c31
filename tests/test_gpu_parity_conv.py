"""GPU parity of SnnCv / SnnCvGrad against the oracle, through the C ABI."""
import numpy as np
import pytest

import oracle as O
from tests import parity as P

pytestmark = pytest.mark.gpu

# (seed, B, H, W, C, Kh, Kw, Sh, Sw, Kc, biasvolt, padding, dist); kernel 2..6, stride 1..3, SAME/VALID,
# bias on/off as randomised by test-snn-cv-forward.py:23-29
CONV_CASES = [
    (41, 2, 7, 9, 3, 3, 2, 2, 1, 5, 1.0, "SAME", "test"),
    (42, 2, 8, 8, 3, 3, 3, 2, 2, 4, 1.0, "SAME", "test"),
    (43, 1, 9, 6, 4, 2, 4, 1, 3, 7, 0.0, "VALID", "test"),
    (44, 2, 6, 6, 8, 3, 3, 1, 1, 16, 1.0, "SAME", "cfg"),
    (45, 2, 6, 6, 8, 3, 3, 1, 1, 16, 0.0, "SAME", "cfg"),
    (46, 1, 10, 10, 2, 5, 5, 2, 2, 3, 1.0, "SAME", "test"),
    (47, 3, 12, 11, 5, 6, 3, 3, 2, 33, 1.0, "VALID", "test"),
    (48, 2, 16, 16, 64, 3, 3, 1, 1, 128, 0.0, "SAME", "cfg"),
    (49, 4, 8, 8, 3, 3, 3, 1, 1, 64, 1.0, "SAME", "cfg"),
    (50, 1, 5, 5, 1, 1, 1, 1, 1, 1, 1.0, "SAME", "test"),
    (51, 2, 9, 9, 16, 7, 7, 2, 2, 40, 1.0, "SAME", "cfg"),
    (52, 5, 64, 64, 3, 3, 3, 1, 1, 64, 1.0, "SAME", "cfg"),   # 20480 rows: many more than resident warps
]


def _ids(c):
    return "s%d_B%d_%dx%dx%d_K%dx%d_S%d%d_Kc%d_b%g_%s_%s" % c


def _run_conv(seed, B, H, W, C, Kh, Kw, Sh, Sw, Kc, bv, padding, dist):
    import torch
    from snntc_2023_b200 import ops
    I = Kh * Kw * C
    x, w = P.make_inputs(seed, (B, H, W, C), (I + (bv > 1e-8), Kc), dist)
    params = O.cv_params(Kh, Kw, Sh, Sw, padding, bv)
    xd, wd = torch.from_numpy(x).cuda(), torch.from_numpy(w).cuda()
    pt, pl, Nh, Nw = ops.conv_geometry(H, W, Kh, Kw, Sh, Sw, padding)
    out = ops.snn_cv(xd, wd, params, pt, pl, Nh, Nw)
    assert out.shape == (2 * B, Nh, Nw, Kc)
    return x, w, params, xd, wd, out, out.cpu().numpy(), (pt, pl, Nh, Nw)


@pytest.mark.parametrize("case", CONV_CASES, ids=_ids)
def test_conv_forward(case):
    import torch
    from snntc_2023_b200 import ops
    seed, B, H, W, C, Kh, Kw, Sh, Sw, Kc, bv, padding, dist = case
    x, w, params, xd, wd, out, outc, geom = _run_conv(*case)
    o32 = O.cv_forward(x, w, params, "f32")
    o64 = O.cv_forward(x, w, params, "f64")
    rows = P.im2col_rows(x, Kh, Kw, Sh, Sw, padding)
    P.check_forward(outc[:B], outc[B:], o32, o64, rows=rows, what="conv fwd %s" % (case,))
    # the reference op's own calling convention: a tensor already padded with MAX / cropped
    xp = O.pad_like_reference(x, Kh, Kw, Sh, Sw, padding)
    out_p = ops.snn_cv(torch.from_numpy(xp).cuda(), wd, params)
    assert torch.equal(out_p, out)


@pytest.mark.parametrize("case", CONV_CASES, ids=_ids)
def test_conv_backward(case):
    import torch
    from snntc_2023_b200 import ops
    seed, B, H, W, C, Kh, Kw, Sh, Sw, Kc, bv, padding, dist = case
    x, w, params, xd, wd, out, outc, (pt, pl, Nh, Nw) = _run_conv(*case)
    g = np.random.default_rng(seed + 1000).standard_normal((B, Nh, Nw, Kc)).astype(np.float32)
    gd = torch.from_numpy(g).cuda()
    dx, dw, dp = ops.snn_cv_grad(gd, xd, wd, params, out, pt, pl)
    ref = O.cv_backward(g, x, w, params, outc[:B], outc[B:], "f64")
    P.check_close(dx.cpu().numpy(), ref["dx"], "conv dX %s" % (case,), abs_sum=ref["dx_abs"])
    P.check_close(dw.cpu().numpy(), ref["dw"], "conv dW %s" % (case,), abs_sum=ref["dw_abs"])
    assert np.all(dp.cpu().numpy() == 0)
    # reference convention: padded input in, padded-shape gradient out; its interior is our dx
    xp = O.pad_like_reference(x, Kh, Kw, Sh, Sw, padding)
    dxp, dwp, _ = ops.snn_cv_grad(gd, torch.from_numpy(xp).cuda(), wd, params, out)
    assert tuple(dxp.shape) == xp.shape
    if padding == "SAME":
        inner = dxp[:, pt:pt + H, pl:pl + W, :]
        assert torch.equal(inner, dx)
        rest = dxp.clone()
        rest[:, pt:pt + H, pl:pl + W, :] = 0
        assert float(rest.abs().max()) == 0.0  # padding positions get no gradient
    assert torch.equal(dwp, dw)
