"""The CUDA path against the reference's OWN GPU operators (snn*_kernels.cu.cc compiled unmodified for
sm_100a under a stand-in TensorFlow header, oracle/_ref/libsnntc_ref_gpu.so). Same inputs, same GPU.
Skipped where that library has not been built."""
import numpy as np
import pytest

import oracle as O
from tests import parity as P

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(O.ref_gpu_lib() is None, reason="reference GPU operators not built")]
MAXV = 1e5


def _compare_forward(mine, ref, o64, what):
    mine, ref = mine.cpu().numpy(), ref.cpu().numpy()
    n = mine.shape[0] // 2
    y, yr = mine[:n].reshape(o64["y"].shape), ref[:n].reshape(o64["y"].shape)
    inv, invr = mine[n:].reshape(o64["y"].shape), ref[n:].reshape(o64["y"].shape)
    f, fr = y < MAXV - 0.1, yr < MAXV - 0.1
    assert ((f != fr) & ~o64["illc"]).sum() == 0, "%s: fire/no-fire differs from the reference GPU kernel" % what
    ok = f & fr & ~o64["illc"]
    if ok.any():
        assert (np.abs(y[ok] - yr[ok]) / np.abs(yr[ok])).max() <= 2e-6, what
        assert (np.abs(inv[ok] - invr[ok]) / np.abs(invr[ok])).max() <= 2e-6, what
    return float(ok.mean())


@pytest.mark.parametrize("seed,B,I,J,bv,dist", [(701, 40, 300, 200, 1.0, "test"), (702, 33, 784, 400, 0.0, "cfg"),
                                                 (703, 17, 65, 10, 1.0, "test"), (704, 64, 513, 96, 0.5, "cfg")])
def test_dense_against_reference_gpu(seed, B, I, J, bv, dist):
    import torch
    from snntc_2023_b200 import ops
    rg = O.RefGpu(256 << 20)
    x, w = P.make_inputs(seed, (B, I), (I + (bv > 1e-8), J), dist)
    p = O.fc_params(biasvolt=bv)
    xd, wd = torch.from_numpy(x).cuda(), torch.from_numpy(w).cuda()
    mine = ops.snn_fc(xd, wd, p)
    ref = rg.fc_forward(xd, wd, p)
    _compare_forward(mine, ref, O.fc_forward(x, w, p, "f64"), "dense %d" % seed)
    g = torch.randn(2 * B, J, device="cuda", generator=torch.Generator("cuda").manual_seed(seed))
    g[B:] = 0
    # both backward passes from the REFERENCE's forward output, so only the gradient kernels differ
    dx, dw, _ = ops.snn_fc_grad(g, xd, wd, p, ref)
    dxr, dwr = rg.fc_backward(g, xd, wd, p, ref)
    refc = ref.cpu().numpy()
    b64 = O.fc_backward(g[:B].cpu().numpy(), x, w, p, refc[:B], refc[B:], "f64")
    P.check_close(dx.cpu().numpy(), dxr.cpu().numpy(), "dense dX vs reference GPU", abs_sum=b64["dx_abs"])
    P.check_close(dw.cpu().numpy(), dwr.cpu().numpy(), "dense dW vs reference GPU", abs_sum=b64["dw_abs"])


@pytest.mark.parametrize("case", [(711, 2, 7, 9, 3, 3, 2, 2, 1, 5, 1.0, "SAME", "test"),
                                  (712, 2, 8, 8, 3, 3, 3, 2, 2, 4, 1.0, "SAME", "test"),
                                  (713, 1, 9, 6, 4, 2, 4, 1, 3, 7, 0.0, "VALID", "test"),
                                  (714, 2, 10, 10, 16, 3, 3, 1, 1, 32, 1.0, "SAME", "cfg"),
                                  (715, 3, 12, 11, 5, 6, 3, 3, 2, 33, 1.0, "VALID", "test")])
def test_conv_against_reference_gpu(case):
    import torch
    from snntc_2023_b200 import ops
    seed, B, H, W, C, Kh, Kw, Sh, Sw, Kc, bv, padding, dist = case
    rg = O.RefGpu(256 << 20)
    x, w = P.make_inputs(seed, (B, H, W, C), (Kh * Kw * C + (bv > 1e-8), Kc), dist)
    p = O.cv_params(Kh, Kw, Sh, Sw, padding, bv)
    xd, wd = torch.from_numpy(x).cuda(), torch.from_numpy(w).cuda()
    xp = torch.from_numpy(O.pad_like_reference(x, Kh, Kw, Sh, Sw, padding)).cuda()
    pt, pl, Nh, Nw = ops.conv_geometry(H, W, Kh, Kw, Sh, Sw, padding)
    mine = ops.snn_cv(xd, wd, p, pt, pl, Nh, Nw)
    ref = rg.cv_forward(xp, wd, p)
    assert tuple(ref.shape) == tuple(mine.shape)
    _compare_forward(mine, ref, O.cv_forward(x, w, p, "f64"), "conv %d" % seed)
    g = torch.randn(2 * B, Nh, Nw, Kc, device="cuda", generator=torch.Generator("cuda").manual_seed(seed))
    g[B:] = 0
    dxp, dw, _ = ops.snn_cv_grad(g, xp, wd, p, ref)           # the reference's calling convention: padded in, padded out
    dxr, dwr = rg.cv_backward(g, xp, wd, p, ref)
    refc = ref.cpu().numpy()
    b64 = O.cv_backward(g[:B].cpu().numpy(), xp.cpu().numpy(), w, O.cv_params(Kh, Kw, Sh, Sw, "VALID", bv), refc[:B], refc[B:], "f64")
    P.check_close(dxp.cpu().numpy(), dxr.cpu().numpy(), "conv dX vs reference GPU", abs_sum=b64["dx_abs"])
    P.check_close(dw.cpu().numpy(), dwr.cpu().numpy(), "conv dW vs reference GPU", abs_sum=b64["dw_abs"])
