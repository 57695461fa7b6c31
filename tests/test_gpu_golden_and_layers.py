"""GPU checks against the committed golden fixtures (outputs of the reference's own CPU operators),
two-layer chains as in the reference's test-snn-*-layers.py, and the layer modules end to end."""
import glob
import os

import numpy as np
import pytest

import oracle as O
from tests import parity as P

pytestmark = pytest.mark.gpu
GOLD = sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "*.npz")))
MAXV = 1e5


@pytest.mark.parametrize("path", GOLD, ids=lambda p: os.path.basename(p)[:-4])
def test_cuda_matches_golden(path):
    import torch
    from snntc_2023_b200 import ops
    d = np.load(path)
    name = os.path.basename(path)
    x, w, p = d["x"], d["w"], d["params"]
    xd, wd = torch.from_numpy(x).cuda(), torch.from_numpy(w).cuda()
    if name.startswith("dense"):
        B = x.shape[0]
        out = ops.snn_fc(xd, wd, p).cpu().numpy()
        y_gpu, y_ref = out[:B], d["out"][:B]
        o64 = O.fc_forward(x, w, p, "f64")
    else:
        Kh, Kw, Sh, Sw = (int(p[i]) for i in (6, 7, 8, 9))
        pt, pl, Nh, Nw = ops.conv_geometry(x.shape[1], x.shape[2], Kh, Kw, Sh, Sw, str(d["padding"]))
        out = ops.snn_cv(xd, wd, p, pt, pl, Nh, Nw).cpu().numpy()
        y_gpu, y_ref = out[:x.shape[0]], d["y"]
        o64 = O.cv_forward(x, w, p, "f64")
    fg, fr = y_gpu < MAXV - 0.1, y_ref < MAXV - 0.1
    assert ((fg != fr) & ~o64["illc"]).sum() == 0
    ok = fg & fr & ~o64["illc"]
    if ok.any():
        tol = np.maximum(1e-4, 4e-7 * o64["cond"][ok])
        rel = np.abs(y_gpu[ok] - y_ref[ok]) / np.abs(y_ref[ok])
        assert (rel / tol).max() <= 1.0, "%s: rel %.3e vs the reference's output" % (name, rel.max())


def test_two_dense_layers_chain():
    """Gradients w.r.t. the input and the second layer's weight through two stacked layers and an MSE
    loss (test-snn-fc-layers.py:46-54); sentinel outputs of layer 1 feed layer 2 as 'never spikes'."""
    import torch
    import SNN_TC_Modules as SNN
    rng = np.random.default_rng(71)
    B, I, H, J = 24, 60, 50, 30
    x = np.exp(np.abs(rng.standard_normal((B, I)))).astype(np.float32)
    w1 = rng.standard_normal((I + 1, H)).astype(np.float32)
    w2 = rng.standard_normal((H + 1, J)).astype(np.float32)
    l1 = SNN.SNN_dense(I, H, weight=w1).cuda(); l2 = SNN.SNN_dense(H, J, weight=w2).cuda()
    xd = torch.from_numpy(x).cuda().requires_grad_(True)
    h = l1(xd); y = l2(h)
    target = torch.zeros_like(y)
    fired = y < MAXV - 0.1
    loss = ((y - target)[fired] ** 2).sum()
    loss.backward()
    # oracle chain
    p = O.fc_params(biasvolt=1.0)
    hc, yc = h.detach().cpu().numpy(), y.detach().cpu().numpy()
    o1 = O.fc_forward(x, w1, p, "f64"); assert ((hc < MAXV - .1) != (o1["y"] < MAXV - .1))[~o1["illc"]].sum() == 0
    assert (hc >= MAXV - 0.1).any(), "the case should contain unfired hidden units"
    g2 = np.where(yc < MAXV - 0.1, 2 * yc, 0).astype(np.float32)
    f2 = O.fc_forward(hc, w2, p, "f32")
    b2 = O.fc_backward(g2, hc, w2, p, yc, f2["inv"], "f64")
    P.check_close(l2.weight.grad.cpu().numpy(), b2["dw"], "chain dW2", abs_sum=b2["dw_abs"])
    f1 = O.fc_forward(x, w1, p, "f32")
    b1 = O.fc_backward(b2["dx"].astype(np.float32), x, w1, p, hc, f1["inv"], "f64")
    P.check_close(xd.grad.cpu().numpy(), b1["dx"], "chain dX", rel=2e-4, l2=1e-4, abs_sum=b1["dx_abs"])
    assert np.all(b2["dx"][hc >= MAXV - 0.1] == 0)   # no gradient through a unit that did not fire


def test_conv_pool_dense_network_step():
    """A small conv -> pool -> dense net: module forward equals the oracle chain, dW lands in the flat
    bucket, and a second identical step reproduces it bit for bit (no atomics on this path)."""
    import torch
    from snntc_2023_b200 import nets
    from oracle import ref_model
    specs = [("conv", 3, 8, 3, 1), ("conv", 8, 8, 3, 1), ("pool", 2), ("flatten",), ("dense", 8 * 4 * 4, 10)]
    weights = nets.spec_weights(specs, 5)
    net = nets.SnnNet(specs, weights=weights, device="cuda")
    rng = np.random.default_rng(6)
    B = 5
    x = np.exp(rng.random((B, 8, 8, 3))).astype(np.float32)
    labels = rng.integers(0, 10, B)
    xd, ld = torch.from_numpy(x).cuda(), torch.from_numpy(labels).cuda()
    loss = net.loss(xd, ld); net.backward(loss)
    g1 = net.flat_grad.clone()
    loss_c, grads_c, _ = ref_model.train_step(specs, weights, x, labels, threads=1, kind="port")
    assert abs(float(loss.detach()) - loss_c) <= 1e-4 * abs(loss_c)
    want = np.concatenate([g.reshape(-1) for g in grads_c])
    got = g1.cpu().numpy()
    assert np.linalg.norm(got - want) <= 1e-4 * np.linalg.norm(want)
    net.flat_grad.zero_()
    loss2 = net.loss(xd, ld); net.backward(loss2)
    assert torch.equal(net.flat_grad, g1) and float(loss2.detach()) == float(loss.detach())
    assert all(l.weight.grad.data_ptr() == l.grad_sink.data_ptr() for l in net.weighted_layers())


def test_minpool_matches_oracle():
    import torch
    from snntc_2023_b200 import ops
    rng = np.random.default_rng(8)
    for (H, W, K, S, padding) in ((8, 8, 2, 2, "SAME"), (7, 9, 3, 2, "SAME"), (9, 7, 2, 2, "VALID"), (5, 5, 3, 1, "SAME")):
        x = np.exp(rng.random((2, H, W, 6))).astype(np.float32)
        x[rng.random(x.shape) < 0.3] = 1e5
        xd = torch.from_numpy(x).cuda().requires_grad_(True)
        y = ops.snn_minpool(xd, K, K, S, S, padding)
        yo, arg = O.minpool(x, K, K, S, S, padding)
        assert np.array_equal(y.detach().cpu().numpy(), yo)
        g = torch.randn_like(y)
        y.backward(g)
        want = np.zeros(x.size, np.float32)
        ok = arg.reshape(-1) >= 0
        np.add.at(want, arg.reshape(-1)[ok], g.cpu().numpy().reshape(-1)[ok])
        assert np.allclose(xd.grad.cpu().numpy().reshape(-1), want, rtol=1e-6, atol=1e-6)
