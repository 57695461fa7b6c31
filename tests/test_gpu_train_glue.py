"""GPU tests of the kernels around the SNN-TC layers (input encoding, loss, weight cost, optimisers) and of the
inference-only forward. These are floating-point kernels: they are compared with plain torch / numpy fp32-fp64
evaluations of the reference's formulas, tolerance stated per test."""
import numpy as np
import pytest

import oracle as O
from tests import parity as P

pytestmark = pytest.mark.gpu


def test_encode_matches_exp_of_one_minus_pixel():
    import torch
    from snntc_2023_b200 import train
    p = torch.rand(7, 28, 28, 1, device="cuda", generator=torch.Generator("cuda").manual_seed(1))
    x = train.encode(p)                       # snntc-mnist.py:75: tf.exp(1.0 * (1.0 - images))
    ref = torch.exp(1.0 - p.double()).float()
    assert torch.allclose(x, ref, rtol=2e-6, atol=0)       # expf is within 2 ulp
    x2 = train.encode(p, scale=0.5, one_minus=False)
    assert torch.allclose(x2, torch.exp(0.5 * p.double()).float(), rtol=2e-6, atol=0)


@pytest.mark.parametrize("B,J", [(1, 10), (37, 10), (256, 1000), (5, 33)])
def test_loss_matches_cross_entropy_on_negated_logits(B, J):
    import torch
    import torch.nn.functional as F
    from snntc_2023_b200 import train
    g = torch.Generator("cuda").manual_seed(B * 1000 + J)
    y = (torch.rand(B, J, device="cuda", generator=g) * 3 + 1)
    y[torch.rand(B, J, device="cuda", generator=g) < 0.3] = 1e5      # outputs that never spiked
    y[0, :] = 1e5                                                     # a sample without any spike: uniform softmax
    lab = torch.randint(0, J, (B,), device="cuda", generator=g)
    y1 = y.clone().requires_grad_(True)
    loss, hits = train.loss_func(y1, lab, with_hits=True)
    (loss * 1.5).backward()
    y2 = y.double().clone().requires_grad_(True)
    ref = F.cross_entropy(-y2, lab)                                   # SNN_TC_Modules.py:286-288, batch mean
    (ref * 1.5).backward()
    assert abs(float(loss) - float(ref)) <= 1e-5 * max(1.0, abs(float(ref)))
    assert torch.allclose(y1.grad.double(), y2.grad, rtol=1e-5, atol=1e-7)
    assert int(hits) == int((y.argmin(1) == lab).sum())
    onehot = F.one_hot(lab, J).float()                                # the reference passes one-hot labels
    assert abs(float(train.loss_func(y, onehot)) - float(ref)) <= 1e-5 * max(1.0, abs(float(ref)))


def test_constraint_cost_matches_reference_formula():
    import torch
    from snntc_2023_b200 import train
    g = torch.Generator("cuda").manual_seed(3)
    ws = [torch.randn(28, 64, device="cuda", generator=g) * 0.3,
          torch.randn(577, 130, device="cuda", generator=g) * 0.05,
          torch.randn(4097, 10, device="cuda", generator=g) * 0.02]
    K, K2 = 100.0, 1e-3
    w1 = [w.clone().requires_grad_(True) for w in ws]
    cost = train.constraint_cost(w1, K, K2)
    (cost * 2.0).backward()
    w2 = [w.double().clone().requires_grad_(True) for w in ws]
    # snntc-mnist.py:55-59
    wsc = sum(torch.clamp(1.0 - w.sum(0), min=0).mean() for w in w2)
    l2 = sum((w ** 2).mean() for w in w2)
    ref = K * wsc + K2 * l2
    (ref * 2.0).backward()
    assert abs(float(cost) - float(ref)) <= 1e-5 * abs(float(ref))
    for a, b in zip(w1, w2):
        assert torch.allclose(a.grad.double(), b.grad, rtol=1e-5, atol=1e-9)


def test_adam_and_sgdm_follow_the_keras_updates():
    import torch
    from snntc_2023_b200 import train
    rng = np.random.default_rng(5)
    n = 100003
    w0 = rng.standard_normal(n).astype(np.float32)
    grads = [rng.standard_normal(n).astype(np.float32) for _ in range(4)]
    # Adam (tf.keras.optimizers.Adam: lr_t = lr*sqrt(1-b2^t)/(1-b1^t), eps added to sqrt(v))
    lr, b1, b2, eps, gs = 1e-2, 0.9, 0.999, 1e-7, 0.5
    w = w0.astype(np.float64); m = np.zeros(n); v = np.zeros(n)
    wd = torch.from_numpy(w0.copy()).cuda(); gd = torch.zeros(n, device="cuda")
    opt = train.Adam(wd, gd, lr=lr, beta1=b1, beta2=b2, eps=eps)
    for t, g in enumerate(grads, 1):
        gd.copy_(torch.from_numpy(g))
        opt.step(grad_scale=gs)
        ge = g.astype(np.float64) * gs
        m += (ge - m) * (1 - b1); v += (ge * ge - v) * (1 - b2)
        w -= lr * np.sqrt(1 - b2 ** t) / (1 - b1 ** t) * m / (np.sqrt(v) + eps)
    assert int(opt.steps) == len(grads)
    assert np.allclose(wd.cpu().numpy(), w, rtol=2e-5, atol=2e-6)
    # SGD with momentum (tf.keras.optimizers.SGD: vel = momentum*vel - lr*g; w += vel)
    w = w0.astype(np.float64); vel = np.zeros(n)
    wd = torch.from_numpy(w0.copy()).cuda()
    opt = train.SGDM(wd, gd, lr=0.05, momentum=0.9)
    for g in grads:
        gd.copy_(torch.from_numpy(g))
        opt.step()
        vel = 0.9 * vel - 0.05 * g.astype(np.float64); w += vel
    assert np.allclose(wd.cpu().numpy(), w, rtol=1e-5, atol=1e-6)


def test_inference_forward_is_the_first_half_of_the_training_forward():
    import torch
    from snntc_2023_b200 import ops
    from snntc_2023_b200.SNN_TC_Modules import SNN_conv, SNN_dense
    x, w = P.make_inputs(61, (33, 70), (71, 64), "test")
    params = O.fc_params(biasvolt=1.0)
    xd, wd = torch.from_numpy(x).cuda(), torch.from_numpy(w).cuda()
    assert torch.equal(ops.snn_fc_infer(xd, wd, params), ops.snn_fc(xd, wd, params)[:33])
    xc, wc = P.make_inputs(62, (2, 9, 9, 8), (3 * 3 * 8 + 1, 130), "cfg")
    pc = O.cv_params(3, 3, 1, 1, "SAME", 1.0)
    pt, pl, Nh, Nw = ops.conv_geometry(9, 9, 3, 3, 1, 1, "SAME")
    xcd, wcd = torch.from_numpy(xc).cuda(), torch.from_numpy(wc).cuda()
    assert torch.equal(ops.snn_cv_infer(xcd, wcd, pc, pt, pl, Nh, Nw), ops.snn_cv(xcd, wcd, pc, pt, pl, Nh, Nw)[:2])
    # the layers take the inference path by themselves when no gradient can be asked for
    conv = SNN_conv(8, 16, 3, 1).cuda()
    dense = SNN_dense(9 * 9 * 16, 10).cuda()
    xin = xcd.clone().requires_grad_(True)
    y_train = dense(conv(xin).reshape(2, -1))
    with torch.no_grad():
        y_eval = dense(conv(xin).reshape(2, -1))
    assert torch.equal(y_train.detach(), y_eval)


def test_inference_forward_against_the_oracle_and_its_causal_set_histogram():
    """snntc_fc_infer / snntc_cv_infer held to the forward protocol directly (not through the training forward),
    and the k histogram against the oracle's count of consumed inputs."""
    import torch
    from snntc_2023_b200 import ops
    # dense, reference tests' distribution: outputs fire early (median k about a third of the fan-in)
    B, I, J = 48, 300, 200
    x, w = P.make_inputs(63, (B, I), (I + 1, J), "test")
    params = O.fc_params(biasvolt=1.0)
    kh = torch.zeros(I + 2, dtype=torch.int32, device="cuda")
    y = ops.snn_fc_infer(torch.from_numpy(x).cuda(), torch.from_numpy(w).cuda(), params, khist=kh).cpu().numpy()
    o32, o64 = O.fc_forward(x, w, params, "f32"), O.fc_forward(x, w, params, "f64")
    P.check_forward(y, None, o32, o64, rows=x, what="dense inference forward")
    kh = kh.cpu().numpy()
    assert kh.sum() == B * J
    fired = o64["y"] < 1e5 - 0.1
    want = np.bincount(o64["k"][fired], minlength=I + 2)
    want[I + 1] = (~fired).sum()
    # outputs the oracle flags as ill-conditioned may land one bin away or in the no-spike bin
    assert np.abs(kh - want).sum() <= 2 * o64["illc"].sum() + 2
    assert kh[I + 1] > 0 and kh[:I + 1].sum() > 0
    # conv, a hidden layer of the benchmark networks
    Bc, H, W, C, Kc = 2, 8, 8, 64, 64
    xc, wc = P.make_inputs(64, (Bc, H, W, C), (9 * C + 1, Kc), "ref", bias=True)
    pc = O.cv_params(3, 3, 1, 1, "SAME", 1.0)
    khc = torch.zeros(9 * C + 2, dtype=torch.int32, device="cuda")
    yc = ops.snn_cv_infer(torch.from_numpy(xc).cuda(), torch.from_numpy(wc).cuda(), pc, 1, 1, H, W, khist=khc).cpu().numpy()
    c32, c64 = O.cv_forward(xc, wc, pc, "f32"), O.cv_forward(xc, wc, pc, "f64")
    P.check_forward(yc, None, c32, c64, rows=P.im2col_rows(xc, 3, 3, 1, 1, "SAME"), what="conv inference forward")
    khc = khc.cpu().numpy()
    firedc = c64["y"] < 1e5 - 0.1
    wantc = np.bincount(c64["k"][firedc], minlength=9 * C + 2)
    wantc[9 * C + 1] = (~firedc).sum()
    assert khc.sum() == firedc.size and np.abs(khc - wantc).sum() <= 2 * c64["illc"].sum() + 2


def test_minpool_backward_is_a_gather_for_overlapping_windows():
    """3x3 windows at stride 1 and 2 overlap: an input can win several windows. The backward sums their gradients
    in window order (no atomics): two runs give the same bits, and the sum matches numpy."""
    import torch
    from snntc_2023_b200 import ops
    rng = np.random.default_rng(9)
    for (H, W, K, S) in ((9, 8, 3, 1), (11, 7, 3, 2), (6, 6, 4, 2)):
        x = np.exp(rng.random((3, H, W, 5))).astype(np.float32)
        x[rng.random(x.shape) < 0.4] = 1e5
        xd = torch.from_numpy(x).cuda().requires_grad_(True)
        y = ops.snn_minpool(xd, K, K, S, S, "SAME")
        g = torch.randn_like(y)
        (dx1,) = torch.autograd.grad(y, xd, g, retain_graph=True)
        (dx2,) = torch.autograd.grad(y, xd, g)
        assert torch.equal(dx1, dx2)
        _, arg = O.minpool(x, K, K, S, S, "SAME")
        want = np.zeros(x.size, np.float64)
        ok = arg.reshape(-1) >= 0
        np.add.at(want, arg.reshape(-1)[ok], g.cpu().numpy().reshape(-1)[ok].astype(np.float64))
        assert np.allclose(dx1.cpu().numpy().reshape(-1), want, rtol=1e-5, atol=1e-6)
