"""GPU parity of SnnFc / SnnFcGrad against the oracle, through the C ABI (ctypes) on torch buffers."""
import numpy as np
import pytest

import oracle as O
from tests import parity as P

pytestmark = pytest.mark.gpu

# (seed, B, I, J, biasvolt, dist) -- shapes in the spirit of test-snn-fc-forward.py:25-32 (1..1000, odd sizes)
DENSE_CASES = [
    (11, 37, 300, 200, 1.0, "test"),
    (12, 64, 784, 400, 0.0, "cfg"),
    (13, 5, 1, 1, 1.0, "test"),
    (14, 1, 17, 33, 0.0, "test"),
    (15, 129, 999, 65, 1.0, "test"),
    (16, 70, 513, 10, 1.0, "cfg"),
    (17, 33, 64, 130, 0.5, "test"),
    (18, 16, 2049, 96, 1.0, "cfg"),
    (19, 3, 16000, 40, 1.0, "cfg"),     # too long for two shared-memory sort buffers: bitonic fallback
    (20, 6, 4097, 512, 1.0, "cfg"),
    (22, 40, 31, 64, 1.0, "test"),      # <= 32 inputs: shuffle rank sort
    (23, 40, 33, 128, 0.0, "test"),
    (25, 18945, 24, 64, 1.0, "cfg"),    # many more rows than resident warps, odd row count
    (26, 19000, 40, 36, 0.0, "test"),   # the same with a ragged last block of outputs
    # the dense layers of the benchmark networks at reduced batch, reference initialisation ("ref": inputs with
    # sentinels as a hidden layer sees them) and the benchmark's own weight family ("cfg")
    (61, 8, 784, 400, 1.0, "ref"),      # MNIST-shaped MLP
    (62, 8, 400, 400, 1.0, "ref"),
    (63, 16, 400, 10, 1.0, "ref"),
    (64, 4, 4096, 512, 1.0, "ref"),     # CIFAR-shaped net
    (65, 4, 4096, 512, 1.0, "cfg"),
    (66, 16, 512, 10, 1.0, "ref"),
    (67, 2, 25088, 1024, 1.0, "ref"),   # ImageNet-shaped net: CTA-wide sort for the long row
    (68, 2, 25088, 1024, 1.0, "cfg"),
    (69, 4, 1024, 1000, 1.0, "ref"),
    (70, 4, 1024, 1000, 1.0, "cfg"),
]


def _run_dense(seed, B, I, J, bv, dist):
    import torch
    from snntc_2023_b200 import ops
    x, w = P.make_inputs(seed, (B, I), (I + (bv > 1e-8), J), dist, bias=bv > 1e-8)
    params = O.fc_params(biasvolt=bv)
    dev = torch.device("cuda:0")
    xd, wd = torch.from_numpy(x).to(dev), torch.from_numpy(w).to(dev)
    out = ops.snn_fc(xd, wd, params)
    assert out.shape == (2 * B, J)
    outc = out.cpu().numpy()
    return x, w, params, xd, wd, out, outc


@pytest.mark.parametrize("case", DENSE_CASES, ids=lambda c: "s%d_B%d_I%d_J%d_b%g_%s" % c)
def test_dense_forward(case):
    seed, B, I, J, bv, dist = case
    x, w, params, xd, wd, out, outc = _run_dense(*case)
    o32 = O.fc_forward(x, w, params, "f32")
    o64 = O.fc_forward(x, w, params, "f64")
    P.check_forward(outc[:B], outc[B:], o32, o64, rows=x, what="dense fwd %s" % (case,))


@pytest.mark.parametrize("case", DENSE_CASES, ids=lambda c: "s%d_B%d_I%d_J%d_b%g_%s" % c)
def test_dense_backward(case):
    import torch
    from snntc_2023_b200 import ops
    seed, B, I, J, bv, dist = case
    x, w, params, xd, wd, out, outc = _run_dense(*case)
    rng = np.random.default_rng(seed + 1000)
    g = rng.standard_normal((B, J)).astype(np.float32)
    g2 = np.concatenate([g, np.zeros_like(g)])
    dx, dw, dp = ops.snn_fc_grad(torch.from_numpy(g2).cuda(), xd, wd, params, out)
    ref = O.fc_backward(g, x, w, params, outc[:B], outc[B:], "f64")
    P.check_close(dx.cpu().numpy(), ref["dx"], "dense dX %s" % (case,), abs_sum=ref["dx_abs"])
    P.check_close(dw.cpu().numpy(), ref["dw"], "dense dW %s" % (case,), abs_sum=ref["dw_abs"])
    assert np.all(dp.cpu().numpy() == 0)
    # the unpacked [B,J] gradient gives the same result, and dx may be skipped
    dx2, dw2, _ = ops.snn_fc_grad(torch.from_numpy(g).cuda(), xd, wd, params, out, need_input_grad=False)
    assert dx2 is None
    assert torch.equal(dw2, dw)


def test_dense_sentinel_inputs():
    """Inputs at MAX never spike and get no gradient (snnfc_kernels.cu.cc:45, snnfcgrad_kernels.cu.cc:113)."""
    import torch
    from snntc_2023_b200 import ops
    seed, B, I, J, bv = 21, 9, 40, 50, 1.0
    x, w = P.make_inputs(seed, (B, I), (I + 1, J), "test")
    x[:, ::3] = 1e5
    x[0, :] = 1e5
    params = O.fc_params(biasvolt=bv)
    xd, wd = torch.from_numpy(x).cuda(), torch.from_numpy(w).cuda()
    out = ops.snn_fc(xd, wd, params)
    outc = out.cpu().numpy()
    P.check_forward(outc[:B], outc[B:], O.fc_forward(x, w, params, "f32"), O.fc_forward(x, w, params, "f64"),
                    what="sentinel fwd")
    g = np.random.default_rng(3).standard_normal((B, J)).astype(np.float32)
    dx, dw, _ = ops.snn_fc_grad(torch.from_numpy(g).cuda(), xd, wd, params, out)
    ref = O.fc_backward(g, x, w, params, outc[:B], outc[B:], "f64")
    P.check_close(dx.cpu().numpy(), ref["dx"], "sentinel dX", abs_sum=ref["dx_abs"])
    P.check_close(dw.cpu().numpy(), ref["dw"], "sentinel dW", abs_sum=ref["dw_abs"])
    assert np.all(dx.cpu().numpy()[:, ::3] == 0)


@pytest.mark.parametrize("J", [1, 2, 10, 64, 128, 256])
@pytest.mark.parametrize("bv", [0.0, 1.0])
def test_dense_weight_sum_cancels_exactly(J, bv):
    """sum(w) - theta == +0 after the last input with a positive weighted sum: the reference takes 1/0 = +inf,
    so the spike value is +inf >= MAX and the output reads "no spike" (MAX, 0) (snnfc_kernels.cu.cc:60-68).
    Every way the walk carries its sums (scalar, pairs, negated) has to land on the same side of zero."""
    import torch
    from snntc_2023_b200 import ops
    x = np.array([[1.5, 2.0], [2.0, 1.5], [1.25, 1.75]], np.float32)
    rows = [[0.25] * J, [0.5] * J] + ([[0.25] * J] if bv > 0 else [])   # bias row last
    if bv == 0:
        rows = [[0.5] * J, [0.5] * J]
    w = np.array(rows, np.float32)
    w[:, J // 2:] += np.float32(0.125) * (J > 1)    # other half: an ordinary finite spike beside the cancelled one
    params = O.fc_params(biasvolt=bv)
    out = ops.snn_fc(torch.from_numpy(x).cuda(), torch.from_numpy(w).cuda(), params).cpu().numpy()
    ref = O.fc_forward(x, w, params, "f32")
    assert np.array_equal(out[:3], ref["y"]) and np.array_equal(out[3:], ref["inv"])
    ncancel = J // 2 if J > 1 else 1
    assert np.all(out[:3, :ncancel] == 1e5) and np.all(out[3:, :ncancel] == 0)
    assert np.all(np.isfinite(out))


@pytest.mark.parametrize("odd", ["below_minus_max", "tiny", "huge_grad"])
def test_dense_backward_values_outside_the_scaled_range(odd):
    """The dW kernel's scaled inner loop is exact only for inputs >= -MAX, magnitudes that do not underflow
    when scaled and gradients below 2^100; anything else must take its unscaled loop and still match."""
    import torch
    from snntc_2023_b200 import ops
    seed, B, I, J, bv = 24, 33, 70, 64, 1.0
    x, w = P.make_inputs(seed, (B, I), (I + 1, J), "test")
    g = np.random.default_rng(4).standard_normal((B, J)).astype(np.float32)
    if odd == "below_minus_max":
        x[0, 0] = -3e5
    elif odd == "tiny":
        x[1, 1] = 1e-30
    else:
        g[2, 3] = 1e36
    params = O.fc_params(biasvolt=bv)
    xd, wd = torch.from_numpy(x).cuda(), torch.from_numpy(w).cuda()
    out = ops.snn_fc(xd, wd, params)
    outc = out.cpu().numpy()
    dx, dw, _ = ops.snn_fc_grad(torch.from_numpy(g).cuda(), xd, wd, params, out)
    ref = O.fc_backward(g, x, w, params, outc[:B], outc[B:], "f64")
    with np.errstate(over="ignore", invalid="ignore"):
        P.check_close(dw.cpu().numpy(), ref["dw"], "dW %s" % odd, abs_sum=ref["dw_abs"])
        P.check_close(dx.cpu().numpy(), ref["dx"], "dX %s" % odd, abs_sum=ref["dx_abs"])


def test_dense_repeatable():
    """No atomics on the dense path: two runs give identical bits."""
    import torch
    from snntc_2023_b200 import ops
    x, w, params, xd, wd, out, outc = _run_dense(31, 100, 300, 77, 1.0, "test")
    out2 = ops.snn_fc(xd, wd, params)
    assert torch.equal(out, out2)
    g = torch.randn(100, 77, device="cuda", generator=torch.Generator("cuda").manual_seed(1))
    a = ops.snn_fc_grad(g, xd, wd, params, out)
    b = ops.snn_fc_grad(g, xd, wd, params, out)
    assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])


@pytest.mark.parametrize("I", [1, 31, 32, 33, 64, 70, 100, 147, 170, 200, 255, 256])
def test_dense_short_rows_by_the_register_network_match_the_row_sort(I):
    """Rows of at most 256 inputs are sorted by a network in registers; the per-row radix sort forced through the
    measurement build gives the same lists (equal inputs in index order), hence the same bits. Inputs include
    ties and values that never spike."""
    import torch
    from snntc_2023_b200 import _lib, ops
    rng = np.random.default_rng(I)
    x = np.round(np.exp(rng.random((37, I)) * 2), 2).astype(np.float32)
    x[rng.random(x.shape) < 0.2] = 1e5
    w = (rng.standard_normal((I + 1, 48)) * np.sqrt(15.0 / I)).astype(np.float32)
    params = O.fc_params(biasvolt=1.0)
    xd, wd = torch.from_numpy(x).cuda(), torch.from_numpy(w).cuda()
    a = ops.snn_fc(xd, wd, params, opts=_lib.options(list_builder=1))
    b = ops.snn_fc(xd, wd, params, opts=_lib.options(list_builder=3))
    assert torch.equal(a, b) and torch.equal(b, ops.snn_fc(xd, wd, params))
    bc = b.cpu().numpy()
    P.check_forward(bc[:37], bc[37:], O.fc_forward(x, w, params, "f32"), O.fc_forward(x, w, params, "f64"), rows=x,
                    what="short rows I=%d" % I)


def test_walk_variants_agree_bit_for_bit():
    """The library picks among several walk kernels (output pairs, consecutive outputs per lane, strided outputs,
    1/2/4/8 outputs per lane); forced one by one through the measurement build they must give identical bits."""
    import torch
    from snntc_2023_b200 import _lib, ops
    x, w = P.make_inputs(71, (50, 300), (301, 256), "cfg")
    params = O.fc_params(biasvolt=1.0)
    xd, wd = torch.from_numpy(x).cuda(), torch.from_numpy(w).cuda()
    ref = ops.snn_fc(xd, wd, params)
    for layout in (1, 2, 3, 5, 6, 7):      # 5..7: the same layouts reading list entries straight from global memory
        for outputs in (0, 1, 2, 3, 4):
            out = ops.snn_fc(xd, wd, params, opts=_lib.options(walk_layout=layout, walk_outputs=outputs))
            assert torch.equal(out, ref), "layout %d, outputs-per-lane choice %d" % (layout, outputs)
    # the pairs walk with the weights of 64 outputs staged in shared memory by asynchronous bulk copies (8, 12: with and
    # without staged list entries), one and several slices of 64 outputs, with and without bias row, more rows than warps
    for (B, I, J, bv) in ((50, 300, 256, 1.0), (2100, 37, 64, 1.0), (70, 577, 128, 0.0), (3, 799, 64, 1.0)):
        x, w = P.make_inputs(73 + I, (B, I), (I + (1 if bv else 0), J), "cfg")
        prm = O.fc_params(biasvolt=bv)
        xd, wd = torch.from_numpy(x).cuda(), torch.from_numpy(w).cuda()
        ref = ops.snn_fc(xd, wd, prm, opts=_lib.options(walk_layout=1))
        for layout in (8, 12):
            assert torch.equal(ops.snn_fc(xd, wd, prm, opts=_lib.options(walk_layout=layout)), ref), (B, I, J, bv, layout)
    assert _lib.load_measure().snntc_copy_timeouts() == 0
    # a fan-out that leaves the last block of eight-per-lane outputs partly empty
    x, w = P.make_inputs(72, (20, 100), (101, 1000), "test")
    params = O.fc_params(biasvolt=1.0)
    xd, wd = torch.from_numpy(x).cuda(), torch.from_numpy(w).cuda()
    ref = ops.snn_fc(xd, wd, params, opts=_lib.options(walk_layout=2, walk_outputs=1))
    for outputs in (2, 3, 4):
        assert torch.equal(ops.snn_fc(xd, wd, params, opts=_lib.options(walk_layout=3, walk_outputs=outputs)), ref)


def _small_grid_problem(seed, B, I, J, bv, lo, hi):
    """Inputs and weights on a grid of quarters: every sum of the walk is exact in fp32, so the fp32 restatement IS
    the reference's result and ties between a spike time and an input are exact, not accidents of rounding."""
    rng = np.random.default_rng(seed)
    x = (rng.integers(lo, hi, size=(B, I)) / 4.0).astype(np.float32)
    w = (rng.integers(-12, 13, size=(I + (bv > 1e-8), J)) / 4.0).astype(np.float32)
    return x, w


@pytest.mark.parametrize("J", [1, 2, 64, 128, 256, 250])
@pytest.mark.parametrize("bv", [0.0, 1.0])
def test_dense_exact_ties_between_spike_time_and_next_input(J, bv):
    """The reference fires when the spike time EQUALS the next input (ysumabs <= x*wsumabs,
    snntc/snnfc_kernels.cu.cc:46); with small-integer data such ties are exact and frequent (the reference's
    own tests name them as the source of their mismatches, test-snn-fc-forward.py:74-77). Every walk variant
    must take the reference's side of the tie."""
    import torch
    from snntc_2023_b200 import ops
    x, w = _small_grid_problem(300 + J, 64, 6, J, bv, 4, 17)        # inputs 1.0 .. 4.0, at or above the bias input
    params = O.fc_params(biasvolt=bv)
    out = ops.snn_fc(torch.from_numpy(x).cuda(), torch.from_numpy(w).cuda(), params).cpu().numpy()
    ref = O.fc_forward(x, w, params, "f32")
    fired_ref = ref["y"] < 1e5 - 0.1
    # the case really contains ties: outputs whose spike time equals one of the row's inputs
    ties = (fired_ref & (ref["y"][:, None, :] == x[:, :, None]).any(1)).sum()
    assert ties > 0
    assert np.array_equal(out[:64] < 1e5 - 0.1, fired_ref), "fire/no-fire differs on exactly representable data"
    np.testing.assert_allclose(out[:64][fired_ref], ref["y"][fired_ref], rtol=2e-6, atol=0)
    np.testing.assert_allclose(out[64:][fired_ref], ref["inv"][fired_ref], rtol=2e-6, atol=0)


def _rounded_product_rows(w0, n, seed):
    """Rows (x0, x1, x2) for a no-bias output with first weight w0 and threshold 1: after x0 the sums are
    (w0 - 1, x0*w0); x1 is chosen so that ysum is ABOVE the exact product x1*wsum but not above the product rounded to
    fp32 -- the reference, which compares against the rounded product, fires at x1; the exact sign of ysum - x1*wsum
    says "not yet"."""
    f32 = np.float32
    rng = np.random.default_rng(seed)
    ws = f32(f32(w0) - f32(1.0))
    rows = []
    while len(rows) < n:
        x0 = f32(rng.uniform(1.0, 3.0))
        ys = f32(np.float64(x0) * np.float64(f32(w0)))
        x1 = f32(np.float64(ys) / np.float64(ws))
        for _ in range(2):
            x1 = np.nextafter(x1, f32(-np.inf))
        for _ in range(5):
            prod = np.float64(x1) * np.float64(ws)
            if x1 > x0 and ys > f32(np.float64(x0) * np.float64(ws)) and np.float64(ys) > prod and ys <= f32(prod):
                rows.append((x0, x1, f32(x1 * f32(1.5))))
                break
            x1 = np.nextafter(x1, f32(np.inf))
    return np.array(rows, np.float32)


@pytest.mark.parametrize("J", [4, 64, 128, 256])
def test_dense_decision_by_the_rounded_product_like_the_reference(J):
    """The reference decides "spike time <= next input" as ysum <= fl(x*wsum) (snntc/snnfc_kernels.cu.cc:46-48): it
    can fire while the exact difference ysum - x*wsum is still positive by less than the rounding of the product.
    The walk's sign test alone would miss that step; its margin hands it to the reference's comparison. Constructed
    rows where that happens for output 0, every walk layout, results bit for bit those of the fp32 restatement."""
    import torch
    from snntc_2023_b200 import _lib, ops
    x = _rounded_product_rows(2.3, 96, J)
    rng = np.random.default_rng(J)
    w = rng.uniform(-1.0, 1.5, (3, J)).astype(np.float32)
    w[:, 0] = (2.3, 0.7, 0.9)
    params = O.fc_params(biasvolt=0.0)
    ref = O.fc_forward(x, w, params, "f32")
    assert np.all(ref["k"][:, 0] == 1), "the reference consumes one input and fires at the second"
    xd, wd = torch.from_numpy(x).cuda(), torch.from_numpy(w).cuda()
    outs = [ops.snn_fc(xd, wd, params)]
    outs += [ops.snn_fc(xd, wd, params, opts=_lib.options(walk_layout=lay)) for lay in (1, 2, 3, 8)]
    fired = ref["y"] < 1e5 - 0.1
    assert fired[:, 0].all()
    for o in outs:
        assert torch.equal(o, outs[0])                               # every layout: the same bits
        o = o.cpu().numpy()
        assert np.array_equal(o[:96] < 1e5 - 0.1, fired)
        # 1/(sum w - theta) tells which inputs were consumed: 1/1.3 at the second input, 1/2.0 one input later
        np.testing.assert_allclose(o[96:][fired], ref["inv"][fired], rtol=2e-6, atol=0)
        np.testing.assert_allclose(o[:96][fired], ref["y"][fired], rtol=2e-6, atol=0)


@pytest.mark.parametrize("J", [2, 64, 128, 256])
def test_dense_inputs_below_the_bias_input_fire_with_negative_denominator(J):
    """The reference's tests are sign-safe (snntc/snnfc_kernels.cu.cc:36-38,53-55): with inputs BELOW the bias input
    an output can arm and fire while sum(w) - theta is negative. Sorted inputs at or above the bias input never get
    there, but the operator does not check its inputs, so the walk must follow the reference here too."""
    import torch
    from snntc_2023_b200 import ops
    bv = 2.0
    x, w = _small_grid_problem(400 + J, 96, 5, J, bv, 2, 17)        # inputs 0.5 .. 4.0, bias input at 2.0
    params = O.fc_params(biasvolt=bv)
    out = ops.snn_fc(torch.from_numpy(x).cuda(), torch.from_numpy(w).cuda(), params).cpu().numpy()
    ref = O.fc_forward(x, w, params, "f32")
    fired_ref = ref["y"] < 1e5 - 0.1
    assert (fired_ref & (ref["inv"] < 0)).sum() >= 5, "the case should contain spikes with a negative denominator"
    assert np.array_equal(out[:96] < 1e5 - 0.1, fired_ref)
    np.testing.assert_allclose(out[:96][fired_ref], ref["y"][fired_ref], rtol=2e-6, atol=0)
    np.testing.assert_allclose(out[96:][fired_ref], ref["inv"][fired_ref], rtol=2e-6, atol=0)


def test_dense_unaligned_weight_and_input_pointers():
    """Weights and inputs that start 4 bytes off a 16-byte boundary take the kernels without vector loads."""
    import torch
    from snntc_2023_b200 import ops
    B, I, J = 40, 96, 64
    x, w = P.make_inputs(72, (B, I), (I + 1, J), "test")
    params = O.fc_params(biasvolt=1.0)
    wflat = torch.empty((I + 1) * J + 1, device="cuda")
    wd = wflat[1:].view(I + 1, J)
    wd.copy_(torch.from_numpy(w))
    xflat = torch.empty(B * I + 1, device="cuda")
    xd = xflat[1:].view(B, I)
    xd.copy_(torch.from_numpy(x))
    assert wd.data_ptr() % 16 == 4 and xd.data_ptr() % 16 == 4
    out = ops.snn_fc(xd, wd, params)
    aligned = ops.snn_fc(torch.from_numpy(x).cuda(), torch.from_numpy(w).cuda(), params)
    assert torch.equal(out, aligned)
    g = np.random.default_rng(7).standard_normal((B, J)).astype(np.float32)
    dx, dw, _ = ops.snn_fc_grad(torch.from_numpy(g).cuda(), xd, wd, params, out)
    outc = out.cpu().numpy()
    ref = O.fc_backward(g, x, w, params, outc[:B], outc[B:], "f64")
    P.check_close(dx.cpu().numpy(), ref["dx"], "unaligned dX", abs_sum=ref["dx_abs"])
    P.check_close(dw.cpu().numpy(), ref["dw"], "unaligned dW", abs_sum=ref["dw_abs"])


@pytest.mark.parametrize("span", [1e-4, 0.02, 0.69, 1.5, 2.2, 4.0, 11.0])
def test_dense_forward_over_input_ranges(span):
    """The row sort rebases its keys to the row minimum and sorts only the digits the row's range needs (a top
    digit of one or two bits is a plain split): inputs exp(span*U[0,1)) make the range anything from a few
    hundred key steps to many binades; a mis-sorted row shows up as a wrong causal set."""
    import torch
    from snntc_2023_b200 import ops
    rng = np.random.default_rng(int(span * 1000) + 5)
    B, I, J = 24, 200, 32
    x = np.exp(span * rng.random((B, I))).astype(np.float32)
    x[3, :] = x[3, 0]                      # a row of identical inputs: nothing to sort
    x[4, ::2] = 1e5                        # half of a row never spikes
    w = rng.normal(2.0 / I, 1.0 / np.sqrt(I), (I + 1, J)).astype(np.float32)
    params = O.fc_params(biasvolt=1.0)
    out = ops.snn_fc(torch.from_numpy(x).cuda(), torch.from_numpy(w).cuda(), params).cpu().numpy()
    P.check_forward(out[:B], out[B:], O.fc_forward(x, w, params, "f32"), O.fc_forward(x, w, params, "f64"),
                    rows=x, what="span %g" % span)
