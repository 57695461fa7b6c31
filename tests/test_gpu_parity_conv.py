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
    # the conv layers of the benchmark networks at reduced batch and image size, exact channel counts and fan-in
    # (577, 1153, 2305, 4609 with the bias row); "ref": reference initialisation, inputs with sentinels
    (81, 2, 10, 10, 3, 3, 3, 1, 1, 64, 1.0, "SAME", "cfg"),      # first layer: every input spikes
    (82, 2, 10, 10, 64, 3, 3, 1, 1, 64, 1.0, "SAME", "ref"),
    (83, 2, 8, 8, 64, 3, 3, 1, 1, 128, 1.0, "SAME", "ref"),
    (84, 2, 8, 8, 128, 3, 3, 1, 1, 128, 1.0, "SAME", "ref"),
    (85, 1, 8, 8, 128, 3, 3, 1, 1, 256, 1.0, "SAME", "ref"),
    (86, 1, 8, 8, 256, 3, 3, 1, 1, 256, 1.0, "SAME", "ref"),
    (87, 1, 8, 8, 256, 3, 3, 1, 1, 256, 1.0, "SAME", "cfg"),
    (88, 1, 7, 7, 256, 3, 3, 1, 1, 512, 1.0, "SAME", "ref"),
    (89, 1, 7, 7, 512, 3, 3, 1, 1, 512, 1.0, "SAME", "ref"),
    (90, 2, 32, 32, 3, 7, 7, 2, 2, 64, 1.0, "SAME", "cfg"),      # ImageNet-shaped first layer, 7x7 stride 2
    (91, 2, 32, 32, 64, 3, 3, 1, 1, 128, 0.0, "SAME", "cfg"),    # config 3: 32x32x64 -> 128, no bias
    (92, 4, 32, 32, 64, 3, 3, 1, 1, 64, 1.0, "SAME", "ref"),     # 4096 rows: the row-skipping dW kernel, several slices
    (93, 3, 9, 7, 32, 3, 2, 1, 1, 48, 1.0, "VALID", "ref"),      # merged lists with a 3x2 kernel, VALID, odd sizes
    (94, 2, 6, 9, 20, 2, 3, 1, 1, 12, 0.0, "SAME", "test"),      # 2x3 kernel, asymmetric SAME padding, C not a multiple of 32
    (96, 2, 11, 9, 16, 3, 3, 2, 1, 24, 1.0, "SAME", "test"),     # strides 2x1: the list-walking dX kernel with strided taps
    # shapes of the tensor-map dW kernel beyond the benchmark layers: a map 4 wide (boxes of four image rows), a 2x2
    # kernel (SAME pads only below and right), 32 and 16 channels, a fan-out that is no multiple of 32
    (97, 4, 4, 4, 32, 3, 3, 1, 1, 64, 1.0, "SAME", "ref"),
    (98, 2, 16, 16, 16, 2, 2, 1, 1, 40, 1.0, "SAME", "cfg"),
    (99, 3, 16, 2, 64, 3, 1, 1, 1, 32, 0.0, "SAME", "ref"),      # a map 2 wide, a 3x1 kernel, no bias
    (100, 1, 5, 5, 4, 7, 7, 1, 1, 8, 1.0, "SAME", "test"),       # 4 channels under a 7x7 window: 49 taps, one per lane
    (101, 2, 1, 1, 16, 1, 1, 1, 1, 4, 1.0, "SAME", "test"),      # a 1x1 map, a 1x1 kernel: one field per stage
    (102, 1, 3, 40, 32, 3, 3, 1, 1, 36, 1.0, "SAME", "ref"),     # a map 40 wide: blocks of 16, 16 and 8 columns
]


def _ids(c):
    return "s%d_B%d_%dx%dx%d_K%dx%d_S%d%d_Kc%d_b%g_%s_%s" % c


def _run_conv(seed, B, H, W, C, Kh, Kw, Sh, Sw, Kc, bv, padding, dist):
    import torch
    from snntc_2023_b200 import ops
    I = Kh * Kw * C
    x, w = P.make_inputs(seed, (B, H, W, C), (I + (bv > 1e-8), Kc), dist, bias=bv > 1e-8)
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


# ---- kernel variants against each other (measurement build: the kernel choice of a call is given explicitly)
VARIANT_CASES = [c for c in CONV_CASES if c[0] in (44, 48, 51, 82, 84, 86, 92, 93, 94, 96, 97, 98, 99, 100, 101, 102)]


@pytest.mark.parametrize("case", VARIANT_CASES, ids=_ids)
def test_conv_list_builders_agree(case):
    """Sorted lists by per-field radix sort and by per-pixel sort + merges: the same lists up to the order of equal
    inputs, which can move the last bits of a sum but not a decision on a well-conditioned output."""
    import torch
    from snntc_2023_b200 import _lib, ops
    seed, B, H, W, C, Kh, Kw, Sh, Sw, Kc, bv, padding, dist = case
    x, w, params, xd, wd, out, outc, (pt, pl, Nh, Nw) = _run_conv(*case)
    a = ops.snn_cv(xd, wd, params, pt, pl, Nh, Nw, opts=_lib.options(list_builder=1)).cpu().numpy()
    b = ops.snn_cv(xd, wd, params, pt, pl, Nh, Nw, opts=_lib.options(list_builder=2)).cpu().numpy()
    assert np.array_equal(outc, b), "the default list builder of a 3x3 stride-1 layer is the merging one"
    fa, fb = a[:B] < 1e5 - 0.1, b[:B] < 1e5 - 0.1
    assert (fa != fb).sum() <= 1e-4 * fa.size
    both = fa & fb
    np.testing.assert_allclose(a[:B][both], b[:B][both], rtol=2e-6, atol=0)
    # the pre-padded calling convention goes through the same builder
    xp = O.pad_like_reference(x, Kh, Kw, Sh, Sw, padding)
    bp = ops.snn_cv(torch.from_numpy(xp).cuda(), wd, params, opts=_lib.options(list_builder=2)).cpu().numpy()
    assert np.array_equal(bp, b)
    # merges cut into 1, 2, 8 and 32 pieces build the same lists entry for entry
    for k in (0, 1, 3, 5):
        c = ops.snn_cv(xd, wd, params, pt, pl, Nh, Nw, opts=_lib.options(list_builder=2 + 4 * (k + 1))).cpu().numpy()
        assert np.array_equal(c, b), "pieces per merge: %d" % (1 << k)


SMALL_ROW_CASES = [c for c in CONV_CASES if c[5] * c[6] * c[4] <= 256]


@pytest.mark.parametrize("case", SMALL_ROW_CASES, ids=_ids)
def test_conv_small_row_builder_matches_the_row_sort(case):
    """Rows of at most 256 inputs sorted by the register network and by the per-row radix sort: both order equal
    inputs by source index, so the lists and with them every output bit are the same."""
    from snntc_2023_b200 import _lib, ops
    x, w, params, xd, wd, out, outc, (pt, pl, Nh, Nw) = _run_conv(*case)
    a = ops.snn_cv(xd, wd, params, pt, pl, Nh, Nw, opts=_lib.options(list_builder=1)).cpu().numpy()
    b = ops.snn_cv(xd, wd, params, pt, pl, Nh, Nw, opts=_lib.options(list_builder=3)).cpu().numpy()
    assert np.array_equal(a, b)


@pytest.mark.parametrize("case", VARIANT_CASES, ids=_ids)
def test_conv_dw_kernels_agree(case):
    """dW by the dense register-tile kernel and by the row-skipping kernel: the same sums in a different grouping."""
    import torch
    from snntc_2023_b200 import _lib, ops
    seed, B, H, W, C, Kh, Kw, Sh, Sw, Kc, bv, padding, dist = case
    if C % 4 or Kc % 4:
        pytest.skip("the row-skipping kernel needs channel counts that are multiples of 4")
    x, w, params, xd, wd, out, outc, (pt, pl, Nh, Nw) = _run_conv(*case)
    g = np.random.default_rng(seed + 2000).standard_normal((B, Nh, Nw, Kc)).astype(np.float32)
    g[np.random.default_rng(seed).random(g.shape) < 0.5] = 0          # gradients routed through a pooling layer are sparse
    gd = torch.from_numpy(g).cuda()
    _, dw1, _ = ops.snn_cv_grad(gd, xd, wd, params, out, pt, pl, opts=_lib.options(dw_kernel=1))
    dx2, dw2, _ = ops.snn_cv_grad(gd, xd, wd, params, out, pt, pl, opts=_lib.options(dw_kernel=2))
    ref = O.cv_backward(g, x, w, params, outc[:B], outc[B:], "f64")
    P.check_close(dw1.cpu().numpy(), ref["dw"], "dense-tile dW %s" % (case,), abs_sum=ref["dw_abs"])
    P.check_close(dw2.cpu().numpy(), ref["dw"], "row-skipping dW %s" % (case,), abs_sum=ref["dw_abs"])
    P.check_close(dx2.cpu().numpy(), ref["dx"], "dX beside the row-skipping dW %s" % (case,), abs_sum=ref["dx_abs"])
    # twice the same call: no atomics, identical bits
    _, dw3, _ = ops.snn_cv_grad(gd, xd, wd, params, out, pt, pl, opts=_lib.options(dw_kernel=2))
    assert torch.equal(dw2, dw3)
    # the same kernel fed through tensor maps (where the shape allows; elsewhere this is the call above again)
    _, dw5, _ = ops.snn_cv_grad(gd, xd, wd, params, out, pt, pl, opts=_lib.options(dw_kernel=4))
    P.check_close(dw5.cpu().numpy(), ref["dw"], "row-skipping dW through tensor maps %s" % (case,), abs_sum=ref["dw_abs"])
    _, dw6, _ = ops.snn_cv_grad(gd, xd, wd, params, out, pt, pl, opts=_lib.options(dw_kernel=4))
    assert torch.equal(dw5, dw6)
    assert _lib.load_measure().snntc_copy_timeouts() == 0
    # a value outside the range of the scaled inner loop (|u| >= 2^100) sends the kernel through its unscaled loop
    j_fired = int(np.argmax(outc[0, 0, 0, :] < 1e5 - 0.1))
    g[0, 0, 0, j_fired] = 4e30
    gd = torch.from_numpy(g).cuda()
    _, dw4, _ = ops.snn_cv_grad(gd, xd, wd, params, out, pt, pl, opts=_lib.options(dw_kernel=2))
    ref = O.cv_backward(g, x, w, params, outc[:B], outc[B:], "f64")
    with np.errstate(over="ignore", invalid="ignore"):
        P.check_close(dw4.cpu().numpy(), ref["dw"], "row-skipping dW, unscaled loop %s" % (case,), abs_sum=ref["dw_abs"])
        # the tensor-map kernel's unscaled loop: its out-of-image inputs are NaN and must still count as "never spikes"
        _, dw7, _ = ops.snn_cv_grad(gd, xd, wd, params, out, pt, pl, opts=_lib.options(dw_kernel=4))
        P.check_close(dw7.cpu().numpy(), ref["dw"], "tensor-map dW, unscaled loop %s" % (case,), abs_sum=ref["dw_abs"])


@pytest.mark.parametrize("case", VARIANT_CASES, ids=_ids)
def test_conv_dx_kernels_agree(case):
    """dX by the dense register-tile kernels and by the kernel that walks the lists of outputs with a gradient: the
    same terms added in the same order (the skipped ones are zeros), hence the same bits."""
    import torch
    from snntc_2023_b200 import _lib, ops
    seed, B, H, W, C, Kh, Kw, Sh, Sw, Kc, bv, padding, dist = case
    if C % 4 or C < 16:
        pytest.skip("the list-walking kernel needs a channel count that is a multiple of 4, at least 16")
    x, w, params, xd, wd, out, outc, (pt, pl, Nh, Nw) = _run_conv(*case)
    for zero_share in (0.0, 0.8):
        g = np.random.default_rng(seed + 3000).standard_normal((B, Nh, Nw, Kc)).astype(np.float32)
        g[np.random.default_rng(seed + 1).random(g.shape) < zero_share] = 0
        gd = torch.from_numpy(g).cuda()
        dx1, _, _ = ops.snn_cv_grad(gd, xd, wd, params, out, pt, pl, opts=_lib.options(dx_kernel=1))
        dx2, dw2, _ = ops.snn_cv_grad(gd, xd, wd, params, out, pt, pl, opts=_lib.options(dx_kernel=2))
        ref = O.cv_backward(g, x, w, params, outc[:B], outc[B:], "f64")
        P.check_close(dx2.cpu().numpy(), ref["dx"], "list-walking dX %s" % (case,), abs_sum=ref["dx_abs"])
        P.check_close(dw2.cpu().numpy(), ref["dw"], "dW beside the list-walking dX %s" % (case,), abs_sum=ref["dw_abs"])
        assert torch.equal(dx1, dx2), "dense and list-walking dX differ in bits"
        # the library's own choice queues both and lets the device pick by the share of outputs with a gradient (the
        # dense one at no zeros, the list-walking one at 80 % zeros): the same bits either way, and dx fully written
        dx0, _, _ = ops.snn_cv_grad(gd, xd, wd, params, out, pt, pl, opts=_lib.options())
        assert torch.equal(dx0, dx1)
        assert torch.equal(ops.snn_cv_grad(gd, xd, wd, params, out, pt, pl)[0], dx1)   # product library
    # the pre-padded calling convention: padding pixels hold MAX and get a zero gradient
    xp = torch.from_numpy(O.pad_like_reference(x, Kh, Kw, Sh, Sw, padding)).cuda()
    a, _, _ = ops.snn_cv_grad(gd, xp, wd, params, out, opts=_lib.options(dx_kernel=1))
    b, _, _ = ops.snn_cv_grad(gd, xp, wd, params, out, opts=_lib.options(dx_kernel=2))
    assert torch.equal(a, b)


def test_small_fan_in_dw_kernel_matches_the_tile_kernel():
    """A first layer on three channels has 28 weight rows: its dW runs in the kernel for small fan-in (one lane per
    weight row) when there are enough receptive fields, and in the register-tile kernel when forced."""
    import torch
    from snntc_2023_b200 import _lib, ops
    case = [c for c in CONV_CASES if c[0] == 52][0]
    seed, B, H, W, C, Kh, Kw, Sh, Sw, Kc, bv, padding, dist = case
    x, w, params, xd, wd, out, outc, (pt, pl, Nh, Nw) = _run_conv(*case)
    g = np.random.default_rng(seed + 4000).standard_normal((B, Nh, Nw, Kc)).astype(np.float32)
    g[np.random.default_rng(seed + 2).random(g.shape) < 0.6] = 0
    gd = torch.from_numpy(g).cuda()
    _, dw_small, _ = ops.snn_cv_grad(gd, xd, wd, params, out, pt, pl, need_input_grad=False)
    _, dw_tile, _ = ops.snn_cv_grad(gd, xd, wd, params, out, pt, pl, need_input_grad=False, opts=_lib.options(dw_kernel=1))
    ref = O.cv_backward(g, x, w, params, outc[:B], outc[B:], "f64", want_dx=False)
    P.check_close(dw_small.cpu().numpy(), ref["dw"], "small fan-in dW", abs_sum=ref["dw_abs"])
    P.check_close(dw_tile.cpu().numpy(), ref["dw"], "tile dW", abs_sum=ref["dw_abs"])
    _, again, _ = ops.snn_cv_grad(gd, xd, wd, params, out, pt, pl, need_input_grad=False)
    assert torch.equal(again, dw_small)


def test_conv_inputs_that_never_spike_or_are_not_numbers():
    """Whole pixels, whole channels and single inputs at MAX: empty pixel runs, empty row runs and empty lists."""
    import torch
    from snntc_2023_b200 import ops
    B, H, W, C, Kc = 2, 7, 6, 32, 16
    x, w = P.make_inputs(95, (B, H, W, C), (9 * C + 1, Kc), "ref", bias=True)
    x[0, 2, :, :] = 1e5          # a whole image row
    x[:, :, :, 5] = 1e5          # a whole channel
    x[1] = 1e5                   # a whole image: every list empty, only the bias input is left
    params = O.cv_params(3, 3, 1, 1, "SAME", 1.0)
    xd, wd = torch.from_numpy(x).cuda(), torch.from_numpy(w).cuda()
    out = ops.snn_cv(xd, wd, params, 1, 1, H, W).cpu().numpy()
    P.check_forward(out[:B], out[B:], O.cv_forward(x, w, params, "f32"), O.cv_forward(x, w, params, "f64"),
                    rows=P.im2col_rows(x, 3, 3, 1, 1, "SAME"), what="conv with empty lists")
