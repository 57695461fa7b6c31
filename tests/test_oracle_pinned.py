"""Pins the oracle (the CPU restatement every GPU parity test trusts) to the reference's own code:
against the committed golden fixtures, which the reference's CPU operators produced, and, where the
compiled reference is present, against it live on further seeded inputs.

The reference CPU and GPU kernels differ in documented ways (strict `x<y` mask and a recomputed
denominator in the CPU gradients; `sum w - theta` instead of its reciprocal in the dense forward
output), so spike values are compared tightly and gradients with the looser bound those differences
allow. Fire/no-fire must agree except where the float64 oracle flags the decision ill-conditioned.
"""
import glob
import os

import numpy as np
import pytest

import oracle as O

GOLD = sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "*.npz")))
MAXV = 1e5


def _fire_and_values(y_ref, o32, o64, what):
    fr = y_ref < MAXV - 0.1
    fo = o32["y"] < MAXV - 0.1
    bad = (fr != fo) & ~o64["illc"]
    assert bad.sum() == 0, "%s: %d fire/no-fire mismatches vs the reference" % (what, bad.sum())
    ok = fr & fo & ~o64["illc"]
    if ok.any():
        tol = np.maximum(1e-4, 4e-7 * o64["cond"][ok])
        rel = np.abs(y_ref[ok] - o32["y"][ok]) / np.abs(o32["y"][ok])
        assert (rel / tol).max() <= 1.0, "%s: spike values differ by rel %.3e" % (what, rel.max())
    return ok


def _grad_close(a, b, what, l2=5e-3):
    nb = np.linalg.norm(b)
    if nb == 0:
        assert np.linalg.norm(a) == 0, what
        return
    r = np.linalg.norm(np.asarray(a, np.float64) - b) / nb
    assert r <= l2, "%s: relative L2 %.3e" % (what, r)


def test_fixtures_present():
    assert len(GOLD) >= 8


@pytest.mark.parametrize("path", GOLD, ids=lambda p: os.path.basename(p)[:-4])
def test_oracle_matches_golden(path):
    d = np.load(path)
    name = os.path.basename(path)
    if name.startswith("dense"):
        x, w, p, g = d["x"], d["w"], d["params"], d["g"]
        B = x.shape[0]
        o32, o64 = O.fc_forward(x, w, p, "f32"), O.fc_forward(x, w, p, "f64")
        ok = _fire_and_values(d["out"][:B], o32, o64, name)
        # the reference CPU op stores (sum w - theta); the GPU op and the oracle store its reciprocal
        if ok.any():
            tol = np.maximum(1e-4, 4e-7 * o64["cond"][ok])
            rel = np.abs(1.0 / d["out"][B:][ok] - o32["inv"][ok]) / np.abs(o32["inv"][ok])
            assert (rel / tol).max() <= 1.0
        bw = O.fc_backward(g, x, w, p, o32["y"], o32["inv"], "f64")
        clean = not ((d["out"][:B] < MAXV - 0.1) != (o32["y"] < MAXV - 0.1)).any()
        if clean:
            _grad_close(d["dx"], bw["dx"], name + " dX")
            _grad_close(d["dw"], bw["dw"], name + " dW")
    else:
        x, w, p, g = d["x"], d["w"], d["params"], d["g"]
        Kh, Kw, Sh, Sw = (int(p[i]) for i in (6, 7, 8, 9))
        padding = str(d["padding"])
        B, H, W, C = x.shape
        o32, o64 = O.cv_forward(x, w, p, "f32"), O.cv_forward(x, w, p, "f64")
        assert o32["y"].shape == d["y"].shape
        _fire_and_values(d["y"], o32, o64, name)
        clean = not ((d["y"] < MAXV - 0.1) != (o32["y"] < MAXV - 0.1)).any()
        bw = O.cv_backward(g, x, w, p, o32["y"], o32["inv"], "f64")
        pt, pl, _, _, Hp, Wp = O.conv_geometry(H, W, Kh, Kw, Sh, Sw, padding)
        if clean:
            inner = d["dxp"][:, pt:pt + min(H, Hp), pl:pl + min(W, Wp), :]
            _grad_close(inner, bw["dx"][:, :inner.shape[1], :inner.shape[2], :], name + " dX")
            _grad_close(d["dw"], bw["dw"], name + " dW")
            if padding == "SAME":   # padding positions receive no gradient in the reference either
                rest = d["dxp"].copy()
                rest[:, pt:pt + H, pl:pl + W, :] = 0
                assert np.abs(rest).max() == 0


needs_ref = pytest.mark.skipif(O.ref_lib() is None, reason="compiled reference CPU operators not present")


@needs_ref
@pytest.mark.parametrize("seed,B,I,J,dist", [(601, 16, 300, 200, "test"), (602, 8, 784, 400, "cfg"), (603, 4, 33, 7, "test")])
def test_oracle_vs_reference_dense_live(seed, B, I, J, dist):
    from tests import parity as P
    x, w = P.make_inputs(seed, (B, I), (I, J), dist)
    p = O.fc_params(biasvolt=0.0)
    out = O.ref_fc_forward(x, w, p)
    o32, o64 = O.fc_forward(x, w, p, "f32"), O.fc_forward(x, w, p, "f64")
    _fire_and_values(out[:B], o32, o64, "dense live %d" % seed)


@needs_ref
@pytest.mark.parametrize("case", [(611, 2, 7, 9, 3, 3, 2, 2, 1, 5, 1.0, "SAME", "test"),
                                  (612, 2, 8, 8, 3, 3, 3, 2, 2, 4, 1.0, "SAME", "test"),
                                  (613, 1, 9, 6, 4, 2, 4, 1, 3, 7, 0.0, "VALID", "test"),
                                  (614, 2, 6, 6, 8, 3, 3, 1, 1, 16, 1.0, "SAME", "cfg"),
                                  (615, 1, 10, 10, 2, 5, 5, 2, 2, 3, 1.0, "SAME", "test")])
def test_oracle_vs_reference_conv_live(case):
    from tests import parity as P
    seed, B, H, W, C, Kh, Kw, Sh, Sw, Kc, bv, padding, dist = case
    x, w = P.make_inputs(seed, (B, H, W, C), (Kh * Kw * C + (bv > 1e-8), Kc), dist)
    p = O.cv_params(Kh, Kw, Sh, Sw, padding, bv)
    y = O.ref_cv_forward(O.pad_like_reference(x, Kh, Kw, Sh, Sw, padding), w, p)
    o32, o64 = O.cv_forward(x, w, p, "f32"), O.cv_forward(x, w, p, "f64")
    _fire_and_values(y, o32, o64, "conv live %d" % seed)


@needs_ref
def test_biased_dense_through_reference_conv_op():
    """A dense layer WITH bias is a 1x1 convolution with C = fan-in; the reference's conv CPU op
    handles bias (its dense CPU op does not), so this pins the bias-first rule of the dense oracle."""
    from tests import parity as P
    B, I, J = 12, 50, 30
    x, w = P.make_inputs(621, (B, I), (I + 1, J), "test")
    w[I, :5] = 1.7  # bias weight above the threshold: the bias alone arms these outputs
    y = O.ref_cv_forward(x.reshape(B, 1, 1, I), w, O.cv_params(1, 1, 1, 1, "VALID", 1.0)).reshape(B, J)
    p = O.fc_params(biasvolt=1.0)
    _fire_and_values(y, O.fc_forward(x, w, p, "f32"), O.fc_forward(x, w, p, "f64"), "dense+bias via conv op")
