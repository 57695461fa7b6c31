"""Shared parity protocol of the tests (oracle = CPU restatement of the reference GPU kernels).

Forward: fire/no-fire and causal-set size must agree exactly with the float64 oracle except on
outputs the oracle flags as ill-conditioned (a fire decision within 1e-5 of flipping). Spike values
and 1/(sum w - theta): within 2e-6 of the fp32 restatement (same order of operations as the
reference GPU kernel), and within rel max(1e-4, 4e-7*cond) of the float64 oracle, where
cond = (theta+sum|w|)/|sum w - theta| is the factor by which fp32 rounding of the two running sums
is amplified in y (no fp32 evaluation, the reference's included, can hold 1e-4 when cond > 100). Backward: computed from the SAME forward output,
elementwise |a-b| <= 1e-4*|b| + 1e-5*rms(b) and relative L2 <= 1e-5 against the float64 oracle.
"""
import numpy as np

import oracle as O

REL = 1e-4


def make_inputs(seed, shape_x, shape_w, dist, rng=None):
    """'test': the reference tests' distribution x=exp|randn|, w=randn (test-snn-fc-forward.py:25-32);
    'cfg': benchmark family x=exp(U[0,1)), w~N(2/I, 1/I)."""
    rng = rng or np.random.default_rng(seed)
    I = shape_w[0]
    if dist == "test":
        x = np.exp(np.abs(rng.standard_normal(shape_x))).astype(np.float32)
        w = rng.standard_normal(shape_w).astype(np.float32)
    else:
        x = np.exp(rng.random(shape_x)).astype(np.float32)
        w = rng.normal(2.0 / I, 1.0 / np.sqrt(I), shape_w).astype(np.float32)
    return x, w


def causal_count(rows, y, maxv=1e5):
    """k := #{i : x_i <= y} per (row, output); rows [R,I], y [R,J]."""
    xs = np.sort(rows, axis=1)
    out = np.empty(y.shape, np.int64)
    for r in range(rows.shape[0]):
        out[r] = np.searchsorted(xs[r], y[r], side="right")
    return out


def check_forward(y_gpu, inv_gpu, o32, o64, rows=None, maxv=1e5, what=""):
    y_gpu = np.asarray(y_gpu).reshape(o64["y"].shape)
    inv_gpu = np.asarray(inv_gpu).reshape(o64["y"].shape)
    ill = o64["illc"]
    fired_g = y_gpu < maxv - 0.1
    fired_o = o64["y"] < maxv - 0.1
    bad = (fired_g != fired_o) & ~ill
    assert bad.sum() == 0, "%s: %d fire/no-fire mismatches on well-conditioned outputs" % (what, bad.sum())
    assert ill.mean() < 0.25, "%s: %.3f of outputs flagged ill-conditioned" % (what, ill.mean())
    ok = fired_g & fired_o & ~ill
    if ok.any():
        tol = np.maximum(REL, 4e-7 * o64["cond"][ok])
        rel = np.abs(y_gpu[ok] - o64["y"][ok]) / np.abs(o64["y"][ok])
        assert (rel / tol).max() <= 1.0, "%s: spike value rel err %.3e (%.2fx tolerance)" % (what, rel.max(), (rel / tol).max())
        reli = np.abs(inv_gpu[ok] - o64["inv"][ok]) / np.abs(o64["inv"][ok])
        assert (reli / tol).max() <= 1.0, "%s: 1/wsum rel err %.3e" % (what, reli.max())
    # unfired outputs are exactly MAX with a zero reciprocal
    assert np.all(y_gpu[~fired_g] >= maxv - 0.1)
    assert np.all(inv_gpu[y_gpu >= maxv] == 0)
    # against the fp32 restatement (same order of operations) the agreement is much tighter
    same = fired_g & (o32["y"] < maxv - 0.1) & ~ill
    if same.any():
        rel32 = np.abs(y_gpu[same] - o32["y"][same]) / np.abs(o32["y"][same])
        assert rel32.max() <= 2e-6, "%s: vs fp32 restatement rel err %.3e" % (what, rel32.max())
    if rows is not None:
        R = rows.shape[0]
        kg = causal_count(rows, y_gpu.reshape(R, -1))
        ko = causal_count(rows, o64["y"].reshape(R, -1).astype(np.float32))
        okf = ok.reshape(R, -1)
        assert np.all(kg[okf] == ko[okf]), "%s: causal-set size differs on %d outputs" % (what, (kg[okf] != ko[okf]).sum())
    return dict(flagged=int(ill.sum()), fired=float(fired_g.mean()))


def check_close(a, b, what, rel=REL, rms_atol=1e-5, l2=1e-5, abs_sum=None):
    a = np.asarray(a, np.float64); b = np.asarray(b, np.float64)
    assert a.shape == b.shape, "%s: shape %s vs %s" % (what, a.shape, b.shape)
    rms = np.sqrt(np.mean(b * b)) if b.size else 0.0
    err = np.abs(a - b)
    tol = rel * np.abs(b) + rms_atol * rms + 1e-30
    if abs_sum is not None:
        tol = tol + 1e-6 * abs_sum
    worst = (err / tol).max() if b.size else 0.0
    assert worst <= 1.0, "%s: elementwise error %.2fx tolerance (max abs %.3e, rms %.3e)" % (what, worst, err.max(), rms)
    nb = np.linalg.norm(b)
    if nb > 0:
        bound = l2 * nb + (4e-7 * np.linalg.norm(abs_sum) if abs_sum is not None else 0.0)
        r = np.linalg.norm(a - b)
        assert r <= bound, "%s: L2 error %.3e vs bound %.3e (relative %.3e)" % (what, r, bound, r / nb)


def im2col_rows(x, Kh, Kw, Sh, Sw, padding, maxv=1e5):
    xp = O.pad_like_reference(x, Kh, Kw, Sh, Sw, padding, maxv)
    B, Hp, Wp, C = xp.shape
    Nh, Nw = (Hp - Kh) // Sh + 1, (Wp - Kw) // Sw + 1
    rows = np.stack([xp[b, nh * Sh:nh * Sh + Kh, nw * Sw:nw * Sw + Kw, :].reshape(-1)
                     for b in range(B) for nh in range(Nh) for nw in range(Nw)])
    return rows
