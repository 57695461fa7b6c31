"""Parity protocol shared by the tests and the bench's in-run check -- TEST INFRASTRUCTURE ONLY
(oracle = CPU restatement of the reference GPU kernels, see oracle.py).

Forward: fire/no-fire and causal-set size must agree exactly with the float64 oracle except on
outputs the oracle flags as ill-conditioned (a fire decision within 1e-5 of flipping). Spike values
and 1/(sum w - theta): within 2e-6 of the fp32 restatement (same order of operations as the
reference GPU kernel), and within rel max(1e-4, 4e-7*cond) of the float64 oracle, where
cond = (theta+sum|w|)/|sum w - theta| is the factor by which fp32 rounding of the two running sums
is amplified in y (no fp32 evaluation, the reference's included, can hold 1e-4 when cond > 250).
Backward: computed from the SAME forward output, elementwise
|a-b| <= 1e-4*|b| + 1e-5*rms(b) + 1e-6*sum|terms| and relative L2 <= 1e-5 against the float64 oracle.

How much of each tensor was held to which bound is REPORTED, not only asserted: `check_forward`
returns the fraction of outputs that were flagged (exempt from the float64 comparison), the fraction
whose bound was wider than 1e-4, and how many outputs -- flagged or not -- take a different fire
decision than the fp32 restatement, which follows the reference kernel's operation order and is
therefore expected to agree on flagged outputs too. Every call appends its figures to `REPORT`.
"""
import json
import os

import numpy as np

from . import oracle as O

REL = 1e-4
REPORT = []   # one dict per check_forward call of this process


def flagged_limit(fan_in):
    """Largest flagged fraction a case may show. A row of I inputs takes up to I fire decisions per
    output, each of which lands within 1e-5 (relative) of a tie with a probability of the same
    order, so the flagged share grows linearly with the fan-in: 1 % plus 1.5e-5 per input."""
    return 0.01 + 1.5e-5 * fan_in


def make_inputs(seed, shape_x, shape_w, dist, rng=None, bias=False, sentinels=0.5):
    """'test': the reference tests' distribution x=exp|randn|, w=randn (test-snn-fc-forward.py:25-32);
    'cfg': benchmark family x=exp(U[0,1)), w~N(2/I, 1/I);
    'ref': what a hidden layer of the benchmark networks sees: x=exp(1.5*U[0,1)) with a share
           `sentinels` of the inputs at MAX (outputs of the previous layer that never spiked), weights
           by the reference initialisation randn*sqrt(15/I) with a zero bias row last
           (SNN_TC_Modules.py:19-25; pass bias=True when shape_w includes that row)."""
    rng = rng or np.random.default_rng(seed)
    I = shape_w[0]
    if dist == "test":
        x = np.exp(np.abs(rng.standard_normal(shape_x))).astype(np.float32)
        w = rng.standard_normal(shape_w).astype(np.float32)
    elif dist == "ref":
        x = np.exp(1.5 * rng.random(shape_x)).astype(np.float32)
        x[rng.random(shape_x) < sentinels] = np.float32(1e5)
        fan_in = I - (1 if bias else 0)
        w = (rng.standard_normal(shape_w) * np.sqrt(15.0 / fan_in)).astype(np.float32)
        if bias:
            w[-1, :] = 0
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


def check_forward(y_gpu, inv_gpu, o32, o64, rows=None, maxv=1e5, what="", fan_in=None, max_flagged=None):
    """Asserts the forward protocol and returns its figures. `inv_gpu` may be None (inference forward).
    `fan_in` sets the flagged-fraction limit (see flagged_limit); `max_flagged` overrides it."""
    y_gpu = np.asarray(y_gpu).reshape(o64["y"].shape)
    ill = o64["illc"]
    fired_g = y_gpu < maxv - 0.1
    fired_o = o64["y"] < maxv - 0.1
    fired_32 = o32["y"] < maxv - 0.1
    bad = (fired_g != fired_o) & ~ill
    assert bad.sum() == 0, "%s: %d fire/no-fire mismatches on well-conditioned outputs" % (what, bad.sum())
    if fan_in is None and rows is not None:
        fan_in = rows.shape[1]
    limit = max_flagged if max_flagged is not None else flagged_limit(fan_in or 0)
    flagged = float(ill.mean())
    assert flagged <= limit, ("%s: %.4f of outputs flagged ill-conditioned, limit %.4f (1 %% + 1.5e-5 per input: every "
                              "input is one more decision that can land within 1e-5 of a tie)" % (what, flagged, limit))
    # flagged or not, the decision should be the fp32 restatement's (same operation order as the reference kernel);
    # the few that differ are the outputs whose spike time ties an input to the last bits
    differ32 = int((fired_g != fired_32).sum())
    assert differ32 <= max(2, 1e-3 * ill.size), "%s: %d outputs decide differently from the fp32 restatement" % (what, differ32)
    ok = fired_g & fired_o & ~ill
    wide = 0.0
    worst = 0.0
    if ok.any():
        tol = np.maximum(REL, 4e-7 * o64["cond"][ok])
        wide = float((tol > REL).sum()) / ill.size
        rel = np.abs(y_gpu[ok] - o64["y"][ok]) / np.abs(o64["y"][ok])
        worst = float((rel / tol).max())
        assert worst <= 1.0, "%s: spike value rel err %.3e (%.2fx tolerance)" % (what, rel.max(), worst)
        if inv_gpu is not None:
            inv_gpu = np.asarray(inv_gpu).reshape(o64["y"].shape)
            reli = np.abs(inv_gpu[ok] - o64["inv"][ok]) / np.abs(o64["inv"][ok])
            assert (reli / tol).max() <= 1.0, "%s: 1/wsum rel err %.3e" % (what, reli.max())
    # unfired outputs are exactly MAX with a zero reciprocal
    assert np.all(y_gpu[~fired_g] >= maxv - 0.1)
    if inv_gpu is not None:
        inv_gpu = np.asarray(inv_gpu).reshape(o64["y"].shape)
        assert np.all(inv_gpu[y_gpu >= maxv] == 0)
    # against the fp32 restatement (same order of operations) the agreement is much tighter
    same = fired_g & fired_32 & ~ill
    rel32 = 0.0
    if same.any():
        rel32 = float((np.abs(y_gpu[same] - o32["y"][same]) / np.abs(o32["y"][same])).max())
        assert rel32 <= 2e-6, "%s: vs fp32 restatement rel err %.3e" % (what, rel32)
    if rows is not None:
        R = rows.shape[0]
        kg = causal_count(rows, y_gpu.reshape(R, -1))
        ko = causal_count(rows, o64["y"].reshape(R, -1).astype(np.float32))
        okf = ok.reshape(R, -1)
        assert np.all(kg[okf] == ko[okf]), "%s: causal-set size differs on %d outputs" % (what, (kg[okf] != ko[okf]).sum())
    stats = dict(case=str(what), outputs=int(ill.size), flagged_frac=flagged, flagged_limit=limit,
                 over_1e4_frac=wide, worst_of_tolerance=worst, differ_from_fp32=differ32, max_rel_vs_fp32=rel32,
                 fired=float(fired_g.mean()))
    REPORT.append(stats)
    return stats


def summary(report=None):
    """The figures a bench line or a test log carries: how many cases, the largest flagged share and the
    largest share of outputs that needed a bound above 1e-4."""
    report = REPORT if report is None else report
    if not report:
        return dict(cases=0, flagged_frac_max=None, over_1e4_frac_max=None, differ_from_fp32=0)
    return dict(cases=len(report),
                flagged_frac_max=max(r["flagged_frac"] for r in report),
                over_1e4_frac_max=max(r["over_1e4_frac"] for r in report),
                differ_from_fp32=int(sum(r["differ_from_fp32"] for r in report)),
                outputs=int(sum(r["outputs"] for r in report)))


def dump_report(path):
    d = os.path.dirname(path)
    if d:
        os.makedirs(d, exist_ok=True)
    with open(path, "w") as f:
        json.dump(dict(summary=summary(), cases=REPORT), f, indent=1)


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
