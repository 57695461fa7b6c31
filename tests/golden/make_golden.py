"""Generates the golden fixtures in this folder by running the REFERENCE's own CPU operators
(oracle/_ref/libsnntc_ref_cpu.so, compiled unmodified from the reference checkout by oracle/build.py)
on small seeded inputs. Needs the reference checkout; the fixtures it writes are committed so that
the tests can run where the checkout is absent.

    python tests/golden/make_golden.py

Each .npz holds the inputs and what the reference returned:
  dense_*: x, w, params, g, out (reference layout: rows [B,2B) hold sum(w)-theta, not its reciprocal), dx, dw
  conv_* : x (UNPADDED), w, params, g, y (the CPU conv op leaves the second half unwritten), dxp (padded shape), dw
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

import oracle as O  # noqa: E402

# (name, seed, B, I, J, dist) -- the reference's dense CPU pair is only right without bias
DENSE = [("dense_test", 501, 6, 40, 12, "test"), ("dense_cfg", 502, 5, 96, 20, "cfg"), ("dense_one", 503, 3, 1, 2, "test")]
# (name, seed, B, H, W, C, Kh, Kw, Sh, Sw, Kc, biasvolt, padding, dist)
CONV = [("conv_same_bias", 511, 2, 6, 7, 3, 3, 2, 2, 1, 5, 1.0, "SAME", "test"),
        ("conv_valid_nobias", 512, 1, 7, 6, 4, 2, 3, 1, 2, 6, 0.0, "VALID", "test"),
        ("conv_cfg_bias", 513, 2, 5, 5, 8, 3, 3, 1, 1, 9, 1.0, "SAME", "cfg"),
        ("conv_stride3", 514, 1, 9, 9, 2, 5, 5, 3, 3, 4, 0.5, "SAME", "test"),
        # the deterministic inputs of the reference's test-snn-cv-backward.py:57-79 (testmode 1)
        ("conv_arange", None, 2, 4, 4, 2, 3, 3, 2, 2, 2, 1.0, "SAME", "arange")]


def inputs(seed, shape_x, shape_w, dist):
    if dist == "arange":
        x = (np.arange(int(np.prod(shape_x)), dtype=np.float32) + 1.1).reshape(shape_x)
        w = ((np.arange(int(np.prod(shape_w)), dtype=np.float32) + 1) / 10).reshape(shape_w)
        return x, w
    rng = np.random.default_rng(seed)
    I = shape_w[0]
    if dist == "test":
        return (np.exp(np.abs(rng.standard_normal(shape_x))).astype(np.float32),
                rng.standard_normal(shape_w).astype(np.float32))
    return (np.exp(rng.random(shape_x)).astype(np.float32),
            rng.normal(2.0 / I, 1.0 / np.sqrt(I), shape_w).astype(np.float32))


def main():
    if O.ref_lib() is None:
        raise SystemExit("oracle/_ref/libsnntc_ref_cpu.so is missing: run python oracle/build.py where the reference checkout exists")
    for name, seed, B, I, J, dist in DENSE:
        x, w = inputs(seed, (B, I), (I, J), dist)
        p = O.fc_params(biasvolt=0.0)
        g = np.random.default_rng(seed + 1).standard_normal((B, J)).astype(np.float32)
        out = O.ref_fc_forward(x, w, p)
        dx, dw, _ = O.ref_fc_backward(np.concatenate([g, np.zeros_like(g)]), x, w, p, out)
        np.savez(os.path.join(HERE, name + ".npz"), x=x, w=w, params=p, g=g, out=out, dx=dx, dw=dw)
    for name, seed, B, H, W, C, Kh, Kw, Sh, Sw, Kc, bv, padding, dist in CONV:
        I = Kh * Kw * C
        x, w = inputs(seed, (B, H, W, C), (I + (bv > 1e-8), Kc), dist)
        p = O.cv_params(Kh, Kw, Sh, Sw, padding, bv)
        xp = O.pad_like_reference(x, Kh, Kw, Sh, Sw, padding)
        y = O.ref_cv_forward(xp, w, p)
        g = np.random.default_rng((seed or 7) + 1).standard_normal(y.shape).astype(np.float32)
        dxp, dw, _ = O.ref_cv_backward(np.concatenate([g, np.zeros_like(g)]), xp, w, p,
                                       np.concatenate([y, np.zeros_like(y)]))
        np.savez(os.path.join(HERE, name + ".npz"), x=x, w=w, params=p, g=g, y=y, dxp=dxp, dw=dw,
                 padding=np.array(padding))
    print("wrote", len(DENSE) + len(CONV), "fixtures to", HERE)


if __name__ == "__main__":
    main()
