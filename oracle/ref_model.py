"""CPU train step of a sequential SNN-TC network through the reference's own CPU operators
(oracle/_ref) or, where those are not available, through the restated oracle -- TEST INFRASTRUCTURE
and the bench's CPU-baseline leg only.

Layer specs are those of snntc_2023_b200.nets. Dense layers with bias go through the reference's
CONV CPU operator as a 1x1 convolution (H=W=Kh=Kw=1, C=fan-in): the reference's dense CPU pair is
only right without bias (snntc/readme.txt:28-30), its conv pair handles bias. Pooling and the loss
are numpy glue (the reference does them in TensorFlow, SNN_TC_Modules.py:216-246, 286-288). The
reference operators are single-threaded per call, so the batch is split over `threads` workers and
the per-shard weight gradients are summed.
"""
from concurrent.futures import ThreadPoolExecutor

import numpy as np

from . import oracle as O


def _conv_fwd(x, w, k, s, kind):
    p = O.cv_params(k, k, s, s, "SAME", 1.0)
    if kind == "reference":
        xp = O.pad_like_reference(x, k, k, s, s, "SAME")
        y = O.ref_cv_forward(xp, w, p)
        return y, (x, xp, p, y, None)
    o = O.cv_forward(x, w, p, "f32")
    return o["y"], (x, None, p, o["y"], o["inv"])


def _conv_bwd(g, w, ctx, k, s, kind):
    x, xp, p, y, inv = ctx
    if kind == "reference":
        B = x.shape[0]
        g2 = np.concatenate([g, np.zeros_like(g)])
        old = np.concatenate([y, np.zeros_like(y)])
        dxp, dw, _ = O.ref_cv_backward(g2, xp, w, p, old)
        pt, pl, _, _, _, _ = O.conv_geometry(x.shape[1], x.shape[2], k, k, s, s, "SAME")
        return dxp[:, pt:pt + x.shape[1], pl:pl + x.shape[2], :], dw
    r = O.cv_backward(g, x, w, p, y, inv, "f32")
    return r["dx"], r["dw"]


def _dense_fwd(x, w, kind):
    if kind == "reference":
        B, I = x.shape
        p = O.cv_params(1, 1, 1, 1, "VALID", 1.0)
        x4 = np.ascontiguousarray(x.reshape(B, 1, 1, I))
        y = O.ref_cv_forward(x4, w, p)
        return y.reshape(B, -1), (x4, p, y)
    p = O.fc_params(biasvolt=1.0)
    o = O.fc_forward(x, w, p, "f32")
    return o["y"], (x, p, o)


def _dense_bwd(g, w, ctx, kind):
    if kind == "reference":
        x4, p, y = ctx
        B = x4.shape[0]
        g4 = g.reshape(y.shape)
        g2 = np.concatenate([g4, np.zeros_like(g4)])
        old = np.concatenate([y, np.zeros_like(y)])
        dx, dw, _ = O.ref_cv_backward(g2, x4, w, p, old)
        return dx.reshape(B, -1), dw
    x, p, o = ctx
    r = O.fc_backward(g, x, w, p, o["y"], o["inv"], "f32")
    return r["dx"], r["dw"]


def shard_step(specs, weights, x, labels, total_batch, kind):
    """Forward + loss + backward of one batch shard. Returns (sum of sample losses, [dW per weighted layer])."""
    acts = []
    wi = 0
    h = x
    for s in specs:
        if s[0] == "conv":
            h, ctx = _conv_fwd(h, weights[wi], s[3], s[4], kind); acts.append(ctx); wi += 1
        elif s[0] == "dense":
            h, ctx = _dense_fwd(h, weights[wi], kind); acts.append(ctx); wi += 1
        elif s[0] == "pool":
            shape = h.shape
            h, arg = O.minpool(h, s[1], s[1], s[1], s[1], "SAME")
            acts.append((shape, arg))
        elif s[0] == "flatten":
            acts.append(h.shape)
            h = np.ascontiguousarray(h.reshape(h.shape[0], -1))
    z = -h.astype(np.float64)
    z -= z.max(1, keepdims=True)
    logp = z - np.log(np.exp(z).sum(1, keepdims=True))
    n = h.shape[0]
    loss_sum = -logp[np.arange(n), labels].sum()
    dlogit = np.exp(logp)
    dlogit[np.arange(n), labels] -= 1.0
    g = (-dlogit / total_batch).astype(np.float32)  # d(mean CE)/dy with logits = -y
    grads = [None] * len(weights)
    for s, ctx in zip(reversed(specs), reversed(acts)):
        if s[0] == "conv":
            wi -= 1
            g, grads[wi] = _conv_bwd(g, weights[wi], ctx, s[3], s[4], kind)
        elif s[0] == "dense":
            wi -= 1
            g, grads[wi] = _dense_bwd(g, weights[wi], ctx, kind)
        elif s[0] == "pool":
            shape, arg = ctx
            dx = np.zeros(int(np.prod(shape)), np.float32)
            ok = arg.reshape(-1) >= 0
            np.add.at(dx, arg.reshape(-1)[ok], g.reshape(-1)[ok])
            g = dx.reshape(shape)
        elif s[0] == "flatten":
            g = g.reshape(ctx)
    return loss_sum, grads


def train_step(specs, weights, x, labels, threads=1, kind=None):
    """One forward+backward over the batch, split over `threads` workers. Returns (mean loss, grads, kind)."""
    if kind is None:
        kind = "reference" if O.ref_lib() is not None else "port"
    B = x.shape[0]
    threads = max(1, min(threads, B))
    bounds = np.linspace(0, B, threads + 1).astype(int)
    parts = [(x[a:b], labels[a:b]) for a, b in zip(bounds[:-1], bounds[1:]) if b > a]
    if len(parts) == 1:
        res = [shard_step(specs, weights, parts[0][0], parts[0][1], B, kind)]
    else:
        with ThreadPoolExecutor(len(parts)) as ex:
            res = list(ex.map(lambda p: shard_step(specs, weights, p[0], p[1], B, kind), parts))
    loss = sum(r[0] for r in res) / B
    grads = [sum(r[1][i] for r in res) for i in range(len(weights))]
    return loss, grads, kind
