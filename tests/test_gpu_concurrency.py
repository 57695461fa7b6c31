"""Several host threads calling the operators on their own streams at the same time: the library keeps no state
between calls except per-device caches behind a lock, and the auxiliary streams a backward call forks its dX
kernel onto are handed out per call with their own events. Every concurrent result must be the bits of the same
call made alone."""
import threading

import numpy as np
import pytest

import oracle as O
from tests import parity as P

pytestmark = pytest.mark.gpu


def test_two_threads_two_streams_each_bit_identical_to_serial():
    import torch
    from snntc_2023_b200 import ops
    problems = []
    for seed, B, I, J in ((201, 300, 257, 256), (202, 280, 400, 320), (203, 512, 130, 128), (204, 260, 513, 260)):
        x, w = P.make_inputs(seed, (B, I), (I + 1, J), "test")
        g = np.random.default_rng(seed).standard_normal((B, J)).astype(np.float32)
        problems.append(tuple(torch.from_numpy(a).cuda() for a in (x, w, g)))
    params = O.fc_params(biasvolt=1.0)
    serial = []
    for x, w, g in problems:
        out = ops.snn_fc(x, w, params)
        dx, dw, _ = ops.snn_fc_grad(g, x, w, params, out)      # B*J >= 65536: dX runs on an auxiliary stream
        serial.append((out.clone(), dx.clone(), dw.clone()))
    torch.cuda.synchronize()
    errors = []

    def worker(tid):
        try:
            torch.cuda.set_device(0)
            streams = [torch.cuda.Stream(), torch.cuda.Stream()]
            for it in range(50):
                k = (2 * tid + it) % len(problems)
                x, w, g = problems[k]
                with torch.cuda.stream(streams[it & 1]):
                    out = ops.snn_fc(x, w, params)
                    dx, dw, _ = ops.snn_fc_grad(g, x, w, params, out)
                    streams[it & 1].synchronize()
                    ok = torch.equal(out, serial[k][0]) and torch.equal(dx, serial[k][1]) and torch.equal(dw, serial[k][2])
                if not ok:
                    errors.append("thread %d iteration %d problem %d differs from the serial result" % (tid, it, k))
                    return
        except Exception as e:   # pragma: no cover
            errors.append("thread %d: %r" % (tid, e))

    threads = [threading.Thread(target=worker, args=(t,)) for t in range(2)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    torch.cuda.synchronize()
    assert not errors, errors


def test_one_thread_alternating_streams_without_waiting():
    """Backward calls queued back to back on two streams from one thread, nothing synchronised in between."""
    import torch
    from snntc_2023_b200 import ops
    params = O.fc_params(biasvolt=1.0)
    x, w = P.make_inputs(211, (400, 300), (301, 256), "test")
    xd, wd = torch.from_numpy(x).cuda(), torch.from_numpy(w).cuda()
    gs = [torch.randn(400, 256, device="cuda", generator=torch.Generator("cuda").manual_seed(s)) for s in range(6)]
    out = ops.snn_fc(xd, wd, params)
    want = [ops.snn_fc_grad(g, xd, wd, params, out) for g in gs]
    torch.cuda.synchronize()
    streams = [torch.cuda.Stream(), torch.cuda.Stream()]
    got = []
    for i, g in enumerate(gs):
        with torch.cuda.stream(streams[i & 1]):
            got.append(ops.snn_fc_grad(g, xd, wd, params, out))
    torch.cuda.synchronize()
    for a, b in zip(got, want):
        assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])
