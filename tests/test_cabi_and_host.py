"""CPU-side checks: the C-ABI library loads and exports every symbol the header declares, argument
validation answers with the documented status codes before anything touches a device, and the
Python layer keeps the reference's surface (SNN_TC_Modules.py:42-43,103-105,48-49,121-123)."""
import ctypes
import math
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    """(symbols of the product library, symbols of the measurement build only) as the header declares them."""
    text = open(os.path.join(ROOT, "include", "snntc_b200.h")).read()
    head, _, rest = text.partition("#ifdef SNNTC_MEASURE")
    measure, _, tail = rest.partition("#endif /* SNNTC_MEASURE */")
    find = lambda t: sorted(set(re.findall(r"SNNTC_API[^;(]*?\b(snntc_\w+)\s*\(", t)))
    return find(head + tail), find(measure)


def _exported(path):
    import subprocess
    out = subprocess.check_output(["nm", "-D", "--defined-only", path], text=True)
    return {line.split()[-1] for line in out.splitlines() if line.strip()}


def test_library_exports_every_declared_symbol():
    from snntc_2023_b200 import _lib
    lib = _lib.load()
    names, measure_names = _declared_symbols()
    assert len(names) >= 24 and len(measure_names) == 5
    for n in names:
        assert hasattr(lib, n), "libsnntc_b200.so does not export %s" % n
    assert set(names) == set(_lib.SYMBOLS), "ctypes table and header disagree: %s" % (set(names) ^ set(_lib.SYMBOLS))
    assert set(measure_names) == set(_lib.MEASURE_SYMBOLS)
    assert lib.snntc_version().startswith(b"snntc_b200")
    assert lib.snntc_status_string(0) == b"ok"


def test_default_library_has_no_measurement_entry_points():
    """Kernel selection and partial execution exist only in the measurement build: the product library exports
    exactly what the header declares outside SNNTC_MEASURE, and no switch that changes what a call launches."""
    from snntc_2023_b200 import _lib
    names, measure_names = _declared_symbols()
    exported = {s for s in _exported(_lib.LIB_PATH) if s.startswith("snntc_")}
    assert exported == set(names), "unexpected exports: %s" % sorted(exported ^ set(names))
    assert not any("profile" in s or "measure" in s or "probe" in s for s in exported)
    m = _lib.load_measure()
    for n in names + measure_names:
        assert hasattr(m, n), "libsnntc_b200_measure.so does not export %s" % n
    assert b"measurement" in m.snntc_version()


def test_validation_status_codes_without_a_device():
    from snntc_2023_b200 import _lib
    lib = _lib.load()
    p6 = np.array([1e5, 1e-10, 1.0, 0, 0, 1.0], np.float32)
    P = p6.ctypes.data
    fake = 0x1000  # never dereferenced: every call below is rejected during validation
    fwd = lib.snntc_fc_forward
    assert fwd(0, fake, P, fake, 4, 8, 9, 3, 0, 0, 0) == -1                 # null input
    assert fwd(fake, fake, 0, fake, 4, 8, 9, 3, 0, 0, 0) == -1              # null params
    assert fwd(fake, fake, P, fake, 0, 8, 9, 3, 0, 0, 0) == -2              # empty batch
    assert fwd(fake, fake, P, fake, 4, 8, 8, 3, 0, 0, 0) == -3              # bias on, but no bias row
    assert fwd(fake, fake, P, fake, 4, 8, 10, 3, 0, 0, 0) == -3
    assert fwd(fake, fake, P, fake, 70000, 40000, 40001, 3, 0, 0, 0) == -4  # B*I > 2^31-1
    p6[0] = 0.5
    assert fwd(fake, fake, P, fake, 4, 8, 9, 3, 0, 0, 0) == -8              # MAX_SPIKE_TIME must exceed 1
    p12 = np.array([1e5, 0, 0, 1e-10, 1.0, 0, 3, 3, 1, 1, 1, 0.0], np.float32)
    cv = lib.snntc_cv_forward
    assert cv(fake, fake, p12.ctypes.data, fake, 2, 8, 8, 4, 37, 5, 1, 1, 8, 8, 0, 0, 0) == -3   # 3*3*4 = 36 rows expected
    assert cv(fake, fake, p12.ctypes.data, fake, 2, 8, 8, 4, 36, 5, 3, 1, 8, 8, 0, 0, 0) == -2   # pad >= kernel
    p12[6] = 0
    assert cv(fake, fake, p12.ctypes.data, fake, 2, 8, 8, 4, 36, 5, 1, 1, 8, 8, 0, 0, 0) == -8   # Kh = 0
    for code in range(0, -9, -1):
        assert len(lib.snntc_status_string(code)) > 1
    assert lib.snntc_fc_forward_workspace_bytes(256, 784, 400) >= 256 * 784 * 8
    assert lib.snntc_fc_backward_workspace_bytes(1, 25088, 25089, 1024) == 4096 + 256   # u[1,1024] and the range flag: enough tiles, no row split
    # a 3x3 stride-1 convolution also gets the scratch of the merging list builder; a 5x5 one does not
    lists = 2 * 8 * 8 * 288 * 8
    assert lib.snntc_cv_forward_workspace_bytes(2, 8, 8, 32, 16, 3, 3, 8, 8) > lists + 2 * 8 * 8 * 36 * 8
    assert lib.snntc_cv_forward_workspace_bytes(2, 8, 8, 32, 16, 5, 5, 8, 8) < 2 * 8 * 8 * 802 * 8 + 4096


def test_no_cpu_fallback():
    import torch
    from snntc_2023_b200 import ops, _lib
    x = torch.ones(2, 3); w = torch.ones(4, 5)
    with pytest.raises(_lib.SnntcError):
        ops.snn_fc(x, w, np.array([1e5, 1e-10, 1.0, 0, 0, 1.0], np.float32))
    with pytest.raises(ValueError):
        ops.snn_fc(x.double(), w, np.zeros(6, np.float32)) if False else ops._params(np.zeros(5), 6)


def test_layer_surface_matches_reference():
    import torch
    import SNN_TC_Modules as SNN
    d = SNN.SNN_dense(784, 400)
    assert tuple(d.weight.shape) == (785, 400) and d.in_size == 785 and d.out_size == 400
    assert np.allclose(d.Params, [1e5, 1e-10, 1.0, 0, 0, 1.0]) and d.Params.dtype == np.float32
    assert float(d.weight[-1].abs().sum()) == 0.0            # zero bias row, stored last
    d0 = SNN.SNN_dense(10, 4, biasvolt=0)
    assert tuple(d0.weight.shape) == (10, 4) and d0.in_size == 10
    wgt = np.arange(44, dtype=np.float64).reshape(11, 4)
    d1 = SNN.SNN_dense(10, 4, weight=wgt)
    assert d1.weight.dtype == torch.float32 and np.allclose(d1.weight.detach().numpy(), wgt)
    with pytest.raises(ValueError):
        SNN.SNN_dense(10, 4, weight=np.zeros((10, 4)))      # bias on by default: 11 rows expected
    c = SNN.SNN_conv(3, 8, kernel_sizes=[3, 2], strides=2, padding='same', rates=1)
    assert (c.Kh, c.Kw, c.Sh, c.Sw, c.C, c.Kc, c.padding) == (3, 2, 2, 2, 3, 8, 'SAME')
    assert tuple(c.weight.shape) == (3 * 2 * 3 + 1, 8) and c.in_size == 19
    assert np.allclose(c.Params, [1e5, 0, 0, 1e-10, 1.0, 0, 3, 2, 2, 2, 1, 1.0])
    assert float(d.w_sum_cost()) >= 0 and float(c.l2_cost()) >= 0
    assert callable(d.call) and callable(c.call)
    for name in ("snnfc", "snnfc_grad", "snncv", "snncv_grad", "SNN_maxpool2d", "SNN_avgpool2d", "SNN_LRN",
                 "loss_func", "init_weight"):
        assert hasattr(SNN, name)
    w = SNN.init_weight(100, 7, 1.0)
    assert w.shape == (101, 7) and w.dtype == np.float32 and not w[-1].any()
    # loss: softmax cross-entropy on the negated spike values
    logit = torch.tensor([[1.0, 2.0, 0.5]]); label = torch.tensor([[0.0, 0.0, 1.0]])
    z = -logit
    assert abs(float(SNN.loss_func(logit, label)) - float(-(z[0, 2] - torch.logsumexp(z, 1)))) < 1e-6
    assert abs(float(SNN.loss_func(logit, torch.tensor([2]))) - float(SNN.loss_func(logit, label))) < 1e-6


@pytest.mark.parametrize("H,W,Kh,Kw,Sh,Sw", [(32, 32, 3, 3, 1, 1), (224, 224, 7, 7, 2, 2), (7, 9, 3, 2, 2, 1),
                                              (10, 10, 5, 5, 2, 2), (12, 11, 6, 3, 3, 2), (5, 5, 1, 1, 1, 1), (8, 8, 3, 3, 3, 3)])
def test_conv_geometry_matches_reference_formulas(H, W, Kh, Kw, Sh, Sw):
    import oracle as O
    from snntc_2023_b200 import ops
    # SAME: total = (ceil(H/S)-1)*S + K - H, before = int(total/2)  (SNN_TC_Modules.py:147-161)
    th = (math.ceil(H / Sh) - 1) * Sh + Kh - H
    tw = (math.ceil(W / Sw) - 1) * Sw + Kw - W
    pt, pl, Nh, Nw = ops.conv_geometry(H, W, Kh, Kw, Sh, Sw, "SAME")
    assert (pt, pl) == (int(th / 2), int(tw / 2))
    assert (Nh, Nw) == ((H + th - Kh) // Sh + 1, (W + tw - Kw) // Sw + 1) == (math.ceil(H / Sh), math.ceil(W / Sw))
    assert (pt, pl, Nh, Nw) == O.conv_geometry(H, W, Kh, Kw, Sh, Sw, "SAME")[:4]
    # VALID: OutDim = int((H-K)/S + 1), trailing rows/columns dropped (:163-166)
    pt, pl, Nh, Nw = ops.conv_geometry(H, W, Kh, Kw, Sh, Sw, "VALID")
    assert (pt, pl, Nh, Nw) == (0, 0, int((H - Kh) / Sh + 1.0), int((W - Kw) / Sw + 1.0))
    assert (Nh - 1) * Sh + Kh <= H and (Nw - 1) * Sw + Kw <= W


def test_network_specs_and_work_counts():
    from snntc_2023_b200 import nets
    rows = nets.layer_work(nets.CIFAR_CNN, (32, 32, 3))
    assert sum(r["I"] * r["J"] for r in rows) == 3248202                      # parameters of the CIFAR-shaped net
    assert abs(8 * sum(r["R"] * r["I"] * r["J"] for r in rows) / 1e9 - 1.2408) < 1e-3   # GFLOP per sample
    rows = nets.layer_work(nets.IMAGENET_CNN, (224, 224, 3))
    assert sum(r["I"] * r["J"] for r in rows) == 31372264
    ws = nets.spec_weights(nets.MNIST_MLP, 5)
    assert [w.shape for w in ws] == [(785, 400), (401, 400), (401, 10)] and all(not w[-1].any() for w in ws)
    ws2 = nets.spec_weights(nets.MNIST_MLP, 5)
    assert all(np.array_equal(a, b) for a, b in zip(ws, ws2))                 # same seed, same bytes on every rank


def test_sequential_merge_of_sorted_runs_on_the_host():
    """The three-way merge the list-building kernels run per thread (csrc/snntc_merge.cuh) is plain C++: compiled
    for the host here and checked against numpy on random runs, empty runs and ties."""
    import subprocess
    import tempfile
    src = r"""
#include <stdint.h>
#include <string.h>
struct uint2 { unsigned x, y; };
struct uint4 { unsigned x, y, z, w; };
#include "%s"
struct HostMem {
  uint2 w[3][4];
  void load_window(int run, const uint2* src) { memcpy(w[run], src, sizeof(w[run])); }
  uint2 window(int run, int k) const { return w[run][k]; }
  void store4(uint2* dst, const uint2 (&e)[4]) const { memcpy(dst, e, sizeof(e)); }
  void store1(uint2* dst, const uint2& e) const { *dst = e; }
};
// the merge cut into `parts` pieces by value, the pieces run one after the other in reverse order
extern "C" void merge3_split(const uint2* a, const uint2* b, const uint2* c, int na, int nb, int nc, unsigned oa,
                             unsigned ob, unsigned oc, uint2* dst, int parts, int* piece_sizes) {
  const uint2* run[3] = {a, b, c};
  const int n[3] = {na, nb, nc};
  for (int part = parts - 1; part >= 0; --part) {
    int cut[3], end[3];
    snntc::merge3_cut<uint2>(run, n, part, parts, cut);
    snntc::merge3_cut<uint2>(run, n, part + 1, parts, end);
    const int count = end[0] - cut[0] + end[1] - cut[1] + end[2] - cut[2];
    piece_sizes[part] = count;
    HostMem mem;
    snntc::merge3_runs_blocked_range<uint2, HostMem>(a, b, c, oa, ob, oc, cut[0], cut[1], cut[2], count, dst, mem);
  }
}
extern "C" void merge3(const uint2* a, const uint2* b, const uint2* c, unsigned oa, unsigned ob, unsigned oc,
                       int total, uint2* dst, int terminate, int blocked) {
  if (blocked) {
    HostMem mem;
    snntc::merge3_runs_blocked<uint2, HostMem>(a, b, c, oa, ob, oc, total, dst, terminate != 0, mem);
  } else {
    snntc::merge3_runs<uint2, uint4>(a, b, c, oa, ob, oc, total, dst, terminate != 0);
  }
}
""" % os.path.join(ROOT, "snntc_2023_b200", "csrc", "snntc_merge.cuh")
    with tempfile.TemporaryDirectory() as d:
        cpp = os.path.join(d, "m.cpp"); so = os.path.join(d, "m.so")
        open(cpp, "w").write(src)
        subprocess.check_call(["g++", "-O2", "-std=c++17", "-shared", "-fPIC", "-o", so, cpp])
        lib = ctypes.CDLL(so)
        rng = np.random.default_rng(0)
        for trial in range(400):
            blocked = trial >= 200     # the variant that moves four entries per access: runs padded to four entries
            n = [int(rng.integers(0, 40)) if rng.random() > 0.2 else 0 for _ in range(3)]
            runs, offs = [], [int(rng.integers(0, 1000)) for _ in range(3)]
            for k in range(3):
                vals = np.sort(np.round(np.exp(rng.random(n[k]) * 2), 1 if trial % 2 else 6).astype(np.float32))   # odd trials: many ties
                cap = (n[k] + 1 + 3) // 4 * 4
                ent = np.full((cap, 2), 0x12345678, np.uint32)        # whatever lies behind the terminator is never used
                ent[:n[k], 0] = vals.view(np.uint32)
                ent[:n[k], 1] = rng.integers(0, 1 << 20, n[k])
                ent[n[k]] = (0x7f800000, 0)
                runs.append(ent)
            total = sum(n)
            dst = np.full(((total + 1 + 3) // 4 * 4 + 4, 2), 0xDEADBEEF, np.uint32)
            assert dst.ctypes.data % 16 == 0
            ptr = lambda a: a.ctypes.data_as(ctypes.c_void_p)
            lib.merge3(ptr(runs[0]), ptr(runs[1]), ptr(runs[2]), offs[0], offs[1], offs[2], total, ptr(dst), trial % 3 == 0,
                       int(blocked))
            got_x = dst[:total, 0].copy().view(np.float32)
            want = np.concatenate([np.stack([r[:m, 0].view(np.float32), (r[:m, 1] + o).astype(np.float32), np.full(m, k, np.float32)], 1)
                                   for k, (r, m, o) in enumerate(zip(runs, n, offs))]) if total else np.zeros((0, 3), np.float32)
            order = np.lexsort((np.arange(total), want[:, 2], want[:, 0])) if total else []
            assert np.array_equal(got_x, want[order, 0])
            assert np.array_equal(dst[:total, 1], want[order, 1].astype(np.uint32))   # ties: earlier run first, order kept inside a run
            if trial % 3 == 0:
                assert tuple(dst[total]) == (0x7f800000, 0)
            elif not blocked:
                assert dst[total, 0] == 0xDEADBEEF
            if not blocked:
                assert dst[total + 1, 0] == 0xDEADBEEF
            else:   # whole groups of four are written, nothing behind the last group
                assert np.all(dst[(total + 3) // 4 * 4 + (1 if (trial % 3 == 0 and total % 4 == 0) else 0):, 0] == 0xDEADBEEF)
            # the same merge cut into pieces by value: same entries in the same places, nothing written behind them
            for parts in (2, 8, 32):
                dst2 = np.full_like(dst, 0xDEADBEEF)
                sizes = np.zeros(parts, np.int32)
                lib.merge3_split(ptr(runs[0]), ptr(runs[1]), ptr(runs[2]), n[0], n[1], n[2], offs[0], offs[1], offs[2],
                                 ptr(dst2), parts, sizes.ctypes.data_as(ctypes.c_void_p))
                assert int(sizes.sum()) == total and sizes.min() >= 0
                assert np.array_equal(dst2[:total], dst[:total])
                assert np.all(dst2[total:, 0] == 0xDEADBEEF)


def test_bench_reference_arm_prints_exactly_one_json_line():
    """The CPU arm of the benchmark (the reference's operators on the host cores) on a two-sample step: standard output
    holds one line, a JSON object with the keys the contract names; everything else goes to standard error."""
    import json
    import subprocess
    import sys
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1",
                        "--warmup", "0", "--cpu-sample", "2"], capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [l for l in r.stdout.splitlines() if l.strip()]
    assert len(lines) == 1, r.stdout[:500]
    line = json.loads(lines[0])
    assert line["impl"] == "reference" and line["n_gpus"] == 1 and line["steps"] == 1
    assert line["metric"] == "snn_tc_fwd_bwd_samples_per_s" and line["unit"] == "samples/s" and line["higher_is_better"] is True
    assert line["value"] > 0 and line["cpu_baseline"]["kind"] in ("reference", "port") and line["cpu_baseline"]["cores"] >= 1
    assert line["e2e"]["value"] == line["value"] and line["e2e"]["h2d_bytes_per_step"] == 0
    assert line["gpu_launches"] == 0 and line["config"]["workload"] == "cifar"
