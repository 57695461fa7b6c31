"""Benchmark of the SNN-TC hot path: forward+backward samples/s of an SNN-TC train step.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--config cifar|mnist|imagenet|dense1|conv3]
    python bench.py --impl reference ...        # the reference's own CPU operators on the host cores

One "step" is one train step (input encoding z=exp(t), forward, softmax-CE on -y plus the reference
trainers' constraint cost, backward through SnnCvGrad/SnnFcGrad with every weight gradient written
into one flat bucket, all-reduce of that bucket when N>1, Adam update) on one batch of synthetic
input; for the single-layer configs it is the layer's forward plus backward on a seeded upstream
gradient. Rank 0 prints ONE JSON line: the headline workload (--config, default the CIFAR-shaped
network) with its roofline, CPU baseline and reference-GPU leg, then short runs of the other
configurations under "configs", a small parity check against the CPU oracle under "parity", and at
N>1 the data-parallel checks "dp_parity_rel_l2" (gradient) and "dp_param_max_abs_spread" (weights equal on all ranks
after the timed steps) and an ImageNet-shaped step.
"""
import argparse
import json
import os
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "snn_tc_fwd_bwd_samples_per_s"
UNIT = "samples/s"

CONFIGS = {
    # name: (kind, per-GPU batch, description)
    "cifar": ("net", 256, "CIFAR-shaped SNN-TC CNN train step, 32x32x3, conv 64-64 pool 128-128 pool 256-256 pool, dense 4096-512-10"),
    "mnist": ("net", 1024, "MNIST-shaped SNN-TC MLP train step, 784-400-400-10"),
    "imagenet": ("net", 64, "ImageNet-shaped SNN-TC CNN train step, 224x224x3"),
    "dense1": ("layer", 256, "single SNN_dense 784->400 fwd+bwd, no bias"),
    "conv3": ("layer", 128, "single SNN_conv 32x32x64 -> 128, 3x3 SAME fwd+bwd, no bias"),
}


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--config", default="cifar", choices=sorted(CONFIGS))
    ap.add_argument("--batch", type=int, default=0, help="per-GPU batch (default: the config's)")
    ap.add_argument("--cpu-sample", type=int, default=0, help="samples per CPU-baseline step (default: auto)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--profile-reps", type=int, default=3, help="timed repetitions of every kernel in the per-kernel pass")
    ap.add_argument("--no-ref-gpu", action="store_true", help="skip timing the reference's own GPU operators")
    ap.add_argument("--no-graph", action="store_true", help="launch every kernel of the step from Python instead of replaying a CUDA graph")
    ap.add_argument("--no-extras", action="store_true", help="headline workload only: skip the short runs of the other configurations")
    ap.add_argument("--extra-steps", type=int, default=5, help="timed steps of each extra configuration")
    ap.add_argument("--no-parity", action="store_true", help="skip the small in-run parity check against the CPU oracle")
    return ap.parse_args()


# ----------------------------------------------------------------------------------------------- data
def net_spec(config):
    from snntc_2023_b200 import nets
    if config == "cifar":
        return nets.CIFAR_CNN, (32, 32, 3), 10
    if config == "mnist":
        return nets.MNIST_MLP, (784,), 10
    return nets.IMAGENET_CNN, (224, 224, 3), 1000


def host_batches(config, batch, count, seed):
    """`count` batches of spike TIMES t (the device encodes z=exp(t)) and integer labels."""
    rng = np.random.default_rng(seed)
    _, shape, classes = net_spec(config)
    out = []
    for _ in range(count):
        t = rng.random((batch,) + shape, dtype=np.float32)
        if config == "mnist":
            t = (1.0 - t).astype(np.float32)  # t = 1 - pixel
        out.append((t, rng.integers(0, classes, batch).astype(np.int64)))
    return out


def algorithmic_flops_per_sample(config):
    """8*R*I*J per weighted layer (forward 3, dX 2, dW 3; I includes the bias row), no credit for
    early exit or sentinel skipping; dX is not counted for the first layer of a network."""
    from snntc_2023_b200 import nets
    if config == "dense1":
        return 8.0 * 784 * 400
    if config == "conv3":
        return 8.0 * 32 * 32 * 576 * 128
    specs, shape, _ = net_spec(config)
    return float(sum(r["R"] * r["I"] * r["J"] * (8 if r["needs_dx"] else 6) for r in nets.layer_work(specs, shape)))


# ----------------------------------------------------------------------------------------------- clocks
class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.path = tempfile.mktemp(prefix="snntc_clocks_", suffix=".csv")
        self.proc = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(gpu_index), "--query-gpu=" + self.FIELDS,
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        try:
            for line in open(self.path):
                f = [c.strip() for c in line.split(",")]
                if len(f) < 8:
                    continue
                try:
                    sm.append(float(f[0])); mx.append(float(f[1]))
                except ValueError:
                    continue
                for n, v in zip(names, f[4:8]):
                    if v.lower().startswith("active"):
                        reasons.add(n)
            os.unlink(self.path)
        except OSError:
            pass
        busy = [v for v in sm if v > 0.5 * (max(mx) if mx else 1)] or sm
        return {"sm_mhz": float(np.median(busy)) if busy else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ----------------------------------------------------------------------------------------------- CPU arm
def cpu_threads():
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def cpu_step_fn(config, sample, seed):
    """Returns (fn running one CPU step over `sample` samples, kind)."""
    import oracle as O
    from oracle import ref_model
    from snntc_2023_b200 import nets
    kind = "reference" if O.ref_lib() is not None else "port"
    threads = cpu_threads()
    rng = np.random.default_rng(seed)
    if config in ("dense1", "conv3"):
        if config == "dense1":
            x = np.exp(rng.random((sample, 784))).astype(np.float32)
            w = rng.normal(2 / 784, 1 / 28, (784, 400)).astype(np.float32)
            p = O.fc_params(biasvolt=0.0)
            g = rng.standard_normal((sample, 400)).astype(np.float32)
        else:
            x = np.exp(rng.random((sample, 32, 32, 64))).astype(np.float32)
            w = rng.normal(2 / 576, 1 / 24, (576, 128)).astype(np.float32)
            p = O.cv_params(3, 3, 1, 1, "SAME", 0.0)
            g = rng.standard_normal((sample, 32, 32, 128)).astype(np.float32)
        bounds = np.linspace(0, sample, min(threads, sample) + 1).astype(int)

        def one(a, b):
            xs, gs = x[a:b], g[a:b]
            g2 = np.concatenate([gs, np.zeros_like(gs)])
            if kind == "reference" and config == "dense1":
                out = O.ref_fc_forward(xs, w, p)
                O.ref_fc_backward(g2, xs, w, p, out)
            elif kind == "reference":
                xp = O.pad_like_reference(xs, 3, 3, 1, 1, "SAME")
                y = O.ref_cv_forward(xp, w, p)
                O.ref_cv_backward(g2, xp, w, p, np.concatenate([y, np.zeros_like(y)]))
            elif config == "dense1":
                o = O.fc_forward(xs, w, p, "f32"); O.fc_backward(gs, xs, w, p, o["y"], o["inv"], "f32")
            else:
                o = O.cv_forward(xs, w, p, "f32"); O.cv_backward(gs, xs, w, p, o["y"], o["inv"], "f32")

        def fn():
            from concurrent.futures import ThreadPoolExecutor
            with ThreadPoolExecutor(max(1, len(bounds) - 1)) as ex:
                list(ex.map(lambda ab: one(*ab), [(a, b) for a, b in zip(bounds[:-1], bounds[1:]) if b > a]))
        return fn, kind, min(threads, sample)
    specs, shape, classes = net_spec(config)
    weights = nets.spec_weights(specs, 1000 * (list(CONFIGS).index(config) + 1))
    t, labels = host_batches(config, sample, 1, seed)[0]
    x = np.exp(t)

    def fn():
        ref_model.train_step(specs, weights, x, labels, threads=threads, kind=kind)
    return fn, kind, min(threads, sample)


def default_cpu_sample(config):
    per_core = {"cifar": 2, "mnist": 64, "imagenet": 1, "dense1": 64, "conv3": 1}[config]
    return max(1, per_core * cpu_threads()) if config != "imagenet" else max(1, min(cpu_threads(), 8))


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    sample = args.cpu_sample or default_cpu_sample(args.config)
    fn, kind, cores = cpu_step_fn(args.config, sample, 99)
    for _ in range(min(args.warmup, 1)):
        fn()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        fn()
    dt = time.perf_counter() - t0
    value = sample * args.steps / dt
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": min(args.warmup, 1), "ms_per_step": 1000.0 * dt / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": args.config, "description": CONFIGS[args.config][2],
                   "note": "reference CPU operators on host cores; each step is a bounded sample of the workload"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": kind,
                         "sample": "%d samples per step, batch split over %d threads" % (sample, cores)},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    emit(line)


# ----------------------------------------------------------------------------------------------- GPU arm
CONSTRAINT_K, CONSTRAINT_K2 = 100.0, 1e-2   # K, K2 of the reference's CIFAR trainer (snntc-cifar10.py:8-9)


class NetWorkload:
    def __init__(self, config, batch, device, world):
        import torch
        from snntc_2023_b200 import nets
        self.torch = torch
        self.config, self.batch, self.device, self.world = config, batch, device, world
        specs, shape, classes = net_spec(config)
        weights = nets.spec_weights(specs, 1000 * (list(CONFIGS).index(config) + 1))
        self.net = nets.SnnNet(specs, weights=weights, device=device)
        from snntc_2023_b200 import train
        self.train = train
        # Keras-formulation Adam over the flat parameter / gradient buffers (snntc-mnist.py:70), one kernel
        self.opt = train.Adam(self.net.flat_param, self.net.flat_grad, lr=1e-5)
        self.graphed = None
        self.h2d_bytes = batch * int(np.prod(shape)) * 4 + batch * 8
        self.d2h_bytes = 4
        self.optimize = True
        self.collective = True   # switched off for rank-local passes (per-kernel profiling, the gradient check on rank 0)

    def host_batches(self, count, seed):
        return host_batches(self.config, self.batch, count, seed)

    def stage(self, host):
        t, lab = host
        torch = self.torch
        return (torch.from_numpy(t).pin_memory(), torch.from_numpy(lab).pin_memory())

    def to_device(self, pinned):
        return (pinned[0].to(self.device, non_blocking=True), pinned[1].to(self.device, non_blocking=True))

    def enable_graph(self, example_batch):
        """Capture the step once; later steps replay it (snntc_2023_b200.graph.GraphedStep). One process: the whole
        step is one graph. Several: the collective stays an ordinary NCCL call between two graphs -- everything up to
        the gradient (encoding, forward, loss, backward) and the optimiser update -- so that no rank ever captures a
        collective."""
        from snntc_2023_b200.graph import GraphedStep
        if self.world == 1:
            self.graphed = GraphedStep(lambda t, lab: self.eager_step((t, lab)), list(example_batch))
        else:
            self.graphed = SplitGraphedStep(self, list(example_batch))

    def step(self, dev_batch):
        if self.graphed is not None and self.optimize and (self.collective or self.world == 1):
            return self.graphed(*dev_batch)
        return self.eager_step(dev_batch)

    def forward_backward(self, dev_batch):
        t, lab = dev_batch
        z = self.train.encode(t, one_minus=False)
        loss = self.net.loss(z, lab)
        # the reference's train_step adds the constraint cost to the loss (snntc-mnist.py:76-80)
        self.net.backward(loss + self.net.constraint_cost(CONSTRAINT_K, CONSTRAINT_K2))
        return loss.detach()

    def eager_step(self, dev_batch):
        loss = self.forward_backward(dev_batch)
        if self.world > 1 and self.collective:
            from snntc_2023_b200 import ddp
            ddp.allreduce_mean_(self.net.flat_grad, self.world)
        if self.optimize:
            self.opt.step()
        return loss


class SplitGraphedStep:
    """A data-parallel step as two CUDA graphs around one eager all-reduce of the flat gradient bucket."""

    def __init__(self, wl, example_batch):
        from snntc_2023_b200.graph import GraphedStep
        self.wl = wl
        self.fwd_bwd = GraphedStep(lambda t, lab: wl.forward_backward((t, lab)), example_batch)

        def update():
            wl.opt.step()
            return wl.net.flat_param[:1]
        # (no warm-up runs: they would apply this rank's own, not yet reduced, gradient to its copy of the weights)
        self.update = GraphedStep(update, [], warmup=0)
        self.replays = 0
        self.library_launches_per_replay = (self.fwd_bwd.library_launches_per_replay +
                                            self.update.library_launches_per_replay)

    def __call__(self, *inputs):
        from snntc_2023_b200 import ddp
        loss = self.fwd_bwd(*inputs)
        ddp.allreduce_mean_(self.wl.net.flat_grad, self.wl.world)
        self.update()
        self.replays += 1
        return loss


class LayerWorkload:
    def __init__(self, config, batch, device, world):
        import torch
        from snntc_2023_b200 import ops, train
        self.torch, self.ops, self.train = torch, ops, train
        self.config, self.batch, self.device, self.world = config, batch, device, world
        rng = np.random.default_rng(1000 * (list(CONFIGS).index(config) + 1))
        if config == "dense1":
            self.w = torch.from_numpy(rng.normal(2 / 784, 1 / 28, (784, 400)).astype(np.float32)).to(device)
            self.params = np.array([1e5, 1e-10, 1.0, 0, 0, 0.0], np.float32)
            self.xshape, self.gshape = (batch, 784), (batch, 400)
        else:
            self.w = torch.from_numpy(rng.normal(2 / 576, 1 / 24, (576, 128)).astype(np.float32)).to(device)
            self.params = np.array([1e5, 0, 0, 1e-10, 1.0, 0, 3, 3, 1, 1, 1, 0.0], np.float32)
            self.xshape, self.gshape = (batch, 32, 32, 64), (batch, 32, 32, 128)
        self.h2d_bytes = int(np.prod(self.xshape)) * 4 + int(np.prod(self.gshape)) * 4
        self.d2h_bytes = 4
        self.optimize = False
        self.collective = False
        self.graphed = None
        self.tap = None   # set by the per-kernel pass: the single layer's tensors, in the form ops.TAP records

    def host_batches(self, count, seed):
        rng = np.random.default_rng(seed)
        return [(rng.random(self.xshape, dtype=np.float32), rng.standard_normal(self.gshape).astype(np.float32))
                for _ in range(count)]

    def stage(self, host):
        torch = self.torch
        return (torch.from_numpy(host[0]).pin_memory(), torch.from_numpy(host[1]).pin_memory())

    def to_device(self, pinned):
        return (pinned[0].to(self.device, non_blocking=True), pinned[1].to(self.device, non_blocking=True))

    def enable_graph(self, example_batch):
        from snntc_2023_b200.graph import GraphedStep
        self.graphed = GraphedStep(lambda t, g: self.eager_step((t, g)), list(example_batch))

    def step(self, dev_batch):
        if self.graphed is not None:
            return self.graphed(*dev_batch)
        return self.eager_step(dev_batch)

    def eager_step(self, dev_batch):
        ops = self.ops
        t, g = dev_batch
        z = self.train.encode(t, one_minus=False)
        if self.config == "dense1":
            out = ops.snn_fc(z, self.w, self.params)
            dx, dw, _ = ops.snn_fc_grad(g, z, self.w, self.params, out)
            self.tap = [("fc", z, self.w, self.params, None, out, g, True)]
        else:
            out = ops.snn_cv(z, self.w, self.params, 1, 1, 32, 32)
            dx, dw, _ = ops.snn_cv_grad(g, z, self.w, self.params, out, 1, 1)
            self.tap = [("cv", z, self.w, self.params, (1, 1, 32, 32), out, g, True)]
        return dw[0, 0]   # one element of the weight gradient: what the end-to-end loop reads back


def time_region(torch, dist, world, fn, steps):
    """barrier + sync, `steps` calls of fn(i) between two CUDA events on the current stream, sync + barrier."""
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        fn(i)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
        dist.barrier()
    return ms


def tapped_layers(wl, batch):
    """The tensors every weighted layer's backward saw in one eager step (ops.TAP), without optimiser or collective."""
    from snntc_2023_b200 import ops
    if not hasattr(wl, "net"):
        wl.eager_step(batch)
        return list(wl.tap)
    opt, coll = wl.optimize, wl.collective
    wl.optimize, wl.collective = False, False
    ops.TAP = []
    try:
        wl.eager_step(batch)
        recs = ops.TAP
    finally:
        ops.TAP = None
        wl.optimize, wl.collective = opt, coll
    return recs


def profile_kernels(torch, wl, batch, reps):
    """Per-kernel CUDA-event timings: every weighted layer's operator calls are replayed on the tensors of one
    real step (activations, upstream gradients as sparse as the pooling layers leave them), one kernel group at a
    time through the measurement build: the list builder alone, the walk alone (lists kept in the workspace), the
    backward with only dX, the backward with only dW (each backward call also runs the small u kernel)."""
    from snntc_2023_b200 import _lib, ops
    agg = {}

    def timed(fn):
        fn()
        torch.cuda.synchronize()
        e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps

    for kind, X, W, params, geom, out, grad, need_dx in tapped_layers(wl, batch):
        X, W, out, grad = X.detach(), W.detach(), out.detach(), grad.detach()
        rows, J = W.shape
        if kind == "fc":
            R = X.shape[0]
            ws = ops.fc_forward_workspace(R, X.shape[1], J, X.device)
            scratch = torch.empty_like(out)
            fwd = lambda o: ops.snn_fc(X, W, params, opts=o, workspace=ws, out=scratch)
            bwd = lambda o, dx: ops.snn_fc_grad(grad, X, W, params, out, need_input_grad=dx, opts=o)
        else:
            pt, pl, Nh, Nw = geom
            R = X.shape[0] * Nh * Nw
            ws = ops.cv_forward_workspace(X, W, params, Nh, Nw)
            scratch = torch.empty_like(out)
            fwd = lambda o: ops.snn_cv(X, W, params, pt, pl, Nh, Nw, opts=o, workspace=ws, out=scratch)
            bwd = lambda o, dx: ops.snn_cv_grad(grad, X, W, params, out, pt, pl, need_input_grad=dx, opts=o)
        rij = float(R) * rows * J
        parts = [("lists", lambda: fwd(_lib.options(forward_parts=1)), 0.0),
                 ("walk", lambda: fwd(_lib.options(forward_parts=2)), 3.0 * rij),
                 ("dw", lambda: bwd(_lib.options(backward_parts=2), False), 3.0 * rij)]
        if need_dx:
            parts.append(("dx", lambda: bwd(_lib.options(backward_parts=1), True), 2.0 * rij))
        fwd(_lib.options())   # a complete forward first: the walk-only call needs this layer's lists in the workspace
        for name, fn, flops in parts:
            ms = timed(fn)
            a = agg.setdefault((name, kind, R, rows, J), [0.0, 0, flops])
            a[0] += ms; a[1] += 1
        del ws, scratch
    return agg


def measure_fp32_peak(torch):
    import ctypes
    from snntc_2023_b200 import _lib
    lib = _lib.load_measure()
    sink = torch.zeros(4, device="cuda")
    flops = ctypes.c_double(0)
    stream = torch.cuda.current_stream().cuda_stream
    best = 0.0
    for it in range(4):
        e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
        e0.record()
        rc = lib.snntc_fp32_probe(sink.data_ptr(), 1 << 15, 148 * 8, ctypes.byref(flops), stream)
        e1.record()
        torch.cuda.synchronize()
        if rc != 0:
            return None
        if it > 0:
            best = max(best, flops.value / (e0.elapsed_time(e1) * 1e-3) / 1e12)
    return best


def time_reference_gpu(torch, wl, config, batch):
    """Times the reference's OWN GPU operators (snn*_kernels.cu.cc compiled unmodified for sm_100a,
    oracle/_ref/libsnntc_ref_gpu.so) on the same layer inputs as one step of the workload: per weighted
    layer the MAX padding copy SNN_conv.call makes, the forward functor and the gradient functor (which
    always computes dX), with their im2col/sort temporaries and per-launch device syncs. Pooling, loss
    and optimiser are left out of this figure. Returns None when the library is not available."""
    import oracle as O
    if O.ref_gpu_lib() is None:
        return None
    from snntc_2023_b200 import SNN_TC_Modules as M
    import torch.nn.functional as F
    jobs = []   # (kind, x, weight, params, (Kh,Kw,Sh,Sw))
    if hasattr(wl, "net"):
        t, lab = wl.to_device(wl.stage(host_batches(config, batch, 1, 4242)[0]))
        h = torch.exp(t)
        with torch.no_grad():
            for l in wl.net.layers:
                if isinstance(l, M.SNN_conv):
                    jobs.append(("conv", h, l.weight.detach(), l.Params, (l.Kh, l.Kw, l.Sh, l.Sw)))
                elif isinstance(l, M.SNN_dense):
                    jobs.append(("dense", h, l.weight.detach(), l.Params, None))
                h = l(h)
    elif config == "dense1":
        jobs.append(("dense", torch.exp(torch.rand(wl.xshape, device="cuda")), wl.w, wl.params, None))
    else:
        jobs.append(("conv", torch.exp(torch.rand(wl.xshape, device="cuda")), wl.w, wl.params, (3, 3, 1, 1)))
    need = 0
    for kind, x, w, p, k in jobs:
        if kind == "conv":
            B, H, W, C = x.shape
            rows = B * (-(-H // k[2])) * (-(-W // k[3]))
            need = max(need, 7 * rows * k[0] * k[1] * C * 4)
        else:
            need = max(need, 7 * x.numel() * 4)
    rg = O.RefGpu(min(need + (256 << 20), 40 << 30))
    total_ms, per_layer = 0.0, []
    for kind, x, w, p, k in jobs:
        torch.cuda.synchronize()
        e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
        e0.record()
        if kind == "conv":
            B, H, W, C = x.shape
            pt, pl, Nh, Nw, Hp, Wp = O.conv_geometry(H, W, k[0], k[1], k[2], k[3], "SAME")
            xp = F.pad(x, (0, 0, pl, Wp - W - pl, pt, Hp - H - pt), value=float(p[0]))
            out = rg.cv_forward(xp, w, p)
            g = torch.randn_like(out); g[B:] = 0
            e0.record()   # the random upstream gradient is not part of the reference's work
            xp = F.pad(x, (0, 0, pl, Wp - W - pl, pt, Hp - H - pt), value=float(p[0]))
            out = rg.cv_forward(xp, w, p)
            rg.cv_backward(g, xp, w, p, out)
        else:
            B = x.shape[0]
            out = rg.fc_forward(x.contiguous(), w, p)
            g = torch.randn_like(out); g[B:] = 0
            e0.record()
            out = rg.fc_forward(x.contiguous(), w, p)
            rg.fc_backward(g, x.contiguous(), w, p, out)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        total_ms += ms
        per_layer.append({"op": kind, "in": list(x.shape), "out": int(w.shape[1]), "ms": ms})
    del rg
    return {"ms_per_step": total_ms, "value": batch / (total_ms * 1e-3), "unit": UNIT, "layers": per_layer,
            "what": "reference snn*_kernels.cu.cc compiled unmodified for sm_100a, forward+backward of every weighted "
                    "layer incl. its padding copy, temporaries and device syncs; pooling/loss/optimiser excluded"}


def csrc_hash():
    """Content hash of the CUDA sources: a capture under profiles/ records the hash it was taken at."""
    import hashlib
    d = os.path.join(ROOT, "snntc_2023_b200", "csrc")
    h = hashlib.sha256()
    for name in sorted(os.listdir(d)):
        if name.endswith((".cu", ".cuh")):
            h.update(name.encode())
            h.update(open(os.path.join(d, name), "rb").read())
    return h.hexdigest()[:16]


def in_run_parity(torch):
    """Three small operator calls against the CPU oracle (the checker; nothing here is timed): a dense layer, a
    hidden 3x3 conv layer of the benchmark networks and its backward. Returns the protocol's figures."""
    import oracle as O
    from oracle import parity as P
    from snntc_2023_b200 import ops
    before = len(P.REPORT)
    x, w = P.make_inputs(1, (32, 784), (785, 400), "ref", bias=True)
    p = O.fc_params(biasvolt=1.0)
    out = ops.snn_fc(torch.from_numpy(x).cuda(), torch.from_numpy(w).cuda(), p).cpu().numpy()
    P.check_forward(out[:32], out[32:], O.fc_forward(x, w, p, "f32"), O.fc_forward(x, w, p, "f64"), rows=x, what="bench dense 784->400")
    B, H, W, C, Kc = 2, 12, 12, 64, 128
    x, w = P.make_inputs(2, (B, H, W, C), (9 * C + 1, Kc), "ref", bias=True)
    p = O.cv_params(3, 3, 1, 1, "SAME", 1.0)
    xd, wd = torch.from_numpy(x).cuda(), torch.from_numpy(w).cuda()
    outd = ops.snn_cv(xd, wd, p, 1, 1, H, W)
    out = outd.cpu().numpy()
    P.check_forward(out[:B], out[B:], O.cv_forward(x, w, p, "f32"), O.cv_forward(x, w, p, "f64"),
                    rows=P.im2col_rows(x, 3, 3, 1, 1, "SAME"), what="bench conv 64->128")
    g = np.random.default_rng(3).standard_normal((B, H, W, Kc)).astype(np.float32)
    dx, dw, _ = ops.snn_cv_grad(torch.from_numpy(g).cuda(), xd, wd, p, outd, 1, 1)
    ref = O.cv_backward(g, x, w, p, out[:B], out[B:], "f64")
    P.check_close(dx.cpu().numpy(), ref["dx"], "bench conv dX", abs_sum=ref["dx_abs"])
    P.check_close(dw.cpu().numpy(), ref["dw"], "bench conv dW", abs_sum=ref["dw_abs"])
    s = P.summary(P.REPORT[before:])
    s["gradients"] = "dX, dW within 1e-4*|b| + 1e-5*rms + 1e-6*sum|terms| and relative L2 <= 1e-5 of the float64 oracle"
    return s


def build_workload(config, batch, device, world, use_graph):
    """Constructs the workload, stages 4 rotating input batches, warms up and (single GPU) captures the step."""
    import torch
    kind = CONFIGS[config][0]
    wl = (NetWorkload if kind == "net" else LayerWorkload)(config, batch, device, world)
    rank = int(os.environ.get("RANK", "0"))
    nb = 4
    seed = 1000 * (list(CONFIGS).index(config) + 1) + rank
    pinned = [wl.stage(h) for h in wl.host_batches(nb, seed)]
    resident = [wl.to_device(p) for p in pinned]
    torch.cuda.synchronize()
    for i in range(3):   # warm-up (also sizes the caching allocator)
        wl.step(resident[i % nb])
    torch.cuda.synchronize()
    note = "eager launches"
    if use_graph and (world == 1 or kind == "net"):
        try:
            wl.enable_graph(resident[0])
            for i in range(3):
                wl.step(resident[i % nb])
            torch.cuda.synchronize()
            note = "whole step replayed as one CUDA graph" if world == 1 else \
                "forward+backward and optimiser update replayed as two CUDA graphs around one eager NCCL all-reduce"
        except Exception as e:   # capture is an optimisation: fall back to eager launches and say so
            wl.graphed = None
            note = "eager launches (graph capture failed: %s)" % (str(e).splitlines()[0][:120],)
            torch.cuda.synchronize()
    return wl, pinned, resident, note


def measure(torch, dist, lib, wl, pinned, resident, world, steps, warmup):
    """Device-resident and end-to-end throughput of a prepared workload."""
    nb = len(resident)
    for i in range(max(0, warmup - 3)):
        wl.step(resident[i % nb])
    l0 = lib.snntc_launch_count()
    g0 = wl.graphed.replays if wl.graphed is not None else 0
    ms = time_region(torch, dist, world, lambda i: wl.step(resident[i % nb]), steps)
    launches = lib.snntc_launch_count() - l0
    if wl.graphed is not None:   # replayed kernels are not seen by the library's own counter
        launches += (wl.graphed.replays - g0) * wl.graphed.library_launches_per_replay

    # end to end: pinned host -> device every step, one value read back every step
    def e2e_step(i):
        b = wl.to_device(pinned[i % nb])
        float(wl.step(b).item())
    for i in range(2):
        e2e_step(i)
    ms_e2e = time_region(torch, dist, world, e2e_step, steps)
    return ms, ms_e2e, int(launches)


def run_gpu_arm(args):
    import torch
    import torch.distributed as dist
    from snntc_2023_b200 import _lib
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the SNN-TC operators have no CPU path (use --impl reference for the CPU arm)")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        import datetime
        # a short timeout: a rank that misses a collective must end the run in minutes, not hang it
        dist.init_process_group("nccl", device_id=device, timeout=datetime.timedelta(seconds=120))
    lib = _lib.load()
    kind, def_batch, desc = CONFIGS[args.config]
    batch = args.batch or def_batch
    wl, pinned, resident, graph_note = build_workload(args.config, batch, device, world, not args.no_graph)

    # ---- headline: device-resident throughput with clocks sampled during the timed region, then end to end
    sampler = ClockSampler(local) if rank == 0 else None
    ms, ms_e2e, launches = measure(torch, dist, lib, wl, pinned, resident, world, args.steps, max(args.warmup, 3))
    clocks = sampler.stop() if sampler else None
    value = batch * world * args.steps / (ms * 1e-3)
    e2e_value = batch * world * args.steps / (ms_e2e * 1e-3)

    # ---- N > 1: what the all-reduce computed against the gradient of the global batch formed on rank 0 alone
    dp_parity = None
    param_spread = None
    if world > 1 and kind == "net":
        from snntc_2023_b200 import ddp
        # after the timed steps every rank must hold the same weights: largest |w - w of rank 0| over all ranks
        ref_param = wl.net.flat_param.detach().clone()
        dist.broadcast(ref_param, src=0)
        spread = (wl.net.flat_param.detach() - ref_param).abs().max().reshape(1)
        dist.all_reduce(spread, op=dist.ReduceOp.MAX)
        param_spread = float(spread.item())
        opt = wl.optimize
        wl.optimize = False
        wl.eager_step(resident[0])                  # every rank: its own first batch, gradients all-reduced to the mean
        reduced = wl.net.flat_grad.double().clone()
        torch.cuda.synchronize()
        if rank == 0:
            wl.collective = False
            acc = torch.zeros_like(reduced)
            base = 1000 * (list(CONFIGS).index(args.config) + 1)
            for r in range(world):                  # the other ranks' batches are regenerated from their seeds
                b = wl.to_device(wl.stage(wl.host_batches(1, base + r)[0]))
                wl.eager_step(b)
                acc += wl.net.flat_grad.double()
            acc /= world
            dp_parity = float((reduced - acc).norm() / acc.norm())
            wl.collective = True
        wl.optimize = opt
        dist.barrier()

    line = None
    fp32_peak = None
    if rank == 0:
        flops_sample = algorithmic_flops_per_sample(args.config)
        fp32_peak = measure_fp32_peak(torch)
        agg = profile_kernels(torch, wl, resident[0], max(1, args.profile_reps))
        peaks = {}
        try:
            peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        except Exception:
            pass
        hbm_peak, hbm_src = (peaks["hbm_gbs"], "measured") if "hbm_gbs" in peaks else (6650.0, "fallback")
        # group by kernel kind, find the dominant one
        kinds = {}
        layers = []
        for key, (tms, n, flops) in sorted(agg.items()):
            k = kinds.setdefault(key[0], [0.0, 0.0, 0])
            k[0] += tms; k[1] += flops * n; k[2] += n
            layers.append({"kernel": key[0], "op": key[1], "R": key[2], "I": key[3], "J": key[4],
                           "ms": tms / max(n, 1), "tflops": flops / (tms / max(n, 1) * 1e-3) / 1e12})
        total_ms = sum(v[0] for v in kinds.values()) or 1.0
        dom = max(kinds, key=lambda k: kinds[k][0])
        dms, dflops, dn = kinds[dom]
        names = {"lists": "snn_pixel_runs_kernel+snn_row_runs_kernel+snn_field_lists_kernel (3x3 stride-1 conv) / snn_small_rows_kernel / snn_sort_kernel",
                 "walk": "snn_walk_kernel/snn_walk2_smemw_kernel/snn_walk2_kernel(+snn_wbound_kernel)",
                 "dx": "snn_dx_sparse_kernel(+snn_act_lists_kernel, snn_weight_transpose_kernel)/snn_dx_wide_kernel/snn_dx_kernel(+snn_u_kernel)",
                 "dw": "snn_dw_tma_kernel/snn_dw_skip_kernel/snn_dw_small_kernel/snn_dw_kernel(+snn_u_kernel, snn_dw_reduce_kernel)"}
        traffic, traffic_stale = None, None
        try:
            tj = json.load(open(os.path.join(ROOT, "profiles", "traffic.json")))
            traffic = tj.get(args.config, {}).get(dom)
            traffic_stale = tj.get("csrc_sha16") != csrc_hash()
        except Exception:
            pass
        achieved = dflops / (dms * 1e-3) / 1e12
        roofline = {
            "bound": "fp32", "kernel": names[dom], "achieved": achieved, "peak": fp32_peak, "unit": "TFLOP/s",
            "frac": (achieved / fp32_peak) if fp32_peak else None, "traffic": traffic, "traffic_stale": traffic_stale,
            "peak_source": "FMA-only probe kernel timed in this run (MEASURED_PEAKS.json holds no FP32 figure)",
            "launches_per_step": dn, "ms_per_step": dms, "share_of_kernel_time": dms / total_ms,
            "kernel_ms_per_step": {k: v[0] for k, v in kinds.items()},
            "kernel_frac_of_fp32_peak": {k: (v[1] / (v[0] * 1e-3) / 1e12 / fp32_peak) if (fp32_peak and v[1]) else None for k, v in kinds.items()},
            "kernel_shares": {names[k]: v[0] / total_ms for k, v in kinds.items()},
            "how": "every kernel group of every weighted layer replayed alone on the tensors of one real step, CUDA events, mean of %d" % max(1, args.profile_reps),
            "step": {"algorithmic_tflops": flops_sample * batch / (ms / args.steps * 1e-3) / 1e12,
                     "frac_of_fp32_peak": (flops_sample * batch / (ms / args.steps * 1e-3) / 1e12 / fp32_peak) if fp32_peak else None},
            "hbm_peak_gbs": hbm_peak, "hbm_peak_source": hbm_src, "layers": layers,
        }
        cpu = None
        if world == 1 and not args.no_cpu_baseline:
            sample = args.cpu_sample or default_cpu_sample(args.config)
            fn, ckind, cores = cpu_step_fn(args.config, sample, 99)
            t0 = time.perf_counter(); reps = 0
            while True:
                fn(); reps += 1
                if time.perf_counter() - t0 > 10.0 or reps >= 3:
                    break
            dt = time.perf_counter() - t0
            cpu = {"value": sample * reps / dt, "unit": UNIT, "cores": cores, "kind": ckind,
                   "sample": "%d samples per step x %d steps, batch split over %d threads" % (sample, reps, cores)}
        ref_gpu = None
        if world == 1 and not args.no_ref_gpu:
            try:
                ref_gpu = time_reference_gpu(torch, wl, args.config, batch)
            except Exception as e:  # the reference arm must never take the bench line down with it
                ref_gpu = {"unavailable": "%s: %s" % (type(e).__name__, e)}
            if ref_gpu and "value" in ref_gpu:
                ref_gpu["speedup_of_this_build"] = value / ref_gpu["value"]
        parity = None
        if not args.no_parity:
            try:
                parity = in_run_parity(torch)
            except AssertionError as e:
                parity = {"failed": str(e)[:300]}
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": args.config, "description": desc, "per_gpu_batch": batch, "global_batch": batch * world,
                       "parallelism": "dp%d" % world, "weights": "reference init randn*sqrt(15/fan_in), zero bias row" if kind == "net" else "N(2/I,1/I), no bias",
                       "l2": "4 rotating input batches; activations of the conv layers exceed the 126 MB L2",
                       "objective": "softmax-CE on -y + constraint cost (K=100, K2=1e-2)" if kind == "net" else None,
                       "optimizer": "Adam (fused, flat parameter buffer)" if kind == "net" else None,
                       "launch": graph_note},
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": wl.h2d_bytes, "d2h_bytes_per_step": wl.d2h_bytes,
                    "ms_per_step": ms_e2e / args.steps},
            "gpu_launches": int(launches), "clocks": clocks, "roofline": roofline, "cpu_baseline": cpu,
            "reference_gpu": ref_gpu, "parity": parity,
        }
        if dp_parity is not None:
            line["dp_parity_rel_l2"] = dp_parity
            line["dp_param_max_abs_spread"] = param_spread

    # ---- the other configurations, briefly (the headline's objects are released first)
    extras = {}
    if not args.no_extras:
        del wl, pinned, resident
        torch.cuda.empty_cache()
        extra_names = [c for c in ("conv3", "dense1", "mnist", "imagenet") if c != args.config] if world == 1 else \
                      [c for c in ("imagenet",) if c != args.config]
        for cfg in extra_names:
            try:
                b = CONFIGS[cfg][1]
                w2, p2, r2, note2 = build_workload(cfg, b, device, world, not args.no_graph)
                ms2, ms2_e2e, l2 = measure(torch, dist, lib, w2, p2, r2, world, args.extra_steps, 3)
                entry = {"value": b * world * args.extra_steps / (ms2 * 1e-3), "unit": UNIT, "ms_per_step": ms2 / args.extra_steps,
                         "per_gpu_batch": b, "steps": args.extra_steps, "launch": note2, "gpu_launches": l2,
                         "e2e": {"value": b * world * args.extra_steps / (ms2_e2e * 1e-3), "h2d_bytes_per_step": w2.h2d_bytes,
                                 "d2h_bytes_per_step": w2.d2h_bytes}}
                if rank == 0:
                    fs = algorithmic_flops_per_sample(cfg)
                    entry["step_frac_of_fp32"] = (fs * b / (ms2 / args.extra_steps * 1e-3) / 1e12 / fp32_peak) if fp32_peak else None
                    if world == 1 and not args.no_ref_gpu:
                        try:
                            rg = time_reference_gpu(torch, w2, cfg, b)
                            if rg and "value" in rg:
                                entry["reference_gpu_ms_per_step"] = rg["ms_per_step"]
                                entry["reference_gpu_speedup"] = entry["value"] / rg["value"]
                        except Exception as e:
                            entry["reference_gpu_speedup"] = None
                            entry["reference_gpu_error"] = "%s: %s" % (type(e).__name__, str(e)[:120])
                extras[cfg] = entry
                del w2, p2, r2
                torch.cuda.empty_cache()
            except Exception as e:
                extras[cfg] = {"failed": "%s: %s" % (type(e).__name__, str(e)[:200])}
                if world > 1:
                    raise
        if line is not None:
            line["configs"] = extras

    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if line is not None:
        emit(line)


_RESULT_OUT = None


def emit(line):
    """The one JSON line, written to the process's original standard output."""
    out = _RESULT_OUT if _RESULT_OUT is not None else sys.stdout
    out.write(json.dumps(line) + "\n")
    out.flush()


def main():
    global _RESULT_OUT
    args = parse_args()
    # Standard output carries exactly one line, the result. Libraries that write there on their own (NCCL prints its
    # version line to file descriptor 1) are sent to standard error: descriptor 1 is pointed at descriptor 2 for the
    # rest of the process and the result goes to a duplicate of the original.
    sys.stdout.flush()
    _RESULT_OUT = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)
    if args.impl == "reference":
        run_reference_arm(args)
    else:
        run_gpu_arm(args)


if __name__ == "__main__":
    main()
