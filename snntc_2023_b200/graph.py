"""Whole-step CUDA graph for an SNN-TC train step.

A train step of a small network (the MNIST-shaped MLP is ~40 kernels of a few microseconds each) is
bound by launch and Python overhead, not by the GPU. `GraphedStep` captures one full step -- input
encoding, forward, loss, backward (the operators fork their independent kernels onto the library's
auxiliary stream and join them back, which a capture records as ordinary graph edges), the gradient
all-reduce when there is one, and the optimiser update -- into a CUDA graph once, and replays it with
new data copied into the same input buffers. Shapes must not change between steps.
"""
import torch


class GraphedStep:
    def __init__(self, step_fn, example_inputs, warmup=3):
        """step_fn(*tensors) -> scalar loss tensor; it must use only the tensors it is given (plus
        parameters/optimizer state that live across steps). example_inputs fix shapes and dtypes."""
        self.static_inputs = [t.clone() for t in example_inputs]
        self.step_fn = step_fn
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):          # warm up off the default stream, as capture requires
            for _ in range(warmup):
                step_fn(*self.static_inputs)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        from . import _lib
        lib = _lib.load()
        before = lib.snntc_launch_count()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.static_loss = step_fn(*self.static_inputs)
        # kernels of this library recorded in the graph: each replay launches that many
        self.library_launches_per_replay = int(lib.snntc_launch_count() - before)
        self.replays = 0

    def __call__(self, *inputs):
        for dst, src in zip(self.static_inputs, inputs):
            dst.copy_(src, non_blocking=True)
        self.graph.replay()
        self.replays += 1
        return self.static_loss
