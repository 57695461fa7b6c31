"""Sequential SNN-TC networks built from SNN_dense / SNN_conv / SNN_maxpool2d, as the reference's
example trainers stack them (snntc-mnist.py:40-53, snntc-cifar10.py:83-147), plus the flat
parameter/gradient storage a data-parallel step needs.

A network is described by a list of layer specs:
    ("conv", Cin, Cout, k, stride)   SAME padding, bias on
    ("pool", k)                      earliest-spike pooling, stride k, SAME
    ("flatten",)                     NHWC -> [B, H*W*C]
    ("dense", In, Out)
"""
import numpy as np
import torch

from .SNN_TC_Modules import SNN_conv, SNN_dense, SNN_maxpool2d, init_weight, loss_func

MNIST_MLP = [("dense", 784, 400), ("dense", 400, 400), ("dense", 400, 10)]
CIFAR_CNN = [("conv", 3, 64, 3, 1), ("conv", 64, 64, 3, 1), ("pool", 2),
             ("conv", 64, 128, 3, 1), ("conv", 128, 128, 3, 1), ("pool", 2),
             ("conv", 128, 256, 3, 1), ("conv", 256, 256, 3, 1), ("pool", 2),
             ("flatten",), ("dense", 4096, 512), ("dense", 512, 10)]
IMAGENET_CNN = [("conv", 3, 64, 7, 2), ("pool", 2),
                ("conv", 64, 128, 3, 1), ("conv", 128, 128, 3, 1), ("pool", 2),
                ("conv", 128, 256, 3, 1), ("conv", 256, 256, 3, 1), ("pool", 2),
                ("conv", 256, 512, 3, 1), ("conv", 512, 512, 3, 1), ("pool", 2),
                ("flatten",), ("dense", 25088, 1024), ("dense", 1024, 1000)]


def spec_weights(specs, seed, biasvolt=1.0):
    """Reference initialisation (randn*sqrt(15/fan_in), zero bias row last) for every weighted layer,
    drawn from one seeded generator so that every rank and the CPU baseline hold the same values."""
    rng = np.random.RandomState(seed)
    out = []
    for s in specs:
        if s[0] == "conv":
            fan_in, fan_out = s[3] * s[3] * s[1], s[2]
        elif s[0] == "dense":
            fan_in, fan_out = s[1], s[2]
        else:
            continue
        w = rng.randn(fan_in, fan_out) * np.sqrt(15.0 / fan_in)
        if biasvolt > 1e-8:
            w = np.concatenate((w, np.zeros([1, fan_out])), axis=0)
        out.append(w.astype(np.float32))
    return out


def layer_work(specs, in_shape):
    """Per weighted layer (R, I incl. bias row, J) for a batch of ONE sample of shape in_shape (H,W,C) or (N,)."""
    import math
    shape = tuple(in_shape)
    rows = []
    first = True
    for s in specs:
        if s[0] == "conv":
            H, W, _ = shape
            Nh, Nw = math.ceil(H / s[4]), math.ceil(W / s[4])
            rows.append(dict(kind="conv", R=Nh * Nw, I=s[3] * s[3] * s[1] + 1, J=s[2], needs_dx=not first))
            shape = (Nh, Nw, s[2]); first = False
        elif s[0] == "pool":
            H, W, C = shape
            shape = (math.ceil(H / s[1]), math.ceil(W / s[1]), C)
        elif s[0] == "flatten":
            shape = (int(np.prod(shape)),)
        elif s[0] == "dense":
            rows.append(dict(kind="dense", R=1, I=s[1] + 1, J=s[2], needs_dx=not first))
            shape = (s[2],); first = False
    return rows


class SnnNet(torch.nn.Module):
    """The layers of `specs` in order. All weights live in one flat fp32 buffer (`flat_param`) and
    all weight gradients are written by the backward kernels straight into a second flat buffer
    (`flat_grad`), which is what a data-parallel step all-reduces and the optimiser consumes.

    The operators WRITE their dW into flat_grad (they do not accumulate), and autograd is told nothing
    about it. Any other term of the objective that depends on the weights (the reference's
    constraint_cost, snntc-mnist.py:55-59) reaches a weight through autograd's own `.grad`; `backward`
    below runs autograd and then folds those `.grad` tensors into flat_grad, so that flat_grad holds
    the gradient of the whole objective whatever the order in which autograd visited the terms."""

    def __init__(self, specs, weights=None, biasvolt=1.0, device="cuda"):
        super().__init__()
        self.specs = list(specs)
        layers = []
        wi = 0
        for s in self.specs:
            if s[0] == "conv":
                w = None if weights is None else weights[wi]
                layers.append(SNN_conv(s[1], s[2], s[3], s[4], "SAME", biasvolt=biasvolt, weight=w)); wi += 1
            elif s[0] == "dense":
                w = None if weights is None else weights[wi]
                layers.append(SNN_dense(s[1], s[2], biasvolt=biasvolt, weight=w)); wi += 1
            elif s[0] == "pool":
                layers.append(SNN_maxpool2d(s[1], s[1], "SAME"))
            elif s[0] == "flatten":
                layers.append(torch.nn.Flatten())
            else:
                raise ValueError("unknown layer spec %r" % (s,))
        self.layers = torch.nn.ModuleList(layers)
        self.to(device)
        self._flatten_storage()

    def weighted_layers(self):
        return [l for l in self.layers if isinstance(l, (SNN_conv, SNN_dense))]

    def _flatten_storage(self):
        ws = self.weighted_layers()
        total = sum(l.weight.numel() for l in ws)
        dev = ws[0].weight.device
        self.flat_param = torch.empty(total, dtype=torch.float32, device=dev)
        self.flat_grad = torch.zeros(total, dtype=torch.float32, device=dev)
        off = 0
        for l in ws:
            n = l.weight.numel()
            self.flat_param[off:off + n].copy_(l.weight.data.reshape(-1))
            l.weight.data = self.flat_param[off:off + n].view_as(l.weight)
            l.grad_sink = self.flat_grad[off:off + n].view_as(l.weight)
            off += n

    def forward(self, x):
        for l in self.layers:
            x = l(x)
        return x

    def loss(self, x, labels):
        return loss_func(self.forward(x), labels)

    def constraint_cost(self, K, K2):
        """K * sum_layers mean_j max(0, 1 - sum_i w_ij) + K2 * sum_layers mean(w^2) over this network's weights
        (MyModel.constraint_cost of the reference's trainers, snntc-mnist.py:55-59); differentiable."""
        from . import train
        return train.constraint_cost([l.weight for l in self.weighted_layers()], K, K2)

    def backward(self, objective):
        """objective.backward(), after which flat_grad holds d objective / d weights: the operators' dW (written
        by the kernels) plus whatever autograd accumulated in a weight's .grad for the other terms. The .grad
        of every weight is left pointing at its slice of flat_grad, for optimisers that read .grad."""
        ws = self.weighted_layers()
        for l in ws:
            l.weight.grad = None
        objective.backward()
        for l in ws:
            if l.weight.grad is not None:
                l.grad_sink.add_(l.weight.grad)
            l.weight.grad = l.grad_sink
