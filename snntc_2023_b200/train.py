"""What surrounds the SNN-TC layers in a training step of the reference's example trainers, on this
library's own kernels (csrc/snntc_train.cu) instead of framework glue:

    encode(p)                       exp(1 - p) / exp(p) input encoding            snntc-mnist.py:75
    loss_func(logit, label)         softmax cross-entropy on -logit, batch mean   SNN_TC_Modules.py:286-288
    accuracy_count(logit, label)    number of samples whose earliest spike is the label   snntc-mnist.py:82
    constraint_cost(weights, K, K2) K*sum_w mean_j max(0,1-sum_i w_ij) + K2*sum_w mean(w^2)   snntc-mnist.py:55-59
    Adam / SGDM                     Keras-formulation optimisers over one flat parameter buffer and the
                                    flat gradient buffer the backward kernels (and the all-reduce) write

Everything here needs the CUDA library; there is no CPU path.
"""

import torch

from . import _lib
from .ops import _as_cuda_f32, _ptr, _stream


def encode(p, scale=1.0, one_minus=True):
    """x = exp(scale*(1-p)) (pixel intensities -> spike times, the reference's encoding) or exp(scale*p)."""
    lib = _lib.load()
    p = _as_cuda_f32(p, "p")
    x = torch.empty_like(p)
    with torch.cuda.device(p.device):
        rc = lib.snntc_encode(p.data_ptr(), x.data_ptr(), p.numel(), float(scale), 1 if one_minus else 0, _stream(p))
    _lib.check(rc, "encode")
    return x


def _labels(label, device):
    if label.dim() == 2:   # one-hot, as the reference passes it
        label = label.argmax(1)
    return label.to(device=device, dtype=torch.int64).contiguous()


class _LossCE(torch.autograd.Function):
    """One kernel computes the mean loss, the arg-min hits and d loss / d logit."""

    @staticmethod
    def forward(ctx, logit, label):
        lib = _lib.load()
        y = _as_cuda_f32(logit, "logit")
        if y.dim() != 2:
            raise ValueError("loss_func expects logit[B,classes]")
        B, J = y.shape
        lab = _labels(label, y.device)
        sums = torch.zeros(2, dtype=torch.float32, device=y.device)
        grad = torch.empty_like(y)
        with torch.cuda.device(y.device):
            rc = lib.snntc_loss_ce(y.data_ptr(), lab.data_ptr(), grad.data_ptr(), sums.data_ptr(), B, J,
                                   1.0 / B, 1.0 / B, _stream(y))
        _lib.check(rc, "loss_func")
        ctx.save_for_backward(grad)
        ctx.mark_non_differentiable(sums)
        return sums[0].clone(), sums

    @staticmethod
    def backward(ctx, gloss, _gsums):
        (grad,) = ctx.saved_tensors
        return grad * gloss, None


def loss_func(logit=None, label=None, with_hits=False):
    """Mean softmax cross-entropy on the negated spike times. `label`: integer classes [B] or one-hot [B,C].
    with_hits=True also returns the number of samples whose arg-min output equals the label (a 0-d tensor)."""
    loss, sums = _LossCE.apply(logit, label)
    return (loss, sums[1]) if with_hits else loss


def accuracy_count(logit, label):
    with torch.no_grad():
        return loss_func(logit, label, with_hits=True)[1]


class _WeightCost(torch.autograd.Function):
    @staticmethod
    def forward(ctx, K, K2, *weights):
        lib = _lib.load()
        dev = weights[0].device
        cost = torch.zeros(1, dtype=torch.float32, device=dev)
        grads = []
        with torch.cuda.device(dev):
            for w in weights:
                w = _as_cuda_f32(w, "weight")
                rows, J = w.shape
                g = torch.zeros_like(w)
                nbytes = lib.snntc_weight_cost_workspace_bytes(J)
                ws = torch.empty(nbytes, dtype=torch.uint8, device=dev)
                rc = lib.snntc_weight_cost(w.data_ptr(), g.data_ptr(), cost.data_ptr(), rows, J, float(K), float(K2),
                                           _ptr(ws), nbytes, _stream(w))
                _lib.check(rc, "constraint_cost")
                grads.append(g)
        ctx.save_for_backward(*grads)
        return cost[0]

    @staticmethod
    def backward(ctx, gcost):
        return (None, None) + tuple(g * gcost for g in ctx.saved_tensors)


def constraint_cost(weights, K, K2):
    """K * sum over tensors of mean_j max(0, 1 - sum_i w_ij) + K2 * sum over tensors of mean(w^2); each tensor is
    a layer's whole [fan_in(+1), fan_out] weight, bias row included, as in the reference's trainable_variables."""
    weights = list(weights)
    return _WeightCost.apply(K, K2, *weights)


class _FlatOptimizer:
    def __init__(self, param, grad):
        self.param = _as_cuda_f32(param.detach() if isinstance(param, torch.nn.Parameter) else param, "param")
        self.grad = _as_cuda_f32(grad, "grad")
        if self.param.numel() != self.grad.numel():
            raise ValueError("parameter and gradient buffers differ in size")

    def zero_grad(self):
        self.grad.zero_()


class Adam(_FlatOptimizer):
    """tf.keras.optimizers.Adam over one flat fp32 buffer; the step count lives on the device, so step() can be
    captured into a CUDA graph and replayed. grad_scale multiplies the gradient first (1/world for a summed
    all-reduce)."""

    def __init__(self, param, grad, lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-7):
        super().__init__(param, grad)
        self.lr, self.beta1, self.beta2, self.eps = lr, beta1, beta2, eps
        self.m = torch.zeros_like(self.param)
        self.v = torch.zeros_like(self.param)
        self.steps = torch.zeros(1, dtype=torch.int32, device=self.param.device)

    def step(self, grad_scale=1.0):
        lib = _lib.load()
        with torch.cuda.device(self.param.device):
            rc = lib.snntc_adam_step(self.param.data_ptr(), self.grad.data_ptr(), self.m.data_ptr(), self.v.data_ptr(),
                                     self.param.numel(), float(self.lr), float(self.beta1), float(self.beta2),
                                     float(self.eps), float(grad_scale), self.steps.data_ptr(), _stream(self.param))
        _lib.check(rc, "Adam.step")


class SGDM(_FlatOptimizer):
    """tf.keras.optimizers.SGD(momentum=...): vel = momentum*vel - lr*g; w += vel."""

    def __init__(self, param, grad, lr=1e-2, momentum=0.9):
        super().__init__(param, grad)
        self.lr, self.momentum = lr, momentum
        self.vel = torch.zeros_like(self.param)

    def step(self, grad_scale=1.0):
        lib = _lib.load()
        with torch.cuda.device(self.param.device):
            rc = lib.snntc_sgdm_step(self.param.data_ptr(), self.grad.data_ptr(), self.vel.data_ptr(),
                                     self.param.numel(), float(self.lr), float(self.momentum), float(grad_scale),
                                     _stream(self.param))
        _lib.check(rc, "SGDM.step")
