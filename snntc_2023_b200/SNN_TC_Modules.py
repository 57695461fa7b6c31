"""Layer classes of SNN-TC with the reference's Python surface, on torch + libsnntc_b200.so.

Mirrors SNN_TC_Modules.py of the reference (constructor signatures :42-43 and :103-105, weight
layout [fan-in(+1 bias row, last), fan-out], the `Params` vectors :48-49 and :121-123, NHWC inputs,
MAX (1e5) as the no-fire value and as the SAME-padding value). The layers are torch.nn.Modules; the
reference's keras `call` is available under both `forward` and `call`.
"""
import math

import numpy as np
import torch
import torch.nn.functional as F

from . import ops


def init_weight(in_size=1, out_size=1, bias_volt=1.0, init_param=15.0):
    """randn * sqrt(init_param / in_size), plus a zero bias row appended last (reference :19-25)."""
    weight = np.random.randn(in_size, out_size) * np.sqrt(init_param / in_size)
    if bias_volt > 1e-8:
        weight = np.concatenate((weight, np.zeros([1, out_size])), axis=0)
    return weight.astype(np.float32)


def _to_weight(weight):
    if isinstance(weight, torch.Tensor):
        return weight.detach().to(torch.float32).cpu().clone()
    return torch.from_numpy(np.array(weight).astype(np.float32))


class SNN_dense(torch.nn.Module):
    """Fully connected SNN-TC layer (reference SNN_TC_Modules.py:36-84)."""

    def __init__(self, in_size=1, out_size=1, biasvolt=1.0, MAX_SPIKE_TIME=1e5, Epsilon=1e-10,
                 Spike_Threshold=1.0, Thread_per_Block=0, Blocks=0, weight=None, name=None):
        super().__init__()
        self.in_size = in_size
        self.out_size = out_size
        self.biasvolt = float(biasvolt)
        self.Params = np.array([MAX_SPIKE_TIME, Epsilon, Spike_Threshold, Thread_per_Block, Blocks, self.biasvolt],
                               dtype=np.float32)
        if weight is None:
            weight = init_weight(in_size=self.in_size, out_size=self.out_size, bias_volt=self.biasvolt)
        weight = _to_weight(weight)
        self.name = name if name is not None else "fckernel"
        if self.biasvolt > 1e-8:
            self.in_size += 1  # weight rows include the bias row
        if tuple(weight.shape) != (self.in_size, self.out_size):
            raise ValueError("weight must have shape [%d, %d], got %s" % (self.in_size, self.out_size, tuple(weight.shape)))
        self.weight = torch.nn.Parameter(weight)
        self.grad_sink = None  # optional slice of a flat gradient bucket (nets.SnnNet sets it): dW is written there

    def forward(self, X):
        return ops.snn_fc_layer(X, self.weight, self.Params, self.grad_sink)

    call = forward

    def w_sum_cost(self):
        part1 = float(self.Params[2]) - self.weight.sum(0)
        return torch.clamp(part1, min=0).mean()

    def l2_cost(self):
        return (self.weight ** 2).mean()


class SNN_conv(torch.nn.Module):
    """2-D convolutional SNN-TC layer, NHWC (reference SNN_TC_Modules.py:96-179). The MAX padding of
    SAME mode and the crop of VALID mode are done inside the CUDA kernels, not by copying the input."""

    def __init__(self, in_channel=1, out_channel=1, kernel_sizes=1, strides=1, padding='SAME', rates=1,
                 biasvolt=1.0, MAX_SPIKE_TIME=1e5, Spike_Threshold=1.0, Epsilon=1e-10,
                 Thread_per_Block=0, Blocks=0, weight=None, name=None):
        super().__init__()
        if not isinstance(kernel_sizes, (list, tuple)):
            kernel_sizes = [kernel_sizes, kernel_sizes]
        self.Kh, self.Kw = kernel_sizes[0], kernel_sizes[1]
        self.C = in_channel
        self.Kc = out_channel
        if not isinstance(strides, (list, tuple)):
            strides = [strides, strides]
        self.Sh, self.Sw = strides[0], strides[1]
        self.padding = padding.upper()
        self.cudaflag = 0
        if not isinstance(rates, (list, tuple)):
            rates = [rates, rates]
        self.rates = rates  # accepted, not implemented (as in the reference)
        self.biasvolt = float(biasvolt)
        self.Params = np.array([MAX_SPIKE_TIME, Thread_per_Block, Blocks, Epsilon, Spike_Threshold, self.cudaflag,
                                self.Kh, self.Kw, self.Sh, self.Sw, (self.padding == 'SAME'), self.biasvolt],
                               dtype=np.float32)
        self.in_size = self.Kh * self.Kw * self.C
        if weight is None:
            weight = init_weight(in_size=self.in_size, out_size=self.Kc, bias_volt=self.biasvolt)
        weight = _to_weight(weight)
        self.name = name if name is not None else "convkernel"
        if self.biasvolt > 1e-8:
            self.in_size += 1
        if tuple(weight.shape) != (self.in_size, self.Kc):
            raise ValueError("weight must have shape [%d, %d], got %s" % (self.in_size, self.Kc, tuple(weight.shape)))
        self.weight = torch.nn.Parameter(weight)
        self.grad_sink = None

    def forward(self, input):
        B, H, W, C = input.shape
        geom = ops.conv_geometry(H, W, self.Kh, self.Kw, self.Sh, self.Sw, self.padding)
        return ops.snn_cv_layer(input, self.weight, self.Params, geom, self.grad_sink)

    call = forward

    def w_sum_cost(self):
        part1 = float(self.Params[4]) - self.weight.sum(0)
        return torch.clamp(part1, min=0).mean()

    def l2_cost(self):
        return (self.weight ** 2).mean()


def _same_pad_nhwc(input, Kh, Kw, Sh, Sw, value):
    B, H, W, C = input.shape
    th = (math.ceil(H / Sh) - 1) * Sh + Kh - H
    tw = (math.ceil(W / Sw) - 1) * Sw + Kw - W
    pt, pl = int(th / 2), int(tw / 2)
    if th <= 0 and tw <= 0:
        return input
    return F.pad(input, (0, 0, pl, tw - pl, pt, th - pt), mode='constant', value=value)


def _pair(v):
    return list(v) if isinstance(v, (list, tuple)) else [v, v]


class SNN_maxpool2d(torch.nn.Module):
    """Earliest-spike pooling: pad with 1e5 and take the window minimum (reference :216-246 computes
    -MaxPool(-x) after padding with padvalue)."""

    def __init__(self, kernel_sizes=1, strides=1, padding='SAME', padvalue=1e5, name=None):
        super().__init__()
        self.Kh, self.Kw = _pair(kernel_sizes)
        self.Sh, self.Sw = _pair(strides)
        self.padding = padding.upper()
        self.padvalue = padvalue
        self.name = name if name is not None else 'maxpoolkernel'

    def forward(self, input):
        return ops.snn_minpool(input, self.Kh, self.Kw, self.Sh, self.Sw, self.padding, self.padvalue)

    call = forward


class SNN_avgpool2d(torch.nn.Module):
    """Average pooling with 1e5 padding in SAME mode (reference :251-282); plain torch glue."""

    def __init__(self, kernel_sizes=1, strides=1, padding='SAME', padvalue=1e5, name=None):
        super().__init__()
        self.Kh, self.Kw = _pair(kernel_sizes)
        self.Sh, self.Sw = _pair(strides)
        self.padding = padding.upper()
        self.padvalue = padvalue
        self.name = name if name is not None else 'avgpoolkernel'

    def forward(self, input):
        if self.padding == 'SAME':
            input = _same_pad_nhwc(input, self.Kh, self.Kw, self.Sh, self.Sw, self.padvalue)
        x = F.avg_pool2d(input.permute(0, 3, 1, 2), (self.Kh, self.Kw), (self.Sh, self.Sw))
        return x.permute(0, 2, 3, 1).contiguous()

    call = forward


class SNN_LRN(torch.nn.Module):
    """Local response normalisation over channels with 1e5 padding of the squared input (reference :182-213)."""

    def __init__(self, depth_radius=5, bias=2, alpha=0.0001, beta=0.75, **kwargs):
        super().__init__()
        self.depth_radius = depth_radius
        self.bias = bias
        self.alpha = alpha
        self.beta = beta

    def forward(self, x):
        c = x.shape[3]
        half_n = self.depth_radius // 2
        sq = F.pad(x * x, (half_n, half_n), mode='constant', value=1e5)
        scale = self.bias
        for i in range(self.depth_radius):
            scale = scale + self.alpha * sq[:, :, :, i:i + c]
        return x / scale ** self.beta

    call = forward

    def get_config(self):
        return {"alpha": self.alpha, "depth_radius": self.depth_radius, "beta": self.beta, "bias": self.bias}


def loss_func(logit=None, label=None):
    """Softmax cross-entropy on the NEGATED spike values, batch mean (reference :286-288). `label` is
    one-hot [B,classes] as in the reference, or an integer class vector [B]."""
    if logit.is_cuda and logit.dtype == torch.float32 and logit.dim() == 2:
        from . import train   # one kernel for loss and gradient instead of five framework launches
        return train.loss_func(logit, label)
    logp = F.log_softmax(-logit, dim=1)
    if label.dim() == 1 and not label.is_floating_point():
        return F.nll_loss(logp, label)
    return -(label.to(logp.dtype) * logp).sum(1).mean()


# op-level names of the reference module (SNN_TC_Modules.py:29-30, 89-90)
snnfc = ops.snnfc
snnfc_grad = ops.snnfc_grad
snncv = ops.snncv
snncv_grad = ops.snncv_grad
