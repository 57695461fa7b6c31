"""Operator-level API: the four SNN-TC ops on torch CUDA tensors, calling libsnntc_b200.so.

Names, argument order and packed layouts follow the reference's TensorFlow ops
(snntc/snnfc_ops.cc:6-30, snnfcgrad_ops.cc:6-23, snncv_ops.cc:6-35, snncvgrad_ops.cc:6-23):

    snn_fc(in[B,I], weight[I(+1),J], params[6])                      -> out[2B,J]
    snn_fc_grad(grad[2B,J], in, weight, params, oldout[2B,J])         -> (grad_in, grad_weight, grad_params)
    snn_cv(in[B,H,W,C] already padded/cropped, weight, params[12])    -> out[2B,Nh,Nw,Kc]
    snn_cv_grad(grad, in, weight, params, oldout)                     -> (grad_in, grad_weight, grad_params)

`snnfc` / `snncv` are the differentiable forms (what `tf.load_op_library(...).snn_fc` plus
`@ops.RegisterGradient` gave the reference, SNN_TC_Modules.py:29-33, 89-93). The layer classes use
the `*_layer` forms, which take the UNPADDED image plus padding amounts and return only the spike
values, so neither a padded copy nor the packed second half ever goes through autograd.

torch is used for device memory and streams only; all arithmetic is in the CUDA library. There is no
CPU path: a CPU tensor raises.
"""
import numpy as np
import torch

from . import _lib


# ------------------------------------------------------------------------------------------ replay tap
# When TAP is a list, the layer forms below append what their backward was called with:
# (kind, x, weight, params, geom, packed forward output, upstream gradient). bench.py sets it for one step and
# then times the kernels of every layer apart on exactly those tensors; nothing else reads it.
TAP = None


# ------------------------------------------------------------------------------------------ helpers
def _as_cuda_f32(t, name):
    if not isinstance(t, torch.Tensor):
        if hasattr(t, "__dlpack__"):
            t = torch.from_dlpack(t)
        else:
            raise TypeError("%s must be a torch tensor or a DLPack-capable CUDA array" % name)
    if not t.is_cuda:
        raise _lib.SnntcError("%s is not on a CUDA device: the SNN-TC operators have no CPU implementation" % name)
    if t.dtype != torch.float32:
        raise ValueError("%s must be float32 (the operators are fp32 only), got %s" % (name, t.dtype))
    return t.contiguous()


def _params(p, n):
    if isinstance(p, torch.Tensor):
        p = p.detach().cpu().numpy()
    p = np.ascontiguousarray(np.asarray(p, dtype=np.float32).reshape(-1))
    if p.size != n:
        raise ValueError("params must hold %d values, got %d" % (n, p.size))
    return p


def _stream(t):
    return torch.cuda.current_stream(t.device).cuda_stream


def _workspace(nbytes, device):
    if nbytes == 0:
        return None, 0
    ws = torch.empty((nbytes + 3) // 4, dtype=torch.float32, device=device)
    return ws, ws.numel() * 4


def _ptr(t):
    return 0 if t is None else t.data_ptr()


def _opts_ptr(opts):
    import ctypes
    return ctypes.cast(opts, ctypes.c_void_p).value


def conv_geometry(H, W, Kh, Kw, Sh, Sw, padding):
    """(pad_top, pad_left, Nh, Nw) of SNN_conv: SAME pads with MAX by
    total=(ceil(H/S)-1)*S+K-H, before=total//2; VALID drops trailing rows/columns
    (SNN_TC_Modules.py:147-166)."""
    import math
    if str(padding).upper() == "SAME":
        th = (math.ceil(H / Sh) - 1) * Sh + Kh - H
        tw = (math.ceil(W / Sw) - 1) * Sw + Kw - W
        pt, pl = int(th / 2), int(tw / 2)
        Nh, Nw = (H + th - Kh) // Sh + 1, (W + tw - Kw) // Sw + 1
    else:
        pt = pl = 0
        Nh, Nw = int((H - Kh) / Sh + 1.0), int((W - Kw) / Sw + 1.0)
    return pt, pl, Nh, Nw


# ------------------------------------------------------------------------------------------ raw ops
# `opts` (an opts8 vector from _lib.options) selects kernels explicitly through the measurement build of the
# library; `workspace` lets a caller keep the scratch between two calls (lists built by one, walked by the next).
def snn_fc(inp, weight, params, opts=None, workspace=None, out=None):
    x = _as_cuda_f32(inp, "in"); w = _as_cuda_f32(weight, "weight"); p = _params(params, 6)
    if x.dim() != 2 or w.dim() != 2:
        raise ValueError("snn_fc expects in[B,I] and weight[rows,J]")
    B, I = x.shape
    rows, J = w.shape
    lib = _lib.load() if opts is None else _lib.load_measure()
    with torch.cuda.device(x.device):
        if out is None:
            out = torch.empty((2 * B, J), dtype=torch.float32, device=x.device)
        ws, wsb = (workspace, workspace.numel() * 4) if workspace is not None else \
            _workspace(lib.snntc_fc_forward_workspace_bytes(B, I, J), x.device)
        if opts is None:
            rc = lib.snntc_fc_forward(x.data_ptr(), w.data_ptr(), p.ctypes.data, out.data_ptr(), B, I, rows, J,
                                      _ptr(ws), wsb, _stream(x))
        else:
            rc = lib.snntc_measure_fc_forward(x.data_ptr(), w.data_ptr(), p.ctypes.data, out.data_ptr(), B, I, rows, J,
                                              _ptr(ws), wsb, _opts_ptr(opts), _stream(x))
    _lib.check(rc, "SnnFc")
    return out


def fc_forward_workspace(B, I, J, device):
    lib = _lib.load()
    return _workspace(lib.snntc_fc_forward_workspace_bytes(B, I, J), device)[0]


def snn_fc_infer(inp, weight, params, khist=None):
    """Spike values only, [B,J]: SnnFc without the 1/(sum w - theta) half (snntc_fc_infer). `khist`: an int32
    CUDA tensor of I+2 zeros (I without the bias row) that receives the histogram of causal-set sizes."""
    lib = _lib.load()
    x = _as_cuda_f32(inp, "in"); w = _as_cuda_f32(weight, "weight"); p = _params(params, 6)
    if x.dim() != 2 or w.dim() != 2:
        raise ValueError("snn_fc_infer expects in[B,I] and weight[rows,J]")
    B, I = x.shape
    rows, J = w.shape
    if khist is not None and (khist.dtype != torch.int32 or khist.numel() < I + 2 or not khist.is_cuda):
        raise ValueError("khist must be an int32 CUDA tensor of at least fan_in + 2 elements")
    with torch.cuda.device(x.device):
        out = torch.empty((B, J), dtype=torch.float32, device=x.device)
        ws, wsb = _workspace(lib.snntc_fc_forward_workspace_bytes(B, I, J), x.device)
        rc = lib.snntc_fc_infer(x.data_ptr(), w.data_ptr(), p.ctypes.data, out.data_ptr(), _ptr(khist), B, I, rows, J,
                                _ptr(ws), wsb, _stream(x))
    _lib.check(rc, "SnnFc (inference)")
    return out


def snn_fc_grad(grad, inp, weight, params, oldout, need_input_grad=True, grad_weight_out=None, opts=None):
    """grad may be the packed [2B,J] tensor or just its first B rows (only those are read)."""
    g = _as_cuda_f32(grad, "grad"); x = _as_cuda_f32(inp, "in"); w = _as_cuda_f32(weight, "weight")
    y = _as_cuda_f32(oldout, "oldout"); p = _params(params, 6)
    B, I = x.shape
    rows, J = w.shape
    if y.shape[0] != 2 * B or y.shape[1] != J:
        raise ValueError("snn_fc_grad: oldout must be [2B,J]")
    if g.shape[0] not in (B, 2 * B) or g.shape[1] != J:
        raise ValueError("snn_fc_grad: Grad/Oldout batch should be 2 * batch")
    lib = _lib.load() if opts is None else _lib.load_measure()
    with torch.cuda.device(x.device):
        dx = torch.empty_like(x) if need_input_grad else None
        dw = grad_weight_out if grad_weight_out is not None else torch.empty_like(w)
        dp = torch.empty(6, dtype=torch.float32, device=x.device)
        ws, wsb = _workspace(lib.snntc_fc_backward_workspace_bytes(B, I, rows, J), x.device)
        if opts is None:
            rc = lib.snntc_fc_backward(g.data_ptr(), x.data_ptr(), w.data_ptr(), p.ctypes.data, y.data_ptr(),
                                       _ptr(dx), dw.data_ptr(), dp.data_ptr(), B, I, rows, J, _ptr(ws), wsb, _stream(x))
        else:
            rc = lib.snntc_measure_fc_backward(g.data_ptr(), x.data_ptr(), w.data_ptr(), p.ctypes.data, y.data_ptr(),
                                               _ptr(dx), dw.data_ptr(), dp.data_ptr(), B, I, rows, J, _ptr(ws), wsb,
                                               _opts_ptr(opts), _stream(x))
    _lib.check(rc, "SnnFcGrad")
    return dx, dw, dp


def _cv_dims(x, w, p, pad_top, pad_left, Nh, Nw):
    if x.dim() != 4 or w.dim() != 2:
        raise ValueError("snn_cv expects in[B,H,W,C] (NHWC) and weight[rows,Kc]")
    B, H, W, C = x.shape
    rows, Kc = w.shape
    Kh, Kw, Sh, Sw = int(p[6]), int(p[7]), int(p[8]), int(p[9])
    if Nh is None:
        if Kh <= 0 or Kw <= 0 or Sh <= 0 or Sw <= 0:
            raise ValueError("snn_cv: invalid params vector")
        Nh, Nw = (H - Kh) // Sh + 1, (W - Kw) // Sw + 1
    return B, H, W, C, rows, Kc, Kh, Kw, pad_top, pad_left, Nh, Nw


def snn_cv(inp, weight, params, pad_top=0, pad_left=0, Nh=None, Nw=None, opts=None, workspace=None, out=None):
    """With the default pad arguments this is the reference op: `inp` is the tensor SNN_conv.call has
    already padded with MAX (SAME) or cropped (VALID)."""
    x = _as_cuda_f32(inp, "in"); w = _as_cuda_f32(weight, "weight"); p = _params(params, 12)
    B, H, W, C, rows, Kc, Kh, Kw, pt, pl, Nh, Nw = _cv_dims(x, w, p, pad_top, pad_left, Nh, Nw)
    if Nh <= 0 or Nw <= 0:
        raise ValueError("snn_cv: kernel larger than the (padded) input")
    lib = _lib.load() if opts is None else _lib.load_measure()
    with torch.cuda.device(x.device):
        if out is None:
            out = torch.empty((2 * B, Nh, Nw, Kc), dtype=torch.float32, device=x.device)
        ws, wsb = (workspace, workspace.numel() * 4) if workspace is not None else \
            _workspace(lib.snntc_cv_forward_workspace_bytes(B, H, W, C, Kc, Kh, Kw, Nh, Nw), x.device)
        if opts is None:
            rc = lib.snntc_cv_forward(x.data_ptr(), w.data_ptr(), p.ctypes.data, out.data_ptr(), B, H, W, C, rows, Kc,
                                      pt, pl, Nh, Nw, _ptr(ws), wsb, _stream(x))
        else:
            rc = lib.snntc_measure_cv_forward(x.data_ptr(), w.data_ptr(), p.ctypes.data, out.data_ptr(), B, H, W, C,
                                              rows, Kc, pt, pl, Nh, Nw, _ptr(ws), wsb, _opts_ptr(opts), _stream(x))
    _lib.check(rc, "SnnCv")
    return out


def cv_forward_workspace(x, weight, params, Nh, Nw):
    lib = _lib.load()
    p = _params(params, 12)
    B, H, W, C = x.shape
    return _workspace(lib.snntc_cv_forward_workspace_bytes(B, H, W, C, weight.shape[1], int(p[6]), int(p[7]), Nh, Nw),
                      x.device)[0]


def snn_cv_infer(inp, weight, params, pad_top=0, pad_left=0, Nh=None, Nw=None, khist=None):
    """Spike values only, [B,Nh,Nw,Kc]: SnnCv without the 1/(sum w - theta) half (snntc_cv_infer). `khist`: an
    int32 CUDA tensor of Kh*Kw*C+2 zeros that receives the histogram of causal-set sizes."""
    lib = _lib.load()
    x = _as_cuda_f32(inp, "in"); w = _as_cuda_f32(weight, "weight"); p = _params(params, 12)
    B, H, W, C, rows, Kc, Kh, Kw, pt, pl, Nh, Nw = _cv_dims(x, w, p, pad_top, pad_left, Nh, Nw)
    if Nh <= 0 or Nw <= 0:
        raise ValueError("snn_cv_infer: kernel larger than the (padded) input")
    if khist is not None and (khist.dtype != torch.int32 or khist.numel() < Kh * Kw * C + 2 or not khist.is_cuda):
        raise ValueError("khist must be an int32 CUDA tensor of at least fan_in + 2 elements")
    with torch.cuda.device(x.device):
        out = torch.empty((B, Nh, Nw, Kc), dtype=torch.float32, device=x.device)
        ws, wsb = _workspace(lib.snntc_cv_forward_workspace_bytes(B, H, W, C, Kc, Kh, Kw, Nh, Nw), x.device)
        rc = lib.snntc_cv_infer(x.data_ptr(), w.data_ptr(), p.ctypes.data, out.data_ptr(), _ptr(khist), B, H, W, C,
                                rows, Kc, pt, pl, Nh, Nw, _ptr(ws), wsb, _stream(x))
    _lib.check(rc, "SnnCv (inference)")
    return out


def snn_cv_grad(grad, inp, weight, params, oldout, pad_top=0, pad_left=0, need_input_grad=True,
                grad_weight_out=None, opts=None):
    g = _as_cuda_f32(grad, "grad"); x = _as_cuda_f32(inp, "in"); w = _as_cuda_f32(weight, "weight")
    y = _as_cuda_f32(oldout, "oldout"); p = _params(params, 12)
    if y.dim() != 4:
        raise ValueError("snn_cv_grad: oldout must be [2B,Nh,Nw,Kc]")
    B, H, W, C, rows, Kc, Kh, Kw, pt, pl, Nh, Nw = _cv_dims(x, w, p, pad_top, pad_left, y.shape[1], y.shape[2])
    if y.shape[0] != 2 * B or y.shape[3] != Kc:
        raise ValueError("snn_cv_grad: oldout must be [2B,Nh,Nw,Kc]")
    if g.shape[0] not in (B, 2 * B) or tuple(g.shape[1:]) != tuple(y.shape[1:]):
        raise ValueError("snn_cv_grad: Grad/Oldout batch should be 2 * batch")
    lib = _lib.load() if opts is None else _lib.load_measure()
    with torch.cuda.device(x.device):
        dx = torch.empty_like(x) if need_input_grad else None
        dw = grad_weight_out if grad_weight_out is not None else torch.empty_like(w)
        dp = torch.empty(12, dtype=torch.float32, device=x.device)
        ws, wsb = _workspace(lib.snntc_cv_backward_workspace_bytes(B, H, W, C, rows, Kc, Nh, Nw), x.device)
        if opts is None:
            rc = lib.snntc_cv_backward(g.data_ptr(), x.data_ptr(), w.data_ptr(), p.ctypes.data, y.data_ptr(),
                                       _ptr(dx), dw.data_ptr(), dp.data_ptr(), B, H, W, C, rows, Kc, pt, pl, Nh, Nw,
                                       _ptr(ws), wsb, _stream(x))
        else:
            rc = lib.snntc_measure_cv_backward(g.data_ptr(), x.data_ptr(), w.data_ptr(), p.ctypes.data, y.data_ptr(),
                                               _ptr(dx), dw.data_ptr(), dp.data_ptr(), B, H, W, C, rows, Kc, pt, pl,
                                               Nh, Nw, _ptr(ws), wsb, _opts_ptr(opts), _stream(x))
    _lib.check(rc, "SnnCvGrad")
    return dx, dw, dp


# ------------------------------------------------------------------------------------------ autograd
class _SnnFc(torch.autograd.Function):
    """Differentiable SnnFc with the reference's packed [2B,J] output."""

    @staticmethod
    def forward(ctx, X, W, params):
        out = snn_fc(X, W, params)
        ctx.params = _params(params, 6)
        ctx.save_for_backward(X, W, out)
        return out

    @staticmethod
    def backward(ctx, grad):
        X, W, out = ctx.saved_tensors
        dx, dw, _ = snn_fc_grad(grad, X, W, ctx.params, out, need_input_grad=ctx.needs_input_grad[0])
        return dx, dw, None


class _SnnCv(torch.autograd.Function):
    @staticmethod
    def forward(ctx, X, W, params):
        out = snn_cv(X, W, params)
        ctx.params = _params(params, 12)
        ctx.save_for_backward(X, W, out)
        return out

    @staticmethod
    def backward(ctx, grad):
        X, W, out = ctx.saved_tensors
        dx, dw, _ = snn_cv_grad(grad, X, W, ctx.params, out, need_input_grad=ctx.needs_input_grad[0])
        return dx, dw, None


def snnfc(X, W, params):
    return _SnnFc.apply(X, W, params)


def snncv(X, W, params):
    return _SnnCv.apply(X, W, params)


snnfc_grad = snn_fc_grad
snncv_grad = snn_cv_grad


class _SnnFcLayer(torch.autograd.Function):
    """Layer form: returns y[B,J] only. `sink` (optional) is where dW is written instead of being
    handed to autograd -- a slice of the flat gradient bucket that the all-reduce works on."""

    @staticmethod
    def forward(ctx, X, W, params, sink):
        out = snn_fc(X, W, params)
        ctx.params = _params(params, 6)
        ctx.sink = sink
        ctx.save_for_backward(X, W, out)
        B = X.shape[0]
        return out[:B]

    @staticmethod
    def backward(ctx, grad):
        X, W, out = ctx.saved_tensors
        need_dx = ctx.needs_input_grad[0]
        grad = grad.contiguous()
        if TAP is not None:
            TAP.append(("fc", X, W, ctx.params, None, out, grad, need_dx))
        dx, dw, _ = snn_fc_grad(grad, X, W, ctx.params, out, need_input_grad=need_dx,
                                grad_weight_out=ctx.sink)
        return dx, (None if ctx.sink is not None else dw), None, None


class _SnnCvLayer(torch.autograd.Function):
    @staticmethod
    def forward(ctx, X, W, params, geom, sink):
        pt, pl, Nh, Nw = geom
        out = snn_cv(X, W, params, pt, pl, Nh, Nw)
        ctx.params = _params(params, 12)
        ctx.geom = geom
        ctx.sink = sink
        ctx.save_for_backward(X, W, out)
        return out[:X.shape[0]]

    @staticmethod
    def backward(ctx, grad):
        X, W, out = ctx.saved_tensors
        pt, pl, _, _ = ctx.geom
        need_dx = ctx.needs_input_grad[0]
        grad = grad.contiguous()
        if TAP is not None:
            TAP.append(("cv", X, W, ctx.params, ctx.geom, out, grad, need_dx))
        dx, dw, _ = snn_cv_grad(grad, X, W, ctx.params, out, pt, pl, need_input_grad=need_dx,
                                grad_weight_out=ctx.sink)
        return dx, (None if ctx.sink is not None else dw), None, None, None


def _no_grad_needed(X, W):
    return not (torch.is_grad_enabled() and (X.requires_grad or W.requires_grad))


def snn_fc_layer(X, W, params, grad_sink=None):
    if _no_grad_needed(X, W):   # evaluation: nothing will read 1/(sum w - theta)
        return snn_fc_infer(X, W, params)
    return _SnnFcLayer.apply(X, W, params, grad_sink)


def snn_cv_layer(X, W, params, geom, grad_sink=None):
    if _no_grad_needed(X, W):
        pt, pl, Nh, Nw = geom
        return snn_cv_infer(X, W, params, pt, pl, Nh, Nw)
    return _SnnCvLayer.apply(X, W, params, geom, grad_sink)


# ------------------------------------------------------------------------------------------ pooling
class _MinPool(torch.autograd.Function):
    @staticmethod
    def forward(ctx, X, Kh, Kw, Sh, Sw, padding, padvalue):
        lib = _lib.load()
        x = _as_cuda_f32(X, "input")
        B, H, W, C = x.shape
        if str(padding).upper() == "SAME":
            pt, pl, Nh, Nw = conv_geometry(H, W, Kh, Kw, Sh, Sw, "SAME")
        else:
            pt = pl = 0
            Nh, Nw = (H - Kh) // Sh + 1, (W - Kw) // Sw + 1
        with torch.cuda.device(x.device):
            y = torch.empty((B, Nh, Nw, C), dtype=torch.float32, device=x.device)
            arg = torch.empty((B, Nh, Nw, C), dtype=torch.int32, device=x.device)
            rc = lib.snntc_minpool_forward(x.data_ptr(), y.data_ptr(), arg.data_ptr(), B, H, W, C, Kh, Kw, Sh, Sw,
                                           pt, pl, Nh, Nw, float(padvalue), _stream(x))
        _lib.check(rc, "minpool forward")
        ctx.save_for_backward(arg)
        ctx.in_shape = tuple(x.shape)
        ctx.window = (Kh, Kw, Sh, Sw, pt, pl, Nh, Nw)
        return y

    @staticmethod
    def backward(ctx, gy):
        lib = _lib.load()
        (arg,) = ctx.saved_tensors
        gy = gy.contiguous()
        with torch.cuda.device(gy.device):
            dx = torch.empty(ctx.in_shape, dtype=torch.float32, device=gy.device)
            B, H, W, C = ctx.in_shape
            rc = lib.snntc_minpool_backward(gy.data_ptr(), arg.data_ptr(), dx.data_ptr(), B, H, W, C, *ctx.window,
                                            _stream(gy))
        _lib.check(rc, "minpool backward")
        return dx, None, None, None, None, None, None


def snn_minpool(X, Kh, Kw, Sh, Sw, padding="SAME", padvalue=1e5):
    """Window minimum with `padvalue` outside the image (SNN_maxpool2d of the reference)."""
    return _MinPool.apply(X, Kh, Kw, Sh, Sw, padding, padvalue)
