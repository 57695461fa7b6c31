"""ctypes front-end of the CPU oracle -- TEST INFRASTRUCTURE ONLY.

`liboracle.so` is the plain-C restatement of the reference GPU kernels' arithmetic
(snntc/snnfc_kernels.cu.cc:19-71, snnfcgrad_kernels.cu.cc:15-133, snncvgrad_kernels.cu.cc:15-161);
`_ref/libsnntc_ref_cpu.so` is the reference's own CPU operator code compiled unmodified (only
present where the reference checkout was available at build time, or where the built file travelled).
Only tests, the smoke check and the bench's CPU-baseline leg may import this module.
"""
import ctypes
import math
import os

import numpy as np

from . import build as _build

_F = ctypes.POINTER(ctypes.c_float)
_D = ctypes.POINTER(ctypes.c_double)
_I = ctypes.POINTER(ctypes.c_int)
_U8 = ctypes.POINTER(ctypes.c_ubyte)

_lib = None
_ref = None


def _p(a, t):
    return None if a is None else a.ctypes.data_as(t)


def lib():
    global _lib
    if _lib is None:
        path = _build.ORACLE_SO
        if not os.path.exists(path):
            _build.build_oracle()
        _lib = ctypes.CDLL(path)
    return _lib


def ref_lib():
    """The compiled reference CPU operators, or None when they are not available."""
    global _ref
    if _ref is None:
        path = _build.REF_SO
        if not os.path.exists(path):
            return None
        _ref = ctypes.CDLL(path)
    return _ref


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


# ----------------------------------------------------------------------------- geometry helpers
def same_pad(size, k, s):
    """(before, after) padding of SNN_conv's SAME mode (SNN_TC_Modules.py:147-161)."""
    total = (math.ceil(size / s) - 1) * s + k - size
    total = max(total, 0) if total >= 0 else total
    before = int(total / 2)
    return before, total - before


def conv_geometry(H, W, Kh, Kw, Sh, Sw, padding):
    """Returns (pad_top, pad_left, Nh, Nw, Hp, Wp): output grid and the padded/cropped input size the
    reference op would receive (SNN_TC_Modules.py:144-170, snncv_kernels.cc:215)."""
    if padding.upper() == "SAME":
        pt, pb = same_pad(H, Kh, Sh)
        pl, pr = same_pad(W, Kw, Sw)
        Hp, Wp = H + pt + pb, W + pl + pr
    else:
        pt = pl = 0
        Nh, Nw = int((H - Kh) / Sh + 1.0), int((W - Kw) / Sw + 1.0)
        Hp, Wp = (Nh - 1) * Sh + Kh, (Nw - 1) * Sw + Kw
    Nh, Nw = (Hp - Kh) // Sh + 1, (Wp - Kw) // Sw + 1
    return pt, pl, Nh, Nw, Hp, Wp


def pad_like_reference(x, Kh, Kw, Sh, Sw, padding, maxv=1e5):
    """The tensor SNN_conv.call hands to the op: MAX-padded (SAME) or cropped (VALID)."""
    B, H, W, C = x.shape
    pt, pl, Nh, Nw, Hp, Wp = conv_geometry(H, W, Kh, Kw, Sh, Sw, padding)
    if padding.upper() == "SAME":
        out = np.full((B, Hp, Wp, C), np.float32(maxv), np.float32)
        out[:, pt:pt + H, pl:pl + W, :] = x
        return out
    return np.ascontiguousarray(x[:, :Hp, :Wp, :])


def fc_params(maxv=1e5, eps=1e-10, theta=1.0, tpb=0, blocks=0, biasvolt=1.0):
    return np.array([maxv, eps, theta, tpb, blocks, biasvolt], np.float32)


def cv_params(Kh, Kw, Sh, Sw, padding="SAME", biasvolt=1.0, maxv=1e5, eps=1e-10, theta=1.0):
    return np.array([maxv, 0, 0, eps, theta, 0, Kh, Kw, Sh, Sw, float(padding.upper() == "SAME"), biasvolt],
                    np.float32)


# ----------------------------------------------------------------------------- restated operators
def fc_forward(x, w, params6, acc="f32", tol=1e-5):
    """Dense forward. Returns dict(y, inv, k[, illc]); y/inv are [B,J] in float32 (f32) or float64."""
    x, w = _f32(x), _f32(w)
    B, I = x.shape
    J = w.shape[1]
    maxv, theta, bv = float(params6[0]), float(params6[2]), float(params6[5])
    assert w.shape[0] == I + (1 if bv > 1e-8 else 0)
    k = np.zeros((B, J), np.int32)
    if acc == "f32":
        y = np.zeros((B, J), np.float32); inv = np.zeros((B, J), np.float32)
        rc = lib().oracle_rows_forward_f32(_p(x, _F), _p(w, _F), B, I, J, ctypes.c_float(maxv), ctypes.c_float(theta),
                                           ctypes.c_float(bv), _p(y, _F), _p(inv, _F), _p(k, _I), None,
                                           ctypes.c_double(tol), None)
        assert rc == 0
        return dict(y=y, inv=inv, k=k)
    y = np.zeros((B, J), np.float64); inv = np.zeros((B, J), np.float64); ill = np.zeros((B, J), np.uint8)
    cond = np.zeros((B, J), np.float64)
    rc = lib().oracle_rows_forward_f64(_p(x, _F), _p(w, _F), B, I, J, ctypes.c_float(maxv), ctypes.c_float(theta),
                                       ctypes.c_float(bv), _p(y, _D), _p(inv, _D), _p(k, _I), _p(ill, _U8),
                                       ctypes.c_double(tol), _p(cond, _D))
    assert rc == 0
    return dict(y=y, inv=inv, k=k, illc=ill.astype(bool), cond=cond)


def fc_backward(g, x, w, params6, y, inv, acc="f64", want_dx=True):
    """Dense backward from the forward's (y, inv), given as float32 arrays [B,J]."""
    g, x, w, y, inv = _f32(g), _f32(x), _f32(w), _f32(y), _f32(inv)
    B, I = x.shape
    J = w.shape[1]
    maxv, bv = float(params6[0]), float(params6[5])
    dt, pt, fn = (np.float32, _F, lib().oracle_rows_backward_f32) if acc == "f32" else \
                 (np.float64, _D, lib().oracle_rows_backward_f64)
    dx = np.zeros((B, I), dt) if want_dx else None
    dw = np.zeros(w.shape, dt)
    dxa = np.zeros((B, I), np.float64) if want_dx else None
    dwa = np.zeros(w.shape, np.float64)
    rc = fn(_p(g, _F), _p(x, _F), _p(w, _F), _p(y, _F), _p(inv, _F), B, I, J, ctypes.c_float(maxv),
            ctypes.c_float(bv), _p(dx, pt), _p(dw, pt), _p(dxa, _D), _p(dwa, _D))
    assert rc == 0
    return dict(dx=dx, dw=dw, dx_abs=dxa, dw_abs=dwa)


def cv_forward(x, w, params12, acc="f32", tol=1e-5):
    """Conv forward on the UNPADDED NHWC input; geometry from params12 (SAME/VALID as SNN_conv)."""
    x, w = _f32(x), _f32(w)
    B, H, W, C = x.shape
    Kc = w.shape[1]
    maxv, theta, bv = float(params12[0]), float(params12[4]), float(params12[11])
    Kh, Kw, Sh, Sw = (int(params12[i]) for i in (6, 7, 8, 9))
    padding = "SAME" if params12[10] > 0.5 else "VALID"
    pt, pl, Nh, Nw, _, _ = conv_geometry(H, W, Kh, Kw, Sh, Sw, padding)
    assert w.shape[0] == Kh * Kw * C + (1 if bv > 1e-8 else 0)
    shp = (B, Nh, Nw, Kc)
    k = np.zeros(shp, np.int32)
    args = (_p(x, _F), _p(w, _F), B, H, W, C, Kc, Kh, Kw, Sh, Sw, pt, pl, Nh, Nw, ctypes.c_float(maxv),
            ctypes.c_float(theta), ctypes.c_float(bv))
    if acc == "f32":
        y = np.zeros(shp, np.float32); inv = np.zeros(shp, np.float32)
        rc = lib().oracle_cv_forward_f32(*args, _p(y, _F), _p(inv, _F), _p(k, _I), None, ctypes.c_double(tol), None)
        assert rc == 0
        return dict(y=y, inv=inv, k=k)
    y = np.zeros(shp, np.float64); inv = np.zeros(shp, np.float64); ill = np.zeros(shp, np.uint8)
    cond = np.zeros(shp, np.float64)
    rc = lib().oracle_cv_forward_f64(*args, _p(y, _D), _p(inv, _D), _p(k, _I), _p(ill, _U8), ctypes.c_double(tol),
                                     _p(cond, _D))
    assert rc == 0
    return dict(y=y, inv=inv, k=k, illc=ill.astype(bool), cond=cond)


def cv_backward(g, x, w, params12, y, inv, acc="f64", want_dx=True):
    g, x, w, y, inv = _f32(g), _f32(x), _f32(w), _f32(y), _f32(inv)
    B, H, W, C = x.shape
    Kc = w.shape[1]
    maxv, bv = float(params12[0]), float(params12[11])
    Kh, Kw, Sh, Sw = (int(params12[i]) for i in (6, 7, 8, 9))
    padding = "SAME" if params12[10] > 0.5 else "VALID"
    pt, pl, Nh, Nw, _, _ = conv_geometry(H, W, Kh, Kw, Sh, Sw, padding)
    dt, ptr, fn = (np.float32, _F, lib().oracle_cv_backward_f32) if acc == "f32" else \
                  (np.float64, _D, lib().oracle_cv_backward_f64)
    dx = np.zeros(x.shape, dt) if want_dx else None
    dw = np.zeros(w.shape, dt)
    dxa = np.zeros(x.shape, np.float64) if want_dx else None
    dwa = np.zeros(w.shape, np.float64)
    rc = fn(_p(g, _F), _p(x, _F), _p(w, _F), _p(y, _F), _p(inv, _F), B, H, W, C, Kc, Kh, Kw, Sh, Sw, pt, pl,
            Nh, Nw, ctypes.c_float(maxv), ctypes.c_float(bv), _p(dx, ptr), _p(dw, ptr), _p(dxa, _D), _p(dwa, _D))
    assert rc == 0
    return dict(dx=dx, dw=dw, dx_abs=dxa, dw_abs=dwa)


def minpool(x, Kh, Kw, Sh, Sw, padding="SAME", padvalue=1e5):
    x = _f32(x)
    B, H, W, C = x.shape
    if padding.upper() == "SAME":
        pt, pl, Nh, Nw, _, _ = conv_geometry(H, W, Kh, Kw, Sh, Sw, "SAME")
    else:
        pt = pl = 0
        Nh, Nw = (H - Kh) // Sh + 1, (W - Kw) // Sw + 1
    y = np.zeros((B, Nh, Nw, C), np.float32); arg = np.zeros((B, Nh, Nw, C), np.int32)
    lib().oracle_minpool(_p(x, _F), B, H, W, C, Kh, Kw, Sh, Sw, pt, pl, Nh, Nw, ctypes.c_float(padvalue),
                         _p(y, _F), _p(arg, _I))
    return y, arg


# ----------------------------------------------------------------------------- compiled reference CPU ops
def ref_fc_forward(x, w, params6):
    """Reference CPU SnnFc. Returns out[2B,J]; rows [B,2B) hold (sum w - theta), NOT its reciprocal."""
    L = ref_lib(); x, w, p = _f32(x), _f32(w), _f32(params6)
    B, I = x.shape; J = w.shape[1]
    out = np.zeros((2 * B, J), np.float32)
    rc = L.ref_fc_forward(_p(x, _F), B, I, _p(w, _F), w.shape[0], J, _p(p, _F), _p(out, _F))
    if rc: raise ValueError("reference SnnFc rejected the inputs (rc=%d)" % rc)
    return out


def ref_fc_backward(grad2, x, w, params6, oldout2):
    L = ref_lib(); grad2, x, w, p, oldout2 = _f32(grad2), _f32(x), _f32(w), _f32(params6), _f32(oldout2)
    B, I = x.shape; J = w.shape[1]
    dx = np.zeros_like(x); dw = np.zeros_like(w); dp = np.zeros_like(p)
    rc = L.ref_fc_backward(_p(grad2, _F), _p(x, _F), B, I, _p(w, _F), w.shape[0], J, _p(p, _F), _p(oldout2, _F),
                           _p(dx, _F), _p(dw, _F), _p(dp, _F))
    if rc: raise ValueError("reference SnnFcGrad rejected the inputs (rc=%d)" % rc)
    return dx, dw, dp


def ref_cv_forward(xp, w, params12):
    """Reference CPU SnnCv on the ALREADY padded/cropped input. Returns y[B,Nh,Nw,Kc] only (the CPU op
    leaves the second half of its output unwritten)."""
    L = ref_lib(); xp, w, p = _f32(xp), _f32(w), _f32(params12)
    B, H, W, C = xp.shape; Kc = w.shape[1]
    Kh, Kw, Sh, Sw = (int(p[i]) for i in (6, 7, 8, 9))
    Nh, Nw = (H - Kh) // Sh + 1, (W - Kw) // Sw + 1
    out = np.zeros((2 * B, Nh, Nw, Kc), np.float32); nn = (ctypes.c_int * 2)()
    rc = L.ref_cv_forward(_p(xp, _F), B, H, W, C, _p(w, _F), w.shape[0], Kc, _p(p, _F), _p(out, _F), out.size, nn)
    if rc: raise ValueError("reference SnnCv rejected the inputs (rc=%d)" % rc)
    assert (nn[0], nn[1]) == (Nh, Nw)
    return out[:B]


def ref_cv_backward(grad2, xp, w, params12, oldout2):
    L = ref_lib(); grad2, xp, w, p, oldout2 = _f32(grad2), _f32(xp), _f32(w), _f32(params12), _f32(oldout2)
    B, H, W, C = xp.shape; Kc = w.shape[1]
    Nh, Nw = oldout2.shape[1], oldout2.shape[2]
    dx = np.zeros_like(xp); dw = np.zeros_like(w); dp = np.zeros_like(p)
    rc = L.ref_cv_backward(_p(grad2, _F), _p(xp, _F), B, H, W, C, _p(w, _F), w.shape[0], Kc, _p(p, _F),
                           _p(oldout2, _F), Nh, Nw, _p(dx, _F), _p(dw, _F), _p(dp, _F))
    if rc: raise ValueError("reference SnnCvGrad rejected the inputs (rc=%d)" % rc)
    return dx, dw, dp


# ----------------------------------------------------------------------------- compiled reference GPU ops
_ref_gpu = None


def ref_gpu_lib():
    """The reference's own GPU operators compiled for sm_100a, or None when not available."""
    global _ref_gpu
    if _ref_gpu is None:
        path = _build.REF_GPU_SO
        if not os.path.exists(path):
            return None
        _ref_gpu = ctypes.CDLL(path)
    return _ref_gpu


class RefGpu:
    """Runs the reference GPU functors on torch CUDA tensors. `pool_bytes` of device scratch stand in
    for TensorFlow's allocator (the functors materialise im2col patches, sorted copies and indices)."""

    def __init__(self, pool_bytes=1 << 30):
        import torch
        self.torch = torch
        self.lib = ref_gpu_lib()
        assert self.lib is not None
        self.pool = torch.empty(pool_bytes, dtype=torch.uint8, device="cuda")

    def _args(self):
        torch = self.torch
        return (ctypes.c_void_p(self.pool.data_ptr()), ctypes.c_size_t(self.pool.numel()),
                ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))

    @staticmethod
    def _p(t):
        return ctypes.c_void_p(t.data_ptr())

    def fc_forward(self, x, w, params6):
        torch = self.torch
        p = _f32(params6)
        B, I = x.shape
        out = torch.empty((2 * B, w.shape[1]), dtype=torch.float32, device=x.device)
        rc = self.lib.refgpu_fc_forward(self._p(x), self._p(w), _p(p, _F), self._p(out), B, I, w.shape[0], w.shape[1],
                                        *self._args())
        assert rc == 0, "reference GPU SnnFc failed: CUDA error %d" % -rc
        return out

    def fc_backward(self, grad2, x, w, params6, oldout2):
        torch = self.torch
        p = _f32(params6)
        B, I = x.shape
        dx = torch.empty_like(x); dw = torch.empty_like(w); dp = torch.zeros(6, device=x.device)
        rc = self.lib.refgpu_fc_backward(self._p(grad2), self._p(x), self._p(w), _p(p, _F), self._p(oldout2),
                                         self._p(dx), self._p(dw), self._p(dp), B, I, w.shape[0], w.shape[1],
                                         *self._args())
        assert rc == 0, "reference GPU SnnFcGrad failed: CUDA error %d" % -rc
        return dx, dw

    def cv_forward(self, xp, w, params12):
        """xp: the ALREADY padded/cropped NHWC tensor."""
        torch = self.torch
        p = _f32(params12)
        B, H, W, C = xp.shape
        Kh, Kw, Sh, Sw = (int(p[i]) for i in (6, 7, 8, 9))
        Nh, Nw = (H - Kh) // Sh + 1, (W - Kw) // Sw + 1
        out = torch.empty((2 * B, Nh, Nw, w.shape[1]), dtype=torch.float32, device=xp.device)
        rc = self.lib.refgpu_cv_forward(self._p(xp), self._p(w), _p(p, _F), self._p(out), B, H, W, C, w.shape[0],
                                        w.shape[1], Nh, Nw, *self._args())
        assert rc == 0, "reference GPU SnnCv failed: CUDA error %d" % -rc
        return out

    def cv_backward(self, grad2, xp, w, params12, oldout2):
        torch = self.torch
        p = _f32(params12)
        B, H, W, C = xp.shape
        Nh, Nw = oldout2.shape[1], oldout2.shape[2]
        dx = torch.empty_like(xp); dw = torch.empty_like(w); dp = torch.zeros(12, device=xp.device)
        rc = self.lib.refgpu_cv_backward(self._p(grad2), self._p(xp), self._p(w), _p(p, _F), self._p(oldout2),
                                         self._p(dx), self._p(dw), self._p(dp), B, H, W, C, w.shape[0], w.shape[1],
                                         Nh, Nw, *self._args())
        assert rc == 0, "reference GPU SnnCvGrad failed: CUDA error %d" % -rc
        return dx, dw
