"""ctypes binding of libsnntc_b200.so (the C ABI declared in include/snntc_b200.h).

There is no fallback: if the library is missing or a call fails, an exception is raised.
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libsnntc_b200.so")
MEASURE_LIB_PATH = os.path.join(_HERE, "libsnntc_b200_measure.so")

# every symbol include/snntc_b200.h declares: (restype, argtypes)
_F = ctypes.c_void_p  # device/host float pointers travel as integers
_INT = ctypes.c_int
_SZ = ctypes.c_size_t
SYMBOLS = {
    "snntc_status_string": (ctypes.c_char_p, [_INT]),
    "snntc_last_cuda_error": (ctypes.c_char_p, []),
    "snntc_version": (ctypes.c_char_p, []),
    "snntc_fc_forward_workspace_bytes": (_SZ, [_INT] * 3),
    "snntc_fc_forward": (_INT, [_F, _F, _F, _F] + [_INT] * 4 + [_F, _SZ, _F]),
    "snntc_fc_backward_workspace_bytes": (_SZ, [_INT] * 4),
    "snntc_fc_backward": (_INT, [_F] * 8 + [_INT] * 4 + [_F, _SZ, _F]),
    "snntc_cv_forward_workspace_bytes": (_SZ, [_INT] * 9),
    "snntc_cv_forward": (_INT, [_F] * 4 + [_INT] * 10 + [_F, _SZ, _F]),
    "snntc_cv_backward_workspace_bytes": (_SZ, [_INT] * 8),
    "snntc_cv_backward": (_INT, [_F] * 8 + [_INT] * 10 + [_F, _SZ, _F]),
    "snntc_launch_count": (ctypes.c_ulonglong, []),
    "snntc_set_overlap": (None, [_INT]),
    "snntc_copy_timeouts": (ctypes.c_ulonglong, []),
    "snntc_minpool_forward": (_INT, [_F, _F, _F] + [_INT] * 12 + [ctypes.c_float, _F]),
    "snntc_minpool_backward": (_INT, [_F, _F, _F] + [_INT] * 12 + [_F]),
    "snntc_fc_backward_noalloc": (_INT, [_F] * 8 + [_INT] * 4 + [_F]),
    "snntc_noalloc_scratch_bytes": (_SZ, []),
    "snntc_fc_infer": (_INT, [_F] * 5 + [_INT] * 4 + [_F, _SZ, _F]),
    "snntc_cv_infer": (_INT, [_F] * 5 + [_INT] * 10 + [_F, _SZ, _F]),
    "snntc_encode": (_INT, [_F, _F, _SZ, ctypes.c_float, _INT, _F]),
    "snntc_loss_ce": (_INT, [_F, _F, _F, _F, _INT, _INT, ctypes.c_float, ctypes.c_float, _F]),
    "snntc_weight_cost_workspace_bytes": (_SZ, [_INT]),
    "snntc_weight_cost": (_INT, [_F, _F, _F, _INT, _INT, ctypes.c_float, ctypes.c_float, _F, _SZ, _F]),
    "snntc_adam_step": (_INT, [_F, _F, _F, _F, _SZ] + [ctypes.c_float] * 5 + [_F, _F]),
    "snntc_sgdm_step": (_INT, [_F, _F, _F, _SZ] + [ctypes.c_float] * 3 + [_F]),
}
# exported by the measurement build only (include/snntc_b200.h, #ifdef SNNTC_MEASURE)
MEASURE_SYMBOLS = {
    "snntc_measure_fc_forward": (_INT, [_F, _F, _F, _F] + [_INT] * 4 + [_F, _SZ, _F, _F]),
    "snntc_measure_fc_backward": (_INT, [_F] * 8 + [_INT] * 4 + [_F, _SZ, _F, _F]),
    "snntc_measure_cv_forward": (_INT, [_F] * 4 + [_INT] * 10 + [_F, _SZ, _F, _F]),
    "snntc_measure_cv_backward": (_INT, [_F] * 8 + [_INT] * 10 + [_F, _SZ, _F, _F]),
    "snntc_fp32_probe": (_INT, [_F, _INT, _INT, ctypes.POINTER(ctypes.c_double), _F]),
}

_lib = None
_measure = None


class SnntcError(RuntimeError):
    pass


def _open(path, symbols):
    if not os.path.exists(path):
        raise SnntcError(
            "%s not found -- build it with `python -m snntc_2023_b200.build`; "
            "there is no CPU or framework fallback" % path)
    lib = ctypes.CDLL(path)
    for name, (res, args) in symbols.items():
        try:
            fn = getattr(lib, name)
        except AttributeError:
            raise SnntcError("%s does not export %s" % (os.path.basename(path), name))
        fn.restype = res
        fn.argtypes = args
    return lib


def load():
    """Loads the library once; raises if it has not been built (python -m snntc_2023_b200.build)."""
    global _lib
    if _lib is None:
        _lib = _open(LIB_PATH, SYMBOLS)
    return _lib


def load_measure():
    """The measurement build: every symbol of the product library plus the entry points that take the kernel
    choice of a call explicitly. Used by bench.py and by the tests that compare kernel variants."""
    global _measure
    if _measure is None:
        both = dict(SYMBOLS)
        both.update(MEASURE_SYMBOLS)
        _measure = _open(MEASURE_LIB_PATH, both)
    return _measure


def options(forward_parts=3, walk_layout=0, walk_outputs=0, list_builder=0, backward_parts=3, dw_kernel=0, overlap=-1,
            dx_kernel=0):
    """The opts8 vector of the measurement entry points (include/snntc_b200.h)."""
    return (ctypes.c_int * 8)(forward_parts, walk_layout, walk_outputs, list_builder, backward_parts, dw_kernel, overlap,
                              dx_kernel)


def check(status, what):
    """Turns a non-zero status into the exception the reference would have raised as InvalidArgument."""
    if status == 0:
        return
    lib = load()
    msg = lib.snntc_status_string(status).decode()
    if status == -7:
        err = lib.snntc_last_cuda_error().decode()
        if not err and _measure is not None:
            err = _measure.snntc_last_cuda_error().decode()
        raise SnntcError("%s: %s (%s)" % (what, msg, err))
    if status in (-1, -2, -3, -4, -8):
        raise ValueError("%s: %s" % (what, msg))
    raise SnntcError("%s: %s" % (what, msg))
