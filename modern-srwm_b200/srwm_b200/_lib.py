"""ctypes binding of libsrwm_b200.so (declarations mirror include/srwm_b200.h).

The library is prebuilt in-tree (``modern-srwm_b200/csrc/build.py``); there is no JIT
compilation at import time and no fallback: if the shared object is missing, loading
raises with the command that builds it.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
# SRWM_B200_DEBUG=1 selects the debug build of the library (row checks that report through a status
# word instead of faulting; csrc/build.py --debug)
DEBUG_BUILD = os.environ.get("SRWM_B200_DEBUG", "0") not in ("", "0")
LIB_PATH = os.path.join(_HERE, "libsrwm_b200_debug.so" if DEBUG_BUILD else "libsrwm_b200.so")

F32, BF16 = 0, 1
FLAG_NO_SAVE, FLAG_STATE_GRAD_IN, FLAG_RESTORE_STATE, FLAG_INPUT_SOFTMAX, FLAG_ZERO_INIT = 1, 2, 4, 8, 16
OP_SRWM_FWD, OP_SRWM_BWD, OP_DELTA_FWD, OP_DELTA_BWD, OP_SRWM_BWD_DET = 0, 1, 2, 3, 4
ABI_VERSION = 2
STATIC_SCRATCH_BYTES = 4 * 1024 * 1024   # SRWM_B200_STATIC_SCRATCH_BYTES

ERR_NULL, ERR_SHAPE, ERR_HEAD_DIM, ERR_DTYPE, ERR_ALIGN, ERR_VARIANT, ERR_CUDA, ERR_TOO_LARGE, ERR_UNSUPPORTED = (
    -1, -2, -3, -4, -5, -6, -7, -8, -9)


class Seq(C.Structure):
    _fields_ = [("data", C.c_void_p), ("stride_n", C.c_int64), ("stride_h", C.c_int64),
                ("stride_l", C.c_int64)]


class State(C.Structure):
    _fields_ = [("data", C.c_void_p), ("stride_n", C.c_int64), ("stride_h", C.c_int64)]


class SrwmFwdArgs(C.Structure):
    _fields_ = [("N", C.c_int32), ("H", C.c_int32), ("L", C.c_int32), ("E", C.c_int32),
                ("io_dtype", C.c_int32), ("flags", C.c_uint32), ("variant", C.c_int32),
                ("reserved", C.c_int32),
                ("x", Seq), ("W_y", State), ("W_q", State), ("W_k", State), ("w_b", State),
                ("out", Seq), ("q", Seq), ("k", Seq), ("beta", Seq),
                ("y_diff", Seq), ("q_diff", Seq), ("k_diff", Seq), ("beta_diff", Seq)]


class SrwmBwdArgs(C.Structure):
    _fields_ = [("N", C.c_int32), ("H", C.c_int32), ("L", C.c_int32), ("E", C.c_int32),
                ("io_dtype", C.c_int32), ("flags", C.c_uint32), ("variant", C.c_int32),
                ("reserved", C.c_int32),
                ("x", Seq), ("q", Seq), ("k", Seq), ("beta", Seq),
                ("y_diff", Seq), ("q_diff", Seq), ("k_diff", Seq), ("beta_diff", Seq),
                ("grad_out", Seq),
                ("W_y", State), ("W_q", State), ("W_k", State), ("w_b", State),
                ("grad_x", Seq),
                ("grad_W_y", State), ("grad_W_q", State), ("grad_W_k", State), ("grad_w_b", State)]


class SrwmExt(C.Structure):
    _fields_ = [("base_W_y", State), ("base_W_q", State), ("base_W_k", State), ("base_w_b", State),
                ("shift_W_y", State), ("shift_W_q", State), ("shift_W_k", State), ("shift_w_b", State),
                ("done", C.c_void_p), ("done_stride_n", C.c_int64), ("done_stride_l", C.c_int64)]


class SrwmReduce(C.Structure):
    _fields_ = [("grad_base_W_y", State), ("grad_base_W_q", State), ("grad_base_W_k", State),
                ("grad_base_w_b", State), ("accumulate", C.c_int32), ("reserved", C.c_int32),
                ("scratch", C.c_void_p), ("scratch_bytes", C.c_int64)]


class SrwmBwdDetArgs(C.Structure):
    _fields_ = [("N", C.c_int32), ("H", C.c_int32), ("L", C.c_int32), ("E", C.c_int32),
                ("io_dtype", C.c_int32), ("flags", C.c_uint32), ("variant", C.c_int32),
                ("reserved", C.c_int32),
                ("x", Seq), ("k", Seq), ("beta", Seq), ("y_diff", Seq), ("grad_out", Seq),
                ("base_W_y", State), ("shift_W_y", State),
                ("done", C.c_void_p), ("done_stride_n", C.c_int64), ("done_stride_l", C.c_int64),
                ("grad_x", Seq), ("grad_W_y", State)]


class DeltaFwdArgs(C.Structure):
    _fields_ = [("N", C.c_int32), ("H", C.c_int32), ("L", C.c_int32), ("E", C.c_int32),
                ("M", C.c_int32), ("io_dtype", C.c_int32), ("flags", C.c_uint32),
                ("variant", C.c_int32),
                ("Q", Seq), ("K", Seq), ("V", Seq), ("beta", Seq), ("W", State),
                ("out", Seq), ("v_old", Seq), ("v_insert", Seq)]


class DeltaBwdArgs(C.Structure):
    _fields_ = [("N", C.c_int32), ("H", C.c_int32), ("L", C.c_int32), ("E", C.c_int32),
                ("M", C.c_int32), ("io_dtype", C.c_int32), ("flags", C.c_uint32),
                ("variant", C.c_int32),
                ("Q", Seq), ("K", Seq), ("V", Seq), ("beta", Seq),
                ("v_old", Seq), ("v_insert", Seq), ("grad_out", Seq), ("W", State),
                ("grad_Q", Seq), ("grad_K", Seq), ("grad_V", Seq), ("grad_beta", Seq),
                ("grad_W0", State)]


class DeltaPackedFwdArgs(C.Structure):
    _fields_ = [("N", C.c_int32), ("H", C.c_int32), ("L", C.c_int32), ("E", C.c_int32),
                ("io_dtype", C.c_int32), ("flags", C.c_uint32), ("variant", C.c_int32),
                ("norm_eps", C.c_float),
                ("qkvb", Seq), ("W", State), ("out", Seq), ("v_old", Seq), ("v_insert", Seq)]


class DeltaPackedBwdArgs(C.Structure):
    _fields_ = [("N", C.c_int32), ("H", C.c_int32), ("L", C.c_int32), ("E", C.c_int32),
                ("io_dtype", C.c_int32), ("flags", C.c_uint32), ("variant", C.c_int32),
                ("norm_eps", C.c_float),
                ("qkvb", Seq), ("v_old", Seq), ("v_insert", Seq), ("grad_out", Seq), ("W", State),
                ("grad_qkvb", Seq), ("grad_W0", State)]


# name -> (restype, argtypes); also the list of symbols the header declares.
SYMBOLS = {
    "srwm_b200_srwm_forward": (C.c_int, [C.POINTER(SrwmFwdArgs), C.c_void_p]),
    "srwm_b200_srwm_backward": (C.c_int, [C.POINTER(SrwmBwdArgs), C.c_void_p]),
    "srwm_b200_srwm_layer_forward": (C.c_int, [C.POINTER(SrwmFwdArgs), C.POINTER(SrwmExt), C.c_void_p]),
    "srwm_b200_srwm_layer_backward": (C.c_int, [C.POINTER(SrwmBwdArgs), C.POINTER(SrwmExt), C.c_void_p]),
    "srwm_b200_srwm_layer_backward_reduced": (C.c_int, [C.POINTER(SrwmBwdArgs), C.POINTER(SrwmExt),
                                                        C.POINTER(SrwmReduce), C.c_void_p]),
    "srwm_b200_srwm_layer_backward_reduced_static": (C.c_int, [C.POINTER(SrwmBwdArgs), C.POINTER(SrwmExt),
                                                               C.POINTER(SrwmReduce), C.c_void_p]),
    "srwm_b200_srwm_reduce_scratch_bytes": (C.c_size_t, [C.c_int32, C.c_int32, C.c_int32]),
    "srwm_b200_srwm_backward_detached": (C.c_int, [C.POINTER(SrwmBwdDetArgs), C.c_void_p]),
    "srwm_b200_delta_forward": (C.c_int, [C.POINTER(DeltaFwdArgs), C.c_void_p]),
    "srwm_b200_delta_backward": (C.c_int, [C.POINTER(DeltaBwdArgs), C.c_void_p]),
    "srwm_b200_delta_packed_forward": (C.c_int, [C.POINTER(DeltaPackedFwdArgs), C.c_void_p]),
    "srwm_b200_delta_packed_backward": (C.c_int, [C.POINTER(DeltaPackedBwdArgs), C.c_void_p]),
    "srwm_b200_reduce_batch": (C.c_int, [C.c_void_p, C.c_int64, C.c_int32, C.c_int64, C.c_void_p,
                                         C.c_int32, C.c_void_p]),
    "srwm_b200_debug_status": (C.c_int, [C.POINTER(C.c_uint64)]),
    "srwm_b200_debug_selftest": (C.c_int, [C.c_void_p]),
    "srwm_b200_abi_version": (C.c_int, []),
    "srwm_b200_head_dim_supported": (C.c_int, [C.c_int32]),
    "srwm_b200_num_variants": (C.c_int, [C.c_int32, C.c_int32]),
    "srwm_b200_strerror": (C.c_char_p, [C.c_int]),
    "srwm_b200_last_cuda_error": (C.c_int, []),
    "srwm_b200_describe": (C.c_int, [C.c_int32, C.c_int32, C.c_int32, C.c_int32,
                                     C.POINTER(C.c_int32 * 4)]),
    "srwm_b200_describe_for_grid": (C.c_int, [C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int64, C.c_int32,
                                              C.POINTER(C.c_int32 * 5)]),
}

_lib = None


def load():
    """Load the shared library once; raise loudly if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with "
            "`python modern-srwm_b200/csrc/build.py" + (" --debug" if DEBUG_BUILD else "") +
            "` (there is no fallback implementation)")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SYMBOLS.items():
        fn = getattr(lib, name, None)
        if fn is None:
            continue        # optional symbols are checked by their users
        fn.restype = res
        fn.argtypes = args
    if lib.srwm_b200_abi_version() != ABI_VERSION:
        raise RuntimeError("libsrwm_b200.so ABI version mismatch")
    _lib = lib
    return lib


class SrwmError(RuntimeError):
    def __init__(self, code, what):
        self.code = code
        lib = load()
        msg = lib.srwm_b200_strerror(code).decode()
        if code == ERR_CUDA:
            msg += f" [cudaError {lib.srwm_b200_last_cuda_error()}]"
        super().__init__(f"{what}: {msg} (code {code})")


def check(code, what):
    if code != 0:
        raise SrwmError(code, what)


def describe(op, E, io_dtype=F32, variant=0, grid=None, num_sms=0):
    """Kernel configuration of a call; with ``grid`` (= N*H sequences) what variant 0 resolves to there."""
    if grid is None:
        out = (C.c_int32 * 4)()
        check(load().srwm_b200_describe(op, E, io_dtype, variant, C.byref(out)), "describe")
        return dict(P=out[0], R=out[1], T=out[2], smem=out[3])
    out = (C.c_int32 * 5)()
    check(load().srwm_b200_describe_for_grid(op, E, io_dtype, variant, grid, num_sms, C.byref(out)), "describe")
    return dict(P=out[0], R=out[1], T=out[2], smem=out[3], id=out[4])


def debug_status():
    """(compiled_in, word): the debug build's status word (0 = no violation), cleared by the read."""
    w = C.c_uint64(0)
    rc = load().srwm_b200_debug_status(C.byref(w))
    if rc == 1:
        return False, 0
    check(rc, "debug_status")
    return True, int(w.value)
