"""ctypes binding of ``libskv.so`` (the C ABI declared in ``include/skv.h``).

There is no fallback: if the library is missing or a call returns an error code, an exception is
raised.  Tensors are passed as raw device addresses (``tensor.data_ptr()``)."""

from __future__ import annotations

import ctypes as C
import os

import torch

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libskv.so")

SKV_BF16, SKV_F32 = 0, 1
FLAG_DRIFT, FLAG_RESET = 1, 2
ST_NO_SLOT, ST_SPLIT_TOO_BIG, ST_BAD_INDEX, ST_WAIT_TIMEOUT = 1, 2, 4, 8

EXPORTS = ("skv_version", "skv_error_string", "skv_last_cuda_error", "skv_attend_splits",
           "skv_attend_workspace_bytes", "skv_attend", "skv_attend_static", "skv_attend_weighted", "skv_attend_labels", "skv_step", "skv_step_clusters", "skv_step_workspace_bytes", "skv_debug_step_probe", "skv_merge", "skv_select_workspace_bytes", "skv_select", "skv_debug_select_probe", "skv_debug_attend_probe", "skv_set_overlap", "skv_insert",
           "skv_insert_max_members", "skv_fit_tensor_cores", "skv_fit_workspace_bytes", "skv_fit", "skv_rebin",
           "skv_add_rmsnorm", "skv_qk_rope_cache", "skv_silu_mul", "skv_gemv", "skv_gemv_attended", "skv_gemv_supported", "skv_gemv_tp", "skv_comm_bytes", "skv_comm_alloc",
           "skv_comm_export", "skv_comm_open", "skv_comm_close", "skv_comm_free", "skv_comm_view", "skv_comm_tick", "skv_comm_push", "skv_comm_reduce", "skv_comm_status")


class SkvError(RuntimeError):
    pass


class SkvComm(C.Structure):
    """``skv_comm`` of include/skv.h: one rank's view of the exchange buffers of a tensor-parallel group."""
    _fields_ = [("world", C.c_int32), ("rank", C.c_int32), ("cap_elems", C.c_int32), ("wait_kpolls", C.c_int32),
                ("data", C.c_void_p * 8), ("tick", C.c_void_p), ("status", C.c_void_p)]


class SkvRope(C.Structure):
    """``skv_rope`` of include/skv.h: QK-norm + rotary + cache write folded into the selection launch."""
    _fields_ = [("qkv", C.c_void_p), ("q_norm_w", C.c_void_p), ("k_norm_w", C.c_void_p), ("cos_table", C.c_void_p),
                ("sin_table", C.c_void_p), ("pos", C.c_void_p), ("q_out", C.c_void_p), ("k_cache", C.c_void_p),
                ("v_cache", C.c_void_p), ("H", C.c_int32), ("H_kv", C.c_int32), ("cache_batch_stride", C.c_int64),
                ("cache_head_stride", C.c_int64), ("cache_row_stride", C.c_int64), ("eps", C.c_float),
                ("pos_per_seq", C.c_int32)]


class SkvState(C.Structure):
    """Mirror of ``struct skv_state``."""
    _fields_ = [("heads", C.c_int32), ("C", C.c_int32), ("d", C.c_int32), ("capacity", C.c_int32),
                ("summary_bits", C.c_int32), ("reserved", C.c_int32),
                ("sum_dir", C.c_void_p), ("cent", C.c_void_p), ("dir8", C.c_void_p), ("cent8", C.c_void_p),
                ("mmax", C.c_void_p), ("mmin", C.c_void_p), ("count", C.c_void_p), ("n_c", C.c_void_p),
                ("cap", C.c_void_p), ("vthr", C.c_void_p), ("rbar", C.c_void_p), ("ksum", C.c_void_p), ("mu_ref", C.c_void_p),
                ("flags", C.c_void_p), ("status", C.c_void_p), ("nsplit", C.c_void_p), ("end", C.c_void_p),
                ("need", C.c_void_p), ("labels", C.c_void_p)]


_lib = None


def _declare(lib) -> None:
    vp, i32, i64, f32, f64 = C.c_void_p, C.c_int, C.c_int64, C.c_float, C.c_double
    lib.skv_version.restype = i32
    lib.skv_error_string.restype = C.c_char_p
    lib.skv_error_string.argtypes = [i32]
    lib.skv_last_cuda_error.restype = C.c_char_p
    lib.skv_attend_splits.restype = i32
    lib.skv_attend_splits.argtypes = [i32]
    lib.skv_attend_workspace_bytes.restype = i64
    lib.skv_attend_workspace_bytes.argtypes = [i32, i32, i32, i32]
    lib.skv_attend.restype = i32
    lib.skv_attend.argtypes = [vp, vp, vp, vp, vp, vp, i32, vp, vp, vp, i32, i32, i32, i32, i64, i64, i64, i64, i64, i32,
                               i32, f32, vp]
    lib.skv_attend_static.restype = i32
    lib.skv_attend_static.argtypes = [vp, vp, vp, vp, vp, vp, i32, vp, vp, i32, i32, i32, i32, i64, i64, i64, i64, i64,
                                      i32, i32, f32, vp]
    lib.skv_attend_weighted.restype = i32
    lib.skv_attend_weighted.argtypes = [vp, vp, vp, vp, i64, vp, i32, vp, i32, vp, vp, vp, i32, i32, i32, i32, i64, i64,
                                        i64, i64, i32, f32, vp]
    lib.skv_merge.restype = i32
    lib.skv_merge.argtypes = [vp, vp, vp, vp, i32, i32, i32, i32, vp]
    lib.skv_select.restype = i32
    lib.skv_select.argtypes = [C.POINTER(SkvState), vp, i32, i32, vp, i32, vp, vp, vp, i64, vp, vp, vp, vp, vp, f32, i32,
                               C.POINTER(SkvRope), vp]
    lib.skv_select_workspace_bytes.restype = i64
    lib.skv_select_workspace_bytes.argtypes = [i32, i32, i32]
    lib.skv_debug_select_probe.restype = None
    lib.skv_debug_select_probe.argtypes = [vp]
    lib.skv_set_overlap.restype = None
    lib.skv_set_overlap.argtypes = [i32]
    lib.skv_debug_attend_probe.restype = None
    lib.skv_debug_attend_probe.argtypes = [vp]
    lib.skv_attend_labels.restype = i32
    lib.skv_attend_labels.argtypes = [vp, vp, vp, vp, i64, vp, i32, vp, i32, vp, vp, vp, vp, i32, i32, i32, i32, i64, i64,
                                      i64, i64, i32, f32, vp]
    lib.skv_step_clusters.restype = i32
    lib.skv_step_clusters.argtypes = [i32, i32, i32, i32]
    lib.skv_step_workspace_bytes.restype = i64
    lib.skv_step_workspace_bytes.argtypes = [i32, i32, i32]
    lib.skv_step.restype = i32
    lib.skv_step.argtypes = [C.POINTER(SkvState), vp, i32, vp, i32, vp, vp, i64, i64, i64, i64, vp, vp, vp, vp, vp, i32, f32,
                             C.POINTER(SkvRope), vp]
    lib.skv_debug_step_probe.restype = None
    lib.skv_debug_step_probe.argtypes = [vp]
    lib.skv_insert.restype = i32
    lib.skv_insert.argtypes = [C.POINTER(SkvState), vp, i32, i32, i64, i64, vp, i32, i32, f64, f32, i32, i32, f32, i32, vp]
    lib.skv_insert_max_members.restype = i32
    lib.skv_fit_tensor_cores.restype = None
    lib.skv_fit_tensor_cores.argtypes = [i32]
    lib.skv_fit_workspace_bytes.restype = i64
    lib.skv_fit_workspace_bytes.argtypes = [i32, i32, i32, i32]
    lib.skv_fit.restype = i32
    lib.skv_fit.argtypes = [C.POINTER(SkvState), vp, i32, i64, i64, i32, i32, i32, i32, vp, f32, f32, f32, f32, vp, i32,
                            vp, i32, vp, i64, vp]
    lib.skv_add_rmsnorm.restype = i32
    lib.skv_add_rmsnorm.argtypes = [vp, vp, vp, vp, i32, i32, f32, vp]
    lib.skv_qk_rope_cache.restype = i32
    lib.skv_qk_rope_cache.argtypes = [vp, vp, vp, vp, vp, vp, i32, vp, vp, vp, i32, i32, i32, i32, i64, i64, i64, f32, vp]
    lib.skv_silu_mul.restype = i32
    lib.skv_silu_mul.argtypes = [vp, vp, i32, i32, vp]
    lib.skv_gemv_tp.restype = i32
    lib.skv_gemv_tp.argtypes = [vp, i32, i32, vp, i32, i32, vp, vp, vp, vp, f32, C.POINTER(SkvComm), i32,
                                C.POINTER(SkvComm), i32, vp]
    lib.skv_comm_bytes.restype = i64
    lib.skv_comm_bytes.argtypes = [i32, i32]
    lib.skv_comm_alloc.restype = i32
    lib.skv_comm_alloc.argtypes = [i64, C.POINTER(C.c_void_p)]
    lib.skv_comm_export.restype = i32
    lib.skv_comm_export.argtypes = [vp, vp]
    lib.skv_comm_open.restype = i32
    lib.skv_comm_open.argtypes = [vp, C.POINTER(C.c_void_p)]
    lib.skv_comm_close.restype = i32
    lib.skv_comm_close.argtypes = [vp]
    lib.skv_comm_free.restype = i32
    lib.skv_comm_free.argtypes = [vp]
    lib.skv_comm_view.restype = i32
    lib.skv_comm_view.argtypes = [C.POINTER(SkvComm), C.POINTER(C.c_void_p), i32, i32, i32]
    lib.skv_comm_tick.restype = i32
    lib.skv_comm_tick.argtypes = [C.POINTER(SkvComm), vp]
    lib.skv_comm_status.restype = i32
    lib.skv_comm_status.argtypes = [C.POINTER(SkvComm)]
    lib.skv_comm_reduce.restype = i32
    lib.skv_comm_reduce.argtypes = [C.POINTER(SkvComm), i32, vp, i32, i32, vp]
    lib.skv_comm_push.restype = i32
    lib.skv_comm_push.argtypes = [C.POINTER(SkvComm), i32, vp, i32, i32, vp]
    lib.skv_gemv_attended.restype = i32
    lib.skv_gemv_attended.argtypes = [vp, i32, i32, vp, i32, vp, i32, i32, vp, C.POINTER(SkvComm), i32, vp]
    lib.skv_gemv_supported.restype = i32
    lib.skv_gemv_supported.argtypes = [i32, i32, i32, i32]
    lib.skv_gemv.restype = i32
    lib.skv_gemv.argtypes = [vp, i32, i32, vp, i32, i32, vp, vp, vp, vp, vp, f32, vp]
    lib.skv_rebin.restype = i32
    lib.skv_rebin.argtypes = [C.POINTER(SkvState), vp, i32, i32, vp, i32, i64, i64, f32, i32, f32, vp, i64, vp]


def lib():
    """The loaded library; raises when it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise SkvError(f"{LIB_PATH} is missing: build it with `python -m sparse_kv_reads_b200.build` "
                           "(there is no CPU or PyTorch fallback for the CUDA kernels)")
        handle = C.CDLL(LIB_PATH)
        _declare(handle)
        _lib = handle
    return _lib


# entry points that launch exactly one kernel each: counted, so that a caller can tell how many of the library's
# kernels a captured decode step holds (GraphDecoder.launches_per_step)
_ONE_LAUNCH = {"skv_insert", "skv_select", "skv_attend", "skv_attend_weighted", "skv_attend_labels", "skv_step", "skv_gemv", "skv_gemv_tp", "skv_gemv_attended",
               "skv_add_rmsnorm", "skv_qk_rope_cache", "skv_silu_mul", "skv_comm_push", "skv_comm_reduce", "skv_comm_tick"}
launches = 0


def check(code: int, what: str) -> None:
    global launches
    if what in _ONE_LAUNCH:
        launches += 1
    if code != 0:
        L = lib()
        msg = L.skv_error_string(code).decode()
        if code == -7:
            msg += ": " + L.skv_last_cuda_error().decode()
        raise SkvError(f"{what} failed ({code}): {msg}")


def ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.bfloat16:
        return SKV_BF16
    if dt == torch.float32:
        return SKV_F32
    raise ValueError(f"unsupported cache dtype {dt}; the kernels take bfloat16 or float32")


def stream_ptr(device=None) -> int:
    return torch.cuda.current_stream(device).cuda_stream
