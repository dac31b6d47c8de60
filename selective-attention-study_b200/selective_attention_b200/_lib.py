"""ctypes binding of libselective_attention_b200.so (declarations: include/selective_attention_b200.h).

There is no fallback: if the library is missing or a call returns a non-zero status, an exception is
raised.  Build the library with ``python -m selective_attention_b200.build``.
"""

from __future__ import annotations

import ctypes
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libselective_attention_b200.so")

SA_OK = 0
STATUS_NAMES = {1: "BAD_ARGUMENT", 2: "UNSUPPORTED", 3: "ALIGNMENT", 4: "WORKSPACE", 5: "CUDA", 6: "DEVICE_TIMEOUT",
                7: "TOO_LARGE"}
DTYPE_F32, DTYPE_BF16, DTYPE_F16 = 0, 1, 2
ENGINE_SIMT, ENGINE_TCGEN05 = 0, 1
DAMP_CODES = {"none": 0, "linear": 1, "sqrt": 2}

# every symbol include/selective_attention_b200.h declares
EXPORTS = ("sa_abi_version", "sa_status_string", "sa_last_cuda_error", "sa_engine_available", "sa_engine_supports", "sa_carry_rows", "sa_carry_checkpoints", "sa_forward",
           "sa_backward_workspace_bytes", "sa_backward", "sa_decode_workspace_bytes", "sa_decode_step", "sa_device_status", "sa_selftest_tcgen05", "sa_profile_enable",
           "sa_profile_collect", "sa_static_scratch_floats", "sa_forward_static_scratch", "sa_forward_selector",
           "sa_backward_selector", "sa_forward_fused", "sa_backward_fused", "sa_prefill_extend", "sa_selection_carry", "sa_launch_count", "sa_selftest_wait_timeout",
           "sa_tile_table_bytes", "sa_forward_live_tiles", "sa_backward_live_tiles", "sa_prefill_extend_live_tiles", "sa_decode_step_live_keys")


class Problem(ctypes.Structure):
    _fields_ = [("struct_bytes", ctypes.c_int32), ("dtype", ctypes.c_int32), ("engine", ctypes.c_int32),
                ("batch", ctypes.c_int32), ("heads", ctypes.c_int32), ("seq", ctypes.c_int32),
                ("head_dim", ctypes.c_int32), ("exempt", ctypes.c_int32), ("damp", ctypes.c_int32),
                ("train_len", ctypes.c_int32), ("q_stride", ctypes.c_int64 * 3), ("k_stride", ctypes.c_int64 * 3),
                ("v_stride", ctypes.c_int64 * 3)]


class Selector(ctypes.Structure):
    _fields_ = [("struct_bytes", ctypes.c_int32), ("reserved", ctypes.c_int32), ("q0", ctypes.c_void_p),
                ("k0", ctypes.c_void_p), ("q0_stride", ctypes.c_int64 * 2), ("k0_stride", ctypes.c_int64 * 2)]


class Tensor(ctypes.Structure):
    """sa_tensor: rows of head_dim contiguous elements at batch / head / token strides."""
    _fields_ = [("ptr", ctypes.c_void_p), ("dtype", ctypes.c_int32), ("reserved", ctypes.c_int32),
                ("stride", ctypes.c_int64 * 3)]


class LibraryError(RuntimeError):
    def __init__(self, fn: str, status: int, detail: str):
        super().__init__(f"{fn} failed: SA_ERR_{STATUS_NAMES.get(status, status)} ({detail})")
        self.status = status


_lib = None


def available() -> bool:
    return os.path.exists(LIB_PATH)


def load() -> ctypes.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    if not available():
        raise RuntimeError(f"{LIB_PATH} is missing: build it with `python -m selective_attention_b200.build` "
                           "(there is no fallback path)")
    lib = ctypes.CDLL(LIB_PATH)
    vp, i32, sz, f32p = ctypes.c_void_p, ctypes.c_int, ctypes.c_size_t, ctypes.c_void_p
    pp = ctypes.POINTER(Problem)
    lib.sa_abi_version.restype = i32
    lib.sa_status_string.restype = ctypes.c_char_p
    lib.sa_status_string.argtypes = [i32]
    lib.sa_last_cuda_error.restype = i32
    lib.sa_engine_available.restype = i32
    lib.sa_engine_available.argtypes = [i32]
    lib.sa_engine_supports.restype = i32
    lib.sa_engine_supports.argtypes = [i32] * 4
    lib.sa_carry_rows.restype = i32
    lib.sa_carry_rows.argtypes = [i32]
    lib.sa_carry_checkpoints.restype = i32
    lib.sa_carry_checkpoints.argtypes = [i32, i32]
    lib.sa_forward.restype = i32
    lib.sa_forward.argtypes = [pp, vp, vp, vp, f32p, f32p, f32p, f32p, vp]
    sp = ctypes.POINTER(Selector)
    lib.sa_forward_selector.restype = i32
    lib.sa_forward_selector.argtypes = [pp, vp, vp, vp, sp, f32p, f32p, f32p, f32p, vp]
    lib.sa_backward_selector.restype = i32
    lib.sa_backward_selector.argtypes = [pp, vp, vp, vp, sp, f32p, f32p, f32p, vp, i32, vp, vp, vp, f32p, f32p, vp, sz, vp]
    tp = ctypes.POINTER(Tensor)
    lib.sa_forward_fused.restype = i32
    lib.sa_forward_fused.argtypes = [pp, vp, vp, vp, sp, f32p, tp, f32p, f32p, f32p, vp]
    lib.sa_backward_fused.restype = i32
    lib.sa_backward_fused.argtypes = [pp, vp, vp, vp, sp, f32p, f32p, f32p, tp, tp, tp, tp, f32p, f32p, vp, sz, vp]
    lib.sa_tile_table_bytes.restype = sz
    lib.sa_tile_table_bytes.argtypes = [pp]
    lib.sa_forward_live_tiles.restype = i32
    lib.sa_forward_live_tiles.argtypes = [pp, vp, vp, vp, sp, f32p, tp, f32p, f32p, f32p, vp, sz, vp]
    lib.sa_backward_live_tiles.restype = i32
    lib.sa_backward_live_tiles.argtypes = [pp, vp, vp, vp, sp, f32p, f32p, f32p, tp, tp, tp, tp, f32p, f32p, vp, sz, vp, vp]
    lib.sa_prefill_extend_live_tiles.restype = i32
    lib.sa_prefill_extend_live_tiles.argtypes = [pp, i32, vp, vp, vp, f32p, ctypes.c_int64, f32p, f32p, f32p, f32p, vp, sz, vp]
    lib.sa_prefill_extend.restype = i32
    lib.sa_prefill_extend.argtypes = [pp, i32, vp, vp, vp, f32p, ctypes.c_int64, f32p, f32p, f32p, f32p, vp]
    lib.sa_selection_carry.restype = i32
    lib.sa_selection_carry.argtypes = [pp, vp, vp, sp, f32p, f32p, vp]
    lib.sa_launch_count.restype = ctypes.c_ulonglong
    lib.sa_selftest_wait_timeout.restype = i32
    lib.sa_selftest_wait_timeout.argtypes = [ctypes.c_uint, vp]
    lib.sa_backward_workspace_bytes.restype = sz
    lib.sa_backward_workspace_bytes.argtypes = [pp]
    lib.sa_backward.restype = i32
    lib.sa_backward.argtypes = [pp, vp, vp, vp, f32p, f32p, f32p, vp, i32, vp, vp, vp, vp, sz, vp]
    lib.sa_decode_workspace_bytes.restype = sz
    lib.sa_decode_workspace_bytes.argtypes = [i32] * 5
    lib.sa_decode_step.restype = i32
    lib.sa_decode_step.argtypes = [i32] * 8 + [vp] * 8 + [sz, vp]
    lib.sa_decode_step_live_keys.restype = i32
    lib.sa_decode_step_live_keys.argtypes = [i32] * 8 + [vp] * 9 + [sz, vp]
    lib.sa_device_status.restype = i32
    lib.sa_device_status.argtypes = [ctypes.POINTER(ctypes.c_uint), i32]
    lib.sa_selftest_tcgen05.restype = i32
    lib.sa_selftest_tcgen05.argtypes = [vp, vp, vp]
    lib.sa_static_scratch_floats.restype = sz
    lib.sa_forward_static_scratch.restype = i32
    lib.sa_forward_static_scratch.argtypes = [pp, vp, vp, vp, f32p, f32p, f32p, vp]
    lib.sa_profile_enable.restype = i32
    lib.sa_profile_enable.argtypes = [i32]
    lib.sa_profile_collect.restype = i32
    lib.sa_profile_collect.argtypes = [ctypes.POINTER(ctypes.c_float), i32]
    _lib = lib
    return lib


KERNEL_IDS = {"none": 0, "tc_colsum": 1, "tc_scan": 2, "tc_forward": 3, "tc_backward": 4, "dbar": 5, "decode": 6}


def profile_enable(kernel: str) -> None:
    check("sa_profile_enable", load().sa_profile_enable(KERNEL_IDS[kernel]))


def profile_collect(capacity: int = 512) -> list[float]:
    """Durations (ms) of the launches of the enabled kernel since the last collect."""
    buf = (ctypes.c_float * capacity)()
    n = load().sa_profile_collect(buf, capacity)
    if n < 0:
        raise RuntimeError("sa_profile_collect failed")
    return [buf[i] for i in range(n)]


def launch_count() -> int:
    """Kernels of the library launched by this process so far."""
    return int(load().sa_launch_count())


def device_status(clear: bool = True) -> int:
    """Status word of the tensor-core engine's bounded waits on the current device (0 = fine)."""
    value = ctypes.c_uint(0)
    check("sa_device_status", load().sa_device_status(ctypes.byref(value), int(clear)))
    return value.value


def check(fn: str, status: int) -> None:
    if status != SA_OK:
        lib = load()
        detail = lib.sa_status_string(status).decode()
        if status == 5:
            detail += f", cudaError {lib.sa_last_cuda_error()}"
        if status == 6:
            detail += "; results of the launch that gave up are invalid; read and clear the word with device_status()"
        raise LibraryError(fn, status, detail)
