"""ctypes binding of libvarq_b200.so (declarations in include/varq_b200.h).

There is no CPU implementation behind this module: if the shared library has not been
built, or a tensor does not live on a CUDA device, the callers raise.
"""
import ctypes
import os
import threading

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libvarq_b200.so")

OK, ERR_ARG, ERR_UNSUPPORTED, ERR_CUDA, ERR_WORKSPACE = 0, -1, -2, -3, -4
F32, F16, BF16 = 0, 1, 2
DTYPES = {torch.float32: F32, torch.float16: F16, torch.bfloat16: BF16}

# every symbol include/varq_b200.h declares
SYMBOLS = (
    "varq_version", "varq_last_error", "varq_launch_count", "varq_device_status", "varq_pack_int8", "varq_unpack_int8",
    "varq_quant_workspace_bytes", "varq_quant_pack", "varq_quant_pack_static",
    "varq_quant_static_scratch_bytes", "varq_unpack_dequant",
    "varq_attn_workspace_bytes", "varq_attn_fwd", "varq_attn_force_path",
    "varq_qk_norm_stats", "varq_quant_pack_prestats",
)


class Tensor(ctypes.Structure):
    _fields_ = [("ptr", ctypes.c_void_p), ("dtype", ctypes.c_int32), ("_pad", ctypes.c_int32),
                ("stride_b", ctypes.c_int64), ("stride_l", ctypes.c_int64), ("stride_h", ctypes.c_int64)]


class QParams(ctypes.Structure):
    _fields_ = [("scale", ctypes.c_void_p), ("zp", ctypes.c_void_p), ("row_of_token", ctypes.c_void_p),
                ("stride_b", ctypes.c_int64), ("stride_r", ctypes.c_int64), ("stride_h", ctypes.c_int64),
                ("stride_g", ctypes.c_int64),
                ("share_b", ctypes.c_int32), ("share_l", ctypes.c_int32), ("share_h", ctypes.c_int32),
                ("group", ctypes.c_int32),
                ("row_begin", ctypes.c_void_p), ("n_rows", ctypes.c_int32), ("_pad", ctypes.c_int32)]


_lib = None
_lock = threading.Lock()


def _declare(lib):
    i32, i64, vp, f32, sz = ctypes.c_int32, ctypes.c_int64, ctypes.c_void_p, ctypes.c_float, ctypes.c_size_t
    T, Q = ctypes.POINTER(Tensor), ctypes.POINTER(QParams)
    lib.varq_version.restype = ctypes.c_char_p
    lib.varq_version.argtypes = []
    lib.varq_last_error.restype = ctypes.c_char_p
    lib.varq_last_error.argtypes = []
    lib.varq_launch_count.restype = ctypes.c_uint64
    lib.varq_launch_count.argtypes = []
    lib.varq_device_status.restype = i32
    lib.varq_device_status.argtypes = [ctypes.POINTER(ctypes.c_int32)]
    lib.varq_pack_int8.restype = i32
    lib.varq_pack_int8.argtypes = [vp, i64, i32, i32, vp, vp]
    lib.varq_unpack_int8.restype = i32
    lib.varq_unpack_int8.argtypes = [vp, i64, i32, i32, vp, vp]
    lib.varq_quant_workspace_bytes.restype = sz
    lib.varq_quant_workspace_bytes.argtypes = [i32, i32, i32, i32, i32, i32, Q]
    lib.varq_quant_pack.restype = i32
    lib.varq_quant_pack.argtypes = [T, i32, i32, i32, i32, i32, i32, f32, T, Q, vp, sz, vp]
    lib.varq_quant_pack_prestats.restype = i32
    lib.varq_quant_pack_prestats.argtypes = [T, i32, i32, i32, i32, i32, i32, f32, T, Q, vp, sz, vp]
    lib.varq_qk_norm_stats.restype = i32
    lib.varq_qk_norm_stats.argtypes = [T, T, T, i32, i32, i32, i32, vp, f32, T, T, Q, vp, Q, vp, vp]
    lib.varq_quant_pack_static.restype = i32
    lib.varq_quant_pack_static.argtypes = [T, i32, i32, i32, i32, i32, i32, f32, T, Q, vp]
    lib.varq_quant_static_scratch_bytes.restype = sz
    lib.varq_quant_static_scratch_bytes.argtypes = []
    lib.varq_unpack_dequant.restype = i32
    lib.varq_unpack_dequant.argtypes = [T, i32, i32, i32, i32, i32, Q, T, vp]
    lib.varq_attn_workspace_bytes.restype = sz
    lib.varq_attn_workspace_bytes.argtypes = [i32, i32, i32, i32, i32, i32, i32]
    lib.varq_attn_force_path.restype = i32
    lib.varq_attn_force_path.argtypes = [i32]
    lib.varq_attn_fwd.restype = i32
    lib.varq_attn_fwd.argtypes = [T, T, T, Q, Q, i32, i32, i32, i32, i32, i32, i32, f32, T, vp, sz, vp]
    return lib


def lib():
    """The loaded library; raises if it has not been built."""
    global _lib
    if _lib is None:
        with _lock:
            if _lib is None:
                if not os.path.exists(LIB_PATH):
                    raise ImportError(
                        f"{LIB_PATH} is missing: build it with `python var-q_b200/build.py` "
                        "(needs nvcc; the library targets sm_100a and has no CPU fallback)")
                _lib = _declare(ctypes.CDLL(LIB_PATH))
    return _lib


def check(rc: int):
    if rc == OK:
        return
    msg = lib().varq_last_error().decode("utf-8", "replace")
    if rc in (ERR_ARG, ERR_UNSUPPORTED, ERR_WORKSPACE):
        raise ValueError(f"[VAR-Q] {msg}")
    raise RuntimeError(f"[VAR-Q] {msg}")


def require_cuda(t: torch.Tensor, what: str):
    if not t.is_cuda:
        raise RuntimeError(f"[VAR-Q] {what} must be a CUDA tensor: this build runs on the GPU only "
                           "(no CPU fallback exists)")


def stream_ptr(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def tensor_desc(ptr: int, dtype_code: int, sb: int, sl: int, sh: int) -> Tensor:
    return Tensor(ptr, dtype_code, 0, sb, sl, sh)


_workspaces = {}


def workspace(device, nbytes: int) -> torch.Tensor:
    """Scratch buffer of the current stream on `device`; it only grows.

    Kernels on one stream are ordered and may share scratch; kernels on two streams may overlap, so
    every stream gets its own buffer.  A buffer that is outgrown goes back to torch's caching
    allocator, which reuses a block only in the order of the stream it was allocated on.
    """
    index = device.index if device.index is not None else torch.cuda.current_device()
    key = (index, torch.cuda.current_stream(device).cuda_stream)
    buf = _workspaces.get(key)
    if buf is None or buf.numel() < nbytes:
        with torch.cuda.device(index):
            buf = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _workspaces[key] = buf
    return buf


ATTN_PATHS = {None: 0, "auto": 0, "small": 1, "stream": 2, "tc": 3, "mid": 4}


def force_attn_path(name):
    """Pin the attention kernel for later calls ("small", "stream", "tc", "mid"; None = automatic).  Test hook."""
    check(lib().varq_attn_force_path(ATTN_PATHS[name]))


def device_status() -> int:
    """First expired-wait code recorded by a kernel since the last call (0 = none); synchronises."""
    out = ctypes.c_int32(0)
    check(lib().varq_device_status(ctypes.byref(out)))
    return int(out.value)
