"""ctypes binding of ``libb200attn.so`` (the C ABI declared in ``include/b200attn.h``).

The library holds sm_100a code only.  There is no fallback of any kind: if the
shared object is missing or a call fails, a ``RuntimeError`` carrying the
library's own error text is raised.
"""
from __future__ import annotations

import ctypes as C
import os
import threading
from typing import Dict, Optional, Tuple

import torch

ABI_VERSION = 1

F16, BF16, F32 = 0, 1, 2
DENSE, RAGGED, PAGED = 0, 1, 2

DTYPE_CODE = {torch.float16: F16, torch.bfloat16: BF16, torch.float32: F32}

_LIB_NAME = "libb200attn.so"
_PKG_ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

EXPORTS = (
    "b200attn_abi_version",
    "b200attn_last_error",
    "b200attn_device_info",
    "b200attn_prefill_workspace_bytes",
    "b200attn_decode_workspace_bytes",
    "b200attn_prefill",
    "b200attn_decode",
    "b200attn_decode_static",
    "b200attn_decode_static_check",
    "b200attn_selftest_wait_expiry",
    "b200attn_paged_append",
    "b200attn_softmax",
    "b200attn_check_workspace",
)


class DeviceInfo(C.Structure):
    _fields_ = [
        ("sm_count", C.c_int32),
        ("cc_major", C.c_int32),
        ("cc_minor", C.c_int32),
        ("max_smem_optin", C.c_int32),
    ]


class PrefillArgs(C.Structure):
    _fields_ = [
        ("q", C.c_void_p),
        ("k", C.c_void_p),
        ("v", C.c_void_p),
        ("out", C.c_void_p),
        ("q_indptr", C.c_void_p),
        ("kv_indptr", C.c_void_p),
        ("k_table", C.c_void_p),
        ("v_table", C.c_void_p),
        ("workspace", C.c_void_p),
        ("workspace_bytes", C.c_size_t),
        ("total_q", C.c_int64),
        ("total_kv", C.c_int64),
        ("table_stride", C.c_int64),
        ("dtype", C.c_int32),
        ("layout", C.c_int32),
        ("indptr_is_i64", C.c_int32),
        ("batch", C.c_int32),
        ("q_heads", C.c_int32),
        ("kv_heads", C.c_int32),
        ("max_q", C.c_int32),
        ("max_kv", C.c_int32),
        ("head_dim", C.c_int32),
        ("page_size", C.c_int32),
        ("is_causal", C.c_int32),
        ("device", C.c_int32),
        ("sm_scale", C.c_float),
    ]


class DecodeArgs(C.Structure):
    _fields_ = [
        ("q", C.c_void_p),
        ("k", C.c_void_p),
        ("v", C.c_void_p),
        ("out", C.c_void_p),
        ("kv_indptr", C.c_void_p),
        ("k_table", C.c_void_p),
        ("v_table", C.c_void_p),
        ("workspace", C.c_void_p),
        ("workspace_bytes", C.c_size_t),
        ("total_kv", C.c_int64),
        ("table_stride", C.c_int64),
        ("dtype", C.c_int32),
        ("layout", C.c_int32),
        ("indptr_is_i64", C.c_int32),
        ("batch", C.c_int32),
        ("q_heads", C.c_int32),
        ("kv_heads", C.c_int32),
        ("q_len", C.c_int32),
        ("max_kv", C.c_int32),
        ("head_dim", C.c_int32),
        ("page_size", C.c_int32),
        ("causal_drafts", C.c_int32),
        ("device", C.c_int32),
        ("sm_scale", C.c_float),
    ]


class PagedAppendArgs(C.Structure):
    _fields_ = [
        ("src", C.c_void_p),
        ("cache", C.c_void_p),
        ("src_indptr", C.c_void_p),
        ("dst_pos", C.c_void_p),
        ("table", C.c_void_p),
        ("workspace", C.c_void_p),
        ("workspace_bytes", C.c_size_t),
        ("total_rows", C.c_int64),
        ("cache_rows", C.c_int64),
        ("table_stride", C.c_int64),
        ("row_bytes", C.c_int32),
        ("indptr_is_i64", C.c_int32),
        ("batch", C.c_int32),
        ("page_size", C.c_int32),
        ("device", C.c_int32),
    ]


class SoftmaxArgs(C.Structure):
    _fields_ = [
        ("x", C.c_void_p),
        ("out", C.c_void_p),
        ("rows", C.c_int64),
        ("cols", C.c_int64),
        ("dtype", C.c_int32),
        ("log_softmax", C.c_int32),
        ("device", C.c_int32),
    ]


_lib: Optional[C.CDLL] = None
_lib_lock = threading.Lock()


def library_path() -> str:
    return os.environ.get("B200ATTN_LIBRARY", os.path.join(_PKG_ROOT, _LIB_NAME))


def lib() -> C.CDLL:
    """Load the shared object once; raise loudly if it is not there."""
    global _lib
    if _lib is not None:
        return _lib
    with _lib_lock:
        if _lib is not None:
            return _lib
        path = library_path()
        if not os.path.exists(path):
            raise RuntimeError(
                f"{_LIB_NAME} not found at {path}. Build it with `make -C {os.path.join(_PKG_ROOT, 'csrc')}` "
                "(needs nvcc with sm_100a support). There is no CPU or Triton fallback."
            )
        handle = C.CDLL(path)
        handle.b200attn_abi_version.restype = C.c_int
        handle.b200attn_last_error.restype = C.c_char_p
        handle.b200attn_device_info.argtypes = [C.c_int, C.POINTER(DeviceInfo)]
        handle.b200attn_device_info.restype = C.c_int
        handle.b200attn_prefill_workspace_bytes.argtypes = [C.POINTER(PrefillArgs)]
        handle.b200attn_prefill_workspace_bytes.restype = C.c_size_t
        handle.b200attn_decode_workspace_bytes.argtypes = [C.POINTER(DecodeArgs)]
        handle.b200attn_decode_workspace_bytes.restype = C.c_size_t
        handle.b200attn_prefill.argtypes = [C.POINTER(PrefillArgs), C.c_void_p]
        handle.b200attn_prefill.restype = C.c_int
        handle.b200attn_decode.argtypes = [C.POINTER(DecodeArgs), C.c_void_p]
        handle.b200attn_decode.restype = C.c_int
        handle.b200attn_decode_static.argtypes = [C.POINTER(DecodeArgs), C.c_void_p]
        handle.b200attn_decode_static.restype = C.c_int
        handle.b200attn_decode_static_check.argtypes = [C.c_int, C.c_void_p, C.POINTER(C.c_int32)]
        handle.b200attn_decode_static_check.restype = C.c_int
        handle.b200attn_selftest_wait_expiry.argtypes = [C.c_int, C.c_void_p, C.c_uint32, C.c_void_p]
        handle.b200attn_selftest_wait_expiry.restype = C.c_int
        handle.b200attn_paged_append.argtypes = [C.POINTER(PagedAppendArgs), C.c_void_p]
        handle.b200attn_paged_append.restype = C.c_int
        handle.b200attn_softmax.argtypes = [C.POINTER(SoftmaxArgs), C.c_void_p]
        handle.b200attn_softmax.restype = C.c_int
        handle.b200attn_check_workspace.argtypes = [C.c_void_p, C.c_void_p, C.POINTER(C.c_int32)]
        handle.b200attn_check_workspace.restype = C.c_int
        got = handle.b200attn_abi_version()
        if got != ABI_VERSION:
            raise RuntimeError(f"{path}: ABI version {got}, expected {ABI_VERSION}")
        _lib = handle
        return _lib


def last_error() -> str:
    msg = lib().b200attn_last_error()
    return msg.decode("utf-8", "replace") if msg else ""


def check(status: int, what: str) -> None:
    if status != 0:
        raise RuntimeError(f"{what} failed with status {status}: {last_error()}")


def device_info(device: int) -> DeviceInfo:
    info = DeviceInfo()
    check(lib().b200attn_device_info(int(device), C.byref(info)), "b200attn_device_info")
    return info


# ---------------------------------------------------------------------------
# Workspace: one zero-initialised byte buffer per (device, stream), grown on demand.
# Word 0 is the device error code; kernels of the same stream reuse the rest.
# ---------------------------------------------------------------------------
_workspaces: Dict[Tuple[int, int], torch.Tensor] = {}
# buffers replaced by a larger one: a kernel still running may yet set its error word in one of them, so they are
# kept (alive and un-reused) until the next error check has read them
_retired: Dict[Tuple[int, int], list] = {}


def workspace(device: torch.device, stream_ptr: int, nbytes: int) -> torch.Tensor:
    key = (device.index if device.index is not None else torch.cuda.current_device(), int(stream_ptr))
    buf = _workspaces.get(key)
    if buf is None or buf.numel() < nbytes:
        size = max(int(nbytes), 1 << 20)
        size = (size + 255) & ~255
        if buf is not None:
            _retired.setdefault(key, []).append(buf)
        buf = torch.zeros(size, dtype=torch.uint8, device=device)
        _workspaces[key] = buf
    return buf


def check_device_errors() -> None:
    """Synchronise and raise if any kernel launched so far recorded a device-side error
    (bounded wait expired, block-table entry out of range, planner overflow)."""
    code = C.c_int32(0)
    first_error = None
    for (dev, stream_ptr), buf in list(_workspaces.items()):
        for b in [buf] + _retired.pop((dev, stream_ptr), []):
            status = lib().b200attn_check_workspace(C.c_void_p(b.data_ptr()), C.c_void_p(stream_ptr), C.byref(code))
            if status != 0 and first_error is None:
                first_error = (status, f"device error check on cuda:{dev}", last_error())
    if first_error is not None:
        raise RuntimeError(f"{first_error[1]} failed with status {first_error[0]}: {first_error[2]}")


def release_workspaces() -> None:
    _workspaces.clear()
    _retired.clear()
