"""ctypes binding of libb200ops.so, the C-ABI library that holds every CUDA kernel.

It plays the role of the reference's lazily loaded kernel modules
(torch_mojo_backend/eager_kernels/aten_fast.py:4495-4534: import once, latch failures) with the
same calling contract as its native bridges (raw pointers, element strides, dtype enums, stream;
torch_mojo_backend/eager_kernels/bf16_matmul_ops.mojo:25-63).

There is no fallback: if the library is missing, cannot be loaded or speaks another ABI version,
`lib()` raises and every op that needs a kernel fails loudly.
"""

from __future__ import annotations

import ctypes
import os
from pathlib import Path

import torch

ABI_VERSION = 2

F32 = 0
BF16 = 1

REDUCE_SUM = 0
REDUCE_MEAN = 1
REDUCE_AMAX = 2

EPILOGUE_NONE = 0
EPILOGUE_GELU_TANH = 1
EPILOGUE_GELU_ERF = 2

ROUTE_AUTO = 0
ROUTE_SIMT = 1
ROUTE_TCGEN05 = 2
ROUTE_SKINNY = 3
ROUTE_SPLIT3 = 4

ERR_DEVICE_TIMEOUT = -6

# bits of the per-device status word (b200_device_status)
STATUS_GEMM_TIMEOUT = 1
STATUS_SDPA_TIMEOUT = 2
STATUS_TEST_TIMEOUT = 4
STATUS_INDEX_OUT_OF_RANGE = 8

STATIC_SCRATCH_BYTES = 8 * 1024 * 1024  # B200_STATIC_SCRATCH_BYTES of include/b200ops.h

PACKAGE_ROOT = Path(__file__).resolve().parent.parent
LIBRARY_PATH = PACKAGE_ROOT / "libb200ops.so"

# Every symbol include/b200ops.h declares; checked at load time and by the CPU test-suite.
EXPORTED_SYMBOLS = (
    "b200_abi_version",
    "b200_status_string",
    "b200_last_error",
    "b200_device_status",
    "b200_debug_wait_timeout",
    "b200_layer_norm",
    "b200_softmax_lastdim",
    "b200_softmax_masked",
    "b200_gelu",
    "b200_reduce_lastdim",
    "b200_gelu_backward",
    "b200_softmax_backward",
    "b200_layer_norm_backward_workspace_bytes",
    "b200_layer_norm_backward",
    "b200_sum_rows_workspace_bytes",
    "b200_sum_rows",
    "b200_embedding_sum",
    "b200_argmax_lastdim",
    "b200_copy_rows",
    "b200_gemm_route",
    "b200_gemm_workspace_bytes",
    "b200_gemm",
    "b200_gemm_small_m_static",
    "b200_sdpa_route",
    "b200_sdpa_fwd",
    "b200_sdpa_bwd_workspace_bytes",
    "b200_sdpa_bwd",
)


class NativeLibraryError(RuntimeError):
    """libb200ops.so is missing, unloadable or incompatible."""


class KernelError(RuntimeError):
    """A C-ABI entry point returned a non-zero status."""

    def __init__(self, op: str, status: int, detail: str):
        self.op = op
        self.status = status
        self.detail = detail
        super().__init__(f"{op} failed with status {status}: {detail}")


class GemmArgs(ctypes.Structure):
    _fields_ = [
        ("a", ctypes.c_void_p),
        ("b", ctypes.c_void_p),
        ("bias", ctypes.c_void_p),
        ("residual", ctypes.c_void_p),
        ("c", ctypes.c_void_p),
        ("m", ctypes.c_int64),
        ("n", ctypes.c_int64),
        ("k", ctypes.c_int64),
        ("batch", ctypes.c_int64),
        ("a_row_stride", ctypes.c_int64),
        ("a_col_stride", ctypes.c_int64),
        ("a_batch_stride", ctypes.c_int64),
        ("b_row_stride", ctypes.c_int64),
        ("b_col_stride", ctypes.c_int64),
        ("b_batch_stride", ctypes.c_int64),
        ("c_row_stride", ctypes.c_int64),
        ("c_batch_stride", ctypes.c_int64),
        ("bias_row_stride", ctypes.c_int64),
        ("residual_row_stride", ctypes.c_int64),
        ("alpha", ctypes.c_float),
        ("beta", ctypes.c_float),
        ("in_dtype", ctypes.c_int32),
        ("bias_dtype", ctypes.c_int32),
        ("residual_dtype", ctypes.c_int32),
        ("out_dtype", ctypes.c_int32),
        ("epilogue", ctypes.c_int32),
        ("route", ctypes.c_int32),
    ]


class SdpaArgs(ctypes.Structure):
    _fields_ = [
        ("q", ctypes.c_void_p),
        ("k", ctypes.c_void_p),
        ("v", ctypes.c_void_p),
        ("o", ctypes.c_void_p),
        ("lse", ctypes.c_void_p),
        ("batch", ctypes.c_int64),
        ("heads", ctypes.c_int64),
        ("q_len", ctypes.c_int64),
        ("kv_len", ctypes.c_int64),
        ("head_dim", ctypes.c_int64),
        ("q_strides", ctypes.c_int64 * 3),
        ("k_strides", ctypes.c_int64 * 3),
        ("v_strides", ctypes.c_int64 * 3),
        ("o_strides", ctypes.c_int64 * 3),
        ("scale", ctypes.c_float),
        ("causal", ctypes.c_int32),
        ("dtype", ctypes.c_int32),
        ("route", ctypes.c_int32),
    ]


class SdpaBwdArgs(ctypes.Structure):
    _fields_ = [
        ("q", ctypes.c_void_p),
        ("k", ctypes.c_void_p),
        ("v", ctypes.c_void_p),
        ("o", ctypes.c_void_p),
        ("d_out", ctypes.c_void_p),
        ("lse", ctypes.c_void_p),
        ("dq", ctypes.c_void_p),
        ("dk", ctypes.c_void_p),
        ("dv", ctypes.c_void_p),
        ("workspace", ctypes.c_void_p),
        ("workspace_bytes", ctypes.c_size_t),
        ("batch", ctypes.c_int64),
        ("heads", ctypes.c_int64),
        ("q_len", ctypes.c_int64),
        ("kv_len", ctypes.c_int64),
        ("head_dim", ctypes.c_int64),
        ("q_strides", ctypes.c_int64 * 3),
        ("k_strides", ctypes.c_int64 * 3),
        ("v_strides", ctypes.c_int64 * 3),
        ("o_strides", ctypes.c_int64 * 3),
        ("d_out_strides", ctypes.c_int64 * 3),
        ("dq_strides", ctypes.c_int64 * 3),
        ("dk_strides", ctypes.c_int64 * 3),
        ("dv_strides", ctypes.c_int64 * 3),
        ("scale", ctypes.c_float),
        ("causal", ctypes.c_int32),
        ("dtype", ctypes.c_int32),
    ]


_lib: ctypes.CDLL | None = None
_load_error: NativeLibraryError | None = None

# Number of kernel-launching C-ABI calls made by this process (bench.py reports it).
launch_count = 0


class KernelProfiler:
    """Optional per-launch timing with CUDA events on the launching stream. While installed
    (`native.profiler = KernelProfiler()`), every op records (name, algorithmic work, events);
    `summary()` synchronises and returns per-op totals. Off by default: events cost host time."""

    def __init__(self):
        self.records = []

    def begin(self, device):
        ev = torch.cuda.Event(enable_timing=True)
        ev.record(torch.cuda.current_stream(device))
        return ev

    def end(self, device, start, name, flops, bytes_):
        ev = torch.cuda.Event(enable_timing=True)
        ev.record(torch.cuda.current_stream(device))
        self.records.append((name, flops, bytes_, start, ev))

    def summary(self):
        torch.cuda.synchronize()
        out = {}
        for name, flops, bytes_, start, end in self.records:
            agg = out.setdefault(name, {"launches": 0, "ms": 0.0, "flops": 0.0, "bytes": 0.0})
            agg["launches"] += 1
            agg["ms"] += start.elapsed_time(end)
            agg["flops"] += flops
            agg["bytes"] += bytes_
        return out


profiler: KernelProfiler | None = None


def _declare(dll: ctypes.CDLL) -> None:
    i32, i64, f32, vp = ctypes.c_int32, ctypes.c_int64, ctypes.c_float, ctypes.c_void_p
    dll.b200_abi_version.restype = i32
    dll.b200_abi_version.argtypes = []
    dll.b200_status_string.restype = ctypes.c_char_p
    dll.b200_status_string.argtypes = [i32]
    dll.b200_last_error.restype = ctypes.c_char_p
    dll.b200_last_error.argtypes = []
    dll.b200_device_status.restype = i32
    dll.b200_device_status.argtypes = [ctypes.POINTER(ctypes.c_uint32)]
    dll.b200_debug_wait_timeout.restype = i32
    dll.b200_debug_wait_timeout.argtypes = [ctypes.c_uint64, vp]
    dll.b200_layer_norm.restype = i32
    dll.b200_layer_norm.argtypes = [vp, vp, vp, vp, vp, vp, i64, i64, i64, f32, i32, i32, i32, vp]
    dll.b200_softmax_lastdim.restype = i32
    dll.b200_softmax_lastdim.argtypes = [vp, vp, i64, i64, i64, f32, i32, i64, i32, i32, vp]
    dll.b200_softmax_masked.restype = i32
    dll.b200_softmax_masked.argtypes = [vp, vp, vp, i64, i64, i64, i64, i64, i32, f32, f32, i32, i32, vp]
    dll.b200_gelu.restype = i32
    dll.b200_gelu.argtypes = [vp, vp, i64, i32, i32, vp]
    dll.b200_reduce_lastdim.restype = i32
    dll.b200_reduce_lastdim.argtypes = [vp, vp, i64, i64, i64, i32, i32, i32, vp]
    dll.b200_gelu_backward.restype = i32
    dll.b200_gelu_backward.argtypes = [vp, vp, vp, i64, i32, i32, vp]
    dll.b200_softmax_backward.restype = i32
    dll.b200_softmax_backward.argtypes = [vp, vp, vp, i64, i64, i64, i64, ctypes.c_float, i32, i32, vp]
    dll.b200_layer_norm_backward_workspace_bytes.restype = ctypes.c_size_t
    dll.b200_layer_norm_backward_workspace_bytes.argtypes = [i64, i64]
    dll.b200_layer_norm_backward.restype = i32
    dll.b200_layer_norm_backward.argtypes = [
        vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, ctypes.c_size_t, i64, i64, i64, i64, i32, i32, i32, i32, i32, vp,
    ]
    dll.b200_sum_rows_workspace_bytes.restype = ctypes.c_size_t
    dll.b200_sum_rows_workspace_bytes.argtypes = [i64, i64, i32]
    dll.b200_sum_rows.restype = i32
    dll.b200_sum_rows.argtypes = [vp, vp, vp, ctypes.c_size_t, i64, i64, i64, i32, i32, vp]
    dll.b200_embedding_sum.restype = i32
    dll.b200_embedding_sum.argtypes = [vp, vp, i64, i64, vp, vp, i64, i64, i64, vp, i64, i64, i32, i32, vp]
    dll.b200_argmax_lastdim.restype = i32
    dll.b200_argmax_lastdim.argtypes = [vp, vp, i64, i64, i64, i32, vp]
    dll.b200_copy_rows.restype = i32
    dll.b200_copy_rows.argtypes = [vp, vp, i64, i64, i64, i64, i32, vp]
    dll.b200_gemm_route.restype = i32
    dll.b200_gemm_route.argtypes = [ctypes.POINTER(GemmArgs)]
    dll.b200_gemm_workspace_bytes.restype = ctypes.c_size_t
    dll.b200_gemm_workspace_bytes.argtypes = [ctypes.POINTER(GemmArgs)]
    dll.b200_gemm.restype = i32
    dll.b200_gemm.argtypes = [ctypes.POINTER(GemmArgs), vp, ctypes.c_size_t, vp]
    dll.b200_gemm_small_m_static.restype = i32
    dll.b200_gemm_small_m_static.argtypes = [ctypes.POINTER(GemmArgs), vp]
    dll.b200_sdpa_route.restype = i32
    dll.b200_sdpa_route.argtypes = [ctypes.POINTER(SdpaArgs)]
    dll.b200_sdpa_fwd.restype = i32
    dll.b200_sdpa_fwd.argtypes = [ctypes.POINTER(SdpaArgs), vp]
    dll.b200_sdpa_bwd_workspace_bytes.restype = ctypes.c_size_t
    dll.b200_sdpa_bwd_workspace_bytes.argtypes = [ctypes.POINTER(SdpaBwdArgs)]
    dll.b200_sdpa_bwd.restype = i32
    dll.b200_sdpa_bwd.argtypes = [ctypes.POINTER(SdpaBwdArgs), vp]


def lib() -> ctypes.CDLL:
    """The loaded library; raises NativeLibraryError (every time) when it is unusable."""
    global _lib, _load_error
    if _lib is not None:
        return _lib
    if _load_error is not None:
        raise _load_error
    path = Path(os.environ.get("B200OPS_LIBRARY", LIBRARY_PATH))
    try:
        if not path.exists():
            raise NativeLibraryError(
                f"{path} does not exist. Build it with `python -c 'import __graft_entry__ as g; "
                f"g.build()'` or `make -C {PACKAGE_ROOT / 'csrc'}`. There is no CPU or PyTorch "
                "fallback for the b200 kernels."
            )
        try:
            dll = ctypes.CDLL(str(path))
        except OSError as e:
            raise NativeLibraryError(f"cannot load {path}: {e}") from e
        missing = [s for s in EXPORTED_SYMBOLS if not hasattr(dll, s)]
        if missing:
            raise NativeLibraryError(f"{path} lacks symbols {missing}")
        _declare(dll)
        version = dll.b200_abi_version()
        if version != ABI_VERSION:
            raise NativeLibraryError(f"{path} has ABI version {version}, expected {ABI_VERSION}")
    except NativeLibraryError as e:
        _load_error = e
        raise
    _lib = dll
    return dll


def check(op: str, status: int) -> None:
    if status != 0:
        dll = lib()
        detail = dll.b200_last_error().decode() or dll.b200_status_string(status).decode()
        raise KernelError(op, status, detail)


def dtype_enum(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise TypeError(f"the b200 kernels take float32 and bfloat16 tensors, not {dtype}")


def supported_dtype(dtype: torch.dtype) -> bool:
    return dtype in (torch.float32, torch.bfloat16)


def current_stream(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def require_cuda(op: str, *tensors: torch.Tensor | None) -> torch.device:
    device = None
    for t in tensors:
        if t is None:
            continue
        if t.device.type != "cuda":
            raise RuntimeError(
                f"b200::{op} got a tensor on {t.device}; the b200 kernels run on CUDA tensors only "
                "and there is no CPU fallback."
            )
        if device is None:
            device = t.device
        elif t.device != device:
            raise RuntimeError(f"b200::{op} got tensors on {device} and {t.device}")
    assert device is not None
    return device


def device_status() -> int:
    """Status word of the current device (0 = no kernel gave up a bounded wait). Synchronises."""
    word = ctypes.c_uint32(0)
    status = lib().b200_device_status(ctypes.byref(word))
    if status not in (0, ERR_DEVICE_TIMEOUT):
        check("device_status", status)
    return word.value
