"""The C-ABI boundary without a GPU: the library loads, exports every symbol the header declares,
and the ctypes structs have the layout a C compiler gives the header's structs."""

import ctypes
import re
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
HEADER = ROOT / "include" / "b200ops.h"


@pytest.fixture(scope="module")
def native():
    from torch_mojo_backend import native as n

    return n


def declared_symbols():
    text = HEADER.read_text()
    return sorted(set(re.findall(r"B200_API\s+[\w\s\*]+?\b(b200_\w+)\s*\(", text)))


def test_header_declares_what_python_expects(native):
    assert declared_symbols() == sorted(native.EXPORTED_SYMBOLS)


def test_library_loads_and_exports_every_declared_symbol(native):
    assert native.LIBRARY_PATH.exists(), "libb200ops.so is not built (run __graft_entry__.build())"
    dll = native.lib()
    for name in declared_symbols():
        assert hasattr(dll, name), name
    assert dll.b200_abi_version() == native.ABI_VERSION
    assert dll.b200_status_string(0) == b"ok"
    assert b"invalid" in dll.b200_status_string(-1)


def test_struct_layout_matches_c(native, tmp_path):
    src = tmp_path / "layout.c"
    src.write_text(
        '#include <stdio.h>\n#include <stddef.h>\n#include "b200ops.h"\n'
        "int main(void) {\n"
        '  printf("%zu %zu %zu %zu %zu\\n", sizeof(b200_gemm_args), offsetof(b200_gemm_args, m),'
        " offsetof(b200_gemm_args, alpha), offsetof(b200_gemm_args, in_dtype), offsetof(b200_gemm_args, route));\n"
        '  printf("%zu %zu %zu %zu %zu\\n", sizeof(b200_sdpa_args), offsetof(b200_sdpa_args, batch),'
        " offsetof(b200_sdpa_args, q_strides), offsetof(b200_sdpa_args, scale), offsetof(b200_sdpa_args, route));\n"
        "  return 0;\n}\n"
    )
    exe = tmp_path / "layout"
    subprocess.run(["gcc", "-std=c99", "-I", str(ROOT / "include"), str(src), "-o", str(exe)], check=True)
    out = subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.split("\n")
    g, s = native.GemmArgs, native.SdpaArgs
    assert [int(v) for v in out[0].split()] == [
        ctypes.sizeof(g), g.m.offset, g.alpha.offset, g.in_dtype.offset, g.route.offset]
    assert [int(v) for v in out[1].split()] == [
        ctypes.sizeof(s), s.batch.offset, s.q_strides.offset, s.scale.offset, s.route.offset]


def test_validation_errors_need_no_gpu(native):
    """Argument validation runs before any CUDA call, so it can be exercised on a CPU-only box."""
    dll = native.lib()
    st = dll.b200_layer_norm(None, None, None, None, None, None, 4, 8, 8, 1e-5, 0, 0, 0, None)
    assert st == -1 and b"null pointer" in dll.b200_last_error()
    st = dll.b200_gelu(None, None, -1, 0, 0, None)
    assert st == -1
    st = dll.b200_softmax_lastdim(None, None, 4, 8, 8, 1.0, 0, 0, 0, 1, None)
    assert st == -2  # fp32 -> bf16 is not a softmax signature
    g = native.GemmArgs()
    g.m, g.n, g.k, g.batch = 4, 4, 4, 1
    g.in_dtype = 7
    assert dll.b200_gemm(ctypes.byref(g), None, 0, None) == -1
    with pytest.raises(native.KernelError, match="bad dtype"):
        native.check("gemm", dll.b200_gemm(ctypes.byref(g), None, 0, None))
    # empty problems succeed without touching the device
    assert dll.b200_gelu(None, None, 0, 0, 0, None) == 0
    assert dll.b200_reduce_lastdim(None, None, 0, 5, 5, 0, 0, 0, None) == 0


def test_missing_library_fails_loudly(native, monkeypatch, tmp_path):
    monkeypatch.setattr(native, "_lib", None)
    monkeypatch.setattr(native, "_load_error", None)
    monkeypatch.setenv("B200OPS_LIBRARY", str(tmp_path / "nope.so"))
    with pytest.raises(native.NativeLibraryError, match="no CPU or PyTorch fallback"):
        native.lib()
    # the failure is latched: later calls raise the same error instead of retrying silently
    with pytest.raises(native.NativeLibraryError):
        native.lib()


@pytest.mark.gpu
def test_bounded_wait_runs_out_and_reports_a_status(native):
    """A device-side wait whose limit runs out (a barrier nothing signals, 100 us) ends the kernel
    with a status bit instead of hanging: the host reads B200_ERR_DEVICE_TIMEOUT once, the word is
    cleared by the read, and the next kernel on the device runs and is correct."""
    import torch

    from torch_mojo_backend import ops

    lib = native.lib()
    assert native.device_status() == 0
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert lib.b200_debug_wait_timeout(0, stream) == -1          # limit validated on the host
    assert lib.b200_debug_wait_timeout(10**9, stream) == -1
    assert lib.b200_debug_wait_timeout(100_000, stream) == 0
    torch.cuda.synchronize()  # returns: the kernel gave up by itself
    word = ctypes.c_uint32(0)
    assert lib.b200_device_status(ctypes.byref(word)) == native.ERR_DEVICE_TIMEOUT
    assert word.value == native.STATUS_TEST_TIMEOUT
    assert lib.b200_device_status(ctypes.byref(word)) == 0 and word.value == 0  # cleared by the first read
    a = torch.randn((256, 128), device="cuda").bfloat16()
    w = torch.randn((192, 128), device="cuda").bfloat16()
    y = ops.gemm(a, w.t(), None, None, 1.0, 1.0, 0, torch.float32)
    torch.testing.assert_close(y.cpu(), a.float().cpu() @ w.float().cpu().t(), rtol=1e-4, atol=1e-3)
    assert native.device_status() == 0
