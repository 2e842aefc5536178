"""The allocation-free small-M GEMM entry point, called straight through the C ABI.

Some callers cannot give the library a workspace: they run inside another engine's fixed memory
budget, or their binding only passes the operand buffers through. `b200_gemm_small_m_static` keeps
its scratch in a static device array inside the library instead. This file is collected last on
purpose: if it fails, a run that stops at the first failure has already run every other test.
"""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _problem(m, k, n, seed):
    g = torch.Generator().manual_seed(seed)
    a = (torch.randn((m, k), generator=g) * 0.5).to(torch.bfloat16).cuda()
    w = (torch.randn((n, k), generator=g) * 0.1).to(torch.bfloat16).cuda()
    bias = torch.randn((n,), generator=g).to(torch.bfloat16).cuda()
    res = torch.randn((m, n), generator=g).cuda()
    return a, w.t(), bias, res


@pytest.mark.parametrize("m,k,n", [(16, 6400, 1600), (64, 3072, 768)])
def test_static_scratch_entry_matches_workspace_entry(m, k, n):
    from torch_mojo_backend import native, ops

    lib = native.lib()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    for call in range(2):  # two calls in a row share the static array
        a, b, bias, res = _problem(m, k, n, seed=100 + call)
        want = torch.empty((m, n), dtype=torch.float32, device="cuda")
        got = torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda")
        g_ws = ops.fill_gemm_args(a, b, bias, res, want, 1.0, 1.0, native.EPILOGUE_GELU_TANH, native.ROUTE_AUTO)
        assert lib.b200_gemm_route(ctypes.byref(g_ws)) == native.ROUTE_SKINNY
        need = lib.b200_gemm_workspace_bytes(ctypes.byref(g_ws))
        assert 0 < need <= native.STATIC_SCRATCH_BYTES
        workspace = torch.empty(need, dtype=torch.uint8, device="cuda")
        native.check("gemm", lib.b200_gemm(ctypes.byref(g_ws), workspace.data_ptr(), need, stream))

        g_static = ops.fill_gemm_args(a, b, bias, res, got, 1.0, 1.0, native.EPILOGUE_GELU_TANH, native.ROUTE_AUTO)
        torch.cuda.synchronize()
        reserved_before = torch.cuda.memory_reserved()
        free_before, _ = torch.cuda.mem_get_info()
        native.check("gemm_small_m_static", lib.b200_gemm_small_m_static(ctypes.byref(g_static), stream))
        torch.cuda.synchronize()
        # torch's allocator did not grow, and neither did the device's own count of used memory (a
        # cudaMalloc inside the library would not show in the first figure, it does in the second);
        # the first call's one-time lookup of the static array's address allocates nothing either
        assert torch.cuda.memory_reserved() == reserved_before
        assert torch.cuda.mem_get_info()[0] >= free_before
        # same kernels, same fixed reduction order: the two entry points agree bit for bit, which is
        # inside the 1e-4 fp32 tolerance the other GEMM tests use
        assert torch.equal(got, want), f"call {call}: max|diff| {(got - want).abs().max().item():.3e}"
        ref = torch.nn.functional.gelu(a.float() @ b.float() + bias.float(), approximate="tanh") + res
        torch.testing.assert_close(got, ref, rtol=1e-4, atol=1e-4 * ref.abs().max().item())


def test_static_scratch_entry_validates_like_the_workspace_entry():
    """Same host-side checks as b200_gemm, before any launch: a misaligned output or residual
    pointer, a row pitch shorter than a row and a bad enum are refused with a status."""
    from torch_mojo_backend import native, ops

    lib = native.lib()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    a, b, bias, res = _problem(16, 6400, 1600, seed=9)
    out = torch.empty((16, 1600), dtype=torch.float32, device="cuda")
    before = native.launch_count

    def args():
        return ops.fill_gemm_args(a, b, bias, res, out, 1.0, 1.0, 0, 0)

    g = args()
    g.c = out.data_ptr() + 2  # fp32 output at a 2-byte offset
    assert lib.b200_gemm_small_m_static(ctypes.byref(g), stream) == -3
    assert lib.b200_gemm(ctypes.byref(g), None, 0, stream) == -3
    g = args()
    g.residual = res.data_ptr() + 1
    assert lib.b200_gemm_small_m_static(ctypes.byref(g), stream) == -3
    g = args()
    g.bias = bias.data_ptr() + 1
    assert lib.b200_gemm_small_m_static(ctypes.byref(g), stream) == -3
    g = args()
    g.c_row_stride = 1599  # rows would overlap
    assert lib.b200_gemm_small_m_static(ctypes.byref(g), stream) == -1
    g = args()
    g.route = 17
    assert lib.b200_gemm_small_m_static(ctypes.byref(g), stream) == -1
    g = args()
    g.epilogue = 9
    assert lib.b200_gemm_small_m_static(ctypes.byref(g), stream) == -1
    torch.cuda.synchronize()
    assert native.launch_count == before and native.device_status() == 0


def test_static_scratch_entry_refuses_what_it_cannot_hold():
    from torch_mojo_backend import native, ops

    lib = native.lib()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    # a large-M problem does not take the split-K route at all
    a, b, bias, res = _problem(512, 1024, 512, seed=7)
    out = torch.empty((512, 512), dtype=torch.float32, device="cuda")
    g = ops.fill_gemm_args(a, b, None, None, out, 1.0, 1.0, 0, 0)
    assert lib.b200_gemm_small_m_static(ctypes.byref(g), stream) == -2
    assert b"use b200_gemm" in lib.b200_last_error()
    # a split-K problem whose partial sums exceed the static array: 2 x 128 x 9472 floats = 9.7 MB
    a, b, bias, res = _problem(128, 16384, 9472, seed=8)
    out = torch.empty((128, 9472), dtype=torch.float32, device="cuda")
    g = ops.fill_gemm_args(a, b, None, None, out, 1.0, 1.0, 0, 0)
    assert lib.b200_gemm_route(ctypes.byref(g)) == native.ROUTE_SKINNY
    assert lib.b200_gemm_workspace_bytes(ctypes.byref(g)) > native.STATIC_SCRATCH_BYTES
    assert lib.b200_gemm_small_m_static(ctypes.byref(g), stream) == -4
    assert b"static array holds" in lib.b200_last_error()
