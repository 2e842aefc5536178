"""Host-side marshalling and lowering logic, checked on a CPU-only box (the pattern of the
reference's fake-device wiring tests, tests/test_fa4_host_wiring.py:13-168): what the C ABI
would be called with, and that no path computes on the CPU instead."""

import pytest
import torch
import torch.nn.functional as F

from torch_mojo_backend import native, ops


def test_cpu_tensors_are_refused():
    x = torch.randn(4, 8)
    for call in (
        lambda: ops.layer_norm(x, None, None, 1e-5),
        lambda: ops.softmax(x),
        lambda: ops.gelu(x),
        lambda: ops.reduce(x, 0),
        lambda: ops.gemm(x, x.t()),
        lambda: ops.sdpa(x.view(1, 1, 4, 8), x.view(1, 1, 4, 8), x.view(1, 1, 4, 8)),
    ):
        with pytest.raises(RuntimeError, match="no CPU fallback"):
            call()


def test_gemm_args_carry_view_strides():
    a = torch.empty(16, 40, dtype=torch.bfloat16)[:, :32]  # row pitch 40
    w = torch.empty(24, 32, dtype=torch.bfloat16)           # nn.Linear weight [N, K]
    c = torch.empty(16, 24, dtype=torch.float32)
    bias = torch.empty(24, dtype=torch.bfloat16)
    g = ops.fill_gemm_args(a, w.t(), bias, None, c, 2.0, 0.5, native.EPILOGUE_GELU_TANH, native.ROUTE_AUTO)
    assert (g.m, g.n, g.k, g.batch) == (16, 24, 32, 1)
    assert (g.a_row_stride, g.a_col_stride) == (40, 1)
    assert (g.b_row_stride, g.b_col_stride) == (1, 32)  # t() view: K contiguous
    assert g.c_row_stride == 24 and g.bias_row_stride == 0
    assert (g.in_dtype, g.bias_dtype, g.out_dtype) == (native.BF16, native.BF16, native.F32)
    assert (g.alpha, g.beta, g.epilogue) == (2.0, 0.5, native.EPILOGUE_GELU_TANH)
    assert g.a == a.data_ptr() and g.b == w.data_ptr() and g.residual is None


def test_gemm_args_batched():
    a = torch.empty(12, 128, 64)
    b = torch.empty(12, 128, 64).transpose(1, 2)
    c = torch.empty(12, 128, 128)
    g = ops.fill_gemm_args(a, b, None, None, c, 1.0, 1.0, 0, 0)
    assert (g.batch, g.m, g.n, g.k) == (12, 128, 128, 64)
    assert (g.a_batch_stride, g.b_batch_stride, g.c_batch_stride) == (128 * 64, 128 * 64, 128 * 128)
    assert (g.b_row_stride, g.b_col_stride) == (1, 64)


def test_bias_normalisation():
    n = ops._normalise_bias
    row = torch.arange(6.0)
    assert n(row, 4, 6) is row
    assert n(row.view(1, 6), 4, 6).shape == (6,)
    col = torch.arange(4.0).view(4, 1)
    full = n(col, 4, 6)
    assert full.shape == (4, 6) and full.stride(1) == 1 and torch.equal(full[:, 0], col[:, 0])
    scalar = n(torch.tensor(3.0), 4, 6)
    assert scalar.shape == (4, 6) and (scalar == 3).all()
    assert n(None, 4, 6) is None


def test_rows_view_avoids_copies_when_it_can():
    x = torch.empty(8, 4, 16)
    t, rows, cols, stride = ops._as_rows(x)
    assert t is x and (rows, cols, stride) == (32, 16, 16)
    v = torch.empty(8, 32)[:, :16]
    t, rows, cols, stride = ops._as_rows(v)
    assert t is v and (rows, cols, stride) == (8, 16, 32)
    tr = torch.empty(16, 8).t()
    t, rows, cols, stride = ops._as_rows(tr)
    assert t.is_contiguous() and (rows, cols, stride) == (8, 16, 16)


def test_sdpa_args_from_fused_qkv_views():
    B, T, H, D = 2, 10, 4, 8
    qkv = torch.empty(B, T, 3 * H * D, dtype=torch.bfloat16)
    q, k, v = (t.view(B, T, H, D).transpose(1, 2) for t in qkv.split(H * D, dim=2))
    o = torch.empty(B, T, H, D, dtype=torch.bfloat16).transpose(1, 2)
    lse = torch.empty(B, H, T)
    s = ops.fill_sdpa_args(q, k, v, o, lse, True, 0.125, native.ROUTE_AUTO)
    assert (s.batch, s.heads, s.q_len, s.kv_len, s.head_dim) == (B, H, T, T, D)
    assert list(s.q_strides) == [T * 3 * H * D, D, 3 * H * D]
    assert list(s.o_strides) == [T * H * D, D, H * D]
    assert s.k - s.q == H * D * 2 and s.v - s.k == H * D * 2  # zero-copy views of one buffer
    assert s.causal == 1 and s.dtype == native.BF16


def test_meta_implementations_give_traced_shapes():
    with torch._subclasses.FakeTensorMode():
        x = torch.empty(4, 6, 16, device="cuda", dtype=torch.bfloat16)
        y, mean, rstd = ops.layer_norm(x, None, None, 1e-5, torch.float32)
        assert y.shape == x.shape and y.dtype == torch.float32 and mean.shape == (4, 6)
        assert ops.softmax(x, 1.0, False, 0, torch.float32).dtype == torch.float32
        assert ops.reduce(x, 0).shape == (4, 6)
        a = torch.empty(3, 5, 7, device="cuda")
        assert ops.gemm(a, torch.empty(3, 7, 2, device="cuda")).shape == (3, 5, 2)
        q = torch.empty(2, 4, 10, 8, device="cuda", dtype=torch.bfloat16)
        o, lse = ops.sdpa(q, q, q, True)
        assert o.shape == q.shape and o.stride() == (320, 8, 32, 1) and lse.shape == (2, 4, 10)
        with pytest.raises(RuntimeError, match="cannot be multiplied"):
            ops.gemm(torch.empty(3, 4, device="cuda"), torch.empty(5, 6, device="cuda"))


def test_gemm_fake_output_has_the_real_ops_strides():
    """The Meta implementation (what FakeTensor tracing sees) must describe the tensor the CUDA
    implementation returns, padded row pitch of a wide unaligned output included."""
    a = torch.empty(16, 64, dtype=torch.bfloat16, device="meta")
    w = torch.empty(64, 50257, dtype=torch.bfloat16, device="meta")
    y = ops.gemm(a, w, None, None, 1.0, 1.0, 0, torch.float32)
    assert tuple(y.shape) == (16, 50257) and y.stride() == (50264, 1)
    small = ops.gemm(a, torch.empty(64, 1000, dtype=torch.bfloat16, device="meta"))
    assert small.stride() == (1000, 1)
    one_row = ops.gemm(a[:1], w)
    assert one_row.stride() == (50257, 1)


def test_view_lowering_copies_when_the_runtime_layout_is_not_the_traced_one():
    from torch_mojo_backend import aten_functions as af

    padded = torch.arange(4 * 8, dtype=torch.float32).reshape(4, 8)[:, :5]  # row pitch 8, 5 columns
    flat = af.aten_view(padded, [-1])
    assert flat.shape == (20,) and torch.equal(flat, padded.reshape(-1))
    split = af.aten__unsafe_view(padded, [2, 2, 5])  # splitting the row dim stays a view
    assert split.data_ptr() == padded.data_ptr()
