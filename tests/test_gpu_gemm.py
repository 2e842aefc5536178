"""GPU parity of mm / addmm / bmm: every route of b200_gemm against the CPU oracle."""

import pytest
import torch
from conftest import assert_parity

from oracle import ref_ops

pytestmark = pytest.mark.gpu

ROUTE_AUTO, ROUTE_SIMT, ROUTE_TC = 0, 1, 2


def gen(shape, dtype, seed, std=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * std).to(dtype)


@pytest.fixture(scope="module")
def ops():
    from torch_mojo_backend import ops as _ops

    return _ops


def cpu_gemm(a, b, bias=None, alpha=1.0, beta=1.0, out_dtype=None):
    """fp32 CPU matmul of the stored (possibly bf16-rounded) values: the oracle for big shapes."""
    y = alpha * (a.float() @ b.float())
    if bias is not None:
        y = y + beta * bias.float()
    return y.to(out_dtype or a.dtype)


# ---- exact-fp32 route ------------------------------------------------------------------------
def test_simt_golden_odd_shape(ops, golden):
    a, b, bias = (torch.from_numpy(golden[k]).cuda() for k in ("mm_a", "mm_b", "mm_bias"))
    assert_parity(ops.gemm(a, b), torch.from_numpy(golden["mm_y"]), bf16=False)
    y = ops.gemm(a, b, bias, None, 2.0, 0.5)
    assert_parity(y, torch.from_numpy(golden["addmm_y"]), bf16=False)
    yb = ops.gemm(torch.from_numpy(golden["bmm_a"]).cuda(), torch.from_numpy(golden["bmm_b"]).cuda())
    assert_parity(yb, torch.from_numpy(golden["bmm_y"]), bf16=False)


@pytest.mark.parametrize("ta", [False, True])
@pytest.mark.parametrize("tb", [False, True])
def test_simt_fp32_layouts(ops, ta, tb):
    m, n, k = 257, 130, 75
    a = gen((k, m) if ta else (m, k), torch.float32, 1)
    b = gen((n, k) if tb else (k, n), torch.float32, 2)
    a_cpu, a_gpu = (a.t(), a.cuda().t()) if ta else (a, a.cuda())
    b_cpu, b_gpu = (b.t(), b.cuda().t()) if tb else (b, b.cuda())
    assert_parity(ops.gemm(a_gpu, b_gpu), ref_ops.mm(a_cpu, b_cpu), bf16=False)


def test_simt_fp32_gpt2_shape_and_2d_bias(ops):
    a, b = gen((128, 768), torch.float32, 3), gen((768, 2304), torch.float32, 4, 0.02)
    bias = gen((2304,), torch.float32, 5, 0.02)
    assert_parity(ops.gemm(a.cuda(), b.cuda(), bias.cuda()), ref_ops.addmm(bias, a, b), bf16=False)
    bias2 = gen((128, 2304), torch.float32, 6)
    assert_parity(ops.gemm(a.cuda(), b.cuda(), bias2.cuda()), ref_ops.addmm(bias2, a, b), bf16=False)
    col = gen((128, 1), torch.float32, 7)
    assert_parity(ops.gemm(a.cuda(), b.cuda(), col.cuda()), ref_ops.addmm(col, a, b), bf16=False)


def test_simt_degenerate(ops):
    a = torch.empty((0, 8), device="cuda")
    b = torch.randn((8, 5), device="cuda")
    assert ops.gemm(a, b).shape == (0, 5)
    z = ops.gemm(torch.randn((4, 0), device="cuda"), torch.randn((0, 5), device="cuda"))
    assert torch.equal(z.cpu(), torch.zeros(4, 5))  # k == 0: empty sum
    one = ops.gemm(torch.full((1, 1), 3.0, device="cuda"), torch.full((1, 1), 4.0, device="cuda"))
    assert one.item() == 12.0


def test_simt_bf16_forced(ops):
    a, b = gen((100, 72), torch.bfloat16, 8), gen((72, 90), torch.bfloat16, 9)
    y = ops.gemm(a.cuda(), b.cuda(), None, None, 1.0, 1.0, 0, None, ROUTE_SIMT)
    assert_parity(y, cpu_gemm(a, b), bf16=True)


# ---- tensor-core route -----------------------------------------------------------------------
KN = [(768, 2304), (768, 768), (768, 3072), (3072, 768)]


@pytest.mark.parametrize("k,n", KN)
@pytest.mark.parametrize("b_layout", ["nk", "kn"])
def test_tcgen05_addmm_m8192(ops, k, n, b_layout):
    """M = 8192 GPT-2 shapes, both weight layouts: contiguous [K, N] (HF Conv1D) and the t() view
    of a contiguous [N, K] (nn.Linear)."""
    m = 8192
    a = gen((m, k), torch.bfloat16, 10)
    bias = gen((n,), torch.bfloat16, 12, 0.02)
    if b_layout == "nk":
        w = gen((n, k), torch.bfloat16, 11)
        b_cpu, b_gpu = w.t(), w.cuda().t()
    else:
        b_cpu = gen((k, n), torch.bfloat16, 11)
        b_gpu = b_cpu.cuda()
    y = ops.gemm(a.cuda(), b_gpu, bias.cuda(), None, 1.0, 1.0, 0, None, ROUTE_TC)
    want = cpu_gemm(a, b_cpu, bias)
    # reference's bf16 GEMM bar: atol 0.03125, rtol 0.02 on N(0,1) operands (tests/test_eager_kernels.py:5126-5129)
    torch.testing.assert_close(y.cpu(), want, atol=0.03125 * (k / 192) ** 0.5, rtol=0.02)
    y32 = ops.gemm(a.cuda(), b_gpu, bias.cuda(), None, 1.0, 1.0, 0, torch.float32, ROUTE_TC)
    assert y32.dtype == torch.float32
    assert_parity(y32, cpu_gemm(a, b_cpu, bias, out_dtype=torch.float32), bf16=False, scale=k**0.5 * 4)


@pytest.mark.parametrize("b_layout", ["nk", "kn"])
def test_lm_head_m8192_n50257(ops, b_layout):
    """The widest cell of the GEMM sweep, [8192, 768] x [768, 50257] in bf16 with fp32 logits: the
    tied-head layout (t() view of [N, K], the tensor-core route with a ragged last column tile and
    a padded output pitch) and a contiguous [K, N] weight (its 100514-byte row pitch cannot be
    described to TMA, so AUTO must fall to the strided CUDA-core kernel, never to a wrong answer).
    Rows from the first, a middle and the last row tile against the CPU oracle."""
    m, k, n = 8192, 768, 50257
    g = torch.Generator(device="cuda").manual_seed(81)
    a = torch.randn((m, k), generator=g, device="cuda").bfloat16()
    w = (torch.randn((n, k), generator=g, device="cuda") * 0.1).bfloat16()
    b_gpu = w.t() if b_layout == "nk" else w.t().contiguous()
    y = ops.gemm(a, b_gpu, None, None, 1.0, 1.0, 0, torch.float32)
    assert y.shape == (m, n) and y.dtype == torch.float32
    rows = torch.tensor([0, 1, 127, 128, 255, 256, 4095, 4096, 8063, 8064, 8191])
    want = a[rows.cuda()].float().cpu() @ w.float().cpu().t()
    assert_parity(y[rows.cuda()], want, bf16=False, scale=k**0.5 * 0.4)
    # bf16 output of the same product (the aten.mm contract for bf16 operands)
    yb = ops.gemm(a[:512], b_gpu)
    assert yb.dtype == torch.bfloat16
    assert_parity(yb, (a[:512].float().cpu() @ w.float().cpu().t()), bf16=True)


@pytest.mark.parametrize("m", [1, 16, 64])
@pytest.mark.parametrize("k,n", [(768, 2304), (768, 768), (768, 3072), (3072, 768), (768, 50257)])
@pytest.mark.parametrize("b_layout", ["nk", "kn"])
def test_decode_shapes_of_the_sweep(ops, m, k, n, b_layout):
    """M in {1, 16, 64} on every (K, N) of the GEMM sweep, both weight layouts, bias, route AUTO
    (whatever it resolves to: split-K, plain tensor-core or the strided kernel), bf16 and fp32
    results against the CPU oracle."""
    a = gen((m, k), torch.bfloat16, 90)
    bias = gen((n,), torch.bfloat16, 92, 0.02)
    if b_layout == "nk":
        w = gen((n, k), torch.bfloat16, 91, 0.1)
        b_cpu, b_gpu = w.t(), w.cuda().t()
    else:
        b_cpu = gen((k, n), torch.bfloat16, 91, 0.1)
        b_gpu = b_cpu.cuda()
    want = a.float() @ b_cpu.float() + bias.float()
    y32 = ops.gemm(a.cuda(), b_gpu, bias.cuda(), None, 1.0, 1.0, 0, torch.float32)
    assert_parity(y32, want, bf16=False)
    y16 = ops.gemm(a.cuda(), b_gpu, bias.cuda())
    assert y16.dtype == torch.bfloat16 and y16.shape == (m, n)
    assert_parity(y16, want, bf16=True)


@pytest.mark.parametrize("m", [1, 3, 16, 17, 64])
@pytest.mark.parametrize("k,n", [(768, 2304), (768, 768), (768, 3072), (3072, 768), (768, 50257)])
@pytest.mark.parametrize("b_layout", ["nk", "kn"])
def test_decode_shapes_of_the_sweep_fp32(ops, m, k, n, b_layout):
    """The fp32 half of the decode cells: M in {1, 16, 64} (and two ragged row counts) on every
    (K, N) of the sweep, both weight layouts, bias + residual, route AUTO; 1e-4 relative against an
    fp64 oracle."""
    a = gen((m, k), torch.float32, 93)
    bias, res = gen((n,), torch.float32, 95, 0.02), gen((m, n), torch.float32, 96)
    if b_layout == "nk":
        w = gen((n, k), torch.float32, 94, 0.1)
        b_cpu, b_gpu = w.t(), w.cuda().t()
    else:
        b_cpu = gen((k, n), torch.float32, 94, 0.1)
        b_gpu = b_cpu.cuda()
    want = (a.double() @ b_cpu.double() + bias.double() + res.double()).float()
    y = ops.gemm(a.cuda(), b_gpu, bias.cuda(), res.cuda())
    assert y.dtype == torch.float32 and y.shape == (m, n)
    assert_parity(y, want, bf16=False)


@pytest.mark.parametrize("m,n,k", [(1000, 50257, 768), (129, 200, 72), (33, 72, 200), (128, 256, 64), (300, 1000, 1600)])
def test_tcgen05_ragged(ops, m, n, k):
    a = gen((m, k), torch.bfloat16, 13)
    w = gen((n, k), torch.bfloat16, 14)
    y = ops.gemm(a.cuda(), w.cuda().t(), None, None, 1.0, 1.0, 0, torch.float32, ROUTE_TC)
    assert_parity(y, cpu_gemm(a, w.t(), out_dtype=torch.float32), bf16=False, scale=k**0.5 * 4)


@pytest.mark.parametrize("tile_n", [128, 192, 256])
@pytest.mark.parametrize("b_layout", ["nk", "kn"])
def test_tcgen05_every_tile_width(ops, monkeypatch, tile_n, b_layout):
    """Each tile width on a shape with ragged M, N and K tails, bias, gelu, fp32 residual."""
    monkeypatch.setenv("B200_GEMM_TILE_N", str(tile_n))
    m, n, k = 700, 1000, 328
    a = gen((m, k), torch.bfloat16, 40, 0.5)
    if b_layout == "nk":
        w = gen((n, k), torch.bfloat16, 41, 0.1)
        b_cpu, b_gpu = w.t(), w.cuda().t()
    else:
        b_cpu = gen((k, n), torch.bfloat16, 41, 0.1)
        b_gpu = b_cpu.cuda()
    bias = gen((n,), torch.bfloat16, 42)
    res = gen((m, n), torch.float32, 43)
    y = ops.gemm(a.cuda(), b_gpu, bias.cuda(), res.cuda(), 1.0, 1.0, 1, torch.float32, ROUTE_TC)
    want = torch.nn.functional.gelu(a.float() @ b_cpu.float() + bias.float(), approximate="tanh") + res
    assert_parity(y, want, bf16=False)
    # interior (branch-free) epilogue path: aligned pitch, full tiles
    m2, n2 = 512, 768
    a2, w2 = gen((m2, k), torch.bfloat16, 44, 0.5), gen((n2, k), torch.bfloat16, 45, 0.1)
    y2 = ops.gemm(a2.cuda(), w2.cuda().t(), bias[:n2].cuda(), None, 1.0, 1.0, 0, torch.bfloat16, ROUTE_TC)
    assert_parity(y2, a2.float() @ w2.float().t() + bias[:n2].float(), bf16=True)


@pytest.mark.parametrize("tile_n", [128, 192, 256])
def test_tcgen05_cta_pair_kernel(ops, monkeypatch, tile_n):
    """The CTA-pair kernel (two CTAs share a 256-row tile), forced on shapes it would not pick by
    itself: ragged tails in M (second CTA partly or wholly past the last row), N and K, bias +
    gelu + fp32 residual, batches; and bit-for-bit agreement with the single-CTA kernel."""
    monkeypatch.setenv("B200_GEMM_TILE_N", str(tile_n))
    for m, n, k in ((700, 1000, 328), (100, 520, 64), (1024, 768, 1600)):
        a = gen((m, k), torch.bfloat16, 50, 0.5)
        w = gen((n, k), torch.bfloat16, 51, 0.1)
        bias = gen((n,), torch.bfloat16, 52)
        res = gen((m, n), torch.float32, 53)
        outs = {}
        for pair in ("0", "1"):
            monkeypatch.setenv("B200_GEMM_PAIR", pair)
            outs[pair] = ops.gemm(a.cuda(), w.cuda().t(), bias.cuda(), res.cuda(), 1.0, 1.0, 1, torch.float32, ROUTE_TC)
        want = torch.nn.functional.gelu(a.float() @ w.float().t() + bias.float(), approximate="tanh") + res
        assert_parity(outs["1"], want, bf16=False)
        assert torch.equal(outs["0"], outs["1"])
    # batched, bf16 out
    monkeypatch.setenv("B200_GEMM_PAIR", "1")
    a3, w3 = gen((3, 300, 136), torch.bfloat16, 54, 0.5), gen((3, 200, 136), torch.bfloat16, 55, 0.1)
    y3 = ops.gemm(a3.cuda(), w3.cuda().transpose(1, 2), None, None, 1.0, 1.0, 0, torch.bfloat16, ROUTE_TC)
    assert_parity(y3, torch.bmm(a3.float(), w3.float().transpose(1, 2)), bf16=True)


@pytest.mark.parametrize("tile_n", [128, 256])
def test_tcgen05_cta_pair_kernel_mn_major_b(ops, monkeypatch, tile_n):
    """The CTA-pair kernel on a contiguous [K, N] weight (HF Conv1D layout): each CTA stages its half
    of the tile's columns as 64-column boxes. Forced on ragged shapes, with bias + gelu + fp32
    residual; bit-for-bit equal to the single-CTA kernel; and the default for large problems."""
    monkeypatch.setenv("B200_GEMM_TILE_N", str(tile_n))
    for m, n, k in ((700, 1000, 328), (100, 520, 64), (1024, 768, 1600), (512, 2304, 768)):
        a = gen((m, k), torch.bfloat16, 58, 0.5)
        b = gen((k, n), torch.bfloat16, 59, 0.1)
        bias = gen((n,), torch.bfloat16, 60)
        res = gen((m, n), torch.float32, 61)
        outs = {}
        for pair in ("0", "1"):
            monkeypatch.setenv("B200_GEMM_PAIR", pair)
            outs[pair] = ops.gemm(a.cuda(), b.cuda(), bias.cuda(), res.cuda(), 1.0, 1.0, 1, torch.float32, ROUTE_TC)
        want = torch.nn.functional.gelu(a.float() @ b.float() + bias.float(), approximate="tanh") + res
        assert_parity(outs["1"], want, bf16=False)
        assert torch.equal(outs["0"], outs["1"])
    monkeypatch.delenv("B200_GEMM_PAIR", raising=False)
    monkeypatch.delenv("B200_GEMM_TILE_N", raising=False)
    a, b = gen((2048, 512), torch.bfloat16, 62, 0.5), gen((512, 1536), torch.bfloat16, 63, 0.1)
    y = ops.gemm(a.cuda(), b.cuda(), None, None, 1.0, 1.0, 0, torch.bfloat16, ROUTE_TC)
    assert_parity(y, a.float() @ b.float(), bf16=True)


def test_tcgen05_cta_pair_kernel_is_the_default_for_large_problems(ops, monkeypatch):
    """Without any override a large K-major problem takes the pair kernel; its result must equal
    the single-CTA kernel's."""
    m, n, k = 2048, 1536, 512
    a, w = gen((m, k), torch.bfloat16, 56, 0.5), gen((n, k), torch.bfloat16, 57, 0.1)
    monkeypatch.delenv("B200_GEMM_PAIR", raising=False)
    y_default = ops.gemm(a.cuda(), w.cuda().t(), None, None, 1.0, 1.0, 0, torch.bfloat16, ROUTE_TC)
    monkeypatch.setenv("B200_GEMM_PAIR", "0")
    y_single = ops.gemm(a.cuda(), w.cuda().t(), None, None, 1.0, 1.0, 0, torch.bfloat16, ROUTE_TC)
    assert_parity(y_default, a.float() @ w.float().t(), bf16=True)
    assert torch.equal(y_default, y_single)


def test_tcgen05_epilogues(ops):
    m, n, k = 512, 640, 256
    a, w = gen((m, k), torch.bfloat16, 15, 0.5), gen((n, k), torch.bfloat16, 16, 0.1)
    bias = gen((n,), torch.float32, 17)
    res = gen((m, n), torch.float32, 18)
    acc = a.float() @ w.float().t()
    y = ops.gemm(a.cuda(), w.cuda().t(), bias.cuda(), res.cuda(), 0.5, 2.0, 1, torch.float32, ROUTE_TC)
    want = torch.nn.functional.gelu(0.5 * acc + 2.0 * bias, approximate="tanh") + res
    assert_parity(y, want, bf16=False)
    y2 = ops.gemm(a.cuda(), w.cuda().t(), bias.cuda(), None, 1.0, 1.0, 2, torch.bfloat16, ROUTE_TC)
    assert_parity(y2, torch.nn.functional.gelu(acc + bias), bf16=True)
    bias2 = gen((m, n), torch.bfloat16, 19)
    y3 = ops.gemm(a.cuda(), w.cuda().t(), bias2.cuda(), None, 1.0, 1.0, 0, None, ROUTE_TC)
    assert_parity(y3, acc + bias2.float(), bf16=True)


@pytest.mark.parametrize("shape", [((12, 128, 64), (12, 64, 128), True), ((12, 128, 128), (12, 128, 64), False),
                                   ((5, 200, 72), (5, 72, 136), False)])
def test_tcgen05_bmm(ops, shape):
    """bmm shapes of the decomposed attention: Q K^T (B as a transposed view) and P V."""
    sa, sb, b_transposed = shape
    a = gen(sa, torch.bfloat16, 20)
    if b_transposed:
        bt = gen((sb[0], sb[2], sb[1]), torch.bfloat16, 21)
        b_cpu, b_gpu = bt.transpose(1, 2), bt.cuda().transpose(1, 2)
    else:
        b_cpu = gen(sb, torch.bfloat16, 21)
        b_gpu = b_cpu.cuda()
    y = ops.gemm(a.cuda(), b_gpu, None, None, 1.0, 1.0, 0, torch.float32, ROUTE_TC)
    assert_parity(y, torch.bmm(a.float(), b_cpu.float()), bf16=False, scale=sa[2] ** 0.5 * 4)


ROUTE_SKINNY = 3


@pytest.mark.parametrize("m", [1, 16, 64, 100])
@pytest.mark.parametrize("k,n,b_layout", [(6400, 1600, "nk"), (3072, 768, "kn"), (1600, 1600, "nk")])
def test_small_m_split_k_route(ops, m, k, n, b_layout):
    """Decode shapes: K is split across CTAs into a scratch buffer and reduced in a fixed order.
    Checked against the oracle, against the unsplit tensor-core route, and for run-to-run
    bitwise determinism."""
    import ctypes

    from torch_mojo_backend import native

    a = gen((m, k), torch.bfloat16, 50, 0.5)
    if b_layout == "nk":
        w = gen((n, k), torch.bfloat16, 51, 0.1)
        b_cpu, b_gpu = w.t(), w.cuda().t()
    else:
        b_cpu = gen((k, n), torch.bfloat16, 51, 0.1)
        b_gpu = b_cpu.cuda()
    bias = gen((n,), torch.bfloat16, 52)
    res = gen((m, n), torch.float32, 53)
    ag = a.cuda()
    c = torch.empty((m, n), dtype=torch.float32, device="cuda")
    g = ops.fill_gemm_args(ag, b_gpu, bias.cuda(), res.cuda(), c, 1.0, 1.0, 1, 0)
    auto = native.lib().b200_gemm_route(ctypes.byref(g))
    need = native.lib().b200_gemm_workspace_bytes(ctypes.byref(g))
    # up to eight rows against a K-contiguous weight: partial sums, their sum and the epilogue are one
    # launch (the slices of a column block form a cluster) and nothing is written to scratch
    one_launch = auto == ROUTE_SKINNY and m <= 8 and b_layout == "nk"
    assert (auto == ROUTE_SKINNY and not one_launch) == (need > 0)
    want = torch.nn.functional.gelu(a.float() @ b_cpu.float() + bias.float(), approximate="tanh") + res
    y = ops.gemm(ag, b_gpu, bias.cuda(), res.cuda(), 1.0, 1.0, 1, torch.float32)
    assert_parity(y, want, bf16=False)
    if auto == ROUTE_SKINNY:
        y_again = ops.gemm(ag, b_gpu, bias.cuda(), res.cuda(), 1.0, 1.0, 1, torch.float32)
        assert torch.equal(y, y_again), "fixed-order reduction must be bitwise reproducible"
        y_tc = ops.gemm(ag, b_gpu, bias.cuda(), res.cuda(), 1.0, 1.0, 1, torch.float32, ROUTE_TC)
        assert_parity(y, y_tc, bf16=False)
        # a missing workspace is an error, not a silent reroute
        st = native.lib().b200_gemm(ctypes.byref(g), None, 0, None)
        assert st == (0 if one_launch else -4)


def test_auto_route_choices(ops):
    import ctypes

    from torch_mojo_backend import native

    def route(a, b):
        c = torch.empty((a.shape[0], b.shape[1]), dtype=a.dtype, device="cuda")
        g = ops.fill_gemm_args(a, b, None, None, c, 1.0, 1.0, 0, 0)
        return native.lib().b200_gemm_route(ctypes.byref(g))

    bf = torch.bfloat16
    assert route(torch.empty((256, 64), dtype=bf, device="cuda"), torch.empty((64, 256), dtype=bf, device="cuda")) == ROUTE_TC
    assert route(torch.empty((256, 64), device="cuda"), torch.empty((64, 256), device="cuda")) == ROUTE_SIMT
    # K-contiguity / 16-byte pitch rules of the TMA route
    assert route(torch.empty((256, 60), dtype=bf, device="cuda"), torch.empty((60, 256), dtype=bf, device="cuda")) == ROUTE_SIMT
    # a transposed A (m contiguous, the operand of a weight gradient) is taken as it lies when its pitch is 16-byte
    assert route(torch.empty((64, 256), dtype=bf, device="cuda").t(), torch.empty((64, 256), dtype=bf, device="cuda")) == ROUTE_TC
    assert route(torch.empty((64, 252), dtype=bf, device="cuda").t(), torch.empty((64, 256), dtype=bf, device="cuda")) == ROUTE_SIMT
    assert route(torch.empty((64, 512), dtype=bf, device="cuda")[:, ::2].t(), torch.empty((64, 256), dtype=bf, device="cuda")) == ROUTE_SIMT


def test_forced_route_refused_loudly(ops):
    a, b = torch.randn((8, 8), device="cuda"), torch.randn((8, 8), device="cuda")
    with pytest.raises(RuntimeError, match="tcgen05 route refused"):
        ops.gemm(a, b, None, None, 1.0, 1.0, 0, None, ROUTE_TC)


def test_no_device_timeout_recorded():
    from torch_mojo_backend import native

    assert native.device_status() == 0


ROUTE_SPLIT3 = 4


@pytest.mark.parametrize("k,n", KN)
@pytest.mark.parametrize("b_layout", ["nk", "kn"])
def test_fp32_m8192_split_precision_route(ops, k, n, b_layout):
    """fp32 operands at M = 8192 on the four (K, N) of the sweep, both weight layouts, bias: AUTO
    resolves to the split-precision tensor-core route (operands as bf16 hi / lo halves, three products
    accumulated in fp32 by one tensor-core launch) and must meet the fp32 bar, 1e-4 relative,
    against an fp64 oracle; the exact CUDA-core route must agree with it to the same bar."""
    import ctypes

    from torch_mojo_backend import native

    m = 8192
    g = torch.Generator(device="cuda").manual_seed(100)
    a = torch.randn((m, k), generator=g, device="cuda")
    bias = torch.randn((n,), generator=g, device="cuda") * 0.02
    w = torch.randn((n, k) if b_layout == "nk" else (k, n), generator=g, device="cuda")
    b = w.t() if b_layout == "nk" else w
    c = torch.empty((m, n), device="cuda")
    args = ops.fill_gemm_args(a, b, bias, None, c, 1.0, 1.0, 0, 0)
    assert native.lib().b200_gemm_route(ctypes.byref(args)) == ROUTE_SPLIT3
    assert native.lib().b200_gemm_workspace_bytes(ctypes.byref(args)) >= (m + n) * 2 * k * 2
    y = ops.gemm(a, b, bias)
    assert y.dtype == torch.float32
    want = torch.addmm(bias.double(), a.double(), b.double())
    scale = want.abs().max().item()
    err = (y.double() - want).abs().max().item()
    assert err <= 1e-4 * scale, f"max|diff| {err:.3e} at scale {scale:.3e}"
    rows = slice(0, 512)
    exact = ops.gemm(a[rows], b, bias, None, 1.0, 1.0, 0, None, ROUTE_SIMT)
    assert (exact.double() - want[rows]).abs().max().item() <= 1e-4 * scale
    # a missing workspace is an error, not a silent reroute
    assert native.lib().b200_gemm(ctypes.byref(args), None, 0, None) == -4


@pytest.mark.parametrize("m,n,k", [(257, 130, 75), (1000, 1000, 333), (300, 50257, 768), (4096, 33, 4096)])
@pytest.mark.parametrize("ta,tb", [(False, False), (False, True), (True, False)])
def test_fp32_split_precision_odd_shapes_and_layouts(ops, m, n, k, ta, tb):
    """Forced split-precision route on ragged extents (K not a multiple of the 64-element k-block,
    unaligned pitches, the 50257-column logits) and on transposed views of either operand, with
    alpha / beta / gelu / residual in the epilogue."""
    a = gen((k, m) if ta else (m, k), torch.float32, 110)
    b = gen((n, k) if tb else (k, n), torch.float32, 111, 0.1)
    a_cpu, a_gpu = (a.t(), a.cuda().t()) if ta else (a, a.cuda())
    b_cpu, b_gpu = (b.t(), b.cuda().t()) if tb else (b, b.cuda())
    bias, res = gen((n,), torch.float32, 112), gen((m, n), torch.float32, 113)
    y = ops.gemm(a_gpu, b_gpu, bias.cuda(), res.cuda(), 0.5, 2.0, 1, None, ROUTE_SPLIT3)
    acc = 0.5 * (a_cpu.double() @ b_cpu.double()) + 2.0 * bias.double()
    want = torch.nn.functional.gelu(acc, approximate="tanh") + res.double()
    assert_parity(y, want.float(), bf16=False)


@pytest.mark.parametrize("level,rtol", [("highest", 1e-4), ("high", 1e-4), ("medium", 2e-2)])
def test_fp32_matmul_precision_levels(level, rtol):
    """fp32 mm / addmm through the lowering: "highest" and "high" meet the fp32 bar (on the tensor
    cores, in split precision, for a product of this size), "medium" rounds the operands to bf16;
    one GEMM call either way."""
    from torch_mojo_backend import aten_functions as af
    from torch_mojo_backend import native

    m, k, n = 1024, 768, 1536
    a, w, bias = gen((m, k), torch.float32, 70), gen((n, k), torch.float32, 71, 0.05), gen((n,), torch.float32, 72)
    want = torch.addmm(bias.double(), a.double(), w.double().t()).float()
    old = torch.get_float32_matmul_precision()
    try:
        torch.set_float32_matmul_precision(level)
        before = native.launch_count
        got = af.aten_addmm(bias.cuda(), a.cuda(), w.cuda().t())
        launches = native.launch_count - before
        got_mm = af.aten_mm(a.cuda(), w.cuda().t())
    finally:
        torch.set_float32_matmul_precision(old)
    assert launches == 1
    assert got.dtype == torch.float32
    scale = want.abs().max().item()
    assert (got.cpu() - want).abs().max().item() <= rtol * scale
    assert (got_mm.cpu() - (want - bias)).abs().max().item() <= rtol * scale


def test_tcgen05_output_beyond_2_31_elements(ops):
    """LM-head shape at the benchmark's largest forward: [65536, 64] x [64, 50257] -> fp32 logits,
    3.3e9 output elements (13 GB), so every output offset that is not computed in 64 bits wraps.
    Checked on rows from the first, a middle and the last tile against the CPU oracle."""
    m, k, n = 65536, 64, 50257
    g = torch.Generator(device="cuda").manual_seed(80)
    a = torch.randn((m, k), generator=g, device="cuda").bfloat16()
    w = (torch.randn((n, k), generator=g, device="cuda") * 0.1).bfloat16()
    y = ops.gemm(a, w.t(), None, None, 1.0, 1.0, 0, torch.float32, ROUTE_TC)
    assert y.shape == (m, n) and y.dtype == torch.float32
    rows = torch.tensor([0, 1, 127, 128, 255, 256, 32767, 32768, 42719, 65279, 65280, 65535])
    want = a[rows.cuda()].float().cpu() @ w.float().cpu().t()
    assert_parity(y[rows.cuda()], want, bf16=False, scale=k**0.5 * 0.4)
    del y
    torch.cuda.empty_cache()
