"""GPU parity of the row kernels against the CPU oracle, through torch.ops.b200 -> C ABI."""

import json

import pytest
import torch
import torch.nn.functional as F
from conftest import GOLDEN_DIR, assert_parity

from oracle import ref_ops

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


def gen(shape, dtype, seed=0, mean=0.0, std=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * std + mean).to(dtype)


@pytest.fixture(scope="module")
def ops():
    from torch_mojo_backend import ops as _ops

    return _ops


# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", [(8192, 768), (8192, 1600), (33, 40), (5, 7), (3, 5000), (2, 3, 64), (1, 8)])
def test_layer_norm(ops, dtype, shape):
    cols = shape[-1]
    x = gen(shape, dtype, 1)
    w = gen((cols,), dtype, 2, mean=1.0, std=0.02)
    b = gen((cols,), dtype, 3, std=0.02)
    y, mean, rstd = ops.layer_norm(x.cuda(), w.cuda(), b.cuda(), 1e-5)
    ry, rmean, rrstd = ref_ops.layer_norm(x, [cols], w, b, 1e-5)
    assert y.dtype == dtype and mean.dtype == torch.float32
    assert_parity(y, ry, bf16=dtype == torch.bfloat16, what="y")
    assert_parity(mean, rmean.reshape(mean.shape), bf16=False, scale=1.0, what="mean")
    assert_parity(rstd, rrstd.reshape(rstd.shape), bf16=False, what="rstd")


def test_layer_norm_mixed_dtypes_and_no_affine(ops):
    x = gen((257, 768), torch.float32, 5)
    w = gen((768,), torch.float32, 6, mean=1.0, std=0.02)
    b = gen((768,), torch.float32, 7, std=0.02)
    y, _, _ = ops.layer_norm(x.cuda(), w.cuda(), b.cuda(), 1e-5, torch.bfloat16)
    assert y.dtype == torch.bfloat16
    assert_parity(y, ref_ops.layer_norm(x, [768], w, b, 1e-5, torch.bfloat16)[0], bf16=True)
    y2, _, _ = ops.layer_norm(x.cuda(), None, None, 1e-3)
    assert_parity(y2, ref_ops.layer_norm(x, [768], None, None, 1e-3)[0], bf16=False)
    xb = x.bfloat16()
    y3, _, _ = ops.layer_norm(xb.cuda(), w.cuda(), b.cuda(), 1e-5, torch.float32)  # bf16 in, fp32 params/out
    assert_parity(y3, ref_ops.layer_norm(xb, [768], w, b, 1e-5, torch.float32)[0], bf16=False)


def test_layer_norm_strided_rows_and_nonfinite(ops):
    big = gen((64, 1024), torch.float32, 8).cuda()
    view = big[:, :768]  # row stride 1024, 768 columns
    y, _, _ = ops.layer_norm(view, None, None, 1e-5)
    assert_parity(y, ref_ops.layer_norm(view.cpu(), [768], None, None, 1e-5)[0], bf16=False)
    x = gen((4, 64), torch.float32, 9)
    x[1, 3] = float("inf")
    x[2, 5] = float("nan")
    y, mean, rstd = ops.layer_norm(x.cuda(), None, None, 1e-5)
    # non-finite rows give NaN statistics and outputs; other rows are untouched
    assert torch.isnan(y[1]).all() and torch.isnan(y[2]).all() and torch.isnan(rstd[1]) and torch.isnan(mean[2])
    assert_parity(y[[0, 3]], ref_ops.layer_norm(x[[0, 3]], [64], None, None, 1e-5)[0], bf16=False)


def test_layer_norm_golden(ops, golden):
    x, w, b = (torch.from_numpy(golden[k]) for k in ("ln_x", "ln_w", "ln_b"))
    y, mean, rstd = ops.layer_norm(x.cuda(), w.cuda(), b.cuda(), 1e-5)
    assert_parity(y, torch.from_numpy(golden["ln_y"]), bf16=False)
    assert_parity(mean, torch.from_numpy(golden["ln_mean"]).reshape(-1), bf16=False, scale=1.0)
    assert_parity(rstd, torch.from_numpy(golden["ln_rstd"]).reshape(-1), bf16=False)


# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", [(8, 1024, 1024), (3, 5, 7), (4, 33, 2048), (2, 5000), (7, 1)])
def test_softmax(ops, dtype, shape):
    x = gen(shape, dtype, 11, std=3.0)
    y = ops.softmax(x.cuda())
    assert y.dtype == dtype
    assert_parity(y, ref_ops.softmax(x, -1), bf16=dtype == torch.bfloat16, scale=1.0)


def test_softmax_half_to_float_and_minus_inf(ops):
    x = gen((16, 256), torch.bfloat16, 12)
    y = ops.softmax(x.cuda(), 1.0, False, 0, torch.float32)
    assert y.dtype == torch.float32
    assert_parity(y, ref_ops.softmax(x, -1, torch.float32), bf16=False, scale=1.0)
    # pre-masked input, as the traced masked_fill -> _softmax graph produces it
    s = gen((2, 64, 64), torch.float32, 13)
    mask = torch.tril(torch.ones(64, 64, dtype=torch.bool))
    sm = s.masked_fill(~mask, float("-inf"))
    y = ops.softmax(sm.cuda())
    assert_parity(y, ref_ops.softmax(sm, -1), bf16=False, scale=1.0)
    assert (y.cpu().triu(1) == 0).all()
    allinf = torch.full((2, 8), float("-inf"))
    assert torch.isnan(ops.softmax(allinf.cuda())).all()  # same as torch for a fully masked row


@pytest.mark.parametrize("dtype", DTYPES)
def test_softmax_fused_scale_causal(ops, dtype):
    B, T = 6, 128
    x = gen((B, T, T), dtype, 14, std=2.0)
    y = ops.softmax(x.cuda(), 0.125, True, T)
    want = ref_ops.softmax_rows(x, scale=0.125, causal=True, q_len=T)
    assert_parity(y, want, bf16=dtype == torch.bfloat16, scale=1.0)
    assert (y.float().cpu().triu(1) == 0).all(), "masked columns must be exact zeros"
    # kv longer than q (cols > q_len) and the vectorised oracle as an independent check
    x2 = gen((2, 16, 40), dtype, 15)
    y2 = ops.softmax(x2.cuda(), 1.0, True, 16)
    assert_parity(y2, ref_ops.softmax_rows(x2, causal=True, q_len=16), bf16=dtype == torch.bfloat16, scale=1.0)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("cols,offset", [(64, 0), (200, 0), (77, 0), (128, 3)])
def test_softmax_masked(ops, dtype, cols, offset):
    """scale -> masked_fill -> softmax in one kernel: a [T, S] mask shared by batch and heads, read
    as a strided slice of a larger buffer (with an odd byte offset it takes the scalar kernel),
    both polarities, -inf and finite fills; oracle = the unfused chain in fp64."""
    B, H, T = 2, 3, 40
    x = gen((B, H, T, cols), dtype, 17, std=2.0)
    g = torch.Generator().manual_seed(18)
    buf = torch.rand(1, 1, 64, 256, generator=g) > 0.4
    buf[..., offset] = False  # at least one visible key per row
    mask = buf[:, :, :T, offset : offset + cols]
    for fill in (float("-inf"), -3.0):
        want = torch.softmax((x.double() * 0.3).masked_fill(mask, fill), -1).to(dtype)
        y = ops.softmax_masked(x.cuda(), buf.cuda()[:, :, :T, offset : offset + cols], fill, 0.3, False)
        assert y.dtype == dtype
        assert_parity(y, want, bf16=dtype == torch.bfloat16, scale=1.0)
        if fill == float("-inf"):
            assert (y.cpu().float().masked_select(mask.expand_as(x)) == 0).all()
        keep = ~mask
        y2 = ops.softmax_masked(x.cuda(), keep.contiguous().cuda(), fill, 0.3, True)
        # (the dense `keep` may take the vector kernel where the offset slice took the scalar one)
        assert_parity(y2, want, bf16=dtype == torch.bfloat16, scale=1.0)
        if offset == 0:
            assert torch.equal(y2, y), "where(keep, x, fill) form must agree with masked_fill(mask, fill)"
    # row-broadcast mask [S] and the rejection of a mask that varies over heads
    m1 = buf[0, 0, 0, :cols]
    y3 = ops.softmax_masked(x.cuda(), m1.cuda(), float("-inf"), 1.0, False)
    assert_parity(y3, torch.softmax(x.double().masked_fill(m1, float("-inf")), -1).to(dtype), bf16=dtype == torch.bfloat16, scale=1.0)
    with pytest.raises(ValueError, match="not one"):
        ops.softmax_masked(x.cuda(), mask.expand(1, H, T, cols).contiguous().cuda(), 0.0, 1.0, False)


@pytest.mark.parametrize("dtype", DTYPES)
def test_softmax_full_size_properties(ops, dtype):
    """Scores of 8 batch x 12 heads x 1024 x 1024 with the strict upper triangle at -inf: rows sum
    to one, masked entries are exact zeros, and a slice matches the oracle."""
    g = torch.Generator(device="cuda").manual_seed(16)
    x = torch.randn((96, 1024, 1024), generator=g, device="cuda", dtype=torch.float32).to(dtype)
    mask = torch.ones(1024, 1024, dtype=torch.bool, device="cuda").tril()
    x.masked_fill_(~mask, float("-inf"))
    y = ops.softmax(x)
    sums = y.float().sum(-1)
    tol = 2e-2 if dtype == torch.bfloat16 else 1e-4
    assert (sums - 1).abs().max().item() < tol
    assert (y.masked_select(~mask) == 0).all()
    assert_parity(y[5, 100:164], ref_ops.softmax(x[5, 100:164].cpu(), -1), bf16=dtype == torch.bfloat16, scale=1.0)
    fused = ops.softmax(torch.where(mask, x, torch.zeros_like(x)), 1.0, True, 1024)
    assert torch.equal(fused, y), "fused causal form must agree bit for bit with the pre-masked form"


# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("approximate", ["none", "tanh"])
@pytest.mark.parametrize("shape", [(8192, 3072), (257,), (3, 5, 7), (1,)])
def test_gelu(ops, dtype, approximate, shape):
    x = gen(shape, dtype, 21, std=2.0)
    y = ops.gelu(x.cuda(), approximate)
    assert y.dtype == dtype and y.shape == x.shape
    want = F.gelu(x.float(), approximate=approximate).to(dtype) if x.numel() > 100000 else ref_ops.gelu(x, approximate)
    assert_parity(y, want, bf16=dtype == torch.bfloat16)


@pytest.mark.parametrize("approximate", ["none", "tanh"])
def test_gelu_reference_known_answers(ops, approximate):
    """The reference's frozen bf16 bit patterns (tests/test_eager_kernels.py:1998-2032)."""
    ka = json.loads((GOLDEN_DIR / "gelu_bf16_known_answers.json").read_text())
    bits = torch.tensor([int(b, 16) for b in ka["input_bits"]], dtype=torch.int32).to(torch.uint16)
    x = bits.view(torch.bfloat16)
    # once through the vector kernel (padded to a full 16-byte vector) and once through the scalar tail
    for pad in (16 - len(bits), 0):
        xin = torch.cat([x, torch.zeros(pad, dtype=torch.bfloat16)]).cuda()
        y = ops.gelu(xin, approximate).cpu()[: len(bits)]
        yb = y.view(torch.uint16)
        assert int(yb[0]) == 0x0000 and int(yb[1]) == 0x8000
        assert torch.isposinf(y[2]) and torch.isnan(y[3]) and torch.isnan(y[4])
        probes = [hex(int(yb[i])) for i in ka["probe_indices"]]
        assert probes == [b.lower() for b in ka["probe_bits"][approximate]], probes
        assert torch.equal(xin.cpu()[: len(bits)].view(torch.uint16), bits), "input must be untouched"


@pytest.mark.parametrize("approximate", ["none", "tanh"])
def test_gelu_bf16_every_bit_pattern(ops, approximate):
    """All 65536 bf16 inputs against the formula evaluated in float64 and rounded once: the kernel's
    approximations (MUFU ex2 / rcp, the erfc fit of the erf form) must land on the correctly rounded
    bf16 value nearly everywhere and never more than one bf16 step away; NaN and infinity classes must
    agree. Inputs whose exact result is subnormal, and the left tail where the float64 formula itself
    cancels (x < -5.5), are held to an absolute bound instead."""
    bits = torch.arange(65536, dtype=torch.int32).to(torch.uint16)
    x = bits.view(torch.bfloat16)
    got = ops.gelu(x.cuda(), approximate).cpu()
    assert torch.equal(x.view(torch.uint16), bits)
    xd = x.double()
    want64 = F.gelu(xd, approximate=approximate)
    want = want64.to(torch.bfloat16)
    finite_in = torch.isfinite(xd)
    assert torch.equal(torch.isnan(got), torch.isnan(want))
    assert torch.equal(torch.isposinf(got), torch.isposinf(want))
    body = finite_in & (xd > -5.5) & (want64.abs() >= 2.0**-120) & torch.isfinite(want.float())
    gb = got.view(torch.int16).to(torch.int32)[body]
    wb = want.view(torch.int16).to(torch.int32)[body]
    steps = (gb - wb).abs()
    assert int(steps.max()) <= 1, f"{int((steps > 1).sum())} results more than one bf16 step off"
    assert float((steps == 0).double().mean()) >= 0.999
    rest = finite_in & ~body
    assert float((got.double()[rest] - want64[rest]).abs().max()) < 1e-9


def test_gelu_unaligned_offset(ops):
    base = gen((1000,), torch.float32, 22).cuda()
    x = base[3:900]  # 12-byte offset: vector path must not be taken blindly
    assert_parity(ops.gelu(x, "tanh"), ref_ops.gelu(x.cpu(), "tanh"), bf16=False)


# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("op,name", [(0, "sum"), (1, "mean"), (2, "amax")])
@pytest.mark.parametrize("shape", [(8192, 768), (33, 65), (4, 6, 9), (2, 70000), (600, 4)])
def test_reduce_lastdim(ops, dtype, op, name, shape):
    x = gen(shape, dtype, 31)
    y = ops.reduce(x.cuda(), op)
    want = ref_ops.reduce(x, name, -1)
    assert y.dtype == dtype and y.shape == want.shape
    scale = {"sum": shape[-1] ** 0.5, "mean": 1.0, "amax": 4.0}[name]
    assert_parity(y, want, bf16=dtype == torch.bfloat16, scale=scale)


def test_reduce_nan_and_empty(ops):
    x = gen((600, 16), torch.float32, 32)
    x[7, 3] = float("nan")
    assert torch.isnan(ops.reduce(x.cuda(), 2)[7])  # amax propagates NaN like torch.amax
    assert ops.reduce(torch.empty((0, 5), device="cuda"), 0).shape == (0,)
    assert torch.equal(ops.reduce(torch.empty((3, 0), device="cuda"), 0).cpu(), torch.zeros(3))


def test_no_device_timeout_recorded():
    from torch_mojo_backend import native

    assert native.device_status() == 0
