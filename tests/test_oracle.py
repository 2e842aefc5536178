"""Pins the CPU oracle: against the golden vectors generated from PyTorch CPU eager, against live
PyTorch CPU eager on fresh seeds, and against the reference's bf16 GELU known answers."""

import json

import pytest
import torch
import torch.nn.functional as F
from conftest import GOLDEN_DIR

from oracle import ref_ops


def t(a, dtype=torch.float32):
    return torch.from_numpy(a).to(dtype)


def close(a, b, atol=1e-6, rtol=1e-5):
    torch.testing.assert_close(a, b, atol=atol, rtol=rtol)


def bf16_one_ulp(got, want):
    """bf16 results of "widen, compute, round once" agree within one bf16 ulp (2^-7 relative);
    values that underflow in fp32 but not in fp64 differ by a denormal-sized absolute amount."""
    assert got.dtype == want.dtype == torch.bfloat16
    torch.testing.assert_close(got.float(), want.float(), rtol=2.0**-7, atol=1e-6, equal_nan=True)


def test_layer_norm_golden(golden):
    y, mean, rstd = ref_ops.layer_norm(t(golden["ln_x"]), [40], t(golden["ln_w"]), t(golden["ln_b"]), 1e-5)
    close(y, t(golden["ln_y"]), atol=2e-6)
    close(mean, t(golden["ln_mean"]))
    close(rstd, t(golden["ln_rstd"]), rtol=1e-5)
    y2, mean2, rstd2 = ref_ops.layer_norm(t(golden["ln2_x"]), [4, 10], None, None, 1e-3)
    close(y2, t(golden["ln2_y"]), atol=2e-6)
    assert mean2.shape == (3, 1, 1) and rstd2.shape == (3, 1, 1)
    close(mean2, t(golden["ln2_mean"]))
    close(rstd2, t(golden["ln2_rstd"]))


def test_softmax_golden(golden):
    x = t(golden["sm_x"])
    for d in range(3):
        close(ref_ops.softmax(x, d), t(golden[f"sm_y{d}"]))
    # causal + scale fused form against masked_fill -> softmax
    got = ref_ops.softmax_rows(t(golden["csm_x"]), scale=0.25, causal=True, q_len=8)
    close(got, t(golden["csm_y"]))
    assert (got.triu(1) == 0).all(), "masked columns must be exact zeros"


def test_softmax_rows_q_len_wraps():
    x = torch.randn(6, 4, generator=torch.Generator().manual_seed(3))
    got = ref_ops.softmax_rows(x, causal=True, q_len=3)  # rows 0..2 and 3..5 are two query blocks
    mask = torch.tril(torch.ones(3, 4, dtype=torch.bool)).repeat(2, 1)
    want = torch.softmax(x.masked_fill(~mask, float("-inf")), -1)
    close(got, want)


@pytest.mark.parametrize("approximate", ["none", "tanh"])
def test_gelu_golden(golden, approximate):
    close(ref_ops.gelu(t(golden["gelu_x"]), approximate), t(golden[f"gelu_{approximate}"]), atol=1e-6)
    xb = t(golden["gelu_bf16_x"], torch.bfloat16)
    want = t(golden[f"gelu_bf16_{approximate}"], torch.bfloat16)
    got = ref_ops.gelu(xb, approximate)
    bf16_one_ulp(got, want)


@pytest.mark.parametrize("approximate", ["none", "tanh"])
def test_gelu_reference_known_answers(approximate):
    """Bit patterns asserted by the reference (tests/test_eager_kernels.py:1998-2032), checked on
    both the oracle restatement and PyTorch CPU eager."""
    ka = json.loads((GOLDEN_DIR / "gelu_bf16_known_answers.json").read_text())
    bits = torch.tensor([int(b, 16) for b in ka["input_bits"]], dtype=torch.int32).to(torch.uint16)
    x = bits.view(torch.bfloat16)
    for name, fn in (("oracle", lambda v: ref_ops.gelu(v, approximate)),
                     ("torch", lambda v: F.gelu(v, approximate=approximate))):
        y = fn(x)
        yb = y.view(torch.uint16)
        assert int(yb[0]) == 0x0000, name
        assert int(yb[1]) == 0x8000, name
        if name == "oracle" or approximate == "tanh":
            # PyTorch's CPU erf kernel returns NaN for gelu(+inf); the reference's frozen answer
            # (and the formula 0.5 * inf * (1 + 1)) is +inf, which the restatement follows.
            assert torch.isposinf(y[2]), name
        assert torch.isnan(y[3]) and torch.isnan(y[4]), name
        probes = tuple(int(yb[i]) for i in ka["probe_indices"])
        assert probes == tuple(int(b, 16) for b in ka["probe_bits"][approximate]), (name, [hex(p) for p in probes])


def test_reductions_golden(golden):
    x = t(golden["red_x"])
    close(ref_ops.reduce(x, "sum", -1), t(golden["red_sum_last"]), atol=1e-5)
    close(ref_ops.reduce(x, "mean", (0, 1)), t(golden["red_mean_01"]))
    close(ref_ops.reduce(x, "amax", 1, keepdim=True), t(golden["red_amax_1k"]))
    close(ref_ops.reduce(x, "sum"), t(golden["red_sum_all"]), atol=1e-4)


def test_gemm_family_golden(golden):
    a, b, bias = t(golden["mm_a"]), t(golden["mm_b"]), t(golden["mm_bias"])
    close(ref_ops.mm(a, b), t(golden["mm_y"]), atol=1e-5)
    close(ref_ops.addmm(bias, a, b, beta=0.5, alpha=2.0), t(golden["addmm_y"]), atol=1e-5)
    close(ref_ops.bmm(t(golden["bmm_a"]), t(golden["bmm_b"])), t(golden["bmm_y"]), atol=1e-5)


@pytest.mark.parametrize("kv", [6, 10, 64])
def test_sdpa_golden(golden, kv):
    q, k, v = (t(golden[f"sdpa{kv}_{n}"]) for n in "qkv")
    out, lse = ref_ops.sdpa(q, k, v, causal=True)
    close(out, t(golden[f"sdpa{kv}_causal"]), atol=2e-6)
    out_full, _ = ref_ops.sdpa(q, k, v, causal=False)
    close(out_full, t(golden[f"sdpa{kv}_full"]), atol=2e-6)
    # lse is the natural log of the softmax denominator of the scaled, masked scores
    s = (q @ k.transpose(-1, -2)) / 4.0
    s = s.masked_fill(~torch.tril(torch.ones(kv, kv, dtype=torch.bool)), float("-inf"))
    close(lse, torch.logsumexp(s, -1), atol=1e-5)


@pytest.mark.parametrize("seed", [0, 1])
def test_oracle_matches_torch_eager_on_fresh_inputs(seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(17, 96, generator=g)
    w, b = torch.randn(96, generator=g), torch.randn(96, generator=g)
    close(ref_ops.layer_norm(x, [96], w, b, 1e-5)[0], F.layer_norm(x, (96,), w, b, 1e-5), atol=3e-6)
    close(ref_ops.softmax(x, -1), torch.softmax(x, -1))
    close(ref_ops.gelu(x, "tanh"), F.gelu(x, approximate="tanh"), atol=1e-6)
    xb = x.to(torch.bfloat16)
    # bf16 in, fp32 math, bf16 out
    got = ref_ops.layer_norm(xb, [96], w.bfloat16(), b.bfloat16(), 1e-5)[0]
    want = F.layer_norm(xb.float(), (96,), w.bfloat16().float(), b.bfloat16().float(), 1e-5).bfloat16()
    bf16_one_ulp(got, want)


@pytest.mark.parametrize("attention", ["sdpa", "masked_softmax"])
def test_gpt2_tiny_golden(golden, attention):
    """The model definition is deterministic from its seed, and the whole-model oracle (fp32 CPU
    eager of the device model's parameter values) reproduces the stored logits."""
    from demo_scripts.gpt2 import GPT2, GPTConfig

    cfg = GPTConfig(vocab_size=211, block_size=32, n_layer=2, n_head=4, n_embd=64)
    ids = torch.from_numpy(golden["gpt_ids"])
    model = GPT2(cfg, attention).init_weights(0).eval()
    close(ref_ops.gpt2_logits_fp32(model, ids), t(golden[f"gpt_logits_{attention}"]), atol=1e-5)
    # bf16 policy: oracle uses the bf16-rounded weights in fp32 math
    model.set_precision("bf16")
    ref = ref_ops.gpt2_logits_fp32(model, ids)
    assert ref.dtype == torch.float32
    assert next(model.h[0].attn.c_attn.parameters()).dtype == torch.bfloat16  # oracle left the model alone
    rel = (ref - t(golden[f"gpt_logits_{attention}"])).norm() / t(golden[f"gpt_logits_{attention}"]).norm()
    assert rel < 2e-2


@pytest.mark.parametrize("seed", [0, 1])
def test_backward_oracle_matches_torch_autograd(seed):
    """The backward restatements against PyTorch CPU autograd of the forward ops (the reference pins
    its backward kernels the same way, tests/test_eager_kernels.py: gradients vs torch eager)."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(13, 40, generator=g, requires_grad=True)
    dy = torch.randn(13, 40, generator=g)
    for approximate in ("none", "tanh"):
        (want,) = torch.autograd.grad(F.gelu(x, approximate=approximate), x, dy)
        close(ref_ops.gelu_backward(dy, x.detach(), approximate), want, atol=2e-6)
    y = torch.softmax(x * 0.3, -1)
    (want,) = torch.autograd.grad(y, x, dy)
    close(ref_ops.softmax_backward(dy, y.detach(), 0.3), want, atol=1e-6)
    w = torch.randn(40, generator=g, requires_grad=True)
    b = torch.randn(40, generator=g, requires_grad=True)
    out, mean, rstd = torch.native_layer_norm(x, (40,), w, b, 1e-5)
    want = torch.autograd.grad(out, (x, w, b), dy)
    got = ref_ops.layer_norm_backward(dy, x.detach(), mean.detach(), rstd.detach(), w.detach())
    for a, e in zip(got, want):
        close(a, e, atol=2e-5)
    close(ref_ops.sum_rows(dy), dy.sum(0), atol=1e-5)
    q, k, v = (torch.randn(2, 3, 9, 8, generator=g, requires_grad=True) for _ in range(3))
    d_out = torch.randn(2, 3, 9, 8, generator=g)
    for causal in (False, True):
        want = torch.autograd.grad(F.scaled_dot_product_attention(q, k, v, is_causal=causal, scale=0.4), (q, k, v), d_out)
        got = ref_ops.sdpa_backward(d_out, q.detach(), k.detach(), v.detach(), causal, 0.4)
        for a, e in zip(got, want):
            close(a, e, atol=2e-6)
