"""The scaled-dot-product-attention overloads that sit beside the flash one on the same path:
math (bool / additive / broadcast masks, mask + causal, grouped-query heads), efficient and cuDNN
attention (their output tuples and log-sum-exp shapes), and operands no attention kernel takes.
Cases follow the reference's tests/test_aten_functions.py:20-202; the oracle is PyTorch CPU eager.
"""

import math

import pytest
import torch
import torch.nn.functional as F
from conftest import assert_parity

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def af():
    from torch_mojo_backend import aten_functions

    return aten_functions


def rnd(shape, seed, dtype=torch.float32):
    return torch.randn(shape, generator=torch.Generator().manual_seed(seed)).to(dtype)


def cpu_reference(q, k, v, mask=None, causal=False, scale=None):
    """softmax(q k^T * scale + mask) v in fp32 on the CPU, mask semantics as torch's (bool keeps
    where True, float is added), causal on top; also the natural-log LSE."""
    q, k, v = q.float(), k.float(), v.float()
    if k.shape[1] != q.shape[1]:
        rep = q.shape[1] // k.shape[1]
        k, v = k.repeat_interleave(rep, 1), v.repeat_interleave(rep, 1)
    scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    s = q @ k.transpose(-2, -1) * scale
    if mask is not None:
        s = s.masked_fill(~mask, float("-inf")) if mask.dtype == torch.bool else s + mask.float()
    if causal:
        L, S = s.shape[-2:]
        s = s.masked_fill(~torch.ones(L, S, dtype=torch.bool).tril(), float("-inf"))
    return torch.softmax(s, -1) @ v, torch.logsumexp(s, -1)


B, H, L, D = 2, 4, 6, 16


def test_math_additive_causal_mask(af, call_checker):
    call_checker.register(af.aten__scaled_dot_product_attention_math)
    q, k, v = rnd((B, H, L, D), 1), rnd((B, H, L, D), 2), rnd((B, H, L, D), 3)
    mask = torch.tril(torch.ones(L, L))
    mask = mask.masked_fill(mask == 0, float("-inf")).masked_fill(mask == 1, 0.0)
    out, _ = af.aten__scaled_dot_product_attention_math(q.cuda(), k.cuda(), v.cuda(), attn_mask=mask.cuda())
    assert_parity(out, cpu_reference(q, k, v, mask)[0], bf16=False)
    assert_parity(out, torch.ops.aten._scaled_dot_product_attention_math(q, k, v, attn_mask=mask)[0], bf16=False)


def test_math_broadcast_per_head_mask(af):
    q, k, v = rnd((B, H, L, D), 4), rnd((B, H, L, D), 5), rnd((B, H, L, D), 6)
    mask = rnd((H, L, L), 7)  # broadcasts across the batch
    out, _ = af.aten__scaled_dot_product_attention_math(q.cuda(), k.cuda(), v.cuda(), attn_mask=mask.cuda())
    assert_parity(out, cpu_reference(q, k, v, mask)[0], bf16=False)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_math_bool_mask_and_mask_with_causal(af, dtype):
    q, k, v = rnd((B, H, 40, 64), 8, dtype), rnd((B, H, 48, 64), 9, dtype), rnd((B, H, 48, 64), 10, dtype)
    keep = torch.rand((B, 1, 40, 48), generator=torch.Generator().manual_seed(11)) > 0.3
    keep[..., 0] = True  # no row fully masked
    out, _ = af.aten__scaled_dot_product_attention_math(q.cuda(), k.cuda(), v.cuda(), attn_mask=keep.cuda())
    assert_parity(out, cpu_reference(q, k, v, keep)[0], bf16=dtype == torch.bfloat16)
    both, _ = af.aten__scaled_dot_product_attention_math(q.cuda(), k.cuda(), v.cuda(), attn_mask=keep.cuda(), is_causal=True)
    assert_parity(both, cpu_reference(q, k, v, keep, causal=True)[0], bf16=dtype == torch.bfloat16)
    # additive mask together with causal
    add = rnd((40, 48), 12)
    both2 = af.aten_scaled_dot_product_attention(q.cuda(), k.cuda(), v.cuda(), attn_mask=add.cuda().to(dtype), is_causal=True)
    assert_parity(both2, cpu_reference(q, k, v, add.to(dtype), causal=True)[0], bf16=dtype == torch.bfloat16)


def test_math_no_mask_reaches_the_attention_kernel(af):
    from torch_mojo_backend import native

    q, k, v = rnd((B, H, L, D), 13), rnd((B, H, L, D), 14), rnd((B, H, L, D), 15)
    before = native.launch_count
    out, _ = af.aten__scaled_dot_product_attention_math(q.cuda(), k.cuda(), v.cuda())
    assert native.launch_count == before + 1  # one attention kernel, not GEMM + softmax + GEMM
    assert_parity(out, cpu_reference(q, k, v)[0], bf16=False)
    out2 = af.aten_scaled_dot_product_attention(q.cuda(), k.cuda(), v.cuda(), scale=0.3, is_causal=True)
    assert_parity(out2, cpu_reference(q, k, v, causal=True, scale=0.3)[0], bf16=False)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("with_mask", [False, True])
def test_grouped_query_heads(af, dtype, with_mask):
    """8 query heads share 2 K/V heads (enable_gqa): each K/V head serves 4 consecutive query heads."""
    q = rnd((2, 8, 70, 64), 16, dtype)
    k, v = rnd((2, 2, 70, 64), 17, dtype), rnd((2, 2, 70, 64), 18, dtype)
    mask = (torch.rand((70, 70), generator=torch.Generator().manual_seed(19)) > 0.2) if with_mask else None
    if mask is not None:
        mask[:, 0] = True
    out = af.aten_scaled_dot_product_attention(q.cuda(), k.cuda(), v.cuda(), attn_mask=None if mask is None else mask.cuda(),
                                               is_causal=not with_mask, enable_gqa=True)
    want = cpu_reference(q, k, v, mask, causal=not with_mask)[0]
    assert_parity(out, want, bf16=dtype == torch.bfloat16)
    assert_parity(out, F.scaled_dot_product_attention(q.float(), k.float(), v.float(), attn_mask=mask,
                                                      is_causal=not with_mask, enable_gqa=True), bf16=dtype == torch.bfloat16)


@pytest.mark.parametrize("with_bias", [False, True])
@pytest.mark.parametrize("compute_lse", [False, True])
def test_efficient_attention_tuple(af, with_bias, compute_lse):
    """(output, logsumexp [B, H, T padded to 32] or [B, H, 0], philox seed, philox offset); the
    logsumexp is the real one with or without a bias."""
    T = 70
    q, k, v = rnd((B, H, T, 64), 20), rnd((B, H, T, 64), 21), rnd((B, H, T, 64), 22)
    bias = rnd((B, H, T, T), 23) if with_bias else None
    out, lse, seed, offset = af.aten__scaled_dot_product_efficient_attention(
        q.cuda(), k.cuda(), v.cuda(), None if bias is None else bias.cuda(), compute_lse, 0.0, not with_bias)
    want, want_lse = cpu_reference(q, k, v, bias, causal=not with_bias)
    assert_parity(out, want, bf16=False)
    assert seed.dtype == torch.int64 and offset.dtype == torch.int64
    if compute_lse:
        assert lse.shape == (B, H, 96) and lse.dtype == torch.float32
        assert_parity(lse[..., :T], want_lse, bf16=False, scale=max(want_lse.abs().max().item(), 1.0))
    else:
        assert lse.shape == (B, H, 0)


@pytest.mark.parametrize("with_bias", [False, True])
def test_cudnn_attention_tuple(af, with_bias):
    """Nine outputs; logsumexp is [B, H, T, 1]; max_q / max_k are the lengths."""
    T = 33
    q, k, v = (rnd((B, H, T, 64), 24 + i, torch.bfloat16) for i in range(3))
    bias = rnd((1, 1, T, T), 27, torch.bfloat16) if with_bias else None
    res = af.aten__scaled_dot_product_cudnn_attention(q.cuda(), k.cuda(), v.cuda(), None if bias is None else bias.cuda(),
                                                      True, 0.0, not with_bias)
    assert len(res) == 9 and res[4] == T and res[5] == T
    want, want_lse = cpu_reference(q, k, v, bias, causal=not with_bias)
    assert_parity(res[0], want, bf16=True)
    assert res[1].shape == (B, H, T, 1)
    assert_parity(res[1].squeeze(-1), want_lse, bf16=False, scale=max(want_lse.abs().max().item(), 1.0) * 10)


def test_flash_attention_tuple_and_lse(af, call_checker):
    call_checker.register(af.aten__scaled_dot_product_flash_attention)
    q, k, v = (rnd((1, 2, 130, 64), 30 + i, torch.bfloat16) for i in range(3))
    res = af.aten__scaled_dot_product_flash_attention(q.cuda(), k.cuda(), v.cuda(), 0.0, True, False, scale=0.125)
    assert len(res) == 9 and res[4] == 130 and res[5] == 130
    want, want_lse = cpu_reference(q, k, v, causal=True, scale=0.125)
    assert_parity(res[0], want, bf16=True)
    assert res[1].shape == (1, 2, 130)
    assert_parity(res[1], want_lse, bf16=False, scale=max(want_lse.abs().max().item(), 1.0) * 10)


def test_head_dim_beyond_the_attention_kernels_goes_through_gemm_and_softmax(af):
    """head_dim 256 has no attention kernel: the lowering computes it as GEMM -> softmax -> GEMM on
    the same library (never a vendor kernel), LSE included."""
    from torch_mojo_backend import native

    q, k, v = (rnd((1, 2, 40, 256), 33 + i, torch.bfloat16) for i in range(3))
    before = native.launch_count
    res = af.aten__scaled_dot_product_flash_attention(q.cuda(), k.cuda(), v.cuda(), 0.0, True)
    assert native.launch_count - before == 3
    want, want_lse = cpu_reference(q, k, v, causal=True)
    assert_parity(res[0], want, bf16=True)
    assert_parity(res[1], want_lse, bf16=False, scale=max(want_lse.abs().max().item(), 1.0) * 10)


def test_dropout_is_refused(af):
    q = rnd((1, 1, 4, 8), 40).cuda()
    with pytest.raises(NotImplementedError, match="dropout"):
        af.aten_scaled_dot_product_attention(q, q, q, dropout_p=0.1)
