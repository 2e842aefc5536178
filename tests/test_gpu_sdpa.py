"""GPU parity of scaled-dot-product attention against the CPU oracle."""

import pytest
import torch
import torch.nn.functional as F
from conftest import assert_parity

from oracle import ref_ops

pytestmark = pytest.mark.gpu


def gen(shape, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(shape, generator=g).to(dtype)


@pytest.fixture(scope="module")
def ops():
    from torch_mojo_backend import ops as _ops

    return _ops


@pytest.mark.parametrize("kv", [6, 10, 64])
@pytest.mark.parametrize("causal", [False, True])
def test_sdpa_golden(ops, golden, kv, causal):
    q, k, v = (torch.from_numpy(golden[f"sdpa{kv}_{n}"]).cuda() for n in "qkv")
    out, lse = ops.sdpa(q, k, v, causal)
    assert_parity(out, torch.from_numpy(golden[f"sdpa{kv}_{'causal' if causal else 'full'}"]), bf16=False)
    _, ref_lse = ref_ops.sdpa(q.cpu(), k.cpu(), v.cpu(), causal)
    assert_parity(lse, ref_lse, bf16=False)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", [(2, 3, 100, 64), (1, 2, 257, 128), (2, 2, 33, 16), (1, 1, 1, 8)])
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("route", [0, 1])
def test_sdpa_shapes(ops, dtype, shape, causal, route):
    q, k, v = gen(shape, dtype, 1), gen(shape, dtype, 2), gen(shape, dtype, 3)
    out, lse = ops.sdpa(q.cuda(), k.cuda(), v.cuda(), causal, None, route)
    want, want_lse = ref_ops.sdpa(q, k, v, causal)
    assert out.dtype == dtype and out.shape == q.shape and lse.shape == shape[:3]
    assert_parity(out, want, bf16=dtype == torch.bfloat16)
    assert_parity(lse, want_lse, bf16=dtype == torch.bfloat16, scale=max(want_lse.abs().max().item(), 1.0))


def test_sdpa_fused_qkv_strided_views_and_kv_longer(ops):
    """Q/K/V as views into one fused [B, T, 3C] projection (the layout GPT-2 produces), and a
    kv_len != q_len case with the top-left aligned causal mask."""
    B, T, H, D = 2, 96, 4, 64
    qkv = gen((B, T, 3 * H * D), torch.bfloat16, 4)
    q, k, v = (t.view(B, T, H, D).transpose(1, 2) for t in qkv.split(H * D, dim=2))
    qg, kg, vg = (t.view(B, T, H, D).transpose(1, 2) for t in qkv.cuda().split(H * D, dim=2))
    out, _ = ops.sdpa(qg, kg, vg, True)
    assert_parity(out, ref_ops.sdpa(q, k, v, True)[0], bf16=True)
    # output memory is [B, T, H, D] so that transpose(1, 2).reshape(B, T, C) is a view
    assert out.transpose(1, 2).is_contiguous()
    q2, k2, v2 = gen((1, 2, 16, 32), torch.float32, 5), gen((1, 2, 40, 32), torch.float32, 6), gen((1, 2, 40, 32), torch.float32, 7)
    out2, _ = ops.sdpa(q2.cuda(), k2.cuda(), v2.cuda(), True)
    assert_parity(out2, ref_ops.sdpa(q2, k2, v2, True)[0], bf16=False)


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("q_len,kv_len", [(1, 1), (77, 300), (64, 200), (129, 129), (300, 77), (128, 64),
                                          (256, 256), (257, 513), (384, 384), (512, 300), (640, 640), (130, 1000)])
def test_sdpa_tensor_core_route_ragged_lengths(ops, causal, q_len, kv_len):
    """head_dim 64 bf16 takes the tcgen05 kernel: ragged tiles, kv_len != q_len (causal mask is
    top-left aligned), single-row and single-key cases; forced route so that a silent reroute fails."""
    q = gen((2, 3, q_len, 64), torch.bfloat16, 30)
    k = gen((2, 3, kv_len, 64), torch.bfloat16, 31)
    v = gen((2, 3, kv_len, 64), torch.bfloat16, 32)
    out, lse = ops.sdpa(q.cuda(), k.cuda(), v.cuda(), causal, None, 2)
    want, want_lse = ref_ops.sdpa(q, k, v, causal)
    assert_parity(out, want, bf16=True)
    assert_parity(lse, want_lse, bf16=False, scale=max(want_lse.abs().max().item(), 1.0) * 10)


def test_sdpa_route_selection(ops):
    import ctypes

    from torch_mojo_backend import native

    def route(shape, dtype):
        q = torch.empty(shape, dtype=dtype, device="cuda")
        o = torch.empty(shape, dtype=dtype, device="cuda")
        lse = torch.empty(shape[:3], device="cuda")
        s = ops.fill_sdpa_args(q, q, q, o, lse, True, 0.125, 0)
        return native.lib().b200_sdpa_route(ctypes.byref(s))

    assert route((8, 12, 1024, 64), torch.bfloat16) == 2
    assert route((4, 25, 2048, 64), torch.bfloat16) == 2
    assert route((8, 12, 1024, 64), torch.float32) == 1   # exact-fp32 route
    assert route((2, 2, 128, 128), torch.bfloat16) == 1   # head_dim other than 64


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("head_dim", [32, 64, 128])
@pytest.mark.parametrize("q_len,kv_len,causal", [(1, 1, False), (1, 7, False), (1, 1024, False), (1, 5000, False),
                                                 (3, 333, False), (3, 333, True), (16, 9, True), (2, 32768, False)])
def test_sdpa_decode_route(ops, dtype, head_dim, q_len, kv_len, causal):
    """Few query rows against a KV cache: the split-KV cluster kernel, forced (route 3) so that a
    silent reroute fails. Keys fewer than the eight CTAs of a cluster, a ragged last chunk, the
    largest supported cache, and the top-left aligned causal mask."""
    b, h = (1, 2) if kv_len > 8192 else (2, 3)
    q = gen((b, h, q_len, head_dim), dtype, 60)
    k = gen((b, h, kv_len, head_dim), dtype, 61)
    v = gen((b, h, kv_len, head_dim), dtype, 62)
    out, lse = ops.sdpa(q.cuda(), k.cuda(), v.cuda(), causal, None, 3)
    want, want_lse = ref_ops.sdpa(q, k, v, causal)
    assert out.dtype == dtype and out.shape == q.shape
    assert_parity(out, want, bf16=dtype == torch.bfloat16)
    assert_parity(lse, want_lse, bf16=False, scale=max(want_lse.abs().max().item(), 1.0) * (10 if dtype == torch.bfloat16 else 1))


def test_sdpa_decode_route_strided_cache_view(ops):
    """K and V as the first T positions of a longer preallocated cache [B, H, T_max, D] (strides
    that are not the dense ones) and Q as a slice of a fused projection; AUTO picks the decode
    kernel for one query row."""
    import ctypes

    from torch_mojo_backend import native

    B, H, T, T_max, D = 2, 5, 300, 512, 64
    cache_k, cache_v = gen((B, H, T_max, D), torch.bfloat16, 63), gen((B, H, T_max, D), torch.bfloat16, 64)
    qkv = gen((B, 1, 3 * H * D), torch.bfloat16, 65)
    q = qkv[..., : H * D].view(B, 1, H, D).transpose(1, 2)
    kg, vg = cache_k.cuda()[:, :, :T], cache_v.cuda()[:, :, :T]
    qg = qkv.cuda()[..., : H * D].view(B, 1, H, D).transpose(1, 2)
    o = torch.empty((B, H, 1, D), dtype=torch.bfloat16, device="cuda")
    lse = torch.empty((B, H, 1), device="cuda")
    args = ops.fill_sdpa_args(qg, kg, vg, o, lse, False, D**-0.5, 0)
    assert native.lib().b200_sdpa_route(ctypes.byref(args)) == 3
    out, _ = ops.sdpa(qg, kg, vg, False)
    assert_parity(out, ref_ops.sdpa(q, cache_k[:, :, :T], cache_v[:, :, :T], False)[0], bf16=True)


@pytest.mark.parametrize("shape", [(8, 12, 1024, 64), (4, 25, 2048, 64)])
def test_sdpa_benchmark_shapes_bf16(ops, shape):
    """The two causal bf16 configurations; oracle = PyTorch CPU SDPA in fp32 on the bf16 values."""
    q, k, v = gen(shape, torch.bfloat16, 8), gen(shape, torch.bfloat16, 9), gen(shape, torch.bfloat16, 10)
    out, lse = ops.sdpa(q.cuda(), k.cuda(), v.cuda(), True)
    B = 2  # the CPU oracle on two batches keeps the test short; the rest is checked by the LSE identity
    want = F.scaled_dot_product_attention(q[:B].float(), k[:B].float(), v[:B].float(), is_causal=True)
    assert_parity(out[:B], want, bf16=True)
    # size-independent property at full size: row 0 attends only to key 0, so out[..., 0, :] == v[..., 0, :]
    assert torch.equal(out[:, :, 0, :].cpu(), v[:, :, 0, :])
    # and LSE of row 0 is the single scaled score q0.k0 / sqrt(d)
    s00 = (q[:, :, 0, :].float() * k[:, :, 0, :].float()).sum(-1) / shape[-1] ** 0.5
    assert_parity(lse[:, :, 0], s00, bf16=False, scale=max(s00.abs().max().item(), 1.0))


def test_sdpa_many_items_per_cta_and_l2_groups(ops):
    """More work items than CTAs and more (batch, head) pairs than one L2 group holds (the
    kernel walks pairs in groups sized for L2 and, inside a group, query tiles heaviest first):
    every item must still land on its own rows. Checked on a sample of pairs against the oracle."""
    B, H, T = 3, 67, 768   # 201 pairs, 3 query-tile pairs each: 603 items on 148 CTAs
    q, k, v = gen((B, H, T, 64), torch.bfloat16, 40), gen((B, H, T, 64), torch.bfloat16, 41), gen((B, H, T, 64), torch.bfloat16, 42)
    out, lse = ops.sdpa(q.cuda(), k.cuda(), v.cuda(), True, None, 2)
    for b, h in ((0, 0), (0, 66), (1, 33), (2, 13), (2, 66)):
        want, want_lse = ref_ops.sdpa(q[b:b + 1, h:h + 1], k[b:b + 1, h:h + 1], v[b:b + 1, h:h + 1], True)
        assert_parity(out[b:b + 1, h:h + 1], want, bf16=True, what=f"pair ({b},{h})")
        assert_parity(lse[b:b + 1, h:h + 1], want_lse, bf16=False, scale=max(want_lse.abs().max().item(), 1.0) * 10)
    # size-independent property over every pair: row 0 attends only to key 0
    assert torch.equal(out[:, :, 0, :].cpu(), v[:, :, 0, :])


def test_sdpa_large_scores_trigger_lazy_rescale(ops):
    """Scores whose running maximum keeps growing along the keys (so the accumulator in tensor
    memory has to be rescaled after the first tile, the rare path of the lazy-rescale scheme)."""
    B, H, T = 1, 2, 512
    q = gen((B, H, T, 64), torch.bfloat16, 43)
    k = gen((B, H, T, 64), torch.bfloat16, 44)
    # keys grow along the sequence so that later tiles hold much larger scores
    k = (k.float() * torch.linspace(0.5, 6.0, T).view(1, 1, T, 1)).to(torch.bfloat16)
    v = gen((B, H, T, 64), torch.bfloat16, 45)
    for causal in (False, True):
        out, lse = ops.sdpa(q.cuda(), k.cuda(), v.cuda(), causal, None, 2)
        want, want_lse = ref_ops.sdpa(q, k, v, causal)
        assert_parity(out, want, bf16=True)
        assert_parity(lse, want_lse, bf16=False, scale=max(want_lse.abs().max().item(), 1.0) * 10)


def test_no_device_timeout_recorded():
    from torch_mojo_backend import native

    assert native.device_status() == 0
