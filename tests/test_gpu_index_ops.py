"""GPU parity of the index-driven row kernels: embedding (+ second table), arg-max over the last
dim, concatenation and the in-place KV-cache append. Integer and copy work is checked bit for bit,
sums within the fp32 / bf16 tolerance; the oracle is PyTorch CPU eager."""

import ctypes

import pytest
import torch
import torch.nn.functional as F
from conftest import assert_parity

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from torch_mojo_backend import ops as _ops

    return _ops


def rnd(shape, seed, dtype=torch.float32):
    return torch.randn(shape, generator=torch.Generator().manual_seed(seed)).to(dtype)


@pytest.mark.parametrize("table_dtype,out_dtype", [(torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16),
                                                   (torch.bfloat16, torch.float32)])
@pytest.mark.parametrize("cols", [1600, 768, 50])  # 50: not a multiple of the 16-byte vector -> scalar kernel
def test_embedding_sum(ops, table_dtype, out_dtype, cols):
    wte, wpe = rnd((1000, cols), 1, table_dtype), rnd((64, cols), 2, table_dtype)
    idx = torch.randint(0, 1000, (3, 64), generator=torch.Generator().manual_seed(3))
    pos = torch.arange(64)
    got = ops.embedding_sum(wte.cuda(), idx.cuda(), wpe.cuda(), pos.cuda(), out_dtype)
    want = (F.embedding(idx, wte).float() + F.embedding(pos, wpe).float()).to(out_dtype)
    assert got.dtype == out_dtype and got.shape == (3, 64, cols)
    if out_dtype == torch.float32:
        assert torch.equal(got.cpu(), want)  # one fp32 add of exactly representable inputs
    else:
        assert_parity(got, want, bf16=True)
    single = ops.embedding_sum(wte.cuda(), idx.cuda())
    assert torch.equal(single.cpu(), F.embedding(idx, wte))


def test_embedding_through_the_lowering_and_strided_table(ops):
    from torch_mojo_backend import aten_functions as af

    big = rnd((200, 96), 4, torch.bfloat16)
    table = big[:, :64]  # row pitch 96, width 64
    idx = torch.randint(0, 200, (7,), generator=torch.Generator().manual_seed(5))
    got = af.aten_embedding(table.cuda(), idx.cuda())
    assert torch.equal(got.cpu(), F.embedding(idx, table))
    empty = af.aten_embedding(table.cuda(), torch.empty((0, 4), dtype=torch.long, device="cuda"))
    assert empty.shape == (0, 4, 64)


def test_embedding_index_out_of_range_is_reported_not_read(ops):
    from torch_mojo_backend import native

    table = rnd((10, 64), 6).cuda()
    idx = torch.tensor([0, 9, 10, -1], device="cuda")
    got = ops.embedding_sum(table, idx)
    torch.cuda.synchronize()
    assert torch.equal(got[:2], table[[0, 9]]) and torch.count_nonzero(got[2:]) == 0
    word = ctypes.c_uint32(0)
    assert native.lib().b200_device_status(ctypes.byref(word)) == native.ERR_DEVICE_TIMEOUT
    assert word.value == native.STATUS_INDEX_OUT_OF_RANGE
    assert native.device_status() == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_argmax_rows(ops, dtype):
    x = rnd((4, 33, 1000), 7, dtype)
    assert torch.equal(ops.argmax(x.cuda()).cpu(), torch.argmax(x.float(), -1))
    # the logits layout: 50257 columns with a padded row pitch, rows that start off a 16-byte boundary
    logits = rnd((64, 50264), 8, dtype)[:, :50257]
    got = ops.argmax(logits.cuda())
    assert torch.equal(got.cpu(), torch.argmax(logits.float(), -1))
    unaligned = rnd((9, 50257), 9, dtype)
    assert torch.equal(ops.argmax(unaligned.cuda()).cpu(), torch.argmax(unaligned.float(), -1))
    short = rnd((5, 3), 10, dtype)
    assert torch.equal(ops.argmax(short.cuda()).cpu(), torch.argmax(short.float(), -1))


def test_argmax_ties_nan_and_lowering(ops):
    from torch_mojo_backend import aten_functions as af

    x = torch.zeros((3, 700))
    x[0, [5, 300, 699]] = 2.0           # ties: the first index wins
    x[1, 400] = float("nan")            # a NaN is the maximum
    x[1, 10] = 9.0
    x[2] = float("-inf")                # nothing finite: index 0
    assert ops.argmax(x.cuda()).tolist() == [5, 400, 0]
    y = rnd((6, 5, 40), 11)
    for dim, keep in ((-1, False), (1, True), (0, False), (None, False)):
        assert torch.equal(af.aten_argmax(y.cuda(), dim, keep).cpu(), torch.argmax(y, dim, keep)), (dim, keep)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.int64, torch.bool])
@pytest.mark.parametrize("dim", [0, 1, 2, -1])
def test_cat(ops, dtype, dim):
    def make(shape, seed):
        t = rnd(shape, seed)
        return (t > 0) if dtype == torch.bool else t.mul(10).to(dtype)

    shapes = {0: [(2, 3, 5), (4, 3, 5), (1, 3, 5)], 1: [(2, 3, 5), (2, 1, 5), (2, 7, 5)],
              2: [(2, 3, 5), (2, 3, 8), (2, 3, 1)], -1: [(2, 3, 5), (2, 3, 3)]}[dim]
    parts = [make(s, 20 + i) for i, s in enumerate(shapes)]
    got = ops.cat([p.cuda() for p in parts], dim)
    assert torch.equal(got.cpu(), torch.cat(parts, dim))
    # a non-contiguous input and the KV-cache shape (16-byte vector path)
    k_cache, k_new = rnd((2, 4, 300, 64), 30, torch.bfloat16), rnd((2, 4, 1, 64), 31, torch.bfloat16)
    got = ops.cat([k_cache.cuda(), k_new.cuda().transpose(1, 2).contiguous().transpose(1, 2)], 2)
    assert torch.equal(got.cpu(), torch.cat([k_cache, k_new], 2))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_kv_append_in_place(ops, dtype):
    """The decode-loop alternative to cat: the new token's rows are written into a preallocated
    cache; nothing else in the cache changes and no memory is allocated."""
    B, H, T_max, D = 2, 3, 40, 64
    cache = rnd((B, H, T_max, D), 40, dtype).cuda()
    before = cache.clone()
    ptr = cache.data_ptr()
    for step, t in ((17, 1), (18, 3)):
        new = rnd((B, H, t, D), 41 + step, dtype).cuda()
        ops.kv_append(cache, new, step)
        before[:, :, step:step + t] = new
        assert cache.data_ptr() == ptr and torch.equal(cache, before)
    with pytest.raises(RuntimeError, match="outside a cache"):
        ops.kv_append(cache, rnd((B, H, 2, D), 50, dtype).cuda(), T_max - 1)
    with pytest.raises(RuntimeError, match="do not match"):
        ops.kv_append(cache, rnd((B, H + 1, 1, D), 51, dtype).cuda(), 0)


def test_decode_loop_with_preallocated_cache_matches_cat(ops):
    """Three decode steps: cache grown by kv_append + attention over the filled prefix (a strided
    view of the cache) equals cat + attention."""
    from oracle import ref_ops

    B, H, D, T0, T_max = 2, 4, 64, 50, 64
    k_hist, v_hist = rnd((B, H, T0, D), 60, torch.bfloat16), rnd((B, H, T0, D), 61, torch.bfloat16)
    k_cache = torch.zeros((B, H, T_max, D), dtype=torch.bfloat16, device="cuda")
    v_cache = torch.zeros_like(k_cache)
    ops.kv_append(k_cache, k_hist.cuda(), 0)
    ops.kv_append(v_cache, v_hist.cuda(), 0)
    for step in range(3):
        q, k_new, v_new = (rnd((B, H, 1, D), 70 + 3 * step + i, torch.bfloat16) for i in range(3))
        ops.kv_append(k_cache, k_new.cuda(), T0 + step)
        ops.kv_append(v_cache, v_new.cuda(), T0 + step)
        k_hist, v_hist = torch.cat([k_hist, k_new], 2), torch.cat([v_hist, v_new], 2)
        n = T0 + step + 1
        out, _ = ops.sdpa(q.cuda(), k_cache[:, :, :n], v_cache[:, :, :n], False)
        assert_parity(out, ref_ops.sdpa(q, k_hist, v_hist, False)[0], bf16=True)


def test_no_device_status_left_behind():
    from torch_mojo_backend import native

    assert native.device_status() == 0
