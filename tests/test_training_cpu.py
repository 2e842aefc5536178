"""A training step (forward + backward) through the backend on a CPU-only box. The kernel ops are
replaced by torch stand-ins (installed by the test, never shipped), which checks the wiring of the
backward lowerings -- which aten nodes stay whole, operand order, dtypes, shapes, transposed GEMM
operands -- against plain eager autograd."""

import pytest
import torch
import torch.nn.functional as F

from test_fusion_cpu import _StandIns
from torch_mojo_backend import aten_functions as af
from torch_mojo_backend import mojo_backend


class _TrainingStandIns(_StandIns):
    @staticmethod
    def layer_norm(x, w, b, eps, out_dtype=None):
        _StandIns._record(x, ("layer_norm", out_dtype))
        xf = x.float()
        mean = xf.mean(-1)
        rstd = torch.rsqrt(xf.var(-1, unbiased=False) + eps)
        y = (xf - mean[..., None]) * rstd[..., None]
        if w is not None:
            y = y * w.float()
        if b is not None:
            y = y + b.float()
        return y.to(out_dtype or x.dtype), mean, rstd

    @staticmethod
    def softmax(x, scale=1.0, causal=False, q_len=0, out_dtype=None):
        out_dtype = out_dtype or x.dtype
        x = x.float() * scale
        if causal:  # the kernel's fused flag: column j of row r is visible when j <= r % q_len
            x = x.masked_fill(~torch.ones(x.shape[-2], x.shape[-1], dtype=torch.bool).tril(), float("-inf"))
        return torch.softmax(x, -1).to(out_dtype)

    @staticmethod
    def gelu_backward(dy, x, approximate="none"):
        _StandIns._record(x, ("gelu_backward", approximate))
        return torch.ops.aten.gelu_backward(dy, x, approximate=approximate)

    @staticmethod
    def softmax_backward(dy, y, scale=1.0, out_dtype=None):
        _StandIns._record(y, ("softmax_backward", scale))
        yf, gf = y.float(), dy.float()
        return (scale * yf * (gf - (gf * yf).sum(-1, keepdim=True))).to(out_dtype or y.dtype)

    @staticmethod
    def layer_norm_backward(dy, x, mean, rstd, weight, want_weight=True, want_bias=True, dx_add=None, dx_dtype=None):
        _StandIns._record(x, ("layer_norm_backward", want_weight, want_bias, dx_add is not None, dx_dtype))
        assert dx_dtype in (None, dy.dtype) or (dy.dtype, x.dtype, dx_dtype) == (torch.bfloat16, torch.float32, torch.float32)
        assert dx_add is None or (dx_add.shape == x.shape and dx_add.dtype == (dx_dtype or dy.dtype))
        cols = x.shape[-1]
        xf, gf = x.float().reshape(-1, cols), dy.float().reshape(-1, cols)
        xh = (xf - mean.reshape(-1, 1).float()) * rstd.reshape(-1, 1).float()
        g = gf * (weight.float() if weight is not None else 1.0)
        dx = rstd.reshape(-1, 1).float() * (g - g.mean(-1, keepdim=True) - xh * (g * xh).mean(-1, keepdim=True))
        pd = weight.dtype if weight is not None else x.dtype
        return (
            (dx.reshape(x.shape) + (dx_add.float() if dx_add is not None else 0.0)).to(dx_dtype or dy.dtype),
            (gf * xh).sum(0).to(pd) if want_weight else None,
            gf.sum(0).to(pd) if want_bias else None,
        )

    @staticmethod
    def layer_norm_backward_with_copy(dy, x, mean, rstd, weight, want_weight=True, want_bias=True, dx_add=None,
                                      dx_dtype=None, want_cast=False, sum_dtype=None):
        dx, dg, db = _TrainingStandIns.layer_norm_backward(dy, x, mean, rstd, weight, want_weight, want_bias, dx_add, dx_dtype)
        _StandIns._record(x, ("layer_norm_backward_with_copy", want_cast, sum_dtype))
        assert not want_cast or dx.dtype == torch.float32
        narrow = dx.to(torch.bfloat16) if want_cast else None
        summed = narrow if narrow is not None else dx
        sums = summed.reshape(-1, x.shape[-1]).float().sum(0).to(sum_dtype) if sum_dtype is not None else None
        return dx, dg, db, narrow, sums

    @staticmethod
    def sum_rows(x, out_dtype=None):
        _StandIns._record(x, ("sum_rows",))
        return x.float().reshape(-1, x.shape[-1]).sum(0).to(out_dtype or x.dtype)


@pytest.fixture()
def training_stand_ins(monkeypatch, reset_compiler):
    _StandIns.calls = []
    monkeypatch.setattr(af, "ops", _TrainingStandIns)
    return _TrainingStandIns


def _grads(model):
    return {n: p.grad.clone() for n, p in model.named_parameters() if p.grad is not None}


@pytest.mark.parametrize("attention", ["masked_softmax", "sdpa"])
def test_gpt2_training_step_matches_eager_autograd(training_stand_ins, attention):
    from demo_scripts.gpt2 import GPT2, GPTConfig

    cfg = GPTConfig(vocab_size=97, block_size=16, n_layer=2, n_head=2, n_embd=32)
    model = GPT2(cfg, attention).init_weights(0).train()
    g = torch.Generator().manual_seed(1)
    ids = torch.randint(0, 97, (2, 16), generator=g)
    targets = torch.randint(0, 97, (2, 16), generator=g)

    def loss_of(m):
        return F.cross_entropy(m(ids).reshape(-1, 97).float(), targets.reshape(-1))

    want_loss = loss_of(model)
    want_loss.backward()
    want = _grads(model)
    model.zero_grad()

    before = {f: f.call_count for f in (af.aten_gelu_backward, af.aten_native_layer_norm_backward)}
    got_loss = loss_of(torch.compile(model, backend=mojo_backend))
    got_loss.backward()
    got = _grads(model)

    torch.testing.assert_close(got_loss, want_loss, rtol=1e-5, atol=1e-6)
    assert got.keys() == want.keys() and len(got) > 10
    for name in want:
        torch.testing.assert_close(got[name], want[name], rtol=1e-4, atol=1e-5, msg=lambda m: f"{name}: {m}")
    # the backward graph kept these ops whole and they went through the lowerings (and the stand-ins)
    assert af.aten_gelu_backward.call_count > before[af.aten_gelu_backward]
    assert af.aten_native_layer_norm_backward.call_count > before[af.aten_native_layer_norm_backward]
    kinds = {c[0] for c in training_stand_ins.calls}
    assert {"gelu_backward", "layer_norm_backward", "sum_rows"} <= kinds
    if attention == "masked_softmax":
        assert "softmax_backward" in kinds


def test_bf16_policy_training_graph_folds_the_layer_norm_cast(training_stand_ins):
    """In the bf16 policy every LayerNorm output is cast to bf16 for the next GEMM; the forward of a
    training step also keeps mean and rstd for the backward. The cast is folded into the LayerNorm
    launch there too, and the gradients still match eager autograd."""
    from demo_scripts.gpt2 import GPT2, GPTConfig

    cfg = GPTConfig(vocab_size=97, block_size=16, n_layer=2, n_head=2, n_embd=32)
    model = GPT2(cfg, "masked_softmax").init_weights(0).train().set_precision("bf16")
    g = torch.Generator().manual_seed(1)
    ids = torch.randint(0, 97, (2, 16), generator=g)
    targets = torch.randint(0, 97, (2, 16), generator=g)

    def loss_of(m):
        return F.cross_entropy(m(ids).reshape(-1, 97).float(), targets.reshape(-1))

    loss_of(model).backward()
    want = _grads(model)
    model.zero_grad()
    before = af.fused_layer_norm_with_statistics.call_count
    before_backward = af.fused_layer_norm_backward.call_count
    loss_of(torch.compile(model, backend=mojo_backend)).backward()
    got = _grads(model)
    assert af.fused_layer_norm_with_statistics.call_count > before
    assert ("layer_norm", torch.bfloat16) in training_stand_ins.calls
    # backward: all five LayerNorm gradients read the bf16 gradient of the GEMM before them and write
    # fp32; the four inside the blocks also add the gradient of the residual branch in the same launch
    assert af.fused_layer_norm_backward.call_count > before_backward
    kinds = [c for c in training_stand_ins.calls if c[0] == "layer_norm_backward"]
    assert len(kinds) == 5 and all(c[4] == torch.float32 for c in kinds)
    assert sum(1 for c in kinds if c[3]) == 4
    # all five residual-stream gradients also leave the launch as bf16: four feed a projection's backward,
    # one the embedding's
    copies = [c for c in training_stand_ins.calls if c[0] == "layer_norm_backward_with_copy"]
    assert sum(1 for c in copies if c[1] and c[2] is None) == 5
    for name in want:
        scale = float(want[name].float().abs().max())
        err = float((got[name].float() - want[name].float()).abs().max())
        assert err <= 6e-2 * max(scale, 1e-8), f"{name}: {err:.3e} against {scale:.3e}"


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("with_bias", [False, True])
def test_attention_backward_composition_matches_autograd(training_stand_ins, causal, with_bias):
    g = torch.Generator().manual_seed(2)
    B, H, T, D = 2, 3, 8, 4
    q, k, v = (torch.randn(B, H, T, D, generator=g, requires_grad=True) for _ in range(3))
    bias = torch.randn(1, H, T, T, generator=g, requires_grad=True) if with_bias else None
    d_out = torch.randn(B, H, T, D, generator=g)
    scale = 0.37
    scores = (q @ k.transpose(-1, -2)) * scale
    if bias is not None:
        scores = scores + bias
    if causal:
        scores = scores.masked_fill(~torch.ones(T, T, dtype=torch.bool).tril(), float("-inf"))
    out = torch.softmax(scores, -1) @ v
    want = torch.autograd.grad(out, [q, k, v] + ([bias] if with_bias else []), d_out)

    dq, dk, dv, dbias = af._sdpa_backward(
        d_out, q.detach(), k.detach(), v.detach(), None if bias is None else bias.detach(), causal, scale, with_bias
    )
    for got, ref in zip((dq, dk, dv), want[:3]):
        torch.testing.assert_close(got, ref, rtol=1e-4, atol=1e-5)
    if with_bias:
        torch.testing.assert_close(dbias, want[3], rtol=1e-4, atol=1e-5)


def test_cat_of_slices_that_tile_one_buffer_is_a_view():
    """`aten_cat` returns the common buffer when its inputs tile it exactly and in order (the dq | dk | dv
    slices of a packed attention gradient); anything else takes the copying path."""
    packed = torch.arange(2 * 8 * 3 * 2 * 4, dtype=torch.float32).reshape(2, 8, 3, 2, 4).clone()
    parts = [packed[:, :, i].reshape(2, 8, 8) for i in range(3)]  # [B, T, H * D] views, row pitch 3 * H * D
    assert all(p._base is packed for p in parts)
    whole = af._tiles_of_one_buffer(parts, 2)
    assert whole is not None and whole.data_ptr() == packed.data_ptr() and whole.is_contiguous()
    assert torch.equal(whole, torch.cat(parts, 2))
    assert torch.equal(af._tiles_of_one_buffer(parts, -1), whole)
    # wrong order, a subset, another dim, a different base, tensors that own their memory
    assert af._tiles_of_one_buffer([parts[1], parts[0], parts[2]], 2) is None
    assert af._tiles_of_one_buffer(parts[:2], 2) is None
    assert af._tiles_of_one_buffer(parts, 1) is None
    other = torch.zeros(2, 8, 3, 2, 4)
    assert af._tiles_of_one_buffer([parts[0], other[:, :, 1].reshape(2, 8, 8), parts[2]], 2) is None
    assert af._tiles_of_one_buffer([p.clone() for p in parts], 2) is None
    # a buffer with room after the slices is not "exactly tiled"
    roomy = torch.zeros(2, 8, 4, 2, 4)
    assert af._tiles_of_one_buffer([roomy[:, :, i].reshape(2, 8, 8) for i in range(3)], 2) is None


def test_packed_attention_gradient_buffers():
    from torch_mojo_backend import ops

    dq, dk, dv = ops._sdpa_gradient_buffers(2, 3, 16, 16, 64, torch.bfloat16, "cpu")
    assert dq._base is dk._base is dv._base and dq._base.shape == (2, 16, 3, 3, 64)
    assert dq.shape == dk.shape == dv.shape == (2, 3, 16, 64)
    assert dq.stride() == (16 * 3 * 3 * 64, 64, 3 * 3 * 64, 1)
    assert dk.storage_offset() - dq.storage_offset() == 3 * 64
    # the views the backward graph builds from them concatenate back to the buffer
    flat = [t.transpose(1, 2).reshape(2, 16, 3 * 64) for t in (dq, dk, dv)]
    assert af._tiles_of_one_buffer(flat, 2).data_ptr() == dq._base.data_ptr()
    # cross attention: separate buffers in the same [B, T, H, D] memory order
    dq, dk, dv = ops._sdpa_gradient_buffers(2, 3, 16, 24, 64, torch.bfloat16, "cpu")
    assert dq._base is not dk._base and dk.shape == (2, 3, 24, 64) and dk.transpose(1, 2).is_contiguous()


def test_repitched_operand_is_kept_on_its_base_tensor():
    from torch_mojo_backend import ops

    dl = torch.randn(4096, 1031).to(torch.bfloat16)  # 2062-byte pitch: not a multiple of 16
    view = dl[:]                                      # what a graph's view node hands to the GEMM
    a = ops._tma_pitch(view)
    assert a.stride(0) % 8 == 0 and torch.equal(a, dl)
    assert ops._tma_pitch(dl[:]) is a, "a second view of the same tensor shares the copy"
    at = ops._tma_pitch(dl[:].t())                    # the weight gradient reads the transposed view
    assert at.shape == (1031, 4096) and at.data_ptr() == a.data_ptr()
    dl.add_(1.0)                                      # written to: the copy is stale and is made again
    b = ops._tma_pitch(dl[:])
    assert b is not a and torch.equal(b, dl)
    small = torch.randn(64, 1031).to(torch.bfloat16)
    assert ops._tma_pitch(small) is small             # too small to be worth a copy
    with torch.inference_mode():                      # no version counter to tell a write by: copied every time
        frozen = torch.randn(4096, 1031).to(torch.bfloat16)
        first, second = ops._tma_pitch(frozen), ops._tma_pitch(frozen)
        assert first is not second and torch.equal(first, frozen) and torch.equal(second, frozen)
    aligned = torch.randn(4096, 1024).to(torch.bfloat16)
    assert ops._tma_pitch(aligned) is aligned
