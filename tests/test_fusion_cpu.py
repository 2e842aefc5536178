"""The graph fusion pass on a CPU-only box. The rewritten graphs are executed with torch stand-ins
for the kernel ops (installed by the test, never shipped), which checks the wiring of the fused
nodes -- operands, bias, residual, epilogue, dtypes, shapes -- against plain eager execution."""

import pytest
import torch
import torch.nn.functional as F

from torch_mojo_backend import aten_functions as af
from torch_mojo_backend import mojo_backend, native
from torch_mojo_backend.torch_compile_backend import compiler, fusion


class _StandIns:
    """torch implementations with the signatures of torch.ops.b200.* (test doubles)."""

    calls = []

    @staticmethod
    def _record(t, entry):
        # the compile-time dry run calls the lowerings on FakeTensors; count real executions only
        if not isinstance(t, torch._subclasses.FakeTensor):
            _StandIns.calls.append(entry)

    @staticmethod
    def gemm(a, b, bias=None, residual=None, alpha=1.0, beta=1.0, epilogue=0, out_dtype=None, route=0):
        _StandIns._record(a, ("gemm", epilogue, out_dtype, residual is not None))
        acc = alpha * (a.float() @ b.float())
        if bias is not None:
            acc = acc + beta * bias.float()
        if epilogue == native.EPILOGUE_GELU_TANH:
            acc = F.gelu(acc, approximate="tanh")
        elif epilogue == native.EPILOGUE_GELU_ERF:
            acc = F.gelu(acc)
        if residual is not None:
            acc = acc + residual.float()
        return acc.to(out_dtype or a.dtype)

    @staticmethod
    def layer_norm(x, w, b, eps, out_dtype=None):
        _StandIns._record(x, ("layer_norm", out_dtype))
        y = F.layer_norm(x.float(), (x.shape[-1],), None if w is None else w.float(), None if b is None else b.float(), eps)
        mean = x.float().mean(-1)
        return y.to(out_dtype or x.dtype), mean, mean

    @staticmethod
    def softmax(x, scale=1.0, causal=False, q_len=0, out_dtype=None):
        return torch.softmax(x.float() * scale, -1).to(out_dtype or x.dtype)

    @staticmethod
    def mask_rows_of(x, mask):
        from torch_mojo_backend import ops

        return ops.mask_rows_of(x, mask)

    @staticmethod
    def softmax_masked(x, mask, fill, scale=1.0, invert=False, out_dtype=None):
        _StandIns._record(x, ("softmax_masked", fill, scale, invert))
        masked = mask != invert
        return torch.softmax(torch.where(masked, torch.tensor(fill), x.float() * scale), -1).to(out_dtype or x.dtype)

    @staticmethod
    def gelu(x, approximate="none"):
        return F.gelu(x, approximate=approximate)

    @staticmethod
    def reduce(x, op, out_dtype=None):
        return [x.sum(-1), x.mean(-1), x.amax(-1)][op].to(out_dtype or x.dtype)

    @staticmethod
    def embedding_sum(table, indices, table2=None, indices2=None, out_dtype=None):
        _StandIns._record(table, ("embedding_sum", table2 is not None, out_dtype))
        y = F.embedding(indices, table).float()
        if table2 is not None:
            y = y + F.embedding(indices2, table2).float()
        return y.to(out_dtype or table.dtype)

    @staticmethod
    def argmax(x):
        return torch.argmax(x, -1)

    @staticmethod
    def cat(tensors, dim=0):
        return torch.cat(list(tensors), dim)

    @staticmethod
    def sdpa_backward_supported(q, k, v):
        return False

    @staticmethod
    def sdpa(q, k, v, causal=False, scale=None, route=0):
        out = F.scaled_dot_product_attention(q, k, v, is_causal=causal, scale=scale)
        return out, torch.zeros(q.shape[:3])


@pytest.fixture()
def stand_ins(monkeypatch, reset_compiler):
    _StandIns.calls = []
    monkeypatch.setattr(af, "ops", _StandIns)
    # the compile-time dry run compares against the trace; stand-ins produce the same metadata
    return _StandIns


def test_gpt2_bf16_policy_chains_are_folded(stand_ins):
    from demo_scripts.gpt2 import GPT2, GPTConfig

    cfg = GPTConfig(vocab_size=211, block_size=32, n_layer=2, n_head=4, n_embd=64)
    model = GPT2(cfg, "masked_softmax").init_weights(0).eval().set_precision("bf16")
    ids = torch.randint(0, 211, (2, 16), generator=torch.Generator().manual_seed(0))
    with torch.no_grad():
        want = model(ids)
        got = torch.compile(model, backend=mojo_backend)(ids)
    # fused graph computes in fp32 where eager rounds to bf16, so it is at least as close to the
    # fp32 oracle; against bf16 eager it agrees to bf16 accuracy
    torch.testing.assert_close(got, want, rtol=2e-2, atol=2e-2)
    gemms = [c for c in stand_ins.calls if c[0] == "gemm"]
    lns = [c for c in stand_ins.calls if c[0] == "layer_norm"]
    assert all(c[1] == torch.bfloat16 for c in lns) and len(lns) == 2 * 2 + 1, "every LayerNorm writes bf16 directly"
    assert sum(1 for c in gemms if c[1] == native.EPILOGUE_GELU_TANH) == 2, "MLP up-projection carries the GELU"
    assert sum(1 for c in gemms if c[3]) == 4, "both projections of each block carry the residual add"
    assert gemms[-1][2] == torch.float32 and not gemms[-1][3], "LM head stores fp32 logits"
    assert [c for c in stand_ins.calls if c[0] == "embedding_sum"] == [("embedding_sum", True, torch.float32)], \
        "token + positional embeddings are one gather that writes the fp32 residual stream"


def test_fused_gemm_wiring_matches_eager(stand_ins):
    def fn(x, w1, b1, w2, b2, res):
        h = F.gelu(F.linear(x, w1, b1), approximate="tanh")          # addmm -> view -> gelu
        y = F.linear(h, w2, b2).float()                              # addmm -> view -> _to_copy
        return res + y                                               # residual on the left

    g = torch.Generator().manual_seed(0)
    bf = torch.bfloat16
    x = torch.randn(2, 5, 16, generator=g).to(bf)
    w1, b1 = torch.randn(32, 16, generator=g).to(bf), torch.randn(32, generator=g).to(bf)
    w2, b2 = torch.randn(16, 32, generator=g).to(bf), torch.randn(16, generator=g).to(bf)
    res = torch.randn(2, 5, 16, generator=g)
    got = torch.compile(fn, backend=mojo_backend)(x, w1, b1, w2, b2, res)
    assert got.dtype == torch.float32 and got.shape == (2, 5, 16)
    torch.testing.assert_close(got, fn(x, w1, b1, w2, b2, res), rtol=2e-2, atol=5e-2)
    assert [c for c in stand_ins.calls if c[0] == "gemm"] == [
        ("gemm", native.EPILOGUE_GELU_TANH, bf, False), ("gemm", 0, torch.float32, True)]


def test_embedding_sum_fusion_and_its_limits(stand_ins):
    wte = torch.randn(50, 16, generator=torch.Generator().manual_seed(1)).to(torch.bfloat16)
    wpe = torch.randn(12, 16, generator=torch.Generator().manual_seed(2)).to(torch.bfloat16)
    idx = torch.randint(0, 50, (3, 12), generator=torch.Generator().manual_seed(3))

    def fused(idx, wte, wpe):
        pos = torch.arange(idx.shape[1])
        return F.embedding(idx, wte).float() + F.embedding(pos, wpe).float()

    got = torch.compile(fused, backend=mojo_backend)(idx, wte, wpe)
    torch.testing.assert_close(got, fused(idx, wte, wpe))
    assert [c for c in stand_ins.calls if c[0] == "embedding_sum"] == [("embedding_sum", True, torch.float32)]

    # an embedding whose result has a second consumer keeps its own gather
    stand_ins.calls.clear()
    torch._dynamo.reset()

    def shared(idx, wte, wpe):
        tok = F.embedding(idx, wte)
        return tok + F.embedding(torch.arange(idx.shape[1]), wpe), tok.sum()

    got2 = torch.compile(shared, backend=mojo_backend)(idx, wte, wpe)
    torch.testing.assert_close(got2[0], shared(idx, wte, wpe)[0])
    assert [c[1] for c in stand_ins.calls if c[0] == "embedding_sum"] == [False, False]


def test_chain_with_a_second_consumer_is_not_folded(stand_ins):
    def fn(x, w, b):
        y = F.linear(x, w, b)
        return F.gelu(y), y  # y itself is needed: the GELU cannot move into the GEMM

    g = torch.Generator().manual_seed(1)
    x, w, b = torch.randn(4, 8, generator=g), torch.randn(6, 8, generator=g), torch.randn(6, generator=g)
    got = torch.compile(fn, backend=mojo_backend)(x, w, b)
    for a, e in zip(got, fn(x, w, b)):
        torch.testing.assert_close(a, e, rtol=1e-5, atol=1e-5)
    assert [c[1] for c in stand_ins.calls if c[0] == "gemm"] == [0]


def test_fusion_can_be_switched_off(stand_ins, monkeypatch):
    monkeypatch.setenv("TORCH_MOJO_BACKEND_NO_FUSION", "1")

    def fn(x, w, b):
        return F.gelu(F.linear(x, w, b), approximate="tanh")

    g = torch.Generator().manual_seed(2)
    args = (torch.randn(4, 8, generator=g), torch.randn(6, 8, generator=g), torch.randn(6, generator=g))
    torch.testing.assert_close(torch.compile(fn, backend=mojo_backend)(*args), fn(*args), rtol=1e-5, atol=1e-5)
    assert [c[1] for c in stand_ins.calls if c[0] == "gemm"] == [0]


def test_attention_output_copy_is_dropped_only_for_fresh_outputs():
    """Graph-level check on a hand-built graph (the CUDA attention overloads cannot be traced
    here): clone of a transposed attention output becomes an alias, a clone of an input stays."""
    graph = torch.fx.Graph()
    q = graph.placeholder("q")
    fake = torch.empty(2, 4, 8, 16)
    q.meta["val"] = fake
    att = graph.call_function(torch.ops.aten._scaled_dot_product_flash_attention.default, (q, q, q, 0.0, True))
    att.meta["val"] = (fake,)
    o = graph.call_function(__import__("operator").getitem, (att, 0))
    o.meta["val"] = fake
    tr = graph.call_function(torch.ops.aten.transpose.int, (o, 1, 2))
    tr.meta["val"] = fake.transpose(1, 2)
    c1 = graph.call_function(torch.ops.aten.clone.default, (tr,), {"memory_format": torch.contiguous_format})
    c1.meta["val"] = fake.transpose(1, 2).contiguous()
    c2 = graph.call_function(torch.ops.aten.clone.default, (q,), {"memory_format": torch.contiguous_format})
    c2.meta["val"] = fake
    graph.output((c1, c2))
    gm = torch.fx.GraphModule(torch.nn.Module(), graph)
    stats = fusion.fuse_graph(gm)
    assert stats["attention_output_copy"] == 1
    targets = [n.target for n in gm.graph.nodes if n.op == "call_function"]
    assert af.contiguous_or_alias in targets and torch.ops.aten.clone.default in targets
    x = torch.randn(3, 4).t()
    assert af.contiguous_or_alias(x).is_contiguous()
    xc = x.contiguous()
    assert af.contiguous_or_alias(xc) is xc


def test_masked_softmax_chain_is_folded(stand_ins):
    """scale -> masked_fill -> softmax (GPT-2 demo form) and div -> where -> softmax (HF form)
    each become one masked softmax; the fused node gets the unscaled scores, the mask as it is
    and the scale / fill / polarity of the chain."""
    T = 12
    tril = torch.tril(torch.ones(T, T)).view(1, 1, T, T)

    def demo_form(att, bias):
        att = att * 0.25
        att = att.masked_fill(bias[:, :, :T, :T] == 0, float("-inf"))
        return torch.softmax(att, dim=-1)

    def hf_form(att, keep):
        att = att / 4.0
        att = torch.where(keep, att, torch.full([], -1e9))
        return torch.nn.functional.softmax(att, dim=-1)

    g = torch.Generator().manual_seed(0)
    att = torch.randn(2, 3, T, T, generator=g)
    for fn, second, entry in ((demo_form, tril, ("softmax_masked", float("-inf"), 0.25, False)),
                              (hf_form, tril.bool(), ("softmax_masked", -1e9, 0.25, True))):
        torch._dynamo.reset()
        stand_ins.calls.clear()
        with torch.no_grad():
            got = torch.compile(fn, backend=mojo_backend)(att, second)
        torch.testing.assert_close(got, fn(att, second))
        assert stand_ins.calls == [entry]


def test_masked_softmax_is_left_alone_when_the_mask_varies_over_heads(stand_ins):
    """A mask with a real head dimension is not one [T, S] matrix: the chain stays unfused."""
    g = torch.Generator().manual_seed(1)
    att = torch.randn(2, 3, 8, 8, generator=g)
    mask = torch.rand(1, 3, 8, 8, generator=g) > 0.5
    mask[..., 0] = False

    def fn(att, mask):
        return torch.softmax(att.masked_fill(mask, float("-inf")), dim=-1)

    with torch.no_grad():
        got = torch.compile(fn, backend=mojo_backend)(att, mask)
    torch.testing.assert_close(got, fn(att, mask))
    assert not [c for c in stand_ins.calls if c[0] == "softmax_masked"]


def test_export_with_frozen_weights_matches_eager(stand_ins):
    """export_to_max_graph: parameters and buffers become plan constants, only the user inputs
    are passed at run time, a [K, N]-contiguous weight used directly by mm is repacked K-major,
    and the result equals eager."""
    from torch_mojo_backend.torch_compile_backend.exporter import export_to_max_graph

    class Net(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.fc = torch.nn.Linear(16, 32)
            self.ln = torch.nn.LayerNorm(32)
            self.conv1d_weight = torch.nn.Parameter(torch.randn(32, 24) * 0.1)  # [K, N] like HF Conv1D
            self.register_buffer("shift", torch.arange(24, dtype=torch.float32) * 0.01)

        def forward(self, x):
            h = self.ln(F.gelu(self.fc(x), approximate="tanh"))
            return h @ self.conv1d_weight + self.shift, h.sum(-1)

    torch.manual_seed(0)
    net = Net().eval()
    x = torch.randn(5, 16)
    exported = export_to_max_graph(net, (x,))
    assert exported.num_user_inputs == 1
    frozen = [c for _, c in exported.plan.constants]
    assert len(frozen) == 6  # fc.weight, fc.bias, ln.weight, ln.bias, conv1d_weight, shift
    repacked = [c for c in frozen if c.shape == (32, 24)]
    assert repacked and repacked[0].stride() == (1, 32), "the [K, N] weight is stored K-major"
    with torch.no_grad():
        want = net(x)
    got = exported.execute(x)
    for g, w in zip(got, want):
        torch.testing.assert_close(g, w, rtol=1e-5, atol=1e-5)
    x2 = torch.randn(5, 16)
    with torch.no_grad():
        torch.testing.assert_close(exported(x2)[0], net(x2)[0], rtol=1e-5, atol=1e-5)
    with pytest.raises(TypeError, match="expected 1 inputs"):
        exported.execute(x, x)


def test_fp32_gemm_precision_levels_wiring(stand_ins, monkeypatch):
    """fp32 mm / addmm: "highest" and "high" hand the fp32 operands to one b200 GEMM call (whose own
    routing puts all but small products on the tensor cores in split precision), "medium" rounds
    the operands to bf16 first, and TORCH_MOJO_BACKEND_EXACT_FP32 pins the exact CUDA-core route."""
    g = torch.Generator().manual_seed(0)
    a, b, bias = torch.randn(256, 512, generator=g), torch.randn(512, 192, generator=g) * 0.05, torch.randn(192, generator=g)
    want = torch.addmm(bias.double(), a.double(), b.double()).float()
    seen = []
    real_gemm = stand_ins.gemm

    def spy(a_, b_, *rest):
        seen.append((a_.dtype, rest[6] if len(rest) > 6 else 0))
        return real_gemm(a_, b_, *rest)

    monkeypatch.setattr(stand_ins, "gemm", staticmethod(spy))
    old = torch.get_float32_matmul_precision()
    try:
        for level, dtype, tol in (("highest", torch.float32, 1e-5), ("high", torch.float32, 1e-5), ("medium", torch.bfloat16, 2e-2)):
            torch.set_float32_matmul_precision(level)
            seen.clear()
            got = af.aten_addmm(bias, a, b)
            assert seen == [(dtype, 0)], level
            assert got.dtype == torch.float32
            assert (got - want).abs().max().item() <= tol * want.abs().max().item()
        monkeypatch.setenv("TORCH_MOJO_BACKEND_EXACT_FP32", "1")
        seen.clear()
        af.aten_mm(a, b)
        assert seen == [(torch.float32, native.ROUTE_SIMT)]
    finally:
        torch.set_float32_matmul_precision(old)
