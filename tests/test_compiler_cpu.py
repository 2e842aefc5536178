"""Host logic of the compile backend on a CPU-only box: registry semantics, the error-message
contract, the launch plan's bookkeeping (driven through shape-glue ops, which run on any device),
and compile-time lowering of whole GPT-2 graphs on FakeTensors. Kernels are never computed on the
CPU: graphs that contain them compile here but refuse to run."""

import operator

import pytest
import torch
import torch.nn.functional as F
from torch._dynamo.exc import BackendCompilerFailed

import torch_mojo_backend
from torch_mojo_backend import MAPPING_TORCH_ATEN_TO_MOJO, MojoCompilerError, mojo_backend
from torch_mojo_backend import aten_functions as af
from torch_mojo_backend.torch_compile_backend import compiler

aten = torch.ops.aten


@pytest.fixture(autouse=True)
def _reset(reset_compiler):
    yield


def test_public_surface():
    assert set(torch_mojo_backend.__all__) == {
        "mojo_backend", "get_accelerators", "MAPPING_TORCH_ATEN_TO_MOJO", "MojoCompilerError",
            "make_torch_op_from_mojo"}
    assert torch_mojo_backend.get_accelerators() == []  # no CUDA device here, and no CPU device is offered
    for op in (aten.mm, aten.addmm, aten.bmm, aten._softmax, aten.native_layer_norm, aten.gelu, aten.sum,
               aten.mean, aten.amax, aten._scaled_dot_product_flash_attention, operator.getitem):
        assert op in MAPPING_TORCH_ATEN_TO_MOJO


def test_mapped_ops_leave_the_decomposition_table():
    # packets: every overload is removed (reference tests/test_compiler.py:701-766)
    for overload in (aten._softmax.default, aten.gelu.default, aten.native_layer_norm.default, aten.addmm.default):
        assert overload not in af.DECOMPOSITION_TABLE
    # unmapped ops are still decomposed, e.g. the CPU flash-attention entry point
    assert aten._scaled_dot_product_flash_attention_for_cpu.default in af.DECOMPOSITION_TABLE
    assert af.number_of_decompositions_removed > 0


def test_map_to_single_overload_and_type_check(monkeypatch):
    table = dict(af.DECOMPOSITION_TABLE)
    monkeypatch.setattr(af, "DECOMPOSITION_TABLE", table)
    mapping = dict(MAPPING_TORCH_ATEN_TO_MOJO)
    monkeypatch.setattr(af, "MAPPING_TORCH_ATEN_TO_MOJO", mapping)
    assert aten.lerp.Scalar in table and aten.lerp.Tensor in table

    @af.map_to(aten.lerp.Scalar)
    def aten_lerp(x, end, weight):
        return x + weight * (end - x)

    assert aten.lerp.Scalar not in table and aten.lerp.Tensor in table
    assert mapping[aten.lerp.Scalar] is aten_lerp
    assert aten_lerp.call_count == 0  # test runs instrument lowerings with call counters
    with pytest.raises(TypeError):
        af.map_to("aten.lerp")(lambda x: x)


def test_error_message_op_not_supported(monkeypatch):
    monkeypatch.delitem(MAPPING_TORCH_ATEN_TO_MOJO, aten.add)

    def fn(x, y):
        return x + y

    with pytest.raises(BackendCompilerFailed) as exc_info:
        torch.compile(backend=mojo_backend)(fn)(torch.randn(2, 3), torch.randn(2, 3))
    msg = str(exc_info.value)
    assert "return x + y" in msg
    assert "torch._ops.aten.aten::add" in msg
    assert "https://github.com/gabrieldemarmiesse/torch-mojo-backend/issues" in msg
    assert "is not supported" in msg


def test_error_message_exception_in_op(monkeypatch):
    def not_working_add(x, y):
        raise RuntimeError("Ho no crash!")

    monkeypatch.setitem(MAPPING_TORCH_ATEN_TO_MOJO, aten.add, not_working_add)

    def fn(x, y):
        return x + y

    with pytest.raises(RuntimeError) as exc_info:
        torch.compile(backend=mojo_backend)(fn)(torch.randn(2, 3), torch.randn(2, 3))
    msg = str(exc_info.value)
    for needle in ("return x + y", "Ho no crash!", "torch._ops.aten.aten::add", "not_working_add",
                   "https://github.com/gabrieldemarmiesse/torch-mojo-backend/issues"):
        assert needle in msg, needle


def test_lowering_that_disagrees_with_the_trace_is_a_compile_error(monkeypatch):
    monkeypatch.setitem(MAPPING_TORCH_ATEN_TO_MOJO, aten.tanh, lambda x: x.double())
    with pytest.raises(RuntimeError, match="where the traced graph has"):
        torch.compile(backend=mojo_backend)(lambda x: x.tanh())(torch.randn(4))


def test_plan_runs_glue_graphs_and_returns_a_list():
    """Slots, constants, multiple outputs and None outputs, on ops that are pure shape glue."""

    def fn(x, y):
        z = (x + y).tanh().view(-1)
        a, b = z.split(3)
        return a * 2, b, x.t()

    x, y = torch.randn(2, 3), torch.randn(2, 3)
    out = torch.compile(backend=mojo_backend)(fn)(x, y)
    for got, want in zip(out, fn(x, y)):
        torch.testing.assert_close(got, want)

    gm = torch.fx.symbolic_trace(lambda x: (x + 1, None))
    backend_out = compiler.mojo_backend(gm, [torch.randn(3)])(torch.ones(3))
    assert isinstance(backend_out, list) and backend_out[1] is None
    torch.testing.assert_close(backend_out[0], torch.full((3,), 2.0))


def test_plan_releases_dead_values_and_keeps_outputs():
    def fn(x):
        a = x + 1
        b = a * 2
        c = b - 3
        return c, a

    holder = {}

    class Probe(compiler.BaseMaxCompiler):
        def __init__(self, gm, example_inputs):
            super().__init__(gm, example_inputs)
            holder["plan"] = self.plan

    def backend(gm, inputs):
        from functorch.compile import make_boxed_func
        from torch._dynamo.backends.common import aot_autograd

        return aot_autograd(fw_compiler=lambda g, i: make_boxed_func(Probe(g, i).__call__),
                            decompositions=af.DECOMPOSITION_TABLE)(gm, inputs)

    out = torch.compile(fn, backend=backend)(torch.zeros(4))
    torch.testing.assert_close(out[0], torch.full((4,), -1.0))
    plan = holder["plan"]
    released = [s for step in plan.steps for s in step.release]
    assert len(released) == len(set(released)), "a slot is released once"
    assert not set(released) & set(plan.output_slots), "outputs must survive"
    assert len(released) >= 1  # `b` dies after the subtraction


def test_get_attr_constants_and_dynamic_dim_output():
    const = torch.arange(3.0)

    def fn(x):
        return x + const, x.shape[0] * 2

    compiled = torch.compile(fn, backend=mojo_backend, dynamic=True)
    for n in (4, 7):
        x = torch.randn(n, 3)
        got, dim = compiled(x)
        torch.testing.assert_close(got, x + const)
        assert dim == 2 * n


def test_mark_dynamic_compiles_once():
    from torch._dynamo.testing import CompileCounterWithBackend

    counter = CompileCounterWithBackend(mojo_backend)

    def fn(x):
        return x * 2 + x.shape[0]

    compiled = torch.compile(fn, backend=counter)
    for n in (5, 9, 12):
        x = torch.randn(n, 3)
        torch._dynamo.mark_dynamic(x, 0)
        torch.testing.assert_close(compiled(x), fn(x))
    assert counter.frame_count == 1


@pytest.mark.parametrize("attention", ["sdpa", "masked_softmax"])
@pytest.mark.parametrize("precision", ["fp32", "bf16"])
def test_gpt2_graph_lowers_completely_and_refuses_cpu(attention, precision, capsys, monkeypatch):
    """Every node of the traced forward has a lowering (the compile-time dry run on FakeTensors
    passes), the hot ops stay whole, and running on CPU tensors is refused."""
    from demo_scripts.gpt2 import GPT2, GPTConfig

    monkeypatch.setenv("TORCH_MOJO_BACKEND_VERBOSE", "1")
    cfg = GPTConfig(vocab_size=211, block_size=32, n_layer=2, n_head=4, n_embd=64)
    model = GPT2(cfg, attention).init_weights(0).eval().set_precision(precision)
    ids = torch.randint(0, 211, (2, 16))
    with torch.no_grad(), pytest.raises(RuntimeError, match="no CPU fallback"):
        torch.compile(model, backend=mojo_backend)(ids)
    printed = capsys.readouterr().out
    for op in ("aten::addmm", "aten::native_layer_norm", "aten::gelu", "aten::mm", "aten::bmm", "aten::_softmax"):
        assert op in printed, f"{op} missing from the traced graph"
    assert "LaunchPlan(" in printed


def test_only_first_output_used_sees_the_current_node():
    seen = {}

    def fn(x, w, b):
        return F.layer_norm(x, (8,), w, b)

    original = MAPPING_TORCH_ATEN_TO_MOJO[aten.native_layer_norm]

    def spy(*args, **kwargs):
        seen["first_only"] = af._only_first_output_used()
        return original(*args, **kwargs)

    MAPPING_TORCH_ATEN_TO_MOJO[aten.native_layer_norm] = spy
    try:
        with torch.no_grad(), pytest.raises(RuntimeError, match="no CPU fallback"):
            torch.compile(fn, backend=mojo_backend)(torch.randn(4, 8), torch.randn(8), torch.randn(8))
    finally:
        MAPPING_TORCH_ATEN_TO_MOJO[aten.native_layer_norm] = original
    assert seen["first_only"] is True


@pytest.mark.parametrize("dtype", [torch.float16, torch.float64])
def test_hot_ops_refuse_floating_dtypes_without_a_kernel(dtype):
    """No silent trip through a vendor library: a float16 / float64 operand of one of the ops this
    backend exists for is an error in the lowering (which the graph walk turns into a
    MojoCompilerError while it builds the plan)."""
    from torch_mojo_backend import aten_functions as af

    x = torch.zeros((4, 8), dtype=dtype)
    for call in (
        lambda: af.aten_mm(x, x.t()),
        lambda: af.aten_addmm(x[:, :4], x, x.t()),
        lambda: af.aten_bmm(x[None], x.t()[None]),
        lambda: af.aten__softmax(x, -1, False),
        lambda: af.aten_native_layer_norm(x, [8], None, None, 1e-5),
        lambda: af.aten_gelu(x),
        lambda: af.aten_sum(x, [-1]),
        lambda: af.aten_mean(x, [-1]),
        lambda: af.aten_amax(x, [-1]),
        lambda: af.aten_scaled_dot_product_attention(x[None, None], x[None, None], x[None, None]),
    ):
        with pytest.raises(NotImplementedError, match="not supported by the b200 kernels"):
            call()


def test_glue_targets_of_the_reference_registry_run_through_the_backend():
    """Elementwise, fill, allocation and multi-tensor (optimizer) targets that the reference's registry
    names beside the hot ops: shape glue here (stock torch ops on any device), so a graph that uses
    them compiles instead of raising. Checked against eager on the CPU."""
    from torch_mojo_backend.testing import check_functions_are_equivalent

    def elementwise(x, y):
        a = torch.cos(x) + torch.sin(x) * torch.tan(x * 0.1) + torch.cosh(x * 0.1) - torch.sinh(x * 0.1)
        b = torch.acos(torch.clamp(x * 0.1, -0.9, 0.9)) + torch.asinh(x) + torch.atanh(torch.clamp(y * 0.1, -0.9, 0.9))
        c = torch.floor(x) + torch.ceil(y) + torch.sign(x) + torch.log1p(x.abs()) + torch.remainder(x, 1.5)
        return a + b + c, torch.isnan(x / y), torch.logical_xor(x > 0, y > 0), (x > 0).int() ^ (y > 0).int()

    def fills_and_pads(x, y):
        padded = torch.nn.functional.pad(x, (1, 2, 0, 1), value=-1.0)
        filled = torch.full_like(x, 0.0).fill_(3.0)
        scattered = torch.select_scatter(x, y[0], 0, 1)
        return padded, filled + torch.addcmul(x, x, y, value=0.5) + torch.addcdiv(x, x, y.abs() + 1.0, value=2.0), scattered

    def reductions(x, y):
        return x.var(dim=1), x.argmin(dim=1), torch.isin(x.int(), torch.tensor([0, 1, 2]))

    def optimizer_like(p0, p1, g0, g1):
        # what a compiled multi-tensor optimizer step is made of
        avg = torch._foreach_mul([g0, g1], 0.9)
        sq = torch._foreach_addcmul([p0.abs(), p1.abs()], [g0, g1], [g0, g1], 0.1)
        denom = torch._foreach_sqrt(torch._foreach_add(sq, 1e-8))
        step = torch._foreach_addcdiv([p0, p1], avg, denom, -0.01)
        step = torch._foreach_sub(step, torch._foreach_div(torch._foreach_neg(avg), 4.0))
        return tuple(torch._foreach_pow(torch._foreach_reciprocal(torch._foreach_add(torch._foreach_mul(step, step), 1.0)), 2.0))

    g = torch.Generator().manual_seed(5)
    x, y = torch.randn(4, 6, generator=g), torch.randn(4, 6, generator=g)
    for fn, inputs in ((elementwise, [x, y]), (fills_and_pads, [x, y]), (reductions, [x, y]),
                       (optimizer_like, [x, y, x * 0.5, y * 0.5])):
        torch._dynamo.reset()
        compiled = torch.compile(fn, backend=mojo_backend, fullgraph=True)
        check_functions_are_equivalent(fn, None, inputs, fn_compiled=compiled, rtol=1e-6, atol=1e-6)
