"""torch.export front end: one launch plan per module with its weights frozen in.

Mirror of the reference's `export_to_max_graph`
(torch_mojo_backend/torch_compile_backend/exporter.py:17-35): `torch.export.export(strict=True)`,
the same decomposition table as the `torch.compile` path, parameters embedded as graph constants,
the same FX walk (`_GraphFactory(replace_inputs)`). Where the reference hands the graph to MAX and
returns a `max.engine.Model`, this returns an `ExportedPlan` whose `execute(*inputs)` replays the
launch plan on the b200 kernels. Differences, all supersets: buffers and lifted tensor constants
are frozen as well as parameters (the reference leaves them as inputs), the fusion pass runs on
the exported graph, `[K, N]`-contiguous weights that feed a GEMM directly (HF Conv1D layout) are
repacked once to K-major so that every large GEMM takes the CTA-pair tensor-core kernel, and the
plan can be replayed from a CUDA graph.
"""

from __future__ import annotations

import torch
import torch.export
from torch.export.graph_signature import InputKind

from torch_mojo_backend.aten_functions import DECOMPOSITION_TABLE
from torch_mojo_backend.torch_compile_backend import fusion
from torch_mojo_backend.torch_compile_backend.compiler import OutputBlueprintKind, _GraphFactory

aten = torch.ops.aten

_FROZEN_KINDS = (InputKind.PARAMETER, InputKind.BUFFER, InputKind.CONSTANT_TENSOR)


class ExportedPlan:
    """A frozen-weights launch plan. `execute(*inputs)` (also `__call__`) takes the module's
    positional inputs and returns the list of its outputs, like `max.engine.Model.execute`."""

    def __init__(self, plan, output_blueprint, num_user_inputs: int, cuda_graph: bool):
        self.plan = plan
        self.output_blueprint = output_blueprint
        self.num_user_inputs = num_user_inputs
        self._runner = None
        self._cuda_graph = cuda_graph

    def execute(self, *inputs) -> list:
        if len(inputs) != self.num_user_inputs:
            raise TypeError(f"expected {self.num_user_inputs} inputs, got {len(inputs)}")
        # frozen placeholders take no argument: their positions are None in plan.input_slots
        it = iter(inputs)
        flat = [None if slot is None else next(it) for slot in self.plan.input_slots]
        if self._cuda_graph:
            from torch_mojo_backend.torch_compile_backend.graph_replay import GraphRunner

            if self._runner is None:
                self._runner = GraphRunner(self.plan)
            outputs = self._runner.run(flat)
        else:
            outputs = self.plan.run(flat)
        return [None if kind is OutputBlueprintKind.NONE else outputs[index] for kind, index in self.output_blueprint]

    __call__ = execute


def _repack_gemm_weights(graph: torch.fx.Graph, frozen: dict[str, torch.Tensor]) -> int:
    """Frozen 2-D weights used directly as the B operand of mm / addmm in `[K, N]`-contiguous
    layout are re-stored K-major (same shape and values, strides (1, K))."""
    count = 0
    for node in graph.nodes:
        if node.op != "call_function" or node.target not in (aten.mm.default, aten.addmm.default):
            continue
        b = node.args[1] if node.target is aten.mm.default else node.args[2]
        if not isinstance(b, torch.fx.Node) or b.op != "placeholder" or b.name not in frozen:
            continue
        w = frozen[b.name]
        if w.dim() == 2 and w.is_contiguous() and w.shape[0] > 1 and w.shape[1] > 1 and len(b.users) == 1:
            frozen[b.name] = w.t().contiguous().t()
            count += 1
    return count


def export_to_max_graph(
    model: torch.nn.Module, example_inputs: tuple[torch.Tensor, ...], force_device=None, cuda_graph: bool = False
) -> ExportedPlan:
    """Exports `model` with its weights frozen. `force_device` (a torch device or string) is where
    the frozen weights are placed; by default they stay where the module has them."""
    exported_program = torch.export.export(model, example_inputs, strict=True)
    with torch.no_grad():
        exported_program = exported_program.run_decompositions(decomp_table=DECOMPOSITION_TABLE)
    state = dict(model.state_dict(keep_vars=False))
    state.update(dict(model.named_buffers()))  # non-persistent buffers are not in the state dict
    constants = getattr(exported_program, "constants", {})
    frozen: dict[str, torch.Tensor] = {}
    num_user_inputs = 0
    for spec in exported_program.graph_signature.input_specs:
        if spec.kind == InputKind.USER_INPUT:
            num_user_inputs += 1
            continue
        if spec.kind not in _FROZEN_KINDS:
            continue
        value = state.get(spec.target)
        if value is None:
            value = constants.get(spec.target)
        if value is None:
            raise KeyError(f"no value for exported input {spec.arg.name!r} (target {spec.target!r})")
        value = value.detach()
        if force_device is not None:
            value = value.to(force_device)
        frozen[spec.arg.name] = value

    gm = exported_program.graph_module
    # repack first: the fusion pass rewrites mm / addmm nodes into fused nodes this pass does not match
    _repack_gemm_weights(gm.graph, frozen)
    if fusion.fusion_enabled():
        fusion.fuse_graph(gm)
    plan, blueprint = _GraphFactory(frozen).create_graph(gm.graph)
    return ExportedPlan(plan, blueprint, num_user_inputs, cuda_graph)
