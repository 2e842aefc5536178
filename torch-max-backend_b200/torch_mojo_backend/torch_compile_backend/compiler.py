"""`torch.compile(backend=mojo_backend)`: lowers an aten FX graph to a launch plan of CUDA kernels.

Public surface and control flow follow the reference backend
(torch_mojo_backend/torch_compile_backend/compiler.py): `mojo_backend(gm, example_inputs)` wraps
AOTAutograd with the trimmed `DECOMPOSITION_TABLE` (:573-583); its forward compiler builds the
graph once (`BaseMaxCompiler.__init__`, :455-481) by walking the FX nodes and calling
`MAPPING_TORCH_ATEN_TO_MOJO[target](*args, **kwargs)` for each (`_GraphFactory`, :153-403), and
every later call marshals inputs, executes, and rebuilds the outputs from a blueprint
(`__call__` / `reconstruct_from_blueprint`, :483-532).

The difference is the thing being built. The reference builds a MAX graph and lets MAX compile
and run it. Here the walk produces a `LaunchPlan`: a flat list of steps, each a registry function
bound to value slots. At compile time the walk executes every step once on the FakeTensors that
AOTAutograd recorded (`node.meta["val"]`), so an unsupported op or a failing lowering is reported
as a `MojoCompilerError` before anything runs on the GPU, with the same message contract as the
reference (:287-306). At run time the plan is replayed on the real CUDA tensors: the registry
functions enqueue kernels from libb200ops on the current stream; nothing is traced again.
"""

from __future__ import annotations

import datetime as dt
import operator
import time
import traceback
from dataclasses import dataclass, field
from enum import Enum
from typing import Any

import torch
from functorch.compile import make_boxed_func
from torch._dynamo.backends.common import aot_autograd

from torch_mojo_backend.aten_functions import (
    CURRENT_FX_NODE,
    DECOMPOSITION_TABLE,
    MAPPING_TORCH_ATEN_TO_MOJO,
)
from torch_mojo_backend.flags import cuda_graphs_enabled, profiling_enabled, verbose_enabled
from torch_mojo_backend.torch_compile_backend import debug, fusion
from torch_mojo_backend.torch_compile_backend.utils import (
    get_accelerators,
    get_error_message,
    get_fully_qualified_name,
)

__all__ = [
    "MAPPING_TORCH_ATEN_TO_MOJO",
    "MojoCompilerError",
    "get_accelerators",
    "mojo_backend",
    "BaseMaxCompiler",
]


class MojoCompilerError(Exception):
    pass


def gather_stats_on_graph(gm: torch.fx.GraphModule):
    """Print how often each function appears in the graph, most frequent first."""
    function_counts: dict[str, int] = {}
    for node in gm.graph.nodes:
        if node.op in ("call_function", "call_method"):
            name = get_fully_qualified_name(node.target)
            function_counts[name] = function_counts.get(name, 0) + 1
    print("Function call counts:")
    for name, count in sorted(function_counts.items(), key=lambda x: x[1], reverse=True):
        print(f"{name}: {count}")


class _Ref:
    """Marks a position in a step's arguments that is filled from a value slot at run time."""

    __slots__ = ("slot",)

    def __init__(self, slot: int):
        self.slot = slot

    def __repr__(self):
        return f"%{self.slot}"


class TensorsBook:
    """Node name -> value slot, plus the compile-time (fake) value of every node.

    `convert_to_max` keeps the reference's name (compiler.py:89-129): it turns an FX argument
    structure into what a registry function receives. Here it is used for the compile-time dry
    run, so nodes resolve to their FakeTensor / SymInt values.
    """

    def __init__(self):
        self.slots: dict[str, int] = {}
        self.tensors: dict[str, Any] = {}

    def __setitem__(self, name: str, value):
        self.tensors[name] = value

    def slot_of(self, node: torch.fx.Node) -> int:
        if node.name not in self.slots:
            self.slots[node.name] = len(self.slots)
        return self.slots[node.name]

    def convert_to_max(self, something):
        if isinstance(something, torch.fx.Node):
            value = self.tensors[something.name]
            if isinstance(value, NotImplementedError):
                raise value
            return value
        if isinstance(something, (str, int, float, bool)) or something is None:
            return something
        if isinstance(something, slice):
            return slice(
                self.convert_to_max(something.start),
                self.convert_to_max(something.stop),
                self.convert_to_max(something.step),
            )
        if isinstance(something, (list, torch.fx.immutable_collections.immutable_list)):
            return [self.convert_to_max(x) for x in something]
        if isinstance(something, tuple):
            return tuple(self.convert_to_max(x) for x in something)
        if isinstance(something, (torch.device, torch.dtype, torch.layout, torch.memory_format)):
            return something
        if isinstance(something, NotImplementedError):
            raise something
        if something is ...:
            return ...
        if isinstance(something, (torch.nn.Module, torch._ops.OpOverload)):
            return something
        raise ValueError(f"Unsupported type when reading the graph: {type(something)}")

    def to_spec(self, something):
        """Same traversal, but nodes become `_Ref(slot)` placeholders for run-time binding."""
        if isinstance(something, torch.fx.Node):
            return _Ref(self.slots[something.name])
        if isinstance(something, slice):
            return slice(self.to_spec(something.start), self.to_spec(something.stop), self.to_spec(something.step))
        if isinstance(something, (list, torch.fx.immutable_collections.immutable_list)):
            return [self.to_spec(x) for x in something]
        if isinstance(something, tuple):
            return tuple(self.to_spec(x) for x in something)
        return something


def _has_ref(spec) -> bool:
    if isinstance(spec, _Ref):
        return True
    if isinstance(spec, (list, tuple)):
        return any(_has_ref(x) for x in spec)
    if isinstance(spec, slice):
        return _has_ref(spec.start) or _has_ref(spec.stop) or _has_ref(spec.step)
    return False


def _bind(spec, env):
    if isinstance(spec, _Ref):
        value = env[spec.slot]
        if isinstance(value, NotImplementedError):
            raise value
        return value
    if isinstance(spec, list):
        return [_bind(x, env) for x in spec]
    if isinstance(spec, tuple):
        return tuple(_bind(x, env) for x in spec)
    if isinstance(spec, slice):
        return slice(_bind(spec.start, env), _bind(spec.stop, env), _bind(spec.step, env))
    return spec


def fetch_attr(gm: torch.fx.GraphModule, target: str):
    """Fetch a (dotted) attribute from the module hierarchy of `gm`."""
    attr_itr = gm
    atoms = target.split(".")
    for i, atom in enumerate(atoms):
        if not hasattr(attr_itr, atom):
            raise RuntimeError(f"Node referenced nonexistent target {'.'.join(atoms[: i + 1])}")
        attr_itr = getattr(attr_itr, atom)
    return attr_itr


class OutputBlueprintKind(Enum):
    NONE = 1
    TENSOR = 2
    DIM = 3


@dataclass
class Step:
    fn: Any
    args: tuple
    kwargs: dict
    out_slot: int
    node: torch.fx.Node | None
    needs_node: bool
    dynamic_args: bool  # any _Ref inside args/kwargs
    release: tuple = ()  # slots whose last use is this step


@dataclass
class LaunchPlan:
    """What `create_graph` returns in place of a MAX graph: an ordered list of bound steps."""

    num_slots: int = 0
    input_slots: list[int | None] = field(default_factory=list)  # per placeholder, None = unused
    constants: list[tuple[int, Any]] = field(default_factory=list)
    steps: list[Step] = field(default_factory=list)
    output_slots: list[int] = field(default_factory=list)

    def run(self, flat_args) -> list:
        env: list[Any] = [None] * self.num_slots
        for slot, value in zip(self.input_slots, flat_args):
            if slot is not None:
                env[slot] = value
        for slot, value in self.constants:
            env[slot] = value
        for step in self.steps:
            if step.dynamic_args:
                args = _bind(step.args, env)
                kwargs = {k: _bind(v, env) for k, v in step.kwargs.items()} if step.kwargs else {}
            else:
                args, kwargs = step.args, step.kwargs
            if step.needs_node:
                token = CURRENT_FX_NODE.set(step.node)
                try:
                    env[step.out_slot] = step.fn(*args, **kwargs)
                finally:
                    CURRENT_FX_NODE.reset(token)
            else:
                env[step.out_slot] = step.fn(*args, **kwargs)
            for slot in step.release:
                env[slot] = None
        return [env[s] for s in self.output_slots]

    def __str__(self):
        lines = [f"LaunchPlan({len(self.steps)} steps, {self.num_slots} slots)"]
        for i, step in enumerate(self.steps):
            name = getattr(step.fn, "__name__", str(step.fn))
            lines.append(f"  {i:4d}: %{step.out_slot} = {name}{step.args} {step.kwargs or ''}")
        lines.append(f"  outputs: {self.output_slots}")
        return "\n".join(lines)


class _GraphFactory:
    """Walks one FX graph and builds its LaunchPlan (one instance per graph).

    `replace_inputs` maps placeholder names to tensors that become plan constants instead of
    call arguments (frozen parameters; reference: compiler.py:153-176 and exporter.py).
    """

    def __init__(self, replace_inputs: dict[str, torch.Tensor] | None = None, validate: bool = True):
        self.tensor_book = TensorsBook()
        self.plan = LaunchPlan()
        self.replace_inputs = replace_inputs or {}
        self.validate = validate
        self.fake_mode = None

    # -- placeholders ---------------------------------------------------------------------
    def handle_placeholder(self, node: torch.fx.Node):
        slot = self.tensor_book.slot_of(node)
        example_value = node.meta.get("example_value", node.meta.get("val"))
        self.tensor_book[node.name] = example_value
        if node.name in self.replace_inputs:
            self.plan.constants.append((slot, self.replace_inputs[node.name]))
            self.plan.input_slots.append(None)
            return
        if isinstance(example_value, torch.Tensor) and self.fake_mode is None:
            self.fake_mode = getattr(example_value, "fake_mode", None)
        self.plan.input_slots.append(slot)

    # -- call_function / call_method ------------------------------------------------------
    def handle_call_function(self, node_idx: int, node: torch.fx.Node):
        book = self.tensor_book
        func_args = [book.convert_to_max(x) for x in node.args]
        func_kwargs = {k: book.convert_to_max(v) for k, v in node.kwargs.items()}
        spec_args = tuple(book.to_spec(x) for x in node.args)
        spec_kwargs = {k: book.to_spec(v) for k, v in node.kwargs.items()}

        if isinstance(node.target, torch._higher_order_ops.auto_functionalize.AutoFunctionalizedV2):
            # A user custom op kept in the graph (no graph break): registered under its
            # "namespace.name" string, called with the mutated bases first, then the inputs
            # (reference: compiler.py:262-277).
            key = str(func_args[0]).removesuffix(".default")
            if key not in MAPPING_TORCH_ATEN_TO_MOJO:
                raise MojoCompilerError(
                    "The custom op is not supported by the Mojo backend yet. "
                    + get_error_message(node, node_idx, func_args, func_kwargs)
                    + "You can register it in the MAPPING_TORCH_ATEN_TO_MOJO dictionary under "
                    f"the key {key!r}."
                )
            mapping_func = MAPPING_TORCH_ATEN_TO_MOJO[key]
            visible = [k for k in node.kwargs if not k.startswith("_")]
            spec_args = (*spec_kwargs["_all_bases"], *[spec_kwargs[k] for k in visible])
            func_args = [*func_kwargs["_all_bases"], *[func_kwargs[k] for k in visible]]
            spec_kwargs, func_kwargs = {}, {}
        else:
            key = node.target
            if key not in MAPPING_TORCH_ATEN_TO_MOJO and getattr(key, "overloadpacket", None) in MAPPING_TORCH_ATEN_TO_MOJO:
                key = key.overloadpacket
            if key not in MAPPING_TORCH_ATEN_TO_MOJO:
                raise MojoCompilerError(
                    "The aten function is not supported by the Mojo backend yet. "
                    + get_error_message(node, node_idx, func_args, func_kwargs)
                    + "You can try to write it yourself and insert it in the MAPPING_TORCH_ATEN_TO_MOJO dictionary."
                )
            mapping_func = MAPPING_TORCH_ATEN_TO_MOJO[key]

        # Shape glue registered for a whole packet is bound to the node's exact overload.
        run_func = mapping_func
        passthrough = getattr(mapping_func, "passthrough_of", None)
        if passthrough is not None and isinstance(node.target, torch._ops.OpOverload):
            run_func = node.target

        if self.validate:
            try:
                token = CURRENT_FX_NODE.set(node)
                try:
                    func_output = self._dry_run(mapping_func, func_args, func_kwargs)
                finally:
                    CURRENT_FX_NODE.reset(token)
                self._check_against_trace(node, func_output)
            except Exception as e:
                raise MojoCompilerError(
                    get_error_message(node, node_idx, func_args, func_kwargs)
                    + "There was an error when executing the function. See the original error below. \n"
                    f"{e}\n"
                    f"{traceback.format_exc()}"
                )
        else:
            func_output = node.meta.get("val")

        slot = book.slot_of(node)
        book[node.name] = func_output
        needs_node = passthrough is None and run_func not in (operator.getitem,)
        self.plan.steps.append(
            Step(
                fn=run_func,
                args=spec_args,
                kwargs=spec_kwargs,
                out_slot=slot,
                node=node,
                needs_node=needs_node,
                dynamic_args=_has_ref(spec_args) or _has_ref(tuple(spec_kwargs.values())),
            )
        )

    def _dry_run(self, mapping_func, func_args, func_kwargs):
        if self.fake_mode is not None:
            with self.fake_mode:
                return mapping_func(*func_args, **func_kwargs)
        return mapping_func(*func_args, **func_kwargs)

    @staticmethod
    def _check_against_trace(node: torch.fx.Node, produced):
        """The lowering must produce what AOTAutograd recorded for the node: same shape and dtype
        for every tensor that is present in both."""
        traced = node.meta.get("val")
        if traced is None:
            return
        pairs = []
        if isinstance(traced, torch.Tensor):
            pairs.append((traced, produced))
        elif isinstance(traced, (tuple, list)) and isinstance(produced, (tuple, list)):
            pairs.extend(zip(traced, produced))
        for want, got in pairs:
            if not isinstance(want, torch.Tensor) or not isinstance(got, torch.Tensor):
                continue
            if tuple(want.shape) != tuple(got.shape) or want.dtype != got.dtype:
                raise RuntimeError(
                    f"lowering produced {tuple(got.shape)} {got.dtype} where the traced graph has "
                    f"{tuple(want.shape)} {want.dtype}"
                )

    # -- get_attr -------------------------------------------------------------------------
    def handle_get_attr(self, node: torch.fx.Node):
        attr_value = fetch_attr(node.graph.owning_module, node.target)
        slot = self.tensor_book.slot_of(node)
        self.plan.constants.append((slot, attr_value))
        fake_value = attr_value
        if isinstance(attr_value, torch.Tensor):
            fake_value = node.meta.get("val")
            if fake_value is None and self.fake_mode is not None:
                fake_value = self.fake_mode.from_tensor(attr_value)
            elif fake_value is None:
                fake_value = attr_value
        self.tensor_book[node.name] = fake_value

    # -- output ---------------------------------------------------------------------------
    def handle_output(self, node: torch.fx.Node) -> list[tuple[OutputBlueprintKind, int | None]]:
        """Returns the blueprint of the final output list: NONE (a None is required there),
        TENSOR or DIM (an int computed from shapes), with the index into the plan's outputs
        (reference: compiler.py:329-369)."""
        blueprint: list[tuple[OutputBlueprintKind, int | None]] = []
        for x in node.args[0]:
            if x is None:
                blueprint.append((OutputBlueprintKind.NONE, None))
                continue
            if not isinstance(x, torch.fx.Node):
                # A python constant required as an output: carried as a plan constant.
                slot = len(self.tensor_book.slots)
                self.tensor_book.slots[f"__const_out_{slot}"] = slot
                self.plan.constants.append((slot, x))
                blueprint.append((OutputBlueprintKind.DIM, len(self.plan.output_slots)))
                self.plan.output_slots.append(slot)
                continue
            value = self.tensor_book.tensors[x.name]
            if isinstance(value, NotImplementedError):
                raise value
            kind = OutputBlueprintKind.TENSOR if isinstance(value, torch.Tensor) else OutputBlueprintKind.DIM
            if value is None:
                blueprint.append((OutputBlueprintKind.NONE, None))
                continue
            blueprint.append((kind, len(self.plan.output_slots)))
            self.plan.output_slots.append(self.tensor_book.slots[x.name])
        return blueprint

    def create_graph(self, graph: torch.fx.Graph):
        output_blueprint = None
        for node_idx, node in enumerate(graph.nodes):
            if node.op == "placeholder":
                self.handle_placeholder(node)
            elif node.op in ("call_function", "call_method"):
                self.handle_call_function(node_idx, node)
            elif node.op == "get_attr":
                self.handle_get_attr(node)
            elif node.op == "output":
                output_blueprint = self.handle_output(node)
            else:
                raise ValueError(f"Unsupported node type: {node.op}")
        if output_blueprint is None:
            raise ValueError("No output node found in the graph, this should never happen.")
        self._finish_plan()
        return self.plan, output_blueprint

    def _finish_plan(self):
        """Slot lifetimes: each slot is dropped after its last reader so that intermediate
        activations return to the caching allocator as early as in eager execution."""
        plan = self.plan
        plan.num_slots = len(self.tensor_book.slots)
        last_use: dict[int, int] = {}

        def visit(spec, idx):
            if isinstance(spec, _Ref):
                last_use[spec.slot] = idx
            elif isinstance(spec, (list, tuple)):
                for x in spec:
                    visit(x, idx)
            elif isinstance(spec, slice):
                visit(spec.start, idx), visit(spec.stop, idx), visit(spec.step, idx)

        for idx, step in enumerate(plan.steps):
            visit(step.args, idx)
            visit(tuple(step.kwargs.values()), idx)
            last_use.setdefault(step.out_slot, idx)
        keep = set(plan.output_slots) | {s for s, _ in plan.constants}
        releases: dict[int, list[int]] = {}
        for slot, idx in last_use.items():
            if slot not in keep:
                releases.setdefault(idx, []).append(slot)
        for idx, slots in releases.items():
            plan.steps[idx].release = tuple(slots)


class BaseMaxCompiler:
    """Forward compiler handed to AOTAutograd: builds the plan once, replays it per call."""

    def __init__(self, gm: torch.fx.GraphModule, example_inputs: list, mode=None):
        self.gm = gm
        if profiling_enabled():
            compiler_start = time.time_ns()
        if verbose_enabled():
            print(f"Graph has {len(gm.graph.nodes)} nodes.")
            gather_stats_on_graph(gm)
            gm.graph.print_tabular()

        if fusion.fusion_enabled():
            fusion_stats = fusion.fuse_graph(gm)
            if verbose_enabled():
                print(f"Fused chains: {fusion_stats}")
        self.plan, self.output_blueprint = _GraphFactory().create_graph(gm.graph)
        self._graph_runner = None
        if verbose_enabled():
            print(self.plan)
        if profiling_enabled():
            defining = dt.timedelta(microseconds=(time.time_ns() - compiler_start) / 1000)
            print(f"Defining the launch plan in {defining}")

    def reconstruct_from_blueprint(self, plan_outputs: list) -> list[torch.Tensor | int | float | None]:
        result = []
        for kind, index in self.output_blueprint:
            if kind is OutputBlueprintKind.NONE:
                result.append(None)
            else:
                result.append(plan_outputs[index])
        return result

    def __call__(self, *args) -> list[torch.Tensor | int | float | None]:
        if profiling_enabled():
            start_inference_time = time.time_ns()
        if cuda_graphs_enabled():
            from torch_mojo_backend.torch_compile_backend.graph_replay import GraphRunner

            if self._graph_runner is None:
                self._graph_runner = GraphRunner(self.plan)
            outputs = self._graph_runner.run(args)
        else:
            outputs = self.plan.run(args)
        debug.debug_graph_if_required(self.gm, args, outputs, self.plan)
        result = self.reconstruct_from_blueprint(outputs)
        if profiling_enabled():
            duration = dt.timedelta(microseconds=(time.time_ns() - start_inference_time) / 1000)
            print(f"Running the launch plan in {duration} (host time; kernels run asynchronously)")
        return result


def boxed_func(*args, **kwargs):
    return make_boxed_func(BaseMaxCompiler(*args, **kwargs).__call__)


class mojo_backend:
    """Pass as `torch.compile(model, backend=mojo_backend)`."""

    def __init__(self, gm: torch.fx.GraphModule, example_inputs: list):
        self.func_to_execute = aot_autograd(fw_compiler=boxed_func, decompositions=DECOMPOSITION_TABLE)(
            gm, example_inputs
        )

    def __call__(self, *args) -> list[torch.Tensor | int | float | None]:
        result = self.func_to_execute(*args)
        if isinstance(result, tuple):
            return list(result)
        return result


def dummy_compiler(gm: torch.fx.GraphModule, example_inputs: list):
    return make_boxed_func(gm.forward)


# Runs the same AOTAutograd pipeline on stock torch ops: tells backend faults from tracing faults.
dummy_backend = aot_autograd(fw_compiler=dummy_compiler)
