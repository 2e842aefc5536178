"""TORCH_MOJO_BACKEND_DEBUG_GRAPH=1: after a call, re-run the FX graph node by node on stock torch
ops and report, per node, how far the launch plan's value is from it. Same purpose as the
reference's per-node comparison (torch_mojo_backend/torch_compile_backend/debug.py:23-128), without
the MAX print ops: both sides are torch tensors here, so they are compared directly."""

from __future__ import annotations

import torch

from torch_mojo_backend.flags import debug_graph


class _Recorder(torch.fx.Interpreter):
    def __init__(self, gm):
        super().__init__(gm)
        self.values: dict[str, object] = {}

    def run_node(self, n):
        out = super().run_node(n)
        self.values[n.name] = out
        return out


def _max_abs_diff(a, b) -> float | None:
    if isinstance(a, torch.Tensor) and isinstance(b, torch.Tensor) and a.shape == b.shape:
        if a.numel() == 0:
            return 0.0
        return (a.double() - b.double()).abs().max().item()
    return None


def compare_plan_with_reference(gm: torch.fx.GraphModule, args, plan) -> list[tuple[str, str, float]]:
    """Runs both executions and returns (node name, op, max abs difference) for tensor nodes."""
    from torch_mojo_backend.torch_compile_backend.compiler import _bind

    recorder = _Recorder(gm)
    recorder.run(*args)
    env = [None] * plan.num_slots
    for slot, value in zip(plan.input_slots, args):
        if slot is not None:
            env[slot] = value
    for slot, value in plan.constants:
        env[slot] = value
    report = []
    for step in plan.steps:
        a = _bind(step.args, env)
        kw = {k: _bind(v, env) for k, v in step.kwargs.items()}
        env[step.out_slot] = step.fn(*a, **kw)
        want = recorder.values.get(step.node.name) if step.node is not None else None
        got = env[step.out_slot]
        pairs = zip(want, got) if isinstance(want, (tuple, list)) and isinstance(got, (tuple, list)) else [(want, got)]
        for w, g in pairs:
            d = _max_abs_diff(w, g)
            if d is not None:
                report.append((step.node.name, str(step.node.target), d))
    return report


def debug_graph_if_required(gm: torch.fx.GraphModule, args, outputs=None, plan=None):
    if not debug_graph() or plan is None:
        return
    for name, op, diff in compare_plan_with_reference(gm, args, plan):
        print(f"[debug_graph] {name:40s} {op:50s} max|diff| = {diff:.3e}")
