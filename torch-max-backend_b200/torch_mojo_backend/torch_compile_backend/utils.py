"""Helpers of the compile backend: device listing and the error-message contract
(reference: torch_mojo_backend/torch_compile_backend/utils.py)."""

from __future__ import annotations

from collections.abc import Callable

import torch

ISSUES_URL = "https://github.com/gabrieldemarmiesse/torch-mojo-backend/issues"


def get_accelerators() -> list[torch.device]:
    """The devices this backend can run on: every visible CUDA device. (The reference appends a
    CPU device so that `mojo:0` always resolves; this backend has no CPU execution path.)"""
    if not torch.cuda.is_available():
        return []
    return [torch.device("cuda", i) for i in range(torch.cuda.device_count())]


def get_fully_qualified_name(func: Callable | str) -> str:
    if isinstance(func, str):
        return f"torch.Tensor.{func}"
    result = ""
    if hasattr(func, "__module__"):
        result += func.__module__ + "."
    if hasattr(func, "__qualname__"):
        result += func.__qualname__
    result += " of type " + str(type(func)) + " "
    return result


def get_error_message(node: torch.fx.Node, node_idx: int, func_args, func_kwargs) -> str:
    if node.stack_trace is None:
        stack_trace = "No stack trace available, likely because this node is the result of a decomposition."
    else:
        stack_trace = node.stack_trace
    return (
        f"Failing at node {node_idx} when executing function {get_fully_qualified_name(node.target)}. "
        f"inputs of node were: args={func_args}, kwargs={func_kwargs}. "
        f"You can open an issue at {ISSUES_URL} . "
        f"It comes from there in your code: \n"
        f"{stack_trace}\n"
    )
