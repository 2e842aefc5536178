"""Environment switches, same names and meaning as the reference (torch_mojo_backend/flags.py):
TORCH_MOJO_BACKEND_PROFILE / _VERBOSE / _DEBUG_GRAPH, also accepted with a PYTORCH_ prefix."""

import os

POSITIVE_VALUES = ("1", "true", "yes")


def _flag(name: str) -> bool:
    for prefix in ("TORCH_", "PYTORCH_"):
        if os.environ.get(f"{prefix}MOJO_BACKEND_{name}", "0").lower() in POSITIVE_VALUES:
            return True
    return False


def profiling_enabled() -> bool:
    """Print plan-build and per-call times."""
    return _flag("PROFILE")


def verbose_enabled() -> bool:
    """Print the op histogram, the fx graph and the launch plan at compile time."""
    return _flag("VERBOSE")


def debug_graph() -> bool:
    """After every call, re-run the graph node by node on stock torch ops and compare."""
    return _flag("DEBUG_GRAPH")


def cuda_graphs_enabled() -> bool:
    """Replay static-shape plans from a captured CUDA graph (TORCH_MOJO_BACKEND_CUDA_GRAPHS=1)."""
    return _flag("CUDA_GRAPHS")
