"""The parity helpers of torch_mojo_backend.testing on graphs that are shape glue only (views, slices,
integer arithmetic: stock torch ops on any device), so they run without a GPU."""

import pytest
import torch

from torch_mojo_backend.testing import Conf, check_functions_are_equivalent, check_outputs, to_device


def glue(x):
    return x.reshape(-1)[::2] + 1


def two_outputs(x, y):
    return x.t().contiguous(), (y * 2).view(-1)


def test_check_functions_are_equivalent_passes_and_fails():
    x = torch.arange(24, dtype=torch.int64).reshape(4, 6)
    check_functions_are_equivalent(glue, "cpu", [x])
    check_functions_are_equivalent(two_outputs, None, [x, torch.arange(6)])
    with pytest.raises(AssertionError):
        check_functions_are_equivalent(glue, "cpu", [x], fn_compiled=lambda t: t.reshape(-1)[::2] + 2)
    with pytest.raises(AssertionError, match="dtype"):
        check_functions_are_equivalent(glue, "cpu", [x], fn_compiled=lambda t: (t.reshape(-1)[::2] + 1).int())
    with pytest.raises(AssertionError, match="shape"):
        check_functions_are_equivalent(glue, "cpu", [x], fn_compiled=lambda t: t.reshape(-1)[::3] + 1)


def test_check_outputs_runs_both_ways_against_cpu_eager():
    x = torch.arange(24, dtype=torch.int64).reshape(4, 6)
    for conf in (Conf("cpu", False), Conf("cpu", True)):
        check_outputs(glue, conf, [x])
        check_outputs(two_outputs, conf, [x, torch.arange(6)])
    assert str(Conf("cuda", True)) == "cuda, compiled" and str(Conf("cpu", False)) == "cpu, eager"

    def with_device(t, device):
        return t + torch.ones(1, dtype=t.dtype, device=device)

    check_outputs(with_device, Conf("cpu", True), [x])


def test_to_device_copies():
    x = torch.zeros(3)
    (y,) = to_device([x], "cpu")
    y += 1
    assert float(x.sum()) == 0.0
