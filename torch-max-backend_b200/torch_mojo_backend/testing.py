"""Helpers for parity tests of compiled functions, with the names and argument meaning of the
reference's `torch_mojo_backend/testing.py:139-229`: the oracle is eager PyTorch, on the CPU for
`check_outputs` and on the inputs' own device for `check_functions_are_equivalent`.

Nothing here is used by the product path; tests and user code import it.
"""

from __future__ import annotations

import inspect
from collections.abc import Callable, Sequence
from dataclasses import dataclass

import torch

from torch_mojo_backend.torch_compile_backend.compiler import mojo_backend


def _as_list(outputs):
    return [outputs] if isinstance(outputs, torch.Tensor) else list(outputs)


def _compare(expected: Sequence[torch.Tensor], produced: Sequence[torch.Tensor], *, rtol, atol, same_device: bool):
    if len(expected) != len(produced):
        raise AssertionError(f"{len(expected)} outputs expected, {len(produced)} produced")
    for i, (want, got) in enumerate(zip(expected, produced)):
        assert want.shape == got.shape, f"Issue with output {i}: shape {tuple(got.shape)}, expected {tuple(want.shape)}"
        assert want.dtype == got.dtype, f"Issue with output {i}: dtype {got.dtype}, expected {want.dtype}"
        if same_device:
            assert want.device == got.device, f"Issue with output {i}: device {got.device}, expected {want.device}"
        torch.testing.assert_close(got.to(want.device), want, rtol=rtol, atol=atol)


def check_functions_are_equivalent(fn: Callable, device: str | None, inputs: list[torch.Tensor],
                                   fn_compiled: Callable | None = None, rtol=None, atol=None):
    """`fn` compiled with `mojo_backend` (or `fn_compiled`) against `fn` itself on the same inputs,
    moved to `device` first when one is given. The compiled function runs first: it never writes to
    its inputs, `fn` might."""
    fn_compiled = fn_compiled or torch.compile(backend=mojo_backend)(fn)
    if device is not None:
        inputs = [t.to(device) for t in inputs]
    produced = fn_compiled(*inputs)
    expected = fn(*inputs)
    assert type(expected) is type(produced), f"{type(produced).__name__} returned where eager returns {type(expected).__name__}"
    _compare(_as_list(expected), _as_list(produced), rtol=rtol, atol=atol, same_device=True)


@dataclass
class Conf:
    """Where and how a test runs a function: on `device`, compiled with `mojo_backend` or eagerly."""

    device: str
    compile: bool

    def __str__(self) -> str:
        return f"{self.device}, {'compiled' if self.compile else 'eager'}"


def to_device(tensors: list[torch.Tensor], device: str) -> list[torch.Tensor]:
    """Fresh copies on `device` (a function under test may write to its inputs)."""
    return [torch.clone(t).to(device) for t in tensors]


def check_outputs(fn: Callable, conf: Conf, inputs: list[torch.Tensor], *, rtol=None, atol=None):
    """`fn` run as `conf` says against `fn` run eagerly on the CPU. A `device` parameter of `fn`, when
    it has one, receives the device of the run."""
    takes_device = "device" in inspect.signature(fn).parameters

    def run(f, tensors, device):
        return f(*tensors, device=device) if takes_device else f(*tensors)

    expected = _as_list(run(fn, to_device(inputs, "cpu"), "cpu"))
    runner = torch.compile(fn, backend=mojo_backend) if conf.compile else fn
    produced = _as_list(run(runner, to_device(inputs, conf.device), conf.device))
    want_device = torch.device(conf.device)
    for i, got in enumerate(produced):
        on = got.device if want_device.index is not None else torch.device(got.device.type)
        if on != want_device:
            raise AssertionError(f"Issue with output {i}, expected device {want_device!r} but got {got.device!r}")
    _compare(expected, produced, rtol=rtol, atol=atol, same_device=False)
