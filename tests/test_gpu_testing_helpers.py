"""torch_mojo_backend.testing on a B200: a compiled function against CPU eager (`check_outputs`, the form
of the reference's tests/test_aten_functions.py) and against itself run eagerly on the same device."""

import pytest
import torch
import torch.nn.functional as F

from torch_mojo_backend import native
from torch_mojo_backend.testing import Conf, check_functions_are_equivalent, check_outputs

pytestmark = pytest.mark.gpu


def mlp(x, w1, b1, w2):
    return F.layer_norm(F.gelu(x @ w1 + b1, approximate="tanh") @ w2, (w2.shape[1],))


def _inputs():
    g = torch.Generator().manual_seed(11)
    return [torch.randn(96, 128, generator=g), torch.randn(128, 256, generator=g) * 0.1,
            torch.randn(256, generator=g) * 0.1, torch.randn(256, 64, generator=g) * 0.1]


def test_check_outputs_compiled_on_cuda_against_cpu_eager(reset_compiler):
    before = native.launch_count
    check_outputs(mlp, Conf("cuda", True), _inputs(), rtol=1e-3, atol=1e-3)
    assert native.launch_count > before, "the compiled function ran on the library's kernels"
    with pytest.raises(AssertionError, match="expected device"):
        check_outputs(lambda x: x.cpu() + 1, Conf("cuda", False), [torch.zeros(3)])


def test_check_functions_are_equivalent_on_cuda(reset_compiler):
    check_functions_are_equivalent(mlp, "cuda", _inputs(), rtol=1e-3, atol=1e-3)
