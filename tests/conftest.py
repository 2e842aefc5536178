import os
import sys
from pathlib import Path

# Before the package is imported: lowerings get call counters (map_to) in test runs.
os.environ.setdefault("TORCH_MOJO_BACKEND_TESTING", "1")
# The GEMM tuning switches (B200_GEMM_PAIR / B200_GEMM_TILE_N) are read once per process unless
# this is set; the GEMM tests flip them between calls.
os.environ.setdefault("B200_GEMM_ENV_LIVE", "1")

ROOT = Path(__file__).resolve().parents[1]
for p in (ROOT, ROOT / "torch-max-backend_b200"):
    if str(p) not in sys.path:
        sys.path.insert(0, str(p))

import numpy as np  # noqa: E402
import pytest  # noqa: E402
import torch  # noqa: E402

GOLDEN_DIR = Path(__file__).parent / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def golden():
    return np.load(GOLDEN_DIR / "ops_golden.npz")


@pytest.fixture()
def reset_compiler():
    torch._dynamo.reset()
    yield
    torch._dynamo.reset()


class CallChecker:
    """Asserts that a registered lowering ran (reference: torch_mojo_backend/testing.py:32-136)."""

    def __init__(self):
        self._funcs = None
        self._before = None

    def register(self, *funcs):
        self._funcs = funcs
        self._before = [f.call_count for f in funcs]

    def check_was_called(self):
        assert self._funcs is not None, "call register() first"
        if not any(f.call_count > b for f, b in zip(self._funcs, self._before)):
            names = ", ".join(f.__name__ for f in self._funcs)
            raise AssertionError(f"Expected one of [{names}] to be called at least once, but none was")


@pytest.fixture()
def call_checker():
    checker = CallChecker()
    yield checker
    if checker._funcs is not None:
        checker.check_was_called()


# ---- tolerances of the parity bar -----------------------------------------------------------
# fp32: 1e-4 relative. bf16 with fp32 accumulation: 2e-2 relative. "Relative" is meant the way
# torch.testing.assert_close (and the reference's run_hf_mojo.py:22,51) means it:
# |got - want| <= atol + rtol * |want| with atol tied to the scale of the expected values, so
# that entries near zero are judged against the magnitude of the tensor, not their own.
FP32_RTOL = 1e-4
BF16_RTOL = 2e-2


def assert_parity(got: torch.Tensor, want: torch.Tensor, *, bf16: bool, scale: float | None = None, what=""):
    got = got.detach().float().cpu()
    want = want.detach().float().cpu()
    assert got.shape == want.shape, f"{what}: shape {tuple(got.shape)} != {tuple(want.shape)}"
    rtol = BF16_RTOL if bf16 else FP32_RTOL
    finite = torch.isfinite(want)
    if scale is None:
        scale = want[finite].abs().max().item() if finite.any() else 1.0
    atol = rtol * max(scale, 1e-30)
    torch.testing.assert_close(got, want, rtol=rtol, atol=atol, equal_nan=True, msg=lambda m: f"{what}: {m}")
