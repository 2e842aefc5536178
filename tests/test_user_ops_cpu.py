"""User CUDA kernels as ops of a compiled graph, the part that needs no GPU: the kernel directory
compiles for sm_100a, the library exports the ops, the torch custom op has the destination-passing
schema, a graph with the op traces and lowers, and running it on CPU tensors fails loudly.
Mirrors the registration half of the reference's tests/test_compiler.py:781-826."""

from pathlib import Path

import pytest
import torch

from torch_mojo_backend import MAPPING_TORCH_ATEN_TO_MOJO, make_torch_op_from_mojo, mojo_backend

KERNELS = Path(__file__).parent / "dummy_cuda_kernels"


def allocate_outputs_grayscale(pic: torch.Tensor) -> torch.Tensor:
    return pic.new_empty(pic.shape[:-1], dtype=torch.float32)


def allocate_outputs_grayscale_multi(pic: torch.Tensor, noise: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    return tuple(pic.new_empty(noise.shape, dtype=torch.float32) for _ in range(2))


def test_registration_builds_the_library_and_the_schema():
    fn = make_torch_op_from_mojo(KERNELS, "grayscale", allocate_outputs_grayscale)
    assert fn.library.path.exists() and fn.library.path.parent == KERNELS / "_build"
    assert str(torch.ops.dummy_cuda_kernels.grayscale.default._schema) == (
        "dummy_cuda_kernels::grayscale(Tensor(a0!) out0, Tensor pic) -> ()"
    )
    assert "dummy_cuda_kernels.grayscale" in MAPPING_TORCH_ATEN_TO_MOJO
    multi = make_torch_op_from_mojo(KERNELS, "grayscale_multi", allocate_outputs_grayscale_multi)
    assert multi.library is fn.library, "one shared library per kernel directory"
    assert str(torch.ops.dummy_cuda_kernels.grayscale_multi.default._schema) == (
        "dummy_cuda_kernels::grayscale_multi(Tensor(a0!) out0, Tensor(a1!) out1, Tensor pic, Tensor noise) -> ()"
    )
    again = make_torch_op_from_mojo(KERNELS, "grayscale", allocate_outputs_grayscale)  # registering twice is allowed
    assert again.library is fn.library


def test_registration_errors():
    with pytest.raises(AttributeError, match="exports no function 'sepia'"):
        make_torch_op_from_mojo(KERNELS, "sepia", allocate_outputs_grayscale)
    with pytest.raises(FileNotFoundError):
        make_torch_op_from_mojo(KERNELS / "nowhere", "grayscale", allocate_outputs_grayscale)

    def unannotated(pic):
        return pic.new_empty(pic.shape[:-1])

    with pytest.raises(ValueError, match="return annotation"):
        make_torch_op_from_mojo(KERNELS, "grayscale", unannotated)
    assert callable(make_torch_op_from_mojo(KERNELS, "grayscale", unannotated, num_outputs=1))


def test_no_cpu_fallback_eager_and_compiled():
    fn = make_torch_op_from_mojo(KERNELS, "grayscale", allocate_outputs_grayscale)
    img = torch.zeros(8, 8, 3, dtype=torch.uint8)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        fn(img)

    def graph(x):
        return fn(x + 8) - 16

    # the graph is captured whole (fullgraph=True would raise on a break) and lowered; the launch then refuses
    compiled = torch.compile(graph, backend=mojo_backend, fullgraph=True)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        compiled(img)


def test_wrong_number_of_outputs_is_reported():
    def two(pic: torch.Tensor) -> torch.Tensor:
        return (pic.new_empty(pic.shape[:-1]), pic.new_empty(pic.shape[:-1]))

    fn = make_torch_op_from_mojo(KERNELS, "grayscale", two)
    with pytest.raises(ValueError, match="has 1 outputs"):
        fn(torch.zeros(2, 2, 3, dtype=torch.uint8))
    with pytest.raises(ValueError, match="must return a torch.Tensor"):
        make_torch_op_from_mojo(KERNELS, "grayscale", lambda pic: 3, num_outputs=1)(torch.zeros(2, 2, 3))
