"""B200-native drop-in for the compile path of torch-mojo-backend.

Public names match the reference package (torch_mojo_backend/__init__.py:11-33) for the part that
is in scope: `mojo_backend`, `MAPPING_TORCH_ATEN_TO_MOJO`, `MojoCompilerError`, `get_accelerators`,
and `make_torch_op_from_mojo` (user kernels, here CUDA sources, as ops of a compiled graph);
`torch_mojo_backend.testing` has the reference's parity helpers (`check_outputs`,
`check_functions_are_equivalent`). The eager
`mojo` device (`register_mojo_devices`, `TorchMojoTensor`, `log_aten_calls`) belongs to a subsystem
that is not part of this path.
"""

from torch_mojo_backend.custom_torch_ops_in_cuda import make_torch_op_from_mojo

from torch_mojo_backend.torch_compile_backend.compiler import (
    MAPPING_TORCH_ATEN_TO_MOJO,
    MojoCompilerError,
    get_accelerators,
    mojo_backend,
)

__all__ = [
    "mojo_backend",
    "get_accelerators",
    "MAPPING_TORCH_ATEN_TO_MOJO",
    "MojoCompilerError",
    "make_torch_op_from_mojo",
]
