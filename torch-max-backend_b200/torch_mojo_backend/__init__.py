"""B200-native drop-in for the compile path of torch-mojo-backend.

Public names match the reference package (torch_mojo_backend/__init__.py:11-33) for the part that
is in scope: `mojo_backend`, `MAPPING_TORCH_ATEN_TO_MOJO`, `MojoCompilerError`, `get_accelerators`.
The eager `mojo` device (`register_mojo_devices`, `TorchMojoTensor`, `log_aten_calls`) and
`make_torch_op_from_mojo` belong to subsystems that are not part of this path.
"""

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
]
