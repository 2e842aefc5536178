from torch_mojo_backend.custom_torch_ops_in_cuda.torch_custom_ops import (
    UserKernelLibrary,
    UserTensor,
    make_torch_op_from_mojo,
)

__all__ = ["make_torch_op_from_mojo", "UserKernelLibrary", "UserTensor"]
