"""Type aliases used in lowering signatures (reference: torch_mojo_backend/types.py). In this
backend a graph value is a torch.Tensor on a CUDA device (or a FakeTensor at compile time)."""

import torch

MaxTensor = torch.Tensor
Scalar = int | float | torch.SymInt | torch.SymFloat
SymIntType = int | torch.SymInt
