"""User-written CUDA kernels as torch custom ops that compiled graphs launch without a graph break.

Same entry point and argument meaning as the reference's
`make_torch_op_from_mojo(path_to_kernels, mojo_custom_op_str, allocate_outputs_fn)`
(torch_mojo_backend/custom_torch_ops_in_mojo/torch_custom_ops.py:13-92); the kernel directory holds
CUDA sources instead of Mojo sources:

  * `path_to_kernels` is a directory of `.cu` files. They are compiled together for sm_100a into one
    shared library (once per content hash, kept under `<directory>/_build/`, or under
    `$B200_USER_OP_BUILD_DIR/<directory name>/` when that is set).
  * the op `NAME` is the `extern "C"` function `NAME` of that library with the calling convention of
    `include/b200_user_op.h`: outputs first, then inputs, then the stream (destination passing, as the
    reference's ops are).
  * `allocate_outputs_fn(*inputs)` returns the output tensor, or a tuple / list of them, for given
    inputs. Its signature names the op's inputs; its return annotation (or `num_outputs=`) says how
    many outputs there are.

The op is registered as `torch.library.custom_op("<directory name>::NAME", mutates_args=<outputs>)`
and, under the key `"<directory name>.NAME"`, in `MAPPING_TORCH_ATEN_TO_MOJO`, where the graph
walk finds it when AOTAutograd hands the op over as an `auto_functionalized_v2` node (reference:
torch_compile_backend/compiler.py:262-277). The returned function allocates the outputs and calls
the op; eager calls and compiled graphs run the same launch. There is no CPU implementation: a
tensor that is not on a CUDA device is an error.
"""

from __future__ import annotations

import ctypes
import hashlib
import inspect
import os
import shutil
import subprocess
import threading
import typing
from collections.abc import Callable
from pathlib import Path

import torch

MAX_RANK = 8
_DTYPE_CODES = {
    torch.uint8: 0, torch.int8: 1, torch.int16: 2, torch.int32: 3, torch.int64: 4,
    torch.float16: 5, torch.bfloat16: 6, torch.float32: 7, torch.float64: 8, torch.bool: 9,
}
_INCLUDE_DIR = Path(__file__).resolve().parents[3] / "include"
_NVCC_FLAGS = ("-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo", "-shared",
               "--cudart", "static", "-Xcompiler", "-fPIC")


class UserTensor(ctypes.Structure):
    """`b200_user_tensor` of include/b200_user_op.h."""

    _fields_ = [
        ("data", ctypes.c_void_p),
        ("dtype", ctypes.c_int32),
        ("rank", ctypes.c_int32),
        ("shape", ctypes.c_int64 * MAX_RANK),
        ("strides", ctypes.c_int64 * MAX_RANK),
    ]

    @classmethod
    def describe(cls, op: str, t: torch.Tensor) -> "UserTensor":
        if not isinstance(t, torch.Tensor):
            raise TypeError(f"{op}: user CUDA ops take tensors, got {type(t).__name__}")
        if t.device.type != "cuda":
            raise RuntimeError(f"{op} got a tensor on {t.device}; user CUDA ops run on CUDA tensors only and there is no CPU fallback.")
        if t.dtype not in _DTYPE_CODES:
            raise TypeError(f"{op}: dtype {t.dtype} has no code in b200_user_dtype")
        if t.dim() > MAX_RANK:
            raise RuntimeError(f"{op}: rank {t.dim()} exceeds B200_USER_MAX_RANK = {MAX_RANK}")
        d = cls()
        d.data = t.data_ptr()
        d.dtype = _DTYPE_CODES[t.dtype]
        d.rank = t.dim()
        for i in range(t.dim()):
            d.shape[i] = t.shape[i]
            d.strides[i] = t.stride(i)
        return d


def _nvcc() -> str:
    for candidate in (os.environ.get("NVCC"), shutil.which("nvcc"),
                      os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")):
        if candidate and os.path.exists(candidate):
            return candidate
    raise RuntimeError("nvcc was not found (set NVCC or CUDA_HOME): user CUDA kernels are compiled for sm_100a when first used")


class UserKernelLibrary:
    """The shared library built from the `.cu` files of one kernel directory (one per directory and process)."""

    _lock = threading.Lock()
    _loaded: dict[Path, "UserKernelLibrary"] = {}

    def __init__(self, directory: Path):
        self.directory = directory
        self.sources = sorted(directory.glob("*.cu"))
        if not directory.is_dir() or not self.sources:
            raise FileNotFoundError(f"{directory} is not a directory with .cu kernel sources")
        digest = hashlib.sha256()
        for extra in sorted(directory.glob("*.cuh")) + sorted(directory.glob("*.h")) + self.sources:
            digest.update(extra.name.encode())
            digest.update(extra.read_bytes())
        digest.update((_INCLUDE_DIR / "b200_user_op.h").read_bytes())
        digest.update(" ".join(_NVCC_FLAGS).encode())
        base = os.environ.get("B200_USER_OP_BUILD_DIR")
        self.build_dir = Path(base) / directory.name if base else directory / "_build"
        self.path = self.build_dir / f"lib{directory.name}_{digest.hexdigest()[:16]}.so"
        if not self.path.exists():
            self._compile()
        self.dll = ctypes.CDLL(str(self.path))

    def _compile(self) -> None:
        self.build_dir.mkdir(parents=True, exist_ok=True)
        tmp = self.path.with_suffix(f".{os.getpid()}.tmp")
        cmd = [_nvcc(), *_NVCC_FLAGS, "-I", str(_INCLUDE_DIR), "-I", str(self.directory),
               *[str(s) for s in self.sources], "-o", str(tmp)]
        done = subprocess.run(cmd, capture_output=True, text=True)
        if done.returncode != 0:
            raise RuntimeError(f"nvcc failed on the kernels of {self.directory}:\n{done.stdout}{done.stderr}")
        os.replace(tmp, self.path)  # atomic: a concurrent process sees the old state or the whole file

    @classmethod
    def of(cls, directory: Path) -> "UserKernelLibrary":
        directory = Path(directory).resolve()
        with cls._lock:
            lib = cls._loaded.get(directory)
            if lib is None:
                lib = cls._loaded[directory] = cls(directory)
            return lib

    def function(self, name: str):
        try:
            fn = getattr(self.dll, name)
        except AttributeError:
            raise AttributeError(
                f"{self.path.name} (built from {self.directory}) exports no function {name!r}; a user op is an "
                'extern "C" function with the signature of b200_user_op_fn'
            ) from None
        fn.restype = ctypes.c_int32
        fn.argtypes = [ctypes.POINTER(UserTensor), ctypes.c_int32, ctypes.POINTER(UserTensor), ctypes.c_int32, ctypes.c_void_p]
        return fn


def _count_outputs(allocate_outputs_fn: Callable, num_outputs: int | None) -> int:
    if num_outputs is not None:
        if num_outputs < 1:
            raise ValueError("a user op has at least one output")
        return num_outputs
    try:
        returns = typing.get_type_hints(allocate_outputs_fn).get("return")
    except Exception:
        returns = inspect.signature(allocate_outputs_fn).return_annotation
    if returns is torch.Tensor:
        return 1
    if typing.get_origin(returns) in (tuple, list):
        args = [a for a in typing.get_args(returns)]
        if args and Ellipsis not in args and all(a is torch.Tensor for a in args):
            return len(args)
    raise ValueError(
        "the number of outputs is read from allocate_outputs_fn's return annotation (torch.Tensor or "
        "tuple[torch.Tensor, ...] with one entry per output); annotate it or pass num_outputs="
    )


def make_torch_op_from_mojo(path_to_kernels: Path, mojo_custom_op_str: str, allocate_outputs_fn: Callable,
                            *, num_outputs: int | None = None) -> Callable:
    import torch_mojo_backend

    path_to_kernels = Path(path_to_kernels)
    name = mojo_custom_op_str
    library = UserKernelLibrary.of(path_to_kernels)
    kernel = library.function(name)
    n_out = _count_outputs(allocate_outputs_fn, num_outputs)
    qualified = f"{path_to_kernels.name}::{name}"

    inputs = list(inspect.signature(allocate_outputs_fn).parameters.values())
    for p in inputs:
        if p.kind not in (p.POSITIONAL_ONLY, p.POSITIONAL_OR_KEYWORD):
            raise TypeError(f"{qualified}: allocate_outputs_fn may only take positional tensor arguments, not {p}")
    out_names = [f"out{i}" for i in range(n_out)]
    in_names = [p.name for p in inputs]
    if set(out_names) & set(in_names):
        raise TypeError(f"{qualified}: the input names {sorted(set(out_names) & set(in_names))} are taken by the outputs")

    def launch(*tensors):
        if len(tensors) != n_out + len(in_names):
            raise TypeError(f"{qualified} takes {n_out} outputs and {len(in_names)} inputs, got {len(tensors)} tensors")
        described = [UserTensor.describe(qualified, t) for t in tensors]
        device = tensors[0].device
        for t in tensors:
            if t.device != device:
                raise RuntimeError(f"{qualified} got tensors on {device} and {t.device}")
        outs = (UserTensor * n_out)(*described[:n_out])
        ins = (UserTensor * max(len(in_names), 1))(*described[n_out:])
        with torch.cuda.device(device):
            stream = torch.cuda.current_stream(device).cuda_stream
            status = kernel(outs, n_out, ins, len(in_names), ctypes.c_void_p(stream))
        if status != 0:
            raise RuntimeError(f"{qualified} returned status {status}")

    # the schema torch infers: (Tensor(a!) out0, ..., Tensor in0, ...) -> ()
    launch.__signature__ = inspect.Signature(
        [inspect.Parameter(n, inspect.Parameter.POSITIONAL_OR_KEYWORD, annotation=torch.Tensor) for n in out_names + in_names],
        return_annotation=None,
    )
    launch.__name__ = name
    try:
        torch_custom_op = torch.library.custom_op(qualified, mutates_args=out_names)(launch)
    except RuntimeError as e:  # defined before in this process (the reference re-registers on every call as well)
        namespace = getattr(torch.ops, path_to_kernels.name)
        if not hasattr(namespace, name):
            raise e
        torch_custom_op = getattr(namespace, name).default

    def compiler_fn(*args):
        """The lowering of the `auto_functionalized_v2` node: the mutated bases (the outputs) come
        first, then the inputs; returns (the op's own result, *the written outputs)."""
        torch_custom_op(*args)
        return (None, *args[:n_out])

    torch_mojo_backend.MAPPING_TORCH_ATEN_TO_MOJO[f"{path_to_kernels.name}.{name}"] = compiler_fn

    def fn(*args):
        output_tensors = allocate_outputs_fn(*args)
        if isinstance(output_tensors, torch.Tensor):
            output_tensors = (output_tensors,)
            single_output = True
        elif isinstance(output_tensors, (tuple, list)):
            single_output = False
            for t in output_tensors:
                if not isinstance(t, torch.Tensor):
                    raise ValueError(
                        "allocate_outputs_fn must return a torch.Tensor or a tuple/list of torch.Tensor. "
                        f"Found a list/tuple with an element of type {type(t)}"
                    )
        else:
            raise ValueError(
                f"allocate_outputs_fn must return a torch.Tensor or a tuple/list of torch.Tensor. Found {type(output_tensors)}"
            )
        if len(output_tensors) != n_out:
            raise ValueError(f"{qualified} has {n_out} outputs; allocate_outputs_fn returned {len(output_tensors)}")
        torch_custom_op(*output_tensors, *args)
        if single_output:
            return output_tensors[0]
        return tuple(output_tensors)

    fn.torch_op = torch_custom_op
    fn.library = library
    return fn
