"""The aten -> kernel registry: `MAPPING_TORCH_ATEN_TO_MOJO`, `map_to`, `DECOMPOSITION_TABLE`.

Same surface and semantics as the reference registry (torch_mojo_backend/aten_functions.py:98-198):
a dict keyed by `OpOverload` / `OpOverloadPacket` / python operator / `"ns.op"` string whose values
are called as `fn(*args, **kwargs)` by the graph walk (torch_compile_backend/compiler.py), and a
`@map_to(op)` decorator that also removes the op (every overload of a packet) from the
decomposition table handed to AOTAutograd so that mapped ops reach the lowering whole.

What differs is what the values do. The reference re-expresses each op as MAX graph ops; here the
values run on `torch.Tensor`s that live on a CUDA device and the ops this backend is about --
mm/addmm/bmm, _softmax, native_layer_norm, gelu, sum/mean/amax and the scaled-dot-product
attention family -- enqueue hand-written sm_100a kernels through `torch.ops.b200.*`. Shape glue
(views, slices, casts, small elementwise ops) stays on stock torch CUDA ops working on views.
"""

from __future__ import annotations

import contextvars
import functools
import math
import operator
import os

import torch
from torch._decomp import core_aten_decompositions
from torch._ops import OpOverload, OpOverloadPacket

import torch_mojo_backend.is_running_tests
from torch_mojo_backend import native, ops
from torch_mojo_backend.flags import verbose_enabled

aten = torch.ops.aten

# The fx node being lowered, set by the graph walk. Multi-output lowerings use it to see which
# outputs are consumed (reference: torch_mojo_backend/aten_functions.py:94-110).
CURRENT_FX_NODE: contextvars.ContextVar = contextvars.ContextVar("CURRENT_FX_NODE", default=None)


def _only_first_output_used() -> bool:
    node = CURRENT_FX_NODE.get()
    if node is None:
        return False
    return all(user.target is operator.getitem and user.args[1] == 0 for user in node.users)


# Ops that are not mapped get decomposed by AOTAutograd with this table.
DECOMPOSITION_TABLE = core_aten_decompositions()
original_decomposition_table_size = len(DECOMPOSITION_TABLE)
MAPPING_TORCH_ATEN_TO_MOJO: dict = {}

IDENTICAL_FUNCTIONS = [
    operator.add, operator.sub, operator.mul, operator.truediv, operator.floordiv, operator.pow,
    operator.mod, operator.matmul, operator.neg, operator.gt, operator.ge, operator.lt,
    operator.le, operator.eq, operator.ne, operator.and_, operator.or_, operator.xor,
    operator.iadd, operator.isub, operator.imul, operator.ifloordiv, operator.ipow,
    operator.imod, operator.getitem, str, max, min,
]
for _func in IDENTICAL_FUNCTIONS:
    MAPPING_TORCH_ATEN_TO_MOJO[_func] = _func

number_of_decompositions_removed = 0


def map_to(func):
    """Register the decorated function as the lowering of `func` (OpOverload or OpOverloadPacket)."""

    def decorator(func_to_map):
        registered = func_to_map
        if torch_mojo_backend.is_running_tests.IS_RUNNING_TESTS:
            # Call counters let tests assert that the registered lowering really ran
            # (reference: torch_mojo_backend/aten_functions.py:167-176).
            @functools.wraps(func_to_map)
            def counted(*args, **kwargs):
                counted.call_count += 1
                return func_to_map(*args, **kwargs)

            counted.call_count = 0
            registered = counted
        MAPPING_TORCH_ATEN_TO_MOJO[func] = registered
        if isinstance(func, OpOverload):
            DECOMPOSITION_TABLE.pop(func, None)
        elif isinstance(func, OpOverloadPacket):
            global number_of_decompositions_removed
            for overload_name in func.overloads():
                popped = DECOMPOSITION_TABLE.pop(getattr(func, overload_name), None)
                if popped is not None:
                    number_of_decompositions_removed += 1
        else:
            raise TypeError(f"Expected OpOverload or OpOverloadPacket, got {type(func)}")
        return registered

    return decorator


def _kernel_dtype(*tensors) -> bool:
    """True when every given tensor has a dtype the b200 kernels take (fp32 / bf16)."""
    return all(t is None or native.supported_dtype(t.dtype) for t in tensors)


def _require_kernel_dtype(op: str, *tensors) -> None:
    """The ops this backend exists for have no second implementation: a floating-point dtype the
    kernels do not take (float16, float64) is an error -- raised while the launch plan is built, so
    the user sees a MojoCompilerError at compile time -- not a silent trip through a vendor library."""
    for t in tensors:
        if t is not None and t.dtype.is_floating_point and not native.supported_dtype(t.dtype):
            raise NotImplementedError(
                f"{op}: dtype {t.dtype} is not supported by the b200 kernels (float32 and bfloat16 are); "
                "there is no library fallback"
            )


# ==============================================================================================
# GEMM family
# ==============================================================================================


def _fp32_gemm(a, b, bias, alpha, beta):
    """alpha * a @ b + beta * bias for 2-D fp32 operands, by torch.get_float32_matmul_precision():
    "highest" and "high" take b200_gemm's own choice for fp32 -- all but small products run on the
    tensor cores as three bf16 products of the operands' (hi, lo) halves accumulated in fp32 by one
    launch (relative error ~2^-16, inside the 1e-4 bar of the fp32 configurations), small ones on
    the exact CUDA-core kernel; "medium" rounds the operands to bf16 (one product).
    TORCH_MOJO_BACKEND_EXACT_FP32=1 pins every fp32 product to the exact kernel."""
    if os.environ.get("TORCH_MOJO_BACKEND_EXACT_FP32", "0").lower() in ("1", "true", "yes"):
        return ops.gemm(a, b, bias, None, alpha, beta, 0, None, native.ROUTE_SIMT)
    if torch.get_float32_matmul_precision() == "medium" and a.shape[0] * a.shape[1] * b.shape[1] >= (1 << 24):
        return ops.gemm(a.bfloat16(), b.bfloat16(), bias, None, alpha, beta, 0, torch.float32)
    return ops.gemm(a, b, bias, None, alpha, beta)


# mm(Tensor self, Tensor mat2) -> Tensor
@map_to(aten.mm)
def aten_mm(x, y):
    _require_kernel_dtype("aten.mm", x, y)
    if not _kernel_dtype(x, y):
        return aten.mm.default(x, y)  # integer matrices: shape glue, not a hot op
    if x.dtype == torch.float32 and y.dtype == torch.float32 and x.dim() == 2 and y.dim() == 2:
        return _fp32_gemm(x, y, None, 1.0, 1.0)
    return ops.gemm(x, y)


# addmm(Tensor self, Tensor mat1, Tensor mat2, *, Scalar beta=1, Scalar alpha=1) -> Tensor
@map_to(aten.addmm)
def aten_addmm(input, mat1, mat2, *, beta=1.0, alpha=1.0):
    # beta * input + alpha * (mat1 @ mat2), input broadcast to [m, n]; the scaling and the add
    # happen in the GEMM epilogue on the fp32 accumulator.
    _require_kernel_dtype("aten.addmm", input, mat1, mat2)
    if not _kernel_dtype(input, mat1, mat2):
        return aten.addmm.default(input, mat1, mat2, beta=beta, alpha=alpha)  # integer matrices: shape glue
    if float(beta) == 0.0:
        input = None  # torch ignores `input` altogether then (a NaN or inf in it must not propagate)
    if mat1.dtype == torch.float32 and mat2.dtype == torch.float32 and mat1.dim() == 2 and mat2.dim() == 2:
        return _fp32_gemm(mat1, mat2, input, float(alpha), float(beta))
    return ops.gemm(mat1, mat2, input, None, float(alpha), float(beta))


# bmm(Tensor self, Tensor mat2) -> Tensor
@map_to(aten.bmm)
def aten_bmm(input, mat2):
    _require_kernel_dtype("aten.bmm", input, mat2)
    if not _kernel_dtype(input, mat2):
        return aten.bmm.default(input, mat2)  # integer matrices: shape glue
    return ops.gemm(input, mat2)


# ==============================================================================================
# Row kernels
# ==============================================================================================


def _move_dim_last(x, dim):
    dim = dim % x.dim() if x.dim() > 0 else 0
    if x.dim() == 0 or dim == x.dim() - 1:
        return x, None
    return x.movedim(dim, -1), dim


# _softmax(Tensor self, int dim, bool half_to_float) -> Tensor
@map_to(aten._softmax)
def aten__softmax(self, dim: int, half_to_float: bool):
    return aten_softmax(self, dim=dim, dtype=torch.float32 if half_to_float else None)


# softmax.int(Tensor self, int dim, ScalarType? dtype=None) -> Tensor
@map_to(aten.softmax)
def aten_softmax(input, dim=-1, dtype=None):
    _require_kernel_dtype("aten._softmax", input)
    if not input.dtype.is_floating_point:
        raise NotImplementedError(f"aten._softmax: dtype {input.dtype} is not a floating-point type")
    if dtype is not None and dtype not in (torch.float32, input.dtype):
        raise NotImplementedError(f"aten._softmax: output dtype {dtype} for input {input.dtype} is not supported")
    if input.dim() == 0:
        return torch.ones_like(input, dtype=dtype or input.dtype)
    if input.dtype == torch.float32:
        dtype = None
    x, moved = _move_dim_last(input, dim)
    y = ops.softmax(x, 1.0, False, 0, dtype)
    return y if moved is None else y.movedim(-1, moved)


# native_layer_norm(Tensor input, SymInt[] normalized_shape, Tensor? weight, Tensor? bias, float eps)
#   -> (Tensor, Tensor, Tensor)
@map_to(aten.native_layer_norm)
def aten_native_layer_norm(input, normalized_shape, weight, bias, eps):
    _require_kernel_dtype("aten.native_layer_norm", input, weight, bias)
    k = len(normalized_shape)
    lead = input.shape[: input.dim() - k]
    cols = math.prod(normalized_shape)
    x = input.reshape(*lead, cols)
    w = weight.reshape(cols) if weight is not None else None
    b = bias.reshape(cols) if bias is not None else None
    y, mean, rstd = ops.layer_norm(x, w, b, eps)
    y = y.reshape(input.shape)
    if _only_first_output_used():
        # Statistics are dead in inference graphs (same observation as the reference makes to
        # pick its fused kernel, torch_mojo_backend/aten_functions.py:2837-2849).
        return y, None, None
    stat_shape = (*lead, *([1] * k))
    # torch reports the statistics in the input dtype on CPU and in fp32 for reduced-precision
    # CUDA inputs; follow what the traced graph recorded for this node.
    stat_dtype = _traced_output_dtype(1, torch.float32)
    return y, mean.reshape(stat_shape).to(stat_dtype), rstd.reshape(stat_shape).to(stat_dtype)


def _traced_output_dtype(index: int, default: torch.dtype) -> torch.dtype:
    node = CURRENT_FX_NODE.get()
    if node is None:
        return default
    val = node.meta.get("val")
    if isinstance(val, (tuple, list)) and index < len(val) and isinstance(val[index], torch.Tensor):
        return val[index].dtype
    return default


# gelu(Tensor self, *, str approximate='none') -> Tensor
@map_to(aten.gelu)
def aten_gelu(input, approximate="none"):
    _require_kernel_dtype("aten.gelu", input)
    return ops.gelu(input, approximate)


# gelu_backward(Tensor grad_output, Tensor self, *, str approximate='none') -> Tensor
@map_to(aten.gelu_backward)
def aten_gelu_backward(grad_output, input, *, approximate="none"):
    """reference: aten_functions.py:2070-2102"""
    if approximate not in ("none", "tanh"):
        raise ValueError(
            f"Invalid approximate argument '{approximate}'. Supported values are 'none' (exact, erf) and 'tanh'."
        )
    _require_kernel_dtype("aten.gelu_backward", grad_output, input)
    if grad_output.dtype != input.dtype:
        grad_output = grad_output.to(input.dtype)
    return ops.gelu_backward(grad_output, input, approximate)


# _softmax_backward_data(Tensor grad_output, Tensor output, int dim, ScalarType input_dtype) -> Tensor
@map_to(aten._softmax_backward_data)
def aten__softmax_backward_data(grad_output, output, dim, input_dtype):
    _require_kernel_dtype("aten._softmax_backward_data", grad_output, output)
    if grad_output.dtype != output.dtype:
        grad_output = grad_output.to(output.dtype)
    g, _ = _move_dim_last(grad_output, dim)
    y, moved = _move_dim_last(output, dim)
    dx = ops.softmax_backward(g, y, 1.0, input_dtype if native.supported_dtype(input_dtype) else None)
    return dx if moved is None else dx.movedim(-1, moved)


# native_layer_norm_backward(Tensor grad_out, Tensor input, SymInt[] normalized_shape, Tensor mean,
#   Tensor rstd, Tensor? weight, Tensor? bias, bool[3] output_mask) -> (Tensor, Tensor, Tensor)
@map_to(aten.native_layer_norm_backward)
def aten_native_layer_norm_backward(grad_out, input, normalized_shape, mean, rstd, weight, bias, output_mask,
                                    *, dx_add=None, dx_dtype=None, want_cast=False, sum_dtype=None, sum_shape=None):
    _require_kernel_dtype("aten.native_layer_norm_backward", grad_out, input, weight)
    norm = 1
    for d in normalized_shape:
        norm *= int(d)
    if weight is not None and weight.numel() != norm:
        raise ValueError(f"native_layer_norm_backward: weight of {weight.numel()} elements for {norm} normalised elements")
    w = weight
    if w is None and norm != input.shape[-1]:
        # no weight to carry the normalised extent: flatten the normalised dims ourselves
        input = input.reshape(*input.shape[: input.dim() - len(normalized_shape)], norm)
        grad_out = grad_out.reshape(input.shape)
    want_w, want_b = bool(output_mask[1]) and weight is not None, bool(output_mask[2]) and bias is not None
    extras = want_cast or sum_dtype is not None
    if extras:
        dx, dgamma, dbeta, dx_cast, dx_sum = ops.layer_norm_backward_with_copy(
            grad_out, input, mean, rstd, w, want_w, want_b, dx_add, dx_dtype, want_cast, sum_dtype)
    else:
        dx, dgamma, dbeta = ops.layer_norm_backward(grad_out, input, mean, rstd, w, want_w, want_b, dx_add, dx_dtype)
    if dx.dtype != input.dtype:
        dx = dx.to(input.dtype)
    dx = dx.reshape(grad_out.shape) if output_mask[0] else None
    if dbeta is not None and bias is not None:
        dbeta = dbeta.reshape(bias.shape)
    if not extras:
        return dx, dgamma, dbeta
    if dx_cast is not None:
        dx_cast = dx_cast.reshape(grad_out.shape)
    if dx_sum is not None and sum_shape is not None:
        dx_sum = dx_sum.reshape(sum_shape)
    return dx, dgamma, dbeta, dx_cast, dx_sum


def _reduce_dims(input, dim, keepdim, op, dtype):
    """sum/mean/amax over `dim` (list, int or None): the reduced dims are moved to the end and
    flattened so that one trailing-dim kernel launch covers any dim list."""
    nd = input.dim()
    if dim is None or (isinstance(dim, (list, tuple)) and len(dim) == 0):
        dims = list(range(nd))
    elif isinstance(dim, int):
        dims = [dim % nd if nd > 0 else 0]
    else:
        dims = sorted({d % nd if nd > 0 else 0 for d in dim})
    if nd == 0:
        x = input.reshape(1)
        out = ops.reduce(x, op, dtype)
        return out
    kept = [d for d in range(nd) if d not in dims]
    if op == native.REDUCE_SUM and kept == [nd - 1] and nd >= 2 and input.stride(-1) == 1:
        # Every dim but the last is summed (a bias gradient): the column-sum kernel reads the rows
        # as they lie instead of transposing them first.
        out = ops.sum_rows(input.reshape(-1, input.shape[-1]), dtype)
        return out.reshape([1] * (nd - 1) + [input.shape[-1]]) if keepdim else out
    x = input.permute(*kept, *dims) if kept + dims != list(range(nd)) else input
    lead = [input.shape[d] for d in kept]
    x = x.reshape(*lead, -1)
    out = ops.reduce(x, op, dtype)
    if keepdim:
        shape = [1 if d in dims else input.shape[d] for d in range(nd)]
        out = out.reshape(shape)
    return out


# sum.dim_IntList(Tensor self, int[1]? dim, bool keepdim=False, *, ScalarType? dtype=None) -> Tensor
@map_to(aten.sum)
def aten_sum(input, dim=None, keepdim=False, *, dtype=None):
    out_dtype = dtype or input.dtype
    _require_kernel_dtype("aten.sum", input)
    if not _kernel_dtype(input) or not native.supported_dtype(out_dtype) or input.numel() == 0:
        # Integer/bool sums (promoted to int64 by torch: token counts, mask sizes) and empty
        # reductions are shape glue, not a hot op.
        if dim is None:
            return torch.sum(input, dtype=dtype)
        return torch.sum(input, dim, keepdim, dtype=dtype)
    return _reduce_dims(input, dim, keepdim, native.REDUCE_SUM, out_dtype)


# mean(Tensor self, *, ScalarType? dtype=None) -> Tensor
# mean.dim(Tensor self, int[1]? dim, bool keepdim=False, *, ScalarType? dtype=None) -> Tensor
@map_to(aten.mean)
def aten_mean(input, dim=None, keepdim=False, *, dtype=None):
    out_dtype = dtype or input.dtype
    _require_kernel_dtype("aten.mean", input)
    if not native.supported_dtype(out_dtype):
        raise NotImplementedError(f"aten.mean: output dtype {out_dtype} is not supported by the b200 kernels")
    if input.numel() == 0:
        if dim is None:
            return torch.mean(input, dtype=dtype)
        return torch.mean(input, dim, keepdim, dtype=dtype)
    return _reduce_dims(input, dim, keepdim, native.REDUCE_MEAN, out_dtype)


# amax(Tensor self, int[1] dim=[], bool keepdim=False) -> Tensor
@map_to(aten.amax)
def aten_amax(input, dim=[], keepdim=False):
    _require_kernel_dtype("aten.amax", input)
    if not _kernel_dtype(input) or input.numel() == 0:
        return torch.amax(input, dim, keepdim)  # integer maxima / empty reductions: shape glue
    return _reduce_dims(input, dim, keepdim, native.REDUCE_AMAX, input.dtype)


# ==============================================================================================
# Attention
# ==============================================================================================


def _repeat_kv_heads(query, key, value):
    """Grouped-query attention: every K/V head serves `rep` consecutive query heads."""
    if key.dim() == 4 and key.shape[1] != query.shape[1]:
        rep = query.shape[1] // key.shape[1]
        key = key.repeat_interleave(rep, dim=1)
        value = value.repeat_interleave(rep, dim=1)
    return key, value


def _kernel_takes_attention(query, key, value) -> bool:
    """Whether b200::sdpa has a kernel for these operands (fp32 / bf16, head_dim <= 128); anything
    else is computed as GEMM -> softmax -> GEMM by `_sdpa_math`."""
    return _kernel_dtype(query, key, value) and query.shape[-1] <= 128 and query.dim() in (3, 4)


def _sdpa_kernel(query, key, value, is_causal, scale):
    """[B, H, T, D] attention through the kernel; 3-D inputs are treated as one batch.
    Returns (out, natural-log LSE [B, H, T])."""
    _require_kernel_dtype("scaled_dot_product_attention", query, key, value)
    if not _kernel_takes_attention(query, key, value):
        return _sdpa_math(query, key, value, None, is_causal, scale, want_lse=True)
    squeeze = query.dim() == 3
    if squeeze:
        query, key, value = query.unsqueeze(0), key.unsqueeze(0), value.unsqueeze(0)
    key, value = _repeat_kv_heads(query, key, value)
    out, lse = ops.sdpa(query, key, value, bool(is_causal), scale)
    if squeeze:
        out, lse = out.squeeze(0), lse.squeeze(0)
    return out, lse


_PLACEHOLDERS: dict = {}


def _placeholder(shape, dtype, device):
    """A zero tensor for the attention outputs that only a backward pass or dropout replay would
    read (philox seed / offset, debug mask). One per (shape, dtype, device), made once: filling a
    fresh one per call costs a kernel launch per attention layer for values nobody reads. While a
    CUDA graph is being captured the tensor made by the eager call that precedes every capture is
    re-used (allocating inside the capture would put a fill kernel into the graph)."""
    if torch._guards.detect_fake_mode() is not None:
        return torch.zeros(shape, dtype=dtype, device=device)  # tracing: nothing is cached
    key = (tuple(shape), dtype, torch.device(device))
    t = _PLACEHOLDERS.get(key)
    if t is None:
        t = torch.zeros(shape, dtype=dtype, device=device)
        capturing = torch.device(device).type == "cuda" and torch.cuda.is_current_stream_capturing()
        if not capturing:
            _PLACEHOLDERS[key] = t
    return t


# _scaled_dot_product_flash_attention(Tensor query, Tensor key, Tensor value, float dropout_p=0.0,
#   bool is_causal=False, bool return_debug_mask=False, *, float? scale=None)
#   -> (Tensor, Tensor, Tensor, Tensor, SymInt, SymInt, Tensor, Tensor, Tensor)
@map_to(aten._scaled_dot_product_flash_attention)
def aten__scaled_dot_product_flash_attention(
    query, key, value, dropout_p=0.0, is_causal=False, return_debug_mask=False, scale=None
):
    if dropout_p != 0.0:
        raise NotImplementedError("attention dropout is not supported (inference forward only)")
    out, lse = _sdpa_kernel(query, key, value, is_causal, scale)
    # The remaining outputs exist for the backward/dropout replay; the reference fabricates
    # placeholders for them too (torch_mojo_backend/aten_functions.py:609-677). Here logsumexp
    # ([B, H, T] fp32, the shape torch gives this overload) is the real one.
    dev = out.device
    rng = _placeholder((2,), torch.int64, dev)
    unused = _placeholder((), torch.int64, dev)
    debug_mask = _placeholder((), out.dtype, dev)
    return (out, lse, None, None, query.shape[2], key.shape[2], rng, unused, debug_mask)


def _lse_padded_to_32(lse):
    """torch's memory-efficient attention reports logsumexp as [B, H, T rounded up to 32] (its
    kernel's alignment); the padding holds +inf there and nothing reads it."""
    t = lse.shape[-1]
    pad = (-t) % 32
    if pad == 0:
        return lse
    return torch.nn.functional.pad(lse, (0, pad), value=float("inf"))


# _scaled_dot_product_efficient_attention(Tensor query, Tensor key, Tensor value, Tensor? attn_bias,
#   bool compute_log_sumexp, float dropout_p=0.0, bool is_causal=False, *, float? scale=None)
#   -> (Tensor output, Tensor log_sumexp, Tensor philox_seed, Tensor philox_offset)
@map_to(aten._scaled_dot_product_efficient_attention)
def aten__scaled_dot_product_efficient_attention(
    query, key, value, attn_bias, compute_log_sumexp, dropout_p=0.0, is_causal=False, *, scale=None
):
    if dropout_p != 0.0:
        raise NotImplementedError("attention dropout is not supported (inference forward only)")
    if attn_bias is not None:
        out, lse = _sdpa_math(query, key, value, attn_bias, is_causal, scale, want_lse=bool(compute_log_sumexp))
    else:
        out, lse = _sdpa_kernel(query, key, value, is_causal, scale)
    dev = out.device
    if compute_log_sumexp:
        lse = _lse_padded_to_32(lse)
    else:
        lse = torch.empty((*query.shape[:-2], 0), dtype=torch.float32, device=dev)
    seed = _placeholder((), torch.int64, dev)
    return out, lse, seed, seed


# _scaled_dot_product_cudnn_attention(Tensor query, Tensor key, Tensor value, Tensor? attn_bias,
#   bool compute_log_sumexp, float dropout_p=0.0, bool is_causal=False, bool return_debug_mask=False,
#   *, float? scale=None) -> (Tensor, Tensor, Tensor, Tensor, SymInt, SymInt, Tensor, Tensor, Tensor)
@map_to(aten._scaled_dot_product_cudnn_attention)
def aten__scaled_dot_product_cudnn_attention(
    query, key, value, attn_bias, compute_log_sumexp, dropout_p=0.0, is_causal=False,
    return_debug_mask=False, *, scale=None,
):
    if dropout_p != 0.0:
        raise NotImplementedError("attention dropout is not supported (inference forward only)")
    if attn_bias is not None:
        out, lse = _sdpa_math(query, key, value, attn_bias, is_causal, scale, want_lse=True)
    else:
        out, lse = _sdpa_kernel(query, key, value, is_causal, scale)
    dev = out.device
    rng = _placeholder((), torch.int64, dev)
    # this overload reports logsumexp as [B, H, T, 1]
    return (out, lse.unsqueeze(-1), None, None, query.shape[2], key.shape[2], rng, rng, None)


def _sdpa_math(query, key, value, attn_mask, is_causal, scale, want_lse=False):
    """Attention with an explicit mask (or operands no attention kernel takes): GEMM -> masked
    softmax kernel -> GEMM (reference: aten__scaled_dot_product_attention_math,
    torch_mojo_backend/aten_functions.py:443-504). A bool mask keeps where it is True, a float
    mask is added to the scaled scores, `is_causal` masks on top of either (top-left aligned).
    Returns (out, lse): lse is the natural-log LSE [..., L] in fp32 when `want_lse`, else None."""
    d = query.shape[-1]
    if scale is None:
        scale = 1.0 / math.sqrt(d)
    lead = query.shape[:-2]
    L, S = query.shape[-2], key.shape[-2]
    key, value = _repeat_kv_heads(query, key, value)
    q3 = query.reshape(-1, L, d)
    k3 = key.reshape(-1, S, d)
    v3 = value.reshape(-1, S, value.shape[-1])
    scores = aten_bmm(q3, k3.transpose(1, 2)).reshape(*lead, L, S)
    lse = None
    if attn_mask is not None or want_lse:
        scores = scores.float() * scale if want_lse else scores * scale
        if attn_mask is not None:
            if attn_mask.dtype == torch.bool:
                scores = scores.masked_fill(~attn_mask, float("-inf"))
            else:
                scores = scores + attn_mask
        if is_causal:
            causal = torch.ones(L, S, dtype=torch.bool, device=query.device).tril()
            scores = scores.masked_fill(~causal, float("-inf"))
        if want_lse:
            lse = torch.logsumexp(scores, dim=-1)  # small reduction over fp32 scores: glue
        probs = aten_softmax(scores, -1)
    else:
        probs = ops.softmax(scores, scale, bool(is_causal), L)
    out = aten_bmm(probs.reshape(-1, L, S).to(v3.dtype), v3)
    return out.reshape(*lead, L, value.shape[-1]), lse


# _scaled_dot_product_attention_math(Tensor query, Tensor key, Tensor value, Tensor? attn_mask=None,
#   float dropout_p=0.0, bool is_causal=False, Tensor? dropout_mask=None, *, float? scale=None,
#   bool enable_gqa=False) -> (Tensor, Tensor)
@map_to(aten._scaled_dot_product_attention_math)
def aten__scaled_dot_product_attention_math(
    query, key, value, attn_mask=None, dropout_p=0.0, is_causal=False, dropout_mask=None, *,
    scale=None, enable_gqa=False,
):
    if dropout_p != 0.0:
        raise NotImplementedError("attention dropout is not supported (inference forward only)")
    if dropout_mask is not None:
        raise NotImplementedError("dropout_mask is not supported in aten._scaled_dot_product_attention_math")
    if attn_mask is None and _kernel_takes_attention(query, key, value):
        out = _sdpa_kernel(query, key, value, is_causal, scale)[0]
    else:
        out = _sdpa_math(query, key, value, attn_mask, is_causal, scale)[0]
    # the second output (attention weights) is materialised by torch only for the backward pass
    return out, torch.zeros((), dtype=out.dtype, device=out.device)


# scaled_dot_product_attention(Tensor query, Tensor key, Tensor value, Tensor? attn_mask=None,
#   float dropout_p=0.0, bool is_causal=False, *, float? scale=None, bool enable_gqa=False) -> Tensor
@map_to(aten.scaled_dot_product_attention)
def aten_scaled_dot_product_attention(
    query, key, value, attn_mask=None, dropout_p=0.0, is_causal=False, *, scale=None, enable_gqa=False
):
    if dropout_p != 0.0:
        raise NotImplementedError("attention dropout is not supported (inference forward only)")
    _require_kernel_dtype("aten.scaled_dot_product_attention", query, key, value)
    if attn_mask is None and _kernel_takes_attention(query, key, value):
        return _sdpa_kernel(query, key, value, is_causal, scale)[0]
    return _sdpa_math(query, key, value, attn_mask, is_causal, scale)[0]


# ==============================================================================================
# Fused forms produced by torch_compile_backend/fusion.py (registered under themselves)
# ==============================================================================================


# ---- attention backward -----------------------------------------------------------------------
# The gradient of softmax(scale Q K^T + bias) V from the library's own GEMM and row kernels: the
# probabilities are recomputed (S = Q K^T, P = softmax), dV = P^T dO, dP = dO V^T,
# dS = scale P (dP - rowsum(dP P)), dQ = dS K, dK = dS^T Q. The T x S matrices exist for a bounded
# number of (batch, head) pairs at a time. (The reference's fused form is
# eager_flash_attention/fa4_bwd_kernel.mojo; its decomposed form is eager_kernels/sdpa_backward_ops.mojo.)
_SDPA_BACKWARD_SCORE_BYTES = 1 << 30


def _sdpa_backward(grad_out, query, key, value, attn_bias, is_causal, scale, want_bias_grad=False, out=None, lse=None):
    _require_kernel_dtype("scaled_dot_product_attention backward", grad_out, query, key, value)
    if (
        attn_bias is None and out is not None and lse is not None and ops.sdpa_backward_supported(query, key, value)
        and out.dtype == query.dtype
    ):
        # the fused tensor-core kernel (bf16, head_dim 64): no T x S matrix is ever materialised
        dq, dk, dv = ops.sdpa_backward(grad_out, query, key, value, out, lse, bool(is_causal), scale)
        return dq, dk, dv, None
    if key.shape[1] != query.shape[1]:
        raise NotImplementedError("attention backward with grouped-query heads is not supported by the b200 kernels")
    B, H, T, D = query.shape
    S = key.shape[2]
    scale = float(scale) if scale is not None else 1.0 / math.sqrt(D)
    dtype = query.dtype
    q = query.reshape(B * H, T, D)
    k = key.reshape(B * H, S, D)
    v = value.reshape(B * H, S, value.shape[3])
    do = grad_out.to(dtype).reshape(B * H, T, value.shape[3])
    bias = None
    if attn_bias is not None:
        bias = attn_bias
        if bias.dtype == torch.bool:
            bias = torch.zeros(bias.shape, dtype=torch.float32, device=bias.device).masked_fill_(~bias, float("-inf"))
        bias = bias.to(torch.float32).expand(B, H, T, S).reshape(B * H, T, S)
    dq = torch.empty_like(q)
    dk = torch.empty_like(k)
    dv = torch.empty_like(v)
    dbias = torch.empty((B * H, T, S), dtype=torch.float32, device=q.device) if want_bias_grad else None
    chunk = max(1, _SDPA_BACKWARD_SCORE_BYTES // (16 * T * S))
    for lo in range(0, B * H, chunk):
        hi = min(B * H, lo + chunk)
        qc, kc, vc, doc = q[lo:hi], k[lo:hi], v[lo:hi], do[lo:hi]
        scores = ops.gemm(qc, kc.transpose(1, 2), None, None, 1.0, 1.0, 0, torch.float32)
        if bias is None:
            p = ops.softmax(scores, scale, bool(is_causal), T)
            fold = scale
        else:
            scores = scores * scale + bias[lo:hi]
            p = ops.softmax(scores, 1.0, bool(is_causal), T)
            fold = 1.0
        del scores
        p_lo = p if dtype == torch.float32 else p.to(dtype)
        dv[lo:hi] = ops.gemm(p_lo.transpose(1, 2), doc)
        dp = ops.gemm(doc, vc.transpose(1, 2), None, None, 1.0, 1.0, 0, torch.float32)
        if dbias is not None:
            ds32 = ops.softmax_backward(dp, p, 1.0)
            dbias[lo:hi] = ds32
            ds = (ds32 * scale).to(dtype)
        else:
            ds = ops.softmax_backward(dp, p, fold if bias is None else scale, dtype)
        del dp, p, p_lo
        dq[lo:hi] = ops.gemm(ds, kc)
        dk[lo:hi] = ops.gemm(ds.transpose(1, 2), qc)
    shape_q, shape_k, shape_v = query.shape, key.shape, value.shape
    if dbias is not None:
        dbias = dbias.reshape(B, H, T, S)
        # sum over the dims the bias was broadcast along
        for d in range(4):
            if attn_bias.dim() == 4 and attn_bias.shape[d] == 1 and dbias.shape[d] != 1:
                dbias = dbias.sum(d, keepdim=True)
        dbias = dbias.to(attn_bias.dtype) if attn_bias.dtype.is_floating_point else None
    return dq.reshape(shape_q), dk.reshape(shape_k), dv.reshape(shape_v), dbias


# _scaled_dot_product_flash_attention_backward(Tensor grad_out, Tensor query, Tensor key, Tensor value,
#   Tensor out, Tensor logsumexp, Tensor cum_seq_q, Tensor cum_seq_k, SymInt max_q, SymInt max_k,
#   float dropout_p, bool is_causal, Tensor philox_seed, Tensor philox_offset, *, float? scale=None)
#   -> (Tensor, Tensor, Tensor)
@map_to(aten._scaled_dot_product_flash_attention_backward)
def aten__scaled_dot_product_flash_attention_backward(
    grad_out, query, key, value, out, logsumexp, cum_seq_q, cum_seq_k, max_q, max_k, dropout_p, is_causal,
    philox_seed, philox_offset, *, scale=None,
):
    if dropout_p != 0.0:
        raise NotImplementedError("attention backward with dropout is not supported by the b200 kernels")
    return _sdpa_backward(grad_out, query, key, value, None, is_causal, scale, out=out, lse=logsumexp)[:3]


# _scaled_dot_product_efficient_attention_backward(Tensor grad_out_, Tensor query, Tensor key, Tensor value,
#   Tensor attn_bias, Tensor out, Tensor logsumexp, Tensor philox_seed, Tensor philox_offset, float dropout_p,
#   bool[4] grad_input_mask, bool is_causal=False, *, float? scale=None) -> (Tensor, Tensor, Tensor, Tensor)
@map_to(aten._scaled_dot_product_efficient_attention_backward)
def aten__scaled_dot_product_efficient_attention_backward(
    grad_out_, query, key, value, attn_bias, out, logsumexp, philox_seed, philox_offset, dropout_p,
    grad_input_mask, is_causal=False, *, scale=None,
):
    if dropout_p != 0.0:
        raise NotImplementedError("attention backward with dropout is not supported by the b200 kernels")
    want_bias = bool(grad_input_mask[3]) and attn_bias is not None
    return _sdpa_backward(grad_out_, query, key, value, attn_bias, is_causal, scale, want_bias, out=out, lse=logsumexp)


# _scaled_dot_product_cudnn_attention_backward(Tensor grad_out, Tensor query, Tensor key, Tensor value,
#   Tensor out, Tensor logsumexp, Tensor philox_seed, Tensor philox_offset, Tensor attn_bias,
#   Tensor cum_seq_q, Tensor cum_seq_k, SymInt max_q, SymInt max_k, float dropout_p, bool is_causal,
#   *, float? scale=None) -> (Tensor, Tensor, Tensor)
@map_to(aten._scaled_dot_product_cudnn_attention_backward)
def aten__scaled_dot_product_cudnn_attention_backward(
    grad_out, query, key, value, out, logsumexp, philox_seed, philox_offset, attn_bias, cum_seq_q, cum_seq_k,
    max_q, max_k, dropout_p, is_causal, *, scale=None,
):
    if dropout_p != 0.0:
        raise NotImplementedError("attention backward with dropout is not supported by the b200 kernels")
    return _sdpa_backward(grad_out, query, key, value, attn_bias, is_causal, scale, out=out, lse=logsumexp)[:3]


# _scaled_dot_product_flash_attention_for_cpu_backward(Tensor grad_out, Tensor query, Tensor key, Tensor value,
#   Tensor out, Tensor logsumexp, float dropout_p, bool is_causal, *, Tensor? attn_mask=None, float? scale=None)
#   -> (Tensor, Tensor, Tensor)
# (what the backward of a graph traced on CPU tensors holds: the forward op is decomposed, this one is not)
@map_to(aten._scaled_dot_product_flash_attention_for_cpu_backward)
def aten__scaled_dot_product_flash_attention_for_cpu_backward(
    grad_out, query, key, value, out, logsumexp, dropout_p, is_causal, *, attn_mask=None, scale=None
):
    if dropout_p != 0.0:
        raise NotImplementedError("attention backward with dropout is not supported by the b200 kernels")
    return _sdpa_backward(grad_out, query, key, value, attn_mask, is_causal, scale)[:3]


def _count_calls(fn):
    if not torch_mojo_backend.is_running_tests.IS_RUNNING_TESTS:
        return fn

    @functools.wraps(fn)
    def counted(*args, **kwargs):
        counted.call_count += 1
        return fn(*args, **kwargs)

    counted.call_count = 0
    return counted


@_count_calls
def fused_layer_norm(input, normalized_shape, weight, bias, eps, *, out_dtype):
    """native_layer_norm whose only consumer was a dtype cast of output 0: the kernel writes
    `out_dtype` directly from its fp32 registers."""
    k = len(normalized_shape)
    lead = input.shape[: input.dim() - k]
    cols = math.prod(normalized_shape)
    w = weight.reshape(cols) if weight is not None else None
    b = bias.reshape(cols) if bias is not None else None
    y, _, _ = ops.layer_norm(input.reshape(*lead, cols), w, b, eps, out_dtype)
    return y.reshape(input.shape)


@_count_calls
def fused_layer_norm_with_statistics(input, normalized_shape, weight, bias, eps, *, out_dtype):
    """native_layer_norm whose output 0 only fed a dtype cast and whose statistics are used as well
    (the forward of a training step): (y in `out_dtype`, mean, rstd) from one launch."""
    k = len(normalized_shape)
    lead = input.shape[: input.dim() - k]
    cols = math.prod(normalized_shape)
    w = weight.reshape(cols) if weight is not None else None
    b = bias.reshape(cols) if bias is not None else None
    y, mean, rstd = ops.layer_norm(input.reshape(*lead, cols), w, b, eps, out_dtype)
    stat_shape = (*lead, *([1] * k))
    stat_dtype = _traced_output_dtype(1, torch.float32)
    return y.reshape(input.shape), mean.reshape(stat_shape).to(stat_dtype), rstd.reshape(stat_shape).to(stat_dtype)


@_count_calls
def fused_layer_norm_backward(grad_out, input, normalized_shape, mean, rstd, weight, bias, output_mask,
                              *, dx_add=None, dx_dtype=None, want_cast=False, sum_dtype=None, sum_shape=None):
    """native_layer_norm_backward whose grad_out was a bf16 tensor widened to fp32 just before it
    (`dx_dtype`: the kernel reads the bf16 tensor and writes fp32), and / or whose dx only fed an add
    with the gradient of the residual branch (`dx_add`: added before dx is stored). With `want_cast` /
    `sum_dtype` the result has two more entries: that sum as bf16 (the operand of the gradient GEMMs
    of the layer before) and the sums of the bf16 tensor over its rows, shaped `sum_shape` (that
    layer's bias gradient)."""
    return aten_native_layer_norm_backward(
        grad_out, input, normalized_shape, mean, rstd, weight, bias, output_mask, dx_add=dx_add, dx_dtype=dx_dtype,
        want_cast=want_cast, sum_dtype=sum_dtype, sum_shape=sum_shape,
    )


@_count_calls
def fused_gemm(a, b, bias, residual, *, alpha, beta, epilogue, out_dtype, out_shape):
    """addmm / mm followed by (views,) gelu, an fp32 cast and/or a residual add, as one GEMM:
    out = act(alpha * a @ b + beta * bias) + residual, stored as `out_dtype`, viewed as `out_shape`."""
    n = b.shape[-1]
    res2d = residual.reshape(-1, n) if residual is not None else None
    y = ops.gemm(a, b, bias, res2d, alpha, beta, epilogue, out_dtype)
    # reshape, not view: a padded-pitch result splits its row dim as a view and copies otherwise
    return y.reshape(out_shape)


@_count_calls
def fused_embedding_sum(table, indices, table2, indices2, *, out_dtype):
    """`embedding(table, indices).to(out_dtype) + embedding(table2, indices2).to(out_dtype)` (token
    plus positional embeddings) as one gather kernel that adds in fp32 and writes `out_dtype`."""
    return ops.embedding_sum(table, indices, table2, indices2, out_dtype)


@_count_calls
def contiguous_or_alias(x):
    """`clone(memory_format=contiguous)` of a fresh kernel output: no copy when the memory is
    already in that order."""
    return x if x.is_contiguous() else x.contiguous()


@_count_calls
def fused_masked_softmax(x, mask, *, fill, scale, invert):
    """`_softmax(masked_fill(x * scale, mask, fill), -1)` (invert=False) or
    `_softmax(where(mask, x * scale, fill), -1)` (invert=True) in one pass over the scores. A mask
    whose run-time layout is not one [T, S] matrix shared by all leading indices is applied with
    torch glue first and only the softmax runs in the kernel."""
    if ops.mask_rows_of(x, mask) is not None:
        return ops.softmax_masked(x, mask, fill, scale, invert)
    masked = torch.where(mask if invert else ~mask, x * scale, fill)
    return ops.softmax(masked)


for _fused in (fused_layer_norm, fused_layer_norm_with_statistics, fused_layer_norm_backward, fused_gemm, contiguous_or_alias, fused_masked_softmax,
               fused_embedding_sum):
    MAPPING_TORCH_ATEN_TO_MOJO[_fused] = _fused


# _assert_tensor_metadata(Tensor a, SymInt[]? size=None, SymInt[]? stride=None, ScalarType? dtype=None,
#                         *, Device? device=None, Layout? layout=None) -> ()
@map_to(aten._assert_tensor_metadata)
def aten__assert_tensor_metadata(a, size=None, stride=None, dtype=None, *, device=None, layout=None):
    """torch.export leaves this check behind dtype / device casts. Shape and dtype are verified
    where the lowering runs (once on the trace's FakeTensors at plan-building time, then per
    call on metadata only: no kernel is launched). The device is not compared: a plan exported
    with `force_device` runs its frozen weights somewhere else than the module had them."""
    if dtype is not None and a.dtype != dtype:
        raise AssertionError(f"tensor dtype mismatch: expected {dtype}, got {a.dtype}")
    if size is not None and list(a.shape) != list(size):
        raise AssertionError(f"tensor size mismatch: expected {list(size)}, got {list(a.shape)}")
    return None


# ==============================================================================================
# Glue: ops kept whole and executed by stock torch on CUDA views
# ==============================================================================================


def _passthrough(op):
    def run(*args, **kwargs):
        return op(*args, **kwargs)

    run.__name__ = "aten_" + str(op).split(".")[-1]
    run.__qualname__ = run.__name__
    # Lets the graph walk call the node's exact OpOverload instead of re-resolving the packet.
    run.passthrough_of = op
    return run


# embedding(Tensor weight, Tensor indices, SymInt padding_idx=-1, bool scale_grad_by_freq=False,
#   bool sparse=False) -> Tensor
@map_to(aten.embedding)
def aten_embedding(weight, indices, padding_idx=-1, scale_grad_by_freq=False, sparse=False):
    # padding_idx, scale_grad_by_freq and sparse only matter for the backward pass
    # (reference: torch_mojo_backend/aten_functions.py:1779-1831)
    if not _kernel_dtype(weight) or weight.dim() != 2:
        return aten.embedding.default(weight, indices, padding_idx, scale_grad_by_freq, sparse)
    return ops.embedding_sum(weight, indices)


# argmax(Tensor self, int? dim=None, bool keepdim=False) -> Tensor
@map_to(aten.argmax)
def aten_argmax(input, dim=None, keepdim=False):
    if not _kernel_dtype(input) or input.numel() == 0 or input.dim() == 0:
        return torch.argmax(input, dim, keepdim)  # integer inputs / degenerate shapes: shape glue
    if dim is None:
        out = ops.argmax(input.reshape(-1))
        return out.reshape([1] * input.dim()) if keepdim else out
    x, moved = _move_dim_last(input, dim)
    out = ops.argmax(x)
    return out.unsqueeze(dim % input.dim()) if keepdim else out


# cat(Tensor[] tensors, int dim=0) -> Tensor
@map_to(aten.cat)
def aten_cat(tensors, dim=0):
    tensors = list(tensors)
    if len({t.dtype for t in tensors}) != 1 or any(t.dim() == 0 for t in tensors):
        return torch.cat(tensors, dim)  # type promotion across inputs: shape glue
    whole = _tiles_of_one_buffer(tensors, dim)
    if whole is not None:
        return whole
    return ops.cat(tensors, dim)


def _tiles_of_one_buffer(tensors, dim):
    """The concatenation as a view, when the inputs are views of ONE buffer that they tile exactly and
    in order along `dim` (the dq | dk | dv slices of the packed gradient an attention backward writes:
    their `cat` is that buffer). None when a copy is needed."""
    first = tensors[0]
    base = first._base
    if base is None or len(tensors) < 2 or not base.is_contiguous():
        return None
    dim = dim % first.dim()
    strides, offset, total = first.stride(), first.storage_offset(), 0
    for t in tensors:
        if t._base is not base or t.stride() != strides or t.storage_offset() != offset or t.dim() != first.dim():
            return None
        if any(t.shape[d] != first.shape[d] for d in range(first.dim()) if d != dim):
            return None
        offset += t.shape[dim] * strides[dim]
        total += t.numel()
    if total != base.numel() or first.storage_offset() != base.storage_offset():
        return None
    shape = list(first.shape)
    shape[dim] = sum(t.shape[dim] for t in tensors)
    out = first.as_strided(shape, strides, first.storage_offset())
    return out if out.is_contiguous() else None


def _view_or_copy(x, size):
    """aten.view / aten._unsafe_view of a tensor whose run-time strides may differ from the ones the
    trace assumed (a GEMM result with a padded row pitch): stay a view when the layout allows it,
    copy otherwise -- never fail on a stride the user's program knows nothing about."""
    try:
        return x.view(size)
    except (RuntimeError, ValueError):  # eager raises RuntimeError, the FakeTensor reference ValueError
        return x.reshape(size)


# view(Tensor(a) self, SymInt[] size) -> Tensor(a)
@map_to(aten.view)
def aten_view(x, size):
    return _view_or_copy(x, size)


# _unsafe_view(Tensor self, SymInt[] size) -> Tensor
@map_to(aten._unsafe_view)
def aten__unsafe_view(x, size):
    return _view_or_copy(x, size)


_GLUE_OPS = [
    aten.reshape, aten.transpose, aten.t, aten.permute, aten.expand,
    aten.clone, aten.contiguous, aten.split, aten.split_with_sizes, aten.slice, aten.select,
    aten.unsqueeze, aten.squeeze, aten.stack, aten.alias, aten.detach, aten.arange,
    aten.full, aten.full_like, aten.zeros, aten.zeros_like, aten.ones, aten.ones_like, aten.empty,
    aten.empty_like, aten.scalar_tensor, aten.tril, aten.triu, aten.eq, aten.ne, aten.lt, aten.le,
    aten.gt, aten.ge, aten.masked_fill, aten.where, aten.add, aten.sub, aten.mul, aten.div,
    aten.neg, aten.pow, aten.tanh, aten.exp, aten.log, aten.sqrt, aten.rsqrt, aten.abs,
    aten.sigmoid, aten.relu, aten.silu, aten.erf, aten.reciprocal, aten.minimum, aten.maximum,
    aten.clamp, aten._to_copy, aten.logical_not, aten.logical_and,
    aten.logical_or, aten.bitwise_and, aten.bitwise_or, aten.bitwise_not, aten.cumsum, aten.all,
    aten.any, aten.index, aten.index_select, aten.gather, aten.sym_size, aten.sym_numel,
    aten.lift_fresh_copy, aten.copy, aten.repeat, aten.flip, aten.unbind, aten.max, aten.min,
    aten.amin, aten.topk, aten.sort, aten.squeeze_copy, aten.native_dropout, aten._local_scalar_dense,
    # loss and embedding gradients of a training step
    aten._log_softmax, aten._log_softmax_backward_data, aten.nll_loss_forward, aten.nll_loss_backward,
    aten.scatter, aten.scatter_add, aten.index_put, aten.embedding_dense_backward, aten.new_zeros,
    # the rest of the elementwise, fill and allocation targets the reference's registry names
    # (torch_mojo_backend/aten_functions.py: acos 781 ... var 3379); none is on the hot path
    aten.acos, aten.asinh, aten.atanh, aten.ceil, aten.floor, aten.cos, aten.cosh, aten.sin, aten.sinh, aten.tan,
    aten.sign, aten.isnan, aten.log1p, aten.remainder, aten.logical_xor, aten.bitwise_xor, aten.addcmul,
    aten.addcdiv, aten.fill, aten.select_scatter, aten.empty_strided, aten.empty_permuted, aten.constant_pad_nd,
    aten.argmin, aten.var, aten.isin,
    # an optimizer step compiled with the backend (the reference maps the same multi-tensor ops)
    aten._foreach_add, aten._foreach_sub, aten._foreach_mul, aten._foreach_div, aten._foreach_neg,
    aten._foreach_pow, aten._foreach_sqrt, aten._foreach_reciprocal, aten._foreach_addcmul, aten._foreach_addcdiv,
]

for _packet in _GLUE_OPS:
    map_to(_packet)(_passthrough(_packet))

if verbose_enabled():
    print(
        f"Removed {number_of_decompositions_removed}/{original_decomposition_table_size} decompositions "
        "from the table (mapped ops stay whole)."
    )
