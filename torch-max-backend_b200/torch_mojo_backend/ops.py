"""torch custom ops (`torch.ops.b200.*`) that marshal tensors into the libb200ops C ABI.

Shape of the boundary: the reference exposes user kernels as `torch.library.custom_op`s whose
Python body allocates the outputs and hands raw buffers to native code
(torch_mojo_backend/custom_torch_ops_in_mojo/torch_custom_ops.py:52-87), and its eager bridges
allocate outputs in Python before the native call (torch_mojo_backend/eager_kernels/aten_fast.py:4587-4600).
The same split is used here: every op below allocates with `torch.empty` (caching allocator,
stream ordered), validates, and enqueues exactly one C-ABI call on the current stream.

Each op has a Meta implementation so that it can run under FakeTensorMode at compile time, and
refuses CPU tensors: there is no CPU fallback.
"""

from __future__ import annotations

import ctypes
import math

import torch

from torch_mojo_backend import native

_lib = torch.library.Library("b200", "DEF")

_lib.define(
    "layer_norm(Tensor x, Tensor? weight, Tensor? bias, float eps, ScalarType? out_dtype=None)"
    " -> (Tensor, Tensor, Tensor)"
)
_lib.define(
    "softmax(Tensor x, float scale=1.0, bool causal=False, int q_len=0, ScalarType? out_dtype=None) -> Tensor"
)
_lib.define(
    "softmax_masked(Tensor x, Tensor mask, float fill, float scale=1.0, bool invert=False,"
    " ScalarType? out_dtype=None) -> Tensor"
)
_lib.define("gelu(Tensor x, str approximate='none') -> Tensor")
_lib.define("reduce(Tensor x, int op, ScalarType? out_dtype=None) -> Tensor")
_lib.define(
    "gemm(Tensor a, Tensor b, Tensor? bias=None, Tensor? residual=None, float alpha=1.0, float beta=1.0,"
    " int epilogue=0, ScalarType? out_dtype=None, int route=0) -> Tensor"
)
_lib.define(
    "sdpa(Tensor q, Tensor k, Tensor v, bool causal=False, float? scale=None, int route=0) -> (Tensor, Tensor)"
)
_lib.define(
    "sdpa_backward(Tensor d_out, Tensor q, Tensor k, Tensor v, Tensor o, Tensor lse, bool causal=False,"
    " float? scale=None) -> (Tensor, Tensor, Tensor)"
)
_lib.define(
    "embedding_sum(Tensor table, Tensor indices, Tensor? table2=None, Tensor? indices2=None,"
    " ScalarType? out_dtype=None) -> Tensor"
)
_lib.define("gelu_backward(Tensor dy, Tensor x, str approximate='none') -> Tensor")
_lib.define("softmax_backward(Tensor dy, Tensor y, float scale=1.0, ScalarType? out_dtype=None) -> Tensor")
_lib.define(
    "layer_norm_backward(Tensor dy, Tensor x, Tensor mean, Tensor rstd, Tensor? weight, bool want_weight=True,"
    " bool want_bias=True, Tensor? dx_add=None, ScalarType? dx_dtype=None) -> (Tensor, Tensor?, Tensor?)"
)
_lib.define(
    "layer_norm_backward_with_copy(Tensor dy, Tensor x, Tensor mean, Tensor rstd, Tensor? weight, bool want_weight=True,"
    " bool want_bias=True, Tensor? dx_add=None, ScalarType? dx_dtype=None, bool want_cast=False,"
    " ScalarType? sum_dtype=None) -> (Tensor, Tensor?, Tensor?, Tensor?, Tensor?)"
)
_lib.define("sum_rows(Tensor x, ScalarType? out_dtype=None) -> Tensor")
_lib.define("argmax(Tensor x) -> Tensor")
_lib.define("cat(Tensor[] tensors, int dim=0) -> Tensor")
_lib.define("kv_append(Tensor(a!) cache, Tensor new, int position) -> ()")


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def _nbytes(*tensors) -> float:
    return float(sum(t.numel() * t.element_size() for t in tensors if t is not None))


def _launched(device, start, name, flops, bytes_):
    """Bookkeeping after a successful launch: launch counter and, when installed, the profiler."""
    native.launch_count += 1
    if start is not None:
        native.profiler.end(device, start, name, flops, bytes_)


def _prof_begin(device):
    return native.profiler.begin(device) if native.profiler is not None else None


def _as_rows(x: torch.Tensor) -> tuple[torch.Tensor, int, int, int]:
    """View x as [rows, cols] with a unit column stride and one row stride (copying only when
    the layout cannot be described that way). Returns (tensor, rows, cols, row_stride)."""
    cols = x.shape[-1] if x.dim() > 0 else 1
    rows = math.prod(x.shape[:-1]) if x.dim() > 0 else 1
    if x.dim() == 0:
        return x.reshape(1, 1), 1, 1, 1
    if x.is_contiguous():
        return x, rows, cols, cols
    if x.dim() == 2 and x.stride(1) == 1 and x.stride(0) >= cols:
        return x, rows, cols, x.stride(0)
    x = x.contiguous()
    return x, rows, cols, cols


# ---- layer_norm -----------------------------------------------------------------------------


def _layer_norm_cuda(x, weight, bias, eps, out_dtype=None):
    device = native.require_cuda("layer_norm", x, weight, bias)
    out_dtype = out_dtype or x.dtype
    xr, rows, cols, row_stride = _as_rows(x)
    param_dtype = weight.dtype if weight is not None else (bias.dtype if bias is not None else x.dtype)
    if weight is not None and bias is not None and weight.dtype != bias.dtype:
        bias = bias.to(weight.dtype)
    if weight is not None:
        weight = weight.contiguous()
    if bias is not None:
        bias = bias.contiguous()
    y = torch.empty(x.shape, dtype=out_dtype, device=device)
    stat_shape = x.shape[:-1]
    mean = torch.empty(stat_shape, dtype=torch.float32, device=device)
    rstd = torch.empty(stat_shape, dtype=torch.float32, device=device)
    start = _prof_begin(device)
    with torch.cuda.device(device):
        status = native.lib().b200_layer_norm(
            xr.data_ptr(), _ptr(weight), _ptr(bias), y.data_ptr(), mean.data_ptr(), rstd.data_ptr(),
            rows, cols, row_stride, eps, native.dtype_enum(x.dtype), native.dtype_enum(param_dtype),
            native.dtype_enum(out_dtype), native.current_stream(device),
        )
    native.check("layer_norm", status)
    _launched(device, start, "layer_norm", 0.0, _nbytes(xr, y) + 8.0 * rows)
    return y, mean, rstd


def _layer_norm_meta(x, weight, bias, eps, out_dtype=None):
    y = torch.empty(x.shape, dtype=out_dtype or x.dtype, device=x.device)
    mean = torch.empty(x.shape[:-1], dtype=torch.float32, device=x.device)
    return y, mean, torch.empty_like(mean)


# ---- softmax --------------------------------------------------------------------------------


def _softmax_cuda(x, scale=1.0, causal=False, q_len=0, out_dtype=None):
    device = native.require_cuda("softmax", x)
    out_dtype = out_dtype or x.dtype
    xr, rows, cols, row_stride = _as_rows(x)
    y = torch.empty(x.shape, dtype=out_dtype, device=device)
    start = _prof_begin(device)
    with torch.cuda.device(device):
        status = native.lib().b200_softmax_lastdim(
            xr.data_ptr(), y.data_ptr(), rows, cols, row_stride, scale, int(causal), q_len,
            native.dtype_enum(x.dtype), native.dtype_enum(out_dtype), native.current_stream(device),
        )
    native.check("softmax", status)
    _launched(device, start, "softmax", 0.0, _nbytes(xr, y))
    return y


def _softmax_meta(x, scale=1.0, causal=False, q_len=0, out_dtype=None):
    return torch.empty(x.shape, dtype=out_dtype or x.dtype, device=x.device)


def mask_rows_of(x: torch.Tensor, mask: torch.Tensor):
    """(mask_rows, mask_row_stride) when `mask` (bool) broadcasts against `x` as one [T, S] matrix
    shared by every leading index of x — the layout the fused kernel reads — else None."""
    if mask.dtype != torch.bool or mask.dim() < 1 or mask.dim() > x.dim() or x.dim() < 1:
        return None
    shape = (1,) * (x.dim() - mask.dim()) + tuple(mask.shape)
    strides = (0,) * (x.dim() - mask.dim()) + tuple(mask.stride())
    if shape[-1] != x.shape[-1] or (shape[-1] > 1 and strides[-1] != 1):
        return None
    if any(d != 1 for d in shape[:-2]):
        return None
    if x.dim() == 1 or shape[-2] == 1:
        return 1, max(int(x.shape[-1]), 1)
    if shape[-2] != x.shape[-2]:
        return None
    return int(shape[-2]), int(strides[-2])


def _softmax_masked_cuda(x, mask, fill, scale=1.0, invert=False, out_dtype=None):
    device = native.require_cuda("softmax_masked", x, mask)
    out_dtype = out_dtype or x.dtype
    layout = mask_rows_of(x, mask)
    if layout is None:
        raise ValueError(
            f"softmax_masked: mask of shape {tuple(mask.shape)} and strides {mask.stride()} is not one [T, S] "
            f"matrix broadcast over the leading dims of x {tuple(x.shape)}"
        )
    mask_rows, mask_stride = layout
    xr, rows, cols, row_stride = _as_rows(x)
    y = torch.empty(x.shape, dtype=out_dtype, device=device)
    start = _prof_begin(device)
    with torch.cuda.device(device):
        status = native.lib().b200_softmax_masked(
            xr.data_ptr(), mask.data_ptr(), y.data_ptr(), rows, cols, row_stride, mask_rows, mask_stride,
            int(invert), fill, scale, native.dtype_enum(x.dtype), native.dtype_enum(out_dtype),
            native.current_stream(device),
        )
    native.check("softmax_masked", status)
    _launched(device, start, "softmax", 0.0, _nbytes(xr, y))
    return y


def _softmax_masked_meta(x, mask, fill, scale=1.0, invert=False, out_dtype=None):
    return torch.empty(x.shape, dtype=out_dtype or x.dtype, device=x.device)


# ---- gelu -----------------------------------------------------------------------------------


def _gelu_cuda(x, approximate="none"):
    device = native.require_cuda("gelu", x)
    if approximate not in ("none", "tanh"):
        raise ValueError(f"gelu: approximate must be 'none' or 'tanh', got {approximate!r}")
    xc = x if x.is_contiguous() else x.contiguous()
    y = torch.empty(x.shape, dtype=x.dtype, device=device)
    start = _prof_begin(device)
    with torch.cuda.device(device):
        status = native.lib().b200_gelu(
            xc.data_ptr(), y.data_ptr(), xc.numel(), int(approximate == "tanh"),
            native.dtype_enum(x.dtype), native.current_stream(device),
        )
    native.check("gelu", status)
    _launched(device, start, "gelu", 0.0, _nbytes(xc, y))
    return y


def _gelu_meta(x, approximate="none"):
    return torch.empty(x.shape, dtype=x.dtype, device=x.device)


# ---- reduce over the last dim ---------------------------------------------------------------


def _reduce_cuda(x, op, out_dtype=None):
    device = native.require_cuda("reduce", x)
    out_dtype = out_dtype or x.dtype
    xr, rows, cols, row_stride = _as_rows(x)
    y = torch.empty(x.shape[:-1], dtype=out_dtype, device=device)
    start = _prof_begin(device)
    with torch.cuda.device(device):
        status = native.lib().b200_reduce_lastdim(
            xr.data_ptr(), y.data_ptr(), rows, cols, row_stride, op, native.dtype_enum(x.dtype),
            native.dtype_enum(out_dtype), native.current_stream(device),
        )
    native.check("reduce", status)
    _launched(device, start, "reduce", 0.0, _nbytes(xr, y))
    return y


def _reduce_meta(x, op, out_dtype=None):
    return torch.empty(x.shape[:-1], dtype=out_dtype or x.dtype, device=x.device)


# ---- backward of the row kernels --------------------------------------------------------------


def _gelu_backward_cuda(dy, x, approximate="none"):
    device = native.require_cuda("gelu_backward", dy, x)
    if approximate not in ("none", "tanh"):
        raise ValueError(f"gelu_backward: approximate must be 'none' or 'tanh', got {approximate!r}")
    if dy.shape != x.shape or dy.dtype != x.dtype:
        raise RuntimeError(f"gelu_backward: dy {tuple(dy.shape)} {dy.dtype} and x {tuple(x.shape)} {x.dtype} differ")
    gc = dy if dy.is_contiguous() else dy.contiguous()
    xc = x if x.is_contiguous() else x.contiguous()
    dx = torch.empty(x.shape, dtype=x.dtype, device=device)
    start = _prof_begin(device)
    with torch.cuda.device(device):
        status = native.lib().b200_gelu_backward(
            gc.data_ptr(), xc.data_ptr(), dx.data_ptr(), xc.numel(), int(approximate == "tanh"),
            native.dtype_enum(x.dtype), native.current_stream(device),
        )
    native.check("gelu_backward", status)
    _launched(device, start, "gelu_backward", 0.0, _nbytes(gc, xc, dx))
    return dx


def _gelu_backward_meta(dy, x, approximate="none"):
    return torch.empty(x.shape, dtype=x.dtype, device=x.device)


def _softmax_backward_cuda(dy, y, scale=1.0, out_dtype=None):
    device = native.require_cuda("softmax_backward", dy, y)
    if dy.shape != y.shape or dy.dtype != y.dtype:
        raise RuntimeError(f"softmax_backward: dy {tuple(dy.shape)} {dy.dtype} and y {tuple(y.shape)} {y.dtype} differ")
    out_dtype = out_dtype or y.dtype
    gr, rows, cols, g_stride = _as_rows(dy)
    yr, _, _, y_stride = _as_rows(y)
    dx = torch.empty(y.shape, dtype=out_dtype, device=device)
    start = _prof_begin(device)
    with torch.cuda.device(device):
        status = native.lib().b200_softmax_backward(
            gr.data_ptr(), yr.data_ptr(), dx.data_ptr(), rows, cols, g_stride, y_stride, float(scale),
            native.dtype_enum(y.dtype), native.dtype_enum(out_dtype), native.current_stream(device),
        )
    native.check("softmax_backward", status)
    _launched(device, start, "softmax_backward", 0.0, _nbytes(gr, yr, dx))
    return dx


def _softmax_backward_meta(dy, y, scale=1.0, out_dtype=None):
    return torch.empty(y.shape, dtype=out_dtype or y.dtype, device=y.device)


def _layer_norm_backward_cuda(dy, x, mean, rstd, weight, want_weight=True, want_bias=True, dx_add=None, dx_dtype=None):
    """dx (+ dx_add, the gradient that reaches x along a residual branch), dgamma, dbeta. dx_dtype
    defaults to dy's dtype; float32 is also accepted for a bfloat16 dy and a float32 x."""
    return _layer_norm_backward_with_copy_cuda(dy, x, mean, rstd, weight, want_weight, want_bias, dx_add, dx_dtype)[:3]


def _layer_norm_backward_with_copy_cuda(dy, x, mean, rstd, weight, want_weight=True, want_bias=True, dx_add=None,
                                        dx_dtype=None, want_cast=False, sum_dtype=None):
    """The same launch with two more results: a bfloat16 copy of a float32 dx (`want_cast`) and the sums
    of dx over the rows as [cols] in `sum_dtype` -- of the bfloat16 copy when there is one. They are what
    the gradient GEMMs and the bias gradient of the layer that produced x read."""
    device = native.require_cuda("layer_norm_backward", dy, x, mean, rstd, weight, dx_add)
    if dy.shape != x.shape:
        raise RuntimeError(f"layer_norm_backward: dy {tuple(dy.shape)} and x {tuple(x.shape)} differ")
    dx_dtype = dx_dtype or dy.dtype
    if dx_add is not None and (dx_add.shape != x.shape or dx_add.dtype != dx_dtype):
        raise RuntimeError(
            f"layer_norm_backward: dx_add {tuple(dx_add.shape)} {dx_add.dtype} is not a {tuple(x.shape)} {dx_dtype} tensor"
        )
    cols = weight.numel() if weight is not None else x.shape[-1]
    if cols == 0 or x.numel() % cols != 0:
        raise RuntimeError(f"layer_norm_backward: {tuple(x.shape)} is not rows of {cols} normalised elements")
    rows = x.numel() // cols
    x2 = x.reshape(rows, cols)
    g2 = dy.reshape(rows, cols)
    x2 = x2 if x2.stride(1) == 1 and (x2.stride(0) >= cols or rows <= 1) else x2.contiguous()
    g2 = g2 if g2.stride(1) == 1 and (g2.stride(0) >= cols or rows <= 1) else g2.contiguous()
    mean_c = mean.reshape(-1).float().contiguous()
    rstd_c = rstd.reshape(-1).float().contiguous()
    if mean_c.numel() != rows or rstd_c.numel() != rows:
        raise RuntimeError(f"layer_norm_backward: mean / rstd have {mean_c.numel()} / {rstd_c.numel()} entries for {rows} rows")
    param_dtype = weight.dtype if weight is not None else x.dtype
    wc = None if weight is None else weight.reshape(-1).contiguous()
    dx = torch.empty(x.shape, dtype=dx_dtype, device=device)
    extra = None if dx_add is None else dx_add.contiguous()
    if want_cast and dx_dtype != torch.float32:
        raise RuntimeError(f"layer_norm_backward: the bfloat16 copy is offered for a float32 dx, not {dx_dtype}")
    dx_cast = torch.empty(x.shape, dtype=torch.bfloat16, device=device) if want_cast else None
    dx_sum = torch.empty(cols, dtype=sum_dtype, device=device) if sum_dtype is not None else None
    dgamma = torch.empty(cols, dtype=param_dtype, device=device) if want_weight else None
    dbeta = torch.empty(cols, dtype=param_dtype, device=device) if want_bias else None
    lib = native.lib()
    ws_bytes = lib.b200_layer_norm_backward_workspace_bytes(rows, cols)
    ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=device)
    start = _prof_begin(device)
    with torch.cuda.device(device):
        status = lib.b200_layer_norm_backward(
            g2.data_ptr(), x2.data_ptr(), mean_c.data_ptr(), rstd_c.data_ptr(), _ptr(wc), _ptr(extra), dx.data_ptr(),
            _ptr(dgamma), _ptr(dbeta), _ptr(dx_cast), _ptr(dx_sum), ws.data_ptr(), ws_bytes, rows, cols,
            g2.stride(0) if rows > 1 else cols, x2.stride(0) if rows > 1 else cols, native.dtype_enum(x.dtype),
            native.dtype_enum(dy.dtype), native.dtype_enum(param_dtype), native.dtype_enum(dx_dtype),
            native.dtype_enum(sum_dtype) if sum_dtype is not None else 0, native.current_stream(device),
        )
    native.check("layer_norm_backward", status)
    _launched(device, start, "layer_norm_backward", 0.0, _nbytes(g2, x2, dx, extra, dx_cast))
    if weight is not None and dgamma is not None:
        dgamma = dgamma.reshape(weight.shape)
        dbeta = dbeta.reshape(weight.shape) if dbeta is not None else None
    return dx, dgamma, dbeta, dx_cast, dx_sum


def _layer_norm_backward_with_copy_meta(dy, x, mean, rstd, weight, want_weight=True, want_bias=True, dx_add=None,
                                        dx_dtype=None, want_cast=False, sum_dtype=None):
    cols = weight.numel() if weight is not None else x.shape[-1]
    return _layer_norm_backward_meta(dy, x, mean, rstd, weight, want_weight, want_bias, dx_add, dx_dtype) + (
        torch.empty(x.shape, dtype=torch.bfloat16, device=x.device) if want_cast else None,
        torch.empty(cols, dtype=sum_dtype, device=x.device) if sum_dtype is not None else None,
    )


def _layer_norm_backward_meta(dy, x, mean, rstd, weight, want_weight=True, want_bias=True, dx_add=None, dx_dtype=None):
    cols = weight.numel() if weight is not None else x.shape[-1]
    shape = weight.shape if weight is not None else (cols,)
    param_dtype = weight.dtype if weight is not None else x.dtype
    return (
        torch.empty(x.shape, dtype=dx_dtype or dy.dtype, device=x.device),
        torch.empty(shape, dtype=param_dtype, device=x.device) if want_weight else None,
        torch.empty(shape, dtype=param_dtype, device=x.device) if want_bias else None,
    )


def _sum_rows_cuda(x, out_dtype=None):
    device = native.require_cuda("sum_rows", x)
    out_dtype = out_dtype or x.dtype
    xr, rows, cols, row_stride = _as_rows(x)
    y = torch.empty(cols, dtype=out_dtype, device=device)
    lib = native.lib()
    ws_bytes = lib.b200_sum_rows_workspace_bytes(rows, cols, native.dtype_enum(x.dtype))
    ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=device)
    start = _prof_begin(device)
    with torch.cuda.device(device):
        status = lib.b200_sum_rows(
            xr.data_ptr(), y.data_ptr(), ws.data_ptr(), ws_bytes, rows, cols, row_stride,
            native.dtype_enum(x.dtype), native.dtype_enum(out_dtype), native.current_stream(device),
        )
    native.check("sum_rows", status)
    _launched(device, start, "sum_rows", 0.0, _nbytes(xr, y))
    return y


def _sum_rows_meta(x, out_dtype=None):
    return torch.empty(x.shape[-1] if x.dim() > 0 else 1, dtype=out_dtype or x.dtype, device=x.device)


# ---- gemm -----------------------------------------------------------------------------------


def _gemm_out_shape(a, b):
    if a.dim() == 2 and b.dim() == 2:
        if a.shape[1] != b.shape[0]:
            raise RuntimeError(f"gemm: shapes {tuple(a.shape)} and {tuple(b.shape)} cannot be multiplied")
        return (a.shape[0], b.shape[1])
    if a.dim() == 3 and b.dim() == 3:
        if a.shape[0] != b.shape[0] or a.shape[2] != b.shape[1]:
            raise RuntimeError(f"gemm: batched shapes {tuple(a.shape)} and {tuple(b.shape)} cannot be multiplied")
        return (a.shape[0], a.shape[1], b.shape[2])
    raise RuntimeError(f"gemm: operands must both be 2-D or both 3-D, got {a.dim()}-D and {b.dim()}-D")


def _gemm_empty_out(out_shape, dtype, device, operand_dim):
    """The output buffer of a GEMM. Rows of a wide 2-D output whose pitch is not a multiple of 16
    bytes (e.g. the 50257-column logits) would be misaligned for vector stores: such an output gets
    a padded pitch and is returned as the [m, n] view of it (the same idea as a padded leading
    dimension in BLAS). Used by the CUDA and the Meta implementation alike."""
    m, n = out_shape[-2], out_shape[-1]
    if operand_dim == 2 and n % 8 != 0 and n >= 1024 and m > 1:
        return torch.empty((m, (n + 7) // 8 * 8), dtype=dtype, device=device)[:, :n]
    return torch.empty(out_shape, dtype=dtype, device=device)


def fill_gemm_args(a, b, bias, residual, c, alpha, beta, epilogue, route) -> native.GemmArgs:
    """Marshals tensors into the C struct; separate from the launch so that tests can inspect it."""
    g = native.GemmArgs()
    batched = a.dim() == 3
    g.a, g.b, g.c = a.data_ptr(), b.data_ptr(), c.data_ptr()
    g.m, g.k = a.shape[-2], a.shape[-1]
    g.n = b.shape[-1]
    g.batch = a.shape[0] if batched else 1
    g.a_row_stride, g.a_col_stride = a.stride(-2), a.stride(-1)
    g.b_row_stride, g.b_col_stride = b.stride(-2), b.stride(-1)
    g.a_batch_stride = a.stride(0) if batched else 0
    g.b_batch_stride = b.stride(0) if batched else 0
    g.c_row_stride = c.stride(-2)
    g.c_batch_stride = c.stride(0) if batched else 0
    g.bias = _ptr(bias)
    g.bias_row_stride = 0
    g.bias_dtype = native.F32
    if bias is not None:
        g.bias_dtype = native.dtype_enum(bias.dtype)
        g.bias_row_stride = 0 if bias.dim() == 1 else bias.stride(0)
    g.residual = _ptr(residual)
    g.residual_row_stride = 0
    g.residual_dtype = native.F32
    if residual is not None:
        g.residual_dtype = native.dtype_enum(residual.dtype)
        g.residual_row_stride = residual.stride(0)
    g.alpha, g.beta = alpha, beta
    g.in_dtype = native.dtype_enum(a.dtype)
    g.out_dtype = native.dtype_enum(c.dtype)
    g.epilogue = epilogue
    g.route = route
    return g


def _normalise_bias(bias, m, n):
    """1-D [n] stays a broadcast row; anything else becomes an [m, n] matrix with unit column stride."""
    if bias is None:
        return None
    if bias.dim() == 1 and bias.shape[0] == n:
        return bias if bias.stride(0) == 1 else bias.contiguous()
    if bias.dim() == 2 and bias.shape[0] == 1 and bias.shape[1] == n:
        row = bias[0]
        return row if row.stride(0) == 1 else row.contiguous()
    full = bias.expand(m, n)
    if full.stride(1) != 1 or full.stride(0) < n:
        full = full.contiguous()
    return full


def _tma_pitch(t):
    """A large 2-D bf16 operand whose rows (or, for a transposed view, columns) are contiguous but
    whose pitch is not a multiple of 16 bytes (the 50257-column gradient of the logits) cannot be
    read by TMA and would take the CUDA-core kernel, ~50x slower: copy it once into a buffer with
    a padded pitch (one pass over the operand) and hand the GEMM the same view of that."""
    if t.dim() != 2 or t.dtype != torch.bfloat16 or min(t.shape) < 64 or t.numel() < (1 << 22):
        return t
    if t.stride(1) == 1 and t.stride(0) % 8 != 0:
        # The copy is kept on the tensor the operand is a view of, for as long as that tensor lives and
        # is not written to: the data and the weight gradient of a layer read the same gradient.
        root = t._base if t._base is not None else t
        try:
            key = (t.storage_offset(), tuple(t.shape), t.stride(), root._version)
        except RuntimeError:  # an inference tensor has no version counter: nothing to tell a write by
            key = None
        kept = getattr(root, "_b200_padded_pitch", None) if key is not None else None
        if kept is not None and kept[0] == key:
            return kept[1]
        rows, cols = t.shape
        padded = torch.empty((rows, (cols + 7) // 8 * 8), dtype=t.dtype, device=t.device)[:, :cols]
        padded.copy_(t)
        if key is not None:
            try:
                root._b200_padded_pitch = (key, padded)
            except (AttributeError, RuntimeError):  # a tensor subclass without attributes: copy again next time
                pass
        return padded
    if t.stride(0) == 1 and t.stride(1) % 8 != 0:
        return _tma_pitch(t.t()).t()
    return t


def _gemm_cuda(a, b, bias=None, residual=None, alpha=1.0, beta=1.0, epilogue=0, out_dtype=None, route=0):
    device = native.require_cuda("gemm", a, b, bias, residual)
    a, b = _tma_pitch(a), _tma_pitch(b)
    if a.dtype != b.dtype:
        raise RuntimeError(f"gemm: operand dtypes differ ({a.dtype} and {b.dtype})")
    out_shape = _gemm_out_shape(a, b)
    out_dtype = out_dtype or a.dtype
    m, n = out_shape[-2], out_shape[-1]
    c = _gemm_empty_out(out_shape, out_dtype, device, a.dim())
    if c.numel() == 0:
        return c
    if a.dim() == 2:
        bias = _normalise_bias(bias, m, n)
        if residual is not None and (residual.shape != c.shape or residual.stride(-1) != 1):
            residual = residual.expand(m, n).contiguous()
    elif bias is not None or residual is not None:
        if residual is not None or not (bias.dim() == 1 and bias.shape[0] == n):
            raise RuntimeError("gemm: batched gemm takes only a 1-D [n] bias")
        bias = bias.contiguous()
    g = fill_gemm_args(a, b, bias, residual, c, alpha, beta, epilogue, route)
    workspace, workspace_bytes = None, 0
    if a.dim() == 2 and (m <= 128 or a.dtype == torch.float32):
        # the routes that need scratch: split-K for small M, split-precision for fp32 operands
        workspace_bytes = native.lib().b200_gemm_workspace_bytes(ctypes.byref(g))
        if workspace_bytes:
            workspace = torch.empty(workspace_bytes, dtype=torch.uint8, device=device)
    start = _prof_begin(device)
    with torch.cuda.device(device):
        status = native.lib().b200_gemm(ctypes.byref(g), _ptr(workspace), workspace_bytes, native.current_stream(device))
    native.check("gemm", status)
    name = "gemm"
    if start is not None and getattr(native.profiler, "by_shape", False):
        # per-shape breakdown for bench_training.py --by-shape: operand layouts tell the three GEMMs of a layer apart
        layout = ("T" if a.stride(-1) != 1 else "N") + ("T" if b.stride(-1) != 1 else "N")
        name = f"gemm {g.m}x{g.k}x{g.n} {layout} {str(a.dtype).split('.')[-1]}->{str(c.dtype).split('.')[-1]}"
    _launched(device, start, name, 2.0 * g.m * g.n * g.k * g.batch, _nbytes(a, b, c, bias, residual))
    return c


def _gemm_meta(a, b, bias=None, residual=None, alpha=1.0, beta=1.0, epilogue=0, out_dtype=None, route=0):
    # same strides as the real op (padded pitch included), so that what the trace records about
    # views of the result holds at run time
    return _gemm_empty_out(_gemm_out_shape(a, b), out_dtype or a.dtype, a.device, a.dim())


# ---- sdpa -----------------------------------------------------------------------------------


def _unit_last_stride(t):
    return t if t.stride(-1) == 1 else t.contiguous()


def fill_sdpa_args(q, k, v, o, lse, causal, scale, route) -> native.SdpaArgs:
    s = native.SdpaArgs()
    s.q, s.k, s.v, s.o = q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr()
    s.lse = _ptr(lse)
    s.batch, s.heads, s.q_len, s.head_dim = q.shape
    s.kv_len = k.shape[2]
    for name, t in (("q_strides", q), ("k_strides", k), ("v_strides", v), ("o_strides", o)):
        arr = getattr(s, name)
        arr[0], arr[1], arr[2] = t.stride(0), t.stride(1), t.stride(2)
    s.scale = scale
    s.causal = int(causal)
    s.dtype = native.dtype_enum(q.dtype)
    s.route = route
    return s


def _sdpa_cuda(q, k, v, causal=False, scale=None, route=0):
    device = native.require_cuda("sdpa", q, k, v)
    if q.dim() != 4 or k.dim() != 4 or v.dim() != 4:
        raise RuntimeError("sdpa: q, k, v must be [batch, heads, length, head_dim]")
    if not (q.dtype == k.dtype == v.dtype):
        raise RuntimeError("sdpa: q, k, v dtypes differ")
    if k.shape[1] != q.shape[1] or v.shape[1] != q.shape[1]:
        raise RuntimeError("sdpa: q, k, v must have the same number of heads (expand GQA heads first)")
    if k.shape[2] != v.shape[2] or k.shape[3] != q.shape[3] or v.shape[3] != q.shape[3]:
        raise RuntimeError("sdpa: inconsistent kv_len / head_dim")
    if scale is None:
        scale = 1.0 / math.sqrt(q.shape[-1])
    q, k, v = _unit_last_stride(q), _unit_last_stride(k), _unit_last_stride(v)
    B, H, T, D = q.shape
    # Output laid out [B, T, H, D] in memory (returned as its [B, H, T, D] view): the layout the
    # following `transpose(1, 2).view(B, T, C)` wants, so that it stays a view.
    o = torch.empty((B, T, H, D), dtype=q.dtype, device=device).transpose(1, 2)
    lse = torch.empty((B, H, T), dtype=torch.float32, device=device)
    if o.numel() == 0:
        return o, lse
    s = fill_sdpa_args(q, k, v, o, lse, causal, scale, route)
    start = _prof_begin(device)
    with torch.cuda.device(device):
        status = native.lib().b200_sdpa_fwd(ctypes.byref(s), native.current_stream(device))
    native.check("sdpa", status)
    flops = 4.0 * B * H * T * k.shape[2] * D * (0.5 if causal else 1.0)
    _launched(device, start, "sdpa", flops, _nbytes(q, k, v, o))
    return o, lse


def _sdpa_meta(q, k, v, causal=False, scale=None, route=0):
    B, H, T, D = q.shape
    o = torch.empty((B, T, H, D), dtype=q.dtype, device=q.device).transpose(1, 2)
    return o, torch.empty((B, H, T), dtype=torch.float32, device=q.device)


_SDPA_BWD_WORKSPACE_BYTES = 2 << 30


def sdpa_backward_supported(q, k, v) -> bool:
    """What b200_sdpa_bwd takes: bf16, head_dim 64, equal head counts."""
    return (
        q.dtype == torch.bfloat16 and k.dtype == torch.bfloat16 and v.dtype == torch.bfloat16
        and q.dim() == 4 and q.shape[-1] == 64 and v.shape[-1] == 64 and k.shape[1] == q.shape[1]
        and q.shape[2] > 0 and k.shape[2] > 0
    )


def _sdpa_backward_cuda(d_out, q, k, v, o, lse, causal=False, scale=None):
    device = native.require_cuda("sdpa_backward", d_out, q, k, v, o, lse)
    if not sdpa_backward_supported(q, k, v):
        raise RuntimeError("sdpa_backward: the kernel takes bf16 tensors with head_dim 64 and equal head counts")
    B, H, T, D = q.shape
    S = k.shape[2]
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    q, k, v, o = _unit_last_stride(q), _unit_last_stride(k), _unit_last_stride(v), _unit_last_stride(o)
    d_out = _unit_last_stride(d_out.to(q.dtype))
    lse_c = lse.reshape(B, H, -1)[:, :, :T].float().contiguous()
    # Gradients laid out [B, T, H, D] in memory (returned as their [B, H, T, D] views), like the forward's
    # output: the `transpose(1, 2)` + `contiguous` that follows in a projection's backward is then a view.
    dq, dk, dv = _sdpa_gradient_buffers(B, H, T, S, D, q.dtype, device)
    lib = native.lib()

    def args_for(b0, b1):
        a = native.SdpaBwdArgs()
        a.q, a.k, a.v, a.o, a.d_out, a.lse = (t[b0:b1].data_ptr() for t in (q, k, v, o, d_out, lse_c))
        a.dq, a.dk, a.dv = dq[b0:b1].data_ptr(), dk[b0:b1].data_ptr(), dv[b0:b1].data_ptr()
        a.batch, a.heads, a.q_len, a.kv_len, a.head_dim = b1 - b0, H, T, S, D
        for name, t in (("q_strides", q), ("k_strides", k), ("v_strides", v), ("o_strides", o), ("d_out_strides", d_out),
                        ("dq_strides", dq), ("dk_strides", dk), ("dv_strides", dv)):
            arr = getattr(a, name)
            arr[0], arr[1], arr[2] = t.stride(0), t.stride(1), t.stride(2)
        a.scale, a.causal, a.dtype = float(scale), int(bool(causal)), native.dtype_enum(q.dtype)
        return a

    # The per-key-tile shares of dQ live in the workspace (kv_tiles x q_tiles x 32 KB per (batch, head)):
    # long sequences are processed a few batch entries at a time so that it stays below ~2 GB.
    per_batch = lib.b200_sdpa_bwd_workspace_bytes(ctypes.byref(args_for(0, 1)))
    step = max(1, min(B, _SDPA_BWD_WORKSPACE_BYTES // max(per_batch, 1)))
    ws = torch.empty(max(per_batch * step, 256), dtype=torch.uint8, device=device)
    start = _prof_begin(device)
    with torch.cuda.device(device):
        for b0 in range(0, B, step):
            a = args_for(b0, min(B, b0 + step))
            a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
            native.check("sdpa_backward", lib.b200_sdpa_bwd(ctypes.byref(a), native.current_stream(device)))
    flops = 10.0 * B * H * T * S * D * (0.5 if causal else 1.0)
    _launched(device, start, "sdpa_backward", flops, _nbytes(q, k, v, o, d_out, dq, dk, dv))
    return dq, dk, dv


def _sdpa_gradient_buffers(B, H, T, S, D, dtype, device):
    """dq, dk, dv as [B, H, T, D] views of memory laid out [B, T, H, D]. For self-attention the three
    share one [B, T, 3, H, D] buffer: the gradient of a fused QKV projection's output, which the graph
    builds with `cat([dq, dk, dv], -1)`, is then that buffer and the concatenation copies nothing."""
    if T == S:
        packed = torch.empty((B, T, 3, H, D), dtype=dtype, device=device)
        return tuple(packed[:, :, i].transpose(1, 2) for i in range(3))
    return (
        torch.empty((B, T, H, D), dtype=dtype, device=device).transpose(1, 2),
        torch.empty((B, S, H, D), dtype=dtype, device=device).transpose(1, 2),
        torch.empty((B, S, H, D), dtype=dtype, device=device).transpose(1, 2),
    )


def _sdpa_backward_meta(d_out, q, k, v, o, lse, causal=False, scale=None):
    B, H, T, D = q.shape
    return _sdpa_gradient_buffers(B, H, T, k.shape[2], D, q.dtype, q.device)


# ---- embedding (+ second table) ---------------------------------------------------------------


def _embedding_sum_cuda(table, indices, table2=None, indices2=None, out_dtype=None):
    device = native.require_cuda("embedding_sum", table, indices, table2, indices2)
    out_dtype = out_dtype or table.dtype
    if table.dim() != 2 or table.stride(1) != 1:
        raise RuntimeError("embedding_sum: the table must be [rows, cols] with a unit column stride")
    if indices.dtype != torch.int64:
        indices = indices.long()
    idx = indices.contiguous()
    rows, cols = idx.numel(), table.shape[1]
    idx2, period = None, 0
    if table2 is not None:
        if table2.dtype != table.dtype or table2.dim() != 2 or table2.shape[1] != cols or table2.stride(1) != 1:
            raise RuntimeError("embedding_sum: the second table must match the first in dtype and width")
        idx2 = (indices2 if indices2.dtype == torch.int64 else indices2.long()).contiguous()
        period = idx2.numel()
        # indices2 broadcasts against indices from the right: its flattened length must tile the rows
        if period == 0 or rows % period != 0 or tuple(indices.shape[indices.dim() - idx2.dim():]) != tuple(idx2.shape):
            raise RuntimeError(
                f"embedding_sum: indices2 {tuple(indices2.shape)} does not broadcast over indices {tuple(indices.shape)}")
    out = torch.empty((*indices.shape, cols), dtype=out_dtype, device=device)
    if out.numel() == 0:
        return out
    start = _prof_begin(device)
    with torch.cuda.device(device):
        status = native.lib().b200_embedding_sum(
            table.data_ptr(), idx.data_ptr(), table.shape[0], table.stride(0), _ptr(table2), _ptr(idx2),
            table2.shape[0] if table2 is not None else 0, table2.stride(0) if table2 is not None else 0, period,
            out.data_ptr(), rows, cols, native.dtype_enum(table.dtype), native.dtype_enum(out_dtype),
            native.current_stream(device),
        )
    native.check("embedding_sum", status)
    nb = rows * cols * (table.element_size() * (2 if table2 is not None else 1) + out.element_size())
    _launched(device, start, "embedding", 0.0, float(nb))
    return out


def _embedding_sum_meta(table, indices, table2=None, indices2=None, out_dtype=None):
    return torch.empty((*indices.shape, table.shape[1]), dtype=out_dtype or table.dtype, device=table.device)


# ---- argmax over the last dim -----------------------------------------------------------------


def _argmax_cuda(x):
    device = native.require_cuda("argmax", x)
    if x.dim() == 0 or x.shape[-1] == 0:
        raise RuntimeError("argmax: needs a non-empty last dim")
    # contiguous tensors and 2-D views with a padded pitch (the logits) are read in place
    xr, rows, cols, row_stride = _as_rows(x)
    out = torch.empty(x.shape[:-1], dtype=torch.int64, device=device)
    if out.numel() == 0:
        return out
    start = _prof_begin(device)
    with torch.cuda.device(device):
        status = native.lib().b200_argmax_lastdim(
            xr.data_ptr(), out.data_ptr(), rows, cols, row_stride, native.dtype_enum(x.dtype), native.current_stream(device))
    native.check("argmax", status)
    _launched(device, start, "argmax", 0.0, float(rows * cols * x.element_size()))
    return out


def _argmax_meta(x):
    return torch.empty(x.shape[:-1], dtype=torch.int64, device=x.device)


# ---- concatenation and cache append (strided block copies) -------------------------------------


def _copy_block(dst, src, dim, device):
    """dst and src have the same shape except that dst may be a slice (along `dim`) of a larger
    contiguous tensor; both are dense from `dim` on."""
    outer = math.prod(src.shape[:dim])
    inner = math.prod(src.shape[dim:])
    if outer == 0 or inner == 0:
        return
    dst_stride = dst.stride(dim - 1) if dim > 0 else inner
    src_stride = src.stride(dim - 1) if dim > 0 else inner
    with torch.cuda.device(device):
        status = native.lib().b200_copy_rows(dst.data_ptr(), src.data_ptr(), outer, inner, dst_stride, src_stride,
                                             src.element_size(), native.current_stream(device))
    native.check("copy_rows", status)
    native.launch_count += 1


def _cat_cuda(tensors, dim=0):
    tensors = [t for t in tensors if not (t.dim() == 1 and t.numel() == 0)]  # torch skips legacy empty tensors
    device = native.require_cuda("cat", *tensors)
    first = tensors[0]
    dim = dim % first.dim()
    dtype = first.dtype
    for t in tensors:
        if t.dtype != dtype:
            raise RuntimeError("cat: mixed dtypes are not supported")
    shape = list(first.shape)
    shape[dim] = sum(t.shape[dim] for t in tensors)
    out = torch.empty(shape, dtype=dtype, device=device)
    start = _prof_begin(device)
    offset = 0
    for t in tensors:
        tc = t if t.is_contiguous() else t.contiguous()
        _copy_block(out.narrow(dim, offset, t.shape[dim]), tc, dim, device)
        offset += t.shape[dim]
    if start is not None:
        native.profiler.end(device, start, "cat", 0.0, 2.0 * out.numel() * out.element_size())
    return out


def _cat_meta(tensors, dim=0):
    tensors = [t for t in tensors if not (t.dim() == 1 and t.numel() == 0)]
    first = tensors[0]
    dim = dim % first.dim()
    shape = list(first.shape)
    shape[dim] = sum(t.shape[dim] for t in tensors)
    return torch.empty(shape, dtype=first.dtype, device=first.device)


def _kv_append_cuda(cache, new, position):
    """cache[..., position : position + t, :] = new, in place: the decode-loop alternative to
    `torch.cat([cache, new], dim=-2)`, which re-copies the whole cache every step. cache is a
    contiguous [..., T_max, D]; new is [..., t, D] with the same leading dims."""
    device = native.require_cuda("kv_append", cache, new)
    if cache.dim() < 2 or new.dim() != cache.dim() or cache.dtype != new.dtype:
        raise RuntimeError("kv_append: cache and new must have the same rank and dtype")
    if tuple(cache.shape[:-2]) != tuple(new.shape[:-2]) or cache.shape[-1] != new.shape[-1]:
        raise RuntimeError(f"kv_append: shapes {tuple(cache.shape)} and {tuple(new.shape)} do not match")
    t = new.shape[-2]
    if position < 0 or position + t > cache.shape[-2]:
        raise RuntimeError(f"kv_append: positions [{position}, {position + t}) outside a cache of {cache.shape[-2]}")
    if not cache.is_contiguous():
        raise RuntimeError("kv_append: the cache must be contiguous")
    nc = new if new.is_contiguous() else new.contiguous()
    _copy_block(cache.narrow(-2, position, t), nc, cache.dim() - 2, device)


def _kv_append_meta(cache, new, position):
    return None


def _refuse_cpu(name):
    def impl(*args, **kwargs):
        raise RuntimeError(
            f"b200::{name} was called with CPU tensors; the b200 kernels run on CUDA tensors only "
            "and there is no CPU fallback."
        )

    return impl


for _name, _cuda, _meta in (
    ("layer_norm", _layer_norm_cuda, _layer_norm_meta),
    ("softmax", _softmax_cuda, _softmax_meta),
    ("softmax_masked", _softmax_masked_cuda, _softmax_masked_meta),
    ("gelu", _gelu_cuda, _gelu_meta),
    ("reduce", _reduce_cuda, _reduce_meta),
    ("gelu_backward", _gelu_backward_cuda, _gelu_backward_meta),
    ("softmax_backward", _softmax_backward_cuda, _softmax_backward_meta),
    ("layer_norm_backward", _layer_norm_backward_cuda, _layer_norm_backward_meta),
    ("layer_norm_backward_with_copy", _layer_norm_backward_with_copy_cuda, _layer_norm_backward_with_copy_meta),
    ("sum_rows", _sum_rows_cuda, _sum_rows_meta),
    ("gemm", _gemm_cuda, _gemm_meta),
    ("sdpa", _sdpa_cuda, _sdpa_meta),
    ("sdpa_backward", _sdpa_backward_cuda, _sdpa_backward_meta),
    ("embedding_sum", _embedding_sum_cuda, _embedding_sum_meta),
    ("argmax", _argmax_cuda, _argmax_meta),
    ("cat", _cat_cuda, _cat_meta),
    ("kv_append", _kv_append_cuda, _kv_append_meta),
):
    _lib.impl(_name, _cuda, "CUDA")
    _lib.impl(_name, _refuse_cpu(_name), "CPU")
    torch.library.register_fake(f"b200::{_name}", _meta, lib=_lib)

layer_norm = torch.ops.b200.layer_norm
softmax = torch.ops.b200.softmax
softmax_masked = torch.ops.b200.softmax_masked
gelu = torch.ops.b200.gelu
reduce = torch.ops.b200.reduce
gelu_backward = torch.ops.b200.gelu_backward
softmax_backward = torch.ops.b200.softmax_backward
layer_norm_backward = torch.ops.b200.layer_norm_backward
layer_norm_backward_with_copy = torch.ops.b200.layer_norm_backward_with_copy
sum_rows = torch.ops.b200.sum_rows
gemm = torch.ops.b200.gemm
sdpa = torch.ops.b200.sdpa
sdpa_backward = torch.ops.b200.sdpa_backward
embedding_sum = torch.ops.b200.embedding_sum
argmax = torch.ops.b200.argmax
cat = torch.ops.b200.cat
kv_append = torch.ops.b200.kv_append
