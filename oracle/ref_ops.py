"""CPU oracle for the aten-lowering hot path. TEST INFRASTRUCTURE ONLY.

Only `tests/`, `__graft_entry__.smoke()` and the CPU-baseline / reference legs of `bench.py` may
import this module; nothing in the shipped package does, and the product path has no CPU route.

What it restates. The reference computes these ops inside Modular MAX
(`max==26.5.0.dev2026072306`, pinned in the reference's pyproject.toml:82-89), a binary wheel that
is not part of the reference tree and cannot be installed offline, so the reference itself cannot
run here. Its own tests pin the path to **PyTorch CPU eager** on the same inputs
(torch_mojo_backend/testing.py:139-166 and 186-229). The oracle therefore is:

  * for each op, a plain numpy restatement (float64 accumulation) of the formula the reference
    lowering or the reference's own CPU loop writes down, each citing file:line below; and
  * PyTorch CPU eager of the same op, which `tests/test_oracle.py` checks the restatements
    against, together with the known-answer vectors the reference's tests hold (bf16 GELU bit
    patterns, tests/test_eager_kernels.py:1998-2032) and the fixtures under `tests/golden/`
    that were generated from PyTorch CPU eager by `tests/golden/make_golden.py`.

Parity status: pinned to PyTorch CPU eager (the reference's own oracle) and to the reference's
known-answer vectors; not pinned to MAX outputs, which cannot be produced here.

bf16 convention ("bf16 with fp32 accumulation"): operands are rounded to bf16 first, the math
runs in fp32/fp64, and the result is rounded once to the output dtype.
"""

from __future__ import annotations

import math

import numpy as np
import torch


def _np(x: torch.Tensor) -> np.ndarray:
    """Tensor -> float64 numpy array of the exact stored values (bf16 widens losslessly)."""
    return x.detach().to(torch.float64).cpu().numpy()


def _out(a, dtype: torch.dtype) -> torch.Tensor:
    a = np.asarray(a)
    return torch.from_numpy(np.ascontiguousarray(a)).reshape(a.shape).to(dtype)


# ---- LayerNorm --------------------------------------------------------------------------------
def layer_norm(x, normalized_shape, weight, bias, eps, out_dtype=None):
    """(y, mean, rstd) with two-pass centred variance and rstd = 1/sqrt(var + eps).

    Follows the reference's CPU loop (torch_mojo_backend/eager_kernels/nn_ops.mojo:299-326) and
    its graph lowering (torch_mojo_backend/aten_functions.py:2851-2868): mean over the normalised
    dims, variance of the centred values, then scale and shift. mean/rstd are fp32 and keep
    the normalised dims as size 1.
    """
    k = len(normalized_shape)
    a = _np(x)
    axes = tuple(range(a.ndim - k, a.ndim))
    mean = a.mean(axis=axes, keepdims=True)
    centered = a - mean
    var = (centered * centered).mean(axis=axes, keepdims=True)
    rstd = 1.0 / np.sqrt(var + eps)
    y = centered * rstd
    if weight is not None:
        y = y * _np(weight)
    if bias is not None:
        y = y + _np(bias)
    return _out(y, out_dtype or x.dtype), _out(mean, torch.float32), _out(rstd, torch.float32)


# ---- softmax ----------------------------------------------------------------------------------
def softmax_rows(x, scale=1.0, causal=False, q_len=0, out_dtype=None):
    """Row softmax over the last dim with optional scale and top-left-aligned causal mask.

    Follows the reference's CPU loop (torch_mojo_backend/eager_kernels/nn_ops.mojo:428-455): for
    row r, `allowed = min(cols, r % q_len + 1)`; the maximum and the denominator run over the
    allowed columns of `x * scale`; masked columns are written as exact 0. Without the mask it
    is the lowering's `exp(x - amax) / sum` (torch_mojo_backend/aten_functions.py:690-714).
    """
    a = _np(x) * scale
    cols = a.shape[-1]
    flat = a.reshape(-1, cols)
    out = np.zeros_like(flat)
    for r in range(flat.shape[0]):
        allowed = min(cols, r % q_len + 1) if causal else cols
        row = flat[r, :allowed]
        m = row.max() if allowed > 0 else 0.0
        with np.errstate(invalid="ignore"):
            e = np.exp(row - m)
            out[r, :allowed] = e / e.sum()
    return _out(out.reshape(a.shape), out_dtype or x.dtype)


def softmax(x, dim=-1, out_dtype=None):
    """`aten._softmax` / `aten.softmax` along any dim (torch_mojo_backend/aten_functions.py:680-714)."""
    a = np.moveaxis(_np(x), dim, -1)
    with np.errstate(invalid="ignore"):
        e = np.exp(a - a.max(axis=-1, keepdims=True))
        y = e / e.sum(axis=-1, keepdims=True)
    return _out(np.moveaxis(y, -1, dim), out_dtype or x.dtype)


# ---- GELU -------------------------------------------------------------------------------------
_erf = np.vectorize(math.erf, otypes=[np.float64])


def gelu(x, approximate="none"):
    """Elementwise GELU, exact (erf) or tanh form; widen, compute, round once.

    Formulas of `aten.gelu` that the reference lowers one-to-one
    (torch_mojo_backend/aten_functions.py:2062-2067) and that its bf16 kernels implement as
    "widen -> fp32 -> round once"
    (torch_mojo_backend/eager_kernels/activation_forward_kernels.mojo:22-56).
    """
    a = _np(x)
    with np.errstate(invalid="ignore", over="ignore"):
        if approximate == "tanh":
            inner = math.sqrt(2.0 / math.pi) * (a + 0.044715 * a * a * a)
            y = 0.5 * a * (1.0 + np.tanh(inner))
        else:
            y = 0.5 * a * (1.0 + _erf(a / math.sqrt(2.0)))
    return _out(y, x.dtype)


def gelu_backward(dy, x, approximate="none"):
    """dy * gelu'(x), formulas of the reference's kernels
    (torch_mojo_backend/eager_kernels/activation_backward_ops.mojo:44-72: exact
    Phi(x) + x phi(x); tanh 0.5 (1 + t) + 0.5 x (1 - t^2) beta (1 + 3 kappa x^2))."""
    a, g = _np(x), _np(dy)
    with np.errstate(invalid="ignore", over="ignore"):
        if approximate == "tanh":
            beta, kappa = math.sqrt(2.0 / math.pi), 0.044715
            t = np.tanh(beta * (a + kappa * a * a * a))
            d = 0.5 * (1.0 + t) + 0.5 * a * (1.0 - t * t) * beta * (1.0 + 3.0 * kappa * a * a)
        else:
            d = 0.5 * (1.0 + _erf(a / math.sqrt(2.0))) + a * np.exp(-0.5 * a * a) / math.sqrt(2.0 * math.pi)
    return _out(g * d, x.dtype)


# ---- backward of the row kernels ----------------------------------------------------------------
def softmax_backward(dy, y, scale=1.0, out_dtype=None):
    """scale * y * (dy - sum_j dy_j y_j) over the last dim: aten._softmax_backward_data (scale 1), and
    with the score scale folded in, the softmax backward of the reference's decomposed attention
    (torch_mojo_backend/eager_kernels/sdpa_backward_ops.mojo:28-78)."""
    g, p = _np(dy), _np(y)
    return _out(scale * p * (g - (g * p).sum(-1, keepdims=True)), out_dtype or y.dtype)


def layer_norm_backward(dy, x, mean, rstd, weight):
    """(dx, dgamma, dbeta) from the forward's statistics
    (torch_mojo_backend/eager_kernels/normalization_backward_dx.mojo:66-175 for dx,
    normalization_backward_params.mojo:75-180 for the parameter sums):
    xhat = (x - mean) rstd, g = dy gamma, dx = rstd (g - mean(g) - xhat mean(g xhat)),
    dgamma = sum_rows dy xhat, dbeta = sum_rows dy."""
    cols = x.shape[-1]
    a, g = _np(x).reshape(-1, cols), _np(dy).reshape(-1, cols)
    mu, rs = _np(mean).reshape(-1, 1), _np(rstd).reshape(-1, 1)
    xh = (a - mu) * rs
    gg = g * (_np(weight) if weight is not None else 1.0)
    dx = rs * (gg - gg.mean(-1, keepdims=True) - xh * (gg * xh).mean(-1, keepdims=True))
    pd = weight.dtype if weight is not None else x.dtype
    return _out(dx.reshape(x.shape), dy.dtype), _out((g * xh).sum(0), pd), _out(g.sum(0), pd)


def sum_rows(x, out_dtype=None):
    """Sum over every dim but the last (a bias gradient; torch_mojo_backend/aten_functions.py:2323-2380)."""
    return _out(_np(x).reshape(-1, x.shape[-1]).sum(0), out_dtype or x.dtype)


def sdpa_backward(d_out, q, k, v, causal=False, scale=None):
    """(dq, dk, dv) of softmax(scale q k^T [+ causal mask]) v in float64: P recomputed, dV = P^T dO,
    dP = dO V^T, dS = scale P (dP - rowsum(dP P)), dQ = dS K, dK = dS^T Q (the math of
    torch_mojo_backend/eager_flash_attention/fa4_bwd_kernel.mojo)."""
    Q, K, V, dO = _np(q), _np(k), _np(v), _np(d_out)
    T, S, D = Q.shape[-2], K.shape[-2], Q.shape[-1]
    scale = float(scale) if scale is not None else 1.0 / math.sqrt(D)
    s = np.einsum("...td,...sd->...ts", Q, K) * scale
    if causal:
        s = np.where(np.tril(np.ones((T, S), dtype=bool)), s, -np.inf)
    s = s - s.max(-1, keepdims=True)
    p = np.exp(s)
    p = p / p.sum(-1, keepdims=True)
    dv = np.einsum("...ts,...td->...sd", p, dO)
    dp = np.einsum("...td,...sd->...ts", dO, V)
    ds = scale * p * (dp - (dp * p).sum(-1, keepdims=True))
    dq = np.einsum("...ts,...sd->...td", ds, K)
    dk = np.einsum("...ts,...td->...sd", ds, Q)
    return _out(dq, q.dtype), _out(dk, k.dtype), _out(dv, v.dtype)


# ---- reductions -------------------------------------------------------------------------------
def reduce(x, op, dim=None, keepdim=False, out_dtype=None):
    """sum / mean / amax over `dim` (list, int or None = all dims).

    Semantics of the reference lowerings: one reduction per listed axis followed by squeezes
    (sum: torch_mojo_backend/aten_functions.py:3310-3346, mean: :2554-2603, amax: :1001-1020).
    """
    a = _np(x)
    if dim is None or (isinstance(dim, (list, tuple)) and len(dim) == 0):
        axes = tuple(range(a.ndim))
    elif isinstance(dim, int):
        axes = (dim,)
    else:
        axes = tuple(dim)
    fn = {"sum": np.sum, "mean": np.mean, "amax": np.max}[op]
    return _out(fn(a, axis=axes, keepdims=keepdim), out_dtype or x.dtype)


# ---- GEMM family ------------------------------------------------------------------------------
def mm(a, b, out_dtype=None):
    """`x @ y` (torch_mojo_backend/aten_functions.py:2631-2634)."""
    return _out(_np(a) @ _np(b), out_dtype or a.dtype)


def addmm(inp, mat1, mat2, beta=1.0, alpha=1.0, out_dtype=None):
    """`beta * input + alpha * (mat1 @ mat2)`, scaling applied in that order
    (torch_mojo_backend/aten_functions.py:970-992)."""
    prod = _np(mat1) @ _np(mat2)
    if alpha != 1.0:
        prod = prod * alpha
    scaled = _np(inp) * beta if beta != 1.0 else _np(inp)
    return _out(scaled + prod, out_dtype or mat1.dtype)


def bmm(a, b, out_dtype=None):
    """Batched matmul (torch_mojo_backend/aten_functions.py:1414-1428)."""
    return _out(np.matmul(_np(a), _np(b)), out_dtype or a.dtype)


# ---- attention --------------------------------------------------------------------------------
def sdpa(q, k, v, causal=False, scale=None):
    """(out, lse) of softmax(scale * Q K^T + mask) V per (batch, head), [B, H, T, D] tensors.

    The math of the reference's matmul formulation
    (torch_mojo_backend/aten_functions.py:573-599 and :443-504), with the causal mask top-left
    aligned (key j visible to query i iff j <= i;
    torch_mojo_backend/eager_kernels/nn_ops.mojo:394-397) and the default scale 1/sqrt(D)
    (aten_functions.py:560-566). lse is the natural-log log-sum-exp of the scaled, masked scores,
    fp32 [B, H, T] (torch_mojo_backend/eager_flash_attention/fa4_fwd_kernel.mojo:958-980).
    """
    qa, ka, va = _np(q), _np(k), _np(v)
    d = qa.shape[-1]
    if scale is None:
        scale = 1.0 / math.sqrt(d)
    s = np.matmul(qa, np.swapaxes(ka, -1, -2)) * scale
    if causal:
        L, S = s.shape[-2], s.shape[-1]
        mask = np.tril(np.ones((L, S), dtype=bool))
        s = np.where(mask, s, -np.inf)
    m = s.max(axis=-1, keepdims=True)
    with np.errstate(invalid="ignore"):
        e = np.exp(s - m)
        denom = e.sum(axis=-1, keepdims=True)
        out = np.matmul(e / denom, va)
    lse = (m + np.log(denom))[..., 0]
    return _out(out, q.dtype), _out(lse, torch.float32)


# ---- whole-model oracle -----------------------------------------------------------------------
def gpt2_logits_fp32(model: torch.nn.Module, idx: torch.Tensor) -> torch.Tensor:
    """PyTorch CPU eager forward in fp32 of a GPT-2 whose parameters hold the values the device
    model uses (for the bf16 policy: the bf16-rounded weights, widened to fp32). This is the
    oracle the reference's tests use for whole models (run_hf_mojo.py:26-55)."""
    import copy

    ref = copy.deepcopy(model).to("cpu")
    ref.set_precision("fp32")  # widens bf16 parameters losslessly; all math in fp32
    ref.eval()
    with torch.no_grad():
        return ref(idx.to("cpu"))
