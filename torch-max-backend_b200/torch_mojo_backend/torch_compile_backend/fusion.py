"""Graph-level fusion run on the aten FX graph before the launch plan is built.

The reference leaves fusion to MAX (its lowerings emit separate matmul / mul / add graph ops,
torch_mojo_backend/aten_functions.py:970-992, and MAX fuses elementwise chains). Here the kernels
are hand-written, so the chains that matter are matched explicitly and folded into kernel
epilogues:

  * `native_layer_norm -> getitem[0] -> _to_copy(dtype)`         => LayerNorm that writes `dtype`
  * `addmm | mm -> views -> [gelu] -> views -> [_to_copy(float32)] -> views -> [add(residual, .)]`
        => one GEMM whose epilogue applies bias, GELU, the residual add and the output dtype to
           the fp32 accumulator (an fp32 result is stored as computed, without the intermediate
           bf16 rounding the unfused graph would do)
  * `[_to_copy(bf16 -> float32)] -> native_layer_norm_backward -> getitem[0] -> [add(residual grad, .)]`
        => one LayerNorm backward that reads the bf16 gradient and adds the residual branch's
           gradient before it stores dx (the backward of a pre-norm transformer block)
  * `sdpa -> getitem[0] -> transpose -> clone(contiguous)`        => no copy: the attention kernel
        already writes its output in the [B, T, H, D] order that `clone` would produce
  * `[mul | div (scalar)] -> masked_fill(mask, value) | where(keep, ., value) -> _softmax(-1)`
        => one masked softmax over the scores of a decomposed attention (the reference's fused
           contract is SoftmaxRows(scale, causal, q_len), eager_kernels/nn_ops.mojo:392-409; the
           mask here is explicit, so nothing is assumed about its values)

  * `embedding(wte, idx)[.to(dt)] + embedding(wpe, pos)[.to(dt)]`  => one gather kernel that reads
        both tables, adds in fp32 and writes `dt` (token + positional embeddings)

Every intermediate node of a chain must have exactly one user; chains with symbolic shapes are
left alone. Fused nodes call functions registered in MAPPING_TORCH_ATEN_TO_MOJO under themselves,
so the graph walk treats them like any other lowering. TORCH_MOJO_BACKEND_NO_FUSION=1 disables
the pass.
"""

from __future__ import annotations

import operator
import os

import torch

from torch_mojo_backend import aten_functions as af
from torch_mojo_backend import native

aten = torch.ops.aten

VIEW_OPS = (aten.view.default, aten._unsafe_view.default, aten.reshape.default)
ALIAS_OPS = VIEW_OPS + (aten.transpose.int, aten.permute.default, aten.t.default, operator.getitem)
SDPA_OPS = (
    aten._scaled_dot_product_flash_attention.default,
    aten._scaled_dot_product_efficient_attention.default,
    aten._scaled_dot_product_cudnn_attention.default,
    aten.scaled_dot_product_attention.default,
    # the gradients of the fused backward come out in [B, T, H, D] memory order as well
    aten._scaled_dot_product_flash_attention_backward.default,
    aten._scaled_dot_product_efficient_attention_backward.default,
    aten._scaled_dot_product_cudnn_attention_backward.default,
)


def fusion_enabled() -> bool:
    return os.environ.get("TORCH_MOJO_BACKEND_NO_FUSION", "0").lower() not in ("1", "true", "yes")


def _val(node):
    return node.meta.get("val") if isinstance(node, torch.fx.Node) else None


def _static_tensor(node) -> bool:
    v = _val(node)
    return isinstance(v, torch.Tensor) and all(isinstance(d, int) for d in v.shape)


def _only_user(node):
    if len(node.users) != 1:
        return None
    return next(iter(node.users))


def _is_call(node, *targets) -> bool:
    return node is not None and node.op == "call_function" and node.target in targets


def _skip_views(node):
    while True:
        user = _only_user(node)
        if _is_call(user, *VIEW_OPS) and user.args[0] is node and _static_tensor(user):
            node = user
        else:
            return node


def _plain_cast(node) -> torch.dtype | None:
    """dtype of a `_to_copy` that only changes dtype, else None."""
    if not _is_call(node, aten._to_copy.default):
        return None
    source = _val(node.args[0])
    for key, value in node.kwargs.items():
        if key == "dtype" or value in (None, False):
            continue
        # autograd spells the layout and the device out; they change nothing when they are the input's
        if key == "layout" and value == torch.strided:
            continue
        if key == "device" and isinstance(source, torch.Tensor) and torch.device(value) == source.device:
            continue
        return None
    return node.kwargs.get("dtype")


def _replace(graph, old, func, args, kwargs):
    with graph.inserting_after(old):
        new = graph.call_function(func, args=args, kwargs=kwargs)
    new.meta = dict(old.meta)
    old.replace_all_uses_with(new)
    return new


def _fuse_layer_norm(graph) -> int:
    count = 0
    for node in list(graph.nodes):
        if not _is_call(node, aten.native_layer_norm.default):
            continue
        get0 = _only_user(node)
        if not (_is_call(get0, operator.getitem) and get0.args[1] == 0):
            continue
        cast = _only_user(get0)
        dtype = _plain_cast(cast)
        x = _val(node.args[0])
        if dtype is None or not native.supported_dtype(dtype) or not isinstance(x, torch.Tensor):
            continue
        if not native.supported_dtype(x.dtype):
            continue
        _replace(graph, cast, af.fused_layer_norm, tuple(node.args), {"out_dtype": dtype})
        count += 1
    return count


def _fuse_layer_norm_with_statistics(graph) -> int:
    """The same fold in a graph that also uses the statistics (the forward of a training step keeps
    mean and rstd for the backward): output 0 -> cast becomes output 0 of a node that returns
    (y in the cast's dtype, mean, rstd)."""
    count = 0
    for node in list(graph.nodes):
        if not _is_call(node, aten.native_layer_norm.default):
            continue
        items = {}
        for user in node.users:
            if not (_is_call(user, operator.getitem) and user.args[0] is node and user.args[1] in (0, 1, 2)):
                items = None
                break
            if user.args[1] in items:
                items = None
                break
            items[user.args[1]] = user
        if not items or 0 not in items or len(items) < 2:
            continue  # no statistics in use: _fuse_layer_norm's case
        cast = _only_user(items[0])
        dtype = _plain_cast(cast)
        x = _val(node.args[0])
        if dtype is None or not native.supported_dtype(dtype) or not isinstance(x, torch.Tensor):
            continue
        if not native.supported_dtype(x.dtype):
            continue
        with graph.inserting_after(node):
            new = graph.call_function(af.fused_layer_norm_with_statistics, args=tuple(node.args), kwargs={"out_dtype": dtype})
        old_val = _val(node)
        new.meta = dict(node.meta)
        if isinstance(old_val, (tuple, list)):
            new.meta["val"] = (_val(cast),) + tuple(old_val[1:])
        with graph.inserting_after(new):
            y = graph.call_function(operator.getitem, args=(new, 0))
        y.meta = dict(cast.meta)
        cast.replace_all_uses_with(y)
        for index in (1, 2):
            if index in items:
                items[index].args = (new, index)
        count += 1
    return count


def _fuse_layer_norm_backward(graph) -> int:
    """`_to_copy(bf16 -> fp32) -> native_layer_norm_backward -> getitem[0] -> add(residual gradient, .)`
    as one launch: the kernel reads the bf16 gradient, and adds the gradient of the residual branch
    before it stores dx. Either half of the chain is folded on its own when the other is absent."""
    order = {node: i for i, node in enumerate(graph.nodes)}
    count = 0
    for node in list(graph.nodes):
        if not _is_call(node, aten.native_layer_norm_backward.default) or node.kwargs:
            continue
        grad, x = node.args[0], node.args[1]
        vg, vx = _val(grad), _val(x)
        if not (isinstance(vg, torch.Tensor) and isinstance(vx, torch.Tensor) and _static_tensor(x)):
            continue
        if vg.dtype != torch.float32 or vx.dtype != torch.float32 or not node.args[7][0]:
            continue
        kwargs = {}
        source = grad
        while _is_call(source, *VIEW_OPS):
            source = source.args[0]
        narrow = source.args[0] if _plain_cast(source) == torch.float32 else None
        if (
            narrow is not None
            and source is grad  # views between the cast and the kernel would have to be replayed
            and len(grad.users) == 1
            and isinstance(_val(narrow), torch.Tensor)
            and _val(narrow).dtype == torch.bfloat16
        ):
            grad = narrow
            kwargs["dx_dtype"] = torch.float32
        dx = next((u for u in node.users if _is_call(u, operator.getitem) and u.args[1] == 0), None)
        add = _only_user(dx) if dx is not None else None
        target = None
        if (
            _is_call(add, aten.add.Tensor)
            and add.kwargs.get("alpha", 1) == 1
            and len(add.args) == 2
            and all(isinstance(a, torch.fx.Node) for a in add.args)
        ):
            other = add.args[1] if add.args[0] is dx else add.args[0]
            vo = _val(other)
            if (
                other is not dx
                and isinstance(vo, torch.Tensor)
                and vo.dtype == torch.float32
                and tuple(vo.shape) == tuple(vx.shape) == tuple(_val(add).shape)
                and order[other] < order[node]  # already computed where the kernel runs
            ):
                kwargs["dx_add"] = other
                target = add
        # What reads the fp32 sum next is `_to_copy(bf16) -> view [rows, C] -> {mm, t -> mm, sum([0])}`, the
        # gradient GEMMs and the bias gradient of the layer before: the bf16 tensor leaves the same
        # launch. (The kernel can also emit that tensor's column sums, the bias gradient; the extra
        # shared-memory accumulator made the launch 21 us slower at [8192, 1600] where the separate
        # column-sum kernel over the L2-resident bf16 tensor takes 10 us, so the sum stays a node.)
        total = target if target is not None else dx
        cast = None
        if total is not None and kwargs:
            casts = [u for u in total.users if _plain_cast(u) == torch.bfloat16 and u.args[0] is total]
            if len(casts) == 1 and _static_tensor(casts[0]) and tuple(_val(casts[0]).shape) == tuple(vx.shape):
                cast = casts[0]
        if not kwargs:
            continue
        if cast is not None:
            kwargs["want_cast"] = True
        with graph.inserting_after(node):
            new = graph.call_function(af.fused_layer_norm_backward, args=(grad,) + tuple(node.args[1:]), kwargs=kwargs)
        new.meta = dict(node.meta)
        node.replace_all_uses_with(new)
        if target is not None:
            target.replace_all_uses_with(dx)
        if cast is not None:
            old_val = _val(node)
            new.meta["val"] = tuple(old_val) + (_val(cast), None)
            with graph.inserting_after(dx):
                narrow = graph.call_function(operator.getitem, args=(new, 3))
            narrow.meta = dict(cast.meta)
            cast.replace_all_uses_with(narrow)
        count += 1
    return count


def _fuse_gemm_epilogues(graph) -> int:
    count = 0
    for node in list(graph.nodes):
        if _is_call(node, aten.addmm.default):
            bias, a, b = node.args[:3]
            alpha, beta = node.kwargs.get("alpha", 1), node.kwargs.get("beta", 1)
        elif _is_call(node, aten.mm.default):
            a, b = node.args[:2]
            bias, alpha, beta = None, 1, 1
        else:
            continue
        va, vb = _val(a), _val(b)
        if not (_static_tensor(node) and isinstance(va, torch.Tensor) and isinstance(vb, torch.Tensor)):
            continue
        if va.dtype != vb.dtype or not native.supported_dtype(va.dtype):
            continue
        if bias is not None and not native.supported_dtype(_val(bias).dtype):
            continue
        if not isinstance(alpha, (int, float)) or not isinstance(beta, (int, float)):
            continue

        epilogue, out_dtype, residual = native.EPILOGUE_NONE, None, None
        cur = _skip_views(node)
        user = _only_user(cur)
        if _is_call(user, aten.gelu.default) and user.args[0] is cur:
            approximate = user.kwargs.get("approximate", "none")
            epilogue = native.EPILOGUE_GELU_TANH if approximate == "tanh" else native.EPILOGUE_GELU_ERF
            cur = _skip_views(user)
            user = _only_user(cur)
        if _plain_cast(user) == torch.float32 and user.args[0] is cur and _static_tensor(user):
            out_dtype = torch.float32
            cur = _skip_views(user)
            user = _only_user(cur)
        if (
            _is_call(user, aten.add.Tensor)
            and user.kwargs.get("alpha", 1) == 1
            and len(user.args) == 2
            and all(isinstance(x, torch.fx.Node) for x in user.args)
            and _static_tensor(user)
        ):
            other = user.args[1] if user.args[0] is cur else user.args[0]
            vo, vc = _val(other), _val(cur)
            if (
                other is not cur
                and isinstance(vo, torch.Tensor)
                and tuple(vo.shape) == tuple(vc.shape) == tuple(_val(user).shape)
                and native.supported_dtype(vo.dtype)
                and _val(user).dtype == (out_dtype or va.dtype)
            ):
                residual = other
                cur = user
        if epilogue == native.EPILOGUE_NONE and out_dtype is None and residual is None:
            continue
        out_val = _val(cur)
        _replace(
            graph, cur, af.fused_gemm, (a, b, bias, residual),
            {"alpha": float(alpha), "beta": float(beta), "epilogue": epilogue,
             "out_dtype": out_val.dtype, "out_shape": [int(d) for d in out_val.shape]},
        )
        count += 1
    return count


def _alias_root(node):
    while _is_call(node, *ALIAS_OPS):
        node = node.args[0]
    return node


def _drop_attention_output_copies(graph) -> int:
    count = 0
    for node in list(graph.nodes):
        if not _is_call(node, aten.clone.default):
            continue
        if node.kwargs.get("memory_format") not in (None, torch.contiguous_format):
            continue
        root = _alias_root(node.args[0])
        if not _is_call(root, *SDPA_OPS):
            continue
        # a fresh kernel output that nothing mutates: an alias is indistinguishable from a copy
        _replace(graph, node, af.contiguous_or_alias, (node.args[0],), {})
        count += 1
    return count


def _constant_fill(node):
    """Python float of a `where` fill operand built in the graph as a constant, else None."""
    if isinstance(node, (int, float)):
        return float(node)
    if _is_call(node, aten.scalar_tensor.default) and isinstance(node.args[0], (int, float)):
        return float(node.args[0])
    if _is_call(node, aten.full.default) and list(node.args[0]) == [] and isinstance(node.args[1], (int, float)):
        return float(node.args[1])
    return None


def _fuse_masked_softmax(graph) -> int:
    from torch_mojo_backend import ops

    count = 0
    for node in list(graph.nodes):
        if not _is_call(node, aten._softmax.default) or not _static_tensor(node):
            continue
        src, dim, half_to_float = node.args[:3]
        v = _val(node)
        if half_to_float or dim not in (-1, v.dim() - 1) or not native.supported_dtype(v.dtype):
            continue
        if not isinstance(src, torch.fx.Node) or len(src.users) != 1:
            continue
        if _is_call(src, aten.masked_fill.Scalar):
            x, mask, fill = src.args
            invert = False
        elif _is_call(src, aten.where.self):
            mask, x, fill = src.args
            fill = _constant_fill(fill)
            invert = True
        else:
            continue
        if not isinstance(fill, (int, float)) or not isinstance(x, torch.fx.Node):
            continue
        vx, vm = _val(x), _val(mask)
        if not (isinstance(vx, torch.Tensor) and isinstance(vm, torch.Tensor) and vx.dtype == v.dtype):
            continue
        if tuple(vx.shape) != tuple(v.shape) or ops.mask_rows_of(vx, vm) is None:
            continue
        scale = 1.0
        if len(x.users) == 1 and _is_call(x, aten.mul.Tensor, aten.div.Tensor) and _static_tensor(x):
            inner, factor = x.args
            vi = _val(inner)
            if (
                isinstance(factor, (int, float))
                and isinstance(vi, torch.Tensor)
                and vi.dtype == vx.dtype
                and tuple(vi.shape) == tuple(vx.shape)
                and (x.target is aten.mul.Tensor or factor != 0)
            ):
                scale = float(factor) if x.target is aten.mul.Tensor else 1.0 / float(factor)
                x = inner
        _replace(graph, node, af.fused_masked_softmax, (x, mask),
                 {"fill": float(fill), "scale": scale, "invert": invert})
        count += 1
    return count


def _embedding_operand(node):
    """(table, indices, cast dtype or None) when `node` is `embedding(table, indices)` or a plain
    dtype cast of one, each link with a single user; else None."""
    dtype = None
    cast = _plain_cast(node)
    if cast is not None:
        if len(node.users) != 1:
            return None
        dtype = cast
        node = node.args[0]
    if not _is_call(node, aten.embedding.default) or len(node.users) != 1 or not _static_tensor(node):
        return None
    table, indices = node.args[:2]
    vt, vi = _val(table), _val(indices)
    if not (isinstance(vt, torch.Tensor) and isinstance(vi, torch.Tensor)) or vt.dim() != 2:
        return None
    if not native.supported_dtype(vt.dtype) or vi.dtype not in (torch.int64, torch.int32):
        return None
    return table, indices, dtype


def _fuse_embedding_sum(graph) -> int:
    """`embedding(wte, idx)[.to(dt)] + embedding(wpe, pos)[.to(dt)]`, pos broadcasting over idx from
    the right (the token + positional embeddings of a GPT-style model; reference contract:
    aten_embedding, torch_mojo_backend/aten_functions.py:1779-1831, followed by aten_add)."""
    count = 0
    for node in list(graph.nodes):
        if not (_is_call(node, aten.add.Tensor) and node.kwargs.get("alpha", 1) == 1 and len(node.args) == 2):
            continue
        if not all(isinstance(x, torch.fx.Node) for x in node.args) or not _static_tensor(node):
            continue
        lhs, rhs = _embedding_operand(node.args[0]), _embedding_operand(node.args[1])
        if lhs is None or rhs is None or node.args[0] is node.args[1]:
            continue
        # the operand whose indices carry the full shape goes first
        if _val(lhs[1]).dim() < _val(rhs[1]).dim():
            lhs, rhs = rhs, lhs
        (t1, i1, d1), (t2, i2, d2) = lhs, rhs
        v1, v2, vt1, vt2, vo = _val(i1), _val(i2), _val(t1), _val(t2), _val(node)
        if d1 != d2 or vt1.dtype != vt2.dtype or vt1.shape[1] != vt2.shape[1]:
            continue
        out_dtype = d1 or vt1.dtype
        if vo.dtype != out_dtype or not native.supported_dtype(out_dtype):
            continue
        if vt1.dtype == torch.float32 and out_dtype != torch.float32:
            continue
        if v2.dim() > v1.dim() or tuple(v1.shape[v1.dim() - v2.dim():]) != tuple(v2.shape) or v2.numel() == 0:
            continue
        if tuple(vo.shape) != (*v1.shape, vt1.shape[1]):
            continue
        _replace(graph, node, af.fused_embedding_sum, (t1, i1, t2, i2), {"out_dtype": out_dtype})
        count += 1
    return count


def fuse_graph(gm: torch.fx.GraphModule) -> dict[str, int]:
    """Rewrites gm.graph in place and returns how many chains of each kind were folded."""
    graph = gm.graph
    stats = {
        "layer_norm_cast": _fuse_layer_norm(graph) + _fuse_layer_norm_with_statistics(graph),
        "layer_norm_backward": _fuse_layer_norm_backward(graph),
        "gemm_epilogue": _fuse_gemm_epilogues(graph),
        "attention_output_copy": _drop_attention_output_copies(graph),
        "masked_softmax": _fuse_masked_softmax(graph),
        "embedding_sum": _fuse_embedding_sum(graph),
    }
    if any(stats.values()):
        graph.eliminate_dead_code()
        graph.lint()
        gm.recompile()
    return stats
