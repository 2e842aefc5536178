"""Generates tests/golden/ops_golden.npz from PyTorch CPU eager -- the implementation the
reference's own tests pin this path to (torch_mojo_backend/testing.py:139-229). The reference
package cannot be imported here (it needs Modular MAX), so its oracle is what produces the vectors.

Run from the repository root:  python tests/golden/make_golden.py
bf16 tensors are stored widened to float32 (exact); the `*_dtype` entries say what they were.
"""

import sys
from pathlib import Path

import numpy as np
import torch
import torch.nn.functional as F

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT / "torch-max-backend_b200"))

from demo_scripts.gpt2 import GPT2, GPTConfig  # noqa: E402


def f32(t):
    return t.detach().to(torch.float32).numpy()


def main():
    torch.manual_seed(0)
    g = torch.Generator().manual_seed(1234)
    out = {}

    # native_layer_norm, the shapes of tests/test_aten_functions.py:380-445 in spirit: affine,
    # none-affine, two normalised dims.
    x = torch.randn(6, 40, generator=g)
    w = torch.randn(40, generator=g)
    b = torch.randn(40, generator=g)
    y, mean, rstd = torch.ops.aten.native_layer_norm(x, [40], w, b, 1e-5)
    out.update(ln_x=f32(x), ln_w=f32(w), ln_b=f32(b), ln_y=f32(y), ln_mean=f32(mean), ln_rstd=f32(rstd))
    x2 = torch.randn(3, 4, 10, generator=g)
    y2, mean2, rstd2 = torch.ops.aten.native_layer_norm(x2, [4, 10], None, None, 1e-3)
    out.update(ln2_x=f32(x2), ln2_y=f32(y2), ln2_mean=f32(mean2), ln2_rstd=f32(rstd2))

    # softmax over every dim (tests/test_high_level_ops.py:3883-3920) and the causal-masked form
    s = torch.randn(3, 5, 7, generator=g)
    for d in range(3):
        out[f"sm_y{d}"] = f32(torch.softmax(s, d))
    out["sm_x"] = f32(s)
    scores = torch.randn(2, 8, 8, generator=g)
    mask = torch.tril(torch.ones(8, 8, dtype=torch.bool))
    out["csm_x"] = f32(scores)
    out["csm_y"] = f32(torch.softmax((scores * 0.25).masked_fill(~mask, float("-inf")), -1))

    # gelu none / tanh (tests/test_high_level_ops.py:3859-3880), fp32 and bf16
    gx = torch.randn(257, generator=g) * 3
    out["gelu_x"] = f32(gx)
    out["gelu_none"] = f32(F.gelu(gx))
    out["gelu_tanh"] = f32(F.gelu(gx, approximate="tanh"))
    gxb = gx.to(torch.bfloat16)
    out["gelu_bf16_x"] = f32(gxb)
    out["gelu_bf16_none"] = f32(F.gelu(gxb))
    out["gelu_bf16_tanh"] = f32(F.gelu(gxb, approximate="tanh"))

    # sum / mean / amax
    r = torch.randn(4, 6, 9, generator=g)
    out["red_x"] = f32(r)
    out["red_sum_last"] = f32(r.sum(-1))
    out["red_mean_01"] = f32(r.mean((0, 1)))
    out["red_amax_1k"] = f32(r.amax(1, keepdim=True))
    out["red_sum_all"] = f32(r.sum())

    # addmm with alpha/beta and 1-D bias (tests/test_high_level_ops.py:4307-4352), bmm (:4355-4393),
    # and the odd-shape case m,n,k = 33,65,31 (tests/test_eager_kernels.py:5196-5244)
    bias = torch.randn(65, generator=g)
    m1 = torch.randn(33, 31, generator=g)
    m2 = torch.randn(31, 65, generator=g)
    out.update(mm_bias=f32(bias), mm_a=f32(m1), mm_b=f32(m2))
    out["mm_y"] = f32(m1 @ m2)
    out["addmm_y"] = f32(torch.addmm(bias, m1, m2, beta=0.5, alpha=2.0))
    ba = torch.randn(3, 5, 7, generator=g)
    bb = torch.randn(3, 7, 4, generator=g)
    out.update(bmm_a=f32(ba), bmm_b=f32(bb), bmm_y=f32(torch.bmm(ba, bb)))

    # causal and full SDPA, kv_len in the reference's set {6, 10, 64} (tests/test_eager_kernels.py:5606-5619)
    for kv in (6, 10, 64):
        q = torch.randn(2, 3, kv, 16, generator=g)
        k = torch.randn(2, 3, kv, 16, generator=g)
        v = torch.randn(2, 3, kv, 16, generator=g)
        out[f"sdpa{kv}_q"], out[f"sdpa{kv}_k"], out[f"sdpa{kv}_v"] = f32(q), f32(k), f32(v)
        out[f"sdpa{kv}_causal"] = f32(F.scaled_dot_product_attention(q, k, v, is_causal=True))
        out[f"sdpa{kv}_full"] = f32(F.scaled_dot_product_attention(q, k, v))

    # a tiny GPT-2 (2 layers, width 64, 4 heads) from seed 0: logits for 2 x 16 token ids
    cfg = GPTConfig(vocab_size=211, block_size=32, n_layer=2, n_head=4, n_embd=64)
    ids = torch.randint(0, cfg.vocab_size, (2, 16), generator=torch.Generator().manual_seed(0))
    out["gpt_ids"] = ids.numpy()
    for attention in ("sdpa", "masked_softmax"):
        model = GPT2(cfg, attention).init_weights(0).eval()
        with torch.no_grad():
            out[f"gpt_logits_{attention}"] = f32(model(ids))

    path = Path(__file__).with_name("ops_golden.npz")
    np.savez_compressed(path, **out)
    print(f"wrote {path} ({path.stat().st_size} bytes, {len(out)} arrays)")


if __name__ == "__main__":
    main()
