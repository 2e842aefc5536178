"""Forward + backward of GPT-2 through `torch.compile(backend=mojo_backend)` on one GPU: tokens/s of a
training step without the optimizer, and where its time goes.

  python torch-max-backend_b200/bench_training.py [--model xl|small] [--batch 8] [--seq 1024] [--steps 5]

Prints one JSON line: tokens/s (CUDA events around `steps` steps after `warmup`), and the per-op share
of one further step timed with CUDA events around every launch of the library (`ops`) -- time outside
the library's kernels (the elementwise glue of the loss, dtype casts, gradient accumulation) is the
difference to the step time. Synthetic ids and targets, seeded random weights.
"""

from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.nn.functional as F

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", choices=["xl", "small"], default="xl")
    ap.add_argument("--precision", choices=["bf16", "fp32"], default="bf16")
    ap.add_argument("--attention", choices=["sdpa", "masked_softmax"], default="sdpa")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--seq", type=int, default=1024)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--by-shape", action="store_true", help="break the GEMM time of the profiled step down by shape")
    args = ap.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("bench_training.py needs a CUDA device: the b200 kernels have no CPU fallback")

    import torch_mojo_backend
    from demo_scripts.gpt2 import GPT2, GPTConfig, flops_per_token
    from torch_mojo_backend import native

    native.lib()
    cfg = GPTConfig.xl() if args.model == "xl" else GPTConfig.small()
    model = GPT2(cfg, args.attention).init_weights(0).train().cuda().set_precision(args.precision)
    compiled = torch.compile(model, backend=torch_mojo_backend.mojo_backend)
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(0, cfg.vocab_size, (args.batch, args.seq), generator=g).cuda()
    targets = torch.randint(0, cfg.vocab_size, (args.batch, args.seq), generator=g).cuda()

    def step():
        model.zero_grad(set_to_none=True)
        loss = F.cross_entropy(compiled(ids).reshape(-1, cfg.vocab_size).float(), targets.reshape(-1))
        loss.backward()
        return loss

    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    before = native.launch_count
    t0.record()
    for _ in range(args.steps):
        loss = step()
    t1.record()
    torch.cuda.synchronize()
    ms = t0.elapsed_time(t1) / args.steps
    launches = (native.launch_count - before) // args.steps

    native.profiler = native.KernelProfiler()
    native.profiler.by_shape = args.by_shape
    step()
    per_op = native.profiler.summary()
    native.profiler = None
    tokens = args.batch * args.seq
    print(json.dumps({
        "metric": "gpt2_forward_backward_tokens_per_s", "value": tokens / (ms * 1e-3), "unit": "tokens/s",
        "ms_per_step": ms, "config": {"model": args.model, "precision": args.precision, "attention": args.attention,
                                      "batch": args.batch, "seq_len": args.seq, "optimizer": "none"},
        "tflops": 3 * flops_per_token(cfg, args.seq) * tokens / (ms * 1e-3) / 1e12,
        "library_launches_per_step": launches, "loss": float(loss),
        "ops": {k: {"launches": v["launches"], "ms": round(v["ms"], 3)} for k, v in sorted(per_op.items(), key=lambda kv: -kv[1]["ms"])},
        "device_status": native.device_status(),
    }))


if __name__ == "__main__":
    main()
