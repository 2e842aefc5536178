"""Per-kernel timings for the GEMM sweep, the row ops and causal attention at the benchmark
shapes, each reported against its roofline (measured HBM copy bandwidth / measured bf16 peak).

  python torch-max-backend_b200/bench_kernels.py [--ops gemm,layer_norm,...] [--iters 50] [--quick]
  python torch-max-backend_b200/bench_kernels.py --ops gemm --only "8192x768x2304" --iters 3 --no-graph   # for ncu

Method (the reference's own protocol, bench_gemm.py:152-169, plus L2 hygiene): inputs rotate over
enough copies to exceed twice the 126 MB L2, so every launch reads cold data; `iters` launches
are captured in one CUDA graph and the replay is timed with CUDA events, so that microsecond
kernels are not hidden behind Python launch overhead; at least 5 warm-up replays. Algorithmic
work per launch: GEMM 2*M*N*K flops and s*(M*K + K*N + M*N + N) bytes (bench_gemm.py:239-240),
row ops numel*size*(reads + writes), causal SDPA 4*B*H*T^2*d/2 flops.
One JSON line per case on stdout.
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent
for _p in (ROOT, ROOT.parent):
    if str(_p) not in sys.path:
        sys.path.insert(0, str(_p))

import torch  # noqa: E402

L2_BYTES = 126 * 1024 * 1024


def peaks():
    path = ROOT.parent / "MEASURED_PEAKS.json"
    if path.exists():
        d = json.loads(path.read_text())
        return d["hbm_gbs"], d["bf16_tflops"], "measured"
    return 6650.0, 1590.0, "fallback"


def rotations(bytes_per_copy: float) -> int:
    return int(max(2, min(64, -(-2 * L2_BYTES // max(1, int(bytes_per_copy))))))


def time_case(make_inputs, run, bytes_per_copy, iters, use_graph):
    """make_inputs(i) -> inputs of copy i; run(inputs) launches the kernel once."""
    r = rotations(bytes_per_copy)
    copies = [make_inputs(i) for i in range(r)]
    for i in range(5):
        run(copies[i % r])
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if use_graph:
        graph = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            run(copies[0])
        torch.cuda.current_stream().wait_stream(side)
        with torch.cuda.graph(graph):
            for i in range(iters):
                run(copies[i % r])
        for _ in range(5):
            graph.replay()
        torch.cuda.synchronize()
        reps = 3
        start.record()
        for _ in range(reps):
            graph.replay()
        end.record()
        torch.cuda.synchronize()
        return start.elapsed_time(end) * 1e3 / (iters * reps), r
    start.record()
    for i in range(iters):
        run(copies[i % r])
    end.record()
    torch.cuda.synchronize()
    return start.elapsed_time(end) * 1e3 / iters, r


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ops", default="gemm,gemm_fused,gemm_fp32_routes,layer_norm,softmax,gelu,reduce,embedding,argmax,sdpa,sdpa_decode,backward")
    ap.add_argument("--iters", type=int, default=40)
    ap.add_argument("--only", default="", help="substring filter on the case name")
    ap.add_argument("--no-graph", action="store_true", help="plain launches (what an ncu capture wants)")
    ap.add_argument("--quick", action="store_true", help="skip the largest GEMM (N=50257 at M=8192)")
    args = ap.parse_args()

    from torch_mojo_backend import native, ops

    native.lib()
    dev = torch.device("cuda")
    hbm, tf, src = peaks()
    wanted = set(args.ops.split(","))
    gen = torch.Generator(device="cuda").manual_seed(0)

    def randn(shape, dtype, std=1.0, mean=0.0):
        return (torch.randn(shape, generator=gen, device=dev, dtype=torch.float32) * std + mean).to(dtype)

    def report(name, us, rot, flops=0.0, nbytes=0.0, bound="hbm"):
        line = {"case": name, "us": round(us, 3), "rotating_copies": rot, "bound": bound}
        if flops:
            line["tflops"] = round(flops / us / 1e6, 2)
        if nbytes:
            line["gbs"] = round(nbytes / us / 1e3, 1)
        if bound == "tensor":
            line["frac"] = round(flops / us / 1e6 / tf, 4)
            line["peak"] = f"{tf} TFLOP/s bf16 burst, {src}"
        else:
            line["frac"] = round(nbytes / us / 1e3 / hbm, 4)
            line["peak"] = f"{hbm} GB/s copy, {src}"
        print(json.dumps(line), flush=True)

    def keep(name):
        return args.only in name

    use_graph = not args.no_graph

    if "gemm" in wanted:
        kn = [(768, 2304), (768, 768), (768, 3072), (3072, 768), (1600, 4800), (1600, 6400), (6400, 1600)]
        if not args.quick:
            kn += [(768, 50257), (1600, 50257)]
        for dtype, dname in ((torch.bfloat16, "bf16"), (torch.float32, "fp32")):
            for m in (8192, 64, 16, 1):
                for k, n in kn:
                    if dtype == torch.float32 and (n > 6400 or k > 3072) and m == 8192:
                        continue
                    for layout in ("nk", "kn"):
                        name = f"gemm {dname} {m}x{k}x{n} B={layout} +bias"
                        if not keep(name):
                            continue
                        s = 2 if dtype == torch.bfloat16 else 4
                        nbytes = s * (m * k + k * n + m * n + n)

                        def make(i, m=m, k=k, n=n, layout=layout, dtype=dtype):
                            a = randn((m, k), dtype)
                            b = randn((n, k), dtype).t() if layout == "nk" else randn((k, n), dtype)
                            return a, b, randn((n,), dtype, 0.02)

                        us, rot = time_case(make, lambda t: ops.gemm(t[0], t[1], t[2]), nbytes, args.iters, use_graph)
                        bound = "tensor" if m >= 512 else "hbm"
                        report(name, us, rot, 2.0 * m * n * k, nbytes, bound)

    if "gemm_fp32_routes" in wanted:
        # fp32 operands: the exact CUDA-core route against the default (split precision on the tensor
        # cores: operands as bf16 hi / lo halves, three products accumulated in fp32 by one launch).
        for m, k, n in ((8192, 768, 2304), (8192, 1600, 6400)):
            for label, route in (("exact", 1), ("split", 4)):
                name = f"gemm_fp32_routes {label} {m}x{k}x{n} B=nk +bias"
                if not keep(name):
                    continue
                nbytes = 4 * (m * k + k * n + m * n + n)

                def make(i, m=m, k=k, n=n):
                    return randn((m, k), torch.float32), randn((n, k), torch.float32, 0.05).t(), randn((n,), torch.float32, 0.02)

                us, rot = time_case(make, lambda t, route=route: ops.gemm(t[0], t[1], t[2], None, 1.0, 1.0, 0, None, route),
                                    nbytes, max(4, args.iters // 4), use_graph)
                report(name, us, rot, 2.0 * m * n * k, nbytes, "tensor")

    if "gemm_fused" in wanted:
        # The GEMMs of one GPT-2 XL block (and the LM head) as the fused graph launches them.
        m, d = 8192, 1600
        bf, f32 = torch.bfloat16, torch.float32
        cases = [
            ("xl qkv  bias", d, 3 * d, False, 0, bf),
            ("xl proj bias+residual f32", d, d, True, 0, f32),
            ("xl fc   bias+gelu_tanh", d, 4 * d, False, 1, bf),
            ("xl out  bias+residual f32", 4 * d, d, True, 0, f32),
            ("xl lm_head f32 logits", d, 50257, False, 0, f32),
        ]
        for label, k, n, with_res, epi, out_dtype in cases:
            name = f"gemm_fused {label} {m}x{k}x{n}"
            if not keep(name):
                continue
            out_s = 4 if out_dtype == f32 else 2
            nbytes = 2 * (m * k + k * n) + out_s * m * n + (4 * m * n if with_res else 0)

            def make(i, k=k, n=n, with_res=with_res, label=label):
                a = randn((m, k), bf)
                w = randn((n, k), bf, 0.02).t()
                bias = None if "lm_head" in label else randn((n,), bf, 0.02)
                res = randn((m, n), f32) if with_res else None
                return a, w, bias, res

            us, rot = time_case(make, lambda t, epi=epi, out_dtype=out_dtype: ops.gemm(t[0], t[1], t[2], t[3], 1.0, 1.0, epi, out_dtype),
                                nbytes, args.iters, use_graph)
            report(name, us, rot, 2.0 * m * n * k, nbytes, "tensor")

    if "layer_norm" in wanted:
        for dtype, dname in ((torch.bfloat16, "bf16"), (torch.float32, "fp32")):
            for rows, cols in ((8192, 768), (8192, 1600), (65536, 1600)):
                name = f"layer_norm {dname} {rows}x{cols}"
                if not keep(name):
                    continue
                s = 2 if dtype == torch.bfloat16 else 4
                nbytes = 2 * rows * cols * s + 8 * rows
                make = lambda i, rows=rows, cols=cols, dtype=dtype: (randn((rows, cols), dtype), randn((cols,), dtype, 0.02, 1.0), randn((cols,), dtype, 0.02))
                us, rot = time_case(make, lambda t: ops.layer_norm(t[0], t[1], t[2], 1e-5), nbytes, args.iters, use_graph)
                report(name, us, rot, nbytes=nbytes)

        # the variant the fused GPT-2 graph launches: fp32 residual stream in, bf16 GEMM operand out
        for rows, cols in ((8192, 1600), (65536, 1600)):
            name = f"layer_norm fp32->bf16 {rows}x{cols}"
            if keep(name):
                nbytes = rows * cols * (4 + 2) + 8 * rows
                make = lambda i, rows=rows, cols=cols: (randn((rows, cols), torch.float32), randn((cols,), torch.float32, 0.02, 1.0), randn((cols,), torch.float32, 0.02))
                us, rot = time_case(make, lambda t: ops.layer_norm(t[0], t[1], t[2], 1e-5, torch.bfloat16), nbytes, args.iters, use_graph)
                report(name, us, rot, nbytes=nbytes)

    if "softmax" in wanted:
        for dtype, dname in ((torch.bfloat16, "bf16"), (torch.float32, "fp32")):
            shape = (96, 1024, 1024)
            s = 2 if dtype == torch.bfloat16 else 4
            nbytes = 2 * 96 * 1024 * 1024 * s
            mask = torch.ones(1024, 1024, dtype=torch.bool, device=dev).tril()
            name = f"softmax {dname} 96x1024x1024 pre-masked(-inf)"
            if keep(name):
                make = lambda i, dtype=dtype: (randn(shape, dtype).masked_fill_(~mask, float("-inf")),)
                us, rot = time_case(make, lambda t: ops.softmax(t[0]), nbytes, args.iters, use_graph)
                report(name, us, rot, nbytes=nbytes)
            name = f"softmax {dname} 96x1024x1024 fused scale+causal"
            if keep(name):
                make = lambda i, dtype=dtype: (randn(shape, dtype),)
                us, rot = time_case(make, lambda t: ops.softmax(t[0], 0.125, True, 1024), nbytes, args.iters, use_graph)
                # masked columns are never read: algorithmic bytes = half the reads + all the writes
                report(name, us, rot, nbytes=0.75 * nbytes)

            name = f"softmax {dname} 96x1024x1024 fused scale+explicit mask"
            if keep(name):
                make = lambda i, dtype=dtype: (randn(shape, dtype),)
                blocked = ~mask
                us, rot = time_case(make, lambda t: ops.softmax_masked(t[0], blocked, float("-inf"), 0.125, False),
                                    nbytes + 1024 * 1024, args.iters, use_graph)
                # every score is read (the mask's values are not known to be triangular) + the 1 MB mask
                report(name, us, rot, nbytes=nbytes + 1024 * 1024)

    if "gelu" in wanted:
        for dtype, dname in ((torch.bfloat16, "bf16"), (torch.float32, "fp32")):
            for approx in ("tanh", "none"):
                name = f"gelu {dname} {approx} 8192x3072"
                if not keep(name):
                    continue
                s = 2 if dtype == torch.bfloat16 else 4
                nbytes = 2 * 8192 * 3072 * s
                make = lambda i, dtype=dtype: (randn((8192, 3072), dtype),)
                us, rot = time_case(make, lambda t, approx=approx: ops.gelu(t[0], approx), nbytes, args.iters, use_graph)
                report(name, us, rot, nbytes=nbytes)

    if "reduce" in wanted:
        # [8192,768] is one hidden-state matrix of the small configuration (12 - 25 MB: a 4 - 6 us kernel,
        # launch ramp included); [65536,1600] is the benchmark's, large enough to show the sustained rate.
        for R, C in ((8192, 768), (65536, 1600)):
            for dtype, dname in ((torch.bfloat16, "bf16"), (torch.float32, "fp32")):
                for op, oname in ((0, "sum"), (1, "mean"), (2, "amax")):
                    name = f"reduce {oname} {dname} {R}x{C}"
                    if not keep(name):
                        continue
                    s = 2 if dtype == torch.bfloat16 else 4
                    nbytes = R * C * s
                    make = lambda i, dtype=dtype, R=R, C=C: (randn((R, C), dtype),)
                    us, rot = time_case(make, lambda t, op=op: ops.reduce(t[0], op), nbytes, args.iters, use_graph)
                    report(name, us, rot, nbytes=nbytes)

    if "backward" in wanted:
        # The backward kernels on the shapes of a GPT-2 XL training step over 8 x 1024 tokens
        # (and LayerNorm / bias sums also on the benchmark's 64 x 1024).
        bf, f32 = torch.bfloat16, torch.float32
        for approx in ("tanh", "none"):
            name = f"gelu_backward bf16 {approx} 8192x6400"
            if keep(name):
                nbytes = 3 * 8192 * 6400 * 2
                make = lambda i: (randn((8192, 6400), bf), randn((8192, 6400), bf))
                us, rot = time_case(make, lambda t, approx=approx: ops.gelu_backward(t[0], t[1], approx), nbytes, args.iters, use_graph)
                report(name, us, rot, nbytes=nbytes)
        name = "gelu_backward fp32 tanh 8192x3072"
        if keep(name):
            nbytes = 3 * 8192 * 3072 * 4
            make = lambda i: (randn((8192, 3072), f32), randn((8192, 3072), f32))
            us, rot = time_case(make, lambda t: ops.gelu_backward(t[0], t[1], "tanh"), nbytes, args.iters, use_graph)
            report(name, us, rot, nbytes=nbytes)
        for dtype, dname in ((bf, "bf16"), (f32, "fp32")):
            name = f"softmax_backward {dname} 96x1024x1024"
            if keep(name):
                s_ = 2 if dtype == bf else 4
                nbytes = 3 * 96 * 1024 * 1024 * s_
                make = lambda i, dtype=dtype: (randn((96, 1024, 1024), dtype), torch.softmax(randn((96, 1024, 1024), f32), -1).to(dtype))
                us, rot = time_case(make, lambda t: ops.softmax_backward(t[0], t[1], 0.125), nbytes, args.iters, use_graph)
                report(name, us, rot, nbytes=nbytes)
        for rows in (8192, 65536):
            # x fp32 (residual stream), dy bf16 (gradient of the GEMM operand), dx bf16
            name = f"layer_norm_backward x fp32, dy bf16 {rows}x1600"
            if keep(name):
                nbytes = rows * 1600 * (4 + 2 + 2) + 8 * rows
                make = lambda i, rows=rows: (randn((rows, 1600), bf), randn((rows, 1600), f32), randn((rows,), f32),
                                             randn((rows,), f32).abs() + 0.5, randn((1600,), f32, 0.02, 1.0))
                us, rot = time_case(make, lambda t: ops.layer_norm_backward(t[0], t[1], t[2], t[3], t[4]), nbytes, args.iters, use_graph)
                report(name, us, rot, nbytes=nbytes)
            # the training graph's form: bf16 dy widened in the kernel, fp32 dx with the residual gradient added
            name = f"layer_norm_backward x fp32, dy bf16, dx fp32 + residual gradient {rows}x1600"
            if keep(name):
                nbytes = rows * 1600 * (4 + 2 + 4 + 4) + 8 * rows
                make = lambda i, rows=rows: (randn((rows, 1600), bf), randn((rows, 1600), f32), randn((rows,), f32),
                                             randn((rows,), f32).abs() + 0.5, randn((1600,), f32, 0.02, 1.0),
                                             randn((rows, 1600), f32))
                us, rot = time_case(make, lambda t: ops.layer_norm_backward(t[0], t[1], t[2], t[3], t[4], True, True, t[5], f32),
                                    nbytes, args.iters, use_graph)
                report(name, us, rot, nbytes=nbytes)
            # ... and with the bf16 copy of dx and its column sums (the next projection's operand and bias gradient)
            name = f"layer_norm_backward x fp32, dy bf16, dx fp32 + residual gradient + bf16 copy + sums {rows}x1600"
            if keep(name):
                nbytes = rows * 1600 * (4 + 2 + 4 + 4 + 2) + 8 * rows
                make = lambda i, rows=rows: (randn((rows, 1600), bf), randn((rows, 1600), f32), randn((rows,), f32),
                                             randn((rows,), f32).abs() + 0.5, randn((1600,), f32, 0.02, 1.0),
                                             randn((rows, 1600), f32))
                us, rot = time_case(make, lambda t: ops.layer_norm_backward_with_copy(t[0], t[1], t[2], t[3], t[4], True, True,
                                                                                     t[5], f32, True, bf),
                                    nbytes, args.iters, use_graph)
                report(name, us, rot, nbytes=nbytes)
            name = f"layer_norm_backward x fp32, dy bf16, dx fp32 + residual gradient + bf16 copy {rows}x1600"
            if keep(name):
                nbytes = rows * 1600 * (4 + 2 + 4 + 4 + 2) + 8 * rows
                make = lambda i, rows=rows: (randn((rows, 1600), bf), randn((rows, 1600), f32), randn((rows,), f32),
                                             randn((rows,), f32).abs() + 0.5, randn((1600,), f32, 0.02, 1.0),
                                             randn((rows, 1600), f32))
                us, rot = time_case(make, lambda t: ops.layer_norm_backward_with_copy(t[0], t[1], t[2], t[3], t[4], True, True,
                                                                                     t[5], f32, True, None),
                                    nbytes, args.iters, use_graph)
                report(name, us, rot, nbytes=nbytes)
            name = f"layer_norm_backward fp32 {rows}x1600"
            if keep(name):
                nbytes = rows * 1600 * 12 + 8 * rows
                make = lambda i, rows=rows: (randn((rows, 1600), f32), randn((rows, 1600), f32), randn((rows,), f32),
                                             randn((rows,), f32).abs() + 0.5, randn((1600,), f32, 0.02, 1.0))
                us, rot = time_case(make, lambda t: ops.layer_norm_backward(t[0], t[1], t[2], t[3], t[4]), nbytes, args.iters, use_graph)
                report(name, us, rot, nbytes=nbytes)
        for rows, cols in ((8192, 6400), (65536, 1600)):
            name = f"sum_rows bf16 {rows}x{cols}"
            if keep(name):
                nbytes = rows * cols * 2
                make = lambda i, rows=rows, cols=cols: (randn((rows, cols), bf),)
                us, rot = time_case(make, lambda t: ops.sum_rows(t[0], f32), nbytes, args.iters, use_graph)
                report(name, us, rot, nbytes=nbytes)
        for B, H, T in ((8, 25, 1024), (64, 25, 1024)):
            name = f"sdpa_backward bf16 causal {B}x{H}x{T}x64"
            if keep(name):
                flops = 10.0 * B * H * T * T * 64 * 0.5
                nbytes = 8 * B * H * T * 64 * 2  # q, k, v, o, dO read; dq, dk, dv written

                def make(i, B=B, H=H, T=T):
                    qkv = randn((B, T, 3 * H * 64), bf)
                    q, k, v = (t.view(B, T, H, 64).transpose(1, 2) for t in qkv.split(H * 64, dim=2))
                    o, lse = ops.sdpa(q, k, v, True)
                    return randn((B, T, H, 64), bf).transpose(1, 2), q, k, v, o, lse

                us, rot = time_case(make, lambda t: ops.sdpa_backward(t[0], t[1], t[2], t[3], t[4], t[5], True), nbytes, args.iters, use_graph)
                report(name, us, rot, flops, nbytes, "tensor")
        # weight gradients dW = X^T dY (A stored transposed, K = tokens) and data gradients dX = dY W
        m_tok, d = 8192, 1600
        for label, kin, nout in (("fc", d, 4 * d), ("out", 4 * d, d)):
            name = f"gemm wgrad xl {label} {kin}x{nout}x{m_tok} (A transposed)"
            if keep(name):
                nbytes = 2 * (m_tok * kin + m_tok * nout) + 4 * kin * nout
                make = lambda i, kin=kin, nout=nout: (randn((m_tok, kin), bf), randn((m_tok, nout), bf))
                us, rot = time_case(make, lambda t: ops.gemm(t[0].t(), t[1], None, None, 1.0, 1.0, 0, f32), nbytes, args.iters, use_graph)
                report(name, us, rot, 2.0 * m_tok * kin * nout, nbytes, "tensor")
            name = f"gemm dgrad xl {label} {m_tok}x{nout}x{kin}"
            if keep(name):
                nbytes = 2 * (m_tok * nout + kin * nout + m_tok * kin)
                make = lambda i, kin=kin, nout=nout: (randn((m_tok, nout), bf), randn((nout, kin), bf, 0.02))
                us, rot = time_case(make, lambda t: ops.gemm(t[0], t[1]), nbytes, args.iters, use_graph)
                report(name, us, rot, 2.0 * m_tok * kin * nout, nbytes, "tensor")

    if "embedding" in wanted:
        # token + positional embeddings of a GPT-2 XL batch: bf16 tables, fp32 residual stream out
        for B, T, C in ((8, 1024, 1600), (64, 1024, 1600)):
            name = f"embedding_sum bf16->fp32 {B}x{T}x{C}"
            if not keep(name):
                continue
            nbytes = B * T * C * (2 + 2 + 4)
            wte, wpe = randn((50257, C), torch.bfloat16, 0.02), randn((1024, C), torch.bfloat16, 0.02)
            pos = torch.arange(T, device=dev)
            make = lambda i, B=B, T=T: (torch.randint(0, 50257, (B, T), device=dev, generator=gen),)
            us, rot = time_case(make, lambda t: ops.embedding_sum(wte, t[0], wpe, pos, torch.float32), nbytes, args.iters, use_graph)
            report(name, us, rot, nbytes=nbytes)

    if "argmax" in wanted:
        # top-1 over the fp32 logits (50257 columns, padded pitch) of 8 and 64 sequences
        for rows in (8192, 65536):
            name = f"argmax fp32 {rows}x50257"
            if not keep(name):
                continue
            nbytes = rows * 50257 * 4
            reps = 1 if rows > 8192 else 2
            make = lambda i, rows=rows: (randn((rows, 50264), torch.float32)[:, :50257],)
            if rows > 8192:
                one = make(0)
                make = lambda i, one=one: one  # 13 GB: one copy, far larger than L2
            us, rot = time_case(make, lambda t: ops.argmax(t[0]), nbytes, max(3, args.iters // 4), use_graph)
            report(name, us, rot, nbytes=nbytes)

    if "sdpa" in wanted:
        for B, H, T, D in ((8, 12, 1024, 64), (4, 25, 2048, 64), (8, 25, 1024, 64), (16, 25, 1024, 64), (64, 25, 1024, 64)):
            name = f"sdpa bf16 causal {B}x{H}x{T}x{D}"
            if not keep(name):
                continue
            nbytes = 4 * B * H * T * D * 2
            flops = 4.0 * B * H * T * T * D / 2

            def make(i, B=B, H=H, T=T, D=D):
                qkv = randn((B, T, 3 * H * D), torch.bfloat16)
                return tuple(t.view(B, T, H, D).transpose(1, 2) for t in qkv.split(H * D, dim=2))

            us, rot = time_case(make, lambda t: ops.sdpa(t[0], t[1], t[2], True), nbytes, args.iters, use_graph)
            report(name, us, rot, flops, nbytes, "tensor")

    if "sdpa_decode" in wanted:
        # One new token against a KV cache: K and V are read once, so the bound is HBM.
        for B, H, T, D in ((8, 25, 1024, 64), (64, 25, 1024, 64), (8, 25, 8192, 64), (32, 32, 4096, 128)):
            name = f"sdpa_decode bf16 {B}x{H}x1x{T}x{D}"
            if not keep(name):
                continue
            nbytes = 2 * B * H * T * D * 2 + 2 * B * H * D * 2

            def make(i, B=B, H=H, T=T, D=D):
                return (randn((B, H, 1, D), torch.bfloat16), randn((B, H, T, D), torch.bfloat16), randn((B, H, T, D), torch.bfloat16))

            us, rot = time_case(make, lambda t: ops.sdpa(t[0], t[1], t[2], False), nbytes, args.iters, use_graph)
            report(name, us, rot, nbytes=nbytes)

    status = native.device_status()
    if status != 0:
        raise SystemExit(f"a kernel reported a bounded-wait timeout (status word {status:#x})")


if __name__ == "__main__":
    main()
