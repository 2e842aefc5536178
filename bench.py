"""Benchmark of the hot path: GPT-2 XL forward (bf16 operands, fp32 accumulation) through
torch.compile(backend=mojo_backend), batch-sharded over N GPUs of one box.

  python bench.py [--gpus N] [--steps K] [--warmup W]            # this backend
  python bench.py --impl reference [--gpus N] [--steps K] ...    # CPU baseline arm (host cores)

Workload: 48 layers, d_model 1600, 25 heads, MLP 6400, ctx 1024, vocab 50257, tied head, weights
N(0, 0.02) from seed 0, token ids uniform in [0, 50257); global batch 64 x 1024 split evenly over
the ranks (strong scaling), weights replicated, no collective on the data path. One step = one
forward over the rank's shard (one forward call per --micro-batch sequences, by default the whole
shard at once). Synthetic data stands in for the HF prompts the reference's own benchmarks use.

  python bench.py --model small --precision fp32 --batch 1 --seq 128   # the CPU-runnable configuration

Prints one JSON line (rank 0). `value` is whole-job tokens/s with token ids resident in HBM,
timed with CUDA events, max over ranks. `e2e` is the same forward through the public API with
the ids in pinned host memory: H2D of the ids, the forward, the arg-max over the logits (this
library's kernel) and D2H of the step's result (the top-1 token id per position) are inside the
timed region. `roofline` is the GEMM kernel's achieved TFLOP/s
(algorithmic 2*M*N*K over CUDA-event time of every GEMM launch of one instrumented step)
against the measured bf16 peak. `cpu_baseline` is the same model on the host cores (PyTorch CPU
eager, the reference's own oracle) on a bounded sample.
"""

from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
for _p in (ROOT, ROOT / "torch-max-backend_b200"):
    if str(_p) not in sys.path:
        sys.path.insert(0, str(_p))

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

GLOBAL_BATCH = 64
SEQ_LEN = 1024
# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the GEMM with the largest time share
# (MLP down-projection, 8192 x 6400 x 1600 + fp32 residual, algorithmic 229 MB), from an ncu capture
NCU_DRAM_BYTES_MLP_DOWN = 252.54e6 + 38.88e6
MICRO_BATCH = 64  # sequences per forward call: the rank's whole shard when it has no more than this
VOCAB = 50257


def parse_args():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=5)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--impl", choices=["b200", "reference"], default="b200")
    p.add_argument("--model", choices=["xl", "small"], default="xl")
    p.add_argument("--precision", choices=["bf16", "fp32"], default="bf16",
                   help="bf16: bf16 GEMM/attention operands, fp32 accumulation, residual stream and logits; fp32: all fp32")
    p.add_argument("--batch", type=int, default=GLOBAL_BATCH, help="global batch (sequences), split over the ranks")
    p.add_argument("--seq", type=int, default=SEQ_LEN, help="tokens per sequence")
    p.add_argument("--cpu-sample-tokens", type=int, default=1024)
    p.add_argument("--no-cpu-baseline", action="store_true")
    p.add_argument("--micro-batch", type=int, default=MICRO_BATCH, help="sequences per forward call")
    return p.parse_args()


def measured_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        d = json.loads(path.read_text())
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"],
                "bf16_tflops_sustained": d.get("bf16_tflops_sustained", d["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML while the timed region runs.
    Read-only: nothing about the GPU is changed."""

    REASONS = {
        0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap",
    }

    def __init__(self, index: int):
        self.samples, self.reasons = [], set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self._nvml = pynvml
            self._handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._handle, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._nvml = None

    def _loop(self):
        n = self._nvml
        while not self._stop.is_set():
            try:
                self.samples.append(n.nvmlDeviceGetClockInfo(self._handle, n.NVML_CLOCK_SM))
                mask = n.nvmlDeviceGetCurrentClocksThrottleReasons(self._handle)
                for bit, name in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(0.1)

    def __enter__(self):
        if self._nvml is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2] if s else None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(s)}


def physical_gpu_index(local_rank: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local_rank])
        except (ValueError, IndexError):
            pass
    return local_rank


def build_model(name: str):
    from demo_scripts.gpt2 import GPT2, GPTConfig

    cfg = GPTConfig.xl() if name == "xl" else GPTConfig.small()
    return GPT2(cfg).init_weights(0).eval(), cfg


def cpu_forward_tokens_per_s(model, cfg, sample_tokens: int, reps: int, warmup: int = 1, seq_len: int = SEQ_LEN):
    """PyTorch CPU eager (fp32 math on the bf16-rounded weights), all host threads."""
    import copy

    ref = copy.deepcopy(model).to("cpu").set_precision("fp32").eval()
    seq = min(sample_tokens, seq_len)
    nseq = max(1, sample_tokens // seq)
    ids = torch.randint(0, cfg.vocab_size, (nseq, seq), generator=torch.Generator().manual_seed(1))
    times = []
    with torch.no_grad():
        for i in range(warmup + reps):
            t0 = time.perf_counter()
            ref(ids)
            dt_ = time.perf_counter() - t0
            if i >= warmup:
                times.append(dt_)
    per_step = sum(times) / len(times)
    return nseq * seq / per_step, per_step, f"{nseq} x {seq} tokens per step, mean of {reps} steps after {warmup} warm-up"


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    # torchrun exports OMP_NUM_THREADS=1; the CPU arm uses every host thread it is allowed to
    torch.set_num_threads(len(os.sched_getaffinity(0)))
    model, cfg = build_model(args.model)
    model.set_precision(args.precision)
    cores = torch.get_num_threads()
    tps, per_step, sample = cpu_forward_tokens_per_s(model, cfg, args.cpu_sample_tokens, args.steps,
                                                     min(args.warmup, 1), args.seq)
    line = {
        "impl": "reference",
        "metric": f"gpt2_{args.model}_forward_tokens_per_s", "value": tps, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": min(args.warmup, 1), "ms_per_step": per_step * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"gpt2-{args.model} forward, PyTorch CPU eager on host cores, {sample}",
                   "global_batch": args.batch, "seq_len": args.seq},
        "cpu_baseline": {"value": tps, "unit": "tokens/s", "cores": cores, "host_cpus": os.cpu_count(),
                         "kind": "port", "sample": sample},
        "e2e": {"value": tps, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "the reference's MAX CPU execution cannot be installed offline; PyTorch CPU eager, the "
                "oracle the reference's tests pin this path to, is what runs",
    }
    print(json.dumps(line), flush=True)


def main():
    args = parse_args()
    if args.impl == "reference":
        run_reference(args)
        return

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the b200 kernels have no CPU fallback")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    # Every micro-batch launches the same ~340 kernels with the same shapes: replay them from a
    # CUDA graph (the backend's own switch; export TORCH_MOJO_BACKEND_CUDA_GRAPHS=0 for the eager plan).
    os.environ.setdefault("TORCH_MOJO_BACKEND_CUDA_GRAPHS", "1")
    if world > 1:
        dist.init_process_group("nccl", device_id=device)

    import torch_mojo_backend
    from demo_scripts.gpt2 import flops_per_token
    from torch_mojo_backend import native
    from torch_mojo_backend.sharding import aggregate_throughput, shard_range

    native.lib()  # fail now, loudly, if the kernels are missing

    model, cfg = build_model(args.model)
    model.set_precision(args.precision)
    cpu_model = model if (rank == 0 and world == 1 and not args.no_cpu_baseline) else None
    if cpu_model is not None:
        import copy

        cpu_model = copy.deepcopy(model)
    model = model.to(device)
    compiled = torch.compile(model, backend=torch_mojo_backend.mojo_backend)

    global_batch, seq_len = args.batch, args.seq
    start, end = shard_range(global_batch, rank, world)
    my_seqs = end - start
    all_ids = torch.randint(0, cfg.vocab_size, (global_batch, seq_len), generator=torch.Generator().manual_seed(0))
    ids_host = all_ids[start:end].contiguous().pin_memory()
    ids_dev = ids_host.to(device)
    micro = [(i, min(i + args.micro_batch, my_seqs)) for i in range(0, my_seqs, args.micro_batch)]

    def step_resident():
        out = None
        for lo, hi in micro:
            out = compiled(ids_dev[lo:hi])
        return out

    top1_host = torch.empty((my_seqs, seq_len), dtype=torch.int64).pin_memory()

    def step_e2e():
        for lo, hi in micro:
            x = ids_host[lo:hi].to(device, non_blocking=True)
            logits = compiled(x)
            # top-1 token ids with this library's arg-max kernel (no vendor kernel in the timed region)
            top1_host[lo:hi].copy_(torch.ops.b200.argmax(logits), non_blocking=True)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(step_fn, steps):
        barrier()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        launches_before = native.launch_count
        t0.record()
        for _ in range(steps):
            step_fn()
        t1.record()
        torch.cuda.synchronize()
        elapsed = t0.elapsed_time(t1)
        barrier()
        return elapsed, native.launch_count - launches_before

    with torch.no_grad():
        for _ in range(max(args.warmup, 3)):
            step_resident()
        with ClockSampler(physical_gpu_index(local_rank)) as clocks:
            elapsed_ms, launches = timed(step_resident, args.steps)
        for _ in range(2):
            step_e2e()
        e2e_ms, _ = timed(step_e2e, args.steps)

        # one instrumented step: CUDA events around every kernel launch of this library (the eager
        # plan: inside a replayed CUDA graph there is nothing to bracket)
        graphs_flag = os.environ.get("TORCH_MOJO_BACKEND_CUDA_GRAPHS")
        os.environ["TORCH_MOJO_BACKEND_CUDA_GRAPHS"] = "0"
        native.profiler = native.KernelProfiler()
        step_resident()
        prof = native.profiler.summary()
        native.profiler = None
        if graphs_flag is None:
            os.environ.pop("TORCH_MOJO_BACKEND_CUDA_GRAPHS", None)
        else:
            os.environ["TORCH_MOJO_BACKEND_CUDA_GRAPHS"] = graphs_flag

    tokens = float(my_seqs * seq_len * args.steps)
    agg = aggregate_throughput(tokens, elapsed_ms, device)
    agg_e2e = aggregate_throughput(tokens, e2e_ms, device)
    launch_total = aggregate_throughput(float(launches), 0.0, device)["units"]
    status = native.device_status()

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peaks = measured_peaks()
    value = agg["units"] / (agg["ms"] / 1e3)
    gemm = prof.get("gemm", {"launches": 0, "ms": 0.0, "flops": 0.0})
    achieved = gemm["flops"] / (gemm["ms"] / 1e3) / 1e12 if gemm["ms"] > 0 else 0.0
    peak = peaks["bf16_tflops_sustained"]
    roofline = {
        "bound": "tensor", "kernel": "gemm_tcgen05_kernel", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
        "frac": achieved / peak,
        # measured DRAM bytes of one launch of the MLP down-projection GEMM (captured at 8192 rows per
        # launch; operand, residual and output bytes all grow with the row count, so the figure is
        # scaled to the rows one launch of this run processes)
        "traffic": NCU_DRAM_BYTES_MLP_DOWN * (min(args.micro_batch, my_seqs) * seq_len / 8192.0)
        if args.model == "xl" and args.precision == "bf16" else None,
        "traffic_unit": "bytes per launch (ncu capture of the MLP down-projection GEMM at 8192 rows, scaled by rows)",
        "peak_source": f"{peaks['source']} (sustained cuBLAS bf16)",
        "launches_timed": gemm["launches"],
        "per_op_ms": {k: round(v["ms"], 3) for k, v in prof.items()},
    }
    line = {
        "metric": "gpt2_xl_forward_tokens_per_s" if args.model == "xl" else "gpt2_small_forward_tokens_per_s",
        "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": agg["ms"] / args.steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "bf16" if args.precision == "bf16" else "f32", "data": "synthetic",
        "config": {"workload": f"gpt2-{args.model} forward, {args.precision}, global batch {global_batch} x {seq_len} "
                               f"batch-sharded, {min(args.micro_batch, my_seqs)} sequences per forward call",
                   "global_batch": global_batch, "seq_len": seq_len, "parallelism": f"batch-shard x{world}, no collective",
                   "l2": "inputs larger than L2 (weights 3 GB, activations 52 MB per tensor)" if args.model == "xl"
                         else "weights (0.5 GB in fp32) larger than L2",
                   "launch": "CUDA-graph replay of the launch plan"
                             if os.environ.get("TORCH_MOJO_BACKEND_CUDA_GRAPHS", "0") == "1" else "eager launch plan"},
        "tflops_per_gpu": value / world * flops_per_token(cfg, seq_len) / 1e12,
        "clocks": clocks.summary(),
        "e2e": {"value": agg_e2e["units"] / (agg_e2e["ms"] / 1e3), "unit": "tokens/s",
                "h2d_bytes_per_step": my_seqs * seq_len * 8, "d2h_bytes_per_step": my_seqs * seq_len * 8,
                "result": "top-1 token id per position (int64, this library's arg-max kernel over the fp32 "
                          "logits), read back to pinned host memory"},
        "gpu_launches": int(launch_total),
        "roofline": roofline,
        "device_status": status,
    }
    if cpu_model is not None:
        torch.set_num_threads(len(os.sched_getaffinity(0)))
        tps, per_step, sample = cpu_forward_tokens_per_s(cpu_model, cfg, args.cpu_sample_tokens, reps=2, seq_len=seq_len)
        line["cpu_baseline"] = {"value": tps, "unit": "tokens/s", "cores": torch.get_num_threads(),
                                "host_cpus": os.cpu_count(), "kind": "port", "sample": sample}
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
