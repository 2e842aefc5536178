"""CUDA-graph replay of a launch plan (TORCH_MOJO_BACKEND_CUDA_GRAPHS=1).

A plan over static shapes launches the same kernels with the same arguments on every call, so
after one eager warm-up call it is captured into a CUDA graph and later calls replay it: one
graph launch instead of hundreds of kernel launches, which is what bounds small-batch forwards.

Tensor arguments whose address is the same on every call (parameters) are read in place;
arguments whose address changed between the first two calls are copied into buffers owned by the
runner before each replay. Outputs live in the graph's memory pool and are overwritten by the
next replay (the usual CUDA-graph contract); callers that keep results across calls must clone.
Any change of shape, dtype, device or of a non-tensor argument falls back to eager replay of the
plan and re-captures.
"""

from __future__ import annotations

import torch

from torch_mojo_backend import native


def _signature(args):
    sig = []
    for a in args:
        if isinstance(a, torch.Tensor):
            sig.append((tuple(a.shape), a.dtype, a.device, tuple(a.stride())))
        else:
            sig.append(a)
    return tuple(sig)


class GraphRunner:
    def __init__(self, plan):
        self.plan = plan
        self._sig = None
        self._first_ptrs = None
        self._graph = None
        self._static_args = None
        self._copy_idx = ()
        self._pinned_ptrs = {}
        self._outputs = None
        self._kernels = 0  # kernels of this library inside the captured graph
        self.replays = 0
        self._eager_only = False

    def _reset(self):
        self._eager_only = False
        self._graph = None
        self._static_args = None
        self._outputs = None
        self._first_ptrs = None

    def run(self, args):
        args = list(args)
        sig = _signature(args)
        ptrs = [a.data_ptr() if isinstance(a, torch.Tensor) else None for a in args]
        if sig != self._sig or not all(isinstance(a, torch.Tensor) and a.is_cuda or not isinstance(a, torch.Tensor) for a in args):
            self._sig = sig
            self._reset()
        if self._eager_only:
            return self.plan.run(args)
        if self._graph is None:
            if self._first_ptrs is None:
                # first call with this signature: eager warm-up, remember addresses
                self._first_ptrs = ptrs
                return self.plan.run(args)
            if not self._try_capture(args, ptrs):
                return self.plan.run(args)
        else:
            for i, p in self._pinned_ptrs.items():
                if ptrs[i] != p:
                    # an argument assumed static moved: capture again with it as a copied input
                    self._first_ptrs = [None if j == i else q for j, q in enumerate(self._first_ptrs)]
                    self._graph = None
                    if not self._try_capture(args, ptrs):
                        return self.plan.run(args)
                    break
        for i in self._copy_idx:
            self._static_args[i].copy_(args[i], non_blocking=True)
        self._graph.replay()
        self.replays += 1
        native.launch_count += self._kernels  # the replay launched them; the op wrappers did not run
        return self._outputs

    def _try_capture(self, args, ptrs) -> bool:
        """Captures the plan; a plan that cannot be captured (an op that synchronises, e.g.
        `_local_scalar_dense`, `nonzero`, boolean-mask indexing) is latched to the eager launch plan
        for this signature instead of failing on every call."""
        try:
            self._capture(args, ptrs)
            return True
        except Exception as e:  # noqa: BLE001 -- whatever the capture raised, the eager plan still works
            import warnings

            self._graph = None
            self._eager_only = True
            torch.cuda.synchronize()
            warnings.warn(f"CUDA-graph capture of the launch plan failed ({type(e).__name__}: {e}); "
                          "running this signature eagerly", RuntimeWarning, stacklevel=3)
            return False

    def _capture(self, args, ptrs):
        self._copy_idx = tuple(
            i for i, a in enumerate(args) if isinstance(a, torch.Tensor) and ptrs[i] != self._first_ptrs[i]
        )
        self._static_args = list(args)
        for i in self._copy_idx:
            self._static_args[i] = args[i].clone()
        self._pinned_ptrs = {
            i: ptrs[i] for i, a in enumerate(args) if isinstance(a, torch.Tensor) and i not in self._copy_idx
        }
        device = next(a.device for a in args if isinstance(a, torch.Tensor))
        stream = torch.cuda.Stream(device)
        stream.wait_stream(torch.cuda.current_stream(device))
        with torch.cuda.stream(stream):
            self.plan.run(self._static_args)  # warm-up on the side stream (allocator, attributes)
        torch.cuda.current_stream(device).wait_stream(stream)
        graph = torch.cuda.CUDAGraph()
        before = native.launch_count
        with torch.cuda.graph(graph):
            self._outputs = self.plan.run(self._static_args)
        # recorded, not launched: they count once per replay instead
        self._kernels = native.launch_count - before
        native.launch_count = before
        self._graph = graph
