"""One CUDA graph per forward call of a module whose step is a long chain of small launches.

The diffusion token stack is about 500 launches of a few microseconds each per step: issued one by one the GPU waits
for the host between them. ``GraphedModule`` captures one forward call (all kernels, on every stream the module uses)
into a ``torch.cuda.CUDAGraph`` and replays it; inputs are copied into the buffers the graph was captured with, so they
may be device tensors or pinned host tensors (the copy is then the upload). Shapes, dtypes and which arguments are
``None`` are fixed at capture time.
"""

from __future__ import annotations

import torch


class GraphedModule:
    """``GraphedModule(fn, *example_args, warmup=2)(*args) -> the outputs of fn``, replayed from a CUDA graph.

    ``fn`` must be a pure function of its tensor arguments and of state that does not change between calls (module
    parameters; for ``DiffusionTransformer`` with ``hoist_pair_bias`` also the pair tensor: the projections captured
    in the graph are those of the pair tensor seen at capture time). The returned tensors are the graph's own output
    buffers: they are overwritten by the next call.
    """

    def __init__(self, fn, *example_args, warmup: int = 2):
        self._static_in = [None if a is None else a.detach().clone() for a in example_args]
        if not all(a is None or a.is_cuda for a in self._static_in):
            raise ValueError("GraphedModule needs CUDA example arguments")
        dev = next(a.device for a in self._static_in if a is not None)
        cur = torch.cuda.current_stream(dev)
        side = torch.cuda.Stream(dev)
        side.wait_stream(cur)
        with torch.no_grad(), torch.cuda.stream(side):
            for _ in range(max(1, warmup)):   # workspaces, packed weights and caches exist before the capture
                fn(*self._static_in)
        cur.wait_stream(side)
        torch.cuda.synchronize(dev)
        self.graph = torch.cuda.CUDAGraph()
        with torch.no_grad(), torch.cuda.graph(self.graph):
            self._static_out = fn(*self._static_in)

    def __call__(self, *args):
        if len(args) != len(self._static_in):
            raise ValueError(f"expected {len(self._static_in)} arguments, got {len(args)}")
        for dst, src in zip(self._static_in, args):
            if (dst is None) != (src is None):
                raise ValueError("an argument that was None at capture time must stay None, and the reverse")
            if dst is not None and src is not dst:
                if src.shape != dst.shape or src.dtype != dst.dtype:
                    raise ValueError(f"argument of shape {tuple(src.shape)} / {src.dtype}: the graph was captured with "
                                     f"{tuple(dst.shape)} / {dst.dtype}")
                dst.copy_(src, non_blocking=True)
        self.graph.replay()
        return self._static_out
