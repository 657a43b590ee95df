"""Replays a fixed-shape inference forward as one CUDA graph.

A forward pass of the network is a few hundred short kernels (the fused convolution-fit layers, the ReLU fixed point,
normalisations, packing); launched one by one they leave the GPU idle between launches. All kernels of this library
run on the stream they are given, allocate through torch's caching allocator and never synchronise, so the whole pass
can be captured once and replayed with a single launch.
"""
import torch


class GraphedForward:
    """graph = GraphedForward(fn, example_input); out = graph(x) for x of the example's shape, dtype and device.

    `fn` must be free of host synchronisation (no .item(), no data-dependent Python control flow) and is run under
    torch.no_grad(). The returned tensor is the graph's static output buffer: it is overwritten by the next call.
    Whatever `fn` derives from parameters on the Python side and caches (the kernel mixtures of the convolution
    layers) is frozen into the graph: capture again after changing parameters."""

    def __init__(self, fn, example_input: torch.Tensor, warmup: int = 3):
        if not example_input.is_cuda:
            raise ValueError("GraphedForward needs a CUDA tensor")
        self._fn = fn
        self._static_in = example_input.clone()
        side = torch.cuda.Stream(device=example_input.device)
        side.wait_stream(torch.cuda.current_stream(example_input.device))
        with torch.cuda.stream(side), torch.no_grad():
            for _ in range(max(1, warmup)):       # lazy initialisation (function attributes, allocator pools)
                fn(self._static_in)
        torch.cuda.current_stream(example_input.device).wait_stream(side)
        self._graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self._graph), torch.no_grad():
            self._static_out = fn(self._static_in)

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        if x.shape != self._static_in.shape or x.dtype != self._static_in.dtype or x.device != self._static_in.device:
            raise ValueError("input does not match the captured shape / dtype / device")
        self._static_in.copy_(x, non_blocking=True)
        self._graph.replay()
        return self._static_out
