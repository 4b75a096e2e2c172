"""CUDA-graph runner for the stand-alone backbone.

A VMamba forward is about 120 kernel launches of 5 to 300 microseconds; replaying them from one captured
graph removes the per-launch host cost (the reference's own throughput loop, classification/main.py:350-363,
pays it on every step).  `GraphedBackbone` captures one forward of a fixed batch shape with static input and
output buffers and offers three calls:

    runner = GraphedBackbone(model, (128, 3, 224, 224))
    runner.replay()                      # input already in runner.input (device); result in runner.output
    logits = runner(device_images)       # copies into the static input, replays, returns runner.output
    runner.infer_host(pinned_images, pinned_logits)    # host -> device -> forward -> host, asynchronous

`infer_host` uploads on a stream of its own into one of two staging buffers, so the upload of one call
overlaps the forward of the previous one; the caller synchronises (stream or `runner.done` event) before
reading `pinned_logits`.
"""
from __future__ import annotations

from typing import Callable, Optional, Sequence

import torch

from . import _lib


class GraphedBackbone:
    def __init__(self, model, batch_shape: Sequence[int], *, features: bool = False,
                 out_indices: Sequence[int] = (0, 1, 2, 3), dtype: Optional[torch.dtype] = None,
                 device: Optional[torch.device] = None, warmup: int = 2):
        if not torch.cuda.is_available():
            raise RuntimeError("GraphedBackbone needs a CUDA device (there is no CPU path)")
        self.model = model
        self.device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.dtype = dtype or getattr(model, "dtype", torch.bfloat16)
        fn: Callable = (lambda x: model.features(x, out_indices)) if features else model
        with torch.cuda.device(self.device):
            self.input = torch.zeros(tuple(batch_shape), device=self.device, dtype=self.dtype)
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):            # warm-up outside capture: lazy initialisation, allocator pools
                for _ in range(max(1, warmup)):
                    fn(self.input)
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            self.graph = torch.cuda.CUDAGraph()
            l0 = _lib.launch_count()
            with torch.cuda.graph(self.graph):
                self.output = fn(self.input)
            self.launches_per_forward = _lib.launch_count() - l0      # kernels of this library in one forward
            self._copy_stream = torch.cuda.Stream()
            self._staging = [torch.empty_like(self.input) for _ in range(2)]
            self._h2d_done = [torch.cuda.Event() for _ in range(2)]
            self._consumed = [torch.cuda.Event() for _ in range(2)]
            self.done = torch.cuda.Event()
            self._calls = 0

    def replay(self):
        """One forward on whatever `self.input` holds; the result is `self.output` (static buffers)."""
        self.graph.replay()
        return self.output

    def __call__(self, images: torch.Tensor):
        if images.shape != self.input.shape:
            raise RuntimeError(f"captured for batch shape {tuple(self.input.shape)}, got {tuple(images.shape)}")
        self.input.copy_(images, non_blocking=True)
        return self.replay()

    def fence_uploads(self):
        """No upload of a later `infer_host` call starts before the work queued so far on the current stream."""
        self._copy_stream.wait_stream(torch.cuda.current_stream())

    def infer_host(self, host_images: torch.Tensor, host_out=None):
        """Pinned host batch in, pinned host result out (a tensor, or a list of tensors for `features=True`).
        Everything is queued asynchronously; `self.done` is recorded behind the last copy."""
        if host_images.shape != self.input.shape:
            raise RuntimeError(f"captured for batch shape {tuple(self.input.shape)}, got {tuple(host_images.shape)}")
        k = self._calls & 1
        self._calls += 1
        cur = torch.cuda.current_stream()
        self._copy_stream.wait_event(self._consumed[k])           # staging[k] has been read by its previous call
        with torch.cuda.stream(self._copy_stream):
            self._staging[k].copy_(host_images, non_blocking=True)
            self._h2d_done[k].record(self._copy_stream)
        cur.wait_event(self._h2d_done[k])
        self.input.copy_(self._staging[k], non_blocking=True)
        self._consumed[k].record(cur)
        self.graph.replay()
        outs = self.output if isinstance(self.output, (list, tuple)) else [self.output]
        if host_out is None:
            host_out = [torch.empty(o.shape, dtype=o.dtype).pin_memory() for o in outs]
        hosts = host_out if isinstance(host_out, (list, tuple)) else [host_out]
        for h, o in zip(hosts, outs):
            h.copy_(o, non_blocking=True)
        self.done.record(cur)
        return host_out if isinstance(self.output, (list, tuple)) else hosts[0]
