"""Host orchestration of prefill and per-token steps over the ring cache.

Mirror of the reference ``Generator._prefill`` / ``Generator._step`` (inference/generate.py:220-248) for a
stack of attention layers: prefill fills the ring layer by layer from inside the projection kernel (the rows
``bulk_write_packed`` would write, no copy pass); each step hands every
layer the ring itself (no per-layer chronological ``view`` copy, no separate ``write``) and advances once.
Sampling, embeddings and the MLPs are outside this path; the runner works on hidden states.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch

from .attention import B200CausalSelfAttention, WindowMask
from .kv_cache import B200KVCache


class StepRunner:
    def __init__(self, layers: Sequence[B200CausalSelfAttention], window: int, cache_capacity: Optional[int] = None,
                 batch: int = 1, device="cuda", dtype=torch.bfloat16):
        assert len(layers) > 0
        self.layers = list(layers)
        self.window = int(window)
        a = self.layers[0]
        cap = int(cache_capacity if cache_capacity is not None else window)
        self.cache = B200KVCache(L=len(self.layers), B=batch, H=a.num_heads, W=cap, D=a.head_dim, device=device, dtype=dtype)

    def reset_history(self):
        self.cache.reset_history()
        for a in self.layers:
            a.reset_history()

    @torch.inference_mode()
    def _prefill(self, x: torch.Tensor) -> torch.Tensor:
        """``x [B,T,dim]`` through every layer's ``prefill`` (each layer sees the previous layer's output),
        the cache receives the rows ``Generator._prefill`` stores through ``bulk_write_packed``."""
        T = x.size(1)
        for i, a in enumerate(self.layers):
            # the projection's epilogue stores the rows bulk_write_packed keeps straight into their ring slots
            x, _, _ = a.prefill_ring(x, None, self.cache, i, attn_mask=WindowMask(self.window))
        self.cache.set_position(T)
        return x

    # ------------------------------------------------------------------ CUDA-graph step
    @torch.inference_mode()
    def capture_step(self, batch: int, dim: int) -> None:
        """Record one token step of all layers into a CUDA graph.  The position lives in ``cache.t_dev`` and is
        advanced inside the graph, the input and output are fixed buffers: ``_step_graph`` then costs one copy
        and one graph launch per token instead of four launches per layer issued from Python."""
        dev = self.cache.device
        self._gx = torch.zeros(batch, 1, dim, device=dev, dtype=torch.bfloat16)
        t_saved = self.cache.t_dev.clone()
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):                              # warm-up outside the capture (lazy initialisation);
            self._graph_body(write_ring=False)                     # it must not store its dummy row into the ring
        torch.cuda.current_stream(dev).wait_stream(side)
        self.cache.t_dev.copy_(t_saved)                            # the warm-up advanced the device counter
        self._graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self._graph):
            self._gy = self._graph_body()
        self.cache.t_dev.copy_(t_saved)

    def _graph_body(self, write_ring: bool = True) -> torch.Tensor:
        x = self._gx
        for i, a in enumerate(self.layers):
            x = a.step_ring_dev(x, self.cache, i, self.window, write_ring=write_ring)
        self.cache.t_dev += 1
        return x

    @torch.inference_mode()
    def _step_graph(self, x: torch.Tensor) -> torch.Tensor:
        """``_step`` through the captured graph.  Neither the warm-up run (made without the ring store) nor the
        capture itself (which executes nothing) has touched the ring, so a capture is safe at any position, also
        with a window larger than the ring, where the slot of the next token is the oldest row still attended."""
        self._gx.copy_(x)
        self._graph.replay()
        self.cache.t += 1                                          # host mirror; the device counter moved in the graph
        return self._gy

    @torch.inference_mode()
    def _step(self, x: torch.Tensor) -> torch.Tensor:
        """One token ``x [B,1,dim]``: every layer reads the ring in place and stores its new row; one advance."""
        pos = self.cache.t
        for i, a in enumerate(self.layers):
            x, _, _ = a.step_ring(x, self.cache, i, pos, None, self.window)
        self.cache.advance()
        return x
