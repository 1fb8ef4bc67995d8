"""Host orchestration of prefill and per-token steps over the ring cache.

Mirror of the reference ``Generator._prefill`` / ``Generator._step`` (inference/generate.py:220-248) for a
stack of attention layers: prefill fills the ring through ``bulk_write_packed``; each step hands every
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
        then the cache is filled from the stacked k,v exactly as ``Generator._prefill`` does."""
        T = x.size(1)
        ks: List[torch.Tensor] = []
        vs: List[torch.Tensor] = []
        for a in self.layers:
            x, k, v = a.prefill(x, None, attn_mask=WindowMask(self.window))
            ks.append(k); vs.append(v)
        self.cache.bulk_write_packed(torch.stack([torch.stack(ks), torch.stack(vs)]), T)
        return x

    @torch.inference_mode()
    def _step(self, x: torch.Tensor) -> torch.Tensor:
        """One token ``x [B,1,dim]``: every layer reads the ring in place and stores its new row; one advance."""
        pos = self.cache.t
        for i, a in enumerate(self.layers):
            x, _, _ = a.step_ring(x, self.cache, i, pos, None, self.window)
        self.cache.advance()
        return x
