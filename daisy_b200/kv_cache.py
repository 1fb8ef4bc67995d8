"""Ring-buffer sliding-window KV cache on the GPU.

Same constructor, attributes and six methods as the reference ``KVCache``
(inference/kv_cache.py:4-68): storage ``k, v [L, B, H, W, D]``, token ``p`` of the sequence
lives in row ``p % W``, ``t`` counts committed tokens.  ``view`` / ``write`` /
``bulk_write_packed`` keep the reference's shapes and ordering; in addition ``ring(layer)``
hands the in-place ring to the decode kernel so the per-token chronological copy that
``view`` makes once the ring has wrapped is never needed on the hot path.
"""
from __future__ import annotations

import torch

from . import ops


def ring_segment(t: int, staged: bool, W: int):
    """Host-side index arithmetic of ``view`` (inference/kv_cache.py:27-35): returns ``(first_pos, n)``
    -- the n = min(t + staged, W) most recent tokens start at sequence position ``first_pos``."""
    m = t + (1 if staged else 0)
    n = min(m, W)
    return m - n, n


class B200KVCache:
    def __init__(self, L, B, H, W, D, device, dtype=torch.bfloat16):
        dev = torch.device(device)
        if dev.type != "cuda":
            raise ValueError("B200KVCache lives in GPU memory; daisy_b200 has no CPU path")
        self.L, self.B, self.H, self.W, self.D = L, B, H, W, D
        self.device, self.dtype = dev, dtype
        self.reset_history()

    def reset_history(self):
        shape = (self.L, self.B, self.H, self.W, self.D)
        self.k = torch.zeros(shape, device=self.device, dtype=self.dtype)
        self.v = torch.zeros(shape, device=self.device, dtype=self.dtype)
        self.t = 0
        # the same counter in device memory, for decode launches that must not depend on host values
        # (CUDA-graph replays); kept in step with `t` by stream-ordered updates, never read back
        self.t_dev = torch.zeros(1, device=self.device, dtype=torch.int64)
        self._staged = [False] * self.L

    # ------------------------------------------------------------------ reference API
    def view(self, layer):
        """Chronological ``(k, v)`` as ``[B, n, H, D]`` (inference/kv_cache.py:26-42).  A view of the
        ring when the rows are contiguous, otherwise a gathered copy."""
        first, n = ring_segment(self.t, self._staged[layer], self.W)
        if n == 0:
            return self.k[layer, :, :, :0].transpose(1, 2), self.v[layer, :, :, :0].transpose(1, 2)
        start = first % self.W
        if start + n <= self.W:
            return (self.k[layer, :, :, start:start + n].transpose(1, 2),
                    self.v[layer, :, :, start:start + n].transpose(1, 2))
        k = torch.empty(self.B, self.H, n, self.D, device=self.device, dtype=self.dtype)
        v = torch.empty_like(k)
        ops.ring_copy_rows(self.k[layer], k, first, to_ring=False)
        ops.ring_copy_rows(self.v[layer], v, first, to_ring=False)
        return k.transpose(1, 2), v.transpose(1, 2)

    def write(self, layer, k_new, v_new):
        """Stage the new token's row at slot ``t % W`` (inference/kv_cache.py:44-51); accepts
        ``[B,1,H,D]`` or ``[B,H,1,D]``."""
        if k_new.size(1) == 1:
            k_new, v_new = k_new.transpose(1, 2), v_new.transpose(1, 2)
        k_new = k_new.to(self.dtype)
        v_new = v_new.to(self.dtype)
        if k_new.stride(-1) != 1:
            k_new, v_new = k_new.contiguous(), v_new.contiguous()
        ops.ring_copy_rows(self.k[layer], k_new, self.t, to_ring=True)
        ops.ring_copy_rows(self.v[layer], v_new, self.t, to_ring=True)
        self._staged[layer] = True

    def advance(self):
        self.t += 1
        self.t_dev += 1
        self._staged = [False] * self.L

    def bulk_write_packed(self, kv, pos):
        """Fill from prefill output ``kv [2, L, B, H, T, D]``: the last ``min(pos, W-1)`` rows go to
        slots ``p % W`` (inference/kv_cache.py:57-68)."""
        r = min(pos, max(self.W - 1, 0))
        if r > 0:
            k, v = kv[0].to(self.dtype), kv[1].to(self.dtype)
            for layer in range(self.L):
                ops.ring_copy_rows(self.k[layer], k[layer][:, :, pos - r:pos], pos - r, to_ring=True)
                ops.ring_copy_rows(self.v[layer], v[layer][:, :, pos - r:pos], pos - r, to_ring=True)
        self.t = pos
        self.t_dev.fill_(pos)
        self._staged = [False] * self.L

    def bulk_write_layer(self, layer, k, v, pos):
        """One layer of ``bulk_write_packed`` straight from that layer's prefill output ``k, v [B,H,T,D]`` (any
        strides): the runner fills the ring layer by layer and never builds the stacked ``[2,L,B,H,T,D]`` tensor
        (models/daisy/daisy_core.py:358-369).  Call :meth:`set_position` once after the last layer."""
        r = min(pos, max(self.W - 1, 0))
        if r > 0:
            ops.ring_copy_rows(self.k[layer], k.to(self.dtype)[:, :, pos - r:pos], pos - r, to_ring=True)
            ops.ring_copy_rows(self.v[layer], v.to(self.dtype)[:, :, pos - r:pos], pos - r, to_ring=True)

    def set_position(self, pos):
        self.t = pos
        self.t_dev.fill_(pos)
        self._staged = [False] * self.L

    # ------------------------------------------------------------------ in-place access for the decode kernel
    def ring(self, layer):
        """``(k_ring, v_ring)`` as ``[B, H, W, D]`` views of the storage (no copy)."""
        return self.k[layer], self.v[layer]

    def mark_written(self, layer):
        """Record that the decode kernel stored the new row of ``layer`` itself."""
        self._staged[layer] = True
