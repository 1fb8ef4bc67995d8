"""Host-buffer entry points: the same hot-path calls for callers whose tensors live in (pinned) host memory.

Batch rows are independent, so a call is cut into per-row chunks that flow through three CUDA streams --
host-to-device copy, kernels, device-to-host copy -- with double-buffered device staging.  PCIe is full
duplex, so a step costs about max(copy-in, copy-out, compute) instead of their sum.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import ops


class HostPrefill:
    """Windowed prefill on pinned host tensors ``q,k,v [B,T,H,D]`` bf16 -> pinned host ``out [B,T,H,D]``
    (and optionally k', v').  Device staging buffers are allocated once and reused."""

    def __init__(self, T: int, H: int, D: int, device="cuda", rows_per_chunk: int = 1, return_kv: bool = False):
        self.dev = torch.device(device)
        self.T, self.H, self.D, self.rows = T, H, D, rows_per_chunk
        self.return_kv = return_kv
        mk = lambda: torch.empty(rows_per_chunk, T, H, D, dtype=torch.bfloat16, device=self.dev)
        self.stage = [dict(q=mk(), k=mk(), v=mk(), out=mk(), ko=mk(), vo=mk()) for _ in range(2)]
        self.ws = [torch.empty(ops._lib.lib().daisy_b200_swa_prefill_workspace_bytes(rows_per_chunk, T, H, D),
                               dtype=torch.uint8, device=self.dev) for _ in range(2)]
        self.s_in, self.s_run, self.s_out = (torch.cuda.Stream(self.dev) for _ in range(3))
        self.ev_in = [torch.cuda.Event() for _ in range(2)]
        self.ev_run = [torch.cuda.Event() for _ in range(2)]
        self.ev_out = [torch.cuda.Event() for _ in range(2)]

    def __call__(self, q, k, v, cos, sin, window: Optional[int], out, k_out=None, v_out=None, scale: float = ops.ATTN_SCALE,
                 eps: float = 1.1920929e-07):
        for t in (q, k, v, out):
            assert not t.is_cuda and t.is_pinned(), "host tensors must be pinned"
        B = q.shape[0]
        cur = torch.cuda.current_stream(self.dev)
        for s in (self.s_in, self.s_run, self.s_out):
            s.wait_stream(cur)
        n = 0
        for b0 in range(0, B, self.rows):
            b1 = min(B, b0 + self.rows)
            r = b1 - b0
            st, i = self.stage[n & 1], n & 1
            with torch.cuda.stream(self.s_in):
                if n >= 2:
                    self.s_in.wait_event(self.ev_run[i])           # staging inputs free again
                st["q"][:r].copy_(q[b0:b1], non_blocking=True)
                st["k"][:r].copy_(k[b0:b1], non_blocking=True)
                st["v"][:r].copy_(v[b0:b1], non_blocking=True)
                self.ev_in[i].record(self.s_in)
            with torch.cuda.stream(self.s_run):
                self.s_run.wait_event(self.ev_in[i])
                if n >= 2:
                    self.s_run.wait_event(self.ev_out[i])          # staging outputs drained
                ops.swa_prefill(st["q"][:r], st["k"][:r], st["v"][:r], cos, sin, window, scale, eps,
                                workspace=self.ws[i], out=st["out"][:r], k_out=st["ko"][:r], v_out=st["vo"][:r])
                self.ev_run[i].record(self.s_run)
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(self.ev_run[i])
                out[b0:b1].copy_(st["out"][:r], non_blocking=True)
                if self.return_kv and k_out is not None:
                    k_out[b0:b1].copy_(st["ko"][:r], non_blocking=True)
                    v_out[b0:b1].copy_(st["vo"][:r], non_blocking=True)
                self.ev_out[i].record(self.s_out)
            n += 1
        for s in (self.s_in, self.s_run, self.s_out):
            cur.wait_stream(s)
        return out
