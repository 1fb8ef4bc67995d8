"""Drop-in for the reference ``CausalSelfAttention`` (models/daisy/attention.py:73-202).

Same constructor, parameters (``qkvo_w [4, dim, dim]`` bf16, ``g_ve``), attributes and the three
``AttentionProtocol`` entry points (models/daisy/attention_protocol.py:5-42).  The two
projections stay cuBLAS GEMMs; everything between them -- q/k/v RMS norm, RoPE, the windowed
softmax attention, the ring-cache read and write -- runs in the hand-written sm_100a kernels of
``libdaisy_b200.so``.  There is no other code path: on a machine without the library or without a
GPU the calls raise.

Masking.  The kernels implement the reference's inference mask (models/daisy/daisy_core.py:53-69,
one document): key visible iff ``0 <= q - k < window``.  ``attn_mask`` therefore is a
``WindowMask(window)`` (or ``None`` for plain causal) instead of a dense ``[1,1,T,T]`` tensor.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Optional

import torch
from torch import nn, Tensor
import torch.nn.functional as F

from . import ops
from ._lib import NORM_Q, NORM_K, NORM_V, ROPE, QKV_DEFAULT
from .kv_cache import B200KVCache


@dataclass(frozen=True)
class WindowMask:
    """Stands in for the dense additive mask of ``build_attn_mask`` (models/daisy/daisy_core.py:53-69): causal,
    ``window`` most recent keys and, with ``doc_start``, only keys of the query's own document.
    ``doc_start`` is an integer tensor ``[T]`` or ``[B,T]`` holding each token's first document position
    (:func:`doc_starts` builds it from the token ids the way the reference numbers documents)."""
    window: Optional[int]
    doc_start: Optional[Tensor] = None

    @classmethod
    def from_tokens(cls, input_seq: Tensor, window: Optional[int], eos_token_id: int) -> "WindowMask":
        """Same arguments as ``build_attn_mask(input_seq, window_size, eos_token_id)``."""
        return cls(window, doc_starts(input_seq, eos_token_id))


WINDOW_BLOCK_SIZE = 128      # models/daisy/daisy_core.py: WINDOW_BLOCK_SIZE, also the kernels' key tile


@dataclass(frozen=True)
class BlockWindowMask:
    """Stands in for one flex-attention ``BlockMask`` of ``DaisyCore.create_blockmasks``
    (models/daisy/daisy_core.py:182-229), the training-form mask: causal and same-document per token, and
    only the ``window_blocks`` nearest key blocks of 128 tokens (key block >= query block - window_blocks + 1).
    That is what the reference's block lists select: its "full" blocks are clamped to the ``window_blocks - 1``
    nearest, its "partial" blocks (the diagonal and blocks a document boundary crosses) to
    ``max(window_blocks - #full, 1)`` nearest, and together these are always the nearest ``window_blocks``
    blocks that hold any visible key."""
    window_blocks: int
    doc_start: Optional[Tensor] = None


def create_blockmasks(input_seq: Tensor, sliding_window_num_blocks: int, L: int, eos_token_id: int):
    """One mask per layer in the reference's long/short cycle (daisy_core.py:224-228): ``long`` uses
    ``sliding_window_num_blocks``, ``short`` half of it; layers cycle long, short, short, short and the last
    layer is long."""
    torch._assert(input_seq.shape[-1] % WINDOW_BLOCK_SIZE == 0, "input_seq length must be divisible by the block size")
    ds = doc_starts(input_seq, eos_token_id)
    wb = int(sliding_window_num_blocks)
    long_bm, short_bm = BlockWindowMask(wb, ds), BlockWindowMask(wb // 2, ds)
    cycle = [long_bm] + [short_bm] * 3
    return (cycle * ((L + 3) // 4))[:L - 1] + [long_bm]


def doc_starts(input_seq: Tensor, eos_token_id: int) -> Tensor:
    """First position of each token's document, int32, shape of ``input_seq`` without a leading batch of 1.
    The reference counts ``docs = (input_seq == eos).cumsum(0)``: an EOS token opens the next document, so the
    start is the position of the last EOS at or before the token (0 if there is none)."""
    seq = input_seq.squeeze(0) if input_seq.dim() == 2 and input_seq.size(0) == 1 else input_seq
    pos = torch.arange(seq.shape[-1], device=seq.device).expand_as(seq)
    marks = torch.where(seq == eos_token_id, pos, torch.zeros_like(pos))
    return torch.cummax(marks, dim=-1).values.to(torch.int32)


class Rotary(nn.Module):
    """cos/sin tables of the reference's half-truncated RoPE (models/daisy/attention.py:26-47):
    head_dim//4 frequencies ``(1/1024)**linspace(0,1,head_dim//4)`` followed by zeros."""

    def __init__(self, dim: int, max_seq_len: int, base: float = 1024.0):
        super().__init__()
        half, keep = dim // 2, dim // 4
        if keep == 0:
            freq = (1 / base) ** torch.linspace(0, 1, steps=half, dtype=torch.float32)
        else:
            active = (1 / base) ** torch.linspace(0, 1, steps=keep, dtype=torch.float32)
            freq = torch.cat([active, active.new_zeros(half - keep)])
        self.inv_freq = nn.Buffer(freq, persistent=False)
        theta = torch.einsum("i,j -> ij", torch.arange(max_seq_len, dtype=torch.float32), freq)
        self.cos = nn.Buffer(theta.cos(), persistent=False)
        self.sin = nn.Buffer(theta.sin(), persistent=False)
        self._max_seq_len = int(max_seq_len)

    def tables(self, L: int):
        torch._assert(L <= self.cos.shape[0], f"Rotary buffers too small {self.cos.shape[0]} < {L}")
        return self.cos, self.sin


def _init_linear(w: Tensor):
    # models/daisy/functional.py:11-14
    std = 0.5 * (w.size(-1) ** -0.5)
    bound = (3 ** 0.5) * std
    return w.uniform_(-bound, bound)


class B200CausalSelfAttention(nn.Module):
    def __init__(self, dim: int, num_heads: int, head_dim, receives_ve: bool = False,
                 layer_idx: Optional[int] = None, max_seq_len: int = 131072):
        super().__init__()
        torch._assert(dim % num_heads == 0, "dim must be divisible by num_heads")
        torch._assert(head_dim == 128, "the B200 kernels implement head_dim == 128")
        torch._assert(dim == num_heads * head_dim, "dim must equal num_heads * head_dim")
        self.num_heads = num_heads
        self.head_dim = head_dim
        self.m_dim = dim
        with torch.no_grad():
            self.qkvo_w = nn.Parameter(_init_linear(torch.empty(4, dim, dim)).bfloat16())
            if os.getenv("DISABLE_O_ZERO_INIT", "") != "1":
                self.qkvo_w.detach()[3].zero_()
        self.rotary = Rotary(head_dim, max_seq_len)
        self.attn_scale = 0.12
        # F.rms_norm(x, (D,)) with eps=None uses finfo(x.dtype).eps (models/daisy/functional.py:7)
        self.norm_eps = float(torch.finfo(torch.bfloat16).eps)
        self.last_q = None
        self.last_k = None
        self.receives_ve = receives_ve
        # True (default): forward / prefill run the projections on this library's tcgen05 GEMM, the norm and RoPE in
        # the QKV epilogue (measured faster than cuBLAS followed by the norm/RoPE pass); False or
        # DAISY_NATIVE_GEMM=0: F.linear (cuBLAS) + qkv_prep.  Single-token steps always take the F.linear form.
        self.native_gemm = os.environ.get("DAISY_NATIVE_GEMM", "1") == "1"
        if receives_ve:
            init = {0: 0.3228, 1: 0.0, 2: -1.5163, 21: -2.4423, 22: -2.9444, 23: 10.0}.get(layer_idx, 0.0) \
                if layer_idx is not None else 0.0
            self.g_ve = nn.Parameter(torch.tensor(init))
        else:
            self.g_ve = None

    def reset_history(self):
        self.last_q = None
        self.last_k = None

    # ------------------------------------------------------------------ helpers
    def _project(self, x: Tensor):
        B, T = x.size(0), x.size(1)
        x = x.to(self.qkvo_w.dtype)
        qkv = F.linear(x, self.qkvo_w[:3].flatten(end_dim=1)).view(B, T, 3 * self.num_heads, self.head_dim)
        return qkv.chunk(3, dim=-2)                       # strided views, no copies

    @staticmethod
    def _window_of(attn_mask):
        """-> (window or None, doc_start tensor or None[, True when the window counts 128-token blocks])"""
        if attn_mask is None:
            return None, None
        if isinstance(attn_mask, WindowMask):
            return attn_mask.window, attn_mask.doc_start
        if isinstance(attn_mask, BlockWindowMask):
            torch._assert(attn_mask.window_blocks >= 1, "a block window keeps at least the diagonal block")
            return attn_mask.window_blocks, attn_mask.doc_start, True
        if isinstance(attn_mask, int):
            return attn_mask, None
        raise TypeError("attn_mask must be None, an int window or WindowMask(window[, doc_start]); dense mask "
                        "tensors are not consumed by the B200 kernels")

    def _attend(self, x: Tensor, ve: Optional[Tensor], mask):
        window, doc_start = mask[0], mask[1]
        in_blocks = len(mask) > 2 and mask[2]
        B, T = x.size(0), x.size(1)
        cos, sin = self.rotary.tables(T)
        if self.native_gemm and self.m_dim % 64 == 0:
            # every kernel hand-written: QKV GEMM with norm + RoPE (+ the value-embedding gate) in its epilogue,
            # attention, output GEMM
            w = self.qkvo_w
            ve_kw = {}
            if self.receives_ve:
                torch._assert(ve is not None, "ve must be provided when receives_ve=True")
                ve_kw = dict(ve=ve.to(torch.bfloat16), ve_gate_logit=self.g_ve.detach().float().reshape(1))
            qp, kp, vp = ops.qkv_gemm(x.to(w.dtype), w[:3].flatten(end_dim=1), cos, sin, self.num_heads, self.norm_eps,
                                      **ve_kw)
            y = ops.swa_attend(qp, kp, vp, window, self.attn_scale, bounded_qk=True, doc_start=doc_start,
                               window_in_blocks=in_blocks)
            y = ops.gemm_nt(y.view(B, T, self.m_dim), w[3])
            return y, kp.transpose(1, 2), vp.transpose(1, 2), qp.transpose(1, 2)
        q, k, v = self._project(x)
        if self.receives_ve:
            torch._assert(ve is not None, "ve must be provided when receives_ve=True")
            # the gate v' = sigmoid(g_ve) * norm(v) + (1 - sigmoid(g_ve)) * ve rides on the norm/RoPE pass
            ve_ = ve.view(B, T, self.num_heads, self.head_dim).to(torch.bfloat16)
            qp, kp, vp = ops.qkv_prep(q, k, v, cos, sin, self.norm_eps, ve=ve_,
                                      ve_gate_logit=self.g_ve.detach().float().reshape(1))
            y = ops.swa_attend(qp, kp, vp, window, self.attn_scale, bounded_qk=True,   # q, k are RMS-normalised
                               doc_start=doc_start, window_in_blocks=in_blocks)
            qp, kp, vp = qp.transpose(1, 2), kp.transpose(1, 2), vp.transpose(1, 2)
        else:
            y, kp, vp = ops.swa_prefill(q, k, v, cos, sin, window, self.attn_scale, self.norm_eps, doc_start=doc_start,
                                        window_in_blocks=in_blocks)
            qp = None
        y = F.linear(y.view(B, T, self.m_dim), self.qkvo_w[3])
        return y, kp, vp, qp

    # ------------------------------------------------------------------ AttentionProtocol
    def forward(self, x: Tensor, ve: Optional[Tensor], block_mask=None, attn_mask=None):
        # block_mask: a BlockWindowMask (what create_blockmasks returns here) selects the training-form mask of
        # forward_flex (models/daisy/attention.py:156-162); otherwise attn_mask as in forward_sdpa
        if block_mask is not None:
            torch._assert(isinstance(block_mask, BlockWindowMask), "block_mask must be a daisy_b200 BlockWindowMask")
            torch._assert(x.size(1) % WINDOW_BLOCK_SIZE == 0, "the block-granular mask needs T divisible by 128")
            y, _, _, _ = self._attend(x, ve, self._window_of(block_mask))
            return y
        y, _, _, _ = self._attend(x, ve, self._window_of(attn_mask))
        return y

    def prefill(self, x: Tensor, ve: Optional[Tensor], attn_mask=None, debug: bool = False):
        """Returns ``(y [B,T,dim], k [B,H,T,D], v [B,H,T,D])`` (models/daisy/attention.py:173-179)."""
        y, k, v, q = self._attend(x, ve, self._window_of(attn_mask))
        if debug:
            self.last_q = None if q is None else q.transpose(1, 2)
            self.last_k = k.transpose(1, 2)
        return y, k, v

    def step(self, x, k_ctx: Optional[Tensor], v_ctx: Optional[Tensor], pos: int, ve: Optional[Tensor],
             window: Optional[int]):
        """One token against a chronological context ``[B,n,H,D]`` (models/daisy/attention.py:181-202).
        Returns ``(y [B,1,dim], k_new [B,1,H,D], v_new [B,1,H,D])``."""
        B = x.size(0)
        q, k, v = self._project(x)
        n = 0 if k_ctx is None else k_ctx.size(1)
        kc = None if n == 0 else k_ctx.transpose(1, 2)        # logical [B,H,n,D]
        vc = None if n == 0 else v_ctx.transpose(1, 2)
        if kc is not None and kc.dtype != torch.bfloat16:     # reference casts the context to q's dtype
            kc, vc = kc.to(torch.bfloat16), vc.to(torch.bfloat16)
        y, k_new, v_new = self._decode(q, k, v, kc, vc, n, n, pos, ve, window, write_ring=False)
        y = F.linear(y.view(B, 1, self.m_dim), self.qkvo_w[3])
        return y, k_new, v_new

    def step_ring(self, x, cache: B200KVCache, layer: int, pos: int, ve: Optional[Tensor], window: Optional[int]):
        """``step`` fused with the cache: reads the ring in place and stores the new row into it
        (replaces ``cache.view(layer)`` + ``step`` + ``cache.write(layer, ...)`` of
        inference/generate.py:231-246).  The caller still calls ``cache.advance()`` once per token."""
        B = x.size(0)
        q, k, v = self._project(x)
        kr, vr = cache.ring(layer)
        y, k_new, v_new = self._decode(q, k, v, kr, vr, cache.t, cache.W, pos, ve, window, write_ring=True)
        cache.mark_written(layer)
        y = F.linear(y.view(B, 1, self.m_dim), self.qkvo_w[3])
        return y, k_new, v_new

    def step_ring_dev(self, x, cache: B200KVCache, layer: int, window: Optional[int]):
        """``step_ring`` with the position read from ``cache.t_dev`` on the device: nothing in the launch
        sequence depends on the token index, so it can be captured once in a CUDA graph and replayed
        (``StepRunner.capture_step``).  Position = tokens in the cache, as in ``Generator._step``."""
        torch._assert(not self.receives_ve, "the graph step does not take value embeddings")
        B = x.size(0)
        q, k, v = self._project(x)
        kr, vr = cache.ring(layer)
        y = ops.swa_decode_step_dev(q, k, v, kr, vr, cache.t_dev, cache.W, window, self.rotary.cos, self.rotary.sin,
                                    self.attn_scale, self.norm_eps, QKV_DEFAULT, write_ring=True)
        return F.linear(y.view(B, 1, self.m_dim), self.qkvo_w[3])

    def _decode(self, q, k, v, kc, vc, t, cap, pos, ve, window, write_ring):
        cos, sin = self.rotary.tables(pos + 1)
        flags = QKV_DEFAULT
        if self.receives_ve:
            torch._assert(ve is not None, "ve must be provided when receives_ve=True")
            vf = v.float()
            vf = vf * torch.rsqrt(vf.pow(2).mean(-1, keepdim=True) + self.norm_eps)
            g = torch.sigmoid(self.g_ve).float()
            v = (g * vf + (1.0 - g) * ve.view_as(v).float()).to(torch.bfloat16)
            flags = NORM_Q | NORM_K | ROPE
        return ops.swa_decode_step(q, k, v, kc, vc, t, cap, window, cos[pos], sin[pos], self.attn_scale,
                                   self.norm_eps, flags, write_ring=write_ring)
