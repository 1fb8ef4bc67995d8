"""Drop-in for the reference ``CausalSelfAttention`` (models/daisy/attention.py:73-202).

Same constructor, parameters (``qkvo_w [4, dim, dim]`` bf16, ``g_ve``), attributes and the three
``AttentionProtocol`` entry points (models/daisy/attention_protocol.py:5-42).  ``forward`` and ``prefill``
run on hand-written sm_100a kernels of ``libdaisy_b200.so`` only: the merged QKV projection with the RMS
norm, RoPE and value-embedding gate in its epilogue, the windowed softmax attention, the output projection.
The single-token ``step`` forms are three launches: the token's merged QKV projection (a weight-streaming
kernel), the single-launch ring-cache decode (norm, RoPE, value-embedding gate, split-KV attention, merge, ring
store) and the output projection.  There is no other code path and no switch that selects one: on a machine without the library
or without a GPU the calls raise.

Masking.  The kernels evaluate the reference's inference mask (models/daisy/daisy_core.py:53-69)
analytically: key visible iff ``0 <= q - k < window`` and both tokens lie in one document.  ``attn_mask`` is
a ``WindowMask(window[, doc_start])``, an int, ``None`` (plain causal) -- or the reference's own dense additive
``[1,1,T,T]`` tensor, which is read once on the device to recover each row's first visible key
(:func:`band_of_dense_mask`) and rejected if it is not such a band.

Training.  When a call needs gradients (grad mode on and the input or a parameter requires them) ``forward``
takes the differentiable route: ``F.linear`` projections (autograd supplies their gradients) around
``daisy_b200.autograd.swa_attention``, whose backward is this library's tcgen05 backward kernels.  In a layer that
receives a value embedding the norm of v and the gate are torch operations on that route, so the gate parameter and
``ve`` get their gradients too.  The cache-writing ``prefill`` / ``step`` forms have no backward and raise.
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
    # the reference clamps a layer's partial-block count to at least 1 (daisy_core.py:216), so the short layers
    # of a one-block window keep the diagonal block
    long_bm, short_bm = BlockWindowMask(wb, ds), BlockWindowMask(max(wb // 2, 1), ds)
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


def band_of_dense_mask(mask: Tensor) -> Tensor:
    """First visible key of every query row of a dense attention mask, int32 ``[T]`` or ``[B,T]``.

    ``mask`` is what the reference passes to ``F.scaled_dot_product_attention``: additive float (0 = visible,
    -inf = masked; models/daisy/daisy_core.py:53-69) or boolean (True = visible), shape ``[T,T]``,
    ``[1,1,T,T]`` or ``[B,1,T,T]``.  The kernels can express exactly the masks of that builder -- row q sees the
    contiguous keys ``first[q] .. q`` with ``first`` non-decreasing (causal, sliding window, documents) -- so the
    tensor is checked to be such a band on the device (one pass over T x T and one host synchronisation; pass a
    ``WindowMask`` to avoid both) and ``ValueError`` is raised otherwise."""
    if mask.dim() == 4:
        torch._assert(mask.size(1) == 1, "a dense mask must broadcast over heads: [B,1,T,T]")
        mask = mask[:, 0]
    if mask.dim() == 2:
        mask = mask[None]
    torch._assert(mask.dim() == 3 and mask.size(-1) == mask.size(-2), "a dense mask must be [T,T], [1,1,T,T] or [B,1,T,T]")
    if not mask.is_cuda:
        raise ValueError("the dense mask must be a CUDA tensor (daisy_b200 has no CPU path)")
    T = mask.size(-1)
    vis = mask if mask.dtype == torch.bool else (mask == 0)
    cnt = vis.sum(-1)
    first = vis.to(torch.uint8).argmax(-1)
    last = (T - 1) - vis.flip(-1).to(torch.uint8).argmax(-1)
    q = torch.arange(T, device=mask.device)
    ok = (cnt > 0) & (last == q) & (cnt == q - first + 1)
    ok = ok.all() & (first[:, 1:] >= first[:, :-1]).all()
    if not bool(ok):
        raise ValueError("the dense attn_mask is not a causal band (window / document mask): the B200 kernels cannot express it")
    first = first.to(torch.int32)
    return first[0] if first.size(0) == 1 else first


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
    def _linear(self, x: Tensor, w: Tensor) -> Tensor:
        """``F.linear(x, w)`` on this library's kernels: the weight-streaming one for the few rows of a decode step,
        the tcgen05 GEMM otherwise."""
        rows = x.numel() // x.size(-1)
        return ops.gemm_skinny(x, w) if rows <= 64 else ops.gemm_nt(x, w)

    def _project(self, x: Tensor):
        self._no_autograd(x)
        B, T = x.size(0), x.size(1)
        w = self.qkvo_w.detach()
        qkv = self._linear(x.detach().to(w.dtype), w[:3].flatten(end_dim=1)).view(B, T, 3 * self.num_heads, self.head_dim)
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
        if isinstance(attn_mask, Tensor):
            # the reference's dense mask: causal + "first visible key per row" says everything it can hold
            return None, band_of_dense_mask(attn_mask)
        raise TypeError("attn_mask must be None, an int window, WindowMask(window[, doc_start]) or the dense mask tensor of "
                        "build_attn_mask")

    def _needs_grad(self, x: Tensor) -> bool:
        return torch.is_grad_enabled() and (x.requires_grad or self.qkvo_w.requires_grad
                                            or (self.g_ve is not None and self.g_ve.requires_grad))

    def _no_autograd(self, x: Tensor):
        if self._needs_grad(x):
            raise NotImplementedError("this call has no backward pass (only forward() does): call "
                                      "it under torch.no_grad() / inference_mode(), or detach the input and freeze the parameters")

    def _attend_autograd(self, x: Tensor, ve: Optional[Tensor], mask):
        """The differentiable forward: same arithmetic as ``_attend`` with the norm / RoPE as their own pass.  In a layer
        with a value embedding the norm of v and the gate ``v = s(g_ve) norm(v) + (1 - s(g_ve)) ve``
        (models/daisy/attention.py:125,132-135) are torch operations, so autograd supplies the gradients of ``g_ve`` and
        ``ve`` as well, and the kernels get a v they must not normalise again."""
        from .autograd import swa_attention
        window, doc_start = mask[0], mask[1]
        in_blocks = len(mask) > 2 and mask[2]
        B, T = x.size(0), x.size(1)
        cos, sin = self.rotary.tables(T)
        w = self.qkvo_w
        qkv = F.linear(x.to(w.dtype), w[:3].flatten(end_dim=1)).view(B, T, 3 * self.num_heads, self.head_dim)
        q, k, v = qkv.chunk(3, dim=-2)
        flags = QKV_DEFAULT
        if self.receives_ve:
            torch._assert(ve is not None, "ve must be provided when receives_ve=True")
            vn = F.rms_norm(v.float(), (self.head_dim,), eps=self.norm_eps)
            g = torch.sigmoid(self.g_ve.float())
            v = (g * vn + (1.0 - g) * ve.view_as(v).float()).to(q.dtype)
            flags = QKV_DEFAULT & ~NORM_V
        y = swa_attention(q, k, v, cos, sin, window, self.attn_scale, self.norm_eps, flags, doc_start, in_blocks)
        return F.linear(y.view(B, T, self.m_dim), w[3])

    def _attend(self, x: Tensor, ve: Optional[Tensor], mask, ring=None, ring_first: int = 0):
        """Every kernel hand-written: QKV GEMM with norm + RoPE (+ the value-embedding gate) in its epilogue,
        attention, output GEMM.  Returns ``(y, k', v', q')`` with k', v', q' shaped ``[B,H,T,D]``.  ``ring``: one
        layer of a KV ring the projection's epilogue also fills from position ``ring_first`` on."""
        self._no_autograd(x)
        window, doc_start = mask[0], mask[1]
        in_blocks = len(mask) > 2 and mask[2]
        B, T = x.size(0), x.size(1)
        cos, sin = self.rotary.tables(T)
        w = self.qkvo_w.detach()
        ve_kw = {}
        if self.receives_ve:
            torch._assert(ve is not None, "ve must be provided when receives_ve=True")
            ve_kw = dict(ve=ve.to(torch.bfloat16), ve_gate_logit=self.g_ve.detach().float().reshape(1))
        qp, kp, vp = ops.qkv_gemm(x.detach().to(w.dtype), w[:3].flatten(end_dim=1), cos, sin, self.num_heads, self.norm_eps,
                                  ring=ring, ring_first=ring_first, **ve_kw)
        y = ops.swa_attend(qp, kp, vp, window, self.attn_scale, bounded_qk=True, doc_start=doc_start,   # q, k are RMS-normalised
                           window_in_blocks=in_blocks)
        y = ops.gemm_nt(y.view(B, T, self.m_dim), w[3])
        return y, kp.transpose(1, 2), vp.transpose(1, 2), qp.transpose(1, 2)

    # ------------------------------------------------------------------ AttentionProtocol
    def forward(self, x: Tensor, ve: Optional[Tensor], block_mask=None, attn_mask=None):
        # block_mask: a BlockWindowMask (what create_blockmasks returns here) selects the training-form mask of
        # forward_flex (models/daisy/attention.py:156-162); otherwise attn_mask as in forward_sdpa
        if block_mask is not None:
            torch._assert(isinstance(block_mask, BlockWindowMask), "block_mask must be a daisy_b200 BlockWindowMask")
            torch._assert(x.size(1) % WINDOW_BLOCK_SIZE == 0, "the block-granular mask needs T divisible by 128")
            attn_mask = block_mask
        mask = self._window_of(attn_mask)
        if self._needs_grad(x) or (ve is not None and torch.is_grad_enabled() and ve.requires_grad):
            return self._attend_autograd(x, ve, mask)
        y, _, _, _ = self._attend(x, ve, mask)
        return y

    def prefill(self, x: Tensor, ve: Optional[Tensor], attn_mask=None, debug: bool = False):
        """Returns ``(y [B,T,dim], k [B,H,T,D], v [B,H,T,D])`` (models/daisy/attention.py:173-179)."""
        y, k, v, q = self._attend(x, ve, self._window_of(attn_mask))
        if debug:
            self.last_q = q.transpose(1, 2)
            self.last_k = k.transpose(1, 2)
        return y, k, v

    def prefill_ring(self, x: Tensor, ve: Optional[Tensor], cache: B200KVCache, layer: int, attn_mask=None):
        """``prefill`` that fills layer ``layer`` of the ring cache itself: the projection kernel stores the rows
        ``KVCache.bulk_write_packed`` would keep (the last ``min(T, W - 1)``, inference/kv_cache.py:57-68) into their
        slots as it produces them, so the prompt's k, v are neither stacked (models/daisy/daisy_core.py:358-369) nor
        copied afterwards.  The caller sets the cache position once after the last layer
        (``cache.set_position(T)``).  Returns ``(y, k, v)`` like ``prefill``."""
        T = x.size(1)
        r = min(T, max(cache.W - 1, 0))
        ring = cache.ring(layer) if r > 0 else None
        y, k, v, _ = self._attend(x, ve, self._window_of(attn_mask), ring=ring, ring_first=T - r)
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
        y = self._linear(y.view(B, 1, self.m_dim), self.qkvo_w.detach()[3])
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
        y = self._linear(y.view(B, 1, self.m_dim), self.qkvo_w.detach()[3])
        return y, k_new, v_new

    def step_ring_dev(self, x, cache: B200KVCache, layer: int, window: Optional[int], write_ring: bool = True,
                      ve: Optional[Tensor] = None):
        """``step_ring`` with the position read from ``cache.t_dev`` on the device: nothing in the launch
        sequence depends on the token index, so it can be captured once in a CUDA graph and replayed
        (``StepRunner.capture_step``).  Position = tokens in the cache, as in ``Generator._step``.  Three launches,
        all of this library: the merged QKV projection of the token (weight-streaming kernel), the single-launch
        ring decode (norm, RoPE, value-embedding gate, split-KV attention, merge, ring store), the output
        projection."""
        self._no_autograd(x)
        B = x.size(0)
        H, D = self.num_heads, self.head_dim
        w = self.qkvo_w.detach()
        qkv = ops.gemm_skinny(x.detach().to(w.dtype).view(B, self.m_dim), w[:3].flatten(end_dim=1)).view(B, 1, 3 * H, D)
        q, k, v = qkv[:, :, :H], qkv[:, :, H:2 * H], qkv[:, :, 2 * H:]
        kr, vr = cache.ring(layer)
        ve_kw = {}
        if self.receives_ve:
            torch._assert(ve is not None, "ve must be provided when receives_ve=True")
            ve_kw = dict(ve=ve.to(torch.bfloat16), ve_gate_logit=self.g_ve.detach().float().reshape(1))
        key = (B, cache.W, window)
        if getattr(self, "_fused_ws_key", None) != key:                   # zeroed once; every call leaves the tickets zero
            r = cache.W if not window else min(cache.W, window - 1)
            self._fused_splits = ops.decode_splits(B, H, r)
            self._fused_ws = ops.decode_fused_workspace(B, H, D, self._fused_splits, x.device)
            self._fused_ws_key = key
        y = ops.swa_decode_step_fused(q, k, v, kr, vr, cache.t_dev, cache.W, window, self.rotary.cos, self.rotary.sin,
                                      self.attn_scale, self.norm_eps, QKV_DEFAULT, write_ring=write_ring,
                                      splits=self._fused_splits, workspace=self._fused_ws, **ve_kw)
        return ops.gemm_skinny(y.view(B, self.m_dim), w[3]).view(B, 1, self.m_dim)

    def _decode(self, q, k, v, kc, vc, t, cap, pos, ve, window, write_ring):
        cos, sin = self.rotary.tables(pos + 1)
        ve_kw = {}
        if self.receives_ve:
            torch._assert(ve is not None, "ve must be provided when receives_ve=True")
            ve_kw = dict(ve=ve.to(torch.bfloat16), ve_gate_logit=self.g_ve.detach().float().reshape(1))
        return ops.swa_decode_step_fused(q, k, v, kc, vc, int(t), cap, window, cos[pos], sin[pos], self.attn_scale,
                                         self.norm_eps, QKV_DEFAULT, write_ring=write_ring, return_new_kv=True, **ve_kw)
