"""fp32 CPU oracle: sliding-window causal attention + ring KV cache.

Test infrastructure only (see ``oracle/__init__.py``).  Every function cites the
reference lines it restates; paths are relative to the reference project root.
All math is done in ``torch.float32`` (or the dtype of the inputs when they are
float64) on the CPU with plain tensor ops -- no fused attention kernels.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch

ATTN_SCALE = 0.12          # models/daisy/attention.py:88
ROPE_BASE_REFERENCE = 1024  # models/daisy/attention.py:32
FP32_EPS = float(torch.finfo(torch.float32).eps)   # models/daisy/functional.py:7 with fp32 inputs
BF16_EPS = float(torch.finfo(torch.bfloat16).eps)  # same call with bf16 inputs


# --------------------------------------------------------------------------- norm / rope

def rms_norm(x: torch.Tensor, eps: float) -> torch.Tensor:
    """Weightless RMS norm over the last dim (models/daisy/functional.py:6-7).

    ``F.rms_norm(x, (D,))`` with ``eps=None`` uses ``finfo(x.dtype).eps``; the
    caller passes that value explicitly."""
    ms = x.pow(2).mean(dim=-1, keepdim=True)
    return x * torch.rsqrt(ms + eps)


def rope_tables(head_dim: int, max_len: int, base: float = ROPE_BASE_REFERENCE,
                truncate: bool = True) -> Tuple[torch.Tensor, torch.Tensor]:
    """cos/sin tables ``[max_len, head_dim//2]`` fp32 (models/daisy/attention.py:26-47).

    ``truncate=True`` is the reference's half-truncated RoPE: only the first
    ``head_dim//4`` frequencies are non-zero, ``(1/base)**linspace(0,1,head_dim//4)``,
    the rest are zero (identity rotation).  ``truncate=False`` gives a full
    table with ``head_dim//2`` frequencies on the same linspace form."""
    half = head_dim // 2
    keep = head_dim // 4
    if keep == 0 or not truncate:
        freq = (1.0 / base) ** torch.linspace(0, 1, steps=half, dtype=torch.float32)
    else:
        active = (1.0 / base) ** torch.linspace(0, 1, steps=keep, dtype=torch.float32)
        freq = torch.cat([active, active.new_zeros(half - keep)])
    t = torch.arange(max_len, dtype=torch.float32)
    theta = torch.einsum("i,j->ij", t, freq)
    return theta.cos(), theta.sin()


def apply_rope(x_bthd: torch.Tensor, cos_td: torch.Tensor, sin_td: torch.Tensor) -> torch.Tensor:
    """Rotate halves (models/daisy/attention.py:16-20): ``y1 = x1 cos + x2 sin``,
    ``y2 = -x1 sin + x2 cos`` with ``x1 = x[..., :D/2]``, ``x2 = x[..., D/2:]``.
    ``cos_td``/``sin_td`` are ``[T, D/2]`` and broadcast over batch and heads."""
    x1, x2 = x_bthd.chunk(2, dim=-1)
    c = cos_td[None, :, None, :].to(x_bthd.dtype)
    s = sin_td[None, :, None, :].to(x_bthd.dtype)
    return torch.cat((x1 * c + x2 * s, -x1 * s + x2 * c), dim=-1)


def qkv_transform(q, k, v, cos_td, sin_td, eps: float, norm_q=True, norm_k=True, norm_v=True,
                  rope=True):
    """What ``CausalSelfAttention._calc_qkv`` does after the projection
    (models/daisy/attention.py:121-125): RMS-norm q, k and v; RoPE q and k.
    Inputs/outputs ``[B, T, H, D]``; ``cos_td`` rows are the positions of the T tokens."""
    q, k, v = q.float(), k.float(), v.float()
    if norm_q:
        q = rms_norm(q, eps)
    if norm_k:
        k = rms_norm(k, eps)
    if norm_v:
        v = rms_norm(v, eps)
    if rope:
        q = apply_rope(q, cos_td, sin_td)
        k = apply_rope(k, cos_td, sin_td)
    return q, k, v


# --------------------------------------------------------------------------- prefill

def doc_starts(input_seq: torch.Tensor, eos_token_id: int) -> torch.Tensor:
    """For every position t of ``input_seq [T]`` (or ``[B,T]``) the first position of its document, int32.
    ``build_attn_mask`` numbers documents ``docs = (input_seq == eos).cumsum(0)``
    (models/daisy/daisy_core.py:60), so an EOS token opens the next document and belongs to it:
    document of t = [last EOS position <= t (or 0), next EOS position)."""
    is_eos = input_seq == eos_token_id
    pos = torch.arange(input_seq.shape[-1]).expand_as(input_seq)
    marks = torch.where(is_eos, pos, torch.zeros_like(pos))
    return torch.cummax(marks, dim=-1).values.to(torch.int32)


BLOCK = 128      # WINDOW_BLOCK_SIZE of the reference (models/daisy/daisy_core.py)


def flex_block_lists(docs: torch.Tensor, window_blocks: int):
    """The key-block lists ``build_bm(window_blocks)`` hands to ``BlockMask.from_kv_blocks``
    (models/daisy/daisy_core.py:196-221), restated: per query block, the selected *partial* blocks (some but not
    all (q,k) pairs pass ``document_causal``) and *full* blocks (all pass), as Python sets.  ``docs [T]`` are the
    document numbers ``(input_seq == eos).cumsum(0)``.  Both kinds are listed nearest first; full blocks are cut
    to the ``window_blocks - 1`` nearest, partial ones to ``max(window_blocks - #full, 1)`` nearest."""
    nb = docs.numel() // BLOCK
    lo, hi = docs.view(nb, BLOCK)[:, 0], docs.view(nb, BLOCK)[:, -1]
    partial, full = [], []
    for qb in range(nb):
        any_ = [kb for kb in range(qb, -1, -1) if lo[qb] <= hi[kb] and hi[qb] >= lo[kb]]           # nearest first
        all_ = [kb for kb in range(qb - 1, -1, -1) if lo[qb] == hi[kb] and hi[qb] == lo[kb]]
        part = [kb for kb in any_ if kb not in all_]
        n_full = len(all_)
        full.append(set(all_[:max(min(n_full, window_blocks - 1), 0)]))
        partial.append(set(part[:min(len(part), max(window_blocks - n_full, 1))]))
    return partial, full


def window_mask(q_lo: int, q_hi: int, k_lo: int, k_hi: int, window: Optional[int],
                doc_start: Optional[torch.Tensor] = None, window_blocks: Optional[int] = None) -> torch.Tensor:
    """Additive mask block for query rows [q_lo,q_hi) x key cols [k_lo,k_hi): 0 where
    ``0 <= q - k < window`` and q, k lie in the same document, else -inf
    (models/daisy/daisy_core.py:53-69).  ``window=None`` means plain causal; ``doc_start [T]`` (see
    :func:`doc_starts`) None means one document.  With causality, "same document" is ``k >= doc_start[q]``."""
    qi = torch.arange(q_lo, q_hi)[:, None]
    ki = torch.arange(k_lo, k_hi)[None, :]
    d = qi - ki
    bad = d < 0
    if window is not None:
        bad = bad | (d >= window)
    if doc_start is not None:
        bad = bad | (ki < doc_start[q_lo:q_hi].to(torch.int64)[:, None])
    if window_blocks is not None:
        # training form (flex BlockMasks of create_blockmasks, daisy_core.py:182-229): the lists of
        # :func:`flex_block_lists` always amount to the window_blocks nearest key blocks
        bad = bad | (ki // BLOCK < qi // BLOCK - window_blocks + 1)
    m = torch.zeros(q_hi - q_lo, k_hi - k_lo, dtype=torch.float32)
    m[bad] = float("-inf")
    return m


def attend_windowed(q, k, v, window: Optional[int], scale: float = ATTN_SCALE, block: int = 512,
                    doc_start: Optional[torch.Tensor] = None, window_blocks: Optional[int] = None):
    """``softmax(scale * q k^T + M) v`` with the window (and document) mask, on already
    normalised / rotated ``[B, T, H, D]`` tensors (models/daisy/attention.py:141-148).
    Evaluated in blocks of ``block`` query rows against only the keys the mask can
    admit, which is the same arithmetic as the dense ``[T, T]`` mask.  ``doc_start`` is ``[T]`` (shared by the
    batch, as the reference's single ``input_seq``) or ``[B,T]``."""
    B, T, H, D = q.shape
    qh, kh, vh = (x.permute(0, 2, 1, 3) for x in (q, k, v))       # [B,H,T,D]
    out = torch.empty(B, H, T, D, dtype=q.dtype)
    for q0 in range(0, T, block):
        q1 = min(T, q0 + block)
        k0 = 0 if window is None else max(0, q0 - window + 1)
        s = torch.matmul(qh[:, :, q0:q1], kh[:, :, k0:q1].transpose(-1, -2)) * scale
        if doc_start is not None and doc_start.dim() == 2:
            m = torch.stack([window_mask(q0, q1, k0, q1, window, doc_start[b], window_blocks) for b in range(B)])[:, None]
        else:
            m = window_mask(q0, q1, k0, q1, window, doc_start, window_blocks)
        s = s + m.to(s.dtype)
        p = torch.softmax(s, dim=-1)
        out[:, :, q0:q1] = torch.matmul(p, vh[:, :, k0:q1])
    return out.permute(0, 2, 1, 3).contiguous()                   # [B,T,H,D]


def swa_prefill(q, k, v, cos_td, sin_td, window: Optional[int], scale: float = ATTN_SCALE,
                eps: float = FP32_EPS, norm_q=True, norm_k=True, norm_v=True, rope=True,
                block: int = 512, doc_start: Optional[torch.Tensor] = None, window_blocks: Optional[int] = None):
    """Projection-to-projection part of ``CausalSelfAttention.prefill``
    (models/daisy/attention.py:121-125,141-148,173-179): takes raw projected
    q,k,v ``[B,T,H,D]``, returns ``(y [B,T,H,D], k' [B,H,T,D], v' [B,H,T,D])`` in fp32."""
    qn, kn, vn = qkv_transform(q, k, v, cos_td, sin_td, eps, norm_q, norm_k, norm_v, rope)
    y = attend_windowed(qn, kn, vn, window, scale, block, doc_start, window_blocks)
    return y, kn.permute(0, 2, 1, 3).contiguous(), vn.permute(0, 2, 1, 3).contiguous()


# --------------------------------------------------------------------------- decode step

def decode_step(q_new, k_new, v_new, k_ctx, v_ctx, pos: int, window: Optional[int],
                cos_td, sin_td, scale: float = ATTN_SCALE, eps: float = FP32_EPS,
                norm_q=True, norm_k=True, norm_v=True, rope=True):
    """Projection-to-projection part of ``CausalSelfAttention.step``
    (models/daisy/attention.py:181-200).

    ``q_new,k_new,v_new`` raw ``[B,1,H,D]``; ``k_ctx,v_ctx`` chronological
    ``[B,n,H,D]`` (already normalised/rotated rows, as stored in the cache).  Uses
    the last ``r = min(n, window-1)`` context rows plus the new row.  Returns
    ``(y [B,1,H,D], k' [B,1,H,D], v' [B,1,H,D])``."""
    c = cos_td[pos:pos + 1] if rope else None
    s = sin_td[pos:pos + 1] if rope else None
    qn, kn, vn = qkv_transform(q_new, k_new, v_new, c, s, eps, norm_q, norm_k, norm_v, rope)
    n = k_ctx.size(1)
    r = n if window is None else min(n, max(window - 1, 0))
    K = torch.cat([k_ctx[:, n - r:n].float(), kn], 1).permute(0, 2, 1, 3)   # [B,H,r+1,D]
    V = torch.cat([v_ctx[:, n - r:n].float(), vn], 1).permute(0, 2, 1, 3)
    Q = qn.permute(0, 2, 1, 3)                                               # [B,H,1,D]
    p = torch.softmax(torch.matmul(Q, K.transpose(-1, -2)) * scale, dim=-1)
    y = torch.matmul(p, V).permute(0, 2, 1, 3).contiguous()
    return y, kn, vn


# --------------------------------------------------------------------------- ring KV cache

class RingKVCache:
    """Restatement of the reference ``KVCache`` (inference/kv_cache.py:4-68).

    Storage ``k, v [L, B, H, W, D]``; ``t`` counts tokens ever committed; token
    ``p`` lives in slot ``p % W``.  ``view`` returns the last ``min(t+staged, W)``
    rows in chronological order as ``[B, n, H, D]``."""

    def __init__(self, L, B, H, W, D, dtype=torch.float32):
        self.L, self.B, self.H, self.W, self.D = L, B, H, W, D
        self.dtype = dtype
        self.reset_history()

    def reset_history(self):                                  # kv_cache.py:19-23
        shape = (self.L, self.B, self.H, self.W, self.D)
        self.k = torch.zeros(shape, dtype=self.dtype)
        self.v = torch.zeros(shape, dtype=self.dtype)
        self.t = 0
        self._staged = [False] * self.L

    def view(self, layer):                                    # kv_cache.py:26-42
        staged = 1 if self._staged[layer] else 0
        n = min(self.t + staged, self.W)
        if n == 0:
            return (self.k[layer, :, :, :0].transpose(1, 2), self.v[layer, :, :, :0].transpose(1, 2))
        end = (self.t % self.W + staged) % self.W
        start = (end - n) % self.W
        idx = (start + torch.arange(n)) % self.W
        return (self.k[layer][:, :, idx].transpose(1, 2), self.v[layer][:, :, idx].transpose(1, 2))

    def write(self, layer, k_new, v_new):                     # kv_cache.py:44-51
        if k_new.size(1) == 1:                                # accepts [B,1,H,D] or [B,H,1,D]
            k_new, v_new = k_new.transpose(1, 2), v_new.transpose(1, 2)
        i = self.t % self.W
        self.k[layer, :, :, i:i + 1] = k_new
        self.v[layer, :, :, i:i + 1] = v_new
        self._staged[layer] = True

    def advance(self):                                        # kv_cache.py:53-55
        self.t += 1
        self._staged = [False] * self.L

    def bulk_write_packed(self, kv, pos):                     # kv_cache.py:57-68
        k, v = kv[0], kv[1]
        r = min(pos, max(self.W - 1, 0))
        if r > 0:
            idx = torch.arange(pos - r, pos) % self.W
            self.k[:, :, :, idx] = k[:, :, :, pos - r:pos].to(self.dtype)
            self.v[:, :, :, idx] = v[:, :, :, pos - r:pos].to(self.dtype)
        self.t = pos
        self._staged = [False] * self.L


# --------------------------------------------------------------------------- whole module

def project_qkv(x, qkvo_w, num_heads: int, head_dim: int):
    """Merged QKV projection and head split (models/daisy/attention.py:118-120):
    ``F.linear(x, W[:3].flatten(0,1)).view(B,T,3H,D).chunk(3,-2)``."""
    B, T, _ = x.shape
    w = qkvo_w[:3].reshape(-1, qkvo_w.shape[-1]).float()
    qkv = torch.matmul(x.float(), w.t()).view(B, T, 3 * num_heads, head_dim)
    return qkv.chunk(3, dim=-2)


def csa_prefill(x, qkvo_w, num_heads, head_dim, window, cos_td, sin_td, eps=FP32_EPS,
                scale=ATTN_SCALE, doc_start=None):
    """Whole ``CausalSelfAttention.prefill`` with ``ve=None``
    (models/daisy/attention.py:141-150,173-179): returns ``(y [B,T,dim], k', v' [B,H,T,D])``."""
    B, T, dim = x.shape
    q, k, v = project_qkv(x, qkvo_w, num_heads, head_dim)
    y, kn, vn = swa_prefill(q, k, v, cos_td[:T], sin_td[:T], window, scale, eps, doc_start=doc_start)
    y = torch.matmul(y.reshape(B, T, dim), qkvo_w[3].float().t())
    return y, kn, vn


def csa_backward(x, qkvo_w, num_heads, head_dim, window, cos_td, sin_td, cot, eps=FP32_EPS, scale=ATTN_SCALE,
                 doc_start=None):
    """Gradients of ``sum(forward(x) * cot)`` with respect to ``x`` and the merged weights, by ``torch.autograd``
    over :func:`csa_prefill` in fp32 -- what training computes through the reference module's forward
    (models/daisy/attention.py:164-171).  Returns ``(y, dx, dw)``."""
    x = x.detach().float().requires_grad_(True)
    w = qkvo_w.detach().float().requires_grad_(True)
    y, _, _ = csa_prefill(x, w, num_heads, head_dim, window, cos_td, sin_td, eps, scale, doc_start)
    (y * cot.float()).sum().backward()
    return y.detach(), x.grad, w.grad


def attend_backward(q, k, v, d_out, window, scale=ATTN_SCALE, doc_start=None, window_blocks=None):
    """Gradients of :func:`attend_windowed` with respect to its prepared inputs for the cotangent ``d_out``, by
    ``torch.autograd`` in fp32.  Returns ``(out, dq, dk, dv)``."""
    q, k, v = (t.detach().float().requires_grad_(True) for t in (q, k, v))
    out = attend_windowed(q, k, v, window, scale, doc_start=doc_start, window_blocks=window_blocks)
    (out * d_out.float()).sum().backward()
    return out.detach(), q.grad, k.grad, v.grad


def csa_step(x, qkvo_w, num_heads, head_dim, k_ctx, v_ctx, pos, window, cos_td, sin_td,
             eps=FP32_EPS, scale=ATTN_SCALE):
    """Whole ``CausalSelfAttention.step`` with ``ve=None`` (models/daisy/attention.py:181-202)."""
    B, _, dim = x.shape
    q, k, v = project_qkv(x, qkvo_w, num_heads, head_dim)
    y, kn, vn = decode_step(q, k, v, k_ctx, v_ctx, pos, window, cos_td, sin_td, scale, eps)
    y = torch.matmul(y.reshape(B, 1, dim), qkvo_w[3].float().t())
    return y, kn, vn


# --------------------------------------------------------------------------- work counts

def window_pairs(T: int, window: Optional[int]) -> int:
    """Number of (query, key) pairs the window mask admits."""
    W = T if window is None else min(window, T)
    return W * (W + 1) // 2 + (T - W) * W


def prefill_flops(B, T, H, D, window) -> float:
    """Algorithmic FLOPs of the windowed attention (QK^T and PV, 2 per multiply-add)."""
    return 4.0 * D * window_pairs(T, window) * B * H


def decode_bytes(B, H, D, ctx_rows: int, elem: int = 2) -> float:
    """Algorithmic HBM bytes of one decode step: K and V context rows read, new q,k,v
    read, output written, new k,v rows written to the ring."""
    return float(B * H * ctx_rows * D * elem * 2 + B * H * D * elem * 6)
