"""Tensor-level wrappers over the C ABI: torch supplies device memory and the stream, nothing else.

Every function requires CUDA tensors and calls into ``libdaisy_b200.so``; there is no CPU path.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import _lib
from ._lib import (NORM_Q, NORM_K, NORM_V, ROPE, QKV_DEFAULT, WRITE_RING, OUT_BTHD, KV_BHTD, Q_IN_KERNEL, KDA_L2NORM_QK,
                   KDA_OUT_FP32)

ATTN_SCALE = 0.12            # reference models/daisy/attention.py:88

_status_words = {}


def _stream(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def status_word(device) -> torch.Tensor:
    """Per-device int32 word that kernels write a DAISY_E* code into when a bounded wait runs out."""
    dev = torch.device(device)
    key = dev.index if dev.index is not None else torch.cuda.current_device()
    if key not in _status_words:
        _status_words[key] = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", key))
    return _status_words[key]


def check_device_status(device) -> None:
    """Synchronise and raise if any kernel reported a device-side error since the last check."""
    w = status_word(device)
    code = int(w.item())
    if code != 0:
        w.zero_()
        raise _lib.DaisyB200Error(code, "device-side status")


def _req(t: torch.Tensor, name: str, dtype=torch.bfloat16):
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor (daisy_b200 has no CPU path)")
    if t.dtype != dtype:
        raise TypeError(f"{name} must be {dtype}, got {t.dtype}")
    if t.stride(-1) != 1:
        raise ValueError(f"{name} must be contiguous in its last dimension")


def _f32c(t: torch.Tensor, name: str) -> torch.Tensor:
    if not t.is_cuda or t.dtype != torch.float32 or not t.is_contiguous():
        raise ValueError(f"{name} must be a contiguous float32 CUDA tensor")
    return t


def qkv_prep(q, k, v, cos, sin, eps: float, flags: int = QKV_DEFAULT, bhtd: bool = False,
             ve: Optional[torch.Tensor] = None, ve_gate_logit: Optional[torch.Tensor] = None):
    """RMS-norm / RoPE raw ``[B,T,H,D]`` projections.  Returns three ``[B,T,H,D]`` contiguous tensors, or
    ``[B,H,T,D]`` contiguous ones with ``bhtd=True``.  With ``ve`` (bf16, viewable as ``[B,T,H,D]``) and
    ``ve_gate_logit`` (float32 scalar tensor on the device) the value-embedding gate is applied to the
    normalised v: ``v' = g * norm(v) + (1 - g) * ve``, ``g = sigmoid(logit)``."""
    for n, t in (("q", q), ("k", k), ("v", v)):
        _req(t, n)
    B, T, H, D = q.shape
    ve_args = (None, 0, 0, 0, None)
    if ve is not None:
        if ve_gate_logit is None:
            raise ValueError("ve needs ve_gate_logit")
        ve = ve.view(B, T, H, D)
        _req(ve, "ve")
        if not (ve_gate_logit.is_cuda and ve_gate_logit.dtype == torch.float32 and ve_gate_logit.numel() == 1):
            raise ValueError("ve_gate_logit must be a float32 scalar CUDA tensor")
        ve_args = (ve.data_ptr(), ve.stride(0), ve.stride(1), ve.stride(2), ve_gate_logit.data_ptr())
    if flags & ROPE:
        cos, sin = _f32c(cos, "cos"), _f32c(sin, "sin")
        assert cos.shape[0] >= T and cos.shape[1] == D // 2
    shape = (B, H, T, D) if bhtd else (B, T, H, D)
    outs = [torch.empty(shape, dtype=torch.bfloat16, device=q.device) for _ in range(3)]
    rc = _lib.lib().daisy_b200_qkv_prep(
        q.data_ptr(), k.data_ptr(), v.data_ptr(),
        q.stride(0), q.stride(1), q.stride(2), k.stride(0), k.stride(1), k.stride(2),
        v.stride(0), v.stride(1), v.stride(2), cos.data_ptr() if cos is not None else None,
        sin.data_ptr() if sin is not None else None,
        outs[0].data_ptr(), outs[1].data_ptr(), outs[2].data_ptr(), *ve_args, B, T, H, D, eps,
        flags | (0 if bhtd else OUT_BTHD), _stream(q))
    _lib.check(rc, "daisy_b200_qkv_prep")
    return tuple(outs)


def qkv_gemm(x, w_qkv, cos, sin, num_heads: int, eps: float, flags: int = QKV_DEFAULT,
             ve: Optional[torch.Tensor] = None, ve_gate_logit: Optional[torch.Tensor] = None,
             ring: Optional[Tuple[torch.Tensor, torch.Tensor]] = None, ring_first: int = 0):
    """``x [B,T,dim]`` times the merged ``w_qkv [3*H*128, dim]`` (``qkvo_w[:3].flatten(end_dim=1)``) with the RMS
    norm and RoPE applied in the GEMM epilogue: returns prepared ``q', k', v'`` as ``[B,T,H,128]`` contiguous.
    ``ve [B,T,H*128]`` (bf16) with ``ve_gate_logit`` (float32 scalar on the device) mixes the value embedding into
    the normalised v: ``v' = g * norm(v) + (1 - g) * ve``.  ``ring = (k_ring, v_ring)``, one layer of a KV ring
    ``[B,H,cap,128]`` (bf16 or float16): the epilogue also stores rows ``t >= ring_first`` of k', v' into slot
    ``t % cap`` -- the rows ``KVCache.bulk_write_packed`` keeps when ``ring_first = T - min(T, cap - 1)``."""
    _req(x, "x"); _req(w_qkv, "w_qkv")
    B, T, dim = x.shape
    H, D = int(num_heads), 128
    if w_qkv.shape != (3 * H * D, dim):
        raise ValueError(f"w_qkv must be [{3 * H * D}, {dim}], got {tuple(w_qkv.shape)}")
    x2 = x.reshape(B * T, dim)
    if x2.stride(1) != 1:
        x2 = x2.contiguous()
    if flags & ROPE:
        cos, sin = _f32c(cos, "cos"), _f32c(sin, "sin")
        assert cos.shape[0] >= T and cos.shape[1] == D // 2
    ve_args = (None, 0, None)
    if ve is not None:
        if ve_gate_logit is None or not (ve_gate_logit.is_cuda and ve_gate_logit.dtype == torch.float32 and ve_gate_logit.numel() == 1):
            raise ValueError("ve needs ve_gate_logit, a float32 scalar CUDA tensor")
        ve2 = ve.reshape(B * T, H * D)
        _req(ve2, "ve")
        ve_args = (ve2.data_ptr(), ve2.stride(0), ve_gate_logit.data_ptr())
    outs = [torch.empty(B, T, H, D, dtype=torch.bfloat16, device=x.device) for _ in range(3)]
    ring_args = (None, None, 0, 0, 0, 0, 0)
    if ring is not None:
        rk, rv = ring
        f16 = rk.dtype == torch.float16
        _req(rk, "ring k", rk.dtype if f16 else torch.bfloat16); _req(rv, "ring v", rk.dtype)
        if rk.shape != rv.shape or rk.stride() != rv.stride() or rk.shape[0] != B or rk.shape[1] != H or rk.shape[3] != D:
            raise ValueError(f"ring tensors must both be [{B}, {H}, cap, {D}] with equal strides")
        ring_args = (rk.data_ptr(), rv.data_ptr(), rk.stride(0), rk.stride(1), rk.stride(2), rk.shape[2], int(ring_first))
        flags = flags | (_lib.CACHE_FP16 if f16 else 0)
    rc = _lib.lib().daisy_b200_qkv_gemm_ring(
        x2.data_ptr(), x2.stride(0), w_qkv.data_ptr(), w_qkv.stride(0),
        cos.data_ptr() if cos is not None else None, sin.data_ptr() if sin is not None else None,
        outs[0].data_ptr(), outs[1].data_ptr(), outs[2].data_ptr(), *ve_args, *ring_args, B, T, H, D, dim, eps, flags,
        status_word(x.device).data_ptr(), _stream(x))
    _lib.check(rc, "daisy_b200_qkv_gemm_ring")
    return tuple(outs)


def gemm_nt(x, w):
    """``x [..., K] @ w[N, K]^T`` in bf16 with fp32 accumulation (``F.linear(x, w)``) on the tcgen05 GEMM kernel."""
    _req(x, "x"); _req(w, "w")
    K = x.shape[-1]
    x2 = x.reshape(-1, K)
    if x2.stride(1) != 1:
        x2 = x2.contiguous()
    M, N = x2.shape[0], w.shape[0]
    c = torch.empty(M, N, dtype=torch.bfloat16, device=x.device)
    rc = _lib.lib().daisy_b200_gemm_nt(x2.data_ptr(), x2.stride(0), w.data_ptr(), w.stride(0), c.data_ptr(), c.stride(0),
                                       M, N, K, status_word(x.device).data_ptr(), _stream(x))
    _lib.check(rc, "daisy_b200_gemm_nt")
    return c.view(*x.shape[:-1], N)


def gemm_skinny(x, w, out: Optional[torch.Tensor] = None):
    """``F.linear(x, w)`` for at most 64 rows (a decode step's projections): weight-streaming kernel, bf16 in and out."""
    _req(x, "x"); _req(w, "w")
    K = x.shape[-1]
    x2 = x.reshape(-1, K)
    if x2.stride(1) != 1:
        x2 = x2.contiguous()
    M, N = x2.shape[0], w.shape[0]
    if out is None:
        out = torch.empty(*x.shape[:-1], N, dtype=torch.bfloat16, device=x.device)
    y2 = out.view(M, N)
    rc = _lib.lib().daisy_b200_gemm_skinny(x2.data_ptr(), x2.stride(0), w.data_ptr(), w.stride(0), y2.data_ptr(), y2.stride(0),
                                           M, N, K, _stream(x))
    _lib.check(rc, "daisy_b200_gemm_skinny")
    return out


def _doc_arg(doc_start: Optional[torch.Tensor], B: int, T: int, device):
    """``doc_start`` ([T] shared by the batch, or [B,T]) -> (int32 contiguous tensor or None, pointer, batch stride)."""
    if doc_start is None:
        return None, None, 0
    if not doc_start.is_cuda:
        raise ValueError("doc_start must be a CUDA tensor")
    d = doc_start.to(device=device, dtype=torch.int32).contiguous()
    if d.dim() == 1 and d.shape[0] == T:
        return d, d.data_ptr(), 0
    if d.dim() == 2 and d.shape == (B, T):
        return d, d.data_ptr(), T
    raise ValueError(f"doc_start must have shape [{T}] or [{B},{T}], got {tuple(d.shape)}")


def swa_attend(q, k, v, window: Optional[int], scale: float = ATTN_SCALE,
               out: Optional[torch.Tensor] = None, bounded_qk: bool = False,
               doc_start: Optional[torch.Tensor] = None, window_in_blocks: bool = False, return_lse: bool = False):
    """Windowed causal attention on prepared tensors of logical shape ``[B,T,H,D]`` (any batch / token /
    head strides, D contiguous); returns ``[B,T,H,D]``.  ``bounded_qk=True`` promises RMS-normalised q and k
    (every logit bounded), which selects the kernel without a running maximum.  ``doc_start`` (int, ``[T]`` or
    ``[B,T]``): first position of each token's document; keys before it are masked.  ``window_in_blocks``:
    ``window`` counts blocks of 128 tokens (key block >= query block - window + 1), the training-form mask.
    ``return_lse``: also return ``lse2 [B,H,T]`` float32 (base-2 log of each row's softmax denominator), what
    :func:`swa_attend_bwd` needs."""
    for n, t in (("q", q), ("k", k), ("v", v)):
        _req(t, n)
    B, T, H, D = q.shape
    assert k.shape == q.shape and v.shape == q.shape
    if out is None:
        out = torch.empty(B, T, H, D, dtype=torch.bfloat16, device=q.device)
    _doc, doc_ptr, doc_sb = _doc_arg(doc_start, B, T, q.device)
    if return_lse:
        lse = torch.empty(B, H, T, dtype=torch.float32, device=q.device)
        rc = _lib.lib().daisy_b200_swa_attend_lse(
            q.data_ptr(), k.data_ptr(), v.data_ptr(),
            q.stride(0), q.stride(1), q.stride(2), k.stride(0), k.stride(1), k.stride(2),
            v.stride(0), v.stride(1), v.stride(2), out.data_ptr(),
            out.stride(0), out.stride(1), out.stride(2), lse.data_ptr(), B, T, H, D, int(window or 0), scale, doc_ptr, doc_sb,
            (_lib.BOUNDED_QK if bounded_qk else 0) | (_lib.WINDOW_BLOCKS if window_in_blocks else 0),
            status_word(q.device).data_ptr(), _stream(q))
        _lib.check(rc, "daisy_b200_swa_attend_lse")
        return out, lse
    rc = _lib.lib().daisy_b200_swa_attend(
        q.data_ptr(), k.data_ptr(), v.data_ptr(),
        q.stride(0), q.stride(1), q.stride(2), k.stride(0), k.stride(1), k.stride(2),
        v.stride(0), v.stride(1), v.stride(2), out.data_ptr(),
        out.stride(0), out.stride(1), out.stride(2), B, T, H, D, int(window or 0), scale, doc_ptr, doc_sb,
        (_lib.BOUNDED_QK if bounded_qk else 0) | (_lib.WINDOW_BLOCKS if window_in_blocks else 0),
        status_word(q.device).data_ptr(), _stream(q))
    _lib.check(rc, "daisy_b200_swa_attend")
    return out


def swa_attend_bwd(q, k, v, o, d_o, lse2, window: Optional[int], scale: float = ATTN_SCALE,
                   doc_start: Optional[torch.Tensor] = None, window_in_blocks: bool = False):
    """Gradients of :func:`swa_attend` w.r.t. its prepared inputs: ``(dq, dk, dv)``, each ``[B,T,H,D]`` bf16 contiguous.
    ``q, k, v, o, d_o`` logical ``[B,T,H,D]`` (any strides, D contiguous); ``lse2`` from ``swa_attend(...,
    return_lse=True)``.  Deterministic (no atomics)."""
    for n, t in (("q", q), ("k", k), ("v", v), ("o", o), ("d_o", d_o)):
        _req(t, n)
    B, T, H, D = q.shape
    lse2 = _f32c(lse2, "lse2")
    assert lse2.shape == (B, H, T)
    dq, dk, dv = (torch.empty(B, T, H, D, dtype=torch.bfloat16, device=q.device) for _ in range(3))
    L = _lib.lib()
    ws = torch.empty(L.daisy_b200_swa_attend_bwd_workspace_bytes(B, T, H), dtype=torch.uint8, device=q.device)
    _doc, doc_ptr, doc_sb = _doc_arg(doc_start, B, T, q.device)
    st = lambda t: (t.stride(0), t.stride(1), t.stride(2))
    rc = L.daisy_b200_swa_attend_bwd(
        q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), d_o.data_ptr(), *st(q), *st(k), *st(v), *st(o), *st(d_o),
        lse2.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), B, T, H, D, int(window or 0), scale, doc_ptr, doc_sb,
        _lib.WINDOW_BLOCKS if window_in_blocks else 0, ws.data_ptr(), ws.numel(), status_word(q.device).data_ptr(), _stream(q))
    _lib.check(rc, "daisy_b200_swa_attend_bwd")
    return dq, dk, dv


def qkv_prep_bwd(q, k, v, cos, sin, dq_p, dk_p, dv_p, eps: float, flags: int = QKV_DEFAULT):
    """Backward of :func:`qkv_prep` (without a value embedding): raw ``q, k, v`` ``[B,T,H,D]`` (any strides) and the
    gradients w.r.t. the prepared tensors (``[B,T,H,D]`` contiguous) -> gradients w.r.t. the raw tensors."""
    for n, t in (("q", q), ("k", k), ("v", v), ("dq_p", dq_p), ("dk_p", dk_p), ("dv_p", dv_p)):
        _req(t, n)
    B, T, H, D = q.shape
    for t in (dq_p, dk_p, dv_p):
        assert t.shape == (B, T, H, D) and t.is_contiguous()
    if flags & ROPE:
        cos, sin = _f32c(cos, "cos"), _f32c(sin, "sin")
    outs = [torch.empty(B, T, H, D, dtype=torch.bfloat16, device=q.device) for _ in range(3)]
    st = lambda t: (t.stride(0), t.stride(1), t.stride(2))
    rc = _lib.lib().daisy_b200_qkv_prep_bwd(
        q.data_ptr(), k.data_ptr(), v.data_ptr(), *st(q), *st(k), *st(v), cos.data_ptr() if cos is not None else None,
        sin.data_ptr() if sin is not None else None, dq_p.data_ptr(), dk_p.data_ptr(), dv_p.data_ptr(),
        outs[0].data_ptr(), outs[1].data_ptr(), outs[2].data_ptr(), B, T, H, D, eps, flags, _stream(q))
    _lib.check(rc, "daisy_b200_qkv_prep_bwd")
    return tuple(outs)


def swa_prefill(q, k, v, cos, sin, window: Optional[int], scale: float = ATTN_SCALE, eps: float = 1.1920929e-07,
                flags: int = QKV_DEFAULT, workspace: Optional[torch.Tensor] = None,
                out: Optional[torch.Tensor] = None, k_out=None, v_out=None,
                doc_start: Optional[torch.Tensor] = None, window_in_blocks: bool = False
                ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Raw projections ``[B,T,H,D]`` -> ``(y [B,T,H,D], k' [B,H,T,D], v' [B,H,T,D])``.  Like the reference's
    ``prefill`` the returned k', v' are ``[B,H,T,D]``-shaped views of ``[B,T,H,D]`` memory; pass
    ``k_out``/``v_out`` as ``[B,T,H,D]`` contiguous buffers to reuse storage."""
    for n, t in (("q", q), ("k", k), ("v", v)):
        _req(t, n)
    B, T, H, D = q.shape
    cos, sin = _f32c(cos, "cos"), _f32c(sin, "sin")
    assert cos.shape[0] >= T and cos.shape[1] == D // 2
    L = _lib.lib()
    need = L.daisy_b200_swa_prefill_workspace_bytes(B, T, H, D)
    if workspace is None:
        workspace = torch.empty(need, dtype=torch.uint8, device=q.device)
    if out is None:
        out = torch.empty(B, T, H, D, dtype=torch.bfloat16, device=q.device)
    if k_out is None:
        k_out = torch.empty(B, T, H, D, dtype=torch.bfloat16, device=q.device)
    if v_out is None:
        v_out = torch.empty(B, T, H, D, dtype=torch.bfloat16, device=q.device)
    assert k_out.shape == (B, T, H, D) and k_out.is_contiguous() and v_out.shape == (B, T, H, D) and v_out.is_contiguous()
    _doc, doc_ptr, doc_sb = _doc_arg(doc_start, B, T, q.device)
    rc = L.daisy_b200_swa_prefill_fwd(
        q.data_ptr(), k.data_ptr(), v.data_ptr(),
        q.stride(0), q.stride(1), q.stride(2), k.stride(0), k.stride(1), k.stride(2),
        v.stride(0), v.stride(1), v.stride(2), cos.data_ptr(), sin.data_ptr(),
        out.data_ptr(), out.stride(0), out.stride(1), out.stride(2), k_out.data_ptr(), v_out.data_ptr(),
        B, T, H, D, int(window or 0), scale, eps, doc_ptr, doc_sb,
        flags | (_lib.WINDOW_BLOCKS if window_in_blocks else 0), workspace.data_ptr(), workspace.numel(),
        status_word(q.device).data_ptr(), _stream(q))
    _lib.check(rc, "daisy_b200_swa_prefill_fwd")
    return out, k_out.transpose(1, 2), v_out.transpose(1, 2)


def decode_splits(B: int, H: int, ctx_rows: int) -> int:
    L = _lib.lib()
    return L.daisy_b200_swa_decode_splits(B, H, ctx_rows, L.daisy_b200_sm_count())


def swa_decode_step(q_new, k_new, v_new, kcache, vcache, t: int, cap: int, window: Optional[int],
                    cos_row, sin_row, scale: float = ATTN_SCALE, eps: float = 1.1920929e-07,
                    flags: int = QKV_DEFAULT, write_ring: bool = False, splits: Optional[int] = None,
                    workspace: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
                    return_new_kv: bool = True):
    """One decode step.  ``q_new,k_new,v_new`` raw ``[B,1,H,D]``; ``kcache,vcache`` logical ``[B,H,cap,D]``
    (any batch/head/row strides, D contiguous) holding token p in row ``p % cap``; ``t`` tokens are in it.
    Returns ``(y [B,1,H,D], k' [B,1,H,D] or None, v' or None)``."""
    for n, x in (("q_new", q_new), ("k_new", k_new), ("v_new", v_new)):
        _req(x, n)
    B, one, H, D = q_new.shape
    assert one == 1
    L = _lib.lib()
    r = min(t, cap)
    if window is not None and window > 0:
        r = min(r, window - 1)
    if splits is None:
        splits = decode_splits(B, H, r)
    need = L.daisy_b200_swa_decode_workspace_bytes(B, H, D, splits)
    if workspace is None:
        workspace = torch.empty(need, dtype=torch.uint8, device=q_new.device)
    if out is None:
        out = torch.empty(B, 1, H, D, dtype=torch.bfloat16, device=q_new.device)
    k_o = torch.empty(B, 1, H, D, dtype=torch.bfloat16, device=q_new.device) if return_new_kv else None
    v_o = torch.empty(B, 1, H, D, dtype=torch.bfloat16, device=q_new.device) if return_new_kv else None
    cache_f16 = kcache is not None and kcache.dtype == torch.float16
    if kcache is not None:
        _req(kcache, "kcache", kcache.dtype if cache_f16 else torch.bfloat16)
        _req(vcache, "vcache", kcache.dtype if cache_f16 else torch.bfloat16)
        assert kcache.shape == vcache.shape and kcache.stride() == vcache.stride()
        kc_ptr, vc_ptr = kcache.data_ptr(), vcache.data_ptr()
        c_sb, c_sh, c_sr = kcache.stride(0), kcache.stride(1), kcache.stride(2)
    else:
        kc_ptr = vc_ptr = None
        c_sb = c_sh = c_sr = 0
    if flags & ROPE:
        cos_row, sin_row = _f32c(cos_row, "cos_row"), _f32c(sin_row, "sin_row")
    f = flags | (WRITE_RING if write_ring else 0) | (_lib.CACHE_FP16 if cache_f16 else 0)
    rc = L.daisy_b200_swa_decode_step(
        q_new.data_ptr(), k_new.data_ptr(), v_new.data_ptr(),
        q_new.stride(0), q_new.stride(2), k_new.stride(0), k_new.stride(2), v_new.stride(0), v_new.stride(2),
        kc_ptr, vc_ptr, c_sb, c_sh, c_sr, int(t), int(cap), int(window or 0),
        cos_row.data_ptr() if cos_row is not None else None, sin_row.data_ptr() if sin_row is not None else None,
        out.data_ptr(), out.stride(0), out.stride(2),
        k_o.data_ptr() if k_o is not None else None, v_o.data_ptr() if v_o is not None else None,
        B, H, D, scale, eps, f, workspace.data_ptr(), workspace.numel(), splits,
        status_word(q_new.device).data_ptr(), _stream(q_new))
    _lib.check(rc, "daisy_b200_swa_decode_step")
    return out, k_o, v_o


def swa_decode_step_dev(q_new, k_new, v_new, kcache, vcache, t_dev: torch.Tensor, cap: int, window: Optional[int],
                        cos_table, sin_table, scale: float = ATTN_SCALE, eps: float = 1.1920929e-07,
                        flags: int = QKV_DEFAULT, write_ring: bool = True, splits: Optional[int] = None,
                        workspace: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None):
    """:func:`swa_decode_step` with the position in device memory (``t_dev``: int64 tensor of one element), so the
    launch can sit inside a CUDA graph and be replayed for every token.  ``cos_table, sin_table`` are whole
    ``[rows, D/2]`` tables; the kernels pick row ``t_dev[0]``.  Returns ``y [B,1,H,D]``."""
    for n, x in (("q_new", q_new), ("k_new", k_new), ("v_new", v_new)):
        _req(x, n)
    cache_f16 = kcache.dtype == torch.float16
    _req(kcache, "kcache", kcache.dtype if cache_f16 else torch.bfloat16)
    _req(vcache, "vcache", kcache.dtype if cache_f16 else torch.bfloat16)
    if not (t_dev.is_cuda and t_dev.dtype == torch.int64 and t_dev.numel() == 1):
        raise ValueError("t_dev must be an int64 CUDA tensor with one element")
    B, one, H, D = q_new.shape
    assert one == 1 and kcache.shape == vcache.shape and kcache.stride() == vcache.stride()
    cos_table, sin_table = _f32c(cos_table, "cos_table"), _f32c(sin_table, "sin_table")
    L = _lib.lib()
    r = cap if not window else min(cap, window - 1)
    if splits is None:
        splits = decode_splits(B, H, r)
    need = L.daisy_b200_swa_decode_workspace_bytes(B, H, D, splits)
    if workspace is None:
        workspace = torch.empty(need, dtype=torch.uint8, device=q_new.device)
    if out is None:
        out = torch.empty(B, 1, H, D, dtype=torch.bfloat16, device=q_new.device)
    rc = L.daisy_b200_swa_decode_step_dev(
        q_new.data_ptr(), k_new.data_ptr(), v_new.data_ptr(),
        q_new.stride(0), q_new.stride(2), k_new.stride(0), k_new.stride(2), v_new.stride(0), v_new.stride(2),
        kcache.data_ptr(), vcache.data_ptr(), kcache.stride(0), kcache.stride(1), kcache.stride(2),
        t_dev.data_ptr(), int(cap), int(window or 0), cos_table.data_ptr(), sin_table.data_ptr(), cos_table.shape[0],
        out.data_ptr(), out.stride(0), out.stride(2), None, None,
        B, H, D, scale, eps, flags | (WRITE_RING if write_ring else 0) | (_lib.CACHE_FP16 if cache_f16 else 0),
        workspace.data_ptr(), workspace.numel(), splits,
        status_word(q_new.device).data_ptr(), _stream(q_new))
    _lib.check(rc, "daisy_b200_swa_decode_step_dev")
    return out


def decode_fused_workspace(B: int, H: int, D: int, splits: int, device) -> torch.Tensor:
    """Workspace of :func:`swa_decode_step_fused`, zero-filled: its tail holds one ticket per (batch, head) that must
    be zero before the first call (every call leaves it zero)."""
    n = _lib.lib().daisy_b200_swa_decode_fused_workspace_bytes(B, H, D, splits)
    return torch.zeros(n, dtype=torch.uint8, device=device)


def swa_decode_step_fused(q_new, k_new, v_new, kcache, vcache, t, cap: int, window: Optional[int], cos, sin,
                          scale: float = ATTN_SCALE, eps: float = 1.1920929e-07, flags: int = QKV_DEFAULT,
                          write_ring: bool = True, splits: Optional[int] = None, workspace: Optional[torch.Tensor] = None,
                          out: Optional[torch.Tensor] = None, ve: Optional[torch.Tensor] = None,
                          ve_gate_logit: Optional[torch.Tensor] = None, return_new_kv: bool = False):
    """The decode step as one launch.  ``t``: an int (``cos, sin`` are then the table rows of the position) or an
    int64 CUDA tensor of one element (``cos, sin`` are whole tables, the kernels pick row ``t[0]``).  ``ve``
    ``[B,1,H,D]`` with ``ve_gate_logit`` mixes the value embedding into the new token's normalised v.  ``workspace``
    must come from :func:`decode_fused_workspace` (zeroed tickets).  ``kcache`` may be None (no context yet, nothing
    to store).  Returns ``y [B,1,H,D]``, or ``(y, k', v')`` with ``return_new_kv``."""
    for n, x in (("q_new", q_new), ("k_new", k_new), ("v_new", v_new)):
        _req(x, n)
    B, one, H, D = q_new.shape
    assert one == 1
    cache_f16 = kcache is not None and kcache.dtype == torch.float16
    if kcache is not None:
        _req(kcache, "kcache", kcache.dtype if cache_f16 else torch.bfloat16)
        _req(vcache, "vcache", kcache.dtype if cache_f16 else torch.bfloat16)
        assert kcache.shape == vcache.shape and kcache.stride() == vcache.stride()
        c_args = (kcache.data_ptr(), vcache.data_ptr(), kcache.stride(0), kcache.stride(1), kcache.stride(2))
    else:
        c_args = (None, None, 0, 0, 0)
    on_dev = isinstance(t, torch.Tensor)
    if on_dev and not (t.is_cuda and t.dtype == torch.int64 and t.numel() == 1):
        raise ValueError("a device-side position must be an int64 CUDA tensor with one element")
    cos, sin = _f32c(cos, "cos"), _f32c(sin, "sin")
    L = _lib.lib()
    r = min(cap, int(t)) if not on_dev else cap
    if window:
        r = min(r, window - 1)
    if splits is None:
        splits = decode_splits(B, H, r)
    if workspace is None:
        workspace = decode_fused_workspace(B, H, D, splits, q_new.device)
    if out is None:
        out = torch.empty(B, 1, H, D, dtype=torch.bfloat16, device=q_new.device)
    ve_args = (None, 0, 0, None)
    if ve is not None:
        ve = ve.view(B, 1, H, D)
        _req(ve, "ve")
        if ve_gate_logit is None or not (ve_gate_logit.is_cuda and ve_gate_logit.dtype == torch.float32 and ve_gate_logit.numel() == 1):
            raise ValueError("ve needs ve_gate_logit, a float32 scalar CUDA tensor")
        ve_args = (ve.data_ptr(), ve.stride(0), ve.stride(2), ve_gate_logit.data_ptr())
    k_o = torch.empty(B, 1, H, D, dtype=torch.bfloat16, device=q_new.device) if return_new_kv else None
    v_o = torch.empty(B, 1, H, D, dtype=torch.bfloat16, device=q_new.device) if return_new_kv else None
    rc = L.daisy_b200_swa_decode_step_fused(
        q_new.data_ptr(), k_new.data_ptr(), v_new.data_ptr(),
        q_new.stride(0), q_new.stride(2), k_new.stride(0), k_new.stride(2), v_new.stride(0), v_new.stride(2),
        *c_args,
        0 if on_dev else int(t), t.data_ptr() if on_dev else None, int(cap), int(window or 0),
        cos.data_ptr(), sin.data_ptr(), cos.shape[0] if on_dev else 0,
        out.data_ptr(), out.stride(0), out.stride(2), k_o.data_ptr() if return_new_kv else None,
        v_o.data_ptr() if return_new_kv else None, *ve_args,
        B, H, D, scale, eps, flags | (WRITE_RING if write_ring else 0) | (_lib.CACHE_FP16 if cache_f16 else 0),
        workspace.data_ptr(), workspace.numel(), splits, status_word(q_new.device).data_ptr(), _stream(q_new))
    _lib.check(rc, "daisy_b200_swa_decode_step_fused")
    return (out, k_o, v_o) if return_new_kv else out


def ring_copy_rows(ring_bhcd, lin_bhnd, first_pos: int, to_ring: bool) -> None:
    """Copy rows between a ring ``[B,H,cap,D]`` and a chronological ``[B,H,n,D]`` tensor (any strides
    with D contiguous): row i of ``lin`` <-> ring row ``(first_pos + i) % cap``."""
    assert ring_bhcd.is_cuda and lin_bhnd.is_cuda and ring_bhcd.dtype == lin_bhnd.dtype
    assert ring_bhcd.stride(-1) == 1 and lin_bhnd.stride(-1) == 1
    B, H, cap, D = ring_bhcd.shape
    n = lin_bhnd.shape[2]
    assert lin_bhnd.shape == (B, H, n, D)
    rc = _lib.lib().daisy_b200_ring_copy_rows(
        ring_bhcd.data_ptr(), ring_bhcd.stride(0), ring_bhcd.stride(1), ring_bhcd.stride(2),
        lin_bhnd.data_ptr(), lin_bhnd.stride(0), lin_bhnd.stride(1), lin_bhnd.stride(2),
        B, H, D, cap, int(first_pos), n, ring_bhcd.element_size(), 1 if to_ring else 0, _stream(ring_bhcd))
    _lib.check(rc, "daisy_b200_ring_copy_rows")


def kda_chunk_fwd(q, k, v, g, beta, scale: Optional[float] = None, initial_state=None,
                  output_final_state: bool = False, l2norm_qk: bool = True, out_fp32: bool = False):
    """KDA chunked forward.  ``q,k [B,T,H,K]`` ``v [B,T,H,V]`` bf16; ``g [B,T,H,K]`` fp32 log-decay; ``beta
    [B,T,H]`` fp32; state ``[B,H,K,V]`` fp32.  Returns ``(o [B,T,H,V], final_state or None)``."""
    for n, t in (("q", q), ("k", k), ("v", v)):
        _req(t, n)
        if not t.is_contiguous():
            raise ValueError(f"{n} must be contiguous")
    g, beta = _f32c(g, "g"), _f32c(beta, "beta")
    B, T, H, K = q.shape
    V = v.shape[-1]
    L = _lib.lib()
    o = torch.empty(B, T, H, V, dtype=torch.float32 if out_fp32 else torch.bfloat16, device=q.device)
    hT = torch.empty(B, H, K, V, dtype=torch.float32, device=q.device) if output_final_state else None
    if initial_state is not None:
        initial_state = _f32c(initial_state, "initial_state")
    need = L.daisy_b200_kda_workspace_bytes(B, T, H, K, V)
    ws = torch.empty(max(need, 16), dtype=torch.uint8, device=q.device)
    flags = (KDA_L2NORM_QK if l2norm_qk else 0) | (KDA_OUT_FP32 if out_fp32 else 0)
    rc = L.daisy_b200_kda_chunk_fwd(
        q.data_ptr(), k.data_ptr(), v.data_ptr(), g.data_ptr(), beta.data_ptr(),
        initial_state.data_ptr() if initial_state is not None else None, o.data_ptr(),
        hT.data_ptr() if hT is not None else None, B, T, H, K, V, 64,
        float(scale) if scale is not None else 0.0, flags, ws.data_ptr(), ws.numel(),
        status_word(q.device).data_ptr(), _stream(q))
    _lib.check(rc, "daisy_b200_kda_chunk_fwd")
    return o, hT


def kda_varlen_tables(cu_seqlens, device, chunk: int = 64):
    """Chunk and token tables of a packed batch, from its ``cu_seqlens`` (N + 1 offsets, host integers or a tensor --
    a tensor costs one device-to-host read, as the reference's own chunk-index preparation does).  Returns
    ``(chunk_tab [n_chunks, 2], seq_ptr [N + 1], tok_tab [T_total, 2], n_chunks)`` as int32 device tensors: first token
    and length of every chunk, the first chunk of every sequence, and for every token its sequence's first token and
    number."""
    cu = [int(c) for c in (cu_seqlens.tolist() if torch.is_tensor(cu_seqlens) else cu_seqlens)]
    if len(cu) < 2 or cu[0] != 0 or any(b < a for a, b in zip(cu, cu[1:])):
        raise ValueError("cu_seqlens must start at 0 and not decrease")
    chunks, ptr, tok = [], [0], []
    for n, (a, b) in enumerate(zip(cu, cu[1:])):
        chunks.extend((t, min(chunk, b - t)) for t in range(a, b, chunk))
        ptr.append(len(chunks))
        tok.extend((a, n) for _ in range(b - a))
    mk = lambda rows, w: torch.tensor(rows, dtype=torch.int32).reshape(-1, w).to(device)
    return mk(chunks, 2), torch.tensor(ptr, dtype=torch.int32, device=device), mk(tok, 2), len(chunks)


def kda_chunk_fwd_varlen(q, k, v, g, beta, cu_seqlens, scale: Optional[float] = None, initial_state=None,
                         output_final_state: bool = False, l2norm_qk: bool = True, out_fp32: bool = False, tables=None):
    """KDA chunked forward over packed sequences: ``q,k [1,T,H,K]``, ``v [1,T,H,V]`` bf16, ``g`` fp32, ``beta [1,T,H]``,
    ``cu_seqlens`` the N + 1 sequence offsets; state ``[N,H,K,V]`` fp32.  ``tables``: the result of
    :func:`kda_varlen_tables` when the caller already has it."""
    for n, t in (("q", q), ("k", k), ("v", v)):
        _req(t, n)
        if not t.is_contiguous():
            raise ValueError(f"{n} must be contiguous")
    if q.shape[0] != 1:
        raise ValueError("packed sequences come as one row: q must be [1, T_total, H, K]")
    g, beta = _f32c(g, "g"), _f32c(beta, "beta")
    _, T, H, K = q.shape
    V = v.shape[-1]
    chunk_tab, seq_ptr, _tok, n_chunks = tables if tables is not None else kda_varlen_tables(cu_seqlens, q.device)
    N = seq_ptr.numel() - 1
    if int(_tok.shape[0]) != T:
        raise ValueError(f"cu_seqlens covers {int(_tok.shape[0])} tokens, the inputs hold {T}")
    L = _lib.lib()
    o = torch.empty(1, T, H, V, dtype=torch.float32 if out_fp32 else torch.bfloat16, device=q.device)
    if initial_state is not None:
        initial_state = _f32c(initial_state, "initial_state")
        if tuple(initial_state.shape) != (N, H, K, V):
            raise ValueError(f"initial_state must be [{N}, {H}, {K}, {V}]")
    hT = torch.empty(N, H, K, V, dtype=torch.float32, device=q.device) if output_final_state else None
    if T == 0 or n_chunks == 0:
        if hT is not None:
            hT.copy_(initial_state) if initial_state is not None else hT.zero_()
        return o, hT
    need = L.daisy_b200_kda_varlen_workspace_bytes(n_chunks, H, K, V)
    ws = torch.empty(max(need, 16), dtype=torch.uint8, device=q.device)
    flags = (KDA_L2NORM_QK if l2norm_qk else 0) | (KDA_OUT_FP32 if out_fp32 else 0)
    rc = L.daisy_b200_kda_chunk_fwd_varlen(
        q.data_ptr(), k.data_ptr(), v.data_ptr(), g.data_ptr(), beta.data_ptr(),
        initial_state.data_ptr() if initial_state is not None else None, o.data_ptr(),
        hT.data_ptr() if hT is not None else None, T, H, K, V, 64,
        float(scale) if scale is not None else 0.0, flags, chunk_tab.data_ptr(), n_chunks, seq_ptr.data_ptr(), N,
        ws.data_ptr(), ws.numel(), status_word(q.device).data_ptr(), _stream(q))
    _lib.check(rc, "daisy_b200_kda_chunk_fwd_varlen")
    return o, hT


def kda_recurrent_fwd(q, k, v, g, beta, scale: Optional[float] = None, initial_state=None,
                      output_final_state: bool = False, l2norm_qk: bool = True, out_fp32: bool = False,
                      state_in_place: bool = False):
    """KDA token-by-token recurrence (short inputs, decode steps); same arguments and layouts as
    :func:`kda_chunk_fwd`.  ``state_in_place=True`` updates ``initial_state`` itself and returns it."""
    for n, t in (("q", q), ("k", k), ("v", v)):
        _req(t, n)
        if not t.is_contiguous():
            raise ValueError(f"{n} must be contiguous")
    g, beta = _f32c(g, "g"), _f32c(beta, "beta")
    B, T, H, K = q.shape
    V = v.shape[-1]
    o = torch.empty(B, T, H, V, dtype=torch.float32 if out_fp32 else torch.bfloat16, device=q.device)
    if initial_state is not None:
        if state_in_place and not (initial_state.dtype == torch.float32 and initial_state.is_contiguous()):
            raise ValueError("an in-place state must be a contiguous float32 tensor")
        initial_state = _f32c(initial_state, "initial_state")
    if state_in_place:
        if initial_state is None:
            raise ValueError("state_in_place needs an initial_state")
        hT = initial_state
    else:
        hT = torch.empty(B, H, K, V, dtype=torch.float32, device=q.device) if output_final_state else None
    flags = (KDA_L2NORM_QK if l2norm_qk else 0) | (KDA_OUT_FP32 if out_fp32 else 0)
    rc = _lib.lib().daisy_b200_kda_recurrent_fwd(
        q.data_ptr(), k.data_ptr(), v.data_ptr(), g.data_ptr(), beta.data_ptr(),
        initial_state.data_ptr() if initial_state is not None else None, o.data_ptr(),
        hT.data_ptr() if hT is not None else None, B, T, H, K, V,
        float(scale) if scale is not None else 0.0, flags, _stream(q))
    _lib.check(rc, "daisy_b200_kda_recurrent_fwd")
    return o, hT


def kda_gate(g: torch.Tensor, a_log: torch.Tensor, head_k_dim: int, g_bias: Optional[torch.Tensor] = None,
             beta: float = 1.0, threshold: float = 20.0, round_bf16: Optional[bool] = None) -> torch.Tensor:
    """``-exp(A_log[h]) * softplus(g + bias)`` for ``g [..., H*D]`` (bf16 or fp32) -> fp32 ``[..., H, D]``.
    ``round_bf16`` (default: when ``g`` is bf16) rounds the values to bf16 before storing them as fp32, the
    reference's cast of the gate back to the activation dtype."""
    if not g.is_cuda:
        raise ValueError("g must be a CUDA tensor")
    if g.dtype not in (torch.bfloat16, torch.float32):
        g = g.float()
    g = g.contiguous()
    HD = g.shape[-1]
    H = HD // int(head_k_dim)
    if H * int(head_k_dim) != HD:
        raise ValueError("last dim must be divisible by head_k_dim")
    a = a_log.to(device=g.device, dtype=torch.float32).reshape(-1).contiguous()
    if a.numel() != H:
        raise ValueError(f"A_log must hold {H} values")
    bias = None
    if g_bias is not None:
        bias = g_bias.to(device=g.device, dtype=torch.float32)
        bias = (bias.reshape(H, 1).expand(H, head_k_dim) if bias.numel() == H else bias).reshape(-1).contiguous()
        if bias.numel() != HD:
            raise ValueError("g_bias must hold H or H*D values")
    if round_bf16 is None:
        round_bf16 = g.dtype == torch.bfloat16
    out = torch.empty(*g.shape[:-1], H, int(head_k_dim), dtype=torch.float32, device=g.device)
    rows = g.numel() // HD
    rc = _lib.lib().daisy_b200_kda_gate(g.data_ptr(), 1 if g.dtype == torch.bfloat16 else 0, a.data_ptr(),
                                        bias.data_ptr() if bias is not None else None, out.data_ptr(), rows, H,
                                        int(head_k_dim), float(beta), float(threshold),
                                        _lib.KDA_GATE_ROUND_BF16 if round_bf16 else 0, _stream(g))
    _lib.check(rc, "daisy_b200_kda_gate")
    return out


def kda_short_conv(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
                   state: Optional[torch.Tensor] = None, output_final_state: bool = False, silu: bool = True,
                   inplace_state: bool = False):
    """Causal depthwise convolution (+ SiLU) of ``x [B,T,C]`` bf16 with ``weight [C,W]`` (or the Conv1d layout
    ``[C,1,W]``), W <= 4.  ``state [B,C,W]`` holds the W inputs before ``x`` (oldest first).  Returns
    ``(y, final_state or None)``; with ``inplace_state`` (T <= 32 only) the final state overwrites ``state``."""
    _req(x, "x")
    if x.dim() != 3:
        raise ValueError("x must be [B, T, C]")
    if x.stride(2) != 1:
        x = x.contiguous()
    B, T, C = x.shape
    w = weight.reshape(C, -1)
    w = (w if w.dtype == torch.bfloat16 else w.to(torch.bfloat16)).contiguous()
    W = w.shape[1]
    if bias is not None:
        bias = bias.to(device=x.device, dtype=torch.bfloat16).contiguous()
    s_out = None
    if state is not None:
        if state.shape != (B, C, W) or state.dtype != torch.bfloat16 or not state.is_contiguous():
            raise ValueError(f"state must be a contiguous bf16 [{B}, {C}, {W}] tensor")
    if output_final_state:
        s_out = state if (inplace_state and state is not None) else torch.empty(B, C, W, dtype=torch.bfloat16, device=x.device)
    y = torch.empty(B, T, C, dtype=torch.bfloat16, device=x.device)
    rc = _lib.lib().daisy_b200_kda_short_conv(x.data_ptr(), x.stride(0), x.stride(1), w.data_ptr(),
                                              bias.data_ptr() if bias is not None else None,
                                              state.data_ptr() if state is not None else None,
                                              s_out.data_ptr() if s_out is not None else None,
                                              y.data_ptr(), y.stride(0), y.stride(1), B, T, C, W,
                                              _lib.KDA_CONV_SILU if silu else 0, _stream(x))
    _lib.check(rc, "daisy_b200_kda_short_conv")
    return y, s_out


def kda_short_conv_varlen(x: torch.Tensor, weight: torch.Tensor, tok_tab: torch.Tensor, n_seq: int,
                          bias: Optional[torch.Tensor] = None, state: Optional[torch.Tensor] = None,
                          output_final_state: bool = False, silu: bool = True):
    """:func:`kda_short_conv` over packed sequences ``x [1, T_total, C]``: the window stops at each sequence's first
    token.  ``tok_tab`` is the third table of :func:`kda_varlen_tables`; ``state`` and the returned final state are
    ``[n_seq, C, W]``."""
    _req(x, "x")
    if x.dim() != 3 or x.shape[0] != 1:
        raise ValueError("x must be [1, T_total, C]")
    if x.stride(2) != 1:
        x = x.contiguous()
    _, T, C = x.shape
    w = weight.reshape(C, -1)
    w = (w if w.dtype == torch.bfloat16 else w.to(torch.bfloat16)).contiguous()
    W = w.shape[1]
    if tok_tab.dtype != torch.int32 or tuple(tok_tab.shape) != (T, 2) or not tok_tab.is_contiguous():
        raise ValueError(f"tok_tab must be a contiguous int32 [{T}, 2] tensor")
    if bias is not None:
        bias = bias.to(device=x.device, dtype=torch.bfloat16).contiguous()
    if state is not None and (tuple(state.shape) != (n_seq, C, W) or state.dtype != torch.bfloat16 or not state.is_contiguous()):
        raise ValueError(f"state must be a contiguous bf16 [{n_seq}, {C}, {W}] tensor")
    s_out = None
    if output_final_state:       # sequences without tokens keep their state
        s_out = state.clone() if state is not None else torch.zeros(n_seq, C, W, dtype=torch.bfloat16, device=x.device)
    y = torch.empty(1, T, C, dtype=torch.bfloat16, device=x.device)
    if T == 0:
        return y, s_out
    rc = _lib.lib().daisy_b200_kda_short_conv_varlen(x.data_ptr(), x.stride(1), w.data_ptr(),
                                                     bias.data_ptr() if bias is not None else None,
                                                     state.data_ptr() if state is not None else None,
                                                     s_out.data_ptr() if s_out is not None else None,
                                                     y.data_ptr(), y.stride(1), T, C, W, tok_tab.data_ptr(),
                                                     _lib.KDA_CONV_SILU if silu else 0, _stream(x))
    _lib.check(rc, "daisy_b200_kda_short_conv_varlen")
    return y, s_out


def kda_out_norm(o: torch.Tensor, gate: torch.Tensor, weight: Optional[torch.Tensor] = None, eps: float = 1e-6,
                 mode: int = _lib.KDA_NORM_SWISH_SIGMOID, gate_bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Gated RMS norm over the last dimension (128) of ``o [..., H, 128]`` (bf16 or fp32) with the gate
    pre-activation ``gate`` (bf16, same shape); bf16 result of ``o``'s shape.  ``mode``: ``_lib.KDA_NORM_*``.
    ``gate_bias [H*128]``: added to the gate inside the kernel (the bias of the projection that produced it)."""
    if not o.is_cuda:
        raise ValueError("o must be a CUDA tensor")
    if o.dtype not in (torch.bfloat16, torch.float32):
        o = o.to(torch.bfloat16)
    o = o.contiguous()
    gate = gate.to(device=o.device, dtype=torch.bfloat16).contiguous()
    if gate.shape != o.shape:
        raise ValueError("gate must have the shape of o")
    D = o.shape[-1]
    if weight is not None:
        weight = weight.to(device=o.device, dtype=torch.bfloat16).contiguous()
    H = 1
    if gate_bias is not None:
        if o.dim() < 2 or gate_bias.numel() != o.shape[-2] * D:
            raise ValueError("gate_bias must hold H*D values for o [..., H, D]")
        H = o.shape[-2]
        gate_bias = gate_bias.to(device=o.device, dtype=torch.bfloat16).contiguous()
    y = torch.empty(o.shape, dtype=torch.bfloat16, device=o.device)
    rc = _lib.lib().daisy_b200_kda_out_norm(o.data_ptr(), 1 if o.dtype == torch.float32 else 0, gate.data_ptr(),
                                            gate_bias.data_ptr() if gate_bias is not None else None, H,
                                            weight.data_ptr() if weight is not None else None, y.data_ptr(),
                                            o.numel() // D, D, float(eps), int(mode), _stream(o))
    _lib.check(rc, "daisy_b200_kda_out_norm")
    return y


def selftest_umma(a: torch.Tensor, b: torch.Tensor, mode: int) -> torch.Tensor:
    """C[128,128] fp32 = A[128,K] x B (B is [128,K] for mode 0, [K,128] for modes 1 and 2)."""
    _req(a, "a"); _req(b, "b")
    K = a.shape[1]
    c = torch.zeros(128, 128, dtype=torch.float32, device=a.device)
    rc = _lib.lib().daisy_b200_selftest_umma(a.contiguous().data_ptr(), b.contiguous().data_ptr(), c.data_ptr(), K, mode,
                                             status_word(a.device).data_ptr(), _stream(a))
    _lib.check(rc, "daisy_b200_selftest_umma")
    return c
