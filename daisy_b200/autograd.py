"""The attention core under ``torch.autograd``: forward and backward on the B200 kernels.

``swa_attention(q, k, v, cos, sin, window, ...)`` takes the RAW projections ``[B,T,H,D]`` (views of the merged QKV
projection are fine) and returns the attention output ``[B,T,H,D]``; its backward runs
``daisy_b200_swa_attend_bwd`` (three launches, deterministic) and the norm / RoPE backward.  This is what the
reference gets from autograd through ``F.rms_norm``, ``_apply_rope`` and ``scaled_dot_product_attention`` /
``flex_attention`` inside ``CausalSelfAttention.forward`` during training (models/daisy/attention.py:116-127,
141-162).  The projections either side stay ordinary ``F.linear`` calls, so their weight and input gradients come
from autograd's own matmul rules.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import ops
from ._lib import NORM_Q, NORM_K, QKV_DEFAULT


class _SwaAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, cos, sin, window, scale, eps, flags, doc_start, window_in_blocks):
        qp, kp, vp = ops.qkv_prep(q, k, v, cos, sin, eps, flags)
        bounded = bool(flags & NORM_Q) and bool(flags & NORM_K)
        y, lse = ops.swa_attend(qp, kp, vp, window, scale, bounded_qk=bounded, doc_start=doc_start,
                                window_in_blocks=window_in_blocks, return_lse=True)
        ctx.save_for_backward(q, k, v, qp, kp, vp, y, lse, cos, sin, doc_start if doc_start is not None else torch.empty(0))
        ctx.args = (window, scale, eps, flags, doc_start is not None, window_in_blocks)
        return y

    @staticmethod
    def backward(ctx, dy):
        q, k, v, qp, kp, vp, y, lse, cos, sin, doc = ctx.saved_tensors
        window, scale, eps, flags, has_doc, in_blocks = ctx.args
        dy = dy.to(torch.bfloat16)
        if dy.stride(-1) != 1:
            dy = dy.contiguous()
        dqp, dkp, dvp = ops.swa_attend_bwd(qp, kp, vp, y, dy, lse, window, scale, doc_start=doc if has_doc else None,
                                           window_in_blocks=in_blocks)
        dq, dk, dv = ops.qkv_prep_bwd(q, k, v, cos, sin, dqp, dkp, dvp, eps, flags)
        return dq, dk, dv, None, None, None, None, None, None, None, None


def swa_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor,
                  window: Optional[int], scale: float = ops.ATTN_SCALE, eps: float = 1.1920929e-07,
                  flags: int = QKV_DEFAULT, doc_start: Optional[torch.Tensor] = None,
                  window_in_blocks: bool = False) -> torch.Tensor:
    """Differentiable ``rms_norm -> RoPE -> windowed causal softmax attention`` on raw ``[B,T,H,D]`` bf16 projections."""
    return _SwaAttention.apply(q, k, v, cos, sin, window, scale, eps, flags, doc_start, window_in_blocks)
