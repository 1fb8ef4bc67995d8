"""Drop-in for the ``chunk_kda`` call of the reference's Kimi-delta-attention layer
(models/daisy/attention_kimi.py:133-134), same argument names and return convention:

    o, final_state = chunk_kda(q=q, k=k, v=v, g=g, beta=beta, initial_state=rec,
                               output_final_state=use_cache, use_qk_l2norm_in_kernel=True, cu_seqlens=None)

``q,k [B,T,H,K]`` and ``v [B,T,H,V]`` bf16, ``g [B,T,H,K]`` log-decay (any float dtype, used in fp32),
``beta [B,T,H]``, state ``[B,H,K,V]`` fp32; K = V = 128.  Runs the hand-written sm_100a kernels only.
Inputs of at most ``RECURRENT_MAX_T`` tokens (decode steps: the reference calls the same function with T = 1
and the cached state, attention_kimi.py:144-149,175-180) take the token-by-token kernel, longer ones the
chunked pair.

``fused_kda_gate`` mirrors the gate call one line above it (attention_kimi.py:132; forward of
``_gate_impl``, models/daisy/fla_custom_ops.py:71-103).
"""
from __future__ import annotations

from typing import Optional

import torch

from . import ops

RECURRENT_MAX_T = 4      # up to this many tokens the state is carried token by token in registers


def chunk_kda(q, k, v, g, beta, scale: Optional[float] = None, initial_state: Optional[torch.Tensor] = None,
              output_final_state: bool = False, use_qk_l2norm_in_kernel: bool = False, cu_seqlens=None,
              out_fp32: bool = False):
    if cu_seqlens is not None:
        raise NotImplementedError("variable-length packing (cu_seqlens) is not implemented by the B200 KDA kernels")
    q, k, v = (x.contiguous() if x.dtype == torch.bfloat16 else x.to(torch.bfloat16).contiguous() for x in (q, k, v))
    g = g.float().contiguous()
    beta = beta.float().contiguous()
    if initial_state is not None:
        initial_state = initial_state.float().contiguous()
    fwd = ops.kda_recurrent_fwd if q.shape[1] <= RECURRENT_MAX_T else ops.kda_chunk_fwd
    o, hT = fwd(q, k, v, g, beta, scale, initial_state, output_final_state,
                l2norm_qk=use_qk_l2norm_in_kernel, out_fp32=out_fp32)
    return o, hT


def fused_kda_gate(g, A_log, head_k_dim: int, g_bias=None, b=None, beta: float = 1.0, threshold: float = 20.0):
    """``(y, b_sigmoid)`` like the reference op: ``y [..., H, D]`` = ``-exp(A_log) * softplus(g + g_bias)``
    in ``g.dtype`` (computed in fp32), ``b_sigmoid = sigmoid(b)`` or zeros ``[..., H]`` when ``b`` is None.
    ``chunk_kda`` takes the fp32 values; pass ``ops.kda_gate(...)`` directly to skip the cast back."""
    y32 = ops.kda_gate(g, A_log, head_k_dim, g_bias, beta, threshold)
    y = y32 if g.dtype == torch.float32 else y32.to(g.dtype)
    H = g.shape[-1] // int(head_k_dim)
    if b is None:
        b_sigmoid = torch.zeros(*g.shape[:-1], H, device=g.device, dtype=g.dtype)
    else:
        b_sigmoid = torch.sigmoid(b.to(device=g.device, dtype=g.dtype))
    return y, b_sigmoid
