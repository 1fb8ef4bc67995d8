"""Drop-in for the ``chunk_kda`` call of the reference's Kimi-delta-attention layer
(models/daisy/attention_kimi.py:133-134), same argument names and return convention:

    o, final_state = chunk_kda(q=q, k=k, v=v, g=g, beta=beta, initial_state=rec,
                               output_final_state=use_cache, use_qk_l2norm_in_kernel=True, cu_seqlens=None)

``q,k [B,T,H,K]`` and ``v [B,T,H,V]`` bf16, ``g [B,T,H,K]`` log-decay (any float dtype, used in fp32),
``beta [B,T,H]``, state ``[B,H,K,V]`` fp32; K = V = 128.  Runs the hand-written sm_100a kernels only.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import ops


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
    o, hT = ops.kda_chunk_fwd(q, k, v, g, beta, scale, initial_state, output_final_state,
                              l2norm_qk=use_qk_l2norm_in_kernel, out_fp32=out_fp32)
    return o, hT
