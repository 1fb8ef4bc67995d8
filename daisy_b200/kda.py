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


def smoke_kda() -> None:
    """One small KDA forward on cuda:0 against the fp32 token recurrence."""
    from oracle import kda as okda
    g_ = torch.Generator().manual_seed(0)
    B, T, H, K = 1, 160, 2, 128
    q, k, v = (torch.randn(B, T, H, K, generator=g_).bfloat16() for _ in range(3))
    g = torch.nn.functional.logsigmoid(torch.randn(B, T, H, K, generator=g_))
    beta = torch.sigmoid(torch.randn(B, T, H, generator=g_))
    o_ref, s_ref = okda.kda_recurrent(q.float(), k.float(), v.float(), g, beta)
    o, s = chunk_kda(q.cuda(), k.cuda(), v.cuda(), g.cuda(), beta.cuda(), output_final_state=True,
                     use_qk_l2norm_in_kernel=True, out_fp32=True)
    ops.check_device_status("cuda")
    rel = ((o.cpu() - o_ref).norm() / o_ref.norm()).item()
    rel_s = ((s.cpu() - s_ref).norm() / s_ref.norm()).item()
    assert rel < 1e-3 and rel_s < 1e-3, ("kda", rel, rel_s)
