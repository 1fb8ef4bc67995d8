"""CPU oracle: Kimi delta attention (KDA), token-by-token recurrence.

Test infrastructure only (see ``oracle/__init__.py``).

The reference calls ``fla.ops.kda.chunk_kda(q, k, v, g, beta, initial_state,
output_final_state, use_qk_l2norm_in_kernel=True, cu_seqlens)`` at
``models/daisy/attention_kimi.py:133-134``; the arithmetic is in the
third-party, unpinned ``flash-linear-attention`` package (0.5.1 in the build
container), not in the reference tree.  This file restates the published
recurrence of that operator:

    S      <- diag(exp(g_t)) S                     (per key channel decay, S in R^{K x V})
    u_t    =  beta_t (v_t - S^T k_t)
    S      <- S + k_t u_t^T
    o_t    =  S^T (scale * q_t)

with q, k L2-normalised over K when ``l2norm_qk`` (eps 1e-6 added to the squared
norm inside the square root, as the third-party kernel does), ``scale = K**-0.5`` by
default, layouts ``q,k,g [B,T,H,K]``, ``v,o [B,T,H,V]``, ``beta [B,T,H]``,
state ``[B,H,K,V]``.  It is checked against ``fla.ops.kda.naive.naive_recurrent_kda``
through the committed fixture ``tests/golden/kda_naive_small.npz``.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch


def l2norm(x: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    return x * torch.rsqrt(x.pow(2).sum(dim=-1, keepdim=True) + eps)


def kda_recurrent(q, k, v, g, beta, scale: Optional[float] = None,
                  initial_state: Optional[torch.Tensor] = None, l2norm_qk: bool = True,
                  dtype=torch.float32) -> Tuple[torch.Tensor, torch.Tensor]:
    """Returns ``(o [B,T,H,V], final_state [B,H,K,V])`` in ``dtype`` (fp32 or fp64)."""
    B, T, H, K = q.shape
    V = v.shape[-1]
    q, k, v, g, beta = (x.to(dtype) for x in (q, k, v, g, beta))
    if l2norm_qk:
        q, k = l2norm(q), l2norm(k)
    if scale is None:
        scale = K ** -0.5
    q = q * scale
    S = torch.zeros(B, H, K, V, dtype=dtype)
    if initial_state is not None:
        S = S + initial_state.to(dtype)
    o = torch.empty(B, T, H, V, dtype=dtype)
    for t in range(T):
        kt, vt, qt = k[:, t], v[:, t], q[:, t]                  # [B,H,K], [B,H,V]
        S = S * g[:, t].exp().unsqueeze(-1)
        u = beta[:, t].unsqueeze(-1) * (vt - torch.einsum("bhkv,bhk->bhv", S, kt))
        S = S + kt.unsqueeze(-1) * u.unsqueeze(-2)
        o[:, t] = torch.einsum("bhkv,bhk->bhv", S, qt)
    return o, S


def kda_gate(g: torch.Tensor, A_log: torch.Tensor, head_k_dim: int, g_bias: Optional[torch.Tensor] = None,
             beta: float = 1.0, threshold: float = 20.0) -> torch.Tensor:
    """Log-decay gate of the KDA layer, ``[..., H*D] -> [..., H, D]`` in ``g.dtype``:

        y = -exp(A_log[h]) * softplus(g + g_bias, beta, threshold)        (fp32 math, then cast)

    Restates ``_gate_impl`` (models/daisy/fla_custom_ops.py:71-103) as called from
    ``KimiLinearSelfAttention._kda_eager`` (models/daisy/attention_kimi.py:132:
    ``fused_kda_gate(g, A_log, head_k_dim, dt_bias, None, 1.0, 20.0)``).  softplus(x) = log1p(exp(beta x)) / beta
    and exactly x where beta x > threshold (torch.nn.functional.softplus).  ``A_log`` is ``[H]``, ``g_bias``
    ``[H*D]`` or None."""
    H = g.shape[-1] // head_k_dim
    x = g.float().reshape(*g.shape[:-1], H, head_k_dim)
    if g_bias is not None:
        x = x + g_bias.float().reshape(H, head_k_dim)
    bx = x * beta
    sp = torch.where(bx > threshold, x, torch.log1p(torch.exp(torch.clamp(bx, max=threshold))) / beta)
    y = -torch.exp(A_log.float().reshape(H, 1)) * sp
    return y.to(g.dtype)


def kda_bytes_per_token_head(K: int = 128, V: int = 128) -> int:
    """Algorithmic HBM bytes per (token, head): q,k bf16, v bf16, g fp32, beta fp32, o bf16."""
    return 2 * K * 2 + V * 2 + K * 4 + 4 + V * 2


def kda_flops_per_token_head(K: int = 128, V: int = 128, C: int = 64) -> float:
    """Chunked-form FLOPs per (token, head): two gated CxC Gram products over K, the CxC
    unit-lower-triangular solve, W = T(beta k e^G) and U = T(beta v), W S, Q S, A U and the
    state update K^T U -- per chunk, divided by C."""
    per_chunk = (2 * 2 * C * C * K          # A_kk, A_qk
                 + C * C * C / 3.0          # forward substitution
                 + 2 * C * C * K            # W
                 + 2 * C * C * V            # U
                 + 2 * C * K * V            # W S
                 + 2 * C * K * V            # Q S
                 + 2 * C * C * V            # A_qk U
                 + 2 * C * K * V)           # K^T U
    return per_chunk / C
