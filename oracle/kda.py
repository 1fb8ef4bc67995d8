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


def kda_recurrent_varlen(q, k, v, g, beta, cu_seqlens, scale: Optional[float] = None,
                         initial_state: Optional[torch.Tensor] = None, l2norm_qk: bool = True,
                         dtype=torch.float32) -> Tuple[torch.Tensor, torch.Tensor]:
    """The packed form the reference reaches with an attention mask (``cu_seqlens`` from ``get_unpad_data``,
    models/daisy/attention_kimi.py:150-154, passed to ``chunk_kda`` at :133-134): the sequences lie end to end in one
    row ``[1, T_total, ...]`` and each runs the recurrence on its own, from its own initial state.  Returns
    ``(o [1,T_total,H,V], final_state [N,H,K,V])``."""
    cu = [int(c) for c in cu_seqlens]
    N, H, K, V = len(cu) - 1, q.shape[2], q.shape[3], v.shape[3]
    o = torch.zeros(1, q.shape[1], H, V, dtype=dtype)
    S = torch.zeros(N, H, K, V, dtype=dtype)
    for n, (a, b) in enumerate(zip(cu, cu[1:])):
        h0 = initial_state[n:n + 1] if initial_state is not None else None
        if b == a:
            if h0 is not None:
                S[n] = h0[0].to(dtype)
            continue
        o[:, a:b], S[n:n + 1] = kda_recurrent(q[:, a:b], k[:, a:b], v[:, a:b], g[:, a:b], beta[:, a:b], scale, h0,
                                              l2norm_qk, dtype)
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


def short_conv(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
               state: Optional[torch.Tensor] = None, activation: Optional[str] = "silu"
               ) -> Tuple[torch.Tensor, torch.Tensor]:
    """Short causal depthwise convolution of the KDA layer's q / k / v projections, fp32.

    Restates the ``ShortConvolution`` calls of ``KimiLinearSelfAttention._forward_core``
    (models/daisy/attention_kimi.py:160-162; modules built at :88-91 with ``activation="silu"``).  The class is
    third-party (``fla.modules``): a depthwise ``nn.Conv1d(C, C, W, groups=C, padding=W-1)`` truncated to the
    first T outputs, so with cross-correlation taps ``w[c, 0..W-1]``

        y[b, t, c] = act(bias[c] + sum_j w[c, j] * in[b, t - (W-1) + j, c])

    where ``in`` is ``x`` preceded by the carried ``state [B, C, W]`` (the W inputs before x, oldest first; zeros
    when None).  Returns ``(y [B,T,C], final_state [B,C,W])``, final_state[..., j] = in[T - W + j]: the decode
    step's cache update (shift left by one, newest input last) is the T = 1 case."""
    B, T, C = x.shape
    w = weight.float().reshape(C, -1)
    W = w.shape[1]
    hist = state.float().transpose(1, 2) if state is not None else torch.zeros(B, W, C)
    full = torch.cat([hist, x.float()], dim=1)                     # [B, W+T, C]; row W+t is input t
    y = torch.zeros(B, T, C)
    for j in range(W):
        y = y + w[:, j] * full[:, 1 + j:1 + j + T]                 # input t-(W-1)+j = row t+1+j
    if bias is not None:
        y = y + bias.float()
    if activation in ("silu", "swish"):
        y = y * torch.sigmoid(y)
    return y, full[:, T:T + W].transpose(1, 2).contiguous()


def short_conv_varlen(x: torch.Tensor, weight: torch.Tensor, cu_seqlens, bias: Optional[torch.Tensor] = None,
                      state: Optional[torch.Tensor] = None, activation: Optional[str] = "silu"
                      ) -> Tuple[torch.Tensor, torch.Tensor]:
    """``short_conv`` over packed sequences ``x [1, T_total, C]`` (the ``cu_seqlens`` argument of the calls at
    models/daisy/attention_kimi.py:160-162): every sequence is convolved on its own, preceded by its own state
    ``state[n]`` (zeros when None).  Returns ``(y [1,T_total,C], final_state [N,C,W])``; an empty sequence keeps its
    state."""
    cu = [int(c) for c in cu_seqlens]
    N, C = len(cu) - 1, x.shape[2]
    W = weight.reshape(C, -1).shape[1]
    y = torch.zeros(1, x.shape[1], C)
    fin = state.float().clone() if state is not None else torch.zeros(N, C, W)
    for n, (a, b) in enumerate(zip(cu, cu[1:])):
        if b > a:
            y[:, a:b], fin[n:n + 1] = short_conv(x[:, a:b], weight, bias, state[n:n + 1] if state is not None else None,
                                                 activation)
    return y, fin


def gated_rms_norm(o: torch.Tensor, gate: torch.Tensor, weight: Optional[torch.Tensor] = None,
                   eps: float = 1e-6, mode: str = "swish_sigmoid") -> torch.Tensor:
    """Gated RMS norm of the KDA output over the head dimension, fp32 result.

    Restates ``CompilableFusedRMSNormGated.forward`` (models/daisy/attention_kimi.py:52-60) as called at :137.  It
    calls the third-party ``fla.modules.fused_norm_gate.rms_norm_gated(x, gate, weight, bias)`` with that function's
    defaults (swish gate, eps 1e-6): ``n = x * rsqrt(mean(x^2) + eps) * weight * gate * sigmoid(gate)`` in fp32,
    rounded to x's dtype -- and then multiplies by ``sigmoid(gate)`` once more in that dtype.  ``mode``:
    "swish_sigmoid" (the reference: both factors, with the bf16 roundings in between), "swish", "sigmoid" (the
    single-factor forms of the third-party operator)."""
    x, g = o.float(), gate.float()
    n = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps)
    if weight is not None:
        n = n * weight.float()
    sg = torch.sigmoid(g)
    if mode == "sigmoid":
        return n * sg
    if mode == "swish":
        return n * g * sg
    return (n * g * sg).bfloat16().float() * sg.bfloat16().float()


def kimi_layer_forward(x: torch.Tensor, params: dict, num_heads: int, head_dim: int,
                       state: Optional[dict] = None, round_stages: bool = True):
    """The KDA layer end to end, ``x [B,T,dim] -> (y [B,T,dim], state)``: what
    ``KimiLinearSelfAttention._forward_core`` / ``_kda_eager`` (models/daisy/attention_kimi.py:128-193) compute,
    composed from the restatements above -- q/k/v projections, short convolutions with SiLU (:160-162), decay gate
    ``fused_kda_gate(f_proj(x), A_log, head_k_dim, dt_bias, None, 1.0, 20.0)`` (:132), ``beta = sigmoid(b_proj(x))``
    (:178), KDA with L2-normalised q, k (:133-134), gated norm with ``g_proj(x)`` (:135-137), output projection
    (:189).  ``params`` maps the module's parameter names to tensors.  ``state`` carries ``{"rec", "conv"}`` between
    calls (prefill -> steps).  With ``round_stages`` every stage output is rounded to bf16 where the bf16 module
    stores one, so that a bf16 device run can be compared tightly."""
    r = (lambda t: t.bfloat16().float()) if round_stages else (lambda t: t)
    P = {k: v.float() for k, v in params.items()}
    B, T, _ = x.shape
    x = x.float()
    lin = lambda t, w, b=None: r(torch.nn.functional.linear(t, w, b))
    st = state or {}
    conv_in = st.get("conv", (None, None, None))
    qkv, conv_out = [], []
    for name, cs in zip("qkv", conv_in):
        y, s_new = short_conv(lin(x, P[f"{name}_proj.weight"]), P[f"{name}_conv1d.weight"],
                              P.get(f"{name}_conv1d.bias"), state=cs)
        qkv.append(r(y).view(B, T, num_heads, head_dim)); conv_out.append(s_new)
    g = kda_gate(lin(lin(x, P["f_proj.0.weight"]), P["f_proj.1.weight"]), P["A_log"].reshape(-1), head_dim, P["dt_bias"])
    beta = r(torch.sigmoid(lin(x, P["b_proj.weight"])))
    o, rec = kda_recurrent(qkv[0], qkv[1], qkv[2], r(g), beta, None, st.get("rec"), True)
    gp = lin(lin(x, P["g_proj.0.weight"]), P["g_proj.1.weight"], P["g_proj.1.bias"]).view(B, T, num_heads, head_dim)
    o = gated_rms_norm(r(o), gp, P["o_norm.weight"], mode="swish_sigmoid")
    y = lin(r(o).reshape(B, T, num_heads * head_dim), P["o_proj.weight"])
    return y, {"rec": rec, "conv": tuple(conv_out)}


def kimi_layer_forward_masked(x: torch.Tensor, params: dict, num_heads: int, head_dim: int, attn_mask: torch.Tensor,
                              round_stages: bool = True):
    """The layer with an attention mask (models/daisy/attention_kimi.py:150-154,193): the tokens a row's mask keeps
    (its last T columns) form that row's sequence, the layer runs on each sequence alone, and the outputs return to
    their positions with zeros at the padding.  Returns ``(y [B,T,dim], [state of row 0, state of row 1, ...])``."""
    B, T, _ = x.shape
    keep = attn_mask[:, -T:].bool()
    y = torch.zeros(B, T, params["o_proj.weight"].shape[0])
    states = []
    for b in range(B):
        idx = keep[b].nonzero().flatten()
        if idx.numel() == 0:
            states.append(None)
            continue
        yb, st = kimi_layer_forward(x[b:b + 1, idx], params, num_heads, head_dim, None, round_stages)
        y[b, idx] = yb[0]
        states.append(st)
    return y, states


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
