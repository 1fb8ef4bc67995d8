"""Algorithmic work of the hot-path kernels: the FLOP and byte counts the roofline figures are computed from.
Pure arithmetic on shapes; no tensors."""
from __future__ import annotations

from typing import Optional

FP32_EPS = 2.0 ** -23      # torch.finfo(torch.float32).eps: F.rms_norm's eps for fp32 inputs


def window_pairs(T: int, window: Optional[int]) -> int:
    """(query, key) pairs the causal window mask admits: query i sees keys max(0, i - window + 1) .. i."""
    W = T if window is None else min(window, T)
    return W * (W + 1) // 2 + (T - W) * W


def prefill_flops(B: int, T: int, H: int, D: int, window: Optional[int]) -> float:
    """Windowed attention: QK^T and PV over the admitted pairs, 2 FLOPs per multiply-add."""
    return 4.0 * D * window_pairs(T, window) * B * H


def decode_bytes(B: int, H: int, D: int, ctx_rows: int, elem: int = 2) -> float:
    """One decode step: K and V context rows read; new q, k, v read, output written, new k, v written to the ring."""
    return float(B * H * ctx_rows * D * elem * 2 + B * H * D * elem * 6)


def kda_bytes_per_token_head(K: int = 128, V: int = 128) -> int:
    """q, k bf16; v bf16; g fp32; beta fp32; o bf16."""
    return 2 * K * 2 + V * 2 + K * 4 + 4 + V * 2


def kda_flops_per_token_head(K: int = 128, V: int = 128, C: int = 64) -> float:
    """Chunked KDA per (token, head): two gated C x C Gram products over K, the unit-lower-triangular solve,
    W and U, W S, Q S, A U and the state update, per chunk of C tokens, divided by C."""
    per_chunk = (2 * 2 * C * C * K + C * C * C / 3.0 + 2 * C * C * K + 2 * C * C * V
                 + 2 * C * K * V + 2 * C * K * V + 2 * C * C * V + 2 * C * K * V)
    return per_chunk / C
