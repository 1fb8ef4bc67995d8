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

``B200ShortConvolution``, ``B200FusedRMSNormGated`` and ``B200KimiLinearSelfAttention`` mirror the rest of the
layer (attention_kimi.py:41-62, 65-211): same constructors, parameter names and call protocol, on the kernels of
``csrc/kda_layer.cu``; the layer adds ``capture_step`` / ``step_graph`` (one CUDA-graph replay per decoded token).
"""
from __future__ import annotations

from typing import Optional

import torch

from . import ops

RECURRENT_MAX_T = 4      # up to this many tokens the state is carried token by token in registers


def chunk_kda(q, k, v, g, beta, scale: Optional[float] = None, initial_state: Optional[torch.Tensor] = None,
              output_final_state: bool = False, use_qk_l2norm_in_kernel: bool = False, cu_seqlens=None,
              out_fp32: bool = False, varlen_tables=None):
    q, k, v = (x.contiguous() if x.dtype == torch.bfloat16 else x.to(torch.bfloat16).contiguous() for x in (q, k, v))
    g = g.float().contiguous()
    beta = beta.float().contiguous()
    if initial_state is not None:
        initial_state = initial_state.float().contiguous()
    if cu_seqlens is not None or varlen_tables is not None:
        # packed sequences [1, T_total, ...]: states are per sequence, no chunk spans two of them
        return ops.kda_chunk_fwd_varlen(q, k, v, g, beta, cu_seqlens, scale, initial_state, output_final_state,
                                        l2norm_qk=use_qk_l2norm_in_kernel, out_fp32=out_fp32, tables=varlen_tables)
    fwd = ops.kda_recurrent_fwd if q.shape[1] <= RECURRENT_MAX_T else ops.kda_chunk_fwd
    o, hT = fwd(q, k, v, g, beta, scale, initial_state, output_final_state,
                l2norm_qk=use_qk_l2norm_in_kernel, out_fp32=out_fp32)
    return o, hT


def get_unpad_data(attention_mask: torch.Tensor):
    """``(indices, cu_seqlens, max_len)`` of a ``[B, S]`` 0/1 mask, as the helper the reference imports
    (models/daisy/attention_kimi.py:19, used at :150): the flat positions of the kept tokens, the N + 1 offsets of the
    rows' kept counts, and the largest count."""
    m = attention_mask.to(torch.bool)
    lens = m.sum(dim=-1, dtype=torch.int32)
    indices = torch.nonzero(m.flatten(), as_tuple=False).flatten()
    cu = torch.nn.functional.pad(torch.cumsum(lens, 0, dtype=torch.int32), (1, 0))
    return indices, cu, int(lens.max().item()) if lens.numel() else 0


def index_first_axis(x: torch.Tensor, indices: torch.Tensor) -> torch.Tensor:
    """Rows ``indices`` of ``x [(B S), ...]`` (attention_kimi.py:153)."""
    return x.index_select(0, indices)


def pad_input(x: torch.Tensor, indices: torch.Tensor, batch: int, seqlen: int) -> torch.Tensor:
    """Inverse of :func:`index_first_axis`: ``x [T_total, ...]`` back to ``[batch, seqlen, ...]``, zeros at the dropped
    positions (attention_kimi.py:193)."""
    out = x.new_zeros(batch * seqlen, *x.shape[1:])
    out.index_copy_(0, indices, x)
    return out.view(batch, seqlen, *x.shape[1:])


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


# ----------------------------------------------------------------------------------------------- the layer
class B200ShortConvolution(torch.nn.Conv1d):
    """The ``ShortConvolution`` the reference's KDA layer builds (models/daisy/attention_kimi.py:88-91; third-party
    ``fla.modules``): a depthwise causal ``Conv1d`` (weight ``[C, 1, W]``, so checkpoints load unchanged) with SiLU,
    called as ``y, cache = conv(x=..., cache=..., output_final_state=...)`` (:160-162).  ``cache [B, C, W]`` holds the
    last W inputs; on decode steps it is updated in place, as the reference's is."""

    def __init__(self, hidden_size: int, kernel_size: int, bias: bool = False, activation: Optional[str] = "silu",
                 device=None, dtype=None):
        super().__init__(hidden_size, hidden_size, kernel_size, groups=hidden_size, bias=bias,
                         padding=kernel_size - 1, device=device, dtype=dtype)
        if activation not in (None, "silu", "swish"):
            raise ValueError(f"activation {activation!r} not supported")
        self.hidden_size, self.activation = hidden_size, activation

    def forward(self, x, cache=None, output_final_state: bool = False, cu_seqlens=None, varlen_tables=None, **_):
        if cache is not None and cache.dtype != torch.bfloat16:
            cache = cache.to(torch.bfloat16)
        if cu_seqlens is not None or varlen_tables is not None:
            # packed sequences x [1, T_total, C]; cache and final state [N, C, W]
            tabs = varlen_tables if varlen_tables is not None else ops.kda_varlen_tables(cu_seqlens, x.device)
            return ops.kda_short_conv_varlen(x if x.dtype == torch.bfloat16 else x.to(torch.bfloat16), self.weight,
                                             tabs[2], tabs[1].numel() - 1, self.bias, state=cache,
                                             output_final_state=output_final_state, silu=self.activation is not None)
        step = cache is not None and x.shape[1] <= 32
        return ops.kda_short_conv(x if x.dtype == torch.bfloat16 else x.to(torch.bfloat16), self.weight, self.bias,
                                  state=cache, output_final_state=output_final_state or step,
                                  silu=self.activation is not None, inplace_state=step)


class B200FusedRMSNormGated(torch.nn.Module):
    """``CompilableFusedRMSNormGated`` (models/daisy/attention_kimi.py:41-62): ``rms_norm_gated(x, gate, weight)`` with
    that function's default swish gate and eps 1e-6, times ``sigmoid(gate)`` -- one kernel here."""

    def __init__(self, hidden_size: int, activation: str = "sigmoid", dtype=torch.bfloat16):
        if activation != "sigmoid":
            raise ValueError("Only sigmoid activation is supported")
        super().__init__()
        self.hidden_size, self.activation = hidden_size, activation
        self.weight = torch.nn.Parameter(torch.ones(hidden_size, dtype=dtype))
        self.bias = None

    def forward(self, x, gate, gate_bias=None):
        return ops.kda_out_norm(x, gate, self.weight, eps=1e-6, gate_bias=gate_bias)


def _linear(x, weight, bias=None):
    """``F.linear`` on this library's GEMM where its tiles apply (at least 64 rows, N % 128 == 0, K % 64 == 0);
    the narrow ones (the per-head beta projection, single decode rows) go to torch's."""
    N, K = weight.shape
    if x.numel() // K >= 64 and N % 128 == 0 and K % 64 == 0 and weight.dtype == torch.bfloat16 and x.dtype == torch.bfloat16:
        y = ops.gemm_nt(x, weight)
        return y if bias is None else y.add_(bias)
    return torch.nn.functional.linear(x, weight, bias)


class B200KimiLinearSelfAttention(torch.nn.Module):
    """The reference's ``KimiLinearSelfAttention`` (models/daisy/attention_kimi.py:65-211) with the same constructor,
    parameter names and ``forward`` / ``prefill`` / ``step`` / ``reset_history`` protocol, running on the B200 kernels:
    projections -> short convolutions (:160-162) -> decay gate (:132) -> KDA (:133-134; chunked for prompts, the
    recurrent step for decode) -> gated norm (:135-137) -> output projection.  The reference's ``forward`` cannot
    run as written (it passes five arguments to a four-parameter ``_forward_core`` whose body then reads an
    undefined ``sa_lambdas``); this class implements what those lines evidently intend, with ``sa_lambdas``
    threaded through.  The batch-size-1 assertion (:151) is lifted.  ``attn_mask [B, S_total]`` (1 = token, 0 =
    padding) packs the kept tokens of the last ``T`` columns into one row, runs the convolutions and the KDA per
    sequence (cu_seqlens, :150-162) and scatters the result back with zeros at the padding (:193); the cached states
    are then one per batch row, so decode steps continue from them."""

    def __init__(self, dim: int, num_heads: int, max_seq_len: int, head_dim: int, expand_v: float = 1.0,
                 mode: str = "chunk", use_short_conv: bool = True, allow_neg_eigval: bool = False, conv_size: int = 4,
                 conv_bias: bool = False, layer_idx: int = 0, receives_ve: bool = False):
        if allow_neg_eigval or mode != "chunk":
            raise ValueError("allow_neg_eigval=False and mode='chunk' only, as in the reference")
        super().__init__()
        nn, bf = torch.nn, torch.bfloat16
        self.hidden_size, self.num_heads, self.head_dim = dim, num_heads, head_dim
        self.head_k_dim, self.head_v_dim = head_dim, int(head_dim * expand_v)
        self.key_dim, self.value_dim = num_heads * self.head_k_dim, num_heads * self.head_v_dim
        self.use_short_conv, self.conv_size, self.layer_idx = use_short_conv, conv_size, layer_idx
        self.q_proj = nn.Linear(dim, self.key_dim, bias=False, dtype=bf)
        self.k_proj = nn.Linear(dim, self.key_dim, bias=False, dtype=bf)
        self.v_proj = nn.Linear(dim, self.value_dim, bias=False, dtype=bf)
        if use_short_conv:
            self.q_conv1d = B200ShortConvolution(self.key_dim, conv_size, bias=conv_bias, dtype=bf)
            self.k_conv1d = B200ShortConvolution(self.key_dim, conv_size, bias=conv_bias, dtype=bf)
            self.v_conv1d = B200ShortConvolution(self.value_dim, conv_size, bias=conv_bias, dtype=bf)
        self.f_proj = nn.Sequential(nn.Linear(dim, self.head_v_dim, bias=False, dtype=bf),
                                    nn.Linear(self.head_v_dim, self.key_dim, bias=False, dtype=bf))
        self.b_proj = nn.Linear(dim, num_heads, bias=False, dtype=bf)
        self.A_log = nn.Parameter(torch.log(torch.empty(num_heads, dtype=torch.float32).uniform_(1, 16)).view(1, 1, -1, 1))
        self.dt_bias = nn.Parameter(torch.zeros(self.key_dim, dtype=torch.float32))
        self.g_proj = nn.Sequential(nn.Linear(dim, self.head_v_dim, bias=False, dtype=bf),
                                    nn.Linear(self.head_v_dim, self.value_dim, bias=True, dtype=bf))
        self.o_norm = B200FusedRMSNormGated(self.head_v_dim, activation="sigmoid", dtype=bf)
        self.o_proj = nn.Linear(self.value_dim, dim, bias=False, dtype=bf)
        self.reset_history()

    def reset_history(self):
        self._recurrent_state, self._conv_state, self._seen = None, None, 0

    def _forward_core(self, x, ve, sa_lambdas, attn_mask, use_cache: bool):
        if torch.is_grad_enabled() and (x.requires_grad or any(p.requires_grad for p in self.parameters())):
            # the kernels return tensors without a grad_fn: autograd would treat the layer as a constant
            raise NotImplementedError("daisy_b200 implements the forward pass only: call under torch.no_grad() / "
                                      "inference_mode(), or detach the input and freeze the parameters")
        B0, T0, _ = x.shape
        indices = tabs = None
        if attn_mask is not None:                                          # attention_kimi.py:150-154
            indices, cu_seqlens, _ = get_unpad_data(attn_mask[:, -T0:])
            x = index_first_axis(x.reshape(B0 * T0, -1), indices).unsqueeze(0)
            if ve is not None:
                ve = index_first_axis(ve.reshape(B0 * T0, -1), indices).unsqueeze(0)
            tabs = ops.kda_varlen_tables(cu_seqlens, x.device)
            if x.shape[1] == 0:
                return x.new_zeros(B0, T0, self.hidden_size)
        B, T, _ = x.shape
        H = self.num_heads
        q, k, v = _linear(x, self.q_proj.weight), _linear(x, self.k_proj.weight), _linear(x, self.v_proj.weight)
        if self.use_short_conv:
            cs = self._conv_state if (use_cache and self._conv_state is not None) else (None, None, None)
            q, cs_q = self.q_conv1d(x=q, cache=cs[0], output_final_state=use_cache, varlen_tables=tabs)
            k, cs_k = self.k_conv1d(x=k, cache=cs[1], output_final_state=use_cache, varlen_tables=tabs)
            v, cs_v = self.v_conv1d(x=v, cache=cs[2], output_final_state=use_cache, varlen_tables=tabs)
            conv_state = (cs_q, cs_k, cs_v)
        else:
            q, k, v = (torch.nn.functional.silu(t) for t in (q, k, v))
            conv_state = None
        q, k = q.view(B, T, H, self.head_k_dim), k.view(B, T, H, self.head_k_dim)
        v = v.view(B, T, H, self.head_v_dim)
        if sa_lambdas is not None and ve is not None:                      # attention_kimi.py:118-126
            v = sa_lambdas[0].to(v.dtype) * v + sa_lambdas[1].to(v.dtype) * ve.to(dtype=v.dtype, device=v.device).view_as(v)
        g = _linear(_linear(x, self.f_proj[0].weight), self.f_proj[1].weight)
        g = ops.kda_gate(g, self.A_log, self.head_k_dim, self.dt_bias, 1.0, 20.0)
        beta = torch.nn.functional.linear(x, self.b_proj.weight).sigmoid().float()
        rec = self._recurrent_state if use_cache else None
        if tabs is None and rec is not None and T <= RECURRENT_MAX_T and rec.dtype == torch.float32 and rec.is_contiguous():
            # decode step: the cached state is updated where it lies (no allocation: the step can be graph-captured)
            o, rec = ops.kda_recurrent_fwd(q.contiguous(), k.contiguous(), v.contiguous(), g, beta, None, rec, True,
                                           l2norm_qk=True, state_in_place=True)
        else:
            o, rec = chunk_kda(q=q, k=k, v=v, g=g, beta=beta, initial_state=rec, output_final_state=use_cache,
                               use_qk_l2norm_in_kernel=True, varlen_tables=tabs)
        gp = _linear(_linear(x, self.g_proj[0].weight), self.g_proj[1].weight)        # its bias is added in the norm kernel
        o = self.o_norm(o, gp.view(B, T, H, self.head_v_dim), self.g_proj[1].bias)
        if use_cache:
            self._recurrent_state, self._conv_state = rec, conv_state
            self._seen += T0
        y = _linear(o.view(B, T, self.value_dim), self.o_proj.weight)
        return y if indices is None else pad_input(y.squeeze(0), indices, B0, T0)

    # ------------------------------------------------------------------ CUDA-graph decode step
    @torch.inference_mode()
    def capture_step(self, batch: int = 1) -> None:
        """Record one single-token ``step`` (no value embedding) into a CUDA graph.  Needs the states a ``prefill``
        leaves; they are updated in place by the replayed kernels, input and output are fixed buffers.
        ``step_graph(x)`` then costs one copy and one graph launch instead of ~17 launches issued from Python."""
        if self._recurrent_state is None or (self.use_short_conv and self._conv_state is None):
            raise RuntimeError("capture_step needs the cached states of a prefill")
        dev = self._recurrent_state.device
        self._gx = torch.zeros(batch, 1, self.hidden_size, device=dev, dtype=torch.bfloat16)
        saved = [self._recurrent_state.clone()] + [c.clone() for c in (self._conv_state or ())]
        seen = self._seen

        def restore():
            self._recurrent_state.copy_(saved[0])
            for c, s_ in zip(self._conv_state or (), saved[1:]):
                c.copy_(s_)
            self._seen = seen

        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):                              # warm-up outside the capture (lazy initialisation)
            self._forward_core(self._gx, None, None, None, use_cache=True)
        torch.cuda.current_stream(dev).wait_stream(side)
        restore()
        self._graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self._graph):
            self._gy = self._forward_core(self._gx, None, None, None, use_cache=True)
        restore()

    @torch.inference_mode()
    def step_graph(self, x):
        """``step`` through the captured graph: ``x [batch, 1, dim]`` -> ``y`` (a fixed buffer, overwritten by the next call)."""
        self._gx.copy_(x)
        self._graph.replay()
        self._seen += 1
        return self._gy

    def forward(self, x, ve=None, sa_lambdas=None, attn_mask=None, sliding_window_num_blocks=None, block_mask=None):
        assert block_mask is None, "block_mask not supported for KimiLinearSelfAttention"
        return self._forward_core(x, ve, sa_lambdas, attn_mask, use_cache=False)

    def prefill(self, x, ve=None, sa_lambdas=None, attn_mask=None, debug: bool = False):
        return self._forward_core(x, ve, sa_lambdas, attn_mask, use_cache=True), None, None

    def step(self, x, k_ctx=None, v_ctx=None, pos: int = 0, ve=None, sa_lambdas=None, window=None):
        return self._forward_core(x, ve, sa_lambdas, None, use_cache=True), None, None
