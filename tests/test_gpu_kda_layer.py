"""The row-wise passes of the KDA layer through the C ABI: short causal convolution + SiLU, gated RMS norm.
Checked against the fp32 oracle, the committed fixture, chaining through the carried state, and -- where the
third-party package runs on this GPU -- fla's own Triton kernels, which are what the reference executes."""
import os

import numpy as np
import pytest
import torch

from gpu_util import assert_close_bf16
from oracle import kda as okda

pytestmark = pytest.mark.gpu


def _conv_inputs(B, T, C, W, seed, bias=False):
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(B, T, C, device="cuda", generator=g).bfloat16()
    w = (torch.randn(C, W, device="cuda", generator=g) * 0.5).bfloat16()
    b = (torch.randn(C, device="cuda", generator=g) * 0.3).bfloat16() if bias else None
    return x, w, b


@pytest.mark.parametrize("W", [4, 3, 2, 1])
@pytest.mark.parametrize("T", [1, 2, 3, 5, 31, 32, 33, 64, 100, 517])
def test_short_conv_matches_oracle(T, W):
    from daisy_b200 import ops
    x, w, b = _conv_inputs(2, T, 256, W, 100 + T + W, bias=(W == 3))
    y, s = ops.kda_short_conv(x, w, b, output_final_state=True)
    ref, s_ref = okda.short_conv(x.float().cpu(), w.float().cpu(), None if b is None else b.float().cpu())
    assert_close_bf16(y, ref, f"T={T} W={W}")
    assert torch.equal(s.float().cpu(), s_ref)
    y_lin, _ = ops.kda_short_conv(x, w, b, silu=False)
    ref_lin, _ = okda.short_conv(x.float().cpu(), w.float().cpu(), None if b is None else b.float().cpu(), activation=None)
    assert_close_bf16(y_lin, ref_lin, "no activation")


def test_short_conv_fixture(golden_dir):
    from daisy_b200 import ops
    d = np.load(os.path.join(golden_dir, "kda_layer_small.npz"))
    for W in (4, 3, 2):
        x, w, b, ref = (torch.from_numpy(d[f"conv_w{W}_{n}"]) for n in ("x", "weight", "bias", "y"))
        xb, wb = x.bfloat16(), w.bfloat16()
        bb = b.bfloat16() if b.numel() else None
        y, _ = ops.kda_short_conv(xb.cuda(), wb.cuda(), None if bb is None else bb.cuda())
        # the kernel sees bf16 inputs: compare with the oracle on the same rounded values, and loosely with the
        # fp32 fixture itself
        ref_b, _ = okda.short_conv(xb.float(), wb.float().reshape(-1, W), None if bb is None else bb.float())
        assert_close_bf16(y, ref_b, f"fixture W={W}")
        assert (y.float().cpu() - ref).abs().max().item() <= 6e-2


@pytest.mark.parametrize("W", [4, 2])
def test_short_conv_state_chain_is_bit_exact(W):
    """Prefill + decode steps through the carried state (updated in place, as the reference's cache is) give the
    bits of one call over the whole sequence; so do two long calls chained through a fresh state tensor."""
    from daisy_b200 import ops
    B, T, C = 3, 150, 512
    x, w, b = _conv_inputs(B, T, C, W, 7)
    y_all, s_all = ops.kda_short_conv(x, w, b, output_final_state=True)
    y0, s = ops.kda_short_conv(x[:, :97], w, b, output_final_state=True)
    ys = [y0]
    for t in range(97, T):
        yt, s2 = ops.kda_short_conv(x[:, t:t + 1], w, b, state=s, output_final_state=True, inplace_state=True)
        assert s2 is s
        ys.append(yt)
    assert torch.equal(torch.cat(ys, 1), y_all) and torch.equal(s, s_all)
    ya, sa = ops.kda_short_conv(x[:, :70], w, b, output_final_state=True)
    yb, sb = ops.kda_short_conv(x[:, 70:], w, b, state=sa, output_final_state=True)
    assert torch.equal(torch.cat([ya, yb], 1), y_all) and torch.equal(sb, s_all) and sb is not sa
    # a one-token prompt: the state keeps the zero padding in front
    _, s1 = ops.kda_short_conv(x[:, :1], w, b, output_final_state=True)
    assert not s1[..., :-1].any() and torch.equal(s1[..., -1], x[:, 0])
    # in place over more than one time block is refused, not raced
    big = torch.zeros(B, C, W, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(Exception):
        ops.kda_short_conv(x, w, b, state=big, output_final_state=True, inplace_state=True)


def test_short_conv_strided_input():
    """q, k, v read as column slices of one merged projection [B, T, 3C]."""
    from daisy_b200 import ops
    B, T, C = 2, 77, 256
    x3, w, _ = _conv_inputs(B, T, 3 * C, 4, 9)
    for i in range(3):
        xs = x3[:, :, i * C:(i + 1) * C]
        y, _ = ops.kda_short_conv(xs, w[i * C:(i + 1) * C])
        y_ref, _ = ops.kda_short_conv(xs.contiguous(), w[i * C:(i + 1) * C].contiguous())
        assert torch.equal(y, y_ref)


@pytest.mark.parametrize("rows", [(1,), (17,), (2, 31, 3), (4, 128, 16)])
def test_out_norm_matches_oracle(rows):
    from daisy_b200 import ops, _lib
    g_ = torch.Generator(device="cuda").manual_seed(sum(rows))
    o = (torch.randn(*rows, 128, device="cuda", generator=g_) * 2).bfloat16()
    gate = (torch.randn(*rows, 128, device="cuda", generator=g_) * 3).bfloat16()
    w = (1 + 0.2 * torch.randn(128, device="cuda", generator=g_)).bfloat16()
    for mode, name in ((_lib.KDA_NORM_SIGMOID, "sigmoid"), (_lib.KDA_NORM_SWISH, "swish"),
                       (_lib.KDA_NORM_SWISH_SIGMOID, "swish_sigmoid")):
        y = ops.kda_out_norm(o, gate, w, mode=mode)
        ref = okda.gated_rms_norm(o.float().cpu(), gate.float().cpu(), w.float().cpu(), mode=name)
        assert y.shape == o.shape
        assert_close_bf16(y, ref, f"{name} rows={rows}")
    if len(rows) >= 2:                                               # gate bias per (head, channel), added in the kernel
        H = rows[-1]
        gb = (torch.randn(H * 128, device="cuda", generator=g_) * 0.5).bfloat16()
        yb = ops.kda_out_norm(o, gate, w, gate_bias=gb)
        gsum = (gate.float() + gb.float().view(H, 128)).bfloat16()
        assert torch.equal(yb, ops.kda_out_norm(o, gsum, w))
    y32 = ops.kda_out_norm(o.float(), gate, None)
    assert_close_bf16(y32, okda.gated_rms_norm(o.float().cpu(), gate.float().cpu(), None), "fp32 input, no weight")


def test_out_norm_fixture(golden_dir):
    from daisy_b200 import ops
    d = np.load(os.path.join(golden_dir, "kda_layer_small.npz"))
    x, g, w = (torch.from_numpy(d[n]).bfloat16().cuda() for n in ("norm_x", "norm_gate", "norm_weight"))
    y = ops.kda_out_norm(x, g, w).float().cpu()
    ref = torch.from_numpy(d["norm_ref_bf16_as_fp32"])
    assert ((y - ref).abs() <= ref.abs() * 2.0 ** -6 + 1e-6).all()
    assert (y == ref).float().mean().item() > 0.98


def _fla_or_skip():
    try:
        from fla.modules import ShortConvolution
        from fla.modules.fused_norm_gate import rms_norm_gated
        return ShortConvolution, rms_norm_gated
    except Exception as e:                                           # package absent or unusable here
        pytest.skip(f"fla not importable: {e}")


def test_against_fla_triton_kernels():
    """The third-party kernels the reference itself runs (ShortConvolution, rms_norm_gated), when they work on
    this GPU: prefill with a final state, a decode step on the cache, and the module's two-factor gated norm."""
    ShortConvolution, rms_norm_gated = _fla_or_skip()
    from daisy_b200 import ops
    B, T, C, W = 2, 200, 256, 4
    x, w, _ = _conv_inputs(B, T, C, W, 21)
    try:
        conv = ShortConvolution(C, W, activation="silu", dtype=torch.bfloat16).cuda()
        with torch.no_grad():
            conv.weight.copy_(w.view(C, 1, W))
            y_ref, cache = conv(x=x, cache=None, output_final_state=True)
            x1 = torch.randn(B, 1, C, device="cuda").bfloat16()
            cache_before = cache.clone()
            y1_ref, cache_after = conv(x=x1, cache=cache, output_final_state=True)
            o = (torch.randn(B, T, 2, 128, device="cuda") * 2).bfloat16()
            gate = (torch.randn(B, T, 2, 128, device="cuda") * 3).bfloat16()
            nw = (1 + 0.2 * torch.randn(128, device="cuda")).bfloat16()
            n_ref = rms_norm_gated(o, gate, nw, None)
            n_ref = n_ref * torch.sigmoid(gate)
        torch.cuda.synchronize()
    except Exception as e:
        pytest.skip(f"fla's Triton kernels did not run here: {type(e).__name__}: {e}")
    y, s = ops.kda_short_conv(x, w, output_final_state=True)
    assert_close_bf16(y, y_ref.float().cpu(), "conv vs fla")
    assert (y == y_ref).float().mean().item() > 0.99
    assert torch.equal(s, cache_before.to(s.dtype))
    y1, s1 = ops.kda_short_conv(x1, w, state=s, output_final_state=True)
    assert_close_bf16(y1, y1_ref.float().cpu(), "conv step vs fla")
    assert torch.equal(s1, cache_after.to(s1.dtype))
    yn = ops.kda_out_norm(o, gate, nw)
    assert_close_bf16(yn, n_ref.float().cpu(), "gated norm vs fla")
    assert (yn == n_ref).float().mean().item() > 0.98


def _layer(dim=256, H=2, seed=3):
    from daisy_b200 import B200KimiLinearSelfAttention
    torch.manual_seed(seed)
    m = B200KimiLinearSelfAttention(dim, H, 4096, 128).cuda().eval()
    with torch.no_grad():
        for n, p in m.named_parameters():
            if n.endswith("conv1d.weight"):
                p.copy_(torch.randn_like(p) * 0.5)
            elif n == "dt_bias":
                p.copy_(torch.randn_like(p) * 0.5)
            elif n == "o_norm.weight":
                p.copy_(1 + 0.1 * torch.randn_like(p))
            elif n == "g_proj.1.bias":
                p.copy_(torch.randn_like(p) * 0.2)
    return m


@pytest.mark.parametrize("T", [96, 200])
def test_layer_forward_matches_oracle(T):
    """The whole KDA layer (projections, convolutions, gate, KDA, gated norm, output projection) against the oracle's
    composition with the same bf16 stage roundings."""
    m = _layer()
    x = torch.randn(2, T, 256, device="cuda").bfloat16()
    with torch.inference_mode():
        y = m(x, None, None)
    params = {n: p.detach().cpu() for n, p in m.named_parameters()}
    y_ref, _ = okda.kimi_layer_forward(x.cpu(), params, 2, 128)
    rel = ((y.float().cpu() - y_ref).norm() / y_ref.norm()).item()
    assert y.shape == x.shape and rel <= 2e-2, rel


def test_layer_prefill_then_steps():
    """prefill + single-token steps (convolution cache updated in place, recurrent state carried) reproduce the
    forward over the whole sequence, and the oracle's chained run."""
    m = _layer(seed=5)
    B, T0, T = 2, 130, 138
    x = torch.randn(B, T, 256, device="cuda").bfloat16()
    with torch.inference_mode():
        y_all = m(x, None, None)
        m.reset_history()
        y0, _, _ = m.prefill(x[:, :T0], None, None)
        ys = [y0]
        conv_ptrs = [c.data_ptr() for c in m._conv_state]
        for t in range(T0, T):
            yt, _, _ = m.step(x[:, t:t + 1], None, None, t, None, None, None)
            ys.append(yt)
        assert [c.data_ptr() for c in m._conv_state] == conv_ptrs and m._seen == T
    y_chain = torch.cat(ys, 1).float().cpu()
    rel = ((y_chain - y_all.float().cpu()).norm() / y_all.float().norm().cpu()).item()
    assert rel <= 2e-2, rel
    params = {n: p.detach().cpu() for n, p in m.named_parameters()}
    y_ref, st = okda.kimi_layer_forward(x[:, :T0].cpu(), params, 2, 128)
    refs = [y_ref]
    for t in range(T0, T):
        yt, st = okda.kimi_layer_forward(x[:, t:t + 1].cpu(), params, 2, 128, state=st)
        refs.append(yt)
    y_ref = torch.cat(refs, 1)
    rel = ((y_chain - y_ref).norm() / y_ref.norm()).item()
    assert rel <= 2e-2, rel
    m.reset_history()
    assert m._recurrent_state is None and m._conv_state is None and m._seen == 0


def test_layer_step_graph_matches_eager():
    """The captured single-token step replays to the bits of the step launched kernel by kernel, states included."""
    m = _layer(seed=9)
    B, T0, n = 2, 70, 6
    x = torch.randn(B, T0 + n, 256, device="cuda").bfloat16()
    with torch.inference_mode():
        m.prefill(x[:, :T0], None, None)
        eager = [m.step(x[:, t:t + 1], None, None, t, None, None, None)[0].clone() for t in range(T0, T0 + n)]
        rec_e, conv_e = m._recurrent_state.clone(), [c.clone() for c in m._conv_state]
        m.reset_history()
        m.prefill(x[:, :T0], None, None)
        m.capture_step(batch=B)
        graph = [m.step_graph(x[:, t:t + 1]).clone() for t in range(T0, T0 + n)]
    for a, b in zip(eager, graph):
        assert torch.equal(a, b)
    assert torch.equal(m._recurrent_state, rec_e) and all(torch.equal(a, b) for a, b in zip(m._conv_state, conv_e))
    assert m._seen == T0 + n


# ------------------------------------------------------------------------------------ packed variable-length batches
@pytest.mark.parametrize("W", [4, 2])
@pytest.mark.parametrize("cu", [[0, 40], [0, 1, 2, 3, 4, 40], [0, 2, 2, 35, 67, 200], [0, 31, 32, 33, 96, 97]])
def test_short_conv_varlen_matches_oracle(cu, W):
    """The convolution over packed sequences: the window stops at each sequence's first token (sequences of 1 and 2
    tokens, an empty one, boundaries on and next to the 32-row blocks of the kernel), with and without carried states;
    each sequence gives the bits of the dense call on it alone."""
    from daisy_b200 import ops
    N, T, C = len(cu) - 1, cu[-1], 512
    x, w, b = _conv_inputs(1, T, C, W, 21 + T + W, bias=True)
    tabs = ops.kda_varlen_tables(cu, "cuda")
    st = torch.randn(N, C, W, device="cuda").bfloat16()
    for state in (None, st):
        y, s = ops.kda_short_conv_varlen(x, w, tabs[2], N, b, state=state, output_final_state=True)
        ref, s_ref = okda.short_conv_varlen(x.float().cpu(), w.float().cpu(), cu, b.float().cpu(),
                                            None if state is None else state.float().cpu())
        assert_close_bf16(y, ref, f"cu={cu} W={W}")
        assert torch.equal(s.float().cpu(), s_ref)
        for n, (a, e) in enumerate(zip(cu, cu[1:])):
            if e > a:
                yd, sd = ops.kda_short_conv(x[:, a:e], w, b, state=None if state is None else state[n:n + 1],
                                            output_final_state=True)
                assert torch.equal(y[:, a:e], yd) and torch.equal(s[n:n + 1], sd), f"sequence {n}"
    assert s is not st


def test_layer_attn_mask_matches_oracle_and_continues():
    """forward / prefill with an attention mask (left padding, right padding, a hole, a full row): kept tokens match
    the layer run on each row's kept tokens alone, padding positions return zeros, and the cached states are one per
    row, so that the following single-token steps match the oracle's chained run."""
    m = _layer(seed=13)
    B, T, D = 4, 150, 256
    x = torch.randn(B, T, D, device="cuda").bfloat16()
    mask = torch.ones(B, T + 10, dtype=torch.long, device="cuda")         # longer than T: the last T columns count
    mask[0, 10:10 + 37] = 0                                                # left padding
    mask[1, -20:] = 0                                                      # right padding
    mask[2, 60:75] = 0                                                     # a hole
    with torch.inference_mode():
        y = m(x, None, None, attn_mask=mask)
        m.reset_history()
        yp, _, _ = m.prefill(x, None, None, attn_mask=mask)
    assert y.shape == x.shape and torch.equal(y, yp)
    params = {n: p.detach().cpu() for n, p in m.named_parameters()}
    y_ref, states = okda.kimi_layer_forward_masked(x.cpu(), params, 2, 128, mask.cpu())
    keep = mask[:, -T:].bool().cpu()
    assert not y.float().cpu()[~keep].any()
    for b in range(B):
        rel = ((y[b].float().cpu()[keep[b]] - y_ref[b][keep[b]]).norm() / y_ref[b][keep[b]].norm()).item()
        assert rel <= 2e-2, (b, rel)
    assert m._recurrent_state.shape == (B, 2, 128, 128) and m._conv_state[0].shape[0] == B
    x1 = torch.randn(B, 1, D, device="cuda").bfloat16()
    with torch.inference_mode():
        y1, _, _ = m.step(x1, None, None, T, None, None, None)
    for b in range(B):
        r1, _ = okda.kimi_layer_forward(x1[b:b + 1].cpu(), params, 2, 128, state=states[b])
        rel = ((y1[b].float().cpu() - r1[0]).norm() / r1[0].norm()).item()
        assert rel <= 2e-2, (b, rel)


def test_short_conv_varlen_against_fla_triton():
    ShortConvolution, _ = _fla_or_skip()
    from daisy_b200 import B200ShortConvolution
    cu, C, W = [0, 3, 50, 51, 200], 256, 4
    torch.manual_seed(2)
    ref = ShortConvolution(C, W, bias=False, activation="silu").cuda().bfloat16()
    ours = B200ShortConvolution(C, W, bias=False, activation="silu", dtype=torch.bfloat16).cuda()
    ours.load_state_dict(ref.state_dict())
    x = torch.randn(1, cu[-1], C, device="cuda").bfloat16()
    cu_t = torch.tensor(cu, dtype=torch.int32, device="cuda")
    try:
        with torch.no_grad():
            y_ref, s_ref = ref(x=x, cache=None, output_final_state=True, cu_seqlens=cu_t.long())
        torch.cuda.synchronize()
    except Exception as e:
        pytest.skip(f"fla's Triton kernels did not run here: {type(e).__name__}: {e}")
    with torch.no_grad():
        y, s = ours(x=x, cache=None, output_final_state=True, cu_seqlens=cu_t)
    assert_close_bf16(y, y_ref.float().cpu(), "varlen conv vs fla")
    assert s.shape == s_ref.shape and torch.equal(s.float().cpu(), s_ref.float().cpu())
