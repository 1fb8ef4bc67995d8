"""Backward pass of the windowed attention (the training form): the tcgen05 backward kernels against
``torch.autograd`` over the fp32 oracle, on the (T, window, documents, block window) grid of the forward tests;
bitwise run-to-run determinism; the norm / RoPE backward; the module under autograd against the reference-generated
fixture."""
import os

import numpy as np
import pytest
import torch

from gpu_util import assert_close_bf16, bf16_randn
from oracle import swa

pytestmark = pytest.mark.gpu
D = 128


def _prepared(B, T, H, seed):
    """RMS-normalised, rotated q, k and normalised v as bf16 (what the forward kernel consumes)."""
    q, k, v = (bf16_randn(B, T, H, D, seed=seed + i, device="cpu").float() for i in range(3))
    cos, sin = swa.rope_tables(D, T)
    qn, kn, vn = swa.qkv_transform(q, k, v, cos, sin, swa.FP32_EPS)
    return qn.bfloat16(), kn.bfloat16(), vn.bfloat16()


def _check_grads(got, ref, what, cancelling=False):
    """bf16 bar of the forward tests, plus relative L2 <= 2e-2.  ``cancelling``: windows of one or two keys, where the
    exact dq and dk are (nearly) zero as the difference dP - delta of two terms of magnitude |dO||v| ~ 10..40: delta
    is formed from the bf16 output O, which carries the forward's bf16 rounding of P (2^-9 relative), so an
    absolute error of 2^-8 * max|dP| * scale * max|k| ~ 0.05 remains -- the same in any implementation that takes
    delta from the stored output."""
    for g, r, n in zip(got, ref, ("dq", "dk", "dv")):
        if cancelling and n != "dv":
            assert_close_bf16(g, r, f"{what} {n}", max_tol=0.1, mean_tol=0.01)
            continue
        assert_close_bf16(g, r, f"{what} {n}")
        rel = ((g.float().cpu() - r).norm() / r.norm().clamp_min(1e-20)).item()
        assert rel <= 2e-2, f"{what} {n}: relative L2 {rel}"


@pytest.mark.parametrize("T,window", [(128, None), (300, 64), (256, 128), (257, 1), (640, 200), (1000, 129), (131, 500), (512, 2)])
def test_attend_backward_matches_autograd_oracle(T, window):
    from daisy_b200 import ops
    B, H = 2, 2
    q, k, v = _prepared(B, T, H, seed=T)
    d_o = bf16_randn(B, T, H, D, seed=T + 9, device="cpu")
    y_ref, *ref = swa.attend_backward(q.float(), k.float(), v.float(), d_o.float(), window)
    qc, kc, vc, gc = (t.cuda() for t in (q, k, v, d_o))
    y, lse = ops.swa_attend(qc, kc, vc, window, bounded_qk=True, return_lse=True)
    got = ops.swa_attend_bwd(qc, kc, vc, y, gc, lse, window)
    ops.check_device_status("cuda")
    assert_close_bf16(y, y_ref, "forward with lse")
    _check_grads(got, ref, f"T={T} W={window}", cancelling=window is not None and window <= 2)
    # the general (running-maximum) forward form stores the same quantity
    y2, lse2 = ops.swa_attend(qc, kc, vc, window, bounded_qk=False, return_lse=True)
    assert (lse2 - lse).abs().max().item() <= 2e-2
    again = ops.swa_attend_bwd(qc, kc, vc, y, gc, lse, window)
    assert all(torch.equal(a, b) for a, b in zip(got, again)), "backward is not run-to-run deterministic"


@pytest.mark.parametrize("T,window,n_docs,per_batch", [(384, 100, 3, False), (700, None, 12, False), (512, 64, 5, True)])
def test_attend_backward_with_documents(T, window, n_docs, per_batch):
    from daisy_b200 import ops
    B, H = 2, 2
    q, k, v = _prepared(B, T, H, seed=T + 1)
    d_o = bf16_randn(B, T, H, D, seed=T + 5, device="cpu")
    g = torch.Generator().manual_seed(T)
    rows = []
    for _ in range(B if per_batch else 1):
        cuts = torch.sort(torch.randperm(T - 1, generator=g)[:n_docs - 1] + 1).values
        ds = torch.zeros(T, dtype=torch.int32)
        for c in cuts.tolist():
            ds[c:] = c
        rows.append(ds)
    ds = torch.stack(rows) if per_batch else rows[0]
    _, *ref = swa.attend_backward(q.float(), k.float(), v.float(), d_o.float(), window, doc_start=ds)
    qc, kc, vc, gc = (t.cuda() for t in (q, k, v, d_o))
    y, lse = ops.swa_attend(qc, kc, vc, window, bounded_qk=True, doc_start=ds.cuda(), return_lse=True)
    got = ops.swa_attend_bwd(qc, kc, vc, y, gc, lse, window, doc_start=ds.cuda())
    ops.check_device_status("cuda")
    _check_grads(got, ref, f"docs T={T}")


@pytest.mark.parametrize("T,wb,n_docs", [(512, 2, 1), (768, 1, 4), (640, 3, 6)])
def test_attend_backward_block_window_training_form(T, wb, n_docs):
    """The flex-attention form: the window counts 128-token key blocks (models/daisy/daisy_core.py:182-229)."""
    from daisy_b200 import ops
    B, H = 1, 2
    q, k, v = _prepared(B, T, H, seed=T + 2)
    d_o = bf16_randn(B, T, H, D, seed=T + 6, device="cpu")
    g = torch.Generator().manual_seed(T + wb)
    ds = torch.zeros(T, dtype=torch.int32)
    for c in torch.sort(torch.randperm(T - 1, generator=g)[:n_docs - 1] + 1).values.tolist():
        ds[c:] = c
    _, *ref = swa.attend_backward(q.float(), k.float(), v.float(), d_o.float(), None, doc_start=ds, window_blocks=wb)
    qc, kc, vc, gc = (t.cuda() for t in (q, k, v, d_o))
    y, lse = ops.swa_attend(qc, kc, vc, wb, bounded_qk=True, doc_start=ds.cuda(), window_in_blocks=True, return_lse=True)
    got = ops.swa_attend_bwd(qc, kc, vc, y, gc, lse, wb, doc_start=ds.cuda(), window_in_blocks=True)
    ops.check_device_status("cuda")
    _check_grads(got, ref, f"block window T={T} wb={wb}")


def test_prep_backward_matches_autograd():
    """Norm / RoPE backward on strided views of a merged projection."""
    from daisy_b200 import ops
    B, T, H = 2, 150, 3
    qkv = bf16_randn(B, T, 3 * H, D, seed=1)
    q, k, v = qkv.chunk(3, dim=-2)
    gs = [bf16_randn(B, T, H, D, seed=20 + i) for i in range(3)]
    cos, sin = swa.rope_tables(D, T)
    leaves = [t.float().cpu().requires_grad_(True) for t in (q, k, v)]
    outs = swa.qkv_transform(*leaves, cos, sin, swa.FP32_EPS)
    sum((o * g.float().cpu()).sum() for o, g in zip(outs, gs)).backward()
    got = ops.qkv_prep_bwd(q, k, v, cos.cuda(), sin.cuda(), *gs, swa.FP32_EPS)
    for g_, leaf, n in zip(got, leaves, "qkv"):
        assert_close_bf16(g_, leaf.grad, f"d{n} raw")


def test_module_forward_under_autograd_matches_reference_fixture(golden_dir):
    """``loss.backward()`` through ``B200CausalSelfAttention.forward`` with the document mask: input and weight
    gradients against the reference module's own autograd results (fp32, CPU)."""
    from daisy_b200 import B200CausalSelfAttention, WindowMask
    d = np.load(os.path.join(golden_dir, "csa_backward_small.npz"))
    attn = B200CausalSelfAttention(dim=256, num_heads=2, head_dim=128, max_seq_len=256).cuda()
    attn.norm_eps = swa.FP32_EPS
    with torch.no_grad():
        attn.qkvo_w.copy_(torch.from_numpy(d["qkvo_w"]).to(attn.qkvo_w.dtype))
    x = torch.from_numpy(d["x"]).cuda().bfloat16().requires_grad_(True)
    mask = WindowMask.from_tokens(torch.from_numpy(d["seq"]).cuda(), int(d["window"]), int(d["eos"]))
    y = attn(x, None, attn_mask=mask)
    assert y.requires_grad
    (y.float() * torch.from_numpy(d["cot"]).cuda()).sum().backward()
    assert_close_bf16(y.detach(), torch.from_numpy(d["y"]), "y", max_tol=4e-2, mean_tol=4e-3)
    assert_close_bf16(x.grad, torch.from_numpy(d["dx"]), "dx", max_tol=4e-2, mean_tol=4e-3)
    assert_close_bf16(attn.qkvo_w.grad, torch.from_numpy(d["dw"]), "dw", max_tol=4e-2, mean_tol=4e-3)
    # and the inference route computes the same forward
    with torch.inference_mode():
        y_inf = attn(x.detach(), None, attn_mask=mask)
    assert_close_bf16(y_inf, y.detach().float().cpu(), "inference vs training forward", max_tol=3e-2, mean_tol=3e-3)


def test_value_embedding_layer_under_autograd():
    """A layer that receives a value embedding, trained: the gate ``v = s(g_ve) norm(v) + (1 - s(g_ve)) ve``
    (models/daisy/attention.py:132-135) sits between the norm and the attention, and ``loss.backward()`` must reach x, the
    merged weights, the gate parameter and ve.  Compared with ``torch.autograd`` over the fp32 oracle functions."""
    from daisy_b200 import B200CausalSelfAttention, WindowMask
    os.environ["DISABLE_O_ZERO_INIT"] = "1"
    torch.manual_seed(3)
    H, T, W = 2, 200, 64
    m = B200CausalSelfAttention(H * D, H, D, receives_ve=True, layer_idx=2).cuda()
    m.norm_eps = swa.FP32_EPS
    x = torch.randn(1, T, H * D, device="cuda").bfloat16().requires_grad_(True)
    ve = torch.randn(1, T, H * D, device="cuda").bfloat16().requires_grad_(True)
    cot = torch.randn(1, T, H * D, device="cuda")
    y = m(x, ve, attn_mask=WindowMask(W))
    assert y.requires_grad
    (y.float() * cot).sum().backward()
    # oracle: the same computation in fp32 on the CPU
    xo = x.detach().float().cpu().requires_grad_(True)
    vo = ve.detach().float().cpu().requires_grad_(True)
    wo = m.qkvo_w.detach().float().cpu().requires_grad_(True)
    go = m.g_ve.detach().float().cpu().requires_grad_(True)
    q, k, v = swa.project_qkv(xo, wo, H, D)
    cos, sin = swa.rope_tables(D, T)
    qn, kn, vn = swa.qkv_transform(q, k, v, cos, sin, swa.FP32_EPS)
    gate = torch.sigmoid(go)
    vn = gate * vn + (1 - gate) * vo.view_as(vn)
    yo = swa.attend_windowed(qn, kn, vn, W).reshape(1, T, H * D) @ wo[3].t()
    (yo * cot.cpu()).sum().backward()
    assert_close_bf16(y.detach(), yo.detach(), "y", max_tol=4e-2, mean_tol=4e-3)
    assert_close_bf16(x.grad, xo.grad, "dx", max_tol=4e-2, mean_tol=4e-3)
    assert_close_bf16(ve.grad, vo.grad, "d ve", max_tol=4e-2, mean_tol=4e-3)
    assert_close_bf16(m.qkvo_w.grad, wo.grad, "dw", max_tol=4e-2, mean_tol=4e-3)
    g_got, g_ref = m.g_ve.grad.float().cpu().reshape(-1), go.grad.reshape(-1)
    assert torch.allclose(g_got, g_ref, rtol=5e-2, atol=5e-2 * float(g_ref.abs().max()) + 1e-3), (g_got, g_ref)
    # the inference route computes the same forward
    with torch.inference_mode():
        y_inf = m(x.detach(), ve.detach(), attn_mask=WindowMask(W))
    assert_close_bf16(y_inf, y.detach().float().cpu(), "inference vs training forward", max_tol=3e-2, mean_tol=3e-3)
