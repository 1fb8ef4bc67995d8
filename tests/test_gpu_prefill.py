"""Prefill path (q/k/v preparation + tcgen05 windowed attention) against the fp32 oracle and the
reference-generated fixture."""
import os

import numpy as np
import pytest
import torch

from gpu_util import bf16_randn, assert_close_bf16
from oracle import swa

pytestmark = pytest.mark.gpu
D = 128


def test_qkv_prep_matches_oracle():
    from daisy_b200 import ops
    B, T, H = 2, 77, 3
    qkv = bf16_randn(B, T, 3 * H, D, seed=0)
    q, k, v = qkv.chunk(3, dim=-2)
    cos, sin = swa.rope_tables(D, T)
    qn, kn, vn = swa.qkv_transform(q.float().cpu(), k.float().cpu(), v.float().cpu(), cos, sin, swa.FP32_EPS)
    qp, kp, vp = ops.qkv_prep(q, k, v, cos.cuda(), sin.cuda(), swa.FP32_EPS)
    for got, ref, n in ((qp, qn, "q"), (kp, kn, "k"), (vp, vn, "v")):
        assert got.shape == (B, T, H, D)
        assert_close_bf16(got, ref, n)
    qb, kb, vb = ops.qkv_prep(q, k, v, cos.cuda(), sin.cuda(), swa.FP32_EPS, bhtd=True)
    assert qb.shape == (B, H, T, D) and torch.equal(qb, qp.transpose(1, 2)) and torch.equal(vb, vp.transpose(1, 2))


@pytest.mark.parametrize("T,window", [(1, None), (5, 3), (63, 16), (128, None), (128, 128), (129, 128), (131, 128),
                                      (256, 1), (300, 2), (300, 64), (300, 200), (300, 1000), (513, 129),
                                      (700, 256), (1024, 512)])
def test_attend_matches_oracle(T, window):
    from daisy_b200 import ops
    B, H = 1, 2
    q, k, v = (bf16_randn(B, T, H, D, seed=10 + i) for i in range(3))
    cos, sin = swa.rope_tables(D, T)
    y_ref, k_ref, v_ref = swa.swa_prefill(q.float().cpu(), k.float().cpu(), v.float().cpu(), cos, sin, window)
    out = torch.full((B, T, H, D), float("nan"), dtype=torch.bfloat16, device="cuda")
    y, kp, vp = ops.swa_prefill(q, k, v, cos.cuda(), sin.cuda(), window, out=out)
    ops.check_device_status(q.device)
    assert_close_bf16(y, y_ref, f"T={T} W={window}")
    assert_close_bf16(kp, k_ref, "k'")
    assert_close_bf16(vp, v_ref, "v'")


def test_attend_reference_fixture_base10000(golden_dir):
    """Reference inner functions (norm, _apply_rope, SDPA with the window mask) on a full base-10000 table."""
    from daisy_b200 import ops
    z = np.load(os.path.join(golden_dir, "swa_inner_small.npz"))
    q, k, v = (torch.from_numpy(z[n]).bfloat16().cuda() for n in ("q", "k", "v"))
    cos, sin = torch.from_numpy(z["cos"]).cuda(), torch.from_numpy(z["sin"]).cuda()
    # the fixture was computed from fp32 inputs; recompute the oracle on the bf16-rounded inputs the kernel sees
    y_ref, _, _ = swa.swa_prefill(q.float().cpu(), k.float().cpu(), v.float().cpu(), cos.cpu(), sin.cpu(), int(z["window"]))
    y, _, _ = ops.swa_prefill(q, k, v, cos, sin, int(z["window"]))
    assert_close_bf16(y, y_ref, "fixture (bf16 inputs)")
    assert_close_bf16(y, torch.from_numpy(z["y"]), "fixture (reference fp32 output)", max_tol=3e-2, mean_tol=3e-3)


def test_attend_batch_heads_and_determinism():
    from daisy_b200 import ops
    B, T, H, window = 3, 520, 4, 192
    qkv = bf16_randn(B, T, 3 * H, D, seed=5)
    q, k, v = qkv.chunk(3, dim=-2)
    cos, sin = swa.rope_tables(D, T)
    y_ref, _, _ = swa.swa_prefill(q.float().cpu(), k.float().cpu(), v.float().cpu(), cos, sin, window)
    y1, _, _ = ops.swa_prefill(q, k, v, cos.cuda(), sin.cuda(), window)
    y2, _, _ = ops.swa_prefill(q, k, v, cos.cuda(), sin.cuda(), window)
    ops.check_device_status(q.device)
    assert_close_bf16(y1, y_ref, "batched")
    assert torch.equal(y1, y2), "prefill is not run-to-run deterministic"


def test_attend_large_logits_rescale_path():
    """Scores that grow along the key axis force the lazy accumulator rescale (max jumps by > 8)."""
    from daisy_b200 import ops
    B, T, H, window = 1, 640, 1, 512
    g = torch.Generator().manual_seed(3)
    q = torch.randn(B, T, H, D, generator=g)
    k = torch.randn(B, T, H, D, generator=g) * torch.linspace(0.2, 6.0, T)[None, :, None, None]
    v = torch.randn(B, T, H, D, generator=g)
    q, k, v = (x.bfloat16().cuda() for x in (q, k, v))
    y_ref = swa.attend_windowed(q.float().cpu(), k.float().cpu(), v.float().cpu(), window, scale=0.5)
    y = ops.swa_attend(q, k, v, window, scale=0.5)
    # the same tensors in [B,H,T,D] memory order reach the kernel through different strides
    yb = ops.swa_attend(*(x.transpose(1, 2).contiguous().transpose(1, 2) for x in (q, k, v)), window, scale=0.5)
    assert torch.equal(y, yb)
    ops.check_device_status(q.device)
    assert_close_bf16(y, y_ref, "rescale", max_tol=4e-2, mean_tol=4e-3)


@pytest.mark.parametrize("T,window", [(7, None), (300, 64), (513, 129), (1300, 512), (2100, 1024)])
def test_attend_bounded_qk_kernel_matches(T, window):
    """DAISY_BOUNDED_QK on prepared (RMS-normalised, rotated) q and k: the kernel with two softmax warpgroups per
    stream and no running maximum gives the oracle's result, and agrees with the general kernel."""
    from daisy_b200 import ops
    B, H = 2, 3
    qkv = bf16_randn(B, T, 3 * H, D, seed=91)
    q, k, v = qkv.chunk(3, dim=-2)
    cos, sin = swa.rope_tables(D, T)
    qp, kp, vp = ops.qkv_prep(q, k, v, cos.cuda(), sin.cuda(), swa.FP32_EPS)
    y_ref = swa.attend_windowed(qp.float().cpu(), kp.float().cpu(), vp.float().cpu(), window)
    y_b = ops.swa_attend(qp, kp, vp, window, bounded_qk=True)
    y_g = ops.swa_attend(qp, kp, vp, window)
    ops.check_device_status(q.device)
    assert_close_bf16(y_b, y_ref, "bounded")
    assert_close_bf16(y_b, y_g.float().cpu(), "bounded vs general", max_tol=1e-2, mean_tol=1e-3)


def test_bounded_qk_is_a_caller_promise():
    """``DAISY_BOUNDED_QK`` promises |q.k| * scale * log2(e) <= 60 for every pair.  The entry point can only check
    what it can see on the host -- the scale against the head dimension (RMS-normalised q and k give |q.k| <= D) --
    and falls back to the general kernel when that bound is out of reach; the tensors themselves are not
    inspected.  When the data break the promise, 2^x without a reference maximum overflows: the affected rows are
    undefined (typically non-finite), rows whose logits stay in range are unaffected, and the general kernel
    (the flag left off) gives the right answer for all of them.  The module path always normalises q and k."""
    from daisy_b200 import ops
    B, T, H, window = 1, 256, 1, 64
    q, k, v = (bf16_randn(B, T, H, D, seed=60 + i) for i in range(3))
    cos, sin = swa.rope_tables(D, T)
    qp, kp, vp = ops.qkv_prep(q, k, v, cos.cuda(), sin.cuda(), swa.FP32_EPS)
    y_ok = ops.swa_attend(qp, kp, vp, window, bounded_qk=True)
    # (1) a scale the bound cannot cover: the flag is ignored, the general kernel runs -- same answer as without it
    y_big_scale = ops.swa_attend(qp, kp, vp, window, scale=0.5, bounded_qk=True)      # 0.5 * 1.4427 * 128 > 60
    assert torch.equal(y_big_scale, ops.swa_attend(qp, kp, vp, window, scale=0.5))
    # (2) the promise broken by the data: rows 128.. of q are 40 x too large (logits up to ~ 40 * 128 * 0.12)
    q_bad = qp.clone()
    q_bad[:, 128:] *= 40.0
    y_gen = ops.swa_attend(q_bad, kp, vp, window)
    ref = swa.attend_windowed(q_bad.float().cpu(), kp.float().cpu(), vp.float().cpu(), window)
    assert_close_bf16(y_gen, ref, "general kernel on out-of-bound logits", max_tol=4e-2, mean_tol=4e-3)
    y_bad = ops.swa_attend(q_bad, kp, vp, window, bounded_qk=True)
    ops.check_device_status("cuda")
    assert torch.equal(y_bad[:, :128], y_ok[:, :128])                    # rows that keep the promise: untouched


@pytest.mark.parametrize("T,window", [(5, 3), (300, 64), (513, 129), (1300, 512)])
def test_q_prepared_in_kernel_matches(T, window):
    """DAISY_Q_IN_KERNEL: Q is normalised and rotated inside the attention kernel (in the swizzled tile, one
    item ahead); same result as the prepared-Q path and the oracle."""
    from daisy_b200 import ops, _lib
    B, H = 2, 3
    qkv = bf16_randn(B, T, 3 * H, D, seed=77)
    q, k, v = qkv.chunk(3, dim=-2)
    cos, sin = swa.rope_tables(D, T)
    y_ref, _, _ = swa.swa_prefill(q.float().cpu(), k.float().cpu(), v.float().cpu(), cos, sin, window)
    y0, k0, _ = ops.swa_prefill(q, k, v, cos.cuda(), sin.cuda(), window)
    y1, k1, _ = ops.swa_prefill(q, k, v, cos.cuda(), sin.cuda(), window, flags=_lib.QKV_DEFAULT | _lib.Q_IN_KERNEL)
    ops.check_device_status(q.device)
    assert_close_bf16(y1, y_ref, "q in kernel")
    assert torch.equal(k0, k1)
    assert (y0.float() - y1.float()).abs().max().item() <= 2e-2
    # flags off: raw attention through the same entry point
    y2, _, _ = ops.swa_prefill(q, k, v, cos.cuda(), sin.cuda(), window, flags=_lib.Q_IN_KERNEL)
    y2r = swa.attend_windowed(q.float().cpu(), k.float().cpu(), v.float().cpu(), window)
    assert_close_bf16(y2, y2r, "no transform")


def _random_doc_starts(B, T, n_docs, seed, per_batch):
    g = torch.Generator().manual_seed(seed)
    rows = []
    for _ in range(B if per_batch else 1):
        cuts = torch.randperm(max(T - 1, 1), generator=g)[:n_docs].sort().values + (1 if T > 1 else 0)
        ds = torch.zeros(T, dtype=torch.int32)
        for c in cuts.tolist():
            if c < T:
                ds[c:] = c
        rows.append(ds)
    return torch.stack(rows) if per_batch else rows[0]


@pytest.mark.parametrize("T,window,n_docs,per_batch", [(9, 4, 2, False), (300, 64, 5, True), (520, None, 3, False),
                                                        (1300, 512, 4, True), (2100, 1024, 7, True),
                                                        (700, 300, 40, False)])
def test_document_mask_matches_oracle(T, window, n_docs, per_batch):
    """Keys before the start of the query's document are invisible (the EOS document mask of
    build_attn_mask); documents start at arbitrary positions, also inside a tile and per batch row."""
    from daisy_b200 import ops
    B, H = 2, 3
    qkv = bf16_randn(B, T, 3 * H, D, seed=T)
    q, k, v = qkv.chunk(3, dim=-2)
    cos, sin = swa.rope_tables(D, T)
    ds = _random_doc_starts(B, T, n_docs, seed=T + 1, per_batch=per_batch)
    y_ref, _, _ = swa.swa_prefill(q.float().cpu(), k.float().cpu(), v.float().cpu(), cos, sin, window, doc_start=ds)
    y, _, _ = ops.swa_prefill(q, k, v, cos.cuda(), sin.cuda(), window, doc_start=ds.cuda())
    ops.check_device_status(q.device)
    assert_close_bf16(y, y_ref, "doc mask, fused step")
    # the attention core alone, both kernels
    qp, kp, vp = ops.qkv_prep(q, k, v, cos.cuda(), sin.cuda(), swa.FP32_EPS)
    for bounded in (True, False):
        ya = ops.swa_attend(qp, kp, vp, window, bounded_qk=bounded, doc_start=ds.cuda())
        assert_close_bf16(ya, y_ref, f"doc mask, attend bounded={bounded}")
    # and the mask really bites: without it the result differs
    y_nodoc, _, _ = ops.swa_prefill(q, k, v, cos.cuda(), sin.cuda(), window)
    assert (y_nodoc.float() - y.float()).abs().max().item() > 1e-2
    ops.check_device_status(q.device)


@pytest.mark.parametrize("logit", [-1.5163, 0.0, 10.0])
def test_prep_value_embedding_gate(logit):
    """qkv_prep with ``ve``: v' = g * norm(v) + (1 - g) * ve with g = sigmoid(g_ve)
    (models/daisy/attention.py:129-136), q' and k' untouched by it; ``ve`` arrives as a strided view."""
    from daisy_b200 import ops
    B, T, H = 2, 77, 3
    qkv = bf16_randn(B, T, 3 * H, D, seed=8)
    q, k, v = qkv.chunk(3, dim=-2)
    ve_wide = bf16_randn(B, T, 2 * H * D, seed=9)
    ve = ve_wide[:, :, H * D:].unflatten(-1, (H, D))               # [B,T,H,D] with a padded token stride
    cos, sin = swa.rope_tables(D, T)
    g = torch.tensor([logit], device="cuda")
    qp, kp, vp = ops.qkv_prep(q, k, v, cos.cuda(), sin.cuda(), swa.FP32_EPS, ve=ve, ve_gate_logit=g)
    q0, k0, v0 = ops.qkv_prep(q, k, v, cos.cuda(), sin.cuda(), swa.FP32_EPS)
    assert torch.equal(qp, q0) and torch.equal(kp, k0)
    gate = torch.sigmoid(torch.tensor(logit))
    ref = gate * swa.rms_norm(v.float().cpu(), swa.FP32_EPS) + (1 - gate) * ve.float().cpu()
    assert_close_bf16(vp, ref, "ve gate")
    with pytest.raises(ValueError):
        ops.qkv_prep(q, k, v, cos.cuda(), sin.cuda(), swa.FP32_EPS, ve=ve)


@pytest.mark.parametrize("T,wb,n_docs", [(256, 1, 0), (1024, 2, 3), (1536, 4, 6), (2048, 3, 30), (1280, 20, 2)])
def test_block_window_training_form_matches_oracle(T, wb, n_docs):
    """DAISY_WINDOW_BLOCKS: the mask the flex BlockMasks of create_blockmasks select -- causal and same
    document per token, the wb nearest key blocks of 128 tokens."""
    from daisy_b200 import ops
    B, H = 2, 2
    qkv = bf16_randn(B, T, 3 * H, D, seed=T + wb)
    q, k, v = qkv.chunk(3, dim=-2)
    cos, sin = swa.rope_tables(D, T)
    ds = _random_doc_starts(B, T, n_docs, seed=wb, per_batch=True) if n_docs else None
    y_ref, _, _ = swa.swa_prefill(q.float().cpu(), k.float().cpu(), v.float().cpu(), cos, sin, None,
                                  doc_start=ds, window_blocks=wb)
    dsc = ds.cuda() if ds is not None else None
    y, _, _ = ops.swa_prefill(q, k, v, cos.cuda(), sin.cuda(), wb, doc_start=dsc, window_in_blocks=True)
    ops.check_device_status(q.device)
    assert_close_bf16(y, y_ref, "block window, fused step")
    qp, kp, vp = ops.qkv_prep(q, k, v, cos.cuda(), sin.cuda(), swa.FP32_EPS)
    ya = ops.swa_attend(qp, kp, vp, wb, doc_start=dsc, window_in_blocks=True)       # the general kernel
    assert_close_bf16(ya, y_ref, "block window, attend")
    if T // 128 > wb and n_docs <= 6:                             # differs from the token-exact window of wb * 128
        y_tok, _, _ = ops.swa_prefill(q, k, v, cos.cuda(), sin.cuda(), wb * 128, doc_start=dsc)
        assert (y_tok.float() - y.float()).abs().max().item() > 1e-3
