"""Decode kernel (split-KV over the ring cache) against the fp32 oracle."""
import pytest
import torch

from gpu_util import bf16_randn, assert_close_bf16
from oracle import swa

pytestmark = pytest.mark.gpu

B, H, D = 2, 3, 128


def _oracle_ctx(ring_k, ring_v, t, cap):
    """Chronological [B,n,H,D] context the reference's KVCache.view would return (n = min(t,cap))."""
    n = min(t, cap)
    idx = (torch.arange(t - n, t) % cap)
    return ring_k[:, :, idx].transpose(1, 2).float().cpu(), ring_v[:, :, idx].transpose(1, 2).float().cpu()


@pytest.mark.parametrize("t", [0, 1, 5, 15, 16, 47, 48, 49, 100, 1000])
@pytest.mark.parametrize("window,cap", [(16, 48), (48, 48), (100, 48), (None, 48)])
@pytest.mark.parametrize("splits", [1, 3])
def test_decode_ring_matches_oracle(t, window, cap, splits):
    from daisy_b200 import ops
    ring_k, ring_v = bf16_randn(B, H, cap, D, seed=t), bf16_randn(B, H, cap, D, seed=t + 7)
    q, k, v = (bf16_randn(B, 1, H, D, seed=100 + i + t) for i in range(3))
    cos, sin = swa.rope_tables(D, t + 1)
    kc, vc = _oracle_ctx(ring_k, ring_v, t, cap)
    y_ref, k_ref, v_ref = swa.decode_step(q.float().cpu(), k.float().cpu(), v.float().cpu(), kc, vc, t, window, cos, sin)
    before_k = ring_k.clone()
    y, k_new, v_new = ops.swa_decode_step(q, k, v, ring_k, ring_v, t, cap, window, cos[t].cuda(), sin[t].cuda(),
                                          write_ring=True, splits=splits)
    ops.check_device_status(q.device)
    assert_close_bf16(y, y_ref, f"y t={t} w={window}")
    assert_close_bf16(k_new, k_ref, "k_new")
    assert_close_bf16(v_new, v_ref, "v_new")
    # ring: only slot t % cap changed, and it holds the new row
    slot = t % cap
    assert torch.equal(ring_k[:, :, slot], k_new[:, 0])
    assert torch.equal(ring_v[:, :, slot], v_new[:, 0])
    mask = torch.ones(cap, dtype=torch.bool); mask[slot] = False
    assert torch.equal(ring_k[:, :, mask], before_k[:, :, mask])


def test_decode_plain_context_tensor():
    """A chronological [B,n,H,D] context (what the protocol's step() receives) is the ring special case cap=n."""
    from daisy_b200 import ops
    n, window = 37, 20
    ctx_k, ctx_v = bf16_randn(B, n, H, D, seed=1), bf16_randn(B, n, H, D, seed=2)
    q, k, v = (bf16_randn(B, 1, H, D, seed=3 + i) for i in range(3))
    cos, sin = swa.rope_tables(D, n + 1)
    y_ref, _, _ = swa.decode_step(q.float().cpu(), k.float().cpu(), v.float().cpu(), ctx_k.float().cpu(),
                                  ctx_v.float().cpu(), n, window, cos, sin)
    y, _, _ = ops.swa_decode_step(q, k, v, ctx_k.transpose(1, 2), ctx_v.transpose(1, 2), n, n, window,
                                  cos[n].cuda(), sin[n].cuda())
    assert_close_bf16(y, y_ref, "plain ctx")


def test_decode_strided_qkv_and_flags():
    """q,k,v as views of a merged [B,1,3H,D] projection; transform flags off = raw attention."""
    from daisy_b200 import ops, _lib
    cap, t, window = 64, 200, 33
    ring_k, ring_v = bf16_randn(B, H, cap, D, seed=11), bf16_randn(B, H, cap, D, seed=12)
    qkv = bf16_randn(B, 1, 3 * H, D, seed=13)
    q, k, v = qkv.chunk(3, dim=-2)
    idx = torch.arange(t - cap, t) % cap
    kc = ring_k[:, :, idx].transpose(1, 2).float().cpu(); vc = ring_v[:, :, idx].transpose(1, 2).float().cpu()
    y_ref, _, _ = swa.decode_step(q.float().cpu(), k.float().cpu(), v.float().cpu(), kc, vc, t, window, None, None,
                                  norm_q=False, norm_k=False, norm_v=False, rope=False)
    y, _, _ = ops.swa_decode_step(q, k, v, ring_k, ring_v, t, cap, window, None, None, flags=0)
    assert_close_bf16(y, y_ref, "flags=0")


def test_decode_long_window_many_splits():
    from daisy_b200 import ops
    cap, t, window = 4096, 5000, 4096
    ring_k, ring_v = bf16_randn(1, 2, cap, D, seed=21), bf16_randn(1, 2, cap, D, seed=22)
    q, k, v = (bf16_randn(1, 1, 2, D, seed=23 + i) for i in range(3))
    cos, sin = swa.rope_tables(D, t + 1)
    idx = torch.arange(t - cap, t) % cap
    kc = ring_k[:, :, idx].transpose(1, 2).float().cpu(); vc = ring_v[:, :, idx].transpose(1, 2).float().cpu()
    y_ref, _, _ = swa.decode_step(q.float().cpu(), k.float().cpu(), v.float().cpu(), kc, vc, t, window, cos, sin)
    for splits in (None, 1, 7, 32):
        y, _, _ = ops.swa_decode_step(q, k, v, ring_k, ring_v, t, cap, window, cos[t].cuda(), sin[t].cuda(), splits=splits)
        assert_close_bf16(y, y_ref, f"splits={splits}")
    y2, _, _ = ops.swa_decode_step(q, k, v, ring_k, ring_v, t, cap, window, cos[t].cuda(), sin[t].cuda(), splits=32)
    assert torch.equal(y, y2), "decode is not run-to-run deterministic"


@pytest.mark.parametrize("t,window,cap", [(0, 16, 48), (30, 16, 48), (100, None, 48), (1000, 100, 48)])
def test_decode_float16_ring(t, window, cap):
    """The ring may hold float16 rows (the reference Generator's default cache dtype, inference/generate.py:62)
    while q, k, v are bf16: rows are read as fp16, the new row is stored as fp16 and attended at that precision."""
    from daisy_b200 import ops
    ring_k = bf16_randn(B, H, cap, D, seed=t).to(torch.float16)
    ring_v = bf16_randn(B, H, cap, D, seed=t + 7).to(torch.float16)
    q, k, v = (bf16_randn(B, 1, H, D, seed=200 + i + t) for i in range(3))
    cos, sin = swa.rope_tables(D, t + 1)
    kc, vc = _oracle_ctx(ring_k, ring_v, t, cap)
    y_ref, k_ref, v_ref = swa.decode_step(q.float().cpu(), k.float().cpu(), v.float().cpu(), kc, vc, t, window, cos, sin)
    y, k_new, v_new = ops.swa_decode_step(q, k, v, ring_k, ring_v, t, cap, window, cos[t].cuda(), sin[t].cuda(), write_ring=True)
    ops.check_device_status(q.device)
    assert_close_bf16(y, y_ref, f"y fp16 ring t={t}")
    slot = t % cap
    assert ring_k.dtype == torch.float16
    assert (ring_k[:, :, slot].float().cpu() - k_ref[:, 0]).abs().max().item() <= 4e-3 * max(1.0, k_ref.abs().max().item())
    assert (ring_v[:, :, slot].float().cpu() - v_ref[:, 0]).abs().max().item() <= 4e-3 * max(1.0, v_ref.abs().max().item())


@pytest.mark.parametrize("t,window,cap,splits", [(0, 16, 48, None), (30, 16, 48, 3), (100, None, 48, None), (1000, 100, 48, 2),
                                                 (5000, 4096, 4096, 13), (20, 40, 16, None)])
@pytest.mark.parametrize("f16", [False, True])
def test_fused_single_launch_decode_equals_two_launch_form(t, window, cap, splits, f16):
    """``daisy_b200_swa_decode_step_fused`` (the last split CTA of a (batch, head) merges the partials itself) gives the
    bits of the partial + combine pair: outputs, new rows, ring contents -- with the position on the host and on the
    device, called twice in a row on one workspace (the tickets must come back to zero)."""
    from daisy_b200 import ops
    mk = lambda seed: bf16_randn(B, H, cap, D, seed=seed).to(torch.float16 if f16 else torch.bfloat16)
    ring0 = (mk(t), mk(t + 5))
    q, k, v = (bf16_randn(B, 1, H, D, seed=300 + i + t) for i in range(3))
    cos, sin = swa.rope_tables(D, t + 2)
    cos, sin = cos.cuda(), sin.cuda()
    rk, rv = ring0[0].clone(), ring0[1].clone()
    y_ref, k_ref, v_ref = ops.swa_decode_step(q, k, v, rk, rv, t, cap, window, cos[t], sin[t], write_ring=True, splits=splits)
    r = min(t, cap) if not window else min(t, cap, window - 1)
    sp = splits or ops.decode_splits(B, H, r)
    ws = ops.decode_fused_workspace(B, H, D, sp, q.device)
    for rep in range(2):
        fk, fv = ring0[0].clone(), ring0[1].clone()
        y, kn, vn = ops.swa_decode_step_fused(q, k, v, fk, fv, t, cap, window, cos[t], sin[t], splits=sp, workspace=ws,
                                              return_new_kv=True)
        assert torch.equal(y, y_ref) and torch.equal(kn, k_ref) and torch.equal(vn, v_ref), f"host position, call {rep}"
        assert torch.equal(fk, rk) and torch.equal(fv, rv)
    fk, fv = ring0[0].clone(), ring0[1].clone()
    t_dev = torch.tensor([t], device="cuda", dtype=torch.int64)
    r_max = cap if not window else min(cap, window - 1)
    sp_dev = ops.decode_splits(B, H, r_max)
    y = ops.swa_decode_step_fused(q, k, v, fk, fv, t_dev, cap, window, cos, sin, splits=sp_dev)
    ops.check_device_status(q.device)
    y2, _, _ = ops.swa_decode_step(q, k, v, ring0[0].clone(), ring0[1].clone(), t, cap, window, cos[t], sin[t], write_ring=True, splits=sp_dev)
    assert torch.equal(y, y2), "device position"
    assert torch.equal(fk, rk) and torch.equal(fv, rv)
    assert int(ws.view(torch.int32)[-B * H:].abs().sum()) == 0, "tickets must be left at zero"


def test_fused_decode_value_embedding_gate():
    """The value-embedding gate on the new token inside the decode kernel (models/daisy/attention.py:132-135 on the
    single-token path): v = g * norm(v) + (1 - g) * ve, against the oracle with the mixed v fed in."""
    from daisy_b200 import ops, _lib
    t, window, cap = 77, 40, 64
    ring_k, ring_v = bf16_randn(B, H, cap, D, seed=1), bf16_randn(B, H, cap, D, seed=2)
    q, k, v = (bf16_randn(B, 1, H, D, seed=400 + i) for i in range(3))
    ve = bf16_randn(B, 1, H * D, seed=404)
    logit = torch.tensor([-1.5163], device="cuda")
    cos, sin = swa.rope_tables(D, t + 1)
    kc, vc = _oracle_ctx(ring_k, ring_v, t, cap)
    g = torch.sigmoid(torch.tensor(-1.5163))
    v_mixed = g * swa.rms_norm(v.float().cpu(), swa.FP32_EPS) + (1 - g) * ve.float().cpu().view(B, 1, H, D)
    y_ref, _, v_ref = swa.decode_step(q.float().cpu(), k.float().cpu(), v_mixed, kc, vc, t, window, cos, sin, norm_v=False)
    y, _, v_new = ops.swa_decode_step_fused(q, k, v, ring_k, ring_v, t, cap, window, cos[t].cuda(), sin[t].cuda(),
                                            ve=ve, ve_gate_logit=logit, return_new_kv=True)
    ops.check_device_status(q.device)
    assert_close_bf16(y, y_ref, "y with ve")
    assert_close_bf16(v_new, v_ref, "v' with ve")
    assert torch.equal(ring_v[:, :, t % cap], v_new[:, 0])
