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
