"""The benchmark configurations at their full sizes, checked through properties that do not need a
full-size CPU run: sampled (batch, head) slices and query blocks against the fp32 oracle, shard invariance
(a batch row / a head group computed alone gives bit-identical results: the multi-GPU sharding relies on it),
state chaining for the KDA, and finiteness everywhere."""
import pytest
import torch

from gpu_util import assert_close_bf16
from oracle import swa
from oracle import kda as okda

pytestmark = pytest.mark.gpu
D = 128


def _randn_bf16(shape, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return torch.randn(*shape, device="cuda", generator=g).bfloat16()


def _rope(T, base=10000.0):
    cos, sin = swa.rope_tables(D, T, base=base, truncate=False)
    return cos.cuda(), sin.cuda()


def test_prefill_c2_full_size():
    """B=8, T=8192, 16 heads, window 2048 (the headline prefill configuration)."""
    from daisy_b200 import ops
    B, T, H, W = 8, 8192, 16, 2048
    q, k, v = (_randn_bf16((B, T, H, D), 10 + i) for i in range(3))
    cos, sin = _rope(T)
    y, kp, vp = ops.swa_prefill(q, k, v, cos, sin, W, eps=swa.FP32_EPS)
    ops.check_device_status("cuda")
    assert torch.isfinite(y.float()).all()
    # sampled (b, h) slices against the oracle on the same raw inputs
    for b, h in ((0, 0), (5, 11), (7, 15)):
        sl = lambda x: x[b:b + 1, :, h:h + 1].float().cpu()
        y_ref, k_ref, v_ref = swa.swa_prefill(sl(q), sl(k), sl(v), cos.cpu(), sin.cpu(), W)
        assert_close_bf16(y[b:b + 1, :, h:h + 1], y_ref, f"y[{b},{h}]")
        assert_close_bf16(kp[b:b + 1, h:h + 1], k_ref, f"k'[{b},{h}]")
        assert_close_bf16(vp[b:b + 1, h:h + 1], v_ref, f"v'[{b},{h}]")
    # shard invariance: one batch row alone, and a head group alone (strided views), bit for bit
    y1, _, _ = ops.swa_prefill(q[3:4], k[3:4], v[3:4], cos, sin, W, eps=swa.FP32_EPS)
    assert torch.equal(y1[0], y[3])
    y2, _, _ = ops.swa_prefill(q[:, :, 4:8], k[:, :, 4:8], v[:, :, 4:8], cos, sin, W, eps=swa.FP32_EPS)
    assert torch.equal(y2, y[:, :, 4:8])


def test_prefill_c4_full_size():
    """B=1, T=65536, 16 heads, window 8192 (the long-context prefill configuration): sampled query blocks of sampled heads."""
    from daisy_b200 import ops
    B, T, H, W = 1, 65536, 16, 8192
    q, k, v = (_randn_bf16((B, T, H, D), 20 + i) for i in range(3))
    cos, sin = _rope(T)
    qp, kp, vp = ops.qkv_prep(q, k, v, cos, sin, swa.FP32_EPS)
    y = ops.swa_attend(qp, kp, vp, W, bounded_qk=True)
    ops.check_device_status("cuda")
    assert torch.isfinite(y.float()).all()
    for h, q0 in ((0, 0), (3, 8100), (9, 30000), (15, T - 256)):
        q1, k0 = q0 + 256, max(0, q0 - W + 1)
        qs = qp[:, q0:q1, h:h + 1].float().cpu()
        ks, vs = kp[:, k0:q1, h:h + 1].float().cpu(), vp[:, k0:q1, h:h + 1].float().cpu()
        s = torch.einsum("bqhd,bkhd->bhqk", qs, ks) * swa.ATTN_SCALE
        s = s + swa.window_mask(q0, q1, k0, q1, W)
        ref = torch.einsum("bhqk,bkhd->bqhd", torch.softmax(s, dim=-1), vs)
        assert_close_bf16(y[:, q0:q1, h:h + 1], ref, f"block h={h} q0={q0}")
    # head shards 16 -> 2 x 8 as in the multi-GPU partition: identical bits
    y_lo = ops.swa_attend(qp[:, :, :8], kp[:, :, :8], vp[:, :, :8], W, bounded_qk=True)
    assert torch.equal(y_lo, y[:, :, :8])


def test_decode_c3_full_size():
    """Batch 64, 16 heads, ring capacity 32768, window 4096, steps that wrap the ring (the decode configuration)."""
    from daisy_b200 import ops
    B, H, cap, W = 64, 16, 32768, 4096
    kc = torch.empty(B, H, cap, D, dtype=torch.bfloat16, device="cuda")
    vc = torch.empty_like(kc)
    g = torch.Generator(device="cuda").manual_seed(31)
    for b in range(B):                                             # 8.6 GB per tensor, filled row by row
        kc[b] = torch.randn(H, cap, D, device="cuda", generator=g).bfloat16()
        vc[b] = torch.randn(H, cap, D, device="cuda", generator=g).bfloat16()
    cos, sin = swa.rope_tables(D, cap + 8, base=10000.0, truncate=False)
    t = cap + 1                                                    # the ring has wrapped once
    for step in range(3):
        qn, kn, vn = (_randn_bf16((B, 1, H, D), 40 + 3 * step + i) for i in range(3))
        # the oracle's chronological context for sampled (b, h), gathered before the step overwrites a slot
        samples = ((0, 0), (17, 5), (63, 15))
        idx = (torch.arange(t - (W - 1), t) % cap).cuda()
        ctx = {bh: (kc[bh[0], bh[1]][idx].float().cpu(), vc[bh[0], bh[1]][idx].float().cpu()) for bh in samples}
        y, k_new, v_new = ops.swa_decode_step(qn, kn, vn, kc, vc, t, cap, W, cos[t].cuda(), sin[t].cuda(), write_ring=True)
        ops.check_device_status("cuda")
        assert torch.isfinite(y.float()).all()
        for (b, h), (ck, cv) in ctx.items():
            sl = lambda x: x[b:b + 1, :, h:h + 1].float().cpu()
            y_ref, k_ref, _ = swa.decode_step(sl(qn), sl(kn), sl(vn), ck[None, :, None], cv[None, :, None], t, W, cos, sin)
            assert_close_bf16(y[b:b + 1, :, h:h + 1], y_ref, f"step {step} y[{b},{h}]")
            assert_close_bf16(k_new[b:b + 1, :, h:h + 1], k_ref, "k_new")
        assert torch.equal(kc[:, :, t % cap], k_new[:, 0])         # the new row landed in its slot
        t += 1


def test_kda_c5_full_size():
    """B=4, T=16384, 16 heads, K=V=128 (the KDA configuration): sampled (b, h) against the fp32 recurrence --
    prefixes, and for one pair the WHOLE length (every output row, the last 256 rows on their own, the final
    state), so drift of the fp32 state over 256 chunks is compared with the recurrence and not only with the
    kernel itself; one call over T against two calls over T/2 chained through the state; and the per-GPU shapes of
    the multi-GPU partition (8 (batch, head) pairs = half the heads of one batch row) give the same bits."""
    from daisy_b200 import ops
    B, T, H = 4, 16384, 16
    g_ = torch.Generator(device="cuda").manual_seed(50)
    q, k, v = (torch.randn(B, T, H, D, device="cuda", generator=g_).bfloat16() for _ in range(3))
    g = torch.nn.functional.logsigmoid(torch.randn(B, T, H, D, device="cuda", generator=g_))
    beta = torch.sigmoid(torch.randn(B, T, H, device="cuda", generator=g_))
    o, s = ops.kda_chunk_fwd(q, k, v, g, beta, None, None, True, out_fp32=True)
    ops.check_device_status("cuda")
    assert torch.isfinite(o).all() and torch.isfinite(s).all()
    n = 1024
    for b, h in ((0, 0), (3, 15)):
        sl = lambda x: x[b:b + 1, :n, h:h + 1].float().cpu()
        o_ref, _ = okda.kda_recurrent(sl(q), sl(k), sl(v), sl(g), beta[b:b + 1, :n, h:h + 1].cpu())
        rel = ((o[b:b + 1, :n, h:h + 1].cpu() - o_ref).norm() / o_ref.norm()).item()
        assert rel <= 1e-3, rel
    # full length for one (b, h): 16384 steps of the CPU recurrence (seconds)
    b, h = 2, 7
    sl = lambda x: x[b:b + 1, :, h:h + 1].float().cpu()
    o_ref, s_ref = okda.kda_recurrent(sl(q), sl(k), sl(v), sl(g), beta[b:b + 1, :, h:h + 1].cpu())
    o_bh = o[b:b + 1, :, h:h + 1].cpu()
    assert ((o_bh - o_ref).norm() / o_ref.norm()).item() <= 1e-3
    assert ((o_bh[:, -256:] - o_ref[:, -256:]).norm() / o_ref[:, -256:].norm()).item() <= 1e-3
    assert ((s[b:b + 1, h:h + 1].cpu() - s_ref).norm() / s_ref.norm()).item() <= 1e-3
    # the shard one GPU of eight computes: heads 0..7 of batch row 2, as its own contiguous tensors
    shard = lambda x: x[b:b + 1, :, :8].contiguous()
    o_sh, s_sh = ops.kda_chunk_fwd(shard(q), shard(k), shard(v), shard(g), shard(beta), None, None, True, out_fp32=True)
    # (8 pairs per GPU run the state pass with the K dimension split over four warps: another summation order)
    rel = lambda a, r: ((a - r).norm() / r.norm()).item()
    assert rel(o_sh, o[b:b + 1, :, :8]) <= 1e-4 and rel(s_sh, s[b:b + 1, :8]) <= 1e-4
    half = T // 2
    cut = lambda x, a, b_: x[:, a:b_].contiguous()
    o1, s1 = ops.kda_chunk_fwd(cut(q, 0, half), cut(k, 0, half), cut(v, 0, half), cut(g, 0, half), cut(beta, 0, half),
                               None, None, True, out_fp32=True)
    o2, s2 = ops.kda_chunk_fwd(cut(q, half, T), cut(k, half, T), cut(v, half, T), cut(g, half, T), cut(beta, half, T),
                               None, s1, True, out_fp32=True)
    assert torch.equal(o1, o[:, :half])                            # chunks are independent of what follows
    assert ((o2 - o[:, half:]).norm() / o[:, half:].norm()).item() <= 1e-6
    assert ((s2 - s).norm() / s.norm()).item() <= 1e-6


def test_backward_c2_full_size():
    """The attention backward at the headline shape (B=8, T=8192, 16 heads, window 2048): dq, dk, dv of sampled
    (batch, head) pairs against ``torch.autograd`` over the fp32 oracle run on that pair's whole sequence; one batch row
    computed alone gives the same bits; two runs give the same bits."""
    from daisy_b200 import ops
    B, T, H, W = 8, 8192, 16, 2048
    q, k, v = (_randn_bf16((B, T, H, D), 60 + i) for i in range(3))
    cos, sin = _rope(T)
    qp, kp, vp = ops.qkv_prep(q, k, v, cos, sin, swa.FP32_EPS)
    d_o = _randn_bf16((B, T, H, D), 64)
    y, lse = ops.swa_attend(qp, kp, vp, W, bounded_qk=True, return_lse=True)
    dq, dk, dv = ops.swa_attend_bwd(qp, kp, vp, y, d_o, lse, W)
    ops.check_device_status("cuda")
    assert all(torch.isfinite(t.float()).all() for t in (dq, dk, dv))
    for b, h in ((0, 0), (6, 13)):
        sl = lambda x: x[b:b + 1, :, h:h + 1].float().cpu()
        y_ref, *ref = swa.attend_backward(sl(qp), sl(kp), sl(vp), sl(d_o), W)
        assert_close_bf16(y[b:b + 1, :, h:h + 1], y_ref, f"y[{b},{h}]")
        for got, r, n in zip((dq, dk, dv), ref, ("dq", "dk", "dv")):
            g = got[b:b + 1, :, h:h + 1]
            assert_close_bf16(g, r, f"{n}[{b},{h}]")
            rel = ((g.float().cpu() - r).norm() / r.norm()).item()
            assert rel <= 2e-2, f"{n}[{b},{h}]: relative L2 {rel}"
    again = ops.swa_attend_bwd(qp, kp, vp, y, d_o, lse, W)
    assert all(torch.equal(a, b_) for a, b_ in zip((dq, dk, dv), again))
    row = ops.swa_attend_bwd(qp[2:3], kp[2:3], vp[2:3], y[2:3], d_o[2:3], lse[2:3], W)
    assert all(torch.equal(a[0], b_[2]) for a, b_ in zip(row, (dq, dk, dv)))
