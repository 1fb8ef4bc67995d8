"""KDA chunked forward against the fp32 token-by-token recurrence (oracle.kda) and the fixture produced
by the third-party naive recurrence.  Tolerance: relative L2 error <= 1e-3 on the fp32-output variant
(bf16 rounding of the output alone is 1.7e-3, so the bf16 variant is checked against the bf16-rounded
oracle)."""
import os

import numpy as np
import pytest
import torch

from oracle import kda as okda

pytestmark = pytest.mark.gpu
REL_TOL = 1e-3


def _inputs(B, T, H, seed, K=128, gate_scale=1.0):
    g_ = torch.Generator().manual_seed(seed)
    q, k, v = (torch.randn(B, T, H, K, generator=g_).bfloat16() for _ in range(3))
    g = gate_scale * torch.nn.functional.logsigmoid(torch.randn(B, T, H, K, generator=g_))
    beta = torch.sigmoid(torch.randn(B, T, H, generator=g_))
    return q, k, v, g, beta


def _rel(a, b):
    return ((a.float().cpu() - b).norm() / b.norm().clamp_min(1e-20)).item()


def _run(q, k, v, g, beta, **kw):
    from daisy_b200.kda import chunk_kda
    from daisy_b200 import ops
    o, s = chunk_kda(q.cuda(), k.cuda(), v.cuda(), g.cuda(), beta.cuda(), use_qk_l2norm_in_kernel=True, **kw)
    ops.check_device_status("cuda")
    return o, s


@pytest.mark.parametrize("B,T,H", [(1, 64, 1), (1, 1, 2), (1, 100, 2), (2, 300, 3), (1, 640, 2),
                                   (3, 130, 10), (4, 70, 12)])
def test_kda_matches_recurrence(B, T, H):
    q, k, v, g, beta = _inputs(B, T, H, seed=T + H)
    o_ref, s_ref = okda.kda_recurrent(q.float(), k.float(), v.float(), g, beta)
    o, s = _run(q, k, v, g, beta, output_final_state=True, out_fp32=True)
    assert o.dtype == torch.float32 and o.shape == o_ref.shape and s.shape == s_ref.shape
    assert _rel(o, o_ref) <= REL_TOL, f"o rel {_rel(o, o_ref)}"
    assert _rel(s, s_ref) <= REL_TOL, f"state rel {_rel(s, s_ref)}"
    # bf16 output: same numbers rounded once
    ob, _ = _run(q, k, v, g, beta)
    assert ob.dtype == torch.bfloat16
    assert _rel(ob, o_ref.bfloat16().float()) <= 3e-3
    assert (ob.float().cpu() - o_ref).abs().max().item() <= 2e-2


def test_kda_third_party_fixture(golden_dir):
    z = np.load(os.path.join(golden_dir, "kda_naive_small.npz"))
    q, k, v = (torch.from_numpy(z[n]).bfloat16() for n in ("q", "k", "v"))
    g, beta, h0 = (torch.from_numpy(z[n]) for n in ("g", "beta", "h0"))
    o, s = _run(q, k, v, g, beta, output_final_state=True, out_fp32=True)
    assert _rel(o, torch.from_numpy(z["o"])) <= REL_TOL
    assert _rel(s, torch.from_numpy(z["s"])) <= REL_TOL
    o, s = _run(q, k, v, g, beta, initial_state=h0.cuda(), output_final_state=True, out_fp32=True)
    assert _rel(o, torch.from_numpy(z["o_h0"])) <= REL_TOL
    assert _rel(s, torch.from_numpy(z["s_h0"])) <= REL_TOL


def test_kda_strong_decay_and_zero_beta():
    """Per-token log-decay down to about -40 (a factor e^-600 over a 16-token block): every exponent the
    kernel forms is a difference G_i - G_j <= 0, so nothing overflows."""
    q, k, v, g, beta = _inputs(1, 200, 2, seed=5, gate_scale=8.0)
    beta[:, 50:80] = 0.0
    o_ref, s_ref = okda.kda_recurrent(q.float(), k.float(), v.float(), g, beta)
    o, s = _run(q, k, v, g, beta, output_final_state=True, out_fp32=True)
    assert torch.isfinite(o).all() and torch.isfinite(s).all()
    assert _rel(o, o_ref) <= REL_TOL and _rel(s, s_ref) <= REL_TOL


def test_kda_no_l2norm_custom_scale_and_determinism():
    from daisy_b200.kda import chunk_kda
    q, k, v, g, beta = _inputs(1, 192, 2, seed=9)
    qn, kn = okda.l2norm(q.float()).bfloat16(), okda.l2norm(k.float()).bfloat16()
    o_ref, _ = okda.kda_recurrent(qn.float(), kn.float(), v.float(), g, beta, scale=0.2, l2norm_qk=False)
    o1, _ = chunk_kda(qn.cuda(), kn.cuda(), v.cuda(), g.cuda(), beta.cuda(), scale=0.2, out_fp32=True)
    o2, _ = chunk_kda(qn.cuda(), kn.cuda(), v.cuda(), g.cuda(), beta.cuda(), scale=0.2, out_fp32=True)
    assert _rel(o1, o_ref) <= REL_TOL
    assert torch.equal(o1, o2)


def test_kda_chunked_state_carry():
    """Two calls of 128 tokens chained through the final state == one call of 256 tokens."""
    q, k, v, g, beta = _inputs(2, 256, 2, seed=11)
    o_full, s_full = _run(q, k, v, g, beta, output_final_state=True, out_fp32=True)
    o_a, s_a = _run(q[:, :128], k[:, :128], v[:, :128], g[:, :128], beta[:, :128], output_final_state=True, out_fp32=True)
    o_b, s_b = _run(q[:, 128:], k[:, 128:], v[:, 128:], g[:, 128:], beta[:, 128:], initial_state=s_a,
                    output_final_state=True, out_fp32=True)
    assert _rel(torch.cat([o_a, o_b], 1), o_full.cpu()) <= 1e-5
    assert _rel(s_b, s_full.cpu()) <= 1e-5
