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


def test_kda_decode_steps_carry_state():
    """Prefill through the chunked kernels, then single-token calls (the token-by-token kernel) that carry
    the state: the reference's decode pattern (chunk_kda with T = 1 and the cached state)."""
    from daisy_b200 import ops
    from daisy_b200.kda import chunk_kda, RECURRENT_MAX_T
    B, T0, n_steps, H = 2, 130, 6, 3
    q, k, v, g, beta = _inputs(B, T0 + n_steps + 3, H, seed=21)
    o_ref, s_ref = okda.kda_recurrent(q.float(), k.float(), v.float(), g, beta)
    dev = [x.cuda() for x in (q, k, v, g, beta)]
    cut = lambda a, b: [x[:, a:b].contiguous() for x in dev]
    o0, state = chunk_kda(*cut(0, T0), output_final_state=True, use_qk_l2norm_in_kernel=True, out_fp32=True)
    outs = [o0]
    for t in range(T0, T0 + n_steps):
        o1, state = chunk_kda(*cut(t, t + 1), initial_state=state, output_final_state=True,
                              use_qk_l2norm_in_kernel=True, out_fp32=True)
        outs.append(o1)
    # a short multi-token block, state updated in place
    assert 3 <= RECURRENT_MAX_T
    o3, state2 = ops.kda_recurrent_fwd(*cut(T0 + n_steps, T0 + n_steps + 3), initial_state=state,
                                       l2norm_qk=True, out_fp32=True, state_in_place=True)
    assert state2.data_ptr() == state.data_ptr()
    outs.append(o3)
    ops.check_device_status("cuda")
    o = torch.cat(outs, dim=1)
    assert _rel(o, o_ref) <= REL_TOL
    assert _rel(state, s_ref) <= REL_TOL


@pytest.mark.parametrize("T", [1, 2, 4])
def test_kda_recurrent_kernel_matches_oracle_and_chunk_kernel(T):
    from daisy_b200 import ops
    B, H = 3, 5
    q, k, v, g, beta = _inputs(B, T, H, seed=40 + T)
    h0 = torch.randn(B, H, 128, 128, generator=torch.Generator().manual_seed(T)) * 0.3
    o_ref, s_ref = okda.kda_recurrent(q.float(), k.float(), v.float(), g, beta, initial_state=h0)
    dev = [x.cuda() for x in (q, k, v, g, beta)]
    o_r, s_r = ops.kda_recurrent_fwd(*dev, initial_state=h0.cuda(), output_final_state=True, out_fp32=True)
    o_c, s_c = ops.kda_chunk_fwd(*dev, initial_state=h0.cuda(), output_final_state=True, out_fp32=True)
    ops.check_device_status("cuda")
    assert _rel(o_r, o_ref) <= 1e-5 and _rel(s_r, s_ref) <= 1e-5          # fp32 arithmetic end to end
    assert _rel(o_c, o_ref) <= REL_TOL and _rel(s_c, s_ref) <= REL_TOL
    o_b, _ = ops.kda_recurrent_fwd(*dev, initial_state=h0.cuda())
    assert o_b.dtype == torch.bfloat16 and _rel(o_b, o_ref.bfloat16().float()) <= 4e-3


def test_kda_gate_matches_reference_fixture(golden_dir):
    """The gate kernel against values produced by the reference's own ``_gate_impl``
    (models/daisy/fla_custom_ops.py:71-103): fp32 input, bf16 input (result rounded to bf16 like the
    reference's cast), no bias; softplus threshold crossed on both sides."""
    from daisy_b200 import ops
    from daisy_b200.kda import fused_kda_gate
    d = np.load(os.path.join(golden_dir, "kda_gate_small.npz"))
    x, A, bias = (torch.from_numpy(d[n]).cuda() for n in ("x", "A_log", "bias"))
    y = ops.kda_gate(x, A, 128, bias)
    ref = torch.from_numpy(d["y_fp32"])
    assert y.shape == ref.shape
    assert ((y.cpu() - ref).abs() <= 2e-6 * ref.abs() + 1e-6).all()
    y_nb = ops.kda_gate(x, A, 128, None)
    ref_nb = torch.from_numpy(d["y_nobias"])
    assert ((y_nb.cpu() - ref_nb).abs() <= 2e-6 * ref_nb.abs() + 1e-6).all()
    yb, bs = fused_kda_gate(x.bfloat16(), A, 128, bias)
    refb = torch.from_numpy(d["y_bf16_as_fp32"])
    assert yb.dtype == torch.bfloat16 and bs.shape == (*x.shape[:-1], 3) and not bs.any()
    # identical up to one bf16 ulp where the fp32 value sits on a rounding boundary
    assert ((yb.float().cpu() - refb).abs() <= refb.abs() * 2.0 ** -7).all()
    assert (yb.float().cpu() == refb).float().mean().item() > 0.999


def test_chunk_kda_against_fla_triton():
    """The function the reference itself calls (fla.ops.kda.chunk_kda, models/daisy/attention_kimi.py:133-134, with
    use_qk_l2norm_in_kernel=True), run on this GPU where the third-party package works: same inputs, with an
    initial state and the final state returned, T not a multiple of the chunk.  Skips if fla / Triton cannot run."""
    try:
        from fla.ops.kda import chunk_kda as fla_chunk_kda
    except Exception as e:
        pytest.skip(f"fla not importable: {e}")
    from daisy_b200.kda import chunk_kda
    B, T, H, K = 2, 333, 4, 128
    g_ = torch.Generator(device="cuda").manual_seed(77)
    q, k, v = (torch.randn(B, T, H, K, device="cuda", generator=g_).bfloat16() for _ in range(3))
    g = torch.nn.functional.logsigmoid(torch.randn(B, T, H, K, device="cuda", generator=g_))
    beta = torch.sigmoid(torch.randn(B, T, H, device="cuda", generator=g_))
    h0 = torch.randn(B, H, K, K, device="cuda", generator=g_) * 0.1
    try:
        with torch.no_grad():
            o_ref, s_ref = fla_chunk_kda(q=q, k=k, v=v, g=g, beta=beta, initial_state=h0.clone(), output_final_state=True,
                                         use_qk_l2norm_in_kernel=True)
        torch.cuda.synchronize()
    except Exception as e:
        pytest.skip(f"fla's Triton kernels did not run here: {type(e).__name__}: {e}")
    o, s = chunk_kda(q=q, k=k, v=v, g=g, beta=beta, initial_state=h0, output_final_state=True,
                     use_qk_l2norm_in_kernel=True)
    rel_o = ((o.float() - o_ref.float()).norm() / o_ref.float().norm()).item()
    rel_s = ((s.float() - s_ref.float()).norm() / s_ref.float().norm()).item()
    # both sides round their output to bf16 (1.7e-3 of rounding noise each) and differ in internal precision
    assert rel_o <= 5e-3, rel_o
    assert rel_s <= 5e-3, rel_s
    # and both sit equally close to the fp32 recurrence
    o_or, s_or = okda.kda_recurrent(q.float().cpu(), k.float().cpu(), v.float().cpu(), g.cpu(), beta.cpu(), None, h0.cpu(), True)
    ours = ((o.float().cpu() - o_or).norm() / o_or.norm()).item()
    theirs = ((o_ref.float().cpu() - o_or).norm() / o_or.norm()).item()
    assert ours <= max(3e-3, 1.5 * theirs), (ours, theirs)


# ------------------------------------------------------------------------------------ packed variable-length batches
VARLEN_CASES = [[0, 64], [0, 1], [0, 5, 69], [0, 100, 100, 164, 421], [0, 64, 128, 192], [0, 63, 65, 130, 700],
                [0, 0, 7], [0, 1000, 1001]]


@pytest.mark.parametrize("cu", VARLEN_CASES)
@pytest.mark.parametrize("with_state", [False, True])
def test_kda_varlen_matches_per_sequence_recurrence(cu, with_state):
    """chunk_kda(..., cu_seqlens=...): sequences of ragged lengths (one token, empty, chunk multiples, a partial last
    chunk next to the following sequence's first tokens) packed into one row; each must equal the recurrence run on
    it alone, from its own initial state."""
    N, T, H = len(cu) - 1, cu[-1], 3
    q, k, v, g, beta = _inputs(1, T, H, seed=11 + T + N)
    h0 = torch.randn(N, H, 128, 128, generator=torch.Generator().manual_seed(5)) * 0.1 if with_state else None
    o_ref, s_ref = okda.kda_recurrent_varlen(q.float(), k.float(), v.float(), g, beta, cu, None, h0)
    o, s = _run(q, k, v, g, beta, cu_seqlens=torch.tensor(cu, dtype=torch.int32, device="cuda"),
                initial_state=None if h0 is None else h0.cuda(), output_final_state=True, out_fp32=True)
    assert o.shape == o_ref.shape and s.shape == s_ref.shape
    assert _rel(o, o_ref) <= REL_TOL, f"o rel {_rel(o, o_ref)}"
    assert _rel(s, s_ref) <= REL_TOL, f"state rel {_rel(s, s_ref)}"
    for n, (a, b) in enumerate(zip(cu, cu[1:])):                    # per sequence, so that a short one cannot hide
        if b > a:
            assert _rel(o[:, a:b], o_ref[:, a:b]) <= 2 * REL_TOL, f"sequence {n}"
        assert _rel(s[n], s_ref[n]) <= 2 * REL_TOL or s_ref[n].norm() == 0, f"state of sequence {n}"
    if not with_state and 0 in [b - a for a, b in zip(cu, cu[1:])]:
        n = [b - a for a, b in zip(cu, cu[1:])].index(0)
        assert not s[n].any()


def test_kda_varlen_equals_dense_per_sequence():
    """A packed batch gives, sequence by sequence, the bits of the dense call on that sequence alone (the chunking
    starts at each sequence's own first token)."""
    cu = [0, 130, 194, 500]
    q, k, v, g, beta = _inputs(1, cu[-1], 2, seed=41)
    o, s = _run(q, k, v, g, beta, cu_seqlens=cu, output_final_state=True)
    for n, (a, b) in enumerate(zip(cu, cu[1:])):
        od, sd = _run(q[:, a:b].contiguous(), k[:, a:b].contiguous(), v[:, a:b].contiguous(), g[:, a:b].contiguous(),
                      beta[:, a:b].contiguous(), output_final_state=True)
        assert torch.equal(o[:, a:b], od) and torch.equal(s[n], sd[0]), f"sequence {n}"


def test_kda_varlen_against_fla_triton():
    """fla.ops.kda.chunk_kda with cu_seqlens on this GPU, the call the reference makes for a masked batch."""
    try:
        from fla.ops.kda import chunk_kda as fla_chunk_kda
    except Exception as e:
        pytest.skip(f"fla not importable: {e}")
    from daisy_b200.kda import chunk_kda
    cu, H, K = [0, 70, 333, 400], 4, 128
    T, N = cu[-1], len(cu) - 1
    g_ = torch.Generator(device="cuda").manual_seed(78)
    q, k, v = (torch.randn(1, T, H, K, device="cuda", generator=g_).bfloat16() for _ in range(3))
    g = torch.nn.functional.logsigmoid(torch.randn(1, T, H, K, device="cuda", generator=g_))
    beta = torch.sigmoid(torch.randn(1, T, H, device="cuda", generator=g_))
    h0 = torch.randn(N, H, K, K, device="cuda", generator=g_) * 0.1
    cu_t = torch.tensor(cu, dtype=torch.int32, device="cuda")
    try:
        with torch.no_grad():
            o_ref, s_ref = fla_chunk_kda(q=q, k=k, v=v, g=g, beta=beta, initial_state=h0.clone(), output_final_state=True,
                                         use_qk_l2norm_in_kernel=True, cu_seqlens=cu_t.long())
        torch.cuda.synchronize()
    except Exception as e:
        pytest.skip(f"fla's Triton kernels did not run here: {type(e).__name__}: {e}")
    o, s = chunk_kda(q=q, k=k, v=v, g=g, beta=beta, initial_state=h0, output_final_state=True,
                     use_qk_l2norm_in_kernel=True, cu_seqlens=cu_t)
    assert ((o.float() - o_ref.float()).norm() / o_ref.float().norm()).item() <= 5e-3
    assert ((s.float() - s_ref.float()).norm() / s_ref.float().norm()).item() <= 5e-3
