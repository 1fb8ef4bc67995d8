"""The CPU oracle against fixtures produced by the reference's own code
(tests/golden/make_golden.py).  These pin the oracle; the GPU parity tests then
compare the CUDA path with the oracle."""
import os

import numpy as np
import pytest
import torch

from oracle import swa, kda


def _load(golden_dir, name):
    z = np.load(os.path.join(golden_dir, name))
    return {k: (torch.from_numpy(z[k]) if z[k].ndim else z[k].item()) for k in z.files}


def test_csa_prefill_matches_reference(golden_dir):
    g = _load(golden_dir, "csa_prefill_small.npz")
    H, D, W = int(g["heads"]), int(g["head_dim"]), int(g["window"])
    cos, sin = swa.rope_tables(D, g["x"].shape[1])
    y, k, v = swa.csa_prefill(g["x"], g["qkvo_w"], H, D, W, cos, sin)
    assert (y - g["y"]).abs().max().item() < 2e-5
    assert (k - g["k"]).abs().max().item() < 1e-5
    assert (v - g["v"]).abs().max().item() < 1e-5


@pytest.mark.parametrize("window", [4, 12])
def test_csa_step_chain_matches_reference(golden_dir, window):
    g = _load(golden_dir, "csa_step_small.npz")
    H, D, CAP = int(g["heads"]), int(g["head_dim"]), int(g["cap"])
    x = g["x"]
    T = x.shape[1]
    cos, sin = swa.rope_tables(D, T)
    cache = swa.RingKVCache(1, 1, H, CAP, D)
    ys, ks = [], []
    for t in range(T):
        kc, vc = cache.view(0)
        y, k, v = swa.csa_step(x[:, t:t + 1], g["qkvo_w"], H, D, kc, vc, cache.t, window, cos, sin)
        cache.write(0, k, v)
        cache.advance()
        ys.append(y); ks.append(k)
    assert (torch.cat(ys, 1) - g[f"y_steps_w{window}"]).abs().max().item() < 2e-5
    assert (torch.cat(ks, 1) - g[f"k_steps_w{window}"]).abs().max().item() < 1e-5
    assert (cache.k[0] - g[f"ring_k_w{window}"]).abs().max().item() < 1e-5


def test_csa_bulk_write_then_steps(golden_dir):
    g = _load(golden_dir, "csa_step_small.npz")
    H, D, CAP = int(g["heads"]), int(g["head_dim"]), int(g["cap"])
    x = g["x"]
    T, P, window = x.shape[1], 13, 4
    cos, sin = swa.rope_tables(D, T)
    y_p, k_p, v_p = swa.csa_prefill(x[:, :P], g["qkvo_w"], H, D, window, cos, sin)
    assert (y_p - g["y_prefill13_w4"]).abs().max().item() < 2e-5
    cache = swa.RingKVCache(1, 1, H, CAP, D)
    cache.bulk_write_packed(torch.stack([k_p[None], v_p[None]]), P)
    ys = []
    for t in range(P, T):
        kc, vc = cache.view(0)
        y, k, v = swa.csa_step(x[:, t:t + 1], g["qkvo_w"], H, D, kc, vc, cache.t, window, cos, sin)
        cache.write(0, k, v)
        cache.advance()
        ys.append(y)
    assert (torch.cat(ys, 1) - g["y_after_bulk_w4"]).abs().max().item() < 2e-5


def test_swa_inner_base10000(golden_dir):
    g = _load(golden_dir, "swa_inner_small.npz")
    y, kn, vn = swa.swa_prefill(g["q"], g["k"], g["v"], g["cos"], g["sin"], int(g["window"]), block=64)
    assert (y - g["y"]).abs().max().item() < 2e-5
    assert (kn.permute(0, 2, 1, 3) - g["kn"]).abs().max().item() < 1e-5
    assert (vn.permute(0, 2, 1, 3) - g["vn"]).abs().max().item() < 1e-5


def test_blockwise_equals_dense_mask():
    torch.manual_seed(0)
    B, T, H, D, W = 1, 150, 1, 16, 37
    q, k, v = (torch.randn(B, T, H, D) for _ in range(3))
    a = swa.attend_windowed(q, k, v, W, block=32)
    b = swa.attend_windowed(q, k, v, W, block=1000)
    assert (a - b).abs().max().item() < 1e-5
    # per-token definition: keys max(0, t+1-W) .. t  (reference tests/test_attention.py:66-67)
    t = 100
    s = (q[0, t, 0] @ k[0, t + 1 - W:t + 1, 0].T) * swa.ATTN_SCALE
    ref = torch.softmax(s, -1) @ v[0, t + 1 - W:t + 1, 0]
    assert (a[0, t, 0] - ref).abs().max().item() < 1e-5


def test_kda_matches_third_party_naive(golden_dir):
    g = _load(golden_dir, "kda_naive_small.npz")
    o, s = kda.kda_recurrent(g["q"], g["k"], g["v"], g["g"], g["beta"])
    assert (o - g["o"]).abs().max().item() < 1e-5
    assert (s - g["s"]).abs().max().item() < 1e-5
    o, s = kda.kda_recurrent(g["q"], g["k"], g["v"], g["g"], g["beta"], initial_state=g["h0"])
    assert (o - g["o_h0"]).abs().max().item() < 1e-5
    assert (s - g["s_h0"]).abs().max().item() < 1e-5


def test_kv_cache_view_order_and_contract():
    """Ported from the reference's tests/test_kv_cache.py:105-133 (integer fills, wrap order)."""
    W, steps, L, B, H, D = 4, 6, 2, 1, 3, 5
    cache = swa.RingKVCache(L, B, H, W, D)
    for t in range(steps):
        for layer in range(L):
            assert cache.view(layer)[0].size(1) == min(t, W)
        new = torch.full((B, H, 1, D), float(t))
        for layer in range(L):
            cache.write(layer, new, new)
        for layer in range(L):
            got = cache.view(layer)[0][0, :, 0, 0].to(torch.int64).tolist()
            n = min(t + 1, W)
            assert got == list(range(max(0, t - n + 1), t + 1))
        cache.advance()


def test_work_counts():
    assert swa.window_pairs(1024, 512) == 393472
    assert swa.prefill_flops(8, 8192, 16, 128, 2048) == pytest.approx(9.6214e11, rel=1e-4)
    assert swa.prefill_flops(1, 65536, 16, 128, 8192) == pytest.approx(4.1232e12, rel=1e-4)
    assert swa.decode_bytes(64, 16, 128, 4095) == pytest.approx(2.1485e9, rel=1e-4)
    assert kda.kda_bytes_per_token_head() == 1540


def test_kda_gate_against_reference_fixture(golden_dir):
    """oracle.kda.kda_gate vs values produced by the reference's own ``_gate_impl``
    (models/daisy/fla_custom_ops.py:71-103)."""
    import numpy as np
    d = np.load(os.path.join(golden_dir, "kda_gate_small.npz"))
    x, A, bias = (torch.from_numpy(d[n]) for n in ("x", "A_log", "bias"))
    for got, ref in ((kda.kda_gate(x, A, 128, bias), d["y_fp32"]), (kda.kda_gate(x, A, 128, None), d["y_nobias"])):
        ref = torch.from_numpy(ref)
        assert got.shape == ref.shape and ((got - ref).abs() <= 1e-6 * ref.abs() + 1e-7).all()
    got = kda.kda_gate(x.bfloat16(), A, 128, bias)
    assert got.dtype == torch.bfloat16 and torch.equal(got.float(), torch.from_numpy(d["y_bf16_as_fp32"]))


def test_document_mask_against_reference_fixture(golden_dir):
    """oracle window_mask / doc_starts / csa_prefill vs ``build_attn_mask`` with EOS tokens
    (models/daisy/daisy_core.py:53-69) and the module's forward under that mask."""
    d = np.load(os.path.join(golden_dir, "doc_mask_small.npz"))
    seq = torch.from_numpy(d["seq"])[0]
    T, W = seq.numel(), int(d["window"])
    ds = swa.doc_starts(seq, int(d["eos"]))
    assert torch.equal(swa.window_mask(0, T, 0, T, W, ds), torch.from_numpy(d["mask"]))
    assert torch.equal(swa.window_mask(10, 90, 3, 77, W, ds), torch.from_numpy(d["mask"])[10:90, 3:77])
    y, _, _ = swa.csa_prefill(torch.from_numpy(d["x"]), torch.from_numpy(d["qkvo_w"]), 2, 128, W,
                              torch.from_numpy(d["cos"]), torch.from_numpy(d["sin"]), doc_start=ds)
    assert (y - torch.from_numpy(d["y"])).abs().max().item() < 1e-5


def test_backward_against_reference_autograd_fixture(golden_dir):
    """oracle ``csa_backward`` (autograd over the restatement) vs the reference module's own CPU SDPA path under
    autograd, with the dense window + document mask: output, input gradient, weight gradient."""
    d = np.load(os.path.join(golden_dir, "csa_backward_small.npz"))
    seq = torch.from_numpy(d["seq"])[0]
    T, W = seq.numel(), int(d["window"])
    ds = swa.doc_starts(seq, int(d["eos"]))
    cos, sin = swa.rope_tables(128, T)
    y, dx, dw = swa.csa_backward(torch.from_numpy(d["x"]), torch.from_numpy(d["qkvo_w"]), 2, 128, W, cos, sin,
                                 torch.from_numpy(d["cot"]), doc_start=ds)
    for got, name in ((y, "y"), (dx, "dx"), (dw, "dw")):
        ref = torch.from_numpy(d[name])
        assert (got - ref).abs().max().item() <= 2e-5 * max(1.0, ref.abs().max().item()), name


def test_flex_block_lists_against_reference_fixture(golden_dir):
    """The block lists of ``DaisyCore.create_blockmasks`` (models/daisy/daisy_core.py:182-229), produced by the
    reference itself for documents of many lengths and several window sizes, against the oracle's restatement;
    and the token-level rule the kernels implement (causal, same document, key block >= query block -
    window_blocks + 1) selects exactly the union of those lists."""
    d = np.load(os.path.join(golden_dir, "flex_blockmask_lists.npz"))
    eos, checked = int(d["eos"]), 0
    for case in range(3):
        seq = torch.from_numpy(d[f"seq{case}"])
        docs, T = (seq == eos).cumsum(0), seq.numel()
        nb = T // swa.BLOCK
        ds = swa.doc_starts(seq, eos)
        for wb in (2, 3, 6, 8):
            for name, w in (("long", wb), ("short", wb // 2)):
                key = f"c{case}_wb{wb}_{name}"
                if key + "_pn" not in d.files:
                    continue
                part, full = swa.flex_block_lists(docs, w)
                for qb in range(nb):
                    ref_p = set(d[key + "_pi"][qb][:d[key + "_pn"][qb]].tolist())
                    ref_f = set(d[key + "_fi"][qb][:d[key + "_fn"][qb]].tolist())
                    assert ref_p == part[qb] and ref_f == full[qb], (key, qb)
                    m = swa.window_mask(qb * swa.BLOCK, (qb + 1) * swa.BLOCK, 0, T, None, ds, w)
                    vis = torch.isfinite(m).any(0).view(nb, swa.BLOCK)
                    assert set(vis.any(1).nonzero().flatten().tolist()) == (ref_p | ref_f), (key, qb)
                    for kb in ref_f:                                # a "full" block is visible to every row
                        assert bool(vis[kb].all()) and bool(torch.isfinite(m[:, kb * swa.BLOCK:(kb + 1) * swa.BLOCK]).all())
                    checked += 1
    assert checked == 384


def test_kda_layer_passes_against_fixture(golden_dir):
    """oracle.kda.short_conv vs torch's Conv1d forward on fla's ShortConvolution instances (taps 4, 3 with bias, 2),
    in one piece and as prefill + single-token steps through the carried state; oracle.kda.gated_rms_norm vs the
    torch.nn.functional evaluation in the order of CompilableFusedRMSNormGated.forward
    (models/daisy/attention_kimi.py:52-60)."""
    d = np.load(os.path.join(golden_dir, "kda_layer_small.npz"))
    for W in (4, 3, 2):
        x, w, b, ref = (torch.from_numpy(d[f"conv_w{W}_{n}"]) for n in ("x", "weight", "bias", "y"))
        b = b if b.numel() else None
        y, s = kda.short_conv(x, w, b)
        assert (y - ref).abs().max().item() <= 2e-6
        assert torch.equal(s, x[:, -W:].transpose(1, 2))
        # prefill of 13 tokens, then 8 single-token steps on the state
        y0, s = kda.short_conv(x[:, :13], w, b)
        ys = [y0]
        for t in range(13, x.shape[1]):
            yt, s = kda.short_conv(x[:, t:t + 1], w, b, state=s)
            ys.append(yt)
        assert (torch.cat(ys, 1) - ref).abs().max().item() <= 2e-6
        # a prompt shorter than the taps keeps the zero padding in the state
        _, s1 = kda.short_conv(x[:, :1], w, b)
        assert not s1[..., :-1].any() and torch.equal(s1[..., -1], x[:, 0])
    x, g, w = (torch.from_numpy(d[n]) for n in ("norm_x", "norm_gate", "norm_weight"))
    assert (kda.gated_rms_norm(x, g, w, mode="swish") - torch.from_numpy(d["norm_swish"])).abs().max() <= 1e-5
    assert (kda.gated_rms_norm(x, g, w, mode="sigmoid") - torch.from_numpy(d["norm_sigmoid"])).abs().max() <= 1e-5
    got = kda.gated_rms_norm(x.bfloat16(), g.bfloat16(), w.bfloat16()).bfloat16().float()
    ref = torch.from_numpy(d["norm_ref_bf16_as_fp32"])
    assert (got == ref).float().mean().item() > 0.995 and ((got - ref).abs() <= ref.abs() * 2.0 ** -6 + 1e-30).all()
