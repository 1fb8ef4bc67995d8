"""B200CausalSelfAttention / B200KVCache as drop-ins: the reference's own test scenarios
(tests/test_attention.py, tests/test_causal_self_attention_equivalence.py, tests/test_kv_cache.py,
tests/test_generator.py cache contract) re-stated for head_dim 128 on the GPU, plus the
reference-generated fixtures."""
import os

import numpy as np
import pytest
import torch

from gpu_util import assert_close_bf16
from oracle import swa

pytestmark = pytest.mark.gpu


def _module(dim, H, D, w=None, eps=None):
    os.environ["DISABLE_O_ZERO_INIT"] = "1"
    from daisy_b200 import B200CausalSelfAttention
    m = B200CausalSelfAttention(dim=dim, num_heads=H, head_dim=D).cuda().eval()
    if w is not None:
        with torch.no_grad():
            m.qkvo_w.copy_(w.to(m.qkvo_w.dtype))
    if eps is not None:
        m.norm_eps = eps
    return m


def _fixture(golden_dir, name):
    z = np.load(os.path.join(golden_dir, name))
    return {k: (torch.from_numpy(z[k]) if z[k].ndim else z[k].item()) for k in z.files}


def test_prefill_matches_reference_fixture(golden_dir):
    from daisy_b200 import WindowMask
    g = _fixture(golden_dir, "csa_prefill_small.npz")
    H, D, W = int(g["heads"]), int(g["head_dim"]), int(g["window"])
    m = _module(H * D, H, D, g["qkvo_w"], eps=swa.FP32_EPS)
    x = g["x"].bfloat16().cuda()
    with torch.inference_mode():
        y, k, v = m.prefill(x, None, attn_mask=WindowMask(W))
        y_fwd = m.forward(x, None, attn_mask=WindowMask(W))
    assert torch.equal(y, y_fwd)
    assert k.shape == g["k"].shape and v.shape == g["v"].shape
    # oracle on the bf16-rounded weights/activations the module actually sees
    cos, sin = swa.rope_tables(D, x.shape[1])
    y_o, k_o, v_o = swa.csa_prefill(x.float().cpu(), g["qkvo_w"].bfloat16().float(), H, D, W, cos, sin)
    assert_close_bf16(y, y_o, "y vs oracle(bf16 weights)")
    assert_close_bf16(k, k_o, "k", max_tol=4e-2)
    assert_close_bf16(v, v_o, "v", max_tol=4e-2)
    # and against the reference's own fp32 output
    assert_close_bf16(y, g["y"], "y vs reference fp32", max_tol=4e-2, mean_tol=4e-3)


@pytest.mark.parametrize("window", [4, 12])
@pytest.mark.parametrize("fused", [False, True])
def test_step_chain_matches_reference_fixture(golden_dir, window, fused):
    """21 tokens from an empty cache of capacity 8 (window 4, and window 12 > capacity)."""
    from daisy_b200 import B200KVCache
    g = _fixture(golden_dir, "csa_step_small.npz")
    H, D, CAP = int(g["heads"]), int(g["head_dim"]), int(g["cap"])
    m = _module(H * D, H, D, g["qkvo_w"], eps=swa.FP32_EPS)
    x = g["x"].bfloat16().cuda()
    T = x.shape[1]
    cache = B200KVCache(L=1, B=1, H=H, W=CAP, D=D, device="cuda", dtype=torch.bfloat16)
    ys = []
    with torch.inference_mode():
        for t in range(T):
            if fused:
                y, k, v = m.step_ring(x[:, t:t + 1], cache, 0, cache.t, None, window)
            else:
                kc, vc = cache.view(0)
                assert kc.size(1) == min(t, CAP)
                y, k, v = m.step(x[:, t:t + 1], kc, vc, pos=cache.t, ve=None, window=window)
                cache.write(0, k, v)
            cache.advance()
            ys.append(y)
    y = torch.cat(ys, 1)
    assert_close_bf16(y, g[f"y_steps_w{window}"], f"steps w={window}", max_tol=4e-2, mean_tol=4e-3)
    assert_close_bf16(cache.k[0], g[f"ring_k_w{window}"], "ring contents", max_tol=4e-2)


def test_bulk_write_then_steps_matches_reference_fixture(golden_dir):
    from daisy_b200 import B200KVCache, WindowMask
    g = _fixture(golden_dir, "csa_step_small.npz")
    H, D, CAP = int(g["heads"]), int(g["head_dim"]), int(g["cap"])
    m = _module(H * D, H, D, g["qkvo_w"], eps=swa.FP32_EPS)
    x = g["x"].bfloat16().cuda()
    T, P, window = x.shape[1], 13, 4
    with torch.inference_mode():
        y_p, k_p, v_p = m.prefill(x[:, :P], None, attn_mask=WindowMask(window))
        assert_close_bf16(y_p, g["y_prefill13_w4"], "prefill", max_tol=4e-2, mean_tol=4e-3)
        cache = B200KVCache(L=1, B=1, H=H, W=CAP, D=D, device="cuda")
        cache.bulk_write_packed(torch.stack([k_p[None], v_p[None]]), P)
        ys = []
        for t in range(P, T):
            y, _, _ = m.step_ring(x[:, t:t + 1], cache, 0, cache.t, None, window)
            cache.advance()
            ys.append(y)
    assert_close_bf16(torch.cat(ys, 1), g["y_after_bulk_w4"], "after bulk", max_tol=4e-2, mean_tol=4e-3)


@pytest.mark.parametrize("T,W", [(128, 128), (131, 128)])
def test_forward_equals_step(T, W):
    """tests/test_causal_self_attention_equivalence.py:15-52: full forward == token-by-token step."""
    from daisy_b200 import WindowMask
    torch.manual_seed(0)
    H, D = 2, 128
    m = _module(H * D, H, D)
    x = torch.randn(1, T, H * D, device="cuda", dtype=torch.bfloat16)
    with torch.inference_mode():
        y_full = m.forward(x, None, attn_mask=WindowMask(W))
        K = torch.empty(1, 0, H, D, device="cuda", dtype=torch.bfloat16)
        V = torch.empty(1, 0, H, D, device="cuda", dtype=torch.bfloat16)
        ys = []
        for pos in range(T):
            y, k, v = m.step(x[:, pos:pos + 1], k_ctx=K, v_ctx=V, pos=pos, ve=None, window=W)
            K, V = torch.cat([K, k], 1), torch.cat([V, v], 1)
            ys.append(y)
    y_step = torch.cat(ys, 1)
    assert y_full.shape == y_step.shape
    assert torch.allclose(y_full.float(), y_step.float(), atol=2e-2, rtol=2e-2), \
        f"max_err={(y_full.float() - y_step.float()).abs().max().item()}"


def test_value_embedding_gate():
    from daisy_b200 import B200CausalSelfAttention, WindowMask
    os.environ["DISABLE_O_ZERO_INIT"] = "1"
    torch.manual_seed(1)
    H, D, T, W = 2, 128, 70, 32
    m = B200CausalSelfAttention(H * D, H, D, receives_ve=True, layer_idx=2).cuda().eval()
    m.norm_eps = swa.FP32_EPS
    x = torch.randn(1, T, H * D, device="cuda", dtype=torch.bfloat16)
    ve = torch.randn(1, T, H * D, device="cuda", dtype=torch.bfloat16)
    with torch.inference_mode():
        y = m.forward(x, ve, attn_mask=WindowMask(W))
    # oracle: models/daisy/attention.py:129-139 (gate after the norm, before attention)
    w = m.qkvo_w.detach().float().cpu()
    q, k, v = swa.project_qkv(x.float().cpu(), w, H, D)
    cos, sin = swa.rope_tables(D, T)
    qn, kn, vn = swa.qkv_transform(q, k, v, cos, sin, swa.FP32_EPS)
    gate = torch.sigmoid(m.g_ve.detach().float().cpu())
    vn = gate * vn + (1 - gate) * ve.float().cpu().view_as(vn)
    y_o = swa.attend_windowed(qn, kn, vn, W).reshape(1, T, H * D) @ w[3].t()
    assert_close_bf16(y, y_o, "ve gate", max_tol=4e-2, mean_tol=4e-3)


# ----------------------------------------------------------------------------- KV cache (tests/test_kv_cache.py)

def test_kvcache_empty_view_and_reset():
    from daisy_b200 import B200KVCache
    L, B, H, W, D = 2, 2, 2, 3, 128
    c = B200KVCache(L, B, H, W, D, device="cuda", dtype=torch.float32)
    k, v = c.view(1)
    assert k.shape == (B, 0, H, D) and v.shape == (B, 0, H, D)
    for i in range(2):
        c.write(0, torch.full((B, H, 1, D), 30.0 + i, device="cuda"), torch.full((B, H, 1, D), 1030.0 + i, device="cuda"))
        c.advance()
    c.reset_history()
    assert c.t == 0 and c.view(0)[0].shape == (B, 0, H, D)


@pytest.mark.parametrize("W,steps", [(4, 3), (3, 5)])
def test_kvcache_write_and_view_order(W, steps):
    from daisy_b200 import B200KVCache
    L, B, H, D = 1, 2, 2, 128
    c = B200KVCache(L, B, H, W, D, device="cuda", dtype=torch.float32)
    vals = [20.0 + i for i in range(steps)]
    for val in vals:
        c.write(0, torch.full((B, H, 1, D), val, device="cuda"), torch.full((B, H, 1, D), val + 1000, device="cuda"))
        c.advance()
    k, v = c.view(0)
    exp = vals[-W:]
    assert k.shape == (B, len(exp), H, D)
    assert k[0, :, 0, 0].tolist() == exp and v[1, :, 1, 5].tolist() == [e + 1000 for e in exp]


def test_kvcache_accepts_b1hd_and_contract():
    from daisy_b200 import B200KVCache
    L, B, H, W, D, steps = 2, 1, 3, 4, 128, 6
    c = B200KVCache(L, B, H, W, D, device="cuda", dtype=torch.bfloat16)
    for t in range(steps):
        for layer in range(L):
            assert c.view(layer)[0].size(1) == min(t, W)
        new = torch.full((B, 1, H, D), float(t), device="cuda", dtype=torch.bfloat16)   # [B,1,H,D] form
        for layer in range(L):
            c.write(layer, new, new)
        for layer in range(L):
            got = c.view(layer)[0][0, :, 0, 0].to(torch.int64).tolist()
            n = min(t + 1, W)
            assert got == list(range(max(0, t - n + 1), t + 1))
        c.advance()


def test_step_runner_matches_layerwise_oracle():
    """Generator-style orchestration (inference/generate.py:220-248) over two layers: prefill 40 tokens into a
    capacity-32 ring, then 12 fused steps; every step equals the oracle's prefill of the whole prefix."""
    from daisy_b200 import B200CausalSelfAttention, StepRunner
    os.environ["DISABLE_O_ZERO_INIT"] = "1"
    torch.manual_seed(3)
    H, D, W, P, N = 2, 128, 24, 40, 12
    layers = [B200CausalSelfAttention(H * D, H, D).cuda().eval() for _ in range(2)]
    for m in layers:
        m.norm_eps = swa.FP32_EPS
        with torch.no_grad():
            m.qkvo_w.mul_(4.0)                      # keep activations O(1) through two layers
    x = torch.randn(1, P + N, H * D, device="cuda", dtype=torch.bfloat16)
    run = StepRunner(layers, window=W, cache_capacity=32)
    y_p = run._prefill(x[:, :P])
    ys = [run._step(x[:, P + i:P + i + 1]) for i in range(N)]
    assert run.cache.t == P + N
    # oracle: full prefill of all P+N tokens through both layers in fp32 on the bf16 weights
    cos, sin = swa.rope_tables(D, P + N)
    h = x.float().cpu()
    for m in layers:
        h, _, _ = swa.csa_prefill(h.bfloat16().float(), m.qkvo_w.detach().float().cpu(), H, D, W, cos, sin)
    assert_close_bf16(y_p, h[:, :P], "prefill part", max_tol=6e-2, mean_tol=6e-3)
    assert_close_bf16(torch.cat(ys, 1), h[:, P:], "stepped part", max_tol=6e-2, mean_tol=6e-3)


def test_host_buffer_prefill_equals_device_call():
    """HostPrefill (pinned host tensors, three-stream pipeline over batch rows) == the device-resident call."""
    from daisy_b200 import ops
    from daisy_b200.host_api import HostPrefill
    B, T, H, D, W = 5, 260, 2, 128, 100
    g = torch.Generator().manual_seed(8)
    hq, hk, hv = (torch.randn(B, T, H, D, generator=g).bfloat16().pin_memory() for _ in range(3))
    cos, sin = swa.rope_tables(D, T)
    cos, sin = cos.cuda(), sin.cuda()
    y_dev, k_dev, _ = ops.swa_prefill(hq.cuda(), hk.cuda(), hv.cuda(), cos, sin, W)
    for rows in (1, 2):
        hout = torch.zeros(B, T, H, D, dtype=torch.bfloat16).pin_memory()
        hk_out, hv_out = torch.zeros_like(hout).pin_memory(), torch.zeros_like(hout).pin_memory()
        call = HostPrefill(T, H, D, rows_per_chunk=rows, return_kv=True)
        call(hq, hk, hv, cos, sin, W, hout, hk_out, hv_out)
        call(hq, hk, hv, cos, sin, W, hout, hk_out, hv_out)          # staging reuse
        torch.cuda.synchronize()
        assert torch.equal(hout, y_dev.cpu())
        assert torch.equal(hk_out.transpose(1, 2), k_dev.cpu())


def test_forward_with_eos_document_mask_matches_reference_fixture(golden_dir):
    """``forward`` under ``build_attn_mask`` with EOS tokens in the sequence (document masking),
    against the reference module's own output."""
    import numpy as np
    from daisy_b200 import B200CausalSelfAttention, WindowMask
    d = np.load(os.path.join(golden_dir, "doc_mask_small.npz"))
    x = torch.from_numpy(d["x"])
    attn = B200CausalSelfAttention(dim=256, num_heads=2, head_dim=128, max_seq_len=256).cuda()
    with torch.no_grad():
        attn.qkvo_w.copy_(torch.from_numpy(d["qkvo_w"]).to(attn.qkvo_w.dtype))
    seq = torch.from_numpy(d["seq"]).cuda()
    mask = WindowMask.from_tokens(seq, int(d["window"]), int(d["eos"]))
    with torch.inference_mode():
        y = attn(x.cuda().bfloat16(), None, attn_mask=mask)
    ref = torch.from_numpy(d["y"])
    err = (y.float().cpu() - ref).abs()
    scale = max(1.0, ref.abs().max().item())
    assert err.max().item() <= 4e-2 * scale and err.mean().item() <= 4e-3 * scale
    # the reference's own dense additive mask tensor (what DaisyCore.prefill passes, daisy_core.py:338-346), as
    # [1,1,T,T], as [T,T] and as a boolean mask: same bits as the analytic form
    dense = torch.from_numpy(d["mask"]).cuda()
    with torch.inference_mode():
        for mk in (dense[None, None], dense, dense == 0):
            y_d, k_d, v_d = attn.prefill(x.cuda().bfloat16(), None, attn_mask=mk)
            assert torch.equal(y_d, y)
    from daisy_b200.attention import band_of_dense_mask
    T = dense.shape[0]
    first = band_of_dense_mask(dense[None, None])
    want = torch.maximum(mask.doc_start.cuda().view(-1), (torch.arange(T, device="cuda") - int(d["window"]) + 1).clamp_min(0).int())
    assert torch.equal(first, want.to(torch.int32))
    # masks the kernels cannot express are refused, not approximated
    assert float(dense[140, 120]) == 0.0
    holed = dense.clone(); holed[140, 120] = float("-inf")
    future = dense.clone(); future[10, 11] = 0.0
    for bad in (holed, future, torch.full_like(dense, float("-inf"))):
        with pytest.raises(ValueError, match="causal band"):
            band_of_dense_mask(bad)
    # the cache-writing form has no backward pass: a call that would need gradients raises
    with pytest.raises(NotImplementedError, match="no backward pass"):
        attn.prefill(x.cuda().bfloat16(), None, attn_mask=mask)


def test_forward_with_block_mask_training_form():
    """``forward(x, ve, block_mask=...)`` with the masks of ``create_blockmasks`` (long / short cycle) against
    the oracle's block-granular mask."""
    from daisy_b200 import B200CausalSelfAttention, create_blockmasks
    H, T, eos = 2, 768, 5
    m = _module(H * 128, H, 128, eps=swa.FP32_EPS)
    g = torch.Generator().manual_seed(12)
    seq = torch.randint(6, 50, (T,), generator=g)
    seq[[100, 300, 301, 640]] = eos
    x = torch.randn(1, T, H * 128, generator=g).bfloat16()
    masks = create_blockmasks(seq.cuda(), 4, 6, eos)
    assert [bm.window_blocks for bm in masks] == [4, 2, 2, 2, 4, 4]
    w = m.qkvo_w.detach().float().cpu()
    ds = swa.doc_starts(seq, eos)
    for bm in (masks[0], masks[1]):
        with torch.inference_mode():
            y = m(x.cuda(), None, block_mask=bm)
        q, k, v = swa.project_qkv(x.float(), w, H, 128)
        yo, _, _ = swa.swa_prefill(q, k, v, m.rotary.cos[:T].cpu(), m.rotary.sin[:T].cpu(), None, doc_start=ds,
                                   window_blocks=bm.window_blocks)
        yo = torch.matmul(yo.reshape(1, T, H * 128), w[3].t())
        assert_close_bf16(y, yo, f"block mask wb={bm.window_blocks}", max_tol=4e-2, mean_tol=4e-3)


def test_step_through_cuda_graph_equals_eager_steps():
    """``StepRunner.capture_step`` / ``_step_graph``: one captured launch sequence with the position in device
    memory, replayed per token, gives bit-identical outputs and ring contents to the eager ``_step`` -- through
    the ramp-up (fewer context rows than the window), the steady state and the ring wrap."""
    from daisy_b200 import B200CausalSelfAttention, StepRunner
    os.environ["DISABLE_O_ZERO_INIT"] = "1"
    torch.manual_seed(4)
    B, H, D, W, cap, P, N = 2, 2, 128, 24, 32, 10, 45
    layers = [B200CausalSelfAttention(H * D, H, D, max_seq_len=256).cuda().eval() for _ in range(2)]
    for m in layers:
        with torch.no_grad():
            m.qkvo_w.mul_(4.0)
    x = torch.randn(B, P + N, H * D, device="cuda", dtype=torch.bfloat16)
    eager = StepRunner(layers, window=W, cache_capacity=cap, batch=B)
    graph = StepRunner(layers, window=W, cache_capacity=cap, batch=B)
    eager._prefill(x[:, :P])
    graph._prefill(x[:, :P])
    graph.capture_step(B, H * D)
    for i in range(N):
        xi = x[:, P + i:P + i + 1]
        y_e = eager._step(xi)
        y_g = graph._step_graph(xi).clone()
        assert torch.equal(y_e, y_g), f"step {i} (t={P + i})"
    from daisy_b200 import ops
    ops.check_device_status("cuda")
    assert graph.cache.t == eager.cache.t == P + N and int(graph.cache.t_dev.item()) == P + N
    assert torch.equal(graph.cache.k, eager.cache.k) and torch.equal(graph.cache.v, eager.cache.v)


@pytest.mark.parametrize("T,cap,dtype", [(40, 32, torch.bfloat16), (300, 64, torch.bfloat16), (20, 64, torch.bfloat16),
                                         (200, 48, torch.float16), (1, 8, torch.bfloat16)])
def test_prefill_fills_the_ring_like_bulk_write_packed(T, cap, dtype):
    """``prefill_ring``: the projection epilogue stores the prompt's last min(T, cap - 1) k', v' rows into their ring
    slots; same ring contents, bit for bit, as ``prefill`` followed by ``KVCache.bulk_write_packed`` (the reference's
    sequence, inference/generate.py:220-229), and the same outputs."""
    from daisy_b200 import B200KVCache, WindowMask
    B, H, D = 2, 2, 128
    m = _module(H * D, H, D)
    x = torch.randn(B, T, H * D, device="cuda", dtype=torch.bfloat16)
    with torch.inference_mode():
        y0, k0, v0 = m.prefill(x, None, attn_mask=WindowMask(24))
        ref = B200KVCache(1, B, H, cap, D, "cuda", dtype)
        ref.k.fill_(7.0); ref.v.fill_(7.0)                       # slots the fill must leave alone keep their contents
        ref.bulk_write_packed(torch.stack([k0[None], v0[None]]), T)
        got = B200KVCache(1, B, H, cap, D, "cuda", dtype)
        got.k.fill_(7.0); got.v.fill_(7.0)
        y1, k1, v1 = m.prefill_ring(x, None, got, 0, attn_mask=WindowMask(24))
        got.set_position(T)
    from daisy_b200 import ops
    ops.check_device_status("cuda")
    assert torch.equal(y1, y0) and torch.equal(k1, k0) and torch.equal(v1, v0)
    assert torch.equal(got.k, ref.k) and torch.equal(got.v, ref.v) and got.t == ref.t == T


def test_graph_capture_after_the_ring_wrapped_with_window_larger_than_capacity():
    """Capturing the graph step must leave the ring alone: with a window larger than the ring capacity the slot of
    the next token holds the oldest row the next step still attends to.  Eager steps first (so that slot holds a real
    row), then the capture, then graph steps against eager ones."""
    from daisy_b200 import B200CausalSelfAttention, StepRunner
    os.environ["DISABLE_O_ZERO_INIT"] = "1"
    torch.manual_seed(8)
    B, H, D, W, cap, P, E, N = 1, 2, 128, 40, 16, 10, 12, 20
    layers = [B200CausalSelfAttention(H * D, H, D, max_seq_len=256).cuda().eval() for _ in range(2)]
    for m in layers:
        with torch.no_grad():
            m.qkvo_w.mul_(4.0)
    x = torch.randn(B, P + E + N, H * D, device="cuda", dtype=torch.bfloat16)
    eager = StepRunner(layers, window=W, cache_capacity=cap, batch=B)
    graph = StepRunner(layers, window=W, cache_capacity=cap, batch=B)
    for run in (eager, graph):
        run._prefill(x[:, :P])
        for i in range(E):
            run._step(x[:, P + i:P + i + 1])
    assert graph.cache.t == P + E > cap
    before = (graph.cache.k.clone(), graph.cache.v.clone())
    graph.capture_step(B, H * D)
    assert torch.equal(graph.cache.k, before[0]) and torch.equal(graph.cache.v, before[1])
    for i in range(N):
        xi = x[:, P + E + i:P + E + i + 1]
        assert torch.equal(eager._step(xi), graph._step_graph(xi).clone()), f"step {i}"
    assert torch.equal(graph.cache.k, eager.cache.k) and torch.equal(graph.cache.v, eager.cache.v)


def test_graph_step_with_value_embedding_layer():
    """A layer that receives a value embedding through ``step_ring_dev`` (what the CUDA-graph step runs): same bits as
    the eager ``step_ring``, and the step chain matches the windowed forward under the same embeddings."""
    from daisy_b200 import B200CausalSelfAttention, B200KVCache, WindowMask
    os.environ["DISABLE_O_ZERO_INIT"] = "1"
    torch.manual_seed(3)
    H, D, T, W, cap = 2, 128, 40, 16, 32
    m = B200CausalSelfAttention(H * D, H, D, receives_ve=True, layer_idx=2, max_seq_len=128).cuda().eval()
    m.norm_eps = swa.FP32_EPS
    with torch.no_grad():
        m.qkvo_w.mul_(4.0)
    x = torch.randn(1, T, H * D, device="cuda", dtype=torch.bfloat16)
    ve = torch.randn(1, T, H * D, device="cuda", dtype=torch.bfloat16)
    with torch.inference_mode():
        y_full = m.forward(x, ve, attn_mask=WindowMask(W))
        ca, cb = B200KVCache(1, 1, H, cap, D, "cuda"), B200KVCache(1, 1, H, cap, D, "cuda")
        for t in range(T):
            ya, _, _ = m.step_ring(x[:, t:t + 1], ca, 0, ca.t, ve[:, t:t + 1], W)
            yb = m.step_ring_dev(x[:, t:t + 1], cb, 0, W, ve=ve[:, t:t + 1])
            ca.advance(); cb.advance()
            assert torch.equal(ya, yb), f"token {t}"
            assert_close_bf16(ya, y_full[:, t:t + 1].float().cpu(), f"token {t} vs forward", max_tol=6e-2, mean_tol=6e-3)
    assert torch.equal(ca.k, cb.k) and torch.equal(ca.v, cb.v)


def test_step_runner_with_float16_cache():
    """The runner with ``dtype=torch.float16`` for the cache, as ``Generator`` defaults to: prefill fills the fp16
    ring, eager and CUDA-graph steps read and extend it; results stay within the bf16 bar of the oracle."""
    from daisy_b200 import B200CausalSelfAttention, StepRunner
    os.environ["DISABLE_O_ZERO_INIT"] = "1"
    torch.manual_seed(6)
    H, D, W, P, N = 2, 128, 24, 40, 10
    layers = [B200CausalSelfAttention(H * D, H, D, max_seq_len=128).cuda().eval() for _ in range(2)]
    for m in layers:
        m.norm_eps = swa.FP32_EPS
        with torch.no_grad():
            m.qkvo_w.mul_(4.0)
    x = torch.randn(1, P + N, H * D, device="cuda", dtype=torch.bfloat16)
    run = StepRunner(layers, window=W, cache_capacity=32, dtype=torch.float16)
    assert run.cache.k.dtype == torch.float16
    run._prefill(x[:, :P])
    ys = [run._step(x[:, P + i:P + i + 1]) for i in range(N // 2)]
    run.capture_step(1, H * D)
    ys += [run._step_graph(x[:, P + i:P + i + 1]).clone() for i in range(N // 2, N)]
    cos, sin = swa.rope_tables(D, P + N)
    h = x.float().cpu()
    for m in layers:
        h, _, _ = swa.csa_prefill(h.bfloat16().float(), m.qkvo_w.detach().float().cpu(), H, D, W, cos, sin)
    assert_close_bf16(torch.cat(ys, 1), h[:, P:], "stepped part, fp16 cache", max_tol=6e-2, mean_tol=6e-3)
