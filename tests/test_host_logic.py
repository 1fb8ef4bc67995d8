"""Host-side logic that needs no GPU: ring index arithmetic, mask descriptor parsing, module construction,
and the sharding arithmetic of the multi-GPU bench (world_size-2 gloo)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import swa


def test_ring_segment_matches_reference_view():
    from daisy_b200 import ring_segment
    for W in (1, 3, 4, 8):
        c = swa.RingKVCache(1, 1, 1, W, 2)
        for t in range(3 * W + 2):
            for staged in (False, True):
                first, n = ring_segment(t, staged, W)
                assert n == min(t + staged, W) and first == t + staged - n
            k = torch.full((1, 1, 1, 2), float(t))
            kc, _ = c.view(0)
            first, n = ring_segment(c.t, False, W)
            assert kc[0, :, 0, 0].tolist() == [float(x) for x in range(first, first + n)]
            c.write(0, k, k)
            kc, _ = c.view(0)
            first, n = ring_segment(c.t, True, W)
            assert kc[0, :, 0, 0].tolist() == [float(x) for x in range(first, first + n)]
            c.advance()


def test_module_construction_and_mask_parsing(monkeypatch):
    monkeypatch.setenv("DISABLE_O_ZERO_INIT", "")
    from daisy_b200 import B200CausalSelfAttention, WindowMask
    m = B200CausalSelfAttention(256, 2, 128, max_seq_len=64)
    assert m.qkvo_w.shape == (4, 256, 256) and m.qkvo_w.dtype == torch.bfloat16
    assert float(m.qkvo_w[3].abs().max()) == 0.0               # W_o zero-initialised like the reference
    assert m.attn_scale == 0.12 and m.num_heads == 2 and m.head_dim == 128
    cos, sin = swa.rope_tables(128, 64)
    assert torch.equal(m.rotary.cos, cos) and torch.equal(m.rotary.sin, sin)
    assert m._window_of(None) == (None, None) and m._window_of(WindowMask(5)) == (5, None) and m._window_of(7) == (7, None)
    from daisy_b200.attention import doc_starts
    seq = torch.tensor([[3, 9, 4, 4, 9, 9, 2]])
    assert doc_starts(seq, 9).tolist() == [0, 1, 1, 1, 4, 5, 5]              # an EOS opens the next document
    assert WindowMask.from_tokens(seq, 4, 9).doc_start.tolist() == [0, 1, 1, 1, 4, 5, 5]
    with pytest.raises(TypeError):
        m._window_of("causal")
    with pytest.raises(ValueError, match="CUDA tensor"):       # the dense mask is read on the device
        m._window_of(torch.zeros(1, 1, 4, 4))
    # calls without a backward pass that would need gradients raise instead of returning a constant
    with pytest.raises(NotImplementedError, match="no backward pass"):
        m.prefill(torch.zeros(1, 4, 256, dtype=torch.bfloat16), None)
    from daisy_b200.attention import create_blockmasks
    assert [bm.window_blocks for bm in create_blockmasks(torch.zeros(128, dtype=torch.long), 1, 3, 9)] == [1, 1, 1]
    with pytest.raises(Exception):
        B200CausalSelfAttention(128, 2, 64)                    # head_dim must be 128
    g = B200CausalSelfAttention(256, 2, 128, receives_ve=True, layer_idx=2, max_seq_len=8)
    assert abs(float(g.g_ve) + 1.5163) < 1e-6


def test_cpu_tensors_are_rejected():
    from daisy_b200 import ops, B200KVCache
    x = torch.zeros(1, 4, 2, 128, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="no CPU path"):
        ops.qkv_prep(x, x, x, torch.zeros(4, 64), torch.zeros(4, 64), 1e-6)
    with pytest.raises(ValueError, match="no CPU path"):
        B200KVCache(1, 1, 2, 4, 128, device="cpu")


def _free_port():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); p = s.getsockname()[1]; s.close()
    return p


def _shard_worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from bench import shard_bounds
    # independent (batch) units are sharded with no data-path collective; outputs are all-gathered afterwards
    B, T, H, D = 6, 16, 2, 8
    g = torch.Generator().manual_seed(0)
    qkv = torch.randn(3, B, T, H, D, generator=g)
    lo, hi = shard_bounds(B, world, rank)
    y_local = swa.attend_windowed(qkv[0, lo:hi], qkv[1, lo:hi], qkv[2, lo:hi], 5)
    parts = [torch.empty(shard_bounds(B, world, r)[1] - shard_bounds(B, world, r)[0], T, H, D) for r in range(world)]
    dist.all_gather(parts, y_local) if len({p.shape for p in parts}) == 1 else dist.all_gather_object(parts, y_local)
    t = torch.tensor([float(rank + 1)])
    dist.all_reduce(t, op=dist.ReduceOp.MAX)                    # the bench's max-over-ranks timing reduction
    if rank == 0:
        y = torch.cat(parts, 0)
        y_ref = swa.attend_windowed(qkv[0], qkv[1], qkv[2], 5)
        q.put((float((y - y_ref).abs().max()), float(t)))
    dist.destroy_process_group()


def test_two_rank_gloo_sharding():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_shard_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    err, tmax = q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert err < 1e-6 and tmax == 2.0


def test_shard_bounds_cover_everything():
    from bench import shard_bounds
    for n in (1, 7, 8, 64):
        for w in (1, 2, 4, 8):
            spans = [shard_bounds(n, w, r) for r in range(w)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [b - a for a, b in spans]
            assert max(sizes) - min(sizes) <= 1


def test_kda_layer_module_has_the_reference_parameters(golden_dir):
    """B200KimiLinearSelfAttention registers the parameters of the reference's KimiLinearSelfAttention
    (models/daisy/attention_kimi.py:65-112), name for name, shape for shape, dtype for dtype: the list in the
    fixture was written from the reference class."""
    import numpy as np
    from daisy_b200 import B200KimiLinearSelfAttention
    want = sorted(np.load(os.path.join(golden_dir, "kda_layer_small.npz"))["layer_parameters"].tolist())
    m = B200KimiLinearSelfAttention(256, 2, 64, 128)
    got = sorted(f"{n}:{'x'.join(map(str, p.shape))}:{str(p.dtype).replace('torch.', '')}" for n, p in m.named_parameters())
    assert got == want


def test_varlen_tables_and_unpad_helpers():
    """Host side of the packed (cu_seqlens) KDA path: chunk / sequence / token tables, and the unpad helpers the
    reference imports (models/daisy/attention_kimi.py:19, used at :150-154,193)."""
    from daisy_b200 import ops
    from daisy_b200.kda import get_unpad_data, index_first_axis, pad_input
    chunk_tab, seq_ptr, tok_tab, n = ops.kda_varlen_tables([0, 5, 5, 135, 199], "cpu")
    assert n == 5 and chunk_tab.tolist() == [[0, 5], [5, 64], [69, 64], [133, 2], [135, 64]]
    assert seq_ptr.tolist() == [0, 1, 1, 4, 5]
    assert tok_tab.shape == (199, 2) and tok_tab[4].tolist() == [0, 0] and tok_tab[5].tolist() == [5, 2]
    assert tok_tab[198].tolist() == [135, 3] and chunk_tab.dtype == seq_ptr.dtype == tok_tab.dtype == torch.int32
    t2 = ops.kda_varlen_tables(torch.tensor([0, 64]), "cpu")
    assert t2[0].tolist() == [[0, 64]] and t2[3] == 1
    for bad in ([1, 5], [0, 5, 3], [0]):
        with pytest.raises(ValueError):
            ops.kda_varlen_tables(bad, "cpu")
    mask = torch.tensor([[0, 0, 1, 1, 1], [1, 1, 0, 1, 0], [0, 0, 0, 0, 0]])
    idx, cu, mx = get_unpad_data(mask)
    assert idx.tolist() == [2, 3, 4, 5, 6, 8] and cu.tolist() == [0, 3, 6, 6] and mx == 3 and cu.dtype == torch.int32
    x = torch.arange(15 * 2, dtype=torch.float32).view(15, 2)
    packed = index_first_axis(x, idx)
    back = pad_input(packed, idx, 3, 5)
    assert back.shape == (3, 5, 2) and torch.equal(back.view(15, 2)[idx], packed)
    assert not back.view(15, 2)[[0, 1, 7, 9, 10, 14]].any()


def test_oracle_varlen_is_the_per_sequence_recurrence(golden_dir):
    """The packed restatements against the pinned dense ones: the third-party fixture's two batch rows laid end to end
    (plus an empty sequence) give each row's fixture output and state; the convolution likewise."""
    import os
    import numpy as np
    from oracle import kda as okda
    z = np.load(os.path.join(golden_dir, "kda_naive_small.npz"))
    q, k, v, g, beta, h0 = (torch.from_numpy(z[n]) for n in ("q", "k", "v", "g", "beta", "h0"))
    B, T = q.shape[:2]
    pack = lambda t: t.reshape(1, B * T, *t.shape[2:])
    cu = [0] + [T * (i + 1) for i in range(B)]
    cu = cu[:1] + cu[:1] + cu[1:]                                   # an empty sequence in front
    h0e = torch.cat([torch.ones_like(h0[:1]), h0])
    o, s = okda.kda_recurrent_varlen(pack(q), pack(k), pack(v), pack(g), pack(beta), cu, None, h0e)
    o_d, s_d = okda.kda_recurrent(q, k, v, g, beta, None, h0)
    assert torch.allclose(o.view_as(o_d), o_d, atol=1e-6) and torch.allclose(s[1:], s_d, atol=1e-6)
    assert torch.equal(s[0], h0e[0])
    x = torch.randn(2, 9, 16)
    w, st = torch.randn(16, 4), torch.randn(2, 16, 4)
    y, f = okda.short_conv_varlen(x.reshape(1, 18, 16), w, [0, 9, 18], None, st)
    y_d, f_d = okda.short_conv(x, w, None, st)
    assert torch.allclose(y.view_as(y_d), y_d, atol=1e-6) and torch.allclose(f, f_d)


def test_accounting_matches_the_oracle_formulas():
    """The package's FLOP / byte counts (what bench.py's roofline figures use) equal the oracle's."""
    from daisy_b200 import accounting as a
    from oracle import kda
    for B, T, H, D, W in ((8, 8192, 16, 128, 2048), (1, 65536, 16, 128, 8192), (2, 100, 3, 128, None), (1, 5, 1, 128, 9)):
        assert a.prefill_flops(B, T, H, D, W) == swa.prefill_flops(B, T, H, D, W)
    assert a.decode_bytes(64, 16, 128, 4095) == swa.decode_bytes(64, 16, 128, 4095)
    assert a.kda_bytes_per_token_head() == kda.kda_bytes_per_token_head() == 1540
    assert a.kda_flops_per_token_head() == kda.kda_flops_per_token_head()
    assert a.FP32_EPS == swa.FP32_EPS
