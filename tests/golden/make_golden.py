"""Generate the golden fixtures in this directory from the REFERENCE's own code.

Run once in a container that has the reference tree (its root is taken from ``DAISY_REFERENCE_ROOT``,
default ``../reference`` beside the repository's parent directory) and, for the KDA fixture, the third-party
``flash-linear-attention`` package:

    python tests/golden/make_golden.py

It imports ``models.daisy.attention.CausalSelfAttention``, ``inference.kv_cache.KVCache``
and ``models.daisy.daisy_core.build_attn_mask`` from the reference, runs them in fp32
on the CPU exactly the way the reference's tests do (``tests/test_attention.py:6-13``:
weights cast to fp32, W_o re-initialised non-zero), and stores inputs and outputs as
``.npz``.  The fixtures travel with the repository; the reference does not.
"""
import os
import sys

import numpy as np
import torch

REF = os.environ.get("DAISY_REFERENCE_ROOT",
                     os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))), "reference"))
HERE = os.path.dirname(os.path.abspath(__file__))
os.environ["DISABLE_O_ZERO_INIT"] = "1"
sys.path.insert(0, REF)
import tempfile                                                       # noqa: E402
os.chdir(tempfile.mkdtemp(prefix="daisy_golden_"))                    # the reference's logger creates ./logs

from models.daisy.attention import CausalSelfAttention, _apply_rope   # noqa: E402
from models.daisy.daisy_core import build_attn_mask                   # noqa: E402
from models.daisy.functional import norm                              # noqa: E402
from inference.kv_cache import KVCache                                # noqa: E402

EOS = 50256


def make_attn(dim, heads, head_dim, seed):
    torch.manual_seed(seed)
    attn = CausalSelfAttention(dim=dim, num_heads=heads, head_dim=head_dim)
    attn.qkvo_w = torch.nn.Parameter(attn.qkvo_w.float())
    with torch.no_grad():
        attn.qkvo_w.normal_(mean=0.0, std=dim ** -0.5)
    return attn.eval()


def mask_for(T, window):
    ids = torch.zeros(1, T, dtype=torch.long)          # no EOS -> single document
    return build_attn_mask(ids, window, EOS)


@torch.no_grad()
def csa_prefill_case():
    B, T, H, D, W = 2, 96, 2, 128, 40
    dim = H * D
    attn = make_attn(dim, H, D, seed=0)
    x = torch.randn(B, T, dim)
    m = mask_for(T, W)
    y_fwd = attn.forward(x, None, attn_mask=m)
    y, k, v = attn.prefill(x, None, attn_mask=m)
    assert torch.equal(y, y_fwd)
    np.savez_compressed(os.path.join(HERE, "csa_prefill_small.npz"),
                        x=x.numpy(), qkvo_w=attn.qkvo_w.detach().numpy(), window=W, heads=H, head_dim=D,
                        y=y.numpy(), k=k.contiguous().numpy(), v=v.contiguous().numpy())


@torch.no_grad()
def csa_step_case():
    """Step chain through the reference KVCache: capacity 8, window 4 and window 12 (> capacity),
    21 tokens from an empty cache; then prefill of 13 tokens + bulk_write_packed + 8 steps."""
    B, H, D, CAP, T = 1, 2, 128, 8, 21
    dim = H * D
    attn = make_attn(dim, H, D, seed=1)
    x = torch.randn(B, T, dim)
    out = dict(x=x.numpy(), qkvo_w=attn.qkvo_w.detach().numpy(), heads=H, head_dim=D, cap=CAP)
    for window in (4, 12):
        cache = KVCache(L=1, B=B, H=H, W=CAP, D=D, device="cpu", dtype=torch.float32)
        ys, ks = [], []
        for t in range(T):
            kc, vc = cache.view(0)
            y, k, v = attn.step(x[:, t:t + 1], kc, vc, pos=cache.t, ve=None, window=window)
            cache.write(0, k, v)
            cache.advance()
            ys.append(y); ks.append(k)
        out[f"y_steps_w{window}"] = torch.cat(ys, 1).numpy()
        out[f"k_steps_w{window}"] = torch.cat(ks, 1).numpy()
        out[f"ring_k_w{window}"] = cache.k[0].numpy()
    # prefill + bulk write + steps (window 4)
    window, P = 4, 13
    y_p, k_p, v_p = attn.prefill(x[:, :P], None, attn_mask=mask_for(P, window))
    cache = KVCache(L=1, B=B, H=H, W=CAP, D=D, device="cpu", dtype=torch.float32)
    cache.bulk_write_packed(torch.stack([k_p[None], v_p[None]]), P)
    ys = []
    for t in range(P, T):
        kc, vc = cache.view(0)
        y, k, v = attn.step(x[:, t:t + 1], kc, vc, pos=cache.t, ve=None, window=window)
        cache.write(0, k, v)
        cache.advance()
        ys.append(y)
    out["y_prefill13_w4"] = y_p.numpy()
    out["y_after_bulk_w4"] = torch.cat(ys, 1).numpy()
    np.savez_compressed(os.path.join(HERE, "csa_step_small.npz"), **out)


@torch.no_grad()
def swa_inner_case():
    """Inner functions on post-projection q,k,v with a full base-10000 RoPE table
    (the benchmark configs name base 10000; the reference module hard-codes 1024):
    norm -> _apply_rope -> SDPA(attn_mask, scale=0.12), as models/daisy/attention.py:121-125,145."""
    B, T, H, D, W = 1, 200, 2, 128, 64
    g = torch.Generator().manual_seed(2)
    q, k, v = (torch.randn(B, T, H, D, generator=g) for _ in range(3))
    freq = (1.0 / 10000.0) ** torch.linspace(0, 1, steps=D // 2, dtype=torch.float32)
    theta = torch.einsum("i,j->ij", torch.arange(T, dtype=torch.float32), freq)
    cos, sin = theta.cos(), theta.sin()
    qn, kn, vn = norm(q), norm(k), norm(v)
    qn = _apply_rope(qn, cos[None, :, None, :], sin[None, :, None, :])
    kn = _apply_rope(kn, cos[None, :, None, :], sin[None, :, None, :])
    y = torch.nn.functional.scaled_dot_product_attention(
        qn.transpose(1, 2), kn.transpose(1, 2), vn.transpose(1, 2), is_causal=False,
        attn_mask=mask_for(T, W), scale=0.12).transpose(1, 2)
    np.savez_compressed(os.path.join(HERE, "swa_inner_small.npz"),
                        q=q.numpy(), k=k.numpy(), v=v.numpy(), cos=cos.numpy(), sin=sin.numpy(), window=W,
                        y=y.contiguous().numpy(), kn=kn.numpy(), vn=vn.numpy())


@torch.no_grad()
def kda_case():
    """Third-party naive recurrence (fla.ops.kda.naive.naive_recurrent_kda, fla 0.5.1) on
    bf16-representable inputs; q,k are L2-normalised before the call with the same formula
    the chunk kernel applies when use_qk_l2norm_in_kernel=True."""
    import fla
    from fla.ops.kda.naive import naive_recurrent_kda
    B, T, H, K, V = 1, 96, 2, 128, 128
    g_ = torch.Generator().manual_seed(3)
    bf = lambda t: t.bfloat16().float()
    q, k, v = (bf(torch.randn(B, T, H, K, generator=g_)) for _ in range(3))
    g = torch.nn.functional.logsigmoid(torch.randn(B, T, H, K, generator=g_))
    beta = torch.sigmoid(torch.randn(B, T, H, generator=g_))
    h0 = 0.1 * torch.randn(B, H, K, V, generator=g_)
    l2 = lambda t: t * torch.rsqrt(t.pow(2).sum(-1, keepdim=True) + 1e-6)
    o, s = naive_recurrent_kda(l2(q), l2(k), v, g, beta, output_final_state=True)
    o2, s2 = naive_recurrent_kda(l2(q), l2(k), v, g, beta, initial_state=h0.clone(), output_final_state=True)
    np.savez_compressed(os.path.join(HERE, "kda_naive_small.npz"),
                        q=q.numpy(), k=k.numpy(), v=v.numpy(), g=g.numpy(), beta=beta.numpy(), h0=h0.numpy(),
                        o=o.numpy(), s=s.numpy(), o_h0=o2.numpy(), s_h0=s2.numpy(), fla_version=fla.__version__)


def doc_mask_case():
    """``build_attn_mask`` with EOS tokens in the sequence (document masking, daisy_core.py:53-69) and the
    module's ``forward`` under that mask."""
    torch.manual_seed(5)
    dim, heads, hd, T, window, eos = 256, 2, 128, 200, 64, 7
    attn = make_attn(dim, heads, hd, seed=5)
    g = torch.Generator().manual_seed(6)
    seq = torch.randint(8, 100, (1, T), generator=g)
    for p in (0, 1, 40, 41, 90, 150, 199):
        seq[0, p] = eos
    x = torch.randn(1, T, dim, generator=g)
    mask = build_attn_mask(seq, window, eos)
    with torch.no_grad():
        y = attn(x, None, attn_mask=mask)
    np.savez_compressed(os.path.join(HERE, "doc_mask_small.npz"),
                        seq=seq.numpy(), eos=np.int64(eos), window=np.int64(window), x=x.numpy(),
                        qkvo_w=attn.qkvo_w.detach().numpy(), mask=mask[0, 0].numpy(), y=y.numpy(),
                        cos=attn.rotary.cos[:T].numpy(), sin=attn.rotary.sin[:T].numpy())
    print("doc_mask_small", tuple(y.shape))


def csa_backward_case():
    """The reference module's CPU SDPA path under autograd (the training form evaluated where flex-attention is not
    available, models/daisy/attention.py:141-154,164-171): forward with the dense window + document mask, a fixed
    cotangent, gradients with respect to the input and the merged weights."""
    dim, heads, hd, T, window, eos = 256, 2, 128, 160, 48, 7
    attn = make_attn(dim, heads, hd, seed=11)
    g = torch.Generator().manual_seed(12)
    seq = torch.randint(8, 100, (1, T), generator=g)
    for p_ in (30, 31, 100):
        seq[0, p_] = eos
    x = torch.randn(1, T, dim, generator=g).requires_grad_(True)
    cot = torch.randn(1, T, dim, generator=g)
    mask = build_attn_mask(seq, window, eos)
    y = attn(x, None, attn_mask=mask)
    (y * cot).sum().backward()
    np.savez_compressed(os.path.join(HERE, "csa_backward_small.npz"),
                        seq=seq.numpy(), eos=np.int64(eos), window=np.int64(window), x=x.detach().numpy(), cot=cot.numpy(),
                        qkvo_w=attn.qkvo_w.detach().numpy(), y=y.detach().numpy(), dx=x.grad.numpy(),
                        dw=attn.qkvo_w.grad.numpy())
    print("csa_backward_small", tuple(y.shape), float(x.grad.abs().max()), float(attn.qkvo_w.grad.abs().max()))


def flex_blockmask_case():
    """Block lists of ``DaisyCore.create_blockmasks`` (daisy_core.py:182-229) for sequences with documents
    of many lengths: kv_num_blocks / kv_indices / full_kv_num_blocks / full_kv_indices of the long and the short
    mask, for several window sizes.  (The CPU path of ``flex_attention`` applies ``mask_mod`` densely and ignores
    the lists, so the lists themselves are the fixture; the compiled GPU kernel visits exactly the listed
    blocks and applies ``mask_mod`` inside the partial ones.)"""
    import types
    from models.daisy.daisy_core import DaisyCore
    eos, T = 7, 2048
    g = torch.Generator().manual_seed(17)
    out = {}
    for case in range(3):
        seq = torch.randint(8, 100, (T,), generator=g)
        n_eos = (3, 12, 40)[case]
        seq[torch.randperm(T, generator=g)[:n_eos]] = eos
        if case == 1:
            seq[640:1400] = 9                                      # one long document
        out[f"seq{case}"] = seq.numpy()
        for wb in (2, 3, 6, 8):
            bms = DaisyCore.create_blockmasks(types.SimpleNamespace(eos_token_id=eos), seq,
                                              torch.tensor(wb, dtype=torch.int32), 2)
            for name, bm in (("long", bms[-1]), ("short", bms[0] if wb // 2 >= 1 else None)):
                if bm is None:
                    continue
                bm = bms[-1] if name == "long" else DaisyCore.create_blockmasks(
                    types.SimpleNamespace(eos_token_id=eos), seq, torch.tensor(wb, dtype=torch.int32), 5)[1]
                key = f"c{case}_wb{wb}_{name}"
                out[key + "_pn"] = bm.kv_num_blocks[0, 0].numpy()
                out[key + "_pi"] = bm.kv_indices[0, 0].numpy()
                out[key + "_fn"] = bm.full_kv_num_blocks[0, 0].numpy()
                out[key + "_fi"] = bm.full_kv_indices[0, 0].numpy()
    out["eos"] = np.int64(eos)
    np.savez_compressed(os.path.join(HERE, "flex_blockmask_lists.npz"), **out)
    print("flex_blockmask_lists", len(out))


def kda_gate_case():
    """``fused_kda_gate`` as the KDA layer calls it (attention_kimi.py:132), through the reference's own
    pure-PyTorch implementation ``_gate_impl`` (fla_custom_ops.py:71-103): fp32 and bf16 inputs, with the
    softplus threshold (20) exercised on both sides."""
    from models.daisy.fla_custom_ops import _gate_impl
    g = torch.Generator().manual_seed(11)
    H, Dk = 3, 128
    x = torch.randn(2, 37, H * Dk, generator=g) * 6.0
    x[0, 0, :8] = torch.tensor([19.5, 20.0, 20.5, 25.0, -30.0, 0.0, 35.0, -0.5])
    A_log = torch.log(torch.empty(H).uniform_(1.0, 16.0, generator=g))
    bias = torch.randn(H * Dk, generator=g)
    y32, _ = _gate_impl(x, A_log, Dk, bias, None, 1.0, 20.0)
    ybf, _ = _gate_impl(x.bfloat16(), A_log, Dk, bias, None, 1.0, 20.0)
    ynb, _ = _gate_impl(x, A_log, Dk, None, None, 1.0, 20.0)
    np.savez_compressed(os.path.join(HERE, "kda_gate_small.npz"),
                        x=x.numpy(), A_log=A_log.numpy(), bias=bias.numpy(), y_fp32=y32.numpy(),
                        y_bf16_as_fp32=ybf.float().numpy(), y_nobias=ynb.numpy())
    print("kda_gate_small", tuple(y32.shape))


def kda_layer_case():
    """The two row-wise passes of the KDA layer whose kernels are third-party Triton code that has no CPU path:
    the short convolution through ``torch.nn.Conv1d``'s own forward on an ``fla.modules.ShortConvolution``
    instance (the class *is* that Conv1d: its parameters, groups and padding define the operator), in one piece
    and as prefill + single-token steps through the carried state; and the gated norm through
    ``torch.nn.functional.rms_norm`` / ``silu`` / ``sigmoid`` in the order of
    ``CompilableFusedRMSNormGated.forward`` (attention_kimi.py:52-60)."""
    from fla.modules import ShortConvolution
    g = torch.Generator().manual_seed(12)
    out = {}
    for W, use_bias in ((4, False), (3, True), (2, False)):
        C, B, T = 64, 2, 21
        conv = ShortConvolution(C, W, bias=use_bias, activation="silu")
        with torch.no_grad():
            conv.weight.copy_(torch.randn(C, 1, W, generator=g) * 0.5)
            if use_bias:
                conv.bias.copy_(torch.randn(C, generator=g) * 0.3)
            x = torch.randn(B, T, C, generator=g)
            y = torch.nn.functional.silu(torch.nn.Conv1d.forward(conv, x.transpose(1, 2))[..., :T]).transpose(1, 2)
        tag = f"conv_w{W}"
        out[tag + "_x"] = x.numpy(); out[tag + "_weight"] = conv.weight.detach().numpy()
        out[tag + "_bias"] = conv.bias.detach().numpy() if use_bias else np.zeros(0, np.float32)
        out[tag + "_y"] = y.contiguous().numpy()
    D = 128
    x = torch.randn(3, 9, 2, D, generator=g) * 2.0
    gate = torch.randn(3, 9, 2, D, generator=g) * 3.0
    wgt = 1.0 + 0.2 * torch.randn(D, generator=g)
    F = torch.nn.functional
    normed = F.rms_norm(x, (D,), wgt, 1e-6) * F.silu(gate)
    xb, gb, wb = x.bfloat16(), gate.bfloat16(), wgt.bfloat16()
    normed_b = (F.rms_norm(xb.float(), (D,), wb.float(), 1e-6) * F.silu(gb.float())).bfloat16()
    y_b = normed_b * torch.sigmoid(gb)                               # bf16 x bf16, as the module's last line
    out.update(norm_x=x.numpy(), norm_gate=gate.numpy(), norm_weight=wgt.numpy(), norm_swish=normed.numpy(),
               norm_sigmoid=(F.rms_norm(x, (D,), wgt, 1e-6) * torch.sigmoid(gate)).numpy(),
               norm_ref_bf16_as_fp32=y_b.float().numpy())
    # the layer's parameter names and shapes, from the reference class itself (state-dict compatibility)
    from models.daisy.attention_kimi import KimiLinearSelfAttention
    ref_layer = KimiLinearSelfAttention(256, 2, 64, 128)
    names = sorted(f"{n}:{'x'.join(map(str, p.shape))}:{str(p.dtype).replace('torch.', '')}" for n, p in ref_layer.named_parameters())
    out["layer_parameters"] = np.array(names)
    np.savez_compressed(os.path.join(HERE, "kda_layer_small.npz"), **out)
    print("kda_layer_small", sorted(out))


if __name__ == "__main__":
    csa_prefill_case()
    csa_step_case()
    swa_inner_case()
    kda_case()
    kda_gate_case()
    kda_layer_case()
    doc_mask_case()
    csa_backward_case()
    flex_blockmask_case()
    for f in sorted(os.listdir(HERE)):
        if f.endswith(".npz"):
            print(f, os.path.getsize(os.path.join(HERE, f)))
