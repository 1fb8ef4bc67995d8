"""The tcgen05 projection GEMM: plain bf16 output (the output projection) and the QKV form whose epilogue applies
the RMS norm and RoPE (the merged projection plus the element-wise tail of ``_calc_qkv``), against fp32 matmuls
and the oracle's transform on the same bf16 inputs."""
import pytest
import torch

from gpu_util import bf16_randn, assert_close_bf16
from oracle import swa

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (300, 256, 128), (77, 384, 192), (1000, 2048, 768), (4096, 768, 2048)])
def test_gemm_nt_matches_fp32_matmul(M, N, K):
    from daisy_b200 import ops
    x = bf16_randn(M, K, seed=M) * 0.5
    w = bf16_randn(N, K, seed=N + 1) * (K ** -0.5)
    c = ops.gemm_nt(x, w)
    ops.check_device_status(x.device)
    ref = x.float().cpu() @ w.float().cpu().t()
    assert_close_bf16(c, ref, f"gemm {M}x{N}x{K}")


def test_gemm_nt_strided_rows_and_batch_shape():
    from daisy_b200 import ops
    xw = bf16_randn(3, 50, 2 * 256, seed=4)
    x = xw[..., :256]                                              # row stride 512
    w = bf16_randn(512, 256, seed=5) * 0.06
    c = ops.gemm_nt(x, w)
    assert c.shape == (3, 50, 512)
    assert_close_bf16(c, x.float().cpu() @ w.float().cpu().t(), "strided")


@pytest.mark.parametrize("B,T,H,dim", [(1, 128, 2, 256), (2, 300, 2, 256), (1, 1024, 6, 768), (3, 77, 3, 384)])
def test_qkv_gemm_epilogue_matches_oracle(B, T, H, dim):
    """H = 3 makes 3*H*128 = 1152 columns, not a multiple of 256: the 128-column tile variant."""
    from daisy_b200 import ops
    D = 128
    x = bf16_randn(B, T, dim, seed=T)
    w = bf16_randn(3 * H * D, dim, seed=dim) * (dim ** -0.5)
    cos, sin = swa.rope_tables(D, T)
    qp, kp, vp = ops.qkv_gemm(x, w, cos.cuda(), sin.cuda(), H, swa.FP32_EPS)
    ops.check_device_status(x.device)
    qkv = (x.float().cpu() @ w.float().cpu().t()).view(B, T, 3 * H, D)
    q, k, v = qkv.chunk(3, dim=-2)
    qn, kn, vn = swa.qkv_transform(q, k, v, cos, sin, swa.FP32_EPS)
    assert_close_bf16(qp, qn, "q'")
    assert_close_bf16(kp, kn, "k'")
    assert_close_bf16(vp, vn, "v'")


def test_module_forward_matches_library_gemm_composition(golden_dir):
    """The module's forward runs on hand-written kernels only (fused QKV GEMM, attention, output GEMM); the same
    forward composed here from torch's GEMMs and the separate norm / RoPE pass agrees within bf16 rounding, and both
    meet the reference fixture's bar."""
    import os
    import numpy as np
    import torch.nn.functional as F
    from daisy_b200 import B200CausalSelfAttention, WindowMask, ops
    z = np.load(os.path.join(golden_dir, "csa_prefill_small.npz"))
    H, D, W = int(z["heads"]), int(z["head_dim"]), int(z["window"])
    os.environ["DISABLE_O_ZERO_INIT"] = "1"
    m = B200CausalSelfAttention(H * D, H, D).cuda().eval()
    m.norm_eps = swa.FP32_EPS
    with torch.no_grad():
        m.qkvo_w.copy_(torch.from_numpy(z["qkvo_w"]).to(m.qkvo_w.dtype))
    x = torch.from_numpy(z["x"]).bfloat16().cuda()
    B, T = x.shape[:2]
    with torch.inference_mode():
        y_nat = m(x, None, attn_mask=WindowMask(W))
        q, k, v = F.linear(x, m.qkvo_w[:3].flatten(end_dim=1)).view(B, T, 3 * H, D).chunk(3, dim=-2)
        y_lib, _, _ = ops.swa_prefill(q, k, v, m.rotary.cos, m.rotary.sin, W, m.attn_scale, m.norm_eps)
        y_lib = F.linear(y_lib.view(B, T, H * D), m.qkvo_w[3])
    ref = torch.from_numpy(z["y"])
    assert_close_bf16(y_nat, ref, "native forward vs reference fixture", max_tol=4e-2, mean_tol=4e-3)
    assert_close_bf16(y_nat, y_lib.float().cpu(), "native vs library projections", max_tol=3e-2, mean_tol=3e-3)


def test_qkv_gemm_value_embedding_gate():
    """The value-embedding gate in the GEMM epilogue: v' = g * norm(v) + (1 - g) * ve, q' and k' unaffected."""
    from daisy_b200 import ops
    B, T, H, D, dim = 2, 200, 2, 128, 256
    x = bf16_randn(B, T, dim, seed=3)
    w = bf16_randn(3 * H * D, dim, seed=4) * (dim ** -0.5)
    ve = bf16_randn(B, T, H * D, seed=5)
    cos, sin = swa.rope_tables(D, T)
    logit = torch.tensor([-1.5163], device="cuda")
    qp, kp, vp = ops.qkv_gemm(x, w, cos.cuda(), sin.cuda(), H, swa.FP32_EPS, ve=ve, ve_gate_logit=logit)
    q0, k0, v0 = ops.qkv_gemm(x, w, cos.cuda(), sin.cuda(), H, swa.FP32_EPS)
    ops.check_device_status(x.device)
    assert torch.equal(qp, q0) and torch.equal(kp, k0)
    v = (x.float().cpu() @ w.float().cpu().t()).view(B, T, 3 * H, D)[:, :, 2 * H:]
    g = torch.sigmoid(torch.tensor(-1.5163))
    ref = g * swa.rms_norm(v, swa.FP32_EPS) + (1 - g) * ve.float().cpu().view(B, T, H, D)
    assert_close_bf16(vp, ref, "ve gate in the epilogue")


@pytest.mark.parametrize("M,N,K", [(1, 6144, 2048), (2, 2048, 2048), (5, 392, 256), (8, 777, 1024), (17, 2048, 512), (64, 256, 2048),
                                   (3, 512, 12288), (8, 130, 16384)])
def test_skinny_gemm_matches_fp32_reference(M, N, K):
    """The weight-streaming projection of a decode step: F.linear for up to 64 rows."""
    from daisy_b200 import ops
    x = bf16_randn(M, K, seed=M + N)
    w = bf16_randn(N, K, seed=K) * (K ** -0.5)
    y = ops.gemm_skinny(x, w)
    ref = x.float().cpu() @ w.float().cpu().t()
    assert_close_bf16(y, ref, f"skinny {M}x{N}x{K}")
    # a [B,1,K] input and a strided weight view (rows of a larger matrix), as the module passes them
    big = bf16_randn(2 * N, K, seed=K + 1) * (K ** -0.5)
    y3 = ops.gemm_skinny(x.view(M, 1, K), big[N:])
    assert y3.shape == (M, 1, N)
    assert_close_bf16(y3.view(M, N), x.float().cpu() @ big[N:].float().cpu().t(), "strided weight")
    assert torch.equal(ops.gemm_skinny(x, w), y), "not run-to-run deterministic"


def test_skinny_gemm_after_a_kernel_that_writes_its_operands():
    """The skinny projection is launched as a dependent grid and hints its weight rows into L2 before it waits for the
    preceding kernel.  Both operands are produced by kernels launched immediately before it on the same stream, again
    and again with new values: every result must see the latest ones."""
    from daisy_b200 import ops
    M, N, K = 2, 2048, 2048
    w = torch.empty(N, K, device="cuda", dtype=torch.bfloat16)
    x = torch.empty(M, K, device="cuda", dtype=torch.bfloat16)
    g = torch.Generator(device="cuda").manual_seed(5)
    srcs = [((torch.randn(N, K, device="cuda", generator=g) * K ** -0.5).bfloat16(),
             torch.randn(M, K, device="cuda", generator=g).bfloat16()) for _ in range(6)]
    outs = []
    for ws, xs in srcs:
        w.copy_(ws)                                               # a kernel that writes the weights ...
        x.copy_(xs)                                               # ... and one that writes the rows, right before the call
        outs.append(ops.gemm_skinny(x, w).clone())
    for (ws, xs), y in zip(srcs, outs):
        assert_close_bf16(y, xs.float().cpu() @ ws.float().cpu().t(), "operands written by the preceding kernels")
