"""The allocation-free decode entry point (scratch inside the library) against the workspace entry point.

For hosts that cannot call cudaMalloc -- a stream capture in progress, a plugin under a pool allocator, an
FFI embedder holding only the tensors it was given -- `daisy_b200_swa_decode_step_static` must give exactly
what `daisy_b200_swa_decode_step` gives.  Checked through the C ABI, twice in a row (the built-in array keeps
the previous call's contents), and for the size limit.  Collected last on purpose."""
import pytest
import torch

from gpu_util import bf16_randn

pytestmark = pytest.mark.gpu


def _args(q, k, v, rk, rv, t, cap, window, cos, sin, out, flags):
    B, _, H, D = q.shape
    return [q.data_ptr(), k.data_ptr(), v.data_ptr(), q.stride(0), q.stride(2), k.stride(0), k.stride(2),
            v.stride(0), v.stride(2), rk.data_ptr(), rv.data_ptr(), rk.stride(0), rk.stride(1), rk.stride(2),
            t, cap, window, cos.data_ptr(), sin.data_ptr(), out.data_ptr(), out.stride(0), out.stride(2),
            None, None, B, H, D, 0.12, 1.1920929e-07, flags]


def test_static_decode_equals_workspace_decode():
    from daisy_b200 import _lib
    from oracle import swa
    L = _lib.lib()
    B, H, D, cap, window, splits = 3, 4, 128, 512, 300, 5
    st = torch.cuda.current_stream().cuda_stream
    assert L.daisy_b200_swa_decode_static_capacity() == 4096
    cos, sin = swa.rope_tables(D, 2048)
    cos, sin = cos.cuda(), sin.cuda()
    ws = torch.empty(L.daisy_b200_swa_decode_workspace_bytes(B, H, D, splits), dtype=torch.uint8, device="cuda")
    for call, t in enumerate((700, 701)):                        # two calls in a row, ring wrapped
        rk, rv = bf16_randn(B, H, cap, D, seed=40 + call), bf16_randn(B, H, cap, D, seed=50 + call)
        q, k, v = (bf16_randn(B, 1, H, D, seed=60 + 3 * call + i) for i in range(3))
        ref = torch.empty(B, 1, H, D, dtype=torch.bfloat16, device="cuda")
        got = torch.full_like(ref, float("nan"))
        a = _args(q, k, v, rk, rv, t, cap, window, cos[t], sin[t], ref, _lib.QKV_DEFAULT)
        assert L.daisy_b200_swa_decode_step(*a, ws.data_ptr(), ws.numel(), splits, None, st) == 0
        a = _args(q, k, v, rk, rv, t, cap, window, cos[t], sin[t], got, _lib.QKV_DEFAULT)
        assert L.daisy_b200_swa_decode_step_static(*a, splits, None, st) == 0
        torch.cuda.synchronize()
        assert torch.isfinite(got.float()).all()
        assert torch.equal(got, ref), f"call {call}: max diff {(got.float() - ref.float()).abs().max().item()}"


def test_static_decode_rejects_oversize():
    from daisy_b200 import _lib
    from oracle import swa
    L = _lib.lib()
    B, H, D, cap = 2, 4, 128, 64
    rk, rv = bf16_randn(B, H, cap, D, seed=1), bf16_randn(B, H, cap, D, seed=2)
    q, k, v = (bf16_randn(B, 1, H, D, seed=3 + i) for i in range(3))
    cos, sin = swa.rope_tables(D, 64)
    cos, sin = cos.cuda(), sin.cuda()
    out = torch.empty(B, 1, H, D, dtype=torch.bfloat16, device="cuda")
    a = _args(q, k, v, rk, rv, 10, cap, 16, cos[10], sin[10], out, _lib.QKV_DEFAULT)
    too_many = 4096 // (B * H) + 1
    assert L.daisy_b200_swa_decode_step_static(*a, too_many, None, torch.cuda.current_stream().cuda_stream) == _lib.EWORKSPACE
