"""tcgen05 building blocks: smem x smem (K-major B), smem x smem (MN-major B) and TMEM x smem products
against a float32 matmul of the same bf16 values."""
import pytest
import torch

from gpu_util import bf16_randn

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("K", [64, 128])
@pytest.mark.parametrize("mode", [0, 1, 2])
def test_umma_product(mode, K):
    from daisy_b200 import ops
    a = bf16_randn(128, K, seed=1)
    b = bf16_randn(128, K, seed=2) if mode == 0 else bf16_randn(K, 128, seed=2)
    c = ops.selftest_umma(a, b, mode)
    ops.check_device_status(a.device)
    ref = a.float() @ (b.float().t() if mode == 0 else b.float())
    err = (c - ref).abs().max().item()
    assert err < 1e-3, f"mode {mode} K {K}: max err {err}"


def test_bounded_wait_reports_timeout_and_context_survives():
    """A device-side wait that nothing satisfies runs into its time limit: the kernel raises its abort flag,
    writes DAISY_ETIMEOUT into the status word, frees its TMEM and returns; the host reads the status, and the
    context keeps working (the next launches allocate TMEM and compute correctly)."""
    from daisy_b200 import ops, _lib
    a, b = bf16_randn(128, 128, seed=1), bf16_randn(128, 128, seed=2)
    ops.selftest_umma(a, b, 3)
    with pytest.raises(_lib.DaisyB200Error) as e:
        ops.check_device_status(a.device)
    assert e.value.code == _lib.ETIMEOUT
    c = ops.selftest_umma(a, b, 0)
    ops.check_device_status(a.device)                              # the status word was cleared by the read above
    assert (c - a.float() @ b.float().t()).abs().max().item() < 1e-3
