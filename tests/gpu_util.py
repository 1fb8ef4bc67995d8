"""Helpers shared by the GPU parity tests."""
import torch

MAX_ABS_TOL = 2e-2     # bf16 outputs vs the fp32 oracle: max-abs <= 2e-2 ...
MEAN_ABS_TOL = 2e-3    # ... and mean-abs <= 2e-3


def bf16_randn(*shape, seed=0, device="cuda"):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(*shape, generator=g).bfloat16().to(device)


def assert_close_bf16(got, ref, what="", max_tol=MAX_ABS_TOL, mean_tol=MEAN_ABS_TOL):
    """The stated tolerances are absolute and meant for outputs of magnitude <= 1 (an average over a
    window of unit-RMS values).  A bf16 value of magnitude m carries a rounding error of up to m * 2^-8, so
    for tensors whose entries exceed 1 (tiny windows, the normalised k/v rows themselves) both bounds scale
    with max|ref|."""
    got, ref = got.float().cpu(), ref.float().cpu()
    mag = max(1.0, ref.abs().max().item()) if ref.numel() else 1.0
    max_tol, mean_tol = max_tol * mag, mean_tol * mag
    assert got.shape == ref.shape, (got.shape, ref.shape)
    assert torch.isfinite(got).all(), f"{what}: non-finite values"
    err = (got - ref).abs()
    assert err.max().item() <= max_tol, f"{what}: max-abs {err.max().item():.4g} > {max_tol}"
    assert err.mean().item() <= mean_tol, f"{what}: mean-abs {err.mean().item():.4g} > {mean_tol}"
