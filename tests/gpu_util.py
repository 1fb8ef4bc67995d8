"""Helpers shared by the GPU parity tests."""
import torch

MAX_ABS_TOL = 2e-2     # bf16 outputs vs the fp32 oracle: max-abs <= 2e-2 ...
MEAN_ABS_TOL = 2e-3    # ... and mean-abs <= 2e-3


def bf16_randn(*shape, seed=0, device="cuda"):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(*shape, generator=g).bfloat16().to(device)


def assert_close_bf16(got, ref, what="", max_tol=MAX_ABS_TOL, mean_tol=MEAN_ABS_TOL):
    got, ref = got.float().cpu(), ref.float().cpu()
    assert got.shape == ref.shape, (got.shape, ref.shape)
    assert torch.isfinite(got).all(), f"{what}: non-finite values"
    err = (got - ref).abs()
    assert err.max().item() <= max_tol, f"{what}: max-abs {err.max().item():.4g} > {max_tol}"
    assert err.mean().item() <= mean_tol, f"{what}: mean-abs {err.mean().item():.4g} > {mean_tol}"
