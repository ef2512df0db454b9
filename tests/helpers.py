"""Shared pieces of the parity tests: tolerances, error metric and the oracle calls."""
import torch

from oracle import c_oracle

# max |x - ref| / max |ref| per output tensor; the reference states no tolerance
# (its tests print norms, clusten/test_qk_kernel.py:48-50), these are the targets of this build
TOL = {torch.float32: 1e-5, torch.float64: 1e-12, torch.float16: 2e-3, torch.bfloat16: 2e-2}


def rel_err(x, ref):
    x = x.detach().double().cpu()
    ref = ref.detach().double().cpu()
    denom = ref.abs().max().clamp_min(1e-30)
    return ((x - ref).abs().max() / denom).item()


def assert_close(x, ref, dtype, what):
    assert x.shape == ref.shape, f"{what}: shape {tuple(x.shape)} vs {tuple(ref.shape)}"
    assert torch.isfinite(x.float()).all(), f"{what}: non-finite values"
    err = rel_err(x, ref)
    assert err <= TOL[dtype], f"{what}: relative error {err:.3e} > {TOL[dtype]:.1e}"


def exact(op, direction, *tensors):
    """fp64 C-oracle result on the (already dtype-rounded) inputs, as CPU double tensors."""
    args = [t.detach().cpu().double() if t.is_floating_point() else t.detach().cpu() for t in tensors]
    return getattr(c_oracle, f"{op}_{direction}")(*args)
