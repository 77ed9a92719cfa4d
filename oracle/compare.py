"""Comparator oracle (test infrastructure; see the package docstring).

Vectorised restatement of ``compare_tile_output_values``
(src/open_cake_ir/evaluation/core.py:645-696): every element is compared with
``|a - r| <= atol + rtol*|r|``; a non-finite pair matches only under the ``_ieee`` rule and
only as NaN with NaN or as equal infinities (core.py:681-686); a finite observed value
beyond the fp32 range is a mismatch.  ``inputs_unchanged`` restates the bitwise input check
(core.py:602-636).
"""
from __future__ import annotations

import torch


def compare(observed: torch.Tensor, reference: torch.Tensor, *, atol: float, rtol: float,
            ieee: bool = False):
    """Returns (ok, mismatches, max_abs_error) over all elements."""
    a = observed.detach().cpu().double().reshape(-1)
    r = reference.detach().cpu().double().reshape(-1)
    if a.numel() != r.numel():
        return False, max(a.numel(), r.numel()), float("nan")
    finite = torch.isfinite(a) & torch.isfinite(r)
    mismatch = torch.zeros_like(finite)
    nf = ~finite
    if ieee:
        same = (torch.isnan(a) & torch.isnan(r)) | (torch.isinf(a) & (a == r))
        mismatch |= nf & ~same
    else:
        mismatch |= nf
    err = (a - r).abs()
    mismatch |= finite & (err > atol + rtol * r.abs())
    mismatch |= finite & (a.abs() > 3.4028234663852886e38)
    max_err = float(err[finite].max()) if bool(finite.any()) else 0.0
    count = int(mismatch.sum())
    return count == 0, count, max_err


def bitwise_equal(a: torch.Tensor, b: torch.Tensor) -> bool:
    a = a.detach().cpu().contiguous(); b = b.detach().cpu().contiguous()
    return (a.dtype == b.dtype and a.shape == b.shape
            and torch.equal(a.view(torch.uint8), b.view(torch.uint8)))


def inputs_unchanged(before: dict, after: dict) -> bool:
    return set(before) == set(after) and all(bitwise_equal(before[k], after[k]) for k in before)


def rel_frobenius(observed: torch.Tensor, reference: torch.Tensor) -> float:
    a = observed.detach().cpu().double(); r = reference.detach().cpu().double()
    denom = float(r.norm())
    return float((a - r).norm()) / denom if denom > 0 else float((a - r).norm())
