"""Two-output residual add + RMSNorm oracle (test infrastructure; see the package docstring).

Follows src/open_cake_ir/tasks/add_rmsnorm.py:131-143 (``reference_outputs``):
``z = RN_bf16(delta + residual)`` element-wise (the sum of two bf16 values is exact in double,
so one rounding to fp32 and one to bf16, both to nearest even -- the reference's ``_round``,
src/open_cake_ir/tasks/tiles/workload.py:132-142 -- land on the same value), ``residual_out = z``,
and per row ``out = RN_bf16(z * (1/sqrt(fsum(z*z)/width + eps)) * weight)`` with the row sum an
exactly rounded ``math.fsum`` and every product in double.  The input materialiser restates
add_rmsnorm.py:103-128 (``random.Random(seed)``, one stream for delta/residual pairs and then the
weights).
"""
from __future__ import annotations

import math
import random
import struct

import numpy as np
import torch

EPSILON = 1e-6
CASES = {"primary": ("uniform", 7601), "zeros": ("zeros", 7602), "rounding_ties": ("rounding_ties", 7603),
         "cancellation": ("cancellation", 7604), "mixed_magnitude": ("mixed_magnitude", 7605)}


def _round_bf16(value: float) -> float:
    bits = struct.unpack("<I", struct.pack("<f", value))[0]
    bits = (bits + 0x7FFF + ((bits >> 16) & 1)) & 0xFFFF0000
    return struct.unpack("<f", struct.pack("<I", bits))[0]


def _bf16_tensor(values64: np.ndarray) -> torch.Tensor:
    """double -> fp32 (nearest even) -> bf16 (nearest even), as the reference's ``_round`` does."""
    return torch.from_numpy(values64.astype(np.float32)).to(torch.bfloat16)


def add_rmsnorm_reference(delta: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor, eps: float = EPSILON):
    """delta, residual bf16 [R, C]; weight bf16 [C] -> {"out": bf16 [R, C], "residual_out": bf16 [R, C]}."""
    z = _bf16_tensor(delta.double().numpy() + residual.double().numpy())
    zd = z.double().numpy()
    w = weight.double().numpy()
    rows, width = zd.shape
    out = np.empty_like(zd)
    squares = zd * zd
    for r in range(rows):
        inverse = 1.0 / math.sqrt(math.fsum(squares[r].tolist()) / width + eps)
        out[r] = zd[r] * inverse * w
    return {"out": _bf16_tensor(out), "residual_out": z}


def materialize_reference_case(case_id: str, rows: int = 128, columns: int = 2560) -> dict[str, torch.Tensor]:
    """Inputs of one reference case (add_rmsnorm.py:103-128)."""
    _, seed = CASES[case_id]
    count = rows * columns
    rng = random.Random(seed)
    delta, residual = np.empty(count), np.empty(count)
    for i in range(count):
        if case_id == "zeros":
            d, r = (-0.0, -0.0) if i % 2 else (0.0, 0.0)
        elif case_id == "rounding_ties":
            d, r = 2 ** -8, 1.0 + (i % 2) * 2 ** -7
        elif case_id == "cancellation":
            r = _round_bf16(rng.uniform(-2, 2))
            d = -r if i % 2 else _round_bf16(-r + 2 ** -8)
        elif case_id == "mixed_magnitude":
            d, r = ((-1) ** i * 2.0 ** rng.randint(-12, 8), (-1) ** (i + 1) * 2.0 ** rng.randint(-12, 8))
        else:
            d, r = rng.uniform(-2, 2), rng.uniform(-2, 2)
        delta[i], residual[i] = d, r
    weights = np.array([1.0 if i == 0 else (0.0 if (i + 1) % 17 == 0 else rng.uniform(-1.5, 1.5)) for i in range(columns)])
    return {"delta": _bf16_tensor(delta).reshape(rows, columns), "residual": _bf16_tensor(residual).reshape(rows, columns),
            "weight": _bf16_tensor(weights)}
