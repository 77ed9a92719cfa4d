"""RMSNorm oracle (test infrastructure; see the package docstring).

Follows src/open_cake_ir/tasks/solx_fib/workload.py:334-358 (``reference_outputs``): the
row sum of squares is an exactly rounded ``math.fsum`` in double precision, the inverse is
``1/sqrt(sum/width + eps)`` in double, every output is ``value*inverse*weight`` in double,
rounded first to fp32 and then to bf16, both round-to-nearest-even (the reference's
``_round``, src/open_cake_ir/tasks/tiles/workload.py:132-142).  The fused variant first
rounds ``x + residual`` to fp32 (workload.py:348-349).
"""
from __future__ import annotations

import math
import random

import numpy as np
import torch


def _to_bf16_via_fp32(values64: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(values64.astype(np.float32)).to(torch.bfloat16)


def rmsnorm_reference(x: torch.Tensor, weight: torch.Tensor, eps: float,
                      residual: torch.Tensor | None = None) -> torch.Tensor:
    """x, residual: bf16 [R, C]; weight: bf16 [C] -> bf16 [R, C]."""
    values = x.double().numpy()
    if residual is not None:
        values = (values + residual.double().numpy()).astype(np.float32).astype(np.float64)
    w = weight.double().numpy()
    rows, width = values.shape
    out = np.empty_like(values)
    squares = values * values  # exact in double: inputs carry at most 24 significant bits
    for r in range(rows):
        inverse = 1.0 / math.sqrt(math.fsum(squares[r].tolist()) / width + eps)
        out[r] = values[r] * inverse * w
    return _to_bf16_via_fp32(out)


def rmsnorm_fast(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """Multi-threaded torch restatement used only as the timed CPU baseline: the same
    definition with the row reduction in fp64 by torch instead of ``math.fsum``."""
    v = x.double()
    inverse = torch.rsqrt(v.square().mean(dim=1, keepdim=True) + eps)
    return (v * inverse * weight.double()).float().to(torch.bfloat16)


# --- the reference's input materialiser, restated (workload.py:307-331) ------------------
_MODES = {"primary": "uniform", "zeros": "zeros", "near_zero": "near_zero",
          "alternating": "alternating", "mixed_magnitude": "mixed_magnitude"}
_CASE_INDEX = {"primary": 0, "zeros": 1, "near_zero": 2, "alternating": 3, "mixed_magnitude": 4}


def materialize_reference_case(case_id: str, rows: int, width: int, base_seed: int,
                               residual: bool = False) -> dict[str, torch.Tensor]:
    """Inputs of one reference RMSNorm case: ``random.Random(seed + 10000*abi_position)`` per
    tensor, values rounded to bf16 after generation; ``base_seed`` is the task seed
    (2501 for h4096, 2671 for h7168; workload.py:94-106) and the case seed adds the case
    index (workload.py:113-119)."""
    mode = _MODES[case_id]
    seed = base_seed + _CASE_INDEX[case_id]
    names = ["x"] + (["residual"] if residual else []) + ["weight"]
    result = {}
    for position, name in enumerate(names):
        rng = random.Random(seed + position * 10000)
        count = width if name == "weight" else rows * width
        values = np.empty(count, dtype=np.float64)
        for index in range(count):
            if name == "weight":
                value = 0.0 if (index + 1) % 17 == 0 else rng.uniform(-1.5, 1.5)
            elif mode == "zeros":
                value = -0.0 if index % 2 else 0.0
            elif mode == "near_zero":
                value = rng.uniform(-1e-4, 1e-4)
            elif mode == "alternating":
                value = (1 if index % 2 else -1) * (1 + (index % 17) / 16)
            elif mode == "mixed_magnitude":
                value = (1 if index % 2 else -1) * 2.0 ** rng.randint(-12, 8)
            else:
                value = rng.uniform(-2, 2)
            values[index] = value
        tensor = _to_bf16_via_fp32(values)
        result[name] = tensor if name == "weight" else tensor.reshape(rows, width)
    return result
