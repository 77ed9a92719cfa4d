"""Block-scaled FP8 GEMM oracle (test infrastructure; see the package docstring).

Follows tools/kernel_oracles.py:98-112 (``_block_scaled_gemm_oracle``): dequantise both
operands with their block scales, contract in fp32.  Scale layouts are the contract's
(docs/adr/0023-block-scales-are-axis-relations.md:21-27): ``sfa[k//128, m]`` for the
activation operand, ``sfb[n//128, k//128]`` for the weight operand, B stored ``[N, K]``.
The reference oracle holds a single 128-row weight group; more groups are the same relation
repeated along N.  The bf16 rounding of the output is this build's contract (the smoke
schedule keeps fp32).
"""
from __future__ import annotations

import torch


def dequant_a(a: torch.Tensor, sfa: torch.Tensor, dtype=torch.float32) -> torch.Tensor:
    k = a.shape[1]
    return a.to(dtype) * sfa.t().to(dtype).repeat_interleave(128, dim=1)[:, :k]


def dequant_b(b: torch.Tensor, sfb: torch.Tensor, dtype=torch.float32) -> torch.Tensor:
    n, k = b.shape
    return b.to(dtype) * sfb.to(dtype).repeat_interleave(128, dim=0)[:n].repeat_interleave(128, dim=1)[:, :k]


def block_scaled_gemm_reference(a, sfa, b, sfb, *, out_dtype=torch.bfloat16, dtype=torch.float32):
    """a e4m3 [M,K], sfa fp32 [K/128,M], b e4m3 [N,K], sfb fp32 [N/128,K/128] -> [M,N]."""
    c = dequant_a(a, sfa, dtype) @ dequant_b(b, sfb, dtype).t()
    return c if out_dtype is None else c.to(out_dtype)
