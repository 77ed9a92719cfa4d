"""B200 (sm_100a) native target for open-cake-ir's inference workload contracts.

The product is ``libcake_b200.so`` -- hand-written CUDA behind a C ABI (``include/cake_b200.h``).
This package is the Python host side a user of the reference calls instead of the reference's
emitted Triton launch plans: the same operators, tensor names, layouts, dtypes and scale
conventions (``operators``), thin ctypes bindings (``_lib``), the operator objects that own a
native handle (``ops``) and seeded synthetic inputs at serving shapes (``workloads``).
There is no CPU fallback: every operator raises if the native library is missing.
"""
from . import _lib, operators, ops, workloads  # noqa: F401
from .ops import (AddRmsNorm, BlockScaledGemm, CsaTopk, GqaCausalPrefill, MlaCausalPrefill, Fp8Moe, GqaPagedDecode, MlaPagedDecode, MoePermute, MoeRouting, RmsNorm, SparseMlaDecode, V4MoeGate,
                  add_rmsnorm, block_scaled_gemm, csa_topk, gqa_causal_prefill, mla_causal_prefill, fp8_moe, gqa_paged_decode, mla_paged_decode, moe_permute, moe_routing, rmsnorm, sparse_mla_decode, v4_moe_gate)

__all__ = ["AddRmsNorm", "BlockScaledGemm", "CsaTopk", "GqaCausalPrefill", "MlaCausalPrefill", "gqa_causal_prefill", "mla_causal_prefill", "SparseMlaDecode", "V4MoeGate", "sparse_mla_decode", "csa_topk", "v4_moe_gate", "Fp8Moe", "GqaPagedDecode", "MlaPagedDecode", "MoePermute", "MoeRouting", "RmsNorm",
           "add_rmsnorm", "block_scaled_gemm", "fp8_moe", "gqa_paged_decode", "mla_paged_decode", "moe_permute", "moe_routing",
           "rmsnorm", "operators", "ops", "workloads"]
