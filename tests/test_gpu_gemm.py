"""GPU parity: block-scaled FP8 GEMM (tcgen05) through the C ABI against the oracle
(tools/kernel_oracles.py:98-112 semantics).  Tolerances: bf16 output within rtol 2e-2 / atol 2e-2
element-wise and relative Frobenius error <= 1e-2 of the dequantised fp32 reference."""
import pytest
import torch

import open_cake_ir_b200 as cake
from gpu_util import poison, snapshot, unchanged
from oracle import block_scaled_gemm as oracle_gemm, compare

pytestmark = pytest.mark.gpu


def run(m, n, k, salt=0):
    cpu = cake.workloads.block_scaled_gemm_inputs(m, n, k, device="cpu", salt=salt)
    want = oracle_gemm.block_scaled_gemm_reference(cpu["a"], cpu["sfa"], cpu["b"], cpu["sfb"], out_dtype=None)
    dev = {key: v.cuda() for key, v in cpu.items()}
    before = snapshot(dev)
    c, guard = poison((m, n), torch.bfloat16)
    op = cake.BlockScaledGemm(dev["a"], dev["sfa"], dev["b"], dev["sfb"], c)
    op.launch()
    assert op.status() == 0
    guard()
    assert unchanged(before, dev)
    return c, want


@pytest.mark.parametrize("m,n,k", [(16, 128, 256), (128, 256, 128), (200, 384, 512), (1, 256, 1024), (517, 1024, 896)])
def test_small_shapes(m, n, k):
    c, want = run(m, n, k)
    ok, bad, err = compare.compare(c, want, atol=2e-2, rtol=2e-2)
    assert ok, f"{bad} mismatches, max abs err {err}"
    assert compare.rel_frobenius(c, want) <= 1e-2


def test_reference_smoke_shape_with_reference_value_ranges():
    """The reference's smoke schedule: a[16,256], b[128,256], sfa[2,16], sfb[1,2] (block-scaled-gemm-b1-smoke.json)."""
    g = torch.Generator().manual_seed(20260825)
    a = ((torch.rand((16, 256), generator=g) - 0.5) * 4).to(torch.float8_e4m3fn)
    b = ((torch.rand((128, 256), generator=g) - 0.5) * 4).to(torch.float8_e4m3fn)
    sfa = 0.5 + torch.rand((2, 16), generator=g); sfb = 0.5 + torch.rand((1, 2), generator=g)
    want = oracle_gemm.block_scaled_gemm_reference(a, sfa, b, sfb, out_dtype=None)
    c = cake.block_scaled_gemm(a.cuda(), sfa.cuda(), b.cuda(), sfb.cuda())
    ok, bad, err = compare.compare(c, want, atol=2e-2, rtol=2e-2)
    assert ok, f"{bad} mismatches, max abs err {err}"


def test_serving_shape():
    c, want = run(8192, 4096, 7168)
    assert compare.rel_frobenius(c, want) <= 1e-2
    ok, bad, err = compare.compare(c, want, atol=2e-2, rtol=2e-2)
    assert ok, f"{bad} mismatches, max abs err {err}"


def test_linearity_in_scales():
    """Size-independent property: doubling every A scale doubles C exactly (powers of two commute with rounding)."""
    cpu = cake.workloads.block_scaled_gemm_inputs(256, 512, 768, device="cpu", salt=3)
    dev = {key: v.cuda() for key, v in cpu.items()}
    c1 = cake.block_scaled_gemm(dev["a"], dev["sfa"], dev["b"], dev["sfb"])
    c2 = cake.block_scaled_gemm(dev["a"], dev["sfa"] * 2, dev["b"], dev["sfb"])
    assert torch.equal((c1.float() * 2).to(torch.bfloat16), c2)
