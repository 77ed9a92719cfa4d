"""GPU parity: RMSNorm through the C ABI against the oracle, on the reference's cases and at the
serving shape.  Tolerance is the contract's: atol 2**-16, rtol 2**-7, every element
(src/open_cake_ir/tasks/solx_fib/workload.py:128-129, :271-273)."""
import pytest
import torch

import open_cake_ir_b200 as cake
from gpu_util import poison, snapshot, unchanged
from oracle import compare, rmsnorm

pytestmark = pytest.mark.gpu
ATOL, RTOL = 2.0 ** -16, 2.0 ** -7
CASES = ["primary", "zeros", "near_zero", "alternating", "mixed_magnitude"]


@pytest.mark.parametrize("rows,width,seed,eps,fused", [(170, 4096, 2501, 1e-5, False), (64, 7168, 2671, 1e-6, False),
                                                       (170, 4096, 2471, 1e-5, True)])
@pytest.mark.parametrize("case", CASES)
def test_reference_cases(golden, rows, width, seed, eps, fused, case):
    if fused:
        meta = golden.index[f"rmsnorm/solx-fib-fused-add-rmsnorm-h4096-bf16-triton-b300-r170-v1/{case}"]
        seed, eps = meta["seed"] - CASES.index(case), meta["epsilon"]
    cpu = rmsnorm.materialize_reference_case(case, rows, width, seed, residual=fused)
    want = rmsnorm.rmsnorm_reference(cpu["x"], cpu["weight"], eps, cpu.get("residual"))
    dev = {k: v.cuda() for k, v in cpu.items()}
    before = snapshot(dev)
    out, guard = poison((rows, width), torch.bfloat16)
    cake.RmsNorm(dev["x"], dev["weight"], out, eps, dev.get("residual")).launch()
    torch.cuda.synchronize()
    guard()
    assert unchanged(before, dev)
    ok, bad, err = compare.compare(out, want, atol=ATOL, rtol=RTOL)
    assert ok, f"{bad} mismatches, max abs err {err}"


@pytest.mark.parametrize("rows,width", [(4096, 4096), (1, 8), (3, 2048 + 8), (5, 16384), (0, 4096)])
def test_serving_and_edge_shapes(rows, width):
    inputs, meta = cake.workloads.rmsnorm_inputs(rows, width, device="cpu")
    want = rmsnorm.rmsnorm_reference(inputs["x"], inputs["weight"], meta["epsilon"]) if rows else inputs["x"]
    out, guard = poison((rows, width), torch.bfloat16)
    cake.RmsNorm(inputs["x"].cuda(), inputs["weight"].cuda(), out, meta["epsilon"]).launch()
    torch.cuda.synchronize()
    guard()
    ok, bad, err = compare.compare(out, want, atol=ATOL, rtol=RTOL)
    assert ok, f"{bad} mismatches, max abs err {err}"


def test_rejects_bad_arguments():
    x = torch.zeros((4, 12), dtype=torch.bfloat16, device="cuda")   # width not a multiple of 8
    with pytest.raises(cake._lib.CakeError):
        cake.RmsNorm(x, torch.zeros(12, dtype=torch.bfloat16, device="cuda"), torch.empty_like(x), 1e-6)
    with pytest.raises(ValueError):
        cake.RmsNorm(x.cpu(), torch.zeros(12, dtype=torch.bfloat16), torch.empty_like(x.cpu()), 1e-6)
