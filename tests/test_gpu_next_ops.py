"""GPU parity of the operators either side of the hot path through the C ABI: the two-output add +
RMSNorm (src/open_cake_ir/tasks/add_rmsnorm.py) and the DeepSeek-V4 MoE gate and CSA indexer top-k
(src/open_cake_ir/tasks/deepseek_v4/workload.py), against the reference's golden outputs on its own
cases and against the oracle at larger sizes.  Tolerances are the contracts': add + RMSNorm ``out``
atol 2**-16 rtol 1/64, ``residual_out`` bit for bit (add_rmsnorm.py:84-86); gate weights atol 2e-6 rtol
2e-5, every index bit for bit (deepseek_v4/workload.py:103-104)."""
import json
from pathlib import Path

import numpy as np
import pytest
import torch

import open_cake_ir_b200 as cake
from gpu_util import poison, snapshot, unchanged
from oracle import add_rmsnorm, compare, deepseek_v4

pytestmark = pytest.mark.gpu
BASE = Path(__file__).resolve().parent / "golden"
INDEX = json.loads((BASE / "next_index.json").read_text())
ARRAYS = np.load(BASE / "next_outputs.npz")


def run_add_rmsnorm(cpu, eps):
    dev = {k: v.cuda() for k, v in cpu.items()}
    before = snapshot(dev)
    shape = tuple(cpu["delta"].shape)
    out, g1 = poison(shape, torch.bfloat16)
    res, g2 = poison(shape, torch.bfloat16)
    cake.AddRmsNorm(dev["delta"], dev["residual"], dev["weight"], out, res, eps).launch()
    torch.cuda.synchronize()
    g1(); g2()
    assert unchanged(before, dev)
    return out, res


@pytest.mark.parametrize("case", list(add_rmsnorm.CASES))
def test_add_rmsnorm_reference_cases(case):
    meta = INDEX[f"add_rmsnorm/{case}"]
    cpu = add_rmsnorm.materialize_reference_case(case, meta["rows"], meta["width"])
    out, res = run_add_rmsnorm(cpu, meta["epsilon"])
    want_out = torch.from_numpy(ARRAYS[f"add_rmsnorm/{case}/out"].copy()).view(torch.bfloat16)
    want_res = torch.from_numpy(ARRAYS[f"add_rmsnorm/{case}/residual_out"].copy()).view(torch.bfloat16)
    assert torch.equal(res.cpu().view(torch.int16), want_res.view(torch.int16)), "residual_out must be byte-equal"
    ok, bad, err = compare.compare(out, want_out, atol=2.0 ** -16, rtol=1 / 64)
    assert ok, f"{bad} mismatches, max abs err {err}"


@pytest.mark.parametrize("rows,width", [(4096, 4096), (1, 8), (3, 2048 + 8), (7, 8192), (5, 16384), (0, 256)])
def test_add_rmsnorm_serving_and_edge_shapes(rows, width):
    g = torch.Generator().manual_seed(rows * 31 + width)
    cpu = {"delta": torch.randn((rows, width), generator=g).to(torch.bfloat16),
           "residual": torch.randn((rows, width), generator=g).to(torch.bfloat16),
           "weight": (1 + 0.1 * torch.randn(width, generator=g)).to(torch.bfloat16)}
    out, res = run_add_rmsnorm(cpu, 1e-6)
    if rows == 0:
        return
    sample = slice(0, rows, max(1, rows // 64))          # the fsum oracle is a Python loop per row
    want = add_rmsnorm.add_rmsnorm_reference(cpu["delta"][sample], cpu["residual"][sample], cpu["weight"], 1e-6)
    assert torch.equal(res.cpu()[sample].view(torch.int16), want["residual_out"].view(torch.int16))
    whole = (cpu["delta"].float() + cpu["residual"].float()).to(torch.bfloat16)      # every row of residual_out
    assert torch.equal(res.cpu().view(torch.int16), whole.view(torch.int16))
    ok, bad, err = compare.compare(out[sample], want["out"], atol=2.0 ** -16, rtol=1 / 64)
    assert ok, f"{bad} mismatches, max abs err {err}"


# ---- DeepSeek-V4 gate and indexer -----------------------------------------------------------
def accepted(task):
    return [c for c in deepseek_v4.CASES[task] if "refused" not in INDEX[f"deepseek_v4/{task}/{c}"]]


@pytest.mark.parametrize("case", accepted("moe_gate"))
def test_gate_reference_cases(case):
    cpu = deepseek_v4.materialize_reference_case("moe_gate", case)
    dev = {k: v.cuda() for k, v in cpu.items()}
    before = snapshot(dev)
    weights, g1 = poison((4, 6), torch.float32)
    ids, g2 = poison((4, 6), torch.int32)
    cake.V4MoeGate(dev["router_logits"], dev["selection_bias"], weights, ids).launch()
    torch.cuda.synchronize()
    g1(); g2()
    assert unchanged(before, dev)
    key = f"deepseek_v4/moe_gate/{case}"
    assert ids.cpu().reshape(-1).tolist() == ARRAYS[key + "/expert_ids"].tolist()
    want = torch.from_numpy(ARRAYS[key + "/weights"].copy()).view(torch.float32).reshape(4, 6)
    ok, bad, err = compare.compare(weights, want, atol=2e-6, rtol=2e-5)
    assert ok, f"{bad} mismatches, max abs err {err}"


@pytest.mark.parametrize("tokens,experts,top_k", [(4096, 384, 6), (37, 256, 8), (5, 40, 3), (0, 384, 6)])
def test_gate_serving_shapes(tokens, experts, top_k):
    g = torch.Generator().manual_seed(experts + tokens)
    logits = torch.randn((tokens, experts), generator=g) * 2
    bias = torch.rand(experts, generator=g) * 0.5
    weights, ids = cake.v4_moe_gate(logits.cuda(), bias.cuda(), top_k=top_k)
    torch.cuda.synchronize()
    if tokens == 0:
        return
    sample = torch.arange(0, tokens, max(1, tokens // 256))
    want = deepseek_v4.moe_gate_reference(logits[sample], bias, top_k=top_k)
    assert ids.cpu()[sample].tolist() == want["expert_ids"].tolist()
    ok, bad, err = compare.compare(weights[sample.cuda()], want["weights"], atol=2e-6, rtol=2e-5)
    assert ok, f"{bad} mismatches, max abs err {err}"


def test_gate_ties_go_to_the_lower_expert():
    logits = torch.zeros((2, 384)); bias = torch.zeros(384)
    logits[1, 100] = 1.0
    weights, ids = cake.v4_moe_gate(logits.cuda(), bias.cuda())
    assert ids.cpu().tolist() == [[0, 1, 2, 3, 4, 5], [100, 0, 1, 2, 3, 4]]
    torch.testing.assert_close(weights.cpu()[0], torch.full((6,), 2.5 / 6))


@pytest.mark.parametrize("case", accepted("csa_indexer_topk"))
def test_indexer_reference_cases(case):
    cpu = deepseek_v4.materialize_reference_case("csa_indexer_topk", case)
    scores = cpu["index_scores"].cuda()
    before = snapshot({"s": scores})
    indices, guard = poison((4, 1024), torch.int32)
    cake.CsaTopk(scores, indices).launch()
    torch.cuda.synchronize()
    guard()
    assert unchanged(before, {"s": scores})
    assert indices.cpu().reshape(-1).tolist() == ARRAYS[f"deepseek_v4/csa_indexer_topk/{case}/indices"].tolist()


@pytest.mark.parametrize("rows,candidates,top_k", [(512, 2048, 1024), (3, 2048, 2048), (5, 1000, 17), (2, 1, 1)])
def test_indexer_shapes(rows, candidates, top_k):
    g = torch.Generator().manual_seed(candidates)
    scores = torch.randn((rows, candidates), generator=g)
    got = cake.csa_topk(scores.cuda(), top_k).cpu()
    want = torch.argsort(scores, dim=1, descending=True, stable=True)[:, :top_k].int()
    assert torch.equal(got, want)


def test_indexer_ties_and_signed_zeros_order_by_position():
    scores = torch.zeros((1, 2048)); scores[0, ::2] = -0.0; scores[0, 7] = 1.0; scores[0, 9] = float("-inf")
    got = cake.csa_topk(scores.cuda(), 2048).cpu()[0].tolist()
    assert got[0] == 7 and got[-1] == 9 and got[1:-1] == [i for i in range(2048) if i not in (7, 9)]
