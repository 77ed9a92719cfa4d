"""GPU parity: MoE routing, permute and the whole FP8 expert layer through the C ABI.

Routing indices and the permutation are compared bit for bit (ties to the lower expert id).
The layer output is compared (a) with the reference's own six cases at the contract tolerance
atol = rtol = 1e-2 on every element (src/open_cake_ir/tasks/solx_fib/moe.py:72-73) in the
two-term activation mode, and (b) in the single-term FP8 activation mode with the oracle that
has the identical quantiser inserted, at 1e-2 relative Frobenius error and bf16 rtol/atol 2e-2."""
import pytest
import torch

import open_cake_ir_b200 as cake
from conftest import moe_reference_case
from gpu_util import snapshot, unchanged
from oracle import compare, moe as oracle_moe, permute as oracle_permute, routing as oracle_routing

pytestmark = pytest.mark.gpu


def near_tie_tokens(logits, bias, mode):
    """Tokens whose selection hangs on two scores closer than a few fp32 ulps: a device exp() one
    ulp off the host's may legitimately pick the other expert there."""
    return oracle_routing.score_gap(logits, bias, mode=mode) < 4e-7


@pytest.mark.parametrize("mode", ["ds", "softmax"])
@pytest.mark.parametrize("tokens,experts", [(4096, 256), (1, 256), (37, 64), (5, 512)])
def test_routing_bit_exact(mode, tokens, experts):
    g = torch.Generator().manual_seed(100 + tokens)
    logits = torch.randn((tokens, experts), generator=g)
    bias = (torch.rand(experts, generator=g) * 0.015).to(torch.bfloat16) if mode == "ds" else torch.zeros(experts, dtype=torch.bfloat16)
    factor = torch.tensor([2.5])
    if mode == "ds":
        want_ids, want_w = oracle_routing.routing_ds(logits, bias, 2.5)
    else:
        want_ids, want_w = oracle_routing.routing_softmax_topk(logits); want_w = want_w * 2.5
    ids, w = cake.moe_routing(logits.cuda(), bias.cuda(), factor.cuda(), mode=mode)
    ids, w = ids.cpu(), w.cpu()
    differs = (ids.long() != want_ids).any(1)
    excused = near_tie_tokens(logits, bias, mode) if mode == "ds" else torch.zeros(tokens, dtype=torch.bool)
    assert not bool((differs & ~excused).any()), f"{int((differs & ~excused).sum())} tokens differ without a near tie"
    assert int(differs.sum()) <= max(1, tokens // 500), "too many near-tie tokens to be rounding"
    same = ~differs
    torch.testing.assert_close(w[same], want_w[same], rtol=2e-6, atol=1e-7)


def test_routing_known_answers():
    logits = torch.full((1, 256), -6.0)
    for group in [0, 2, 3, 4]:
        logits[0, group * 32:group * 32 + 2] = 3.0
    logits[0, 32] = 6.0
    zeros = torch.zeros(256, dtype=torch.bfloat16)
    ids, w = cake.moe_routing(logits.cuda(), zeros.cuda(), torch.tensor([2.5]).cuda(), mode="ds")
    assert ids.cpu().tolist() == [[0, 1, 64, 65, 96, 97, 128, 129]]          # test_solx_fib_launch_plans.py:104-111
    torch.testing.assert_close(w.cpu(), torch.full((1, 8), 2.5 / 8))
    scores = torch.full((2, 256), -float("inf"))
    scores[:, :8] = torch.tensor([10.0, 10.0, 9.0, 9.0, 8.0, 8.0, -float("inf"), -float("inf")])
    ids, _ = cake.moe_routing(scores.cuda(), zeros.cuda(), torch.tensor([1.0]).cuda(), mode="softmax")
    assert ids.cpu().tolist() == [[0, 1, 2, 3, 4, 5, 6, 7]] * 2                # tools/kernel_oracles.py:77-95
    ties = torch.zeros((1, 256)); ties[0, 7] = -0.0
    ids, w = cake.moe_routing(ties.cuda(), zeros.cuda(), torch.tensor([2.5]).cuda(), mode="ds")
    want, _ = oracle_routing.routing_ds(ties, zeros, 2.5)
    assert ids.cpu().tolist() == want.tolist()


@pytest.mark.parametrize("tokens,experts,offset,local", [(4096, 256, 0, 256), (4096, 256, 96, 32), (1, 256, 224, 32),
                                                          (50, 64, 0, 1), (300, 64, 60, 4)])
def test_permute_bit_exact(tokens, experts, offset, local):
    g = torch.Generator().manual_seed(tokens + experts)
    ids = torch.stack([torch.randperm(experts, generator=g)[:8] for _ in range(tokens)]).int()
    want = oracle_permute.permute_reference(ids, offset, local)
    got = cake.moe_permute(ids.cuda(), torch.tensor([offset], dtype=torch.int32).cuda(), local)
    got = {k: v.cpu() for k, v in got.items()}
    n = int(want["offsets"][-1])
    assert torch.equal(got["counts"], want["counts"]) and torch.equal(got["offsets"], want["offsets"])
    assert torch.equal(got["sorted_pairs"][:n], want["sorted_pairs"])
    assert torch.equal(got["inv_perm"], want["inv_perm"])
    assert oracle_permute.check_ownership(ids, offset, local, got["counts"], got["offsets"], got["sorted_pairs"], got["inv_perm"]) == []


def run_layer(cpu, **options):
    dev = {k: v.cuda() for k, v in cpu.items()}
    before = snapshot(dev)
    tokens, hidden = cpu["hidden_states"].shape
    out = torch.full((tokens, hidden), float("nan"), dtype=torch.bfloat16, device="cuda")
    op = cake.Fp8Moe(dev, out, **options)
    op.launch()
    assert op.status() == 0
    assert unchanged(before, dev)
    return out, op


@pytest.mark.parametrize("case", list(oracle_moe.CASES))
def test_reference_cases_at_contract_tolerance(golden, case):
    cpu = moe_reference_case(case)
    out, op = run_layer(cpu, routing="ds", act_mode="split")
    assert op.intermediate("expert_ids").cpu().tolist() == golden.int32(f"moe/{case}/expert_ids").reshape(-1).tolist()
    want = golden.bf16(f"moe/{case}/output").reshape(1, 7168)
    ok, bad, err = compare.compare(out, want, atol=1e-2, rtol=1e-2)
    assert ok, f"{bad} mismatches, max abs err {err}"
    if case in ("zero_hidden", "all_nonlocal", "ties"):
        assert not bool(out.float().abs().any())


SMALL = dict(tokens=96, hidden=512, inter=256, experts=32, local_experts=32, local_offset=0)


@pytest.mark.parametrize("routing", ["softmax", "ds"])
@pytest.mark.parametrize("shape", [SMALL, dict(SMALL, tokens=1), dict(SMALL, tokens=700, experts=16, local_experts=4, local_offset=8),
                                   dict(tokens=256, hidden=7168, inter=2048, experts=256, local_experts=8, local_offset=40)])
def test_layer_fp8_activation_mode(routing, shape):
    cpu = cake.workloads.moe_inputs(**shape, routing=routing, device="cpu")
    n_group = 8 if shape["experts"] % 8 == 0 and shape["experts"] >= 32 else 1
    out, op = run_layer(cpu, experts=shape["experts"], routing=routing, act_mode="fp8", n_group=n_group,
                        topk_group=max(1, n_group // 2))
    if routing == "ds" and n_group != 8:
        pytest.skip("oracle routing is the 8-group definition")
    want = oracle_moe.moe_reference(cpu, routing=routing, act_quant="fp8", dtype=torch.float32, return_parts=True)
    ids = op.intermediate("expert_ids").cpu().reshape(shape["tokens"], 8)
    same = (ids.long() == want["expert_ids"]).all(1)
    assert int((~same).sum()) <= 1
    assert compare.rel_frobenius(out[same.cuda()], want["output"][same]) <= 1e-2
    ok, bad, err = compare.compare(out[same.cuda()], want["output"][same], atol=2e-2, rtol=2e-2)
    assert ok, f"{bad} mismatches, max abs err {err}"


def test_layer_split_mode_against_unquantised_oracle():
    cpu = cake.workloads.moe_inputs(**SMALL, routing="softmax", device="cpu")
    out, _ = run_layer(cpu, experts=32, routing="softmax", act_mode="split")
    want = oracle_moe.moe_reference(cpu, routing="softmax", act_quant="none")
    assert compare.rel_frobenius(out, want["output"]) <= 4e-3
    one, _ = run_layer(cpu, experts=32, routing="softmax", act_mode="fp8")
    assert compare.rel_frobenius(one, want["output"]) <= 6e-2      # the quantisation error of the single-term mode, reported


def test_layer_serving_size_token_subset():
    """Full DeepSeek-V3 layer size (4096 tokens, 256 local experts) on the device; the oracle follows a
    subset of tokens through every expert they use."""
    shape = dict(tokens=4096, hidden=7168, inter=2048, experts=256, local_experts=256, local_offset=0)
    dev = cake.workloads.moe_inputs(**shape, routing="softmax", device="cuda", gen_device="cuda")
    out = torch.empty((4096, 7168), dtype=torch.bfloat16, device="cuda")
    op = cake.Fp8Moe(dev, out, routing="softmax", act_mode="fp8")
    op.launch()
    assert op.status() == 0
    counts = op.intermediate("counts").cpu()
    assert int(counts.sum()) == 4096 * 8 and torch.equal(op.intermediate("offsets").cpu()[1:], counts.cumsum(0).int())
    pick = torch.arange(0, 4096, 512)
    sub = {k: v.cpu() for k, v in dev.items() if not k.startswith("gemm")}
    sub["routing_logits"] = sub["routing_logits"][pick].contiguous()
    sub["hidden_states"] = sub["hidden_states"][pick].contiguous()
    sub["hidden_states_scale"] = sub["hidden_states_scale"][:, pick].contiguous()
    ids, _ = oracle_routing.routing_softmax_topk(sub["routing_logits"])
    used = sorted(set(ids.reshape(-1).tolist()))
    remap = {e: i for i, e in enumerate(used)}
    for name in ("gemm1_weights", "gemm1_weights_scale", "gemm2_weights", "gemm2_weights_scale"):
        sub[name] = dev[name][used].cpu()
    # route among the used experts only: rewrite logits so the same experts win in the compacted numbering
    logits = torch.full((pick.numel(), len(used)), -1e30)
    for t in range(pick.numel()):
        for e in ids[t].tolist():
            logits[t, remap[e]] = sub["routing_logits"][t, e]
    sub["routing_logits"] = logits
    sub["routing_bias"] = torch.zeros(len(used), dtype=torch.bfloat16)
    want = oracle_moe.moe_reference(sub, routing="softmax", act_quant="fp8", dtype=torch.float32)
    assert compare.rel_frobenius(out[pick.cuda()], want["output"]) <= 1e-2
