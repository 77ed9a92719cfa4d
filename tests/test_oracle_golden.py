"""CPU tests: the oracle restatements against outputs of the reference's own oracles
(tests/golden) and against the known-answer vectors held in the reference's contract tests."""
import math

import pytest
import torch

from conftest import moe_reference_case, sha256
from oracle import attention, block_scaled_gemm, compare, moe, permute, rmsnorm, routing

RMS = {"solx-fib-rmsnorm-h4096-bf16-triton-b300-r170-v1": (170, 4096, 2501, False),
       "solx-fib-rmsnorm-h7168-bf16-triton-b300-r64-v1": (64, 7168, 2671, False),
       "solx-fib-fused-add-rmsnorm-h4096-bf16-triton-b300-r170-v1": (170, 4096, None, True)}


@pytest.mark.parametrize("stem", list(RMS))
@pytest.mark.parametrize("case", ["primary", "zeros", "near_zero", "alternating", "mixed_magnitude"])
def test_rmsnorm_oracle_is_bit_identical_to_reference(golden, stem, case):
    rows, width, base_seed, fused = RMS[stem]
    meta = golden.index[f"rmsnorm/{stem}/{case}"]
    assert (meta["rows"], meta["width"]) == (rows, width)
    case_index = ["primary", "zeros", "near_zero", "alternating", "mixed_magnitude"].index(case)
    inputs = rmsnorm.materialize_reference_case(case, rows, width, meta["seed"] - case_index, residual=fused)
    for name, digest in meta["inputs_sha256"].items():
        assert sha256(inputs[name]) == digest, f"materialiser differs on {name}"
    out = rmsnorm.rmsnorm_reference(inputs["x"], inputs["weight"], meta["epsilon"], inputs.get("residual"))
    assert sha256(out) == meta["out_sha256"]
    assert torch.equal(out[:4].view(torch.int16), golden.bf16(f"rmsnorm/{stem}/{case}/out_head").view(torch.int16).reshape(4, width))
    if case == "zeros":      # reference test_solx_fib_workloads.py:191-196: zeros stay zero
        assert not bool(out.float().abs().any())


def test_rmsnorm_fast_baseline_matches_oracle_within_contract_tolerance():
    inputs = rmsnorm.materialize_reference_case("primary", 64, 7168, 2671)
    a = rmsnorm.rmsnorm_reference(inputs["x"], inputs["weight"], 1e-6)
    b = rmsnorm.rmsnorm_fast(inputs["x"], inputs["weight"], 1e-6)
    ok, bad, _ = compare.compare(b, a, atol=2.0 ** -16, rtol=2.0 ** -7)
    assert ok, bad


DECODE = [(t, v, c) for t in ("gqa_kv4", "gqa_kv8", "mla_h16") for v in ("captured", "boundary") for c in attention.CASES]


@pytest.mark.parametrize("task,variant,case", DECODE)
def test_decode_oracle_is_bit_identical_to_reference(golden, task, variant, case):
    key = f"decode/{task}/{variant}/{case}"
    inputs = attention.materialize_reference_case(task, variant, case)
    for name, digest in golden.index[key]["inputs_sha256"].items():
        assert sha256(inputs[name]) == digest, f"materialiser differs on {name}"
    result = attention.paged_decode_reference(inputs, mla=task.startswith("mla"), page_size=1)
    assert torch.equal(result["output"].view(torch.int16), golden.bf16(key + "/output").view(torch.int16).reshape(result["output"].shape))
    want = golden.fp32(key + "/lse").reshape(result["lse"].shape)
    assert torch.equal(result["lse"].view(torch.int32), want.view(torch.int32))
    if variant == "boundary" and case == "segmented":     # test_solx_fib_launch_plans.py:78-91
        assert not bool(result["output"][:1].float().abs().any()) and bool(torch.isneginf(result["lse"][:1]).all())
    # the all-heads-at-once evaluation used at serving sizes agrees within the contract tolerance
    fast = attention.paged_decode_reference(inputs, mla=task.startswith("mla"), page_size=1, per_head_loop=False)
    assert compare.compare(fast["output"], result["output"], atol=2.0 ** -16, rtol=2.0 ** -7)[0]
    assert compare.compare(fast["lse"], result["lse"], atol=1e-4, rtol=1e-5, ieee=True)[0]


def test_zero_query_known_answer():
    """test_solx_fib_launch_plans.py:93-102: zero query => output = mean of the V rows, lse = log2(L)."""
    inputs = attention.materialize_reference_case("gqa_kv4", "boundary", "zeros")
    result = attention.paged_decode_reference(inputs, mla=False, page_size=1)
    for b in range(2):
        lo, hi = inputs["kv_indptr"][b:b + 2].tolist()
        ids = inputs["kv_indices"][lo:hi].long()
        expected = inputs["v_cache"][ids, 0].double().mean(0).repeat_interleave(8, 0).to(torch.bfloat16)
        torch.testing.assert_close(result["output"][b], expected, rtol=0, atol=0)
        torch.testing.assert_close(result["lse"][b], torch.full((32,), math.log2(hi - lo)), rtol=1e-6, atol=1e-6)


def test_paged_addressing_reduces_to_page_size_one():
    """page_size > 1 (not held by the reference): regrouping the same tokens into pages of 4 with a
    ragged last page must not change any result bit."""
    g = torch.Generator().manual_seed(7)
    lens = [0, 1, 4, 9, 13]
    batch, hq, hkv, d, page = len(lens), 8, 2, 128, 4
    total = sum(lens)
    tokens_k = (torch.rand((total, hkv, d), generator=g) - 0.5).to(torch.bfloat16)
    tokens_v = (torch.rand((total, hkv, d), generator=g) - 0.5).to(torch.bfloat16)
    q = (torch.rand((batch, hq, d), generator=g) - 0.5).to(torch.bfloat16)
    scale = torch.tensor([0.09], dtype=torch.float32)
    flat_ptr = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32)
    perm = torch.randperm(total, generator=g)
    k1 = torch.zeros((total, 1, hkv, d), dtype=torch.bfloat16); v1 = torch.zeros_like(k1)
    k1[perm, 0] = tokens_k; v1[perm, 0] = tokens_v
    one = attention.paged_decode_reference({"q": q, "k_cache": k1, "v_cache": v1, "kv_indptr": flat_ptr,
                                            "kv_indices": perm.int(), "sm_scale": scale}, mla=False, page_size=1)
    pages = [(n + page - 1) // page for n in lens]
    pool = sum(pages) + 3
    page_perm = torch.randperm(pool, generator=g)[:sum(pages)]
    kp = torch.zeros((pool, page, hkv, d), dtype=torch.bfloat16); vp = torch.zeros_like(kp)
    indptr = [0]; last = []; cursor = 0; tok = 0
    for n, np_ in zip(lens, pages):
        for j in range(n):
            pg = page_perm[cursor + j // page]
            kp[pg, j % page] = tokens_k[tok + j]; vp[pg, j % page] = tokens_v[tok + j]
        tok += n; cursor += np_; indptr.append(cursor)
        last.append(0 if n == 0 else n - (np_ - 1) * page)
    paged = attention.paged_decode_reference(
        {"q": q, "k_cache": kp, "v_cache": vp, "kv_indptr": torch.tensor(indptr, dtype=torch.int32),
         "kv_indices": page_perm.int(), "kv_last_page_len": torch.tensor(last, dtype=torch.int32), "sm_scale": scale},
        mla=False, page_size=page)
    assert torch.equal(one["output"].view(torch.int16), paged["output"].view(torch.int16))
    assert torch.equal(one["lse"].view(torch.int32), paged["lse"].view(torch.int32))
    assert bool(torch.isneginf(paged["lse"][0]).all())


def test_group_routing_known_answer():
    """test_solx_fib_launch_plans.py:104-111."""
    logits = torch.full((1, 256), -6.0)
    for group in [0, 2, 3, 4]:
        logits[0, group * 32:group * 32 + 2] = 3.0
    logits[0, 32] = 6.0
    selected, weights = routing.routing_ds(logits, torch.zeros(256, dtype=torch.bfloat16), 2.5)
    assert selected.tolist() == [[0, 1, 64, 65, 96, 97, 128, 129]]
    torch.testing.assert_close(weights, torch.full((1, 8), 2.5 / 8, dtype=torch.float32))


def test_top_k_prefix_tie_known_answer():
    """tools/kernel_oracles.py:77-95: ties and -inf in a fixed prefix resolve to the lowest index."""
    scores = torch.full((3, 256), -float("inf"))
    scores[:, :8] = torch.tensor([10.0, 10.0, 9.0, 9.0, 8.0, 8.0, -float("inf"), -float("inf")])
    ids, w = routing.routing_softmax_topk(scores, 8)
    assert ids.tolist() == [[0, 1, 2, 3, 4, 5, 6, 7]] * 3


def test_softmax_routing_known_answer():
    logits = torch.zeros((2, 256)); logits[0, 200] = 1.0; logits[1, 5] = -0.0
    ids, w = routing.routing_softmax_topk(logits, 8)
    assert ids[0].tolist() == [200, 0, 1, 2, 3, 4, 5, 6] and ids[1].tolist() == list(range(8))
    e = math.e
    torch.testing.assert_close(w[0], torch.tensor([e / (e + 7)] + [1 / (e + 7)] * 7))
    torch.testing.assert_close(w[1], torch.full((8,), 0.125))


@pytest.mark.parametrize("case", ["primary", "zero_hidden", "all_nonlocal", "mixed_local", "scaled", "ties"])
def test_moe_oracle_is_bit_identical_to_reference(golden, case):
    inputs = moe_reference_case(case)
    for name, digest in golden.index[f"moe/{case}"]["inputs_sha256"].items():
        assert sha256(inputs[name]) == digest, f"materialiser differs on {name}"
    result = moe.moe_reference(inputs, routing="ds", return_parts=True)
    assert result["expert_ids"].int().tolist() == golden.int32(f"moe/{case}/expert_ids").tolist()
    assert torch.equal(result["route_weights"].view(torch.int32), golden.fp32(f"moe/{case}/route_weights").view(torch.int32).reshape(1, 8))
    assert torch.equal(result["output"].view(torch.int16), golden.bf16(f"moe/{case}/output").view(torch.int16).reshape(1, 7168))
    if case == "ties":     # all scores equal: lowest indices win everywhere (moe.py:63)
        assert result["expert_ids"].tolist() == [[0, 1, 32, 33, 64, 65, 96, 97]] or result["expert_ids"].tolist()[0] == sorted(result["expert_ids"].tolist()[0])


def test_permute_reference_order_and_ownership():
    g = torch.Generator().manual_seed(3)
    ids = torch.stack([torch.randperm(64, generator=g)[:8] for _ in range(100)])
    out = permute.permute_reference(ids, 16, 32)
    assert permute.check_ownership(ids, 16, 32, **out) == []
    sp = out["sorted_pairs"].long()
    experts = ids.reshape(-1)[sp]
    assert bool((experts[1:] >= experts[:-1]).all())
    same = experts[1:] == experts[:-1]
    assert bool((sp[1:][same] > sp[:-1][same]).all())     # stable: ascending pair index inside an expert
    broken = dict(out); broken["counts"] = out["counts"].clone(); broken["counts"][0] += 1
    assert "counts" in permute.check_ownership(ids, 16, 32, **broken)


def test_block_scaled_gemm_oracle_matches_partial_dot_form():
    """The emitted reference kernel scales each 128-wide partial dot (corpus/expected/
    block-scaled-gemm-accepted.txt:74-76); dequantise-then-matmul must agree with it."""
    g = torch.Generator().manual_seed(5)
    a = ((torch.rand((16, 256), generator=g) - 0.5) * 4).to(torch.float8_e4m3fn)
    b = ((torch.rand((128, 256), generator=g) - 0.5) * 4).to(torch.float8_e4m3fn)
    sfa = 0.5 + torch.rand((2, 16), generator=g); sfb = 0.5 + torch.rand((1, 2), generator=g)
    want = torch.zeros((16, 128), dtype=torch.float64)
    for kb in range(2):
        part = a[:, kb * 128:(kb + 1) * 128].double() @ b[:, kb * 128:(kb + 1) * 128].double().T
        want += part * sfa[kb].double()[:, None] * sfb[0, kb].double()
    got = block_scaled_gemm.block_scaled_gemm_reference(a, sfa, b, sfb, out_dtype=None, dtype=torch.float64)
    torch.testing.assert_close(got, want, rtol=1e-12, atol=1e-12)


def test_comparator_truth_table():
    """test_solx_fib_launch_plans.py:59-73."""
    inf, nan = float("inf"), float("nan")
    for expected, actual, ok in [([-inf], [-inf], True), ([-inf], [0.0], False), ([-inf], [inf], False),
                                 ([nan], [nan], True), ([nan], [12345.0], False), ([0.0], [nan], False)]:
        assert compare.compare(torch.tensor(actual), torch.tensor(expected), atol=0.0, rtol=0.0, ieee=True)[0] == ok
    assert not compare.compare(torch.tensor([-inf]), torch.tensor([-inf]), atol=0.0, rtol=0.0)[0]
    assert compare.compare(torch.tensor([1.0, 2.0]), torch.tensor([1.0, 2.01]), atol=0.0, rtol=1e-2)[0]
    assert not compare.compare(torch.tensor([1.0, 2.0]), torch.tensor([1.0, 2.03]), atol=0.0, rtol=1e-2)[0]


def test_activation_quantiser_round_trip():
    g = torch.Generator().manual_seed(11)
    act = torch.randn((5, 256), generator=g) * 3
    act[2] = 0
    q, s = moe.quantize_rows_e4m3(act)
    assert s.shape == (2, 5) and float(s[0, 2]) == 1.0
    back = moe.dequantize_rows(q, s, torch.float32)
    assert float((back - act).abs().max()) <= float(act.abs().max()) / 16 + 1e-6
    assert float(back.abs().max()) <= float(act.abs().max()) * (1 + 1e-6)
