"""The restated oracles of the operators either side of the hot path (two-output add + RMSNorm, the
DeepSeek-V4 MoE gate and CSA indexer top-k, causal prefill attention) against outputs of the reference's own oracles
(tests/golden/make_golden_next.py): regenerated inputs hash-equal, outputs bit-identical, and the
cases the reference's oracle refuses are refused here too."""
import json
from pathlib import Path

import numpy as np
import pytest
import torch

from conftest import sha256
from oracle import add_rmsnorm, attention, deepseek_v4

BASE = Path(__file__).resolve().parent / "golden"
INDEX = json.loads((BASE / "next_index.json").read_text())
ARRAYS = np.load(BASE / "next_outputs.npz")


def bf16(key):
    return torch.from_numpy(ARRAYS[key].copy()).view(torch.bfloat16)


@pytest.mark.parametrize("case", list(add_rmsnorm.CASES))
def test_add_rmsnorm_oracle_is_bit_identical_to_reference(case):
    meta = INDEX[f"add_rmsnorm/{case}"]
    inputs = add_rmsnorm.materialize_reference_case(case, meta["rows"], meta["width"])
    for name, digest in meta["inputs_sha256"].items():
        assert sha256(inputs[name].reshape(-1)) == digest, f"materialiser differs on {name}"
    got = add_rmsnorm.add_rmsnorm_reference(inputs["delta"], inputs["residual"], inputs["weight"], meta["epsilon"])
    for name in ("out", "residual_out"):
        want = bf16(f"add_rmsnorm/{case}/{name}")
        assert torch.equal(got[name].view(torch.int16), want.view(torch.int16).reshape(got[name].shape)), name
    if case == "zeros":      # signed zeros survive the add: -0 + -0 = -0 (add_rmsnorm.py:110-111)
        assert int((got["residual_out"].view(torch.int16).reshape(-1)[1::2] != -32768).sum()) == 0


@pytest.mark.parametrize("task,case", [(t, c) for t in deepseek_v4.CASES for c in deepseek_v4.CASES[t]])
def test_deepseek_v4_oracles_are_bit_identical_to_reference(task, case):
    meta = INDEX[f"deepseek_v4/{task}/{case}"]
    rows = meta["shape"]["Q" if task == "csa_indexer_topk" else "T"]
    inputs = deepseek_v4.materialize_reference_case(task, case, rows)
    for name, digest in meta["inputs_sha256"].items():
        assert sha256(inputs[name].reshape(-1)) == digest, f"materialiser differs on {name}"
    if "refused" in meta:
        with pytest.raises(ValueError):
            (deepseek_v4.csa_topk_reference(inputs["index_scores"]) if task == "csa_indexer_topk"
             else deepseek_v4.moe_gate_reference(inputs["router_logits"], inputs["selection_bias"]))
        return
    key = f"deepseek_v4/{task}/{case}"
    if task == "csa_indexer_topk":
        got = deepseek_v4.csa_topk_reference(inputs["index_scores"])
        assert got.reshape(-1).tolist() == ARRAYS[key + "/indices"].tolist()
    else:
        got = deepseek_v4.moe_gate_reference(inputs["router_logits"], inputs["selection_bias"])
        assert got["expert_ids"].reshape(-1).tolist() == ARRAYS[key + "/expert_ids"].tolist()
        want = torch.from_numpy(ARRAYS[key + "/weights"].copy()).view(torch.float32)
        assert torch.equal(got["weights"].reshape(-1).view(torch.int32), want.view(torch.int32))


def test_gate_known_answers():
    """Weights sum to the route scale and ids are six distinct experts in descending biased score
    (tests/contracts/test_deepseek_v4_workloads.py:45-54); a selection bias changes the ids, not the
    weight formula (:56-65)."""
    inputs = deepseek_v4.materialize_reference_case("moe_gate", "primary")
    base = deepseek_v4.moe_gate_reference(inputs["router_logits"], inputs["selection_bias"])
    assert all(len(set(row)) == 6 for row in base["expert_ids"].tolist())
    torch.testing.assert_close(base["weights"].sum(1), torch.full((4,), 2.5), rtol=2e-6, atol=2e-6)
    bias = deepseek_v4.materialize_reference_case("moe_gate", "bias_changes_selection")["selection_bias"]
    changed = deepseek_v4.moe_gate_reference(inputs["router_logits"], bias)
    assert changed["expert_ids"].tolist() != base["expert_ids"].tolist() and bool((changed["weights"] > 0).all())


@pytest.mark.parametrize("task", list(attention.PREFILL_TASKS))
@pytest.mark.parametrize("variant", ["captured", "boundary"])
@pytest.mark.parametrize("case", attention.CASES)
def test_prefill_oracle_is_bit_identical_to_reference(task, variant, case):
    meta = INDEX[f"prefill/{task}/{variant}/{case}"]
    inputs = attention.materialize_prefill_case(task, variant, case)
    for name, digest in meta["inputs_sha256"].items():
        assert sha256(inputs[name]) == digest, f"materialiser differs on {name}"
    mla, paged = attention.PREFILL_TASKS[task][:2]
    assert attention.prefill_nan_rule(task) == meta["nan_for_masked"]
    got = attention.causal_prefill_reference(inputs, mla=mla, paged=paged, nan_for_masked=meta["nan_for_masked"])
    key = f"prefill/{task}/{variant}/{case}"
    want_out = bf16(key + "/output").reshape(meta["output_shape"])
    want_lse = torch.from_numpy(ARRAYS[key + "/lse"].copy()).view(torch.float32).reshape(meta["output_shape"][:2])
    assert torch.equal(got["output"].view(torch.int16), want_out.view(torch.int16))
    assert torch.equal(got["lse"].view(torch.int32), want_lse.view(torch.int32))


def test_prefill_causal_mask_known_answers():
    """Bottom-right aligned causal mask (attention.py:170): with as many query rows as KV rows, row i sees i + 1 rows;
    with more query rows than KV rows the leading rows see nothing and are NaN (ragged) or zero (paged GQA)."""
    g = torch.Generator().manual_seed(1)
    k = (torch.rand((3, 4, 128), generator=g) - 0.5).to(torch.bfloat16)
    v = (torch.rand((3, 4, 128), generator=g) - 0.5).to(torch.bfloat16)
    q = torch.zeros((5, 32, 128), dtype=torch.bfloat16)             # zero query: uniform weights over the visible rows
    inputs = {"q": q, "k": k, "v": v, "qo_indptr": torch.tensor([0, 5], dtype=torch.int32),
              "kv_indptr": torch.tensor([0, 3], dtype=torch.int32), "sm_scale": torch.tensor([1.0])}
    got = attention.causal_prefill_reference(inputs, mla=False, paged=False, nan_for_masked=True)
    assert bool(torch.isnan(got["output"][:2].float()).all()) and bool(torch.isinf(got["lse"][:2]).all())
    for i, visible in ((2, 1), (3, 2), (4, 3)):
        expected = v[:visible].double().mean(0).repeat_interleave(8, 0).to(torch.bfloat16)
        assert torch.equal(got["output"][i].view(torch.int16), expected.view(torch.int16))
        torch.testing.assert_close(got["lse"][i], torch.full((32,), float(np.log2(visible))), rtol=1e-6, atol=1e-6)
    zero = attention.causal_prefill_reference(inputs, mla=False, paged=False, nan_for_masked=False)
    assert not bool(zero["output"][:2].float().abs().any())
