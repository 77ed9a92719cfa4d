"""The restated oracles of the operators either side of the hot path (two-output add + RMSNorm, the
DeepSeek-V4 MoE gate and CSA indexer top-k) against outputs of the reference's own oracles
(tests/golden/make_golden_next.py): regenerated inputs hash-equal, outputs bit-identical, and the
cases the reference's oracle refuses are refused here too."""
import json
from pathlib import Path

import numpy as np
import pytest
import torch

from conftest import sha256
from oracle import add_rmsnorm, deepseek_v4

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
