"""GPU parity of causal prefill (GQA paged and ragged, MLA paged) through the C ABI: the reference's fifty
cases against its golden outputs, then larger ragged-length problems with pages of more than one token
against the oracle.  Tolerances are the contract's (src/open_cake_ir/tasks/solx_fib/attention.py:76-79):
output atol 2**-16 rtol 2**-7, lse atol 1e-4 rtol 1e-5, NaN and infinities matched by the IEEE rule."""
import json
from pathlib import Path

import numpy as np
import pytest
import torch

import open_cake_ir_b200 as cake
from gpu_util import poison, snapshot, unchanged
from oracle import attention, compare

pytestmark = pytest.mark.gpu
BASE = Path(__file__).resolve().parent / "golden"
INDEX = json.loads((BASE / "next_index.json").read_text())
ARRAYS = np.load(BASE / "next_outputs.npz")
O_ATOL, O_RTOL, L_ATOL, L_RTOL = 2.0 ** -16, 2.0 ** -7, 1e-4, 1e-5


def run(cpu, *, mla, paged, nan, max_kv_len):
    dev = {k: v.cuda() for k, v in cpu.items()}
    before = snapshot(dev)
    q = cpu["q_nope"] if mla else cpu["q"]
    out, g1 = poison(tuple(q.shape), torch.bfloat16)
    lse, g2 = poison(tuple(q.shape[:2]), torch.float32)
    last = dev.get("kv_last_page_len")
    if mla:
        op = cake.MlaCausalPrefill(dev["q_nope"], dev["q_pe"], dev["ckv_cache"], dev["kpe_cache"], dev["qo_indptr"], dev["kv_indptr"],
                                   dev["kv_indices"], last, dev["sm_scale"], out, lse, max_kv_len=max_kv_len, nan_for_masked=nan)
    elif paged:
        op = cake.GqaCausalPrefill(dev["q"], dev["k_cache"], dev["v_cache"], dev["qo_indptr"], dev["kv_indptr"], dev["kv_indices"],
                                   last, dev["sm_scale"], out, lse, max_kv_len=max_kv_len, nan_for_masked=nan)
    else:
        op = cake.GqaCausalPrefill(dev["q"], dev["k"], dev["v"], dev["qo_indptr"], dev["kv_indptr"], None, None, dev["sm_scale"],
                                   out, lse, max_kv_len=max_kv_len, nan_for_masked=nan)
    op.launch()
    assert op.status() == 0
    g1(); g2()
    assert unchanged(before, dev)
    return out, lse


def check(out, lse, want):
    ok, bad, err = compare.compare(out, want["output"], atol=O_ATOL, rtol=O_RTOL, ieee=True)
    assert ok, f"output: {bad} mismatches, max abs err {err}"
    ok, bad, err = compare.compare(lse, want["lse"], atol=L_ATOL, rtol=L_RTOL, ieee=True)
    assert ok, f"lse: {bad} mismatches, max abs err {err}"


@pytest.mark.parametrize("task", list(attention.PREFILL_TASKS))
@pytest.mark.parametrize("variant", ["captured", "boundary"])
@pytest.mark.parametrize("case", attention.CASES)
def test_reference_cases(task, variant, case):
    key = f"prefill/{task}/{variant}/{case}"
    meta = INDEX[key]
    mla, paged = attention.PREFILL_TASKS[task][:2]
    cpu = attention.materialize_prefill_case(task, variant, case)
    shape = meta["output_shape"]
    want = {"output": torch.from_numpy(ARRAYS[key + "/output"].copy()).view(torch.bfloat16).reshape(shape),
            "lse": torch.from_numpy(ARRAYS[key + "/lse"].copy()).view(torch.float32).reshape(shape[:2])}
    out, lse = run(cpu, mla=mla, paged=paged, nan=meta["nan_for_masked"], max_kv_len=64)
    check(out, lse, want)


def ragged_problem(seed, segments, q_range, kv_range, *, mla, paged, page_size, heads, kv_heads):
    g = torch.Generator().manual_seed(seed)
    q_lens = torch.randint(q_range[0], q_range[1] + 1, (segments,), generator=g)
    kv_lens = torch.randint(kv_range[0], kv_range[1] + 1, (segments,), generator=g)
    kv_lens[0] = 0 if segments > 2 else kv_lens[0]                  # a segment without KV rows
    total_q = int(q_lens.sum())
    cpu = {"qo_indptr": torch.cat([torch.zeros(1, dtype=torch.long), q_lens.cumsum(0)]).int(),
           "sm_scale": torch.tensor([1.0 / (192.0 if mla else 128.0) ** 0.5])}
    if paged:
        pages = (kv_lens + page_size - 1) // page_size
        cpu["kv_indptr"] = torch.cat([torch.zeros(1, dtype=torch.long), pages.cumsum(0)]).int()
        pool = int(pages.sum()) + 7
        cpu["kv_indices"] = torch.randperm(pool, generator=g)[:int(pages.sum())].int()
        cpu["kv_last_page_len"] = torch.where(pages > 0, kv_lens - (pages - 1) * page_size, torch.zeros_like(kv_lens)).int()
        if mla:
            cpu["ckv_cache"] = torch.randn((pool, page_size, 512), generator=g).to(torch.bfloat16)
            cpu["kpe_cache"] = torch.randn((pool, page_size, 64), generator=g).to(torch.bfloat16)
        else:
            cpu["k_cache"] = torch.randn((pool, page_size, kv_heads, 128), generator=g).to(torch.bfloat16)
            cpu["v_cache"] = torch.randn((pool, page_size, kv_heads, 128), generator=g).to(torch.bfloat16)
    else:
        cpu["kv_indptr"] = torch.cat([torch.zeros(1, dtype=torch.long), kv_lens.cumsum(0)]).int()
        total_kv = int(kv_lens.sum())
        cpu["k"] = torch.randn((total_kv, kv_heads, 128), generator=g).to(torch.bfloat16)
        cpu["v"] = torch.randn((total_kv, kv_heads, 128), generator=g).to(torch.bfloat16)
    if mla:
        cpu["q_nope"] = torch.randn((total_q, heads, 512), generator=g).to(torch.bfloat16)
        cpu["q_pe"] = torch.randn((total_q, heads, 64), generator=g).to(torch.bfloat16)
    else:
        cpu["q"] = torch.randn((total_q, heads, 128), generator=g).to(torch.bfloat16)
    return cpu, int(kv_lens.max())


@pytest.mark.parametrize("mla,paged,page_size,heads,kv_heads,segments,q_range,kv_range,nan", [
    (False, True, 16, 32, 8, 4, (1, 40), (0, 300), False), (False, True, 1, 32, 4, 3, (5, 9), (1, 6), False),
    (False, False, 1, 32, 8, 5, (1, 30), (0, 200), True), (False, False, 1, 16, 2, 2, (64, 64), (64, 64), True),
    (True, True, 64, 16, 1, 3, (1, 20), (0, 500), True), (True, True, 4, 128, 1, 2, (3, 6), (2, 40), True)])
def test_serving_like_shapes(mla, paged, page_size, heads, kv_heads, segments, q_range, kv_range, nan):
    cpu, max_len = ragged_problem(7 + page_size + heads, segments, q_range, kv_range, mla=mla, paged=paged, page_size=page_size,
                                  heads=heads, kv_heads=kv_heads)
    want = attention.causal_prefill_reference(cpu, mla=mla, paged=paged, page_size=page_size, nan_for_masked=nan, per_head_loop=False)
    out, lse = run(cpu, mla=mla, paged=paged, nan=nan, max_kv_len=max(max_len, 1))
    check(out, lse, want)
