"""GPU parity: paged GQA and MLA decode through the C ABI against the reference's cases (golden
outputs) and against the oracle at serving shapes.  Tolerances are the contract's
(src/open_cake_ir/tasks/solx_fib/attention.py:76-79): output atol 2**-16 rtol 2**-7; lse atol 1e-4
rtol 1e-5 with the IEEE rule for -inf."""
import pytest
import torch

import open_cake_ir_b200 as cake
from gpu_util import poison, snapshot, unchanged
from oracle import attention, compare

pytestmark = pytest.mark.gpu
O_ATOL, O_RTOL, L_ATOL, L_RTOL = 2.0 ** -16, 2.0 ** -7, 1e-4, 1e-5


def run_gqa(cpu, max_kv_len):
    dev = {k: v.cuda() for k, v in cpu.items()}
    before = snapshot(dev)
    out, g1 = poison(tuple(cpu["q"].shape), torch.bfloat16)
    lse, g2 = poison(tuple(cpu["q"].shape[:2]), torch.float32)
    op = cake.GqaPagedDecode(dev["q"], dev["k_cache"], dev["v_cache"], dev["kv_indptr"], dev["kv_indices"],
                             dev["kv_last_page_len"], dev["sm_scale"], out, lse, max_kv_len=max_kv_len)
    op.launch()
    torch.cuda.synchronize()
    g1(); g2()
    assert unchanged(before, dev)
    return out, lse


def run_mla(cpu, max_kv_len):
    dev = {k: v.cuda() for k, v in cpu.items()}
    before = snapshot(dev)
    out, g1 = poison(tuple(cpu["q_nope"].shape), torch.bfloat16)
    lse, g2 = poison(tuple(cpu["q_nope"].shape[:2]), torch.float32)
    op = cake.MlaPagedDecode(dev["q_nope"], dev["q_pe"], dev["ckv_cache"], dev["kpe_cache"], dev["kv_indptr"],
                             dev["kv_indices"], dev["kv_last_page_len"], dev["sm_scale"], out, lse, max_kv_len=max_kv_len)
    op.launch()
    torch.cuda.synchronize()
    g1(); g2()
    assert unchanged(before, dev)
    return out, lse


def check(out, lse, want):
    ok, bad, err = compare.compare(out, want["output"], atol=O_ATOL, rtol=O_RTOL)
    assert ok, f"output: {bad} mismatches, max abs err {err}"
    ok, bad, err = compare.compare(lse, want["lse"], atol=L_ATOL, rtol=L_RTOL, ieee=True)
    assert ok, f"lse: {bad} mismatches, max abs err {err}"


def with_last_page(inputs):
    pages = inputs["kv_indptr"][1:] - inputs["kv_indptr"][:-1]
    inputs = dict(inputs)
    inputs["kv_last_page_len"] = (pages > 0).to(torch.int32)
    return inputs


@pytest.mark.parametrize("task", ["gqa_kv4", "gqa_kv8", "mla_h16"])
@pytest.mark.parametrize("variant", ["captured", "boundary"])
@pytest.mark.parametrize("case", attention.CASES)
def test_reference_cases(golden, task, variant, case):
    key = f"decode/{task}/{variant}/{case}"
    cpu = with_last_page(attention.materialize_reference_case(task, variant, case))
    shape = golden.index[key]["output_shape"]
    want = {"output": golden.bf16(key + "/output").reshape(shape), "lse": golden.fp32(key + "/lse").reshape(shape[:2])}
    n = int(cpu["kv_indices"].numel())
    out, lse = (run_mla if task.startswith("mla") else run_gqa)(cpu, max_kv_len=max(n, 1))
    check(out, lse, want)


@pytest.mark.parametrize("batch,hq,hkv,page,lens", [(64, 32, 8, 16, (512, 4096)), (5, 32, 4, 16, (1, 70)),
                                                    (3, 8, 8, 1, (1, 300)), (7, 16, 8, 5, (0, 133)),
                                                    # KV head counts that take the other range/pair mappings of the kernel
                                                    (3, 8, 1, 16, (1, 900)), (4, 16, 2, 8, (0, 500)), (2, 24, 3, 16, (5, 700)),
                                                    (3, 64, 16, 16, (1, 600)), (1, 32, 8, 16, (9000, 9000)),
                                                    # more than 1024 sequences: the plan kernel's second pass and its carries
                                                    (1500, 8, 2, 4, (0, 40))])
def test_gqa_serving_shapes(batch, hq, hkv, page, lens):
    pool = 20000 if batch == 64 else max(400, batch * (lens[1] // page + 2))
    cpu, meta = cake.workloads.gqa_decode_inputs(batch, hq, hkv, 128, page, lens, pool, device="cpu")
    want = attention.paged_decode_reference(cpu, mla=False, page_size=page, per_head_loop=False)
    out, lse = run_gqa(cpu, meta["max_kv_len"])
    check(out, lse, want)


@pytest.mark.parametrize("batch,heads,page,lens", [(32, 128, 64, (1024, 8192)), (3, 16, 1, (1, 200)), (4, 128, 64, (0, 700)),
                                                   (2, 80, 7, (33, 400)), (2, 256, 16, (10, 300)), (1, 128, 64, (20000, 20000)),
                                                   # more than 1024 sequences: the plan kernel's second pass and its carry
                                                   (1500, 16, 4, (0, 40))])
def test_mla_serving_shapes(batch, heads, page, lens):
    cpu, meta = cake.workloads.mla_decode_inputs(batch, heads, page, lens, device="cpu")
    want = attention.paged_decode_reference(cpu, mla=True, page_size=page, per_head_loop=False)
    out, lse = run_mla(cpu, meta["max_kv_len"])
    check(out, lse, want)


def test_zero_query_known_answer_on_device():
    """Zero query => uniform weights: output = mean of the V rows, lse = log2(L)
    (tests/contracts/test_solx_fib_launch_plans.py:93-102)."""
    import math
    cpu = with_last_page(attention.materialize_reference_case("gqa_kv4", "boundary", "zeros"))
    out, lse = run_gqa(cpu, 8)
    for b in range(2):
        lo, hi = cpu["kv_indptr"][b:b + 2].tolist()
        ids = cpu["kv_indices"][lo:hi].long()
        expected = cpu["v_cache"][ids, 0].double().mean(0).repeat_interleave(8, 0).to(torch.bfloat16)
        assert compare.compare(out[b], expected, atol=O_ATOL, rtol=O_RTOL)[0]
        torch.testing.assert_close(lse[b].cpu(), torch.full((32,), math.log2(hi - lo)), rtol=1e-5, atol=1e-5)
