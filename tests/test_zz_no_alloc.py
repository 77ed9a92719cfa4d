"""GPU test of the allocation-free paged GQA decode entry point (collected last on purpose).

``cake_b200_gqa_decode_noalloc`` serves hosts that may not call the CUDA allocator and have no
workspace to lend (a server whose pool owns all device memory, a plug-in sandbox, a loop that
cannot take an allocation's synchronisation): its split-KV scratch is a fixed array inside the
library.  The test drives it through the C ABI only, twice in a row on different problems -- the
second smaller than the first, so stale scratch from the first call would show -- and compares
each result with the workspace-based entry point AND with the CPU oracle on the same inputs at the
decode tolerances (output atol 2**-16 rtol 2**-7, lse atol 1e-4 rtol 1e-5).  It also checks the
refusal above the scratch limit.  (That the call allocates nothing is a property of its source --
it names no allocating routine; what torch's allocator counter can show, and the test checks, is
only that the binding around it made no torch allocation.)"""
import ctypes

import pytest
import torch

import open_cake_ir_b200 as cake
from oracle import attention, compare

pytestmark = pytest.mark.gpu


def call_noalloc(dev, cfg, out, lse):
    lib = cake._lib.library()
    order = [dev["q"], dev["k_cache"], dev["v_cache"], dev["kv_indptr"], dev["kv_indices"], dev["kv_last_page_len"],
             dev["sm_scale"], out, lse]
    pointers = (ctypes.c_void_p * len(order))(*[t.data_ptr() for t in order])
    return lib.cake_b200_gqa_decode_noalloc(pointers, ctypes.byref(cfg), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))


def one_problem(batch, hq, hkv, page, lens, pool, salt):
    cpu, meta = cake.workloads.gqa_decode_inputs(batch, hq, hkv, 128, page, lens, pool, device="cpu", salt=salt)
    dev = {k: v.cuda() for k, v in cpu.items()}
    want_out, want_lse = cake.gqa_paged_decode(dev["q"], dev["k_cache"], dev["v_cache"], dev["kv_indptr"], dev["kv_indices"],
                                               dev["sm_scale"], dev["kv_last_page_len"], meta["max_kv_len"])
    cfg = cake._lib.GqaDecodeConfig(batch, hq, hkv, 128, page, meta["max_kv_len"])
    out = torch.full_like(want_out, float("nan"))
    lse = torch.full_like(want_lse, float("nan"))
    before = torch.cuda.memory_allocated()
    code = call_noalloc(dev, cfg, out, lse)
    torch.cuda.synchronize()
    assert code == 0, code
    assert torch.cuda.memory_allocated() == before
    ok, bad, err = compare.compare(out, want_out, atol=2.0 ** -16, rtol=2.0 ** -7)
    assert ok, f"output: {bad} mismatches, max abs err {err}"
    ok, bad, err = compare.compare(lse, want_lse, atol=1e-4, rtol=1e-5, ieee=True)
    assert ok, f"lse: {bad} mismatches, max abs err {err}"
    oracle = attention.paged_decode_reference(cpu, mla=False, page_size=page, per_head_loop=False)
    ok, bad, err = compare.compare(out, oracle["output"], atol=2.0 ** -16, rtol=2.0 ** -7)
    assert ok, f"output vs oracle: {bad} mismatches, max abs err {err}"
    ok, bad, err = compare.compare(lse, oracle["lse"], atol=1e-4, rtol=1e-5, ieee=True)
    assert ok, f"lse vs oracle: {bad} mismatches, max abs err {err}"


def test_two_calls_in_a_row_match_the_workspace_entry_point():
    one_problem(16, 32, 8, 16, (300, 2000), 2200, salt=1)
    one_problem(5, 32, 4, 16, (0, 90), 64, salt=2)


def test_problems_beyond_the_scratch_limit_are_refused():
    lib = cake._lib.library()
    assert lib.cake_b200_gqa_decode_noalloc_scratch_limit() == 16 << 20
    cpu, meta = cake.workloads.gqa_decode_inputs(2, 32, 8, 128, 16, (1, 40), 16, device="cpu")
    dev = {k: v.cuda() for k, v in cpu.items()}
    out = torch.empty_like(dev["q"]); lse = torch.empty((2, 32), dtype=torch.float32, device="cuda")
    huge = cake._lib.GqaDecodeConfig(60000, 32, 8, 128, 16, 4096)        # 60000 * 2 * 32 * 516 B > 16 MiB
    assert call_noalloc(dev, huge, out, lse) == 20004
    assert lib.cake_b200_gqa_decode_noalloc(None, ctypes.byref(huge), None) == 20001
