"""The failure path of the tensor-core kernels, exercised without hanging or faulting anything: every device-side
wait is bounded, and when one runs out the kernel records a code in its status word, all of its roles unwind,
copies in flight are given time to land, tensor memory is freed and the kernel RETURNS.  The test shortens the
wait budget to about a millisecond of clocks and makes the first CTA leave one operand load out
(``cake_b200_test_hooks``), checks the status word, and checks that the next ordinary launch on the same handle
is correct -- the context stays usable (the reference keeps every teardown failure instead of aborting,
src/open_cake_ir/evaluation/cuda_driver.py:147-183)."""
import pytest
import torch

import open_cake_ir_b200 as cake
from oracle import attention, block_scaled_gemm, compare

pytestmark = pytest.mark.gpu


@pytest.fixture
def hooks():
    lib = cake._lib.library()
    yield lib.cake_b200_test_hooks
    assert lib.cake_b200_test_hooks(0, 0) == 0


def test_gemm_wait_runs_out_and_the_handle_stays_usable(hooks):
    g = cake.workloads.block_scaled_gemm_inputs(256, 512, 1024, device="cpu")
    dev = {k: v.cuda() for k, v in g.items()}
    c = torch.zeros((256, 512), dtype=torch.bfloat16, device="cuda")
    op = cake.BlockScaledGemm(dev["a"], dev["sfa"], dev["b"], dev["sfb"], c)
    assert hooks(2048, 1) == 0                 # waits give up after 2 Mi clocks; CTA 0 never receives its second K block
    op.launch()
    assert op.status() == 1                    # the MMA issuer's wait for a filled ring slot ran out
    assert hooks(0, 0) == 0
    op.launch()
    assert op.status() == 0
    want = block_scaled_gemm.block_scaled_gemm_reference(g["a"], g["sfa"], g["b"], g["sfb"], out_dtype=None)
    assert compare.rel_frobenius(c, want) <= 1e-2


def test_mla_decode_wait_runs_out_and_the_handle_stays_usable(hooks):
    cpu, meta = cake.workloads.mla_decode_inputs(2, 128, 64, (6000, 9000), device="cpu")      # every CTA meets three tiles or more
    dev = {k: v.cuda() for k, v in cpu.items()}
    out = torch.zeros_like(dev["q_nope"]); lse = torch.zeros((2, 128), dtype=torch.float32, device="cuda")
    op = cake.MlaPagedDecode(dev["q_nope"], dev["q_pe"], dev["ckv_cache"], dev["kpe_cache"], dev["kv_indptr"], dev["kv_indices"],
                             dev["kv_last_page_len"], dev["sm_scale"], out, lse, max_kv_len=meta["max_kv_len"])
    assert hooks(2048, 1) == 0
    op.launch()
    assert op.status() != 0                    # a ring wait of CTA 0 ran out (which role notices first is not fixed)
    assert hooks(0, 0) == 0
    op.launch()
    assert op.status() == 0
    want = attention.paged_decode_reference(cpu, mla=True, page_size=64, per_head_loop=False)
    assert compare.compare(out, want["output"], atol=2.0 ** -16, rtol=2.0 ** -7)[0]
    assert compare.compare(lse, want["lse"], atol=1e-4, rtol=1e-5, ieee=True)[0]


def test_push_exchange_wait_for_a_rank_that_never_arrives_runs_out(hooks):
    """Two ranks of the push exchange live on this GPU (ordinary buffers in place of the symmetric ones); only rank 0
    runs its step, so the flag it waits for is one that nothing sets.  With the wait budget shortened the wait runs
    out in about a millisecond, the kernel returns, the status word says so, and the context stays usable: two
    fresh ranks then complete steps in lock step with the right result."""
    from open_cake_ir_b200 import ep
    shape, tokens, world = dict(hidden=1024, inter=512, experts=32), 256, 2

    def make_ranks():
        sym = ep.PushExpertParallelMoe.symmetric_bytes(tokens // world, shape["hidden"], 8, world, shape["experts"])
        buffers = [torch.zeros(sym + 256, dtype=torch.uint8, device="cuda") for _ in range(world)]
        ranks = []
        for rank in range(world):
            dev = cake.workloads.moe_inputs(tokens=tokens // world, **shape, local_experts=shape["experts"] // world,
                                            local_offset=rank * shape["experts"] // world, routing="softmax", device="cuda",
                                            gen_device="cpu", first_token=rank * tokens // world, total_tokens=tokens)
            ranks.append(ep.PushExpertParallelMoe(dev, dev["routing_logits"], dev["routing_bias"], dev["hidden_states"],
                                                  dev["hidden_states_scale"], experts=shape["experts"], routing="softmax",
                                                  virtual=(rank, world, buffers)))
        return ranks

    lonely = make_ranks()
    assert hooks(2048, 0) == 0                 # waits for another rank give up after 2 Mi clocks
    parts = lonely[0]._parts()
    parts[0]()                                 # rank 0 routes, plans and pushes its rows ...
    parts[1]()                                 # ... and waits for rank 1's rows, which never come
    torch.cuda.synchronize()
    assert lonely[0].status() == 5 and lonely[1].status() == 0
    assert hooks(0, 0) == 0
    for layer in lonely:
        layer.close()

    ranks = make_ranks()
    whole = cake.workloads.moe_inputs(tokens=tokens, **shape, local_experts=shape["experts"], local_offset=0,
                                      routing="softmax", device="cuda", gen_device="cpu")
    want = cake.fp8_moe(whole, experts=shape["experts"], routing="softmax", act_mode="fp8")
    for _ in range(2):
        step_parts = [layer._parts() for layer in ranks]
        for i in range(len(step_parts[0])):
            for rank_parts in step_parts:
                rank_parts[i]()
        torch.cuda.synchronize()
        got = torch.cat([layer.output for layer in ranks])
        assert all(layer.status() == 0 for layer in ranks)
        assert compare.rel_frobenius(got.cpu(), want.cpu()) <= 1e-2
