"""GPU test of the expert-parallel layer on two B200s (skipped where only one is visible): tokens and
experts sharded over two NCCL ranks with all-to-all dispatch and combine must reproduce the
single-GPU native layer over all tokens and experts.  Partial rows travel as bf16 and are added in
fp32, so the comparison is at the bf16 tolerance (rtol 2e-2 / atol 2e-2, Frobenius <= 1e-2)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import open_cake_ir_b200 as cake
from open_cake_ir_b200 import ep
from oracle import compare

pytestmark = pytest.mark.gpu
SHAPE = dict(hidden=1024, inter=512, experts=32)
TOKENS = 512


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, results, native):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        t_local, e_local = TOKENS // world, SHAPE["experts"] // world
        dev = cake.workloads.moe_inputs(tokens=t_local, **SHAPE, local_experts=e_local, local_offset=rank * e_local,
                                        routing="softmax", device=f"cuda:{rank}", gen_device="cpu",
                                        first_token=rank * t_local, total_tokens=TOKENS)
        args = [dev[k] for k in ("routing_logits", "routing_bias", "routed_scaling_factor", "hidden_states", "hidden_states_scale")]
        if native in ("native", "push"):
            cls = ep.NativeExpertParallelMoe if native == "native" else ep.PushExpertParallelMoe
            layer = cls(dev, dev["routing_logits"], dev["routing_bias"], dev["hidden_states"],
                        dev["hidden_states_scale"], experts=SHAPE["experts"], routing="softmax")
            for _ in range(3):      # several steps: buffers, flags and step numbers are reused between steps
                out = layer.forward()
            if native == "push":
                assert layer.status() == 0
                layer.capture()     # and once more as a CUDA graph
                out = layer.forward()
                assert layer.status() == 0
        else:
            route_factory, local_layer = ep.native_layer(dev, capacity=TOKENS, experts=SHAPE["experts"], device=f"cuda:{rank}")
            layer = ep.ExpertParallelMoe(experts=SHAPE["experts"], top_k=8, hidden=SHAPE["hidden"], capacity=TOKENS,
                                         route=route_factory("softmax"), local_layer=local_layer, device=f"cuda:{rank}")
            for _ in range(2):
                out = layer.forward(*args)
        torch.cuda.synchronize()
        results[rank] = out.cpu()
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("native", ["native", "push", "torch"], ids=["nccl-exchange", "push-exchange", "torch-exchange"])
def test_two_rank_layer_equals_single_gpu_layer(native):
    world = 2
    results = mp.Manager().dict()
    mp.spawn(_worker, args=(world, _free_port(), results, native), nprocs=world, join=True)
    whole = cake.workloads.moe_inputs(tokens=TOKENS, **SHAPE, local_experts=SHAPE["experts"], local_offset=0,
                                      routing="softmax", device="cuda:0", gen_device="cpu")
    want = cake.fp8_moe(whole, experts=SHAPE["experts"], routing="softmax", act_mode="fp8").cpu()
    got = torch.cat([results[r] for r in range(world)])
    assert compare.rel_frobenius(got, want) <= 1e-2
    ok, bad, err = compare.compare(got, want, atol=2e-2, rtol=2e-2)
    assert ok, f"{bad} mismatches, max abs err {err}"


def test_single_rank_exchange_is_the_identity():
    """World size 1 (one GPU is enough): plan, pack, unpack and reduce around the rank-local layer must
    reproduce the plain layer bit for bit, since one bf16 partial per token is added to nothing."""
    dev = cake.workloads.moe_inputs(tokens=200, **SHAPE, local_experts=SHAPE["experts"], local_offset=0, routing="softmax",
                                    device="cuda", gen_device="cpu")
    want = cake.fp8_moe(dev, experts=SHAPE["experts"], routing="softmax", act_mode="fp8")
    layer = ep.NativeExpertParallelMoe(dev, dev["routing_logits"], dev["routing_bias"], dev["hidden_states"],
                                       dev["hidden_states_scale"], experts=SHAPE["experts"], routing="softmax")
    got = layer.forward()
    torch.cuda.synchronize()
    assert torch.equal(got.view(torch.int16), want.view(torch.int16))
    assert int((layer.slot_of.cpu()[:, 0] != torch.arange(200)).sum()) == 0


def test_single_rank_push_exchange_is_the_identity():
    """The push exchange with a world of one: the rank writes its rows into its own receive block, waits for its own
    flags, and must reproduce the plain layer bit for bit over several steps (flags and step numbers are reused)."""
    dev = cake.workloads.moe_inputs(tokens=200, **SHAPE, local_experts=SHAPE["experts"], local_offset=0, routing="softmax",
                                    device="cuda", gen_device="cpu")
    want = cake.fp8_moe(dev, experts=SHAPE["experts"], routing="softmax", act_mode="fp8")
    layer = ep.PushExpertParallelMoe(dev, dev["routing_logits"], dev["routing_bias"], dev["hidden_states"],
                                     dev["hidden_states_scale"], experts=SHAPE["experts"], routing="softmax")
    for _ in range(3):
        got = layer.forward()
        torch.cuda.synchronize()
        assert layer.status() == 0
        assert torch.equal(got.view(torch.int16), want.view(torch.int16))
    assert layer.rows_sent() == 200
    layer.capture()
    got = layer.forward()
    torch.cuda.synchronize()
    assert layer.status() == 0 and torch.equal(got.view(torch.int16), want.view(torch.int16))


def _virtual_ranks_step(layers):
    """One step of `layers` (the ranks of one expert-parallel group, all in this process on one GPU): every part of
    the step on every rank before the next part, so that each wait finds its flags already set."""
    parts = [layer._parts() for layer in layers]
    for i in range(len(parts[0])):
        for rank_parts in parts:
            rank_parts[i]()
    torch.cuda.synchronize()
    return torch.cat([layer.output for layer in layers])


@pytest.mark.parametrize("world,tokens,shape", [
    (4, 512, dict(hidden=1024, inter=512, experts=32)),
    (4, 4096, dict(hidden=7168, inter=512, experts=256)),
    (8, 4096, dict(hidden=7168, inter=512, experts=256)),
    (8, 1000 // 8 * 8, dict(hidden=1024, inter=512, experts=64)),
], ids=["4-ranks-small", "4-ranks-serving-rows", "8-ranks-serving-rows", "8-ranks-ragged"])
def test_push_exchange_with_virtual_ranks_on_one_gpu(world, tokens, shape):
    """The push exchange at 4 and 8 ranks without 4 or 8 GPUs: all ranks live on one GPU with ordinary buffers in
    place of the symmetric ones and run the parts of a step in lock step.  The result must be the single-GPU layer's
    over all tokens and experts, at the tolerance of bf16 partial rows, over several steps."""
    t_local, e_local = tokens // world, shape["experts"] // world
    sym = ep.PushExpertParallelMoe.symmetric_bytes(t_local, shape["hidden"], 8, world, shape["experts"])
    buffers = [torch.zeros(sym + 256, dtype=torch.uint8, device="cuda") for _ in range(world)]
    layers = []
    for rank in range(world):
        dev = cake.workloads.moe_inputs(tokens=t_local, **shape, local_experts=e_local, local_offset=rank * e_local,
                                        routing="softmax", device="cuda", gen_device="cuda",
                                        first_token=rank * t_local, total_tokens=tokens)
        layers.append(ep.PushExpertParallelMoe(dev, dev["routing_logits"], dev["routing_bias"], dev["hidden_states"],
                                               dev["hidden_states_scale"], experts=shape["experts"], routing="softmax",
                                               virtual=(rank, world, buffers)))
    whole = cake.workloads.moe_inputs(tokens=tokens, **shape, local_experts=shape["experts"], local_offset=0,
                                      routing="softmax", device="cuda", gen_device="cuda")
    want = cake.fp8_moe(whole, experts=shape["experts"], routing="softmax", act_mode="fp8")
    for _ in range(3):
        got = _virtual_ranks_step(layers)
        assert all(layer.status() == 0 for layer in layers)
        assert compare.rel_frobenius(got.cpu(), want.cpu()) <= 1e-2
        assert compare.compare(got.cpu(), want.cpu(), atol=2e-2, rtol=2e-2)[0]
    assert sum(layer.rows_sent() for layer in layers) >= tokens
