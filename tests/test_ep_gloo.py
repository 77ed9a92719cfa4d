"""CPU test of the expert-parallel exchange (world size 2, gloo): the dispatch plan, packing, the
two all-to-alls and the rank-ordered combine, with the CPU oracle standing in for the native
rank-local layer.  The joined result must equal the single-rank layer over all tokens and experts."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import open_cake_ir_b200 as cake
from open_cake_ir_b200 import ep
from oracle import compare, moe as oracle_moe, routing as oracle_routing

SHAPE = dict(hidden=256, inter=128, experts=16)
TOKENS = 48


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        per_rank_tokens, per_rank_experts = TOKENS // world, SHAPE["experts"] // world
        mine = cake.workloads.moe_inputs(tokens=per_rank_tokens, **SHAPE, local_experts=per_rank_experts,
                                         local_offset=rank * per_rank_experts, routing="softmax", device="cpu",
                                         first_token=rank * per_rank_tokens, total_tokens=TOKENS)

        def route(logits, bias, factor):
            ids, w = oracle_routing.routing_softmax_topk(logits)
            return ids.int(), (w * float(factor[0])).float()

        def local_layer(hidden, scale, ids, w):
            inputs = dict(mine)
            inputs.update(hidden_states=hidden, hidden_states_scale=scale, expert_ids=ids, route_weights=w)
            return oracle_moe.moe_reference(inputs, routing="external", act_quant="fp8", dtype=torch.float32)["output"]

        layer = ep.ExpertParallelMoe(experts=SHAPE["experts"], top_k=8, hidden=SHAPE["hidden"], capacity=TOKENS,
                                     route=route, local_layer=local_layer, device="cpu")
        out = layer.forward(mine["routing_logits"], mine["routing_bias"], mine["routed_scaling_factor"],
                            mine["hidden_states"], mine["hidden_states_scale"])
        results[rank] = (out, layer.last_counts)
    finally:
        dist.destroy_process_group()


def test_exchange_plan_sends_each_token_once_per_destination_rank():
    ids = torch.tensor([[0, 1, 2, 3], [4, 5, 6, 7], [0, 4, 1, 5], [7, 6, 5, 4]], dtype=torch.int32)
    send_tokens, counts, slot_of = ep.exchange_plan(ids, world=2, experts=8)
    assert counts.tolist() == [2, 3]
    assert send_tokens.tolist() == [0, 2, 1, 2, 3]
    assert slot_of.tolist() == [[0, -1], [-1, 2], [1, 3], [-1, 4]]
    assert ep.row_bytes(7168, 8) == 7168 + 224 + 64


def test_two_rank_layer_equals_single_rank_layer():
    world = 2
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_worker, args=(world, _free_port(), results), nprocs=world, join=True)
    whole = cake.workloads.moe_inputs(tokens=TOKENS, **SHAPE, local_experts=SHAPE["experts"], local_offset=0,
                                      routing="softmax", device="cpu")
    want = oracle_moe.moe_reference(whole, routing="softmax", act_quant="fp8", dtype=torch.float32)["output"]
    got = torch.cat([results[r][0] for r in range(world)])
    assert compare.rel_frobenius(got, want) <= 1e-2
    ok, bad, err = compare.compare(got, want, atol=2e-2, rtol=2e-2)
    assert ok, f"{bad} mismatches, max abs err {err}"
    for r in range(world):      # what one rank sends the other receives
        send, recv = results[r][1]
        assert send[1 - r] == results[1 - r][1][1][r]
        assert sum(send) <= TOKENS // world * world
