"""GPU parity of sparse MLA decode (contracts/workloads/dsa-attention-sparse-mla-decode-v1.json) through the
C ABI against the fp64 restatement of the contract's definition, at the contract's geometry (16 heads,
page 64, top-k 2048) with its tolerance (atol = rtol = 1e-2 on at least 99.9 % of the elements) and at this
build's tighter decode tolerance; plus the reduction to the pinned paged-decode oracle when the index list is
a sequence's rows in order.  Inputs are seeded synthetic tensors of the contract's shapes (its captured index
lists are not part of the reference checkout)."""
import pytest
import torch

import open_cake_ir_b200 as cake
from gpu_util import poison, snapshot, unchanged
from oracle import attention, compare

pytestmark = pytest.mark.gpu
SCALE = cake.SparseMlaDecode.SM_SCALE


def make_inputs(tokens, heads, pages, top_k, present, seed, page_size=64):
    g = torch.Generator().manual_seed(seed)
    rows = pages * page_size
    cpu = {"q_nope": (torch.rand((tokens, heads, 512), generator=g) - 0.5).to(torch.bfloat16),
           "q_pe": (torch.rand((tokens, heads, 64), generator=g) - 0.5).to(torch.bfloat16),
           "ckv_cache": torch.randn((pages, page_size, 512), generator=g).to(torch.bfloat16),
           "kpe_cache": torch.randn((pages, page_size, 64), generator=g).to(torch.bfloat16)}
    idx = torch.full((tokens, top_k), -1, dtype=torch.int32)
    for t in range(tokens):
        n = present(t)
        chosen = torch.randperm(rows, generator=g)[:n].int()
        where = torch.randperm(top_k, generator=g)[:n] if t % 2 else torch.arange(n)     # absent entries anywhere / trailing
        idx[t, where] = chosen
    cpu["sparse_indices"] = idx
    return cpu


def run(cpu):
    dev = {k: v.cuda() for k, v in cpu.items()}
    before = snapshot(dev)
    out, guard = poison(tuple(cpu["q_nope"].shape), torch.bfloat16)
    op = cake.SparseMlaDecode(dev["q_nope"], dev["q_pe"], dev["ckv_cache"], dev["kpe_cache"], dev["sparse_indices"], out)
    op.launch()
    assert op.status() == 0
    guard()
    assert unchanged(before, dev)
    return out


@pytest.mark.parametrize("tokens,heads,pages,top_k,present", [
    (8, 16, 128, 2048, lambda t: 2048), (7, 16, 128, 2048, lambda t: (0, 1, 31, 33, 500, 2047, 2048)[t]),
    (1, 16, 40, 2048, lambda t: 1200), (3, 128, 16, 256, lambda t: 100 + t), (2, 16, 4, 64, lambda t: 0)])
def test_against_the_contract_definition(tokens, heads, pages, top_k, present):
    cpu = make_inputs(tokens, heads, pages, top_k, present, seed=tokens * 1000 + top_k)
    want = attention.sparse_mla_decode_reference(cpu, SCALE)
    out = run(cpu)
    ok, bad, err = compare.compare(out, want, atol=1e-2, rtol=1e-2)
    assert bad <= 0.001 * out.numel(), f"{bad} of {out.numel()} elements outside atol = rtol = 1e-2 (max abs err {err})"
    ok, bad, err = compare.compare(out, want, atol=2.0 ** -16, rtol=2.0 ** -7)      # the paged decode contract's tolerance
    assert ok, f"{bad} mismatches at the decode tolerance, max abs err {err}"


def test_reduces_to_paged_decode_when_the_list_is_a_sequence():
    pages, page_size, length = 12, 64, 700
    g = torch.Generator().manual_seed(5)
    cpu = make_inputs(2, 16, pages, 1024, lambda t: 0, seed=9)
    order = torch.randperm(pages, generator=g)[:11].int()
    rows = (order.long()[:, None] * page_size + torch.arange(page_size)[None, :]).reshape(-1)[:length].int()
    cpu["sparse_indices"][:, :length] = rows
    paged = dict(cpu, kv_indptr=torch.tensor([0, 11, 22], dtype=torch.int32), kv_indices=torch.cat([order, order]),
                 kv_last_page_len=torch.tensor([length - 10 * page_size] * 2, dtype=torch.int32),
                 sm_scale=torch.tensor([SCALE], dtype=torch.float32))
    want = attention.paged_decode_reference(paged, mla=True, page_size=page_size, per_head_loop=False)["output"]
    assert torch.equal(attention.sparse_mla_decode_reference(cpu, SCALE).view(torch.int16), want.view(torch.int16))
    out = run(cpu)
    ok, bad, err = compare.compare(out, want, atol=2.0 ** -16, rtol=2.0 ** -7)
    assert ok, f"{bad} mismatches, max abs err {err}"
