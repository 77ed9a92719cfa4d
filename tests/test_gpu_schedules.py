"""The work plans the decode operators' plan kernels write on the device, read back through
``cake_b200_decode_plan_view`` and held to the host-side restatement of tests/test_schedules.py (which the
CPU suite checks for the properties the kernels rely on)."""
import random

import pytest
import torch

from test_schedules import PIECE_COST, SEQ_COST, gqa_pieces, mla_segments

pytestmark = pytest.mark.gpu


def read_ints(pointer: int, count: int) -> list[int]:
    """`count` int32 from device memory, one at a time through the library's own status reader."""
    from open_cake_ir_b200 import _lib
    stream = torch.cuda.current_stream().cuda_stream
    return [_lib.read_status(pointer + 4 * i, stream) for i in range(count)]


def paged_lengths(lens, page_size):
    pages = [(n + page_size - 1) // page_size for n in lens]
    indptr = [0]
    for p in pages:
        indptr.append(indptr[-1] + p)
    last = [((n - 1) % page_size) + 1 if n else 0 for n in lens]
    return indptr, last


@pytest.mark.parametrize("seed", range(4))
def test_mla_device_plan_is_the_restated_one(seed):
    import open_cake_ir_b200 as cake
    from open_cake_ir_b200 import _lib
    rng = random.Random(seed)
    batch = [3, 32, 100, 1500][seed]
    lens = [rng.choice([0, 1, 31, 32, 33, 500, rng.randrange(0, 3000)]) for _ in range(batch)]
    page = 64
    indptr, last = paged_lengths(lens, page)
    pool = indptr[-1] + 1
    dev = "cuda"
    heads = 16
    q_nope = torch.zeros((batch, heads, 512), dtype=torch.bfloat16, device=dev)
    q_pe = torch.zeros((batch, heads, 64), dtype=torch.bfloat16, device=dev)
    ckv = torch.zeros((pool, page, 512), dtype=torch.bfloat16, device=dev)
    kpe = torch.zeros((pool, page, 64), dtype=torch.bfloat16, device=dev)
    op = cake.MlaPagedDecode(q_nope, q_pe, ckv, kpe, torch.tensor(indptr, dtype=torch.int32, device=dev),
                             torch.arange(indptr[-1], dtype=torch.int32, device=dev), torch.tensor(last, dtype=torch.int32, device=dev),
                             torch.tensor([0.1], device=dev), torch.empty_like(q_nope),
                             torch.empty((batch, heads), dtype=torch.float32, device=dev), max_kv_len=max(lens))
    op.launch()
    pointer, count = _lib.decode_plan_view("mla_decode", op.native.handle, 0)
    _, workers = _lib.decode_plan_view("mla_decode", op.native.handle, 1)
    assert count == batch + 1 and workers >= 1
    _, prefix, _, tiles = mla_segments(lens, workers)
    assert read_ints(pointer, count) == prefix
    assert prefix[-1] == sum(t + SEQ_COST for t in tiles if t)
    assert op.status() == 0


@pytest.mark.parametrize("seed", range(4))
def test_gqa_device_plan_is_the_restated_one(seed):
    import open_cake_ir_b200 as cake
    from open_cake_ir_b200 import _lib
    rng = random.Random(50 + seed)
    batch = [2, 64, 200, 1500][seed]
    lens = [rng.choice([0, 1, 15, 16, 17, 700, rng.randrange(0, 2000)]) for _ in range(batch)]
    page = 16
    indptr, last = paged_lengths(lens, page)
    pool = indptr[-1] + 1
    dev = "cuda"
    q = torch.zeros((batch, 32, 128), dtype=torch.bfloat16, device=dev)
    k = torch.zeros((pool, page, 8, 128), dtype=torch.bfloat16, device=dev)
    op = cake.GqaPagedDecode(q, k, torch.zeros_like(k), torch.tensor(indptr, dtype=torch.int32, device=dev),
                             torch.arange(indptr[-1], dtype=torch.int32, device=dev), torch.tensor(last, dtype=torch.int32, device=dev),
                             torch.tensor([0.1], device=dev), torch.empty_like(q),
                             torch.empty((batch, 32), dtype=torch.float32, device=dev), max_kv_len=max(lens))
    op.launch()
    items_ptr, capacity = _lib.decode_plan_view("gqa_decode", op.native.handle, 0)
    first_ptr, ranges = _lib.decode_plan_view("gqa_decode", op.native.handle, 1)
    count_ptr, _ = _lib.decode_plan_view("gqa_decode", op.native.handle, 2)
    items, range_first, range_count, _ = gqa_pieces(lens, ranges)
    assert len(items) <= capacity
    got = read_ints(items_ptr, 4 * len(items))
    want = []
    for b, count, begin, first, end in items:
        want += [b | (count << 16), begin, first, end]
    assert got == want
    assert read_ints(count_ptr, ranges) == range_count
    got_first = read_ints(first_ptr, ranges)
    assert [None if c == 0 else f for f, c in zip(got_first, range_count)] == [None if c == 0 else f for f, c in zip(range_first, range_count)]
    assert PIECE_COST == 32 and op.status() == 0
