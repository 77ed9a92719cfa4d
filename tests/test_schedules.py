"""Host-side restatement of the two device-side work schedules of the decode operators, checked for
the properties the kernels rely on (no GPU needed).

* MLA (csrc/decode_mla.cu, mla_plan_kernel / tiles_per_worker): the 32-token tiles of all sequences form
  one list; worker w of W takes the w-th of W equal consecutive ranges; a (worker, sequence) pair
  that meets writes its partial result to slot worker + sequence.
* GQA (csrc/decode_gqa.cu, gqa_plan_kernel): the tokens of all sequences form one list, cut into equal
  consecutive ranges (a multiple of the 16-token tile); the pieces of sequences the ranges hold are
  listed in token order, so the pieces of a range, and the pieces of a sequence, are consecutive.
"""
import random

import pytest


SEQ_COST = 14      # units charged at the start of a sequence (kSeqCost)


def mla_segments(lens, workers, tile=32):
    tiles = [(n + tile - 1) // tile for n in lens]
    prefix = [0]
    for t in tiles:
        prefix.append(prefix[-1] + (t + SEQ_COST if t else 0))
    total = prefix[-1]
    per = (total + workers - 1) // workers if total > 0 else 1
    segments = []
    for w in range(workers):
        at, stop = w * per, min(total, (w + 1) * per)
        while at < stop:
            lo, hi = 0, len(lens)
            while hi - lo > 1:               # largest b with prefix[b] <= at, as in the kernel
                mid = (lo + hi) // 2
                if prefix[mid] <= at:
                    lo = mid
                else:
                    hi = mid
            b = lo
            upto = min(prefix[b + 1], stop)
            first = max(at - prefix[b] - SEQ_COST, 0)
            n = upto - prefix[b] - SEQ_COST - first
            at = upto
            if n > 0:
                segments.append((w, b, first, n))
    return segments, prefix, per, tiles


@pytest.mark.parametrize("seed", range(6))
def test_mla_ranges_cover_every_tile_once_and_slots_are_unique(seed):
    rng = random.Random(seed)
    batch = rng.choice([1, 2, 7, 32, 100])
    lens = [rng.choice([0, 1, 31, 32, 33, 500, 4097, rng.randrange(0, 9000)]) for _ in range(batch)]
    workers = rng.choice([1, 3, 37, 64])
    segments, prefix, per, tiles = mla_segments(lens, workers)
    covered = {}
    slots = set()
    for w, b, first, n in segments:
        assert n > 0 and first + n <= tiles[b]
        for t in range(first, first + n):
            assert (b, t) not in covered
            covered[(b, t)] = w
        slot = w + b
        assert slot not in slots and slot < workers + batch
        slots.add(slot)
    assert len(covered) == sum(tiles)
    # the reduce kernel finds a sequence's partial results from the prefix alone
    for b, n in enumerate(lens):
        if n == 0:
            continue
        first_w, last_w = (prefix[b] + SEQ_COST) // per, (prefix[b + 1] - 1) // per
        assert {w + b for w in range(first_w, last_w + 1)} == {w + bb for w, bb, _, _ in segments if bb == b}
    # equal shares: no worker has more than `per` units (tiles + a start-up share per sequence start)
    load = {}
    for w, _, _, n in segments:
        load[w] = load.get(w, 0) + n
    assert max(load.values(), default=0) <= per


PIECE_COST = 32    # token units charged at the start of a sequence (kPieceCost)


def gqa_pieces(lens, ranges):
    total = sum(n + PIECE_COST for n in lens if n > 0)
    per = max(16, (((total + ranges - 1) // ranges) + 15) & ~15)
    items, range_first, range_count = [], [None] * ranges, [0] * ranges
    before = 0
    for b, n in enumerate(lens):
        if n == 0:
            continue
        start = before + PIECE_COST                      # where the sequence's tokens begin, in units
        first_range, count = start // per, (start + n - 1) // per - start // per + 1
        first = len(items)
        for k in range(count):
            range_start = (first_range + k) * per
            begin, end = max(start, range_start), min(start + n, range_start + per)
            r = first_range + k
            range_first[r] = len(items) if range_first[r] is None else min(range_first[r], len(items))
            range_count[r] += 1
            items.append((b, count, begin - start, first, end - start))
        before += n + PIECE_COST
    return items, range_first, range_count, per


@pytest.mark.parametrize("seed", range(5))
def test_gqa_ranges_partition_the_token_list(seed):
    rng = random.Random(100 + seed)
    lens = [rng.choice([0, 1, 15, 16, 17, 700, 4096, rng.randrange(0, 5000)]) for _ in range(rng.choice([1, 5, 64]))]
    ranges = rng.choice([1, 18, 148, 1184])
    items, range_first, range_count, per = gqa_pieces(lens, ranges)
    assert per % 16 == 0 and len(items) <= ranges + len(lens)
    # pieces of a sequence: consecutive entries, tiling it exactly
    for b, n in enumerate(lens):
        mine = [(i, it) for i, it in enumerate(items) if it[0] == b]
        assert [i for i, _ in mine] == list(range(mine[0][0], mine[0][0] + len(mine))) if mine else n == 0
        pos = 0
        for i, (_, count, begin, first, end) in mine:
            assert count == len(mine) and first == mine[0][0] and begin == pos and end > begin
            pos = end
        assert pos == n
    # pieces of a range: consecutive entries, every entry in exactly one range, no range above its share
    seen = []
    for r in range(ranges):
        if range_count[r]:
            seen.extend(range(range_first[r], range_first[r] + range_count[r]))
            units = sum(end - begin for _, _, begin, _, end in items[range_first[r]:range_first[r] + range_count[r]])
            assert units <= per
    assert seen == list(range(len(items)))
