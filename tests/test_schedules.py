"""Host-side restatement of the two device-side work schedules of the decode operators, checked for
the properties the kernels rely on (no GPU needed).

* MLA (csrc/decode_mla.cu, mla_plan_kernel / tiles_per_worker): the 32-token tiles of all sequences form
  one list; worker w of W takes the w-th of W equal consecutive ranges; a (worker, sequence) pair
  that meets writes its partial result to slot worker + sequence.
* GQA (csrc/decode_gqa.cu, gqa_plan_kernel / chunk_at): every sequence is cut into chunks of one
  size, a multiple of 64 tokens between 192 and the base chunk, chosen from the work left.
"""
import random

import pytest


def mla_segments(lens, workers, tile=32):
    tiles = [(n + tile - 1) // tile for n in lens]
    prefix = [0]
    for t in tiles:
        prefix.append(prefix[-1] + t)
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
            n = min(prefix[b + 1], stop) - at
            segments.append((w, b, at - prefix[b], n))
            at += n
    return segments, prefix, per


@pytest.mark.parametrize("seed", range(6))
def test_mla_ranges_cover_every_tile_once_and_slots_are_unique(seed):
    rng = random.Random(seed)
    batch = rng.choice([1, 2, 7, 32, 100])
    lens = [rng.choice([0, 1, 31, 32, 33, 500, 4097, rng.randrange(0, 9000)]) for _ in range(batch)]
    workers = rng.choice([1, 3, 37, 64])
    segments, prefix, per = mla_segments(lens, workers)
    covered = {}
    slots = set()
    for w, b, first, n in segments:
        assert n > 0 and first + n <= prefix[b + 1] - prefix[b]
        for t in range(first, first + n):
            assert (b, t) not in covered
            covered[(b, t)] = w
        slot = w + b
        assert slot not in slots and slot < workers + batch
        slots.add(slot)
    assert len(covered) == prefix[-1]
    # the reduce kernel finds a sequence's partial results from the prefix alone
    for b, n in enumerate(lens):
        if n == 0:
            continue
        first_w, last_w = prefix[b] // per, (prefix[b + 1] - 1) // per
        assert {w + b for w in range(first_w, last_w + 1)} == {w + bb for w, bb, _, _ in segments if bb == b}
    # equal shares: no worker has more than `per` tiles
    load = {}
    for w, _, _, n in segments:
        load[w] = load.get(w, 0) + n
    assert max(load.values(), default=0) <= per


def gqa_chunks(lens, hkv, workers, base, guide_div=2, guide_min=192):
    total = sum(lens)
    share = float(hkv) / (float(workers) * guide_div)
    out, before = [], 0
    for n in lens:
        c = int(min((total - before) * share, 4096.0)) & ~63
        c = min(guide_min, base) if c < guide_min else min(c, base)
        out.append([(pos, min(c, n - pos)) for pos in range(0, n, c)])
        before += n
    return out


@pytest.mark.parametrize("seed", range(4))
def test_gqa_chunks_tile_every_sequence(seed):
    rng = random.Random(100 + seed)
    lens = [rng.choice([0, 1, 63, 64, 65, 700, 4096, rng.randrange(0, 5000)]) for _ in range(rng.choice([1, 5, 64]))]
    base = rng.choice([64, 256, 512])
    chunks = gqa_chunks(lens, hkv=8, workers=1184, base=base)
    sizes = set()
    for n, seq in zip(lens, chunks):
        pos = 0
        for begin, tokens in seq:
            assert begin == pos and begin % 64 == 0 and 0 < tokens <= 1024     # what the record packs: begin/64, 11 bits of tokens
            pos += tokens
        assert pos == n
        if len(seq) > 1:
            sizes.add(seq[0][1])
    assert all(s % 64 == 0 and min(192, base) <= s <= base for s in sizes)
    # sizes never grow along the list: the head of the queue has the largest chunks
    firsts = [seq[0][1] for seq in chunks if len(seq) > 1]
    assert firsts == sorted(firsts, reverse=True)
