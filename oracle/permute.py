"""Token-permute oracle (test infrastructure; see the package docstring).

The reference defines no canonical permutation: its building blocks are an unordered atomic
reservation judged "by ownership invariants, never an invented lane order"
(tools/kernel_oracles.py:186-190) and a padded gather by (expert id, row id)
(tools/kernel_oracles.py:137-156).  This build fixes the order so that results are
reproducible: routed (token, slot) pairs whose expert lies in the local interval
[offset, offset+local_experts) are stably sorted by expert, i.e. by (expert, token, slot).
``check_ownership`` restates the reference's order-free invariants for any permutation.
"""
from __future__ import annotations

import torch


def permute_reference(expert_ids: torch.Tensor, local_offset: int, local_experts: int):
    """expert_ids int [T, K] -> dict(counts[E_local], offsets[E_local+1], sorted_pairs[n],
    inv_perm[T*K]) as int32; a pair is ``token*K + slot``; inv_perm is -1 for pairs routed to
    experts this rank does not own."""
    flat = expert_ids.reshape(-1).long() - local_offset
    local = (flat >= 0) & (flat < local_experts)
    pairs = torch.nonzero(local).reshape(-1)
    order = torch.argsort(flat[pairs], stable=True)
    sorted_pairs = pairs[order]
    counts = torch.bincount(flat[pairs], minlength=local_experts)
    offsets = torch.zeros(local_experts + 1, dtype=torch.int64)
    offsets[1:] = torch.cumsum(counts, 0)
    inv = torch.full((flat.numel(),), -1, dtype=torch.int64)
    inv[sorted_pairs] = torch.arange(sorted_pairs.numel())
    return {"counts": counts.int(), "offsets": offsets.int(),
            "sorted_pairs": sorted_pairs.int(), "inv_perm": inv.int()}


def check_ownership(expert_ids: torch.Tensor, local_offset: int, local_experts: int,
                    counts, offsets, sorted_pairs, inv_perm) -> list[str]:
    """Order-free invariants every valid permutation satisfies; returns violated ones."""
    problems = []
    flat = expert_ids.reshape(-1).long() - local_offset
    local = (flat >= 0) & (flat < local_experts)
    expect = torch.bincount(flat[local], minlength=local_experts)
    if not torch.equal(expect, counts.long()):
        problems.append("counts")
    if int(offsets[0]) != 0 or not torch.equal(offsets[1:].long() - offsets[:-1].long(), expect):
        problems.append("offsets")
    n = int(expect.sum())
    sp = sorted_pairs[:n].long()
    if sp.unique().numel() != n or not bool(local[sp].all()):
        problems.append("sorted_pairs not a set of local pairs")
    for e in range(local_experts):
        seg = sp[int(offsets[e]):int(offsets[e + 1])]
        if not bool((flat[seg] == e).all()):
            problems.append(f"segment {e} holds foreign pairs")
            break
    inv = inv_perm.long()
    if not bool((inv[~local] == -1).all()) or not torch.equal(sp[inv[local]], torch.nonzero(local).reshape(-1)):
        problems.append("inv_perm")
    return problems
