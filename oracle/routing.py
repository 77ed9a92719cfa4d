"""MoE routing oracles (test infrastructure; see the package docstring).

``routing_ds`` follows src/open_cake_ir/tasks/solx_fib/moe.py:275-287
(``routing_reference``) with the token axis generalised from 1 to T: sigmoid scores, bias
added for choice only, group score = sum of the two best biased scores of each group, best
``topk_group`` groups kept, best ``top_k`` experts among them, weights = unbiased sigmoid of
the selected experts normalised by their sum (+1e-20) times the scaling factor.  All order
decisions are stable descending sorts, so ties go to the lowest index (moe.py:63).

``routing_softmax_topk`` is the second routing definition this build supports (top-k of the
raw logits, softmax over the selected k logits).  The reference holds no such operator; its
tie rule is the same lowest-index rule and it is pinned by its own known-answer tests.
"""
from __future__ import annotations

import torch


def routing_ds(logits: torch.Tensor, bias: torch.Tensor, factor: float, *, n_group: int = 8,
               topk_group: int = 4, top_k: int = 8):
    """logits fp32 [T, E], bias bf16/fp32 [E] -> (expert ids int64 [T, top_k], weights fp32)."""
    tokens, experts = logits.shape
    per_group = experts // n_group
    s = 1 / (1 + torch.exp(-logits.float()))
    biased = (s + bias.float()).reshape(tokens, n_group, per_group)
    group_scores = torch.sort(biased, dim=2, descending=True, stable=True).values[:, :, :2].sum(2)
    groups = torch.argsort(group_scores, dim=1, descending=True, stable=True)[:, :topk_group]
    mask = torch.zeros((tokens, n_group), dtype=torch.bool).scatter_(1, groups, True)
    mask = mask.repeat_interleave(per_group, 1)
    scores = (s + bias.float()).masked_fill(~mask, -float("inf"))
    selected = torch.argsort(scores, dim=1, descending=True, stable=True)[:, :top_k]
    selected_s = s.gather(1, selected)
    weights = selected_s / (selected_s.sum(1, keepdim=True) + 1e-20) * factor
    return selected, weights


def routing_softmax_topk(logits: torch.Tensor, top_k: int = 8):
    """Top-k of the raw fp32 logits (ties to the lower expert id, result in descending score
    order) and fp32 softmax over the selected logits only."""
    selected = torch.argsort(logits.float(), dim=1, descending=True, stable=True)[:, :top_k]
    chosen = logits.float().gather(1, selected)
    weights = torch.softmax(chosen, dim=1)
    return selected, weights


def score_gap(logits: torch.Tensor, bias: torch.Tensor, *, mode: str, top_k: int = 8,
              n_group: int = 8, topk_group: int = 4) -> torch.Tensor:
    """Smallest relative gap, per token, between two scores whose order decides a selection
    (k-th vs (k+1)-th expert, and for the group-limited mode also the group cut and the
    in-group second/third score).  A device exp() that differs from the host's by an ulp can
    only change the chosen set where this gap is of that order, so parity tests use it to
    name such tokens instead of failing on them."""
    if mode == "softmax":
        return torch.zeros(logits.shape[0]) + float("inf")  # raw logits: comparisons are exact
    tokens, experts = logits.shape
    per_group = experts // n_group
    s = 1 / (1 + torch.exp(-logits.float()))
    biased = s + bias.float()
    grouped = torch.sort(biased.reshape(tokens, n_group, per_group), dim=2, descending=True).values
    in_group = ((grouped[:, :, 1] - grouped[:, :, 2]).abs() / grouped[:, :, 1].abs()).amin(1)
    group_scores = grouped[:, :, :2].sum(2)
    gs = torch.sort(group_scores, dim=1, descending=True).values
    group_cut = (gs[:, topk_group - 1] - gs[:, topk_group]).abs() / gs[:, topk_group - 1].abs()
    groups = torch.argsort(group_scores, dim=1, descending=True, stable=True)[:, :topk_group]
    mask = torch.zeros((tokens, n_group), dtype=torch.bool).scatter_(1, groups, True)
    scores = biased.masked_fill(~mask.repeat_interleave(per_group, 1), -float("inf"))
    es = torch.sort(scores, dim=1, descending=True).values
    adjacent = ((es[:, :top_k] - es[:, 1:top_k + 1]).abs() / es[:, :top_k].abs()).amin(1)
    return torch.minimum(torch.minimum(in_group, group_cut), adjacent)
