"""DeepSeek-V4 routing-stage oracles: the MoE gate and the CSA indexer top-k (test infrastructure; see
the package docstring).

Both follow src/open_cake_ir/tasks/deepseek_v4/workload.py:184-202 (``reference_outputs``):

* gate (:190-201): ``score = RN_fp32(sqrt(log1p(exp(x))))`` in double then rounded to fp32; the experts
  are ranked by ``score + selection_bias`` (a double sum of two fp32 values, exact), the best six in
  descending order are the ``expert_ids``; ``weights = RN_fp32(2.5 * score / fsum(selected scores))``.
* indexer (:188-189): the positions of the 1024 largest of 2048 fp32 scores, in descending order.

The reference refuses rows with tied scores (:175-181); so do these.  The materialiser restates :153-172.
"""
from __future__ import annotations

import math
import random

import numpy as np
import torch

CSA_CANDIDATES, CSA_TOPK = 2048, 1024
MOE_EXPERTS, MOE_TOPK, MOE_ROUTE_SCALE = 384, 6, 2.5
CASES = {
    "csa_indexer_topk": {"primary": ("uniform_distinct", 9501), "skewed": ("skewed_distinct", 9502),
                         "boundary": ("boundary_distinct", 9503), "tail": ("tail_distinct", 9504)},
    "moe_gate": {"primary": ("uniform_distinct", 9601), "bias_changes_selection": ("biased_distinct", 9602),
                 "negative": ("negative_distinct", 9603), "tail": ("tail_distinct", 9604)},
}


def _rank_unique(values: np.ndarray, count: int) -> np.ndarray:
    """values double [rows, width] -> indices int64 [rows, count] of the `count` largest, descending."""
    rows, width = values.shape
    out = np.empty((rows, count), dtype=np.int64)
    for r in range(rows):
        if len(set(values[r].tolist())) != width:
            raise ValueError("tied scores are outside the contract")
        out[r] = np.argsort(-values[r], kind="stable")[:count]
    return out


def csa_topk_reference(index_scores: torch.Tensor, top_k: int = CSA_TOPK) -> torch.Tensor:
    """index_scores fp32 [Q, S] -> indices int32 [Q, top_k]."""
    return torch.from_numpy(_rank_unique(index_scores.double().numpy(), top_k)).to(torch.int32)


def moe_gate_reference(router_logits: torch.Tensor, selection_bias: torch.Tensor, top_k: int = MOE_TOPK,
                       route_scale: float = MOE_ROUTE_SCALE):
    """router_logits fp32 [T, E], selection_bias fp32 [E] -> {"weights": fp32 [T, top_k], "expert_ids": int32 [T, top_k]}."""
    x = router_logits.double().numpy()
    scores = np.array([[math.sqrt(math.log1p(math.exp(v))) for v in row] for row in x.tolist()]).astype(np.float32).astype(np.float64)
    selection = scores + selection_bias.double().numpy()[None, :]
    ids = _rank_unique(selection, top_k)
    weights = np.empty(ids.shape, dtype=np.float32)
    for t in range(ids.shape[0]):
        chosen = scores[t, ids[t]]
        total = math.fsum(chosen.tolist())
        weights[t] = np.array([route_scale * v / total for v in chosen.tolist()]).astype(np.float32)
    return {"weights": torch.from_numpy(weights), "expert_ids": torch.from_numpy(ids).to(torch.int32)}


def materialize_reference_case(task: str, case_id: str, rows: int = 4) -> dict[str, torch.Tensor]:
    """Inputs of one reference case (deepseek_v4/workload.py:153-172): one ``random.Random(seed + 10000*position)``
    per input tensor, values rounded to fp32."""
    mode, seed = CASES[task][case_id]
    shapes = ({"index_scores": (rows, CSA_CANDIDATES)} if task == "csa_indexer_topk"
              else {"router_logits": (rows, MOE_EXPERTS), "selection_bias": (MOE_EXPERTS,)})
    result = {}
    for position, (name, shape) in enumerate(shapes.items()):
        rng = random.Random(seed + position * 10000)
        count = math.prod(shape)
        values = np.empty(count)
        for index in range(count):
            if mode == "negative_distinct":
                value = -1.0 - index / (count + 1)
            elif mode == "skewed_distinct":
                value = 8.0 - index / (count + 1)
            elif mode == "boundary_distinct":
                value = 16.0 - 32.0 * index / max(count - 1, 1)
            elif mode == "biased_distinct" and name == "selection_bias":
                value = 4.0 - index / (count + 1)
            elif mode == "tail_distinct":
                value = (index % 31) / 32.0 + rng.uniform(-1e-5, 1e-5)
            else:
                value = rng.uniform(-2.0, 2.0) + index / (count + 1) * 1e-3
            values[index] = value
        result[name] = torch.from_numpy(values.astype(np.float32)).reshape(shape)
    return result
