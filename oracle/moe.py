"""FP8 block-scaled MoE expert-layer oracle (test infrastructure; see the package docstring).

Follows src/open_cake_ir/tasks/solx_fib/moe.py:122-155 (``reference_tensors``) with the
hard-coded ``T=1`` / 32 local experts generalised to any token count and any local expert
interval: route, and for every (token, slot) whose expert is local dequantise the hidden row
and both weight matrices with their 128-element block scales in float64, ``first = a @ W13^T``,
``act = first[:, :I] * silu(first[:, I:])`` (silu on the SECOND half, moe.py:150-151),
``contribution = (act @ W2^T) * route_weight``; contributions of one token are added in slot
order 0..K-1 (moe.py:143-154) and the sum is rounded once to bf16.

Options beyond the reference (pinned by their own tests, not by the reference):
``act_quant="fp8"`` inserts the e4m3 per-(row, 128) amax/448 quantiser between SwiGLU and the
second GEMM -- the reference keeps that intermediate in float64 (moe.py:150-154);
``routing="softmax"`` selects the second routing definition of ``oracle.routing``.
"""
from __future__ import annotations

import torch

from .routing import routing_ds, routing_softmax_topk

E4M3_MAX = 448.0
INPUT_ORDER = ("routing_logits", "routing_bias", "hidden_states", "hidden_states_scale",
               "gemm1_weights", "gemm1_weights_scale", "gemm2_weights", "gemm2_weights_scale",
               "local_expert_offset", "routed_scaling_factor")


def quantize_rows_e4m3(act: torch.Tensor, group: int = 128):
    """Per-(row, 128-group) quantiser: scale = amax/448 in fp32 (1.0 where amax is 0),
    q = e4m3(act/scale) round-to-nearest-even, saturating.  Returns (q e4m3 [R, C],
    scale fp32 [C/group, R]) -- the scale is stored K-block-major like the contract's
    ``hidden_states_scale``."""
    rows, cols = act.shape
    a = act.float().reshape(rows, cols // group, group)
    amax = a.abs().amax(dim=2)
    scale = torch.where(amax > 0, amax / E4M3_MAX, torch.ones_like(amax))
    q = (a / scale[:, :, None]).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn)
    return q.reshape(rows, cols), scale.t().contiguous()


def dequantize_rows(q: torch.Tensor, scale: torch.Tensor, dtype=torch.float64, group: int = 128):
    return q.to(dtype) * scale.t().to(dtype).repeat_interleave(group, 1)


def dequantize_weight(w: torch.Tensor, scale: torch.Tensor, dtype=torch.float64):
    out = w.to(dtype)
    out *= scale.to(dtype).repeat_interleave(128, 0).repeat_interleave(128, 1)
    return out


def route(inputs, routing: str, top_k: int = 8):
    factor = float(inputs["routed_scaling_factor"][0])
    if routing == "ds":
        return routing_ds(inputs["routing_logits"], inputs["routing_bias"], factor, top_k=top_k)
    if routing == "softmax":
        ids, w = routing_softmax_topk(inputs["routing_logits"], top_k)
        return ids, w * factor
    if routing == "external":     # routing decided elsewhere (expert-parallel receive side); ids outside the local interval are ignored
        return inputs["expert_ids"].long(), inputs["route_weights"].float()
    raise ValueError("routing must be 'ds', 'softmax' or 'external'")


def moe_reference(inputs: dict, *, routing: str = "ds", act_quant: str = "none",
                  dtype=torch.float64, top_k: int = 8, return_parts: bool = False):
    """Rank-local MoE layer.  ``inputs`` carries the contract's ten input tensors
    (moe.py:13-20 names and layouts; T tokens, E_local = gemm1_weights.shape[0])."""
    hidden = inputs["hidden_states"]
    tokens, width = hidden.shape
    local_experts, two_i, _ = inputs["gemm1_weights"].shape
    inter = two_i // 2
    offset = int(inputs["local_expert_offset"][0])
    selected, weights = route(inputs, routing, top_k)
    a = hidden.to(dtype) * inputs["hidden_states_scale"].T.to(dtype).repeat_interleave(128, 1)
    contributions = torch.zeros((tokens, top_k, width), dtype=dtype)
    local = selected - offset
    for e in range(local_experts):
        where = torch.nonzero(local == e)
        if where.numel() == 0:
            continue
        tok, slot = where[:, 0], where[:, 1]
        w1 = dequantize_weight(inputs["gemm1_weights"][e], inputs["gemm1_weights_scale"][e], dtype)
        first = a[tok] @ w1.T
        x1, x2 = first[:, :inter], first[:, inter:]
        activation = x1 * (x2 / (1 + torch.exp(-x2)))
        if act_quant == "fp8":
            q, s = quantize_rows_e4m3(activation)
            activation = dequantize_rows(q, s, dtype)
        elif act_quant != "none":
            raise ValueError("act_quant must be 'none' or 'fp8'")
        w2 = dequantize_weight(inputs["gemm2_weights"][e], inputs["gemm2_weights_scale"][e], dtype)
        contributions[tok, slot] = (activation @ w2.T) * weights[tok, slot].to(dtype)[:, None]
    output = torch.zeros((tokens, width), dtype=dtype)
    for slot in range(top_k):
        output += contributions[:, slot]
    result = {"output": output.to(torch.bfloat16)}
    if return_parts:
        result.update(expert_ids=selected, route_weights=weights, output_wide=output)
    return result


# --- the reference's input materialiser, restated (moe.py:90-119) -------------------------
CASES = ("primary", "zero_hidden", "all_nonlocal", "mixed_local", "scaled", "ties")
REF_TENSORS = {
    "routing_logits": ([1, 256], "fp32"), "routing_bias": ([256], "bf16"),
    "hidden_states": ([1, 7168], "fp8_e4m3"), "hidden_states_scale": ([56, 1], "fp32"),
    "gemm1_weights": ([32, 4096, 7168], "fp8_e4m3"), "gemm1_weights_scale": ([32, 32, 56], "fp32"),
    "gemm2_weights": ([32, 7168, 2048], "fp8_e4m3"), "gemm2_weights_scale": ([32, 56, 16], "fp32"),
    "local_expert_offset": ([1], "int32"), "routed_scaling_factor": ([1], "fp32"),
}


def materialize_reference_case(case_id: str) -> dict[str, torch.Tensor]:
    """Inputs of one of the reference's six cases: one CPU generator seeded 2901+case index
    consumed in the contract's tensor order; FP8 tensors are ``(rand-0.5)*scale`` cast to
    e4m3 in 4 Mi-element chunks; scales ``0.5+rand``; logits a 256-point linspace."""
    g = torch.Generator(device="cpu").manual_seed(2901 + CASES.index(case_id))
    values = {}
    for name, (shape, dtype) in REF_TENSORS.items():
        if dtype == "fp8_e4m3":
            scale = 0.5 if name == "hidden_states" else 0.125
            value = torch.empty(shape, dtype=torch.float8_e4m3fn)
            flat = value.reshape(-1)
            step = 4 * 1024 * 1024
            for start in range(0, flat.numel(), step):
                end = min(start + step, flat.numel())
                flat[start:end] = ((torch.rand((end - start,), generator=g) - 0.5) * scale).to(torch.float8_e4m3fn)
            values[name] = value
        elif name.endswith("_scale"):
            values[name] = 0.5 + torch.rand(shape, generator=g)
    values["routing_logits"] = torch.linspace(-2, 2, 256, dtype=torch.float32).reshape(1, 256)
    values["routing_bias"] = (torch.rand((256,), generator=g) * 0.015).to(torch.bfloat16)
    offset = 224
    if case_id == "all_nonlocal":
        offset = 0
    if case_id == "mixed_local":
        values["routing_logits"][0, 216:224] += 0.5
    if case_id in {"zero_hidden", "ties"}:
        values["hidden_states"].zero_()
    if case_id == "ties":
        values["routing_logits"].zero_(); values["routing_bias"].zero_()
    factor = 0.75 if case_id == "scaled" else 2.5
    values["local_expert_offset"] = torch.tensor([offset], dtype=torch.int32)
    values["routed_scaling_factor"] = torch.tensor([factor], dtype=torch.float32)
    return {name: values[name] for name in INPUT_ORDER}
