"""Operator objects: each owns one native handle created from torch CUDA tensors passed in the
workload contract's ABI order, and launches on the caller's stream.

The checks before ``create`` are the reference loader's (src/open_cake_ir/evaluation/cuda_driver.py:
shape, dtype, contiguity, one device, and no output aliasing any other buffer, :219-220).  torch
is used for device memory and streams only; all arithmetic runs in ``libcake_b200.so``.
"""
from __future__ import annotations

import torch

from . import _lib

_DTYPES = {"fp32": torch.float32, "bf16": torch.bfloat16, "fp8_e4m3": torch.float8_e4m3fn, "int32": torch.int32}


def _check(name: str, tensor: torch.Tensor, dtype: str, shape) -> torch.Tensor:
    if not isinstance(tensor, torch.Tensor):
        raise TypeError(f"{name} must be a torch tensor")
    if tensor.device.type != "cuda":
        raise ValueError(f"{name} must live on a CUDA device (this target has no CPU path)")
    if tensor.dtype != _DTYPES[dtype]:
        raise ValueError(f"{name} must be {dtype}, got {tensor.dtype}")
    if shape is not None and tuple(tensor.shape) != tuple(shape):
        raise ValueError(f"{name} must have shape {tuple(shape)}, got {tuple(tensor.shape)}")
    if not tensor.is_contiguous():
        raise ValueError(f"{name} must be contiguous row-major")
    return tensor


def _no_alias(outputs: dict, everything: dict) -> None:
    def span(t):
        return t.data_ptr(), t.data_ptr() + t.numel() * t.element_size()
    for out_name, out in outputs.items():
        lo, hi = span(out)
        for name, other in everything.items():
            if other is out or other.numel() == 0 or out.numel() == 0:
                continue
            a, b = span(other)
            if lo < b and a < hi:
                raise ValueError(f"output {out_name} aliases {name}")


def _stream(stream) -> int:
    if stream is None:
        return torch.cuda.current_stream().cuda_stream
    return stream.cuda_stream if hasattr(stream, "cuda_stream") else int(stream)


class _Operator:
    stem = ""

    def _create(self, tensors: list, config, workspace_bytes: int = 0):
        devices = {t.device for t in tensors}
        if len(devices) != 1:
            raise ValueError("all tensors must be on one device")
        self.device = devices.pop()
        self._keep = list(tensors)
        self.workspace = None
        pointers = [t.data_ptr() for t in tensors]
        with torch.cuda.device(self.device):
            if workspace_bytes:
                self.workspace = torch.empty(workspace_bytes + 256, dtype=torch.uint8, device=self.device)
                base = (self.workspace.data_ptr() + 255) // 256 * 256
                self.workspace_ptr = base
                pointers.append(base)
            self.native = _lib.NativeHandle(self.stem, pointers, config)

    def _create_with_optional(self, tensors: list, config, workspace_bytes: int):
        """As ``_create`` for an ABI with optional buffers: ``None`` entries are passed as null pointers."""
        present = [t for t in tensors if t is not None]
        devices = {t.device for t in present}
        if len(devices) != 1:
            raise ValueError("all tensors must be on one device")
        self.device = devices.pop()
        self._keep = present
        pointers = [0 if t is None else t.data_ptr() for t in tensors]
        with torch.cuda.device(self.device):
            self.workspace = torch.empty(workspace_bytes + 256, dtype=torch.uint8, device=self.device)
            self.workspace_ptr = (self.workspace.data_ptr() + 255) // 256 * 256
            pointers.append(self.workspace_ptr)
            self.native = _lib.NativeHandle(self.stem, pointers, config)

    def launch(self, stream=None) -> None:
        with torch.cuda.device(self.device):
            self.native.launch(_stream(stream))

    def status(self, stream=None) -> int:
        """Device status word (0 = all bounded waits completed); synchronises the stream."""
        if self.workspace is None:
            return 0
        with torch.cuda.device(self.device):
            return _lib.read_status(self.workspace_ptr, _stream(stream))

    def close(self) -> None:
        self.native.close()


class RmsNorm(_Operator):
    """``out = bf16(z * weight / sqrt(mean(z^2) + eps))`` with ``z = x`` or ``fp32(x + residual)``
    (src/open_cake_ir/tasks/solx_fib/workload.py:214-218)."""
    stem = "rmsnorm"

    def __init__(self, x, weight, out, epsilon: float, residual=None):
        rows, width = x.shape
        _check("x", x, "bf16", None); _check("weight", weight, "bf16", (width,)); _check("out", out, "bf16", (rows, width))
        tensors = {"x": x, "weight": weight, "out": out}
        order = [x]
        if residual is not None:
            _check("residual", residual, "bf16", (rows, width))
            tensors["residual"] = residual
            order.append(residual)
        order += [weight, out]
        _no_alias({"out": out}, tensors)
        cfg = _lib.RmsNormConfig(rows, width, float(epsilon), 1 if residual is not None else 0)
        self._create(order, cfg)


class AddRmsNorm(_Operator):
    """``z = bf16(delta + residual); residual_out = z; out = bf16(fp32(z) * rsqrt(mean z^2 + eps) * weight)``
    (src/open_cake_ir/tasks/add_rmsnorm.py:66): two fresh outputs, the rounded sum is what is normalised."""
    stem = "add_rmsnorm"

    def __init__(self, delta, residual, weight, out, residual_out, epsilon: float = 1e-6):
        rows, width = delta.shape
        _check("delta", delta, "bf16", None); _check("residual", residual, "bf16", (rows, width))
        _check("weight", weight, "bf16", (width,)); _check("out", out, "bf16", (rows, width))
        _check("residual_out", residual_out, "bf16", (rows, width))
        _no_alias({"out": out, "residual_out": residual_out},
                  {"delta": delta, "residual": residual, "weight": weight, "out": out, "residual_out": residual_out})
        self._create([delta, residual, weight, out, residual_out], _lib.AddRmsNormConfig(rows, width, float(epsilon)))


class BlockScaledGemm(_Operator):
    """``c = bf16((a*sfa) @ (b*sfb)^T)``; a e4m3 [M,K], sfa fp32 [K/128,M], b e4m3 [N,K],
    sfb fp32 [N/128,K/128] (corpus/schedules/block-scaled-gemm-b1-smoke.json)."""
    stem = "block_scaled_gemm"

    def __init__(self, a, sfa, b, sfb, c):
        m, k = a.shape
        n = b.shape[0]
        _check("a", a, "fp8_e4m3", None); _check("sfa", sfa, "fp32", (k // 128, m))
        _check("b", b, "fp8_e4m3", (n, k)); _check("sfb", sfb, "fp32", (n // 128, k // 128))
        _check("c", c, "bf16", (m, n))
        _no_alias({"c": c}, {"a": a, "sfa": sfa, "b": b, "sfb": sfb, "c": c})
        cfg = _lib.GemmConfig(m, n, k)
        self._create([a, sfa, b, sfb, c], cfg, _lib.workspace_bytes(self.stem, cfg))


class MoeRouting(_Operator):
    """Routing stages of the MoE plan (src/open_cake_ir/tasks/solx_fib/moe.py:275-287).
    mode "ds": DeepSeek-V3 group-limited sigmoid; "softmax": top-k logits, softmax over them."""
    stem = "moe_routing"

    def __init__(self, routing_logits, routing_bias, routed_scaling_factor, expert_ids, route_weights, *,
                 top_k=8, n_group=8, topk_group=4, mode="ds"):
        tokens, experts = routing_logits.shape
        _check("routing_logits", routing_logits, "fp32", None); _check("routing_bias", routing_bias, "bf16", (experts,))
        _check("routed_scaling_factor", routed_scaling_factor, "fp32", (1,))
        _check("expert_ids", expert_ids, "int32", (tokens, top_k)); _check("route_weights", route_weights, "fp32", (tokens, top_k))
        _no_alias({"expert_ids": expert_ids, "route_weights": route_weights},
                  {"routing_logits": routing_logits, "routing_bias": routing_bias, "f": routed_scaling_factor,
                   "expert_ids": expert_ids, "route_weights": route_weights})
        cfg = _lib.RoutingConfig(tokens, experts, top_k, n_group, topk_group, {"ds": 0, "softmax": 1}[mode])
        self._create([routing_logits, routing_bias, routed_scaling_factor, expert_ids, route_weights], cfg)


class V4MoeGate(_Operator):
    """DeepSeek-V4 gate: sqrt-softplus scores, top-k of score + selection_bias, weights = route_scale *
    score / sum over the selection (src/open_cake_ir/tasks/deepseek_v4/workload.py:190-201).  Outputs in the
    contract's order: ``weights`` then ``expert_ids``."""
    stem = "v4_moe_gate"

    def __init__(self, router_logits, selection_bias, weights, expert_ids, *, top_k=6, route_scale=2.5):
        tokens, experts = router_logits.shape
        _check("router_logits", router_logits, "fp32", None); _check("selection_bias", selection_bias, "fp32", (experts,))
        _check("weights", weights, "fp32", (tokens, top_k)); _check("expert_ids", expert_ids, "int32", (tokens, top_k))
        _no_alias({"weights": weights, "expert_ids": expert_ids},
                  {"router_logits": router_logits, "selection_bias": selection_bias, "weights": weights, "expert_ids": expert_ids})
        self._create([router_logits, selection_bias, weights, expert_ids], _lib.V4GateConfig(tokens, experts, top_k, float(route_scale)))


class CsaTopk(_Operator):
    """DeepSeek-V4 CSA indexer: positions of the ``top_k`` largest of each row's scores, descending
    (src/open_cake_ir/tasks/deepseek_v4/workload.py:188-189)."""
    stem = "csa_topk"

    def __init__(self, index_scores, indices):
        rows, candidates = index_scores.shape
        top_k = indices.shape[1]
        _check("index_scores", index_scores, "fp32", None); _check("indices", indices, "int32", (rows, top_k))
        _no_alias({"indices": indices}, {"index_scores": index_scores, "indices": indices})
        self._create([index_scores, indices], _lib.TopkConfig(rows, candidates, top_k))


class MoePermute(_Operator):
    """Stable sort of the local (token, slot) pairs by expert: counts, offsets, sorted_pairs, inv_perm."""
    stem = "moe_permute"

    def __init__(self, expert_ids, local_expert_offset, counts, offsets, sorted_pairs, inv_perm):
        tokens, top_k = expert_ids.shape
        local_experts = counts.shape[0]
        _check("expert_ids", expert_ids, "int32", None); _check("local_expert_offset", local_expert_offset, "int32", (1,))
        _check("counts", counts, "int32", (local_experts,)); _check("offsets", offsets, "int32", (local_experts + 1,))
        _check("sorted_pairs", sorted_pairs, "int32", (tokens * top_k,)); _check("inv_perm", inv_perm, "int32", (tokens * top_k,))
        cfg = _lib.PermuteConfig(tokens, top_k, local_experts)
        self._create([expert_ids, local_expert_offset, counts, offsets, sorted_pairs, inv_perm], cfg)


MOE_INPUTS = ("routing_logits", "routing_bias", "hidden_states", "hidden_states_scale", "gemm1_weights",
              "gemm1_weights_scale", "gemm2_weights", "gemm2_weights_scale", "local_expert_offset",
              "routed_scaling_factor")


class Fp8Moe(_Operator):
    """Rank-local FP8 block-scaled MoE layer; tensors as in src/open_cake_ir/tasks/solx_fib/moe.py:13-20.

    ``act_mode="fp8"`` requantises the SwiGLU output to one e4m3 term per (row,128) group;
    ``"split"`` keeps a second e4m3 term for the residual, which meets the reference contract's
    tolerance against its unquantised oracle.  With ``external_routing`` the first two inputs
    are ``expert_ids`` int32 [T,top_k] and ``route_weights`` fp32 [T,top_k] instead of logits/bias.
    """
    stem = "moe"

    def __init__(self, inputs: dict, output, *, experts=256, top_k=8, n_group=8, topk_group=4, routing="ds",
                 act_mode="fp8", external_routing=False):
        hidden_states = inputs["hidden_states"]
        tokens, hidden = hidden_states.shape
        local_experts, two_i, _ = inputs["gemm1_weights"].shape
        inter = two_i // 2
        if external_routing:
            _check("expert_ids", inputs["expert_ids"], "int32", (tokens, top_k))
            _check("route_weights", inputs["route_weights"], "fp32", (tokens, top_k))
            first = [inputs["expert_ids"], inputs["route_weights"]]
        else:
            _check("routing_logits", inputs["routing_logits"], "fp32", (tokens, experts))
            _check("routing_bias", inputs["routing_bias"], "bf16", (experts,))
            first = [inputs["routing_logits"], inputs["routing_bias"]]
        _check("hidden_states", hidden_states, "fp8_e4m3", None)
        _check("hidden_states_scale", inputs["hidden_states_scale"], "fp32", (hidden // 128, tokens))
        _check("gemm1_weights", inputs["gemm1_weights"], "fp8_e4m3", (local_experts, 2 * inter, hidden))
        _check("gemm1_weights_scale", inputs["gemm1_weights_scale"], "fp32", (local_experts, 2 * inter // 128, hidden // 128))
        _check("gemm2_weights", inputs["gemm2_weights"], "fp8_e4m3", (local_experts, hidden, inter))
        _check("gemm2_weights_scale", inputs["gemm2_weights_scale"], "fp32", (local_experts, hidden // 128, inter // 128))
        _check("local_expert_offset", inputs["local_expert_offset"], "int32", (1,))
        _check("routed_scaling_factor", inputs["routed_scaling_factor"], "fp32", (1,))
        _check("output", output, "bf16", (tokens, hidden))
        rest = [inputs[n] for n in MOE_INPUTS[2:]]
        everything = {f"in{i}": t for i, t in enumerate(first + rest)}
        everything["output"] = output
        _no_alias({"output": output}, everything)
        cfg = _lib.MoeConfig(tokens, hidden, inter, experts, local_experts, top_k, n_group, topk_group,
                             {"ds": 0, "softmax": 1}[routing], {"fp8": 0, "split": 1}[act_mode], int(external_routing))
        self.config = cfg
        self._create(first + rest + [output], cfg, _lib.workspace_bytes(self.stem, cfg))
        self.tokens, self.top_k, self.local_experts = tokens, top_k, local_experts

    STAGES = ("route_permute_gather", "gemm1_swiglu", "gemm2", "combine")

    def launch_stage(self, stage: int, stream=None) -> None:
        """One part of the layer (see STAGES); the four in order are exactly ``launch``."""
        with torch.cuda.device(self.device):
            code = _lib.library().cake_b200_moe_launch_stage(self.native.handle, stage, _stream(stream))
        if code:
            raise _lib.CakeError("cake_b200_moe_launch_stage", code)

    def intermediate(self, name: str) -> torch.Tensor:
        """Device view of an intermediate in the workspace (expert_ids, route_weights, counts, offsets,
        sorted_pairs, inv_perm, contributions) -- contents are valid after a launch has completed."""
        import ctypes
        which = ["expert_ids", "route_weights", "counts", "offsets", "sorted_pairs", "inv_perm", "contributions"].index(name)
        ptr = ctypes.c_void_p()
        code = _lib.library().cake_b200_moe_intermediate(self.native.handle, which, ctypes.byref(ptr))
        if code:
            raise _lib.CakeError("cake_b200_moe_intermediate", code)
        pairs = self.tokens * self.top_k
        offset = ptr.value - self.workspace.data_ptr()
        if name == "contributions":
            nbytes = pairs * self.config.hidden * 2
            return self.workspace[offset:offset + nbytes].view(torch.bfloat16).view(pairs, self.config.hidden)
        count = {"counts": self.local_experts, "offsets": self.local_experts + 1}.get(name, pairs)
        dtype = torch.float32 if name == "route_weights" else torch.int32
        if not 0 <= offset <= self.workspace.numel() - count * 4:
            raise RuntimeError(f"{name} is not inside the workspace (routing is external)")
        return self.workspace[offset:offset + count * 4].view(dtype)


class GqaPagedDecode(_Operator):
    """Paged GQA decode; tensors as in attention_specs.py:44-84 plus ``kv_last_page_len``."""
    stem = "gqa_decode"

    def __init__(self, q, k_cache, v_cache, kv_indptr, kv_indices, kv_last_page_len, sm_scale, output, lse, *,
                 max_kv_len: int):
        batch, hq, d = q.shape
        pages, page_size, hkv, _ = k_cache.shape
        _check("q", q, "bf16", None); _check("k_cache", k_cache, "bf16", (pages, page_size, hkv, d))
        _check("v_cache", v_cache, "bf16", (pages, page_size, hkv, d)); _check("kv_indptr", kv_indptr, "int32", (batch + 1,))
        _check("kv_indices", kv_indices, "int32", None); _check("kv_last_page_len", kv_last_page_len, "int32", (batch,))
        _check("sm_scale", sm_scale, "fp32", (1,)); _check("output", output, "bf16", (batch, hq, d))
        _check("lse", lse, "fp32", (batch, hq))
        tensors = [q, k_cache, v_cache, kv_indptr, kv_indices, kv_last_page_len, sm_scale, output, lse]
        _no_alias({"output": output, "lse": lse}, {str(i): t for i, t in enumerate(tensors)})
        cfg = _lib.GqaDecodeConfig(batch, hq, hkv, d, page_size, int(max_kv_len))
        self._create(tensors, cfg, _lib.workspace_bytes(self.stem, cfg))


class MlaPagedDecode(_Operator):
    """Paged MLA decode (absorbed); tensors as in attention_specs.py:249-292 plus ``kv_last_page_len``."""
    stem = "mla_decode"

    def __init__(self, q_nope, q_pe, ckv_cache, kpe_cache, kv_indptr, kv_indices, kv_last_page_len, sm_scale, output,
                 lse, *, max_kv_len: int):
        batch, heads, dc = q_nope.shape
        pages, page_size, _ = ckv_cache.shape
        dp = q_pe.shape[2]
        _check("q_nope", q_nope, "bf16", None); _check("q_pe", q_pe, "bf16", (batch, heads, dp))
        _check("ckv_cache", ckv_cache, "bf16", (pages, page_size, dc)); _check("kpe_cache", kpe_cache, "bf16", (pages, page_size, dp))
        _check("kv_indptr", kv_indptr, "int32", (batch + 1,)); _check("kv_indices", kv_indices, "int32", None)
        _check("kv_last_page_len", kv_last_page_len, "int32", (batch,)); _check("sm_scale", sm_scale, "fp32", (1,))
        _check("output", output, "bf16", (batch, heads, dc)); _check("lse", lse, "fp32", (batch, heads))
        tensors = [q_nope, q_pe, ckv_cache, kpe_cache, kv_indptr, kv_indices, kv_last_page_len, sm_scale, output, lse]
        _no_alias({"output": output, "lse": lse}, {str(i): t for i, t in enumerate(tensors)})
        cfg = _lib.MlaDecodeConfig(batch, heads, dc, dp, page_size, int(max_kv_len))
        self._create(tensors, cfg, _lib.workspace_bytes(self.stem, cfg))


class SparseMlaDecode(_Operator):
    """Sparse MLA decode (contracts/workloads/dsa-attention-sparse-mla-decode-v1.json): per query row the cache
    rows named by the non-negative entries of ``sparse_indices`` (token-level row numbers), softmax over them,
    output only; ``sm_scale`` is a number of the contract."""
    stem = "sparse_mla_decode"
    SM_SCALE = 0.1352337788608801

    def __init__(self, q_nope, q_pe, ckv_cache, kpe_cache, sparse_indices, output, *, sm_scale: float = SM_SCALE):
        tokens, heads, dc = q_nope.shape
        pages, page_size, _ = ckv_cache.shape
        dp = q_pe.shape[2]
        top_k = sparse_indices.shape[1]
        _check("q_nope", q_nope, "bf16", None); _check("q_pe", q_pe, "bf16", (tokens, heads, dp))
        _check("ckv_cache", ckv_cache, "bf16", (pages, page_size, dc)); _check("kpe_cache", kpe_cache, "bf16", (pages, page_size, dp))
        _check("sparse_indices", sparse_indices, "int32", (tokens, top_k)); _check("output", output, "bf16", (tokens, heads, dc))
        tensors = [q_nope, q_pe, ckv_cache, kpe_cache, sparse_indices, output]
        _no_alias({"output": output}, {str(i): t for i, t in enumerate(tensors)})
        cfg = _lib.SparseMlaDecodeConfig(tokens, pages * page_size, heads, dc, dp, top_k, float(sm_scale))
        self._create(tensors, cfg, _lib.workspace_bytes(self.stem, cfg))


class GqaCausalPrefill(_Operator):
    """Causal GQA prefill over a paged (``kv_indices`` given) or ragged (``kv_indices`` None; ``k``/``v`` are
    ``[total_kv, Hkv, D]``) KV store; tensors as in attention_specs.py:85-248 plus the optional ``kv_last_page_len``.
    ``nan_for_masked``: a row of a non-empty segment that sees no KV row is NaN (the reference's ragged tasks) instead of zero."""
    stem = "gqa_prefill"

    def __init__(self, q, k, v, qo_indptr, kv_indptr, kv_indices, kv_last_page_len, sm_scale, output, lse, *, max_kv_len: int,
                 nan_for_masked: bool | None = None):
        total_q, hq, d = q.shape
        ragged = kv_indices is None
        segments = qo_indptr.shape[0] - 1
        if ragged:
            total_kv, hkv, _ = k.shape
            page_size = 1
            _check("k", k, "bf16", (total_kv, hkv, d)); _check("v", v, "bf16", (total_kv, hkv, d))
        else:
            pages, page_size, hkv, _ = k.shape
            _check("k_cache", k, "bf16", (pages, page_size, hkv, d)); _check("v_cache", v, "bf16", (pages, page_size, hkv, d))
            _check("kv_indices", kv_indices, "int32", None)
        _check("q", q, "bf16", None); _check("qo_indptr", qo_indptr, "int32", (segments + 1,))
        _check("kv_indptr", kv_indptr, "int32", (segments + 1,)); _check("sm_scale", sm_scale, "fp32", (1,))
        _check("output", output, "bf16", (total_q, hq, d)); _check("lse", lse, "fp32", (total_q, hq))
        if kv_last_page_len is not None:
            _check("kv_last_page_len", kv_last_page_len, "int32", (segments,))
        present = [t for t in (q, k, v, qo_indptr, kv_indptr, kv_indices, kv_last_page_len, sm_scale, output, lse) if t is not None]
        _no_alias({"output": output, "lse": lse}, {str(i): t for i, t in enumerate(present)})
        nan = ragged if nan_for_masked is None else bool(nan_for_masked)
        cfg = _lib.GqaPrefillConfig(total_q, segments, hq, hkv, d, page_size, int(ragged), int(nan), int(max_kv_len))
        self._create_with_optional([q, k, v, qo_indptr, kv_indptr, kv_indices, kv_last_page_len, sm_scale, output, lse], cfg,
                                   _lib.workspace_bytes(self.stem, cfg))


class MlaCausalPrefill(_Operator):
    """Causal MLA prefill over a paged latent cache; tensors as in attention_specs.py:293-338 plus the optional
    ``kv_last_page_len``.  A row of a non-empty segment that sees no KV row is NaN (attention.py:47)."""
    stem = "mla_prefill"

    def __init__(self, q_nope, q_pe, ckv_cache, kpe_cache, qo_indptr, kv_indptr, kv_indices, kv_last_page_len, sm_scale, output,
                 lse, *, max_kv_len: int, nan_for_masked: bool = True):
        total_q, heads, dc = q_nope.shape
        pages, page_size, _ = ckv_cache.shape
        dp = q_pe.shape[2]
        segments = qo_indptr.shape[0] - 1
        _check("q_nope", q_nope, "bf16", None); _check("q_pe", q_pe, "bf16", (total_q, heads, dp))
        _check("ckv_cache", ckv_cache, "bf16", (pages, page_size, dc)); _check("kpe_cache", kpe_cache, "bf16", (pages, page_size, dp))
        _check("qo_indptr", qo_indptr, "int32", (segments + 1,)); _check("kv_indptr", kv_indptr, "int32", (segments + 1,))
        _check("kv_indices", kv_indices, "int32", None); _check("sm_scale", sm_scale, "fp32", (1,))
        _check("output", output, "bf16", (total_q, heads, dc)); _check("lse", lse, "fp32", (total_q, heads))
        if kv_last_page_len is not None:
            _check("kv_last_page_len", kv_last_page_len, "int32", (segments,))
        present = [t for t in (q_nope, q_pe, ckv_cache, kpe_cache, qo_indptr, kv_indptr, kv_indices, kv_last_page_len, sm_scale,
                               output, lse) if t is not None]
        _no_alias({"output": output, "lse": lse}, {str(i): t for i, t in enumerate(present)})
        cfg = _lib.MlaPrefillConfig(total_q, segments, heads, dc, dp, page_size, int(nan_for_masked), int(max_kv_len))
        self._create_with_optional([q_nope, q_pe, ckv_cache, kpe_cache, qo_indptr, kv_indptr, kv_indices, kv_last_page_len,
                                    sm_scale, output, lse], cfg, _lib.workspace_bytes(self.stem, cfg))


# ---- functional forms: allocate the outputs, run once on the current stream ------------------
def rmsnorm(x, weight, epsilon, residual=None):
    out = torch.empty_like(x)
    RmsNorm(x, weight, out, epsilon, residual).launch()
    return out


def add_rmsnorm(delta, residual, weight, epsilon: float = 1e-6):
    out, residual_out = torch.empty_like(delta), torch.empty_like(delta)
    AddRmsNorm(delta, residual, weight, out, residual_out, epsilon).launch()
    return out, residual_out


def block_scaled_gemm(a, sfa, b, sfb):
    c = torch.empty((a.shape[0], b.shape[0]), dtype=torch.bfloat16, device=a.device)
    op = BlockScaledGemm(a, sfa, b, sfb, c)
    op.launch()
    if op.status():
        raise RuntimeError("block_scaled_gemm: a device-side wait ran out")
    return c


def moe_routing(routing_logits, routing_bias, routed_scaling_factor, *, top_k=8, n_group=8, topk_group=4, mode="ds"):
    tokens = routing_logits.shape[0]
    ids = torch.empty((tokens, top_k), dtype=torch.int32, device=routing_logits.device)
    weights = torch.empty((tokens, top_k), dtype=torch.float32, device=routing_logits.device)
    MoeRouting(routing_logits, routing_bias, routed_scaling_factor, ids, weights, top_k=top_k, n_group=n_group,
               topk_group=topk_group, mode=mode).launch()
    return ids, weights


def v4_moe_gate(router_logits, selection_bias, *, top_k=6, route_scale=2.5):
    tokens = router_logits.shape[0]
    weights = torch.empty((tokens, top_k), dtype=torch.float32, device=router_logits.device)
    ids = torch.empty((tokens, top_k), dtype=torch.int32, device=router_logits.device)
    V4MoeGate(router_logits, selection_bias, weights, ids, top_k=top_k, route_scale=route_scale).launch()
    return weights, ids


def csa_topk(index_scores, top_k=1024):
    indices = torch.empty((index_scores.shape[0], top_k), dtype=torch.int32, device=index_scores.device)
    CsaTopk(index_scores, indices).launch()
    return indices


def moe_permute(expert_ids, local_expert_offset, local_experts: int):
    pairs = expert_ids.numel()
    dev = expert_ids.device
    counts = torch.empty(local_experts, dtype=torch.int32, device=dev)
    offsets = torch.empty(local_experts + 1, dtype=torch.int32, device=dev)
    sorted_pairs = torch.full((pairs,), -1, dtype=torch.int32, device=dev)
    inv_perm = torch.full((pairs,), -2, dtype=torch.int32, device=dev)
    MoePermute(expert_ids, local_expert_offset, counts, offsets, sorted_pairs, inv_perm).launch()
    return {"counts": counts, "offsets": offsets, "sorted_pairs": sorted_pairs, "inv_perm": inv_perm}


def fp8_moe(inputs: dict, **options):
    hidden_states = inputs["hidden_states"]
    output = torch.empty(hidden_states.shape, dtype=torch.bfloat16, device=hidden_states.device)
    op = Fp8Moe(inputs, output, **options)
    op.launch()
    if op.status():
        raise RuntimeError("fp8_moe: a device-side wait ran out")
    return output


def _default_last_page_len(kv_indptr, page_size):
    pages = kv_indptr[1:] - kv_indptr[:-1]
    return torch.where(pages > 0, torch.full_like(pages, page_size), torch.zeros_like(pages)).to(torch.int32)


def gqa_paged_decode(q, k_cache, v_cache, kv_indptr, kv_indices, sm_scale, kv_last_page_len=None, max_kv_len=None):
    page_size = k_cache.shape[1]
    if kv_last_page_len is None:
        kv_last_page_len = _default_last_page_len(kv_indptr, page_size)
    if max_kv_len is None:
        max_kv_len = int((kv_indptr[1:] - kv_indptr[:-1]).max().item()) * page_size if q.shape[0] else 0
    output = torch.empty_like(q)
    lse = torch.empty(q.shape[:2], dtype=torch.float32, device=q.device)
    GqaPagedDecode(q, k_cache, v_cache, kv_indptr, kv_indices, kv_last_page_len, sm_scale, output, lse,
                   max_kv_len=max_kv_len).launch()
    return output, lse


def mla_paged_decode(q_nope, q_pe, ckv_cache, kpe_cache, kv_indptr, kv_indices, sm_scale, kv_last_page_len=None,
                     max_kv_len=None):
    page_size = ckv_cache.shape[1]
    if kv_last_page_len is None:
        kv_last_page_len = _default_last_page_len(kv_indptr, page_size)
    if max_kv_len is None:
        max_kv_len = int((kv_indptr[1:] - kv_indptr[:-1]).max().item()) * page_size if q_nope.shape[0] else 0
    output = torch.empty_like(q_nope)
    lse = torch.empty(q_nope.shape[:2], dtype=torch.float32, device=q_nope.device)
    MlaPagedDecode(q_nope, q_pe, ckv_cache, kpe_cache, kv_indptr, kv_indices, kv_last_page_len, sm_scale, output, lse,
                   max_kv_len=max_kv_len).launch()
    return output, lse


def sparse_mla_decode(q_nope, q_pe, ckv_cache, kpe_cache, sparse_indices, sm_scale: float = SparseMlaDecode.SM_SCALE):
    output = torch.empty_like(q_nope)
    op = SparseMlaDecode(q_nope, q_pe, ckv_cache, kpe_cache, sparse_indices, output, sm_scale=sm_scale)
    op.launch()
    if op.status():
        raise RuntimeError("sparse_mla_decode: a device-side wait ran out")
    return output


def gqa_causal_prefill(q, k, v, qo_indptr, kv_indptr, sm_scale, kv_indices=None, kv_last_page_len=None, max_kv_len=None,
                       nan_for_masked=None):
    page_size = 1 if kv_indices is None else k.shape[1]
    if max_kv_len is None:
        max_kv_len = int((kv_indptr[1:] - kv_indptr[:-1]).max().item()) * page_size
    output = torch.empty_like(q)
    lse = torch.empty(q.shape[:2], dtype=torch.float32, device=q.device)
    GqaCausalPrefill(q, k, v, qo_indptr, kv_indptr, kv_indices, kv_last_page_len, sm_scale, output, lse, max_kv_len=max_kv_len,
                     nan_for_masked=nan_for_masked).launch()
    return output, lse


def mla_causal_prefill(q_nope, q_pe, ckv_cache, kpe_cache, qo_indptr, kv_indptr, kv_indices, sm_scale, kv_last_page_len=None,
                       max_kv_len=None, nan_for_masked=True):
    if max_kv_len is None:
        max_kv_len = int((kv_indptr[1:] - kv_indptr[:-1]).max().item()) * ckv_cache.shape[1]
    output = torch.empty_like(q_nope)
    lse = torch.empty(q_nope.shape[:2], dtype=torch.float32, device=q_nope.device)
    MlaCausalPrefill(q_nope, q_pe, ckv_cache, kpe_cache, qo_indptr, kv_indptr, kv_indices, kv_last_page_len, sm_scale, output, lse,
                     max_kv_len=max_kv_len, nan_for_masked=nan_for_masked).launch()
    return output, lse
