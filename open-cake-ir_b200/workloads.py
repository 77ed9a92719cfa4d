"""Seeded synthetic inputs at serving shapes for the operators of this target.

Shapes, value distributions and layouts are those of the five configurations the build is
measured on (RMSNorm 4096x4096; block-scaled FP8 GEMM 8192x4096x7168; paged GQA decode batch 64;
paged MLA decode batch 32; DeepSeek-V3 FP8 MoE layer with 4096 tokens).  They stand in for the
FlashInfer-Bench / SOL-ExecBench captures the reference's contracts name, which are not
distributed with it: the reference too takes only the mathematical definition from that pack
and generates its own inputs (src/open_cake_ir/tasks/solx_fib/moe.py:68-69, attention.py:71-72).

One ``torch.Generator`` per tensor, seed = BASE_SEED + 1000*config + tensor index.  Values are
drawn on ``gen_device`` ("cpu" reproduces the same bytes everywhere; "cuda" is for the tensors
too large to draw on the host in reasonable time) and returned on ``device``.  Quantisation to
e4m3 with amax/448 block scales is part of input materialisation, never of a candidate kernel
(moe.py:97 says the same of the reference's inputs).
"""
from __future__ import annotations

import math

import torch

BASE_SEED = 20261125
E4M3_MAX = 448.0
CONFIG_INDEX = {"rmsnorm": 0, "block_scaled_gemm": 1, "gqa_paged_decode": 2, "mla_paged_decode": 3, "fp8_moe": 4}


def _gen(config: str, index: int, gen_device: str, salt: int = 0) -> torch.Generator:
    g = torch.Generator(device=gen_device)
    g.manual_seed(BASE_SEED + 1000 * CONFIG_INDEX[config] + index + 100000 * salt)
    return g


def _randn(shape, g, gen_device, mean=0.0, std=1.0):
    return torch.randn(shape, generator=g, device=gen_device, dtype=torch.float32) * std + mean


def quantize_rows_1x128(x: torch.Tensor):
    """fp32 [R, K] -> (e4m3 [R, K], fp32 scales [K/128, R]); scale = amax/448 per (row, 128 group)."""
    rows, k = x.shape
    g = x.reshape(rows, k // 128, 128)
    amax = g.abs().amax(dim=2)
    scale = torch.where(amax > 0, amax / E4M3_MAX, torch.ones_like(amax))
    q = (g / scale[:, :, None]).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn)
    return q.reshape(rows, k), scale.t().contiguous()


def quantize_blocks_128x128(w: torch.Tensor):
    """fp32 [N, K] -> (e4m3 [N, K], fp32 scales [N/128, K/128]); scale = amax/448 per 128x128 block."""
    n, k = w.shape
    g = w.reshape(n // 128, 128, k // 128, 128)
    amax = g.abs().amax(dim=(1, 3))
    scale = torch.where(amax > 0, amax / E4M3_MAX, torch.ones_like(amax))
    q = (g / scale[:, None, :, None]).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn)
    return q.reshape(n, k), scale.contiguous()


def rmsnorm_inputs(rows=4096, width=4096, *, device="cuda", gen_device="cpu", salt=0):
    """x ~ N(0,1) bf16 [rows,width]; weight ~ N(1,0.1) bf16 [width]; eps 1e-6."""
    x = _randn((rows, width), _gen("rmsnorm", 0, gen_device, salt), gen_device).to(torch.bfloat16)
    w = _randn((width,), _gen("rmsnorm", 1, gen_device, salt), gen_device, 1.0, 0.1).to(torch.bfloat16)
    return {"x": x.to(device), "weight": w.to(device)}, {"epsilon": 1e-6}


def block_scaled_gemm_inputs(m=8192, n=4096, k=7168, *, device="cuda", gen_device="cpu", salt=0):
    """A, B ~ N(0,1) quantised to e4m3 with amax/448 scales: A per 1x128 row group ([K/128,M]),
    B ([N,K]) per 128x128 block ([N/128,K/128])."""
    a, sfa = quantize_rows_1x128(_randn((m, k), _gen("block_scaled_gemm", 0, gen_device, salt), gen_device))
    b, sfb = quantize_blocks_128x128(_randn((n, k), _gen("block_scaled_gemm", 1, gen_device, salt), gen_device))
    return {"a": a.to(device), "sfa": sfa.to(device), "b": b.to(device), "sfb": sfb.to(device)}


def _paged_layout(batch, page_size, len_range, pool_pages, g):
    """Sequence lengths uniform in len_range; pages = the first sum(ceil(len/P)) entries of a seeded
    permutation of the pool; kv_indptr counts pages."""
    lo, hi = len_range
    lens = torch.randint(lo, hi + 1, (batch,), generator=g, device="cpu") if batch else torch.zeros(0, dtype=torch.int64)
    pages = (lens + page_size - 1) // page_size
    indptr = torch.zeros(batch + 1, dtype=torch.int32)
    indptr[1:] = torch.cumsum(pages, 0).int()
    total = int(indptr[-1])
    if total > pool_pages:
        raise ValueError("page pool too small for the drawn lengths")
    perm = torch.randperm(pool_pages, generator=g, device="cpu")[:total].int()
    last = torch.where(pages > 0, lens - (pages - 1) * page_size, torch.zeros_like(lens)).int()
    return lens, indptr, perm, last


def gqa_decode_inputs(batch=64, hq=32, hkv=8, d=128, page_size=16, len_range=(512, 4096), pool_pages=20000, *,
                      device="cuda", gen_device="cpu", salt=0):
    c = "gqa_paged_decode"
    lens, indptr, indices, last = _paged_layout(batch, page_size, len_range, pool_pages, _gen(c, 3, "cpu", salt))
    q = _randn((batch, hq, d), _gen(c, 0, gen_device, salt), gen_device).to(torch.bfloat16)
    k = _randn((pool_pages, page_size, hkv, d), _gen(c, 1, gen_device, salt), gen_device).to(torch.bfloat16)
    v = _randn((pool_pages, page_size, hkv, d), _gen(c, 2, gen_device, salt), gen_device).to(torch.bfloat16)
    inputs = {"q": q, "k_cache": k, "v_cache": v, "kv_indptr": indptr, "kv_indices": indices,
              "kv_last_page_len": last, "sm_scale": torch.tensor([1.0 / math.sqrt(d)], dtype=torch.float32)}
    return {n: t.to(device) for n, t in inputs.items()}, {"kv_lens": lens, "max_kv_len": len_range[1]}


def mla_decode_inputs(batch=32, heads=128, page_size=64, len_range=(1024, 8192), pool_pages=None, *,
                      device="cuda", gen_device="cpu", salt=0):
    c = "mla_paged_decode"
    if pool_pages is None:
        pool_pages = batch * ((len_range[1] + page_size - 1) // page_size) + 64
    lens, indptr, indices, last = _paged_layout(batch, page_size, len_range, pool_pages, _gen(c, 4, "cpu", salt))
    qn = _randn((batch, heads, 512), _gen(c, 0, gen_device, salt), gen_device).to(torch.bfloat16)
    qp = _randn((batch, heads, 64), _gen(c, 1, gen_device, salt), gen_device).to(torch.bfloat16)
    ckv = _randn((pool_pages, page_size, 512), _gen(c, 2, gen_device, salt), gen_device).to(torch.bfloat16)
    kpe = _randn((pool_pages, page_size, 64), _gen(c, 3, gen_device, salt), gen_device).to(torch.bfloat16)
    inputs = {"q_nope": qn, "q_pe": qp, "ckv_cache": ckv, "kpe_cache": kpe, "kv_indptr": indptr, "kv_indices": indices,
              "kv_last_page_len": last, "sm_scale": torch.tensor([1.0 / math.sqrt(192.0)], dtype=torch.float32)}
    return {n: t.to(device) for n, t in inputs.items()}, {"kv_lens": lens, "max_kv_len": len_range[1]}


def moe_inputs(tokens=4096, hidden=7168, inter=2048, experts=256, local_experts=256, local_offset=0, *, routing="softmax",
               device="cuda", gen_device="cpu", salt=0, first_token=0, total_tokens=None):
    """DeepSeek-V3-shaped layer.  hidden ~ N(0,1) -> e4m3 + 1x128 scales [H/128,T]; weights ~ N(0,1)/sqrt(K)
    -> e4m3 + 128x128 scales, drawn expert by expert with seed index 10+global expert id so that a rank
    holding experts [local_offset, +local_experts) draws the same bytes as the single-GPU layer; logits ~ N(0,1);
    bias 0 for softmax routing, U(0,0.015) bf16 for DeepSeek routing (moe.py:108); factor 2.5.
    ``first_token``/``total_tokens`` select a token slice of the same global draw (expert parallelism)."""
    c = "fp8_moe"
    total = tokens if total_tokens is None else total_tokens
    sl = slice(first_token, first_token + tokens)
    logits = _randn((total, experts), _gen(c, 0, gen_device, salt), gen_device)[sl].contiguous()
    if routing == "softmax":
        bias = torch.zeros(experts, dtype=torch.bfloat16, device=gen_device)
    else:
        bias = (torch.rand(experts, generator=_gen(c, 1, gen_device, salt), device=gen_device) * 0.015).to(torch.bfloat16)
    h, hs = quantize_rows_1x128(_randn((total, hidden), _gen(c, 2, gen_device, salt), gen_device)[sl].contiguous())
    w13 = torch.empty((local_experts, 2 * inter, hidden), dtype=torch.float8_e4m3fn, device=device)
    s13 = torch.empty((local_experts, 2 * inter // 128, hidden // 128), dtype=torch.float32, device=device)
    w2 = torch.empty((local_experts, hidden, inter), dtype=torch.float8_e4m3fn, device=device)
    s2 = torch.empty((local_experts, hidden // 128, inter // 128), dtype=torch.float32, device=device)
    for e in range(local_experts):
        q13, sc13, q2, sc2 = moe_expert_weights(local_offset + e, hidden, inter, gen_device=gen_device, salt=salt)
        w13[e].copy_(q13); s13[e].copy_(sc13)
        w2[e].copy_(q2); s2[e].copy_(sc2)
    inputs = {"routing_logits": logits, "routing_bias": bias, "hidden_states": h, "hidden_states_scale": hs,
              "gemm1_weights": w13, "gemm1_weights_scale": s13, "gemm2_weights": w2, "gemm2_weights_scale": s2,
              "local_expert_offset": torch.tensor([local_offset], dtype=torch.int32),
              "routed_scaling_factor": torch.tensor([2.5], dtype=torch.float32)}
    return {n: t.to(device) for n, t in inputs.items()}


def moe_expert_weights(expert: int, hidden=7168, inter=2048, *, gen_device="cpu", salt=0):
    """The weights of ONE global expert id as ``moe_inputs`` draws them: (w13 e4m3 [2I,H], scales [2I/128,H/128],
    w2 e4m3 [H,I], scales [H/128,I/128]).  Any rank can regenerate any expert, whoever owns it."""
    g = _gen("fp8_moe", 10 + expert, gen_device, salt)
    q13, s13 = quantize_blocks_128x128(_randn((2 * inter, hidden), g, gen_device, 0.0, 1.0 / math.sqrt(hidden)))
    q2, s2 = quantize_blocks_128x128(_randn((hidden, inter), g, gen_device, 0.0, 1.0 / math.sqrt(inter)))
    return q13, s13, q2, s2


def moe_flops(tokens, hidden, inter, top_k=8) -> int:
    """2*T*K*(H*2I + I*H): the two grouped GEMMs of every routed (token, expert) pair."""
    return 2 * tokens * top_k * (hidden * 2 * inter + inter * hidden)


def moe_weight_bytes(local_experts, hidden, inter) -> int:
    return local_experts * (2 * inter * hidden + hidden * inter)
