"""Paged GQA / MLA decode oracle (test infrastructure; see the package docstring).

Follows src/open_cake_ir/tasks/solx_fib/attention.py:132-183 (``reference_tensors``), decode
branch: for every sequence b and query head h, ``logits = (K . q) * sm_scale`` in float64 (for
MLA ``ckv . q_nope + kpe . q_pe``, attention.py:175-177), ``lse = logsumexp(logits)/ln 2``
(base 2, fp32), ``out = bf16(softmax(logits) @ V)`` with V = ckv for MLA (absorbed form,
attention.py:164-165); an empty sequence leaves out = 0 and lse = -inf (attention.py:157-162);
GQA head h reads KV head ``h // (heads // kv_heads)`` (attention.py:179).

Generalisation the reference does not hold: page_size > 1.  The reference reads slot 0 of each
page (attention.py:165-168, page_size 1).  Here ``kv_indptr`` counts pages, ``kv_indices``
holds page ids and ``kv_last_page_len[b]`` the tokens used in the last page; token j of
sequence b lives at ``cache[kv_indices[kv_indptr[b] + j // P], j % P]``.  With P = 1 and
last_page_len = 1 this is the reference addressing.
"""
from __future__ import annotations

import math

import torch


def sequence_length(kv_indptr, kv_last_page_len, b: int, page_size: int) -> int:
    pages = int(kv_indptr[b + 1]) - int(kv_indptr[b])
    return 0 if pages <= 0 else (pages - 1) * page_size + int(kv_last_page_len[b])


def _gather_rows(cache: torch.Tensor, kv_indptr, kv_indices, kv_last_page_len, b, page_size):
    length = sequence_length(kv_indptr, kv_last_page_len, b, page_size)
    start = int(kv_indptr[b])
    j = torch.arange(length)
    pages = kv_indices[start + j // page_size].long()
    return cache[pages, j % page_size]


def paged_decode_reference(inputs: dict, *, mla: bool, page_size: int = 1,
                           per_head_loop: bool = True):
    """inputs: q | (q_nope, q_pe), k_cache & v_cache | (ckv_cache, kpe_cache), kv_indptr,
    kv_indices, sm_scale and optionally kv_last_page_len (defaults to a full last page).
    ``per_head_loop=True`` evaluates head by head with exactly the reference's operations
    (bit-identical on its cases); False contracts all heads of a sequence at once (same
    mathematics, different float64 summation order) for serving-size inputs."""
    q = inputs["q_nope"] if mla else inputs["q"]
    count, heads, _ = q.shape
    kv_indptr = inputs["kv_indptr"]
    last = inputs.get("kv_last_page_len")
    if last is None:
        last = torch.full((count,), page_size, dtype=torch.int32)
    width = 512 if mla else q.shape[2]
    if mla:
        width = inputs["ckv_cache"].shape[-1]
    result = torch.zeros((count, heads, width), dtype=torch.bfloat16)
    lse = torch.full((count, heads), -float("inf"), dtype=torch.float32)
    scale = float(inputs["sm_scale"][0])
    for b in range(count):
        if sequence_length(kv_indptr, last, b, page_size) == 0:
            continue
        args = (kv_indptr, inputs["kv_indices"], last, b, page_size)
        if mla:
            keys = _gather_rows(inputs["ckv_cache"], *args).double()
            positions = _gather_rows(inputs["kpe_cache"], *args).double()
            values = keys
        else:
            keys = _gather_rows(inputs["k_cache"], *args).double()
            values = _gather_rows(inputs["v_cache"], *args).double()
            group = heads // keys.shape[1]
        if per_head_loop:
            for h in range(heads):
                if mla:
                    logits = (keys @ inputs["q_nope"][b, h].double()
                              + positions @ inputs["q_pe"][b, h].double()) * scale
                    vals = values
                else:
                    kh = h // group
                    logits = (keys[:, kh] @ q[b, h].double()) * scale
                    vals = values[:, kh]
                lse[b, h] = torch.logsumexp(logits, 0) / math.log(2)
                result[b, h] = (torch.softmax(logits, 0) @ vals).to(torch.bfloat16)
        else:
            if mla:
                logits = (keys @ inputs["q_nope"][b].double().T
                          + positions @ inputs["q_pe"][b].double().T) * scale       # [L, heads]
                probs = torch.softmax(logits, 0)
                out = probs.T @ values                                              # [heads, 512]
            else:
                kv_heads = keys.shape[1]
                qb = q[b].double().reshape(kv_heads, group, -1)                      # [kvh, g, d]
                logits = torch.einsum("lkd,kgd->lkg", keys, qb) * scale             # [L, kvh, g]
                probs = torch.softmax(logits, 0)
                out = torch.einsum("lkg,lkd->kgd", probs, values).reshape(heads, -1)
                logits = logits.reshape(logits.shape[0], heads)
            lse[b] = (torch.logsumexp(logits, 0) / math.log(2)).float()
            result[b] = out.to(torch.bfloat16)
    return {"output": result, "lse": lse}


# --- the reference's input materialiser, restated (attention.py:101-129) ------------------
CASES = ("primary", "zeros", "permuted", "scaled", "segmented")
DECODE_TASKS = {
    # task: (mla, heads, kv_heads, captured axes, captured scale)   attention_specs.py:3-84, :249-292
    "gqa_kv4": (False, 32, 4, dict(batch_size=1, num_pages=8, len_indptr=2, num_kv_indices=7),
                0.0883883461356163),
    "gqa_kv8": (False, 32, 8, dict(batch_size=1, num_pages=9316, len_indptr=2, num_kv_indices=73),
                0.08838834764831843),
    "mla_h16": (True, 16, 1, dict(batch_size=1, num_pages=989669, len_indptr=2, num_kv_indices=8),
                0.1352337747812271),
}
BOUNDARY_AXES = dict(len_indptr=3, batch_size=2, num_pages=11, num_kv_indices=5)  # attention.py:16-28


def materialize_reference_case(task: str, variant: str, case_id: str) -> dict[str, torch.Tensor]:
    """Inputs of one reference decode case: one generator seeded 2801+case index draws every
    bf16 input in ABI order as ``rand-0.5``; indptr splits the kv entries evenly over the batch
    (``segmented`` empties the first sequence); page ids are ``(3i+1) mod pages`` (reversed for
    ``permuted``); ``scaled`` multiplies the captured softmax scale by 1.75; ``zeros`` zeroes q."""
    mla, heads, kv_heads, axes, scale = DECODE_TASKS[task]
    axes = dict(axes) if variant == "captured" else dict(BOUNDARY_AXES)
    batch = axes["len_indptr"] - 1
    kvcount = axes["num_kv_indices"]
    pages = axes["num_pages"]
    g = torch.Generator(device="cpu").manual_seed(2801 + CASES.index(case_id))
    if mla:
        shapes = {"q_nope": (axes["batch_size"], heads, 512), "q_pe": (axes["batch_size"], heads, 64),
                  "ckv_cache": (pages, 1, 512), "kpe_cache": (pages, 1, 64)}
    else:
        shapes = {"q": (axes["batch_size"], heads, 128), "k_cache": (pages, 1, kv_heads, 128),
                  "v_cache": (pages, 1, kv_heads, 128)}
    inputs = {}
    for name, shape in shapes.items():
        inputs[name] = (torch.rand(shape, generator=g, dtype=torch.float32) - 0.5).to(torch.bfloat16)
    kptr = [i * kvcount // batch for i in range(batch + 1)]
    if case_id == "segmented" and batch > 1:
        kptr[1] = 0
    inputs["kv_indptr"] = torch.tensor(kptr, dtype=torch.int32)
    ids = (torch.arange(kvcount, dtype=torch.int64) * 3 + 1) % pages
    if case_id == "permuted":
        ids = ids.flip(0)
    inputs["kv_indices"] = ids.to(torch.int32)
    inputs["sm_scale"] = torch.tensor([scale * (1.75 if case_id == "scaled" else 1.0)], dtype=torch.float32)
    if case_id == "zeros":
        for name in ("q", "q_nope", "q_pe"):
            if name in inputs:
                inputs[name].zero_()
    return inputs


def sparse_mla_decode_reference(inputs: dict, sm_scale: float):
    """Sparse MLA decode as the contract states it (contracts/workloads/dsa-attention-sparse-mla-decode-v1.json,
    ``semantics.definition``; validator src/open_cake_ir/tasks/dsa/contract.py:5-78): for each query row and head
    gather the cache rows named by the non-negative token-level ``sparse_indices``, logits =
    (q_nope . ckv + q_pe . kpe) * sm_scale, softmax over the present entries, times the ckv rows; no present entry
    gives a row of zeros.  PARITY UNPINNED: the reference holds no executable oracle and no golden vectors for this
    operator (its baseline is a black box outside the checkout); this restates the definition in fp64, and reduces
    to ``paged_decode_reference`` (which IS pinned) when the list names a sequence's rows in order."""
    q_nope, q_pe = inputs["q_nope"], inputs["q_pe"]
    ckv = inputs["ckv_cache"].reshape(-1, inputs["ckv_cache"].shape[-1]).double()
    kpe = inputs["kpe_cache"].reshape(-1, inputs["kpe_cache"].shape[-1]).double()
    tokens, heads, width = q_nope.shape
    out = torch.zeros((tokens, heads, width), dtype=torch.bfloat16)
    scale = float(torch.tensor(sm_scale, dtype=torch.float32))      # the fp32 number a device receives
    for t in range(tokens):
        idx = inputs["sparse_indices"][t].long()
        idx = idx[idx >= 0]
        if idx.numel() == 0:
            continue
        keys, positions = ckv[idx], kpe[idx]
        logits = (keys @ q_nope[t].double().T + positions @ q_pe[t].double().T) * scale        # [L, heads]
        out[t] = (torch.softmax(logits, 0).T @ keys).to(torch.bfloat16)
    return out


# --- causal prefill --------------------------------------------------------------------------
PREFILL_TASKS = {
    # task: (mla, paged, heads, kv_heads, captured axes, captured scale)   attention_specs.py:85-248, :293-338
    "gqa_paged_prefill_kv4": (False, True, 32, 4, dict(len_indptr=2, total_q=1, num_kv_indices=33, num_pages=50), 0.08838834764831843),
    "gqa_paged_prefill_kv8": (False, True, 32, 8, dict(len_indptr=2, total_q=34, num_kv_indices=1, num_pages=2), 0.08838834764831843),
    "gqa_ragged_prefill_kv4": (False, False, 32, 4, dict(len_indptr=2, total_q=6, total_kv=6), 0.0883883461356163),
    "gqa_ragged_prefill_kv8": (False, False, 32, 8, dict(len_indptr=2, total_q=7, total_kv=7), 0.0883883461356163),
    "mla_paged_prefill_h16": (True, True, 16, 1, dict(len_indptr=2, total_q=33, num_kv_indices=34, num_pages=989669), 0.1352337747812271),
}


def prefill_nan_rule(task: str) -> bool:
    """A fully masked row of a non-empty segment is NaN for the MLA and the ragged tasks, zero for paged GQA
    (attention.py:47: ``nan_masked = not decode and (mla or not paged)``)."""
    mla, paged = PREFILL_TASKS[task][:2]
    return mla or not paged


def causal_prefill_reference(inputs: dict, *, mla: bool, paged: bool, page_size: int = 1, nan_for_masked: bool,
                             per_head_loop: bool = True):
    """The prefill branches of attention.py:132-183, with the page size and the last page's fill generalised
    exactly as for decode.  Segment b: query rows [qo_indptr[b], qo_indptr[b+1]), KV rows of its pages (paged) or
    rows [kv_indptr[b], kv_indptr[b+1]) of ``k``/``v`` (ragged); query row qi sees its first
    ``min(kv_len, qi - qs + 1 + kv_len - q_len)`` KV rows (:170); a row that sees none is NaN or zero by the task's
    rule with lse -inf (:171-173); segments without query or KV rows are skipped (:160-162)."""
    q = inputs["q_nope"] if mla else inputs["q"]
    count, heads, _ = q.shape
    qptr, kvptr = inputs["qo_indptr"].tolist(), inputs["kv_indptr"].tolist()
    last = inputs.get("kv_last_page_len")
    width = inputs["ckv_cache"].shape[-1] if mla else q.shape[2]
    result = torch.zeros((count, heads, width), dtype=torch.bfloat16)
    lse = torch.full((count, heads), -float("inf"), dtype=torch.float32)
    scale = float(inputs["sm_scale"][0])
    for b in range(len(kvptr) - 1):
        qs, qe = qptr[b:b + 2]
        ks, ke = kvptr[b:b + 2]
        if qs == qe or ks == ke:
            continue
        if paged:
            full_last = torch.full((len(kvptr) - 1,), page_size, dtype=torch.int32) if last is None else last
            args = (inputs["kv_indptr"], inputs["kv_indices"], full_last, b, page_size)
            if mla:
                keys = _gather_rows(inputs["ckv_cache"], *args).double()
                positions = _gather_rows(inputs["kpe_cache"], *args).double()
                values = keys
            else:
                keys = _gather_rows(inputs["k_cache"], *args).double()
                values = _gather_rows(inputs["v_cache"], *args).double()
        else:
            keys, values = inputs["k"][ks:ke].double(), inputs["v"][ks:ke].double()
        kv_len = keys.shape[0]
        if kv_len == 0:
            continue
        for qi in range(qs, qe):
            valid = min(kv_len, qi - qs + 1 + kv_len - (qe - qs))
            if valid <= 0:
                if nan_for_masked:
                    result[qi].fill_(float("nan"))
                continue
            if per_head_loop:
                for h in range(heads):
                    if mla:
                        logits = (keys[:valid] @ inputs["q_nope"][qi, h].double() + positions[:valid] @ inputs["q_pe"][qi, h].double()) * scale
                        vals = values[:valid]
                    else:
                        kh = h // (heads // keys.shape[1])
                        logits = (keys[:valid, kh] @ q[qi, h].double()) * scale
                        vals = values[:valid, kh]
                    lse[qi, h] = torch.logsumexp(logits, 0) / math.log(2)
                    result[qi, h] = (torch.softmax(logits, 0) @ vals).to(torch.bfloat16)
            else:
                if mla:
                    logits = (keys[:valid] @ inputs["q_nope"][qi].double().T + positions[:valid] @ inputs["q_pe"][qi].double().T) * scale
                    out = torch.softmax(logits, 0).T @ values[:valid]
                else:
                    kv_heads = keys.shape[1]
                    qb = q[qi].double().reshape(kv_heads, heads // kv_heads, -1)
                    logits = torch.einsum("lkd,kgd->lkg", keys[:valid], qb) * scale
                    out = torch.einsum("lkg,lkd->kgd", torch.softmax(logits, 0), values[:valid]).reshape(heads, -1)
                    logits = logits.reshape(valid, heads)
                lse[qi] = (torch.logsumexp(logits, 0) / math.log(2)).float()
                result[qi] = out.to(torch.bfloat16)
    return {"output": result, "lse": lse}


def materialize_prefill_case(task: str, variant: str, case_id: str) -> dict[str, torch.Tensor]:
    """Inputs of one reference prefill case (attention.py:101-129): as for decode, plus ``qo_indptr`` splitting the
    query rows evenly over the segments; the boundary variant has two segments, six query rows and five KV
    entries (attention.py:16-28)."""
    mla, paged, heads, kv_heads, axes, scale = PREFILL_TASKS[task]
    if variant == "captured":
        axes = dict(axes)
    else:
        axes = dict(len_indptr=3, total_q=6)
        axes.update(dict(num_pages=11, num_kv_indices=5) if paged else dict(total_kv=5))
    batch = axes["len_indptr"] - 1
    qcount = axes["total_q"]
    kvcount = axes["num_kv_indices"] if paged else axes["total_kv"]
    g = torch.Generator(device="cpu").manual_seed(2801 + CASES.index(case_id))
    if mla:
        shapes = {"q_nope": (qcount, heads, 512), "q_pe": (qcount, heads, 64),
                  "ckv_cache": (axes["num_pages"], 1, 512), "kpe_cache": (axes["num_pages"], 1, 64)}
    elif paged:
        shapes = {"q": (qcount, heads, 128), "k_cache": (axes["num_pages"], 1, kv_heads, 128), "v_cache": (axes["num_pages"], 1, kv_heads, 128)}
    else:
        shapes = {"q": (qcount, heads, 128), "k": (kvcount, kv_heads, 128), "v": (kvcount, kv_heads, 128)}
    inputs = {}
    for name, shape in shapes.items():
        inputs[name] = (torch.rand(shape, generator=g, dtype=torch.float32) - 0.5).to(torch.bfloat16)
    qptr = [i * qcount // batch for i in range(batch + 1)]
    kptr = [i * kvcount // batch for i in range(batch + 1)]
    if case_id == "segmented" and batch > 1:
        kptr[1] = 0
    inputs["kv_indptr"] = torch.tensor(kptr, dtype=torch.int32)
    inputs["qo_indptr"] = torch.tensor(qptr, dtype=torch.int32)
    if paged:
        ids = (torch.arange(kvcount, dtype=torch.int64) * 3 + 1) % axes["num_pages"]
        if case_id == "permuted":
            ids = ids.flip(0)
        inputs["kv_indices"] = ids.to(torch.int32)
    inputs["sm_scale"] = torch.tensor([scale * (1.75 if case_id == "scaled" else 1.0)], dtype=torch.float32)
    if case_id == "zeros":
        for name in ("q", "q_nope", "q_pe"):
            if name in inputs:
                inputs[name].zero_()
    return inputs
