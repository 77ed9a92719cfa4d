"""Golden fixtures for the operators either side of the hot path, from the reference's own oracles.

``python tests/golden/make_golden_next.py <path-to-reference>`` imports, from ``<reference>/src``, the
two-output add + RMSNorm task (``open_cake_ir.tasks.add_rmsnorm``, five cases at R=128, C=2560) and the
two DeepSeek-V4 routing tasks (``open_cake_ir.tasks.deepseek_v4.workload``: MoE gate and CSA indexer
top-k, four cases each at four rows) and the five causal-prefill attention tasks
(``open_cake_ir.tasks.solx_fib.attention``: captured and boundary variants, five cases each), materialises every case with the reference's materialiser, runs
the reference's oracle and stores the oracle OUTPUTS (or, where the reference's oracle refuses its own
case because scores tie after rounding, the refusal) plus a SHA-256 of every INPUT tensor in
``next_outputs.npz`` / ``next_index.json``.  The test-suite regenerates the inputs with the restated
materialisers under ``oracle/`` and checks the hashes first.
"""
from __future__ import annotations

import json
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE))
from make_golden import raw, sha  # noqa: E402


def main(reference: str) -> None:
    sys.path.insert(0, str(Path(reference) / "src"))
    from open_cake_ir.evaluation.workload import WorkloadContract
    from open_cake_ir.tasks import add_rmsnorm
    from open_cake_ir.tasks.deepseek_v4 import workload as v4
    index, arrays = {}, {}

    w = WorkloadContract(add_rmsnorm.workload_document())
    for case in w.case_ids:
        inputs = add_rmsnorm.materialize_case(w, case)
        ref = add_rmsnorm.reference_outputs(w, case, inputs)
        shape = w.case(case)["shape"]
        key = f"add_rmsnorm/{case}"
        tensors = {n: torch.tensor(v, dtype=torch.float64).float().to(torch.bfloat16) for n, v in inputs.items()}
        index[key] = {"rows": shape["R"], "width": shape["C"], "epsilon": add_rmsnorm.EPSILON,
                      "inputs_sha256": {n: sha(t) for n, t in tensors.items()}}
        for name in ("out", "residual_out"):
            arrays[f"{key}/{name}"] = raw(torch.tensor(ref[name], dtype=torch.float64).float().to(torch.bfloat16)
                                          .reshape(shape["R"], shape["C"]))
        print(key, flush=True)

    for task in ("moe_gate", "csa_indexer_topk"):
        w = WorkloadContract(v4.workload_document(task))
        for case in w.case_ids:
            inputs = v4.materialize_case(w, case)
            key = f"deepseek_v4/{task}/{case}"
            index[key] = {"shape": w.case(case)["shape"],
                          "inputs_sha256": {n: sha(torch.tensor(v, dtype=torch.float64).float()) for n, v in inputs.items()}}
            try:
                ref = v4.reference_outputs(w, case, inputs)
            except ValueError as refusal:      # the reference's oracle refuses rows whose scores tie after rounding
                index[key]["refused"] = str(refusal)
                print(key, "refused:", refusal, flush=True)
                continue
            for name, values in ref.items():
                if name in ("indices", "expert_ids"):
                    arrays[f"{key}/{name}"] = np.asarray(values, dtype=np.int32)
                else:
                    arrays[f"{key}/{name}"] = raw(torch.tensor(values, dtype=torch.float64).float())
            print(key, flush=True)

    # Causal prefill: GQA paged kv4 / kv8, GQA ragged kv4 / kv8 and MLA paged, captured + boundary, five cases each.
    from open_cake_ir.tasks import workloads as registry
    from open_cake_ir.tasks.solx_fib import attention
    contracts = Path(reference) / "contracts" / "workloads"
    for task, stem in (("gqa_paged_prefill_kv4", "solx-fib-gqa-paged-prefill-causal-h32-kv4-d128-ps1-bf16-b300-{v}-v1"),
                       ("gqa_paged_prefill_kv8", "solx-fib-gqa-paged-prefill-causal-h32-kv8-d128-ps1-bf16-b300-{v}-v1"),
                       ("gqa_ragged_prefill_kv4", "solx-fib-gqa-ragged-prefill-causal-h32-kv4-d128-bf16-b300-{v}-v1"),
                       ("gqa_ragged_prefill_kv8", "solx-fib-gqa-ragged-prefill-causal-h32-kv8-d128-bf16-b300-{v}-v1"),
                       ("mla_paged_prefill_h16", "solx-fib-mla-paged-prefill-causal-h16-ckv512-kpe64-ps1-bf16-b300-{v}-v1")):
        for variant in ("captured", "boundary"):
            w = registry.load_workload(contracts / (stem.format(v=variant) + ".json"))
            for case in w.case_ids:
                inputs = attention.materialize_tensors(w, case)
                ref = attention.reference_tensors(w, case, inputs)
                key = f"prefill/{task}/{variant}/{case}"
                index[key] = {"inputs_sha256": {n: sha(t) for n, t in inputs.items()}, "output_shape": list(ref["output"].shape),
                              "nan_for_masked": w.document["semantics"]["fully_masked_nonempty_segment_output"] == "nan"}
                arrays[key + "/output"] = raw(ref["output"])
                arrays[key + "/lse"] = raw(ref["lse"])
                print(key, flush=True)

    np.savez_compressed(HERE / "next_outputs.npz", **arrays)
    (HERE / "next_index.json").write_text(json.dumps(index, indent=1, sort_keys=True) + "\n")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit(f"usage: python {Path(__file__).name} <path of a checkout of the reference>")
    main(sys.argv[1])
