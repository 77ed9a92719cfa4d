"""Generate the golden fixtures in this directory from the reference's own oracles.

Run once, in a container that holds the reference checkout, as
``python tests/golden/make_golden.py <path-to-reference>``: it imports the reference's task
modules from ``<reference>/src``, materialises every case of the hot-path contracts with the
reference's materialisers, runs the reference's CPU oracles and stores, per case, the oracle
OUTPUTS (bf16/fp32 as raw little-endian integers) and a SHA-256 of every INPUT tensor's
bytes.  Inputs are not stored (the MoE weights alone are ~1.4 GB per case): the test-suite
regenerates them with the restated materialisers under ``oracle/`` and first checks the
hashes.  The fixtures travel with the repository; the reference checkout does not.
"""
from __future__ import annotations

import hashlib
import json
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent


def sha(t: torch.Tensor) -> str:
    return hashlib.sha256(t.contiguous().view(torch.uint8).numpy().tobytes()).hexdigest()


def raw(t: torch.Tensor) -> np.ndarray:
    t = t.contiguous()
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy()
    if t.dtype == torch.float32:
        return t.view(torch.int32).numpy()
    return t.numpy()


def main(reference: str) -> None:
    sys.path.insert(0, str(Path(reference) / "src"))
    from open_cake_ir.tasks import workloads as registry
    from open_cake_ir.tasks.solx_fib import attention, moe, workload as rms
    contracts = Path(reference) / "contracts" / "workloads"
    index = {}
    arrays = {}

    # RMSNorm: h4096 (R=170, eps 1e-5) and h7168 (R=64, eps 1e-6), five modes each.
    for stem in ("solx-fib-rmsnorm-h4096-bf16-triton-b300-r170-v1",
                 "solx-fib-rmsnorm-h7168-bf16-triton-b300-r64-v1",
                 "solx-fib-fused-add-rmsnorm-h4096-bf16-triton-b300-r170-v1"):
        w = registry.load_workload(contracts / (stem + ".json"))
        for case in w.case_ids:
            inputs = rms.materialize_case(w, case)
            out = rms.reference_outputs(w, case, inputs)["out"]
            shape = w.case(case)["shape"]
            key = f"rmsnorm/{stem}/{case}"
            tensors = {n: torch.tensor(v, dtype=torch.float64).float().to(torch.bfloat16) for n, v in inputs.items()}
            index[key] = {"rows": shape["R"], "width": shape["C"], "seed": w.case(case)["seed"],
                          "epsilon": w.document["semantics"]["epsilon"],
                          "inputs_sha256": {n: sha(t) for n, t in tensors.items()}}
            out_t = torch.tensor(out, dtype=torch.float64).float().to(torch.bfloat16).reshape(shape["R"], shape["C"])
            index[key]["out_sha256"] = sha(out_t)            # the whole output, by hash
            arrays[key + "/out_head"] = raw(out_t[:4])        # and its first four rows, by value
            print(key, flush=True)

    # Paged decode: GQA kv4 / kv8 and MLA h16, captured + boundary, five cases each.
    for task, stem in (("gqa_kv4", "solx-fib-gqa-paged-decode-h32-kv4-d128-ps1-bf16-b300-{v}-v1"),
                       ("gqa_kv8", "solx-fib-gqa-paged-decode-h32-kv8-d128-ps1-bf16-b300-{v}-v1"),
                       ("mla_h16", "solx-fib-mla-paged-decode-h16-ckv512-kpe64-ps1-bf16-b300-{v}-v1")):
        for variant in ("captured", "boundary"):
            w = registry.load_workload(contracts / (stem.format(v=variant) + ".json"))
            for case in w.case_ids:
                inputs = attention.materialize_tensors(w, case)
                ref = attention.reference_tensors(w, case, inputs)
                key = f"decode/{task}/{variant}/{case}"
                index[key] = {"inputs_sha256": {n: sha(t) for n, t in inputs.items()},
                              "output_shape": list(ref["output"].shape)}
                arrays[key + "/output"] = raw(ref["output"])
                arrays[key + "/lse"] = raw(ref["lse"])
                print(key, flush=True)

    # FP8 MoE: six cases at T=1, 32 local experts.
    w = registry.load_workload(contracts / "solx-fib-moe-fp8-block-scale-ds-routing-topk8-ng8-kg4-e32-h7168-i2048-bf16-b300-t1-v1.json")
    for case in w.case_ids:
        inputs = moe.materialize_tensors(w, case)
        ref = moe.reference_tensors(w, case, inputs)
        sel, wts = moe.routing_reference(inputs["routing_logits"], inputs["routing_bias"],
                                         float(inputs["routed_scaling_factor"][0]))
        key = f"moe/{case}"
        index[key] = {"inputs_sha256": {n: sha(t) for n, t in inputs.items()}}
        arrays[key + "/output"] = raw(ref["output"])
        arrays[key + "/expert_ids"] = sel.to(torch.int32).numpy()
        arrays[key + "/route_weights"] = raw(wts.float())
        print(key, flush=True)

    np.savez_compressed(HERE / "reference_outputs.npz", **arrays)
    (HERE / "reference_index.json").write_text(json.dumps(index, indent=1, sort_keys=True) + "\n")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit(f"usage: python {Path(__file__).name} <path of a checkout of the reference>")
    main(sys.argv[1])
