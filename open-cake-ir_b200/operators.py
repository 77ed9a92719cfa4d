"""The workload contracts this target implements, as data: per operator the ordered tensor ABI
(name, dtype, symbolic shape, mode) in the reference's convention -- inputs then outputs, all
contiguous row-major, scalars as one-element tensors (src/open_cake_ir/evaluation/workload.py:147-190)
-- and the native host-ABI entry that runs it.  Names, layouts and scale conventions are the
reference's (src/open_cake_ir/tasks/solx_fib/moe.py:13-20, attention_specs.py:44-84 and :249-292,
workload.py:214-218, corpus/schedules/block-scaled-gemm-b1-smoke.json)."""
from __future__ import annotations

import json
from pathlib import Path

TARGET_FILE = Path(__file__).resolve().parent / "targets" / "sm_100a_native.json"


def target() -> dict:
    """The target document: hardware facts in the schema of compiler/targets/sm_100a.json plus the
    operator -> host ABI registry."""
    return json.loads(TARGET_FILE.read_text())


def tensor_abi(operator: str) -> list[dict]:
    return target()["operators"][operator]["tensors"]


def host_abi(operator: str) -> dict:
    return target()["operators"][operator]["host_abi"]
