"""CPU tests of the drop-in boundary: the library loads without a GPU, exports every symbol the
header declares, rejects null arguments before touching the device, and the target document's
tensor ABI agrees with the reference's contract for the same operator."""
import ctypes
import json
import re
from pathlib import Path

import pytest

import open_cake_ir_b200 as cake

ROOT = Path(__file__).resolve().parent.parent
HEADER = (ROOT / "include" / "cake_b200.h").read_text()


def declared_symbols():
    return sorted(set(re.findall(r"\b(cake_b200_[a-z0-9_]+)\s*\(", HEADER)))


def test_library_exports_every_declared_symbol():
    lib = cake._lib.library()
    names = declared_symbols()
    assert len(names) >= 28
    for name in names:
        assert hasattr(lib, name), name
    assert sorted(cake._lib.EXPORTS) == names
    assert lib.cake_b200_abi_version() == 1


def test_every_entry_point_cites_the_reference_interface_it_replaces():
    for block in re.split(r"/\* -{20,}", HEADER)[1:]:
        cites = re.search(r"\b(src/open_cake_ir|corpus|tools)/[\w/.-]+(:\d+)?", block)
        assert cites or "no counterpart in the reference" in block, block[:80]


@pytest.mark.parametrize("stem", list(cake._lib.OPERATORS))
def test_null_arguments_are_rejected_without_a_device(stem):
    lib = cake._lib.library()
    config, _ = cake._lib.OPERATORS[stem]
    handle = ctypes.c_void_p()
    assert getattr(lib, f"cake_b200_{stem}_create")(None, ctypes.byref(config()), ctypes.byref(handle)) == 20001
    assert getattr(lib, f"cake_b200_{stem}_launch")(None, None) == 20001
    assert getattr(lib, f"cake_b200_{stem}_destroy")(None) == 0


def test_workspace_queries_are_pure_host_functions():
    cfg = cake._lib.MoeConfig(4096, 7168, 2048, 256, 256, 8, 8, 4, 1, 0, 0)
    size = cake._lib.workspace_bytes("moe", cfg)
    pairs = 4096 * 8
    assert size >= pairs * (7168 + 2048 + 7168 * 2) and size < 2 * pairs * (7168 + 2048 + 7168 * 2)
    assert cake._lib.workspace_bytes("moe", cake._lib.MoeConfig(4096, 7168 + 1, 2048, 256, 256, 8, 8, 4, 1, 0, 0)) == 0
    g = cake._lib.GqaDecodeConfig(64, 32, 8, 128, 16, 4096)
    assert cake._lib.workspace_bytes("gqa_decode", g) > 64 * 32 * 129 * 4
    assert cake._lib.workspace_bytes("gqa_decode", cake._lib.GqaDecodeConfig(64, 32, 5, 128, 16, 4096)) == 0


def test_operators_refuse_cpu_tensors():
    import torch
    x = torch.zeros((4, 16), dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="no CPU path"):
        cake.rmsnorm(x, torch.ones(16, dtype=torch.bfloat16), 1e-6)


def test_target_document_matches_the_contract_abi():
    doc = cake.operators.target()
    assert doc["nvcc_flags"] == ["--gpu-architecture=compute_100a", "--gpu-code=sm_100a"]
    moe = [t["name"] for t in cake.operators.tensor_abi("fp8_moe")]
    # src/open_cake_ir/tasks/solx_fib/moe.py:13-20, inputs then the output
    assert moe == ["routing_logits", "routing_bias", "hidden_states", "hidden_states_scale", "gemm1_weights",
                   "gemm1_weights_scale", "gemm2_weights", "gemm2_weights_scale", "local_expert_offset",
                   "routed_scaling_factor", "output"]
    gqa = [t["name"] for t in cake.operators.tensor_abi("gqa_paged_decode")]
    assert gqa == ["q", "k_cache", "v_cache", "kv_indptr", "kv_indices", "kv_last_page_len", "sm_scale", "output", "lse"]
    for name, op in doc["operators"].items():
        for verb in ("create", "launch", "destroy"):
            assert op["host_abi"][verb] in HEADER, (name, verb)
        assert all(t["mode"] in ("input", "output") for t in op["tensors"])
    assert json.dumps(doc)      # canonical JSON


def test_target_document_carries_the_launch_metadata_of_the_build():
    """What the reference's consumer validates in a candidate's metadata (tools/native_cuda_contract.py:150-175):
    arguments / argument_order / signature in ABI order, block == [threads_per_cta, 1, 1], dynamic shared bytes, the
    exact architecture selectors and the link libraries -- checked against the build script and the compiled constants."""
    import ctypes
    import importlib.util
    doc = cake.operators.target()
    spec = importlib.util.spec_from_file_location("cake_b200_build", ROOT / "open-cake-ir_b200" / "build.py")
    build = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(build)
    selectors = [f for f in build.NVCC_FLAGS if any(k in f for k in ("gpu-architecture", "gpu-code", "-arch", "gencode"))]
    assert selectors == doc["nvcc_flags"] == ["--gpu-architecture=compute_100a", "--gpu-code=sm_100a"]
    assert [f for f in build.NVCC_FLAGS if f not in selectors and f not in ("-Xptxas", "-v")] == doc["nvcc_other_flags"]
    assert doc["link_libraries"] == ["cudart_static"]
    lib = cake._lib.library()
    for name, op in doc["operators"].items():
        assert op["arguments"] == op["tensors"] and op["argument_order"] == [t["name"] for t in op["tensors"]]
        assert op["signature"] == {t["name"]: "*" + t["dtype"] for t in op["tensors"]}
        kernel = op["main_kernel"]
        assert kernel["block"] == [kernel["threads_per_cta"], 1, 1] and kernel["dynamic_shared_bytes"] >= 0
        threads, smem = ctypes.c_int(), ctypes.c_int()
        if lib.cake_b200_launch_facts(kernel["name"].encode(), ctypes.byref(threads), ctypes.byref(smem)) == 0:
            assert (kernel["threads_per_cta"], kernel["dynamic_shared_bytes"]) == (threads.value, smem.value), name


def test_ep_rows_must_stay_sixteen_byte_aligned():
    """Packed rows are moved with 16-byte loads and stores: configurations whose row width is not a
    multiple of 16 (odd top_k, hidden not a multiple of 512) are refused by returning 0."""
    import ctypes
    lib = cake._lib.library()
    def width(hidden, top_k):
        cfg = cake._lib.EpConfig(64, 64, hidden, top_k, 2, 32)
        return int(lib.cake_b200_ep_row_bytes(ctypes.byref(cfg)))
    assert width(1024, 8) == 1024 + 32 + 64
    assert width(1024, 1) == 0 and width(1024, 7) == 0
    assert width(640, 8) == 0


def test_push_exchange_sizes_and_refusals():
    """The symmetric buffer of the push exchange is flags (1 KiB) | one packed row per (source rank, slot) | one bf16
    partial row per (source rank, slot); a rank outside the world, a world above 64 ranks and a row width that is not
    a multiple of 16 bytes are refused by returning 0."""
    import ctypes
    lib = cake._lib.library()

    def sizes(tokens, hidden, top_k, world, experts, rank):
        cfg = cake._lib.EpPushConfig(tokens, tokens, hidden, top_k, world, experts, rank)
        return (int(lib.cake_b200_ep_push_symmetric_bytes(ctypes.byref(cfg))), int(lib.cake_b200_ep_push_scratch_bytes(ctypes.byref(cfg))))

    sym, scratch = sizes(512, 7168, 8, 8, 256, 3)
    row = 7168 + 4 * 56 + 8 * 8
    assert sym == 1024 + 8 * 512 * row + 8 * 512 * 7168 * 2 and scratch > 0 and scratch % 256 == 0
    assert sizes(512, 7168, 8, 8, 256, 8) == (0, 0)          # rank outside the world
    assert sizes(512, 7168, 8, 128, 256, 0) == (0, 0)        # more ranks than the flag block holds
    assert sizes(512, 7168, 7, 8, 256, 0) == (0, 0)          # odd top_k: rows would lose their 16-byte alignment
    from open_cake_ir_b200 import ep
    assert ep.PushExpertParallelMoe.symmetric_bytes(512, 7168, 8, 8, 256) == sym
