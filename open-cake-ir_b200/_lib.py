"""ctypes bindings of ``libcake_b200.so``: one Python function per ``extern "C"`` symbol of
``include/cake_b200.h``, the config structs, and error translation.  Loading fails loudly when
the library has not been built; nothing here computes on the CPU."""
from __future__ import annotations

import ctypes
from ctypes import POINTER, Structure, c_float, c_int, c_int32, c_int64, c_size_t, c_void_p
from pathlib import Path

import os

# CAKE_B200_LIBRARY points at another build of the same library (e.g. one with bounds checks).
LIBRARY_PATH = Path(os.environ.get("CAKE_B200_LIBRARY") or Path(__file__).resolve().parent / "libcake_b200.so")


class CakeError(RuntimeError):
    def __init__(self, where: str, code: int):
        super().__init__(f"{where} failed with code {code} ({describe(code)})")
        self.code = code


def describe(code: int) -> str:
    own = {20001: "bad argument", 20002: "wrong device", 20003: "device is not sm_100",
           20004: "workspace too small", 20005: "device status word set"}
    if code in own:
        return own[code]
    if code >= 10000:
        return f"CUresult {code - 10000}"
    return f"cudaError_t {code}"


class RmsNormConfig(Structure):
    _fields_ = [("rows", c_int64), ("width", c_int64), ("epsilon", c_float), ("fused_residual", c_int32)]


class AddRmsNormConfig(Structure):
    _fields_ = [("rows", c_int64), ("width", c_int64), ("epsilon", c_float)]


class GemmConfig(Structure):
    _fields_ = [("m", c_int64), ("n", c_int64), ("k", c_int64)]


class RoutingConfig(Structure):
    _fields_ = [("tokens", c_int64), ("experts", c_int32), ("top_k", c_int32), ("n_group", c_int32),
                ("topk_group", c_int32), ("mode", c_int32)]


class V4GateConfig(Structure):
    _fields_ = [("tokens", c_int64), ("experts", c_int32), ("top_k", c_int32), ("route_scale", c_float)]


class TopkConfig(Structure):
    _fields_ = [("rows", c_int64), ("candidates", c_int32), ("top_k", c_int32)]


class PermuteConfig(Structure):
    _fields_ = [("tokens", c_int64), ("top_k", c_int32), ("local_experts", c_int32)]


class MoeConfig(Structure):
    _fields_ = [("tokens", c_int64), ("hidden", c_int32), ("intermediate", c_int32), ("experts", c_int32),
                ("local_experts", c_int32), ("top_k", c_int32), ("n_group", c_int32), ("topk_group", c_int32),
                ("routing_mode", c_int32), ("act_mode", c_int32), ("external_routing", c_int32)]


class EpConfig(Structure):
    _fields_ = [("tokens", c_int64), ("capacity", c_int64), ("hidden", c_int32), ("top_k", c_int32),
                ("world", c_int32), ("experts", c_int32)]


class EpPushConfig(Structure):
    _fields_ = [("tokens", c_int64), ("capacity", c_int64), ("hidden", c_int32), ("top_k", c_int32),
                ("world", c_int32), ("experts", c_int32), ("rank", c_int32)]


class GqaDecodeConfig(Structure):
    _fields_ = [("batch", c_int64), ("num_qo_heads", c_int32), ("num_kv_heads", c_int32), ("head_dim", c_int32),
                ("page_size", c_int32), ("max_kv_len", c_int64)]


class MlaDecodeConfig(Structure):
    _fields_ = [("batch", c_int64), ("num_qo_heads", c_int32), ("head_dim_ckv", c_int32), ("head_dim_kpe", c_int32),
                ("page_size", c_int32), ("max_kv_len", c_int64)]


class GqaPrefillConfig(Structure):
    _fields_ = [("total_q", c_int64), ("segments", c_int32), ("num_qo_heads", c_int32), ("num_kv_heads", c_int32),
                ("head_dim", c_int32), ("page_size", c_int32), ("ragged", c_int32), ("nan_for_masked", c_int32),
                ("max_kv_len", c_int64)]


class MlaPrefillConfig(Structure):
    _fields_ = [("total_q", c_int64), ("segments", c_int32), ("num_qo_heads", c_int32), ("head_dim_ckv", c_int32),
                ("head_dim_kpe", c_int32), ("page_size", c_int32), ("nan_for_masked", c_int32), ("max_kv_len", c_int64)]


class SparseMlaDecodeConfig(Structure):
    _fields_ = [("num_tokens", c_int64), ("num_cache_rows", c_int64), ("num_qo_heads", c_int32), ("head_dim_ckv", c_int32),
                ("head_dim_kpe", c_int32), ("top_k", c_int32), ("sm_scale", c_float)]


# operator stem -> (config struct, has a workspace query)
OPERATORS = {
    "rmsnorm": (RmsNormConfig, False),
    "add_rmsnorm": (AddRmsNormConfig, False),
    "block_scaled_gemm": (GemmConfig, True),
    "moe_routing": (RoutingConfig, False),
    "moe_permute": (PermuteConfig, False),
    "v4_moe_gate": (V4GateConfig, False),
    "csa_topk": (TopkConfig, False),
    "moe": (MoeConfig, True),
    "gqa_decode": (GqaDecodeConfig, True),
    "mla_decode": (MlaDecodeConfig, True),
    "sparse_mla_decode": (SparseMlaDecodeConfig, True),
    "gqa_prefill": (GqaPrefillConfig, True),
    "mla_prefill": (MlaPrefillConfig, True),
}
# every symbol include/cake_b200.h declares
EXPORTS = (["cake_b200_abi_version", "cake_b200_read_status", "cake_b200_test_hooks", "cake_b200_launch_facts", "cake_b200_decode_plan_view", "cake_b200_moe_intermediate", "cake_b200_moe_launch_stage",
            "cake_b200_gqa_decode_noalloc", "cake_b200_gqa_decode_noalloc_scratch_limit",
            "cake_b200_ep_row_bytes", "cake_b200_ep_exchange_create", "cake_b200_ep_exchange_launch_stage",
            "cake_b200_ep_exchange_destroy", "cake_b200_ep_push_symmetric_bytes", "cake_b200_ep_push_scratch_bytes",
            "cake_b200_ep_push_create", "cake_b200_ep_push_launch_stage", "cake_b200_ep_push_destroy"]
           + [f"cake_b200_{stem}_{verb}" for stem in OPERATORS for verb in ("create", "launch", "destroy")]
           + [f"cake_b200_{stem}_workspace_bytes" for stem, (_, ws) in OPERATORS.items() if ws])

_library = None


def library() -> ctypes.CDLL:
    global _library
    if _library is None:
        if not LIBRARY_PATH.exists():
            raise RuntimeError(
                f"{LIBRARY_PATH} is missing: build it with `python open-cake-ir_b200/build.py` "
                "(or __graft_entry__.build()); this package has no CPU fallback")
        lib = ctypes.CDLL(str(LIBRARY_PATH))
        lib.cake_b200_abi_version.restype = c_int
        lib.cake_b200_read_status.argtypes = [c_void_p, c_void_p, POINTER(c_int)]
        lib.cake_b200_test_hooks.argtypes = [c_int, c_int]
        lib.cake_b200_launch_facts.argtypes = [ctypes.c_char_p, POINTER(c_int), POINTER(c_int)]
        lib.cake_b200_decode_plan_view.argtypes = [ctypes.c_char_p, c_void_p, c_int, POINTER(c_void_p), POINTER(c_int)]
        lib.cake_b200_moe_intermediate.argtypes = [c_void_p, c_int, POINTER(c_void_p)]
        lib.cake_b200_moe_launch_stage.argtypes = [c_void_p, c_int, c_void_p]
        lib.cake_b200_gqa_decode_noalloc.argtypes = [POINTER(c_void_p), POINTER(GqaDecodeConfig), c_void_p]
        lib.cake_b200_gqa_decode_noalloc.restype = c_int
        lib.cake_b200_gqa_decode_noalloc_scratch_limit.restype = c_size_t
        lib.cake_b200_ep_row_bytes.argtypes = [POINTER(EpConfig)]
        lib.cake_b200_ep_row_bytes.restype = c_size_t
        lib.cake_b200_ep_exchange_create.argtypes = [POINTER(c_void_p), POINTER(EpConfig), POINTER(c_void_p)]
        lib.cake_b200_ep_exchange_launch_stage.argtypes = [c_void_p, c_int, c_void_p]
        lib.cake_b200_ep_exchange_destroy.argtypes = [c_void_p]
        lib.cake_b200_ep_push_symmetric_bytes.argtypes = [POINTER(EpPushConfig)]
        lib.cake_b200_ep_push_symmetric_bytes.restype = c_size_t
        lib.cake_b200_ep_push_scratch_bytes.argtypes = [POINTER(EpPushConfig)]
        lib.cake_b200_ep_push_scratch_bytes.restype = c_size_t
        lib.cake_b200_ep_push_create.argtypes = [POINTER(c_void_p), POINTER(EpPushConfig), POINTER(c_void_p)]
        lib.cake_b200_ep_push_launch_stage.argtypes = [c_void_p, c_int, c_void_p]
        lib.cake_b200_ep_push_destroy.argtypes = [c_void_p]
        for stem, (config, has_ws) in OPERATORS.items():
            create = getattr(lib, f"cake_b200_{stem}_create")
            create.argtypes = [POINTER(c_void_p), POINTER(config), POINTER(c_void_p)]
            create.restype = c_int
            launch = getattr(lib, f"cake_b200_{stem}_launch")
            launch.argtypes = [c_void_p, c_void_p]
            launch.restype = c_int
            destroy = getattr(lib, f"cake_b200_{stem}_destroy")
            destroy.argtypes = [c_void_p]
            destroy.restype = c_int
            if has_ws:
                query = getattr(lib, f"cake_b200_{stem}_workspace_bytes")
                query.argtypes = [POINTER(config)]
                query.restype = c_size_t
        _library = lib
    return _library


def workspace_bytes(stem: str, config) -> int:
    return int(getattr(library(), f"cake_b200_{stem}_workspace_bytes")(ctypes.byref(config)))


def decode_plan_view(stem: str, handle, which: int) -> tuple[int, int]:
    """(device pointer, element count) of part ``which`` of the work plan a decode handle's plan kernel writes
    (``cake_b200_decode_plan_view``; a test accessor)."""
    pointer, count = c_void_p(), c_int()
    code = library().cake_b200_decode_plan_view(stem.encode(), handle, which, ctypes.byref(pointer), ctypes.byref(count))
    if code != 0:
        raise CakeError("cake_b200_decode_plan_view", code)
    return int(pointer.value or 0), int(count.value)


class NativeHandle:
    """create / launch / destroy around one native handle (the shape of the reference's
    ``NativeHandle`` adapter, tools/native_cuda_evaluate.py:485-520)."""

    def __init__(self, stem: str, pointers: list[int], config):
        lib = library()
        self.stem = stem
        self._launch = getattr(lib, f"cake_b200_{stem}_launch")
        self._destroy = getattr(lib, f"cake_b200_{stem}_destroy")
        self.handle = c_void_p()
        array = (c_void_p * len(pointers))(*pointers)
        code = getattr(lib, f"cake_b200_{stem}_create")(array, ctypes.byref(config), ctypes.byref(self.handle))
        if code != 0 or not self.handle.value:
            raise CakeError(f"cake_b200_{stem}_create", code)
        self.calls = 0

    def launch(self, stream: int) -> None:
        code = self._launch(self.handle, c_void_p(stream))
        if code != 0:
            raise CakeError(f"cake_b200_{self.stem}_launch", code)
        self.calls += 1

    def close(self) -> None:
        if self.handle is not None and self.handle.value:
            code = self._destroy(self.handle)
            self.handle = c_void_p()
            if code != 0:
                raise CakeError(f"cake_b200_{self.stem}_destroy", code)

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def read_status(workspace_ptr: int, stream: int) -> int:
    out = c_int(0)
    code = library().cake_b200_read_status(c_void_p(workspace_ptr), c_void_p(stream), ctypes.byref(out))
    if code != 0:
        raise CakeError("cake_b200_read_status", code)
    return out.value
