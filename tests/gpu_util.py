"""Helpers shared by the GPU parity tests: poison-filled outputs, guard bands around outputs,
bitwise input snapshots (the reference harness's practice, src/open_cake_ir/evaluation/core.py:750-752,
torch_tensor_inputs.py:45-48, core.py:602-636)."""
import torch

GUARD = 4096  # bytes on each side of a guarded buffer


def poison(shape, dtype, device="cuda"):
    """Output buffer with guard bands; returns (view, check) where check() asserts the bands are intact."""
    elem = torch.empty((), dtype=dtype).element_size()
    count = 1
    for s in shape:
        count *= s
    raw = torch.full((count * elem + 2 * GUARD,), 0xA5, dtype=torch.uint8, device=device)
    view = raw[GUARD:GUARD + count * elem].view(dtype).reshape(shape)
    if dtype in (torch.float32, torch.bfloat16, torch.float16):
        view.fill_(float("nan"))
    elif dtype == torch.int32:
        view.fill_(-2 ** 31)

    def check():
        assert bool((raw[:GUARD] == 0xA5).all()) and bool((raw[GUARD + count * elem:] == 0xA5).all()), "guard band overwritten"
    return view, check


def snapshot(tensors: dict) -> dict:
    return {k: v.detach().clone() for k, v in tensors.items()}


def unchanged(before: dict, after: dict) -> bool:
    return all(torch.equal(before[k].reshape(-1).view(torch.uint8), after[k].reshape(-1).view(torch.uint8)) for k in before)
