"""CPU oracle for the B200 inference-kernel path.  TEST INFRASTRUCTURE ONLY.

Every function here restates, on the host CPU (torch CPU / numpy / stdlib), the arithmetic of
one reference operator of qhy991/open-cake-ir and cites the reference file:line it follows.
Nothing in the product package imports this directory: only the test-suite, the smoke check
and the CPU-baseline / reference arm of the benchmark may, and there only as the checker or
as the thing timed *beside* the GPU path, never as a fallback for it.

Parity status: PINNED.  The restatements are checked bit-for-bit against outputs of the
reference's own oracles (imported from the reference checkout when the fixtures under
``tests/golden`` were generated) and against the known-answer vectors held in the
reference's contract tests.  Definitions the reference does not hold (page_size > 1
addressing, softmax top-k routing, the canonical permutation order, FP8 requantisation of the
SwiGLU output) are pinned by reduction to the reference on the cases it does hold plus
known-answer tests of their own.
"""
from . import add_rmsnorm, attention, block_scaled_gemm, compare, deepseek_v4, moe, permute, rmsnorm, routing  # noqa: F401
