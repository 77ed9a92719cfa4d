// Causal prefill over a paged or ragged KV store, expressed as decode over one sequence per query token.
//
// Operator (src/open_cake_ir/tasks/solx_fib/attention.py:132-183, the branches with `not spec['decode']`; specs
// attention_specs.py:85-248 and :293-338): segment b holds query rows [qo_indptr[b], qo_indptr[b+1]) and KV rows
// [kv_indptr[b], kv_indptr[b+1]); query row i of a segment with q_len rows and kv_len rows attends to the first
//   valid = min(kv_len, i + 1 + kv_len - q_len)
// KV rows (the causal mask aligned to the bottom right, attention.py:170).  A segment with no query or no KV rows
// is left at zeros / -inf; a row of a non-empty segment with valid <= 0 is NaN where the contract says so (the
// ragged and MLA tasks, attention.py:47) and zeros otherwise; its lse is -inf either way (:171-173).
//
// `prefill_plan_kernel` writes, per query token, where its KV list starts and how many rows it sees; the decode
// kernels then treat every token as a sequence of its own (their explicit sequence table), and
// `prefill_mark_kernel` writes the NaN rows.  Every query token therefore streams its own prefix of the
// segment's KV rows: correct for any shape, and sized for the short suffix prefills of a serving step, not for
// long prompts, where a kernel that shares KV tiles between query rows is the right tool.
#pragma once
#include "common.cuh"

namespace cake {
namespace prefill {

// One thread per query token.  `kv_unit` = rows per kv_indptr unit (the page size; 1 for ragged K/V);
// last_page_len may be null (every page full).
static __global__ void __launch_bounds__(256)
prefill_plan_kernel(const int* __restrict__ qo_indptr, const int* __restrict__ kv_indptr, const int* __restrict__ last_page_len,
                    int segments, int kv_unit, int total_q, int* __restrict__ seq_start, int* __restrict__ seq_tokens,
                    int* __restrict__ masked) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= total_q) return;
  int lo = 0, hi = segments;                     // largest b with qo_indptr[b] <= t
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (__ldg(qo_indptr + mid) <= t) lo = mid; else hi = mid;
  }
  const int b = lo;
  const int qs = __ldg(qo_indptr + b), qe = __ldg(qo_indptr + b + 1);
  const int ks = __ldg(kv_indptr + b), ke = __ldg(kv_indptr + b + 1);
  int tokens = 0, flag = 0;
  if (t >= qs && t < qe && ke > ks) {
    const int units = ke - ks;
    const int kv_len = last_page_len ? (units - 1) * kv_unit + __ldg(last_page_len + b) : units * kv_unit;
    const int valid = min(kv_len, (t - qs + 1) + kv_len - (qe - qs));
    tokens = max(valid, 0);
    flag = valid <= 0;
  }
  seq_start[t] = ks;
  seq_tokens[t] = tokens;
  masked[t] = flag;
}

// One warp per query token: a fully masked row of a non-empty segment becomes NaN (lse stays -inf).
static __global__ void __launch_bounds__(256)
prefill_mark_kernel(const int* __restrict__ masked, int total_q, __nv_bfloat16* __restrict__ out, int row_elements) {
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (t >= total_q || !masked[t]) return;
  uint16_t* row = reinterpret_cast<uint16_t*>(out) + size_t(t) * row_elements;
  for (int i = lane; i < row_elements; i += 32) row[i] = 0x7fc0;     // bf16 quiet NaN
}

inline size_t table_bytes(int64_t total_q) { return 3 * ((size_t(total_q) * sizeof(int) + 255) & ~size_t(255)); }

}  // namespace prefill
}  // namespace cake
