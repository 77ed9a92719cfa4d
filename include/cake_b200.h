/* cake_b200.h -- C ABI of the B200 (sm_100a) native target for open-cake-ir's inference
 * workload contracts.
 *
 * Every operator follows the host ABI of the reference's native CUDA backend
 * (corpus/expected/native-gemm-bias.txt:170-215, consumed by
 * tools/native_cuda_evaluate.py:485-520 and described in docs/NATIVE_CUDA_DESIGN.md:98-104):
 *
 *     int <op>_create (void** buffers, <config>, void** handle_out);
 *     int <op>_launch (void* handle, void* cuda_stream);
 *     int <op>_destroy(void* handle);
 *
 * `buffers` holds DEVICE pointers in the order of the workload contract's tensor ABI
 * (inputs, then outputs; src/open_cake_ir/evaluation/workload.py:147-190), followed where an
 * operator needs scratch by a caller-owned workspace pointer.  All tensors are contiguous
 * row-major.  The caller owns every buffer, the stream and all synchronisation; `create`
 * validates, records pointers, encodes tensor maps and sets function attributes -- it does
 * not allocate device memory, copy or launch.  `launch` only enqueues kernels on the given
 * stream.  Inputs are never written.  A handle must outlive the launches queued from it and
 * must be used on the device that was current at `create`.
 *
 * Two things the reference ABI does not have, added because these kernels are not
 * shape-specialised source: a per-operator config struct passed to `create` (the reference
 * bakes shapes into emitted code), and a device status word at the start of the workspace
 * that a kernel sets when one of its bounded waits runs out (read it with
 * cake_b200_read_status after synchronising the stream).  The first 256 bytes of a workspace
 * are the library's (the status word, then the counters its kernels draw work items from);
 * `launch` clears what it uses on the stream, so a workspace needs no initialisation.
 * Workspace alignment: 4 bytes for the decode operators and the dense GEMM (16 there), which
 * align what follows the status block themselves inside the size they ask for; 256 bytes for
 * the MoE layer, whose workspace holds TMA-addressed tiles (create returns
 * CAKE_B200_ERR_BAD_ARGUMENT otherwise).
 *
 * Return values: 0 on success; a cudaError_t value; 10000 + CUresult for driver errors
 * (the reference's convention, native-gemm-bias.txt:192,199); 20001.. for this library's
 * own argument errors (see CAKE_B200_ERR_*).  No exceptions, no aborts, no internal threads.
 */
#ifndef CAKE_B200_H
#define CAKE_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define CAKE_B200_ERR_BAD_ARGUMENT 20001
#define CAKE_B200_ERR_WRONG_DEVICE 20002
#define CAKE_B200_ERR_NOT_BLACKWELL 20003
#define CAKE_B200_ERR_WORKSPACE 20004
#define CAKE_B200_ERR_DEVICE_STATUS 20005

/* Library identification: ABI version (bumped on any incompatible change). */
int cake_b200_abi_version(void);

/* Copies the 4-byte status word at the start of `workspace` to the host (synchronous on
 * `cuda_stream`).  0 = every kernel ran to completion; otherwise the code of the first wait
 * that gave up (1 smem-full, 2 smem-empty, 3 tmem-full, 4 tmem-empty, 5 flag). */
int cake_b200_read_status(const void* workspace, void* cuda_stream, int* status_out);

/* Launch facts of a kernel of this library as compiled -- "gemm_fp8_kernel", "gqa_decode_kernel", "mla_decode_kernel":
 * threads per CTA and dynamic shared-memory bytes (what the reference's consumer reads from a candidate's metadata,
 * tools/native_cuda_contract.py:150-175; targets/sm_100a_native.json carries the same numbers and is checked against this). */
int cake_b200_launch_facts(const char* kernel, int* threads_per_cta, int* dynamic_shared_bytes);

/* For tests of the failure path only; never needed by a caller.  Every device-side wait of the tensor-core kernels
 * (block-scaled GEMM, MoE grouped GEMMs, MLA decode) is bounded; these hooks let a test make one run out
 * without hanging or faulting anything: `wait_budget_kiloclocks` > 0 shortens the budget of every wait of later
 * launches to that many x 1024 SM clocks (0 restores the default of about a second), and `skip_load` != 0 makes
 * a later dense-GEMM launch (its first CTA) or MLA-decode launch (every CTA with three tiles or more) leave one
 * operand load out, so that the consumer's wait runs out, the kernel unwinds and returns, and the status word is
 * set.  Process-wide host state. */
int cake_b200_test_hooks(int wait_budget_kiloclocks, int skip_load);

/* Test accessor: where the plan kernel of a decode handle (kind "gqa_decode" or "mla_decode", the handle of the
 * matching _create) leaves the work plan of its latest launch, as a device pointer into the caller's workspace.
 *   gqa_decode: which 0 = pieces, int32 x4 each {sequence | pieces of it << 16, first token, list index of the
 *               sequence's first piece, end token}, count = capacity; 1 = list index of each range's first piece
 *               (INT_MAX where a range is empty); 2 = pieces per range; count = ranges.
 *   mla_decode: which 0 = units (tiles + start-up shares) before each sequence, int32 [batch + 1];
 *               which 1 = no pointer, count = the number of equal ranges the unit list is cut into. */
int cake_b200_decode_plan_view(const char* kind, void* handle, int which, void** device_pointer_out, int* count_out);

/* ------------------------------------------------------------------------------------------
 * RMSNorm.  Replaces the emitted RMSNorm starter (src/open_cake_ir/tasks/solx_fib/authoring.py:9-53)
 * for the operator defined at src/open_cake_ir/tasks/solx_fib/workload.py:214-218, :334-358:
 *   out[r,c] = bf16( z[r,c] * weight[c] / sqrt(mean_j z[r,j]^2 + epsilon) ),  z = x  or  fp32(x + residual)
 * buffers: x bf16 [rows,width], (residual bf16 [rows,width] if fused_residual), weight bf16 [width],
 *          out bf16 [rows,width].  width must be a multiple of 8.  No workspace.
 * ---------------------------------------------------------------------------------------- */
typedef struct {
  int64_t rows;
  int64_t width;
  float epsilon;
  int32_t fused_residual; /* 0: x only; 1: buffers = x, residual, weight, out */
} cake_b200_rmsnorm_config;
int cake_b200_rmsnorm_create(void** buffers, const cake_b200_rmsnorm_config* config, void** handle_out);
int cake_b200_rmsnorm_launch(void* handle, void* cuda_stream);
int cake_b200_rmsnorm_destroy(void* handle);
/* ------------------------------------------------------------------------------------------
 * Residual add + RMSNorm with two outputs.  Replaces the emitted starter of the reference's
 * `add_rmsnorm_bf16` task (src/open_cake_ir/tasks/add_rmsnorm.py:145-181; definition :66, oracle :131-143):
 *   z = bf16(delta + residual)  (fp32 add, round to nearest even);  residual_out = z;
 *   out = bf16( fp32(z) * rsqrt(mean_j fp32(z)^2 + epsilon) * fp32(weight) )
 * The rounded sum is both what is returned as residual_out (compared bit for bit by the contract) and what is
 * normalised.  buffers: delta bf16 [rows,width], residual bf16 [rows,width], weight bf16 [width],
 *          out bf16 [rows,width], residual_out bf16 [rows,width].  width % 8 == 0.  No workspace.
 * ---------------------------------------------------------------------------------------- */
typedef struct {
  int64_t rows;
  int64_t width;
  float epsilon;
} cake_b200_add_rmsnorm_config;
int cake_b200_add_rmsnorm_create(void** buffers, const cake_b200_add_rmsnorm_config* config, void** handle_out);
int cake_b200_add_rmsnorm_launch(void* handle, void* cuda_stream);
int cake_b200_add_rmsnorm_destroy(void* handle);

/* ------------------------------------------------------------------------------------------
 * Block-scaled FP8 GEMM.  Replaces the emitted block-scaled GEMM
 * (corpus/schedules/block-scaled-gemm-b1-smoke.json, golden corpus/expected/block-scaled-gemm-accepted.txt;
 * oracle tools/kernel_oracles.py:98-112):
 *   c[m,n] = bf16( sum_k a[m,k]*sfa[k/128,m] * b[n,k]*sfb[n/128,k/128] ), fp32 accumulation
 * buffers: a e4m3 [M,K], sfa fp32 [K/128,M], b e4m3 [N,K], sfb fp32 [N/128,K/128], c bf16 [M,N],
 *          workspace (>= cake_b200_block_scaled_gemm_workspace_bytes).  K % 128 == 0, N % 128 == 0.
 * ---------------------------------------------------------------------------------------- */
typedef struct {
  int64_t m, n, k;
} cake_b200_gemm_config;
size_t cake_b200_block_scaled_gemm_workspace_bytes(const cake_b200_gemm_config* config);
int cake_b200_block_scaled_gemm_create(void** buffers, const cake_b200_gemm_config* config, void** handle_out);
int cake_b200_block_scaled_gemm_launch(void* handle, void* cuda_stream);
int cake_b200_block_scaled_gemm_destroy(void* handle);

/* ------------------------------------------------------------------------------------------
 * MoE routing.  Replaces the four routing stages of the reference launch plan
 * (src/open_cake_ir/tasks/solx_fib/moe.py:167-215; oracle moe.py:275-287; top-k key order
 * compiler/backends/triton.py:2428-2460).
 *   mode 0 (DeepSeek-V3): s = sigmoid(logits); choice by s + bias; group score = sum of the two best of each
 *     group; best `topk_group` groups; best `top_k` experts inside them; weights = s[sel] / (sum s[sel] + 1e-20) * factor.
 *   mode 1 (softmax top-k): best `top_k` raw logits; weights = softmax over the selected logits * factor.
 *   Ties go to the lower index; results are in descending score order.
 * buffers: routing_logits fp32 [T,E], routing_bias bf16 [E], routed_scaling_factor fp32 [1],
 *          expert_ids int32 [T,top_k], route_weights fp32 [T,top_k].  E <= 512 and E % 32 == 0.
 * ---------------------------------------------------------------------------------------- */
typedef struct {
  int64_t tokens;
  int32_t experts, top_k, n_group, topk_group;
  int32_t mode; /* 0 = DeepSeek-V3 group-limited sigmoid, 1 = softmax over the selected top-k */
} cake_b200_routing_config;
int cake_b200_moe_routing_create(void** buffers, const cake_b200_routing_config* config, void** handle_out);
int cake_b200_moe_routing_launch(void* handle, void* cuda_stream);
int cake_b200_moe_routing_destroy(void* handle);

/* ------------------------------------------------------------------------------------------
 * DeepSeek-V4 MoE gate.  Replaces the emitted program of the reference's `deepseek_v4_moe_gate_fp32` task
 * (contract src/open_cake_ir/tasks/deepseek_v4/workload.py:46-108, oracle :190-201;
 * contracts/workloads/deepseek-v4-moe-gate-fp32-triton-b200-v1.json):
 *   score = fp32(sqrt(log1p(exp(router_logits)))); expert_ids = the top_k of score + selection_bias, descending;
 *   weights = fp32(route_scale * score[expert_ids] / sum(score[expert_ids])).  The bias enters the choice only.
 * buffers (the contract's order, outputs `weights` then `expert_ids`): router_logits fp32 [T,E],
 *          selection_bias fp32 [E], weights fp32 [T,top_k], expert_ids int32 [T,top_k].  E <= 512, top_k <= 32.
 * Equal biased scores, which the contract excludes, go to the lower expert id.
 * ---------------------------------------------------------------------------------------- */
typedef struct {
  int64_t tokens;
  int32_t experts, top_k;
  float route_scale; /* 2.5 in the contract */
} cake_b200_v4_gate_config;
int cake_b200_v4_moe_gate_create(void** buffers, const cake_b200_v4_gate_config* config, void** handle_out);
int cake_b200_v4_moe_gate_launch(void* handle, void* cuda_stream);
int cake_b200_v4_moe_gate_destroy(void* handle);

/* ------------------------------------------------------------------------------------------
 * DeepSeek-V4 CSA indexer top-k.  Replaces the emitted program of the reference's
 * `deepseek_v4_csa_indexer_topk_fp32` task (src/open_cake_ir/tasks/deepseek_v4/workload.py:46-108, oracle :188-189;
 * contracts/workloads/deepseek-v4-csa-indexer-topk-fp32-triton-b200-v1.json):
 *   indices[q,:] = positions of the top_k largest index_scores[q,:], in descending score order.
 * buffers: index_scores fp32 [Q,S], indices int32 [Q,top_k].  S <= 2048 (the contract: S 2048, top_k 1024).
 * Equal scores, which the contract excludes, order by ascending position.
 * ---------------------------------------------------------------------------------------- */
typedef struct {
  int64_t rows;
  int32_t candidates, top_k;
} cake_b200_topk_config;
int cake_b200_csa_topk_create(void** buffers, const cake_b200_topk_config* config, void** handle_out);
int cake_b200_csa_topk_launch(void* handle, void* cuda_stream);
int cake_b200_csa_topk_destroy(void* handle);

/* ------------------------------------------------------------------------------------------
 * Token permute.  Fixes the order the reference leaves open (atomic reservation judged by ownership,
 * tools/kernel_oracles.py:186-190; padded gather :137-156): routed (token, slot) pairs whose expert is in
 * [local_expert_offset, +local_experts) are stably sorted by expert.
 * buffers: expert_ids int32 [T,top_k], local_expert_offset int32 [1],
 *          counts int32 [local_experts], offsets int32 [local_experts+1], sorted_pairs int32 [T*top_k],
 *          inv_perm int32 [T*top_k] (-1 for pairs of other ranks).  No workspace.
 * ---------------------------------------------------------------------------------------- */
typedef struct {
  int64_t tokens;
  int32_t top_k, local_experts;
} cake_b200_permute_config;
int cake_b200_moe_permute_create(void** buffers, const cake_b200_permute_config* config, void** handle_out);
int cake_b200_moe_permute_launch(void* handle, void* cuda_stream);
int cake_b200_moe_permute_destroy(void* handle);

/* ------------------------------------------------------------------------------------------
 * FP8 block-scaled MoE expert layer (rank-local).  Replaces the eight-stage launch plan
 * src/open_cake_ir/tasks/solx_fib/moe.py:158-268 for the operator whose oracle is moe.py:122-155:
 * routing -> permute -> grouped GEMM1 (e4m3 x e4m3, fp32 block scales) + SwiGLU (silu on the second half)
 * -> grouped GEMM2 * route weight -> sum over slots -> bf16.
 * buffers (the contract's order, moe.py:13-20): routing_logits fp32 [T,E], routing_bias bf16 [E],
 *   hidden_states e4m3 [T,H], hidden_states_scale fp32 [H/128,T], gemm1_weights e4m3 [E_local,2I,H],
 *   gemm1_weights_scale fp32 [E_local,2I/128,H/128], gemm2_weights e4m3 [E_local,H,I],
 *   gemm2_weights_scale fp32 [E_local,H/128,I/128], local_expert_offset int32 [1],
 *   routed_scaling_factor fp32 [1], output bf16 [T,H], workspace (>= cake_b200_moe_workspace_bytes).
 * act_mode: 0 = intermediate activation requantised to e4m3 per (row,128) with amax/448 scales (one FP8 term);
 *           1 = two FP8 terms (value + residual), which carries the intermediate at better than bf16
 *               precision and meets the reference contract's tolerance against its unquantised oracle.
 * H % 128 == 0, I % 128 == 0.
 * ---------------------------------------------------------------------------------------- */
typedef struct {
  int64_t tokens;
  int32_t hidden, intermediate;
  int32_t experts, local_experts, top_k, n_group, topk_group;
  int32_t routing_mode; /* as cake_b200_routing_config.mode */
  int32_t act_mode;
  int32_t external_routing; /* 1: buffers[0], buffers[1] are expert_ids int32 [T,top_k] and route_weights fp32
                               [T,top_k] produced elsewhere (e.g. after an expert-parallel dispatch); routing is skipped */
} cake_b200_moe_config;
size_t cake_b200_moe_workspace_bytes(const cake_b200_moe_config* config);
int cake_b200_moe_create(void** buffers, const cake_b200_moe_config* config, void** handle_out);
int cake_b200_moe_launch(void* handle, void* cuda_stream);
/* One part of the layer at a time, in order 0..3 (0 routing + permute + gather, 1 grouped GEMM1 + SwiGLU,
 * 2 grouped GEMM2, 3 combine), so that a caller can put events between the parts; launch == stages 0,1,2,3. */
int cake_b200_moe_launch_stage(void* handle, int stage, void* cuda_stream);
int cake_b200_moe_destroy(void* handle);
/* Device pointers of intermediates inside the workspace, for tests and for expert-parallel callers:
 * which = 0 expert_ids int32 [T,top_k]; 1 route_weights fp32 [T,top_k]; 2 counts; 3 offsets; 4 sorted_pairs; 5 inv_perm;
 * 6 the weighted contribution rows bf16 [T*top_k,H] that GEMM2 writes in sorted order (row inv_perm[t,slot] belongs to
 *   token t's slot; the combine stage, or an expert-parallel caller, adds a token's rows in slot order). */
int cake_b200_moe_intermediate(void* handle, int which, void** device_pointer_out);

/* ------------------------------------------------------------------------------------------
 * Paged GQA decode.  Replaces the four-stage attention launch plan
 * src/open_cake_ir/tasks/solx_fib/attention.py:190-331 for the decode operator whose oracle is
 * attention.py:132-183 (spec attention_specs.py:44-84): one query token per sequence,
 *   out = bf16(softmax(K q * sm_scale) V), lse = logsumexp / ln 2 (base 2, -inf and zero output for an empty sequence).
 * buffers: q bf16 [B,Hq,D], k_cache bf16 [pages,page_size,Hkv,D], v_cache (same), kv_indptr int32 [B+1] (pages),
 *          kv_indices int32 [*], kv_last_page_len int32 [B] (extension for page_size > 1; the reference has page_size 1),
 *          sm_scale fp32 [1], output bf16 [B,Hq,D], lse fp32 [B,Hq], workspace.  D == 128; Hq/Hkv in 1..8;
 *          batch <= 65535; max_kv_len <= 2^21.  A launch is two kernels (work list, then decode + merge); the
 *          work is cut on the device from the sequence lengths, so max_kv_len does not enter the workspace size.
 * ---------------------------------------------------------------------------------------- */
typedef struct {
  int64_t batch;
  int32_t num_qo_heads, num_kv_heads, head_dim, page_size;
  int64_t max_kv_len; /* upper bound of any sequence's length, used only to size the split-KV schedule */
} cake_b200_gqa_decode_config;
size_t cake_b200_gqa_decode_workspace_bytes(const cake_b200_gqa_decode_config* config);
int cake_b200_gqa_decode_create(void** buffers, const cake_b200_gqa_decode_config* config, void** handle_out);
int cake_b200_gqa_decode_launch(void* handle, void* cuda_stream);
int cake_b200_gqa_decode_destroy(void* handle);

/* ------------------------------------------------------------------------------------------
 * Paged GQA decode for callers that cannot allocate.  This entry point has no counterpart in the reference.
 * It computes exactly what cake_b200_gqa_decode_* computes, from the same tensors, but takes no workspace and
 * makes no handle: one call validates, launches on `cuda_stream` and returns.  It is meant for hosts that may
 * not touch the CUDA allocator and have no scratch buffer to lend -- a server whose own pool already owns all of
 * device memory, a plug-in sandbox that bans allocator calls, a loop that cannot take the synchronisation an
 * allocation can imply.  The work list, the counters and the split-KV partial results go to a fixed 16 MiB array inside the library image
 * (cake_b200_gqa_decode_noalloc_scratch_limit() returns the size); every GPU that loads the library holds that
 * array until the process exits.  The call uses no cudaMalloc / cudaFree and no allocating library routine.
 *   - Limit: (token ranges + batch) * (num_qo_heads * 129 * 4 + 24) bytes must fit in the array, token ranges being
 *     the SM count (times 8 / num_kv_heads below 8 KV heads); otherwise CAKE_B200_ERR_WORKSPACE (20004).
 *   - The first call on each device looks up the array's device address and sets the kernel's shared-memory
 *     attribute (with that device current); make that first call before starting any stream capture.
 *   - All calls share the array.  Nothing in it has to be cleared: every call rewrites its queue, counters and
 *     work list first and reads back only what it wrote.
 *     Calls that overlap on the GPU race on it; run them one after another.
 * buffers: q, k_cache, v_cache, kv_indptr, kv_indices, kv_last_page_len, sm_scale, output, lse (as above, no workspace).
 * ---------------------------------------------------------------------------------------- */
int cake_b200_gqa_decode_noalloc(void** buffers, const cake_b200_gqa_decode_config* config, void* cuda_stream);
size_t cake_b200_gqa_decode_noalloc_scratch_limit(void);

/* ------------------------------------------------------------------------------------------
 * Paged MLA decode (absorbed form).  Replaces the same four-stage launch plan
 * (src/open_cake_ir/tasks/solx_fib/attention.py:190-331) for the MLA branch of the oracle
 * (attention.py:164-165, :175-177; spec src/open_cake_ir/tasks/solx_fib/attention_specs.py:249-292):
 *   logits = (ckv . q_nope + kpe . q_pe) * sm_scale; out = bf16(softmax(logits) ckv); lse base 2.
 * buffers: q_nope bf16 [B,H,512], q_pe bf16 [B,H,64], ckv_cache bf16 [pages,page_size,512],
 *          kpe_cache bf16 [pages,page_size,64], kv_indptr int32 [B+1], kv_indices int32 [*],
 *          kv_last_page_len int32 [B], sm_scale fp32 [1], output bf16 [B,H,512], lse fp32 [B,H], workspace.
 *          Any H (128 heads per CTA, the last block padded); batch <= 65535.  A launch is three kernels (tile
 *          prefix, decode, merge of the partial results); the work is cut on the device from the sequence
 *          lengths, so max_kv_len does not enter the workspace size.
 * ---------------------------------------------------------------------------------------- */
typedef struct {
  int64_t batch;
  int32_t num_qo_heads, head_dim_ckv, head_dim_kpe, page_size;
  int64_t max_kv_len;
} cake_b200_mla_decode_config;
size_t cake_b200_mla_decode_workspace_bytes(const cake_b200_mla_decode_config* config);
int cake_b200_mla_decode_create(void** buffers, const cake_b200_mla_decode_config* config, void** handle_out);
int cake_b200_mla_decode_launch(void* handle, void* cuda_stream);
int cake_b200_mla_decode_destroy(void* handle);

/* ------------------------------------------------------------------------------------------
 * Causal prefill, GQA over a paged or a ragged KV store.  Replaces the four-stage attention launch plan
 * (src/open_cake_ir/tasks/solx_fib/attention.py:190-331) for the prefill branches of the oracle (attention.py:132-183;
 * specs src/open_cake_ir/tasks/solx_fib/attention_specs.py:85-248): segment b holds query rows
 * [qo_indptr[b], qo_indptr[b+1]) and KV rows [kv_indptr[b], kv_indptr[b+1]) (pages when paged); query row i of a
 * segment with q_len and kv_len rows attends to its first min(kv_len, i + 1 + kv_len - q_len) KV rows (attention.py:170);
 * out bf16, lse base 2.  Empty segments give zeros / -inf; a row of a non-empty segment that sees no KV row gives NaN
 * when nan_for_masked is set (the reference's ragged and MLA tasks, attention.py:47) and zeros otherwise, lse -inf.
 * buffers: q bf16 [total_q,Hq,D], k bf16 and v bf16 ([pages,page_size,Hkv,D] paged; [total_kv,Hkv,D] ragged),
 *          qo_indptr int32 [S+1], kv_indptr int32 [S+1], kv_indices int32 [*] (null when ragged),
 *          kv_last_page_len int32 [S] (null: every page full; null when ragged), sm_scale fp32 [1],
 *          output bf16 [total_q,Hq,D], lse fp32 [total_q,Hq], workspace.  D == 128; Hq/Hkv in 1..8; total_q <= 65535.
 * Every query token is run as a decode sequence of its own over a prefix of its segment's rows.
 * ---------------------------------------------------------------------------------------- */
typedef struct {
  int64_t total_q;
  int32_t segments; /* S */
  int32_t num_qo_heads, num_kv_heads, head_dim, page_size;
  int32_t ragged;         /* 1: k and v are [total_kv,Hkv,D], kv_indptr counts rows, no kv_indices */
  int32_t nan_for_masked; /* 1: a fully masked row of a non-empty segment is NaN */
  int64_t max_kv_len;
} cake_b200_gqa_prefill_config;
size_t cake_b200_gqa_prefill_workspace_bytes(const cake_b200_gqa_prefill_config* config);
int cake_b200_gqa_prefill_create(void** buffers, const cake_b200_gqa_prefill_config* config, void** handle_out);
int cake_b200_gqa_prefill_launch(void* handle, void* cuda_stream);
int cake_b200_gqa_prefill_destroy(void* handle);

/* ------------------------------------------------------------------------------------------
 * Causal prefill, MLA over a paged latent cache (absorbed form); the same rules as above
 * (spec src/open_cake_ir/tasks/solx_fib/attention_specs.py:293-338, oracle attention.py:164-165, :170-177).
 * buffers: q_nope bf16 [total_q,H,512], q_pe bf16 [total_q,H,64], ckv_cache bf16 [pages,page_size,512],
 *          kpe_cache bf16 [pages,page_size,64], qo_indptr int32 [S+1], kv_indptr int32 [S+1], kv_indices int32 [*],
 *          kv_last_page_len int32 [S] (null: every page full), sm_scale fp32 [1], output bf16 [total_q,H,512],
 *          lse fp32 [total_q,H], workspace.  total_q <= 65535.
 * ---------------------------------------------------------------------------------------- */
typedef struct {
  int64_t total_q;
  int32_t segments;
  int32_t num_qo_heads, head_dim_ckv, head_dim_kpe, page_size;
  int32_t nan_for_masked;
  int64_t max_kv_len;
} cake_b200_mla_prefill_config;
size_t cake_b200_mla_prefill_workspace_bytes(const cake_b200_mla_prefill_config* config);
int cake_b200_mla_prefill_create(void** buffers, const cake_b200_mla_prefill_config* config, void** handle_out);
int cake_b200_mla_prefill_launch(void* handle, void* cuda_stream);
int cake_b200_mla_prefill_destroy(void* handle);

/* ------------------------------------------------------------------------------------------
 * Sparse MLA decode (DeepSeek-V3.2 sparse attention).  Implements the operator of the reference's
 * `dsa_attention` contract (contracts/workloads/dsa-attention-sparse-mla-decode-v1.json, validator
 * src/open_cake_ir/tasks/dsa/contract.py:5-78): for each query row and head, the cache rows named by the
 * non-negative entries of sparse_indices[t,:] (token-level row numbers page*page_size + offset; -1 = no entry)
 *   logits = (q_nope . ckv + q_pe . kpe) * sm_scale; out = bf16(softmax over the present entries . ckv);
 *   no present entry => a row of zeros.
 * buffers: q_nope bf16 [T,H,512], q_pe bf16 [T,H,64], ckv_cache bf16 [pages,page_size,512],
 *          kpe_cache bf16 [pages,page_size,64], sparse_indices int32 [T,top_k], output bf16 [T,H,512], workspace.
 * sm_scale is a number of the contract (0.1352337788608801), not a tensor, so it is part of the config.
 * The kernel is the paged MLA decode kernel with the page walk replaced by the index list (16 heads of the
 * contract occupy 16 of its 128 head rows).
 * ---------------------------------------------------------------------------------------- */
typedef struct {
  int64_t num_tokens;      /* query rows */
  int64_t num_cache_rows;  /* pages * page_size: indices must be below it (not checked on the device) */
  int32_t num_qo_heads, head_dim_ckv, head_dim_kpe, top_k;
  float sm_scale;
} cake_b200_sparse_mla_decode_config;
size_t cake_b200_sparse_mla_decode_workspace_bytes(const cake_b200_sparse_mla_decode_config* config);
int cake_b200_sparse_mla_decode_create(void** buffers, const cake_b200_sparse_mla_decode_config* config, void** handle_out);
int cake_b200_sparse_mla_decode_launch(void* handle, void* cuda_stream);
int cake_b200_sparse_mla_decode_destroy(void* handle);

/* ------------------------------------------------------------------------------------------
 * Expert-parallel exchange around the rank-local MoE layer.  The reference holds only the rank-local view
 * (a rank owns experts [local_expert_offset, +local_experts) and other pairs contribute nothing,
 * src/open_cake_ir/tasks/solx_fib/moe.py:139-146); these kernels are the data movement that joins R such ranks.
 * Rank r owns experts [r*experts/world, (r+1)*experts/world).  A token goes once to every rank that owns one
 * of its experts, as a packed row of cake_b200_ep_row_bytes() = H + 4*H/128 + 8*top_k bytes
 * (e4m3 row | K-block scales | expert ids | route weights).  Every rank exchanges exactly `capacity` rows with
 * every peer (unused rows carry expert id -1), so no size ever has to reach the host.
 * buffers: 0 expert_ids int32 [T,top_k], 1 route_weights fp32 [T,top_k], 2 hidden_states e4m3 [T,H],
 *   3 hidden_states_scale fp32 [H/128,T] (inputs, this rank's tokens); 4 slot_of int32 [T,world] (scratch);
 *   5 send u8 [world,capacity,row_bytes] (written by stage 0); 6 recv u8 [world,capacity,row_bytes] (filled by the
 *   caller's all-to-all of `send`); 7..10 the rank-local layer's inputs written by stage 1: hidden e4m3
 *   [world*capacity,H], scales fp32 [H/128,world*capacity], expert_ids int32 and route_weights fp32
 *   [world*capacity,top_k]; 11 returned bf16 [world,capacity,H] (filled by the caller's reverse all-to-all of the
 *   layer's output); 12 output bf16 [T,H] (written by stage 2: partial rows added in rank order in fp32).
 * stages: 0 plan + pack, 1 unpack, 2 reduce.  H % 512 == 0 and top_k even: packed rows are moved with 16-byte loads and
 * stores, so row_bytes must be a multiple of 16; cake_b200_ep_row_bytes returns 0 for any other configuration.
 * ---------------------------------------------------------------------------------------- */
typedef struct {
  int64_t tokens;   /* tokens of this rank */
  int64_t capacity; /* rows exchanged with each peer; >= tokens */
  int32_t hidden, top_k, world, experts;
} cake_b200_ep_config;
size_t cake_b200_ep_row_bytes(const cake_b200_ep_config* config);
int cake_b200_ep_exchange_create(void** buffers, const cake_b200_ep_config* config, void** handle_out);
int cake_b200_ep_exchange_launch_stage(void* handle, int stage, void* cuda_stream);
int cake_b200_ep_exchange_destroy(void* handle);

/* ------------------------------------------------------------------------------------------
 * The same exchange with the ranks writing straight into each other's memory over NVLink instead of through a
 * collective library (no counterpart in the reference, which has no distributed layer).  Every rank owns one
 * SYMMETRIC buffer of cake_b200_ep_push_symmetric_bytes(), zero-filled once, that the host has mapped into every
 * other rank's address space (peer_bases[r] = where rank r's buffer is mapped HERE; peer_bases[rank] = this rank's
 * own).  Only the rows that are needed travel; each side publishes a step number with a system-scope release
 * when its rows are out, and the other side waits for it with a bounded wait (status word 5 on expiry).
 * buffers: 0 expert_ids int32 [T,top_k], 1 route_weights fp32 [T,top_k], 2 hidden_states e4m3 [T,H],
 *   3 hidden_states_scale fp32 [H/128,T] (this rank's tokens); 4 peer_bases uint64 [world] (device array);
 *   5 this rank's symmetric buffer; 6 scratch of cake_b200_ep_push_scratch_bytes(), zero-filled once (its first word
 *   is the status word); 7..10 the rank-local layer's inputs written by stage 1 (hidden e4m3 [world*capacity,H],
 *   scales fp32 [H/128,world*capacity], expert_ids int32 and route_weights fp32 [world*capacity,top_k]; rows beyond
 *   those received carry expert id -1); 11 the layer's contribution rows and 12 its inv_perm
 *   (cake_b200_moe_intermediate 6 and 5; the layer runs its stages 0..2 only); 13 output bf16 [T,H].
 * stages: 0 plan + push rows, 1 wait + unpack, 2 combine + push partial rows back, 3 wait + reduce.  All ranks must
 * run the same sequence of steps; the kernels of a step on different GPUs wait for one another, so they must not
 * share a GPU.
 * ---------------------------------------------------------------------------------------- */
typedef struct {
  int64_t tokens;   /* tokens of this rank */
  int64_t capacity; /* rows a rank can receive from one source; >= the largest `tokens` of any rank */
  int32_t hidden, top_k, world, experts, rank;
} cake_b200_ep_push_config;
size_t cake_b200_ep_push_symmetric_bytes(const cake_b200_ep_push_config* config);
size_t cake_b200_ep_push_scratch_bytes(const cake_b200_ep_push_config* config);
int cake_b200_ep_push_create(void** buffers, const cake_b200_ep_push_config* config, void** handle_out);
int cake_b200_ep_push_launch_stage(void* handle, int stage, void* cuda_stream);
int cake_b200_ep_push_destroy(void* handle);

#ifdef __cplusplus
}
#endif
#endif /* CAKE_B200_H */
