// Allocation-free entry point (this has no counterpart in the reference library).
//
// Some hosts of this library may not allocate device memory once they are running: a serving
// process that hands the whole GPU to its own memory pool at start-up and then forbids cudaMalloc
// (a late allocation would fail, or stall every stream of the device in the middle of a
// latency-critical step), or a plain C/C++ caller that has no tensor framework whose allocator
// could own the scratch.  For them the routing-layout kernel (ep_notify, single rank) is offered
// with all of its scratch memory inside the library: a file-scope device array of
// DEEPEP_NOALLOC_SCRATCH_BYTES (1 MiB) that every GPU which loads this library holds until the
// process exits.  The caller passes only inputs and outputs.
//
// Limits: one rank, at most DEEPEP_NOALLOC_MAX_TOKENS tokens, top-k <= 16, at most 1024 experts.
// Larger problems are rejected with a non-zero return code and a message (deepep_noalloc_last_error).
//
// The first call on a device looks up the device address of the scratch array (with that device
// current) and remembers it; make that first call before any stream capture begins.  All calls
// share the one scratch array and it keeps the previous call's contents: the entry point resets
// what must start from zero, and two calls that overlap on the GPU (different streams, no
// dependency) race on it -- order them.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

#define DEEPEP_NOALLOC_MAX_TOKENS 4096
#define DEEPEP_NOALLOC_SCRATCH_BYTES (1 << 20)

// Expanded-layout routing metadata of one rank that owns all `num_experts` experts.
//   topk_idx      [num_tokens][num_topk] int64 (device), <0 or >= num_experts marks an empty slot
//   topk_weights  [num_tokens][num_topk] fp32 (device) or NULL
// Outputs (device memory owned by the caller):
//   send_slot      [num_tokens]                       staging index of each token (-1: routed nowhere)
//   slot_row       [num_tokens][num_topk]             output row of each slot (-1: empty)
//   stage_meta     [DEEPEP_NOALLOC_MAX_TOKENS][2 + max(2, min(num_topk, num_experts))]
//   chunk_start    [DEEPEP_NOALLOC_MAX_TOKENS / 64 + 1]
//   expert_counts  [num_experts], expert_offsets [num_experts + 1]
//   recv_row_src   [row_capacity]                     token * num_topk + slot of each output row (-1: padding row)
//   recv_weights   [row_capacity] or NULL
//   row_capacity   must be at least num_tokens * min(num_topk, num_experts) + num_experts * (expert_alignment - 1):
//                  with an alignment above 1 every expert's row block is padded up to a multiple of it, and the padding
//                  rows are written too.  A smaller capacity is rejected before anything is launched.
//   info           [4 + num_experts] int32: rows, staged rows, tokens, call number, then the counts again
// Returns 0 on success.  The work is queued on `stream` (a cudaStream_t); outputs are ready once it drains.
int deepep_notify_layout_noalloc(const long long* topk_idx, const float* topk_weights, int num_tokens, int num_topk,
                                 int num_experts, int expert_alignment, int* send_slot, int* slot_row, int* stage_meta,
                                 int* chunk_start, int* expert_counts, int* expert_offsets, int* recv_row_src,
                                 float* recv_weights, long long row_capacity, int* info, void* stream);

// Text of the last failure reported to this thread ("" if none).
const char* deepep_noalloc_last_error(void);

#ifdef __cplusplus
}
#endif
