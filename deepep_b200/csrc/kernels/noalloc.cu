// Allocation-free routing-layout entry point: ep_notify for one rank with library-owned scratch.
// See ../noalloc.h for who needs this and for the limits.  It launches the very same kernel as the
// regular path (launch_notify); only the memory behind the workspace and scratch pointers differs.
#include "../noalloc.h"

#include <mutex>
#include <string>

#include "api.h"

namespace {

using namespace dep;

constexpr int kMaxTokens = DEEPEP_NOALLOC_MAX_TOKENS;
constexpr int kTiles = kMaxTokens / kChunkTokens;

// Layout of the scratch array (byte offsets).  The first part plays the role of a one-rank workspace.
constexpr long long kOffHdr = kControlBytes;
constexpr long long kOffIdx = kOffHdr + 1024;
constexpr long long kOffW = kOffIdx + (long long)kMaxTokens * kMaxTopk * 4;
constexpr long long kOffHist = kOffW + (long long)kMaxTokens * kMaxTopk * 4;
constexpr long long kOffHits = kOffHist + (long long)kTiles * kMaxExperts * 4;
constexpr long long kOffOwnHits = kOffHits + 1024;
constexpr long long kOffCnt = kOffOwnHits + 1024;
constexpr long long kOffRankTokens = kOffCnt + kMaxExperts * 4;
constexpr long long kOffRankRows = kOffRankTokens + 64;
constexpr long long kScratchUsed = kOffRankRows + 64;
static_assert(kScratchUsed <= DEEPEP_NOALLOC_SCRATCH_BYTES, "scratch array is too small for the stated limits");

// Zero-initialised when the module is loaded on a device; lives until the process exits.
static __device__ __align__(256) unsigned char g_scratch[DEEPEP_NOALLOC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
std::mutex g_mutex;
unsigned char* g_device_scratch[kMaxDevices] = {};
thread_local std::string g_error;

int fail(const std::string& message) {
  g_error = message;
  return 1;
}

// Device address of the scratch array on the current device.  In host code `g_scratch` names a host-side
// shadow of the symbol, not device memory: the address a kernel may use has to be asked for, per device.
int scratch_for_current_device(unsigned char** out) {
  int device = -1;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess) return fail(std::string("cudaGetDevice: ") + cudaGetErrorString(e));
  if (device < 0 || device >= kMaxDevices) return fail("device index out of range");
  std::lock_guard<std::mutex> lock(g_mutex);
  if (g_device_scratch[device] == nullptr) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_scratch);
    if (e != cudaSuccess) return fail(std::string("cudaGetSymbolAddress: ") + cudaGetErrorString(e));
    g_device_scratch[device] = static_cast<unsigned char*>(ptr);
  }
  *out = g_device_scratch[device];
  return 0;
}

}  // namespace

extern "C" __attribute__((visibility("default"))) const char* deepep_noalloc_last_error(void) { return g_error.c_str(); }

extern "C" __attribute__((visibility("default"))) int deepep_notify_layout_noalloc(
    const long long* topk_idx, const float* topk_weights, int num_tokens, int num_topk, int num_experts, int expert_alignment,
    int* send_slot, int* slot_row, int* stage_meta, int* chunk_start, int* expert_counts, int* expert_offsets, int* recv_row_src,
    float* recv_weights, long long row_capacity, int* info, void* stream) {
  g_error.clear();
  if (num_tokens < 0 || num_tokens > kMaxTokens)
    return fail("num_tokens exceeds DEEPEP_NOALLOC_MAX_TOKENS (" + std::to_string(kMaxTokens) + "): use the regular entry point");
  if (num_topk < 1 || num_topk > kMaxTopk) return fail("num_topk must be in [1, 16]");
  if (num_experts < 1 || num_experts > kMaxExperts) return fail("num_experts must be in [1, 1024]");
  if (expert_alignment < 1) return fail("expert_alignment must be positive");
  if (!topk_idx || !send_slot || !slot_row || !stage_meta || !chunk_start || !expert_counts || !expert_offsets || !recv_row_src || !info)
    return fail("a required pointer is null");
  // rows the layout can occupy: every routed slot, plus the padding that rounds each expert's block up to the alignment
  const long long rows_needed = (long long)num_tokens * (num_topk < num_experts ? num_topk : num_experts) +
                                (long long)num_experts * (expert_alignment - 1);
  if (row_capacity < rows_needed)
    return fail("row_capacity is smaller than num_tokens * min(num_topk, num_experts) + num_experts * (expert_alignment - 1) = " +
                std::to_string(rows_needed));
  unsigned char* scratch = nullptr;
  if (scratch_for_current_device(&scratch)) return 1;
  cudaStream_t s = static_cast<cudaStream_t>(stream);

  // What must start from zero: the abort word a failed earlier call may have left set.  Epochs and
  // flag words deliberately persist (they only ever grow); every other scratch region is fully
  // rewritten by the kernel before it is read.
  Control* ctl = reinterpret_cast<Control*>(scratch);
  cudaError_t e = cudaMemsetAsync(&ctl->abort, 0, sizeof(int), s);
  if (e != cudaSuccess) return fail(std::string("cudaMemsetAsync: ") + cudaGetErrorString(e));

  NotifyParams p{};
  p.lay.world = 1; p.lay.max_tokens = kMaxTokens; p.lay.hidden = 8; p.lay.topk = num_topk; p.lay.stage_row_bytes = 128;
  p.lay.gather_hdr = kOffHdr; p.lay.gather_idx = kOffIdx; p.lay.gather_w = kOffW;
  p.lay.total = DEEPEP_NOALLOC_SCRATCH_BYTES;
  NotifyArgs& a = p.r[0];
  a.ctx.ws[0] = scratch; a.ctx.status = nullptr; a.ctx.timeout_ns = 2000000000ll; a.ctx.rank = 0; a.ctx.world = 1;
  a.topk_idx = topk_idx; a.topk_w = topk_weights;
  a.T = num_tokens; a.E = num_experts; a.K = num_topk; a.expand = 1; a.alignment = expert_alignment;
  const int per_token = num_topk < num_experts ? num_topk : num_experts;
  a.meta_stride = 2 + (per_token > 2 ? per_token : 2);
  a.hist = reinterpret_cast<int*>(scratch + kOffHist); a.hits = reinterpret_cast<int*>(scratch + kOffHits);
  a.own_hits = reinterpret_cast<int*>(scratch + kOffOwnHits); a.cnt = reinterpret_cast<int*>(scratch + kOffCnt);
  a.rank_tokens = reinterpret_cast<int*>(scratch + kOffRankTokens); a.rank_rows = reinterpret_cast<int*>(scratch + kOffRankRows);
  a.send_slot = send_slot; a.slot_row = slot_row; a.stage_meta = stage_meta; a.chunk_start = chunk_start;
  a.expert_counts = expert_counts; a.expert_offsets = expert_offsets; a.recv_row_src = recv_row_src; a.recv_w = recv_weights;
  a.recv_idx = nullptr; a.mailbox = info; a.rcap = row_capacity;
  e = launch_notify(p, 1, 16, s);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(std::string("kernel launch: ") + cudaGetErrorString(e));
  }
  return 0;
}
