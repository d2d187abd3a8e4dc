// Session: one rank's symmetric workspace and its mappings of every peer's workspace.
//
// Replaces the reference's SHMEM session (csrc/runtime/session.hpp:20-139, session.cpp:40-189):
// instead of a vendor symmetric heap, each rank allocates its workspace with the CUDA runtime,
// exports an IPC handle that the Python layer exchanges through the process group, and maps
// the peers' handles.  All later traffic is loads/stores issued by kernels through these
// mappings over NVLink.  A session also owns the status block and the count mailbox, both in
// mapped pinned host memory, which is how kernels report a wait that ran out without trapping.
#pragma once
#include <cuda_runtime.h>

#include <string>
#include <vector>

#include "../kernels/common.cuh"

namespace dep {

// Seam for host-side fault injection: tests swap the CUDA entry points for doubles.
struct CudaApi {
  cudaError_t (*malloc_)(void**, size_t) = [](void** p, size_t n) { return cudaMalloc(p, n); };
  cudaError_t (*free_)(void*) = [](void* p) { return cudaFree(p); };
  cudaError_t (*memset_)(void*, int, size_t) = [](void* p, int v, size_t n) { return cudaMemset(p, v, n); };
  cudaError_t (*host_alloc_)(void**, size_t, unsigned) = [](void** p, size_t n, unsigned f) { return cudaHostAlloc(p, n, f); };
  cudaError_t (*free_host_)(void*) = [](void* p) { return cudaFreeHost(p); };
  cudaError_t (*host_dev_ptr_)(void**, void*, unsigned) = [](void** d, void* h, unsigned f) { return cudaHostGetDevicePointer(d, h, f); };
  cudaError_t (*ipc_get_)(cudaIpcMemHandle_t*, void*) = [](cudaIpcMemHandle_t* h, void* p) { return cudaIpcGetMemHandle(h, p); };
  cudaError_t (*ipc_open_)(void**, cudaIpcMemHandle_t, unsigned) = [](void** p, cudaIpcMemHandle_t h, unsigned f) { return cudaIpcOpenMemHandle(p, h, f); };
  cudaError_t (*ipc_close_)(void*) = [](void* p) { return cudaIpcCloseMemHandle(p); };
  cudaError_t (*device_sync_)() = []() { return cudaDeviceSynchronize(); };
};
CudaApi& cuda_api();

constexpr int kMaxInstances = 128;
constexpr int kMailboxInts = 4 + kMaxExperts;
constexpr size_t kGuardBytes = 4096;      // canary zone behind the workspace, checked by guard_intact()
constexpr int kGuardPattern = 0xA5;

class Session {
 public:
  Session(int rank, int world, size_t bytes, double timeout_seconds);
  ~Session();
  Session(const Session&) = delete;
  Session& operator=(const Session&) = delete;

  std::string ipc_handle() const;                               // opaque bytes to hand to peers
  void open_peers(const std::vector<std::string>& handles);     // one handle per rank; own entry ignored
  void attach_peers(const std::vector<uintptr_t>& bases);       // same-process peers (virtual ranks)
  void close();                                                 // idempotent; poisons on failure

  RankCtx ctx() const;
  void set_timeout(double seconds) { timeout_seconds_ = seconds; }
  uintptr_t workspace() const { return reinterpret_cast<uintptr_t>(ws_); }
  uintptr_t peer(int r) const { return reinterpret_cast<uintptr_t>(peers_[r]); }
  size_t bytes() const { return bytes_; }
  int rank() const { return rank_; }
  int world() const { return world_; }
  int instance_id() const { return instance_; }
  bool poisoned() const { return poisoned_; }
  bool closed() const { return closed_; }
  bool mapped() const;                                          // every peer mapping is non-null
  StatusBlock status() const { return *status_host_; }
  void clear_status();                                          // also clears the device abort word
  std::string read_control() const;                             // copy of the control block (diagnostics)
  // The allocation carries a canary zone behind the workspace (peers map it too): true while nobody wrote past the end.
  bool guard_intact() const;
  int* mailbox_host() const { return mailbox_host_; }
  int* mailbox_device() const { return mailbox_dev_; }

 private:
  void release_all(bool ignore_errors);
  int rank_, world_, instance_ = -1;
  size_t bytes_;
  double timeout_seconds_;
  uint8_t* ws_ = nullptr;
  uint8_t* peers_[kMaxRanks] = {};
  bool opened_[kMaxRanks] = {};
  StatusBlock* status_host_ = nullptr;
  StatusBlock* status_dev_ = nullptr;
  int* mailbox_host_ = nullptr;
  int* mailbox_dev_ = nullptr;
  bool closed_ = false, poisoned_ = false;
};

int live_instances();

}  // namespace dep
