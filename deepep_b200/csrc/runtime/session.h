// Session: one rank's symmetric workspace and its mappings of every peer's workspace.
//
// Replaces the reference's SHMEM session (csrc/runtime/session.hpp:20-139, session.cpp:40-189): instead of a
// vendor symmetric heap, each rank allocates its workspace, exports a handle that the Python layer passes to
// the peers, and maps the peers' handles.  All later traffic is loads/stores issued by kernels through these
// mappings over NVLink.  Two transports carry the workspace identity:
//   vmm  the workspace is a physical allocation of the CUDA virtual-memory API (cuMemCreate) mapped into a
//        reserved address range; it is exported as a POSIX file descriptor that the peers receive over a Unix
//        socket, import and map into address ranges of their own;
//   ipc  the workspace is a cudaMalloc allocation exported as a CUDA IPC memory handle (64 bytes that travel
//        through the control plane).
// "auto" takes vmm when the driver supports it on this device and falls back to ipc otherwise.
// A session also owns the status block and the count mailbox, both in mapped pinned host memory, which is how
// kernels report a wait that ran out without trapping.
//
// Teardown is two steps so that no rank frees memory a peer still maps (freeing an exported allocation while an
// importer has it open is undefined): close_peers() on every rank, a barrier of the control plane, then close().
#pragma once
#include <cuda_runtime.h>

#include <string>
#include <vector>

#include "../kernels/common.cuh"

namespace dep {

// Seam for host-side fault injection: tests swap the CUDA entry points for doubles (see fake_cuda.cpp).
// The virtual-memory entries wrap the driver API; they return a CUresult as int (0 = success).
struct CudaApi {
  cudaError_t (*get_device_)(int*);
  cudaError_t (*malloc_)(void**, size_t);
  cudaError_t (*free_)(void*);
  cudaError_t (*memset_)(void*, int, size_t);
  cudaError_t (*memcpy_d2h_)(void*, const void*, size_t);
  cudaError_t (*host_alloc_)(void**, size_t, unsigned);
  cudaError_t (*free_host_)(void*);
  cudaError_t (*host_dev_ptr_)(void**, void*, unsigned);
  cudaError_t (*ipc_get_)(cudaIpcMemHandle_t*, void*);
  cudaError_t (*ipc_open_)(void**, cudaIpcMemHandle_t, unsigned);
  cudaError_t (*ipc_close_)(void*);
  cudaError_t (*device_sync_)();
  int (*vmm_supported_)(int device);                                       // 1 when POSIX-fd shareable allocations work here
  int (*mem_granularity_)(size_t* out, int device);
  int (*mem_create_)(unsigned long long* handle, size_t size, int device);
  int (*mem_export_fd_)(int* fd, unsigned long long handle);
  int (*mem_import_fd_)(unsigned long long* handle, int fd);
  int (*mem_reserve_)(void** va, size_t size, size_t alignment);
  int (*mem_map_)(void* va, size_t size, unsigned long long handle);
  int (*mem_set_access_)(void* va, size_t size, int device);
  int (*mem_unmap_)(void* va, size_t size);
  int (*mem_release_)(unsigned long long handle);
  int (*mem_address_free_)(void* va, size_t size);
  int (*close_fd_)(int fd);
};
CudaApi& cuda_api();          // the table in use
CudaApi real_cuda_api();      // the CUDA runtime / driver

constexpr int kMaxInstances = 128;
constexpr int kMailboxInts = 4 + kMaxExperts;
constexpr size_t kGuardBytes = 4096;      // canary zone behind the workspace, checked by guard_intact()
constexpr int kGuardPattern = 0xA5;

enum class Transport : int { kIpc = 0, kVmm = 1 };

class Session {
 public:
  // transport: "auto", "vmm" or "ipc"
  Session(int rank, int world, size_t bytes, double timeout_seconds, const std::string& transport = "auto");
  ~Session();
  Session(const Session&) = delete;
  Session& operator=(const Session&) = delete;

  const char* transport() const { return transport_ == Transport::kVmm ? "vmm" : "ipc"; }
  std::string ipc_handle() const;                               // ipc: opaque bytes to hand to peers
  int export_fd() const;                                        // vmm: a new file descriptor of the allocation (caller closes it)
  void open_peers(const std::vector<std::string>& handles);     // ipc: one handle per rank; own entry ignored
  void open_peer_fds(const std::vector<int>& fds);              // vmm: one descriptor per rank (own entry ignored); they are closed here
  void attach_peers(const std::vector<uintptr_t>& bases);       // same-process peers (virtual ranks)
  void close_peers();                                           // step 1 of teardown: drop every peer mapping; idempotent
  void close();                                                 // step 2: free the workspace; idempotent; poisons on failure

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
  void allocate_vmm();
  void release_own(bool ignore_errors);
  void release_peers(bool ignore_errors);
  int rank_, world_, instance_ = -1, device_ = 0;
  size_t bytes_, alloc_bytes_ = 0;
  double timeout_seconds_;
  Transport transport_ = Transport::kIpc;
  uint8_t* ws_ = nullptr;
  unsigned long long own_handle_ = 0;
  bool own_handle_live_ = false, own_mapped_ = false;
  uint8_t* peers_[kMaxRanks] = {};
  bool opened_[kMaxRanks] = {};
  unsigned long long peer_handle_[kMaxRanks] = {};
  bool peer_handle_live_[kMaxRanks] = {};
  bool peer_mapped_[kMaxRanks] = {};
  StatusBlock* status_host_ = nullptr;
  StatusBlock* status_dev_ = nullptr;
  int* mailbox_host_ = nullptr;
  int* mailbox_dev_ = nullptr;
  bool closed_ = false, poisoned_ = false;
};

int live_instances();
bool vmm_supported_here();    // the current device and driver can share cuMemCreate allocations as file descriptors

}  // namespace dep
