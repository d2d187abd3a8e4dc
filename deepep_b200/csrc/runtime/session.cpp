#include "session.h"

#include <cuda.h>
#include <unistd.h>

#include <cstring>
#include <mutex>
#include <stdexcept>

namespace dep {

// ------------------------------------------------------------------------------------------------ the real CUDA entries
namespace {

// Driver entry points are looked up through the runtime, so the module does not link against libcuda.
template <class Fn> Fn driver_fn(const char* name) {
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint(name, &fn, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) return nullptr;
  return reinterpret_cast<Fn>(fn);
}
#define DRIVER(name, ...)                                                  \
  static auto fn = driver_fn<CUresult (*)(__VA_ARGS__)>(#name);            \
  if (!fn) return (int)CUDA_ERROR_NOT_SUPPORTED

CUmemAllocationProp shareable_prop(int device) {
  CUmemAllocationProp prop{};
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = device;
  prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  return prop;
}

int real_vmm_supported(int device) {
  static auto get_attr = driver_fn<CUresult (*)(int*, CUdevice_attribute, CUdevice)>("cuDeviceGetAttribute");
  if (!get_attr) return 0;
  int vmm = 0, fd = 0;
  if (get_attr(&vmm, CU_DEVICE_ATTRIBUTE_VIRTUAL_MEMORY_MANAGEMENT_SUPPORTED, device) != CUDA_SUCCESS) return 0;
  if (get_attr(&fd, CU_DEVICE_ATTRIBUTE_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR_SUPPORTED, device) != CUDA_SUCCESS) return 0;
  return vmm && fd;
}
int real_mem_granularity(size_t* out, int device) {
  DRIVER(cuMemGetAllocationGranularity, size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags);
  CUmemAllocationProp prop = shareable_prop(device);
  return (int)fn(out, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED);
}
int real_mem_create(unsigned long long* handle, size_t size, int device) {
  DRIVER(cuMemCreate, CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long);
  CUmemAllocationProp prop = shareable_prop(device);
  CUmemGenericAllocationHandle h = 0;
  const CUresult r = fn(&h, size, &prop, 0);
  *handle = h;
  return (int)r;
}
int real_mem_export_fd(int* fd, unsigned long long handle) {
  DRIVER(cuMemExportToShareableHandle, void*, CUmemGenericAllocationHandle, CUmemAllocationHandleType, unsigned long long);
  return (int)fn(fd, handle, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
}
int real_mem_import_fd(unsigned long long* handle, int fd) {
  DRIVER(cuMemImportFromShareableHandle, CUmemGenericAllocationHandle*, void*, CUmemAllocationHandleType);
  CUmemGenericAllocationHandle h = 0;
  const CUresult r = fn(&h, reinterpret_cast<void*>(static_cast<uintptr_t>(fd)), CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
  *handle = h;
  return (int)r;
}
int real_mem_reserve(void** va, size_t size, size_t alignment) {
  DRIVER(cuMemAddressReserve, CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long);
  CUdeviceptr p = 0;
  const CUresult r = fn(&p, size, alignment, 0, 0);
  *va = reinterpret_cast<void*>(p);
  return (int)r;
}
int real_mem_map(void* va, size_t size, unsigned long long handle) {
  DRIVER(cuMemMap, CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long);
  return (int)fn(reinterpret_cast<CUdeviceptr>(va), size, 0, handle, 0);
}
int real_mem_set_access(void* va, size_t size, int device) {
  DRIVER(cuMemSetAccess, CUdeviceptr, size_t, const CUmemAccessDesc*, size_t);
  CUmemAccessDesc desc{};
  desc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  desc.location.id = device;
  desc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  return (int)fn(reinterpret_cast<CUdeviceptr>(va), size, &desc, 1);
}
int real_mem_unmap(void* va, size_t size) {
  DRIVER(cuMemUnmap, CUdeviceptr, size_t);
  return (int)fn(reinterpret_cast<CUdeviceptr>(va), size);
}
int real_mem_release(unsigned long long handle) {
  DRIVER(cuMemRelease, CUmemGenericAllocationHandle);
  return (int)fn(handle);
}
int real_mem_address_free(void* va, size_t size) {
  DRIVER(cuMemAddressFree, CUdeviceptr, size_t);
  return (int)fn(reinterpret_cast<CUdeviceptr>(va), size);
}
#undef DRIVER

}  // namespace

CudaApi real_cuda_api() {
  CudaApi a{};
  a.get_device_ = [](int* d) { return cudaGetDevice(d); };
  a.malloc_ = [](void** p, size_t n) { return cudaMalloc(p, n); };
  a.free_ = [](void* p) { return cudaFree(p); };
  a.memset_ = [](void* p, int v, size_t n) { return cudaMemset(p, v, n); };
  a.memcpy_d2h_ = [](void* d, const void* s, size_t n) { return cudaMemcpy(d, s, n, cudaMemcpyDeviceToHost); };
  a.host_alloc_ = [](void** p, size_t n, unsigned f) { return cudaHostAlloc(p, n, f); };
  a.free_host_ = [](void* p) { return cudaFreeHost(p); };
  a.host_dev_ptr_ = [](void** d, void* h, unsigned f) { return cudaHostGetDevicePointer(d, h, f); };
  a.ipc_get_ = [](cudaIpcMemHandle_t* h, void* p) { return cudaIpcGetMemHandle(h, p); };
  a.ipc_open_ = [](void** p, cudaIpcMemHandle_t h, unsigned f) { return cudaIpcOpenMemHandle(p, h, f); };
  a.ipc_close_ = [](void* p) { return cudaIpcCloseMemHandle(p); };
  a.device_sync_ = []() { return cudaDeviceSynchronize(); };
  a.vmm_supported_ = real_vmm_supported;
  a.mem_granularity_ = real_mem_granularity;
  a.mem_create_ = real_mem_create;
  a.mem_export_fd_ = real_mem_export_fd;
  a.mem_import_fd_ = real_mem_import_fd;
  a.mem_reserve_ = real_mem_reserve;
  a.mem_map_ = real_mem_map;
  a.mem_set_access_ = real_mem_set_access;
  a.mem_unmap_ = real_mem_unmap;
  a.mem_release_ = real_mem_release;
  a.mem_address_free_ = real_mem_address_free;
  a.close_fd_ = [](int fd) { return ::close(fd); };
  return a;
}

CudaApi& cuda_api() {
  static CudaApi api = real_cuda_api();
  return api;
}

// ------------------------------------------------------------------------------------------------ instance registry
namespace {
std::recursive_mutex g_mutex;
bool g_slots[kMaxInstances] = {};

int reserve_instance() {
  std::lock_guard<std::recursive_mutex> lock(g_mutex);
  for (int i = 0; i < kMaxInstances; ++i)
    if (!g_slots[i]) { g_slots[i] = true; return i; }
  throw std::runtime_error("too many live sessions in this process (limit 128)");
}
void release_instance(int id) {
  std::lock_guard<std::recursive_mutex> lock(g_mutex);
  if (id >= 0) g_slots[id] = false;
}
void check(cudaError_t e, const char* what) {
  if (e != cudaSuccess) throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
}
void check_drv(int r, const char* what) {
  if (r != 0) throw std::runtime_error(std::string(what) + ": CUDA driver error " + std::to_string(r));
}
size_t round_up(size_t v, size_t a) { return (v + a - 1) / a * a; }
}  // namespace

int live_instances() {
  std::lock_guard<std::recursive_mutex> lock(g_mutex);
  int n = 0;
  for (bool s : g_slots) n += s;
  return n;
}

bool vmm_supported_here() {
  int device = 0;
  if (cuda_api().get_device_(&device) != cudaSuccess) return false;
  return cuda_api().vmm_supported_(device) != 0;
}

// ------------------------------------------------------------------------------------------------ session
void Session::allocate_vmm() {
  CudaApi& api = cuda_api();
  size_t gran = 0;
  check_drv(api.mem_granularity_(&gran, device_), "cuMemGetAllocationGranularity");
  if (gran == 0) gran = 2u << 20;
  alloc_bytes_ = round_up(bytes_ + kGuardBytes, gran);
  check_drv(api.mem_create_(&own_handle_, alloc_bytes_, device_), "cuMemCreate");
  own_handle_live_ = true;
  void* va = nullptr;
  check_drv(api.mem_reserve_(&va, alloc_bytes_, gran), "cuMemAddressReserve");
  ws_ = static_cast<uint8_t*>(va);
  check_drv(api.mem_map_(ws_, alloc_bytes_, own_handle_), "cuMemMap");
  own_mapped_ = true;
  check_drv(api.mem_set_access_(ws_, alloc_bytes_, device_), "cuMemSetAccess");
}

Session::Session(int rank, int world, size_t bytes, double timeout_seconds, const std::string& transport)
    : rank_(rank), world_(world), bytes_(bytes), timeout_seconds_(timeout_seconds) {
  if (world < 1 || world > kMaxRanks) throw std::invalid_argument("world size must be in [1, 8]");
  if (rank < 0 || rank >= world) throw std::invalid_argument("rank must be in [0, world)");
  if (bytes < (2u << 20) || bytes % (2u << 20)) throw std::invalid_argument("workspace bytes must be a positive multiple of 2 MiB");
  if (!(timeout_seconds > 0) || timeout_seconds > 3600) throw std::invalid_argument("timeout must be in (0, 3600] seconds");
  if (transport != "auto" && transport != "vmm" && transport != "ipc") throw std::invalid_argument("transport must be 'auto', 'vmm' or 'ipc'");
  instance_ = reserve_instance();
  CudaApi& api = cuda_api();
  try {
    check(api.get_device_(&device_), "cudaGetDevice");
    bool want_vmm = transport == "vmm" || (transport == "auto" && api.vmm_supported_(device_) != 0);
    if (want_vmm) {
      try {
        allocate_vmm();
        transport_ = Transport::kVmm;
      } catch (...) {
        release_own(true);
        if (transport == "vmm") throw;
        want_vmm = false;          // "auto": the runtime allocator still works
      }
    }
    if (!want_vmm) {
      transport_ = Transport::kIpc;
      alloc_bytes_ = bytes_ + kGuardBytes;
      check(api.malloc_(reinterpret_cast<void**>(&ws_), alloc_bytes_), "workspace allocation");
    }
    check(api.memset_(ws_, 0, bytes_), "workspace clear");
    check(api.memset_(ws_ + bytes_, kGuardPattern, kGuardBytes), "workspace guard fill");
    check(api.host_alloc_(reinterpret_cast<void**>(&status_host_), sizeof(StatusBlock), cudaHostAllocMapped), "status block allocation");
    std::memset(status_host_, 0, sizeof(StatusBlock));
    check(api.host_dev_ptr_(reinterpret_cast<void**>(&status_dev_), status_host_, 0), "status block mapping");
    check(api.host_alloc_(reinterpret_cast<void**>(&mailbox_host_), kMailboxInts * sizeof(int), cudaHostAllocMapped), "mailbox allocation");
    std::memset(mailbox_host_, 0, kMailboxInts * sizeof(int));
    check(api.host_dev_ptr_(reinterpret_cast<void**>(&mailbox_dev_), mailbox_host_, 0), "mailbox mapping");
    check(api.device_sync_(), "workspace clear (sync)");
  } catch (...) {
    release_own(true);
    release_instance(instance_);
    instance_ = -1;
    throw;
  }
  peers_[rank_] = ws_;
}

Session::~Session() {
  if (!closed_) {
    try { close(); } catch (...) {}
  }
}

std::string Session::ipc_handle() const {
  if (transport_ != Transport::kIpc) throw std::runtime_error("this session shares its workspace as a file descriptor (vmm), not as an IPC handle");
  cudaIpcMemHandle_t h;
  check(cuda_api().ipc_get_(&h, ws_), "cudaIpcGetMemHandle");
  return std::string(reinterpret_cast<const char*>(&h), sizeof(h));
}

int Session::export_fd() const {
  if (transport_ != Transport::kVmm) throw std::runtime_error("this session shares its workspace as an IPC handle, not as a file descriptor");
  int fd = -1;
  check_drv(cuda_api().mem_export_fd_(&fd, own_handle_), "cuMemExportToShareableHandle");
  return fd;
}

void Session::open_peers(const std::vector<std::string>& handles) {
  if (transport_ != Transport::kIpc) throw std::runtime_error("open_peers is the ipc transport's; use open_peer_fds");
  if ((int)handles.size() != world_) throw std::invalid_argument("one handle per rank is required");
  for (int r = 0; r < world_; ++r) {
    if (r == rank_) continue;
    if (handles[r].size() != sizeof(cudaIpcMemHandle_t)) throw std::invalid_argument("malformed IPC handle");
    cudaIpcMemHandle_t h;
    std::memcpy(&h, handles[r].data(), sizeof(h));
    void* p = nullptr;
    check(cuda_api().ipc_open_(&p, h, cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle");
    peers_[r] = static_cast<uint8_t*>(p);
    opened_[r] = true;
  }
}

void Session::open_peer_fds(const std::vector<int>& fds) {
  CudaApi& api = cuda_api();
  auto close_all = [&]() {
    for (int r = 0; r < (int)fds.size(); ++r)
      if (r != rank_ && fds[r] >= 0) api.close_fd_(fds[r]);
  };
  if (transport_ != Transport::kVmm) { close_all(); throw std::runtime_error("open_peer_fds is the vmm transport's; use open_peers"); }
  if ((int)fds.size() != world_) { close_all(); throw std::invalid_argument("one file descriptor per rank is required"); }
  try {
    size_t gran = 0;
    check_drv(api.mem_granularity_(&gran, device_), "cuMemGetAllocationGranularity");
    if (gran == 0) gran = 2u << 20;
    for (int r = 0; r < world_; ++r) {
      if (r == rank_) continue;
      if (fds[r] < 0) throw std::invalid_argument("missing file descriptor of a peer");
      check_drv(api.mem_import_fd_(&peer_handle_[r], fds[r]), "cuMemImportFromShareableHandle");
      peer_handle_live_[r] = true;
      void* va = nullptr;
      check_drv(api.mem_reserve_(&va, alloc_bytes_, gran), "cuMemAddressReserve (peer)");
      peers_[r] = static_cast<uint8_t*>(va);
      opened_[r] = true;
      check_drv(api.mem_map_(va, alloc_bytes_, peer_handle_[r]), "cuMemMap (peer)");
      peer_mapped_[r] = true;
      check_drv(api.mem_set_access_(va, alloc_bytes_, device_), "cuMemSetAccess (peer)");
    }
  } catch (...) {
    close_all();
    release_peers(true);
    throw;
  }
  close_all();     // the imported handles keep the allocations alive; the descriptors are no longer needed
}

void Session::attach_peers(const std::vector<uintptr_t>& bases) {
  if ((int)bases.size() != world_) throw std::invalid_argument("one base pointer per rank is required");
  for (int r = 0; r < world_; ++r)
    if (r != rank_) peers_[r] = reinterpret_cast<uint8_t*>(bases[r]);
}

bool Session::mapped() const {
  for (int r = 0; r < world_; ++r)
    if (peers_[r] == nullptr) return false;
  return true;
}

RankCtx Session::ctx() const {
  if (closed_) throw std::runtime_error("session is closed");
  if (poisoned_) throw std::runtime_error("A previous communication launch failed; restart the distributed job");
  RankCtx c{};
  for (int r = 0; r < world_; ++r) c.ws[r] = peers_[r];
  c.status = status_dev_;
  c.timeout_ns = (long long)(timeout_seconds_ * 1e9);
  c.rank = rank_;
  c.world = world_;
  return c;
}

void Session::clear_status() {
  std::memset(status_host_, 0, sizeof(StatusBlock));
  Control* c = control_of(ws_);
  check(cuda_api().memset_(&c->abort, 0, sizeof(int)), "abort clear");
}

bool Session::guard_intact() const {
  if (!ws_) throw std::runtime_error("the session is closed");
  std::string guard(kGuardBytes, '\0');
  check(cuda_api().memcpy_d2h_(&guard[0], ws_ + bytes_, kGuardBytes), "workspace guard read");
  for (unsigned char c : guard)
    if (c != (unsigned char)kGuardPattern) return false;
  return true;
}

std::string Session::read_control() const {
  std::string out(sizeof(Control), '\0');
  check(cuda_api().memcpy_d2h_(&out[0], ws_, sizeof(Control)), "control block read");
  return out;
}

void Session::release_peers(bool ignore_errors) {
  CudaApi& api = cuda_api();
  std::string first;
  auto note = [&](bool failed, const char* what) { if (failed && first.empty()) first = what; };
  for (int r = 0; r < kMaxRanks; ++r) {
    if (r == rank_) continue;
    if (transport_ == Transport::kVmm) {
      if (peer_mapped_[r]) { note(api.mem_unmap_(peers_[r], alloc_bytes_) != 0, "cuMemUnmap (peer)"); peer_mapped_[r] = false; }
      if (opened_[r]) { note(api.mem_address_free_(peers_[r], alloc_bytes_) != 0, "cuMemAddressFree (peer)"); opened_[r] = false; }
      if (peer_handle_live_[r]) { note(api.mem_release_(peer_handle_[r]) != 0, "cuMemRelease (peer)"); peer_handle_live_[r] = false; }
    } else if (opened_[r]) {
      note(api.ipc_close_(peers_[r]) != cudaSuccess, "cudaIpcCloseMemHandle");
      opened_[r] = false;
    }
    peers_[r] = nullptr;
  }
  if (!ignore_errors && !first.empty()) throw std::runtime_error("session release: " + first + " failed");
}

void Session::release_own(bool ignore_errors) {
  CudaApi& api = cuda_api();
  std::string first;
  auto note = [&](bool failed, const char* what) { if (failed && first.empty()) first = what; };
  if (transport_ == Transport::kVmm || own_handle_live_) {
    if (own_mapped_) { note(api.mem_unmap_(ws_, alloc_bytes_) != 0, "cuMemUnmap"); own_mapped_ = false; }
    if (ws_) { note(api.mem_address_free_(ws_, alloc_bytes_) != 0, "cuMemAddressFree"); ws_ = nullptr; }
    if (own_handle_live_) { note(api.mem_release_(own_handle_) != 0, "cuMemRelease"); own_handle_live_ = false; }
  } else if (ws_) {
    note(api.free_(ws_) != cudaSuccess, "cudaFree");
    ws_ = nullptr;
  }
  if (status_host_) { note(api.free_host_(status_host_) != cudaSuccess, "cudaFreeHost (status)"); status_host_ = nullptr; }
  if (mailbox_host_) { note(api.free_host_(mailbox_host_) != cudaSuccess, "cudaFreeHost (mailbox)"); mailbox_host_ = nullptr; }
  if (!ignore_errors && !first.empty()) throw std::runtime_error("session release: " + first + " failed");
}

void Session::close_peers() {
  if (closed_) return;
  try {
    check(cuda_api().device_sync_(), "device synchronize before unmapping the peers");
    release_peers(false);
  } catch (...) {
    poisoned_ = true;
    throw;
  }
}

void Session::close() {
  if (closed_) return;
  try {
    check(cuda_api().device_sync_(), "device synchronize before close");
    release_peers(false);
    release_own(false);
  } catch (...) {
    poisoned_ = true;   // the instance slot stays reserved: the process must restart
    closed_ = true;
    throw;
  }
  closed_ = true;
  release_instance(instance_);
  instance_ = -1;
}

}  // namespace dep
