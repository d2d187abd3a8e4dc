// Host-memory doubles of the CUDA entry points behind `CudaApi`, with a call log and fault injection.
//
// They let the session life cycle (construction, peer mapping, the two-step teardown, poisoning after a
// failed release) run and be tested on a machine without a GPU, the way the reference drives its Session
// through link-time doubles of its device runtime (tests/runtime/session_test.cpp, tests/runtime/stubs/).
// "Device" memory is host memory here; a virtual-memory allocation is a memfd that is mmap'ed into a reserved
// range, so a descriptor passed to another process really maps the same bytes there.
#include "fake_cuda.h"

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/syscall.h>
#include <time.h>
#include <unistd.h>

#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>

namespace dep {
namespace fake {
namespace {

std::mutex g_mu;
std::vector<std::pair<std::string, double>> g_log;
struct Fault { int nth; int code; };
std::map<std::string, Fault> g_faults;
std::map<std::string, int> g_calls;
std::map<unsigned long long, int> g_handles;      // allocation handle -> memfd
unsigned long long g_next_handle = 1;
bool g_vmm = true;

double now_seconds() {
  timespec ts;
  clock_gettime(CLOCK_MONOTONIC, &ts);
  return ts.tv_sec + ts.tv_nsec * 1e-9;
}

// Records the call and returns the injected error code for it (0: none).
int enter(const char* name) {
  std::lock_guard<std::mutex> lock(g_mu);
  g_log.emplace_back(name, now_seconds());
  const int n = g_calls[name]++;
  auto it = g_faults.find(name);
  if (it != g_faults.end() && it->second.nth == n) return it->second.code;
  return 0;
}
#define RT_ENTER(name)                                                    \
  if (int code = enter(name)) return static_cast<cudaError_t>(code)
#define DRV_ENTER(name)                                                   \
  if (int code = enter(name)) return code

cudaError_t f_get_device(int* d) { RT_ENTER("get_device"); *d = 0; return cudaSuccess; }
cudaError_t f_malloc(void** p, size_t n) { RT_ENTER("malloc"); *p = std::malloc(n); return *p ? cudaSuccess : cudaErrorMemoryAllocation; }
cudaError_t f_free(void* p) { RT_ENTER("free"); std::free(p); return cudaSuccess; }
cudaError_t f_memset(void* p, int v, size_t n) { RT_ENTER("memset"); std::memset(p, v, n); return cudaSuccess; }
cudaError_t f_memcpy_d2h(void* d, const void* s, size_t n) { RT_ENTER("memcpy_d2h"); std::memcpy(d, s, n); return cudaSuccess; }
cudaError_t f_host_alloc(void** p, size_t n, unsigned) { RT_ENTER("host_alloc"); *p = std::calloc(1, n); return *p ? cudaSuccess : cudaErrorMemoryAllocation; }
cudaError_t f_free_host(void* p) { RT_ENTER("free_host"); std::free(p); return cudaSuccess; }
cudaError_t f_host_dev_ptr(void** d, void* h, unsigned) { RT_ENTER("host_dev_ptr"); *d = h; return cudaSuccess; }
cudaError_t f_ipc_get(cudaIpcMemHandle_t* h, void* p) {
  RT_ENTER("ipc_get");
  std::memset(h, 0, sizeof(*h));
  std::memcpy(h, &p, sizeof(p));
  return cudaSuccess;
}
cudaError_t f_ipc_open(void** p, cudaIpcMemHandle_t h, unsigned) { RT_ENTER("ipc_open"); std::memcpy(p, &h, sizeof(*p)); return cudaSuccess; }
cudaError_t f_ipc_close(void*) { RT_ENTER("ipc_close"); return cudaSuccess; }
cudaError_t f_device_sync() { RT_ENTER("device_sync"); return cudaSuccess; }

int f_vmm_supported(int) { return g_vmm ? 1 : 0; }
int f_mem_granularity(size_t* out, int) { DRV_ENTER("mem_granularity"); *out = 2u << 20; return 0; }
int f_mem_create(unsigned long long* handle, size_t size, int) {
  DRV_ENTER("mem_create");
  const int fd = (int)syscall(SYS_memfd_create, "deepep-fake-vmm", 0u);
  if (fd < 0 || ftruncate(fd, (off_t)size) != 0) return 2;   // out of memory
  std::lock_guard<std::mutex> lock(g_mu);
  *handle = g_next_handle++;
  g_handles[*handle] = fd;
  return 0;
}
int f_mem_export_fd(int* fd, unsigned long long handle) {
  DRV_ENTER("mem_export_fd");
  std::lock_guard<std::mutex> lock(g_mu);
  auto it = g_handles.find(handle);
  if (it == g_handles.end()) return 400;                      // invalid handle
  *fd = dup(it->second);
  return *fd >= 0 ? 0 : 999;
}
int f_mem_import_fd(unsigned long long* handle, int fd) {
  DRV_ENTER("mem_import_fd");
  const int mine = dup(fd);
  if (mine < 0) return 400;
  std::lock_guard<std::mutex> lock(g_mu);
  *handle = g_next_handle++;
  g_handles[*handle] = mine;
  return 0;
}
int f_mem_reserve(void** va, size_t size, size_t) {
  DRV_ENTER("mem_reserve");
  void* p = mmap(nullptr, size, PROT_NONE, MAP_PRIVATE | MAP_ANONYMOUS, -1, 0);
  if (p == MAP_FAILED) return 2;
  *va = p;
  return 0;
}
int f_mem_map(void* va, size_t size, unsigned long long handle) {
  DRV_ENTER("mem_map");
  int fd;
  {
    std::lock_guard<std::mutex> lock(g_mu);
    auto it = g_handles.find(handle);
    if (it == g_handles.end()) return 400;
    fd = it->second;
  }
  return mmap(va, size, PROT_READ | PROT_WRITE, MAP_SHARED | MAP_FIXED, fd, 0) == va ? 0 : 2;
}
int f_mem_set_access(void*, size_t, int) { DRV_ENTER("mem_set_access"); return 0; }
int f_mem_unmap(void* va, size_t size) {
  DRV_ENTER("mem_unmap");
  return mmap(va, size, PROT_NONE, MAP_PRIVATE | MAP_ANONYMOUS | MAP_FIXED, -1, 0) == va ? 0 : 999;   // back to a bare reservation
}
int f_mem_release(unsigned long long handle) {
  DRV_ENTER("mem_release");
  std::lock_guard<std::mutex> lock(g_mu);
  auto it = g_handles.find(handle);
  if (it == g_handles.end()) return 400;
  ::close(it->second);
  g_handles.erase(it);
  return 0;
}
int f_mem_address_free(void* va, size_t size) { DRV_ENTER("mem_address_free"); return munmap(va, size) == 0 ? 0 : 999; }
int f_close_fd(int fd) { DRV_ENTER("close_fd"); return ::close(fd); }

}  // namespace

void install(bool vmm_supported) {
  std::lock_guard<std::mutex> lock(g_mu);
  g_vmm = vmm_supported;
  CudaApi a{};
  a.get_device_ = f_get_device; a.malloc_ = f_malloc; a.free_ = f_free; a.memset_ = f_memset; a.memcpy_d2h_ = f_memcpy_d2h;
  a.host_alloc_ = f_host_alloc; a.free_host_ = f_free_host; a.host_dev_ptr_ = f_host_dev_ptr;
  a.ipc_get_ = f_ipc_get; a.ipc_open_ = f_ipc_open; a.ipc_close_ = f_ipc_close; a.device_sync_ = f_device_sync;
  a.vmm_supported_ = f_vmm_supported; a.mem_granularity_ = f_mem_granularity; a.mem_create_ = f_mem_create;
  a.mem_export_fd_ = f_mem_export_fd; a.mem_import_fd_ = f_mem_import_fd; a.mem_reserve_ = f_mem_reserve; a.mem_map_ = f_mem_map;
  a.mem_set_access_ = f_mem_set_access; a.mem_unmap_ = f_mem_unmap; a.mem_release_ = f_mem_release;
  a.mem_address_free_ = f_mem_address_free; a.close_fd_ = f_close_fd;
  cuda_api() = a;
}

void restore() {
  std::lock_guard<std::mutex> lock(g_mu);
  cuda_api() = real_cuda_api();
  g_faults.clear();
}

void fail(const std::string& entry, int nth, int code) {
  std::lock_guard<std::mutex> lock(g_mu);
  if (code == 0) g_faults.erase(entry);
  else g_faults[entry] = Fault{g_calls[entry] + nth, code};
}

std::vector<std::pair<std::string, double>> log() {
  std::lock_guard<std::mutex> lock(g_mu);
  return g_log;
}

void clear() {
  std::lock_guard<std::mutex> lock(g_mu);
  g_log.clear();
  g_faults.clear();
  g_calls.clear();
  for (auto& h : g_handles) ::close(h.second);    // what an injected release failure left behind
  g_handles.clear();
}

int open_allocations() {
  std::lock_guard<std::mutex> lock(g_mu);
  return (int)g_handles.size();
}

}  // namespace fake
}  // namespace dep
