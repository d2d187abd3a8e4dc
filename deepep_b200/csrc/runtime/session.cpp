#include "session.h"

#include <cstring>
#include <mutex>
#include <stdexcept>

namespace dep {

CudaApi& cuda_api() {
  static CudaApi api;
  return api;
}

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
}  // namespace

int live_instances() {
  std::lock_guard<std::recursive_mutex> lock(g_mutex);
  int n = 0;
  for (bool s : g_slots) n += s;
  return n;
}

Session::Session(int rank, int world, size_t bytes, double timeout_seconds)
    : rank_(rank), world_(world), bytes_(bytes), timeout_seconds_(timeout_seconds) {
  if (world < 1 || world > kMaxRanks) throw std::invalid_argument("world size must be in [1, 8]");
  if (rank < 0 || rank >= world) throw std::invalid_argument("rank must be in [0, world)");
  if (bytes < (2u << 20) || bytes % (2u << 20)) throw std::invalid_argument("workspace bytes must be a positive multiple of 2 MiB");
  if (!(timeout_seconds > 0) || timeout_seconds > 3600) throw std::invalid_argument("timeout must be in (0, 3600] seconds");
  instance_ = reserve_instance();
  CudaApi& api = cuda_api();
  try {
    check(api.malloc_(reinterpret_cast<void**>(&ws_), bytes_ + kGuardBytes), "workspace allocation");
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
    release_all(true);
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
  cudaIpcMemHandle_t h;
  check(cuda_api().ipc_get_(&h, ws_), "cudaIpcGetMemHandle");
  return std::string(reinterpret_cast<const char*>(&h), sizeof(h));
}

void Session::open_peers(const std::vector<std::string>& handles) {
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
  check(cudaMemset(&c->abort, 0, sizeof(int)), "abort clear");
}

bool Session::guard_intact() const {
  if (!ws_) throw std::runtime_error("the session is closed");
  std::string guard(kGuardBytes, '\0');
  check(cudaMemcpy(&guard[0], ws_ + bytes_, kGuardBytes, cudaMemcpyDeviceToHost), "workspace guard read");
  for (unsigned char c : guard)
    if (c != (unsigned char)kGuardPattern) return false;
  return true;
}

std::string Session::read_control() const {
  std::string out(sizeof(Control), '\0');
  check(cudaMemcpy(&out[0], ws_, sizeof(Control), cudaMemcpyDeviceToHost), "control block read");
  return out;
}

void Session::release_all(bool ignore_errors) {
  CudaApi& api = cuda_api();
  cudaError_t first = cudaSuccess;
  auto note = [&](cudaError_t e) { if (e != cudaSuccess && first == cudaSuccess) first = e; };
  for (int r = 0; r < kMaxRanks; ++r)
    if (opened_[r]) { note(api.ipc_close_(peers_[r])); opened_[r] = false; peers_[r] = nullptr; }
  if (ws_) { note(api.free_(ws_)); ws_ = nullptr; }
  if (status_host_) { note(api.free_host_(status_host_)); status_host_ = nullptr; }
  if (mailbox_host_) { note(api.free_host_(mailbox_host_)); mailbox_host_ = nullptr; }
  if (!ignore_errors) check(first, "session release");
}

void Session::close() {
  if (closed_) return;
  try {
    check(cuda_api().device_sync_(), "device synchronize before close");
    release_all(false);
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
