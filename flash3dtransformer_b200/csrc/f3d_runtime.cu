// Process-wide runtime state of the library: last-error string, sync flag, RNG seed, scratch workspaces.
// Stands in for the reference's DeviceManagerSingleton (src/common/device_manager.cu:32-119): the
// sync_stream debug flag is kept; the per-device cuRAND state array is replaced by a stateless
// counter-based generator, so only a 64-bit seed lives here (default 3407 as in device_manager.cu:58-67).
#include "f3d_common.cuh"
#include "../../include/f3d_b200.h"
#include <mutex>
#include <map>
#include <atomic>
#include <vector>

namespace f3d {

static thread_local char g_err[512] = "";
static std::atomic<int> g_sync{0};
static std::atomic<uint64_t> g_seed{3407ull};
static std::atomic<unsigned long long> g_launches{0ull};
static std::atomic<uint32_t> g_scene_base{0u};

uint32_t scene_base() { return g_scene_base.load(); }

void count_launches(int n) { g_launches.fetch_add((unsigned long long)n); }

char *err_buf() { return g_err; }

int set_error(int code, const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

bool sync_flag() { return g_sync.load() != 0; }
uint64_t seed() { return g_seed.load(); }

struct Slot { void *ptr = nullptr; size_t bytes = 0; unsigned long long last_use = 0; bool in_graph = false; };
struct SlotKey {
  int device, slot;
  cudaStream_t stream;
  bool operator<(const SlotKey &o) const {
    if (device != o.device) return device < o.device;
    if (slot != o.slot) return slot < o.slot;
    return stream < o.stream;
  }
};
static std::mutex g_ws_mu;
static std::map<SlotKey, Slot> g_ws;
static unsigned long long g_ws_clock = 0;
// blocks that a captured CUDA graph refers to and that were later outgrown: kept until f3d_release_workspaces
static std::vector<std::pair<int, void *>> g_ws_retired;
// blocks kept per (device, slot) before the least recently used one is given back: streams come and go, and a
// handle value may belong to a stream that no longer exists
constexpr int kMaxStreamsPerSlot = 8;

int workspace(int device, int slot, size_t bytes, cudaStream_t stream, void **out) {
  std::lock_guard<std::mutex> lk(g_ws_mu);
  const SlotKey key{device, slot, stream};
  // A call recorded into a CUDA graph bakes the block's address into the graph: the block must exist already (nothing
  // may be allocated while a stream is capturing) and is from then on neither evicted nor freed when outgrown.
  cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
  if (stream != nullptr) F3D_CUDA_TRY(cudaStreamIsCapturing(stream, &cap));
  const bool capturing = cap != cudaStreamCaptureStatusNone;
  auto it = g_ws.find(key);
  if (capturing) {
    if (it == g_ws.end() || it->second.bytes < bytes)
      return set_error(F3D_ERR_UNSUPPORTED, "scratch block %d would have to be allocated while the stream is capturing: run the same "
                       "calls once on this stream before the capture", slot);
    it->second.in_graph = true;
    it->second.last_use = ++g_ws_clock;
    *out = it->second.ptr;
    return F3D_OK;
  }
  if (it == g_ws.end()) {
    // a new stream for this slot: evict the least recently used block when the slot holds too many.  Its stream may
    // be gone, so nothing stream-specific is called on it; cudaFree waits for all work of the device by itself.
    int held = 0;
    auto lru = g_ws.end();
    for (auto jt = g_ws.begin(); jt != g_ws.end(); ++jt)
      if (jt->first.device == device && jt->first.slot == slot && !jt->second.in_graph) {
        ++held;
        if (lru == g_ws.end() || jt->second.last_use < lru->second.last_use) lru = jt;
      }
    if (held >= kMaxStreamsPerSlot && lru != g_ws.end()) {
      if (lru->second.ptr) F3D_CUDA_TRY(cudaFree(lru->second.ptr));
      g_ws.erase(lru);
    }
    it = g_ws.emplace(key, Slot{}).first;
  }
  Slot &s = it->second;
  s.last_use = ++g_ws_clock;
  if (s.bytes < bytes) {
    // round up so that slowly growing requests do not reallocate every call
    size_t want = bytes + bytes / 4 + 4096;
    if (s.ptr && s.in_graph) {
      g_ws_retired.emplace_back(device, s.ptr);          // a graph may still be replayed with this address
      s.ptr = nullptr; s.bytes = 0; s.in_graph = false;
    } else if (s.ptr) {
      // only kernels queued on this stream can still be using the old block
      F3D_CUDA_TRY(cudaStreamSynchronize(stream));
      F3D_CUDA_TRY(cudaFree(s.ptr));
      s.ptr = nullptr; s.bytes = 0;
    }
    F3D_CUDA_TRY(cudaMalloc(&s.ptr, want));
    s.bytes = want;
  }
  *out = s.ptr;
  return F3D_OK;
}

static std::mutex g_attr_mu;
static std::map<std::pair<const void *, int>, int> g_attr;

int ensure_dynamic_smem(const void *kernel, int device, int bytes) {
  std::lock_guard<std::mutex> lk(g_attr_mu);
  auto key = std::make_pair(kernel, device);
  auto it = g_attr.find(key);
  if (it != g_attr.end() && it->second >= bytes) return F3D_OK;
  F3D_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
  g_attr[key] = bytes;
  return F3D_OK;
}

static std::map<int, int> g_sms;

int sm_count(int device) {
  std::lock_guard<std::mutex> lk(g_attr_mu);
  auto it = g_sms.find(device);
  if (it != g_sms.end()) return it->second;
  int n = 148;
  cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device);
  g_sms[device] = n;
  return n;
}

static std::mutex g_st_mu;
static std::map<int, int *> g_status;

// Device word that kernels with bounded waits set (once, with atomicCAS) when a wait is abandoned.
int *status_word(int device) {
  std::lock_guard<std::mutex> lk(g_st_mu);
  if (device < 0) { set_error(F3D_ERR_ARG, "device %d out of range", device); return nullptr; }
  auto it = g_status.find(device);
  if (it == g_status.end()) {
    int *p = nullptr;
    if (cudaMalloc(&p, 256) != cudaSuccess || cudaMemset(p, 0, 256) != cudaSuccess) {
      set_error(F3D_ERR_CUDA, "cannot allocate the device status word");
      return nullptr;
    }
    it = g_status.emplace(device, p).first;
  }
  return it->second;
}

void workspace_release_all() {
  std::lock_guard<std::mutex> lk(g_ws_mu);
  int prev = -1;
  cudaGetDevice(&prev);
  for (auto &kv : g_ws) {
    if (kv.second.ptr) { cudaSetDevice(kv.first.device); cudaFree(kv.second.ptr); }
  }
  g_ws.clear();
  for (auto &r : g_ws_retired) { cudaSetDevice(r.first); cudaFree(r.second); }
  g_ws_retired.clear();
  if (prev >= 0) cudaSetDevice(prev);
}

}  // namespace f3d

extern "C" {

const char *f3d_last_error(void) { return f3d::err_buf(); }

int f3d_version(void) { return 100; }

int f3d_set_sync(int on) {
  int old = f3d::g_sync.exchange(on ? 1 : 0);
  return old;
}

int f3d_get_sync(void) { return f3d::g_sync.load(); }

int f3d_set_seed(uint64_t seed) { f3d::g_seed.store(seed); return F3D_OK; }

uint64_t f3d_get_seed(void) { return f3d::g_seed.load(); }

int f3d_set_scene_base(uint32_t base) { f3d::g_scene_base.store(base); return F3D_OK; }

uint32_t f3d_get_scene_base(void) { return f3d::g_scene_base.load(); }

int f3d_init_device(int device) {
  int n = 0;
  F3D_CUDA_TRY(cudaGetDeviceCount(&n));
  if (device < 0 || device >= n) return f3d::set_error(F3D_ERR_ARG, "device %d out of range [0,%d)", device, n);
  cudaDeviceProp p;
  F3D_CUDA_TRY(cudaGetDeviceProperties(&p, device));
  if (p.major != 10) return f3d::set_error(F3D_ERR_UNSUPPORTED, "device %d is sm_%d%d; this library holds sm_100a code only", device, p.major, p.minor);
  return F3D_OK;
}

int f3d_device_status(int device) {
  f3d::DeviceGuard guard(device);
  int *p = f3d::status_word(device);
  if (!p) return F3D_ERR_CUDA;
  int v = 0;
  F3D_CUDA_TRY(cudaDeviceSynchronize());
  F3D_CUDA_TRY(cudaMemcpy(&v, p, sizeof(int), cudaMemcpyDeviceToHost));
  if (v != 0) {
    cudaMemset(p, 0, sizeof(int));
    return f3d::set_error(F3D_ERR_DEVICE_STATUS, "a kernel abandoned a bounded wait (site code %d)", v);
  }
  return F3D_OK;
}

unsigned long long f3d_launch_count(void) { return f3d::g_launches.load(); }

int f3d_release_workspaces(void) { f3d::workspace_release_all(); return F3D_OK; }

}  // extern "C"
