// The runtime of libtvb200: devices, one in-order stream per device, a caching
// device-memory pool, copies, the thread-local last error.
//
// It stands where the reference's Rust runtime stands behind its C ABI
// (crates/vkcore/src/lib.rs:33-76 Runtime{stream, kernels, pool, ctx};
// crates/pyvk/src/ffi.rs): the pool replaces memory.rs's block allocator
// (256-byte alignment, cached blocks reused in stream order, trimmed on
// empty_cache or when the driver is out of memory, memory.rs:150-210), the
// stream replaces stream.rs's batched in-order submission, and the kernel
// cache has no counterpart (the kernels are compiled into this library).
#include "common.h"

#include <cuda.h>
#include <cudaTypedefs.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <vector>

namespace tvb {
namespace {

thread_local std::string g_last_error;

struct Block {
  void* ptr;
  uint64_t size;
  int device;
};

struct DeviceState {
  bool checked = false;
  bool usable = false;
  std::string why;
  std::string name;
  int sms = 0;
  cudaStream_t own_stream = nullptr;
  cudaStream_t stream = nullptr;
  std::multimap<uint64_t, void*> free_blocks;  // cached, unused: size -> pointer
  uint64_t allocated = 0, reserved = 0, blocks = 0;
  void* ws[4] = {nullptr, nullptr, nullptr, nullptr};
  uint64_t ws_size[4] = {0, 0, 0, 0};
  int* status = nullptr;
  int* status_host = nullptr;  // page-locked copy of the status word, filled by a copy queued ahead of each wait
  // the copy-out lane of tvb_memcpy_d2h_overlapped: a second stream, the event that forks it off the main stream and
  // the event that the main stream waits for when the lane is joined
  cudaStream_t copy_stream = nullptr;
  cudaEvent_t fork_event = nullptr, join_event = nullptr;
  bool copies_pending = false;
};

std::mutex g_mutex;
std::vector<DeviceState> g_devices;
bool g_counted = false;
bool g_shutdown = false;
int g_count = 0;
uint64_t g_dispatches = 0;

bool env_flag(const char* name) {
  const char* v = std::getenv(name);
  return v != nullptr && v[0] != '\0' && std::strcmp(v, "0") != 0;
}

int count_devices_locked() {
  if (g_counted) return g_count;
  int n = 0;
  cudaError_t err = cudaGetDeviceCount(&n);
  if (err != cudaSuccess) {
    cudaGetLastError();
    return fail(std::string("no CUDA device: ") + cudaGetErrorString(err));
  }
  g_devices.resize(n);
  g_count = n;
  g_counted = true;
  return n;
}

// Under g_mutex. Checks and initialises device state on first use.
int state_locked(int device, DeviceState** out) {
  int n = count_devices_locked();
  if (n < 0) return -1;
  if (device < 0 || device >= n) return fail("invalid device index " + std::to_string(device) + " (of " + std::to_string(n) + ")");
  DeviceState& d = g_devices[device];
  if (!d.checked) {
    d.checked = true;
    cudaDeviceProp prop{};
    cudaError_t err = cudaGetDeviceProperties(&prop, device);
    if (err != cudaSuccess) {
      d.why = std::string("cudaGetDeviceProperties: ") + cudaGetErrorString(err);
    } else if (prop.major != 10) {
      d.why = std::string("device ") + prop.name + " is sm_" + std::to_string(prop.major * 10 + prop.minor) +
              "; this library holds sm_100a kernels only";
    } else {
      d.usable = true;
      d.name = prop.name;
      d.sms = prop.multiProcessorCount;
    }
  }
  if (!d.usable) return fail(d.why);
  if (d.own_stream == nullptr) {
    cudaError_t err = cudaSetDevice(device);
    if (err == cudaSuccess) err = cudaStreamCreateWithFlags(&d.own_stream, cudaStreamNonBlocking);
    if (err != cudaSuccess) return fail_cuda("cudaStreamCreateWithFlags", err);
    if (d.stream == nullptr) d.stream = d.own_stream;
  }
  *out = &d;
  return 0;
}

uint64_t round_size(uint64_t n) {
  if (n == 0) n = 1;
  if (n < (1u << 20)) return (n + 511) & ~uint64_t(511);
  return (n + (2u << 20) - 1) & ~uint64_t((2u << 20) - 1);
}

void trim_locked(DeviceState& d) {
  for (auto& kv : d.free_blocks) {
    cudaFree(kv.second);
    d.reserved -= kv.first;
    d.blocks -= 1;
  }
  d.free_blocks.clear();
}

}  // namespace

int fail(const std::string& message) {
  g_last_error = message;
  return -1;
}

int fail_cuda(const char* what, cudaError_t err) {
  cudaGetLastError();
  return fail(std::string(what) + ": " + cudaGetErrorName(err) + " (" + cudaGetErrorString(err) + ")");
}

int enter(int device, cudaStream_t* stream) {
  std::lock_guard<std::mutex> lock(g_mutex);
  if (g_shutdown) return fail("the runtime was shut down");
  DeviceState* d = nullptr;
  if (state_locked(device, &d) != 0) return -1;
  cudaError_t err = cudaSetDevice(device);
  if (err != cudaSuccess) return fail_cuda("cudaSetDevice", err);
  *stream = d->stream;
  return 0;
}

int sm_count(int device) {
  std::lock_guard<std::mutex> lock(g_mutex);
  DeviceState* d = nullptr;
  if (state_locked(device, &d) != 0) return 148;
  return d->sms;
}

int workspace(int device, int slot, uint64_t bytes, void** out) {
  std::lock_guard<std::mutex> lock(g_mutex);
  DeviceState* d = nullptr;
  if (state_locked(device, &d) != 0) return -1;
  if (slot < 0 || slot >= 4) return fail("workspace: bad slot");
  if (d->ws_size[slot] < bytes) {
    TVB_CUDA(cudaSetDevice(device));
    if (d->ws[slot] != nullptr) {
      TVB_CUDA(cudaStreamSynchronize(d->stream));
      cudaFree(d->ws[slot]);
      d->ws[slot] = nullptr;
      d->ws_size[slot] = 0;
    }
    uint64_t size = (bytes + 4095) & ~uint64_t(4095);
    TVB_CUDA(cudaMalloc(&d->ws[slot], size));
    TVB_CUDA(cudaMemsetAsync(d->ws[slot], 0, size, d->stream));
    d->ws_size[slot] = size;
  }
  *out = d->ws[slot];
  return 0;
}

int status_word(int device, int** out) {
  std::lock_guard<std::mutex> lock(g_mutex);
  DeviceState* d = nullptr;
  if (state_locked(device, &d) != 0) return -1;
  if (d->status == nullptr) {
    TVB_CUDA(cudaSetDevice(device));
    TVB_CUDA(cudaMalloc(&d->status, 256));
    TVB_CUDA(cudaMemsetAsync(d->status, 0, 256, d->stream));
    TVB_CUDA(cudaHostAlloc(reinterpret_cast<void**>(&d->status_host), 256, cudaHostAllocDefault));
    *d->status_host = 0;
  }
  *out = d->status;
  return 0;
}

int launched(const char* name, dim3 grid, dim3 block, size_t smem, cudaStream_t stream) {
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) return fail(std::string(name) + ": launch failed: " + cudaGetErrorString(err));
  static const bool trace = env_flag("TVB200_TRACE");
  {
    std::lock_guard<std::mutex> lock(g_mutex);
    g_dispatches++;
  }
  if (trace) {
    std::fprintf(stderr, "[tvb200] %s grid %ux%ux%u block %u smem %zu\n", name, grid.x, grid.y, grid.z, block.x, smem);
    err = cudaStreamSynchronize(stream);
    if (err != cudaSuccess) return fail(std::string(name) + ": " + cudaGetErrorString(err));
  }
  return 0;
}

}  // namespace tvb

using namespace tvb;

extern "C" {

const char* tvb_last_error(void) { return g_last_error.c_str(); }

int tvb_device_count(void) {
  std::lock_guard<std::mutex> lock(g_mutex);
  return count_devices_locked();
}

int tvb_set_device(int device) {
  cudaStream_t s;
  return enter(device, &s);
}

int tvb_current_device(void) {
  int d = 0;
  if (cudaGetDevice(&d) != cudaSuccess) {
    cudaGetLastError();
    return fail("no CUDA device");
  }
  return d;
}

int tvb_device_name(int device, char* buf, size_t n) {
  std::lock_guard<std::mutex> lock(g_mutex);
  DeviceState* d = nullptr;
  if (state_locked(device, &d) != 0) return -1;
  if (buf != nullptr && n > 0) {
    std::strncpy(buf, d->name.c_str(), n - 1);
    buf[n - 1] = '\0';
  }
  return 0;
}

uint32_t tvb_capabilities(int device) {
  std::lock_guard<std::mutex> lock(g_mutex);
  DeviceState* d = nullptr;
  if (state_locked(device, &d) != 0) return 0;
  return 1u | 2u | 4u | 8u | 16u | 32u | 64u;
}

int tvb_alloc(int device, uint64_t nbytes, TvbAlloc* out) {
  TVB_REQUIRE(out != nullptr, "tvb_alloc: out is NULL");
  std::lock_guard<std::mutex> lock(g_mutex);
  if (g_shutdown) return fail("the runtime was shut down");
  DeviceState* d = nullptr;
  if (state_locked(device, &d) != 0) return -1;
  uint64_t size = round_size(nbytes);
  void* ptr = nullptr;
  // best fit among cached blocks, not wasting more than a quarter of the block
  auto it = d->free_blocks.lower_bound(size);
  if (it != d->free_blocks.end() && it->first <= size + size / 4 + 4096) {
    size = it->first;
    ptr = it->second;
    d->free_blocks.erase(it);
  } else {
    TVB_CUDA(cudaSetDevice(device));
    cudaError_t err = cudaMalloc(&ptr, size);
    if (err == cudaErrorMemoryAllocation) {  // (trim and retry, as memory.rs:171-179)
      cudaGetLastError();
      cudaStreamSynchronize(d->stream);
      trim_locked(*d);
      err = cudaMalloc(&ptr, size);
    }
    if (err != cudaSuccess) {
      cudaGetLastError();
      return fail("out of device memory allocating " + std::to_string(size) + " bytes (" + cudaGetErrorString(err) + ")");
    }
    d->reserved += size;
    d->blocks += 1;
  }
  d->allocated += size;
  Block* b = new Block{ptr, size, device};
  out->handle = b;
  out->ptr = ptr;
  out->size = size;
  out->device = device;
  out->pad = 0;
  return 0;
}

void tvb_free(void* handle) {
  if (handle == nullptr) return;
  Block* b = static_cast<Block*>(handle);
  {
    std::lock_guard<std::mutex> lock(g_mutex);
    if (!g_shutdown && b->device < static_cast<int>(g_devices.size())) {
      DeviceState& d = g_devices[b->device];
      // Later users of the block are queued on the same stream, so reuse is ordered after the last use.
      d.free_blocks.emplace(b->size, b->ptr);
      d.allocated -= b->size;
    }
  }
  delete b;
}

int tvb_join_copies(int device) {
  cudaStream_t s;
  if (enter(device, &s) != 0) return -1;
  cudaEvent_t join = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_mutex);
    DeviceState& d = g_devices[device];
    if (d.copies_pending) join = d.join_event;
    d.copies_pending = false;
  }
  if (join != nullptr) TVB_CUDA(cudaStreamWaitEvent(s, join, 0));
  return 0;
}

int tvb_synchronize(int device) {
  cudaStream_t s;
  if (enter(device, &s) != 0) return -1;
  if (tvb_join_copies(device) != 0) return -1;
  int* status = nullptr;
  int* status_host = nullptr;
  void* counters = nullptr;
  uint64_t counter_bytes = 0;
  {
    std::lock_guard<std::mutex> lock(g_mutex);
    status = g_devices[device].status;
    status_host = g_devices[device].status_host;
    counters = g_devices[device].ws[0];
    counter_bytes = std::min<uint64_t>(g_devices[device].ws_size[0], 65536);
  }
  // the status word travels behind the queued work, so the wait below is the only round trip to the device
  if (status != nullptr) TVB_CUDA(cudaMemcpyAsync(status_host, status, sizeof(int), cudaMemcpyDeviceToHost, s));
  TVB_CUDA(cudaStreamSynchronize(s));
  if (status != nullptr) {
    const int code = *static_cast<volatile int*>(status_host);
    if (code != 0) {
      cudaMemset(status, 0, sizeof(int));
      // The kernel that gave up left the decode kernels' tile and CTA counters (the head of workspace slot 0) wherever it
      // stopped; they must read zero again before the next launch, or later launches would miscount arrivals.
      if (counters != nullptr && counter_bytes != 0) cudaMemset(counters, 0, counter_bytes);
      return fail("a kernel gave up a bounded wait and left its result incomplete (status " + std::to_string(code) + ")");
    }
  }
  return 0;
}

int tvb_empty_cache(int device) {
  cudaStream_t s;
  if (enter(device, &s) != 0) return -1;
  cudaError_t err = cudaStreamSynchronize(s);
  {
    std::lock_guard<std::mutex> lock(g_mutex);
    DeviceState& d = g_devices[device];
    trim_locked(d);
    // the kernels' large scratch areas (slot 1: the widened weights of tvb_qmm8) go too; they come back on demand
    for (int slot = 1; slot < 4; slot++) {
      if (d.ws[slot] != nullptr) {
        cudaFree(d.ws[slot]);
        d.ws[slot] = nullptr;
        d.ws_size[slot] = 0;
      }
    }
  }
  if (err != cudaSuccess) return fail_cuda("cudaStreamSynchronize", err);
  return 0;
}

void tvb_memory_stats(int device, uint64_t* allocated, uint64_t* reserved, uint64_t* blocks) {
  std::lock_guard<std::mutex> lock(g_mutex);
  uint64_t a = 0, r = 0, b = 0;
  if (g_counted && device >= 0 && device < static_cast<int>(g_devices.size())) {
    a = g_devices[device].allocated;
    r = g_devices[device].reserved;
    b = g_devices[device].blocks;
  }
  if (allocated) *allocated = a;
  if (reserved) *reserved = r;
  if (blocks) *blocks = b;
}

void* tvb_stream(int device) {
  cudaStream_t s = nullptr;
  if (enter(device, &s) != 0) return nullptr;
  return s;
}

int tvb_set_stream(int device, void* stream) {
  std::lock_guard<std::mutex> lock(g_mutex);
  DeviceState* d = nullptr;
  if (state_locked(device, &d) != 0) return -1;
  cudaStream_t next = stream != nullptr ? static_cast<cudaStream_t>(stream) : d->own_stream;
  if (next != d->stream) {
    // The runtime's scratch (counters, partial sums, the status word, cached blocks) is ordered by one stream per device
    // at a time: work queued on the new stream starts after everything already queued on the old one.
    TVB_CUDA(cudaSetDevice(device));
    cudaEvent_t ev = nullptr;
    TVB_CUDA(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
    cudaError_t err = cudaEventRecord(ev, d->stream);
    if (err == cudaSuccess) err = cudaStreamWaitEvent(next, ev, 0);
    cudaEventDestroy(ev);
    if (err != cudaSuccess) return fail_cuda("tvb_set_stream: ordering the new stream after the old one", err);
    d->stream = next;
  }
  return 0;
}

uint64_t tvb_dispatch_count(void) {
  std::lock_guard<std::mutex> lock(g_mutex);
  return g_dispatches;
}

void tvb_shutdown(void) {
  std::lock_guard<std::mutex> lock(g_mutex);
  if (g_shutdown) return;
  g_shutdown = true;
  for (size_t i = 0; i < g_devices.size(); i++) {
    DeviceState& d = g_devices[i];
    if (d.own_stream == nullptr) continue;
    if (cudaSetDevice(static_cast<int>(i)) != cudaSuccess) continue;
    cudaStreamSynchronize(d.stream);
    trim_locked(d);
    for (int w = 0; w < 4; w++) {
      if (d.ws[w] != nullptr) cudaFree(d.ws[w]);
      d.ws[w] = nullptr;
      d.ws_size[w] = 0;
    }
    if (d.status != nullptr) cudaFree(d.status);
    if (d.status_host != nullptr) cudaFreeHost(d.status_host);
    d.status = nullptr;
    d.status_host = nullptr;
    if (d.copy_stream != nullptr) {
      cudaStreamSynchronize(d.copy_stream);
      cudaStreamDestroy(d.copy_stream);
      cudaEventDestroy(d.fork_event);
      cudaEventDestroy(d.join_event);
      d.copy_stream = nullptr;
    }
    cudaStreamDestroy(d.own_stream);
    d.own_stream = d.stream = nullptr;
  }
  cudaGetLastError();
}

int tvb_host_alloc(uint64_t nbytes, void** out) {
  TVB_REQUIRE(out != nullptr, "tvb_host_alloc: out is NULL");
  *out = nullptr;
  if (nbytes == 0) return 0;
  {
    std::lock_guard<std::mutex> lock(g_mutex);
    if (count_devices_locked() <= 0) return fail("no CUDA device: cannot page-lock host memory");
  }
  TVB_CUDA(cudaHostAlloc(out, nbytes, cudaHostAllocPortable));
  return 0;
}

void tvb_host_free(void* ptr) {
  if (ptr != nullptr && cudaFreeHost(ptr) != cudaSuccess) cudaGetLastError();
}

int tvb_host_register(void* ptr, uint64_t nbytes, void** device_ptr) {
  TVB_REQUIRE(ptr != nullptr && nbytes != 0 && device_ptr != nullptr, "tvb_host_register: NULL pointer or empty range");
  cudaStream_t s;
  if (enter(tvb_current_device(), &s) != 0) return -1;
  TVB_CUDA(cudaHostRegister(ptr, nbytes, cudaHostRegisterPortable | cudaHostRegisterMapped));
  void* dev = nullptr;
  cudaError_t err = cudaHostGetDevicePointer(&dev, ptr, 0);
  if (err != cudaSuccess) {
    cudaHostUnregister(ptr);
    return fail_cuda("cudaHostGetDevicePointer", err);
  }
  *device_ptr = dev;
  return 0;
}

int tvb_host_unregister(void* ptr) {
  TVB_REQUIRE(ptr != nullptr, "tvb_host_unregister: NULL pointer");
  TVB_CUDA(cudaHostUnregister(ptr));
  return 0;
}

int tvb_host_is_pinned(const void* ptr) {
  if (ptr == nullptr) return 0;
  {
    std::lock_guard<std::mutex> lock(g_mutex);
    if (!g_counted || g_count <= 0) return 0;  // (never starts CUDA just to answer)
  }
  cudaPointerAttributes attr{};
  if (cudaPointerGetAttributes(&attr, ptr) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return attr.type == cudaMemoryTypeHost ? 1 : 0;
}

int tvb_graph_begin(int device) {
  cudaStream_t s;
  if (enter(device, &s) != 0) return -1;
  TVB_CUDA(cudaStreamBeginCapture(s, cudaStreamCaptureModeRelaxed));
  return 0;
}

int tvb_graph_end(int device, void** graph_exec) {
  TVB_REQUIRE(graph_exec != nullptr, "tvb_graph_end: NULL pointer");
  cudaStream_t s;
  if (enter(device, &s) != 0) return -1;
  if (tvb_join_copies(device) != 0) return -1;  // a recording cannot end with the copy-out lane still forked off
  cudaGraph_t graph = nullptr;
  TVB_CUDA(cudaStreamEndCapture(s, &graph));
  cudaGraphExec_t exec = nullptr;
  cudaError_t err = cudaGraphInstantiate(&exec, graph, 0);
  cudaGraphDestroy(graph);
  if (err != cudaSuccess) return fail_cuda("cudaGraphInstantiate", err);
  *graph_exec = exec;
  return 0;
}

int tvb_graph_launch(int device, void* graph_exec) {
  TVB_REQUIRE(graph_exec != nullptr, "tvb_graph_launch: NULL graph");
  cudaStream_t s;
  if (enter(device, &s) != 0) return -1;
  TVB_CUDA(cudaGraphLaunch(static_cast<cudaGraphExec_t>(graph_exec), s));
  return 0;
}

void tvb_graph_destroy(void* graph_exec) {
  if (graph_exec != nullptr && cudaGraphExecDestroy(static_cast<cudaGraphExec_t>(graph_exec)) != cudaSuccess) cudaGetLastError();
}

// ---- sharing device memory between the ranks of one node (one process per GPU)

int tvb_ipc_export(int device, const void* ptr, uint8_t* handle64, uint64_t* offset) {
  TVB_REQUIRE(ptr != nullptr && handle64 != nullptr && offset != nullptr, "tvb_ipc_export: NULL pointer");
  cudaStream_t s;
  if (enter(device, &s) != 0) return -1;
  // the handle names the whole allocation: find its base
  static PFN_cuMemGetAddressRange_v3020 range_fn = [] {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &fn, cudaEnableDefault, &q) != cudaSuccess) cudaGetLastError();
    return reinterpret_cast<PFN_cuMemGetAddressRange_v3020>(fn);
  }();
  TVB_REQUIRE(range_fn != nullptr, "tvb_ipc_export: cuMemGetAddressRange is not available");
  CUdeviceptr base = 0;
  size_t size = 0;
  TVB_REQUIRE(range_fn(&base, &size, reinterpret_cast<CUdeviceptr>(ptr)) == CUDA_SUCCESS, "tvb_ipc_export: not a device allocation");
  cudaIpcMemHandle_t h;
  TVB_CUDA(cudaIpcGetMemHandle(&h, reinterpret_cast<void*>(base)));
  static_assert(sizeof(h) == 64, "IPC handles are 64 bytes");
  std::memcpy(handle64, &h, 64);
  *offset = reinterpret_cast<uint64_t>(ptr) - static_cast<uint64_t>(base);
  return 0;
}

int tvb_ipc_import(int device, const uint8_t* handle64, uint64_t offset, void** out) {
  TVB_REQUIRE(handle64 != nullptr && out != nullptr, "tvb_ipc_import: NULL pointer");
  cudaStream_t s;
  if (enter(device, &s) != 0) return -1;
  static std::mutex mutex;
  static std::map<std::string, void*> opened;  // a handle may be opened once per process
  std::lock_guard<std::mutex> lock(mutex);
  std::string key(reinterpret_cast<const char*>(handle64), 64);
  key += static_cast<char>(device);
  auto it = opened.find(key);
  void* base = nullptr;
  if (it != opened.end()) {
    base = it->second;
  } else {
    cudaIpcMemHandle_t h;
    std::memcpy(&h, handle64, 64);
    TVB_CUDA(cudaIpcOpenMemHandle(&base, h, cudaIpcMemLazyEnablePeerAccess));
    opened.emplace(key, base);
  }
  *out = static_cast<uint8_t*>(base) + offset;
  return 0;
}

int tvb_memcpy_h2d(int device, void* dst, const void* src, uint64_t nbytes) {
  cudaStream_t s;
  if (enter(device, &s) != 0) return -1;
  if (nbytes == 0) return 0;
  TVB_CUDA(cudaMemcpyAsync(dst, src, nbytes, cudaMemcpyHostToDevice, s));
  return 0;
}

int tvb_memcpy_d2h(int device, void* dst, const void* src, uint64_t nbytes) {
  cudaStream_t s;
  if (enter(device, &s) != 0) return -1;
  if (nbytes == 0) return 0;
  TVB_CUDA(cudaMemcpyAsync(dst, src, nbytes, cudaMemcpyDeviceToHost, s));
  TVB_CUDA(cudaStreamSynchronize(s));
  return 0;
}

int tvb_memcpy_d2h_async(int device, void* dst, const void* src, uint64_t nbytes) {
  cudaStream_t s;
  if (enter(device, &s) != 0) return -1;
  if (nbytes == 0) return 0;
  TVB_REQUIRE(tvb_host_is_pinned(dst) != 0, "tvb_memcpy_d2h_async: the destination must be page-locked host memory");
  TVB_CUDA(cudaMemcpyAsync(dst, src, nbytes, cudaMemcpyDeviceToHost, s));
  return 0;
}

int tvb_memcpy_d2h_overlapped(int device, void* dst, const void* src, uint64_t nbytes) {
  cudaStream_t s;
  if (enter(device, &s) != 0) return -1;
  if (nbytes == 0) return 0;
  TVB_REQUIRE(tvb_host_is_pinned(dst) != 0, "tvb_memcpy_d2h_overlapped: the destination must be page-locked host memory");
  cudaStream_t lane = nullptr;
  cudaEvent_t fork = nullptr, join = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_mutex);
    DeviceState& d = g_devices[device];
    if (d.copy_stream == nullptr) {
      TVB_CUDA(cudaStreamCreateWithFlags(&d.copy_stream, cudaStreamNonBlocking));
      TVB_CUDA(cudaEventCreateWithFlags(&d.fork_event, cudaEventDisableTiming));
      TVB_CUDA(cudaEventCreateWithFlags(&d.join_event, cudaEventDisableTiming));
    }
    lane = d.copy_stream;
    fork = d.fork_event;
    join = d.join_event;
    d.copies_pending = true;
  }
  // the lane takes up where the main stream stands now (inside a recording this is what makes it part of the recording)
  TVB_CUDA(cudaEventRecord(fork, s));
  TVB_CUDA(cudaStreamWaitEvent(lane, fork, 0));
  TVB_CUDA(cudaMemcpyAsync(dst, src, nbytes, cudaMemcpyDeviceToHost, lane));
  TVB_CUDA(cudaEventRecord(join, lane));
  return 0;
}

int tvb_memcpy_d2d(int device, void* dst, const void* src, uint64_t nbytes) {
  cudaStream_t s;
  if (enter(device, &s) != 0) return -1;
  if (nbytes == 0) return 0;
  TVB_CUDA(cudaMemcpyAsync(dst, src, nbytes, cudaMemcpyDeviceToDevice, s));
  return 0;
}

}  // extern "C"
