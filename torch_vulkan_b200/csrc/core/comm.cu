// Collectives behind the C ABI: the all-gather that assembles the column slices of a sharded product on every rank, for
// hosts that bind the library without PyTorch (tvb_comm_*; the reference has one device and no counterpart:
// crates/pyvk/csrc/backend.cpp:296). NCCL over NVLink does the moving; this file owns the communicator's life cycle the
// way a serving host needs it: non-blocking communicators, every call bounded by a host-side timeout, and abort instead
// of a hang when a peer has gone.
//
// NCCL is not linked: it is looked up at run time (TVB200_NCCL_LIB, else the libnccl.so.2 the process already has or can
// find), so the library loads on hosts that never shard.
#include <cuda_runtime.h>
#include <dlfcn.h>
#include <nccl.h>

#include <chrono>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <thread>

#include "common.h"

namespace tvb {
namespace {

struct NcclApi {
  ncclResult_t (*GetUniqueId)(ncclUniqueId*);
  ncclResult_t (*CommInitRankConfig)(ncclComm_t*, int, ncclUniqueId, int, ncclConfig_t*);
  ncclResult_t (*CommInitAll)(ncclComm_t*, int, const int*);
  ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t);
  ncclResult_t (*CommAbort)(ncclComm_t);
  ncclResult_t (*CommDestroy)(ncclComm_t);
  ncclResult_t (*CommGetAsyncError)(ncclComm_t, ncclResult_t*);
  const char* (*GetErrorString)(ncclResult_t);
  bool ok = false;
  std::string why;
};

NcclApi* nccl() {
  static NcclApi api;
  static std::once_flag once;
  std::call_once(once, [] {
    void* lib = nullptr;
    if (const char* path = std::getenv("TVB200_NCCL_LIB")) lib = dlopen(path, RTLD_NOW | RTLD_GLOBAL);
    if (lib == nullptr) lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);  // the one the process already uses, if any
    if (lib == nullptr) lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (lib == nullptr) lib = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (lib == nullptr) {
      api.why = "NCCL was not found (set TVB200_NCCL_LIB to libnccl.so.2)";
      return;
    }
    auto sym = [&](const char* name) { return dlsym(lib, name); };
    api.GetUniqueId = reinterpret_cast<decltype(api.GetUniqueId)>(sym("ncclGetUniqueId"));
    api.CommInitRankConfig = reinterpret_cast<decltype(api.CommInitRankConfig)>(sym("ncclCommInitRankConfig"));
    api.CommInitAll = reinterpret_cast<decltype(api.CommInitAll)>(sym("ncclCommInitAll"));
    api.AllGather = reinterpret_cast<decltype(api.AllGather)>(sym("ncclAllGather"));
    api.CommAbort = reinterpret_cast<decltype(api.CommAbort)>(sym("ncclCommAbort"));
    api.CommDestroy = reinterpret_cast<decltype(api.CommDestroy)>(sym("ncclCommDestroy"));
    api.CommGetAsyncError = reinterpret_cast<decltype(api.CommGetAsyncError)>(sym("ncclCommGetAsyncError"));
    api.GetErrorString = reinterpret_cast<decltype(api.GetErrorString)>(sym("ncclGetErrorString"));
    api.ok = api.GetUniqueId && api.CommInitRankConfig && api.CommInitAll && api.AllGather && api.CommAbort && api.CommDestroy &&
             api.CommGetAsyncError && api.GetErrorString;
    if (!api.ok) api.why = "the NCCL library lacks a required entry point";
  });
  return &api;
}

struct Comm {
  ncclComm_t comm = nullptr;
  int device = 0, world = 1, rank = 0;
  bool aborted = false;
};

int fail_nccl(const char* what, ncclResult_t rc) { return fail(std::string(what) + ": " + nccl()->GetErrorString(rc)); }

// Polls a non-blocking communicator until its pending call has finished; aborts it when `timeout_ms` runs out or it fails.
int settle(Comm* c, const char* what, int timeout_ms) {
  const auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms);
  for (;;) {
    ncclResult_t state = ncclSuccess;
    ncclResult_t rc = nccl()->CommGetAsyncError(c->comm, &state);
    if (rc != ncclSuccess) state = rc;
    if (state == ncclSuccess) return 0;
    if (state != ncclInProgress || std::chrono::steady_clock::now() > deadline) {
      nccl()->CommAbort(c->comm);
      c->aborted = true;
      if (state == ncclInProgress) return fail(std::string(what) + ": no answer from the other ranks within the time limit; communicator aborted");
      return fail_nccl(what, state);
    }
    std::this_thread::sleep_for(std::chrono::microseconds(200));
  }
}

// [world][m][n_local] (what the all-gather delivers) -> [m][world * n_local], `vec` bytes at a time.
template <typename V>
__global__ void interleave_columns_kernel(const V* __restrict__ src, V* __restrict__ dst, int world, int64_t m, int64_t row_vecs) {
  const int64_t total = static_cast<int64_t>(world) * m * row_vecs;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t v = i % row_vecs, row = (i / row_vecs) % m;
    const int r = static_cast<int>(i / (row_vecs * m));
    dst[(row * world + r) * row_vecs + v] = src[i];
  }
}

constexpr int kDefaultTimeoutMs = 30000;

}  // namespace
}  // namespace tvb

using namespace tvb;

extern "C" int tvb_comm_unique_id(uint8_t* id128) {
  TVB_REQUIRE(id128 != nullptr, "tvb_comm_unique_id: NULL pointer");
  TVB_REQUIRE(nccl()->ok, "tvb_comm_unique_id: " + nccl()->why);
  ncclUniqueId id;
  static_assert(sizeof(id) == 128, "NCCL ids are 128 bytes");
  ncclResult_t rc = nccl()->GetUniqueId(&id);
  if (rc != ncclSuccess) return fail_nccl("ncclGetUniqueId", rc);
  std::memcpy(id128, &id, 128);
  return 0;
}

extern "C" int tvb_comm_init_rank(int device, const uint8_t* id128, int world, int rank, int timeout_ms, void** comm_out) {
  TVB_REQUIRE(id128 != nullptr && comm_out != nullptr, "tvb_comm_init_rank: NULL pointer");
  TVB_REQUIRE(world >= 1 && rank >= 0 && rank < world, "tvb_comm_init_rank: bad rank");
  TVB_REQUIRE(nccl()->ok, "tvb_comm_init_rank: " + nccl()->why);
  cudaStream_t stream;
  if (enter(device, &stream) != 0) return -1;
  ncclUniqueId id;
  std::memcpy(&id, id128, 128);
  ncclConfig_t config = NCCL_CONFIG_INITIALIZER;
  config.blocking = 0;  // every call returns at once; settle() bounds the wait and aborts instead of hanging
  Comm* c = new Comm();
  c->device = device;
  c->world = world;
  c->rank = rank;
  ncclResult_t rc = nccl()->CommInitRankConfig(&c->comm, world, id, rank, &config);
  if (rc != ncclSuccess && rc != ncclInProgress) {
    delete c;
    return fail_nccl("ncclCommInitRankConfig", rc);
  }
  if (settle(c, "tvb_comm_init_rank", timeout_ms > 0 ? timeout_ms : kDefaultTimeoutMs) != 0) {
    delete c;
    return -1;
  }
  *comm_out = c;
  return 0;
}

extern "C" int tvb_comm_init_all(const int* devices, int ndev, void** comms_out) {
  TVB_REQUIRE(devices != nullptr && comms_out != nullptr && ndev >= 1 && ndev <= 64, "tvb_comm_init_all: bad arguments");
  TVB_REQUIRE(nccl()->ok, "tvb_comm_init_all: " + nccl()->why);
  for (int i = 0; i < ndev; i++) {
    cudaStream_t stream;
    if (enter(devices[i], &stream) != 0) return -1;
  }
  ncclComm_t raw[64];
  ncclResult_t rc = nccl()->CommInitAll(raw, ndev, devices);
  if (rc != ncclSuccess) return fail_nccl("ncclCommInitAll", rc);
  for (int i = 0; i < ndev; i++) {
    Comm* c = new Comm();
    c->comm = raw[i];
    c->device = devices[i];
    c->world = ndev;
    c->rank = i;
    comms_out[i] = c;
  }
  return 0;
}

extern "C" int tvb_all_gather(void* comm, const void* send, void* recv, uint64_t nbytes) {
  TVB_REQUIRE(comm != nullptr && send != nullptr && recv != nullptr, "tvb_all_gather: NULL pointer");
  Comm* c = static_cast<Comm*>(comm);
  TVB_REQUIRE(!c->aborted, "tvb_all_gather: the communicator was aborted");
  cudaStream_t stream;
  if (enter(c->device, &stream) != 0) return -1;
  ncclResult_t rc = nccl()->AllGather(send, recv, nbytes, ncclUint8, c->comm, stream);
  if (rc != ncclSuccess && rc != ncclInProgress) return fail_nccl("ncclAllGather", rc);
  return settle(c, "tvb_all_gather", kDefaultTimeoutMs);  // (the call has been queued; the data moves on the stream)
}

extern "C" int tvb_all_gather_columns(void* comm, const void* c_local, void* c_full, int dtype, int64_t m, int64_t n_local) {
  TVB_REQUIRE(comm != nullptr && c_local != nullptr && c_full != nullptr, "tvb_all_gather_columns: NULL pointer");
  TVB_REQUIRE(m >= 1 && n_local >= 1 && dtype_size(dtype) > 0, "tvb_all_gather_columns: bad shape or dtype");
  Comm* c = static_cast<Comm*>(comm);
  const uint64_t row_bytes = static_cast<uint64_t>(n_local) * dtype_size(dtype);
  if (m == 1 || c->world == 1) return tvb_all_gather(comm, c_local, c_full, static_cast<uint64_t>(m) * row_bytes);
  // the ranks' slices arrive one after the other; the rows are then interleaved into [m, world * n_local]
  void* ws = nullptr;
  if (workspace(c->device, 3, 256 + static_cast<uint64_t>(c->world) * m * row_bytes, &ws) != 0) return -1;
  uint8_t* staged = static_cast<uint8_t*>(ws) + 256;  // (the slot's first 256 bytes hold a kernel's counter)
  if (tvb_all_gather(comm, c_local, staged, static_cast<uint64_t>(m) * row_bytes) != 0) return -1;
  cudaStream_t stream;
  if (enter(c->device, &stream) != 0) return -1;
  const bool vec16 = row_bytes % 16 == 0 && (reinterpret_cast<uintptr_t>(c_full) & 15u) == 0;
  const int64_t row_vecs = static_cast<int64_t>(vec16 ? row_bytes / 16 : row_bytes);
  const int64_t total = static_cast<int64_t>(c->world) * m * row_vecs;
  const int grid = static_cast<int>(std::min<int64_t>(ceil_div(total, 256), static_cast<int64_t>(sm_count(c->device)) * 8));
  if (vec16)
    interleave_columns_kernel<uint4><<<grid, 256, 0, stream>>>(reinterpret_cast<const uint4*>(staged), static_cast<uint4*>(c_full), c->world, m, row_vecs);
  else
    interleave_columns_kernel<uint8_t><<<grid, 256, 0, stream>>>(staged, static_cast<uint8_t*>(c_full), c->world, m, row_vecs);
  return launched("interleave_columns", dim3(grid), dim3(256), 0, stream);
}

extern "C" int tvb_comm_wait(void* comm, int timeout_ms) {
  TVB_REQUIRE(comm != nullptr, "tvb_comm_wait: NULL communicator");
  Comm* c = static_cast<Comm*>(comm);
  TVB_REQUIRE(!c->aborted, "tvb_comm_wait: the communicator was aborted");
  cudaStream_t stream;
  if (enter(c->device, &stream) != 0) return -1;
  const auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms > 0 ? timeout_ms : kDefaultTimeoutMs);
  for (;;) {
    cudaError_t q = cudaStreamQuery(stream);
    if (q == cudaSuccess) return 0;
    if (q != cudaErrorNotReady) return fail_cuda("tvb_comm_wait: cudaStreamQuery", q);
    ncclResult_t state = ncclSuccess;
    nccl()->CommGetAsyncError(c->comm, &state);
    if ((state != ncclSuccess && state != ncclInProgress) || std::chrono::steady_clock::now() > deadline) {
      // a peer has gone or is late beyond the limit: abort frees the collective's kernel, so the stream drains
      nccl()->CommAbort(c->comm);
      c->aborted = true;
      return fail("tvb_comm_wait: the collective did not finish within the time limit; communicator aborted");
    }
    std::this_thread::sleep_for(std::chrono::microseconds(200));
  }
}

extern "C" int tvb_comm_abort(void* comm) {
  if (comm == nullptr) return 0;
  Comm* c = static_cast<Comm*>(comm);
  if (!c->aborted && nccl()->ok) nccl()->CommAbort(c->comm);
  c->aborted = true;
  delete c;
  return 0;
}

extern "C" int tvb_comm_destroy(void* comm) {
  if (comm == nullptr) return 0;
  Comm* c = static_cast<Comm*>(comm);
  if (!c->aborted && nccl()->ok) {
    cudaStream_t stream;
    if (enter(c->device, &stream) == 0) cudaStreamSynchronize(stream);
    nccl()->CommDestroy(c->comm);
  }
  delete c;
  return 0;
}
