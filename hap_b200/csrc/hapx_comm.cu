// Communicator: per-rank peer-visible heap, CUDA IPC exchange, status words.
//
// Stands in for the part of dist.init_process_group('nccl', ...) (worker.py:18 in the
// reference) that the uneven collectives need: after the exchange every rank holds a
// device pointer to every other rank's heap, so the collective kernels can load peers'
// inputs directly over NVLink.
#include <atomic>
#include <cstdlib>
#include <cstring>
#include <string>

#include "hapx_internal.h"

namespace hapx {

static thread_local std::string g_error;
static std::atomic<long long> g_launches{0};

void set_error(const std::string& msg) { g_error = msg; }
int fail(int code, const std::string& msg) {
  g_error = msg;
  return code;
}
void count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

static int check_sizes(int world, size_t heap_bytes, size_t stage_bytes) {
  if (world < 1 || world > HAPX_MAX_WORLD)
    return fail(HAPX_ERR_ARGUMENT, "world must be in [1, " + std::to_string(HAPX_MAX_WORLD) + "]");
  if (stage_bytes % 256 != 0) return fail(HAPX_ERR_ARGUMENT, "stage_bytes must be a multiple of 256");
  if (heap_bytes < kCtrlBytes + stage_bytes) return fail(HAPX_ERR_ARGUMENT, "heap_bytes smaller than control block + staging area");
  if (heap_bytes >= (1ull << 40)) return fail(HAPX_ERR_ARGUMENT, "heap_bytes must be below 1 TiB");
  return HAPX_OK;
}

static int common_init(hapx_comm* c) {
  if (const char* e = std::getenv("HAPX_TIMEOUT_MS")) {  // default bound of the device-side waits on peers
    long v = std::atol(e);
    if (v >= 1 && v <= 0x7fffffffL) c->timeout_ms = (int)v;
  }
  HAPX_CUDA(cudaSetDevice(c->device));
  HAPX_CUDA(cudaDeviceGetAttribute(&c->sm_count, cudaDevAttrMultiProcessorCount, c->device));
  HAPX_CUDA(cudaEventCreateWithFlags(&c->last_done, cudaEventDisableTiming));
  void* hs = nullptr;
  HAPX_CUDA(cudaHostAlloc(&hs, 64, cudaHostAllocMapped));
  std::memset(hs, 0, 64);
  c->host_status = static_cast<unsigned*>(hs);
  void* ds = nullptr;
  HAPX_CUDA(cudaHostGetDevicePointer(&ds, hs, 0));
  c->host_status_dev = static_cast<unsigned*>(ds);
  return HAPX_OK;
}

static void common_release(hapx_comm* c) {
  if (c->last_done) cudaEventDestroy(c->last_done);
  if (c->host_status) cudaFreeHost(c->host_status);
  c->last_done = nullptr;
  c->host_status = c->host_status_dev = nullptr;
}

}  // namespace hapx

using namespace hapx;

extern "C" {

const char* hapx_last_error(void) { return g_error.c_str(); }
int hapx_version(void) { return 1; }
int64_t hapx_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

int hapx_comm_create(hapx_comm** out, int world, int rank, int device, size_t heap_bytes, size_t stage_bytes) {
  if (!out) return fail(HAPX_ERR_ARGUMENT, "out is null");
  if (int e = check_sizes(world, heap_bytes, stage_bytes)) return e;
  if (rank < 0 || rank >= world) return fail(HAPX_ERR_ARGUMENT, "rank out of range");
  hapx_comm* c = new hapx_comm();
  c->world = world; c->n_local = 1; c->first_rank = rank; c->device = device;
  c->heap_bytes = heap_bytes; c->stage_bytes = stage_bytes;
  if (int e = common_init(c)) { common_release(c); delete c; return e; }
  void* p = nullptr;
  cudaError_t err = cudaMalloc(&p, heap_bytes);
  if (err != cudaSuccess) { common_release(c); delete c; return fail(HAPX_ERR_CUDA, std::string("cudaMalloc(heap): ") + cudaGetErrorString(err)); }
  cudaMemset(p, 0, kCtrlBytes);
  cudaDeviceSynchronize();
  c->heap[rank] = static_cast<char*>(p);
  c->mapped[rank] = true;
  *out = c;
  return HAPX_OK;
}

int hapx_comm_create_local(hapx_comm** out, int world, int device, size_t heap_bytes, size_t stage_bytes) {
  if (!out) return fail(HAPX_ERR_ARGUMENT, "out is null");
  if (int e = check_sizes(world, heap_bytes, stage_bytes)) return e;
  hapx_comm* c = new hapx_comm();
  c->world = world; c->n_local = world; c->first_rank = 0; c->device = device; c->local_mode = true;
  c->heap_bytes = heap_bytes; c->stage_bytes = stage_bytes;
  if (int e = common_init(c)) { common_release(c); delete c; return e; }
  int coop = 0;
  cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, device);
  if (!coop) { common_release(c); delete c; return fail(HAPX_ERR_CUDA, "device does not support cooperative launch"); }
  for (int r = 0; r < world; ++r) {
    void* p = nullptr;
    cudaError_t err = cudaMalloc(&p, heap_bytes);
    if (err != cudaSuccess) {
      for (int q = 0; q < r; ++q) cudaFree(c->heap[q]);
      common_release(c);
      delete c;
      return fail(HAPX_ERR_CUDA, std::string("cudaMalloc(heap): ") + cudaGetErrorString(err));
    }
    cudaMemset(p, 0, kCtrlBytes);
    c->heap[r] = static_cast<char*>(p);
    c->mapped[r] = true;
  }
  cudaDeviceSynchronize();
  *out = c;
  return HAPX_OK;
}

int hapx_comm_ipc_handle(hapx_comm* c, void* out_handle) {
  if (!c || !out_handle) return fail(HAPX_ERR_ARGUMENT, "null argument");
  if (c->local_mode) return fail(HAPX_ERR_STATE, "a local communicator has no IPC handle");
  static_assert(sizeof(cudaIpcMemHandle_t) == HAPX_IPC_HANDLE_BYTES, "handle size");
  HAPX_CUDA(cudaSetDevice(c->device));
  cudaIpcMemHandle_t h;
  HAPX_CUDA(cudaIpcGetMemHandle(&h, c->heap[c->first_rank]));
  std::memcpy(out_handle, &h, sizeof(h));
  return HAPX_OK;
}

int hapx_comm_open_peers(hapx_comm* c, const void* handles) {
  if (!c || !handles) return fail(HAPX_ERR_ARGUMENT, "null argument");
  if (c->local_mode) return fail(HAPX_ERR_STATE, "a local communicator has no peers to open");
  HAPX_CUDA(cudaSetDevice(c->device));
  const char* hs = static_cast<const char*>(handles);
  for (int p = 0; p < c->world; ++p) {
    if (p == c->first_rank || c->mapped[p]) continue;
    cudaIpcMemHandle_t h;
    std::memcpy(&h, hs + (size_t)p * HAPX_IPC_HANDLE_BYTES, sizeof(h));
    void* ptr = nullptr;
    cudaError_t err = cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess);
    if (err != cudaSuccess)
      return fail(HAPX_ERR_CUDA, "cudaIpcOpenMemHandle(rank " + std::to_string(p) + "): " + cudaGetErrorString(err));
    c->heap[p] = static_cast<char*>(ptr);
    c->mapped[p] = true;
    c->ipc_opened[p] = true;
  }
  return HAPX_OK;
}

int hapx_comm_attach_peer(hapx_comm* c, int peer, void* mapped_base) {
  if (!c || !mapped_base) return fail(HAPX_ERR_ARGUMENT, "null argument");
  if (c->local_mode) return fail(HAPX_ERR_STATE, "a local communicator has no peers to attach");
  if (peer < 0 || peer >= c->world || peer == c->first_rank) return fail(HAPX_ERR_ARGUMENT, "peer out of range");
  c->heap[peer] = static_cast<char*>(mapped_base);
  c->mapped[peer] = true;
  return HAPX_OK;
}

int hapx_comm_close_peers(hapx_comm* c) {
  if (!c) return HAPX_OK;
  cudaSetDevice(c->device);
  cudaDeviceSynchronize();
  for (int p = 0; p < c->world; ++p)
    if (c->ipc_opened[p]) {
      cudaIpcCloseMemHandle(c->heap[p]);
      c->ipc_opened[p] = false;
      c->mapped[p] = false;
      c->heap[p] = nullptr;
    }
  return HAPX_OK;
}

int hapx_comm_destroy(hapx_comm* c) {
  if (!c) return HAPX_OK;
  hapx_comm_close_peers(c);
  if (c->local_mode) {
    for (int p = 0; p < c->world; ++p) cudaFree(c->heap[p]);
  } else {
    cudaFree(c->heap[c->first_rank]);
  }
  common_release(c);
  delete c;
  return HAPX_OK;
}

int hapx_comm_calls_issued(hapx_comm* c, int64_t* calls) {
  if (!c || !calls) return fail(HAPX_ERR_ARGUMENT, "null argument");
  *calls = c->calls;
  return HAPX_OK;
}

int hapx_comm_poll(hapx_comm* c) {
  if (!c) return fail(HAPX_ERR_ARGUMENT, "null communicator");
  if (c->host_status && *static_cast<volatile unsigned*>(c->host_status) != 0u)
    return fail(HAPX_ERR_PEER_TIMEOUT, "an earlier collective of this communicator gave up waiting for a peer; its outputs are not valid "
                                       "(hapx_comm_check reports the details and clears the error)");
  return HAPX_OK;
}

int hapx_comm_world(hapx_comm* c, int* world, int* n_local, int* first_rank) {
  if (!c) return fail(HAPX_ERR_ARGUMENT, "null communicator");
  if (world) *world = c->world;
  if (n_local) *n_local = c->n_local;
  if (first_rank) *first_rank = c->first_rank;
  return HAPX_OK;
}

int hapx_comm_heap(hapx_comm* c, int local_index, void** base, size_t* bytes) {
  if (!c) return fail(HAPX_ERR_ARGUMENT, "null communicator");
  if (local_index < 0 || local_index >= c->n_local) return fail(HAPX_ERR_ARGUMENT, "local_index out of range");
  size_t off = kCtrlBytes + c->stage_bytes;
  if (base) *base = c->heap[c->first_rank + local_index] + off;
  if (bytes) *bytes = c->heap_bytes - off;
  return HAPX_OK;
}

int hapx_comm_set_timeout_ms(hapx_comm* c, int ms) {
  if (!c || ms < 1) return fail(HAPX_ERR_ARGUMENT, "bad timeout");
  c->timeout_ms = ms;
  return HAPX_OK;
}

int hapx_comm_set_max_ctas(hapx_comm* c, int ctas) {
  if (!c || ctas < 0) return fail(HAPX_ERR_ARGUMENT, "bad CTA cap");
  c->max_ctas = ctas;
  return HAPX_OK;
}

int hapx_comm_set_fused_all_reduce(hapx_comm* c, int mode) {
  if (!c || mode < -1 || mode > 2) return fail(HAPX_ERR_ARGUMENT, "bad argument");
  c->fused_all_reduce = mode;
  return HAPX_OK;
}

int hapx_comm_set_stream_ordering(hapx_comm* c, int on) {
  if (!c) return fail(HAPX_ERR_ARGUMENT, "null communicator");
  c->stream_ordering = on != 0;
  c->any_launched = false;
  return HAPX_OK;
}

int hapx_comm_check(hapx_comm* c) {
  if (!c) return fail(HAPX_ERR_ARGUMENT, "null communicator");
  HAPX_CUDA(cudaSetDevice(c->device));
  HAPX_CUDA(cudaDeviceSynchronize());
  int rc = HAPX_OK;
  std::string msg;
  for (int i = 0; i < c->n_local; ++i) {
    int r = c->first_rank + i;
    Ctrl host;
    HAPX_CUDA(cudaMemcpy(&host, c->heap[r], sizeof(Ctrl), cudaMemcpyDeviceToHost));
    if (host.status != 0) {
      rc = -static_cast<int>(host.status);
      msg += "rank " + std::to_string(r) + ": device wait ran out (code " + std::to_string(rc) + ", call #" +
             std::to_string(host.status_info >> 32) + ", waiting for rank " +
             std::to_string(host.status_info & 0xffffffffu) + "); ";
      // clear status and the CTA counter so that the communicator stays usable
      HAPX_CUDA(cudaMemset(c->heap[r] + offsetof(Ctrl, cta_done), 0,
                           sizeof(Ctrl) - offsetof(Ctrl, cta_done)));
    }
  }
  if (c->host_status) *static_cast<volatile unsigned*>(c->host_status) = 0u;
  if (rc != HAPX_OK) return fail(rc, msg);
  return HAPX_OK;
}

}  // extern "C"
