// Internal declarations shared by the hapx translation units.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <string>

#include "hapx.h"

namespace hapx {

// ---- error reporting ---------------------------------------------------------
void set_error(const std::string& msg);
int fail(int code, const std::string& msg);
#define HAPX_CUDA(expr)                                                                      \
  do {                                                                                       \
    cudaError_t _e = (expr);                                                                 \
    if (_e != cudaSuccess)                                                                   \
      return ::hapx::fail(HAPX_ERR_CUDA, std::string(#expr) + ": " + cudaGetErrorString(_e)); \
  } while (0)

void count_launch(int n = 1);

// ---- heap layout -----------------------------------------------------------------
// [0, kCtrlBytes)                  control block (flags written by peers, counters, status)
// [kCtrlBytes, +stage_bytes)       staging area for inputs that live outside the heap
// [.., heap_bytes)                 user area
constexpr size_t kCtrlBytes = 4096;

struct Ctrl {
  unsigned long long start[HAPX_MAX_WORLD];  // peer p writes (seq<<40 | offset of its input in its heap)
  unsigned long long done[HAPX_MAX_WORLD];   // peer p writes seq when it has finished reading this rank
  unsigned long long ready[HAPX_MAX_WORLD];  // all_reduce: peer p writes seq when its reduced slice is complete (and it has read all inputs)
  unsigned long long dst_start[HAPX_MAX_WORLD];  // all_reduce: peer p writes (seq<<40 | offset of its OUTPUT in its heap), all ones = not in the heap
  unsigned int cta_done;                     // CTAs of the running kernel that have finished
  unsigned int cta_phase;                    // all_reduce: CTAs that have finished reducing
  unsigned int status;                       // 0, or a hapx_status code left by a kernel (as a positive number)
  unsigned long long status_info;            // (seq<<32 | peer) of the wait that ran out
};
static_assert(sizeof(Ctrl) <= kCtrlBytes, "control block too large");

inline int dtype_size(int dtype) {
  switch (dtype) {
    case HAPX_F32: case HAPX_B32: return 4;
    case HAPX_BF16: case HAPX_F16: case HAPX_B16: return 2;
    case HAPX_F64: case HAPX_B64: return 8;
    case HAPX_B8: return 1;
    default: return 0;
  }
}

namespace gemm {
// One matrix operand (or the output) of a possibly batched bf16 GEMM.  ld and the batch strides
// are in elements; batch index b = b_out * batch_in + b_in addresses ptr + b_out * s_out + b_in * s_in.
// mn_major: the output index (not the contraction index) is the contiguous one in memory.
struct Operand {
  const void* ptr;
  bool mn_major;
  long long ld, s_in, s_out;
};
// D[b] = A[b] * B[b]^T (+ bias, activation) on the tensor cores; see hapx_gemm_sm100.cu.
int gemm_bf16(const Operand& D, int out_f32, const Operand& A, const Operand& B, const void* bias, int epilogue,
              long long M, long long N, long long Kc, int batch_in, int batch_out, cudaStream_t stream);
}  // namespace gemm

}  // namespace hapx

struct hapx_comm {
  int world = 0, n_local = 0, first_rank = 0, device = 0;
  bool local_mode = false;
  size_t heap_bytes = 0, stage_bytes = 0;
  char* heap[HAPX_MAX_WORLD] = {};  // this process's mapping of every rank's heap
  bool mapped[HAPX_MAX_WORLD] = {};
  bool ipc_opened[HAPX_MAX_WORLD] = {};
  unsigned seq = 0;                 // sequence number of the last collective launched
  long long calls = 0;              // collectives launched so far (never wraps; for callers that count them)
  int timeout_ms = 600000;          // bound of a device-side wait on a peer; HAPX_TIMEOUT_MS overrides the default
  // One word of mapped pinned host memory that a kernel sets (besides the status word in the control
  // block) when a wait runs out: the host reads it at the entry of the next call without synchronising.
  unsigned* host_status = nullptr;      // host address
  unsigned* host_status_dev = nullptr;  // the same word as the device sees it
  int max_ctas = 0;
  int fused_all_reduce = -1;        // large all_reduce: 0 two launches, 1 one launch (pull), 2 one launch that may write results into the peers; -1 = 2 between processes, 0 in single-device emulation
  int order_log2 = 6;               // copy kernels interleave 64 tile streams (see pull_copy_kernel)
  int sm_count = 0;
  cudaEvent_t last_done = nullptr;
  cudaStream_t last_stream = nullptr;
  bool any_launched = false;
  bool stream_ordering = true;      // order calls issued on different streams with an event (off while a CUDA graph is captured)
};
