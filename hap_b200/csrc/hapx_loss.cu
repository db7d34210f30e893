// Loss of the language-model and classification programs: log_softmax over the last dimension
// followed by nll_loss(reduction='sum') (the ops the planner emits at hap.rs:1808 and hap.rs:1858;
// models.py:116-117 in the reference), as one pass over the logits in each direction.
//
// HBM-bound: forward reads the logits once (2 bytes per element in bf16) and writes 8 bytes per
// row; backward reads them once more and writes the gradient (4 bytes per element in bf16).  The
// separate ops move a float copy of the logits, the log-probabilities and two gradients of that
// size instead (about 22 bytes per element).
#include <cuda_bf16.h>
#include <math_constants.h>

#include "hapx_internal.h"

namespace hapx {
namespace loss {

constexpr int kThreads = 256;

template <typename T>
struct Elem;
template <>
struct Elem<float> {
  static constexpr int N = 4;     // elements per 16-byte load
  static __device__ __forceinline__ void unpack(const uint4& v, float (&f)[8]) {
    f[0] = __uint_as_float(v.x); f[1] = __uint_as_float(v.y); f[2] = __uint_as_float(v.z); f[3] = __uint_as_float(v.w);
  }
  static __device__ __forceinline__ uint4 pack(const float (&f)[8]) {
    return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]), __float_as_uint(f[3]));
  }
  static __device__ __forceinline__ float load(const float* p) { return *p; }
  static __device__ __forceinline__ void store(float* p, float x) { *p = x; }
};
template <>
struct Elem<__nv_bfloat16> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void unpack(const uint4& v, float (&f)[8]) {
    const unsigned w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) { f[2 * i] = __uint_as_float(w[i] << 16); f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u); }
  }
  static __device__ __forceinline__ uint4 pack(const float (&f)[8]) {
    unsigned w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const __nv_bfloat162 h = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
      w[i] = *reinterpret_cast<const unsigned*>(&h);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
  }
  static __device__ __forceinline__ float load(const __nv_bfloat16* p) { return __bfloat162float(*p); }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, float x) { *p = __float2bfloat16_rn(x); }
};

// (running maximum, sum of exp(x - maximum)) pairs combine associatively
__device__ __forceinline__ void combine(float& m, float& s, float m2, float s2) {
  const float mx = fmaxf(m, m2);
  if (mx == -CUDART_INF_F) { m = mx; s = 0.f; return; }
  s = s * __expf(m - mx) + s2 * __expf(m2 - mx);
  m = mx;
}

// One block per row: log-sum-exp of the row and the row's loss lse - x[target].
// Rows whose target is outside [0, V) (torch's ignore_index = -100 among them) cost nothing.
template <typename T>
__global__ void __launch_bounds__(kThreads) nll_forward_kernel(const T* __restrict__ logits, const long long* __restrict__ targets,
                                                               float* __restrict__ row_loss, float* __restrict__ row_lse,
                                                               long long rows, int V, long long pitch) {
  using E = Elem<T>;
  __shared__ float s_m[kThreads / 32], s_s[kThreads / 32];
  for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
    const T* x = logits + row * pitch;
    float m = -CUDART_INF_F, s = 0.f;
    const bool vec = ((reinterpret_cast<uintptr_t>(x) & 15u) == 0);
    const int full = vec ? (V / E::N) * E::N : 0;
#pragma unroll 4
    for (int i = threadIdx.x * E::N; i < full; i += kThreads * E::N) {
      float f[8];
      E::unpack(*reinterpret_cast<const uint4*>(x + i), f);
      float vm = f[0];
#pragma unroll
      for (int k = 1; k < E::N; ++k) vm = fmaxf(vm, f[k]);
      if (vm > m) { s *= __expf(m - vm); m = vm; }     // m = -inf at first: s is 0 and stays 0
      if (m != -CUDART_INF_F) {
#pragma unroll
        for (int k = 0; k < E::N; ++k) s += __expf(f[k] - m);
      }
    }
    for (int i = full + threadIdx.x; i < V; i += kThreads) {
      const float f = E::load(x + i);
      if (f > m) { s *= __expf(m - f); m = f; }
      if (m != -CUDART_INF_F) s += __expf(f - m);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float m2 = __shfl_xor_sync(0xffffffffu, m, o), s2 = __shfl_xor_sync(0xffffffffu, s, o);
      combine(m, s, m2, s2);
    }
    if ((threadIdx.x & 31) == 0) { s_m[threadIdx.x >> 5] = m; s_s[threadIdx.x >> 5] = s; }
    __syncthreads();
    if (threadIdx.x == 0) {
      float M = s_m[0], S = s_s[0];
#pragma unroll
      for (int w = 1; w < kThreads / 32; ++w) combine(M, S, s_m[w], s_s[w]);
      const float lse = M + logf(S);
      const long long t = targets[row];
      row_lse[row] = lse;
      row_loss[row] = (t >= 0 && t < V) ? lse - E::load(x + t) : 0.f;
    }
    __syncthreads();
  }
}

// grad[row][c] = gout * (exp(x - lse[row]) - [c == target[row]]); zero rows for ignored targets.
template <typename T>
__global__ void __launch_bounds__(kThreads) nll_backward_kernel(const T* __restrict__ logits, const long long* __restrict__ targets,
                                                                const float* __restrict__ row_lse, const float* __restrict__ gout,
                                                                T* __restrict__ grad, long long rows, int V, long long pitch,
                                                                long long gpitch) {
  using E = Elem<T>;
  const float go = *gout;
  for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
    const T* x = logits + row * pitch;
    T* g = grad + row * gpitch;
    const long long t = targets[row];
    const bool live = t >= 0 && t < V;
    const float lse = row_lse[row], scale = live ? go : 0.f;
    const bool vec = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(g)) & 15u) == 0;
    const int full = vec ? (V / E::N) * E::N : 0;
#pragma unroll 4
    for (int i = threadIdx.x * E::N; i < full; i += kThreads * E::N) {
      float f[8];
      E::unpack(*reinterpret_cast<const uint4*>(x + i), f);
#pragma unroll
      for (int k = 0; k < E::N; ++k) f[k] = scale * (__expf(f[k] - lse) - ((long long)(i + k) == t ? 1.f : 0.f));
      *reinterpret_cast<uint4*>(g + i) = E::pack(f);
    }
    for (int i = full + threadIdx.x; i < V; i += kThreads)
      E::store(g + i, scale * (__expf(E::load(x + i) - lse) - ((long long)i == t ? 1.f : 0.f)));
  }
}

static int grid_rows(long long rows) {
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const long long cap = (long long)sms * 8;
  return (int)(rows < cap ? (rows < 1 ? 1 : rows) : cap);
}

}  // namespace loss
}  // namespace hapx

using namespace hapx;
using namespace hapx::loss;

extern "C" {

int hapx_nll_logsoftmax_forward(const void* logits, const int64_t* targets, float* row_loss, float* row_lse, int dtype,
                                int64_t rows, int64_t classes, int64_t pitch, hapx_stream stream_) {
  if (rows < 0 || classes < 1 || classes > 0x7fffffff || pitch < classes) return fail(HAPX_ERR_ARGUMENT, "nll_logsoftmax_forward: bad extents");
  if (rows == 0) return HAPX_OK;
  if (!logits || !targets || !row_loss || !row_lse) return fail(HAPX_ERR_ARGUMENT, "nll_logsoftmax_forward: null argument");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const int grid = grid_rows(rows);
  if (dtype == HAPX_BF16)
    nll_forward_kernel<__nv_bfloat16><<<grid, kThreads, 0, stream>>>(static_cast<const __nv_bfloat16*>(logits),
                                                                     reinterpret_cast<const long long*>(targets), row_loss, row_lse,
                                                                     rows, (int)classes, pitch);
  else if (dtype == HAPX_F32)
    nll_forward_kernel<float><<<grid, kThreads, 0, stream>>>(static_cast<const float*>(logits), reinterpret_cast<const long long*>(targets),
                                                             row_loss, row_lse, rows, (int)classes, pitch);
  else
    return fail(HAPX_ERR_DTYPE, "nll_logsoftmax_forward: float32 or bfloat16 only");
  HAPX_CUDA(cudaGetLastError());
  count_launch(1);
  return HAPX_OK;
}

int hapx_nll_logsoftmax_backward(const void* logits, const int64_t* targets, const float* row_lse, const float* grad_out, void* grad_logits,
                                 int dtype, int64_t rows, int64_t classes, int64_t pitch, int64_t grad_pitch, hapx_stream stream_) {
  if (rows < 0 || classes < 1 || classes > 0x7fffffff || pitch < classes || grad_pitch < classes)
    return fail(HAPX_ERR_ARGUMENT, "nll_logsoftmax_backward: bad extents");
  if (rows == 0) return HAPX_OK;
  if (!logits || !targets || !row_lse || !grad_out || !grad_logits) return fail(HAPX_ERR_ARGUMENT, "nll_logsoftmax_backward: null argument");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const int grid = grid_rows(rows);
  if (dtype == HAPX_BF16)
    nll_backward_kernel<__nv_bfloat16><<<grid, kThreads, 0, stream>>>(static_cast<const __nv_bfloat16*>(logits),
                                                                      reinterpret_cast<const long long*>(targets), row_lse, grad_out,
                                                                      static_cast<__nv_bfloat16*>(grad_logits), rows, (int)classes, pitch,
                                                                      grad_pitch);
  else if (dtype == HAPX_F32)
    nll_backward_kernel<float><<<grid, kThreads, 0, stream>>>(static_cast<const float*>(logits), reinterpret_cast<const long long*>(targets),
                                                              row_lse, grad_out, static_cast<float*>(grad_logits), rows, (int)classes, pitch,
                                                              grad_pitch);
  else
    return fail(HAPX_ERR_DTYPE, "nll_logsoftmax_backward: float32 or bfloat16 only");
  HAPX_CUDA(cudaGetLastError());
  count_launch(1);
  return HAPX_OK;
}

}  // extern "C"
