// Gradient of an embedding lookup: dweight[v, :] = sum of grad[i, :] over the positions i with idx[i] == v.
//
// The planner's programs look tokens up with torch.nn.functional.embedding (models.py:66-71); torch's backward
// sorts the indices (eight radix-sort launches) and runs two more kernels for a few thousand tokens - 0.2 ms per
// language-model step for 50 MB of mostly zeros.  Here one kernel does it without a sort and without atomics:
// block i looks at all n indices (n * n compares in total: 67 M for 8192 positions, microseconds); if a later
// position holds the same token it leaves, otherwise it is that token's LAST position and sums the gradient
// rows of all positions with the token, in ascending order of position (fixed order: bit-reproducible), in
// float32, and writes the row once.  Rows no position names are zero (one memset).
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <string>

#include "hapx.h"
#include "hapx_internal.h"

namespace hapx {
namespace embed {

constexpr int kThreads = 128;
constexpr int kWindow = 8 * kThreads;      // positions examined per round: eight consecutive ones per thread

template <typename T>
__global__ void __launch_bounds__(kThreads) embedding_backward_kernel(T* __restrict__ dweight, const T* __restrict__ grad,
                                                                       const long long* __restrict__ idx, int n, int E, long long V) {
  __shared__ int s_list[kWindow];
  __shared__ int s_warp[kThreads / 32];
  const int i = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const long long v = idx[i];
  if (v < 0 || v >= V) return;                    // an index outside the table names no row
  // a later position with the same token owns the row
  int later = 0;
  for (int j = i + 1 + tid; j < n; j += kThreads) later |= (__ldg(idx + j) == v);
  if (__syncthreads_or(later)) return;
  constexpr int G = 8;                            // columns per thread and step
  const int groups = E / G;
  float acc[2][G];                                // up to two column groups per thread (rows of up to 2048 elements)
#pragma unroll
  for (int k = 0; k < G; ++k) { acc[0][k] = 0.f; acc[1][k] = 0.f; }
  for (int w0 = 0; w0 <= i; w0 += kWindow) {
    // the matching positions of this window, in ascending order: per-thread counts, an exclusive prefix sum over the block
    int mine[8], m = 0;
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const int j = w0 + 8 * tid + e;
      if (j <= i && __ldg(idx + j) == v) mine[m++] = j;
    }
    int incl = m;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int t = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += t;
    }
    if (lane == 31) s_warp[warp] = incl;
    __syncthreads();
    int base = 0, total = 0;
#pragma unroll
    for (int q = 0; q < kThreads / 32; ++q) {
      if (q < warp) base += s_warp[q];
      total += s_warp[q];
    }
    for (int e = 0; e < m; ++e) s_list[base + incl - m + e] = mine[e];
    __syncthreads();
    for (int c = 0; c < 2; ++c) {
      const int g = tid + c * kThreads;
      if (g >= groups) break;
      for (int q = 0; q < total; ++q) {
        const T* row = grad + (long long)s_list[q] * E + G * g;
        if constexpr (sizeof(T) == 2) {
          const uint4 x = *reinterpret_cast<const uint4*>(row);
          const unsigned u[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
          for (int k = 0; k < 4; ++k) { acc[c][2 * k] += __uint_as_float(u[k] << 16); acc[c][2 * k + 1] += __uint_as_float(u[k] & 0xffff0000u); }
        } else {
          const float4 a = *reinterpret_cast<const float4*>(row), b = *reinterpret_cast<const float4*>(row + 4);
          acc[c][0] += a.x; acc[c][1] += a.y; acc[c][2] += a.z; acc[c][3] += a.w;
          acc[c][4] += b.x; acc[c][5] += b.y; acc[c][6] += b.z; acc[c][7] += b.w;
        }
      }
    }
    __syncthreads();                              // the list is rewritten in the next round
  }
  for (int c = 0; c < 2; ++c) {
    const int g = tid + c * kThreads;
    if (g >= groups) break;
    T* out = dweight + v * E + G * g;
    if constexpr (sizeof(T) == 2) {
      unsigned o[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const __nv_bfloat162 h = __floats2bfloat162_rn(acc[c][2 * k], acc[c][2 * k + 1]);
        o[k] = *reinterpret_cast<const unsigned*>(&h);
      }
      *reinterpret_cast<uint4*>(out) = make_uint4(o[0], o[1], o[2], o[3]);
    } else {
      *reinterpret_cast<float4*>(out) = make_float4(acc[c][0], acc[c][1], acc[c][2], acc[c][3]);
      *reinterpret_cast<float4*>(out + 4) = make_float4(acc[c][4], acc[c][5], acc[c][6], acc[c][7]);
    }
  }
}

}  // namespace embed
}  // namespace hapx

using namespace hapx;

extern "C" int hapx_embedding_backward(void* dweight, const void* grad, const int64_t* idx, int dtype, int64_t n, int64_t V, int64_t E,
                                       hapx_stream stream_) {
  if (dtype != HAPX_F32 && dtype != HAPX_BF16) return fail(HAPX_ERR_DTYPE, "embedding_backward: float32 or bfloat16 only");
  if (n < 0 || V < 0 || E < 8 || (E & 7) != 0 || E > 2048 || n > (1 << 20))
    return fail(HAPX_ERR_EXTENT, "embedding_backward: rows of 8 ... 2048 elements (a multiple of 8), at most 2^20 positions");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (V == 0) return HAPX_OK;
  if (!dweight) return fail(HAPX_ERR_ARGUMENT, "embedding_backward: null pointer");
  HAPX_CUDA(cudaMemsetAsync(dweight, 0, (size_t)(V * E) * (dtype == HAPX_F32 ? 4 : 2), stream));
  if (n == 0) return HAPX_OK;
  if (!grad || !idx) return fail(HAPX_ERR_ARGUMENT, "embedding_backward: null pointer");
  if (dtype == HAPX_BF16)
    embed::embedding_backward_kernel<__nv_bfloat16><<<(unsigned)n, embed::kThreads, 0, stream>>>(
        static_cast<__nv_bfloat16*>(dweight), static_cast<const __nv_bfloat16*>(grad), reinterpret_cast<const long long*>(idx), (int)n, (int)E, (long long)V);
  else
    embed::embedding_backward_kernel<float><<<(unsigned)n, embed::kThreads, 0, stream>>>(
        static_cast<float*>(dweight), static_cast<const float*>(grad), reinterpret_cast<const long long*>(idx), (int)n, (int)E, (long long)V);
  HAPX_CUDA(cudaGetLastError());
  count_launch(1);
  return HAPX_OK;
}
