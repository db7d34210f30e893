// torch.nn.functional.dropout(x, p) as the planner emits it (hap.rs:1446-1464), forward and backward,
// and the generator state shared with the attention kernels' dropout.
//
// y = x * keep / (1 - p), keep ~ Bernoulli(1 - p) from the counter-based generator of hapx_rng.h; the
// backward pass applies the same function to the incoming gradient, re-deriving the mask from
// (seed, iteration, call id, element index) instead of reading a stored one.  HBM bound: one read and
// one write per element, 8 elements per thread and generator evaluation.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <mutex>
#include <string>

#include "hapx_internal.h"
#include "hapx_rng.h"

namespace hapx {

namespace {
rng::State* g_state[64] = {};
std::mutex g_state_mutex;

__global__ void rng_seed_kernel(rng::State* st, unsigned long long seed) { st->seed = seed; st->epoch = 0ull; }
__global__ void rng_advance_kernel(rng::State* st) { st->epoch += 1ull; }

template <typename T>
__global__ void __launch_bounds__(256) dropout_kernel(const T* __restrict__ x, T* __restrict__ y, long long n, unsigned threshold, float scale,
                                                      const rng::State* st, unsigned long long call_id) {
  const rng::Key key = rng::make_key(st, call_id);
  const long long groups = (n + 7) / 8;
  for (long long g = (long long)blockIdx.x * blockDim.x + threadIdx.x; g < groups; g += (long long)gridDim.x * blockDim.x) {
    const unsigned keep = rng::keep_bits(rng::philox(key, (unsigned long long)g), threshold);
    const long long e0 = g * 8;
    if (e0 + 8 <= n && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & (8 * sizeof(T) - 1)) == 0) {
      if constexpr (sizeof(T) == 2) {
        uint4 v = *reinterpret_cast<const uint4*>(x + e0);
        unsigned w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float lo = (keep >> (2 * i)) & 1u ? __uint_as_float(w[i] << 16) * scale : 0.f;
          const float hi = (keep >> (2 * i + 1)) & 1u ? __uint_as_float(w[i] & 0xffff0000u) * scale : 0.f;
          const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
          w[i] = *reinterpret_cast<const unsigned*>(&h);
        }
        *reinterpret_cast<uint4*>(y + e0) = make_uint4(w[0], w[1], w[2], w[3]);
      } else {
        const float4 a = *reinterpret_cast<const float4*>(x + e0), b = *reinterpret_cast<const float4*>(x + e0 + 4);
        float f[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] = (keep >> i) & 1u ? f[i] * scale : 0.f;
        *reinterpret_cast<float4*>(y + e0) = make_float4(f[0], f[1], f[2], f[3]);
        *reinterpret_cast<float4*>(y + e0 + 4) = make_float4(f[4], f[5], f[6], f[7]);
      }
    } else {
      for (int i = 0; i < 8 && e0 + i < n; ++i) {
        const float v = (keep >> i) & 1u ? (float)x[e0 + i] * scale : 0.f;
        y[e0 + i] = (T)v;
      }
    }
  }
}

__global__ void __launch_bounds__(256) dropout_mask_kernel(unsigned char* __restrict__ mask, long long n, unsigned threshold,
                                                           const rng::State* st, unsigned long long call_id) {
  const rng::Key key = rng::make_key(st, call_id);
  const long long groups = (n + 7) / 8;
  for (long long g = (long long)blockIdx.x * blockDim.x + threadIdx.x; g < groups; g += (long long)gridDim.x * blockDim.x) {
    const unsigned keep = rng::keep_bits(rng::philox(key, (unsigned long long)g), threshold);
    for (int i = 0; i < 8 && g * 8 + i < n; ++i) mask[g * 8 + i] = (unsigned char)((keep >> i) & 1u);
  }
}
}  // namespace

int rng_state(rng::State** out) {
  int device = 0;
  HAPX_CUDA(cudaGetDevice(&device));
  if (device < 0 || device >= 64) return fail(HAPX_ERR_ARGUMENT, "rng: device index out of range");
  std::lock_guard<std::mutex> lock(g_state_mutex);
  if (!g_state[device]) {
    void* p = nullptr;
    HAPX_CUDA(cudaMalloc(&p, sizeof(rng::State)));
    const rng::State init = {0x9E3779B97F4A7C15ull, 0ull};
    HAPX_CUDA(cudaMemcpy(p, &init, sizeof(init), cudaMemcpyHostToDevice));
    g_state[device] = static_cast<rng::State*>(p);
  }
  *out = g_state[device];
  return HAPX_OK;
}

static int grid_for(long long n, int* grid) {
  int device = 0, sms = 0;
  HAPX_CUDA(cudaGetDevice(&device));
  HAPX_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
  const long long groups = (n + 7) / 8;
  *grid = (int)std::max<long long>(1, std::min<long long>((groups + 255) / 256, (long long)sms * 8));
  return HAPX_OK;
}

}  // namespace hapx

using namespace hapx;

extern "C" {

int hapx_rng_seed(uint64_t seed, hapx_stream stream) {
  rng::State* st = nullptr;
  if (int e = rng_state(&st)) return e;
  rng_seed_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(st, seed);
  HAPX_CUDA(cudaGetLastError());
  count_launch();
  return HAPX_OK;
}

int hapx_rng_advance(hapx_stream stream) {
  rng::State* st = nullptr;
  if (int e = rng_state(&st)) return e;
  rng_advance_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(st);
  HAPX_CUDA(cudaGetLastError());
  count_launch();
  return HAPX_OK;
}

int hapx_dropout(void* y, const void* x, int dtype, int64_t n, double p, uint64_t call_id, hapx_stream stream_) {
  if (n < 0) return fail(HAPX_ERR_EXTENT, "dropout: negative size");
  if (!(p >= 0.0 && p < 1.0)) return fail(HAPX_ERR_ARGUMENT, "dropout: p must be in [0, 1)");
  if (dtype != HAPX_BF16 && dtype != HAPX_F32) return fail(HAPX_ERR_DTYPE, "dropout: bfloat16 or float32 only");
  if (n == 0) return HAPX_OK;
  if (!y || !x) return fail(HAPX_ERR_ARGUMENT, "dropout: null pointer");
  rng::State* st = nullptr;
  if (int e = rng_state(&st)) return e;
  int grid = 1;
  if (int e = grid_for(n, &grid)) return e;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const unsigned thr = rng::threshold_for(p);
  const float scale = (float)(1.0 / (1.0 - p));
  if (dtype == HAPX_BF16)
    dropout_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(y), n, thr, scale, st, call_id);
  else
    dropout_kernel<float><<<grid, 256, 0, stream>>>(static_cast<const float*>(x), static_cast<float*>(y), n, thr, scale, st, call_id);
  HAPX_CUDA(cudaGetLastError());
  count_launch();
  return HAPX_OK;
}

int hapx_dropout_mask(unsigned char* mask, int64_t n, double p, uint64_t call_id, hapx_stream stream_) {
  if (n < 0) return fail(HAPX_ERR_EXTENT, "dropout_mask: negative size");
  if (!(p >= 0.0 && p < 1.0)) return fail(HAPX_ERR_ARGUMENT, "dropout_mask: p must be in [0, 1)");
  if (n == 0) return HAPX_OK;
  if (!mask) return fail(HAPX_ERR_ARGUMENT, "dropout_mask: null pointer");
  rng::State* st = nullptr;
  if (int e = rng_state(&st)) return e;
  int grid = 1;
  if (int e = grid_for(n, &grid)) return e;
  dropout_mask_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream_)>>>(mask, n, rng::threshold_for(p), st, call_id);
  HAPX_CUDA(cudaGetLastError());
  count_launch();
  return HAPX_OK;
}

}  // extern "C"
