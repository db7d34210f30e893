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

// What one fused elementwise pass computes from `a` (and `b`), 8 elements per thread and generator call:
enum Mode {
  M_DROP = 0,          // y = a * k                      k = keep / (1 - p)
  M_DROP_ADD = 1,      // y = b + a * k                  (residual add after a dropout site)
  M_RELU_DROP = 2,     // y = relu(a) * k
  M_GELU_DROP = 3,     // y = gelu(a) * k                (erf form)
  M_RELU_DROP_BWD = 4, // y = b != 0 ? a / (1 - p) : 0   a = dy, b = the forward's OUTPUT (non-zero iff active and kept)
  M_GELU_DROP_BWD = 5  // y = a * k * gelu'(b)           a = dy, b = the forward's INPUT
};

// Phi(v) = 0.5 (1 + erf(v / sqrt 2)) and the density's exponential e^{-v^2/2}.  FAST (16-bit tensors): erf by the
// rational approximation 7.1.26 of Abramowitz & Stegun, 1 - (a1 t + ... + a5 t^5) e^{-z^2} with t = 1 / (1 + p z),
// absolute error 1.5e-7 - far below a bfloat16 rounding - which shares its exponential with the density: one ex2, one
// rcp and a handful of FMAs where erff() spends several dozen instructions (the GELU passes were bound by them).
template <bool FAST>
__device__ __forceinline__ void normal_cdf(float v, float& cdf, float& e) {
  if constexpr (FAST) {
    const float z = fabsf(v) * 0.70710678118654752f;
    e = __expf(-z * z);
    const float t = __fdividef(1.f, fmaf(0.3275911f, z, 1.f));
    float poly = fmaf(1.061405429f, t, -1.453152027f);
    poly = fmaf(poly, t, 1.421413741f);
    poly = fmaf(poly, t, -0.284496736f);
    poly = fmaf(poly, t, 0.254829592f);
    const float tail = 0.5f * poly * t * e;          // 0.5 (1 - erf z)
    cdf = v >= 0.f ? 1.f - tail : tail;
  } else {
    cdf = 0.5f * (1.f + erff(v * 0.70710678118654752f));
    e = __expf(-0.5f * v * v);
  }
}
template <bool FAST>
__device__ __forceinline__ float gelu_f(float v) {
  float cdf, e;
  normal_cdf<FAST>(v, cdf, e);
  return v * cdf;
}
template <bool FAST>
__device__ __forceinline__ float gelu_grad_f(float v) {
  float cdf, e;
  normal_cdf<FAST>(v, cdf, e);
  return fmaf(v * 0.3989422804014327f, e, cdf);
}

template <int MODE, bool FAST>
__device__ __forceinline__ float fused_value(float a, float b, float k, float scale) {
  switch (MODE) {
    case M_DROP: return a * k;
    case M_DROP_ADD: return fmaf(a, k, b);
    case M_RELU_DROP: return fmaxf(a, 0.f) * k;
    case M_GELU_DROP: return gelu_f<FAST>(a) * k;
    case M_RELU_DROP_BWD: return b != 0.f ? a * scale : 0.f;
    default: return a * k * gelu_grad_f<FAST>(b);
  }
}

template <typename T> struct Vec8;
template <> struct Vec8<__nv_bfloat16> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&f)[8]) {
    const uint4 v = *reinterpret_cast<const uint4*>(p);
    const unsigned w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) { f[2 * i] = __uint_as_float(w[i] << 16); f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u); }
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&f)[8]) {
    unsigned w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const __nv_bfloat162 h = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
      w[i] = *reinterpret_cast<const unsigned*>(&h);
    }
    *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
  }
};
template <> struct Vec8<float> {
  static __device__ __forceinline__ void load(const float* p, float (&f)[8]) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
  }
  static __device__ __forceinline__ void store(float* p, const float (&f)[8]) {
    *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(f[4], f[5], f[6], f[7]);
  }
};

// threshold == 0 means "no dropout" (every element kept, scale 1): the generator is not evaluated.
template <typename T, int MODE>
__global__ void __launch_bounds__(256) dropout_kernel(const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ y, long long n,
                                                      unsigned threshold, float scale, const rng::State* st, unsigned long long call_id) {
  constexpr bool TWO = MODE == M_DROP_ADD || MODE == M_RELU_DROP_BWD || MODE == M_GELU_DROP_BWD;
  constexpr bool NEEDS_MASK = MODE != M_RELU_DROP_BWD;
  rng::Key key = {0u, 0u, 0u, 0u};
  if (NEEDS_MASK && threshold) key = rng::make_key(st, call_id);
  const long long groups = (n + 7) / 8;
  const bool aligned = ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(y) | (TWO ? reinterpret_cast<uintptr_t>(b) : 0)) & (8 * sizeof(T) - 1)) == 0;
  for (long long g = (long long)blockIdx.x * blockDim.x + threadIdx.x; g < groups; g += (long long)gridDim.x * blockDim.x) {
    unsigned keep = 0xffu;
    if (NEEDS_MASK && threshold) keep = rng::keep_bits(rng::philox(key, (unsigned long long)g), threshold);
    const long long e0 = g * 8;
    if (e0 + 8 <= n && aligned) {
      float fa[8], fb[8], fy[8];
      Vec8<T>::load(a + e0, fa);
      if (TWO) Vec8<T>::load(b + e0, fb);
#pragma unroll
      for (int i = 0; i < 8; ++i) fy[i] = fused_value<MODE, sizeof(T) == 2>(fa[i], TWO ? fb[i] : 0.f, (keep >> i) & 1u ? scale : 0.f, scale);
      Vec8<T>::store(y + e0, fy);
    } else {
      for (int i = 0; i < 8 && e0 + i < n; ++i)
        y[e0 + i] = (T)fused_value<MODE, sizeof(T) == 2>((float)a[e0 + i], TWO ? (float)b[e0 + i] : 0.f, (keep >> i) & 1u ? scale : 0.f, scale);
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

static int launch_fused(int mode, void* y, const void* a, const void* b, int dtype, int64_t n, double p, uint64_t call_id, cudaStream_t stream,
                        const char* what) {
  if (n < 0) return fail(HAPX_ERR_EXTENT, std::string(what) + ": negative size");
  if (!(p >= 0.0 && p < 1.0)) return fail(HAPX_ERR_ARGUMENT, std::string(what) + ": p must be in [0, 1)");
  if (dtype != HAPX_BF16 && dtype != HAPX_F32) return fail(HAPX_ERR_DTYPE, std::string(what) + ": bfloat16 or float32 only");
  if (n == 0) return HAPX_OK;
  const bool two = mode == M_DROP_ADD || mode == M_RELU_DROP_BWD || mode == M_GELU_DROP_BWD;
  if (!y || !a || (two && !b)) return fail(HAPX_ERR_ARGUMENT, std::string(what) + ": null pointer");
  const unsigned thr = p > 0.0 ? rng::threshold_for(p) : 0u;
  rng::State* st = nullptr;
  if (thr)
    if (int e = rng_state(&st)) return e;
  int grid = 1;
  if (int e = grid_for(n, &grid)) return e;
  const float scale = (float)(1.0 / (1.0 - p));
#define HAPX_FUSED_CASE(M)                                                                                                             \
  case M:                                                                                                                              \
    if (dtype == HAPX_BF16)                                                                                                            \
      dropout_kernel<__nv_bfloat16, M><<<grid, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(a), static_cast<const __nv_bfloat16*>(b), \
                                                                 static_cast<__nv_bfloat16*>(y), n, thr, scale, st, call_id);         \
    else                                                                                                                               \
      dropout_kernel<float, M><<<grid, 256, 0, stream>>>(static_cast<const float*>(a), static_cast<const float*>(b), static_cast<float*>(y), n, \
                                                         thr, scale, st, call_id);                                                    \
    break;
  switch (mode) {
    HAPX_FUSED_CASE(M_DROP)
    HAPX_FUSED_CASE(M_DROP_ADD)
    HAPX_FUSED_CASE(M_RELU_DROP)
    HAPX_FUSED_CASE(M_GELU_DROP)
    HAPX_FUSED_CASE(M_RELU_DROP_BWD)
    HAPX_FUSED_CASE(M_GELU_DROP_BWD)
    default: return fail(HAPX_ERR_ARGUMENT, std::string(what) + ": unknown mode");
  }
#undef HAPX_FUSED_CASE
  HAPX_CUDA(cudaGetLastError());
  count_launch();
  return HAPX_OK;
}

int hapx_dropout(void* y, const void* x, int dtype, int64_t n, double p, uint64_t call_id, hapx_stream stream_) {
  return launch_fused(M_DROP, y, x, nullptr, dtype, n, p, call_id, static_cast<cudaStream_t>(stream_), "dropout");
}

int hapx_dropout_add(void* y, const void* x, const void* residual, int dtype, int64_t n, double p, uint64_t call_id, hapx_stream stream_) {
  return launch_fused(M_DROP_ADD, y, x, residual, dtype, n, p, call_id, static_cast<cudaStream_t>(stream_), "dropout_add");
}

int hapx_act_dropout(void* y, const void* x, int dtype, int64_t n, int act, double p, uint64_t call_id, hapx_stream stream_) {
  if (act != 1 && act != 2) return fail(HAPX_ERR_ARGUMENT, "act_dropout: act must be 1 (relu) or 2 (gelu)");
  return launch_fused(act == 1 ? M_RELU_DROP : M_GELU_DROP, y, x, nullptr, dtype, n, p, call_id, static_cast<cudaStream_t>(stream_), "act_dropout");
}

int hapx_act_dropout_backward(void* dx, const void* dy, const void* saved, int dtype, int64_t n, int act, double p, uint64_t call_id,
                              hapx_stream stream_) {
  if (act != 1 && act != 2) return fail(HAPX_ERR_ARGUMENT, "act_dropout_backward: act must be 1 (relu) or 2 (gelu)");
  return launch_fused(act == 1 ? M_RELU_DROP_BWD : M_GELU_DROP_BWD, dx, dy, saved, dtype, n, p, call_id, static_cast<cudaStream_t>(stream_),
                      "act_dropout_backward");
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
