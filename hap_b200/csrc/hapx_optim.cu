// Step tail of the SPMD training iteration: gradient clipping by the norm of the LOCAL shards
// followed by Adam, as multi-tensor kernels (worker.py:74, 76 with the optimizer of worker.py:47
// in the reference; torch.nn.utils.clip_grad_norm_ and torch.optim.Adam semantics).
//
// Both kernels are HBM-bound streams over all parameter shards of a rank:
//   sqnorm: reads every gradient once                       (g bytes)
//   apply : reads g, p, m, v and writes p, m, v once        (7 x element size per element)
// Tensor lists travel in the kernel parameters (up to kListMax tensors per launch), so nothing
// is uploaded or allocated per call and the launches can be captured into a CUDA graph.
// The sum of squares is deterministic: every block adds its chunks in a fixed order into its own
// slot of the caller's state buffer, and every consumer adds the slots in slot order.
#include <cuda_bf16.h>

#include "hapx_internal.h"

namespace hapx {
namespace optim {

constexpr int kListMax = 64;            // tensors per launch (kernel parameters stay below 4 KiB)
constexpr int kChunk = 8192;            // elements per block visit
constexpr int kThreads = 256;
constexpr int kUnroll = 4;             // 16-byte loads in flight per thread in the norm kernel
constexpr int kUnrollAdam = 2;         // ... per stream (g, p, m, v) in the update kernel
constexpr int kSlots = HAPX_OPTIM_STATE_FLOATS - 8;   // per-block partial sums of squares

struct NormList {
  const void* g[kListMax];
  long long numel[kListMax];
  int n;
};

struct AdamList {
  void* p[kListMax];
  const void* g[kListMax];
  void* m[kListMax];
  void* v[kListMax];
  long long numel[kListMax];
  int n;
};

__device__ __forceinline__ float to_f(float x) { return x; }
__device__ __forceinline__ float to_f(__nv_bfloat16 x) { return __bfloat162float(x); }
__device__ __forceinline__ void from_f(float& o, float x) { o = x; }
__device__ __forceinline__ void from_f(__nv_bfloat16& o, float x) { o = __float2bfloat16_rn(x); }

// 16 bytes of T as four 32-bit words; word w holds PER consecutive elements.
template <typename T>
struct Words;
template <>
struct Words<float> {
  static constexpr int N = 4, PER = 1;
  static __device__ __forceinline__ void unpack(unsigned w, float (&f)[2]) { f[0] = __uint_as_float(w); }
  static __device__ __forceinline__ unsigned pack(const float (&f)[2]) { return __float_as_uint(f[0]); }
};
template <>
struct Words<__nv_bfloat16> {
  static constexpr int N = 8, PER = 2;
  static __device__ __forceinline__ void unpack(unsigned w, float (&f)[2]) {
    f[0] = __uint_as_float(w << 16);
    f[1] = __uint_as_float(w & 0xffff0000u);
  }
  static __device__ __forceinline__ unsigned pack(const float (&f)[2]) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(f[0], f[1]);   // one conversion per pair
    return *reinterpret_cast<const unsigned*>(&h);
  }
};
__device__ __forceinline__ unsigned word_of(const uint4& v, int i) { return i == 0 ? v.x : (i == 1 ? v.y : (i == 2 ? v.z : v.w)); }
__device__ __forceinline__ void set_word(uint4& v, int i, unsigned w) {
  if (i == 0) v.x = w; else if (i == 1) v.y = w; else if (i == 2) v.z = w; else v.w = w;
}

__device__ __forceinline__ float block_sum(float x) {
  __shared__ float warp_part[kThreads / 32];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
  if ((threadIdx.x & 31) == 0) warp_part[threadIdx.x >> 5] = x;
  __syncthreads();
  float s = 0.f;
  if (threadIdx.x == 0) {
#pragma unroll
    for (int w = 0; w < kThreads / 32; ++w) s += warp_part[w];
  }
  __syncthreads();
  return s;   // valid in thread 0
}

// Work schedule shared by both kernels: the tensors of a list are cut into chunks of kChunk
// elements, numbered through the list; block b takes the chunks b, b + G, b + 2G, ...  Thread 0
// builds the prefix sums of the chunk counts once per block; a chunk's tensor is then found by
// bisection (the same few shared-memory reads in every thread).
template <typename List>
__device__ __forceinline__ long long build_schedule(const List& list, long long* prefix) {
  if (threadIdx.x == 0) {
    long long run = 0;
    for (int t = 0; t < list.n; ++t) {
      prefix[t] = run;
      run += (list.numel[t] + kChunk - 1) / kChunk;
    }
    prefix[list.n] = run;
  }
  __syncthreads();
  return prefix[list.n];
}
__device__ __forceinline__ int tensor_of_chunk(const long long* prefix, int n, long long chunk) {
  int lo = 0, hi = n - 1;            // largest t with prefix[t] <= chunk
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (prefix[mid] <= chunk) lo = mid; else hi = mid - 1;
  }
  return lo;
}

template <typename T>
__global__ void __launch_bounds__(kThreads, 4) sqnorm_kernel(const NormList list, float* state, int reset) {
  __shared__ long long s_prefix[kListMax + 1];
  const long long total_chunks = build_schedule(list, s_prefix);
  float acc = 0.f;
  for (long long gc = blockIdx.x; gc < total_chunks; gc += gridDim.x) {
    const int t = tensor_of_chunk(s_prefix, list.n, gc);
    const long long n = list.numel[t], c = gc - s_prefix[t];
    const T* g = reinterpret_cast<const T*>(list.g[t]);
    const bool vec = (reinterpret_cast<uintptr_t>(g) & 15u) == 0;
    const long long lo = c * kChunk, hi = min(lo + (long long)kChunk, n);
    if (vec) {
      using W = Words<T>;
      constexpr int N = W::N;
      const T* gp = g + lo;                                   // 32-bit offsets inside the chunk
      const int len = (int)(hi - lo), full = (len / N) * N;
      // kUnroll independent 16-byte loads per thread are in flight before any is used
      for (int i0 = threadIdx.x * N; i0 < full; i0 += kThreads * N * kUnroll) {
        uint4 x[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
          const int i = i0 + u * kThreads * N;
          x[u] = (i < full) ? *reinterpret_cast<const uint4*>(gp + i) : make_uint4(0u, 0u, 0u, 0u);   // zeros add nothing
        }
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
#pragma unroll
          for (int w = 0; w < 4; ++w) {
            float f[2] = {0.f, 0.f};
            W::unpack(word_of(x[u], w), f);
#pragma unroll
            for (int k = 0; k < W::PER; ++k) acc = fmaf(f[k], f[k], acc);
          }
        }
      }
      for (int i = full + threadIdx.x; i < len; i += kThreads) { const float f = to_f(gp[i]); acc = fmaf(f, f, acc); }
    } else {
      for (long long i = lo + threadIdx.x; i < hi; i += kThreads) { const float f = to_f(g[i]); acc = fmaf(f, f, acc); }
    }
  }
  const float s = block_sum(acc);
  if (threadIdx.x == 0) {
    float* slot = state + 8 + blockIdx.x;
    *slot = reset ? s : *slot + s;
  }
}

// state[0] = number of optimizer steps taken so far; state[8 + i] = partial sums of squares.
// state[1] (norm) and state[2] (clip coefficient) are written for the host to inspect.
template <typename T>
__global__ void __launch_bounds__(kThreads, 4) clip_adam_kernel(const AdamList list, float* state, int slots, double lr_d, double beta1_d,
                                                             double beta2_d, float eps, float weight_decay, float max_norm) {
  __shared__ float s_coef, s_step_size, s_inv_bc2s;
  // the host-side reference forms 1 - beta in double and rounds it to float once
  const float beta2 = (float)beta2_d, omb1 = (float)(1.0 - beta1_d), omb2 = (float)(1.0 - beta2_d);
  // every block adds the slots in the same order (thread-strided, then a fixed tree), so all blocks clip alike
  __shared__ double s_part[kThreads];
  if (max_norm > 0.f) {
    double part = 0.0;
    for (int i = threadIdx.x; i < slots; i += kThreads) part += (double)state[8 + i];
    s_part[threadIdx.x] = part;
    __syncthreads();
    for (int w = kThreads / 2; w > 0; w >>= 1) {
      if (threadIdx.x < w) s_part[threadIdx.x] += s_part[threadIdx.x + w];
      __syncthreads();
    }
  }
  if (threadIdx.x == 0) {
    float coef = 1.f;
    if (max_norm > 0.f) {
      const double total = s_part[0];
      const float norm = (float)sqrt(total);
      coef = fminf(max_norm / (norm + 1e-6f), 1.f);
      if (blockIdx.x == 0) { state[1] = norm; state[2] = coef; }
    }
    const double step = (double)state[0] + 1.0;      // bias corrections in double, as the host-side reference computes them
    s_coef = coef;
    s_step_size = (float)(lr_d / (1.0 - pow(beta1_d, step)));
    s_inv_bc2s = (float)(1.0 / sqrt(1.0 - pow(beta2_d, step)));
  }
  __syncthreads();
  const float coef = s_coef, step_size = s_step_size, inv_bc2s = s_inv_bc2s;

  // The kernel has to issue about 1.6 elements per clock and SM to keep up with HBM, so the square
  // root and the division are the special-function-unit approximations (about 1 and 2 units in the
  // last place), not the IEEE sequences of a dozen instructions each.
  auto update = [&](float& p, float g, float& m, float& v) {
    g *= coef;
    if (weight_decay != 0.f) g = fmaf(weight_decay, p, g);
    m = fmaf(omb1, g - m, m);                        // exp_avg.lerp_(grad, 1 - beta1)
    v = fmaf(omb2, g * g, beta2 * v);                // exp_avg_sq.mul_(beta2).addcmul_(grad, grad, 1 - beta2)
    float root;
    asm("sqrt.approx.ftz.f32 %0, %1;" : "=f"(root) : "f"(v));
    const float denom = fmaf(root, inv_bc2s, eps);
    p = fmaf(-step_size, __fdividef(m, denom), p);
  };

  __shared__ long long s_prefix[kListMax + 1];
  const long long total_chunks = build_schedule(list, s_prefix);
  for (long long gc = blockIdx.x; gc < total_chunks; gc += gridDim.x) {
    const int t = tensor_of_chunk(s_prefix, list.n, gc);
    const long long n = list.numel[t], c = gc - s_prefix[t];
    T* p = reinterpret_cast<T*>(list.p[t]);
    const T* g = reinterpret_cast<const T*>(list.g[t]);
    T* m = reinterpret_cast<T*>(list.m[t]);
    T* v = reinterpret_cast<T*>(list.v[t]);
    const bool vec = ((reinterpret_cast<uintptr_t>(p) | reinterpret_cast<uintptr_t>(g) | reinterpret_cast<uintptr_t>(m) |
                       reinterpret_cast<uintptr_t>(v)) & 15u) == 0;
    const long long lo = c * kChunk, hi = min(lo + (long long)kChunk, n);
    long long tail = lo;
    if (vec) {
      using W = Words<T>;
      constexpr int N = W::N;
      T* pc = p + lo; const T* gp = g + lo; T* mc = m + lo; T* vc = v + lo;     // 32-bit offsets inside the chunk
      const int full = ((int)(hi - lo) / N) * N;
      for (int i0 = threadIdx.x * N; i0 < full; i0 += kThreads * N * kUnrollAdam) {
        uint4 xp[kUnrollAdam], xg[kUnrollAdam], xm[kUnrollAdam], xv[kUnrollAdam];
#pragma unroll
        for (int u = 0; u < kUnrollAdam; ++u) {          // all loads first: 4 * kUnrollAdam in flight per thread
          const int i = i0 + u * kThreads * N;
          if (i < full) {
            xp[u] = *reinterpret_cast<const uint4*>(pc + i);
            xg[u] = *reinterpret_cast<const uint4*>(gp + i);
            xm[u] = *reinterpret_cast<const uint4*>(mc + i);
            xv[u] = *reinterpret_cast<const uint4*>(vc + i);
          }
        }
#pragma unroll
        for (int u = 0; u < kUnrollAdam; ++u) {
          const int i = i0 + u * kThreads * N;
          if (i < full) {
#pragma unroll
            for (int w = 0; w < 4; ++w) {                  // word by word: 1 (fp32) or 2 (bf16) elements
              float fp[2], fg[2], fm[2], fv[2];
              W::unpack(word_of(xp[u], w), fp); W::unpack(word_of(xg[u], w), fg);
              W::unpack(word_of(xm[u], w), fm); W::unpack(word_of(xv[u], w), fv);
#pragma unroll
              for (int k = 0; k < W::PER; ++k) update(fp[k], fg[k], fm[k], fv[k]);
              set_word(xp[u], w, W::pack(fp)); set_word(xm[u], w, W::pack(fm)); set_word(xv[u], w, W::pack(fv));
            }
            *reinterpret_cast<uint4*>(pc + i) = xp[u];
            *reinterpret_cast<uint4*>(mc + i) = xm[u];
            *reinterpret_cast<uint4*>(vc + i) = xv[u];
          }
        }
      }
      tail = lo + full;
    }
    for (long long i = tail + threadIdx.x; i < hi; i += kThreads) {
      float fp = to_f(p[i]), fm = to_f(m[i]), fv = to_f(v[i]);
      update(fp, to_f(g[i]), fm, fv);
      from_f(p[i], fp); from_f(m[i], fm); from_f(v[i], fv);
    }
  }
}

__global__ void advance_step_kernel(float* state) { state[0] += 1.f; }

static int grid_for(const long long* numel, int n, int sm_count) {
  long long chunks = 0;
  for (int i = 0; i < n; ++i) chunks += (numel[i] + kChunk - 1) / kChunk;
  long long g = (long long)sm_count * 4;   // one resident wave (4 blocks per SM)
  if (g > kSlots) g = kSlots;
  if (chunks < g) g = chunks;
  return g < 1 ? 1 : (int)g;
}

static int sm_count_of_current_device(int* out) {
  int dev = 0;
  HAPX_CUDA(cudaGetDevice(&dev));
  static int cached[64] = {};
  if (dev >= 0 && dev < 64 && cached[dev]) { *out = cached[dev]; return HAPX_OK; }
  int n = 0;
  HAPX_CUDA(cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev));
  if (dev >= 0 && dev < 64) cached[dev] = n;
  *out = n;
  return HAPX_OK;
}

}  // namespace optim
}  // namespace hapx

using namespace hapx;
using namespace hapx::optim;

extern "C" {

int hapx_grad_sqnorm(int n, const void* const* grads, const int64_t* numel, int dtype, float* state, int reset, hapx_stream stream_) {
  if (n < 0 || (n > 0 && (!grads || !numel)) || !state) return fail(HAPX_ERR_ARGUMENT, "grad_sqnorm: null argument");
  if (dtype != HAPX_F32 && dtype != HAPX_BF16) return fail(HAPX_ERR_DTYPE, "grad_sqnorm: float32 or bfloat16 only");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  int sms = 0;
  if (int e = sm_count_of_current_device(&sms)) return e;
  // one grid size for the whole iteration so that every launch uses the same slots
  const int grid = (int)((long long)sms * 8 > kSlots ? kSlots : sms * 8);
  int done = 0;
  bool first = reset != 0;
  do {
    NormList list;
    list.n = 0;
    while (done < n && list.n < kListMax) {
      if (numel[done] < 0) return fail(HAPX_ERR_ARGUMENT, "grad_sqnorm: negative element count");
      if (numel[done] > 0) {
        if (!grads[done]) return fail(HAPX_ERR_ARGUMENT, "grad_sqnorm: null gradient");
        list.g[list.n] = grads[done]; list.numel[list.n] = numel[done]; ++list.n;
      }
      ++done;
    }
    if (list.n == 0 && !first) break;
    if (dtype == HAPX_F32) sqnorm_kernel<float><<<grid, kThreads, 0, stream>>>(list, state, first ? 1 : 0);
    else sqnorm_kernel<__nv_bfloat16><<<grid, kThreads, 0, stream>>>(list, state, first ? 1 : 0);
    HAPX_CUDA(cudaGetLastError());
    count_launch(1);
    first = false;
  } while (done < n);
  return HAPX_OK;
}

int hapx_clip_adam_apply(int n, void* const* params, const void* const* grads, void* const* exp_avg, void* const* exp_avg_sq,
                         const int64_t* numel, int dtype, double lr, double beta1, double beta2, double eps, double weight_decay,
                         double max_norm, float* state, int advance_step, hapx_stream stream_) {
  if (n < 0 || (n > 0 && (!params || !grads || !exp_avg || !exp_avg_sq || !numel)) || !state)
    return fail(HAPX_ERR_ARGUMENT, "clip_adam_apply: null argument");
  if (dtype != HAPX_F32 && dtype != HAPX_BF16) return fail(HAPX_ERR_DTYPE, "clip_adam_apply: float32 or bfloat16 only");
  if (!(beta1 >= 0.0 && beta1 < 1.0) || !(beta2 >= 0.0 && beta2 < 1.0) || !(eps >= 0.0))
    return fail(HAPX_ERR_ARGUMENT, "clip_adam_apply: betas must be in [0, 1) and eps >= 0");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  int sms = 0;
  if (int e = sm_count_of_current_device(&sms)) return e;
  const int slots = (int)((long long)sms * 8 > kSlots ? kSlots : sms * 8);
  int done = 0;
  while (done < n) {
    AdamList list;
    list.n = 0;
    while (done < n && list.n < kListMax) {
      if (numel[done] < 0) return fail(HAPX_ERR_ARGUMENT, "clip_adam_apply: negative element count");
      if (numel[done] > 0) {
        if (!params[done] || !grads[done] || !exp_avg[done] || !exp_avg_sq[done])
          return fail(HAPX_ERR_ARGUMENT, "clip_adam_apply: null tensor");
        list.p[list.n] = params[done]; list.g[list.n] = grads[done]; list.m[list.n] = exp_avg[done];
        list.v[list.n] = exp_avg_sq[done]; list.numel[list.n] = numel[done]; ++list.n;
      }
      ++done;
    }
    if (list.n == 0) break;
    const int grid = grid_for(list.numel, list.n, sms);
    if (dtype == HAPX_F32)
      clip_adam_kernel<float><<<grid, kThreads, 0, stream>>>(list, state, slots, lr, beta1, beta2, (float)eps, (float)weight_decay, (float)max_norm);
    else
      clip_adam_kernel<__nv_bfloat16><<<grid, kThreads, 0, stream>>>(list, state, slots, lr, beta1, beta2, (float)eps, (float)weight_decay, (float)max_norm);
    HAPX_CUDA(cudaGetLastError());
    count_launch(1);
  }
  if (advance_step) {
    advance_step_kernel<<<1, 1, 0, stream>>>(state);
    HAPX_CUDA(cudaGetLastError());
    count_launch(1);
  }
  return HAPX_OK;
}

}  // extern "C"
