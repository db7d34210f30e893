// layer_norm over the last dimension (the torch.nn.functional.layer_norm nodes of the Transformer
// programs: planner handler hap.rs:1637-1660, sharding rules hap.rs:3052; nn.LayerNorm inside the
// reference's encoder layers, models.py:319-320), forward and backward, for bf16 and fp32 rows of
// up to 2048 elements (a multiple of 8).
//
// HBM-bound.  One warp owns a row and keeps it in registers: forward reads x once and writes y
// plus two floats per row; backward reads x and dy once and writes dx, and every block adds the
// weight / bias gradient contributions of its rows into its own row of a partials matrix that a
// second small kernel sums in a fixed order (deterministic, no atomics).
#include <cuda_bf16.h>

#include "hapx_internal.h"

namespace hapx {
namespace norm {

constexpr int kWarpsPerBlock = 4;
constexpr int kThreads = kWarpsPerBlock * 32;
constexpr int kMaxVec = 8;           // 16-byte groups of 8 elements per lane: rows up to 8 * 8 * 32 = 2048 elements

// Eight consecutive elements of a row: kept packed (as loaded) while they wait to be used.
template <typename T>
struct Row;
template <>
struct Row<__nv_bfloat16> {
  struct Packed { uint4 v; };       // one 16-byte load
  static __device__ __forceinline__ Packed load(const __nv_bfloat16* p) { return Packed{*reinterpret_cast<const uint4*>(p)}; }
  static __device__ __forceinline__ void unpack(const Packed& q, float (&f)[8]) {
    const unsigned w[4] = {q.v.x, q.v.y, q.v.z, q.v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) { f[2 * i] = __uint_as_float(w[i] << 16); f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u); }
  }
  static __device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&f)[8]) { unpack(load(p), f); }
  static __device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&f)[8]) {
    unsigned w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const __nv_bfloat162 h = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
      w[i] = *reinterpret_cast<const unsigned*>(&h);
    }
    *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
  }
};
template <>
struct Row<float> {
  struct Packed { float4 a, b; };
  static __device__ __forceinline__ Packed load(const float* p) {
    return Packed{*reinterpret_cast<const float4*>(p), *reinterpret_cast<const float4*>(p + 4)};
  }
  static __device__ __forceinline__ void unpack(const Packed& q, float (&f)[8]) {
    f[0] = q.a.x; f[1] = q.a.y; f[2] = q.a.z; f[3] = q.a.w; f[4] = q.b.x; f[5] = q.b.y; f[6] = q.b.z; f[7] = q.b.w;
  }
  static __device__ __forceinline__ void load8(const float* p, float (&f)[8]) { unpack(load(p), f); }
  static __device__ __forceinline__ void store8(float* p, const float (&f)[8]) {
    *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(f[4], f[5], f[6], f[7]);
  }
};

__device__ __forceinline__ float warp_sum(float x) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
  return x;
}

// Lane l holds the groups g = l, l + 32, ... (< E / 8) of its row: elements [8g, 8g + 8).
template <typename T, int NV>
__global__ void __launch_bounds__(kThreads) layer_norm_forward_kernel(const T* __restrict__ x, const T* __restrict__ gamma,
                                                                      const T* __restrict__ beta, T* __restrict__ y,
                                                                      float* __restrict__ mean_out, float* __restrict__ rstd_out,
                                                                      long long rows, int E, float eps) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int groups = E >> 3;
  float gam[NV][8], bet[NV][8];
#pragma unroll
  for (int v = 0; v < NV; ++v) {
    const int g = lane + 32 * v;
    if (g < groups) {
      Row<T>::load8(gamma + 8 * g, gam[v]);
      if (beta) Row<T>::load8(beta + 8 * g, bet[v]);
      else {
#pragma unroll
        for (int k = 0; k < 8; ++k) bet[v][k] = 0.f;
      }
    }
  }
  const float inv_e = 1.f / (float)E;
  const long long stride = (long long)gridDim.x * kWarpsPerBlock;
  long long row = (long long)blockIdx.x * kWarpsPerBlock + warp;
  typename Row<T>::Packed nxt[NV];            // the next row of this warp is loaded while the current one is worked on
  if (row < rows) {
#pragma unroll
    for (int v = 0; v < NV; ++v)
      if (lane + 32 * v < groups) nxt[v] = Row<T>::load(x + row * E + 8 * (lane + 32 * v));
  }
  for (; row < rows; row += stride) {
    float f[NV][8];
    float s = 0.f;
#pragma unroll
    for (int v = 0; v < NV; ++v) {
      if (lane + 32 * v < groups) {
        Row<T>::unpack(nxt[v], f[v]);
#pragma unroll
        for (int k = 0; k < 8; ++k) s += f[v][k];
      }
    }
    if (row + stride < rows) {
#pragma unroll
      for (int v = 0; v < NV; ++v)
        if (lane + 32 * v < groups) nxt[v] = Row<T>::load(x + (row + stride) * E + 8 * (lane + 32 * v));
    }
    const float mean = warp_sum(s) * inv_e;
    float q = 0.f;
#pragma unroll
    for (int v = 0; v < NV; ++v) {
      if (lane + 32 * v < groups) {
#pragma unroll
        for (int k = 0; k < 8; ++k) { const float d = f[v][k] - mean; q = fmaf(d, d, q); }
      }
    }
    const float rstd = rsqrtf(warp_sum(q) * inv_e + eps);
    T* yr = y + row * E;
#pragma unroll
    for (int v = 0; v < NV; ++v) {
      const int g = lane + 32 * v;
      if (g < groups) {
        float o[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) o[k] = fmaf((f[v][k] - mean) * rstd, gam[v][k], bet[v][k]);
        Row<T>::store8(yr + 8 * g, o);
      }
    }
    if (lane == 0) { mean_out[row] = mean; rstd_out[row] = rstd; }
  }
}

// dx = rstd * (dy*gamma - mean(dy*gamma) - xhat * mean(dy*gamma*xhat)) [+ add];  partial[b][0][e] += dy*xhat, partial[b][1][e] += dy
// `add` (may be null): a second gradient of x - the one that arrives through the residual connection around the
// normalised branch of a pre-LN block - added here instead of by a separate kernel.
template <typename T, int NV, bool ADD>
__global__ void __launch_bounds__(kThreads, (NV <= 3 ? 3 : 2)) layer_norm_backward_kernel(const T* __restrict__ x, const T* __restrict__ dy,
                                                                       const T* __restrict__ gamma, const float* __restrict__ mean_in,
                                                                       const float* __restrict__ rstd_in, const T* __restrict__ add,
                                                                       T* __restrict__ dx, float* __restrict__ partial, long long rows, int E) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int groups = E >> 3;
  float gam[NV][8], dg[NV][8], db[NV][8];
#pragma unroll
  for (int v = 0; v < NV; ++v) {
    const int g = lane + 32 * v;
    if (g < groups) Row<T>::load8(gamma + 8 * g, gam[v]);
#pragma unroll
    for (int k = 0; k < 8; ++k) { dg[v][k] = 0.f; db[v][k] = 0.f; }
  }
  const float inv_e = 1.f / (float)E;
  const long long stride = (long long)gridDim.x * kWarpsPerBlock;
  long long row = (long long)blockIdx.x * kWarpsPerBlock + warp;
  typename Row<T>::Packed nx[NV], ng[NV];      // next row of x and dy, in flight while the current row is worked on
  if (row < rows) {
#pragma unroll
    for (int v = 0; v < NV; ++v) {
      if (lane + 32 * v < groups) {
        nx[v] = Row<T>::load(x + row * E + 8 * (lane + 32 * v));
        ng[v] = Row<T>::load(dy + row * E + 8 * (lane + 32 * v));
      }
    }
  }
  for (; row < rows; row += stride) {
    const float mean = mean_in[row], rstd = rstd_in[row];
    float xh[NV][8], gy[NV][8];
#pragma unroll
    for (int v = 0; v < NV; ++v) {
      if (lane + 32 * v < groups) { Row<T>::unpack(nx[v], xh[v]); Row<T>::unpack(ng[v], gy[v]); }
    }
    if (row + stride < rows) {
#pragma unroll
      for (int v = 0; v < NV; ++v) {
        if (lane + 32 * v < groups) {
          nx[v] = Row<T>::load(x + (row + stride) * E + 8 * (lane + 32 * v));
          ng[v] = Row<T>::load(dy + (row + stride) * E + 8 * (lane + 32 * v));
        }
      }
    }
    if constexpr (ADD) {
      // no registers left to hold the residual gradient across the reductions: pull this row's lines into L2 / L1
      // now (one request per 128-byte line), the loads at the end of the iteration then find them close by
      if ((lane & (sizeof(T) == 2 ? 7 : 3)) == 0) {
#pragma unroll
        for (int v = 0; v < NV; ++v)
          if (lane + 32 * v < groups) asm volatile("prefetch.global.L1 [%0];" ::"l"(add + row * E + 8 * (lane + 32 * v)));
      }
    }
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int v = 0; v < NV; ++v) {
      if (lane + 32 * v < groups) {
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          xh[v][k] = (xh[v][k] - mean) * rstd;
          dg[v][k] = fmaf(gy[v][k], xh[v][k], dg[v][k]);
          db[v][k] += gy[v][k];
          gy[v][k] *= gam[v][k];
          s1 += gy[v][k];
          s2 = fmaf(gy[v][k], xh[v][k], s2);
        }
      }
    }
    const float m1 = warp_sum(s1) * inv_e, m2 = warp_sum(s2) * inv_e;
    T* dr = dx + row * E;
#pragma unroll
    for (int v = 0; v < NV; ++v) {
      const int g = lane + 32 * v;
      if (g < groups) {
        float o[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) o[k] = rstd * (gy[v][k] - m1 - xh[v][k] * m2);
        if constexpr (ADD) {
          float r[8];
          Row<T>::unpack(Row<T>::load(add + row * E + 8 * g), r);
#pragma unroll
          for (int k = 0; k < 8; ++k) o[k] += r[k];
        }
        Row<T>::store8(dr + 8 * g, o);
      }
    }
  }
  // the block's warps add their columns in warp order, then the block writes its partials row
  __shared__ float s_acc[2][kMaxVec * 8 * 32];
  for (int w = 0; w < kWarpsPerBlock; ++w) {
    if (warp == w) {
#pragma unroll
      for (int v = 0; v < NV; ++v) {
        const int g = lane + 32 * v;
        if (g < groups) {
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const int e = 8 * g + k;
            s_acc[0][e] = (w == 0 ? 0.f : s_acc[0][e]) + dg[v][k];
            s_acc[1][e] = (w == 0 ? 0.f : s_acc[1][e]) + db[v][k];
          }
        }
      }
    }
    __syncthreads();
  }
  float* out = partial + (long long)blockIdx.x * 2 * E;
  for (int e = threadIdx.x; e < E; e += kThreads) { out[e] = s_acc[0][e]; out[E + e] = s_acc[1][e]; }
}

// dgamma[e] = sum_b partial[b][0][e], dbeta[e] = sum_b partial[b][1][e].  A thread block owns 32 of the
// 2E columns; its 32 warps add the partial rows w, w + 32, ... (a dozen dependent loads each instead of
// several dozen: the kernel is latency-bound) and the 32 sums are added in warp order.
constexpr int kGradWarps = 32;
template <typename T>
__global__ void __launch_bounds__(kGradWarps * 32) layer_norm_param_grad_kernel(const float* __restrict__ partial, int blocks, int E,
                                                                                T* __restrict__ dgamma, T* __restrict__ dbeta) {
  __shared__ float s_sum[kGradWarps][32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int e = blockIdx.x * 32 + lane;
  float s = 0.f;
  if (e < 2 * E) {
#pragma unroll 4
    for (int b = warp; b < blocks; b += kGradWarps) s += partial[(long long)b * 2 * E + e];
  }
  s_sum[warp][lane] = s;
  __syncthreads();
  if (warp != 0 || e >= 2 * E) return;
#pragma unroll
  for (int w = 1; w < kGradWarps; ++w) s += s_sum[w][lane];
  if (e < E) {
    if (dgamma) { if constexpr (sizeof(T) == 2) dgamma[e] = __float2bfloat16_rn(s); else dgamma[e] = s; }
  } else if (dbeta) {
    if constexpr (sizeof(T) == 2) dbeta[e - E] = __float2bfloat16_rn(s); else dbeta[e - E] = s;
  }
}

static int sm_count() {
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  return sms;
}

template <typename T, int NV>
static void launch_fwd(const void* x, const void* gamma, const void* beta, void* y, float* mean, float* rstd, long long rows, int E,
                       float eps, int grid, cudaStream_t stream) {
  layer_norm_forward_kernel<T, NV><<<grid, kThreads, 0, stream>>>(static_cast<const T*>(x), static_cast<const T*>(gamma),
                                                                  static_cast<const T*>(beta), static_cast<T*>(y), mean, rstd, rows, E, eps);
}
template <typename T, int NV>
static void launch_bwd(const void* x, const void* dy, const void* gamma, const float* mean, const float* rstd, const void* add, void* dx,
                       float* partial, long long rows, int E, int grid, cudaStream_t stream) {
  if (add != nullptr)
    layer_norm_backward_kernel<T, NV, true><<<grid, kThreads, 0, stream>>>(static_cast<const T*>(x), static_cast<const T*>(dy),
                                                                           static_cast<const T*>(gamma), mean, rstd, static_cast<const T*>(add),
                                                                           static_cast<T*>(dx), partial, rows, E);
  else
    layer_norm_backward_kernel<T, NV, false><<<grid, kThreads, 0, stream>>>(static_cast<const T*>(x), static_cast<const T*>(dy),
                                                                            static_cast<const T*>(gamma), mean, rstd, nullptr,
                                                                            static_cast<T*>(dx), partial, rows, E);
}

static int check_common(const char* who, int dtype, int64_t rows, int64_t E) {
  if (dtype != HAPX_F32 && dtype != HAPX_BF16) return fail(HAPX_ERR_DTYPE, std::string(who) + ": float32 or bfloat16 only");
  if (rows < 0 || E < 8 || (E & 7) != 0 || E > kMaxVec * 8 * 32)
    return fail(HAPX_ERR_EXTENT, std::string(who) + ": the normalised dimension must be a multiple of 8 in [8, 2048]");
  return HAPX_OK;
}

}  // namespace norm
}  // namespace hapx

using namespace hapx;
using namespace hapx::norm;

extern "C" {

int hapx_layer_norm_backward_blocks(int64_t rows, int64_t E) {
  // one resident wave: 3 blocks per SM for rows of up to 768 elements, 2 above (register budget)
  const long long cap = (long long)sm_count() * (E <= 768 ? 3 : 2);
  const long long need = (rows + kWarpsPerBlock - 1) / kWarpsPerBlock;
  return (int)(need < 1 ? 1 : (need < cap ? need : cap));
}

int hapx_layer_norm_forward(const void* x, const void* gamma, const void* beta, void* y, float* mean, float* rstd, int dtype,
                            int64_t rows, int64_t E, double eps, hapx_stream stream_) {
  if (int e = check_common("layer_norm_forward", dtype, rows, E)) return e;
  if (rows == 0) return HAPX_OK;
  if (!x || !gamma || !y || !mean || !rstd) return fail(HAPX_ERR_ARGUMENT, "layer_norm_forward: null argument");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const long long need = (rows + kWarpsPerBlock - 1) / kWarpsPerBlock, cap = (long long)sm_count() * 8;
  const int grid = (int)(need < cap ? need : cap);
  const int nv = (int)((E / 8 + 31) / 32);
#define HAPX_LN_FWD(T)                                                                                              \
  switch (nv) {                                                                                                     \
    case 1: launch_fwd<T, 1>(x, gamma, beta, y, mean, rstd, rows, (int)E, (float)eps, grid, stream); break;         \
    case 2: launch_fwd<T, 2>(x, gamma, beta, y, mean, rstd, rows, (int)E, (float)eps, grid, stream); break;         \
    case 3: launch_fwd<T, 3>(x, gamma, beta, y, mean, rstd, rows, (int)E, (float)eps, grid, stream); break;         \
    case 4: launch_fwd<T, 4>(x, gamma, beta, y, mean, rstd, rows, (int)E, (float)eps, grid, stream); break;         \
    default: launch_fwd<T, 8>(x, gamma, beta, y, mean, rstd, rows, (int)E, (float)eps, grid, stream); break;        \
  }
  if (dtype == HAPX_BF16) { HAPX_LN_FWD(__nv_bfloat16) } else { HAPX_LN_FWD(float) }
#undef HAPX_LN_FWD
  HAPX_CUDA(cudaGetLastError());
  count_launch(1);
  return HAPX_OK;
}

int hapx_layer_norm_backward(const void* x, const void* dy, const void* gamma, const float* mean, const float* rstd, void* dx,
                             void* dgamma, void* dbeta, float* partial, int dtype, int64_t rows, int64_t E, hapx_stream stream_) {
  return hapx_layer_norm_backward_add(x, dy, gamma, mean, rstd, nullptr, dx, dgamma, dbeta, partial, dtype, rows, E, stream_);
}

int hapx_layer_norm_backward_add(const void* x, const void* dy, const void* gamma, const float* mean, const float* rstd, const void* add,
                                 void* dx, void* dgamma, void* dbeta, float* partial, int dtype, int64_t rows, int64_t E,
                                 hapx_stream stream_) {
  if (int e = check_common("layer_norm_backward", dtype, rows, E)) return e;
  if (!partial) return fail(HAPX_ERR_ARGUMENT, "layer_norm_backward: null partials buffer");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  int grid = 0;
  if (rows > 0) {
    if (!x || !dy || !gamma || !mean || !rstd || !dx) return fail(HAPX_ERR_ARGUMENT, "layer_norm_backward: null argument");
    grid = hapx_layer_norm_backward_blocks(rows, E);
    const int nv = (int)((E / 8 + 31) / 32);
#define HAPX_LN_BWD(T)                                                                                       \
  switch (nv) {                                                                                              \
    case 1: launch_bwd<T, 1>(x, dy, gamma, mean, rstd, add, dx, partial, rows, (int)E, grid, stream); break;      \
    case 2: launch_bwd<T, 2>(x, dy, gamma, mean, rstd, add, dx, partial, rows, (int)E, grid, stream); break;      \
    case 3: launch_bwd<T, 3>(x, dy, gamma, mean, rstd, add, dx, partial, rows, (int)E, grid, stream); break;      \
    case 4: launch_bwd<T, 4>(x, dy, gamma, mean, rstd, add, dx, partial, rows, (int)E, grid, stream); break;      \
    default: launch_bwd<T, 8>(x, dy, gamma, mean, rstd, add, dx, partial, rows, (int)E, grid, stream); break;     \
  }
    if (dtype == HAPX_BF16) { HAPX_LN_BWD(__nv_bfloat16) } else { HAPX_LN_BWD(float) }
#undef HAPX_LN_BWD
    HAPX_CUDA(cudaGetLastError());
    count_launch(1);
  }
  if (dgamma || dbeta) {
    const int threads = kGradWarps * 32, blocks = (int)((2 * E + 31) / 32);
    if (dtype == HAPX_BF16)
      layer_norm_param_grad_kernel<__nv_bfloat16><<<blocks, threads, 0, stream>>>(partial, grid, (int)E, static_cast<__nv_bfloat16*>(dgamma),
                                                                                  static_cast<__nv_bfloat16*>(dbeta));
    else
      layer_norm_param_grad_kernel<float><<<blocks, threads, 0, stream>>>(partial, grid, (int)E, static_cast<float*>(dgamma),
                                                                          static_cast<float*>(dbeta));
    HAPX_CUDA(cudaGetLastError());
    count_launch(1);
  }
  return HAPX_OK;
}

}  // extern "C"
