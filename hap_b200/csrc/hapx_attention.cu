// Multi-head self-attention on a batch shard: softmax(Q K^T / sqrt(d) + mask) V, forward and backward.
//
// Stands in for the attention core of F.multi_head_attention_forward as the planner emits it
// (hap.rs:1297-1329; only the batch dimension is ever sharded, hap.rs:2903-2926), working directly
// on the packed in-projection output qkv[L, N, 3E] and producing [L, N, E], i.e. in the (L, N, E)
// layout of the reference with no transposed copies: heads and batch entries are batch coordinates
// of the tensor maps.  The contractions run on the batched tcgen05 GEMM (hapx_gemm_sm100.cu):
//
//   forward : S = Q K^T (fp32)  ->  P = softmax(scale * S + mask) (bf16, kept for backward)  ->  O = P V
//   backward: dV = P^T dO;  dP = dO V^T (fp32);  dS = scale * P * (dP - rowsum(dP * P));  dQ = dS K;  dK = dS^T Q
//
// The softmax kernels keep one row per warp in registers (L <= 1024).
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdlib>
#include <string>

#include "hapx_internal.h"

namespace hapx {
namespace attn {

constexpr int kMaxPerLane = 32;  // L <= 1024; the kernels are instantiated for 8, 16 and 32 elements per lane

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// rows = batch * L; row r is query (r % L).  S, P: [rows][Lp] with Lp a multiple of 8, so every lane
// moves groups of 4 consecutive elements: 16-byte loads of fp32 scores, 8-byte stores of bf16
// probabilities.  Lane l owns the groups l, l + 32, ...  mask: additive [L][L] fp32 or null.
__device__ __forceinline__ void store_bf16x4(__nv_bfloat16* p, float a, float b, float c, float d) {
  const __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
  uint2 w;
  w.x = *reinterpret_cast<const unsigned*>(&lo);
  w.y = *reinterpret_cast<const unsigned*>(&hi);
  *reinterpret_cast<uint2*>(p) = w;
}

// The kernel is bound by instruction issue, not by HBM, unless it is written frugally: 32-bit row
// arithmetic (rows < 2^31 is checked on the host), the scale folded with log2(e) into one multiply,
// exp2 on the special-function unit, no work at all for groups of columns the causal rule excludes.
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <int PL>
__global__ void __launch_bounds__(256) softmax_fwd_kernel(const float* __restrict__ S, __nv_bfloat16* __restrict__ P, int L, int Lp,
                                                          long long rows, float scale, int causal, const float* __restrict__ mask) {
  const unsigned row = blockIdx.x * 8u + (threadIdx.x >> 5);
  if (row >= (unsigned)rows) return;
  const int lane = threadIdx.x & 31, q = (int)(row % (unsigned)L);
  const float* s = S + (size_t)row * (unsigned)Lp;
  const int last = causal ? q : L - 1;          // columns after `last` take no part
  constexpr int NG = PL / 4;
  constexpr float kLog2e = 1.4426950408889634f;
  const float scale2 = scale * kLog2e;          // softmax(x) = 2^(x log2 e - max) / sum
  float v[NG][4];
  float mx = -INFINITY;
  const bool mask_vec = mask != nullptr && (L & 3) == 0 && (reinterpret_cast<uintptr_t>(mask) & 15u) == 0;
#pragma unroll
  for (int i = 0; i < NG; ++i) {
    const int j0 = 4 * (lane + 32 * i);
    float4 x = make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
    if (j0 <= last) {                           // last < L <= Lp
      x = *reinterpret_cast<const float4*>(s + j0);
      x.x *= scale2; x.y *= scale2; x.z *= scale2; x.w *= scale2;
      if (mask_vec) {
        const float4 m = *reinterpret_cast<const float4*>(mask + (size_t)q * (unsigned)L + j0);
        x.x = fmaf(m.x, kLog2e, x.x); x.y = fmaf(m.y, kLog2e, x.y); x.z = fmaf(m.z, kLog2e, x.z); x.w = fmaf(m.w, kLog2e, x.w);
      } else if (mask) {
        const float* m = mask + (size_t)q * (unsigned)L + j0;
        x.x = fmaf(m[0], kLog2e, x.x);
        if (j0 + 1 < L) x.y = fmaf(m[1], kLog2e, x.y);
        if (j0 + 2 < L) x.z = fmaf(m[2], kLog2e, x.z);
        if (j0 + 3 < L) x.w = fmaf(m[3], kLog2e, x.w);
      }
      if (j0 + 3 > last) {                      // the group straddles the last column
        if (j0 + 1 > last) x.y = -INFINITY;
        if (j0 + 2 > last) x.z = -INFINITY;
        x.w = -INFINITY;
      }
      mx = fmaxf(fmaxf(mx, fmaxf(x.x, x.y)), fmaxf(x.z, x.w));
    }
    v[i][0] = x.x; v[i][1] = x.y; v[i][2] = x.z; v[i][3] = x.w;
  }
  mx = warp_max(mx);
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < NG; ++i) {
    if (4 * (lane + 32 * i) <= last) {          // 2^(-inf - max) = 0 for excluded columns inside a live group
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        v[i][k] = fast_exp2(v[i][k] - mx);
        sum += v[i][k];
      }
    } else {
      v[i][0] = v[i][1] = v[i][2] = v[i][3] = 0.f;
    }
  }
  sum = warp_sum(sum);
  const float inv = 1.f / sum;
  __nv_bfloat16* p = P + (size_t)row * (unsigned)Lp;
#pragma unroll
  for (int i = 0; i < NG; ++i) {
    const int j0 = 4 * (lane + 32 * i);
    if (j0 < Lp) store_bf16x4(p + j0, v[i][0] * inv, v[i][1] * inv, v[i][2] * inv, v[i][3] * inv);   // excluded columns hold 0
  }
}

template <int PL>
__global__ void __launch_bounds__(256) softmax_bwd_kernel(const __nv_bfloat16* __restrict__ P, const float* __restrict__ dP,
                                                          __nv_bfloat16* __restrict__ dS, int L, int Lp, long long rows, float scale) {
  const unsigned row = blockIdx.x * 8u + (threadIdx.x >> 5);
  if (row >= (unsigned)rows) return;
  const int lane = threadIdx.x & 31;
  const __nv_bfloat16* p = P + (size_t)row * (unsigned)Lp;
  const float* g = dP + (size_t)row * (unsigned)Lp;
  constexpr int NG = PL / 4;
  float pv[NG][4], gv[NG][4];
  float dot = 0.f;
#pragma unroll
  for (int i = 0; i < NG; ++i) {
    const int j0 = 4 * (lane + 32 * i);
    uint2 pw = make_uint2(0u, 0u);
    float4 gw = make_float4(0.f, 0.f, 0.f, 0.f);
    if (j0 < Lp) {                       // P is zero in the padding columns [L, Lp) and where the mask excluded a key
      pw = *reinterpret_cast<const uint2*>(p + j0);
      gw = *reinterpret_cast<const float4*>(g + j0);
    }
    pv[i][0] = __uint_as_float(pw.x << 16); pv[i][1] = __uint_as_float(pw.x & 0xffff0000u);
    pv[i][2] = __uint_as_float(pw.y << 16); pv[i][3] = __uint_as_float(pw.y & 0xffff0000u);
    gv[i][0] = (j0 < L) ? gw.x : 0.f; gv[i][1] = (j0 + 1 < L) ? gw.y : 0.f;
    gv[i][2] = (j0 + 2 < L) ? gw.z : 0.f; gv[i][3] = (j0 + 3 < L) ? gw.w : 0.f;
#pragma unroll
    for (int k = 0; k < 4; ++k) dot = fmaf(pv[i][k], gv[i][k], dot);
  }
  dot = warp_sum(dot);
  __nv_bfloat16* o = dS + (size_t)row * (unsigned)Lp;
#pragma unroll
  for (int i = 0; i < NG; ++i) {
    const int j0 = 4 * (lane + 32 * i);
    if (j0 < Lp)
      store_bf16x4(o + j0, scale * pv[i][0] * (gv[i][0] - dot), scale * pv[i][1] * (gv[i][1] - dot),
                   scale * pv[i][2] * (gv[i][2] - dot), scale * pv[i][3] * (gv[i][3] - dot));
  }
}

static int check(long long L, long long N, long long H, long long D) {
  if (L < 0 || N < 0 || H < 1 || D < 1) return fail(HAPX_ERR_EXTENT, "attention: negative extent");
  if (L > 32 * kMaxPerLane) return fail(HAPX_ERR_EXTENT, "attention: sequence length above 1024 is not supported");
  if (D % 8 != 0) return fail(HAPX_ERR_EXTENT, "attention: head dimension must be a multiple of 8");
  if (N * H > 0x7fffffff || N * H * L > 0x7fffffff) return fail(HAPX_ERR_EXTENT, "attention: too many (batch, head, query) rows");
  return HAPX_OK;
}

}  // namespace attn
}  // namespace hapx

using namespace hapx;
using hapx::gemm::Operand;

extern "C" {

int hapx_attention_forward(void* out, void* probs, void* scores_ws, const void* qkv, int64_t L, int64_t N, int64_t H, int64_t D,
                           int causal, const float* mask, hapx_stream stream_) {
  if (int e = attn::check(L, N, H, D)) return e;
  if (L == 0 || N == 0) return HAPX_OK;   // an empty batch shard (sharding_round may hand a rank nothing)
  if (!out || !probs || !scores_ws || !qkv) return fail(HAPX_ERR_ARGUMENT, "attention_forward: null pointer");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const long long E = H * D, Lp = (L + 7) / 8 * 8, row_qkv = N * 3 * E;
  const __nv_bfloat16* base = static_cast<const __nv_bfloat16*>(qkv);
  const Operand Q{base, false, row_qkv, D, 3 * E}, K{base + E, false, row_qkv, D, 3 * E};
  const Operand Vmn{base + 2 * E, true, row_qkv, D, 3 * E};
  const Operand S{scores_ws, false, Lp, L * Lp, H * L * Lp}, P{probs, false, Lp, L * Lp, H * L * Lp};
  const Operand O{out, false, N * E, D, E};
  // S[b] = Q[b] K[b]^T   (fp32)
  if (int e = gemm::gemm_bf16(S, 1, Q, K, nullptr, 0, L, L, D, (int)H, (int)N, stream)) return e;
  const long long rows = N * H * L;
  {
    const unsigned grid = (unsigned)((rows + 7) / 8);
    const float* sp = static_cast<const float*>(scores_ws);
    __nv_bfloat16* pp = static_cast<__nv_bfloat16*>(probs);
    const float sc = 1.0f / sqrtf((float)D);
    if (Lp <= 256) attn::softmax_fwd_kernel<8><<<grid, 256, 0, stream>>>(sp, pp, (int)L, (int)Lp, rows, sc, causal, mask);
    else if (Lp <= 512) attn::softmax_fwd_kernel<16><<<grid, 256, 0, stream>>>(sp, pp, (int)L, (int)Lp, rows, sc, causal, mask);
    else attn::softmax_fwd_kernel<32><<<grid, 256, 0, stream>>>(sp, pp, (int)L, (int)Lp, rows, sc, causal, mask);
  }
  HAPX_CUDA(cudaGetLastError());
  count_launch();
  // O[b] = P[b] V[b]      (contraction over keys; V is MN-major as stored)
  return gemm::gemm_bf16(O, 0, P, Vmn, nullptr, 0, L, D, L, (int)H, (int)N, stream);
}

int hapx_attention_backward(void* dqkv, void* dscores_ws, void* ds_ws, const void* dout, const void* probs, const void* qkv,
                            int64_t L, int64_t N, int64_t H, int64_t D, hapx_stream stream_) {
  if (int e = attn::check(L, N, H, D)) return e;
  if (L == 0 || N == 0) return HAPX_OK;
  if (!dqkv || !dscores_ws || !ds_ws || !dout || !probs || !qkv) return fail(HAPX_ERR_ARGUMENT, "attention_backward: null pointer");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const long long E = H * D, Lp = (L + 7) / 8 * 8, row_qkv = N * 3 * E;
  const __nv_bfloat16* base = static_cast<const __nv_bfloat16*>(qkv);
  __nv_bfloat16* gbase = static_cast<__nv_bfloat16*>(dqkv);
  const Operand Qmn{base, true, row_qkv, D, 3 * E}, Kmn{base + E, true, row_qkv, D, 3 * E};
  const Operand V{base + 2 * E, false, row_qkv, D, 3 * E};
  const Operand dO{dout, false, N * E, D, E}, dOmn{dout, true, N * E, D, E};
  const Operand P_mn{probs, true, Lp, L * Lp, H * L * Lp};
  const Operand dPf{dscores_ws, false, Lp, L * Lp, H * L * Lp};
  const Operand dS{ds_ws, false, Lp, L * Lp, H * L * Lp}, dSmn{ds_ws, true, Lp, L * Lp, H * L * Lp};
  const Operand dQ{gbase, false, row_qkv, D, 3 * E}, dK{gbase + E, false, row_qkv, D, 3 * E}, dV{gbase + 2 * E, false, row_qkv, D, 3 * E};
  // dV[k, d] = sum_q P[q, k] dO[q, d]
  if (int e = gemm::gemm_bf16(dV, 0, P_mn, dOmn, nullptr, 0, L, D, L, (int)H, (int)N, stream)) return e;
  // dP[q, k] = sum_d dO[q, d] V[k, d]   (fp32)
  if (int e = gemm::gemm_bf16(dPf, 1, dO, V, nullptr, 0, L, L, D, (int)H, (int)N, stream)) return e;
  const long long rows = N * H * L;
  {
    const unsigned grid = (unsigned)((rows + 7) / 8);
    const __nv_bfloat16* pp = static_cast<const __nv_bfloat16*>(probs);
    const float* gp = static_cast<const float*>(dscores_ws);
    __nv_bfloat16* dp = static_cast<__nv_bfloat16*>(ds_ws);
    const float sc = 1.0f / sqrtf((float)D);
    if (Lp <= 256) attn::softmax_bwd_kernel<8><<<grid, 256, 0, stream>>>(pp, gp, dp, (int)L, (int)Lp, rows, sc);
    else if (Lp <= 512) attn::softmax_bwd_kernel<16><<<grid, 256, 0, stream>>>(pp, gp, dp, (int)L, (int)Lp, rows, sc);
    else attn::softmax_bwd_kernel<32><<<grid, 256, 0, stream>>>(pp, gp, dp, (int)L, (int)Lp, rows, sc);
  }
  HAPX_CUDA(cudaGetLastError());
  count_launch();
  // dQ[q, d] = sum_k dS[q, k] K[k, d];   dK[k, d] = sum_q dS[q, k] Q[q, d]
  if (int e = gemm::gemm_bf16(dQ, 0, dS, Kmn, nullptr, 0, L, D, L, (int)H, (int)N, stream)) return e;
  return gemm::gemm_bf16(dK, 0, dSmn, Qmn, nullptr, 0, L, D, L, (int)H, (int)N, stream);
}

}  // extern "C"
