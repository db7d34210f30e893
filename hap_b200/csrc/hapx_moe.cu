// Sparse dispatch / combine of the MoE layers: the dense one-hot contractions of the reference as gathers.
//
// The reference dispatches tokens to expert slots and combines the experts' outputs with two dense einsums
// over (batch, seq, expert, capacity) tensors (models.py:353-366: "bsd,bsec->becd" and "becd,bsec->bsd";
// planner side hap.rs:2255-2276).  The gating function (models.py:477-502) fills those tensors so that every
// (expert, capacity) slot of a batch entry holds at most ONE token and every token sits in at most TWO slots,
// which makes each contraction a row gather:
//
//   index          one pass over the dense tensor: slot -> (token, weight) and token -> (two slots, weights)
//   rows_from_tokens   rows[b, slot, :] = weight * x[b, token(slot), :]          (dispatch; backward of combine)
//   tokens_from_rows   y[b, s, :] = sum_k weight_k * rows[b, slot_k(s), :]        (combine; backward of dispatch)
//   weight_grad        d_dense[b, s, slot_k(s)] = <rows[b, slot_k(s), :], dy[b, s, :]>   (gradient of the combine weights)
//
// All bf16 with fp32 arithmetic, HBM bound: the dense tensor is read once per index pass, every row moves once.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <string>

#include "hapx_internal.h"

namespace hapx {
namespace moe {

// one warp per (b, s) row of the dense tensor [B, S, EC]
__global__ void __launch_bounds__(256) index_kernel(const __nv_bfloat16* __restrict__ dense, int* __restrict__ slot_token,
                                                    float* __restrict__ slot_weight, int* __restrict__ token_slot,
                                                    float* __restrict__ token_weight, long long rows, int S, int EC) {
  __shared__ int count[8];
  const int wib = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * 8 + wib;
  if (row >= rows) return;
  const long long b = row / S;
  const int s = (int)(row - b * S);
  if (lane == 0) count[wib] = 0;
  if (lane < 2) { token_slot[row * 2 + lane] = -1; token_weight[row * 2 + lane] = 0.f; }
  __syncwarp();
  const __nv_bfloat16* src = dense + row * EC;
  auto found = [&](int ec, float v) {
    slot_token[b * EC + ec] = s;
    slot_weight[b * EC + ec] = v;
    const int k = atomicAdd(&count[wib], 1);
    if (k < 2) { token_slot[row * 2 + k] = ec; token_weight[row * 2 + k] = v; }
  };
  if ((EC & 7) == 0 && (reinterpret_cast<uintptr_t>(dense) & 15u) == 0) {
    for (int g = lane; g < EC / 8; g += 32) {
      const uint4 v = *reinterpret_cast<const uint4*>(src + 8 * g);
      if ((v.x | v.y | v.z | v.w) == 0u) continue;             // the common case: eight zeros
      const unsigned w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float lo = __uint_as_float(w[i] << 16), hi = __uint_as_float(w[i] & 0xffff0000u);
        if (lo != 0.f) found(8 * g + 2 * i, lo);
        if (hi != 0.f) found(8 * g + 2 * i + 1, hi);
      }
    }
  } else {
    for (int ec = lane; ec < EC; ec += 32) {
      const float v = __bfloat162float(src[ec]);
      if (v != 0.f) found(ec, v);
    }
  }
}

// Where row (b, slot) of a (b, e, c, d) tensor starts: batch-major memory (cap == 0) or expert-major memory
// (e, b, c, d) with capacity `cap` - the layout the expert GEMMs work on, so that no copy stands between them and
// the gathers.
__device__ __forceinline__ long long row_offset(long long b, int slot, int B, int EC, int cap, int D) {
  if (cap == 0) return (b * EC + slot) * (long long)D;
  const int e = slot / cap, c = slot - e * cap;
  return (((long long)e * B + b) * cap + c) * (long long)D;
}

// rows[b, slot, :] = weight * x[b, token, :] (zero for an empty slot); one block of 128 threads per slot row
__global__ void __launch_bounds__(128) rows_from_tokens_kernel(__nv_bfloat16* __restrict__ rows, const __nv_bfloat16* __restrict__ x,
                                                               const int* __restrict__ slot_token, const float* __restrict__ slot_weight,
                                                               int B, int S, int EC, int D, long long x_sb, long long x_ss, int cap) {
  const long long r = blockIdx.x;             // b * EC + slot
  const long long b = r / EC;
  const int tok = slot_token[r];
  const float w = (tok >= 0) ? (slot_weight ? slot_weight[r] : 1.f) : 0.f;
  __nv_bfloat16* dst = rows + row_offset(b, (int)(r - b * EC), B, EC, cap, D);
  const __nv_bfloat16* src = x + b * x_sb + (tok >= 0 ? tok : 0) * x_ss;
  for (int g = threadIdx.x; g < D / 8; g += blockDim.x) {
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (tok >= 0) {
      v = *reinterpret_cast<const uint4*>(src + 8 * g);
      if (w != 1.f) {
        unsigned q[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(q[i] << 16) * w, __uint_as_float(q[i] & 0xffff0000u) * w);
          q[i] = *reinterpret_cast<const unsigned*>(&h);
        }
        v = make_uint4(q[0], q[1], q[2], q[3]);
      }
    }
    *reinterpret_cast<uint4*>(dst + 8 * g) = v;
  }
}

// y[b, s, :] = sum_k weight_k * rows[b, slot_k, :]; one block of 128 threads per token
__global__ void __launch_bounds__(128) tokens_from_rows_kernel(__nv_bfloat16* __restrict__ y, const __nv_bfloat16* __restrict__ rows,
                                                               const int* __restrict__ token_slot, const float* __restrict__ token_weight,
                                                               int B, int S, int EC, int D, int unit_weights, long long y_sb, long long y_ss, int cap) {
  const long long t = blockIdx.x;             // b * S + s
  const long long b = t / S;
  const int s0 = token_slot[2 * t], s1 = token_slot[2 * t + 1];
  const float w0 = s0 >= 0 ? (unit_weights ? 1.f : token_weight[2 * t]) : 0.f, w1 = s1 >= 0 ? (unit_weights ? 1.f : token_weight[2 * t + 1]) : 0.f;
  const __nv_bfloat16* r0 = rows + row_offset(b, s0 >= 0 ? s0 : 0, B, EC, cap, D);
  const __nv_bfloat16* r1 = rows + row_offset(b, s1 >= 0 ? s1 : 0, B, EC, cap, D);
  __nv_bfloat16* dst = y + b * y_sb + (t - b * S) * y_ss;
  for (int g = threadIdx.x; g < D / 8; g += blockDim.x) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (s0 >= 0) {
      const uint4 v = *reinterpret_cast<const uint4*>(r0 + 8 * g);
      const unsigned q[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) { acc[2 * i] = __uint_as_float(q[i] << 16) * w0; acc[2 * i + 1] = __uint_as_float(q[i] & 0xffff0000u) * w0; }
    }
    if (s1 >= 0) {
      const uint4 v = *reinterpret_cast<const uint4*>(r1 + 8 * g);
      const unsigned q[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) { acc[2 * i] = fmaf(__uint_as_float(q[i] << 16), w1, acc[2 * i]); acc[2 * i + 1] = fmaf(__uint_as_float(q[i] & 0xffff0000u), w1, acc[2 * i + 1]); }
    }
    unsigned o[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const __nv_bfloat162 h = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
      o[i] = *reinterpret_cast<const unsigned*>(&h);
    }
    *reinterpret_cast<uint4*>(dst + 8 * g) = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

// d_dense[b, s, slot_k] = <rows[b, slot_k, :], dy[b, s, :]> for the token's (at most two) slots; one warp per (token, k)
__global__ void __launch_bounds__(256) weight_grad_kernel(__nv_bfloat16* __restrict__ d_dense, const __nv_bfloat16* __restrict__ rows,
                                                          const __nv_bfloat16* __restrict__ dy, const int* __restrict__ token_slot,
                                                          long long pairs, int B, int S, int EC, int D, long long dy_sb, long long dy_ss, int cap) {
  const long long pr = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);      // token * 2 + k
  if (pr >= pairs) return;
  const int lane = threadIdx.x & 31;
  const int slot = token_slot[pr];
  if (slot < 0) return;
  const long long t = pr >> 1, b = t / S;
  const __nv_bfloat16* r = rows + row_offset(b, slot, B, EC, cap, D);
  const __nv_bfloat16* g = dy + b * dy_sb + (t - b * S) * dy_ss;
  float acc = 0.f;
  for (int i = lane; i < D / 8; i += 32) {
    const uint4 a = *reinterpret_cast<const uint4*>(r + 8 * i), c = *reinterpret_cast<const uint4*>(g + 8 * i);
    const unsigned aw[4] = {a.x, a.y, a.z, a.w}, cw[4] = {c.x, c.y, c.z, c.w};
#pragma unroll
    for (int k = 0; k < 4; ++k)
      acc += __uint_as_float(aw[k] << 16) * __uint_as_float(cw[k] << 16) + __uint_as_float(aw[k] & 0xffff0000u) * __uint_as_float(cw[k] & 0xffff0000u);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (lane == 0) d_dense[t * EC + slot] = __float2bfloat16_rn(acc);
}

static int check(const char* what, int64_t B, int64_t S, int64_t EC, int64_t D) {
  if (B < 0 || S < 0 || EC < 0 || D < 0) return fail(HAPX_ERR_EXTENT, std::string(what) + ": negative extent");
  if (D % 8 != 0) return fail(HAPX_ERR_EXTENT, std::string(what) + ": the row width must be a multiple of 8");
  if (B * S > 0x7fffffff || B * EC > 0x7fffffff || S > 0x7fffffff || EC > 0x7fffffff) return fail(HAPX_ERR_EXTENT, std::string(what) + ": extent out of range");
  return HAPX_OK;
}

}  // namespace moe
}  // namespace hapx

using namespace hapx;

extern "C" {

int hapx_moe_index(const void* dense, int32_t* slot_token, float* slot_weight, int32_t* token_slot, float* token_weight, int64_t B,
                   int64_t S, int64_t EC, hapx_stream stream_) {
  if (int e = moe::check("moe_index", B, S, EC, 0)) return e;
  if (B * S * EC == 0) return HAPX_OK;
  if (!dense || !slot_token || !slot_weight || !token_slot || !token_weight) return fail(HAPX_ERR_ARGUMENT, "moe_index: null pointer");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  HAPX_CUDA(cudaMemsetAsync(slot_token, 0xff, (size_t)(B * EC) * sizeof(int32_t), stream));     // -1: empty slot
  const long long rows = B * S;
  moe::index_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(dense), slot_token, slot_weight, token_slot,
                                                                  token_weight, rows, (int)S, (int)EC);
  HAPX_CUDA(cudaGetLastError());
  count_launch();
  return HAPX_OK;
}

static int check_layout(const char* what, int64_t EC, int64_t sb, int64_t ss, int64_t cap) {
  if (sb < 0 || ss < 0 || (sb % 8) != 0 || (ss % 8) != 0) return fail(HAPX_ERR_EXTENT, std::string(what) + ": token strides must be non-negative multiples of 8 elements");
  if (cap < 0 || (cap > 0 && EC % cap != 0)) return fail(HAPX_ERR_EXTENT, std::string(what) + ": the capacity must divide the number of slots");
  return HAPX_OK;
}

int hapx_moe_rows_from_tokens(void* rows, const void* x, const int32_t* slot_token, const float* slot_weight, int64_t B, int64_t S,
                              int64_t EC, int64_t D, hapx_stream stream_) {
  return hapx_moe_rows_from_tokens_strided(rows, x, slot_token, slot_weight, B, S, EC, D, S * D, D, 0, stream_);
}

int hapx_moe_rows_from_tokens_strided(void* rows, const void* x, const int32_t* slot_token, const float* slot_weight, int64_t B, int64_t S,
                                      int64_t EC, int64_t D, int64_t x_stride_b, int64_t x_stride_s, int64_t rows_capacity, hapx_stream stream_) {
  if (int e = moe::check("moe_rows_from_tokens", B, S, EC, D)) return e;
  if (int e = check_layout("moe_rows_from_tokens", EC, x_stride_b, x_stride_s, rows_capacity)) return e;
  if (B * EC * D == 0) return HAPX_OK;
  if (!rows || !x || !slot_token) return fail(HAPX_ERR_ARGUMENT, "moe_rows_from_tokens: null pointer");
  moe::rows_from_tokens_kernel<<<(unsigned)(B * EC), 128, 0, static_cast<cudaStream_t>(stream_)>>>(
      static_cast<__nv_bfloat16*>(rows), static_cast<const __nv_bfloat16*>(x), slot_token, slot_weight, (int)B, (int)S, (int)EC, (int)D,
      (long long)x_stride_b, (long long)x_stride_s, (int)rows_capacity);
  HAPX_CUDA(cudaGetLastError());
  count_launch();
  return HAPX_OK;
}

int hapx_moe_tokens_from_rows(void* y, const void* rows, const int32_t* token_slot, const float* token_weight, int64_t B, int64_t S,
                              int64_t EC, int64_t D, hapx_stream stream_) {
  return hapx_moe_tokens_from_rows_strided(y, rows, token_slot, token_weight, B, S, EC, D, S * D, D, 0, stream_);
}

int hapx_moe_tokens_from_rows_strided(void* y, const void* rows, const int32_t* token_slot, const float* token_weight, int64_t B, int64_t S,
                                      int64_t EC, int64_t D, int64_t y_stride_b, int64_t y_stride_s, int64_t rows_capacity, hapx_stream stream_) {
  if (int e = moe::check("moe_tokens_from_rows", B, S, EC, D)) return e;
  if (int e = check_layout("moe_tokens_from_rows", EC, y_stride_b, y_stride_s, rows_capacity)) return e;
  if (B * S * D == 0) return HAPX_OK;
  if (!y || !rows || !token_slot) return fail(HAPX_ERR_ARGUMENT, "moe_tokens_from_rows: null pointer");
  moe::tokens_from_rows_kernel<<<(unsigned)(B * S), 128, 0, static_cast<cudaStream_t>(stream_)>>>(
      static_cast<__nv_bfloat16*>(y), static_cast<const __nv_bfloat16*>(rows), token_slot, token_weight, (int)B, (int)S, (int)EC, (int)D,
      token_weight == nullptr ? 1 : 0, (long long)y_stride_b, (long long)y_stride_s, (int)rows_capacity);
  HAPX_CUDA(cudaGetLastError());
  count_launch();
  return HAPX_OK;
}

int hapx_moe_weight_grad(void* d_dense, const void* rows, const void* dy, const int32_t* token_slot, int64_t B, int64_t S, int64_t EC,
                         int64_t D, hapx_stream stream_) {
  return hapx_moe_weight_grad_strided(d_dense, rows, dy, token_slot, B, S, EC, D, S * D, D, 0, stream_);
}

int hapx_moe_weight_grad_strided(void* d_dense, const void* rows, const void* dy, const int32_t* token_slot, int64_t B, int64_t S, int64_t EC,
                                 int64_t D, int64_t dy_stride_b, int64_t dy_stride_s, int64_t rows_capacity, hapx_stream stream_) {
  if (int e = moe::check("moe_weight_grad", B, S, EC, D)) return e;
  if (int e = check_layout("moe_weight_grad", EC, dy_stride_b, dy_stride_s, rows_capacity)) return e;
  if (B * S * EC == 0) return HAPX_OK;
  if (!d_dense || !rows || !dy || !token_slot) return fail(HAPX_ERR_ARGUMENT, "moe_weight_grad: null pointer");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  HAPX_CUDA(cudaMemsetAsync(d_dense, 0, (size_t)(B * S * EC) * 2, stream));
  const long long pairs = B * S * 2;
  moe::weight_grad_kernel<<<(unsigned)((pairs + 7) / 8), 256, 0, stream>>>(static_cast<__nv_bfloat16*>(d_dense), static_cast<const __nv_bfloat16*>(rows),
                                                                          static_cast<const __nv_bfloat16*>(dy), token_slot, pairs, (int)B, (int)S, (int)EC, (int)D,
                                                                          (long long)dy_stride_b, (long long)dy_stride_s, (int)rows_capacity);
  HAPX_CUDA(cudaGetLastError());
  count_launch();
  return HAPX_OK;
}

}  // extern "C"
