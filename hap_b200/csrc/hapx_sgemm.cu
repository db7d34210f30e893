// fp32 linear (forward, dgrad, wgrad) on the CUDA cores.
//
// tcgen05 has no fp32 multiply (kind::tf32 keeps 10 mantissa bits), and the fp32 configuration
// of the benchmark must match the reference to 1e-5, so fp32 operands take this FFMA kernel:
// 64 x 64 output tile, 16-deep shared-memory slices, 4 x 4 outputs per thread, fp32 accumulate.
// It serves the correctness configuration (a 2-layer MLP); the throughput path is bf16.
#include <cuda_runtime.h>

#include <string>

#include "hapx_internal.h"

namespace hapx {
namespace sgemm {

constexpr int TM = 64, TN = 64, TK = 16;

// D[i,j] = sum_k A(i,k) * B(j,k) (+ bias[j]); A(i,k) = A[i*a_i + k*a_k], B(j,k) = B[j*b_j + k*b_k].
__global__ void __launch_bounds__(256) sgemm_kernel(const float* __restrict__ A, long long a_i, long long a_k,
                                                    const float* __restrict__ B, long long b_j, long long b_k,
                                                    const float* __restrict__ bias, float* __restrict__ D, long long ldd,
                                                    int M, int N, int K, int epilogue) {
  __shared__ float As[TK][TM + 1];
  __shared__ float Bs[TK][TN + 1];
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int m0 = blockIdx.y * TM, n0 = blockIdx.x * TN;
  float acc[4][4] = {};
  for (int k0 = 0; k0 < K; k0 += TK) {
    // 64 x 16 elements per operand, 256 threads -> 4 each; walk the contiguous direction fastest
    for (int e = threadIdx.x; e < TM * TK; e += 256) {
      int i, k;
      if (a_k == 1) { k = e % TK; i = e / TK; } else { i = e % TM; k = e / TM; }
      const int gi = m0 + i, gk = k0 + k;
      As[k][i] = (gi < M && gk < K) ? A[(long long)gi * a_i + (long long)gk * a_k] : 0.f;
    }
    for (int e = threadIdx.x; e < TN * TK; e += 256) {
      int j, k;
      if (b_k == 1) { k = e % TK; j = e / TK; } else { j = e % TN; k = e / TN; }
      const int gj = n0 + j, gk = k0 + k;
      Bs[k][j] = (gj < N && gk < K) ? B[(long long)gj * b_j + (long long)gk * b_k] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < TK; ++k) {
      float a[4], b[4];
#pragma unroll
      for (int r = 0; r < 4; ++r) { a[r] = As[k][ty * 4 + r]; b[r] = Bs[k][tx * 4 + r]; }
#pragma unroll
      for (int r = 0; r < 4; ++r)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[r][c] = fmaf(a[r], b[c], acc[r][c]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const int gi = m0 + ty * 4 + r;
    if (gi >= M) continue;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const int gj = n0 + tx * 4 + c;
      if (gj >= N) continue;
      float v = acc[r][c] + (bias ? bias[gj] : 0.f);
      if (epilogue == 1) v = v > 0.f ? v : 0.f;
      else if (epilogue == 2) v = 0.5f * v * (1.f + erff(v * 0.70710678118654752f));
      else if (epilogue == 3) v = 1.f / (1.f + expf(-v));
      D[(long long)gi * ldd + gj] = v;
    }
  }
}

// Column sums of g[M,N] in fp32 (bias gradient); one block per 64 columns, rows added in order.
__global__ void __launch_bounds__(256) colsum_f32_kernel(const float* __restrict__ g, long long ldg, int M, int N, float* out) {
  __shared__ float part[4][64];
  const int c = blockIdx.x * 64 + (threadIdx.x & 63), rg = threadIdx.x >> 6;
  float acc = 0.f;
  if (c < N)
    for (int r = rg; r < M; r += 4) acc += g[(long long)r * ldg + c];
  part[rg][threadIdx.x & 63] = acc;
  __syncthreads();
  if (rg == 0 && c < N) out[c] = (part[0][threadIdx.x] + part[1][threadIdx.x]) + (part[2][threadIdx.x] + part[3][threadIdx.x]);
}

int run(const float* A, long long a_i, long long a_k, const float* B, long long b_j, long long b_k, const float* bias, float* D,
        long long ldd, long long M, long long N, long long K, int epilogue, cudaStream_t stream) {
  if (M < 0 || N < 0 || K < 0) return fail(HAPX_ERR_EXTENT, "linear(fp32): negative extent");
  if (M == 0 || N == 0) return HAPX_OK;
  if (M > 0x7fffffff || N > 0x7fffffff || K > 0x7fffffff) return fail(HAPX_ERR_EXTENT, "linear(fp32): extent exceeds 2^31");
  if (!A || !B || !D) return fail(HAPX_ERR_ARGUMENT, "linear(fp32): null pointer");
  dim3 grid((unsigned)((N + TN - 1) / TN), (unsigned)((M + TM - 1) / TM));
  if (grid.y > 65535) return fail(HAPX_ERR_EXTENT, "linear(fp32): too many row tiles");
  sgemm_kernel<<<grid, 256, 0, stream>>>(A, a_i, a_k, B, b_j, b_k, bias, D, ldd, (int)M, (int)N, (int)K, epilogue);
  HAPX_CUDA(cudaGetLastError());
  count_launch();
  return HAPX_OK;
}

int colsum(const float* g, long long m, long long n, float* out, cudaStream_t stream) {
  if (n == 0) return HAPX_OK;
  colsum_f32_kernel<<<(unsigned)((n + 63) / 64), 256, 0, stream>>>(g, n, (int)m, (int)n, out);
  HAPX_CUDA(cudaGetLastError());
  count_launch();
  return HAPX_OK;
}

}  // namespace sgemm
}  // namespace hapx
