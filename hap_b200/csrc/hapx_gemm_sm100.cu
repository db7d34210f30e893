// Uneven-shard GEMMs for F.linear (forward, dgrad, wgrad) on Blackwell tensor cores.
//
// One persistent, warp-specialised kernel: D[M,N] = A[M,Kc] * B[N,Kc]^T (+ bias, activation)
// with bf16 operands and fp32 accumulation in tensor memory.
//
//   warp 0      : TMA producer (cp.async.bulk.tensor, 128-byte swizzle) into a ring of stages
//   warp 1      : allocates TMEM, one elected thread issues tcgen05.mma (cta_group::1, 128 x BN x 16)
//   warps 2..5  : epilogue - tcgen05.ld the accumulator, bias / activation / cast, global stores
//
// Two accumulator buffers in TMEM let the epilogue of tile i run under the main loop of tile
// i+1.  Either operand may be "K-major" (contraction index contiguous in memory) or "MN-major"
// (output index contiguous), which is what dgrad (B = W as stored) and wgrad (A = g^T, B = x^T
// as stored) need: no transposed copies are ever made.  Ragged shard extents (M = 38, N = 2458,
// ...) are handled by TMA's zero fill on loads and by predicated stores, so no operand is padded.
//
// Every mbarrier wait is bounded; on expiry the kernel raises an error word, leaves its loops,
// frees its TMEM and returns.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>
#include <vector>

#include "hapx_internal.h"
#include "hapx_tc.h"

namespace hapx {
namespace gemm {

constexpr int BM = 128;
constexpr int BK = 64;                 // bf16 elements: one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int kThreads = 192;
constexpr int kEpilogueThreads = 128;

enum Epilogue { EPI_NONE = 0, EPI_RELU = 1, EPI_GELU = 2, EPI_SIGMOID = 3 };

struct Params {
  int M, N, Kc;           // D is M x N, contraction length Kc
  long long ldd;          // elements between rows of D
  void* D;
  const void* bias;       // N values of the input dtype, or null
  int epilogue;
  int out_f32;            // D is fp32 instead of bf16
  int m_tiles, n_tiles, k_blocks;
  unsigned* error;        // device word: 0 or a code left by a wait that ran out
  int tma_store;          // D's pitch and base allow bulk tensor stores
  int fast_drain;         // tma_store, no activation, and the bias (if any) can be read as aligned 16-byte groups: see drain_fast
  int splits;             // > 1: the contraction is cut into `splits` ranges of kb_per_split slices, each
  int kb_per_split;       //      writing an fp32 partial tile to rows [split * m_pad, ...) of the workspace
  int m_pad;
  int a_chunked, b_chunked;  // pair kernel: the MN-major operand's map is the 5-D one (two 64-element chunks per load); for B the
                          // 4-D map then travels in the half-width slot
  int tail_begin;         // pair kernel: tiles [tail_begin, m_tiles * n_tiles) are worked on as two half-width units each, so that
                          // the last, partly filled round of tiles takes half as long (only without batching and split-K)
  // batched operation: `batch` independent GEMMs; batch index b = b_out * batch_in + b_in and every
  // tensor map carries (b_in, b_out) as its 3rd and 4th coordinate.  Element strides of D for the
  // direct-store path:
  int batch, batch_in;
  long long d_stride_in, d_stride_out;
  int a_shared_out, b_shared_out;   // operand does not depend on b_out (e.g. expert weights): its maps get coordinate 0
};

using namespace tc;   // PTX wrappers (hapx_tc.h)

// ---- epilogue -------------------------------------------------------------------------------------
constexpr unsigned kStoreTileBytes = 128 * 128;   // staging: 128 rows x 128 bytes (64 bf16 or 32 fp32 columns), two of them
constexpr unsigned kWarpTileBytes = 32 * 128;     // the 32 rows one epilogue warp owns

__device__ __forceinline__ float apply_epilogue(float v, int epi) {
  switch (epi) {
    case EPI_RELU: return v > 0.f ? v : 0.f;
    case EPI_GELU: return 0.5f * v * (1.f + erff(v * 0.70710678118654752f));
    case EPI_SIGMOID: return 1.f / (1.f + __expf(-v));
    default: return v;
  }
}

// Convert 32 accumulator columns (one tcgen05.ld) of this thread's row and put them into the
// warp's swizzled staging tile.  `piece` says which part of the 128-byte staging row they fill.
template <bool OUT_F32, bool BIAS>
__device__ __forceinline__ void stage_columns(const unsigned (&r)[32], unsigned char* tile_row, int sw, int piece,
                                              const __nv_bfloat16* bias, int col, int N) {
  float v[32];
#pragma unroll
  for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
  if constexpr (BIAS) {
#pragma unroll
    for (int g = 0; g < 4; ++g) {   // 8 bias values per 16-byte load, the same address in every lane
      const uint4 raw = __ldg(reinterpret_cast<const uint4*>(bias + ((col + 8 * g + 8 <= N) ? col + 8 * g : 0)));
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __bfloat1622float2(h[e]);
        v[8 * g + 2 * e] += f.x;
        v[8 * g + 2 * e + 1] += f.y;
      }
    }
  }
  if constexpr (OUT_F32) {
#pragma unroll
    for (int j = 0; j < 8; ++j)
      *reinterpret_cast<float4*>(tile_row + ((j ^ sw) << 4)) = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
  } else {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      __nv_bfloat162 h0 = __floats2bfloat162_rn(v[8 * j], v[8 * j + 1]), h1 = __floats2bfloat162_rn(v[8 * j + 2], v[8 * j + 3]);
      __nv_bfloat162 h2 = __floats2bfloat162_rn(v[8 * j + 4], v[8 * j + 5]), h3 = __floats2bfloat162_rn(v[8 * j + 6], v[8 * j + 7]);
      uint4 pk;
      pk.x = *reinterpret_cast<unsigned*>(&h0); pk.y = *reinterpret_cast<unsigned*>(&h1);
      pk.z = *reinterpret_cast<unsigned*>(&h2); pk.w = *reinterpret_cast<unsigned*>(&h3);
      *reinterpret_cast<uint4*>(tile_row + (((4 * piece + j) ^ sw) << 4)) = pk;
    }
  }
}

// The common epilogue (bulk tensor stores, no activation, bias absent or readable in aligned
// 16-byte groups straight from global memory): no shared bias tile and no barrier between the
// epilogue warps, and the tcgen05.ld of the next 32 columns is in flight while the current ones
// are converted.  The output width is a multiple of 8 (bf16) or 4 (fp32) here, so a group of 32
// columns that starts inside the matrix may only overhang it by whole 16-byte groups; the
// overhang is clipped by the tensor map and its bias reads are redirected to the first group
// (with a bias the width is a multiple of 8 for either output type).
template <int BN, bool OUT_F32, bool BIAS>
__device__ __forceinline__ void drain_fast(const Params& p, const CUtensorMap* tmD, unsigned char* stage_gen, unsigned stage_u32,
                                           unsigned t_row, int m0, int n0, int bi, int bo, int q, int lane, int& buf, int width = BN) {
  constexpr int PIECES = OUT_F32 ? 1 : 2;          // 32-column groups per 128-byte staging row
  const int GROUPS = width / 32;
  unsigned char* warp_gen = stage_gen + q * (2 * kWarpTileBytes);
  const unsigned warp_u32 = stage_u32 + q * (2 * kWarpTileBytes);
  const int sw = lane & 7;
  const __nv_bfloat16* bias = reinterpret_cast<const __nv_bfloat16*>(p.bias);
  const int live = min(GROUPS, (p.N - n0 + 31) / 32);   // groups that start inside the matrix (same in every thread)
  unsigned char* row0 = warp_gen + lane * 128;
  // one step: wait for `cur`, start loading the next group into `nxt`, convert and stage `cur`
  auto step = [&](const unsigned (&cur)[32], unsigned (&nxt)[32], int g, int piece) {
    tmem_ld_wait();
    if (g + 1 < live) tmem_ld_32x32(t_row + (unsigned)(32 * (g + 1)), nxt);
    if (piece == 0) {
      if (lane == 0) bulk_wait_read_1();             // the store this warp issued two tiles ago has left the buffer
      __syncwarp();
    }
    stage_columns<OUT_F32, BIAS>(cur, row0 + buf * kWarpTileBytes, sw, piece, bias, n0 + 32 * g, p.N);
    if (piece == PIECES - 1 || g + 1 == live) {
      fence_proxy_async();                           // make the rows visible to the bulk-copy engine
      __syncwarp();
      if (lane == 0) {
        tma_store_4d(tmD, warp_u32 + buf * kWarpTileBytes, n0 + 32 * (g - piece), m0 + q * 32, bi, bo);
        bulk_commit_group();
      }
      buf ^= 1;
    }
  };
  unsigned ra[32], rb[32];
  tmem_ld_32x32(t_row, ra);
#pragma unroll 1
  for (int g = 0; g < live; g += 2) {
    step(ra, rb, g, 0);
    if (g + 1 < live) step(rb, ra, g + 1, PIECES - 1);
  }
}

template <int BN>
__device__ __forceinline__ void drain_fast_any(const Params& p, const CUtensorMap* tmD, unsigned char* stage_gen, unsigned stage_u32,
                                               unsigned t_row, int m0, int n0, int bi, int bo, int q, int lane, int& buf, int width = BN) {
  if (p.out_f32) {
    if (p.bias) drain_fast<BN, true, true>(p, tmD, stage_gen, stage_u32, t_row, m0, n0, bi, bo, q, lane, buf, width);
    else drain_fast<BN, true, false>(p, tmD, stage_gen, stage_u32, t_row, m0, n0, bi, bo, q, lane, buf, width);
  } else {
    if (p.bias) drain_fast<BN, false, true>(p, tmD, stage_gen, stage_u32, t_row, m0, n0, bi, bo, q, lane, buf, width);
    else drain_fast<BN, false, false>(p, tmD, stage_gen, stage_u32, t_row, m0, n0, bi, bo, q, lane, buf, width);
  }
}

// Drain one 128 x BN accumulator tile: this thread owns row (q*32 + lane) of it.
// With `use_tma` every warp works on its own: it converts 128 bytes per row into a private,
// 128-byte-swizzled 32-row staging tile (two of them, used alternately) and its lane 0 sends the
// tile off as one bulk tensor store (coalesced, clipped at the matrix edge by the tensor map).
// No barrier between warps is involved.  Otherwise each thread stores its own row segments
// directly (any row pitch, any alignment).
template <int BN>
__device__ __forceinline__ void drain_tile(const Params& p, const CUtensorMap* tmD, bool use_tma, unsigned char* stage_gen,
                                           unsigned stage_u32, const float* bias_tile, unsigned t_row, int m0, int n0, int bi, int bo,
                                           int q, int lane, int et, int& buf) {
  const int row_in_tile = q * 32 + lane;
  const int row = m0 + row_in_tile;
  if (use_tma) {
    constexpr int CH = 32;   // accumulator columns per tcgen05.ld
    const int cols_per_store = p.out_f32 ? 32 : 64;
    unsigned char* warp_gen = stage_gen + q * (2 * kWarpTileBytes);
    const unsigned warp_u32 = stage_u32 + q * (2 * kWarpTileBytes);
    const int sw = lane & 7;
#pragma unroll 1
    for (int c0 = 0; c0 < BN; c0 += cols_per_store) {
      if (n0 + c0 >= p.N) break;                       // same decision in every thread
      unsigned r0[32], r1[32];
      tmem_ld_32x32(t_row + (unsigned)c0, r0);
      if (!p.out_f32) tmem_ld_32x32(t_row + (unsigned)(c0 + CH), r1);
      tmem_ld_wait();
      if (lane == 0) bulk_wait_read_1();               // the store this warp issued two chunks ago has left the buffer
      __syncwarp();
      unsigned char* tile = warp_gen + buf * kWarpTileBytes + lane * 128;
      if (p.out_f32) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          float4 o;
          o.x = apply_epilogue(__uint_as_float(r0[4 * j]) + bias_tile[c0 + 4 * j], p.epilogue);
          o.y = apply_epilogue(__uint_as_float(r0[4 * j + 1]) + bias_tile[c0 + 4 * j + 1], p.epilogue);
          o.z = apply_epilogue(__uint_as_float(r0[4 * j + 2]) + bias_tile[c0 + 4 * j + 2], p.epilogue);
          o.w = apply_epilogue(__uint_as_float(r0[4 * j + 3]) + bias_tile[c0 + 4 * j + 3], p.epilogue);
          *reinterpret_cast<float4*>(tile + ((j ^ sw) << 4)) = o;
        }
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const unsigned* src = (j < 4) ? r0 : r1;
          const int b = (j & 3) * 8, cb = c0 + j * 8;
          float v[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) v[e] = apply_epilogue(__uint_as_float(src[b + e]) + bias_tile[cb + e], p.epilogue);
          __nv_bfloat162 h0 = __floats2bfloat162_rn(v[0], v[1]), h1 = __floats2bfloat162_rn(v[2], v[3]);
          __nv_bfloat162 h2 = __floats2bfloat162_rn(v[4], v[5]), h3 = __floats2bfloat162_rn(v[6], v[7]);
          uint4 pk;
          pk.x = *reinterpret_cast<unsigned*>(&h0); pk.y = *reinterpret_cast<unsigned*>(&h1);
          pk.z = *reinterpret_cast<unsigned*>(&h2); pk.w = *reinterpret_cast<unsigned*>(&h3);
          *reinterpret_cast<uint4*>(tile + ((j ^ sw) << 4)) = pk;
        }
      }
      fence_proxy_async();                             // make the rows visible to the bulk-copy engine
      __syncwarp();
      if (lane == 0) {
        tma_store_4d(tmD, warp_u32 + buf * kWarpTileBytes, n0 + c0, m0 + q * 32, bi, bo);
        bulk_commit_group();
      }
      buf ^= 1;
    }
    return;
  }
  const bool vec_ok = p.out_f32 ? ((p.ldd & 3) == 0 && (reinterpret_cast<uintptr_t>(p.D) & 15u) == 0)
                                : ((p.ldd & 7) == 0 && (reinterpret_cast<uintptr_t>(p.D) & 15u) == 0);
#pragma unroll 1
  for (int c0 = 0; c0 < BN; c0 += 32) {
    unsigned r[32];
    tmem_ld_32x32(t_row + (unsigned)c0, r);
    tmem_ld_wait();
    if (row < p.M && n0 + c0 < p.N) {
      float v[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] = apply_epilogue(__uint_as_float(r[j]) + bias_tile[c0 + j], p.epilogue);
      const int ncols = min(32, p.N - (n0 + c0));
      if (p.out_f32) {
        float* out = reinterpret_cast<float*>(p.D) + bo * p.d_stride_out + bi * p.d_stride_in + (long long)row * p.ldd + n0 + c0;
        if (vec_ok && ncols == 32) {
#pragma unroll
          for (int j = 0; j < 32; j += 4) *reinterpret_cast<float4*>(out + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) if (j < ncols) out[j] = v[j];
        }
      } else {
        __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.D) + bo * p.d_stride_out + bi * p.d_stride_in + (long long)row * p.ldd + n0 + c0;
        if (vec_ok && ncols == 32) {
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            uint4 pk;
            __nv_bfloat162 h0 = __floats2bfloat162_rn(v[j], v[j + 1]), h1 = __floats2bfloat162_rn(v[j + 2], v[j + 3]);
            __nv_bfloat162 h2 = __floats2bfloat162_rn(v[j + 4], v[j + 5]), h3 = __floats2bfloat162_rn(v[j + 6], v[j + 7]);
            pk.x = *reinterpret_cast<unsigned*>(&h0); pk.y = *reinterpret_cast<unsigned*>(&h1);
            pk.z = *reinterpret_cast<unsigned*>(&h2); pk.w = *reinterpret_cast<unsigned*>(&h3);
            *reinterpret_cast<uint4*>(out + j) = pk;
          }
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) if (j < ncols) out[j] = __float2bfloat16_rn(v[j]);
        }
      }
    }
  }
}


template <int BN, bool A_MN, bool B_MN>
struct Cfg {
  static constexpr int STAGES = (BN >= 256) ? 4 : (BN >= 128 ? 6 : 8);
  static constexpr unsigned A_BYTES = BM * BK * 2;
  static constexpr unsigned B_BYTES = BN * BK * 2;
  static constexpr unsigned STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr unsigned TMEM_COLS = (2 * BN <= 32) ? 32 : (2 * BN <= 64 ? 64 : (2 * BN <= 128 ? 128 : (2 * BN <= 256 ? 256 : 512)));
  // dynamic shared memory: stages (1024-byte aligned) + bias tile + barriers
  static constexpr unsigned SMEM_BYTES = 1024 + STAGES * STAGE_BYTES + 2 * kStoreTileBytes + BN * 4 + 256;
  // instruction descriptor: fp32 accumulate, bf16 x bf16, majors, N >> 3, M >> 4
  static constexpr unsigned IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((A_MN ? 1u : 0u) << 15) | ((B_MN ? 1u : 0u) << 16) |
                                    ((unsigned)(BN >> 3) << 17) | ((unsigned)(BM >> 4) << 24);
};

template <int BN, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(kThreads, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ CUtensorMap tmD, const Params p) {
  using C = Cfg<BN, A_MN, B_MN>;
  extern __shared__ unsigned char smem_raw[];
  const unsigned base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  unsigned char* gen_base = smem_raw + (base - smem_u32(smem_raw));
  constexpr unsigned kOff = C::STAGES * C::STAGE_BYTES + 2 * kStoreTileBytes;   // stages, then the two store tiles
  unsigned char* store_gen = gen_base + C::STAGES * C::STAGE_BYTES;
  const unsigned store_u32 = base + C::STAGES * C::STAGE_BYTES;
  float* bias_tile = reinterpret_cast<float*>(gen_base + kOff);
  const unsigned bars = base + kOff + BN * 4;
  // barrier map (8 bytes each): full[s], empty[s], tmem_full[2], tmem_empty[2]; then the TMEM address slot
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (C::STAGES + s); };
  auto tfull_bar = [&](int a) { return bars + 8u * (2 * C::STAGES + a); };
  auto tempty_bar = [&](int a) { return bars + 8u * (2 * C::STAGES + 2 + a); };
  const unsigned tmem_slot = bars + 8u * (2 * C::STAGES + 4);
  volatile unsigned* tmem_slot_gen = reinterpret_cast<volatile unsigned*>(gen_base + kOff + BN * 4 + 8 * (2 * C::STAGES + 4));
  volatile unsigned* abort_flag = tmem_slot_gen + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_per_batch = p.m_tiles * p.n_tiles;
  const int total_tiles = tiles_per_batch * p.batch;

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(tfull_bar(a), 1); mbar_init(tempty_bar(a), kEpilogueThreads); }
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tensormap(&tmA);
    prefetch_tensormap(&tmB);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, C::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const unsigned tmem_base = *tmem_slot_gen;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      int stage = 0;
      unsigned phase = 0;
      bool ok = true;
      for (int unit = blockIdx.x; unit < total_tiles && ok; unit += gridDim.x) {
        const int b = unit / tiles_per_batch, tile = unit - b * tiles_per_batch;
        const int bo = b / p.batch_in, bi = b - bo * p.batch_in;
        const int boA = p.a_shared_out ? 0 : bo, boB = p.b_shared_out ? 0 : bo;
        const int m0 = (tile % p.m_tiles) * BM, n0 = (tile / p.m_tiles) * BN;
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u)) { ok = false; break; }
          const unsigned sa = base + stage * C::STAGE_BYTES, sb = sa + C::A_BYTES;
          mbar_expect_tx(full_bar(stage), C::STAGE_BYTES);
          const int k0 = kb * BK;
          if (!A_MN) {
            tma_load_4d(sa, &tmA, k0, m0, bi, boA, full_bar(stage));        // box {64 k, 128 m}
          } else {
#pragma unroll
            for (int i = 0; i < BM / 64; ++i)                                // boxes {64 m, 64 k}
              tma_load_4d(sa + i * 8192u, &tmA, m0 + 64 * i, k0, bi, boA, full_bar(stage));
          }
          if (!B_MN) {
            tma_load_4d(sb, &tmB, k0, n0, bi, boB, full_bar(stage));        // box {64 k, BN n}
          } else {
#pragma unroll
            for (int i = 0; i < BN / 64; ++i)                                // boxes {64 n, 64 k}
              tma_load_4d(sb + i * 8192u, &tmB, n0 + 64 * i, k0, bi, boB, full_bar(stage));
          }
          if (++stage == C::STAGES) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok) { *abort_flag = 1; atomicCAS(p.error, 0u, 1u); }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      int stage = 0, acc = 0;
      unsigned phase = 0, acc_phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1u)) { ok = false; break; }
        tc_fence_after();
        const unsigned d_tmem = tmem_base + (unsigned)(acc * BN);
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!mbar_wait(full_bar(stage), phase)) { ok = false; break; }
          tc_fence_after();
          const unsigned sa = base + stage * C::STAGE_BYTES, sb = sa + C::A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            // K-major: 16 elements = 32 bytes further inside the 128-byte swizzle row;
            // MN-major: 16 contraction rows of 128 bytes further
            const unsigned long long da = A_MN ? make_desc(sa + k * 2048u, 8192u, 1024u) : make_desc(sa + k * 32u, 16u, 1024u);
            const unsigned long long db = B_MN ? make_desc(sb + k * 2048u, 8192u, 1024u) : make_desc(sb + k * 32u, 16u, 1024u);
            umma_bf16(d_tmem, da, db, C::IDESC, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit(empty_bar(stage));   // frees the stage once these MMAs have read it
          if (++stage == C::STAGES) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        umma_commit(tfull_bar(acc));       // accumulator complete
        if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
      }
      if (!ok) { *abort_flag = 1; atomicCAS(p.error, 0u, 2u); }
    }
  } else {
    // ---------------- epilogue (warps 2..5) ----------------
    const int q = warp & 3;                       // TMEM lane quarter this warp may read
    const int et = threadIdx.x - 64;              // 0..127
    int acc = 0;
    unsigned acc_phase = 0;
    bool ok = true;
    int store_buf = 0;
    for (int unit = blockIdx.x; unit < total_tiles && ok; unit += gridDim.x) {
      const int b = unit / tiles_per_batch, tile = unit - b * tiles_per_batch;
      const int bo = b / p.batch_in, bi = b - bo * p.batch_in;
      const int m0 = (tile % p.m_tiles) * BM, n0 = (tile / p.m_tiles) * BN;
      if (!p.fast_drain) {
        // bias tile -> shared (fp32)
        asm volatile("bar.sync 1, 128;" ::: "memory");   // previous tile's readers are done with bias_tile
        for (int j = et; j < BN; j += kEpilogueThreads) {
          float b = 0.f;
          if (p.bias != nullptr && n0 + j < p.N) b = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.bias)[n0 + j]);
          bias_tile[j] = b;
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
      }
      ok = epilogue_all(mbar_wait(tfull_bar(acc), acc_phase));
      if (!ok) break;
      tc_fence_after();
      const unsigned t_row = tmem_base + ((unsigned)(q * 32) << 16) + (unsigned)(acc * BN);
      if (p.fast_drain) drain_fast_any<BN>(p, &tmD, store_gen, store_u32, t_row, m0, n0, bi, bo, q, lane, store_buf);
      else drain_tile<BN>(p, &tmD, p.tma_store != 0, store_gen, store_u32, bias_tile, t_row, m0, n0, bi, bo, q, lane, et, store_buf);
      tc_fence_before();
      mbar_arrive(tempty_bar(acc));     // this thread has drained its part of the accumulator
      if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
    }
    if (lane == 0) bulk_wait_all();   // this warp's bulk stores still read its staging tiles
    if (!ok) { *abort_flag = 1; atomicCAS(p.error, 0u, 3u); }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::TMEM_COLS);
  }
}


// ---- two-CTA variant -----------------------------------------------------------------------------
// A cluster of two CTAs (an SM pair) works on one 256 x 256 output tile with tcgen05.mma
// cta_group::2: CTA c holds rows [128c, 128c+128) of A and of the accumulator, and loads only
// HALF of the B tile (columns [128c, 128c+128) of the output); the tensor cores of both SMs read
// both halves.  Per SM this moves 32 KiB of operands per 64-deep slice instead of 48 KiB, which
// is what lifts the kernel off the L2-to-shared-memory bandwidth limit, and leaves room for 6
// pipeline stages.  The leader CTA (cluster rank 0) issues all MMAs; barrier traffic between the
// two CTAs goes through cluster-mapped mbarriers.  No TMA multicast is used.
__device__ __forceinline__ unsigned cluster_ctarank() {
  unsigned r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ unsigned map_to_cta(unsigned smem_addr, unsigned cta) {
  unsigned r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(cta));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(unsigned cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// TMA load whose completion bytes are credited to an mbarrier of the pair's leader CTA.
__device__ __forceinline__ void tma_load_4d_pair(unsigned dst, const CUtensorMap* map, int x, int y, int bi, int bo, unsigned leader_bar) {
  asm volatile(
      "cp.async.bulk.tensor.4d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];" ::"r"(dst),
      "l"(map), "r"(x), "r"(y), "r"(bi), "r"(bo), "r"(leader_bar)
      : "memory");
}
// The same through a 5-D map (64 contiguous elements, contraction row, 64-element chunk, batch_in, batch_out): one
// instruction fetches the two adjacent 64 x 64 chunks of an MN-major operand tile that otherwise take two.
__device__ __forceinline__ void tma_load_5d_pair(unsigned dst, const CUtensorMap* map, int row, int chunk, int bi, int bo, unsigned leader_bar) {
  asm volatile(
      "cp.async.bulk.tensor.5d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5, %6}], [%7];" ::"r"(dst),
      "l"(map), "r"(0), "r"(row), "r"(chunk), "r"(bi), "r"(bo), "r"(leader_bar)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc2(unsigned dst_smem, unsigned cols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish2() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc2(unsigned taddr, unsigned cols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void umma2_bf16(unsigned d_tmem, unsigned long long a_desc, unsigned long long b_desc, unsigned idesc,
                                           unsigned accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive on the mbarrier at the same offset in BOTH CTAs once all MMAs issued so far are done.
__device__ __forceinline__ void umma2_commit_both(unsigned bar) {
  const unsigned short mask = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar),
               "h"(mask)
               : "memory");
}

template <int BN_, bool A_MN, bool B_MN>
struct Cfg2 {
  static constexpr int BN = BN_;                     // output columns per pair tile
  static constexpr int STAGES = (BN_ >= 256) ? 6 : 8;
  static constexpr unsigned A_BYTES = BM * BK * 2;   // this CTA's 128 rows
  static constexpr unsigned B_BYTES = (BN / 2) * BK * 2;
  static constexpr unsigned STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr unsigned TMEM_COLS = 2 * BN_;
  static constexpr unsigned SMEM_BYTES = 1024 + STAGES * STAGE_BYTES + 2 * kStoreTileBytes + BN * 4 + 256;
  static constexpr unsigned IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((A_MN ? 1u : 0u) << 15) | ((B_MN ? 1u : 0u) << 16) |
                                    ((unsigned)(BN >> 3) << 17) | ((unsigned)((2 * BM) >> 4) << 24);
};

template <int BN, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(kThreads, 1)
gemm2_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                  const __grid_constant__ CUtensorMap tmBh, const __grid_constant__ CUtensorMap tmD, const Params p) {
  using C = Cfg2<BN, A_MN, B_MN>;
  extern __shared__ unsigned char smem_raw[];
  const unsigned base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  unsigned char* gen_base = smem_raw + (base - smem_u32(smem_raw));
  constexpr unsigned kOff = C::STAGES * C::STAGE_BYTES + 2 * kStoreTileBytes;   // stages, then the two store tiles
  unsigned char* store_gen = gen_base + C::STAGES * C::STAGE_BYTES;
  const unsigned store_u32 = base + C::STAGES * C::STAGE_BYTES;
  float* bias_tile = reinterpret_cast<float*>(gen_base + kOff);
  const unsigned bars = base + kOff + BN * 4;
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (C::STAGES + s); };
  auto tfull_bar = [&](int a) { return bars + 8u * (2 * C::STAGES + a); };
  auto tempty_bar = [&](int a) { return bars + 8u * (2 * C::STAGES + 2 + a); };
  const unsigned tmem_slot = bars + 8u * (2 * C::STAGES + 4);
  volatile unsigned* tmem_slot_gen = reinterpret_cast<volatile unsigned*>(gen_base + kOff + BN * 4 + 8 * (2 * C::STAGES + 4));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const unsigned cta = cluster_ctarank();            // 0 = leader
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
  const int tiles_per_batch = p.m_tiles * p.n_tiles;
  // work units: (batch, 256-row tile, column tile, contraction range); splits > 1 only without batching.  Tiles from
  // p.tail_begin on (only without batching and split-K) are two units each, one per half of the tile's columns: the
  // last round of tiles, which fills only part of the SM pairs, then takes half as long.
  const int tail_tiles = tiles_per_batch - p.tail_begin;
  const int total_tiles = tiles_per_batch * p.splits * p.batch + tail_tiles;
  // unit -> (tile of its batch entry, first column inside the tile, columns): full tiles first, then the half-width units
  auto unit_tile = [&](int bt_tile, int& col_off, int& width) {
    if (bt_tile < p.tail_begin || tail_tiles == 0) { col_off = 0; width = BN; return bt_tile; }
    const int u = bt_tile - p.tail_begin;
    col_off = (u & 1) * (BN / 2); width = BN / 2;
    return p.tail_begin + (u >> 1);
  };

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(tfull_bar(a), 1); mbar_init(tempty_bar(a), 2 * kEpilogueThreads); }
    fence_barrier_init();
    prefetch_tensormap(&tmA);
    prefetch_tensormap(&tmB);
  }
  if (warp == 1) {
    tmem_alloc2(tmem_slot, C::TMEM_COLS);
    tmem_relinquish2();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                                // both CTAs' barriers and TMEM are ready
  tc_fence_after();
  const unsigned tmem_base = *tmem_slot_gen;

  if (warp == 0) {
    // ---------------- TMA producer (one per CTA) ----------------
    if (lane == 0) {
      struct UnitPos { int m0, n0, bi, boA, boB, width, kb_begin, kb_end; bool valid; };
      auto decode = [&](int unit) {
        UnitPos u;
        u.valid = unit < total_tiles;
        if (!u.valid) return u;
        const int bt = unit / p.splits, sp = unit - bt * p.splits;
        const int per_b = tiles_per_batch + tail_tiles;
        const int b = bt / per_b;
        int col_off;
        const int tile = unit_tile(bt - b * per_b, col_off, u.width);
        const int bo = b / p.batch_in;
        u.bi = b - bo * p.batch_in;
        u.boA = p.a_shared_out ? 0 : bo; u.boB = p.b_shared_out ? 0 : bo;
        u.m0 = (tile % p.m_tiles) * (2 * BM) + (int)cta * BM;
        u.n0 = (tile / p.m_tiles) * BN + col_off + (int)cta * (u.width / 2);
        u.kb_begin = sp * p.kb_per_split; u.kb_end = min(u.kb_begin + p.kb_per_split, p.k_blocks);
        return u;
      };
      int stage = 0;
      unsigned phase = 0;
      bool ok = true;
      UnitPos cur = decode(pair);
      for (int unit = pair; cur.valid && ok; unit += n_pairs) {
        const UnitPos nxt = decode(unit + n_pairs);
        const unsigned tx_bytes = 2 * (C::A_BYTES + (cur.width == BN ? C::B_BYTES : C::B_BYTES / 2));
        for (int kb = cur.kb_begin; kb < cur.kb_end; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u)) { ok = false; break; }
          const unsigned sa = base + stage * C::STAGE_BYTES, sb = sa + C::A_BYTES;
          const unsigned leader_full = map_to_cta(full_bar(stage), 0);
          if (cta == 0) mbar_expect_tx(full_bar(stage), tx_bytes);   // bytes of both CTAs
          const int k0 = kb * BK;
          if (!A_MN) {
            tma_load_4d_pair(sa, &tmA, k0, cur.m0, cur.bi, cur.boA, leader_full);
          } else if (p.a_chunked) {
            tma_load_5d_pair(sa, &tmA, k0, cur.m0 >> 6, cur.bi, cur.boA, leader_full);                         // both 64-row chunks at once
          } else {
#pragma unroll
            for (int i = 0; i < BM / 64; ++i) tma_load_4d_pair(sa + i * 8192u, &tmA, cur.m0 + 64 * i, k0, cur.bi, cur.boA, leader_full);
          }
          if (!B_MN) {
            tma_load_4d_pair(sb, cur.width == BN ? &tmB : &tmBh, k0, cur.n0, cur.bi, cur.boB, leader_full);   // BN/2 (or BN/4) rows of B per CTA
          } else if (p.b_chunked && cur.width == BN) {
            tma_load_5d_pair(sb, &tmB, k0, cur.n0 >> 6, cur.bi, cur.boB, leader_full);                         // both 64-column chunks at once
          } else {
            const CUtensorMap* m4 = p.b_chunked ? &tmBh : &tmB;
            for (int i = 0; i < cur.width / 128; ++i) tma_load_4d_pair(sb + i * 8192u, m4, cur.n0 + 64 * i, k0, cur.bi, cur.boB, leader_full);   // width/2 columns per CTA
          }
          if (++stage == C::STAGES) { stage = 0; phase ^= 1u; }
        }
        cur = nxt;
      }
      if (!ok) atomicCAS(p.error, 0u, 1u);
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (leader CTA only) ----------------
    if (lane == 0 && cta == 0) {
      int stage = 0, acc = 0;
      unsigned phase = 0, acc_phase = 0;
      bool ok = true;
      for (int unit = pair; unit < total_tiles && ok; unit += n_pairs) {
        const int sp = unit % p.splits;
        const int kb_begin = sp * p.kb_per_split, kb_end = min(kb_begin + p.kb_per_split, p.k_blocks);
        int col_off, width;
        {
          const int bt = unit / p.splits, per_b = tiles_per_batch + tail_tiles;
          unit_tile(bt - (bt / per_b) * per_b, col_off, width);
        }
        // the instruction descriptor's N field follows the unit's width
        const unsigned idesc = (C::IDESC & ~(0x3fu << 17)) | ((unsigned)(width >> 3) << 17);
        if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1u)) { ok = false; break; }
        tc_fence_after();
        const unsigned d_tmem = tmem_base + (unsigned)(acc * BN);
        for (int kb = kb_begin; kb < kb_end; ++kb) {
          if (!mbar_wait(full_bar(stage), phase)) { ok = false; break; }
          tc_fence_after();
          const unsigned sa = base + stage * C::STAGE_BYTES, sb = sa + C::A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const unsigned long long da = A_MN ? make_desc(sa + k * 2048u, 8192u, 1024u) : make_desc(sa + k * 32u, 16u, 1024u);
            const unsigned long long db = B_MN ? make_desc(sb + k * 2048u, 8192u, 1024u) : make_desc(sb + k * 32u, 16u, 1024u);
            umma2_bf16(d_tmem, da, db, idesc, (kb != kb_begin || k != 0) ? 1u : 0u);
          }
          umma2_commit_both(empty_bar(stage));
          if (++stage == C::STAGES) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        umma2_commit_both(tfull_bar(acc));
        if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
      }
      if (!ok) atomicCAS(p.error, 0u, 2u);
    }
  } else {
    // ---------------- epilogue: this CTA's 128 rows of the pair tile ----------------
    const int q = warp & 3;
    const int et = threadIdx.x - 64;
    int acc = 0;
    unsigned acc_phase = 0;
    bool ok = true;
    int store_buf = 0;
    for (int unit = pair; unit < total_tiles && ok; unit += n_pairs) {
      const int bt = unit / p.splits, sp = unit - bt * p.splits;
      const int per_b = tiles_per_batch + tail_tiles;
      const int b = bt / per_b;
      int col_off, width;
      const int tile = unit_tile(bt - b * per_b, col_off, width);
      const int bo = b / p.batch_in, bi = b - bo * p.batch_in;
      // with split-K the partial tile goes to the workspace, whose rows are [split][m_pad]
      const int m0 = (tile % p.m_tiles) * (2 * BM) + (int)cta * BM + sp * p.m_pad, n0 = (tile / p.m_tiles) * BN + col_off;
      if (!p.fast_drain) {
        asm volatile("bar.sync 1, 128;" ::: "memory");
        for (int j = et; j < BN; j += kEpilogueThreads) {
          float b = 0.f;
          if (p.bias != nullptr && n0 + j < p.N) b = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.bias)[n0 + j]);
          bias_tile[j] = b;
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
      }
      ok = epilogue_all(mbar_wait(tfull_bar(acc), acc_phase));
      if (!ok) break;
      tc_fence_after();
      const unsigned t_row = tmem_base + ((unsigned)(q * 32) << 16) + (unsigned)(acc * BN);
      if (p.fast_drain) drain_fast_any<BN>(p, &tmD, store_gen, store_u32, t_row, m0, n0, bi, bo, q, lane, store_buf, width);
      else drain_tile<BN>(p, &tmD, p.tma_store != 0, store_gen, store_u32, bias_tile, t_row, m0, n0, bi, bo, q, lane, et, store_buf);
      tc_fence_before();
      mbar_arrive_cluster(map_to_cta(tempty_bar(acc), 0));   // tell the leader this thread has drained its rows
      if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
    }
    if (lane == 0) bulk_wait_all();   // this warp's bulk stores still read its staging tiles
    if (!ok) atomicCAS(p.error, 0u, 3u);
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all();      // neither CTA may leave (or free TMEM) while the other can still signal it
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc2(tmem_base, C::TMEM_COLS);
  }
}

// ---- host side ------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
  });
  return fn;
}

// 4-D tensor map (contiguous index, row, batch_in, batch_out) with 128-byte swizzle.
static int encode_map(CUtensorMap* map, const void* ptr, CUtensorMapDataType type, int es, long long inner, long long rows,
                      long long ld, int batch_in, long long s_in, int batch_out, long long s_out, int box_inner, int box_rows,
                      CUtensorMapL2promotion promo) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fail(HAPX_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  // a batch dimension of extent 1 still needs a legal stride
  const long long bs_in = (batch_in > 1 ? s_in : ld) * es, bs_out = (batch_out > 1 ? s_out : ld) * es;
  cuuint64_t dims[4] = {(cuuint64_t)inner, (cuuint64_t)rows, (cuuint64_t)batch_in, (cuuint64_t)batch_out};
  cuuint64_t strides[3] = {(cuuint64_t)(ld * es), (cuuint64_t)bs_in, (cuuint64_t)bs_out};
  cuuint32_t box[4] = {(cuuint32_t)box_inner, (cuuint32_t)box_rows, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(map, type, 4, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, promo, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(HAPX_ERR_CUDA, "cuTensorMapEncodeTiled failed with code " + std::to_string((int)r));
  return HAPX_OK;
}

// 5-D map of an MN-major bf16 operand whose M / N extent is a multiple of 64: (64 contiguous elements, contraction row,
// chunk of 64, batch_in, batch_out), boxes of 64 x 64 x 2 - in shared memory the two chunks lie 8 KiB apart, exactly as two
// separate 64 x 64 loads leave them.
static int encode_chunked_map(CUtensorMap* map, const void* ptr, long long mn_extent, long long kc, long long ld, int batch_in, long long s_in,
                              int batch_out, long long s_out) {
  typedef CUresult (*Fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                         const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  Fn fn = reinterpret_cast<Fn>(encode_fn());
  if (!fn) return fail(HAPX_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  const long long bs_in = (batch_in > 1 ? s_in : ld) * 2, bs_out = (batch_out > 1 ? s_out : ld) * 2;
  cuuint64_t dims[5] = {64, (cuuint64_t)kc, (cuuint64_t)(mn_extent / 64), (cuuint64_t)batch_in, (cuuint64_t)batch_out};
  cuuint64_t strides[4] = {(cuuint64_t)(ld * 2), 128, (cuuint64_t)bs_in, (cuuint64_t)bs_out};
  cuuint32_t box[5] = {64, 64, 2, 1, 1};
  cuuint32_t estr[5] = {1, 1, 1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 5, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(HAPX_ERR_CUDA, "cuTensorMapEncodeTiled (5-D) failed with code " + std::to_string((int)r));
  return HAPX_OK;
}

static bool strides_ok(const void* ptr, int es, long long ld, int batch_in, long long s_in, int batch_out, long long s_out) {
  if ((reinterpret_cast<uintptr_t>(ptr) & 15u) != 0 || (ld * es) % 16 != 0) return false;
  if (batch_in > 1 && (s_in * es) % 16 != 0) return false;
  if (batch_out > 1 && (s_out * es) % 16 != 0) return false;
  return true;
}

// Tensor map of the output for bulk stores: boxes of 32 rows x 128 bytes.  Returns with *ok = 0
// (and a zeroed map) when D's base, row pitch or batch strides are not multiples of 16 bytes; the
// kernel then stores directly.
static int make_out_map(CUtensorMap* map, int* ok, void* ptr, long long cols, long long rows, long long ld, int out_f32,
                        int batch_in, long long s_in, int batch_out, long long s_out) {
  std::memset(map, 0, sizeof(*map));
  *ok = 0;
  const int es = out_f32 ? 4 : 2;
  if (!strides_ok(ptr, es, ld, batch_in, s_in, batch_out, s_out)) return HAPX_OK;
  if (int e = encode_map(map, ptr, out_f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, es, cols, rows, ld,
                         batch_in, s_in, batch_out, s_out, 128 / es, 32, CU_TENSOR_MAP_L2_PROMOTION_NONE)) return e;
  *ok = 1;
  return HAPX_OK;
}

// bf16 operand map.  K-major operand [rows][contraction contiguous]: box {64, tile rows};
// MN-major operand [contraction rows][M or N contiguous]: box {64, 64}.
int make_map(CUtensorMap* map, const Operand& op, long long mn_extent, long long kc, int tile_rows, int batch_in, int batch_out) {
  if (!strides_ok(op.ptr, 2, op.ld, batch_in, op.s_in, batch_out, op.s_out))
    return fail(HAPX_ERR_EXTENT, "gemm: operand base, row pitch and batch strides must be multiples of 16 bytes (8 bf16 elements)");
  if (op.mn_major)
    return encode_map(map, op.ptr, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, mn_extent, kc, op.ld, batch_in, op.s_in, batch_out, op.s_out, 64, 64,
                      CU_TENSOR_MAP_L2_PROMOTION_L2_256B);
  return encode_map(map, op.ptr, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, kc, mn_extent, op.ld, batch_in, op.s_in, batch_out, op.s_out, BK, tile_rows,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B);
}

struct DeviceState {
  bool ready = false;
  int index = 0;
  int sm_count = 0;
  unsigned* error = nullptr;  // device words: [0] the kernels' error reports, [1] scratch flag for callers
};
static DeviceState g_dev[64];
static std::mutex g_dev_mutex;

static int device_state(DeviceState** out) {
  int device = 0;
  HAPX_CUDA(cudaGetDevice(&device));
  if (device < 0 || device >= 64) return fail(HAPX_ERR_ARGUMENT, "gemm: device index out of range");
  // cuTensorMapEncodeTiled is a driver call: make sure the primary context is current on this
  // thread (autograd's backward threads have selected the device but may not have bound it yet)
  HAPX_CUDA(cudaSetDevice(device));
  std::lock_guard<std::mutex> lock(g_dev_mutex);
  DeviceState& d = g_dev[device];
  if (!d.ready) {
    HAPX_CUDA(cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, device));
    HAPX_CUDA(cudaMalloc(&d.error, 64));
    HAPX_CUDA(cudaMemset(d.error, 0, 64));
    d.index = device;
    d.ready = true;
  }
  *out = &d;
  return HAPX_OK;
}

// The barrier-free epilogue applies when D goes out through bulk tensor stores, there is no
// activation, and a bias can be fetched in aligned groups of 8.
static bool fast_drain_ok(const Params& p) {
  if (!p.tma_store || p.epilogue != EPI_NONE) return false;
  if (p.bias && ((reinterpret_cast<uintptr_t>(p.bias) & 15u) != 0 || (p.N & 7) != 0)) return false;
  return true;
}

template <int BN, bool A_MN, bool B_MN>
static int launch(const Operand& A, const Operand& B, const Operand& Dop, Params& p, cudaStream_t stream, const DeviceState& dev) {
  using C = Cfg<BN, A_MN, B_MN>;
  const int sm_count = dev.sm_count;
  const int batch_out = p.batch / p.batch_in;
  CUtensorMap tmA, tmB, tmD;
  if (int e = make_out_map(&tmD, &p.tma_store, p.D, p.N, p.M, p.ldd, p.out_f32, p.batch_in, Dop.s_in, batch_out, Dop.s_out)) return e;
  p.fast_drain = fast_drain_ok(p);
  if (int e = make_map(&tmA, A, p.M, p.Kc, BM, p.batch_in, p.a_shared_out ? 1 : batch_out)) return e;
  if (int e = make_map(&tmB, B, p.N, p.Kc, BN, p.batch_in, p.b_shared_out ? 1 : batch_out)) return e;
  p.m_tiles = (p.M + BM - 1) / BM;
  p.splits = 1; p.kb_per_split = 0; p.m_pad = 0;
  p.n_tiles = (p.N + BN - 1) / BN;
  p.k_blocks = (p.Kc + BK - 1) / BK;
  auto kernel = gemm_bf16_kernel<BN, A_MN, B_MN>;
  {  // function attributes are per device
    static bool attr_set[64] = {};
    std::lock_guard<std::mutex> lock(g_dev_mutex);
    if (!attr_set[dev.index]) {
      HAPX_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)C::SMEM_BYTES));
      attr_set[dev.index] = true;
    }
  }
  const long long units = (long long)p.m_tiles * p.n_tiles * p.batch;
  if (units > 0x7fffffff) return fail(HAPX_ERR_EXTENT, "gemm: too many tiles");
  const int grid = (int)std::max<long long>(1, std::min<long long>(units, sm_count));
  kernel<<<grid, kThreads, C::SMEM_BYTES, stream>>>(tmA, tmB, tmD, p);
  HAPX_CUDA(cudaGetLastError());
  count_launch();
  return HAPX_OK;
}


// Sum the fp32 partial tiles of a split-K GEMM in split order (deterministic), then bias,
// activation and cast.  ws rows: [split][m_pad], N columns.
__global__ void __launch_bounds__(256) splitk_reduce_kernel(const float* __restrict__ ws, int splits, int M, int N, long long m_pad,
                                                            const void* bias, int epilogue, void* out, int out_f32, long long ldd) {
  // N is a multiple of 4 (checked by the launcher): one thread sums 4 adjacent columns of one row
  const int n4 = N >> 2;
  const long long total = (long long)M * n4;
  for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (long long)gridDim.x * blockDim.x) {
    const int r = (int)(e / n4), c = (int)(e - (long long)r * n4) << 2;
    float4 acc = *reinterpret_cast<const float4*>(ws + (long long)r * N + c);
    for (int s = 1; s < splits; ++s) {
      const float4 v = *reinterpret_cast<const float4*>(ws + ((long long)s * m_pad + r) * N + c);
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    float o[4] = {acc.x, acc.y, acc.z, acc.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (bias) o[j] += __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(bias)[c + j]);
      o[j] = apply_epilogue(o[j], epilogue);
      if (out_f32) reinterpret_cast<float*>(out)[(long long)r * ldd + c + j] = o[j];
      else reinterpret_cast<__nv_bfloat16*>(out)[(long long)r * ldd + c + j] = __float2bfloat16_rn(o[j]);
    }
  }
}

// Scratch for split-K partial tiles and bias-gradient partial sums: one block per device.  The
// block only ever grows, and a block it outgrew is kept until the process exits, because a CUDA
// graph recorded earlier may still write to it on every replay.  Growing allocates and therefore
// cannot happen while the stream is being captured: run the step eagerly first (the step driver's
// capture() does).  The block is shared by all streams of the device: GEMMs that use it (split-K,
// bias gradients) must be ordered against each other, as they are on one stream.
struct Workspace { float* ptr = nullptr; size_t bytes = 0; std::vector<void*> outgrown; };
static Workspace g_ws[64];

static int workspace(int device, cudaStream_t stream, size_t bytes, float** out) {
  std::lock_guard<std::mutex> lock(g_dev_mutex);
  Workspace& w = g_ws[device];
  if (w.bytes < bytes) {
    cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
    HAPX_CUDA(cudaStreamIsCapturing(stream, &capturing));
    if (capturing != cudaStreamCaptureStatusNone)
      return fail(HAPX_ERR_STATE, "gemm: the scratch block of this stream must grow to " + std::to_string(bytes) +
                                      " bytes, which cannot happen during stream capture; run the same step once outside the capture first");
    const size_t want = std::max(bytes, w.bytes + w.bytes / 2);
    void* p = nullptr;
    HAPX_CUDA(cudaMalloc(&p, want));
    if (w.ptr) w.outgrown.push_back(w.ptr);
    w.ptr = static_cast<float*>(p);
    w.bytes = want;
  }
  *out = w.ptr;
  return HAPX_OK;
}

template <int BN, bool A_MN, bool B_MN>
static int launch2(const Operand& A, const Operand& B, const Operand& Dop, Params& p, cudaStream_t stream, const DeviceState& dev) {
  using C = Cfg2<BN, A_MN, B_MN>;
  auto kernel = gemm2_bf16_kernel<BN, A_MN, B_MN>;
  const int sm_count = dev.sm_count;
  static int max_clusters_of[64] = {};      // per device: function attributes and occupancy belong to one
  int max_clusters = 0;
  {
    std::lock_guard<std::mutex> lock(g_dev_mutex);
    max_clusters = max_clusters_of[dev.index];
  }
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = C::SMEM_BYTES;
  cfg.stream = stream;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (max_clusters == 0) {
    HAPX_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)C::SMEM_BYTES));
    cfg.gridDim = dim3(sm_count / 2 * 2);
    int n = 0;
    HAPX_CUDA(cudaOccupancyMaxActiveClusters(&n, kernel, &cfg));
    if (n < 1) return fail(HAPX_ERR_CUDA, "gemm: no SM pair can host the two-CTA kernel");
    max_clusters = n;
    std::lock_guard<std::mutex> lock(g_dev_mutex);
    max_clusters_of[dev.index] = n;
  }
  p.m_tiles = (p.M + 2 * BM - 1) / (2 * BM);
  p.n_tiles = (p.N + C::BN - 1) / C::BN;
  p.k_blocks = (p.Kc + BK - 1) / BK;
  p.splits = 1; p.kb_per_split = p.k_blocks; p.m_pad = 0;
  // A long contraction over few output tiles (weight gradients, the input gradient of the vocabulary
  // projection) leaves SM pairs idle or the last wave nearly empty: cut the contraction into `splits`
  // ranges whose fp32 partial tiles a second kernel adds in a fixed order.  The split count minimises
  // a small cost model, in microseconds: waves x slices per unit x 0.28 (one 256 x 256 x 64 slice on
  // an SM pair) + 3 for the ramp, and for a split the partial tiles written and read back at about
  // 4 TB/s plus the second launch.
  const int tiles = p.m_tiles * p.n_tiles;
  if (p.batch == 1 && p.k_blocks >= 16 && (p.N & 3) == 0) {
    auto waves = [&](long long units) { return (double)((units + max_clusters - 1) / max_clusters); };
    const double out_bytes = (double)p.M * p.N * (p.out_f32 ? 4.0 : 2.0), partial_bytes = (double)p.M * p.N * 4.0;
    int best = 1;
    double best_cost = waves(tiles) * p.k_blocks * 0.28 + 3.0;
    for (int sp = 2; sp <= 16 && sp * 8 <= p.k_blocks; ++sp) {
      const int per = (p.k_blocks + sp - 1) / sp;
      if ((sp - 1) * per >= p.k_blocks) continue;            // an empty last range
      if ((double)sp * partial_bytes > 512e6) break;         // keep the workspace bounded
      const double cost = waves((long long)tiles * sp) * per * 0.28 + 3.0 + 3.0 + (2.0 * sp * partial_bytes + out_bytes) / 4e6;
      if (cost < 0.9 * best_cost) { best = sp; best_cost = cost; }
    }
    if (best > 1) { p.splits = best; p.kb_per_split = (p.k_blocks + best - 1) / best; p.m_pad = p.m_tiles * 2 * BM; }
  }
  Params user = p;   // what the caller asked for (output, bias, activation)
  float* ws = nullptr;
  if (p.splits > 1) {
    if (int e = workspace(dev.index, stream, (size_t)p.splits * p.m_pad * p.N * sizeof(float), &ws)) return e;
    p.D = ws; p.ldd = p.N; p.out_f32 = 1; p.bias = nullptr; p.epilogue = EPI_NONE;
  }
  CUtensorMap tmA, tmB, tmBh, tmD;
  const int batch_out = p.batch / p.batch_in;
  const long long out_rows = p.splits > 1 ? (long long)p.splits * p.m_pad : p.M;
  if (int e = make_out_map(&tmD, &p.tma_store, p.D, p.N, out_rows, p.ldd, p.out_f32, p.batch_in, Dop.s_in, batch_out, Dop.s_out)) return e;
  p.fast_drain = fast_drain_ok(p);
  if (p.splits > 1 && !p.tma_store) return fail(HAPX_ERR_EXTENT, "gemm: split-K needs an output width that is a multiple of 4");
  if (int e = make_map(&tmA, A, p.M, p.Kc, BM, p.batch_in, p.a_shared_out ? 1 : batch_out)) return e;
  if (int e = make_map(&tmB, B, p.N, p.Kc, C::BN / 2, p.batch_in, p.b_shared_out ? 1 : batch_out)) return e;
  if (int e = make_map(&tmBh, B, p.N, p.Kc, C::BN / 4, p.batch_in, p.b_shared_out ? 1 : batch_out)) return e;   // MN-major: the same 64 x 64 boxes
  // MN-major operands whose extent is a whole number of 64-element chunks: one load per stage instead of two
  p.a_chunked = (A_MN && p.M % 64 == 0) ? 1 : 0;
  p.b_chunked = (B_MN && p.N % 64 == 0) ? 1 : 0;
  if (p.a_chunked)
    if (int e = encode_chunked_map(&tmA, A.ptr, p.M, p.Kc, A.ld, p.batch_in, A.s_in, p.a_shared_out ? 1 : batch_out, A.s_out)) return e;
  if (p.b_chunked)
    if (int e = encode_chunked_map(&tmB, B.ptr, p.N, p.Kc, B.ld, p.batch_in, B.s_in, p.b_shared_out ? 1 : batch_out, B.s_out)) return e;
  // A last round that fills at most half of the SM pairs is run as half-width units (no partial sums, no second
  // launch): 96 tiles on 74 pairs take 1.5 tile times instead of 2.
  p.tail_begin = tiles;
  if (p.splits == 1 && p.batch == 1 && p.fast_drain && tiles > max_clusters) {
    const int rest = tiles % max_clusters;
    if (rest > 0 && 2 * rest <= max_clusters) p.tail_begin = tiles - rest;
  }
  const long long units = (long long)tiles * p.splits * p.batch + (tiles - p.tail_begin);
  if (units > 0x7fffffff) return fail(HAPX_ERR_EXTENT, "gemm: too many tiles");
  const int pairs = (int)std::max<long long>(1, std::min<long long>(units, max_clusters));
  cfg.gridDim = dim3(2 * pairs);
  HAPX_CUDA(cudaLaunchKernelEx(&cfg, kernel, tmA, tmB, tmBh, tmD, p));
  count_launch();
  if (p.splits > 1) {
    const long long total = (long long)user.M * (user.N / 4);
    const int grid = (int)std::min<long long>((total + 255) / 256, (long long)sm_count * 8);
    splitk_reduce_kernel<<<grid, 256, 0, stream>>>(ws, p.splits, user.M, user.N, p.m_pad, user.bias, user.epilogue, user.D,
                                                   user.out_f32, user.ldd);
    HAPX_CUDA(cudaGetLastError());
    count_launch();
  }
  return HAPX_OK;
}

// The device word the tensor-core kernels report a timed-out wait into (read by hapx_gemm_status).
int error_word(unsigned** out, int* sm_count) {
  DeviceState* dev = nullptr;
  if (int e = device_state(&dev)) return e;
  *out = dev->error;
  if (sm_count) *sm_count = dev->sm_count;
  return HAPX_OK;
}

// D[b] = A[b] * B[b]^T for b in [0, batch): M x N outputs, contraction length Kc.
int gemm_bf16(const Operand& Dop, int out_f32, const Operand& A, const Operand& B, const void* bias, int epilogue,
              long long M, long long N, long long Kc, int batch_in, int batch_out, cudaStream_t stream) {
  if (M < 0 || N < 0 || Kc < 0 || batch_in < 1 || batch_out < 1) return fail(HAPX_ERR_EXTENT, "gemm: bad extent");
  if (M == 0 || N == 0) return HAPX_OK;
  if (Kc == 0) {  // an empty contraction (e.g. the weight gradient of a rank that holds no samples): D = 0
    if (batch_in * batch_out != 1 || Dop.ld != N || bias != nullptr) return fail(HAPX_ERR_EXTENT, "gemm: empty contraction");
    HAPX_CUDA(cudaMemsetAsync(const_cast<void*>(Dop.ptr), 0, (size_t)M * N * (out_f32 ? 4 : 2), stream));
    return HAPX_OK;
  }
  if (M > 0x7fffffff || N > 0x7fffffff || Kc > 0x7fffffff) return fail(HAPX_ERR_EXTENT, "gemm: extent exceeds 2^31");
  if (!Dop.ptr || !A.ptr || !B.ptr) return fail(HAPX_ERR_ARGUMENT, "gemm: null pointer");
  DeviceState* dev = nullptr;
  if (int e = device_state(&dev)) return e;
  Params p = Params();
  p.M = (int)M; p.N = (int)N; p.Kc = (int)Kc; p.ldd = Dop.ld; p.D = const_cast<void*>(Dop.ptr); p.bias = bias; p.epilogue = epilogue;
  p.out_f32 = out_f32;
  p.error = dev->error;
  p.batch = batch_in * batch_out; p.batch_in = batch_in; p.d_stride_in = Dop.s_in; p.d_stride_out = Dop.s_out;
  p.a_shared_out = (batch_out > 1 && A.s_out == 0) ? 1 : 0;
  p.b_shared_out = (batch_out > 1 && B.s_out == 0) ? 1 : 0;
  const bool a_mn = A.mn_major, b_mn = B.mn_major;
  // SM pairs (256 x 256 tiles, half the B traffic per SM) whenever there is more than one row tile
  if (M > BM && N > 64) {
    // (256 x 128 pair tiles were measured too: slower than 256 x 256 even where they fill the waves better)
    if (!a_mn && !b_mn) return launch2<256, false, false>(A, B, Dop, p, stream, *dev);
    if (!a_mn && b_mn) return launch2<256, false, true>(A, B, Dop, p, stream, *dev);
    if (a_mn && b_mn) return launch2<256, true, true>(A, B, Dop, p, stream, *dev);
  }
  // single-CTA tiles: fewest waves first, then the wider tile
  auto waves = [&](int bn) {
    const long long tiles = ((M + BM - 1) / BM) * ((N + bn - 1) / bn) * p.batch;
    return (double)((tiles + dev->sm_count - 1) / dev->sm_count) * bn;
  };
  const int bn = (waves(256) <= waves(128)) ? 256 : 128;
#define HAPX_GEMM_CASE(BN_, AMN_, BMN_) \
  if (bn == BN_ && a_mn == AMN_ && b_mn == BMN_) return launch<BN_, AMN_, BMN_>(A, B, Dop, p, stream, *dev);
  HAPX_GEMM_CASE(256, false, false)
  HAPX_GEMM_CASE(128, false, false)
  HAPX_GEMM_CASE(256, false, true)
  HAPX_GEMM_CASE(128, false, true)
  HAPX_GEMM_CASE(256, true, true)
  HAPX_GEMM_CASE(128, true, true)
#undef HAPX_GEMM_CASE
  return fail(HAPX_ERR_ARGUMENT, "gemm: unsupported operand layout");
}

// Column sums of g[M,N] (the bias gradient), fp32 accumulation, in two deterministic passes:
// blocks of 64 columns x one slice of the rows write partial sums, a second kernel adds the
// slices in order and casts.
__global__ void __launch_bounds__(256) colsum_partial_kernel(const __nv_bfloat16* __restrict__ g, long long ldg, int M, int N,
                                                             int rows_per_slice, float* __restrict__ partial) {
  __shared__ float part[4][64];
  const int c = blockIdx.x * 64 + (threadIdx.x & 63);
  const int rg = threadIdx.x >> 6;
  const int r0 = blockIdx.y * rows_per_slice, r1 = min(M, r0 + rows_per_slice);
  float acc = 0.f;
  if (c < N)
    for (int r = r0 + rg; r < r1; r += 4) acc += __bfloat162float(g[(long long)r * ldg + c]);
  part[rg][threadIdx.x & 63] = acc;
  __syncthreads();
  if (rg == 0 && c < N)
    partial[(long long)blockIdx.y * N + c] = (part[0][threadIdx.x] + part[1][threadIdx.x]) + (part[2][threadIdx.x] + part[3][threadIdx.x]);
}
// Vector variant for 16-byte aligned rows (pitch and width multiples of 8): a block covers 256 columns
// (32 threads x 8 columns, one 16-byte load each) x 8 row groups of a 64-row slice, so every thread
// has 8 independent loads in flight.
constexpr int kColsumSliceRows = 64;
__global__ void __launch_bounds__(256) colsum_partial_vec_kernel(const __nv_bfloat16* __restrict__ g, long long ldg, int M, int N,
                                                                 float* __restrict__ partial) {
  __shared__ float part[8][256];
  const int ct = threadIdx.x & 31, rg = threadIdx.x >> 5;
  const int c = blockIdx.x * 256 + ct * 8;
  const int r0 = blockIdx.y * kColsumSliceRows;
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  if (c < N) {
    uint4 v[kColsumSliceRows / 8];
#pragma unroll
    for (int i = 0; i < kColsumSliceRows / 8; ++i) {
      const int r = r0 + rg + 8 * i;
      v[i] = (r < M) ? *reinterpret_cast<const uint4*>(g + (long long)r * ldg + c) : make_uint4(0u, 0u, 0u, 0u);
    }
#pragma unroll
    for (int i = 0; i < kColsumSliceRows / 8; ++i) {
      const unsigned w[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        acc[2 * k] += __uint_as_float(w[k] << 16);
        acc[2 * k + 1] += __uint_as_float(w[k] & 0xffff0000u);
      }
    }
  }
#pragma unroll
  for (int k = 0; k < 8; ++k) part[rg][ct * 8 + k] = acc[k];
  __syncthreads();
  const int col = blockIdx.x * 256 + threadIdx.x;
  if (col < N) {
    float s = part[0][threadIdx.x];
#pragma unroll
    for (int q = 1; q < 8; ++q) s += part[q][threadIdx.x];
    partial[(long long)blockIdx.y * N + col] = s;
  }
}
// Adds the slices of 32 columns per block: warp w takes slices w, w + 8, ...; the eight sums are added in warp order.
__global__ void __launch_bounds__(256) colsum_final_kernel(const float* __restrict__ partial, int slices, int N, void* out, int out_f32) {
  __shared__ float s_sum[8][32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + lane;
  float s = 0.f;
  if (c < N) {
#pragma unroll 4
    for (int i = warp; i < slices; i += 8) s += partial[(long long)i * N + c];
  }
  s_sum[warp][lane] = s;
  __syncthreads();
  if (warp != 0 || c >= N) return;
#pragma unroll
  for (int w = 1; w < 8; ++w) s += s_sum[w][lane];
  if (out_f32) reinterpret_cast<float*>(out)[c] = s;
  else reinterpret_cast<__nv_bfloat16*>(out)[c] = __float2bfloat16_rn(s);
}

int colsum_bf16(const void* g, long long m, long long n, void* out, int out_f32, cudaStream_t stream) {
  if (n <= 0) return HAPX_OK;
  if (m < 0 || m > 0x7fffffff || n > 0x7fffffff) return fail(HAPX_ERR_EXTENT, "linear_wgrad: extent out of range");
  int device = 0;
  HAPX_CUDA(cudaGetDevice(&device));
  const bool vec = (n % 8 == 0) && (reinterpret_cast<uintptr_t>(g) & 15u) == 0 && (m + kColsumSliceRows - 1) / kColsumSliceRows <= 65535;
  const int rows_per_slice = vec ? kColsumSliceRows : (int)std::max<long long>(128, (m + 65534) / 65535);
  const int slices = (int)std::max<long long>(1, (m + rows_per_slice - 1) / rows_per_slice);
  float* ws = nullptr;
  if (int e = workspace(device, stream, (size_t)slices * n * sizeof(float), &ws)) return e;
  if (vec) {
    dim3 grid((unsigned)((n + 255) / 256), (unsigned)slices);
    colsum_partial_vec_kernel<<<grid, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(g), n, (int)m, (int)n, ws);
  } else {
    dim3 grid((unsigned)((n + 63) / 64), (unsigned)slices);
    colsum_partial_kernel<<<grid, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(g), n, (int)m, (int)n, rows_per_slice, ws);
  }
  HAPX_CUDA(cudaGetLastError());
  colsum_final_kernel<<<(unsigned)((n + 31) / 32), 256, 0, stream>>>(ws, slices, (int)n, out, out_f32);
  HAPX_CUDA(cudaGetLastError());
  count_launch(2);
  return HAPX_OK;
}

}  // namespace gemm
}  // namespace hapx

namespace hapx { namespace sgemm {
int run(const float* A, long long a_i, long long a_k, const float* B, long long b_j, long long b_k, const float* bias, float* D,
        long long ldd, long long M, long long N, long long K, int epilogue, cudaStream_t stream);
int colsum(const float* g, long long m, long long n, float* out, cudaStream_t stream);
} }

using namespace hapx;

extern "C" {

int hapx_linear_forward(void* y, const void* x, const void* w, const void* bias, int dtype, int out_dtype, int64_t m,
                        int64_t n, int64_t k, int epilogue, hapx_stream stream) {
  if (epilogue < 0 || epilogue > 3) return fail(HAPX_ERR_ARGUMENT, "linear_forward: unknown epilogue");
  if (dtype == HAPX_F32) {  // fp32 operands: CUDA-core path (tcgen05 has no fp32 multiply)
    if (out_dtype != HAPX_F32) return fail(HAPX_ERR_DTYPE, "linear_forward: float32 operands give a float32 result");
    return sgemm::run(static_cast<const float*>(x), k, 1, static_cast<const float*>(w), k, 1, static_cast<const float*>(bias),
                      static_cast<float*>(y), n, m, n, k, epilogue, static_cast<cudaStream_t>(stream));
  }
  if (dtype != HAPX_BF16) return fail(HAPX_ERR_DTYPE, "linear_forward: operands must be bfloat16 or float32");
  if (out_dtype != HAPX_BF16 && out_dtype != HAPX_F32) return fail(HAPX_ERR_DTYPE, "linear_forward: output must be bfloat16 or float32");
  // y[m,n] = x[m,k] * w[n,k]^T : both operands K-major
  return gemm::gemm_bf16({y, false, n, 0, 0}, out_dtype == HAPX_F32, {x, false, k, 0, 0}, {w, false, k, 0, 0}, bias, epilogue, m, n, k, 1, 1,
                         static_cast<cudaStream_t>(stream));
}

int hapx_linear_dgrad(void* dx, const void* g, const void* w, int dtype, int out_dtype, int64_t m, int64_t n, int64_t k,
                      hapx_stream stream) {
  if (dtype == HAPX_F32) {  // dx[m,k] = sum_n g[m,n] w[n,k]
    if (out_dtype != HAPX_F32) return fail(HAPX_ERR_DTYPE, "linear_dgrad: float32 operands give a float32 result");
    return sgemm::run(static_cast<const float*>(g), n, 1, static_cast<const float*>(w), 1, k, nullptr, static_cast<float*>(dx), k,
                      m, k, n, 0, static_cast<cudaStream_t>(stream));
  }
  if (dtype != HAPX_BF16) return fail(HAPX_ERR_DTYPE, "linear_dgrad: operands must be bfloat16 or float32");
  if (out_dtype != HAPX_BF16 && out_dtype != HAPX_F32) return fail(HAPX_ERR_DTYPE, "linear_dgrad: output must be bfloat16 or float32");
  // dx[m,k] = g[m,n] * w[n,k] : contraction over n; A = g is K-major, B[k][n] = w[n][k] is MN-major as stored
  return gemm::gemm_bf16({dx, false, k, 0, 0}, out_dtype == HAPX_F32, {g, false, n, 0, 0}, {w, true, k, 0, 0}, nullptr, 0, m, k, n, 1, 1,
                         static_cast<cudaStream_t>(stream));
}

int hapx_linear_wgrad(void* dw, void* dbias, const void* g, const void* x, int dtype, int out_dtype, int64_t m, int64_t n,
                      int64_t k, hapx_stream stream_) {
  if (dtype == HAPX_F32) {  // dw[n,k] = sum_m g[m,n] x[m,k]
    if (out_dtype != HAPX_F32) return fail(HAPX_ERR_DTYPE, "linear_wgrad: float32 operands give a float32 result");
    cudaStream_t st = static_cast<cudaStream_t>(stream_);
    if (dw)
      if (int e = sgemm::run(static_cast<const float*>(g), 1, n, static_cast<const float*>(x), 1, k, nullptr, static_cast<float*>(dw), k,
                             n, k, m, 0, st)) return e;
    if (dbias) return sgemm::colsum(static_cast<const float*>(g), m, n, static_cast<float*>(dbias), st);
    return HAPX_OK;
  }
  if (dtype != HAPX_BF16) return fail(HAPX_ERR_DTYPE, "linear_wgrad: operands must be bfloat16 or float32");
  if (out_dtype != HAPX_BF16 && out_dtype != HAPX_F32) return fail(HAPX_ERR_DTYPE, "linear_wgrad: output must be bfloat16 or float32");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  // dw[n,k] = g[m,n]^T * x[m,k] : contraction over m; A[n][m] = g[m][n] and B[k][m] = x[m][k] are both MN-major as stored
  if (dw) {
    if (int e = gemm::gemm_bf16({dw, false, k, 0, 0}, out_dtype == HAPX_F32, {g, true, n, 0, 0}, {x, true, k, 0, 0}, nullptr, 0, n, k, m, 1, 1, stream))
      return e;
  }
  if (dbias && n > 0) return gemm::colsum_bf16(g, m, n, dbias, out_dtype == HAPX_F32, stream);
  return HAPX_OK;
}

int hapx_gemm_batched(void* d, const void* a, const void* b, int out_dtype, int a_mn_major, int b_mn_major, int64_t m, int64_t n,
                      int64_t kc, int64_t lda, int64_t ldb, int64_t ldd, int64_t batch_in, int64_t batch_out, int64_t a_stride_in,
                      int64_t a_stride_out, int64_t b_stride_in, int64_t b_stride_out, int64_t d_stride_in, int64_t d_stride_out,
                      hapx_stream stream) {
  if (out_dtype != HAPX_BF16 && out_dtype != HAPX_F32) return fail(HAPX_ERR_DTYPE, "gemm_batched: output must be bfloat16 or float32");
  if (batch_in < 1 || batch_out < 1 || batch_in * batch_out > 0x7fffffff) return fail(HAPX_ERR_EXTENT, "gemm_batched: bad batch counts");
  if (a_mn_major && !b_mn_major) return fail(HAPX_ERR_ARGUMENT, "gemm_batched: A MN-major with B K-major is not built (swap the operands and transpose the result)");
  return gemm::gemm_bf16({d, false, ldd, d_stride_in, d_stride_out}, out_dtype == HAPX_F32, {a, a_mn_major != 0, lda, a_stride_in, a_stride_out},
                         {b, b_mn_major != 0, ldb, b_stride_in, b_stride_out}, nullptr, 0, m, n, kc, (int)batch_in, (int)batch_out,
                         static_cast<cudaStream_t>(stream));
}

int hapx_gemm_status(void) {
  gemm::DeviceState* dev = nullptr;
  if (int e = gemm::device_state(&dev)) return e;
  HAPX_CUDA(cudaDeviceSynchronize());
  unsigned code = 0;
  HAPX_CUDA(cudaMemcpy(&code, dev->error, sizeof(code), cudaMemcpyDeviceToHost));
  if (code != 0) {
    HAPX_CUDA(cudaMemset(dev->error, 0, sizeof(unsigned)));
    return fail(HAPX_ERR_PEER_TIMEOUT, "a GEMM kernel gave up waiting on a barrier (role " + std::to_string(code) +
                                           ": 1 = TMA producer, 2 = MMA issuer, 3 = epilogue)");
  }
  return HAPX_OK;
}

}  // extern "C"
