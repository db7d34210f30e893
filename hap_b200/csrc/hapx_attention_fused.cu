// Fused multi-head self-attention on a batch shard (head dimension 64), forward and backward:
// scores and probabilities never leave the SM.
//
// Stands in for the attention core of F.multi_head_attention_forward as the planner emits it
// (hap.rs:1297-1329 with dropout_p forwarded at hap.rs:1257, 1307, 1319; only the batch dimension is
// sharded, hap.rs:2903-2926; causal -inf mask of models.py:72), on the packed in-projection output
// qkv[L, N, 3E] in the reference's (L, N, E) layout.
//
//   forward : one CTA per (batch entry, head, 128-query tile) walks the key tiles: S = Q K^T into
//             tensor memory (tcgen05.mma), online softmax in registers (one thread per query row),
//             dropout on the probabilities, P as bf16 into swizzled shared memory as the A operand of
//             O += P V; saves only the row log-sum-exp.
//   backward: two launches of one kernel template, both recompute S and dP = dO V^T per tile pair:
//             KEY-major   (one CTA per key tile, walks query tiles):  dV += Pd^T dO, dK += dS^T Q
//             QUERY-major (one CTA per query tile, walks key tiles):  dQ += dS K
//             with dS = P * (dPd * keep / (1-p) - delta) / sqrt(d), delta = rowsum(dO * O).  Nothing of
//             size L x L is ever written to HBM, and nothing is accumulated with atomics: every output
//             element is produced by one CTA in a fixed order (bit-reproducible).
//
// Roles per CTA (192 threads): warp 0 = TMA producer, warp 1 = MMA issuer (one thread), warps 2-5 =
// softmax / gradient math and epilogue (thread = row).  The dropout mask is a pure function of
// (seed, iteration, call id, row, column group) - see hapx_rng.h - so forward and both backward
// launches regenerate it.  All mbarrier waits are bounded; a wait that runs out raises the GEMM
// path's error word (hapx_gemm_status) and every role leaves its loops.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <mutex>
#include <string>

#include "hapx_internal.h"
#include "hapx_rng.h"
#include "hapx_tc.h"

namespace hapx {
namespace fattn {

using namespace tc;

constexpr int BT = 128;                     // rows of a query tile = rows of a key tile
constexpr int HD = 64;                      // head dimension (one 128-byte swizzle row of bf16)
constexpr int kThreads = 192;
constexpr unsigned kTileBytes = BT * HD * 2;        // 16 KiB: one Q / K / V / dO tile
constexpr unsigned kProbBytes = BT * BT * 2;        // 32 KiB: P or dS as bf16, two 64-column chunks of [128][64]
constexpr float kLog2e = 1.4426950408889634f;

// instruction descriptors: fp32 accumulate, bf16 x bf16, M = 128
__host__ __device__ constexpr unsigned idesc(int n, bool a_mn, bool b_mn) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((a_mn ? 1u : 0u) << 15) | ((b_mn ? 1u : 0u) << 16) | ((unsigned)(n >> 3) << 17) |
         ((unsigned)(BT >> 4) << 24);
}

struct Params {
  int L, N, H, E;                  // sequence length, batch entries of this shard, heads, H * 64
  int nt;                          // tiles along the sequence = ceil(L / 128)
  int causal;
  const float* mask;               // additive [L][L] fp32, or null
  const unsigned* mask_is_causal;  // optional device word: non-zero when `mask` is exactly the causal mask
  float scale, scale2;             // 1/sqrt(64) and the same times log2(e)
  unsigned drop_threshold;         // 0: no dropout
  float drop_scale;                // 1 / (1 - p)
  unsigned long long call_id;
  const rng::State* rng;
  __nv_bfloat16* out;              // forward: [L, N, E]
  float* lse2;                     // [N*H, L]: log2-domain log-sum-exp of every row (forward writes, backward reads)
  const float* delta;              // backward: [N*H, L] rowsum(dO * O)
  __nv_bfloat16* dqkv;             // backward: [L, N, 3E]
  unsigned* error;
  int units;                       // work units of the launch
};

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ unsigned pack_bf16(float a, float b) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<const unsigned*>(&h);
}
// Store 32 consecutive columns [32c, 32c+32) of row `row` into a [2 chunks][128 rows][64 columns] bf16 tile
// with the 128-byte swizzle the MMA descriptors and TMA use (16-byte piece j of a row sits at j ^ (row % 8)).
__device__ __forceinline__ void store_prob_columns(unsigned char* tile, int row, int c, const float (&v)[32]) {
  unsigned char* base = tile + (c >> 1) * (BT * 128) + row * 128;
  const int sw = row & 7;
#pragma unroll
  for (int g = 0; g < 4; ++g) {
    uint4 pk;
    pk.x = pack_bf16(v[8 * g], v[8 * g + 1]); pk.y = pack_bf16(v[8 * g + 2], v[8 * g + 3]);
    pk.z = pack_bf16(v[8 * g + 4], v[8 * g + 5]); pk.w = pack_bf16(v[8 * g + 6], v[8 * g + 7]);
    *reinterpret_cast<uint4*>(base + ((((c & 1) * 4 + g) ^ sw) << 4)) = pk;
  }
}
// Keep bits of the 32 columns [col0, col0+32) of probability row (bh, q): four generator groups of 8.
__device__ __forceinline__ unsigned keep32(const rng::Key& key, unsigned threshold, unsigned long long row_groups0, int col0) {
  unsigned bits = 0;
#pragma unroll
  for (int g = 0; g < 4; ++g)
    bits |= rng::keep_bits(rng::philox(key, row_groups0 + (unsigned)((col0 >> 3) + g)), threshold) << (8 * g);
  return bits;
}
// Write one row of 64 fp32 values as bf16 (128 contiguous bytes).
__device__ __forceinline__ void store_row64(__nv_bfloat16* dst, const float (&v)[64], float mul) {
#pragma unroll
  for (int g = 0; g < 8; ++g) {
    uint4 pk;
    pk.x = pack_bf16(v[8 * g] * mul, v[8 * g + 1] * mul); pk.y = pack_bf16(v[8 * g + 2] * mul, v[8 * g + 3] * mul);
    pk.z = pack_bf16(v[8 * g + 4] * mul, v[8 * g + 5] * mul); pk.w = pack_bf16(v[8 * g + 6] * mul, v[8 * g + 7] * mul);
    reinterpret_cast<uint4*>(dst)[g] = pk;
  }
}

// ---- per-chunk math (32 columns of one row, all in registers, no branches) ------------------------------
// PARTIAL: columns after `lim` (relative to the chunk) take no part (causal diagonal, ragged end, rows past L).
// mrow: optional additive mask row, already offset to the chunk's first column (general masks only).
template <bool PARTIAL>
__device__ __forceinline__ float chunk_score(unsigned raw, float scale2, int e, int lim, const float* mrow) {
  float x = __uint_as_float(raw) * scale2;
  if (mrow) x = fmaf(mrow[e], kLog2e, x);
  if (PARTIAL) x = (e <= lim) ? x : -INFINITY;
  return x;
}
template <bool PARTIAL>
__device__ __forceinline__ float chunk_max(const unsigned (&v)[32], float scale2, int lim, const float* mrow, float mx) {
  float m0 = mx, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;
#pragma unroll
  for (int e = 0; e < 32; e += 4) {
    m0 = fmaxf(m0, chunk_score<PARTIAL>(v[e], scale2, e, lim, mrow));
    m1 = fmaxf(m1, chunk_score<PARTIAL>(v[e + 1], scale2, e + 1, lim, mrow));
    m2 = fmaxf(m2, chunk_score<PARTIAL>(v[e + 2], scale2, e + 2, lim, mrow));
    m3 = fmaxf(m3, chunk_score<PARTIAL>(v[e + 3], scale2, e + 3, lim, mrow));
  }
  return fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
}
// exp2(score - shift) of the chunk; returns the sum of the (undropped) values.
template <bool PARTIAL>
__device__ __forceinline__ float chunk_exp(const unsigned (&v)[32], float scale2, float shift, int lim, const float* mrow, float (&pe)[32]) {
  float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
#pragma unroll
  for (int e = 0; e < 32; e += 4) {
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      float x;
      if (mrow) {
        x = chunk_score<PARTIAL>(v[e + u], scale2, e + u, lim, mrow) - shift;
      } else {
        x = fmaf(__uint_as_float(v[e + u]), scale2, -shift);
        if (PARTIAL) x = (e + u <= lim) ? x : -INFINITY;
      }
      pe[e + u] = ex2(x);
    }
    s0 += pe[e]; s1 += pe[e + 1]; s2 += pe[e + 2]; s3 += pe[e + 3];
  }
  return (s0 + s1) + (s2 + s3);
}

// The same for 16 columns (the backward pass, whose sixteen math warps each take 32 columns in two steps).
template <bool PARTIAL>
__device__ __forceinline__ void chunk_exp16(const unsigned (&v)[16], float scale2, float shift, int lim, const float* mrow, float (&pe)[16]) {
#pragma unroll
  for (int e = 0; e < 16; ++e) {
    float x;
    if (mrow) {
      x = chunk_score<PARTIAL>(v[e], scale2, e, lim, mrow) - shift;
    } else {
      x = fmaf(__uint_as_float(v[e]), scale2, -shift);
      if (PARTIAL) x = (e <= lim) ? x : -INFINITY;
    }
    pe[e] = ex2(x);
  }
}
// Store 16 consecutive columns [16c, 16c+16) of row `row` into the swizzled [2 chunks][128 rows][64 columns] tile.
__device__ __forceinline__ void store_prob_columns16(unsigned char* tile, int row, int c, const float (&v)[16]) {
  unsigned char* base = tile + (c >> 2) * (BT * 128) + row * 128;
  const int sw = row & 7;
#pragma unroll
  for (int g = 0; g < 2; ++g) {
    uint4 pk;
    pk.x = pack_bf16(v[8 * g], v[8 * g + 1]); pk.y = pack_bf16(v[8 * g + 2], v[8 * g + 3]);
    pk.z = pack_bf16(v[8 * g + 4], v[8 * g + 5]); pk.w = pack_bf16(v[8 * g + 6], v[8 * g + 7]);
    *reinterpret_cast<uint4*>(base + ((((c & 3) * 2 + g) ^ sw) << 4)) = pk;
  }
}
__device__ __forceinline__ unsigned keep16(const rng::Key& key, unsigned threshold, unsigned long long row_groups0, int col0) {
  unsigned bits = 0;
#pragma unroll
  for (int g = 0; g < 2; ++g)
    bits |= rng::keep_bits(rng::philox(key, row_groups0 + (unsigned)((col0 >> 3) + g)), threshold) << (8 * g);
  return bits;
}
__device__ __forceinline__ void store_row16(__nv_bfloat16* dst, const float (&v)[16]) {
#pragma unroll
  for (int g = 0; g < 2; ++g) {
    uint4 pk;
    pk.x = pack_bf16(v[8 * g], v[8 * g + 1]); pk.y = pack_bf16(v[8 * g + 2], v[8 * g + 3]);
    pk.z = pack_bf16(v[8 * g + 4], v[8 * g + 5]); pk.w = pack_bf16(v[8 * g + 6], v[8 * g + 7]);
    reinterpret_cast<uint4*>(dst)[g] = pk;
  }
}

__device__ __forceinline__ void store_row32(__nv_bfloat16* dst, const float (&v)[32]) {
#pragma unroll
  for (int g = 0; g < 4; ++g) {
    uint4 pk;
    pk.x = pack_bf16(v[8 * g], v[8 * g + 1]); pk.y = pack_bf16(v[8 * g + 2], v[8 * g + 3]);
    pk.z = pack_bf16(v[8 * g + 4], v[8 * g + 5]); pk.w = pack_bf16(v[8 * g + 6], v[8 * g + 7]);
    reinterpret_cast<uint4*>(dst)[g] = pk;
  }
}

// A ring of 16 KiB tiles filled by TMA in load order; slot and phase follow from the load's number.
struct Ring {
  unsigned base, full0, empty0;   // shared-memory addresses: slot 0, full barrier 0, empty barrier 0
  int slots;
  __device__ __forceinline__ unsigned slot_addr(unsigned n) const { return base + (n % slots) * kTileBytes; }
  __device__ __forceinline__ unsigned full(unsigned n) const { return full0 + 8u * (n % slots); }
  __device__ __forceinline__ unsigned empty(unsigned n) const { return empty0 + 8u * (n % slots); }
  __device__ __forceinline__ unsigned phase(unsigned n) const { return (n / slots) & 1u; }
};

// ---------------------------------------------------------------------------------------------------
// forward
// ---------------------------------------------------------------------------------------------------
// Shared memory: Q tile | ring of 3 K/V tiles (loaded K0 V0 K1 V1 ...) | P.  Tensor memory (256 columns):
// S at [0, 128), the P V product of the current key tile at [128, 192).  Two CTAs fit on an SM.
constexpr int kFwdRing = 3;
constexpr unsigned kFwdSmem = 1024 + kTileBytes * (1 + kFwdRing) + kProbBytes + 256;

__global__ void __launch_bounds__(kThreads, 2)
attention_forward_kernel(const __grid_constant__ CUtensorMap tmQKV, const Params p) {
  extern __shared__ unsigned char smem_raw[];
  const unsigned base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  unsigned char* gen = smem_raw + (base - smem_u32(smem_raw));
  const unsigned sQ = base;
  const unsigned sRing = base + kTileBytes;
  unsigned char* sP_gen = gen + kTileBytes * (1 + kFwdRing);
  const unsigned sP = base + kTileBytes * (1 + kFwdRing);
  const unsigned bars = sP + kProbBytes;
  // barriers: q_full, q_empty, s_full, s_empty, p_full, o_full, o_empty, ring full[3], ring empty[3]
  const unsigned q_full = bars, q_empty = bars + 8, s_full = bars + 16, s_empty = bars + 24, p_full = bars + 32, o_full = bars + 40,
                 o_empty = bars + 48;
  const Ring ring{sRing, bars + 56, bars + 56 + 8 * kFwdRing, kFwdRing};
  const unsigned tmem_slot = bars + 56 + 16 * kFwdRing;
  volatile unsigned* tmem_slot_gen = reinterpret_cast<volatile unsigned*>(sP_gen + kProbBytes + 56 + 16 * kFwdRing);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    mbar_init(q_full, 1); mbar_init(q_empty, 1); mbar_init(s_full, 1); mbar_init(s_empty, 128); mbar_init(p_full, 128);
    mbar_init(o_full, 1); mbar_init(o_empty, 128);
    for (int s = 0; s < kFwdRing; ++s) { mbar_init(ring.full0 + 8u * s, 1); mbar_init(ring.empty0 + 8u * s, 1); }
    fence_barrier_init();
    prefetch_tensormap(&tmQKV);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 256);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const unsigned tmem_base = *tmem_slot_gen;
  const unsigned tS = tmem_base, tO = tmem_base + 128;

  const bool causal = p.causal != 0 || (p.mask_is_causal != nullptr && *p.mask_is_causal != 0u);
  const int BH = p.N * p.H;
  // unit -> (query tile i, batch entry b, head h); the heaviest tiles (most key tiles under the causal rule) first
  auto decode = [&](int unit, int& i, int& b, int& h) {
    i = p.nt - 1 - unit / BH;
    const int bh = unit - (unit / BH) * BH;
    b = bh / p.H;
    h = bh - b * p.H;
  };
  auto key_tiles = [&](int i) { return causal ? min(p.nt, i + 1) : p.nt; };

  if (warp == 0) {
    if (lane == 0) {
      unsigned n_q = 0, n_ld = 0;
      bool ok = true;
      for (int unit = blockIdx.x; unit < p.units && ok; unit += gridDim.x) {
        int i, b, h;
        decode(unit, i, b, h);
        if (!mbar_wait(q_empty, (n_q & 1u) ^ 1u)) { ok = false; break; }
        mbar_expect_tx(q_full, kTileBytes);
        tma_load_4d(sQ, &tmQKV, h * HD, i * BT, 0, b, q_full);
        ++n_q;
        const int nk = key_tiles(i);
        for (int j = 0; j < nk && ok; ++j) {
          for (int which = 1; which <= 2; ++which) {           // K_j then V_j
            if (!mbar_wait(ring.empty(n_ld), ring.phase(n_ld) ^ 1u)) { ok = false; break; }
            mbar_expect_tx(ring.full(n_ld), kTileBytes);
            tma_load_4d(ring.slot_addr(n_ld), &tmQKV, which * p.E + h * HD, j * BT, 0, b, ring.full(n_ld));
            ++n_ld;
          }
        }
      }
      if (!ok) atomicCAS(p.error, 0u, 11u);
    }
  } else if (warp == 1) {
    if (lane == 0) {
      unsigned n_q = 0, n_tile = 0, n_s = 0, n_o = 0;   // units, key tiles begun, S products issued, P V products issued
      bool ok = true;
      constexpr unsigned kIdescS = idesc(128, false, false), kIdescO = idesc(64, false, true);
      for (int unit = blockIdx.x; unit < p.units && ok; unit += gridDim.x) {
        int i, b, h;
        decode(unit, i, b, h);
        const int nk = key_tiles(i);
        if (!mbar_wait(q_full, n_q & 1u)) { ok = false; break; }
        auto issue_s = [&](int j) -> bool {          // S = Q K_j^T
          const unsigned ld = 2u * (n_tile + (unsigned)j);
          if (!mbar_wait(ring.full(ld), ring.phase(ld))) return false;
          if (!mbar_wait(s_empty, (n_s & 1u) ^ 1u)) return false;
          tc_fence_after();
          const unsigned sK = ring.slot_addr(ld);
#pragma unroll
          for (int k = 0; k < HD / 16; ++k)
            umma_bf16(tS, make_desc(sQ + k * 32u, 16u, 1024u), make_desc(sK + k * 32u, 16u, 1024u), kIdescS, k != 0 ? 1u : 0u);
          umma_commit(s_full);
          umma_commit(ring.empty(ld));
          if (j == nk - 1) umma_commit(q_empty);     // the unit's last use of Q
          ++n_s;
          return true;
        };
        if (!issue_s(0)) { ok = false; break; }
        for (int j = 0; j < nk; ++j) {
          if (j + 1 < nk && !issue_s(j + 1)) { ok = false; break; }
          const unsigned ld = 2u * (n_tile + (unsigned)j) + 1u;
          if (!mbar_wait(p_full, n_o & 1u) || !mbar_wait(ring.full(ld), ring.phase(ld)) || !mbar_wait(o_empty, (n_o & 1u) ^ 1u)) { ok = false; break; }
          tc_fence_after();
          const unsigned sV = ring.slot_addr(ld);
#pragma unroll
          for (int kk = 0; kk < BT / 16; ++kk)      // 16 keys per instruction: P is K-major (two 64-key chunks), V is MN-major as stored
            umma_bf16(tO, make_desc(sP + (kk >> 2) * (BT * 128u) + (kk & 3) * 32u, 16u, 1024u), make_desc(sV + kk * 2048u, 8192u, 1024u), kIdescO,
                      kk != 0 ? 1u : 0u);
          umma_commit(o_full);
          umma_commit(ring.empty(ld));
          ++n_o;
        }
        n_tile += (unsigned)nk;
        ++n_q;
      }
      if (!ok) atomicCAS(p.error, 0u, 12u);
    }
  } else {
    const int q4 = warp & 3;                       // TMEM lane quarter of this warp
    const int r = q4 * 32 + lane;                  // row of the query tile
    const unsigned lane_off = (unsigned)(q4 * 32) << 16;
    unsigned n_s = 0, n_o = 0;
    bool ok = true;
    rng::Key key = {0u, 0u, 0u, 0u};
    if (p.drop_threshold) key = rng::make_key(p.rng, p.call_id);
    const unsigned long long row_groups = (unsigned long long)((p.L + 7) / 8);
    const bool use_mask = p.mask != nullptr && !(p.mask_is_causal != nullptr && *p.mask_is_causal != 0u);
    for (int unit = blockIdx.x; unit < p.units && ok; unit += gridDim.x) {
      int i, b, h;
      decode(unit, i, b, h);
      const int nk = key_tiles(i);
      const int q = i * BT + r;
      const bool row_ok = q < p.L;
      const float* mrow = (use_mask && row_ok) ? p.mask + (long long)q * p.L : nullptr;
      const unsigned long long rg0 = ((unsigned long long)(b * p.H + h) * (unsigned long long)p.L + (unsigned long long)q) * row_groups;
      float m = -INFINITY, l = 0.f;
      float O[64];
#pragma unroll
      for (int d = 0; d < 64; ++d) O[d] = 0.f;
      for (int j = 0; j < nk; ++j) {
        if (!mbar_wait(s_full, n_s & 1u)) { ok = false; break; }
        tc_fence_after();
        const int k0 = j * BT;
        const int last = row_ok ? (causal ? min(q, p.L - 1) : p.L - 1) : -1;     // last key this row may see
        // tcgen05.ld is a warp-wide instruction: whether a group of 32 columns is read at all must be decided
        // for the whole warp, by the last key that ANY of its 32 rows may see
        const int wq0 = i * BT + q4 * 32;
        const int wlast = wq0 < p.L ? (causal ? min(wq0 + 31, p.L - 1) : p.L - 1) : -1;
        // the smallest `last` of the warp's rows decides, for the whole warp, whether a chunk needs per-element limits
        const int wmin_last = (wq0 + 31 < p.L) ? (causal ? wq0 : p.L - 1) : -1;
        // pass 1 over the scores in tensor memory: the row maximum
        float mx = m;
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          const int c0 = k0 + 32 * c;
          if (c0 > wlast) break;
          unsigned v[32];
          tmem_ld_32x32(tS + lane_off + 32u * c, v);
          tmem_ld_wait();
          const float* mr = mrow ? mrow + c0 : nullptr;
          if (c0 + 31 > wmin_last) mx = chunk_max<true>(v, p.scale2, last - c0, mr, mx);
          else mx = chunk_max<false>(v, p.scale2, 31, mr, mx);
        }
        const float m_use = (mx == -INFINITY) ? 0.f : mx;
        const float alpha = (m == -INFINITY) ? 0.f : ex2(m - m_use);
        // pass 2: probabilities (relative to the running maximum), their sum, dropout, bf16 into shared memory
        float sum = 0.f;
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          const int c0 = k0 + 32 * c;
          float pr[32];
          if (c0 > wlast) {
#pragma unroll
            for (int e = 0; e < 32; ++e) pr[e] = 0.f;
          } else {
            unsigned v[32];
            tmem_ld_32x32(tS + lane_off + 32u * c, v);
            tmem_ld_wait();
            const float* mr = mrow ? mrow + c0 : nullptr;
            if (c0 + 31 > wmin_last) sum += chunk_exp<true>(v, p.scale2, m_use, last - c0, mr, pr);
            else sum += chunk_exp<false>(v, p.scale2, m_use, 31, mr, pr);
            if (p.drop_threshold) {
              const unsigned keep = keep32(key, p.drop_threshold, rg0, c0);
#pragma unroll
              for (int e = 0; e < 32; ++e) pr[e] = (keep >> e) & 1u ? pr[e] : 0.f;
            }
          }
          store_prob_columns(sP_gen, r, c, pr);
        }
        tc_fence_before();
        mbar_arrive(s_empty);                 // the scores have been read: the next S product may overwrite them
        ++n_s;
        fence_proxy_async();                  // P is read by the tensor core through the async proxy
        mbar_arrive(p_full);
        l = l * alpha + sum;
        m = mx;
        if (!mbar_wait(o_full, n_o & 1u)) { ok = false; break; }
        tc_fence_after();
        unsigned o0[32], o1[32];
        tmem_ld_32x32(tO + lane_off, o0);
        tmem_ld_32x32(tO + lane_off + 32u, o1);
        tmem_ld_wait();
        tc_fence_before();
        mbar_arrive(o_empty);
        ++n_o;
#pragma unroll
        for (int d = 0; d < 32; ++d) {
          O[d] = fmaf(O[d], alpha, __uint_as_float(o0[d]));
          O[32 + d] = fmaf(O[32 + d], alpha, __uint_as_float(o1[d]));
        }
      }
      if (!ok) break;
      if (row_ok) {
        const float inv = l > 0.f ? p.drop_scale / l : 0.f;
        store_row64(p.out + ((long long)q * p.N + b) * p.E + h * HD, O, inv);
        p.lse2[(long long)(b * p.H + h) * p.L + q] = (l > 0.f) ? ((m == -INFINITY ? 0.f : m) + log2f(l)) : -INFINITY;
      }
    }
    if (!ok) atomicCAS(p.error, 0u, 13u);
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 256);
  }
}

// ---------------------------------------------------------------------------------------------------
// backward
// ---------------------------------------------------------------------------------------------------
// KEY_MAJOR = true : unit = (batch entry, head, key tile j);   outer tiles K_j, V_j;   inner tiles Q_i, dO_i;   dV, dK
// KEY_MAJOR = false: unit = (batch entry, head, query tile i); outer tiles Q_i, dO_i; inner tiles K_j, V_j;   dQ
// Shared memory: 2 outer tiles | 2 stages x 2 inner tiles | Pd | dS.  Tensor memory (512 columns): S [0,128),
// dPd [128,256), accumulators [256,320) and [320,384).
constexpr int kBwdStages = 2;
constexpr int kBwdThreads = 576;            // TMA warp, MMA warp, 16 math warps: four per tensor-memory lane quarter, each
constexpr int kBwdMath = 512;               // taking a quarter of the columns of its 32 rows (no row reductions are needed here)
constexpr unsigned kBwdSmem = 1024 + kTileBytes * (2 + 2 * kBwdStages) + 2 * kProbBytes + 256;

template <bool KEY_MAJOR>
__global__ void __launch_bounds__(kBwdThreads, 1)
attention_backward_kernel(const __grid_constant__ CUtensorMap tmQKV, const __grid_constant__ CUtensorMap tmDO, const Params p) {
  extern __shared__ unsigned char smem_raw[];
  const unsigned base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  unsigned char* gen = smem_raw + (base - smem_u32(smem_raw));
  const unsigned sOut0 = base, sOut1 = base + kTileBytes;              // K_j, V_j  or  Q_i, dO_i
  const unsigned sIn = base + 2 * kTileBytes;                          // stage s: two tiles at sIn + s * 2 * kTileBytes
  const unsigned off_p = kTileBytes * (2 + 2 * kBwdStages);
  unsigned char* sP_gen = gen + off_p;
  unsigned char* sdS_gen = sP_gen + kProbBytes;
  const unsigned sP = base + off_p, sdS = sP + kProbBytes;
  const unsigned bars = sdS + kProbBytes;
  // barriers: out_full, out_empty, s_full, s_empty, p_full, p_empty, acc_full, acc_empty, in_full[2], in_empty[2]
  const unsigned out_full = bars, out_empty = bars + 8, s_full = bars + 16, s_empty = bars + 24, p_full = bars + 32, p_empty = bars + 40,
                 acc_full = bars + 48, acc_empty = bars + 56, in_full0 = bars + 64, in_empty0 = bars + 64 + 8 * kBwdStages;
  const unsigned tmem_slot = bars + 64 + 16 * kBwdStages;
  volatile unsigned* tmem_slot_gen = reinterpret_cast<volatile unsigned*>(sdS_gen + kProbBytes + 64 + 16 * kBwdStages);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    mbar_init(out_full, 1); mbar_init(out_empty, 1); mbar_init(s_full, 1); mbar_init(s_empty, kBwdMath); mbar_init(p_full, kBwdMath);
    mbar_init(p_empty, 1); mbar_init(acc_full, 1); mbar_init(acc_empty, kBwdMath);
    for (int s = 0; s < kBwdStages; ++s) { mbar_init(in_full0 + 8u * s, 1); mbar_init(in_empty0 + 8u * s, 1); }
    fence_barrier_init();
    prefetch_tensormap(&tmQKV);
    prefetch_tensormap(&tmDO);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const unsigned tmem_base = *tmem_slot_gen;
  const unsigned tS = tmem_base, tDP = tmem_base + 128, tA0 = tmem_base + 256, tA1 = tmem_base + 320;

  const bool causal = p.causal != 0 || (p.mask_is_causal != nullptr && *p.mask_is_causal != 0u);
  const int BH = p.N * p.H;
  // unit -> (outer tile, b, h); heaviest first: key tile 0 sees every query tile, the last query tile sees every key tile
  auto decode = [&](int unit, int& o, int& b, int& h) {
    const int t = unit / BH;
    o = KEY_MAJOR ? t : p.nt - 1 - t;
    const int bh = unit - t * BH;
    b = bh / p.H;
    h = bh - b * p.H;
  };
  // inner tiles that meet outer tile o: [first, end)
  auto inner_first = [&](int o) { return (KEY_MAJOR && causal) ? o : 0; };
  auto inner_end = [&](int o) { return (!KEY_MAJOR && causal) ? min(p.nt, o + 1) : p.nt; };

  if (warp == 0) {
    if (lane == 0) {
      unsigned n_out = 0, n_in = 0;
      bool ok = true;
      for (int unit = blockIdx.x; unit < p.units && ok; unit += gridDim.x) {
        int o, b, h;
        decode(unit, o, b, h);
        if (!mbar_wait(out_empty, (n_out & 1u) ^ 1u)) { ok = false; break; }
        mbar_expect_tx(out_full, 2 * kTileBytes);
        if (KEY_MAJOR) {
          tma_load_4d(sOut0, &tmQKV, p.E + h * HD, o * BT, 0, b, out_full);        // K_j
          tma_load_4d(sOut1, &tmQKV, 2 * p.E + h * HD, o * BT, 0, b, out_full);    // V_j
        } else {
          tma_load_4d(sOut0, &tmQKV, h * HD, o * BT, 0, b, out_full);              // Q_i
          tma_load_4d(sOut1, &tmDO, h * HD, o * BT, 0, b, out_full);               // dO_i
        }
        ++n_out;
        for (int t = inner_first(o); t < inner_end(o); ++t) {
          const unsigned s = n_in % kBwdStages, ph = (n_in / kBwdStages) & 1u;
          if (!mbar_wait(in_empty0 + 8u * s, ph ^ 1u)) { ok = false; break; }
          mbar_expect_tx(in_full0 + 8u * s, 2 * kTileBytes);
          const unsigned dst = sIn + s * 2 * kTileBytes;
          if (KEY_MAJOR) {
            tma_load_4d(dst, &tmQKV, h * HD, t * BT, 0, b, in_full0 + 8u * s);                       // Q_i
            tma_load_4d(dst + kTileBytes, &tmDO, h * HD, t * BT, 0, b, in_full0 + 8u * s);           // dO_i
          } else {
            tma_load_4d(dst, &tmQKV, p.E + h * HD, t * BT, 0, b, in_full0 + 8u * s);                 // K_j
            tma_load_4d(dst + kTileBytes, &tmQKV, 2 * p.E + h * HD, t * BT, 0, b, in_full0 + 8u * s);// V_j
          }
          ++n_in;
        }
      }
      if (!ok) atomicCAS(p.error, 0u, 21u);
    }
  } else if (warp == 1) {
    if (lane == 0) {
      unsigned n_out = 0, n_in = 0;
      bool ok = true;
      constexpr unsigned kIdescS = idesc(128, false, false);
      constexpr unsigned kIdescT = idesc(64, true, true);      // Pd^T dO, dS^T Q : both operands MN-major as stored
      constexpr unsigned kIdescQ = idesc(64, false, true);     // dS K : dS K-major, K MN-major as stored
      for (int unit = blockIdx.x; unit < p.units && ok; unit += gridDim.x) {
        int o, b, h;
        decode(unit, o, b, h);
        if (!mbar_wait(out_full, n_out & 1u)) { ok = false; break; }
        if (!mbar_wait(acc_empty, (n_out & 1u) ^ 1u)) { ok = false; break; }     // the previous unit's accumulators have been read
        const int first = inner_first(o), end = inner_end(o);
        for (int t = first; t < end; ++t) {
          const unsigned s = n_in % kBwdStages, ph = (n_in / kBwdStages) & 1u;
          if (!mbar_wait(in_full0 + 8u * s, ph) || !mbar_wait(s_empty, (n_in & 1u) ^ 1u)) { ok = false; break; }
          tc_fence_after();
          const unsigned in0 = sIn + s * 2 * kTileBytes, in1 = in0 + kTileBytes;
          const unsigned sQt = KEY_MAJOR ? in0 : sOut0, sDOt = KEY_MAJOR ? in1 : sOut1;
          const unsigned sKt = KEY_MAJOR ? sOut0 : in0, sVt = KEY_MAJOR ? sOut1 : in1;
#pragma unroll
          for (int k = 0; k < HD / 16; ++k)       // S = Q K^T
            umma_bf16(tS, make_desc(sQt + k * 32u, 16u, 1024u), make_desc(sKt + k * 32u, 16u, 1024u), kIdescS, k != 0 ? 1u : 0u);
#pragma unroll
          for (int k = 0; k < HD / 16; ++k)       // dPd = dO V^T
            umma_bf16(tDP, make_desc(sDOt + k * 32u, 16u, 1024u), make_desc(sVt + k * 32u, 16u, 1024u), kIdescS, k != 0 ? 1u : 0u);
          umma_commit(s_full);
          if (!mbar_wait(p_full, n_in & 1u)) { ok = false; break; }
          tc_fence_after();
          const unsigned acc = (t != first) ? 1u : 0u;
          if (KEY_MAJOR) {
#pragma unroll
            for (int kk = 0; kk < BT / 16; ++kk)  // dV += Pd^T dO : 16 queries per instruction
              umma_bf16(tA0, make_desc(sP + kk * 2048u, BT * 128u, 1024u), make_desc(sDOt + kk * 2048u, 8192u, 1024u), kIdescT, (acc | (kk != 0)) ? 1u : 0u);
#pragma unroll
            for (int kk = 0; kk < BT / 16; ++kk)  // dK += dS^T Q
              umma_bf16(tA1, make_desc(sdS + kk * 2048u, BT * 128u, 1024u), make_desc(sQt + kk * 2048u, 8192u, 1024u), kIdescT, (acc | (kk != 0)) ? 1u : 0u);
          } else {
#pragma unroll
            for (int kk = 0; kk < BT / 16; ++kk)  // dQ += dS K : 16 keys per instruction
              umma_bf16(tA0, make_desc(sdS + (kk >> 2) * (BT * 128u) + (kk & 3) * 32u, 16u, 1024u), make_desc(sKt + kk * 2048u, 8192u, 1024u), kIdescQ,
                        (acc | (kk != 0)) ? 1u : 0u);
          }
          umma_commit(in_empty0 + 8u * s);
          umma_commit(p_empty);
          ++n_in;
        }
        if (!ok) break;
        umma_commit(acc_full);
        umma_commit(out_empty);
        ++n_out;
      }
      if (!ok) atomicCAS(p.error, 0u, 22u);
    }
  } else {
    const int q4 = warp & 3;                       // tensor-memory lane quarter of this warp
    const int part = (warp - 2) >> 2;              // which 32 of the tile's 128 columns this warp takes
    const int r = q4 * 32 + lane;
    const unsigned lane_off = (unsigned)(q4 * 32) << 16;
    unsigned n_out = 0, n_in = 0;
    bool ok = true;
    rng::Key key = {0u, 0u, 0u, 0u};
    if (p.drop_threshold) key = rng::make_key(p.rng, p.call_id);
    const unsigned long long row_groups = (unsigned long long)((p.L + 7) / 8);
    const bool use_mask = p.mask != nullptr && !(p.mask_is_causal != nullptr && *p.mask_is_causal != 0u);
    for (int unit = blockIdx.x; unit < p.units && ok; unit += gridDim.x) {
      int o, b, h;
      decode(unit, o, b, h);
      const int first = inner_first(o), end = inner_end(o);
      const long long bh = (long long)b * p.H + h;
      for (int t = first; t < end; ++t) {
        const int i = KEY_MAJOR ? t : o, j = KEY_MAJOR ? o : t;     // query tile, key tile
        const int q = i * BT + r, k0 = j * BT;
        const bool row_ok = q < p.L;
        const float lse = row_ok ? p.lse2[bh * p.L + q] : 0.f;
        const float dl = row_ok ? p.delta[bh * p.L + q] : 0.f;
        const float* mrow = (use_mask && row_ok) ? p.mask + (long long)q * p.L : nullptr;
        const unsigned long long rg0 = ((unsigned long long)bh * (unsigned long long)p.L + (unsigned long long)q) * row_groups;
        const int last = row_ok ? (causal ? min(q, p.L - 1) : p.L - 1) : -1;
        // warp-wide decisions for the warp-wide tcgen05.ld (see the forward kernel)
        const int wq0 = i * BT + q4 * 32;
        const int wlast = wq0 < p.L ? (causal ? min(wq0 + 31, p.L - 1) : p.L - 1) : -1;
        const int wmin_last = (wq0 + 31 < p.L) ? (causal ? wq0 : p.L - 1) : -1;
        if (!mbar_wait(s_full, n_in & 1u) || !mbar_wait(p_empty, (n_in & 1u) ^ 1u)) { ok = false; break; }
        tc_fence_after();
#pragma unroll 1
        for (int cc = 0; cc < 2; ++cc) {
          const int c = 2 * part + cc;               // group of 16 columns of the tile
          const int c0 = k0 + 16 * c;
          float pd[16], ds[16];
          if (c0 > wlast) {
#pragma unroll
            for (int e = 0; e < 16; ++e) { pd[e] = 0.f; ds[e] = 0.f; }
          } else {
            unsigned sv[16], gv[16];
            tmem_ld_32x16(tS + lane_off + 16u * c, sv);
            tmem_ld_32x16(tDP + lane_off + 16u * c, gv);
            tmem_ld_wait();
            const float* mr = mrow ? mrow + c0 : nullptr;
            if (c0 + 15 > wmin_last) chunk_exp16<true>(sv, p.scale2, lse, last - c0, mr, pd);
            else chunk_exp16<false>(sv, p.scale2, lse, 15, mr, pd);
            if (p.drop_threshold) {
              const unsigned keep = keep16(key, p.drop_threshold, rg0, c0);
#pragma unroll
              for (int e = 0; e < 16; ++e) {
                const float kd = (keep >> e) & 1u ? p.drop_scale : 0.f;
                ds[e] = pd[e] * p.scale * fmaf(__uint_as_float(gv[e]), kd, -dl);
                pd[e] *= kd;
              }
            } else {
#pragma unroll
              for (int e = 0; e < 16; ++e) ds[e] = pd[e] * p.scale * (__uint_as_float(gv[e]) - dl);
            }
          }
          if (KEY_MAJOR) store_prob_columns16(sP_gen, r, c, pd);
          store_prob_columns16(sdS_gen, r, c, ds);
        }
        tc_fence_before();
        mbar_arrive(s_empty);
        fence_proxy_async();
        mbar_arrive(p_full);
        ++n_in;
      }
      if (!ok) break;
      // epilogue: 16 of the 64 columns of this thread's row of the accumulators (a key row, or a query row)
      if (!mbar_wait(acc_full, n_out & 1u)) { ok = false; break; }
      tc_fence_after();
      const int row = o * BT + r;
      unsigned a0[16];
      float v[16];
      tmem_ld_32x16(tA0 + lane_off + 16u * part, a0);
      tmem_ld_wait();
#pragma unroll
      for (int d = 0; d < 16; ++d) v[d] = __uint_as_float(a0[d]);
      __nv_bfloat16* grow = p.dqkv + ((long long)row * p.N + b) * (3LL * p.E) + h * HD + 16 * part;
      if (KEY_MAJOR) {
        if (row < p.L) store_row16(grow + 2 * p.E, v);               // dV
        tmem_ld_32x16(tA1 + lane_off + 16u * part, a0);
        tmem_ld_wait();
#pragma unroll
        for (int d = 0; d < 16; ++d) v[d] = __uint_as_float(a0[d]);
        if (row < p.L) store_row16(grow + p.E, v);                   // dK
      } else {
        if (row < p.L) store_row16(grow, v);                         // dQ
      }
      tc_fence_before();
      mbar_arrive(acc_empty);
      ++n_out;
    }
    if (!ok) atomicCAS(p.error, 0u, 23u);
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// delta[bh][l] = sum_d dO[l, b, h*64 + d] * O[l, b, h*64 + d]: eight threads per (l, b, h), one 16-byte load of each
// tensor per thread.
__global__ void __launch_bounds__(256) attention_delta_kernel(const __nv_bfloat16* __restrict__ dout, const __nv_bfloat16* __restrict__ out,
                                                              float* __restrict__ delta, int L, int N, int H) {
  const long long total = (long long)L * N * H;
  const long long w = ((long long)blockIdx.x * 256 + threadIdx.x) >> 3;     // (l * N + b) * H + h
  const int part = threadIdx.x & 7;
  float s = 0.f;
  int h = 0;
  long long lb = 0;
  if (w < total) {
    h = (int)(w % H);
    lb = w / H;
    const long long off = w * HD + 8 * part;                                // rows of dout / out are contiguous over (l, b, h, d)
    const uint4 a = *reinterpret_cast<const uint4*>(dout + off), o = *reinterpret_cast<const uint4*>(out + off);
    const unsigned aw[4] = {a.x, a.y, a.z, a.w}, ow[4] = {o.x, o.y, o.z, o.w};
#pragma unroll
    for (int k = 0; k < 4; ++k)
      s += __uint_as_float(aw[k] << 16) * __uint_as_float(ow[k] << 16) + __uint_as_float(aw[k] & 0xffff0000u) * __uint_as_float(ow[k] & 0xffff0000u);
  }
  s += __shfl_xor_sync(0xffffffffu, s, 4);
  s += __shfl_xor_sync(0xffffffffu, s, 2);
  s += __shfl_xor_sync(0xffffffffu, s, 1);
  if (w < total && part == 0) {
    const int b = (int)(lb % N), l = (int)(lb / N);
    delta[((long long)b * H + h) * L + l] = s;
  }
}

// Keep mask of the dropout on the probabilities, as bytes [N*H][L][L] (for tests).
__global__ void __launch_bounds__(256) attention_mask_kernel(unsigned char* __restrict__ mask, int L, long long rows, unsigned threshold,
                                                             const rng::State* st, unsigned long long call_id) {
  const rng::Key key = rng::make_key(st, call_id);
  const long long groups_per_row = (L + 7) / 8, total = rows * groups_per_row;
  for (long long g = (long long)blockIdx.x * blockDim.x + threadIdx.x; g < total; g += (long long)gridDim.x * blockDim.x) {
    const long long row = g / groups_per_row;
    const int c0 = (int)(g - row * groups_per_row) * 8;
    const unsigned keep = rng::keep_bits(rng::philox(key, (unsigned long long)g), threshold);
    for (int e = 0; e < 8 && c0 + e < L; ++e) mask[row * L + c0 + e] = (unsigned char)((keep >> e) & 1u);
  }
}

// *flag stays non-zero when mask[q][k] is 0 for k <= q and -inf for k > q (the language-model mask).  The host
// sets the word to all ones before the launch; any block that finds a deviating entry clears it.
__global__ void __launch_bounds__(256) classify_mask_kernel(const float* __restrict__ mask, int L, unsigned* flag) {
  int ok = 1;
  const long long n = (long long)L * L;
  for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += (long long)gridDim.x * blockDim.x) {
    const int q = (int)(e / L), k = (int)(e - (long long)q * L);
    const float v = mask[e];
    ok &= (k <= q) ? (v == 0.f) : (v == -INFINITY);
  }
  ok = __syncthreads_and(ok);
  if (threadIdx.x == 0 && !ok) atomicAnd(flag, 0u);
}

// ---- host side ----------------------------------------------------------------------------------------
struct Attr { bool fwd = false, bwd_k = false, bwd_q = false; };
static Attr g_attr[64];
static std::mutex g_attr_mutex;

static int check(long long L, long long N, long long H, long long D, double p) {
  if (L < 0 || N < 0 || H < 1) return fail(HAPX_ERR_EXTENT, "attention: negative extent");
  if (D != HD) return fail(HAPX_ERR_EXTENT, "attention: the fused kernels are built for head dimension 64");
  if (L > 0x3fffffff / BT || N * H > 0x7fffffff || N * H * ((L + BT - 1) / BT) > 0x7fffffff) return fail(HAPX_ERR_EXTENT, "attention: too many tiles");
  if (!(p >= 0.0 && p < 1.0)) return fail(HAPX_ERR_ARGUMENT, "attention: dropout_p must be in [0, 1)");
  return HAPX_OK;
}

static int fill(Params& p, long long L, long long N, long long H, int causal, const float* mask, const unsigned* mask_flag, double dropout_p,
                uint64_t call_id, int* sm_count) {
  p = Params();
  p.L = (int)L; p.N = (int)N; p.H = (int)H; p.E = (int)(H * HD);
  p.nt = (int)((L + BT - 1) / BT);
  p.causal = causal;
  p.mask = mask;
  p.scale = 0.125f;
  p.scale2 = 0.125f * kLog2e;
  p.drop_threshold = dropout_p > 0.0 ? rng::threshold_for(dropout_p) : 0u;
  p.drop_scale = (float)(1.0 / (1.0 - dropout_p));
  p.call_id = call_id;
  if (int e = gemm::error_word(&p.error, sm_count)) return e;
  if (p.drop_threshold) {
    rng::State* st = nullptr;
    if (int e = rng_state(&st)) return e;
    p.rng = st;
  }
  p.mask_is_causal = (mask && !causal) ? mask_flag : nullptr;
  return HAPX_OK;
}

}  // namespace fattn
}  // namespace hapx

using namespace hapx;
using hapx::gemm::Operand;

extern "C" {

int hapx_attention_classify_mask(const float* mask, int64_t L, unsigned* flag, hapx_stream stream_) {
  if (!mask || !flag || L < 1 || L > 0x7fff) return fail(HAPX_ERR_ARGUMENT, "attention_classify_mask: bad argument");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  HAPX_CUDA(cudaMemsetAsync(flag, 0xff, sizeof(unsigned), stream));
  const long long n = L * L;
  const int grid = (int)std::max<long long>(1, std::min<long long>((n + 1023) / 1024, 256));
  fattn::classify_mask_kernel<<<grid, 256, 0, stream>>>(mask, (int)L, flag);
  HAPX_CUDA(cudaGetLastError());
  count_launch();
  return HAPX_OK;
}

int hapx_attention_fused_forward(void* out, float* lse2, const void* qkv, int64_t L, int64_t N, int64_t H, int64_t D, int causal,
                                 const float* mask, const unsigned* mask_flag, double dropout_p, uint64_t call_id, hapx_stream stream_) {
  if (int e = fattn::check(L, N, H, D, dropout_p)) return e;
  if (L == 0 || N == 0) return HAPX_OK;
  if (!out || !lse2 || !qkv) return fail(HAPX_ERR_ARGUMENT, "attention_fused_forward: null pointer");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  fattn::Params p;
  int sms = 0;
  if (int e = fattn::fill(p, L, N, H, causal, mask, mask_flag, dropout_p, call_id, &sms)) return e;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.lse2 = lse2;
  p.units = (int)(N * H * p.nt);
  const long long E = H * fattn::HD;
  CUtensorMap tm;
  // packed qkv as (column in [0, 3E), row l, -, batch entry b): boxes of 64 columns x 128 rows
  if (int e = gemm::make_map(&tm, Operand{qkv, false, N * 3 * E, 0, 3 * E}, L, 3 * E, fattn::BT, 1, (int)N)) return e;
  int device = 0;
  HAPX_CUDA(cudaGetDevice(&device));
  {
    std::lock_guard<std::mutex> lock(fattn::g_attr_mutex);
    if (!fattn::g_attr[device].fwd) {
      HAPX_CUDA(cudaFuncSetAttribute(fattn::attention_forward_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)fattn::kFwdSmem));
      fattn::g_attr[device].fwd = true;
    }
  }
  const int grid = std::max(1, std::min(p.units, 2 * sms));
  fattn::attention_forward_kernel<<<grid, fattn::kThreads, fattn::kFwdSmem, stream>>>(tm, p);
  HAPX_CUDA(cudaGetLastError());
  count_launch();
  return HAPX_OK;
}

int hapx_attention_fused_backward(void* dqkv, float* delta_ws, const void* dout, const void* out, const float* lse2, const void* qkv,
                                  int64_t L, int64_t N, int64_t H, int64_t D, int causal, const float* mask, const unsigned* mask_flag,
                                  double dropout_p, uint64_t call_id, hapx_stream stream_) {
  if (int e = fattn::check(L, N, H, D, dropout_p)) return e;
  if (L == 0 || N == 0) return HAPX_OK;
  if (!dqkv || !delta_ws || !dout || !out || !lse2 || !qkv) return fail(HAPX_ERR_ARGUMENT, "attention_fused_backward: null pointer");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  fattn::Params p;
  int sms = 0;
  if (int e = fattn::fill(p, L, N, H, causal, mask, mask_flag, dropout_p, call_id, &sms)) return e;
  p.lse2 = const_cast<float*>(lse2);
  p.delta = delta_ws;
  p.dqkv = static_cast<__nv_bfloat16*>(dqkv);
  p.units = (int)(N * H * p.nt);
  const long long E = H * fattn::HD;
  {
    const long long rows = L * N * H;      // 8 threads each
    fattn::attention_delta_kernel<<<(unsigned)((rows + 31) / 32), 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(dout),
                                                                                 static_cast<const __nv_bfloat16*>(out), delta_ws, (int)L, (int)N, (int)H);
    HAPX_CUDA(cudaGetLastError());
    count_launch();
  }
  CUtensorMap tmQKV, tmDO;
  if (int e = gemm::make_map(&tmQKV, Operand{qkv, false, N * 3 * E, 0, 3 * E}, L, 3 * E, fattn::BT, 1, (int)N)) return e;
  if (int e = gemm::make_map(&tmDO, Operand{dout, false, N * E, 0, E}, L, E, fattn::BT, 1, (int)N)) return e;
  int device = 0;
  HAPX_CUDA(cudaGetDevice(&device));
  {
    std::lock_guard<std::mutex> lock(fattn::g_attr_mutex);
    if (!fattn::g_attr[device].bwd_k) {
      HAPX_CUDA(cudaFuncSetAttribute(fattn::attention_backward_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)fattn::kBwdSmem));
      HAPX_CUDA(cudaFuncSetAttribute(fattn::attention_backward_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)fattn::kBwdSmem));
      fattn::g_attr[device].bwd_k = fattn::g_attr[device].bwd_q = true;
    }
  }
  const int grid = std::max(1, std::min(p.units, sms));
  fattn::attention_backward_kernel<true><<<grid, fattn::kBwdThreads, fattn::kBwdSmem, stream>>>(tmQKV, tmDO, p);
  HAPX_CUDA(cudaGetLastError());
  fattn::attention_backward_kernel<false><<<grid, fattn::kBwdThreads, fattn::kBwdSmem, stream>>>(tmQKV, tmDO, p);
  HAPX_CUDA(cudaGetLastError());
  count_launch(2);
  return HAPX_OK;
}

int hapx_attention_dropout_mask(unsigned char* mask, int64_t L, int64_t N, int64_t H, double dropout_p, uint64_t call_id,
                                hapx_stream stream_) {
  if (L < 0 || N < 0 || H < 1) return fail(HAPX_ERR_EXTENT, "attention_dropout_mask: negative extent");
  if (!(dropout_p >= 0.0 && dropout_p < 1.0)) return fail(HAPX_ERR_ARGUMENT, "attention_dropout_mask: dropout_p must be in [0, 1)");
  if (L == 0 || N == 0) return HAPX_OK;
  if (!mask) return fail(HAPX_ERR_ARGUMENT, "attention_dropout_mask: null pointer");
  rng::State* st = nullptr;
  if (int e = rng_state(&st)) return e;
  const long long rows = N * H * L, groups = rows * ((L + 7) / 8);
  const int grid = (int)std::max<long long>(1, std::min<long long>((groups + 255) / 256, 148 * 8));
  fattn::attention_mask_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream_)>>>(mask, (int)L, rows, rng::threshold_for(dropout_p), st, call_id);
  HAPX_CUDA(cudaGetLastError());
  count_launch();
  return HAPX_OK;
}

}  // extern "C"
