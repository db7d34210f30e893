// Counter-based random bits for the dropout kernels (plain dropout and the dropout on the attention
// probabilities): Philox4x32 with 7 rounds, keyed by
//     (seed, iteration counter read from device memory, id of the call site)
// and counted by the index of a group of 8 consecutive elements.  One evaluation yields 128 bits =
// eight 16-bit numbers, one per element; an element is KEPT when its number is >= round(p * 65536).
// Forward and backward kernels evaluate the same function of the same key and index, so a mask is
// never stored; the iteration counter lives in device memory and is advanced by a kernel, so a
// training step replayed from a CUDA graph draws new masks on every replay.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace hapx {
namespace rng {

struct State {                  // in device memory, one per device
  unsigned long long seed;
  unsigned long long epoch;     // iteration counter
};

struct Key { unsigned k0, k1, c2, c3; };

// Key of one call site in the current iteration.
__device__ __forceinline__ Key make_key(const State* st, unsigned long long call_id) {
  const unsigned long long seed = st->seed, epoch = st->epoch;
  Key k;
  k.k0 = (unsigned)seed ^ (unsigned)(call_id * 0x9E3779B97F4A7C15ull >> 32);
  k.k1 = (unsigned)(seed >> 32) ^ (unsigned)call_id;
  k.c2 = (unsigned)epoch;
  k.c3 = (unsigned)(epoch >> 32);
  return k;
}

// 128 random bits for group `idx` (a 64-bit counter).
__device__ __forceinline__ uint4 philox(const Key& key, unsigned long long idx) {
  unsigned c0 = (unsigned)idx, c1 = (unsigned)(idx >> 32), c2 = key.c2, c3 = key.c3;
  unsigned k0 = key.k0, k1 = key.k1;
#pragma unroll
  for (int r = 0; r < 7; ++r) {
    const unsigned hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
    const unsigned hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
    c0 = hi1 ^ c1 ^ k0; c1 = lo1; c2 = hi0 ^ c3 ^ k1; c3 = lo0;
    k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
  }
  return make_uint4(c0, c1, c2, c3);
}

// Bit j of the result: element j (0..7) of the group is kept.
__device__ __forceinline__ unsigned keep_bits(const uint4& r, unsigned threshold) {
  const unsigned w[4] = {r.x, r.y, r.z, r.w};
  unsigned bits = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    bits |= ((w[i] & 0xffffu) >= threshold ? 1u : 0u) << (2 * i);
    bits |= ((w[i] >> 16) >= threshold ? 1u : 0u) << (2 * i + 1);
  }
  return bits;
}

__host__ __device__ inline unsigned threshold_for(double p) {
  const double t = p * 65536.0 + 0.5;
  return t <= 0.0 ? 0u : (t >= 65536.0 ? 65536u : (unsigned)t);
}

}  // namespace rng

// The device's generator state (allocated on first use; that first use must not be inside a stream capture).
int rng_state(rng::State** out);

}  // namespace hapx
