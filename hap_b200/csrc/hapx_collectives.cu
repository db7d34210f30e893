// Uneven collectives as pull kernels over peer-mapped memory (sm_100a).
//
// One kernel family serves every collective of the reference's collectives.py:
// each rank PULLS what it needs straight out of its peers' input buffers (which live
// in, or were staged into, the peer-visible heap) and writes only its own output.
//
//   all_gather / all_to_all / dynamic_slice : pull_copy_kernel   (bit-exact moves)
//   reduce_scatter / all_reduce             : pull_reduce_kernel (fp32 accumulate in
//                                             rank order, fused scale + cast)
//
// Unequal shard extents are pure address arithmetic: no pad bytes are ever moved.
// A source shard is cut into warp tiles laid on the 16-byte grid of the SOURCE
// address, so every remote load is an aligned 16-byte vector; the (local) stores pick
// the widest width the destination alignment allows.
//
// Synchronisation between ranks uses two flag words per peer in the heap's control
// block (st.release.sys / ld.acquire.sys):
//   start[p] = (call number << 40 | offset of p's input inside p's heap)
//   done[p]  = call number, written by p once all of its CTAs have finished reading
// The last CTA of a rank to finish sends `done` to every peer and waits for theirs, so
// a kernel's completion on the stream means nobody reads this rank's input any more.
// Every wait is bounded by a wall-clock limit; on expiry the kernel records an error
// in the control block, skips the data movement and returns.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <algorithm>
#include <map>
#include <mutex>
#include <type_traits>
#include <string>

#include "hapx_internal.h"

namespace hapx {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kCopyUnroll = 4;                      // 16-byte vectors in flight per lane
constexpr int kCopyTile = 32 * 16 * kCopyUnroll;    // bytes of source per warp tile
constexpr int kRedUnroll = 4;
constexpr int kRedTile = 32 * 16 * kRedUnroll;

enum Op { OP_GATHER = 0, OP_EXCHANGE = 1, OP_SLICE = 2, OP_UNSLICE = 3, OP_REDUCE = 4 };

struct LocalRank {
  int rank;
  int pad;
  const char* src;
  char* dst;
  unsigned long long src_off;  // where peers find this rank's input inside its heap
  unsigned long long dst_off;  // all_reduce: where peers may write this rank's output inside its heap (kNoOffset: they may not)
};
constexpr unsigned long long kNoOffset = (1ull << 40) - 1;

struct PullParams {
  int op, world, n_local, es_in, es_out;
  int self_only;    // no peers involved: skip the flag protocol
  int split_first;  // OP_EXCHANGE: split dim comes before cat dim
  int push;         // all_reduce: results may be written straight into the peers' outputs when every output lies in a heap
  int order_log2;   // copy kernels visit tiles in 2^order_log2 interleaved streams (0 = in order)
  unsigned seq;
  unsigned long long timeout_ns;
  unsigned* host_status;  // mapped host word that mirrors a timeout (may be null)
  float scale;
  long long A, B, C;
  long long L1[HAPX_MAX_WORLD], P1[HAPX_MAX_WORLD], tot1;  // sharded / split dim
  long long L2[HAPX_MAX_WORLD], P2[HAPX_MAX_WORLD], tot2;  // cat dim (OP_EXCHANGE)
  char* heap[HAPX_MAX_WORLD];
  LocalRank lr[HAPX_MAX_WORLD];
};

// One source shard as a grid of rows of `run_b` contiguous bytes.
struct Seg {
  int peer;
  unsigned rows_a, rows_j, tiles_per_row, tile_begin, n_tiles;
  long long run_b;                          // bytes per row, in source element size
  long long src_off_b, src_sa_b, src_sj_b;  // source bytes
  long long dst_off_b, dst_sa_b, dst_sj_b;  // destination bytes (destination element size)
  unsigned long long rows64, tiles64;       // unclamped, for host-side range checks
};

// Geometry of what `rank` pulls from `p`.  Shared by host (validation, grid sizing) and
// device (the kernels rebuild it in shared memory, which keeps the launch parameters small).
__host__ __device__ inline void build_seg(const PullParams& P, int rank, int p, int tile_bytes, Seg& s) {
  long long rows_a = 1, rows_j = 1, run = 0, so = 0, ssa = 0, ssj = 0, d_o = 0, dsa = 0, dsj = 0;
  switch (P.op) {
    case OP_GATHER:  // source (A, L1[p], C) contiguous -> destination (A, tot1, C) at P1[p]
      rows_j = P.A; run = P.L1[p] * P.C; ssj = run; d_o = P.P1[p] * P.C; dsj = P.tot1 * P.C;
      break;
    case OP_SLICE:   // source (A, tot1, C) at P1[rank] -> destination (A, L1[rank], C)
    case OP_REDUCE:
      rows_j = P.A; run = P.L1[rank] * P.C; so = P.P1[rank] * P.C; ssj = P.tot1 * P.C; dsj = run;
      break;
    case OP_UNSLICE:
      rows_j = P.A; run = P.L1[rank] * P.C; ssj = run; d_o = P.P1[rank] * P.C; dsj = P.tot1 * P.C;
      break;
    case OP_EXCHANGE: {
      const long long sl = P.L1[rank], cl = P.L2[p];
      if (P.split_first) {  // source (A, tot1, B, cl, C) -> destination (A, sl, B, tot2, C)
        rows_a = P.A; rows_j = sl * P.B; run = cl * P.C;
        so = P.P1[rank] * P.B * cl * P.C; ssa = P.tot1 * P.B * cl * P.C; ssj = cl * P.C;
        d_o = P.P2[p] * P.C; dsa = sl * P.B * P.tot2 * P.C; dsj = P.tot2 * P.C;
      } else {              // source (A, cl, B, tot1, C) -> destination (A, tot2, B, sl, C)
        rows_a = P.A; rows_j = cl * P.B; run = sl * P.C;
        so = P.P1[rank] * P.C; ssa = cl * P.B * P.tot1 * P.C; ssj = P.tot1 * P.C;
        d_o = P.P2[p] * P.B * sl * P.C; dsa = P.tot2 * P.B * sl * P.C; dsj = sl * P.C;
      }
      break;
    }
  }
  if (run == 0 || rows_j == 0 || rows_a == 0) { rows_a = 1; rows_j = 0; run = 0; }
  // rows that follow each other without a gap on both sides are one longer row
  if (rows_j > 1 && ssj == run && dsj == run) { run *= rows_j; rows_j = 1; }
  if (rows_j == 1 && rows_a > 1) { rows_j = rows_a; rows_a = 1; ssj = ssa; dsj = dsa; }
  if (rows_j > 1 && rows_a == 1 && ssj == run && dsj == run) { run *= rows_j; rows_j = 1; }
  s.peer = p;
  s.run_b = run * P.es_in;
  s.src_off_b = so * P.es_in; s.src_sa_b = ssa * P.es_in; s.src_sj_b = ssj * P.es_in;
  s.dst_off_b = d_o * P.es_out; s.dst_sa_b = dsa * P.es_out; s.dst_sj_b = dsj * P.es_out;
  s.rows64 = (unsigned long long)rows_a * (unsigned long long)rows_j;
  const unsigned long long tpr = (rows_j == 0) ? 0ull : (unsigned long long)((s.run_b + 15 + tile_bytes - 1) / tile_bytes);
  s.tiles64 = s.rows64 * tpr;
  s.rows_a = (unsigned)rows_a; s.rows_j = (unsigned)rows_j;
  s.tiles_per_row = (unsigned)tpr;
  s.n_tiles = (unsigned)s.tiles64;
  s.tile_begin = 0;
}

// ---- device helpers ---------------------------------------------------------------
__device__ __forceinline__ void st_release_sys(unsigned long long* p, unsigned long long v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_acquire_sys(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Spin until (*p >> shift) == want; gives up after timeout_ns (or 2^31 polls).
__device__ inline bool wait_flag(const unsigned long long* p, unsigned shift, unsigned want,
                                 unsigned long long timeout_ns, unsigned long long* value) {
  const unsigned long long t0 = global_ns();
  for (unsigned it = 0; it < 0x7fffffffu; ++it) {
    const unsigned long long v = ld_acquire_sys(p);
    if ((unsigned)(v >> shift) == want) { *value = v; return true; }
    if ((it & 31u) == 31u) {
      if (global_ns() - t0 > timeout_ns) return false;
      __nanosleep(40);
    }
  }
  return false;
}

__device__ inline void report_timeout(Ctrl* my, unsigned seq, int peer, unsigned* host_status) {
  if (atomicCAS(&my->status, 0u, (unsigned)(-HAPX_ERR_PEER_TIMEOUT)) == 0u)
    my->status_info = ((unsigned long long)seq << 32) | (unsigned)peer;
  if (host_status) {   // lets the host notice at its next call, without a synchronisation
    *reinterpret_cast<volatile unsigned*>(host_status) = (unsigned)(-HAPX_ERR_PEER_TIMEOUT);
    __threadfence_system();
  }
}

struct Shared {
  Seg segs[HAPX_MAX_WORLD];
  const char* base[HAPX_MAX_WORLD];  // this rank's view of every rank's input
  unsigned total_tiles;
  int nseg;
  int abort;
  int last;
};

// Announce this rank's input to the peers, wait for theirs, build the segment table.
__device__ inline void begin_collective(const PullParams& P, const LocalRank& lr, Shared& sh, int tile_bytes) {
  const int tid = threadIdx.x, rank = lr.rank;
  if (tid == 0) sh.abort = 0;
  __syncthreads();
  if (tid < P.world) {
    const int p = tid;
    unsigned long long off = lr.src_off;
    if (p != rank && !P.self_only) {
      Ctrl* my = reinterpret_cast<Ctrl*>(P.heap[rank]);
      if (blockIdx.x == 0)
        st_release_sys(&reinterpret_cast<Ctrl*>(P.heap[p])->start[rank],
                       ((unsigned long long)P.seq << 40) | lr.src_off);
      unsigned long long v = 0;
      if (wait_flag(&my->start[p], 40, P.seq, P.timeout_ns, &v)) {
        off = v & ((1ull << 40) - 1);
      } else {
        sh.abort = 1;
        report_timeout(my, P.seq, p, P.host_status);
      }
    }
    sh.base[p] = (p == rank && P.self_only) ? lr.src : (P.heap[p] + off);
    const bool one_seg = (P.op == OP_SLICE || P.op == OP_UNSLICE || P.op == OP_REDUCE);
    if (!one_seg || p == 0) build_seg(P, rank, one_seg ? rank : p, tile_bytes, sh.segs[p]);
  }
  __syncthreads();
  if (tid == 0) {
    const bool one_seg = (P.op == OP_SLICE || P.op == OP_UNSLICE || P.op == OP_REDUCE);
    const int n = one_seg ? 1 : P.world;
    unsigned acc = 0;
    for (int i = 0; i < n; ++i) { sh.segs[i].tile_begin = acc; acc += sh.segs[i].n_tiles; }
    sh.nseg = n;
    sh.total_tiles = sh.abort ? 0u : acc;
  }
  __syncthreads();
}

// Tell the peers that this rank has finished reading them; leave only when they have too.
__device__ inline void end_collective(const PullParams& P, const LocalRank& lr, Shared& sh) {
  if (P.self_only) return;
  const int tid = threadIdx.x, rank = lr.rank;
  Ctrl* my = reinterpret_cast<Ctrl*>(P.heap[rank]);
  __syncthreads();
  if (tid == 0) {
    __threadfence();
    sh.last = (atomicAdd(&my->cta_done, 1u) == gridDim.x - 1);
  }
  __syncthreads();
  if (!sh.last) return;
  if (tid < P.world && tid != rank) {
    const int p = tid;
    st_release_sys(&reinterpret_cast<Ctrl*>(P.heap[p])->done[rank], (unsigned long long)P.seq);
    unsigned long long v;
    if (!sh.abort && !wait_flag(&my->done[p], 0, P.seq, P.timeout_ns, &v)) report_timeout(my, P.seq, p, P.host_status);
  }
  __syncthreads();
  if (tid == 0) my->cta_done = 0;
}

__device__ __forceinline__ uint4 ld16(const char* p) { return __ldcg(reinterpret_cast<const uint4*>(p)); }

// Store `n_words` 32-bit words held in registers to d, which is aligned to `es` bytes only.
template <int NW>
__device__ __forceinline__ void store_words(char* d, const unsigned (&w)[NW]) {
  const unsigned mis = (unsigned)(reinterpret_cast<uintptr_t>(d) & 15u);
  if (NW % 4 == 0 && mis == 0) {
#pragma unroll
    for (int i = 0; i < NW / 4; ++i)
      reinterpret_cast<uint4*>(d)[i] = make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]);
  } else if ((mis & 7u) == 0) {
#pragma unroll
    for (int i = 0; i < NW / 2; ++i) reinterpret_cast<uint2*>(d)[i] = make_uint2(w[2 * i], w[2 * i + 1]);
  } else if ((mis & 3u) == 0) {
#pragma unroll
    for (int i = 0; i < NW; ++i) reinterpret_cast<unsigned*>(d)[i] = w[i];
  } else if ((mis & 1u) == 0) {
#pragma unroll
    for (int i = 0; i < NW; ++i) {
      reinterpret_cast<unsigned short*>(d)[2 * i] = (unsigned short)(w[i] & 0xffffu);
      reinterpret_cast<unsigned short*>(d)[2 * i + 1] = (unsigned short)(w[i] >> 16);
    }
  } else {
#pragma unroll
    for (int i = 0; i < NW; ++i) {
#pragma unroll
      for (int b = 0; b < 4; ++b) reinterpret_cast<unsigned char*>(d)[4 * i + b] = (unsigned char)(w[i] >> (8 * b));
    }
  }
}

__device__ inline void copy_elements(const char* s, char* d, long long bytes, int es) {
  for (long long b = 0; b < bytes; b += es) {
    switch (es) {
      case 8: *reinterpret_cast<unsigned long long*>(d + b) = __ldcg(reinterpret_cast<const unsigned long long*>(s + b)); break;
      case 4: *reinterpret_cast<unsigned*>(d + b) = __ldcg(reinterpret_cast<const unsigned*>(s + b)); break;
      case 2: *reinterpret_cast<unsigned short*>(d + b) = __ldcg(reinterpret_cast<const unsigned short*>(s + b)); break;
      default: *reinterpret_cast<unsigned char*>(d + b) = __ldcg(reinterpret_cast<const unsigned char*>(s + b)); break;
    }
  }
}

// Decode a tile id into (segment, byte offsets of its row, chunk index inside the row).
struct TilePos {
  int si;
  long long src_row_b, dst_row_b;  // byte offsets of the row inside source / destination
  unsigned k;
};
__host__ __device__ __forceinline__ TilePos locate(const Seg* segs, int nseg, unsigned t) {
  TilePos tp;
  int si = 0;
  while (si + 1 < nseg && t >= segs[si + 1].tile_begin) ++si;
  const Seg& s = segs[si];
  const unsigned local = t - s.tile_begin;
  const unsigned row = local / s.tiles_per_row;
  tp.k = local - row * s.tiles_per_row;
  unsigned a = 0, j = row;
  if (s.rows_a > 1) { a = row / s.rows_j; j = row - a * s.rows_j; }
  tp.si = si;
  tp.src_row_b = s.src_off_b + (long long)a * s.src_sa_b + (long long)j * s.src_sj_b;
  tp.dst_row_b = s.dst_off_b + (long long)a * s.dst_sa_b + (long long)j * s.dst_sj_b;
  return tp;
}

// ---- bit-exact pull copy ---------------------------------------------------------------
__device__ __forceinline__ void copy_tiles(const PullParams& P, const LocalRank& lr, Shared& sh) {
  const unsigned lane = threadIdx.x & 31u;
  const unsigned gw = blockIdx.x * kWarps + (threadIdx.x >> 5);
  const unsigned nw = gridDim.x * kWarps;
  const unsigned total = sh.total_tiles;
  // Tiles are numbered source after source.  Walking them in that order would make every
  // rank read the same peer at the same time (one NVLink port saturated, the others idle),
  // so the walk is split into G = 2^order_log2 streams that start G equally spaced places
  // apart: at any moment all sources are being read, each in proportion to its size.
  const unsigned lg = (unsigned)P.order_log2;
  const unsigned G = 1u << lg;
  const unsigned Q = (total + G - 1) >> lg;
  const unsigned long long walk = (unsigned long long)Q << lg;
  for (unsigned long long t0 = gw; t0 < walk; t0 += nw) {
    const unsigned t = ((unsigned)t0 & (G - 1)) * Q + (unsigned)(t0 >> lg);
    if (t >= total) continue;
    const TilePos tp = locate(sh.segs, sh.nseg, t);
    const Seg& s = sh.segs[tp.si];
    const char* srow = sh.base[s.peer] + tp.src_row_b;
    char* drow = lr.dst + tp.dst_row_b;
    if (srow == drow) continue;  // shard already in place
    const unsigned mis = (unsigned)(reinterpret_cast<uintptr_t>(srow) & 15u);
    const long long rel0 = (long long)tp.k * kCopyTile - (long long)mis + (long long)lane * 16;
    const long long run_b = s.run_b;
    uint4 v[kCopyUnroll];
    bool full[kCopyUnroll];
#pragma unroll
    for (int u = 0; u < kCopyUnroll; ++u) {
      const long long rel = rel0 + u * 512;
      full[u] = (rel >= 0) && (rel + 16 <= run_b);
      if (full[u]) v[u] = ld16(srow + rel);
    }
#pragma unroll
    for (int u = 0; u < kCopyUnroll; ++u) {
      const long long rel = rel0 + u * 512;
      if (full[u]) {
        const unsigned w[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
        store_words<4>(drow + rel, w);
      } else {
        const long long lo = rel < 0 ? 0 : rel;
        const long long hi = (rel + 16 < run_b) ? rel + 16 : run_b;
        if (lo < hi) copy_elements(srow + lo, drow + lo, hi - lo, P.es_in);
      }
    }
  }
}

__global__ void __launch_bounds__(kThreads) pull_copy_kernel(const __grid_constant__ PullParams P) {
  __shared__ Shared sh;
  const LocalRank& lr = P.lr[blockIdx.y];
  begin_collective(P, lr, sh, kCopyTile);
  copy_tiles(P, lr, sh);
  end_collective(P, lr, sh);
}

// ---- pull + reduce -----------------------------------------------------------------------
template <typename T> struct Num;
template <> struct Num<float> {
  static constexpr int K = 4;  // elements per 16 bytes
  __device__ static __forceinline__ void unpack(const uint4& v, float (&f)[4]) {
    f[0] = __uint_as_float(v.x); f[1] = __uint_as_float(v.y); f[2] = __uint_as_float(v.z); f[3] = __uint_as_float(v.w);
  }
  __device__ static __forceinline__ float load(const char* p) { return __ldcg(reinterpret_cast<const float*>(p)); }
  __device__ static __forceinline__ void store(char* p, float x) { *reinterpret_cast<float*>(p) = x; }
};
template <> struct Num<__nv_bfloat16> {
  static constexpr int K = 8;
  __device__ static __forceinline__ void unpack(const uint4& v, float (&f)[8]) {
    const unsigned w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) { f[2 * i] = __uint_as_float(w[i] << 16); f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u); }
  }
  __device__ static __forceinline__ float load(const char* p) {
    return __uint_as_float((unsigned)__ldcg(reinterpret_cast<const unsigned short*>(p)) << 16);
  }
  __device__ static __forceinline__ void store(char* p, float x) { *reinterpret_cast<__nv_bfloat16*>(p) = __float2bfloat16_rn(x); }
};
template <> struct Num<__half> {
  static constexpr int K = 8;
  __device__ static __forceinline__ void unpack(const uint4& v, float (&f)[8]) {
    const unsigned w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const __half2 h = *reinterpret_cast<const __half2*>(&w[i]);
      const float2 x = __half22float2(h);
      f[2 * i] = x.x; f[2 * i + 1] = x.y;
    }
  }
  __device__ static __forceinline__ float load(const char* p) {
    const unsigned short u = __ldcg(reinterpret_cast<const unsigned short*>(p));
    return __half2float(*reinterpret_cast<const __half*>(&u));
  }
  __device__ static __forceinline__ void store(char* p, float x) { *reinterpret_cast<__half*>(p) = __float2half_rn(x); }
};

template <typename OutT, int K>
__device__ __forceinline__ void store_values(char* d, const float (&f)[K]) {
  if constexpr (sizeof(OutT) == 4) {
    unsigned w[K];
#pragma unroll
    for (int i = 0; i < K; ++i) w[i] = __float_as_uint(f[i]);
    store_words<K>(d, w);
  } else {
    unsigned w[K / 2];
#pragma unroll
    for (int i = 0; i < K / 2; ++i) {
      unsigned short lo, hi;
      if constexpr (std::is_same<OutT, __nv_bfloat16>::value) {
        lo = __bfloat16_as_ushort(__float2bfloat16_rn(f[2 * i]));
        hi = __bfloat16_as_ushort(__float2bfloat16_rn(f[2 * i + 1]));
      } else {
        lo = __half_as_ushort(__float2half_rn(f[2 * i]));
        hi = __half_as_ushort(__float2half_rn(f[2 * i + 1]));
      }
      w[i] = (unsigned)lo | ((unsigned)hi << 16);
    }
    store_words<K / 2>(d, w);
  }
}

// PUSH: the sums go to every rank's output (`push_dst[q]` + the slice's place in the whole tensor) instead of
// this rank's compact slice buffer.
template <typename InT, typename OutT, bool PUSH = false>
__device__ __forceinline__ void reduce_tiles(const PullParams& P, const LocalRank& lr, Shared& sh, char* const* push_dst = nullptr,
                                             long long push_off_b = 0) {
  constexpr int K = Num<InT>::K;
  const unsigned lane = threadIdx.x & 31u;
  const unsigned gw = blockIdx.x * kWarps + (threadIdx.x >> 5);
  const unsigned nw = gridDim.x * kWarps;
  const unsigned total = sh.total_tiles;
  const int W = P.world;
  const float scale = P.scale;
  for (unsigned t = gw; t < total; t += nw) {
    const TilePos tp = locate(sh.segs, sh.nseg, t);
    const Seg& s = sh.segs[0];
    char* drow = lr.dst + tp.dst_row_b;
    // every rank's input starts on a 16-byte boundary (the host stages it otherwise), so
    // the row has the same misalignment in all of them
    const unsigned mis = (unsigned)(tp.src_row_b & 15);
    const long long rel0 = (long long)tp.k * kRedTile - (long long)mis + (long long)lane * 16;
    const long long run_b = s.run_b;
    float acc[kRedUnroll][K];
    bool full[kRedUnroll];
#pragma unroll
    for (int u = 0; u < kRedUnroll; ++u) {
      const long long rel = rel0 + u * 512;
      full[u] = (rel >= 0) && (rel + 16 <= run_b);
    }
    for (int p = 0; p < W; p += 2) {
      const char* b0 = sh.base[p] + tp.src_row_b + rel0;
      const bool two = (p + 1 < W);
      const char* b1 = two ? sh.base[p + 1] + tp.src_row_b + rel0 : b0;
      uint4 x[kRedUnroll], y[kRedUnroll];
#pragma unroll
      for (int u = 0; u < kRedUnroll; ++u) if (full[u]) x[u] = ld16(b0 + u * 512);
      if (two) {
#pragma unroll
        for (int u = 0; u < kRedUnroll; ++u) if (full[u]) y[u] = ld16(b1 + u * 512);
      }
#pragma unroll
      for (int u = 0; u < kRedUnroll; ++u) {
        if (!full[u]) continue;
        float f[K];
        Num<InT>::unpack(x[u], f);
        if (p == 0) {
#pragma unroll
          for (int i = 0; i < K; ++i) acc[u][i] = f[i];
        } else {
#pragma unroll
          for (int i = 0; i < K; ++i) acc[u][i] += f[i];
        }
        if (two) {
          Num<InT>::unpack(y[u], f);
#pragma unroll
          for (int i = 0; i < K; ++i) acc[u][i] += f[i];
        }
      }
    }
#pragma unroll
    for (int u = 0; u < kRedUnroll; ++u) {
      const long long rel = rel0 + u * 512;
      if (full[u]) {
#pragma unroll
        for (int i = 0; i < K; ++i) acc[u][i] *= scale;
        const long long out_b = (rel / (long long)sizeof(InT)) * (long long)sizeof(OutT);
        if constexpr (PUSH) {
          for (int q = 0; q < W; ++q) store_values<OutT, K>(push_dst[q] + push_off_b + tp.dst_row_b + out_b, acc[u]);
        } else {
          store_values<OutT, K>(drow + out_b, acc[u]);
        }
      } else {
        const long long lo = rel < 0 ? 0 : rel;
        const long long hi = (rel + 16 < run_b) ? rel + 16 : run_b;
        for (long long b = lo; b < hi; b += (long long)sizeof(InT)) {
          float a = 0.f;
          for (int p = 0; p < W; ++p) {
            const float x = Num<InT>::load(sh.base[p] + tp.src_row_b + b);
            a = (p == 0) ? x : a + x;
          }
          const long long out_b = (b / (long long)sizeof(InT)) * (long long)sizeof(OutT);
          if constexpr (PUSH) {
            for (int q = 0; q < W; ++q) Num<OutT>::store(push_dst[q] + push_off_b + tp.dst_row_b + out_b, a * scale);
          } else {
            Num<OutT>::store(drow + out_b, a * scale);
          }
        }
      }
    }
  }
}

template <typename InT, typename OutT>
__global__ void __launch_bounds__(kThreads) pull_reduce_kernel(const __grid_constant__ PullParams P) {
  __shared__ Shared sh;
  const LocalRank& lr = P.lr[blockIdx.y];
  begin_collective(P, lr, sh, kRedTile);
  reduce_tiles<InT, OutT>(P, lr, sh);
  end_collective(P, lr, sh);
}

// ---- all_reduce in one launch -----------------------------------------------------------------
// R: the reduce of an even split (rank r sums slice r of every input into a peer-visible buffer `mid` at
// the same heap offset on every rank); G: the gather of the reduced slices.  Between the two, the CTA that
// finishes a rank's reduce last tells every peer that the slice is complete; a rank gathers once all slices
// are.  Because a peer announces its slice only after it has read every input, the gather may write into the
// buffer the input came from (in-place all_reduce).
template <typename InT, typename OutT>
__global__ void __launch_bounds__(kThreads) pull_allreduce_kernel(const __grid_constant__ PullParams R, const __grid_constant__ PullParams G) {
  __shared__ Shared sh;
  __shared__ char* push_dst[HAPX_MAX_WORLD];
  __shared__ int push_ok;
  const LocalRank& lr = R.lr[blockIdx.y];
  const int tid = threadIdx.x, rank = lr.rank;
  Ctrl* my = reinterpret_cast<Ctrl*>(R.heap[rank]);
  begin_collective(R, lr, sh, kRedTile);
  if (R.push) {
    // Every rank tells the others where its OUTPUT lies in its heap (or that it does not).  If all outputs are
    // reachable, the owner of a slice writes its sums straight into every output: each byte crosses the links
    // once per direction (read as input, written as result), there is no intermediate slice and no second phase.
    if (tid == 0) push_ok = 1;
    __syncthreads();
    if (tid < R.world) {
      const int p = tid;
      unsigned long long off = lr.dst_off;
      if (p != rank) {
        if (blockIdx.x == 0)
          st_release_sys(&reinterpret_cast<Ctrl*>(R.heap[p])->dst_start[rank], ((unsigned long long)R.seq << 40) | lr.dst_off);
        unsigned long long v = 0;
        if (!sh.abort && wait_flag(&my->dst_start[p], 40, R.seq, R.timeout_ns, &v)) {
          off = v & kNoOffset;
        } else if (!sh.abort) {
          sh.abort = 1;
          report_timeout(my, R.seq, p, R.host_status);
        }
      }
      if (off == kNoOffset) push_ok = 0;
      push_dst[p] = R.heap[p] + off;
    }
    __syncthreads();
    if (tid == 0 && sh.abort) sh.total_tiles = 0;
    __syncthreads();
    if (push_ok) {
      reduce_tiles<InT, OutT, true>(R, lr, sh, push_dst, R.P1[rank] * R.C * (long long)sizeof(OutT));
      __threadfence_system();                      // this thread's writes into the peers before the CTA is counted
      __syncthreads();
      if (tid == 0) sh.last = (atomicAdd(&my->cta_phase, 1u) == gridDim.x - 1);
      __syncthreads();
      if (!sh.last) return;
      // the slice is complete in every output, and every input of it has been read: tell everybody (and wait for
      // their slices: then this rank's output is whole and nobody reads its input any more)
      if (tid == 0) { __threadfence_system(); my->cta_phase = 0; }
      __syncthreads();
      if (tid < R.world) {
        st_release_sys(&reinterpret_cast<Ctrl*>(R.heap[tid])->ready[rank], (unsigned long long)R.seq);
        unsigned long long v;
        if (!sh.abort && !wait_flag(&my->ready[tid], 0, R.seq, R.timeout_ns, &v)) report_timeout(my, R.seq, tid, R.host_status);
      }
      return;
    }
  }
  reduce_tiles<InT, OutT>(R, lr, sh);
  // publish this rank's slice when its last CTA has finished reducing
  __syncthreads();
  if (tid == 0) {
    __threadfence_system();
    sh.last = (atomicAdd(&my->cta_phase, 1u) == gridDim.x - 1);
  }
  __syncthreads();
  if (sh.last) {
    if (tid < R.world) st_release_sys(&reinterpret_cast<Ctrl*>(R.heap[tid])->ready[rank], (unsigned long long)R.seq);
    if (tid == 0) my->cta_phase = 0;
  }
  // wait for every rank's slice, then rebuild the segment table for the gather
  if (tid < R.world) {
    unsigned long long v;
    if (!sh.abort && !wait_flag(&my->ready[tid], 0, R.seq, R.timeout_ns, &v)) {
      sh.abort = 1;
      report_timeout(my, R.seq, tid, R.host_status);
    }
    sh.base[tid] = G.heap[tid] + G.lr[blockIdx.y].src_off;
    build_seg(G, rank, tid, kCopyTile, sh.segs[tid]);
  }
  __syncthreads();
  if (tid == 0) {
    unsigned acc = 0;
    for (int i = 0; i < G.world; ++i) { sh.segs[i].tile_begin = acc; acc += sh.segs[i].n_tiles; }
    sh.nseg = G.world;
    sh.total_tiles = sh.abort ? 0u : acc;
  }
  __syncthreads();
  copy_tiles(G, G.lr[blockIdx.y], sh);
  end_collective(R, lr, sh);
}

// ---- local helper: copy an input into the staging area ------------------------------------
__global__ void __launch_bounds__(kThreads) stage_copy_kernel(char* __restrict__ dst, const char* __restrict__ src, long long bytes) {
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long nth = (long long)gridDim.x * blockDim.x;
  if (((reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(src)) & 15u) == 0) {
    const long long nv = bytes >> 4;
    for (long long i = tid; i < nv; i += nth) reinterpret_cast<uint4*>(dst)[i] = __ldcs(reinterpret_cast<const uint4*>(src) + i);
    for (long long b = (nv << 4) + tid; b < bytes; b += nth) dst[b] = src[b];
  } else {
    for (long long b = tid; b < bytes; b += nth) dst[b] = src[b];
  }
}

// ---- host side -------------------------------------------------------------------------------
typedef void (*PullKernel)(const PullParams);

static PullKernel reduce_kernel_for(int in_dtype, int out_dtype) {
#define HAPX_PICK(IN, INT)                                                          \
  if (in_dtype == IN) {                                                             \
    if (out_dtype == HAPX_F32) return pull_reduce_kernel<INT, float>;               \
    if (out_dtype == HAPX_BF16) return pull_reduce_kernel<INT, __nv_bfloat16>;      \
    if (out_dtype == HAPX_F16) return pull_reduce_kernel<INT, __half>;              \
  }
  HAPX_PICK(HAPX_F32, float)
  HAPX_PICK(HAPX_BF16, __nv_bfloat16)
  HAPX_PICK(HAPX_F16, __half)
#undef HAPX_PICK
  return nullptr;
}

typedef void (*AllReduceKernel)(const PullParams, const PullParams);

static AllReduceKernel allreduce_kernel_for(int in_dtype, int out_dtype) {
#define HAPX_PICK(IN, INT)                                                             \
  if (in_dtype == IN) {                                                                \
    if (out_dtype == HAPX_F32) return pull_allreduce_kernel<INT, float>;               \
    if (out_dtype == HAPX_BF16) return pull_allreduce_kernel<INT, __nv_bfloat16>;      \
    if (out_dtype == HAPX_F16) return pull_allreduce_kernel<INT, __half>;              \
  }
  HAPX_PICK(HAPX_F32, float)
  HAPX_PICK(HAPX_BF16, __nv_bfloat16)
  HAPX_PICK(HAPX_F16, __half)
#undef HAPX_PICK
  return nullptr;
}

static unsigned next_seq(hapx_comm* c) {
  ++c->calls;
  c->seq = (c->seq + 1) & 0xffffffu;
  if (c->seq == 0) c->seq = 1;
  return c->seq;
}

static int check_ready(hapx_comm* c) {
  if (!c) return fail(HAPX_ERR_ARGUMENT, "null communicator");
  // a kernel of an earlier call whose wait on a peer ran out has left its outputs unwritten: refuse
  // further work until hapx_comm_check() has reported and cleared it (no synchronisation needed here)
  if (c->host_status && *static_cast<volatile unsigned*>(c->host_status) != 0u)
    return fail(HAPX_ERR_PEER_TIMEOUT, "an earlier collective of this communicator gave up waiting for a peer; its outputs are not valid "
                                       "(hapx_comm_check reports the details and clears the error)");
  for (int p = 0; p < c->world; ++p)
    if (!c->mapped[p]) return fail(HAPX_ERR_STATE, "peer heap of rank " + std::to_string(p) + " is not mapped (call hapx_comm_open_peers)");
  return HAPX_OK;
}

static void fill_prefix(const int64_t* lengths, int world, long long* L, long long* Pfx, long long* total) {
  long long acc = 0;
  for (int i = 0; i < HAPX_MAX_WORLD; ++i) {
    L[i] = (i < world) ? lengths[i] : 0;
    Pfx[i] = acc;
    acc += L[i];
  }
  *total = acc;
}

// Make local rank i's input visible to the peers: use it in place when it already lies in
// the heap (and is aligned as required), otherwise copy it to the staging area at `stage_pos`.
static int publish_input(hapx_comm* c, int i, const void* src, size_t bytes, bool need_16B, size_t stage_pos,
                         cudaStream_t stream, unsigned long long* off_out) {
  const int r = c->first_rank + i;
  const char* lo = c->heap[r] + kCtrlBytes;
  const char* hi = c->heap[r] + c->heap_bytes;
  const char* s = static_cast<const char*>(src);
  if (bytes == 0) { *off_out = kCtrlBytes; return HAPX_OK; }
  if (!src) return fail(HAPX_ERR_ARGUMENT, "null input pointer");
  if (s >= lo && s + bytes <= hi && (!need_16B || (reinterpret_cast<uintptr_t>(s) & 15u) == 0)) {
    *off_out = (unsigned long long)(s - c->heap[r]);
    return HAPX_OK;
  }
  if (stage_pos + bytes > c->stage_bytes)
    return fail(HAPX_ERR_STAGING, "input of " + std::to_string(bytes) + " bytes is outside the peer-visible heap and the staging area holds only " +
                                      std::to_string(c->stage_bytes) + " bytes (raise stage_bytes or allocate the tensor in the heap)");
  char* d = c->heap[r] + kCtrlBytes + stage_pos;
  const long long vecs = (long long)((bytes + 15) / 16);
  int grid = (int)std::min<long long>((vecs + kThreads - 1) / kThreads, (long long)c->sm_count * 8);
  if (grid < 1) grid = 1;
  stage_copy_kernel<<<grid, kThreads, 0, stream>>>(d, s, (long long)bytes);
  HAPX_CUDA(cudaGetLastError());
  count_launch();
  *off_out = kCtrlBytes + stage_pos;
  return HAPX_OK;
}

static int launch_pull(hapx_comm* c, PullKernel kernel, PullParams& P, int tile_bytes, cudaStream_t stream) {
  // validate ranges with the same geometry code the device uses; size the grid
  unsigned long long max_tiles = 0;
  const bool one_seg = (P.op == OP_SLICE || P.op == OP_UNSLICE || P.op == OP_REDUCE);
  for (int i = 0; i < P.n_local; ++i) {
    unsigned long long tiles = 0;
    for (int p = 0; p < (one_seg ? 1 : P.world); ++p) {
      Seg s;
      build_seg(P, P.lr[i].rank, one_seg ? P.lr[i].rank : p, tile_bytes, s);
      if (s.rows64 >= (1ull << 32) || s.tiles64 >= (1ull << 32)) return fail(HAPX_ERR_EXTENT, "tensor too large for 32-bit tile indices");
      tiles += s.tiles64;
    }
    if (tiles >= (1ull << 32)) return fail(HAPX_ERR_EXTENT, "tensor too large for 32-bit tile indices");
    max_tiles = std::max(max_tiles, tiles);
  }
  int per_sm = 0;
  {  // the occupancy query costs microseconds: ask once per kernel
    static std::mutex mu;
    static std::map<const void*, int> cache;
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(reinterpret_cast<const void*>(kernel));
    if (it == cache.end()) {
      HAPX_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kThreads, 0));
      cache[reinterpret_cast<const void*>(kernel)] = per_sm;
    } else {
      per_sm = it->second;
    }
  }
  if (per_sm < 1) return fail(HAPX_ERR_CUDA, "kernel does not fit on an SM");
  long long cap = (long long)c->sm_count * per_sm;
  if (c->local_mode && !P.self_only) cap = std::max<long long>(1, cap / c->world);
  if (c->max_ctas > 0) cap = std::min<long long>(cap, c->max_ctas);
  long long need = (long long)((max_tiles + kWarps - 1) / kWarps);
  int grid_x = (int)std::max<long long>(1, std::min(need, cap));
  dim3 grid(grid_x, P.n_local), block(kThreads);
  if (c->local_mode && !P.self_only && P.n_local > 1) {
    void* args[] = {&P};
    HAPX_CUDA(cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(kernel), grid, block, args, 0, stream));
  } else {
    kernel<<<grid, block, 0, stream>>>(P);
    HAPX_CUDA(cudaGetLastError());
  }
  count_launch();
  return HAPX_OK;
}

static int count_tiles(const PullParams& P, int tile_bytes, unsigned long long* max_tiles) {
  const bool one_seg = (P.op == OP_SLICE || P.op == OP_UNSLICE || P.op == OP_REDUCE);
  for (int i = 0; i < P.n_local; ++i) {
    unsigned long long tiles = 0;
    for (int p = 0; p < (one_seg ? 1 : P.world); ++p) {
      Seg s;
      build_seg(P, P.lr[i].rank, one_seg ? P.lr[i].rank : p, tile_bytes, s);
      if (s.rows64 >= (1ull << 32) || s.tiles64 >= (1ull << 32)) return fail(HAPX_ERR_EXTENT, "tensor too large for 32-bit tile indices");
      tiles += s.tiles64;
    }
    if (tiles >= (1ull << 32)) return fail(HAPX_ERR_EXTENT, "tensor too large for 32-bit tile indices");
    *max_tiles = std::max(*max_tiles, tiles);
  }
  return HAPX_OK;
}

// Launch of the fused all_reduce: one wave of CTAs (they wait on each other's ranks in the middle of the kernel).
static int launch_allreduce(hapx_comm* c, AllReduceKernel kernel, PullParams& R, PullParams& G, cudaStream_t stream) {
  unsigned long long max_tiles = 0;
  if (int e = count_tiles(R, kRedTile, &max_tiles)) return e;
  if (int e = count_tiles(G, kCopyTile, &max_tiles)) return e;
  int per_sm = 0;
  {
    static std::mutex mu;
    static std::map<const void*, int> cache;
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(reinterpret_cast<const void*>(kernel));
    if (it == cache.end()) {
      HAPX_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kThreads, 0));
      cache[reinterpret_cast<const void*>(kernel)] = per_sm;
    } else {
      per_sm = it->second;
    }
  }
  if (per_sm < 1) return fail(HAPX_ERR_CUDA, "kernel does not fit on an SM");
  long long cap = (long long)c->sm_count * per_sm;
  if (c->local_mode) cap = std::max<long long>(1, cap / c->world);
  if (c->max_ctas > 0) cap = std::min<long long>(cap, c->max_ctas);
  const long long need = (long long)((max_tiles + kWarps - 1) / kWarps);
  const int grid_x = (int)std::max<long long>(1, std::min(need, cap));
  dim3 grid(grid_x, R.n_local), block(kThreads);
  if (c->local_mode && R.n_local > 1) {
    void* args[] = {&R, &G};
    HAPX_CUDA(cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(kernel), grid, block, args, 0, stream));
  } else {
    kernel<<<grid, block, 0, stream>>>(R, G);
    HAPX_CUDA(cudaGetLastError());
  }
  count_launch();
  return HAPX_OK;
}

struct CallScope {  // orders calls issued on different streams; one collective in flight per communicator
  hapx_comm* c;
  cudaStream_t stream;
  int enter() {
    HAPX_CUDA(cudaSetDevice(c->device));
    if (!c->stream_ordering) return HAPX_OK;
    if (c->any_launched && c->last_stream != stream) HAPX_CUDA(cudaStreamWaitEvent(stream, c->last_done, 0));
    return HAPX_OK;
  }
  int leave() {
    if (!c->stream_ordering) return HAPX_OK;
    HAPX_CUDA(cudaEventRecord(c->last_done, stream));
    c->last_stream = stream;
    c->any_launched = true;
    return HAPX_OK;
  }
};

static void init_params(hapx_comm* c, PullParams& P, int op, int es_in, int es_out) {
  P = PullParams();
  P.op = op; P.world = c->world; P.n_local = c->n_local; P.es_in = es_in; P.es_out = es_out;
  P.scale = 1.f;
  P.timeout_ns = (unsigned long long)c->timeout_ms * 1000000ull;
  P.host_status = c->host_status_dev;
  P.order_log2 = c->order_log2;
  for (int p = 0; p < c->world; ++p) P.heap[p] = c->heap[p];
}

static int gather_impl(hapx_comm* c, void* const* dst, const void* const* src, int es, long long outer, long long inner,
                       const int64_t* lengths, cudaStream_t stream) {
  PullParams P;
  init_params(c, P, OP_GATHER, es, es);
  P.A = outer; P.C = inner;
  fill_prefix(lengths, c->world, P.L1, P.P1, &P.tot1);
  if (P.A * P.tot1 * P.C == 0) return HAPX_OK;
  CallScope scope{c, stream};
  if (int e = scope.enter()) return e;
  for (int i = 0; i < c->n_local; ++i) {
    const int r = c->first_rank + i;
    P.lr[i].rank = r;
    P.lr[i].src = static_cast<const char*>(src[i]);
    P.lr[i].dst = static_cast<char*>(dst[i]);
    if (!dst[i]) return fail(HAPX_ERR_ARGUMENT, "null output pointer");
    const size_t bytes = (size_t)(outer * P.L1[r] * inner) * es;
    if (c->world == 1) { P.self_only = 1; continue; }     // a world of one: a local copy, nothing to publish
    if (int e = publish_input(c, i, src[i], bytes, false, 0, stream, &P.lr[i].src_off)) return e;
  }
  P.seq = next_seq(c);
  if (int e = launch_pull(c, pull_copy_kernel, P, kCopyTile, stream)) return e;
  return scope.leave();
}

static int reduce_impl(hapx_comm* c, void* const* dst, const void* const* src, int in_dtype, int out_dtype, double scale,
                       long long outer, long long inner, const long long* L, const long long* Pfx, long long total,
                       size_t stage_pos, cudaStream_t stream) {
  PullKernel kernel = reduce_kernel_for(in_dtype, out_dtype);
  if (!kernel) return fail(HAPX_ERR_DTYPE, "reductions support float32, bfloat16 and float16");
  PullParams P;
  init_params(c, P, OP_REDUCE, dtype_size(in_dtype), dtype_size(out_dtype));
  P.A = outer; P.C = inner; P.scale = (float)scale;
  for (int i = 0; i < HAPX_MAX_WORLD; ++i) { P.L1[i] = L[i]; P.P1[i] = Pfx[i]; }
  P.tot1 = total;
  if (P.A * P.tot1 * P.C == 0) return HAPX_OK;
  CallScope scope{c, stream};
  if (int e = scope.enter()) return e;
  for (int i = 0; i < c->n_local; ++i) {
    const int r = c->first_rank + i;
    P.lr[i].rank = r;
    P.lr[i].src = static_cast<const char*>(src[i]);
    P.lr[i].dst = static_cast<char*>(dst[i]);
    if (!dst[i] && L[r] > 0) return fail(HAPX_ERR_ARGUMENT, "null output pointer");
    const size_t bytes = (size_t)(outer * total * inner) * P.es_in;
    // a world of one reads its own input in place (the reduce kernel assumes 16-byte aligned inputs)
    if (c->world == 1 && (reinterpret_cast<uintptr_t>(src[i]) & 15u) == 0 && src[i] != dst[i]) { P.self_only = 1; continue; }
    if (int e = publish_input(c, i, src[i], bytes, true, stage_pos, stream, &P.lr[i].src_off)) return e;
  }
  P.seq = next_seq(c);
  if (int e = launch_pull(c, kernel, P, kRedTile, stream)) return e;
  return scope.leave();
}

static int check_lengths(const int64_t* lengths, int world, const char* what) {
  if (!lengths) return fail(HAPX_ERR_ARGUMENT, std::string(what) + ": null sharding lengths");
  for (int i = 0; i < world; ++i)
    if (lengths[i] < 0) return fail(HAPX_ERR_EXTENT, std::string(what) + ": negative sharding length");
  return HAPX_OK;
}

}  // namespace hapx

using namespace hapx;

extern "C" {

int hapx_all_gather(hapx_comm* c, void* const* dst, const void* const* src, int dtype, int64_t outer, int64_t inner,
                    const int64_t* lengths, int mode, hapx_stream stream) {
  if (int e = check_ready(c)) return e;
  if (!dst || !src) return fail(HAPX_ERR_ARGUMENT, "all_gather: null pointer array");
  if (mode != HAPX_MODE_PADDING && mode != HAPX_MODE_GROUP_CALL) return fail(HAPX_ERR_ARGUMENT, "all_gather: unknown mode");
  const int es = dtype_size(dtype);
  if (!es) return fail(HAPX_ERR_DTYPE, "all_gather: unknown dtype");
  if (outer < 0 || inner < 0) return fail(HAPX_ERR_EXTENT, "all_gather: negative extent");
  if (int e = check_lengths(lengths, c->world, "all_gather")) return e;
  return gather_impl(c, dst, src, es, outer, inner, lengths, static_cast<cudaStream_t>(stream));
}

int hapx_reduce_scatter(hapx_comm* c, void* const* dst, const void* const* src, int in_dtype, int out_dtype, double scale,
                        int64_t outer, int64_t inner, const int64_t* lengths, int mode, hapx_stream stream) {
  if (int e = check_ready(c)) return e;
  if (!dst || !src) return fail(HAPX_ERR_ARGUMENT, "reduce_scatter: null pointer array");
  if (mode != HAPX_MODE_PADDING && mode != HAPX_MODE_GROUP_CALL) return fail(HAPX_ERR_ARGUMENT, "reduce_scatter: unknown mode");
  if (outer < 0 || inner < 0) return fail(HAPX_ERR_EXTENT, "reduce_scatter: negative extent");
  if (int e = check_lengths(lengths, c->world, "reduce_scatter")) return e;
  long long L[HAPX_MAX_WORLD], Pfx[HAPX_MAX_WORLD], total;
  fill_prefix(lengths, c->world, L, Pfx, &total);
  return reduce_impl(c, dst, src, in_dtype, out_dtype, scale, outer, inner, L, Pfx, total, 0, static_cast<cudaStream_t>(stream));
}

int hapx_all_reduce(hapx_comm* c, void* const* dst, const void* const* src, int in_dtype, int out_dtype, double scale,
                    int64_t n, hapx_stream stream_) {
  if (int e = check_ready(c)) return e;
  if (!dst || !src) return fail(HAPX_ERR_ARGUMENT, "all_reduce: null pointer array");
  if (n < 0) return fail(HAPX_ERR_EXTENT, "all_reduce: negative size");
  if (n == 0) return HAPX_OK;
  if (!reduce_kernel_for(in_dtype, out_dtype)) return fail(HAPX_ERR_DTYPE, "reductions support float32, bfloat16 and float16");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const int W = c->world;
  const int es_in = dtype_size(in_dtype), es_out = dtype_size(out_dtype);
  const size_t in_bytes = (size_t)n * es_in;
  for (int i = 0; i < c->n_local; ++i)
    if (dst[i] == src[i] && es_in != es_out) return fail(HAPX_ERR_ARGUMENT, "all_reduce: in-place needs equal dtypes");

  // Small tensors: one shot, every rank sums all inputs itself (one kernel, latency bound).
  // The input is always staged so that an in-place call cannot overwrite what peers still read.
  const size_t one_shot_limit = 256 * 1024;
  if (in_bytes <= one_shot_limit || W == 1) {
    long long L[HAPX_MAX_WORLD], Pfx[HAPX_MAX_WORLD];
    for (int i = 0; i < HAPX_MAX_WORLD; ++i) { L[i] = (i < W) ? n : 0; Pfx[i] = 0; }
    bool alias_in_heap = false;
    for (int i = 0; i < c->n_local; ++i) {
      const char* s = static_cast<const char*>(src[i]);
      const int r = c->first_rank + i;
      if (dst[i] == src[i] && s >= c->heap[r] && s < c->heap[r] + c->heap_bytes) alias_in_heap = true;
    }
    if (alias_in_heap && W > 1) {
      // stage explicitly: publish_input would use the heap-resident buffer in place
      if (in_bytes > c->stage_bytes) return fail(HAPX_ERR_STAGING, "all_reduce: staging area too small");
      const void* staged[HAPX_MAX_WORLD];
      for (int i = 0; i < c->n_local; ++i) {
        char* d = c->heap[c->first_rank + i] + kCtrlBytes;
        HAPX_CUDA(cudaSetDevice(c->device));
        const long long vecs = (long long)((in_bytes + 15) / 16);
        int grid = (int)std::max<long long>(1, std::min<long long>((vecs + kThreads - 1) / kThreads, (long long)c->sm_count * 8));
        if (c->stream_ordering && c->any_launched && c->last_stream != stream) HAPX_CUDA(cudaStreamWaitEvent(stream, c->last_done, 0));
        stage_copy_kernel<<<grid, kThreads, 0, stream>>>(d, static_cast<const char*>(src[i]), (long long)in_bytes);
        HAPX_CUDA(cudaGetLastError());
        count_launch();
        staged[i] = d;
      }
      return reduce_impl(c, dst, staged, in_dtype, out_dtype, scale, 1, 1, L, Pfx, n, 0, stream);
    }
    return reduce_impl(c, dst, src, in_dtype, out_dtype, scale, 1, 1, L, Pfx, n, 0, stream);
  }

  // Two shots: uneven-collective machinery on an even split.  Rank r sums slice r of every
  // input into a peer-visible buffer at the end of its staging area, then everybody gathers.
  const long long vec = 16 / es_in;                                    // keep slices on 16-byte boundaries
  const long long per = ((n + W - 1) / W + vec - 1) / vec * vec;
  int64_t lengths[HAPX_MAX_WORLD];
  long long L[HAPX_MAX_WORLD], Pfx[HAPX_MAX_WORLD], total;
  long long left = n;
  for (int r = 0; r < W; ++r) { lengths[r] = std::min(per, left); left -= lengths[r]; }
  fill_prefix(lengths, W, L, Pfx, &total);
  const size_t mid_bytes = ((size_t)per * es_out + 255) / 256 * 256;
  if (mid_bytes > c->stage_bytes) return fail(HAPX_ERR_STAGING, "all_reduce: staging area too small for the reduced slice");
  const size_t mid_pos = c->stage_bytes - mid_bytes;
  void* mid[HAPX_MAX_WORLD];
  for (int i = 0; i < c->n_local; ++i) {
    mid[i] = c->heap[c->first_rank + i] + kCtrlBytes + mid_pos;
    // a staged input must not run into the reduced slice
    const char* s = static_cast<const char*>(src[i]);
    const int r = c->first_rank + i;
    const bool in_heap = s >= c->heap[r] + kCtrlBytes && s + in_bytes <= c->heap[r] + c->heap_bytes && ((uintptr_t)s & 15u) == 0;
    if (!in_heap && in_bytes > mid_pos)
      return fail(HAPX_ERR_STAGING, "all_reduce: input of " + std::to_string(in_bytes) + " bytes is outside the peer-visible heap and does not fit the staging area");
  }
  if (c->fused_all_reduce == 0 || (c->fused_all_reduce < 0 && c->local_mode)) {
    // single-device emulation: all virtual ranks share the GPU, so there is no launch or flag latency to save and the
    // two phases run best as two launches, each with its own grid
    const void* mid_c[HAPX_MAX_WORLD];
    for (int i = 0; i < c->n_local; ++i) mid_c[i] = mid[i];
    if (int e = reduce_impl(c, mid, src, in_dtype, out_dtype, scale, 1, 1, L, Pfx, total, 0, stream)) return e;
    return gather_impl(c, dst, mid_c, es_out, 1, 1, lengths, stream);
  }
  // one launch: reduce the own slice into `mid`, announce it, gather every rank's slice
  AllReduceKernel kernel = allreduce_kernel_for(in_dtype, out_dtype);
  PullParams R, G;
  init_params(c, R, OP_REDUCE, es_in, es_out);
  R.A = 1; R.C = 1; R.scale = (float)scale;
  for (int i = 0; i < HAPX_MAX_WORLD; ++i) { R.L1[i] = L[i]; R.P1[i] = Pfx[i]; }
  R.tot1 = total;
  init_params(c, G, OP_GATHER, es_out, es_out);
  G.A = 1; G.C = 1;
  fill_prefix(lengths, W, G.L1, G.P1, &G.tot1);
  CallScope scope{c, stream};
  if (int e = scope.enter()) return e;
  for (int i = 0; i < c->n_local; ++i) {
    const int r = c->first_rank + i;
    R.lr[i].rank = r;
    R.lr[i].src = static_cast<const char*>(src[i]);
    R.lr[i].dst = static_cast<char*>(mid[i]);
    if (!dst[i]) return fail(HAPX_ERR_ARGUMENT, "null output pointer");
    if (int e = publish_input(c, i, src[i], in_bytes, true, 0, stream, &R.lr[i].src_off)) return e;
    G.lr[i].rank = r;
    G.lr[i].src = static_cast<const char*>(mid[i]);
    G.lr[i].dst = static_cast<char*>(dst[i]);
    G.lr[i].src_off = kCtrlBytes + mid_pos;
  }
  // Outputs that lie in the peer-visible heap can be written by the slice owners directly; whether all of them
  // do is settled between the ranks inside the kernel (a rank only knows its own).
  R.push = (c->fused_all_reduce == 2 || c->fused_all_reduce < 0) && (in_bytes % 16 == 0) && (((size_t)n * es_out) % 16 == 0);
  // Measured on 8 GPUs: writing into seven peers at once wins up to 64 MiB (1.1 - 2.1 x NCCL) and loses above 128 MiB
  // (1 GiB: 3.14 ms against 3.00 ms for reduce + gather); on 2 and 4 GPUs it is never slower.  Unless forced, wide
  // communicators therefore keep reduce + gather for the largest tensors (a rule of n and W only: every rank agrees).
  if (c->fused_all_reduce < 0 && W > 4 && in_bytes > ((size_t)128 << 20)) R.push = 0;
  for (int i = 0; i < c->n_local; ++i) {
    const int r = c->first_rank + i;
    const char* d = static_cast<const char*>(dst[i]);
    const bool reachable = d >= c->heap[r] + kCtrlBytes && d + (size_t)n * es_out <= c->heap[r] + c->heap_bytes && ((uintptr_t)d & 15u) == 0;
    R.lr[i].dst_off = reachable ? (unsigned long long)(d - c->heap[r]) : kNoOffset;
  }
  R.seq = G.seq = next_seq(c);
  if (int e = launch_allreduce(c, kernel, R, G, stream)) return e;
  return scope.leave();
}

int hapx_all_to_all(hapx_comm* c, void* const* dst, const void* const* src, int dtype, int64_t a, int64_t b, int64_t cc,
                    int split_is_first, const int64_t* split_lengths, const int64_t* cat_lengths, hapx_stream stream_) {
  if (int e = check_ready(c)) return e;
  if (!dst || !src) return fail(HAPX_ERR_ARGUMENT, "all_to_all: null pointer array");
  const int es = dtype_size(dtype);
  if (!es) return fail(HAPX_ERR_DTYPE, "all_to_all: unknown dtype");
  if (a < 0 || b < 0 || cc < 0) return fail(HAPX_ERR_EXTENT, "all_to_all: negative extent");
  if (int e = check_lengths(split_lengths, c->world, "all_to_all")) return e;
  if (int e = check_lengths(cat_lengths, c->world, "all_to_all")) return e;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  PullParams P;
  init_params(c, P, OP_EXCHANGE, es, es);
  P.A = a; P.B = b; P.C = cc; P.split_first = split_is_first ? 1 : 0;
  fill_prefix(split_lengths, c->world, P.L1, P.P1, &P.tot1);
  fill_prefix(cat_lengths, c->world, P.L2, P.P2, &P.tot2);
  if (a * b * cc * P.tot1 * P.tot2 == 0) return HAPX_OK;
  CallScope scope{c, stream};
  if (int e = scope.enter()) return e;
  for (int i = 0; i < c->n_local; ++i) {
    const int r = c->first_rank + i;
    P.lr[i].rank = r;
    P.lr[i].src = static_cast<const char*>(src[i]);
    P.lr[i].dst = static_cast<char*>(dst[i]);
    const size_t bytes = (size_t)(a * P.tot1 * b * P.L2[r] * cc) * es;
    const size_t out_bytes = (size_t)(a * P.L1[r] * b * P.tot2 * cc) * es;
    if (!dst[i] && out_bytes) return fail(HAPX_ERR_ARGUMENT, "null output pointer");
    if (int e = publish_input(c, i, src[i], bytes, false, 0, stream, &P.lr[i].src_off)) return e;
  }
  P.seq = next_seq(c);
  if (int e = launch_pull(c, pull_copy_kernel, P, kCopyTile, stream)) return e;
  return scope.leave();
}

static int slice_impl(int op, void* dst, const void* src, int dtype, int64_t outer, int64_t inner, const int64_t* lengths,
                      int world, int rank, cudaStream_t stream) {
  const int es = dtype_size(dtype);
  if (!es) return fail(HAPX_ERR_DTYPE, "dynamic_slice: unknown dtype");
  if (world < 1 || world > HAPX_MAX_WORLD || rank < 0 || rank >= world) return fail(HAPX_ERR_ARGUMENT, "dynamic_slice: bad world/rank");
  if (outer < 0 || inner < 0) return fail(HAPX_ERR_EXTENT, "dynamic_slice: negative extent");
  if (int e = check_lengths(lengths, world, "dynamic_slice")) return e;
  PullParams P = PullParams();
  P.op = op; P.world = world; P.n_local = 1; P.es_in = es; P.es_out = es; P.self_only = 1; P.scale = 1.f;
  P.A = outer; P.C = inner;
  fill_prefix(lengths, world, P.L1, P.P1, &P.tot1);
  int device = 0, sms = 0;
  HAPX_CUDA(cudaGetDevice(&device));
  HAPX_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
  if (op == OP_UNSLICE) {
    const size_t full = (size_t)(outer * P.tot1 * inner) * es;
    if (full) HAPX_CUDA(cudaMemsetAsync(dst, 0, full, stream));
  }
  if (outer * P.L1[rank] * inner == 0) return HAPX_OK;
  if (!dst || !src) return fail(HAPX_ERR_ARGUMENT, "dynamic_slice: null pointer");
  P.lr[0].rank = rank; P.lr[0].src = static_cast<const char*>(src); P.lr[0].dst = static_cast<char*>(dst);
  hapx_comm tmp;  // only the fields launch_pull reads
  tmp.world = world; tmp.n_local = 1; tmp.sm_count = sms; tmp.local_mode = false; tmp.max_ctas = 0;
  return launch_pull(&tmp, pull_copy_kernel, P, kCopyTile, stream);
}

int hapx_dynamic_slice(void* dst, const void* src, int dtype, int64_t outer, int64_t inner, const int64_t* lengths,
                       int world, int rank, hapx_stream stream) {
  return slice_impl(OP_SLICE, dst, src, dtype, outer, inner, lengths, world, rank, static_cast<cudaStream_t>(stream));
}

int hapx_comm_get(hapx_comm* c, int peer, size_t peer_offset, void* dst, size_t bytes, hapx_stream stream_) {
  if (int e = check_ready(c)) return e;
  if (c->local_mode || c->n_local != 1) return fail(HAPX_ERR_STATE, "comm_get: needs a one-process-per-GPU communicator");
  if (peer < 0 || peer >= c->world) return fail(HAPX_ERR_ARGUMENT, "comm_get: peer out of range");
  const size_t user = kCtrlBytes + c->stage_bytes;
  if (peer_offset > c->heap_bytes - user || bytes > c->heap_bytes - user - peer_offset)
    return fail(HAPX_ERR_EXTENT, "comm_get: range outside the peer's user area");
  if (bytes == 0) return HAPX_OK;
  if (!dst) return fail(HAPX_ERR_ARGUMENT, "comm_get: null destination");
  HAPX_CUDA(cudaSetDevice(c->device));
  // a one-rank "slice" of bytes: the copy kernel without the flag protocol, reading the peer's mapping
  const int64_t one = (int64_t)bytes;
  PullParams P = PullParams();
  P.op = OP_SLICE; P.world = 1; P.n_local = 1; P.es_in = 1; P.es_out = 1; P.self_only = 1; P.scale = 1.f;
  P.order_log2 = 0;
  P.A = 1; P.C = 1;
  fill_prefix(&one, 1, P.L1, P.P1, &P.tot1);
  P.lr[0].rank = 0;
  P.lr[0].src = c->heap[peer] + user + peer_offset;
  P.lr[0].dst = static_cast<char*>(dst);
  hapx_comm tmp;
  tmp.world = 1; tmp.n_local = 1; tmp.sm_count = c->sm_count; tmp.local_mode = false; tmp.max_ctas = c->max_ctas;
  return launch_pull(&tmp, pull_copy_kernel, P, kCopyTile, static_cast<cudaStream_t>(stream_));
}

int hapx_dynamic_slice_backward(void* dst, const void* src, int dtype, int64_t outer, int64_t inner, const int64_t* lengths,
                                int world, int rank, hapx_stream stream) {
  return slice_impl(OP_UNSLICE, dst, src, dtype, outer, inner, lengths, world, rank, static_cast<cudaStream_t>(stream));
}


/* ---- all_reduce for callers that must not allocate ------------------------------------------
 * Same result as hapx_all_reduce on a local (single-device, `world` virtual ranks)
 * communicator, but with no communicator and no allocation of any kind: the control blocks,
 * the staged copies of the inputs and the reduced slices live in the file-scope device array
 * below (16 MiB per GPU that loads the library, held until the process exits), and the same
 * pull_reduce / pull_copy kernels run over it.  It exists for hosts that cannot call cudaMalloc
 * when a collective is due: a process that has already handed all device memory to another
 * allocator (a caching allocator with the whole card reserved, a fixed memory budget), or a
 * latency-critical thread on which the device-wide synchronisation of cudaMalloc / cudaFree
 * would stall every stream.
 *
 * Limits: world <= 8 and 4096 + round256(n * in_size) + round256(ceil(n / world) rounded up to
 * 16 bytes * out_size) <= 2 MiB per rank (about 460 000 float32 elements at world 8); larger
 * calls are rejected with HAPX_ERR_STAGING.
 * The first call on a device looks the array's device address up (cudaGetSymbolAddress); make
 * that first call outside any stream capture.  All calls share the one array: each call
 * clears the control blocks it uses before launching, and two calls whose kernels overlap on
 * the GPU (different streams without ordering between them, or two host threads) race. */
constexpr int kNoAllocMaxWorld = 8;
constexpr size_t kNoAllocRankBytes = 2u << 20;
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocMaxWorld * kNoAllocRankBytes];

namespace {
struct NoAllocDevice {
  bool ready = false;
  char* base = nullptr;   // DEVICE address of g_noalloc_scratch on that device (never the host-side symbol)
  int sm_count = 0;
  unsigned seq = 0;
};
NoAllocDevice g_noalloc_dev[64];
std::mutex g_noalloc_mutex;
}  // namespace

int hapx_local_all_reduce_noalloc(int world, void* const* dst, const void* const* src, int in_dtype, int out_dtype,
                                  double scale, int64_t n, hapx_stream stream_) {
  if (world < 1 || world > kNoAllocMaxWorld)
    return fail(HAPX_ERR_ARGUMENT, "all_reduce_noalloc: world must be in [1, " + std::to_string(kNoAllocMaxWorld) + "]");
  if (!dst || !src) return fail(HAPX_ERR_ARGUMENT, "all_reduce_noalloc: null pointer array");
  if (n < 0) return fail(HAPX_ERR_EXTENT, "all_reduce_noalloc: negative size");
  PullKernel reduce_kernel = reduce_kernel_for(in_dtype, out_dtype);
  if (!reduce_kernel) return fail(HAPX_ERR_DTYPE, "all_reduce_noalloc: reductions support float32, bfloat16 and float16");
  if (n == 0) return HAPX_OK;
  const int es_in = dtype_size(in_dtype), es_out = dtype_size(out_dtype);
  const long long vec = 16 / es_in;
  const long long per = ((n + world - 1) / world + vec - 1) / vec * vec;   // even split on 16-byte boundaries
  const size_t in_bytes = (size_t)n * es_in;
  const size_t in_room = (in_bytes + 255) / 256 * 256;
  const size_t mid_bytes = ((size_t)per * es_out + 255) / 256 * 256;
  if (kCtrlBytes + in_room + mid_bytes > kNoAllocRankBytes)
    return fail(HAPX_ERR_STAGING, "all_reduce_noalloc: " + std::to_string(n) + " elements need " +
                                      std::to_string(kCtrlBytes + in_room + mid_bytes) + " bytes of scratch per rank; the built-in array holds " +
                                      std::to_string(kNoAllocRankBytes) + " (use hapx_all_reduce on a communicator for larger tensors)");
  for (int r = 0; r < world; ++r)
    if (!dst[r] || !src[r]) return fail(HAPX_ERR_ARGUMENT, "all_reduce_noalloc: null tensor pointer");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);

  std::lock_guard<std::mutex> lock(g_noalloc_mutex);
  int device = 0;
  HAPX_CUDA(cudaGetDevice(&device));
  if (device < 0 || device >= 64) return fail(HAPX_ERR_ARGUMENT, "all_reduce_noalloc: device index out of range");
  NoAllocDevice& nd = g_noalloc_dev[device];
  if (!nd.ready) {  // once per device, with that device current
    void* p = nullptr;
    HAPX_CUDA(cudaGetSymbolAddress(&p, g_noalloc_scratch));
    HAPX_CUDA(cudaDeviceGetAttribute(&nd.sm_count, cudaDevAttrMultiProcessorCount, device));
    nd.base = static_cast<char*>(p);
    nd.ready = true;
  }

  // A communicator-shaped view of the array (host struct only; nothing is allocated).
  hapx_comm view;
  view.world = world; view.n_local = world; view.first_rank = 0; view.device = device; view.local_mode = true;
  view.heap_bytes = kNoAllocRankBytes; view.stage_bytes = kNoAllocRankBytes - kCtrlBytes;
  view.sm_count = nd.sm_count;
  for (int r = 0; r < world; ++r) { view.heap[r] = nd.base + (size_t)r * kNoAllocRankBytes; view.mapped[r] = true; }
  // the control blocks keep the previous call's flags and counters: start from zero (the status words
  // behind them stay, so that a wait that ran out is still there for the status query)
  for (int r = 0; r < world; ++r) HAPX_CUDA(cudaMemsetAsync(view.heap[r], 0, offsetof(Ctrl, status), stream));

  int64_t lengths[HAPX_MAX_WORLD];
  long long L[HAPX_MAX_WORLD], Pfx[HAPX_MAX_WORLD], total;
  long long left = n;
  for (int r = 0; r < HAPX_MAX_WORLD; ++r) { lengths[r] = (r < world) ? std::min(per, left) : 0; left -= lengths[r]; }
  fill_prefix(lengths, world, L, Pfx, &total);
  const size_t mid_pos = view.stage_bytes - mid_bytes;

  // 1st launch: rank r sums slice r of every (staged) input into the tail of its staging area
  PullParams P;
  init_params(&view, P, OP_REDUCE, es_in, es_out);
  P.A = 1; P.C = 1; P.scale = (float)scale;
  for (int i = 0; i < HAPX_MAX_WORLD; ++i) { P.L1[i] = L[i]; P.P1[i] = Pfx[i]; }
  P.tot1 = total;
  for (int r = 0; r < world; ++r) {
    P.lr[r].rank = r;
    P.lr[r].src = static_cast<const char*>(src[r]);
    P.lr[r].dst = view.heap[r] + kCtrlBytes + mid_pos;
    if (int e = publish_input(&view, r, src[r], in_bytes, true, 0, stream, &P.lr[r].src_off)) return e;
  }
  nd.seq = (nd.seq + 1) & 0xffffffu;
  if (nd.seq == 0) nd.seq = 1;
  P.seq = nd.seq;
  if (int e = launch_pull(&view, reduce_kernel, P, kRedTile, stream)) return e;

  // 2nd launch: every rank gathers the reduced slices into its output
  PullParams G;
  init_params(&view, G, OP_GATHER, es_out, es_out);
  G.A = 1; G.C = 1;
  fill_prefix(lengths, world, G.L1, G.P1, &G.tot1);
  for (int r = 0; r < world; ++r) {
    G.lr[r].rank = r;
    G.lr[r].src = view.heap[r] + kCtrlBytes + mid_pos;
    G.lr[r].dst = static_cast<char*>(dst[r]);
    G.lr[r].src_off = kCtrlBytes + mid_pos;
  }
  nd.seq = (nd.seq + 1) & 0xffffffu;
  if (nd.seq == 0) nd.seq = 1;
  G.seq = nd.seq;
  return launch_pull(&view, pull_copy_kernel, G, kCopyTile, stream);
}

int hapx_local_all_reduce_noalloc_status(void) {
  std::lock_guard<std::mutex> lock(g_noalloc_mutex);
  int device = 0;
  HAPX_CUDA(cudaGetDevice(&device));
  if (device < 0 || device >= 64) return fail(HAPX_ERR_ARGUMENT, "all_reduce_noalloc_status: device index out of range");
  NoAllocDevice& nd = g_noalloc_dev[device];
  if (!nd.ready) return HAPX_OK;   // nothing has run on this device yet
  HAPX_CUDA(cudaDeviceSynchronize());
  int rc = HAPX_OK;
  std::string msg;
  for (int r = 0; r < kNoAllocMaxWorld; ++r) {
    Ctrl host;
    char* block = nd.base + (size_t)r * kNoAllocRankBytes;
    HAPX_CUDA(cudaMemcpy(&host, block, sizeof(Ctrl), cudaMemcpyDeviceToHost));
    if (host.status != 0) {
      rc = -static_cast<int>(host.status);
      msg += "virtual rank " + std::to_string(r) + ": device wait ran out (waiting for rank " +
             std::to_string(host.status_info & 0xffffffffu) + "); ";
      HAPX_CUDA(cudaMemset(block + offsetof(Ctrl, cta_done), 0, sizeof(Ctrl) - offsetof(Ctrl, cta_done)));
    }
  }
  if (rc != HAPX_OK) return fail(rc, msg);
  return HAPX_OK;
}

/* Diagnostic, host memory only: walks the warp tiling of one rank's pull (the same
 * build_seg / locate code the kernels run) over HOST buffers, checking every byte range
 * against the buffer sizes.  It lets CPU-only tests validate the index arithmetic for a
 * geometry before any kernel touches it.  It is not a compute path: it accepts no device
 * pointers and nothing in the library calls it. */
int hapx_debug_host_walk(int op, int world, int rank, int es, int64_t a, int64_t b, int64_t cc, int split_is_first,
                         const int64_t* l1, const int64_t* l2, const void* const* src_per_rank,
                         const size_t* src_bytes, void* dst, size_t dst_bytes, unsigned char* cover) {
  if (world < 1 || world > HAPX_MAX_WORLD || rank < 0 || rank >= world) return fail(HAPX_ERR_ARGUMENT, "host_walk: bad world/rank");
  if (op != OP_GATHER && op != OP_EXCHANGE && op != OP_SLICE && op != OP_UNSLICE) return fail(HAPX_ERR_ARGUMENT, "host_walk: bad op");
  PullParams P = PullParams();
  P.op = op; P.world = world; P.n_local = 1; P.es_in = es; P.es_out = es; P.split_first = split_is_first;
  P.A = a; P.B = b; P.C = cc;
  fill_prefix(l1, world, P.L1, P.P1, &P.tot1);
  if (l2) fill_prefix(l2, world, P.L2, P.P2, &P.tot2);
  const bool one_seg = (op == OP_SLICE || op == OP_UNSLICE);
  const int nseg = one_seg ? 1 : world;
  Seg segs[HAPX_MAX_WORLD];
  unsigned acc = 0;
  for (int p = 0; p < nseg; ++p) {
    build_seg(P, rank, one_seg ? rank : p, kCopyTile, segs[p]);
    if (segs[p].rows64 >= (1ull << 32) || segs[p].tiles64 >= (1ull << 32)) return fail(HAPX_ERR_EXTENT, "host_walk: too large");
    segs[p].tile_begin = acc;
    acc += segs[p].n_tiles;
  }
  for (unsigned t = 0; t < acc; ++t) {
    const TilePos tp = locate(segs, nseg, t);
    const Seg& s = segs[tp.si];
    const char* sbase = static_cast<const char*>(src_per_rank[s.peer]);
    const long long sbytes = (long long)src_bytes[s.peer];
    // the device aligns tiles to the 16-byte grid of the source ADDRESS; emulate a base that is 16-byte aligned
    const unsigned mis = (unsigned)(tp.src_row_b & 15);
    for (int lane = 0; lane < 32; ++lane) {
      for (int u = 0; u < kCopyUnroll; ++u) {
        const long long rel = (long long)tp.k * kCopyTile - (long long)mis + (long long)lane * 16 + u * 512;
        const long long lo = rel < 0 ? 0 : rel;
        const long long hi = (rel + 16 < s.run_b) ? rel + 16 : s.run_b;
        if (lo >= hi) continue;
        const long long so = tp.src_row_b + lo, d_o = tp.dst_row_b + lo, n = hi - lo;
        if (so < 0 || so + n > sbytes) return fail(HAPX_ERR_EXTENT, "host_walk: source range out of bounds at tile " + std::to_string(t));
        if (d_o < 0 || d_o + n > (long long)dst_bytes) return fail(HAPX_ERR_EXTENT, "host_walk: destination range out of bounds at tile " + std::to_string(t));
        if (n % es != 0 || so % es != 0 || d_o % es != 0) return fail(HAPX_ERR_EXTENT, "host_walk: range splits an element at tile " + std::to_string(t));
        for (long long i = 0; i < n; ++i) {
          static_cast<char*>(dst)[d_o + i] = sbase[so + i];
          if (cover) cover[d_o + i] = (unsigned char)(cover[d_o + i] + 1);  // how often each output byte was written
        }
      }
    }
  }
  return HAPX_OK;
}

}  // extern "C"
