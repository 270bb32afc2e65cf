// Routing: boolean token mask -> per-modality compacted row-index lists.
//
// Replaces the reference's per-tile "is this tile all visual / all text / mixed" test
// (ffn_kernel/linear.py:132-149, ffn_kernel/ffn.py:72-99): once the rows of each modality are
// known as a list, every GEMM tile multiplies one modality's rows by one modality's weights.
//
//   perm[0 .. Mv)            = ascending indices of tokens with mask != 0   (visual)
//   perm[cap .. cap + Mt)    = ascending indices of tokens with mask == 0   (text)
//   counts[0] = Mv, counts[1] = Mt, counts[2] = cap, counts[3] = M,
//   counts[4] = number of runs (maximal stretches of consecutive tokens of one modality); [5..7] unused
//
// Integer work, bit-exact with nonzero(mask) / nonzero(~mask).  One pass over the mask: a
// chained scan with decoupled look-back over tiles in block-index order; the look-back spin is
// bounded, so a tile whose predecessor never publishes reports a status code instead of hanging.
//
// Algorithmic traffic: 1 byte read + 4 bytes written per token.
#include <cuda_bf16.h>

#include <mutex>

#include "ffnk_internal.h"
#include "ptx.cuh"

namespace ffnk {

constexpr int kRouteThreads = 256;
constexpr int kRoutePerThread = 32;                             // two 128-bit loads of mask bytes
constexpr int kRouteTile = kRouteThreads * kRoutePerThread;     // 8192 tokens per tile
constexpr int kLookPerLane = 4;                                 // look-back window: 32 lanes x 4 tiles

// tile state word: [31:30] flag (0 = nothing, 1 = tile aggregate, 2 = inclusive prefix), [29:0] visual count
constexpr uint32_t kFlagAgg = 1u << 30;
constexpr uint32_t kFlagInc = 2u << 30;
constexpr uint32_t kValMask = (1u << 30) - 1;

// The 32 mask bytes of one thread as a bit mask (bit i = token base + i is visual), how many of
// the 32 tokens exist, and how many runs start among them (a token whose modality differs from its
// predecessor's; token 0 always).
struct ThreadTokens {
  uint32_t bits;
  int valid;
  int nruns;
};

// 32 mask bytes (eight words) -> 32 bits.  Four bytes at a time: the high bit of every non-zero byte, then
// one multiply that lines the bits of positions 0, 8, 16, 24 up at 24..27 (no two partial products share
// a bit position).
__device__ __forceinline__ uint32_t mask_words_to_bits(const uint32_t (&w)[kRoutePerThread / 4]) {
  uint32_t bits = 0;
#pragma unroll
  for (int i = 0; i < kRoutePerThread / 4; ++i) {
    const uint32_t nz = (((w[i] & 0x7F7F7F7Fu) + 0x7F7F7F7Fu) | w[i]) & 0x80808080u;
    bits |= ((((nz >> 7) * 0x01020408u) >> 24) & 0xFu) << (4 * i);
  }
  return bits;
}

__device__ __forceinline__ ThreadTokens load_thread_tokens(const uint8_t* __restrict__ mask, int M, int base) {
  uint32_t w[kRoutePerThread / 4] = {};
  int valid = M - base;
  valid = valid < 0 ? 0 : (valid > kRoutePerThread ? kRoutePerThread : valid);
  if (valid == kRoutePerThread && ((reinterpret_cast<uintptr_t>(mask) & 15) == 0)) {
    const uint4 v0 = *reinterpret_cast<const uint4*>(mask + base);
    const uint4 v1 = *reinterpret_cast<const uint4*>(mask + base + 16);
    w[0] = v0.x; w[1] = v0.y; w[2] = v0.z; w[3] = v0.w;
    w[4] = v1.x; w[5] = v1.y; w[6] = v1.z; w[7] = v1.w;
  } else {
#pragma unroll    // fully unrolled: the words stay in registers
    for (int i = 0; i < kRoutePerThread; ++i)
      if (i < valid) w[i >> 2] |= static_cast<uint32_t>(mask[base + i]) << (8 * (i & 3));
  }
  ThreadTokens t;
  t.bits = mask_words_to_bits(w);
  t.valid = valid;
  t.nruns = 0;
  if (valid > 0) {
    const uint32_t prev = base > 0 ? (mask[base - 1] != 0 ? 1u : 0u) : ((t.bits & 1u) ^ 1u);
    const uint32_t vmask = valid == 32 ? 0xFFFFFFFFu : ((1u << valid) - 1u);
    t.nruns = __popc((t.bits ^ ((t.bits << 1) | prev)) & vmask);
  }
  return t;
}

// Block-wide scan of the per-thread visual counts.  Returns the number of visual tokens before
// this thread inside the tile; *tile_v = visual tokens of the tile.  Contains one __syncthreads().
__device__ __forceinline__ int block_exclusive_scan(int nv, int* s_warp, int* tile_v) {
  const int tid = threadIdx.x;
  int incl = nv;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int n = __shfl_up_sync(0xFFFFFFFFu, incl, o);
    if ((tid & 31) >= o) incl += n;
  }
  if ((tid & 31) == 31) s_warp[tid >> 5] = incl;
  __syncthreads();
  int warp_off = 0, total = 0;
#pragma unroll
  for (int i = 0; i < kRouteThreads / 32; ++i) {
    const int c = s_warp[i];
    if (i < (tid >> 5)) warp_off += c;
    total += c;
  }
  *tile_v = total;
  return warp_off + incl - nv;
}

// Compaction inside the tile: visual indices to s_v[0..tile_v), text indices to s_t[0..tile_t), both
// ascending.  Every thread walks its own 32 consecutive tokens and appends each index to its modality's
// list (ev: visual tokens of the tile before this thread; valid: how many of the 32 tokens exist): six
// instructions a token.  Neighbouring lanes write about 16 words apart, a few-way bank conflict per
// store, which costs less than the three shuffles and two population counts per token group of a
// conflict-free warp-transposed order (20 instructions per 32 tokens and lane: the scatter kernel was
// bound by instruction issue, not by DRAM).
__device__ __forceinline__ void compact_tile(int* s_v, int* s_t, int tile, uint32_t bits, int ev, int valid) {
  const int first = static_cast<int>(threadIdx.x) * kRoutePerThread;   // this thread's first token within the tile
  int* pv = s_v + ev;
  int* pt = s_t + (first - ev);
  const int tok0 = tile * kRouteTile + first;
  if (valid == kRoutePerThread) {
#pragma unroll
    for (int i = 0; i < kRoutePerThread; ++i) {
      const bool vis = (bits >> i) & 1u;
      *(vis ? pv : pt) = tok0 + i;
      pv += vis ? 1 : 0;
      pt += vis ? 0 : 1;
    }
  } else {
    for (int i = 0; i < valid; ++i) {
      const bool vis = (bits >> i) & 1u;
      *(vis ? pv : pt) = tok0 + i;
      pv += vis ? 1 : 0;
      pt += vis ? 0 : 1;
    }
  }
}

__global__ void __launch_bounds__(kRouteThreads) route_kernel(const uint8_t* __restrict__ mask, int M, int cap,
                                                              int* __restrict__ perm, int* __restrict__ counts,
                                                              uint32_t* __restrict__ ws,  // [0] run total, [1..tiles] tile state, [tiles+1] finished tiles
                                                              int* __restrict__ status) {
  __shared__ int s_list[kRouteTile];  // visual indices from the front, text indices after them
  __shared__ int s_warp[kRouteThreads / 32];
  __shared__ int s_excl, s_ok, s_runs;

  const int tid = threadIdx.x;
  // Tiles are taken in block-index order.  Blocks are dispatched in that order, so a tile's
  // predecessors are running or done when it looks back; the look-back wait is bounded regardless.
  const int tile = blockIdx.x;
  const int num_tiles = (M + kRouteTile - 1) / kRouteTile;
  volatile uint32_t* state = ws + 1;

  const int base = tile * kRouteTile + tid * kRoutePerThread;
  const ThreadTokens tt = load_thread_tokens(mask, M, base);
  const uint32_t bits = tt.bits;
  const int nv = __popc(bits);
  if (tid == 0) s_runs = 0;
  int tile_v = 0;
  const int ev = block_exclusive_scan(nv, s_warp, &tile_v);   // visual tokens before this thread, in tile
  {
    const int wr = __reduce_add_sync(0xFFFFFFFFu, tt.nruns);
    if ((tid & 31) == 0 && wr) atomicAdd(&s_runs, wr);
  }
  const int tile_len = min(kRouteTile, M - tile * kRouteTile);
  const int tile_t = tile_len - tile_v;

  // publish the tile aggregate, then look back for the exclusive prefix
  if (tid == 0) {
    if (tile == 0) {
      state[0] = kFlagInc | static_cast<uint32_t>(tile_v);
      s_excl = 0;
      s_ok = 1;
    } else {
      state[tile] = kFlagAgg | static_cast<uint32_t>(tile_v);
    }
  }
  if (tile > 0 && tid < 32) {
    // warp 0 walks back 128 tiles at a time (lane l inspects tiles look - 4l - j, j = 0..3): the
    // chain of inclusive prefixes then advances by up to 128 tiles per L2 round trip
    int excl = 0, ok = 1;
    int look = tile - 1;
    const uint64_t t0 = globaltimer_ns();
    while (true) {
      uint32_t st[kLookPerLane];
      int idx[kLookPerLane];
#pragma unroll
      for (int j = 0; j < kLookPerLane; ++j) {
        idx[j] = look - (static_cast<int>(tid) * kLookPerLane + j);
        st[j] = 2u << 30;  // before tile 0: an inclusive prefix of 0
        if (idx[j] >= 0) st[j] = state[idx[j]];
      }
      // wait until every inspected tile has published something (all branches warp-uniform)
      uint32_t polls = 0;
      while (true) {
        bool pending = false;
#pragma unroll
        for (int j = 0; j < kLookPerLane; ++j) pending |= (st[j] >> 30) == 0;
        if (!__any_sync(0xFFFFFFFFu, pending)) break;
#pragma unroll
        for (int j = 0; j < kLookPerLane; ++j)
          if ((st[j] >> 30) == 0) st[j] = state[idx[j]];
        ++polls;
        const bool expired = (polls & 63u) == 0 && globaltimer_ns() - t0 > kWaitBudgetNs;
        if (__any_sync(0xFFFFFFFFu, expired)) { ok = 0; break; }
      }
      if (!ok) break;
      // nearest inclusive prefix in the window; nearer tiles contribute their aggregates, it its prefix
      int my_first = 1 << 20;
#pragma unroll
      for (int j = kLookPerLane - 1; j >= 0; --j)
        if ((st[j] >> 30) == 2) my_first = static_cast<int>(tid) * kLookPerLane + j;
      const int first_inc = __reduce_min_sync(0xFFFFFFFFu, my_first);
      int contrib = 0;
#pragma unroll
      for (int j = 0; j < kLookPerLane; ++j)
        if (static_cast<int>(tid) * kLookPerLane + j <= first_inc) contrib += static_cast<int>(st[j] & kValMask);
      excl += __reduce_add_sync(0xFFFFFFFFu, contrib);
      if (first_inc < (1 << 20)) break;
      look -= 32 * kLookPerLane;
    }
    if (tid == 0) {
      s_excl = excl;
      s_ok = ok;
      if (ok) state[tile] = kFlagInc | static_cast<uint32_t>(excl + tile_v);
      else atomicCAS(status, 0, ST_TIMEOUT_SCAN);
    }
  }

  compact_tile(s_list, s_list + tile_v, tile, bits, ev, tt.valid);
  __syncthreads();
  if (!s_ok) return;
  const int pre_v = s_excl;
  const int pre_t = tile * kRouteTile - pre_v;
  for (int i = tid; i < tile_v; i += kRouteThreads) perm[pre_v + i] = s_list[i];
  for (int i = tid; i < tile_t; i += kRouteThreads) perm[cap + pre_t + i] = s_list[tile_v + i];
  if (tile == num_tiles - 1 && tid == 0) {
    counts[0] = pre_v + tile_v;
    counts[1] = M - (pre_v + tile_v);
    counts[2] = cap;
    counts[3] = M;
  }
  if (tid == 0) {   // s_runs is complete: every warp added to it before the barrier above
    if (num_tiles == 1) {
      counts[4] = s_runs;
    } else {
      // the tile that finishes last publishes the total
      atomicAdd(&ws[0], static_cast<uint32_t>(s_runs));
      __threadfence();
      if (atomicAdd(&ws[1 + num_tiles], 1u) == static_cast<uint32_t>(num_tiles - 1))
        counts[4] = static_cast<int>(atomicAdd(&ws[0], 0u));
    }
  }
}

// -------------------------------------------------------------------------------------------
// Long masks (more than kLookBackMaxTiles tiles): two kernels and no waiting.  With thousands of
// tiles in flight the look-back of route_kernel turns into every tile polling the same few cache
// lines of tile states, and the chain of prefixes, not DRAM, sets the pace (M = 2^26: 1.3 TB/s of
// the 5 bytes per token).  Here the first kernel counts (1 byte per token read) and its last block
// to finish turns the per-tile counts into exclusive prefixes; the second kernel reads the mask
// again and writes the lists (6 bytes per token in all).
// ws: [0] run total, [1..tiles] per-tile visual count -> exclusive prefix, [tiles+1] finished blocks of the count kernel.
// -------------------------------------------------------------------------------------------
constexpr int kLookBackMaxTiles = 128;

constexpr int kCountTiles = 4;       // tiles per block of the count kernel: 128 mask bytes per thread in flight

__global__ void __launch_bounds__(kRouteThreads) route_count_kernel(const uint8_t* __restrict__ mask, int M, int cap,
                                                                    int num_tiles, int* __restrict__ counts,
                                                                    uint32_t* __restrict__ ws) {
  __shared__ int s_cnt[kCountTiles][kRouteThreads / 32];
  __shared__ int s_warp[kRouteThreads / 32];
  __shared__ int s_runs, s_last;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int tile0 = blockIdx.x * kCountTiles;
  if (tid == 0) s_runs = 0;
  uint32_t bits[kCountTiles];
  int nruns = 0;
  if (static_cast<int64_t>(tile0 + kCountTiles) * kRouteTile <= M && (reinterpret_cast<uintptr_t>(mask) & 15) == 0) {
    // whole tiles: all eight 16-byte loads of the thread first (one byte per warp more: the token before
    // the warp's first, for the run count), then the arithmetic
    uint4 v[kCountTiles][2];
    uint32_t prev_byte[kCountTiles];
#pragma unroll
    for (int j = 0; j < kCountTiles; ++j) {
      const int base = (tile0 + j) * kRouteTile + tid * kRoutePerThread;
      v[j][0] = *reinterpret_cast<const uint4*>(mask + base);
      v[j][1] = *reinterpret_cast<const uint4*>(mask + base + 16);
      prev_byte[j] = (lane == 0 && base > 0) ? mask[base - 1] : 0u;
    }
#pragma unroll
    for (int j = 0; j < kCountTiles; ++j) {
      const uint32_t w[8] = {v[j][0].x, v[j][0].y, v[j][0].z, v[j][0].w, v[j][1].x, v[j][1].y, v[j][1].z, v[j][1].w};
      bits[j] = mask_words_to_bits(w);
      // a run starts at every token whose modality differs from its predecessor's (token 0 always)
      uint32_t prev = __shfl_up_sync(0xFFFFFFFFu, bits[j] >> 31, 1);
      if (lane == 0) {
        const int base = (tile0 + j) * kRouteTile + tid * kRoutePerThread;
        prev = base > 0 ? (prev_byte[j] != 0 ? 1u : 0u) : ((bits[j] & 1u) ^ 1u);
      }
      nruns += __popc(bits[j] ^ ((bits[j] << 1) | prev));
    }
  } else {
#pragma unroll
    for (int j = 0; j < kCountTiles; ++j) {
      const ThreadTokens tt = load_thread_tokens(mask, M, (tile0 + j) * kRouteTile + tid * kRoutePerThread);
      bits[j] = tt.bits;
      nruns += tt.nruns;
    }
  }
#pragma unroll
  for (int j = 0; j < kCountTiles; ++j) {
    const int c = __reduce_add_sync(0xFFFFFFFFu, __popc(bits[j]));
    if (lane == 0) s_cnt[j][warp] = c;
  }
  __syncthreads();                     // s_runs is zero, s_cnt is complete
  {
    const int wr = __reduce_add_sync(0xFFFFFFFFu, nruns);
    if (lane == 0 && wr) atomicAdd(&s_runs, wr);
  }
  if (tid < kCountTiles && tile0 + tid < num_tiles) {
    int c = 0;
#pragma unroll
    for (int i = 0; i < kRouteThreads / 32; ++i) c += s_cnt[tid][i];
    ws[1 + tile0 + tid] = static_cast<uint32_t>(c);
    __threadfence();
  }
  __syncthreads();
  if (tid == 0) {
    atomicAdd(&ws[0], static_cast<uint32_t>(s_runs));
    __threadfence();
    s_last = atomicAdd(&ws[1 + num_tiles], 1u) == gridDim.x - 1;
  }
  __syncthreads();
  if (!s_last) return;
  // every other block has published its counts: exclusive prefix over the tiles, in place; 2048 tiles a
  // round, a thread's eight loads issued together (read around L1: other SMs wrote them)
  __threadfence();
  uint32_t* cnt = ws + 1;
  int total = 0;
  for (int base = 0; base < num_tiles; base += kRouteThreads * 8) {
    const int i0 = base + tid * 8;
    int c[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) c[j] = i0 + j < num_tiles ? static_cast<int>(__ldcg(cnt + i0 + j)) : 0;
    int sum = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) sum += c[j];
    int round_total = 0;
    int run = total + block_exclusive_scan(sum, s_warp, &round_total);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (i0 + j < num_tiles) cnt[i0 + j] = static_cast<uint32_t>(run);
      run += c[j];
    }
    total += round_total;
    __syncthreads();     // s_warp is rewritten in the next round
  }
  if (tid == 0) {
    counts[0] = total;
    counts[1] = M - total;
    counts[2] = cap;
    counts[3] = M;
    counts[4] = static_cast<int>(atomicAdd(&ws[0], 0u));
  }
}

// One list of a tile, shared memory -> global memory.  The list was laid out in shared memory with the
// same alignment (modulo four elements) as its destination, so everything between the first and the
// last 16-byte boundary leaves as ONE bulk copy issued by a single thread; at most three elements at
// either end are stored one by one.  `dst` and `src` address element 0 of the list.  `t0`: first of the
// 96 threads that do the work (a different warp triple per list, so the two lists of a tile go out side
// by side).
__device__ __forceinline__ void store_list_bulk(int* dst, const int* src, int n, int t0) {
  const int head = min(n, static_cast<int>((4u - ((reinterpret_cast<uintptr_t>(dst) >> 2) & 3u)) & 3u));
  const int mid = (n - head) & ~3;
  const int tid = static_cast<int>(threadIdx.x) - t0;
  if (tid >= 0 && tid < head) dst[tid] = src[tid];
  else if (tid >= 32 && tid < 32 + (n - head - mid)) dst[head + mid + tid - 32] = src[head + mid + tid - 32];
  if (tid == 64 && mid > 0) {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");     // the list was written by ordinary stores
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst + head),
                 "r"(smem_u32(src + head)), "r"(mid * 4)
                 : "memory");
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
    asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");   // shared memory may be released
  }
}

__global__ void __launch_bounds__(kRouteThreads) route_scatter_kernel(const uint8_t* __restrict__ mask, int M, int cap,
                                                                      int* __restrict__ perm,
                                                                      const uint32_t* __restrict__ ws) {
  __shared__ __align__(16) int s_list[kRouteTile + 16];
  __shared__ int s_warp[kRouteThreads / 32];
  const int tid = threadIdx.x;
  const int tile = blockIdx.x;
  const ThreadTokens tt = load_thread_tokens(mask, M, tile * kRouteTile + tid * kRoutePerThread);
  int tile_v = 0;
  const int ev = block_exclusive_scan(__popc(tt.bits), s_warp, &tile_v);
  const int tile_len = min(kRouteTile, M - tile * kRouteTile);
  const int tile_t = tile_len - tile_v;
  const int pre_v = static_cast<int>(ws[1 + tile]);
  const int pre_t = tile * kRouteTile - pre_v;
  // both lists sit in shared memory at the alignment (mod 4 elements) of their places in perm
  int* s_v = s_list + (pre_v & 3);
  int* s_t = s_list + ((((pre_v & 3) + tile_v + 3) & ~3) + ((cap + pre_t) & 3));
  compact_tile(s_v, s_t, tile, tt.bits, ev, tt.valid);
  __syncthreads();
  store_list_bulk(perm + pre_v, s_v, tile_v, 0);
  store_list_bulk(perm + cap + pre_t, s_t, tile_t, 128);
}

// -------------------------------------------------------------------------------------------
// Long masks whose BITS fit in shared memory (one bit per token: 2^26 tokens are 8 MiB over the whole
// GPU): one launch that reads the mask once.  The grid is exactly what the device holds at once (four
// CTAs per SM); CTA c owns the consecutive tiles [c * T, (c + 1) * T).
//   phase 1: read the owned mask bytes (four tiles' loads in flight per thread), keep them as bits in
//            shared memory, count visual tokens and runs, publish the CTA's count;
//   grid-wide wait (bounded: ST_TIMEOUT_GRID if the CTAs are not all resident at once);
//   the CTA's exclusive prefix = sum of the counts published by the CTAs before it;
//   phase 2: per tile scan + compaction from the bits, lists out by bulk copies as in the scatter kernel.
// 5 bytes per token of DRAM traffic, no chain of prefixes, no second read of the mask.
// ws: [0] run total, [1 .. 1 + gridDim) per-CTA visual count.
// -------------------------------------------------------------------------------------------
constexpr int kResidentPerSm = 4;
constexpr int kResidentSlots = 64;
constexpr int kResidentMaxCtas = 1024;
// grid-wide wait counters, one slot per launch in turn; monotonic (launch n on a slot waits for
// (n + 1) * gridDim arrivals, and the grid size never changes on a device), zero when the library is loaded
static __device__ unsigned long long g_route_barrier[kResidentSlots];

__device__ __forceinline__ unsigned long long route_ld_acquire_u64(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}

// block-wide sums of two values; contains two __syncthreads()
__device__ __forceinline__ void block_sum2(int a, int b, int (*s_red)[kRouteThreads / 32], int* out_a, int* out_b) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  a = __reduce_add_sync(0xFFFFFFFFu, a);
  b = __reduce_add_sync(0xFFFFFFFFu, b);
  __syncthreads();                       // earlier readers of s_red are done
  if (lane == 0) { s_red[0][warp] = a; s_red[1][warp] = b; }
  __syncthreads();
  int ta = 0, tb = 0;
#pragma unroll
  for (int i = 0; i < kRouteThreads / 32; ++i) { ta += s_red[0][i]; tb += s_red[1][i]; }
  *out_a = ta;
  *out_b = tb;
}

__global__ void __launch_bounds__(kRouteThreads, kResidentPerSm)
route_resident_kernel(const uint8_t* __restrict__ mask, int M, int cap, int num_tiles, int tiles_per_cta,
                      int* __restrict__ perm, int* __restrict__ counts, uint32_t* __restrict__ ws, int slot,
                      int* __restrict__ status) {
  extern __shared__ __align__(16) int s_dyn[];   // list staging of one tile, then the owned tiles' bits (256 words a tile)
  int* s_list = s_dyn;
  uint32_t* s_bits = reinterpret_cast<uint32_t*>(s_dyn + kRouteTile + 16);
  __shared__ int s_warp[kRouteThreads / 32];
  __shared__ int s_red[2][kRouteThreads / 32];
  __shared__ int s_ok;
  const int tid = threadIdx.x;
  const int tile_begin = blockIdx.x * tiles_per_cta;
  const int my_tiles = max(0, min(tiles_per_cta, num_tiles - tile_begin));
  const bool aligned = (reinterpret_cast<uintptr_t>(mask) & 15) == 0;

  // ---- phase 1: mask bytes -> bits in shared memory
  int nv = 0;
  for (int t0 = 0; t0 < my_tiles; t0 += kCountTiles) {
    uint32_t bits[kCountTiles];
    if (aligned && static_cast<int64_t>(tile_begin + t0 + kCountTiles) * kRouteTile <= M) {
      uint4 v[kCountTiles][2];
#pragma unroll
      for (int j = 0; j < kCountTiles; ++j) {
        const int base = (tile_begin + t0 + j) * kRouteTile + tid * kRoutePerThread;
        v[j][0] = *reinterpret_cast<const uint4*>(mask + base);
        v[j][1] = *reinterpret_cast<const uint4*>(mask + base + 16);
      }
#pragma unroll
      for (int j = 0; j < kCountTiles; ++j) {
        const uint32_t w[8] = {v[j][0].x, v[j][0].y, v[j][0].z, v[j][0].w, v[j][1].x, v[j][1].y, v[j][1].z, v[j][1].w};
        bits[j] = mask_words_to_bits(w);
      }
    } else {
#pragma unroll
      for (int j = 0; j < kCountTiles; ++j)
        bits[j] = load_thread_tokens(mask, M, (tile_begin + t0 + j) * kRouteTile + tid * kRoutePerThread).bits;
    }
#pragma unroll
    for (int j = 0; j < kCountTiles; ++j) {
      if (t0 + j < my_tiles) {
        s_bits[(t0 + j) * kRouteThreads + tid] = bits[j];
        nv += __popc(bits[j]);
      }
    }
  }
  __syncthreads();
  // runs: a token whose modality differs from its predecessor's (token 0 always); the predecessor of a
  // word's first token is the last bit of the word before it in shared memory
  int nruns = 0;
  for (int t = 0; t < my_tiles; ++t) {
    const int base = (tile_begin + t) * kRouteTile + tid * kRoutePerThread;
    const int valid = min(kRoutePerThread, M - base);
    if (valid > 0) {
      const uint32_t b = s_bits[t * kRouteThreads + tid];
      uint32_t prev;
      if (t == 0 && tid == 0) prev = base > 0 ? (mask[base - 1] != 0 ? 1u : 0u) : ((b & 1u) ^ 1u);
      else prev = s_bits[t * kRouteThreads + tid - 1] >> 31;
      const uint32_t vmask = valid == 32 ? 0xFFFFFFFFu : ((1u << valid) - 1u);
      nruns += __popc((b ^ ((b << 1) | prev)) & vmask);
    }
  }
  int cta_v = 0, cta_runs = 0;
  block_sum2(nv, nruns, s_red, &cta_v, &cta_runs);

  // ---- publish, then wait for the whole grid
  if (tid == 0) {
    ws[1 + blockIdx.x] = static_cast<uint32_t>(cta_v);
    if (cta_runs) atomicAdd(&ws[0], static_cast<uint32_t>(cta_runs));
    __threadfence();
    unsigned long long* bar = &g_route_barrier[slot];
    const unsigned long long ticket = atomicAdd(bar, 1ULL);
    const unsigned long long target = (ticket / gridDim.x + 1ULL) * gridDim.x;
    const uint64_t t0 = globaltimer_ns();
    uint32_t polls = 0;
    int ok = 1;
    while (route_ld_acquire_u64(bar) < target) {
      if ((++polls & 63u) == 0 && globaltimer_ns() - t0 > kWaitBudgetNs) {
        atomicCAS(status, 0, ST_TIMEOUT_GRID);
        ok = 0;
        break;
      }
    }
    s_ok = ok;
  }
  __syncthreads();
  if (!s_ok) return;

  // ---- visual tokens before this CTA's first tile, and in all
  int part = 0, all = 0;
  for (int j = tid; j < static_cast<int>(gridDim.x); j += kRouteThreads) {
    const int c = static_cast<int>(__ldcg(ws + 1 + j));
    all += c;
    if (j < static_cast<int>(blockIdx.x)) part += c;
  }
  int pre_v = 0, total_v = 0;
  block_sum2(part, all, s_red, &pre_v, &total_v);
  if (blockIdx.x == 0 && tid == 0) {
    counts[0] = total_v;
    counts[1] = M - total_v;
    counts[2] = cap;
    counts[3] = M;
    counts[4] = static_cast<int>(__ldcg(ws));
  }

  // ---- phase 2: lists
  for (int t = 0; t < my_tiles; ++t) {
    const int tile = tile_begin + t;
    const uint32_t b = s_bits[t * kRouteThreads + tid];
    int tile_v = 0;
    const int ev = block_exclusive_scan(__popc(b), s_warp, &tile_v);
    const int tile_len = min(kRouteTile, M - tile * kRouteTile);
    const int valid = max(0, min(kRoutePerThread, tile_len - tid * kRoutePerThread));
    const int tile_t = tile_len - tile_v;
    const int pre_t = tile * kRouteTile - pre_v;
    int* s_v = s_list + (pre_v & 3);
    int* s_t = s_list + ((((pre_v & 3) + tile_v + 3) & ~3) + ((cap + pre_t) & 3));
    compact_tile(s_v, s_t, tile, b, ev, valid);
    __syncthreads();
    store_list_bulk(perm + pre_v, s_v, tile_v, 0);
    store_list_bulk(perm + cap + pre_t, s_t, tile_t, 128);
    pre_v += tile_v;
    __syncthreads();      // the bulk copies have read the lists: the next tile may overwrite them
  }
}

// Largest number of tiles per CTA for which kResidentPerSm CTAs of the resident kernel fit on an SM
// (0: the kernel cannot be used on this device); found once per process.
static int resident_max_tiles_per_cta() {
  static int cached = -1;
  static std::mutex mu;
  std::lock_guard<std::mutex> lock(mu);
  if (cached >= 0) return cached;
  cached = 0;
  const DeviceInfo& dev = device_info();
  if (dev.sm_count * kResidentPerSm > kResidentMaxCtas) return cached;
  for (int t = 40; t >= 1; --t) {
    const size_t smem = (kRouteTile + 16) * sizeof(int) + static_cast<size_t>(t) * kRouteThreads * sizeof(uint32_t);
    if (smem > static_cast<size_t>(dev.smem_optin)) continue;
    if (cudaFuncSetAttribute(route_resident_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) !=
        cudaSuccess) {
      cudaGetLastError();
      continue;
    }
    int blocks = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&blocks, route_resident_kernel, kRouteThreads, smem) != cudaSuccess) {
      cudaGetLastError();
      continue;
    }
    if (blocks >= kResidentPerSm) {
      cached = t;
      break;
    }
  }
  return cached;
}

__global__ void route_empty_kernel(int* counts, int cap) {
  counts[0] = 0; counts[1] = 0; counts[2] = cap; counts[3] = 0; counts[4] = 0;
}

// One tile: a single kernel that never looks back (its state word need not be cleared).  Up to
// kLookBackMaxTiles tiles: the single-pass chained scan.  Beyond: count, then scatter.
static int route_launch(const uint8_t* mask, int M, int cap, int* perm, int* counts, uint32_t* ws, int* status,
                        cudaStream_t stream) {
  const int tiles = (M + kRouteTile - 1) / kRouteTile;
  if (tiles > kLookBackMaxTiles) {
    const int grid = device_info().sm_count * kResidentPerSm;
    const int per_cta = (tiles + grid - 1) / grid;
    if (tune_overrides().route_resident != 0 && per_cta <= resident_max_tiles_per_cta()) {
      cudaError_t e = cudaMemsetAsync(ws, 0, sizeof(uint32_t), stream);      // the run total
      if (e != cudaSuccess) return cuda_status(e);
      static unsigned launch_seq = 0;   // successive launches take successive barrier slots
      const int slot = static_cast<int>(__atomic_fetch_add(&launch_seq, 1u, __ATOMIC_RELAXED) % kResidentSlots);
      const size_t smem = (kRouteTile + 16) * sizeof(int) + static_cast<size_t>(per_cta) * kRouteThreads * sizeof(uint32_t);
      route_resident_kernel<<<grid, kRouteThreads, smem, stream>>>(mask, M, cap, tiles, per_cta, perm, counts, ws, slot, status);
      return cuda_status(cudaGetLastError());
    }
  }
  if (tiles > 1) {
    cudaError_t e = cudaMemsetAsync(ws, 0, (static_cast<size_t>(tiles) + 2) * sizeof(uint32_t), stream);
    if (e != cudaSuccess) return cuda_status(e);
  }
  if (tiles <= kLookBackMaxTiles) {
    route_kernel<<<tiles, kRouteThreads, 0, stream>>>(mask, M, cap, perm, counts, ws, status);
    return cuda_status(cudaGetLastError());
  }
  route_count_kernel<<<(tiles + kCountTiles - 1) / kCountTiles, kRouteThreads, 0, stream>>>(mask, M, cap, tiles, counts, ws);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_status(e);
  route_scatter_kernel<<<tiles, kRouteThreads, 0, stream>>>(mask, M, cap, perm, ws);
  return cuda_status(cudaGetLastError());
}

}  // namespace ffnk

using namespace ffnk;

extern "C" int64_t ffnk_route_capacity(int64_t M) { return ((M + 127) / 128) * 128; }

extern "C" int64_t ffnk_route_workspace_bytes(int64_t M) {
  // one word per tile (count + scatter) or per CTA of the resident kernel, plus the run total and a counter
  const int64_t tiles = (M + kRouteTile - 1) / kRouteTile;
  return ((tiles > kResidentMaxCtas ? tiles : kResidentMaxCtas) + 2) * static_cast<int64_t>(sizeof(uint32_t));
}

extern "C" int ffnk_route(const void* mask, int64_t M, int32_t* perm, int32_t* counts, void* workspace,
                          int32_t* status, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (M < 0 || M >= (1ll << 30)) return FFNK_ERR_SHAPE;
  if (!counts || !status) return FFNK_ERR_NULL;
  const int cap = static_cast<int>(ffnk_route_capacity(M));
  if (M == 0) {
    route_empty_kernel<<<1, 1, 0, stream>>>(counts, cap);
    return cuda_status(cudaGetLastError());
  }
  if (!mask || !perm || !workspace) return FFNK_ERR_NULL;
  if (reinterpret_cast<uintptr_t>(perm) & 15) return FFNK_ERR_ALIGN;
  return route_launch(static_cast<const uint8_t*>(mask), static_cast<int>(M), cap, perm, counts,
                      static_cast<uint32_t*>(workspace), status, stream);
}

// -------------------------------------------------------------------------------------------
// Row permutation into routed order: out[routed row of token t] = x[t].
//
// The GEMMs can gather token rows themselves (TMA boxes for runs of consecutive tokens, gather4
// for ragged rows), but every row tile that straddles a run boundary then costs several TMA
// instructions per k-step, and the TMA unit retires only about one instruction per 40 ns.  For
// wide FFNs one extra pass over x (2 * M * d * 2 bytes of HBM traffic, a percent or two of the
// GEMM time) is cheaper: afterwards every A tile is one tiled box whatever the mask looks like.
// Routed layout as for the FFN intermediate: visual rows from row 0, text rows from row
// 256 * ceil(Mv / 256).  HBM bound; algorithmic traffic 4 * d bytes per token.
// -------------------------------------------------------------------------------------------
namespace ffnk {
constexpr int kPermuteThreads = 256;

__global__ void __launch_bounds__(kPermuteThreads) permute_rows_kernel(const uint4* __restrict__ x, int64_t ldx16,
                                                                       const int* __restrict__ perm,
                                                                       const int* __restrict__ counts,
                                                                       uint4* __restrict__ out, int64_t ldo16,
                                                                       int chunks, int only_if_scattered) {
  // optional gate (only_if_scattered = run-length threshold): the copy is wanted only when the mask
  // is scattered; its consumer makes the same test with the same threshold
  if (only_if_scattered && !mask_is_scattered(counts, only_if_scattered)) return;
  const int Mv = counts[0], Mt = counts[1], cap = counts[2];
  const int M = Mv + Mt;
  const int text_base = ((Mv + 255) >> 8) << 8;
  const int warps_per_block = kPermuteThreads / 32;
  const int lane = threadIdx.x & 31;
  for (int i = blockIdx.x * warps_per_block + (threadIdx.x >> 5); i < M; i += gridDim.x * warps_per_block) {
    const bool text = i >= Mv;
    const int tok = text ? perm[cap + (i - Mv)] : perm[i];
    const int64_t dst = text ? static_cast<int64_t>(text_base) + (i - Mv) : i;
    const uint4* src_row = x + static_cast<int64_t>(tok) * ldx16;
    uint4* dst_row = out + dst * ldo16;
    for (int c = lane; c < chunks; c += 128) {
      uint4 v0, v1, v2, v3;
      const bool b1 = c + 32 < chunks, b2 = c + 64 < chunks, b3 = c + 96 < chunks;
      v0 = __ldg(src_row + c);
      if (b1) v1 = __ldg(src_row + c + 32);
      if (b2) v2 = __ldg(src_row + c + 64);
      if (b3) v3 = __ldg(src_row + c + 96);
      dst_row[c] = v0;
      if (b1) dst_row[c + 32] = v1;
      if (b2) dst_row[c + 64] = v2;
      if (b3) dst_row[c + 96] = v3;
    }
  }
}

// Routing and the copy into routed order in ONE launch, for masks of a single tile (M <= 8192): every CTA
// routes the whole mask for itself (8 KiB of mask out of L2, a block scan and a compaction in shared
// memory: a few microseconds, less than a second launch costs), CTA 0 also writes perm and counts for the
// GEMMs that follow, and then every warp copies its share of the rows, reading the row list from shared
// memory.  Same results as route_kernel followed by permute_rows_kernel.
__global__ void __launch_bounds__(kRouteThreads) route_permute_kernel(const uint8_t* __restrict__ mask, int M, int cap,
                                                                      int* __restrict__ perm, int* __restrict__ counts,
                                                                      const uint4* __restrict__ x, int64_t ldx16,
                                                                      uint4* __restrict__ out, int64_t ldo16, int chunks) {
  __shared__ int s_list[kRouteTile];   // visual tokens ascending, then text tokens ascending
  __shared__ int s_warp[kRouteThreads / 32];
  __shared__ int s_runs;
  const int tid = threadIdx.x;
  griddep_launch_dependents();         // the GEMM behind this kernel may set itself up and ask its weights into L2
  const ThreadTokens tt = load_thread_tokens(mask, M, tid * kRoutePerThread);
  if (tid == 0) s_runs = 0;
  int Mv = 0;
  const int ev = block_exclusive_scan(__popc(tt.bits), s_warp, &Mv);
  if (blockIdx.x == 0) {
    const int wr = __reduce_add_sync(0xFFFFFFFFu, tt.nruns);
    if ((tid & 31) == 0 && wr) atomicAdd(&s_runs, wr);
  }
  compact_tile(s_list, s_list + Mv, 0, tt.bits, ev, tt.valid);
  __syncthreads();
  const int Mt = M - Mv;
  if (blockIdx.x == 0) {
    for (int i = tid; i < Mv; i += kRouteThreads) perm[i] = s_list[i];
    for (int i = tid; i < Mt; i += kRouteThreads) perm[cap + i] = s_list[Mv + i];
    if (tid == 0) {
      counts[0] = Mv;
      counts[1] = Mt;
      counts[2] = cap;
      counts[3] = M;
      counts[4] = s_runs;
    }
  }
  const int text_base = ((Mv + 255) >> 8) << 8;
  const int warps_per_block = kRouteThreads / 32;
  const int lane = tid & 31;
  for (int i = blockIdx.x * warps_per_block + (tid >> 5); i < M; i += gridDim.x * warps_per_block) {
    const int tok = s_list[i];
    const int64_t dst = i >= Mv ? static_cast<int64_t>(text_base) + (i - Mv) : i;
    const uint4* src_row = x + static_cast<int64_t>(tok) * ldx16;
    uint4* dst_row = out + dst * ldo16;
    for (int c = lane; c < chunks; c += 128) {
      uint4 v0, v1, v2, v3;
      const bool b1 = c + 32 < chunks, b2 = c + 64 < chunks, b3 = c + 96 < chunks;
      v0 = __ldg(src_row + c);
      if (b1) v1 = __ldg(src_row + c + 32);
      if (b2) v2 = __ldg(src_row + c + 64);
      if (b3) v3 = __ldg(src_row + c + 96);
      dst_row[c] = v0;
      if (b1) dst_row[c + 32] = v1;
      if (b2) dst_row[c + 64] = v2;
      if (b3) dst_row[c + 96] = v3;
    }
  }
}
}  // namespace ffnk

namespace ffnk {
int permute_rows_launch(const void* x, int64_t ldx, const int32_t* perm, const int32_t* counts, void* out, int64_t ldo,
                        int64_t M, int64_t d, int only_if_scattered, void* stream_);
}

extern "C" int64_t ffnk_route_permute_max_tokens(void) { return kRouteTile; }

extern "C" int ffnk_route_permute_rows(const void* mask, int64_t M, const void* x, int64_t ldx, int64_t d, int32_t* perm,
                                       int32_t* counts, void* out, int64_t ldo, void* stream_) {
  if (!counts) return FFNK_ERR_NULL;
  if (M < 0 || M > kRouteTile) return FFNK_ERR_SHAPE;
  const int cap = static_cast<int>(ffnk_route_capacity(M));
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (M == 0) {
    route_empty_kernel<<<1, 1, 0, stream>>>(counts, cap);
    return cuda_status(cudaGetLastError());
  }
  if (!mask || !x || !perm || !out) return FFNK_ERR_NULL;
  if (d < 8 || (d & 7) || d >= (1ll << 30)) return FFNK_ERR_SHAPE;
  if ((ldx & 7) || (ldo & 7) || ldx < d || ldo < d || (reinterpret_cast<uintptr_t>(x) & 15) ||
      (reinterpret_cast<uintptr_t>(out) & 15) || (reinterpret_cast<uintptr_t>(perm) & 15))
    return FFNK_ERR_ALIGN;
  const DeviceInfo& dev = device_info();
  int64_t blocks = (M + 7) / 8;
  const int64_t max_blocks = static_cast<int64_t>(dev.sm_count) * 4;
  if (blocks > max_blocks) blocks = max_blocks;
  route_permute_kernel<<<static_cast<unsigned>(blocks), kRouteThreads, 0, stream>>>(
      static_cast<const uint8_t*>(mask), static_cast<int>(M), cap, perm, counts, static_cast<const uint4*>(x), ldx / 8,
      static_cast<uint4*>(out), ldo / 8, static_cast<int>(d / 8));
  return cuda_status(cudaGetLastError());
}

extern "C" int ffnk_permute_rows(const void* x, int64_t ldx, const int32_t* perm, const int32_t* counts, void* out,
                                 int64_t ldo, int64_t M, int64_t d, void* stream_) {
  return permute_rows_launch(x, ldx, perm, counts, out, ldo, M, d, 0, stream_);
}

int ffnk::permute_rows_launch(const void* x, int64_t ldx, const int32_t* perm, const int32_t* counts, void* out,
                              int64_t ldo, int64_t M, int64_t d, int only_if_scattered, void* stream_) {
  if (M == 0) return 0;
  if (!x || !perm || !counts || !out) return FFNK_ERR_NULL;
  if (M < 0 || M >= (1ll << 30) || d < 8 || (d & 7) || d >= (1ll << 30)) return FFNK_ERR_SHAPE;
  if ((ldx & 7) || (ldo & 7) || ldx < d || ldo < d || (reinterpret_cast<uintptr_t>(x) & 15) ||
      (reinterpret_cast<uintptr_t>(out) & 15))
    return FFNK_ERR_ALIGN;
  const DeviceInfo& dev = device_info();
  int64_t blocks = (M + 7) / 8;
  const int64_t max_blocks = static_cast<int64_t>(dev.sm_count) * 8;
  if (blocks > max_blocks) blocks = max_blocks;
  permute_rows_kernel<<<static_cast<unsigned>(blocks), kPermuteThreads, 0, static_cast<cudaStream_t>(stream_)>>>(
      static_cast<const uint4*>(x), ldx / 8, perm, counts, static_cast<uint4*>(out), ldo / 8, static_cast<int>(d / 8), only_if_scattered);
  return cuda_status(cudaGetLastError());
}

// -------------------------------------------------------------------------------------------
// Sum of row blocks: out[r, c] = sum over b of blocks[b][r][c], bf16 in, fp32 sum, bf16 out.
// Second half of the tensor-parallel reduce-scatter whose first half is the down projection that
// writes every rank's partial rows into their owner's memory (ffnk_ffn_down_to_peers).
// -------------------------------------------------------------------------------------------
namespace ffnk {
__global__ void __launch_bounds__(256) sum_row_blocks_kernel(const uint4* __restrict__ blocks, int nblocks,
                                                             int64_t block_stride16, int64_t ld16, int64_t rows,
                                                             int chunks, uint4* __restrict__ out, int64_t ldo16) {
  const int64_t total = rows * chunks;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = i / chunks;
    const int c = static_cast<int>(i - r * chunks);
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    const uint4* src = blocks + r * ld16 + c;
#pragma unroll 4
    for (int b = 0; b < nblocks; ++b) {
      const uint4 v = __ldg(src + b * block_stride16);
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        acc[2 * e] += __uint_as_float(w[e] << 16);
        acc[2 * e + 1] += __uint_as_float(w[e] & 0xFFFF0000u);
      }
    }
    uint4 o;
    uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const __nv_bfloat162 h2 = __floats2bfloat162_rn(acc[2 * e], acc[2 * e + 1]);
      ow[e] = *reinterpret_cast<const uint32_t*>(&h2);
    }
    out[r * ldo16 + c] = o;
  }
}
}  // namespace ffnk

extern "C" int ffnk_sum_row_blocks(const void* blocks, int nblocks, int64_t rows, int64_t d, int64_t ldb, void* out,
                                   int64_t ldo, void* stream) {
  if (rows == 0) return 0;
  if (!blocks || !out) return FFNK_ERR_NULL;
  if (nblocks < 1 || nblocks > 64 || rows < 0 || rows >= (1ll << 30) || d < 8 || (d & 7) || d >= (1ll << 30))
    return FFNK_ERR_SHAPE;
  if ((ldb & 7) || (ldo & 7) || ldb < d || ldo < d || (reinterpret_cast<uintptr_t>(blocks) & 15) ||
      (reinterpret_cast<uintptr_t>(out) & 15))
    return FFNK_ERR_ALIGN;
  const ffnk::DeviceInfo& dev = ffnk::device_info();
  const int64_t total = rows * (d / 8);
  int64_t grid = (total + 255) / 256;
  const int64_t max_grid = static_cast<int64_t>(dev.sm_count) * 8;
  if (grid > max_grid) grid = max_grid;
  ffnk::sum_row_blocks_kernel<<<static_cast<unsigned>(grid), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(blocks), nblocks, rows * (ldb / 8), ldb / 8, rows, static_cast<int>(d / 8),
      static_cast<uint4*>(out), ldo / 8);
  return ffnk::cuda_status(cudaGetLastError());
}

// -------------------------------------------------------------------------------------------
// Routing without any allocation by anybody.
//
// ffnk_route() needs a few kilobytes of scan state that the caller has to allocate.  Some hosts
// cannot do that at the point where they call us: an inference-server or runtime plugin whose
// execute callback is given all its buffers up front and is forbidden to allocate device memory,
// or a steady-state serving loop that must not touch cudaMalloc because it synchronises the
// whole device.  For them the scan state lives in the fixed array below.  It is part of the
// library image, so every GPU that loads the library carries these 8.25 KiB until the process
// exits, and it bounds the mask length at FFNK_ROUTE_NOALLOC_MAX_TOKENS.
// -------------------------------------------------------------------------------------------
namespace ffnk {
constexpr int64_t kNoAllocMaxTokens = FFNK_ROUTE_NOALLOC_MAX_TOKENS;
constexpr int64_t kNoAllocWords = 2 + (kNoAllocMaxTokens + kRouteTile - 1) / kRouteTile;   // one spare word + tile states
constexpr int64_t kNoAllocWordsPadded = ((kNoAllocWords + 63) / 64) * 64;

static __device__ __align__(256) uint32_t g_route_scratch[kNoAllocWordsPadded];
// the workspace layout of route_launch is [run total][one word per tile][finished tiles]
static_assert(kNoAllocWordsPadded >= (kNoAllocMaxTokens + kRouteTile - 1) / kRouteTile + 2,
              "the fixed array must hold the scan state of a mask of FFNK_ROUTE_NOALLOC_MAX_TOKENS tokens");

// In host code `g_route_scratch` is only a handle for the runtime, not an address a kernel can
// use: the device address is asked for once per device (with that device current) and cached.
static int route_scratch_address(uint32_t** out, cudaStream_t stream) {
  static std::mutex mu;
  static uint32_t* addr[64] = {};
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_status(e);
  if (dev < 0 || dev >= 64) return FFNK_ERR_DEVICE;
  std::lock_guard<std::mutex> lock(mu);
  if (addr[dev] == nullptr) {
    // The lookup is not a stream operation; made while `stream` is being captured it could break the
    // capture and the caller would see only an opaque runtime error.  Refuse instead, launching nothing.
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(stream, &cap) == cudaSuccess && cap != cudaStreamCaptureStatusNone)
      return FFNK_ERR_CAPTURE;
    uint32_t* ptr = nullptr;
    e = cudaGetSymbolAddress((void**)&ptr, g_route_scratch);
    if (e != cudaSuccess) return cuda_status(e);
    if (ptr == nullptr) return FFNK_ERR_DEVICE;
    addr[dev] = ptr;
  }
  *out = addr[dev];
  return 0;
}
}  // namespace ffnk

extern "C" int ffnk_route_noalloc(const void* mask, int64_t M, int32_t* perm, int32_t* counts, int32_t* status,
                                  void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (M < 0) return FFNK_ERR_SHAPE;
  if (M > kNoAllocMaxTokens) return FFNK_ERR_CAPACITY;
  if (!counts || !status) return FFNK_ERR_NULL;
  const int cap = static_cast<int>(ffnk_route_capacity(M));
  if (M == 0) {
    route_empty_kernel<<<1, 1, 0, stream>>>(counts, cap);
    return cuda_status(cudaGetLastError());
  }
  if (!mask || !perm) return FFNK_ERR_NULL;
  if (reinterpret_cast<uintptr_t>(perm) & 15) return FFNK_ERR_ALIGN;
  uint32_t* scratch = nullptr;
  const int r = route_scratch_address(&scratch, stream);
  if (r) return r;
  // the array still holds the previous call's tile states: route_launch clears the part this call uses
  return route_launch(static_cast<const uint8_t*>(mask), static_cast<int>(M), cap, perm, counts, scratch, status,
                      stream);
}
