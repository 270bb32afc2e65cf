// Tensor parallel over h, the part after the down projection: a barrier between the ranks and the
// owner's block sum that hands the finished rows to every rank -- both over peer-mapped memory
// (NVLink), with this library's own kernels.
//
// The down projection (ffnk_ffn_down_to_peers, routed_gemm.cu) has stored every rank's partial rows
// into the block buffer of the rank that owns them.  What remains of the all-reduce is
//   1. a barrier: every rank's partial rows have landed in their owners' buffers,
//   2. per owner: out[row] = bf16(sum over ranks of fp32(partial[rank][row])), stored into the output
//      matrix of EVERY rank (plain 16-byte peer stores, a warp writes 512 contiguous bytes of a row),
//   3. a barrier: every rank's output matrix is complete.
// Only plain loads and stores of peer memory are used: no TMA on peer memory, no multicast, no
// multimem.  The barrier spins on flags in this rank's own memory that the peers set; the spin is
// bounded and reports ST_TIMEOUT_RANK instead of hanging when a rank never arrives.
//
// The reference is single-device (test_linear.py:74 selects device 0); nothing here has a
// counterpart in it.
#include <cuda_bf16.h>

#include "ffnk_internal.h"
#include "ptx.cuh"

namespace ffnk {

constexpr int kMaxPeers = 8;

struct PeerPtrs {
  void* p[kMaxPeers];
};

__device__ __forceinline__ void st_release_sys(int* addr, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* addr) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
  return v;
}

// One warp.  Lane r < world: tell rank r that this rank has arrived (slot `rank` of its flag array),
// then wait until rank r has arrived here (slot r of this rank's own array).  Epochs only grow, so a
// peer that is already one barrier ahead satisfies the wait as well.
__global__ void __launch_bounds__(32) peer_barrier_kernel(const PeerPtrs flags, int world, int rank, int epoch,
                                                          uint64_t budget_ns, int* status) {
  const int lane = threadIdx.x;
  if (lane >= world) return;
  __threadfence_system();   // everything this rank's earlier kernels wrote, to peers too, comes first
  st_release_sys(static_cast<int*>(flags.p[lane]) + rank, epoch);
  const int* mine = static_cast<const int*>(flags.p[rank]) + lane;
  const uint64_t t0 = globaltimer_ns();
  uint32_t polls = 0;
  while (ld_acquire_sys(mine) - epoch < 0) {
    if ((++polls & 63u) == 0 && globaltimer_ns() - t0 > budget_ns) {
      if (status) atomicCAS(status, 0, ST_TIMEOUT_RANK);
      break;
    }
  }
}

// out_r[out_row0 + row][c] = bf16(sum_b fp32(blocks[b][row][c])) for every rank r.
// One thread per 16-byte piece; consecutive threads take consecutive pieces of a row, so a warp
// reads 512 contiguous bytes from each block and stores 512 contiguous bytes to each rank.
__global__ void __launch_bounds__(256) sum_blocks_to_peers_kernel(const uint4* __restrict__ blocks, int nblocks,
                                                                  int64_t block_stride16, int64_t ld16, int64_t rows,
                                                                  int chunks, const PeerPtrs out, int world,
                                                                  int64_t out_row0, int64_t ldo16) {
  const int64_t total = rows * chunks;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = i / chunks;
    const int c = static_cast<int>(i - r * chunks);
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    const uint4* src = blocks + r * ld16 + c;
    uint4 v[kMaxPeers];
#pragma unroll
    for (int b = 0; b < kMaxPeers; ++b)
      if (b < nblocks) v[b] = __ldg(src + b * block_stride16);
#pragma unroll
    for (int b = 0; b < kMaxPeers; ++b) {
      if (b < nblocks) {
        const uint32_t w[4] = {v[b].x, v[b].y, v[b].z, v[b].w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          acc[2 * e] += __uint_as_float(w[e] << 16);
          acc[2 * e + 1] += __uint_as_float(w[e] & 0xFFFF0000u);
        }
      }
    }
    uint4 o;
    uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const __nv_bfloat162 h2 = __floats2bfloat162_rn(acc[2 * e], acc[2 * e + 1]);
      ow[e] = *reinterpret_cast<const uint32_t*>(&h2);
    }
    const int64_t off = (out_row0 + r) * ldo16 + c;
#pragma unroll
    for (int q = 0; q < kMaxPeers; ++q)
      if (q < world) static_cast<uint4*>(out.p[q])[off] = o;
  }
}

}  // namespace ffnk

using namespace ffnk;

extern "C" int ffnk_peer_barrier(void* const* flags, int world, int rank, int32_t epoch, int64_t budget_us,
                                 int32_t* status, void* stream) {
  if (!flags) return FFNK_ERR_NULL;
  if (world < 1 || world > kMaxPeers || rank < 0 || rank >= world || budget_us < 0 || budget_us > 10000000)
    return FFNK_ERR_SHAPE;
  PeerPtrs f{};
  for (int r = 0; r < world; ++r) {
    if (!flags[r]) return FFNK_ERR_NULL;
    if (reinterpret_cast<uintptr_t>(flags[r]) & 3) return FFNK_ERR_ALIGN;
    f.p[r] = flags[r];
  }
  const uint64_t budget_ns = budget_us ? static_cast<uint64_t>(budget_us) * 1000ull : kWaitBudgetNs;
  peer_barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(f, world, rank, epoch, budget_ns, status);
  return cuda_status(cudaGetLastError());
}

extern "C" int ffnk_sum_row_blocks_to_peers(const void* blocks, int nblocks, int64_t block_rows, int64_t rows, int64_t d,
                                            int64_t ldb, void* const* peer_out, int world, int64_t out_row0,
                                            int64_t ldo, int max_ctas, void* stream) {
  if (rows == 0) return 0;
  if (!blocks || !peer_out) return FFNK_ERR_NULL;
  if (nblocks < 1 || nblocks > kMaxPeers || world < 1 || world > kMaxPeers || rows < 0 || rows > block_rows ||
      block_rows >= (1ll << 30) ||
      out_row0 < 0 || out_row0 >= (1ll << 30) || d < 8 || (d & 7) || d >= (1ll << 30) || max_ctas < 0)
    return FFNK_ERR_SHAPE;
  if ((ldb & 7) || (ldo & 7) || ldb < d || ldo < d || (reinterpret_cast<uintptr_t>(blocks) & 15)) return FFNK_ERR_ALIGN;
  PeerPtrs out{};
  for (int r = 0; r < world; ++r) {
    if (!peer_out[r]) return FFNK_ERR_NULL;
    if (reinterpret_cast<uintptr_t>(peer_out[r]) & 15) return FFNK_ERR_ALIGN;
    out.p[r] = peer_out[r];
  }
  const DeviceInfo& dev = device_info();
  const int64_t total = rows * (d / 8);
  int64_t grid = (total + 255) / 256;
  const int64_t max_grid = max_ctas > 0 ? max_ctas : static_cast<int64_t>(dev.sm_count) * 8;
  if (grid > max_grid) grid = max_grid;
  sum_blocks_to_peers_kernel<<<static_cast<unsigned>(grid), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(blocks), nblocks, block_rows * (ldb / 8), ldb / 8, rows, static_cast<int>(d / 8), out, world,
      out_row0, ldo / 8);
  return cuda_status(cudaGetLastError());
}
