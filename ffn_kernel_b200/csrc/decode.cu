// Small-M (decode) MaskedFFN forward: a weight-streaming kernel pair for M <= 32 tokens.
//
// With a handful of tokens the FFN is a matrix-vector product: every weight of each modality
// that is present is read exactly once (3*d*h bf16 per modality) and the arithmetic is tiny,
// so the kernels are built around the HBM stream, not around a 128-row tensor tile:
//   * every lane fetches weights with 128-bit loads straight from the weight's own storage
//     (K-major, the nn.Linear.weight.T view); nothing is staged through shared memory;
//   * the tokens of the modality, in groups of eight, form the N = 8 side of mma.sync.m16n8k16
//     (bf16 in, fp32 accumulate; up to 4 groups per CTA, each weight fragment reused by all).  The k-slots of the instruction are assigned so that one 16-byte chunk of a
//     weight row and the same 16-byte chunk of a token row feed two MMAs directly from
//     registers, with no shuffles: lane (g, t) of the warp holds chunk t of rows g and g+8;
//   * the contraction is split over the warps of a CTA (8 for gate/up, 16 for down) and summed
//     through shared memory; at d = 1024 / h = 2816 every lane issues all of its weight loads
//     in one batch, so a CTA pays HBM latency once.
// The two phases (gate/up with the SiLU(t1)*t3 epilogue, then the down projection) are two
// launches chained with programmatic dependent launch: the second kernel's CTAs start early,
// pull their first weights, and wait for the first kernel only before they read the
// intermediate.
//
// Same contract as MaskedFFN.forward (ffn_kernel/ops.py:28-32); the intermediate is rounded to
// bf16 between the phases as in the reference (ffn_kernel/ffn.py:113).
#include <cuda_bf16.h>

#include "ffnk_internal.h"
#include "ptx.cuh"

namespace ffnk {

// Beyond ~32 tokens the token rows (re-read by every CTA) outweigh the weight stream and the
// tcgen05 GEMM path is faster (measured at d=1024/h=2816: 16 tokens 17 us, 64 tokens 45 us against 39 us).
constexpr int kDecodeMaxTokens = 32;
constexpr int kDecodeRows = 16;   // weight rows per CTA (the M side of m16n8k16)

__device__ __forceinline__ uint4 ld_stream_16(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

__device__ __forceinline__ void mma_bf16_16x8x16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                                 uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait_primary() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

struct DecodeParams {
  const __nv_bfloat16* x;      // [M, K] input rows of this phase (activations, or the intermediate)
  int64_t ldx;
  const __nv_bfloat16* wa[2];  // first weight per modality ([rows, K] storage): gate, or down
  const __nv_bfloat16* wb[2];  // second weight per modality (up); unused in the down phase
  int64_t ldw;                 // elements between weight rows
  const uint8_t* mask;
  __nv_bfloat16* out;          // [M, rows]
  int64_t ldo;
  int M, K, rows;
};

// GATEUP: out[tok, r] = silu(x[tok] . wa[r]) * (x[tok] . wb[r]);  otherwise out[tok, r] = x[tok] . wa[r]
// WAIT_PRIMARY: this launch depends on the previous kernel in the stream for `x`.
// G: token groups of eight (the N side of the MMA) a CTA can hold; the modality's tokens fill
//    them in order and empty groups are skipped.
template <bool GATEUP, bool WAIT_PRIMARY, int WARPS, int UNROLL, int G>
__global__ void __launch_bounds__(WARPS * 32) decode_phase_kernel(const DecodeParams p) {
  constexpr int ACC = GATEUP ? 8 : 4;
  __shared__ float red[G][32][ACC];
  __shared__ int s_tok[G * 8];
  __shared__ int s_ntok;

  const int modality = blockIdx.y;          // 0: mask != 0 (first weight set), 1: mask == 0
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  if constexpr (!WAIT_PRIMARY) pdl_launch_dependents();

  for (int i = threadIdx.x; i < G * 32 * ACC; i += WARPS * 32) (&red[0][0][0])[i] = 0.f;
  if (warp == 0) {
    // 32 mask bytes per round, all loads of a round in flight together; token order is kept
    int base = 0;
#pragma unroll
    for (int r = 0; r < (G * 8 + 31) / 32; ++r) {
      const int idx = r * 32 + lane;
      const bool mine = idx < p.M && ((p.mask[idx] != 0) == (modality == 0));
      const uint32_t ballot = __ballot_sync(0xFFFFFFFFu, mine);
      if (mine) s_tok[base + __popc(ballot & ((1u << lane) - 1u))] = idx;
      base += __popc(ballot);
    }
    if (lane == 0) s_ntok = base;
  }
  __syncthreads();
  const int ntok = s_ntok;
  if (ntok == 0) return;
  const int ngroups = (ntok + 7) >> 3;

  const int r0 = blockIdx.x * kDecodeRows;
  const int row_lo = r0 + g, row_hi = r0 + g + 8;
  const bool lo_ok = row_lo < p.rows, hi_ok = row_hi < p.rows;
  const __nv_bfloat16* wa_lo = p.wa[modality] + static_cast<int64_t>(lo_ok ? row_lo : 0) * p.ldw;
  const __nv_bfloat16* wa_hi = p.wa[modality] + static_cast<int64_t>(hi_ok ? row_hi : 0) * p.ldw;
  const __nv_bfloat16* wb_lo = GATEUP ? p.wb[modality] + static_cast<int64_t>(lo_ok ? row_lo : 0) * p.ldw : nullptr;
  const __nv_bfloat16* wb_hi = GATEUP ? p.wb[modality] + static_cast<int64_t>(hi_ok ? row_hi : 0) * p.ldw : nullptr;
  // this lane supplies token slot g of every group
  const __nv_bfloat16* xrow[G];
#pragma unroll
  for (int gi = 0; gi < G; ++gi) {
    const int slot = gi * 8 + g;
    xrow[gi] = slot < ntok ? p.x + static_cast<int64_t>(s_tok[slot]) * p.ldx : nullptr;
  }

  float acc_a[G][4], acc_b[GATEUP ? G : 1][4];
#pragma unroll
  for (int gi = 0; gi < G; ++gi)
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      acc_a[gi][i] = 0.f;
      if (GATEUP) acc_b[gi][i] = 0.f;
    }
  const uint4 zero = make_uint4(0, 0, 0, 0);
  const int kblocks = (p.K + 31) / 32;      // 32 contraction elements per step: 4 lanes x 16 bytes per row

  bool waited = !WAIT_PRIMARY;
  for (int kb0 = warp; kb0 < kblocks; kb0 += WARPS * UNROLL) {
    uint4 a_lo[UNROLL], a_hi[UNROLL], b_lo[GATEUP ? UNROLL : 1], b_hi[GATEUP ? UNROLL : 1];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int k = (kb0 + u * WARPS) * 32 + t * 8;
      const bool k_ok = (kb0 + u * WARPS) < kblocks && k < p.K;
      a_lo[u] = (k_ok && lo_ok) ? ld_stream_16(wa_lo + k) : zero;
      a_hi[u] = (k_ok && hi_ok) ? ld_stream_16(wa_hi + k) : zero;
      if constexpr (GATEUP) {
        b_lo[u] = (k_ok && lo_ok) ? ld_stream_16(wb_lo + k) : zero;
        b_hi[u] = (k_ok && hi_ok) ? ld_stream_16(wb_hi + k) : zero;
      }
    }
    if (!waited) {   // the weights above do not depend on the previous kernel; the token rows do
      pdl_wait_primary();
      waited = true;
    }
#pragma unroll
    for (int gi = 0; gi < G; ++gi) {
      if (gi < ngroups) {
        uint4 xv[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
          const int k = (kb0 + u * WARPS) * 32 + t * 8;
          const bool k_ok = (kb0 + u * WARPS) < kblocks && k < p.K;
          xv[u] = (k_ok && xrow[gi] != nullptr) ? *reinterpret_cast<const uint4*>(xrow[gi] + k) : zero;
        }
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
          mma_bf16_16x8x16(acc_a[gi], a_lo[u].x, a_hi[u].x, a_lo[u].y, a_hi[u].y, xv[u].x, xv[u].y);
          mma_bf16_16x8x16(acc_a[gi], a_lo[u].z, a_hi[u].z, a_lo[u].w, a_hi[u].w, xv[u].z, xv[u].w);
          if constexpr (GATEUP) {
            mma_bf16_16x8x16(acc_b[gi], b_lo[u].x, b_hi[u].x, b_lo[u].y, b_hi[u].y, xv[u].x, xv[u].y);
            mma_bf16_16x8x16(acc_b[gi], b_lo[u].z, b_hi[u].z, b_lo[u].w, b_hi[u].w, xv[u].z, xv[u].w);
          }
        }
      }
    }
  }
  if (!waited) pdl_wait_primary();

  // sum the partial products of the warps in shared memory, one warp after the other: the order of
  // the fp32 additions is fixed, so the same inputs give the same bits on every run (shared-memory
  // atomics would be a few hundred cycles cheaper and make the last bit depend on warp timing)
#pragma unroll 1
  for (int w = 0; w < WARPS; ++w) {
    if (warp == w) {
#pragma unroll
      for (int gi = 0; gi < G; ++gi) {
        if (gi < ngroups) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            red[gi][lane][i] += acc_a[gi][i];
            if constexpr (GATEUP) red[gi][lane][4 + i] += acc_b[gi][i];
          }
        }
      }
    }
    __syncthreads();
  }
  for (int gi = warp; gi < ngroups; gi += WARPS) {
    // accumulator element i: row (g + 8 * (i >> 1)), token slot (2 t + (i & 1)) of the group
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int row = r0 + g + 8 * (i >> 1);
      const int slot = gi * 8 + 2 * t + (i & 1);
      if (row < p.rows && slot < ntok) {
        float v = red[gi][lane][i];
        if constexpr (GATEUP) v = v * __frcp_rn(1.0f + __expf(-v)) * red[gi][lane][4 + i];
        p.out[static_cast<int64_t>(s_tok[slot]) * p.ldo + row] = __float2bfloat16_rn(v);
      }
    }
  }
}

template <typename Kernel>
static cudaError_t launch_phase(Kernel kernel, dim3 grid, int threads, bool dependent, cudaStream_t stream,
                                const DecodeParams& p) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(threads);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = dependent ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, p);
}

}  // namespace ffnk

using namespace ffnk;

extern "C" int ffnk_decode_max_tokens(void) { return kDecodeMaxTokens; }

extern "C" int ffnk_ffn_decode(const void* x, int64_t ldx, const void* w1, const void* w2, const void* w3,
                               const void* u1, const void* u2, const void* u3, int64_t w13_stride_k,
                               int64_t w13_stride_n, int64_t w2_stride_k, int64_t w2_stride_n, const void* mask,
                               void* inter, void* y, int64_t ldy, int64_t M, int64_t d, int64_t h, int32_t* status,
                               void* stream_) {
  (void)status;
  if (M == 0) return 0;
  if (!x || !w1 || !w2 || !w3 || !u1 || !u2 || !u3 || !mask || !inter || !y) return FFNK_ERR_NULL;
  if (M < 0 || M > kDecodeMaxTokens || d < 8 || h < 8 || (d & 7) || (h & 7) || d >= (1ll << 30) || h >= (1ll << 30))
    return FFNK_ERR_SHAPE;
  // weights must be K-major (the .T view of [out, in] storage): rows are streamed whole
  if (w13_stride_k != 1 || w2_stride_k != 1 || w13_stride_n < d || w2_stride_n < h) return FFNK_ERR_LAYOUT;
  if ((ldx & 7) || (w13_stride_n & 7) || (w2_stride_n & 7) || ldx < d || ldy < d) return FFNK_ERR_ALIGN;
  const void* ptrs[] = {x, w1, w2, w3, u1, u2, u3, inter};
  for (const void* q : ptrs)
    if (reinterpret_cast<uintptr_t>(q) & 15) return FFNK_ERR_ALIGN;
  if (device_info().cc_major != 10) return FFNK_ERR_DEVICE;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  using bf = __nv_bfloat16;

  DecodeParams p1{};
  p1.x = static_cast<const bf*>(x);
  p1.ldx = ldx;
  p1.wa[0] = static_cast<const bf*>(w1);
  p1.wa[1] = static_cast<const bf*>(u1);
  p1.wb[0] = static_cast<const bf*>(w3);
  p1.wb[1] = static_cast<const bf*>(u3);
  p1.ldw = w13_stride_n;
  p1.mask = static_cast<const uint8_t*>(mask);
  p1.out = static_cast<bf*>(inter);
  p1.ldo = h;
  p1.M = static_cast<int>(M);
  p1.K = static_cast<int>(d);
  p1.rows = static_cast<int>(h);
  const dim3 grid1(static_cast<unsigned>((h + kDecodeRows - 1) / kDecodeRows), 2);
  const int groups = static_cast<int>((M + 7) / 8);   // upper bound: every token in one modality
  cudaError_t e;
  if (groups <= 1) e = launch_phase(decode_phase_kernel<true, false, 8, 4, 1>, grid1, 8 * 32, false, stream, p1);
  else if (groups <= 2) e = launch_phase(decode_phase_kernel<true, false, 8, 4, 2>, grid1, 8 * 32, false, stream, p1);
  else e = launch_phase(decode_phase_kernel<true, false, 8, 4, 4>, grid1, 8 * 32, false, stream, p1);
  if (e != cudaSuccess) return cuda_status(e);

  DecodeParams p2{};
  p2.x = static_cast<const bf*>(inter);
  p2.ldx = h;
  p2.wa[0] = static_cast<const bf*>(w2);
  p2.wa[1] = static_cast<const bf*>(u2);
  p2.wb[0] = p2.wb[1] = nullptr;
  p2.ldw = w2_stride_n;
  p2.mask = static_cast<const uint8_t*>(mask);
  p2.out = static_cast<bf*>(y);
  p2.ldo = ldy;
  p2.M = static_cast<int>(M);
  p2.K = static_cast<int>(h);
  p2.rows = static_cast<int>(d);
  const dim3 grid2(static_cast<unsigned>((d + kDecodeRows - 1) / kDecodeRows), 2);
  if (groups <= 1) e = launch_phase(decode_phase_kernel<false, true, 16, 6, 1>, grid2, 16 * 32, true, stream, p2);
  else if (groups <= 2) e = launch_phase(decode_phase_kernel<false, true, 16, 6, 2>, grid2, 16 * 32, true, stream, p2);
  else e = launch_phase(decode_phase_kernel<false, true, 16, 4, 4>, grid2, 16 * 32, true, stream, p2);
  return cuda_status(e);
}
