// Small-M MaskedFFN forward in ONE launch: both phases (gate/up with the SiLU(t1)*t3 epilogue, then the
// down projection) of up to 127 tokens, judged against HBM bandwidth: every weight of each modality
// that has tokens is streamed exactly once (3*d*h bf16 per modality) by 128-bit loads.
//
// One persistent CTA per SM, 16 warps.  A work unit is 8 weight rows over the whole contraction
// (gate and up rows of the same h index together in the first phase); the units of a phase are dealt
// to the CTAs in contiguous, equally long ranges.  Inside a CTA the contraction is split over the 16
// warps (k-blocks of 32 elements, warp w takes k-blocks w, w + 16, ...), loaded two steps ahead of
// their use so that 64 KiB of weight loads per SM are in flight all the time.
//   * the weights are the N = 8 side of mma.sync.m16n8k16 (bf16 in, fp32 accumulate), the modality's
//     tokens, in groups of sixteen, the M = 16 side.  The k-slots of the instruction are assigned so
//     that one 16-byte chunk of a weight row and the same chunk of two token rows feed two MMAs
//     straight from registers, with no shuffles: lane (g, t) holds chunk t of weight row g and of
//     tokens g and g + 8.
//   * a unit ends with a shared-memory reduction over the warps in a fixed order (bitwise reproducible).
//   * the phases are separated by a grid-wide arrive/wait on a counter in device memory (cooperative
//     launch guarantees that all CTAs are resident; the wait is bounded and reports a status code).
//     While the first phase runs, every CTA prefetches the down-projection rows it will need into L2.
// tcgen05 is not used on purpose: with at most 127 rows a 128-row UMMA tile is mostly padding and the
// weights would have to be staged through shared memory; the path is bound by the HBM stream.
//
// Same contract as MaskedFFN.forward (ffn_kernel/ops.py:28-32); the intermediate is rounded to bf16
// between the phases as in the reference (ffn_kernel/ffn.py:113).
#include <cuda_bf16.h>

#include <cstdlib>

#include "ffnk_internal.h"
#include "ptx.cuh"

namespace ffnk {

constexpr int kFusedMaxTokens = 127;
constexpr int kFusedWarps = 16;
constexpr int kFusedThreads = kFusedWarps * 32;
constexpr int kFusedBarrierSlots = 64;

// Grid-barrier counters, one slot per launch in turn (launches that could overlap on the device get
// different slots).  Monotonic: launch n on a slot waits for (n + 1) * gridDim arrivals, so nothing
// is ever reset.  Zero when the library is loaded.
static __device__ unsigned long long g_fused_barrier[kFusedBarrierSlots];

struct FusedParams {
  const __nv_bfloat16* x;
  int64_t ldx;
  const __nv_bfloat16* gate[2];   // [h, d] storage per modality (0: mask != 0)
  const __nv_bfloat16* up[2];
  const __nv_bfloat16* down[2];   // [d, h] storage
  int64_t ld13, ld2;
  const uint8_t* mask;
  __nv_bfloat16* inter;           // [M, h] scratch
  __nv_bfloat16* y;
  int64_t ldy;
  int M, d, h;
  int slot;
  int* status;
};

__device__ __forceinline__ uint4 ldg_stream_16(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ uint4 ldg_cg_16(const void* p) {   // L2 only: data written earlier in this launch
  uint4 v;
  asm volatile("ld.global.cg.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ void prefetch_l2(const void* p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }
__device__ __forceinline__ unsigned long long ld_acquire_gpu_u64(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}

// D[16 tokens x 8 weight rows] += X[16 x 16] * W^T[16 x 8]
__device__ __forceinline__ void mma_tok16_row8(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <bool GLU, int R>
struct StepLoads {
  uint4 a[R];
  uint4 b[GLU ? R : 1];
};

// One phase.  wa/wb: the (one or two) weights per modality, rows of `ldw` elements; xin rows of ldx
// elements (the activations, or the intermediate); out[token][row].
//   G: token groups of sixteen held in accumulators at a time; a modality with more tokens takes several
//      passes over the CTA's units (the second pass finds the weights in L2).
//   R: k-blocks a warp loads per step;  D: steps whose loads are in flight (D * R * 16 or 32 bytes per lane).
// A unit is 8 weight rows, or 4 (half of the lanes idle) when 8-row units would leave the CTAs with
// fewer than four units each and the split uneven.
template <bool GLU, int G, int R, int D>
__device__ __forceinline__ void run_phase(const __nv_bfloat16* const (&wa)[2], const __nv_bfloat16* const (&wb)[2],
                                          int64_t ldw, const __nv_bfloat16* xin, int64_t ldx, int K, int rows,
                                          __nv_bfloat16* out, int64_t ldo, const int (&ntok)[2],
                                          const int (*s_tok)[128], float* s_part, bool x_from_l2) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int present0 = ntok[0] > 0 ? 1 : 0, present1 = ntok[1] > 0 ? 1 : 0;
  const int rpu = ((present0 + present1) * (rows >> 3) < 4 * static_cast<int>(gridDim.x) && (rows & 3) == 0) ? 4 : 8;
  const int units_per_mod = rows / rpu;
  const int units = (present0 + present1) * units_per_mod;
  const int u0 = static_cast<int>(static_cast<long long>(blockIdx.x) * units / gridDim.x);
  const int u1 = static_cast<int>(static_cast<long long>(blockIdx.x + 1) * units / gridDim.x);
  const int nunits = u1 - u0;
  if (nunits <= 0) return;
  const int kblocks = (K + 31) >> 5;
  const int rounds = (kblocks + kFusedWarps * R - 1) / (kFusedWarps * R);
  const int max_tok = max(ntok[0], ntok[1]);
  const int passes = (max_tok + 16 * G - 1) / (16 * G);
  const int steps = passes * nunits * rounds;
  const uint4 zero = make_uint4(0, 0, 0, 0);
  const bool row_lane = g < rpu;      // this lane's weight row exists in the unit

  auto unit_of = [&](int s, int& m, int& rb, int& round, int& pass) {
    round = s % rounds;
    const int ul = (s / rounds) % nunits;
    pass = s / (rounds * nunits);
    const int u = u0 + ul;
    const int which = u / units_per_mod;             // index among the modalities present
    m = present0 ? which : 1;
    rb = u - which * units_per_mod;
  };
  auto load_step = [&](int s, StepLoads<GLU, R>& L) {
    int m, rb, round, pass;
    unit_of(s, m, rb, round, pass);
    const int64_t row_off = static_cast<int64_t>(rb * rpu + g) * ldw;
#pragma unroll
    for (int j = 0; j < R; ++j) {
      const int k = ((round * R + j) * kFusedWarps + warp) * 32 + t * 8;
      const bool ok = row_lane && k < K;
      L.a[j] = ok ? ldg_stream_16(wa[m] + row_off + k) : zero;
      if constexpr (GLU) L.b[j] = ok ? ldg_stream_16(wb[m] + row_off + k) : zero;
    }
  };

  float acc_a[G][4], acc_b[GLU ? G : 1][4];
#pragma unroll
  for (int gi = 0; gi < G; ++gi)
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      acc_a[gi][i] = 0.f;
      if (GLU) acc_b[gi][i] = 0.f;
    }
  int pb = 0;   // which half of the double-buffered partial sums

  auto consume = [&](int s, const StepLoads<GLU, R>& cur) {
    int m, rb, round, pass;
    unit_of(s, m, rb, round, pass);
    const int nt = ntok[m];
    const int groups_left = (nt - pass * 16 * G + 15) >> 4;     // may be <= 0: nothing to do in this pass
#pragma unroll
    for (int gi = 0; gi < G; ++gi) {
      if (gi < groups_left) {
        const int slot_lo = (pass * G + gi) * 16 + g, slot_hi = slot_lo + 8;
        const __nv_bfloat16* xlo = slot_lo < nt ? xin + static_cast<int64_t>(s_tok[m][slot_lo]) * ldx : nullptr;
        const __nv_bfloat16* xhi = slot_hi < nt ? xin + static_cast<int64_t>(s_tok[m][slot_hi]) * ldx : nullptr;
        uint4 vlo[R], vhi[R];
#pragma unroll
        for (int j = 0; j < R; ++j) {
          const int k = ((round * R + j) * kFusedWarps + warp) * 32 + t * 8;
          const bool ok = k < K;
          vlo[j] = vhi[j] = zero;
          if (ok && xlo) vlo[j] = x_from_l2 ? ldg_cg_16(xlo + k) : *reinterpret_cast<const uint4*>(xlo + k);
          if (ok && xhi) vhi[j] = x_from_l2 ? ldg_cg_16(xhi + k) : *reinterpret_cast<const uint4*>(xhi + k);
        }
#pragma unroll
        for (int j = 0; j < R; ++j) {
          mma_tok16_row8(acc_a[gi], vlo[j].x, vhi[j].x, vlo[j].y, vhi[j].y, cur.a[j].x, cur.a[j].y);
          mma_tok16_row8(acc_a[gi], vlo[j].z, vhi[j].z, vlo[j].w, vhi[j].w, cur.a[j].z, cur.a[j].w);
          if constexpr (GLU) {
            mma_tok16_row8(acc_b[gi], vlo[j].x, vhi[j].x, vlo[j].y, vhi[j].y, cur.b[j].x, cur.b[j].y);
            mma_tok16_row8(acc_b[gi], vlo[j].z, vhi[j].z, vlo[j].w, vhi[j].w, cur.b[j].z, cur.b[j].w);
          }
        }
      }
    }
    if (round == rounds - 1) {
      // the unit is complete in this warp: publish the partial sums, add the 16 warps' in warp order
      float* part = s_part + pb * (kFusedWarps * G * 256);
      if (groups_left > 0) {
#pragma unroll
        for (int gi = 0; gi < G; ++gi) {
          if (gi < groups_left) {
            float* mine = part + ((warp * G + gi) * 32 + lane) * 8;
            *reinterpret_cast<float4*>(mine) = make_float4(acc_a[gi][0], acc_a[gi][1], acc_a[gi][2], acc_a[gi][3]);
            if constexpr (GLU)
              *reinterpret_cast<float4*>(mine + 4) = make_float4(acc_b[gi][0], acc_b[gi][1], acc_b[gi][2], acc_b[gi][3]);
          }
        }
      }
      __syncthreads();
      const int ng = groups_left < G ? groups_left : G;
      for (int o = threadIdx.x; o < ng * 128; o += kFusedThreads) {
        const int gi = o >> 7, tau = (o >> 3) & 15, rho = o & 7;
        // accumulator element of (token tau, weight row rho): lane (tau % 8) * 4 + rho / 2, register (tau / 8) * 2 + rho % 2
        const int src = ((tau & 7) << 2) + (rho >> 1), reg = ((tau >> 3) << 1) + (rho & 1);
        const float* col = part + (gi * 32 + src) * 8 + reg;
        float va = 0.f, vb = 0.f;
#pragma unroll
        for (int w = 0; w < kFusedWarps; ++w) {
          va += col[w * G * 256];
          if constexpr (GLU) vb += col[w * G * 256 + 4];
        }
        const int slot = (pass * G + gi) * 16 + tau;
        if (slot < nt && rho < rpu) {
          if constexpr (GLU) va = va * __frcp_rn(1.0f + __expf(-va)) * vb;
          out[static_cast<int64_t>(s_tok[m][slot]) * ldo + rb * rpu + rho] = __float2bfloat16_rn(va);
        }
      }
      pb ^= 1;
#pragma unroll
      for (int gi = 0; gi < G; ++gi)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          acc_a[gi][i] = 0.f;
          if (GLU) acc_b[gi][i] = 0.f;
        }
    }
  };

  StepLoads<GLU, R> buf[D];
#pragma unroll
  for (int i = 0; i < D; ++i)
    if (i < steps) load_step(i, buf[i]);
#pragma unroll 1
  for (int s0 = 0; s0 < steps; s0 += D) {
#pragma unroll
    for (int i = 0; i < D; ++i) {
      const int s = s0 + i;
      if (s < steps) {
        consume(s, buf[i]);
        if (s + D < steps) load_step(s + D, buf[i]);
      }
    }
  }
}

template <int G>
__global__ void __launch_bounds__(kFusedThreads, 1) decode_fused_kernel(const FusedParams p) {
  extern __shared__ float s_part[];          // [2][16 warps][G][32 lanes][8]
  __shared__ int s_tok[2][128];
  __shared__ int s_wcnt[2][4];
  __shared__ int s_ok;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // token lists of the two modalities, ascending
  if (warp < 4) {
    const int idx = warp * 32 + lane;
    const bool valid = idx < p.M;
    const bool vis = valid && p.mask[idx] != 0;
    const uint32_t bv = __ballot_sync(0xFFFFFFFFu, vis), bt = __ballot_sync(0xFFFFFFFFu, valid && !vis);
    if (lane == 0) {
      s_wcnt[0][warp] = __popc(bv);
      s_wcnt[1][warp] = __popc(bt);
    }
    __syncwarp();
  }
  __syncthreads();
  int ntok[2] = {0, 0};
#pragma unroll
  for (int w = 0; w < 4; ++w) {
    ntok[0] += s_wcnt[0][w];
    ntok[1] += s_wcnt[1][w];
  }
  if (warp < 4) {
    const int idx = warp * 32 + lane;
    const bool valid = idx < p.M;
    const bool vis = valid && p.mask[idx] != 0;
    const uint32_t bv = __ballot_sync(0xFFFFFFFFu, vis), bt = __ballot_sync(0xFFFFFFFFu, valid && !vis);
    int off_v = 0, off_t = 0;
    for (int w = 0; w < warp; ++w) {
      off_v += s_wcnt[0][w];
      off_t += s_wcnt[1][w];
    }
    const uint32_t below = (1u << lane) - 1u;
    if (vis) s_tok[0][off_v + __popc(bv & below)] = idx;
    else if (valid) s_tok[1][off_t + __popc(bt & below)] = idx;
  }
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();

  // second-phase weights of this CTA's share of rows into L2 while the first phase streams
  {
    const int present0 = ntok[0] > 0 ? 1 : 0, present1 = ntok[1] > 0 ? 1 : 0;
    const int rows_all = (present0 + present1) * p.d;
    const int r0 = static_cast<int>(static_cast<long long>(blockIdx.x) * rows_all / gridDim.x) & ~7;
    const int r1 = min(rows_all, (static_cast<int>(static_cast<long long>(blockIdx.x + 1) * rows_all / gridDim.x) + 7) & ~7);
    const int lines_per_row = (p.h * 2) >> 7;   // whole 128-byte lines inside the row
    const int total = (r1 - r0) * lines_per_row;
    for (int i = threadIdx.x; i < total; i += kFusedThreads) {
      const int line = i % lines_per_row;
      const int r = r0 + i / lines_per_row;
      const int which = r / p.d;
      const int m = present0 ? which : 1;
      prefetch_l2(reinterpret_cast<const char*>(p.down[m] + static_cast<int64_t>(r - which * p.d) * p.ld2) + line * 128);
    }
  }

  const __nv_bfloat16* const none[2] = {nullptr, nullptr};
  run_phase<true, G, 2, (G <= 2 ? 4 : 2)>(p.gate, p.up, p.ld13, p.x, p.ldx, p.d, p.h, p.inter, static_cast<int64_t>(p.h),
                                          ntok, s_tok, s_part, false);

  // every CTA's part of the intermediate is written: arrive, then wait for the whole grid
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    unsigned long long* bar = &g_fused_barrier[p.slot];
    const unsigned long long ticket = atomicAdd(bar, 1ULL);
    const unsigned long long target = (ticket / gridDim.x + 1ULL) * gridDim.x;
    const uint64_t t0 = globaltimer_ns();
    uint32_t polls = 0;
    while (ld_acquire_gpu_u64(bar) < target) {
      if ((++polls & 63u) == 0 && globaltimer_ns() - t0 > kWaitBudgetNs) {
        if (p.status) atomicCAS(p.status, 0, ST_TIMEOUT_GRID);
        s_ok = 0;
        break;
      }
    }
  }
  __syncthreads();
  if (!s_ok) return;
  run_phase<false, G, 3, (G <= 2 ? 4 : 2)>(p.down, none, p.ld2, p.inter, static_cast<int64_t>(p.h), p.h, p.d, p.y, p.ldy,
                                           ntok, s_tok, s_part, true);
}

}  // namespace ffnk

using namespace ffnk;

extern "C" int ffnk_ffn_small_max_tokens(void) { return kFusedMaxTokens; }

extern "C" int ffnk_ffn_small(const void* x, int64_t ldx, const void* w1, const void* w2, const void* w3, const void* u1,
                              const void* u2, const void* u3, int64_t w13_stride_k, int64_t w13_stride_n,
                              int64_t w2_stride_k, int64_t w2_stride_n, const void* mask, void* inter, void* y,
                              int64_t ldy, int64_t M, int64_t d, int64_t h, int32_t* status, void* stream_) {
  if (M == 0) return 0;
  if (!x || !w1 || !w2 || !w3 || !u1 || !u2 || !u3 || !mask || !inter || !y) return FFNK_ERR_NULL;
  if (M < 0 || M > kFusedMaxTokens || d < 8 || h < 8 || (d & 7) || (h & 7) || d >= (1ll << 24) || h >= (1ll << 24))
    return FFNK_ERR_SHAPE;
  // weights must be K-major (the .T view of [out, in] storage): rows are streamed whole
  if (w13_stride_k != 1 || w2_stride_k != 1 || w13_stride_n < d || w2_stride_n < h) return FFNK_ERR_LAYOUT;
  if ((ldx & 7) || (ldy & 7) || (w13_stride_n & 7) || (w2_stride_n & 7) || ldx < d || ldy < d) return FFNK_ERR_ALIGN;
  const void* ptrs[] = {x, w1, w2, w3, u1, u2, u3, inter, y};
  for (const void* q : ptrs)
    if (reinterpret_cast<uintptr_t>(q) & 15) return FFNK_ERR_ALIGN;
  const DeviceInfo& dev = device_info();
  if (dev.cc_major != 10) return FFNK_ERR_DEVICE;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  using bf = __nv_bfloat16;

  FusedParams p{};
  p.x = static_cast<const bf*>(x);
  p.ldx = ldx;
  p.gate[0] = static_cast<const bf*>(w1);
  p.gate[1] = static_cast<const bf*>(u1);
  p.up[0] = static_cast<const bf*>(w3);
  p.up[1] = static_cast<const bf*>(u3);
  p.down[0] = static_cast<const bf*>(w2);
  p.down[1] = static_cast<const bf*>(u2);
  p.ld13 = w13_stride_n;
  p.ld2 = w2_stride_n;
  p.mask = static_cast<const uint8_t*>(mask);
  p.inter = static_cast<bf*>(inter);
  p.y = static_cast<bf*>(y);
  p.ldy = ldy;
  p.M = static_cast<int>(M);
  p.d = static_cast<int>(d);
  p.h = static_cast<int>(h);
  p.status = status;
  static unsigned launch_seq = 0;   // successive launches take successive barrier slots
  p.slot = static_cast<int>(__atomic_fetch_add(&launch_seq, 1u, __ATOMIC_RELAXED) % kFusedBarrierSlots);

  const int G = M <= 16 ? 1 : (M <= 32 ? 2 : 4);
  const size_t smem = static_cast<size_t>(2) * kFusedWarps * G * 256 * sizeof(float);
  void* args[] = {&p};
  auto go = [&](auto kernel) -> int {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return cuda_status(e);
    static const bool coop = getenv("FFNK_COOP") != nullptr;
    if (coop) {
      e = cudaLaunchCooperativeKernel(reinterpret_cast<void*>(kernel), dim3(dev.sm_count), dim3(kFusedThreads), args, smem,
                                      stream);
      return cuda_status(e);
    }
    kernel<<<dev.sm_count, kFusedThreads, smem, stream>>>(p);
    return cuda_status(cudaGetLastError());
  };
  if (G == 1) return go(decode_fused_kernel<1>);
  if (G == 2) return go(decode_fused_kernel<2>);
  return go(decode_fused_kernel<4>);
}
