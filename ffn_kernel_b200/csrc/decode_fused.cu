// Small-M (decode) MaskedFFN forward in ONE launch: both phases (gate/up with the SiLU(t1)*t3 epilogue, then
// the down projection) of up to 127 tokens, a kernel bound by HBM bandwidth: every weight of each modality
// that has tokens is streamed exactly once (3*d*h bf16 per modality) by 128-bit loads.
//
// One persistent CTA per SM, 16 warps.  A work unit is 8 weight rows over the whole contraction
// (gate and up rows of the same h index together in the first phase); the units of a phase are dealt
// to the CTAs in contiguous, equally long ranges.  Inside a CTA the contraction is split over the 16
// warps (k-blocks of 32 elements, warp w takes k-blocks w, w + 16, ...), loaded two or three steps
// ahead of their use so that 64-96 KiB of weight loads per SM are in flight.
//   * the weights are the N = 8 side of mma.sync.m16n8k16 (bf16 in, fp32 accumulate), the modality's
//     tokens, in groups of sixteen, the M = 16 side.  The k-slots of the instruction are assigned so
//     that one 16-byte chunk of a weight row and the same chunk of two token rows feed two MMAs
//     straight from registers, with no shuffles: lane (g, t) holds chunk t of weight row g and of
//     tokens g and g + 8.
//   * a unit ends with a shared-memory reduction over the warps in a fixed order (bitwise reproducible).
//   * the phases are separated by a grid-wide arrive/wait on a counter in device memory (one CTA per SM,
//     so all CTAs are resident once earlier work has left the SMs; the wait is bounded and reports a
//     status code).  While the first phase runs, every CTA prefetches the down-projection rows it will
//     need into L2, and requests its first ones into registers before it waits.
// tcgen05 is not used on purpose: with at most 127 rows a 128-row UMMA tile is mostly padding and the
// weights would have to be staged through shared memory; the path is bound by the HBM stream.
//
// Same contract as MaskedFFN.forward (ffn_kernel/ops.py:28-32); the intermediate is rounded to bf16
// between the phases as in the reference (ffn_kernel/ffn.py:113).
#include <cuda_bf16.h>

#include "ffnk_internal.h"
#include "ptx.cuh"

namespace ffnk {

constexpr int kFusedMaxTokens = 127;      // what the kernel can take
// Up to this many tokens the tile table sends a forward here; beyond, the token rows (re-read from L2 by
// every CTA) outweigh the weight stream and the tcgen05 GEMM path is faster (measured at d=1024/h=2816,
// both modalities present: 64 tokens 30 us against 37 us, 96 tokens 37 us against 37 us, 127 tokens 50 against 38).
constexpr int kDecodeTableTokens = 80;
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
  long long* prof;                // optional per-CTA cycle stamps (8 per CTA), see ffnk_debug_profile_buffer
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

// Position of a pipeline step inside the CTA's work: pass over the token groups, unit, round of k-blocks.
// Advanced incrementally (no divisions in the loop).
struct StepCursor {
  int round = 0, unit = 0, pass = 0;
  __device__ __forceinline__ void advance(int rounds, int nunits) {
    if (++round == rounds) {
      round = 0;
      if (++unit == nunits) {
        unit = 0;
        ++pass;
      }
    }
  }
};

// One phase.  wa/wb: the (one or two) weights per modality, rows of `ldw` elements; xin rows of ldx
// elements (the activations, or the intermediate); out[token][row].
//   G: token groups of sixteen held in accumulators at a time; a modality with more tokens takes several
//      passes over the CTA's units (the second pass finds the weights in L2).
//   R: k-blocks a warp loads per step;  D (2 or 3): steps whose loads are in flight.
// `before_consume` runs once after the first D steps' weight loads have been issued and before anything
// is multiplied: the place to wait for whatever the token rows depend on (it returns false to give up).
template <bool GLU, int G, int R, int D, typename Hook>
__device__ __forceinline__ void run_phase(const __nv_bfloat16* const (&wa)[2], const __nv_bfloat16* const (&wb)[2],
                                          int64_t ldw, const __nv_bfloat16* xin, int64_t ldx, int K, int rows,
                                          __nv_bfloat16* out, int64_t ldo, int ntok0, int ntok1,
                                          const int (*s_tok)[128], float* s_part, Hook&& before_consume) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int present0 = ntok0 > 0 ? 1 : 0, present1 = ntok1 > 0 ? 1 : 0;
  const int units_per_mod = rows >> 3;
  const int units = (present0 + present1) * units_per_mod;
  // (units < 2^22 and at most a few hundred CTAs: the products fit 32 bits)
  const int u0 = static_cast<int>(blockIdx.x * static_cast<unsigned>(units) / gridDim.x);
  const int u1 = static_cast<int>((blockIdx.x + 1u) * static_cast<unsigned>(units) / gridDim.x);
  const int nunits = u1 - u0;
  if (nunits <= 0) {          // a CTA without work still takes part in whatever the hook waits for
    before_consume();
    return;
  }
  const int kblocks = (K + 31) >> 5;
  const int rounds = (kblocks + kFusedWarps * R - 1) / (kFusedWarps * R);
  const int max_tok = max(ntok0, ntok1);
  const int passes = (max_tok + 16 * G - 1) / (16 * G);
  const int steps = passes * nunits * rounds;
  const uint4 zero = make_uint4(0, 0, 0, 0);
  const int k_lane = warp * 32 + t * 8;                 // this lane's column in the first k-block of a round
  constexpr int K_ROUND = kFusedWarps * 32;             // columns the 16 warps cover per k-block index

  // modality and first row of unit `ul` of this CTA
  auto unit_rows = [&](int ul, int& m, int& row0) {
    const int u = u0 + ul;
    const int second = (present0 && u >= units_per_mod) ? 1 : 0;
    m = present0 ? second : 1;
    row0 = (u - second * units_per_mod) << 3;
  };
  auto load_step = [&](const StepCursor& c, StepLoads<GLU, R>& L) {
    int m, row0;
    unit_rows(c.unit, m, row0);
    const int kbase = k_lane + c.round * (R * K_ROUND);
    const int64_t off = static_cast<int64_t>(row0 + g) * ldw + kbase;
    const __nv_bfloat16* pa = (m ? wa[1] : wa[0]) + off;
    const __nv_bfloat16* pb = GLU ? (m ? wb[1] : wb[0]) + off : nullptr;
#pragma unroll
    for (int j = 0; j < R; ++j) {
      const bool ok = kbase + j * K_ROUND < K;
      L.a[j] = ok ? ldg_stream_16(pa + j * K_ROUND) : zero;
      if constexpr (GLU) L.b[j] = ok ? ldg_stream_16(pb + j * K_ROUND) : zero;
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

  // multiply-accumulate one step's weights with the token rows of the unit's modality
  auto mma_step = [&](const StepCursor& c, const StepLoads<GLU, R>& W, int m, int nt) {
    const int kbase = k_lane + c.round * (R * K_ROUND);
#pragma unroll
    for (int gi = 0; gi < G; ++gi) {
      const int slot_lo = (c.pass * G + gi) * 16 + g, slot_hi = slot_lo + 8;
      if ((c.pass * G + gi) * 16 < nt) {                     // warp-uniform: the group has tokens
        const __nv_bfloat16* xlo = slot_lo < nt ? xin + static_cast<int64_t>(s_tok[m][slot_lo]) * ldx + kbase : nullptr;
        const __nv_bfloat16* xhi = slot_hi < nt ? xin + static_cast<int64_t>(s_tok[m][slot_hi]) * ldx + kbase : nullptr;
        uint4 vlo[R], vhi[R];
#pragma unroll
        for (int j = 0; j < R; ++j) {
          const bool ok = kbase + j * K_ROUND < K;
          vlo[j] = (ok && xlo) ? *reinterpret_cast<const uint4*>(xlo + j * K_ROUND) : zero;
          vhi[j] = (ok && xhi) ? *reinterpret_cast<const uint4*>(xhi + j * K_ROUND) : zero;
        }
#pragma unroll
        for (int j = 0; j < R; ++j) {
          mma_tok16_row8(acc_a[gi], vlo[j].x, vhi[j].x, vlo[j].y, vhi[j].y, W.a[j].x, W.a[j].y);
          mma_tok16_row8(acc_a[gi], vlo[j].z, vhi[j].z, vlo[j].w, vhi[j].w, W.a[j].z, W.a[j].w);
          if constexpr (GLU) {
            mma_tok16_row8(acc_b[gi], vlo[j].x, vhi[j].x, vlo[j].y, vhi[j].y, W.b[j].x, W.b[j].y);
            mma_tok16_row8(acc_b[gi], vlo[j].z, vhi[j].z, vlo[j].w, vhi[j].w, W.b[j].z, W.b[j].w);
          }
        }
      }
    }
  };

  StepLoads<GLU, R> buf0, buf1, buf2;
  auto with_slot = [&](int sl, auto&& f) {
    if (sl == 0) f(buf0);
    else if (D == 2 || sl == 1) f(buf1);
    else f(buf2);
  };
  StepCursor lc, cc;                 // load cursor (D steps ahead), consume cursor
#pragma unroll
  for (int i = 0; i < D; ++i) {
    if (i < steps) {
      with_slot(i, [&](StepLoads<GLU, R>& b) { load_step(lc, b); });
      lc.advance(rounds, nunits);
    }
  }
  if (!before_consume()) return;
  int pb = 0;   // which half of the double-buffered partial sums
  int sl = 0;   // slot of the step being consumed
#pragma unroll 1
  for (int s = 0; s < steps; ++s) {
    int m, row0;
    unit_rows(cc.unit, m, row0);
    const int nt = m ? ntok1 : ntok0;
    with_slot(sl, [&](StepLoads<GLU, R>& b) {
      mma_step(cc, b, m, nt);
      if (s + D < steps) {
        load_step(lc, b);
        lc.advance(rounds, nunits);
      }
    });
    if (++sl == D) sl = 0;
    if (cc.round == rounds - 1) {
      // the unit is complete in this warp: publish the partial sums, add the 16 warps' in warp order
      const int groups_left = (nt - cc.pass * 16 * G + 15) >> 4;     // may be <= 0: nothing to do in this pass
      float* part = s_part + pb * (kFusedWarps * G * 256);
#pragma unroll
      for (int gi = 0; gi < G; ++gi) {
        if (gi < groups_left) {
          float* mine = part + ((warp * G + gi) * 32 + lane) * 8;
          *reinterpret_cast<float4*>(mine) = make_float4(acc_a[gi][0], acc_a[gi][1], acc_a[gi][2], acc_a[gi][3]);
          if constexpr (GLU)
            *reinterpret_cast<float4*>(mine + 4) = make_float4(acc_b[gi][0], acc_b[gi][1], acc_b[gi][2], acc_b[gi][3]);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          acc_a[gi][i] = 0.f;
          if (GLU) acc_b[gi][i] = 0.f;
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
        const int slot = (cc.pass * G + gi) * 16 + tau;
        if (slot < nt) {
          if constexpr (GLU) va = va * __frcp_rn(1.0f + __expf(-va)) * vb;
          out[static_cast<int64_t>(s_tok[m][slot]) * ldo + row0 + rho] = __float2bfloat16_rn(va);
        }
      }
      pb ^= 1;
    }
    cc.advance(rounds, nunits);
  }
}

template <int G>
__global__ void __launch_bounds__(kFusedThreads, 1) decode_fused_kernel(const FusedParams p) {
  extern __shared__ float s_part[];          // [2][16 warps][G][32 lanes][8]
  __shared__ int s_tok[2][128];
  __shared__ int s_ok;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  long long* prof = p.prof ? p.prof + blockIdx.x * 8 : nullptr;
  const long long c_start = clock64();
  auto stamp = [&](int i) {
    if (prof && threadIdx.x == 0) prof[i] = clock64() - c_start;
  };

  // Token lists of the two modalities, ascending.  Every warp reads the (at most 127) mask bytes and counts
  // for itself, so nobody waits for a barrier before the first weight loads go out; warp 0 also writes the
  // lists, which are first read after the barrier that follows those loads.
  int ntok[2] = {0, 0};
  {
    uint32_t bv[4], bt[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int idx = j * 32 + lane;
      const bool valid = idx < p.M;
      const bool vis = valid && p.mask[idx] != 0;
      bv[j] = __ballot_sync(0xFFFFFFFFu, vis);
      bt[j] = __ballot_sync(0xFFFFFFFFu, valid && !vis);
      ntok[0] += __popc(bv[j]);
      ntok[1] += __popc(bt[j]);
    }
    if (warp == 0) {
      const uint32_t below = (1u << lane) - 1u;
      int off_v = 0, off_t = 0;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if ((bv[j] >> lane) & 1u) s_tok[0][off_v + __popc(bv[j] & below)] = j * 32 + lane;
        if ((bt[j] >> lane) & 1u) s_tok[1][off_t + __popc(bt[j] & below)] = j * 32 + lane;
        off_v += __popc(bv[j]);
        off_t += __popc(bt[j]);
      }
    }
    if (threadIdx.x == 0) s_ok = 1;
  }
  stamp(0);          // mask read, tokens counted

  // second-phase weights of this CTA's share of rows into L2 while the first phase streams (issued
  // behind the first gate/up loads, which are what the CTA waits for first)
  auto prefetch_down_rows = [&]() {
    const int present0 = ntok[0] > 0 ? 1 : 0, present1 = ntok[1] > 0 ? 1 : 0;
    const int rows_all = (present0 + present1) * p.d;
    const int u_all = rows_all >> 3;
    const int r0 = static_cast<int>(blockIdx.x * static_cast<unsigned>(u_all) / gridDim.x) << 3;
    const int r1 = static_cast<int>((blockIdx.x + 1u) * static_cast<unsigned>(u_all) / gridDim.x) << 3;
    const int lines_per_row = (p.h * 2) >> 7;   // whole 128-byte lines inside the row
    for (int r = r0 + warp; r < r1; r += kFusedWarps) {
      const int second = r >= p.d ? 1 : 0;
      const int m = present0 ? second : 1;
      const char* row = reinterpret_cast<const char*>(p.down[m] + static_cast<int64_t>(r - second * p.d) * p.ld2);
      for (int line = lane; line < lines_per_row; line += 32) prefetch_l2(row + line * 128);
    }
  };

  const __nv_bfloat16* const none[2] = {nullptr, nullptr};
  constexpr int DEPTH = G <= 2 ? 3 : 2;
  run_phase<true, G, 2, DEPTH>(p.gate, p.up, p.ld13, p.x, p.ldx, p.d, p.h, p.inter, static_cast<int64_t>(p.h), ntok[0],
                               ntok[1], s_tok, s_part, [&]() -> bool {
                                 stamp(1);             // first gate/up weights requested
                                 prefetch_down_rows();
                                 __syncthreads();      // the token lists are in shared memory
                                 return true;
                               });
  stamp(2);          // gate/up done in this CTA

  // The first down-projection weights are requested before the wait (they do not depend on the first
  // phase); then every CTA's part of the intermediate must be written: arrive, wait for the whole grid.
  // The intermediate was written by other SMs before that wait and has never been read by this one, so
  // ordinary (L1-allocating) loads cannot see stale lines.
  run_phase<false, G, 3, DEPTH>(p.down, none, p.ld2, p.inter, static_cast<int64_t>(p.h), p.h, p.d, p.y, p.ldy, ntok[0],
                                ntok[1], s_tok, s_part, [&]() -> bool {
                                  __syncthreads();
                                  stamp(3);           // first down-projection weights requested, before the wait
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
                                  stamp(4);           // the whole grid has finished gate/up
                                  return s_ok != 0;
                                });
  stamp(5);          // down projection done in this CTA
}

}  // namespace ffnk

using namespace ffnk;

extern "C" int ffnk_decode_max_tokens(void) { return kDecodeTableTokens; }

// Tile-table entry: does a forward of M tokens take this kernel?  Both paths stream the weights once; this
// one adds the token rows that every CTA re-reads from L2 for each of its units, the GEMM path (routing and
// row copy in one launch, gate/up GEMM, split-K down projection) has a fixed cost of some 18 us but little
// that grows with M.  Fitted to graph-replayed forwards with both modalities present (a = microseconds the
// weights take at 3.9 TB/s):
//     decode(M) = (a + 6 us) * (1 + (max(M, 8) - 8) / 60)
//     gemm(a)   = through the measured points (a, us): (1.6, 19.7) (3.2, 22.5) (8.9, 27.0) (51.6, 55.7) (138.7, 124)
// d=1024/h=2816 (a = 8.9): decode 14.8 us at 8 tokens, 23.7 at 56, 28.6 at 64; GEMM path 27-28.5 from 8 to 127
// tokens: break-even near 57.  d=512/h=1024: decode 12.8 us at 80 tokens, GEMM path 20.  d=2048/h=8192 and
// d=4096/h=11008: the GEMM path is ahead from two tokens on (8 tokens: 53 against 58 us, 124 against 139 us:
// 0.67 against 0.59 of the HBM peak).  A single token has one modality and half the weights: this
// kernel (31.6 against 50.3 us, 76 against 89 us).
static double gemm_path_us(double a) {
  static const double pts[][2] = {{1.6, 19.7}, {3.2, 22.5}, {8.9, 27.0}, {51.6, 55.7}, {138.7, 124.0}};
  constexpr int n = sizeof(pts) / sizeof(pts[0]);
  if (a <= pts[0][0]) return pts[0][1];
  for (int i = 1; i < n; ++i)
    if (a <= pts[i][0])
      return pts[i - 1][1] + (pts[i][1] - pts[i - 1][1]) * (a - pts[i - 1][0]) / (pts[i][0] - pts[i - 1][0]);
  return pts[n - 1][1] * a / pts[n - 1][0];
}

extern "C" int ffnk_ffn_takes_decode(int64_t M, int64_t d, int64_t h) {
  if (M < 1 || M > kDecodeTableTokens || d < 8 || h < 8) return 0;
  if (M == 1) return 1;
  const double a = 12.0 * static_cast<double>(d) * static_cast<double>(h) / 3.9e6;
  const double m_eff = M < 8 ? 8.0 : static_cast<double>(M);
  const double decode_us = (a + 6.0) * (1.0 + (m_eff - 8.0) / 60.0);
  return decode_us <= gemm_path_us(a) ? 1 : 0;
}
extern "C" int ffnk_decode_capacity(void) { return kFusedMaxTokens; }

extern "C" int ffnk_ffn_decode(const void* x, int64_t ldx, const void* w1, const void* w2, const void* w3, const void* u1,
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
  p.prof = debug_profile_buffer();
  static unsigned launch_seq = 0;   // successive launches take successive barrier slots
  p.slot = static_cast<int>(__atomic_fetch_add(&launch_seq, 1u, __ATOMIC_RELAXED) % kFusedBarrierSlots);

  const int G = M <= 16 ? 1 : (M <= 32 ? 2 : 4);
  const size_t smem = static_cast<size_t>(2) * kFusedWarps * G * 256 * sizeof(float);
  auto go = [&](auto kernel) -> int {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return cuda_status(e);
    // An ordinary launch: one CTA per SM of 512 threads and at most 128 KiB of shared memory always fits, so
    // every CTA becomes resident as soon as the SMs are free of earlier work, and the grid-wide wait (bounded
    // in any case) cannot starve a CTA that has not started.
    kernel<<<dev.sm_count, kFusedThreads, smem, stream>>>(p);
    return cuda_status(cudaGetLastError());
  };
  if (G == 1) return go(decode_fused_kernel<1>);
  if (G == 2) return go(decode_fused_kernel<2>);
  return go(decode_fused_kernel<4>);
}
