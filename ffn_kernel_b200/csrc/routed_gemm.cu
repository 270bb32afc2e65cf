// Routed grouped GEMMs for sm_100a.  Kernels in this file:
//   routed_gemm_kernel       single CTA, 128 x 256 (or 128 x 64) tiles: every forward and dx GEMM
//   routed_gemm_pair_kernel  the same on CTA pairs (cta_group::2), 256 x 256 tiles
//   wgrad_kernel             weight gradients (contraction over token rows), single CTA
//   wgrad_pair_kernel        weight gradients on CTA pairs, operands in routed order
// Epilogues: plain store (to token order, routed order, or straight into the memory of the GPU that
// owns the row: OUT_PEER), SwiGLU, SwiGLU saving its pre-activations, dSwiGLU.
//
// The token rows of each modality are a compacted list (route.cu).  A CTA tile is 128 routed
// rows of ONE modality times 256 accumulator columns, so a tile multiplies by exactly one
// weight set -- the reference instead tiles tokens in natural order and, for a tile holding
// both modalities, computes both products and selects (ffn_kernel/linear.py:142-149,
// ffn_kernel/ffn.py:86-99).
//
// Structure of one persistent CTA (192 or 320 threads, one CTA per SM):
//   warp 0      producer: TMA.  A rows are fetched with gather4 (four arbitrary rows of 128 B
//               per instruction, lane l of the warp owns rows 4l..4l+3 of the tile) or, when A
//               is already in routed order, with one tiled load.  B comes from the weight's own
//               storage, K-major ([N,K], the nn.Linear.weight.T view) or MN-major ([K,N]).
//   warp 1      issues tcgen05.mma (bf16 x bf16 -> fp32 in TMEM), 128x256x16 per instruction,
//               four per 64-wide k-step; owns the TMEM allocation.
//   warps 2..5 (or 2..9 when tiles are short in K: two warps per TMEM lane quarter)  epilogue: tcgen05.ld the accumulator, convert (optionally SiLU(t1)*t3), store
//               bf16 rows to their destination (token order via the list, or routed order).
// Shared-memory stages are handed between producer and MMA with full/empty mbarriers; the
// accumulator is double buffered in TMEM (2 x 256 columns) so the epilogue of tile i runs
// under the main loop of tile i+1.
#include <cuda_bf16.h>

#include <mutex>

#include "ffnk_internal.h"
#include "ptx.cuh"

namespace ffnk {

constexpr int BM = 128;                 // routed rows per tile (UMMA M)
constexpr int BN = 256;                 // accumulator columns per tile (UMMA N)
constexpr int BK = 64;                  // k-step: 64 bf16 = 128 bytes = one swizzle row
constexpr int UMMA_K = 16;
constexpr int STAGES = 4;
constexpr int A_BYTES = BM * BK * 2;    // 16 KiB
constexpr int B_BYTES = BN * BK * 2;    // 32 KiB
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
// The epilogue has one or two warps per TMEM lane quarter (each drains all, or half, of the columns);
// the launch picks 192 or 320 threads: the second set pays off only when tiles are short in K and the
// epilogue would otherwise hold up the MMA issuer (measured: K=1024 gate/up +23 %, K=11008 down -6 %).
constexpr int GEMM_THREADS_MAX = 320;
constexpr int GEMM_THREADS = 192;
__device__ __forceinline__ int epilogue_parts() { return (static_cast<int>(blockDim.x) - 64) >> 7; }
static int gemm_threads_for(int64_t k_len_total) {
  const int forced = tune_overrides().epi_warps;
  if (forced == 4) return GEMM_THREADS;
  if (forced == 8) return GEMM_THREADS_MAX;
  return k_len_total <= 2048 ? GEMM_THREADS_MAX : GEMM_THREADS;
}
constexpr int TMEM_COLS = 512;
constexpr int GEMM_SMEM = STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;

enum { A_GATHER = 0, A_ROUTED = 1 };
// EPI_STORE       : out = acc
// EPI_SWIGLU      : out = silu(gate) * up                         (accumulator = gate | up column halves)
// EPI_SWIGLU_SAVE : same, and gate -> aux0, up -> aux1             (training forward keeps the pre-activations)
// EPI_DSWIGLU     : acc = dH; with t1 = aux0, t3 = aux1 at the same position:
//                   out = dH * t3 * s * (1 + t1 * (1 - s)),  aux2 = dH * t1 * s,  s = sigmoid(t1)
//                   (the element-wise terms of the FFN backward, reference README.md:159-172)
enum { EPI_STORE = 0, EPI_SWIGLU = 1, EPI_SWIGLU_SAVE = 2, EPI_DSWIGLU = 3 };
__host__ __device__ constexpr bool epi_glu(int e) { return e == EPI_SWIGLU || e == EPI_SWIGLU_SAVE; }
// OUT_SCATTER : row of token t -> out[t]            OUT_ROUTED : row i of the routed order -> out[i]
// OUT_PEER    : row of token t -> row block `peer_rank` of the buffer of the rank that owns token t
//               (tensor parallel: every rank hands its partial rows straight to their owner)
enum { OUT_SCATTER = 0, OUT_ROUTED = 1, OUT_PEER = 2 };
constexpr int MAX_PEERS = 8;
constexpr int STORE_STAGING = 8 * 4096;  // one 32-row x 128-byte transposition buffer per epilogue warp
constexpr int GLU_STAGING = 8 * 2048;    // one 32-row x 64-byte transposition buffer per epilogue warp

struct GemmParams {
  const int* perm;      // routing lists
  const int* counts;    // {Mv, Mt, cap, M}
  __nv_bfloat16* out;
  int64_t ldo;          // elements
  int n_out;            // valid output columns
  int k_len;            // contraction length
  int pad_row;          // row index fetched for the padding rows of a tile (>= M: zero fill)
  int group_m;          // m-tiles per super-tile of the tile order
  int max_run_rows;     // largest tiled box used for runs of consecutive tokens (0: gather4 only)
  int* status;
  long long* prof;      // optional per-CTA wait-cycle counters (8 per CTA), see ffnk_debug_profile_buffer
  // extra epilogue operands, addressed like `out` (same row, same leading dimension)
  __nv_bfloat16* aux0 = nullptr;
  __nv_bfloat16* aux1 = nullptr;
  __nv_bfloat16* aux2 = nullptr;
  // Gather mode: when > 0, a routed-order copy of A exists (tensor map m[COPY_MAP]; permute_rows
  // fills it only for scattered masks) and the kernel reads it instead of gathering whenever the
  // mask's average run is shorter than a_copy rows -- decided on the device from counts[4].
  int a_copy = 0;
  // Optional second contraction segment (A_ROUTED + EPI_STORE only): after k_len columns of the
  // first A matrix against the first weight, k_len1 columns of a second A matrix (tensor map
  // m[RUN_LEVELS - 1]) against the second weight (the "1" weight maps) go into the same accumulator.
  int k_len1 = 0;
  // OUT_PEER: peer_out[r] is rank r's buffer of peer_world row blocks, peer_rows rows of ldo elements
  // each, mapped into this process.  Token t is owned by rank t / peer_rows and lands in row
  // peer_rank * peer_rows + t % peer_rows of that rank's buffer.
  __nv_bfloat16* peer_out[MAX_PEERS] = {};
  int peer_world = 0;
  int peer_rank = 0;
  int peer_rows = 1;
  // Split-K (A_ROUTED + EPI_STORE + OUT_SCATTER, single CTAs, K-major weights): ksplit > 1 makes every tile
  // ksplit work items, one per range of k-steps; the items leave fp32 partial tiles in kpart
  // [item][BN_T / 4 column groups][128 rows][4] and the one that arrives last at the tile's counter adds them in item
  // order and stores the rows.  kcount: one counter per tile, zero before and after the launch.
  int ksplit = 1;
  float* kpart = nullptr;
  unsigned int* kcount = nullptr;
  // Early start (single CTAs): pdl != 0 says the kernel was launched with the programmatic-stream-
  // serialization attribute, i.e. it may be running beside its predecessor in the stream.  Until
  // griddep_wait() it touches nothing the predecessor writes; what it does meanwhile, besides its set-up,
  // is ask the weights (up to four matrices of pf_rows rows of pf_row_bytes bytes, pf_stride bytes apart)
  // into L2, every CTA its share.
  int pdl = 0;
  const char* pf_base[4] = {nullptr, nullptr, nullptr, nullptr};
  int64_t pf_stride = 0;
  int pf_rows = 0, pf_row_bytes = 0;
};

// Split-K arrival counters, one row of kSplitKTiles per launch in turn (launches that could overlap on the
// device get different rows); the last arrival at a tile resets its counter, so the rows stay zero between
// launches.  Zero when the library is loaded.
constexpr int kSplitKSlots = 64;
constexpr int kSplitKTiles = 256;
static __device__ unsigned int g_splitk_count[kSplitKSlots][kSplitKTiles];

// Views of one row-gathered activation matrix: m[0] fetches single rows (gather4); m[1 + i]
// fetches boxes of 4 << i consecutive rows (4, 8, ..., 128), 64 columns wide.
// m[RUN_LEVELS + 1] (gather mode only, optional) views a copy of the same matrix in routed order.
constexpr int RUN_LEVELS = 6;
constexpr int COPY_MAP = RUN_LEVELS + 1;
struct AMaps {
  CUtensorMap m[2 + RUN_LEVELS];
};


// Run detection shared by the gathering producers.  Every lane holds four consecutive list
// rows (r0..r3; `valid` = how many of them exist).  A block of 4n rows led by lane L (L a
// multiple of n) can be fetched as one tiled box iff all its rows exist and are consecutive
// tokens.  Returns, for this lane, the number of lanes n of the largest such aligned block
// that contains the lane's rows (0 if not even its own four rows qualify); the lane with
// (lane % n == 0) issues the box.  `lanes` is 32 (whole tile) or 16 (a 64-row k-step).
__device__ __forceinline__ int run_block_lanes(int lane_in_group, int lanes, int r0, int r1, int r2, int r3, int valid,
                                               int max_lanes) {
  const int prev3 = __shfl_up_sync(0xFFFFFFFFu, r3, 1);
  const bool s0 = (valid < 1) || (r0 != prev3 + 1);          // row 4l starts a new run (or is missing)
  const bool s1 = (valid < 2) || (r1 != r0 + 1);
  const bool s2 = (valid < 3) || (r2 != r1 + 1);
  const bool s3 = (valid < 4) || (r3 != r2 + 1);
  const uint32_t b0 = __ballot_sync(0xFFFFFFFFu, s0);
  const uint32_t bi = __ballot_sync(0xFFFFFFFFu, s1 || s2 || s3);
  const uint32_t bv = __ballot_sync(0xFFFFFFFFu, valid == 4);
  const int shift = (threadIdx.x & 31) - lane_in_group;        // 0, or 16 for the upper half-warp
  int best = 0;
#pragma unroll
  for (int n = 1; n <= 32; n <<= 1) {
    if (n > lanes || n > max_lanes) break;
    const int lead = lane_in_group & ~(n - 1);
    const uint32_t range = (n == 32 ? 0xFFFFFFFFu : ((1u << n) - 1u) << lead) << shift;
    const uint32_t inner = range & ~(1u << (lead + shift));
    const bool ok = (bi & range) == 0 && (b0 & inner) == 0 && (bv & range) == range;
    if (ok) best = n;
  }
  return best;
}

struct TileCoord {
  int mt, nt;           // m-tile over [visual tiles | text tiles], n-tile
  int row0;             // first row of the tile inside its modality's list
  int rows;             // valid rows in the tile (1..128)
  int list_off;         // offset of the modality's list inside perm
  bool text;
};

__device__ __forceinline__ TileCoord decode_tile(int t, int tiles_v, int m_tiles, int n_tiles, int group_m, int Mv,
                                                 int Mt, int cap) {
  TileCoord c;
  const int per_super = group_m * n_tiles;
  const int st = t / per_super;
  const int r = t - st * per_super;
  const int m0 = st * group_m;
  const int gm = min(group_m, m_tiles - m0);
  c.nt = r / gm;
  c.mt = m0 + (r - c.nt * gm);
  c.text = c.mt >= tiles_v;
  const int lt = c.text ? c.mt - tiles_v : c.mt;
  c.row0 = lt * BM;
  const int cnt = c.text ? Mt : Mv;
  c.rows = min(BM, cnt - c.row0);
  c.list_off = c.text ? cap : 0;
  return c;
}

__device__ __forceinline__ void report(int* status, int code) {
  if (status) atomicCAS(status, 0, code);
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ float tanh_approx(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// sigmoid(x) = 0.5 + 0.5 * tanh(0.5 x): one special-function instruction instead of an exponential and a
// reciprocal (the epilogues of short-K tiles are bound by that unit); tanh.approx is good to 2^-11
// relative, a quarter of a bf16 rounding step.
__device__ __forceinline__ float sigmoid_fast(float x) { return fmaf(0.5f, tanh_approx(0.5f * x), 0.5f); }

__device__ __forceinline__ float silu_mul(float t1, float t3) {
  // t1 * sigmoid(t1) * t3 (ffn_kernel/ffn.py:107), in fp32: with h = t1 / 2, t1 * sigmoid(t1) = h + h * tanh(h)
  const float h = 0.5f * t1;
  return fmaf(h, tanh_approx(h), h) * t3;
}


// Rows of the routed intermediate: visual rows start at 0, text rows at the next multiple of
// 256 after the visual rows (the largest row tile any kernel variant uses).
__device__ __forceinline__ int text_row_base(int Mv) { return ((Mv + 255) >> 8) << 8; }

// Epilogue of one accumulator row: this thread owns TMEM lane `taddr`'s row, 256 fp32 columns.
// EPI_STORE : out_row[n_base + c] = bf16(acc[c]),                       256 columns
// EPI_SWIGLU: out_row[n_base + c] = bf16(silu(acc[c]) * acc[128 + c]),   128 columns
__device__ __forceinline__ void unpack_bf16x8(const uint4& v, float (&f)[8]) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __uint_as_float(w[i] << 16);
    f[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
  }
}
__device__ __forceinline__ uint4 pack_bf16x8(const float (&f)[8]) {
  uint4 o;
  o.x = pack_bf16(f[0], f[1]);
  o.y = pack_bf16(f[2], f[3]);
  o.z = pack_bf16(f[4], f[5]);
  o.w = pack_bf16(f[6], f[7]);
  return o;
}

// SwiGLU epilogue of one warp's 32 accumulator rows with coalesced stores.  A lane owns one row of
// the accumulator, so storing straight from registers puts 16 bytes into 32 different rows per
// instruction: 32 cache lines per store, and with three outputs per element (H, T1, T3 in the
// training forward) the load/store unit, not the tensor pipe, sets the pace of short-K tiles.
// Each 32-column chunk therefore goes through a 2 KiB shared-memory transposition (XOR-swizzled
// 16-byte pieces spread over the banks) and leaves as 64 contiguous bytes per row, eight rows
// per instruction.  `row_off` = element offset of this lane's destination row, or -1 for no row.
template <int EPI, int BN_T>
__device__ __forceinline__ void epilogue_glu_staged(uint32_t taddr, const GemmParams& p, long long row_off, int n_base,
                                                    int part, int parts, uint8_t* stg, int lane) {
  constexpr int CH = BN_T / 64;
  const int pc = lane & 3;
  long long ro[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) ro[i] = __shfl_sync(0xFFFFFFFFu, row_off, i * 8 + (lane >> 2));
  uint8_t* wr = stg + lane * 64;
  const int wsw = (lane >> 1) & 3;
  auto flush = [&](const float (&v)[32], __nv_bfloat16* base, int n0) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float a[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) a[e] = v[j * 8 + e];
      *reinterpret_cast<uint4*>(wr + ((j ^ wsw) << 4)) = pack_bf16x8(a);
    }
    __syncwarp();
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int r = i * 8 + (lane >> 2);
      const uint4 val = *reinterpret_cast<const uint4*>(stg + r * 64 + ((pc ^ ((r >> 1) & 3)) << 4));
      if (ro[i] >= 0 && n0 + pc * 8 < p.n_out) *reinterpret_cast<uint4*>(base + ro[i] + n0 + pc * 8) = val;
    }
    __syncwarp();
  };
#pragma unroll 1
  for (int c = part * CH / parts; c < (part + 1) * CH / parts; ++c) {
    uint32_t g[32], u[32];
    tmem_ld_32x32(taddr + c * 32, g);              // gate  (t1)
    tmem_ld_32x32(taddr + BN_T / 2 + c * 32, u);   // up    (t3)
    tmem_ld_wait();
    const int n0 = n_base + c * 32;
    if (n0 >= p.n_out) continue;                   // warp-uniform
    float t1[32], t3[32];
#pragma unroll
    for (int e = 0; e < 32; ++e) {
      t1[e] = __uint_as_float(g[e]);
      t3[e] = __uint_as_float(u[e]);
    }
    if constexpr (EPI == EPI_SWIGLU_SAVE) {
      flush(t1, p.aux0, n0);
      flush(t3, p.aux1, n0);
    }
#pragma unroll
    for (int e = 0; e < 32; ++e) t1[e] = silu_mul(t1[e], t3[e]);
    flush(t1, p.out, n0);
  }
}

// dSwiGLU epilogue (FFN backward) with the same shared-memory transposition, for the two loads of
// the saved pre-activations as well as for the two stores: four accesses per element, each of which
// would otherwise touch 32 rows per instruction.
template <int BN_T>
__device__ __forceinline__ void epilogue_dswiglu_staged(uint32_t taddr, const GemmParams& p, long long row_off,
                                                        int n_base, int part, int parts, uint8_t* stg, int lane) {
  constexpr int CH = BN_T / 32;
  const int pc = lane & 3;
  long long ro[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) ro[i] = __shfl_sync(0xFFFFFFFFu, row_off, i * 8 + (lane >> 2));
  uint8_t* mine = stg + lane * 64;
  const int wsw = (lane >> 1) & 3;
  // global loads of one chunk of a saved matrix: 8 rows x 64 bytes per instruction
  auto load4 = [&](uint4 (&l)[4], const __nv_bfloat16* base, int n0) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      l[i] = make_uint4(0, 0, 0, 0);
      if (ro[i] >= 0 && n0 + pc * 8 < p.n_out) l[i] = *reinterpret_cast<const uint4*>(base + ro[i] + n0 + pc * 8);
    }
  };
  // ... transposed through shared memory into this lane's row
  auto spread = [&](float (&v)[32], const uint4 (&l)[4]) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int r = i * 8 + (lane >> 2);
      *reinterpret_cast<uint4*>(stg + r * 64 + ((pc ^ ((r >> 1) & 3)) << 4)) = l[i];
    }
    __syncwarp();
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float a[8];
      unpack_bf16x8(*reinterpret_cast<const uint4*>(mine + ((j ^ wsw) << 4)), a);
#pragma unroll
      for (int e = 0; e < 8; ++e) v[j * 8 + e] = a[e];
    }
    __syncwarp();
  };
  auto flush = [&](const float (&v)[32], __nv_bfloat16* base, int n0) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float a[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) a[e] = v[j * 8 + e];
      *reinterpret_cast<uint4*>(mine + ((j ^ wsw) << 4)) = pack_bf16x8(a);
    }
    __syncwarp();
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int r = i * 8 + (lane >> 2);
      const uint4 val = *reinterpret_cast<const uint4*>(stg + r * 64 + ((pc ^ ((r >> 1) & 3)) << 4));
      if (ro[i] >= 0 && n0 + pc * 8 < p.n_out) *reinterpret_cast<uint4*>(base + ro[i] + n0 + pc * 8) = val;
    }
    __syncwarp();
  };
  const int c_begin = part * CH / parts, c_end = (part + 1) * CH / parts;
  uint4 l1[4], l3[4];
  load4(l1, p.aux0, n_base + c_begin * 32);
  load4(l3, p.aux1, n_base + c_begin * 32);
#pragma unroll 1
  for (int c = c_begin; c < c_end; ++c) {
    uint32_t acc[32];
    tmem_ld_32x32(taddr + c * 32, acc);
    const int n0 = n_base + c * 32;
    float t1[32], t3[32];
    spread(t1, l1);
    spread(t3, l3);
    if (c + 1 < c_end) {             // the next chunk's loads fly while this one is computed and stored
      load4(l1, p.aux0, n0 + 32);
      load4(l3, p.aux1, n0 + 32);
    }
    tmem_ld_wait();
    if (n0 >= p.n_out) continue;   // warp-uniform
#pragma unroll
    for (int e = 0; e < 32; ++e) {
      const float dh = __uint_as_float(acc[e]);
      const float sg = sigmoid_fast(t1[e]);
      const float d1 = dh * t3[e] * sg * (1.0f + t1[e] * (1.0f - sg));
      t3[e] = dh * t1[e] * sg;     // d3
      t1[e] = d1;
    }
    flush(t1, p.out, n0);
    flush(t3, p.aux2, n0);
  }
}

// OUT_PEER: where the row of token `token` goes (nullptr if the token has no owner among the peers).
__device__ __forceinline__ __nv_bfloat16* peer_row(const GemmParams& p, int token) {
  const int owner = token / p.peer_rows;
  if (token < 0 || owner >= p.peer_world) return nullptr;
  __nv_bfloat16* base = p.peer_out[0];
#pragma unroll
  for (int r = 1; r < MAX_PEERS; ++r)
    if (r == owner) base = p.peer_out[r];
  const int64_t row = static_cast<int64_t>(p.peer_rank) * p.peer_rows + (token - owner * p.peer_rows);
  return base + row * p.ldo;
}

// Plain-store epilogue of one warp's 32 accumulator rows, to wherever each row lives: a token row of
// the output (scatter), a row of a routed-order matrix, or a row in another GPU's memory (OUT_PEER).
// A lane owns one accumulator row, so storing from registers would put 16 bytes into 32 different
// rows per instruction; over NVLink that wastes most of every packet, and locally it measured
// 2-6 % slower end to end (M=32768 d=1024 h=2048 down projection 0.116 -> 0.110 ms, M=32768
// K=N=4096 MaskedLinear forward 0.906 -> 0.884 ms).  So each 64-column chunk goes through a
// shared-memory transposition (XOR-swizzled 16-byte pieces: 4.5 wavefronts per 16-byte store
// instruction and 8.5 per load under ncu, against 26 M tensor-pipe wavefronts it is 5 % of the traffic) and is stored
// as 128 contiguous bytes per row, four rows per instruction.
// `dst` is this lane's destination row (nullptr: no row), `stg` the warp's 4 KiB staging area.
template <int BN_T>
__device__ __forceinline__ void epilogue_rows_staged(uint32_t taddr, const GemmParams& p, __nv_bfloat16* dst, int n_base,
                                                   int part, int parts, uint8_t* stg, int lane) {
  constexpr int CH = BN_T / 64;
  const unsigned long long dptr = reinterpret_cast<unsigned long long>(dst);
  const int piece = lane & 7;
#pragma unroll 1
  for (int c = part * CH / parts; c < (part + 1) * CH / parts; ++c) {
    uint32_t v0[32], v1[32];
    tmem_ld_32x32(taddr + c * 64, v0);
    tmem_ld_32x32(taddr + c * 64 + 32, v1);
    tmem_ld_wait();
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float a[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) a[e] = __uint_as_float(j < 4 ? v0[j * 8 + e] : v1[(j - 4) * 8 + e]);
      *reinterpret_cast<uint4*>(stg + lane * 128 + ((j ^ (lane & 7)) << 4)) = pack_bf16x8(a);
    }
    __syncwarp();
    const int n0 = n_base + c * 64 + piece * 8;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int r = i * 4 + (lane >> 3);
      const unsigned long long rp = __shfl_sync(0xFFFFFFFFu, dptr, r);
      const uint4 val = *reinterpret_cast<const uint4*>(stg + r * 128 + ((piece ^ (r & 7)) << 4));
      if (rp != 0ull && n0 < p.n_out) *reinterpret_cast<uint4*>(rp + static_cast<unsigned long long>(n0) * 2ull) = val;
    }
    __syncwarp();
  }
}

// The same row store with the values taken from `nsplit` (at most kMaxSplitK) fp32 partial tiles in memory
// (split-K), added in item order.  A partial tile is stored as [BN_T / 4 column groups][128 rows] of float4,
// so that the 32 lanes of a warp (32 rows) touch 512 contiguous bytes per access; `src` is this lane's row
// in column group 0 of the first partial tile, `stride` the float4 between tiles.  Sixteen columns of every
// partial tile are requested before any is added (up to sixteen 16-byte loads in flight per thread: a
// load-add loop would pay the L2 latency once per split and group).
constexpr int kMaxSplitK = 4;
template <int BN_T>
__device__ __forceinline__ void epilogue_rows_from_partials(const float4* src, int nsplit, int64_t stride, const GemmParams& p,
                                                           __nv_bfloat16* dst, int n_base, int part, int parts,
                                                           uint8_t* stg, int lane) {
  // With two warps per lane quarter (parts == 2) each takes half of every 64-column chunk: 32 columns = two
  // groups of sixteen, stored as 64 contiguous bytes per row, eight rows per instruction.
  constexpr int CH = BN_T / 64;
  const unsigned long long dptr = reinterpret_cast<unsigned long long>(dst);
  const int lanes_per_row = 8 / parts;                       // 16-byte pieces of a row this warp stores
  const int piece = (lane & (lanes_per_row - 1)) + part * lanes_per_row;
#pragma unroll 1
  for (int c = 0; c < CH; ++c) {
#pragma unroll 1
    for (int jp = part * 4 / parts; jp < (part + 1) * 4 / parts; ++jp) {
      float4 t[kMaxSplitK][4];
#pragma unroll
      for (int sp = 0; sp < kMaxSplitK; ++sp) {
#pragma unroll
        for (int k = 0; k < 4; ++k) t[sp][k] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (src != nullptr && sp < nsplit) {
          const float4* q = src + sp * stride + (c * 16 + jp * 4) * BM;
#pragma unroll
          for (int k = 0; k < 4; ++k) t[sp][k] = __ldcg(q + k * BM);
        }
      }
#pragma unroll
      for (int k = 0; k < 4; ++k) {
#pragma unroll
        for (int sp = 1; sp < kMaxSplitK; ++sp) {
          t[0][k].x += t[sp][k].x;
          t[0][k].y += t[sp][k].y;
          t[0][k].z += t[sp][k].z;
          t[0][k].w += t[sp][k].w;
        }
      }
#pragma unroll
      for (int jj = 0; jj < 2; ++jj) {
        const int j = jp * 2 + jj;
        const float a[8] = {t[0][2 * jj].x,     t[0][2 * jj].y,     t[0][2 * jj].z,     t[0][2 * jj].w,
                            t[0][2 * jj + 1].x, t[0][2 * jj + 1].y, t[0][2 * jj + 1].z, t[0][2 * jj + 1].w};
        *reinterpret_cast<uint4*>(stg + lane * 128 + ((j ^ (lane & 7)) << 4)) = pack_bf16x8(a);
      }
    }
    __syncwarp();
    const int n0 = n_base + c * 64 + piece * 8;
    const int rows_per_store = 32 / lanes_per_row;
    for (int i = 0; i < lanes_per_row; ++i) {
      const int r = i * rows_per_store + lane / lanes_per_row;
      const unsigned long long rp = __shfl_sync(0xFFFFFFFFu, dptr, r);
      const uint4 val = *reinterpret_cast<const uint4*>(stg + r * 128 + ((piece ^ (r & 7)) << 4));
      if (rp != 0ull && n0 < p.n_out) *reinterpret_cast<uint4*>(rp + static_cast<unsigned long long>(n0) * 2ull) = val;
    }
    __syncwarp();
  }
}

// BN_T = 128 (6 stages of 32 KiB) sits between the two.
// BN_T = 256 is the throughput tile; BN_T = 64 (K-major weights only) spreads a problem with few row
// tiles over more SMs: 8 stages of 24 KiB, four times as many column tiles.
template <int A_MODE, int EPI, int OUT_MODE, bool B_MN, int BN_T>
__global__ void __launch_bounds__(GEMM_THREADS_MAX, 1)
routed_gemm_kernel(const __grid_constant__ AMaps am, const __grid_constant__ CUtensorMap tmBv0,
                   const __grid_constant__ CUtensorMap tmBv1, const __grid_constant__ CUtensorMap tmBt0,
                   const __grid_constant__ CUtensorMap tmBt1, const GemmParams p) {
  static_assert(BN_T == 256 || ((BN_T == 128 || BN_T == 64) && !B_MN),
                "128- and 64-column tiles exist for K-major weights only");
  constexpr int TB_BYTES = BN_T * BK * 2;
  constexpr int TSTAGE_BYTES = A_BYTES + TB_BYTES;
  constexpr int TSTAGES = (BN_T == 256) ? STAGES : (BN_T == 128 ? 6 : 8);   // 192 KiB of stages either way
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + TSTAGES * TSTAGE_BYTES);
  uint64_t* empty = full + TSTAGES;
  uint64_t* tfull = empty + TSTAGES;   // accumulator ready for the epilogue   [2]
  uint64_t* tempty = tfull + 2;       // accumulator drained by the epilogue  [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < TSTAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tfull[i], 1);
      mbar_init(&tempty[i], 4 * epilogue_parts());
    }
    *abort_flag = 0;
    fence_mbar_init();
    for (int i = 0; i <= COPY_MAP; ++i) tma_prefetch_desc(&am.m[i]);
    tma_prefetch_desc(&tmBv0);
    tma_prefetch_desc(&tmBv1);
    tma_prefetch_desc(&tmBt0);
    tma_prefetch_desc(&tmBt1);
  }
  if (warp == 1) {
    tmem_alloc<1>(tmem_slot, TMEM_COLS);
    tmem_relinquish<1>();
  }
  // a dependent kernel may start its own set-up now (this kernel's CTAs are all resident or done)
  griddep_launch_dependents();
  if (p.pdl) {
    // weights into L2 while the predecessor (routing and row copy, or the gate/up GEMM) is still running
    const int lines_per_row = (p.pf_row_bytes + 127) >> 7;
    const int64_t lines = static_cast<int64_t>(p.pf_rows) * lines_per_row;
#pragma unroll 1
    for (int w = 0; w < 4; ++w) {
      if (p.pf_base[w] == nullptr) continue;
      for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < lines;
           i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int64_t r = i / lines_per_row;
        const int l = static_cast<int>(i - r * lines_per_row);
        prefetch_l2(p.pf_base[w] + r * p.pf_stride + min(l * 128, p.pf_row_bytes - 1));
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  griddep_wait();                       // from here on the predecessor's results (lists, counts, activations) are read

  const int Mv = p.counts[0], Mt = p.counts[1], cap = p.counts[2];
  const int tiles_v = (Mv + BM - 1) / BM;
  const int m_tiles = tiles_v + (Mt + BM - 1) / BM;
  constexpr int N_PER_TILE = epi_glu(EPI) ? BN_T / 2 : BN_T;
  const int n_tiles = (p.n_out + N_PER_TILE - 1) / N_PER_TILE;
  const int total_tiles = m_tiles * n_tiles;
  const int k_steps0 = (p.k_len + BK - 1) / BK;                 // first contraction segment
  const int k_steps = k_steps0 + (p.k_len1 + BK - 1) / BK;      // plus the optional second one
  // split-K: work item = (tile, range of k-steps); consecutive CTAs take the ranges of one tile
  constexpr bool SPLITK = A_MODE == A_ROUTED && EPI == EPI_STORE && OUT_MODE == OUT_SCATTER && !B_MN;
  const int nsplit = SPLITK ? p.ksplit : 1;
  const int total_items = total_tiles * nsplit;

  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    int stage = 0;
    uint32_t phase = 0;
    int issued = 0;
    bool ok = true;
    const bool via_copy = (A_MODE == A_GATHER) && p.a_copy && mask_is_scattered(p.counts, p.a_copy);
    for (int item = blockIdx.x; item < total_items && ok; item += gridDim.x) {
      const int t = item / nsplit, split = item - t * nsplit;
      const int ks_begin = split * k_steps / nsplit, ks_end = (split + 1) * k_steps / nsplit;
      const TileCoord tc = decode_tile(t, tiles_v, m_tiles, n_tiles, p.group_m, Mv, Mt, cap);
      int r0 = p.pad_row, r1 = p.pad_row, r2 = p.pad_row, r3 = p.pad_row;
      // How this lane's rows are fetched: as part of a tiled box of 4 * run_lanes consecutive
      // token rows issued by the block's first lane, or (run_lanes == 0) by a gather4 of its own.
      int run_lanes = 0;
      if constexpr (A_MODE == A_GATHER) {
        const int lr = 4 * lane;  // first of this lane's four rows
        const int valid = min(4, max(0, tc.rows - lr));
        if (valid > 0) {
          const int4 v = *reinterpret_cast<const int4*>(p.perm + tc.list_off + tc.row0 + lr);
          r0 = v.x;
          if (valid > 1) r1 = v.y;
          if (valid > 2) r2 = v.z;
          if (valid > 3) r3 = v.w;
        }
        run_lanes = run_block_lanes(lane, 32, r0, r1, r2, r3, valid, p.max_run_rows >> 2);
      }
      const bool run_lead = run_lanes > 0 && (lane & (run_lanes - 1)) == 0;
      const CUtensorMap* run_map = &am.m[run_lanes > 0 ? 32 - __clz(run_lanes) : 0];
      const CUtensorMap* mB0 = tc.text ? &tmBt0 : &tmBv0;
      const CUtensorMap* mB1 = tc.text ? &tmBt1 : &tmBv1;
      for (int ks = ks_begin; ks < ks_end; ++ks) {
        int w = 1;
        if (lane == 0) w = mbar_wait(&empty[stage], phase ^ 1, abort_flag) ? 1 : 0;
        w = __shfl_sync(0xFFFFFFFFu, w, 0);
        if (!w) {
          if (lane == 0) report(p.status, ST_TIMEOUT_PRODUCER);
          ok = false;
          break;
        }
        uint8_t* sa = smem + stage * TSTAGE_BYTES;
        uint8_t* sb = sa + A_BYTES;
        if (lane == 0) mbar_arrive_expect_tx(&full[stage], TSTAGE_BYTES);
        __syncwarp();
        const bool seg1 = ks >= k_steps0;
        const int kx = (seg1 ? ks - k_steps0 : ks) * BK;
        if constexpr (A_MODE == A_GATHER) {
          if (via_copy) {
            if (lane == 0)
              tma_load_2d(sa, &am.m[COPY_MAP], &full[stage], kx, (tc.text ? text_row_base(Mv) : 0) + tc.row0);
          } else if (run_lanes == 0) {
            tma_gather4(sa + lane * 512, &am.m[0], &full[stage], kx, r0, r1, r2, r3);
          } else if (run_lead) {
            tma_load_2d(sa + lane * 512, run_map, &full[stage], kx, r0);
          }
        } else {
          if (lane == 0)
            tma_load_2d(sa, &am.m[seg1 ? RUN_LEVELS - 1 : RUN_LEVELS], &full[stage], kx,
                        (tc.text ? text_row_base(Mv) : 0) + tc.row0);
        }
        if (lane == 0) {
          // gate/up tiles take their two column halves from two weights; plain tiles take both
          // halves from one weight (the second weight belongs to the second contraction segment)
          const CUtensorMap* mLo = epi_glu(EPI) ? mB0 : (seg1 ? mB1 : mB0);
          const CUtensorMap* mHi = epi_glu(EPI) ? mB1 : mLo;
          if constexpr (!B_MN) {
            // K-major weights: two boxes of BN_T/2 weight rows x 64 k
            const int n0 = epi_glu(EPI) ? tc.nt * (BN_T / 2) : tc.nt * BN_T;
            const int n1 = epi_glu(EPI) ? n0 : n0 + BN_T / 2;
            tma_load_2d(sb, mLo, &full[stage], kx, n0);
            tma_load_2d(sb + TB_BYTES / 2, mHi, &full[stage], kx, n1);
          } else {
            // MN-major weights: four boxes of 64 k rows x 64 output columns
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const CUtensorMap* m = j >= 2 ? mHi : mLo;
              const int n = epi_glu(EPI) ? tc.nt * (BN_T / 2) + (j & 1) * 64 : tc.nt * BN_T + j * 64;
              tma_load_2d(sb + j * (TB_BYTES / 4), m, &full[stage], n, kx);
            }
          }
        }
        ++issued;
        if (++stage == TSTAGES) { stage = 0; phase ^= 1; }
      }
    }
    if (*abort_flag && lane == 0) {
      // let the copies already issued land before the CTA gives its shared memory back
      int s = stage;
      uint32_t ph = phase;
      const int n = issued < TSTAGES ? issued : TSTAGES;
      for (int i = 0; i < n; ++i) {
        if (--s < 0) { s = TSTAGES - 1; ph ^= 1; }
        int dummy = 0;
        mbar_wait(&full[s], ph, &dummy, 1000000ull);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_bf16(BM, BN_T, false, B_MN);
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      long long t_begin = clock64(), t_full = 0, t_tmem = 0;
      for (int item = blockIdx.x; item < total_items && ok; item += gridDim.x, ++it) {
        const int split = item % nsplit;
        const int ks_begin = split * k_steps / nsplit, ks_end = (split + 1) * k_steps / nsplit;
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        long long tw = clock64();
        if (!mbar_wait(&tempty[acc], acc_phase ^ 1, abort_flag)) {
          report(p.status, ST_TIMEOUT_MMA_TMEM);
          break;
        }
        t_tmem += clock64() - tw;
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + acc * BN_T;
        for (int ks = ks_begin; ks < ks_end; ++ks) {
          tw = clock64();
          if (!mbar_wait(&full[stage], phase, abort_flag)) {
            report(p.status, ST_TIMEOUT_MMA_FULL);
            ok = false;
            break;
          }
          t_full += clock64() - tw;
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smem + stage * TSTAGE_BYTES);
          const uint32_t b_addr = a_addr + A_BYTES;
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; ++kk) {
            const uint64_t da = umma_smem_desc(a_addr + kk * (UMMA_K * 2), 16, 1024);
            const uint64_t db = B_MN ? umma_smem_desc(b_addr + kk * (UMMA_K * 128), TB_BYTES / 4, 1024)
                                     : umma_smem_desc(b_addr + kk * (UMMA_K * 2), 16, 1024);
            umma_bf16<1>(tmem_d, da, db, idesc, (ks > ks_begin || kk != 0) ? 1u : 0u);
          }
          umma_commit(&empty[stage]);
          if (++stage == TSTAGES) { stage = 0; phase ^= 1; }
        }
        if (ok) umma_commit(&tfull[acc]);
      }
      if (p.prof) {
        p.prof[blockIdx.x * 8 + 0] = clock64() - t_begin;
        p.prof[blockIdx.x * 8 + 1] = t_full;
        p.prof[blockIdx.x * 8 + 2] = t_tmem;
        p.prof[blockIdx.x * 8 + 7] = it;
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ epilogue
    const int q = warp & 3;              // TMEM lane quarter this warp may read
    const int part = (warp - 2) >> 2;    // which half of the columns it drains
    const int row = q * 32 + lane;       // row of the tile held by this thread
    int it = 0;
    for (int item = blockIdx.x; item < total_items; item += gridDim.x, ++it) {
      const int t = item / nsplit;
      const TileCoord tc = decode_tile(t, tiles_v, m_tiles, n_tiles, p.group_m, Mv, Mt, cap);
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      const bool valid = row < tc.rows;
      int64_t dst_row = 0;
      __nv_bfloat16* peer_dst = nullptr;
      if (valid) {
        if constexpr (OUT_MODE == OUT_PEER) peer_dst = peer_row(p, p.perm[tc.list_off + tc.row0 + row]);
        else if constexpr (OUT_MODE == OUT_SCATTER) dst_row = p.perm[tc.list_off + tc.row0 + row];
        else dst_row = static_cast<int64_t>(tc.text ? text_row_base(Mv) : 0) + tc.row0 + row;
      }
      int w = 1;
      if (lane == 0) w = mbar_wait(&tfull[acc], acc_phase, abort_flag) ? 1 : 0;
      w = __shfl_sync(0xFFFFFFFFu, w, 0);
      if (!w) {
        if (lane == 0) report(p.status, ST_TIMEOUT_EPILOGUE);
        break;
      }
      tc_fence_after();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN_T;
      if constexpr (SPLITK) {
        if (nsplit > 1) {
          // this item's partial tile out (rows that exist only), the accumulator back to the MMA warp at once
          const int parts = epilogue_parts();
          float4* mine = reinterpret_cast<float4*>(p.kpart) + static_cast<int64_t>(item) * (BN_T / 4) * BM + row;
          constexpr int CH32 = BN_T / 32;
#pragma unroll 1
          for (int c = part * CH32 / parts; c < (part + 1) * CH32 / parts; ++c) {
            uint32_t v[32];
            tmem_ld_32x32(taddr + c * 32, v);
            tmem_ld_wait();
            if (valid) {
#pragma unroll
              for (int e = 0; e < 32; e += 4)
                __stcg(mine + (c * 8 + e / 4) * BM,
                       make_float4(__uint_as_float(v[e]), __uint_as_float(v[e + 1]), __uint_as_float(v[e + 2]),
                                   __uint_as_float(v[e + 3])));
            }
          }
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&tempty[acc]);
          __threadfence();
          int* s_last = reinterpret_cast<int*>(const_cast<int*>(abort_flag) + 1);
          asm volatile("bar.sync 1, %0;" ::"r"(128 * parts) : "memory");
          if (warp == 2 && lane == 0) {
            const unsigned int old = atomicAdd(&p.kcount[t], 1u);
            const int last = old == static_cast<unsigned int>(nsplit - 1);
            if (last) p.kcount[t] = 0u;          // everybody has arrived: zero again for the next launch on this slot
            *s_last = last;
          }
          asm volatile("bar.sync 1, %0;" ::"r"(128 * parts) : "memory");
          if (*s_last) {
            __threadfence();
            const float4* first = reinterpret_cast<const float4*>(p.kpart) + static_cast<int64_t>(t) * nsplit * (BN_T / 4) * BM + row;
            epilogue_rows_from_partials<BN_T>(valid ? first : nullptr, nsplit, static_cast<int64_t>(BN_T / 4) * BM, p,
                                              valid ? p.out + dst_row * p.ldo : nullptr, tc.nt * BN_T, part, parts,
                                              smem + TSTAGES * TSTAGE_BYTES + 256 + (warp - 2) * 4096, lane);
          }
          continue;
        }
      }
      if constexpr (epi_glu(EPI))
        epilogue_glu_staged<EPI, BN_T>(taddr, p, valid ? dst_row * p.ldo : -1ll, tc.nt * (BN_T / 2), part,
                                       epilogue_parts(), smem + TSTAGES * TSTAGE_BYTES + 256 + (warp - 2) * 2048, lane);
      else if constexpr (EPI == EPI_DSWIGLU)
        epilogue_dswiglu_staged<BN_T>(taddr, p, valid ? dst_row * p.ldo : -1ll, tc.nt * BN_T, part, epilogue_parts(),
                                      smem + TSTAGES * TSTAGE_BYTES + 256 + (warp - 2) * 2048, lane);
      else
        epilogue_rows_staged<BN_T>(taddr, p, OUT_MODE == OUT_PEER ? peer_dst : (valid ? p.out + dst_row * p.ldo : nullptr),
                                   tc.nt * BN_T, part, epilogue_parts(),
                                   smem + TSTAGES * TSTAGE_BYTES + 256 + (warp - 2) * 4096, lane);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty[acc]);
    }
  }

  // ---------------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc<1>(tmem_base, TMEM_COLS);
  }
}


// -------------------------------------------------------------------------------------------
// CTA-pair variant: two CTAs of a cluster (the two SMs of one TPC) share one
// tcgen05.mma.cta_group::2 of 256 x 256 x 16.  Each CTA fetches its own 128 tile rows of A and
// only HALF of the B tile (128 of the 256 weight rows), so a k-step moves 32 KiB per SM instead
// of 48 and needs two TMA instructions instead of three; six stages fit where four did.
//   * the even CTA (the leader) issues every MMA; its `full` barriers collect the byte counts
//     of both CTAs' loads (the partner's TMA credits the leader's barrier directly);
//   * tcgen05.commit with a two-CTA mask frees the stage in both CTAs and hands the finished
//     accumulator (128 lanes x 256 columns in each CTA's TMEM) to both epilogues;
//   * both CTAs' epilogue warps report back to the leader's `tempty` barrier.
// In the gate/up kernel the leader's B half is the gate weight slice and the partner's the up
// slice, so each CTA's accumulator is again 128 gate columns | 128 up columns.
// -------------------------------------------------------------------------------------------
constexpr int PAIR_STAGES = 6;
constexpr int PAIR_B_BYTES = B_BYTES / 2;                       // 16 KiB: this CTA's half of B
constexpr int PAIR_STAGE_BYTES = A_BYTES + PAIR_B_BYTES;        // 32 KiB
constexpr int PAIR_SMEM = PAIR_STAGES * PAIR_STAGE_BYTES + 1024 + 256;
constexpr int PAIR_BM = 2 * BM;                                 // 256 tile rows per pair

template <int A_MODE, int EPI, int OUT_MODE, bool B_MN>
__global__ void __launch_bounds__(GEMM_THREADS_MAX, 1)
routed_gemm_pair_kernel(const __grid_constant__ AMaps am, const __grid_constant__ CUtensorMap tmBv0,
                        const __grid_constant__ CUtensorMap tmBv1, const __grid_constant__ CUtensorMap tmBt0,
                        const __grid_constant__ CUtensorMap tmBt1, const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + PAIR_STAGES * PAIR_STAGE_BYTES);
  uint64_t* empty = full + PAIR_STAGES;
  uint64_t* tfull = empty + PAIR_STAGES;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();        // 0 = leader
  const int pair_id = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < PAIR_STAGES; ++s) {
      mbar_init(&full[s], 2);      // one arrive.expect_tx per CTA of the pair (used in the leader only)
      mbar_init(&empty[s], 1);     // the leader's commit, delivered to both CTAs
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tfull[i], 1);     // the leader's commit, delivered to both CTAs
      mbar_init(&tempty[i], 8 * epilogue_parts());   // the epilogue warps of both CTAs (used in the leader only)
    }
    *abort_flag = 0;
    fence_mbar_init();
    for (int i = 0; i <= COPY_MAP; ++i) tma_prefetch_desc(&am.m[i]);
    tma_prefetch_desc(&tmBv0);
    tma_prefetch_desc(&tmBv1);
    tma_prefetch_desc(&tmBt0);
    tma_prefetch_desc(&tmBt1);
  }
  if (warp == 1) {
    tmem_alloc<2>(tmem_slot, TMEM_COLS);
    tmem_relinquish<2>();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();              // both CTAs' barriers exist before anybody signals across
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int Mv = p.counts[0], Mt = p.counts[1], cap = p.counts[2];
  const int tiles_v = (Mv + PAIR_BM - 1) / PAIR_BM;
  const int m_tiles = tiles_v + (Mt + PAIR_BM - 1) / PAIR_BM;
  constexpr int N_PER_TILE = epi_glu(EPI) ? BN / 2 : BN;
  const int n_tiles = (p.n_out + N_PER_TILE - 1) / N_PER_TILE;
  const int total_tiles = m_tiles * n_tiles;
  const int k_steps0 = (p.k_len + BK - 1) / BK;                 // first contraction segment
  const int k_steps = k_steps0 + (p.k_len1 + BK - 1) / BK;      // plus the optional second one
  const int text_base = text_row_base(Mv);

  // this CTA's 128 rows of pair tile t
  auto cta_tile = [&](int t) {
    TileCoord c;
    const int per_super = p.group_m * n_tiles;
    const int st = t / per_super;
    const int r = t - st * per_super;
    const int m0 = st * p.group_m;
    const int gm = min(p.group_m, m_tiles - m0);
    c.nt = r / gm;
    c.mt = m0 + (r - c.nt * gm);
    c.text = c.mt >= tiles_v;
    const int lt = c.text ? c.mt - tiles_v : c.mt;
    c.row0 = lt * PAIR_BM + static_cast<int>(rank) * BM;
    const int cnt = c.text ? Mt : Mv;
    c.rows = max(0, min(BM, cnt - c.row0));
    c.list_off = c.text ? cap : 0;
    return c;
  };

  if (warp == 0) {
    // ------------------------------------------------------------------ producer (both CTAs)
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    long long t_begin = clock64(), t_wait = 0;
    const bool via_copy = (A_MODE == A_GATHER) && p.a_copy && mask_is_scattered(p.counts, p.a_copy);
    for (int t = pair_id; t < total_tiles && ok; t += num_pairs) {
      const TileCoord tc = cta_tile(t);
      int r0 = p.pad_row, r1 = p.pad_row, r2 = p.pad_row, r3 = p.pad_row;
      int run_lanes = 0;
      if constexpr (A_MODE == A_GATHER) {
        const int lr = 4 * lane;
        const int valid = min(4, max(0, tc.rows - lr));
        if (valid > 0) {
          const int4 v = *reinterpret_cast<const int4*>(p.perm + tc.list_off + tc.row0 + lr);
          r0 = v.x;
          if (valid > 1) r1 = v.y;
          if (valid > 2) r2 = v.z;
          if (valid > 3) r3 = v.w;
        }
        run_lanes = run_block_lanes(lane, 32, r0, r1, r2, r3, valid, p.max_run_rows >> 2);
      }
      const bool run_lead = run_lanes > 0 && (lane & (run_lanes - 1)) == 0;
      const CUtensorMap* run_map = &am.m[run_lanes > 0 ? 32 - __clz(run_lanes) : 0];
      const bool empty_half = (A_MODE == A_GATHER) && tc.rows == 0;   // nothing to fetch: one out-of-range box
      const CUtensorMap* mB0 = tc.text ? &tmBt0 : &tmBv0;
      const CUtensorMap* mB1 = tc.text ? &tmBt1 : &tmBv1;
      for (int ks = 0; ks < k_steps; ++ks) {
        int w = 1;
        const long long tw = clock64();
        if (lane == 0) w = mbar_wait(&empty[stage], phase ^ 1, abort_flag) ? 1 : 0;
        w = __shfl_sync(0xFFFFFFFFu, w, 0);
        t_wait += clock64() - tw;
        if (!w) {
          if (lane == 0) report(p.status, ST_TIMEOUT_PRODUCER);
          ok = false;
          break;
        }
        uint8_t* sa = smem + stage * PAIR_STAGE_BYTES;
        uint8_t* sb = sa + A_BYTES;
        const uint32_t lead_full = mapa_shared(smem_u32(&full[stage]), 0);
        if (lane == 0) mbar_arrive_expect_tx_cluster(lead_full, PAIR_STAGE_BYTES);
        __syncwarp();
        const bool seg1 = ks >= k_steps0;
        const int kx = (seg1 ? ks - k_steps0 : ks) * BK;
        // gate/up: the leader's half of B is the gate weight, the partner's the up weight;
        // otherwise both halves come from the segment's weight
        const CUtensorMap* mB = epi_glu(EPI) ? (rank ? mB1 : mB0) : (seg1 ? mB1 : mB0);
        if constexpr (A_MODE == A_GATHER) {
          if (via_copy) {
            if (lane == 0) tma_load_2d_pair(sa, &am.m[COPY_MAP], lead_full, kx, (tc.text ? text_base : 0) + tc.row0);
          } else if (empty_half) {
            if (lane == 0) tma_load_2d_pair(sa, &am.m[RUN_LEVELS], lead_full, kx, p.pad_row);
          } else if (run_lanes == 0) {
            tma_gather4_pair(sa + lane * 512, &am.m[0], lead_full, kx, r0, r1, r2, r3);
          } else if (run_lead) {
            tma_load_2d_pair(sa + lane * 512, run_map, lead_full, kx, r0);
          }
        } else {
          if (lane == 0)
            tma_load_2d_pair(sa, &am.m[seg1 ? RUN_LEVELS - 1 : RUN_LEVELS], lead_full, kx,
                             (tc.text ? text_base : 0) + tc.row0);
        }
        if (lane == 0) {
          // this CTA's half of the B tile
          const int n0 = epi_glu(EPI) ? tc.nt * (BN / 2) : tc.nt * BN + static_cast<int>(rank) * (BN / 2);
          if constexpr (!B_MN) {
            tma_load_2d_pair(sb, mB, lead_full, kx, n0);
          } else {
            tma_load_2d_pair(sb, mB, lead_full, n0, kx);
            tma_load_2d_pair(sb + PAIR_B_BYTES / 2, mB, lead_full, n0 + 64, kx);
          }
        }
        if (++stage == PAIR_STAGES) { stage = 0; phase ^= 1; }
      }
    }
    if (p.prof && lane == 0) {
      p.prof[blockIdx.x * 8 + 3] = t_wait;
      p.prof[blockIdx.x * 8 + 4] = clock64() - t_begin;
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (leader only)
    if (rank == 0 && lane == 0) {
      constexpr uint32_t idesc = umma_idesc_bf16(PAIR_BM, BN, false, B_MN);
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      long long t_begin = clock64(), t_full = 0, t_tmem = 0;
      for (int t = pair_id; t < total_tiles && ok; t += num_pairs, ++it) {
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        long long tw = clock64();
        if (!mbar_wait(&tempty[acc], acc_phase ^ 1, abort_flag)) {
          report(p.status, ST_TIMEOUT_MMA_TMEM);
          break;
        }
        t_tmem += clock64() - tw;
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + acc * BN;
        for (int ks = 0; ks < k_steps; ++ks) {
          tw = clock64();
          if (!mbar_wait(&full[stage], phase, abort_flag)) {
            report(p.status, ST_TIMEOUT_MMA_FULL);
            ok = false;
            break;
          }
          t_full += clock64() - tw;
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smem + stage * PAIR_STAGE_BYTES);
          const uint32_t b_addr = a_addr + A_BYTES;
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; ++kk) {
            const uint64_t da = umma_smem_desc(a_addr + kk * (UMMA_K * 2), 16, 1024);
            const uint64_t db = B_MN ? umma_smem_desc(b_addr + kk * (UMMA_K * 128), PAIR_B_BYTES / 2, 1024)
                                     : umma_smem_desc(b_addr + kk * (UMMA_K * 2), 16, 1024);
            umma_bf16<2>(tmem_d, da, db, idesc, (ks | kk) != 0 ? 1u : 0u);
          }
          umma_commit_pair(&empty[stage], 3);
          if (++stage == PAIR_STAGES) { stage = 0; phase ^= 1; }
        }
        if (ok) umma_commit_pair(&tfull[acc], 3);
      }
      if (p.prof) {
        p.prof[blockIdx.x * 8 + 0] = clock64() - t_begin;
        p.prof[blockIdx.x * 8 + 1] = t_full;
        p.prof[blockIdx.x * 8 + 2] = t_tmem;
        p.prof[blockIdx.x * 8 + 7] = it;
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ epilogue (both CTAs)
    const int q = warp & 3;
    const int part = (warp - 2) >> 2;
    const int row = q * 32 + lane;
    int it = 0;
    long long t_begin = clock64(), t_wait = 0;
    for (int t = pair_id; t < total_tiles; t += num_pairs, ++it) {
      const TileCoord tc = cta_tile(t);
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      const bool valid = row < tc.rows;
      int64_t dst_row = 0;
      __nv_bfloat16* peer_dst = nullptr;
      if (valid) {
        if constexpr (OUT_MODE == OUT_PEER) peer_dst = peer_row(p, p.perm[tc.list_off + tc.row0 + row]);
        else if constexpr (OUT_MODE == OUT_SCATTER) dst_row = p.perm[tc.list_off + tc.row0 + row];
        else dst_row = static_cast<int64_t>(tc.text ? text_base : 0) + tc.row0 + row;
      }
      int w = 1;
      const long long tw = clock64();
      if (lane == 0) w = mbar_wait(&tfull[acc], acc_phase, abort_flag) ? 1 : 0;
      w = __shfl_sync(0xFFFFFFFFu, w, 0);
      t_wait += clock64() - tw;
      if (!w) {
        if (lane == 0) report(p.status, ST_TIMEOUT_EPILOGUE);
        break;
      }
      tc_fence_after();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN;
      if constexpr (epi_glu(EPI))
        epilogue_glu_staged<EPI, BN>(taddr, p, valid ? dst_row * p.ldo : -1ll, tc.nt * N_PER_TILE, part,
                                     epilogue_parts(), smem + PAIR_STAGES * PAIR_STAGE_BYTES + 256 + (warp - 2) * 2048, lane);
      else if constexpr (EPI == EPI_DSWIGLU)
        epilogue_dswiglu_staged<BN>(taddr, p, valid ? dst_row * p.ldo : -1ll, tc.nt * N_PER_TILE, part, epilogue_parts(),
                                    smem + PAIR_STAGES * PAIR_STAGE_BYTES + 256 + (warp - 2) * 2048, lane);
      else
        epilogue_rows_staged<BN>(taddr, p, OUT_MODE == OUT_PEER ? peer_dst : (valid ? p.out + dst_row * p.ldo : nullptr),
                                 tc.nt * N_PER_TILE, part, epilogue_parts(),
                                 smem + PAIR_STAGES * PAIR_STAGE_BYTES + 256 + (warp - 2) * 4096, lane);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(mapa_shared(smem_u32(&tempty[acc]), 0));
    }
    if (p.prof && warp == 2 && lane == 0) {
      p.prof[blockIdx.x * 8 + 5] = t_wait;
      p.prof[blockIdx.x * 8 + 6] = clock64() - t_begin;
    }
  }

  // ---------------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();   // the partner's shared memory and barriers stay alive until both CTAs are done
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc<2>(tmem_base, TMEM_COLS);
  }
}

// -------------------------------------------------------------------------------------------
// Weight-gradient GEMM of MaskedLinear backward (replaces _masked_matmul_bwd_db,
// ffn_kernel/linear.py:329-415):   out_g[p, q] = sum over rows r of modality g of P[r, p] * Q[r, q]
// P and Q are the two row-major token matrices (activations and upstream gradient, in the
// order that makes `out` match the weight's storage).  The contraction runs over the
// modality's row list, so both operands are MN-major in shared memory: a k-step is 64 list
// rows, each contributing one 128-byte row per 64-column block, fetched with gather4.  Rows
// past the end of the list are fetched from an out-of-range row index and arrive as zeros.
// The reference streams every token through every tile and zeroes the other modality's rows;
// here a tile only ever touches its own modality's rows.
// -------------------------------------------------------------------------------------------
struct WgradParams {
  const int* perm;
  const int* counts;
  __nv_bfloat16* out_v;
  __nv_bfloat16* out_t;
  int64_t ldo;
  int p_dim;      // output rows    (columns of P)
  int q_dim;      // output columns (columns of Q)
  int pad_row;
  int max_run_rows;
  int* status;
  int routed = 0;   // 1: P and Q are in routed order (row = group base + list position), no index list
  long long* prof = nullptr;   // optional per-CTA wait-cycle counters (8 per CTA), as in GemmParams
};

// Views of one operand of the weight-gradient GEMM: m[0] single rows (gather4), m[1 + i] boxes of
// 4 << i rows (4...64), 64 columns wide.
struct WMaps {
  CUtensorMap m[RUN_LEVELS];
};

struct WgradTile {
  int pt, qt, cnt, list_off;
  bool text;
};

__device__ __forceinline__ WgradTile decode_wgrad_tile(int t, int p_tiles, int q_tiles, int Mv, int Mt, int cap) {
  WgradTile w;
  const int per_group = p_tiles * q_tiles;
  const int gsel = t / per_group;
  const int r = t - gsel * per_group;
  // the modality with more rows goes first so that the long tiles do not end up in the tail
  const bool text_first = Mt > Mv;
  w.text = (gsel == 0) ? text_first : !text_first;
  w.qt = r / p_tiles;
  w.pt = r - w.qt * p_tiles;
  w.cnt = w.text ? Mt : Mv;
  w.list_off = w.text ? cap : 0;
  return w;
}

__global__ void __launch_bounds__(GEMM_THREADS_MAX, 1)
wgrad_kernel(const __grid_constant__ WMaps pm, const __grid_constant__ WMaps qm, const WgradParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* empty = full + STAGES;
  uint64_t* tfull = empty + STAGES;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tfull[i], 1);
      mbar_init(&tempty[i], 4 * epilogue_parts());
    }
    *abort_flag = 0;
    fence_mbar_init();
    for (int i = 0; i < RUN_LEVELS; ++i) {
      tma_prefetch_desc(&pm.m[i]);
      tma_prefetch_desc(&qm.m[i]);
    }
  }
  if (warp == 1) {
    tmem_alloc<1>(tmem_slot, TMEM_COLS);
    tmem_relinquish<1>();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int Mv = p.counts[0], Mt = p.counts[1], cap = p.counts[2];
  const int p_tiles = (p.p_dim + BM - 1) / BM;
  const int q_tiles = (p.q_dim + BN - 1) / BN;
  const int total_tiles = 2 * p_tiles * q_tiles;

  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    int stage = 0;
    uint32_t phase = 0;
    int issued = 0;
    bool ok = true;
    const bool routed = p.routed != 0;
    const WMaps* mp = &pm;
    const WMaps* mq = &qm;
    const int pad_row = p.pad_row;
    const int gi = lane & 15;     // which group of four list rows inside the k-step
    const int half = lane >> 4;   // which 64-column block (of a pair)
    long long t_begin = clock64(), t_wait = 0;
    for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
      const WgradTile wt = decode_wgrad_tile(t, p_tiles, q_tiles, Mv, Mt, cap);
      if (wt.cnt == 0) continue;
      const int k_steps = (wt.cnt + BK - 1) / BK;
      const int* list = p.perm + wt.list_off;
      const int4 pad4 = make_int4(pad_row, pad_row, pad_row, pad_row);
      const int group_base = wt.text ? text_row_base(Mv) : 0;
      int4 nxt = (!routed && 4 * gi < wt.cnt) ? *reinterpret_cast<const int4*>(list + 4 * gi) : pad4;
      for (int ks = 0; ks < k_steps; ++ks) {
        if (routed && (ks + 1) * BK <= wt.cnt) {
          // 64 whole rows of a routed-order matrix: six boxes, one lane each, nothing to detect.
          // (The instruction count of this loop is what the MMA issuer ends up waiting for.)
          int w = 1;
          const long long tw = clock64();
          if (lane == 0) w = mbar_wait(&empty[stage], phase ^ 1, abort_flag) ? 1 : 0;
          w = __shfl_sync(0xFFFFFFFFu, w, 0);
          t_wait += clock64() - tw;
          if (!w) {
            if (lane == 0) report(p.status, ST_TIMEOUT_PRODUCER);
            ok = false;
            break;
          }
          uint8_t* sp = smem + stage * STAGE_BYTES;
          if (lane == 0) mbar_arrive_expect_tx(&full[stage], STAGE_BYTES);
          __syncwarp();
          if (lane < 6) {
            const bool is_p = lane < 2;
            const int b = is_p ? lane : lane - 2;
            tma_load_2d((is_p ? sp : sp + A_BYTES) + b * 8192, is_p ? &mp->m[RUN_LEVELS - 1] : &mq->m[RUN_LEVELS - 1],
                        &full[stage], (is_p ? wt.pt * BM : wt.qt * BN) + b * 64, group_base + ks * BK);
          }
          ++issued;
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
          continue;
        }
        const int lr = ks * BK + 4 * gi;
        int4 v = nxt;
        if (routed) {
          v = make_int4(group_base + lr, group_base + lr + 1, group_base + lr + 2, group_base + lr + 3);
        } else if (ks + 1 < k_steps) {
          // the next k-step's rows are requested now so that the load is hidden behind this step
          nxt = (lr + BK < wt.cnt) ? *reinterpret_cast<const int4*>(list + lr + BK) : pad4;
        }
        int r0 = pad_row, r1 = pad_row, r2 = pad_row, r3 = pad_row;
        const int valid = min(4, max(0, wt.cnt - lr));
        if (valid > 0) {
          r0 = v.x;
          if (valid > 1) r1 = v.y;
          if (valid > 2) r2 = v.z;
          if (valid > 3) r3 = v.w;
        }
        // list rows that are consecutive tokens are fetched as tiled boxes of 4..64 rows per column block
        const int run_lanes = run_block_lanes(gi, 16, r0, r1, r2, r3, valid, p.max_run_rows >> 2);
        const bool run_lead = run_lanes > 0 && (gi & (run_lanes - 1)) == 0;
        const int level = run_lanes > 0 ? 32 - __clz(run_lanes) : 0;
        int w = 1;
        const long long tw = clock64();
        if (lane == 0) w = mbar_wait(&empty[stage], phase ^ 1, abort_flag) ? 1 : 0;
        w = __shfl_sync(0xFFFFFFFFu, w, 0);
        t_wait += clock64() - tw;
        if (!w) {
          if (lane == 0) report(p.status, ST_TIMEOUT_PRODUCER);
          ok = false;
          break;
        }
        uint8_t* sp = smem + stage * STAGE_BYTES;
        uint8_t* sq = sp + A_BYTES;
        if (lane == 0) mbar_arrive_expect_tx(&full[stage], STAGE_BYTES);
        __syncwarp();
        // P: two 64-column blocks; Q: four.  Block b lives at b * 8 KiB, list row j at j * 128 B.
        uint8_t* dp = sp + half * 8192 + gi * 512;
        uint8_t* dq0 = sq + half * 8192 + gi * 512;
        uint8_t* dq1 = sq + (2 + half) * 8192 + gi * 512;
        const int cp = wt.pt * BM + half * 64, cq0 = wt.qt * BN + half * 64, cq1 = wt.qt * BN + (2 + half) * 64;
        if (run_lanes == 0) {
          tma_gather4(dp, &mp->m[0], &full[stage], cp, r0, r1, r2, r3);
          tma_gather4(dq0, &mq->m[0], &full[stage], cq0, r0, r1, r2, r3);
          tma_gather4(dq1, &mq->m[0], &full[stage], cq1, r0, r1, r2, r3);
        } else if (run_lead) {
          tma_load_2d(dp, &mp->m[level], &full[stage], cp, r0);
          tma_load_2d(dq0, &mq->m[level], &full[stage], cq0, r0);
          tma_load_2d(dq1, &mq->m[level], &full[stage], cq1, r0);
        }
        ++issued;
        if (++stage == STAGES) { stage = 0; phase ^= 1; }
      }
    }
    if (p.prof && lane == 0) {
      p.prof[blockIdx.x * 8 + 3] = t_wait;
      p.prof[blockIdx.x * 8 + 4] = clock64() - t_begin;
    }
    if (*abort_flag && lane == 0) {
      int s = stage;
      uint32_t ph = phase;
      const int n = issued < STAGES ? issued : STAGES;
      for (int i = 0; i < n; ++i) {
        if (--s < 0) { s = STAGES - 1; ph ^= 1; }
        int dummy = 0;
        mbar_wait(&full[s], ph, &dummy, 1000000ull);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_bf16(BM, BN, true, true);
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      long long t_begin = clock64(), t_full = 0, t_tmem = 0;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        const WgradTile wt = decode_wgrad_tile(t, p_tiles, q_tiles, Mv, Mt, cap);
        if (wt.cnt == 0) continue;
        const int k_steps = (wt.cnt + BK - 1) / BK;
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        ++it;
        long long tw = clock64();
        if (!mbar_wait(&tempty[acc], acc_phase ^ 1, abort_flag)) {
          report(p.status, ST_TIMEOUT_MMA_TMEM);
          break;
        }
        t_tmem += clock64() - tw;
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + acc * BN;
        for (int ks = 0; ks < k_steps; ++ks) {
          tw = clock64();
          if (!mbar_wait(&full[stage], phase, abort_flag)) {
            report(p.status, ST_TIMEOUT_MMA_FULL);
            ok = false;
            break;
          }
          t_full += clock64() - tw;
          tc_fence_after();
          const uint32_t p_addr = smem_u32(smem + stage * STAGE_BYTES);
          const uint32_t q_addr = p_addr + A_BYTES;
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; ++kk) {
            const uint64_t dp = umma_smem_desc(p_addr + kk * (UMMA_K * 128), 8192, 1024);
            const uint64_t dq = umma_smem_desc(q_addr + kk * (UMMA_K * 128), 8192, 1024);
            umma_bf16<1>(tmem_d, dp, dq, idesc, (ks | kk) != 0 ? 1u : 0u);
          }
          umma_commit(&empty[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (ok) umma_commit(&tfull[acc]);
      }
      if (p.prof) {
        p.prof[blockIdx.x * 8 + 0] = clock64() - t_begin;
        p.prof[blockIdx.x * 8 + 1] = t_full;
        p.prof[blockIdx.x * 8 + 2] = t_tmem;
        p.prof[blockIdx.x * 8 + 7] = it;
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ epilogue
    const int q = warp & 3;
    const int part = (warp - 2) >> 2;
    const int row = q * 32 + lane;
    int it = 0;
    for (int t = blockIdx.x; t < total_tiles; t += gridDim.x) {
      const WgradTile wt = decode_wgrad_tile(t, p_tiles, q_tiles, Mv, Mt, cap);
      const int prow = wt.pt * BM + row;
      const bool valid = prow < p.p_dim;
      __nv_bfloat16* out_row = (wt.text ? p.out_t : p.out_v) + static_cast<int64_t>(prow) * p.ldo;
      const int q_base = wt.qt * BN;
      if (wt.cnt == 0) {
        // a modality without tokens has a zero gradient
        if (valid) {
          for (int c = part * (BN / epilogue_parts()); c < (part + 1) * (BN / epilogue_parts()); c += 8)
            if (q_base + c < p.q_dim) *reinterpret_cast<uint4*>(out_row + q_base + c) = make_uint4(0, 0, 0, 0);
        }
        continue;
      }
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      ++it;
      int w = 1;
      if (lane == 0) w = mbar_wait(&tfull[acc], acc_phase, abort_flag) ? 1 : 0;
      w = __shfl_sync(0xFFFFFFFFu, w, 0);
      if (!w) {
        if (lane == 0) report(p.status, ST_TIMEOUT_EPILOGUE);
        break;
      }
      tc_fence_after();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN;
#pragma unroll 1
      for (int c = part * (BN / 32) / epilogue_parts(); c < (part + 1) * (BN / 32) / epilogue_parts(); ++c) {
        uint32_t v[32];
        tmem_ld_32x32(taddr + c * 32, v);
        tmem_ld_wait();
        const int n0 = q_base + c * 32;
        if (valid && n0 < p.q_dim) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            if (n0 + j * 8 < p.q_dim) {
              uint4 o;
              o.x = pack_bf16(__uint_as_float(v[j * 8 + 0]), __uint_as_float(v[j * 8 + 1]));
              o.y = pack_bf16(__uint_as_float(v[j * 8 + 2]), __uint_as_float(v[j * 8 + 3]));
              o.z = pack_bf16(__uint_as_float(v[j * 8 + 4]), __uint_as_float(v[j * 8 + 5]));
              o.w = pack_bf16(__uint_as_float(v[j * 8 + 6]), __uint_as_float(v[j * 8 + 7]));
              *reinterpret_cast<uint4*>(out_row + n0 + j * 8) = o;
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty[acc]);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc<1>(tmem_base, TMEM_COLS);
  }
}

// -------------------------------------------------------------------------------------------
// Weight gradient on CTA pairs: operands in routed order only (the FFN backward's matrices, or the
// routed-order copies the MaskedLinear backward makes).  One 256 x 256 output tile per pair; each
// CTA fetches its own 128 columns of P and only its half of the 256 columns of Q, i.e. four boxes
// of 64 rows x 64 columns per k-step instead of the single-CTA kernel's six, 32 KiB instead of
// 48 KiB, six pipeline stages instead of four.  (In the single-CTA kernel the MMA issuer spends
// 40-50 % of its time waiting for operands; the TMA requests per k-step are what it waits for.)
// The last k-step of a modality, when it is not 64 whole rows, is fetched row by row (gather4)
// with the missing rows pointed at an out-of-range row, which the TMA unit fills with zeros.
// -------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(GEMM_THREADS_MAX, 1)
wgrad_pair_kernel(const __grid_constant__ WMaps pm, const __grid_constant__ WMaps qm, const WgradParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + PAIR_STAGES * PAIR_STAGE_BYTES);
  uint64_t* empty = full + PAIR_STAGES;
  uint64_t* tfull = empty + PAIR_STAGES;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int pair_id = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < PAIR_STAGES; ++s) {
      mbar_init(&full[s], 2);
      mbar_init(&empty[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tfull[i], 1);
      mbar_init(&tempty[i], 8 * epilogue_parts());
    }
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&pm.m[0]);
    tma_prefetch_desc(&qm.m[0]);
    tma_prefetch_desc(&pm.m[RUN_LEVELS - 1]);
    tma_prefetch_desc(&qm.m[RUN_LEVELS - 1]);
  }
  if (warp == 1) {
    tmem_alloc<2>(tmem_slot, TMEM_COLS);
    tmem_relinquish<2>();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int Mv = p.counts[0], Mt = p.counts[1], cap = p.counts[2];
  const int p_tiles = (p.p_dim + PAIR_BM - 1) / PAIR_BM;
  const int q_tiles = (p.q_dim + BN - 1) / BN;
  const int total_tiles = 2 * p_tiles * q_tiles;

  if (warp == 0) {
    // ------------------------------------------------------------------ producer (both CTAs)
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    long long t_begin = clock64(), t_wait = 0;
    for (int t = pair_id; t < total_tiles && ok; t += num_pairs) {
      const WgradTile wt = decode_wgrad_tile(t, p_tiles, q_tiles, Mv, Mt, cap);
      if (wt.cnt == 0) continue;
      const int k_steps = (wt.cnt + BK - 1) / BK;
      const int group_base = wt.text ? text_row_base(Mv) : 0;
      // lanes 0,1: this CTA's two 64-column blocks of P; lanes 2,3: its two blocks of Q
      const bool is_p = (lane & 2) == 0;
      const int blk = lane & 1;
      const int col = (is_p ? wt.pt * PAIR_BM : wt.qt * BN) + static_cast<int>(rank) * BM + blk * 64;
      const int dst_off = (is_p ? 0 : A_BYTES) + blk * 8192;
      for (int ks = 0; ks < k_steps; ++ks) {
        int w = 1;
        const long long tw = clock64();
        if (lane == 0) w = mbar_wait(&empty[stage], phase ^ 1, abort_flag) ? 1 : 0;
        w = __shfl_sync(0xFFFFFFFFu, w, 0);
        t_wait += clock64() - tw;
        if (!w) {
          if (lane == 0) report(p.status, ST_TIMEOUT_PRODUCER);
          ok = false;
          break;
        }
        uint8_t* st = smem + stage * PAIR_STAGE_BYTES;
        const uint32_t lead_full = mapa_shared(smem_u32(&full[stage]), 0);
        if (lane == 0) mbar_arrive_expect_tx_cluster(lead_full, PAIR_STAGE_BYTES);
        __syncwarp();
        if ((ks + 1) * BK <= wt.cnt) {
          if (lane < 4)
            tma_load_2d_pair(st + dst_off, is_p ? &pm.m[RUN_LEVELS - 1] : &qm.m[RUN_LEVELS - 1], lead_full, col,
                             group_base + ks * BK);
        } else if (lane < 16) {
          // ragged end of the modality: lane g fetches rows 4g..4g+3 of the k-step for all four blocks
          const int lr = ks * BK + 4 * lane;
          const int r0 = lr + 0 < wt.cnt ? group_base + lr + 0 : p.pad_row;
          const int r1 = lr + 1 < wt.cnt ? group_base + lr + 1 : p.pad_row;
          const int r2 = lr + 2 < wt.cnt ? group_base + lr + 2 : p.pad_row;
          const int r3 = lr + 3 < wt.cnt ? group_base + lr + 3 : p.pad_row;
          const int cp = wt.pt * PAIR_BM + static_cast<int>(rank) * BM;
          const int cq = wt.qt * BN + static_cast<int>(rank) * BM;
          tma_gather4_pair(st + lane * 512, &pm.m[0], lead_full, cp, r0, r1, r2, r3);
          tma_gather4_pair(st + 8192 + lane * 512, &pm.m[0], lead_full, cp + 64, r0, r1, r2, r3);
          tma_gather4_pair(st + A_BYTES + lane * 512, &qm.m[0], lead_full, cq, r0, r1, r2, r3);
          tma_gather4_pair(st + A_BYTES + 8192 + lane * 512, &qm.m[0], lead_full, cq + 64, r0, r1, r2, r3);
        }
        if (++stage == PAIR_STAGES) { stage = 0; phase ^= 1; }
      }
    }
    if (p.prof && lane == 0) {
      p.prof[blockIdx.x * 8 + 3] = t_wait;
      p.prof[blockIdx.x * 8 + 4] = clock64() - t_begin;
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (leader only)
    if (rank == 0 && lane == 0) {
      constexpr uint32_t idesc = umma_idesc_bf16(PAIR_BM, BN, true, true);
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      long long t_begin = clock64(), t_full = 0, t_tmem = 0;
      for (int t = pair_id; t < total_tiles && ok; t += num_pairs) {
        const WgradTile wt = decode_wgrad_tile(t, p_tiles, q_tiles, Mv, Mt, cap);
        if (wt.cnt == 0) continue;
        const int k_steps = (wt.cnt + BK - 1) / BK;
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        ++it;
        long long tw = clock64();
        if (!mbar_wait(&tempty[acc], acc_phase ^ 1, abort_flag)) {
          report(p.status, ST_TIMEOUT_MMA_TMEM);
          break;
        }
        t_tmem += clock64() - tw;
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + acc * BN;
        for (int ks = 0; ks < k_steps; ++ks) {
          tw = clock64();
          if (!mbar_wait(&full[stage], phase, abort_flag)) {
            report(p.status, ST_TIMEOUT_MMA_FULL);
            ok = false;
            break;
          }
          t_full += clock64() - tw;
          tc_fence_after();
          const uint32_t p_addr = smem_u32(smem + stage * PAIR_STAGE_BYTES);
          const uint32_t q_addr = p_addr + A_BYTES;
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; ++kk) {
            const uint64_t dp = umma_smem_desc(p_addr + kk * (UMMA_K * 128), 8192, 1024);
            const uint64_t dq = umma_smem_desc(q_addr + kk * (UMMA_K * 128), 8192, 1024);
            umma_bf16<2>(tmem_d, dp, dq, idesc, (ks | kk) != 0 ? 1u : 0u);
          }
          umma_commit_pair(&empty[stage], 3);
          if (++stage == PAIR_STAGES) { stage = 0; phase ^= 1; }
        }
        if (ok) umma_commit_pair(&tfull[acc], 3);
      }
      if (p.prof) {
        p.prof[blockIdx.x * 8 + 0] = clock64() - t_begin;
        p.prof[blockIdx.x * 8 + 1] = t_full;
        p.prof[blockIdx.x * 8 + 2] = t_tmem;
        p.prof[blockIdx.x * 8 + 7] = it;
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ epilogue (both CTAs)
    const int q = warp & 3;
    const int part = (warp - 2) >> 2;
    const int row = q * 32 + lane;
    int it = 0;
    for (int t = pair_id; t < total_tiles; t += num_pairs) {
      const WgradTile wt = decode_wgrad_tile(t, p_tiles, q_tiles, Mv, Mt, cap);
      const int prow = wt.pt * PAIR_BM + static_cast<int>(rank) * BM + row;
      const bool valid = prow < p.p_dim;
      __nv_bfloat16* out_row = (wt.text ? p.out_t : p.out_v) + static_cast<int64_t>(prow) * p.ldo;
      const int q_base = wt.qt * BN;
      if (wt.cnt == 0) {
        if (valid) {
          for (int c = part * (BN / epilogue_parts()); c < (part + 1) * (BN / epilogue_parts()); c += 8)
            if (q_base + c < p.q_dim) *reinterpret_cast<uint4*>(out_row + q_base + c) = make_uint4(0, 0, 0, 0);
        }
        continue;
      }
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      ++it;
      int w = 1;
      if (lane == 0) w = mbar_wait(&tfull[acc], acc_phase, abort_flag) ? 1 : 0;
      w = __shfl_sync(0xFFFFFFFFu, w, 0);
      if (!w) {
        if (lane == 0) report(p.status, ST_TIMEOUT_EPILOGUE);
        break;
      }
      tc_fence_after();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN;
#pragma unroll 1
      for (int c = part * (BN / 32) / epilogue_parts(); c < (part + 1) * (BN / 32) / epilogue_parts(); ++c) {
        uint32_t v[32];
        tmem_ld_32x32(taddr + c * 32, v);
        tmem_ld_wait();
        const int n0 = q_base + c * 32;
        if (valid && n0 < p.q_dim) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            if (n0 + j * 8 < p.q_dim) {
              float a[8];
#pragma unroll
              for (int e = 0; e < 8; ++e) a[e] = __uint_as_float(v[j * 8 + e]);
              *reinterpret_cast<uint4*>(out_row + n0 + j * 8) = pack_bf16x8(a);
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(mapa_shared(smem_u32(&tempty[acc]), 0));
    }
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc<2>(tmem_base, TMEM_COLS);
  }
}

// -------------------------------------------------------------------------------------------
// host side
// -------------------------------------------------------------------------------------------
struct WeightView {
  const void* base;
  int64_t stride_k, stride_n;  // elements
  int64_t K, N;                // logical [K, N]
};

// Tensor map over one weight for the B operand.  K-major: storage rows are output columns.
static int weight_map(CUtensorMap* m, const WeightView& w, bool* mn_major, int box_rows = BN / 2) {
  if (w.stride_k == 1 && (w.stride_n >= w.K || w.N == 1)) {
    *mn_major = false;
    return make_tensor_map_2d(m, w.base, w.K, w.N, w.stride_n, BK, box_rows);
  }
  if (w.stride_n == 1 && (w.stride_k >= w.N || w.K == 1)) {
    *mn_major = true;
    return make_tensor_map_2d(m, w.base, w.N, w.K, w.stride_k, 64, BK);
  }
  return FFNK_ERR_LAYOUT;
}

static int gather_maps(AMaps& a, const void* base, int64_t cols, int64_t rows, int64_t ld) {
  int r = make_tensor_map_2d(&a.m[0], base, cols, rows, ld, BK, 1);
  for (int i = 0; i < RUN_LEVELS && !r; ++i) r = make_tensor_map_2d(&a.m[1 + i], base, cols, rows, ld, BK, 4u << i);
  a.m[COPY_MAP] = a.m[RUN_LEVELS];
  return r;
}

// Largest run box in rows (an override of 0, 4, 8, ..., 128 caps it).
static int max_run_rows() {
  const int v = tune_overrides().max_run_rows;
  return v >= 0 ? v : BM;
}

static long long* g_prof_buffer = nullptr;
long long* debug_profile_buffer() { return g_prof_buffer; }
static int g_sm_margin = 0;   // SMs the persistent GEMM grids leave free (for a concurrent collective)

static int usable_sms(const DeviceInfo& dev) {
  int n = dev.sm_count - g_sm_margin;
  return n < 2 ? 2 : n;
}

// Row tiles per super-tile.  One super-tile of A rows should stay in L2 while the weights stream past
// it: about 32 MiB of A for single CTAs (128-row tiles), about 16 MiB for CTA pairs (256-row tiles).
// Measured with `python -m ffn_kernel_b200.tune`: pairs at K=4096 (MaskedLinear backward, M=32768)
// 8 or 16 row tiles 1.69 ms, 32 row tiles 1.74, 48 row tiles 1.79; pairs at K=2048 (down projection,
// M=32768) 8-16 row tiles 0.103 ms, 64 row tiles 0.109; single CTAs at K=4096 (gate/up) 32 row tiles
// 2.07 ms, 16 row tiles 2.12, 8 row tiles 2.28.
static int pick_group_m(int64_t k_len, bool pair = false) {
  const int forced = tune_overrides().group_m;
  if (forced > 0) return forced;
  int64_t g = pair ? (16ll << 20) / (2 * BM * k_len * 2) : (32ll << 20) / (BM * k_len * 2);
  if (g < 4) g = 4;
  if (g > 64) g = 64;
  return static_cast<int>(g);
}

// Tile table (replaces the reference's JSON lookup, ffn_kernel/utils.py:3-5).
//   pair   : CTA pairs, 256-row tiles.  Measured at d=4096/h=11008, M=16384: +4 % when A arrives as one
//            box per tile and the epilogue is a plain store (down projection), -1...3 % under the
//            two-weight SwiGLU tile, so from M = 4096 it is used for the former, and for the latter
//            only from M = 16384 and when the weights fit in L2.
//   narrow : single CTAs with 64 accumulator columns, for problems with so few row tiles that 256-wide
//            tiles would leave most SMs idle (small M: the weights then stream through 4x as many CTAs).
//   else   : single CTAs, 128 x 256 tiles.
// ffnk_tune_override("pair", 0/1) and ("narrow", 0/1/2: 256-, 64-, 128-column tiles) replace the choice for a measurement.
struct TileChoice {
  bool pair;
  int bn;   // accumulator columns per tile
};

static TileChoice pick_tile(int64_t M, int64_t n_out, int a_mode, int epi, bool k_major_weights,
                            int64_t k_len = int64_t(1) << 30) {
  const int force_pair = tune_overrides().pair;
  const int force_narrow = tune_overrides().narrow;
  TileChoice t{false, BN};
  // Two-weight (SwiGLU) tiles go to pairs only when the four weights (8 d h bytes) stay in L2 and there
  // are many row tiles: the GEMM is then bound by L2 -> SM traffic, which a pair cuts by a third
  // (M=32768 d=1024 h=2048: 0.221 -> 0.214 ms; M=16384 d=4096 h=1376: 0.279 -> 0.257 ms).  With weights
  // streaming from DRAM single CTAs are a percent or two faster (d=4096 h=11008), and at M=4099
  // (d=1024 h=2816) pairs lose 14 %.
  const bool glu_pair = M >= 16384 && k_len * n_out <= (int64_t(8) << 20);
  const bool pair = force_pair >= 0 ? force_pair != 0
                                    : (M >= 4096 && a_mode == A_ROUTED && (!epi_glu(epi) || glu_pair));
  if (pair) {
    t.pair = true;
    return t;
  }
  if (!k_major_weights || force_narrow == 0) return t;
  if (force_narrow == 1 || force_narrow == 2) {
    t.bn = force_narrow == 1 ? 64 : 128;
    return t;
  }
  // Few row tiles: narrower column tiles put more CTAs to work.  Estimate = waves on the SMs times the
  // bytes one CTA pulls per k-step (A 16 KiB + 128 B per accumulator column); the widest tile wins ties.
  const int sms = device_info().sm_count;
  const int64_t m_tiles = (M + BM - 1) / BM + 1;
  int64_t best = -1;
  for (int bn : {256, 128, 64}) {
    const int64_t n_per_tile = epi_glu(epi) ? bn / 2 : bn;
    const int64_t tiles = m_tiles * ((n_out + n_per_tile - 1) / n_per_tile);
    int64_t est = ((tiles + sms - 1) / sms) * (16384 + 128 * bn);
    if (epi_glu(epi) && M <= BM) {
      // One row tile per modality: the token rows come out of L2 and the weights are what streams.  In SM
      // units of one tile's bytes: full waves cost the number of SMs each, a last wave of r tiles costs
      // max(r, SMs / 2) (an SM alone pulls about twice its share of the HBM rate, no more); and however
      // narrow the tile, a CTA issues four MMAs of about 128 cycles per k-step, which bounds the narrowest
      // tiles (d=4096, h=11008, 8 tokens: 256 columns 85 us, 128 columns 79 us, 64 columns 105 us;
      // d=1024, h=2816, 127 tokens: 17.0 / 15.2 / 20.1 us).
      const int64_t full = tiles / sms, rest = tiles % sms;
      const int64_t stream = (full * sms + (rest == 0 ? 0 : (2 * rest > sms ? rest : sms / 2))) * (4096 + 128 * bn);
      const int64_t issue = ((tiles + sms - 1) / sms) * sms * 12288;
      est = stream > issue ? stream : issue;
    }
    if (best < 0 || est < best) {
      best = est;
      t.bn = bn;
    }
  }
  return t;
}

static bool weights_k_major(int64_t stride_k, int64_t stride_n, int64_t K) { return stride_k == 1 && stride_n >= K; }

// Early start of a single-CTA GEMM behind its predecessor (GemmParams::pdl), with up to four K-major
// weights [rows, row_elems] to ask into L2 meanwhile; more than 64 MiB of weights are not prefetched
// (they would push one another out of L2 again).
static void early_start(GemmParams& p, const void* const* weights, int nweights, int64_t rows, int64_t row_elems,
                        int64_t stride_elems, bool k_major) {
  p.pdl = 1;
  if (!k_major || nweights * rows * row_elems * 2 > (int64_t(64) << 20) || rows >= (1ll << 30) || row_elems >= (1ll << 29))
    return;
  for (int i = 0; i < nweights && i < 4; ++i) p.pf_base[i] = static_cast<const char*>(weights[i]);
  p.pf_stride = stride_elems * 2;
  p.pf_rows = static_cast<int>(rows);
  p.pf_row_bytes = static_cast<int>(row_elems * 2);
}

template <int A_MODE, int EPI, int OUT_MODE>
static int launch_gemm(const AMaps& tmA, const CUtensorMap (&tmB)[4], bool b_mn, const GemmParams& p,
                       int64_t M, TileChoice tile, cudaStream_t stream) {
  const DeviceInfo& dev = device_info();
  if (dev.cc_major != 10) return FFNK_ERR_DEVICE;
  const int n_per_tile = epi_glu(EPI) ? tile.bn / 2 : tile.bn;
  const int64_t n_tiles = (p.n_out + n_per_tile - 1) / n_per_tile;
  constexpr int extra_smem = EPI == EPI_STORE ? STORE_STAGING : GLU_STAGING;
  if (tile.pair) {
    GemmParams pp = p;
    pp.group_m = pick_group_m(static_cast<int64_t>(p.k_len) + p.k_len1, true);
    int64_t pairs = ((M + PAIR_BM - 1) / PAIR_BM + 1) * n_tiles;
    if (pairs > usable_sms(dev) / 2) pairs = usable_sms(dev) / 2;
    if (pairs < 1) pairs = 1;
    auto go = [&](auto kernel) -> int {
      cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PAIR_SMEM + extra_smem);
      if (e != cudaSuccess) return cuda_status(e);
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3(static_cast<unsigned>(2 * pairs));
      cfg.blockDim = dim3(gemm_threads_for(static_cast<int64_t>(p.k_len) + p.k_len1));
      cfg.dynamicSmemBytes = PAIR_SMEM + extra_smem;
      cfg.stream = stream;
      cudaLaunchAttribute attr[1];
      attr[0].id = cudaLaunchAttributeClusterDimension;
      attr[0].val.clusterDim.x = 2;
      attr[0].val.clusterDim.y = 1;
      attr[0].val.clusterDim.z = 1;
      cfg.attrs = attr;
      cfg.numAttrs = 1;
      return cuda_status(cudaLaunchKernelEx(&cfg, kernel, tmA, tmB[0], tmB[1], tmB[2], tmB[3], pp));
    };
    return b_mn ? go(routed_gemm_pair_kernel<A_MODE, EPI, OUT_MODE, true>)
                : go(routed_gemm_pair_kernel<A_MODE, EPI, OUT_MODE, false>);
  }
  int64_t grid = ((M + BM - 1) / BM + 1) * n_tiles * (p.ksplit > 1 ? p.ksplit : 1);
  if (grid > usable_sms(dev)) grid = usable_sms(dev);
  if (grid < 1) grid = 1;
  auto go = [&](auto kernel) -> int {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, GEMM_SMEM + extra_smem);
    if (e != cudaSuccess) return cuda_status(e);
    // a split contraction is short per item and ends in a pass over the partial tiles: eight epilogue warps
    const int threads = p.ksplit > 1 ? GEMM_THREADS_MAX : gemm_threads_for(static_cast<int64_t>(p.k_len) + p.k_len1);
    if (p.pdl) {
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3(static_cast<unsigned>(grid));
      cfg.blockDim = dim3(threads);
      cfg.dynamicSmemBytes = GEMM_SMEM + extra_smem;
      cfg.stream = stream;
      cudaLaunchAttribute attr[1];
      attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
      attr[0].val.programmaticStreamSerializationAllowed = 1;
      cfg.attrs = attr;
      cfg.numAttrs = 1;
      return cuda_status(cudaLaunchKernelEx(&cfg, kernel, tmA, tmB[0], tmB[1], tmB[2], tmB[3], p));
    }
    kernel<<<static_cast<unsigned>(grid), threads, GEMM_SMEM + extra_smem, stream>>>(
        tmA, tmB[0], tmB[1], tmB[2], tmB[3], p);
    return cuda_status(cudaGetLastError());
  };
  if (tile.bn == 64) return go(routed_gemm_kernel<A_MODE, EPI, OUT_MODE, false, 64>);
  if (tile.bn == 128) return go(routed_gemm_kernel<A_MODE, EPI, OUT_MODE, false, 128>);
  return b_mn ? go(routed_gemm_kernel<A_MODE, EPI, OUT_MODE, true, BN>)
              : go(routed_gemm_kernel<A_MODE, EPI, OUT_MODE, false, BN>);
}

// out_g[p, q] = sum over the rows of modality g of P[row, p] * Q[row, q], for both modalities.
// rows: token rows picked through the routing lists, or (routed != 0) rows of matrices that are
// already in routed order.  `rows_total` is the height of P and Q.
// Average run length below which a routed-order copy beats gathering rows inside a GEMM with
// `columns` output columns (see mask_is_scattered).
static int copy_threshold(int64_t columns) {
  const int forced = tune_overrides().copy_threshold;
  if (forced >= 0) return forced;
  const int64_t t = columns / 6;
  return static_cast<int>(t < 32 ? 32 : (t > 4096 ? 4096 : t));
}

static int wgrad_maps(WMaps& w, const void* base, int64_t cols, int64_t rows, int64_t ld) {
  int r = make_tensor_map_2d(&w.m[0], base, cols, rows, ld, BK, 1);
  for (int i = 1; i < RUN_LEVELS && !r; ++i) r = make_tensor_map_2d(&w.m[i], base, cols, rows, ld, BK, 2u << i);
  return r;
}

static int launch_wgrad(const void* P, int64_t ldp, int64_t p_dim, const void* Q, int64_t ldq, int64_t q_dim,
                        int64_t rows_total, void* out_v, void* out_t, int64_t ldo, int routed, const int32_t* perm,
                        const int32_t* counts, int32_t* status, cudaStream_t s) {
  const DeviceInfo& dev = device_info();
  WMaps tmP, tmQ;
  int r = wgrad_maps(tmP, P, p_dim, rows_total, ldp);
  if (r) return r;
  if ((r = wgrad_maps(tmQ, Q, q_dim, rows_total, ldq))) return r;
  WgradParams wp{perm, counts, static_cast<__nv_bfloat16*>(out_v), static_cast<__nv_bfloat16*>(out_t), ldo,
                 static_cast<int>(p_dim), static_cast<int>(q_dim), static_cast<int>(rows_total),
                 max_run_rows() < 64 ? max_run_rows() : 64, status, routed};
  wp.prof = g_prof_buffer;
  // operands in routed order and an output big enough for 256 x 256 tiles: the CTA-pair kernel
  // (ffnk_tune_override("wgrad_pair", 0/1) replaces the choice for a measurement)
  const int force_pair = tune_overrides().wgrad_pair;
  const bool pair_ok = routed != 0;
  const bool pair = pair_ok && (force_pair >= 0 ? force_pair != 0 : (p_dim >= 256 && q_dim >= 128 && rows_total >= 1024));
  if (pair) {
    int64_t pairs = 2 * ((p_dim + PAIR_BM - 1) / PAIR_BM) * ((q_dim + BN - 1) / BN);
    if (pairs > usable_sms(dev) / 2) pairs = usable_sms(dev) / 2;
    cudaError_t e = cudaFuncSetAttribute(wgrad_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PAIR_SMEM);
    if (e != cudaSuccess) return cuda_status(e);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(2 * pairs));
    cfg.blockDim = dim3(GEMM_THREADS);
    cfg.dynamicSmemBytes = PAIR_SMEM;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cuda_status(cudaLaunchKernelEx(&cfg, wgrad_pair_kernel, tmP, tmQ, wp));
  }
  int64_t grid = 2 * ((p_dim + BM - 1) / BM) * ((q_dim + BN - 1) / BN);
  if (grid > usable_sms(dev)) grid = usable_sms(dev);
  cudaError_t e = cudaFuncSetAttribute(wgrad_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, GEMM_SMEM);
  if (e != cudaSuccess) return cuda_status(e);
  wgrad_kernel<<<static_cast<unsigned>(grid), GEMM_THREADS, GEMM_SMEM, s>>>(tmP, tmQ, wp);
  return cuda_status(cudaGetLastError());
}

static bool bad_dim(int64_t v) { return v < 8 || (v & 7) || v >= (1ll << 30); }

}  // namespace ffnk

using namespace ffnk;

extern "C" int ffnk_linear_fwd(const void* a, int64_t lda, const void* b1, const void* b2, int64_t b_stride_k,
                               int64_t b_stride_n, const int32_t* perm, const int32_t* counts, void* c, int64_t ldc,
                               void* a_copy, int64_t M, int64_t N, int64_t K, int32_t* status, void* stream) {
  if (M == 0) return 0;
  if (!a || !b1 || !b2 || !perm || !counts || !c) return FFNK_ERR_NULL;
  if (M < 0 || M >= (1ll << 30) || bad_dim(N) || bad_dim(K)) return FFNK_ERR_SHAPE;
  if ((lda & 7) || (ldc & 7) || lda < K || ldc < N || (reinterpret_cast<uintptr_t>(c) & 15)) return FFNK_ERR_ALIGN;
  AMaps tmA;
  CUtensorMap tmB[4];
  int r = gather_maps(tmA, a, K, M, lda);
  if (r) return r;
  if (a_copy) {
    // scattered masks: a routed-order copy of A (made only then) replaces the row gather
    if (reinterpret_cast<uintptr_t>(a_copy) & 15) return FFNK_ERR_ALIGN;
    if ((r = permute_rows_launch(a, lda, perm, counts, a_copy, K, M, K, copy_threshold(N), stream))) return r;
    if ((r = make_tensor_map_2d(&tmA.m[COPY_MAP], a_copy, K, ffnk_route_capacity(M) + 512, K, BK, BM))) return r;
  }
  bool mn1 = false, mn2 = false;
  const TileChoice tile = pick_tile(M, N, A_GATHER, EPI_STORE, weights_k_major(b_stride_k, b_stride_n, K));
  if ((r = weight_map(&tmB[0], WeightView{b1, b_stride_k, b_stride_n, K, N}, &mn1, tile.bn / 2))) return r;
  if ((r = weight_map(&tmB[2], WeightView{b2, b_stride_k, b_stride_n, K, N}, &mn2, tile.bn / 2))) return r;
  tmB[1] = tmB[0];
  tmB[3] = tmB[2];
  GemmParams p{perm, counts, static_cast<__nv_bfloat16*>(c), ldc, static_cast<int>(N), static_cast<int>(K),
               static_cast<int>(M), pick_group_m(K), max_run_rows(), status, g_prof_buffer};
  p.a_copy = a_copy ? copy_threshold(N) : 0;
  return launch_gemm<A_GATHER, EPI_STORE, OUT_SCATTER>(tmA, tmB, mn1, p, M, tile, static_cast<cudaStream_t>(stream));
}

extern "C" int ffnk_ffn_gateup(const void* x, int64_t ldx, const void* w1, const void* w3, const void* u1,
                               const void* u3, int64_t w_stride_k, int64_t w_stride_n, const int32_t* perm,
                               const int32_t* counts, void* out, int64_t ldo, int routed_in, int routed_out, int64_t M,
                               int64_t d, int64_t h, int32_t* status, void* stream) {
  return ffn_gateup_early(x, ldx, w1, w3, u1, u3, w_stride_k, w_stride_n, perm, counts, out, ldo, routed_in, routed_out, M, d,
                          h, 0, status, stream);
}

int ffnk::ffn_gateup_early(const void* x, int64_t ldx, const void* w1, const void* w3, const void* u1, const void* u3,
                           int64_t w_stride_k, int64_t w_stride_n, const int32_t* perm, const int32_t* counts, void* out,
                           int64_t ldo, int routed_in, int routed_out, int64_t M, int64_t d, int64_t h, int early,
                           int32_t* status, void* stream) {
  if (M == 0) return 0;
  if (!x || !w1 || !w3 || !u1 || !u3 || !perm || !counts || !out) return FFNK_ERR_NULL;
  if (M < 0 || M >= (1ll << 30) || bad_dim(d) || bad_dim(h)) return FFNK_ERR_SHAPE;
  if ((ldx & 7) || (ldo & 7) || ldx < d || ldo < h || (reinterpret_cast<uintptr_t>(out) & 15)) return FFNK_ERR_ALIGN;
  AMaps tmA;
  CUtensorMap tmB[4];
  int r;
  if (routed_in) {
    // x is [(cap + 512), d] in routed order (ffnk_permute_rows): one tiled box per A tile
    r = make_tensor_map_2d(&tmA.m[RUN_LEVELS], x, d, ffnk_route_capacity(M) + 512, ldx, BK, BM);
    for (int i = 0; i <= COPY_MAP; ++i)
      if (i != RUN_LEVELS) tmA.m[i] = tmA.m[RUN_LEVELS];
  } else {
    r = gather_maps(tmA, x, d, M, ldx);
  }
  if (r) return r;
  bool mn = false, mn_i = false;
  const void* ws[4] = {w1, w3, u1, u3};
  const TileChoice tile = pick_tile(M, h, routed_in ? A_ROUTED : A_GATHER, EPI_SWIGLU,
                                    weights_k_major(w_stride_k, w_stride_n, d), d);
  for (int i = 0; i < 4; ++i) {
    if ((r = weight_map(&tmB[i], WeightView{ws[i], w_stride_k, w_stride_n, d, h}, &mn_i, tile.bn / 2))) return r;
    mn = mn_i;
  }
  GemmParams p{perm, counts, static_cast<__nv_bfloat16*>(out), ldo, static_cast<int>(h), static_cast<int>(d),
               static_cast<int>(M), pick_group_m(d), max_run_rows(), status, g_prof_buffer};
  if (early && !tile.pair) early_start(p, ws, 4, h, d, w_stride_n, weights_k_major(w_stride_k, w_stride_n, d));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (routed_in)
    return routed_out ? launch_gemm<A_ROUTED, EPI_SWIGLU, OUT_ROUTED>(tmA, tmB, mn, p, M, tile, s)
                      : launch_gemm<A_ROUTED, EPI_SWIGLU, OUT_SCATTER>(tmA, tmB, mn, p, M, tile, s);
  return routed_out ? launch_gemm<A_GATHER, EPI_SWIGLU, OUT_ROUTED>(tmA, tmB, mn, p, M, tile, s)
                    : launch_gemm<A_GATHER, EPI_SWIGLU, OUT_SCATTER>(tmA, tmB, mn, p, M, tile, s);
}

// Split-K plan of the down projection for few row tiles.  One tcgen05.mma of 128 rows takes about 128
// cycles however narrow its N is, so a CTA that walks all of K = h alone issues h/16 of them in a row
// (h = 2816: 22 k cycles, most of the kernel's time at 127 tokens) while most SMs have no tile.  With the
// contraction cut into `splits` ranges the chain shrinks by that factor; the price is a round trip of fp32
// partial tiles through L2, a counter per tile and the last arrival's pass over `splits` partial tiles.
// Estimate in cycles for a tile width bn and a number of ranges (one wave only: the items must fit the SMs):
//   k-steps per item x 505 (four MMAs a k-step) + 400 + 85 x bn + 0.2 x items x bn for the exchange
// (the last arrival reads the partial tiles sixteen columns a round, so narrow tiles are what makes the
// exchange cheap), fitted to graph-replayed forwards at d = 1024, h = 2816, 127 tokens: no split 33.7 us;
// 64-column tiles in 2 / 4 ranges 31.2 / 28.3; 128-column tiles in 4 ranges 31.4; 256-column 38.0.  Other
// points: 256 tokens 33.8 -> 29.9, 384 tokens 36.6 -> 33.6, from 500 tokens on nothing is gained; d = 2048,
// h = 8192, 127 tokens 77.7 -> 60.5; d = 4096, h = 11008, 64 tokens 146 -> 134.  A split is taken when its
// estimate is below 0.85 of the unsplit chain.
struct SplitKPlan {
  int bn = 0;        // 0: no split-K (the table's own tile)
  int splits = 1;
};

static SplitKPlan down_splitk_plan(int64_t M, int64_t d, int64_t h, bool k_major) {
  SplitKPlan plan;
  const int forced = tune_overrides().ksplit;
  if (!k_major || forced == 0 || forced == 1 || M >= 4096 || tune_overrides().pair > 0) return plan;
  const int sms = usable_sms(device_info());
  const int64_t m_tiles = (M + BM - 1) / BM + 1;
  const int64_t k_steps = (h + BK - 1) / BK;
  int64_t best = k_steps * 505 * 85 / 100;
  for (int bn : {64, 128, 256}) {
    const int64_t tiles = m_tiles * ((d + bn - 1) / bn);
    if (tiles > kSplitKTiles) continue;
    for (int sp = 2; sp <= kMaxSplitK; ++sp) {
      if (tiles * sp > sms || k_steps / sp < (forced > 1 ? 1 : 4)) break;
      if (forced > 1 && sp != (forced > kMaxSplitK ? kMaxSplitK : forced)) continue;
      const int64_t est = (k_steps + sp - 1) / sp * 505 + 400 + 85 * bn + tiles * sp * bn / 5;
      if (est < best || (forced > 1 && plan.splits <= 1)) {
        best = est;
        plan = SplitKPlan{bn, sp};
      }
    }
  }
  return plan;
}

namespace ffnk {
int64_t ffn_down_scratch_bytes(int64_t M, int64_t d, int64_t h) {
  // the plan may differ with the weights' layout; reserve for the K-major one (the other never splits)
  const SplitKPlan pl = down_splitk_plan(M, d, h, true);
  if (pl.splits <= 1) return 0;
  const int64_t tiles = ((M + BM - 1) / BM + 1) * ((d + pl.bn - 1) / pl.bn);
  return tiles * pl.splits * BM * pl.bn * static_cast<int64_t>(sizeof(float));
}
}  // namespace ffnk

// the device address of the split-K counters, looked up once per process
static int splitk_counters(unsigned int** out) {
  static unsigned int* cached = nullptr;
  static std::mutex mu;
  std::lock_guard<std::mutex> lock(mu);
  if (!cached) {
    void* ptr = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&ptr, g_splitk_count);
    if (e != cudaSuccess) return cuda_status(e);
    cached = static_cast<unsigned int*>(ptr);
  }
  *out = cached;
  return 0;
}

int ffnk::ffn_down_with_scratch(const void* inter, int64_t ldi, const void* w2, const void* u2, int64_t w_stride_k,
                                int64_t w_stride_n, const int32_t* perm, const int32_t* counts, void* y, int64_t ldy,
                                int64_t M, int64_t d, int64_t h, void* scratch, int64_t scratch_bytes, int early,
                                int32_t* status, void* stream) {
  if (M == 0) return 0;
  if (!inter || !w2 || !u2 || !perm || !counts || !y) return FFNK_ERR_NULL;
  if (M < 0 || M >= (1ll << 30) || bad_dim(d) || bad_dim(h)) return FFNK_ERR_SHAPE;
  if ((ldi & 7) || (ldy & 7) || ldi < h || ldy < d || (reinterpret_cast<uintptr_t>(y) & 15)) return FFNK_ERR_ALIGN;
  const int64_t rows = ffnk_route_capacity(M) + 512;
  AMaps tmA;
  CUtensorMap tmB[4];
  int r = make_tensor_map_2d(&tmA.m[RUN_LEVELS], inter, h, rows, ldi, BK, BM);
  if (r) return r;
  for (int i = 0; i <= COPY_MAP; ++i)
      if (i != RUN_LEVELS) tmA.m[i] = tmA.m[RUN_LEVELS];
  bool mn1 = false, mn2 = false;
  const bool k_major = weights_k_major(w_stride_k, w_stride_n, h);
  TileChoice tile = pick_tile(M, d, A_ROUTED, EPI_STORE, k_major);
  SplitKPlan pl;
  if (scratch && (reinterpret_cast<uintptr_t>(scratch) & 15) == 0) {
    pl = down_splitk_plan(M, d, h, k_major);
    if (pl.splits > 1 && ffn_down_scratch_bytes(M, d, h) <= scratch_bytes) tile = TileChoice{false, pl.bn};
    else pl = SplitKPlan{};
  }
  if ((r = weight_map(&tmB[0], WeightView{w2, w_stride_k, w_stride_n, h, d}, &mn1, tile.bn / 2))) return r;
  if ((r = weight_map(&tmB[2], WeightView{u2, w_stride_k, w_stride_n, h, d}, &mn2, tile.bn / 2))) return r;
  tmB[1] = tmB[0];
  tmB[3] = tmB[2];
  GemmParams p{perm, counts, static_cast<__nv_bfloat16*>(y), ldy, static_cast<int>(d), static_cast<int>(h),
               static_cast<int>(M), pick_group_m(h), max_run_rows(), status, g_prof_buffer};
  if (pl.splits > 1) {
    unsigned int* counters = nullptr;
    if ((r = splitk_counters(&counters))) return r;
    static unsigned launch_seq = 0;   // successive launches take successive rows of counters
    const unsigned slot = __atomic_fetch_add(&launch_seq, 1u, __ATOMIC_RELAXED) % kSplitKSlots;
    p.ksplit = pl.splits;
    p.kpart = static_cast<float*>(scratch);
    p.kcount = counters + static_cast<size_t>(slot) * kSplitKTiles;
  }
  if (early && !tile.pair) {
    const void* ws2[2] = {w2, u2};
    early_start(p, ws2, 2, d, h, w_stride_n, k_major);
  }
  return launch_gemm<A_ROUTED, EPI_STORE, OUT_SCATTER>(tmA, tmB, mn1, p, M, tile, static_cast<cudaStream_t>(stream));
}

extern "C" int ffnk_ffn_down(const void* inter, int64_t ldi, const void* w2, const void* u2, int64_t w_stride_k,
                             int64_t w_stride_n, const int32_t* perm, const int32_t* counts, void* y, int64_t ldy,
                             int64_t M, int64_t d, int64_t h, int32_t* status, void* stream) {
  return ffn_down_with_scratch(inter, ldi, w2, u2, w_stride_k, w_stride_n, perm, counts, y, ldy, M, d, h, nullptr, 0, 0,
                               status, stream);
}

extern "C" int ffnk_ffn_down_to_peers(const void* inter, int64_t ldi, const void* w2, const void* u2,
                                      int64_t w_stride_k, int64_t w_stride_n, const int32_t* perm,
                                      const int32_t* counts, void* const* peer_blocks, int world, int rank,
                                      int64_t rows_per_rank, int64_t ldb, int64_t M, int64_t d, int64_t h,
                                      int32_t* status, void* stream) {
  if (M == 0) return 0;
  if (!inter || !w2 || !u2 || !perm || !counts || !peer_blocks) return FFNK_ERR_NULL;
  if (M < 0 || M >= (1ll << 30) || bad_dim(d) || bad_dim(h)) return FFNK_ERR_SHAPE;
  if (world < 1 || world > MAX_PEERS || rank < 0 || rank >= world || rows_per_rank < 1 ||
      rows_per_rank * world < M || rows_per_rank * world >= (1ll << 30))
    return FFNK_ERR_SHAPE;
  if ((ldi & 7) || (ldb & 7) || ldi < h || ldb < d) return FFNK_ERR_ALIGN;
  for (int r = 0; r < world; ++r) {
    if (!peer_blocks[r]) return FFNK_ERR_NULL;
    if (reinterpret_cast<uintptr_t>(peer_blocks[r]) & 15) return FFNK_ERR_ALIGN;
  }
  const int64_t rows = ffnk_route_capacity(M) + 512;
  AMaps tmA;
  CUtensorMap tmB[4];
  int r = make_tensor_map_2d(&tmA.m[RUN_LEVELS], inter, h, rows, ldi, BK, BM);
  if (r) return r;
  for (int i = 0; i <= COPY_MAP; ++i)
    if (i != RUN_LEVELS) tmA.m[i] = tmA.m[RUN_LEVELS];
  bool mn1 = false, mn2 = false;
  const TileChoice tile = pick_tile(M, d, A_ROUTED, EPI_STORE, weights_k_major(w_stride_k, w_stride_n, h));
  if ((r = weight_map(&tmB[0], WeightView{w2, w_stride_k, w_stride_n, h, d}, &mn1, tile.bn / 2))) return r;
  if ((r = weight_map(&tmB[2], WeightView{u2, w_stride_k, w_stride_n, h, d}, &mn2, tile.bn / 2))) return r;
  tmB[1] = tmB[0];
  tmB[3] = tmB[2];
  GemmParams p{perm, counts, nullptr, ldb, static_cast<int>(d), static_cast<int>(h),
               static_cast<int>(M), pick_group_m(h), max_run_rows(), status, g_prof_buffer};
  for (int i = 0; i < world; ++i) p.peer_out[i] = static_cast<__nv_bfloat16*>(peer_blocks[i]);
  p.peer_world = world;
  p.peer_rank = rank;
  p.peer_rows = static_cast<int>(rows_per_rank);
  return launch_gemm<A_ROUTED, EPI_STORE, OUT_PEER>(tmA, tmB, mn1, p, M, tile, static_cast<cudaStream_t>(stream));
}

// parts: 1 = the routed-order copies of g and a, 2 = the weight gradients, 4 = dx; ffnk_linear_bwd runs
// copies, dx, weight gradients.  A data-parallel caller runs 1|2 first, starts the all-reduce of the weight
// gradients on another stream, and then runs 4 beside it.
extern "C" int ffnk_linear_bwd_parts(const void* g, int64_t ldg, const void* a, int64_t lda, const void* b1,
                                     const void* b2, int64_t b_stride_k, int64_t b_stride_n, const int32_t* perm,
                                     const int32_t* counts, void* da, int64_t ldda, void* db1, void* db2, void* g_copy,
                                     void* a_copy, int64_t M, int64_t N, int64_t K, int parts, int32_t* status,
                                     void* stream) {
  if (parts < 1 || parts > 7) return FFNK_ERR_SHAPE;
  if (!db1 || !db2) return FFNK_ERR_NULL;
  if (bad_dim(N) || bad_dim(K) || M < 0 || M >= (1ll << 30)) return FFNK_ERR_SHAPE;
  const bool k_major = (b_stride_k == 1 && b_stride_n >= K);   // storage [N, K]
  const bool n_major = (b_stride_n == 1 && b_stride_k >= N);   // storage [K, N]
  if (!k_major && !n_major) return FFNK_ERR_LAYOUT;
  if ((reinterpret_cast<uintptr_t>(db1) & 15) || (reinterpret_cast<uintptr_t>(db2) & 15)) return FFNK_ERR_ALIGN;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (M == 0) {
    // no tokens: both weight gradients are zero (strided fill, row by row of the storage)
    const int64_t rows = k_major ? N : K, cols = k_major ? K : N, ld = k_major ? b_stride_n : b_stride_k;
    cudaError_t e = cudaMemset2DAsync(db1, ld * 2, 0, cols * 2, rows, s);
    if (e == cudaSuccess) e = cudaMemset2DAsync(db2, ld * 2, 0, cols * 2, rows, s);
    return cuda_status(e);
  }
  // a may be null when a_copy already holds it in routed order (left there by the forward pass)
  const bool a_prepared = !a && g_copy && a_copy;
  if (!g || (!a && !a_prepared) || !b1 || !b2 || !perm || !counts || !da) return FFNK_ERR_NULL;
  if ((ldg & 7) || (ldda & 7) || ldg < N || ldda < K || (a && ((lda & 7) || lda < K)) ||
      (reinterpret_cast<uintptr_t>(da) & 15))
    return FFNK_ERR_ALIGN;
  const DeviceInfo& dev = device_info();
  if (dev.cc_major != 10) return FFNK_ERR_DEVICE;

  // With scratch for routed-order copies of g and a, every GEMM below reads whole tiles of consecutive
  // rows: dx is then the down-projection kernel of the FFN (routed A, rows scattered back to token
  // order) and the weight gradients run on CTA pairs.  The two copies cost 4 * M * (N + K) bytes of
  // traffic and pay for themselves for every mask (identity routing at M=32768, K=N=4096:
  // 958 -> 1078 TFLOP/s even with the single-CTA weight-gradient kernel).  Without scratch the
  // kernels gather token rows themselves.
  const bool copies = g_copy && a_copy;
  const int64_t copy_rows = ffnk_route_capacity(M) + 512;
  if (copies && ((reinterpret_cast<uintptr_t>(g_copy) | reinterpret_cast<uintptr_t>(a_copy)) & 15)) return FFNK_ERR_ALIGN;
  if (copies && (parts & 1)) {
    int r;
    if ((r = permute_rows_launch(g, ldg, perm, counts, g_copy, N, M, N, 0, stream))) return r;
    if (a && (r = permute_rows_launch(a, lda, perm, counts, a_copy, K, M, K, 0, stream))) return r;
  }
  // dx: the forward kernel on g with the weights seen as [N, K] (contraction over N)
  if (parts & 4) {
    AMaps tmA;
    CUtensorMap tmB[4];
    int r;
    if (copies) {
      if ((r = make_tensor_map_2d(&tmA.m[RUN_LEVELS], g_copy, N, copy_rows, N, BK, BM))) return r;
      for (int i = 0; i <= COPY_MAP; ++i)
        if (i != RUN_LEVELS) tmA.m[i] = tmA.m[RUN_LEVELS];
    } else if ((r = gather_maps(tmA, g, N, M, ldg))) {
      return r;
    }
    bool mn1 = false, mn2 = false;
    const TileChoice tile = pick_tile(M, K, copies ? A_ROUTED : A_GATHER, EPI_STORE,
                                      weights_k_major(b_stride_n, b_stride_k, N));
    if ((r = weight_map(&tmB[0], WeightView{b1, b_stride_n, b_stride_k, N, K}, &mn1, tile.bn / 2))) return r;
    if ((r = weight_map(&tmB[2], WeightView{b2, b_stride_n, b_stride_k, N, K}, &mn2, tile.bn / 2))) return r;
    tmB[1] = tmB[0];
    tmB[3] = tmB[2];
    GemmParams p{perm, counts, static_cast<__nv_bfloat16*>(da), ldda, static_cast<int>(K), static_cast<int>(N),
                 static_cast<int>(M), pick_group_m(N), max_run_rows(), status, g_prof_buffer};
    r = copies ? launch_gemm<A_ROUTED, EPI_STORE, OUT_SCATTER>(tmA, tmB, mn1, p, M, tile, s)
               : launch_gemm<A_GATHER, EPI_STORE, OUT_SCATTER>(tmA, tmB, mn1, p, M, tile, s);
    if (r) return r;
  }
  // dW: output in the weight's storage order; P supplies the storage rows, Q the storage columns
  if (parts & 2) {
    const void* gg = copies ? g_copy : g;
    const void* aa = copies ? a_copy : a;
    const int64_t lg = copies ? N : ldg, la = copies ? K : lda;
    const void* P = k_major ? gg : aa;
    const void* Q = k_major ? aa : gg;
    const int64_t ldp = k_major ? lg : la, ldq = k_major ? la : lg;
    const int64_t p_dim = k_major ? N : K, q_dim = k_major ? K : N;
    return launch_wgrad(P, ldp, p_dim, Q, ldq, q_dim, copies ? copy_rows : M, db1, db2,
                        k_major ? b_stride_n : b_stride_k, copies ? 1 : 0, perm, counts, status, s);
  }
  return 0;
}

extern "C" int ffnk_linear_bwd(const void* g, int64_t ldg, const void* a, int64_t lda, const void* b1, const void* b2,
                               int64_t b_stride_k, int64_t b_stride_n, const int32_t* perm, const int32_t* counts,
                               void* da, int64_t ldda, void* db1, void* db2, void* g_copy, void* a_copy, int64_t M,
                               int64_t N, int64_t K, int32_t* status, void* stream) {
  return ffnk_linear_bwd_parts(g, ldg, a, lda, b1, b2, b_stride_k, b_stride_n, perm, counts, da, ldda, db1, db2, g_copy,
                               a_copy, M, N, K, 7, status, stream);
}

// -------------------------------------------------------------------------------------------
// MaskedFFN with a backward pass.  The reference stops at a forward kernel that would save the
// pre-activations (_masked_ffn_fwd, ffn_kernel/ffn.py:116-221, never launched) and backward
// kernels that do not compile (ffn_kernel/ffn.py:224-524); MaskedFFN.backward raises
// (ffn_kernel/ops.py:34-38).  The formulas are the reference's (README.md:159-172).
//
// Everything between the first and the last GEMM lives in routed order:
//   forward : xr = permute(x);  (t1, t3, hid) = gate/up(xr);  y[token] = hid @ W2
//   backward: gr = permute(dy); (dt1, dt3) = dswiglu(gr @ W2^T; t1, t3)
//             dW2 = gr^T hid | hid^T gr;  dW1 = dt1^T xr;  dW3 = dt3^T xr   (per modality, in storage order)
//             dx[token] = dt1 @ W1^T + dt3 @ W3^T                          (one GEMM, two contraction segments)
// -------------------------------------------------------------------------------------------
extern "C" int ffnk_ffn_forward_train(const void* x, int64_t ldx, const void* w1, const void* w2, const void* w3,
                                      const void* u1, const void* u2, const void* u3, int64_t w13_stride_k,
                                      int64_t w13_stride_n, int64_t w2_stride_k, int64_t w2_stride_n,
                                      const void* mask, int32_t* perm, int32_t* counts, void* scan_workspace, void* xr,
                                      void* t1, void* t3, void* hid, void* y, int64_t ldy, int64_t M, int64_t d,
                                      int64_t h, int32_t* status, void* stream) {
  if (M == 0) return 0;
  if (!x || !w1 || !w2 || !w3 || !u1 || !u2 || !u3 || !mask || !perm || !counts || !scan_workspace || !xr || !t1 ||
      !t3 || !hid || !y)
    return FFNK_ERR_NULL;
  if (M < 0 || M >= (1ll << 30) || bad_dim(d) || bad_dim(h)) return FFNK_ERR_SHAPE;
  if ((ldx & 7) || (ldy & 7) || ldx < d || ldy < d) return FFNK_ERR_ALIGN;
  const void* al[] = {xr, t1, t3, hid, y};
  for (const void* q : al)
    if (reinterpret_cast<uintptr_t>(q) & 15) return FFNK_ERR_ALIGN;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int r;
  if (M <= ffnk_route_permute_max_tokens()) {
    // a mask of one routing tile: routing and the row copy are one launch
    if ((r = ffnk_route_permute_rows(mask, M, x, ldx, d, perm, counts, xr, d, stream))) return r;
  } else {
    if ((r = ffnk_route(mask, M, perm, counts, scan_workspace, status, stream))) return r;
    if ((r = ffnk_permute_rows(x, ldx, perm, counts, xr, d, M, d, stream))) return r;
  }
  const int64_t rows = ffnk_route_capacity(M) + 512;
  {
    AMaps tmA;
    CUtensorMap tmB[4];
    if ((r = make_tensor_map_2d(&tmA.m[RUN_LEVELS], xr, d, rows, d, BK, BM))) return r;
    for (int i = 0; i <= COPY_MAP; ++i)
      if (i != RUN_LEVELS) tmA.m[i] = tmA.m[RUN_LEVELS];
    bool mn = false, mn_i = false;
    const void* ws[4] = {w1, w3, u1, u3};
    const TileChoice tile = pick_tile(M, h, A_ROUTED, EPI_SWIGLU_SAVE, weights_k_major(w13_stride_k, w13_stride_n, d), d);
    for (int i = 0; i < 4; ++i) {
      if ((r = weight_map(&tmB[i], WeightView{ws[i], w13_stride_k, w13_stride_n, d, h}, &mn_i, tile.bn / 2))) return r;
      mn = mn_i;
    }
    GemmParams p{perm, counts, static_cast<__nv_bfloat16*>(hid), h, static_cast<int>(h), static_cast<int>(d),
                 static_cast<int>(rows), pick_group_m(d), max_run_rows(), status, g_prof_buffer};
    p.aux0 = static_cast<__nv_bfloat16*>(t1);
    p.aux1 = static_cast<__nv_bfloat16*>(t3);
    if ((r = launch_gemm<A_ROUTED, EPI_SWIGLU_SAVE, OUT_ROUTED>(tmA, tmB, mn, p, M, tile, s))) return r;
  }
  return ffnk_ffn_down(hid, h, w2, u2, w2_stride_k, w2_stride_n, perm, counts, y, ldy, M, d, h, status, stream);
}

extern "C" int ffnk_ffn_backward(const void* gy, int64_t ldg, const void* xr, const void* t1, const void* t3,
                                 const void* hid, const void* w1, const void* w2, const void* w3, const void* u1,
                                 const void* u2, const void* u3, int64_t w13_stride_k, int64_t w13_stride_n,
                                 int64_t w2_stride_k, int64_t w2_stride_n, const int32_t* perm, const int32_t* counts,
                                 void* gr, void* dt1, void* dt3, void* dx, int64_t lddx, void* dw1, void* dw2,
                                 void* dw3, void* du1, void* du2, void* du3, int64_t M, int64_t d, int64_t h,
                                 int32_t* status, void* stream) {
  if (M == 0) return 0;
  if (!gy || !xr || !t1 || !t3 || !hid || !w1 || !w2 || !w3 || !u1 || !u2 || !u3 || !perm || !counts || !gr || !dt1 ||
      !dt3 || !dx || !dw1 || !dw2 || !dw3 || !du1 || !du2 || !du3)
    return FFNK_ERR_NULL;
  if (M < 0 || M >= (1ll << 30) || bad_dim(d) || bad_dim(h)) return FFNK_ERR_SHAPE;
  if ((ldg & 7) || (lddx & 7) || ldg < d || lddx < d) return FFNK_ERR_ALIGN;
  const bool w13_k = weights_k_major(w13_stride_k, w13_stride_n, d);
  const bool w13_n = w13_stride_n == 1 && w13_stride_k >= h;
  const bool w2_k = weights_k_major(w2_stride_k, w2_stride_n, h);
  const bool w2_n = w2_stride_n == 1 && w2_stride_k >= d;
  if ((!w13_k && !w13_n) || (!w2_k && !w2_n)) return FFNK_ERR_LAYOUT;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int64_t rows = ffnk_route_capacity(M) + 512;
  int r = ffnk_permute_rows(gy, ldg, perm, counts, gr, d, M, d, stream);
  if (r) return r;

  // (dt1, dt3) = dswiglu(gr @ W2^T): contraction over d, output columns over h
  {
    AMaps tmA;
    CUtensorMap tmB[4];
    if ((r = make_tensor_map_2d(&tmA.m[RUN_LEVELS], gr, d, rows, d, BK, BM))) return r;
    for (int i = 0; i <= COPY_MAP; ++i)
      if (i != RUN_LEVELS) tmA.m[i] = tmA.m[RUN_LEVELS];
    bool mn1 = false, mn2 = false;
    const TileChoice tile = pick_tile(M, h, A_ROUTED, EPI_DSWIGLU, weights_k_major(w2_stride_n, w2_stride_k, d));
    if ((r = weight_map(&tmB[0], WeightView{w2, w2_stride_n, w2_stride_k, d, h}, &mn1, tile.bn / 2))) return r;
    if ((r = weight_map(&tmB[2], WeightView{u2, w2_stride_n, w2_stride_k, d, h}, &mn2, tile.bn / 2))) return r;
    tmB[1] = tmB[0];
    tmB[3] = tmB[2];
    GemmParams p{perm, counts, static_cast<__nv_bfloat16*>(dt1), h, static_cast<int>(h), static_cast<int>(d),
                 static_cast<int>(rows), pick_group_m(d), max_run_rows(), status, g_prof_buffer};
    p.aux0 = static_cast<__nv_bfloat16*>(const_cast<void*>(t1));
    p.aux1 = static_cast<__nv_bfloat16*>(const_cast<void*>(t3));
    p.aux2 = static_cast<__nv_bfloat16*>(dt3);
    if ((r = launch_gemm<A_ROUTED, EPI_DSWIGLU, OUT_ROUTED>(tmA, tmB, mn1, p, M, tile, s))) return r;
  }
  // weight gradients, written in each weight's storage order
  if (w2_k) r = launch_wgrad(gr, d, d, hid, h, h, rows, dw2, du2, w2_stride_n, 1, perm, counts, status, s);   // [d][h]
  else r = launch_wgrad(hid, h, h, gr, d, d, rows, dw2, du2, w2_stride_k, 1, perm, counts, status, s);       // [h][d]
  if (r) return r;
  if (w13_k) {                                                                                              // [h][d]
    if ((r = launch_wgrad(dt1, h, h, xr, d, d, rows, dw1, du1, w13_stride_n, 1, perm, counts, status, s))) return r;
    if ((r = launch_wgrad(dt3, h, h, xr, d, d, rows, dw3, du3, w13_stride_n, 1, perm, counts, status, s))) return r;
  } else {                                                                                                  // [d][h]
    if ((r = launch_wgrad(xr, d, d, dt1, h, h, rows, dw1, du1, w13_stride_k, 1, perm, counts, status, s))) return r;
    if ((r = launch_wgrad(xr, d, d, dt3, h, h, rows, dw3, du3, w13_stride_k, 1, perm, counts, status, s))) return r;
  }
  // dx[token] = dt1 @ W1^T + dt3 @ W3^T: two contraction segments of length h into one accumulator
  {
    AMaps tmA;
    CUtensorMap tmB[4];
    if ((r = make_tensor_map_2d(&tmA.m[RUN_LEVELS], dt1, h, rows, h, BK, BM))) return r;
    for (int i = 0; i <= COPY_MAP; ++i)
      if (i != RUN_LEVELS) tmA.m[i] = tmA.m[RUN_LEVELS];
    if ((r = make_tensor_map_2d(&tmA.m[RUN_LEVELS - 1], dt3, h, rows, h, BK, BM))) return r;
    bool mn = false, mn_i = false;
    const void* ws[4] = {w1, w3, u1, u3};
    const TileChoice tile = pick_tile(M, d, A_ROUTED, EPI_STORE, weights_k_major(w13_stride_n, w13_stride_k, h));
    for (int i = 0; i < 4; ++i) {
      if ((r = weight_map(&tmB[i], WeightView{ws[i], w13_stride_n, w13_stride_k, h, d}, &mn_i, tile.bn / 2))) return r;
      mn = mn_i;
    }
    GemmParams p{perm, counts, static_cast<__nv_bfloat16*>(dx), lddx, static_cast<int>(d), static_cast<int>(h),
                 static_cast<int>(rows), pick_group_m(2 * h), max_run_rows(), status, g_prof_buffer};
    p.k_len1 = static_cast<int>(h);
    return launch_gemm<A_ROUTED, EPI_STORE, OUT_SCATTER>(tmA, tmB, mn, p, M, tile, s);
  }
}

extern "C" int ffnk_debug_profile_buffer(void* buffer) {
  g_prof_buffer = static_cast<long long*>(buffer);
  return 0;
}

extern "C" int ffnk_set_sm_margin(int sms) {
  if (sms < 0 || sms > 128) return FFNK_ERR_SHAPE;
  g_sm_margin = sms;
  return 0;
}
