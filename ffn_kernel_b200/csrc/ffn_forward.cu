// The whole MaskedFFN forward behind one C call: routing scan, optional row permutation, gate/up
// GEMM with the SwiGLU epilogue, down projection with the scatter epilogue -- or the
// weight-streaming decode pair for a handful of tokens.  Same contract as MaskedFFN.forward
// (ffn_kernel/ops.py:28-32).  One call keeps the host cost of a forward pass at a few
// microseconds, which is what matters when the kernels themselves take ten.
#include "ffnk_internal.h"

namespace ffnk {

static int64_t align256(int64_t v) { return (v + 255) & ~int64_t(255); }

// Tile-table entry: copy x into routed order before the gate/up GEMM?  The copy moves 4*M*d bytes
// through HBM (measured 5.6-5.9 TB/s); gathering inside the GEMM costs 10-15 % of the GEMM on span
// masks and 3x on i.i.d. masks, because row tiles that straddle run boundaries need many TMA
// instructions per k-step.  The copy costs about 0.73 ps per element of x, the gather about a fifth
// of a GEMM that takes 2.9 fs per element of x and unit of h: break-even near h = 1280 (measured at
// M=16384, d=4096, h=1376: forward 0.499 ms gathering, 0.466 ms copying first).
static bool permute_first(int64_t M, int64_t d, int64_t h) {
  (void)d;
  const int forced = tune_overrides().permute;
  if (forced >= 0) return forced != 0;
  return M < 2048 || h >= 1280;
}

struct FfnWorkspace {
  int64_t perm, counts, scan, xr, inter, kpart, kpart_bytes, total;
};

static FfnWorkspace ffn_workspace(int64_t M, int64_t d, int64_t h) {
  FfnWorkspace w{};
  const int64_t cap = ffnk_route_capacity(M);
  int64_t off = 0;
  w.perm = off;
  off += align256(2 * cap * 4 + 16);
  w.counts = off;
  off += 256;
  w.scan = off;
  off += align256(ffnk_route_workspace_bytes(M));
  w.xr = off;
  if (permute_first(M, d, h)) off += align256((cap + 512) * d * 2);
  w.inter = off;
  off += align256((cap + 512) * h * 2);
  w.kpart = off;
  w.kpart_bytes = ffn_down_scratch_bytes(M, d, h);     // partial tiles of a split-K down projection (few row tiles)
  off += align256(w.kpart_bytes);
  w.total = off;
  return w;
}

}  // namespace ffnk

using namespace ffnk;

extern "C" int ffnk_ffn_permute_first(int64_t M, int64_t d, int64_t h) { return permute_first(M, d, h) ? 1 : 0; }

extern "C" int64_t ffnk_ffn_workspace_bytes(int64_t M, int64_t d, int64_t h) {
  if (M <= 0 || d <= 0 || h <= 0) return 256;
  return ffn_workspace(M, d, h).total;
}

extern "C" int ffnk_ffn_forward(const void* x, int64_t ldx, const void* w1, const void* w2, const void* w3,
                                const void* u1, const void* u2, const void* u3, int64_t w13_stride_k,
                                int64_t w13_stride_n, int64_t w2_stride_k, int64_t w2_stride_n, const void* mask,
                                void* workspace, int64_t workspace_bytes, void* y, int64_t ldy, int64_t M, int64_t d,
                                int64_t h, int allow_decode, int32_t* status, void* stream) {
  if (M == 0) return 0;
  if (!x || !w1 || !w2 || !w3 || !u1 || !u2 || !u3 || !mask || !workspace || !y || !status) return FFNK_ERR_NULL;
  if (M < 0 || M >= (1ll << 30) || d < 8 || h < 8 || (d & 7) || (h & 7)) return FFNK_ERR_SHAPE;
  if (reinterpret_cast<uintptr_t>(workspace) & 255) return FFNK_ERR_ALIGN;
  const FfnWorkspace w = ffn_workspace(M, d, h);
  if (workspace_bytes < w.total) return FFNK_ERR_CAPACITY;
  char* ws = static_cast<char*>(workspace);

  const bool k_major = w13_stride_k == 1 && w2_stride_k == 1;
  if (allow_decode && k_major && ffnk_ffn_takes_decode(M, d, h))
    return ffnk_ffn_decode(x, ldx, w1, w2, w3, u1, u2, u3, w13_stride_k, w13_stride_n, w2_stride_k, w2_stride_n, mask,
                           ws + w.inter, y, ldy, M, d, h, status, stream);

  int32_t* perm = reinterpret_cast<int32_t*>(ws + w.perm);
  int32_t* counts = reinterpret_cast<int32_t*>(ws + w.counts);
  int r;
  const void* a = x;
  int64_t lda = ldx;
  int routed_in = 0;
  if (permute_first(M, d, h)) {
    // a mask of a single routing tile is routed by the kernel that copies the rows: one launch fewer
    if (M <= ffnk_route_permute_max_tokens()) {
      if ((r = ffnk_route_permute_rows(mask, M, x, ldx, d, perm, counts, ws + w.xr, d, stream))) return r;
    } else {
      if ((r = ffnk_route(mask, M, perm, counts, ws + w.scan, status, stream))) return r;
      if ((r = ffnk_permute_rows(x, ldx, perm, counts, ws + w.xr, d, M, d, stream))) return r;
    }
    a = ws + w.xr;
    lda = d;
    routed_in = 1;
  } else if ((r = ffnk_route(mask, M, perm, counts, ws + w.scan, status, stream))) {
    return r;
  }
  // Few row tiles leave most SMs idle: the two GEMMs are launched so that each may set itself up and ask its
  // weights into L2 while its predecessor still runs (programmatic dependent launch; single-CTA tiles only).
  const int early = M < 4096 && tune_overrides().early_start != 0 ? 1 : 0;
  if ((r = ffn_gateup_early(a, lda, w1, w3, u1, u3, w13_stride_k, w13_stride_n, perm, counts, ws + w.inter, h, routed_in,
                            1, M, d, h, early, status, stream)))
    return r;
  return ffn_down_with_scratch(ws + w.inter, h, w2, u2, w2_stride_k, w2_stride_n, perm, counts, y, ldy, M, d, h,
                               w.kpart_bytes ? ws + w.kpart : nullptr, w.kpart_bytes, early, status, stream);
}
