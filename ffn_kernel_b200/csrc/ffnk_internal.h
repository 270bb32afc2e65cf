// Host-side helpers shared by the translation units of libffnk: error mapping, TMA tensor-map
// construction through the driver entry point (no link-time dependency on libcuda).
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/ffnk.h"

namespace ffnk {

// CUDA runtime errors are reported as -(1000 + cudaError_t) so that they cannot be confused with
// argument errors (small negatives) or device status codes (small positives).
inline int cuda_status(cudaError_t e) { return e == cudaSuccess ? 0 : -(1000 + static_cast<int>(e)); }

// Number of SMs / compute capability of the current device (cached per device).
struct DeviceInfo {
  int sm_count = 0;
  int cc_major = 0;
  int smem_optin = 0;
};
const DeviceInfo& device_info();

// 2-D bf16 tensor map with 128-byte swizzle.
//   inner/outer : extents in elements (inner is contiguous)
//   row_stride  : elements between consecutive outer indices
//   box_inner/box_outer : tile extents; box_inner * 2 bytes must be 128
// Returns 0 or FFNK_ERR_*.
int make_tensor_map_2d(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer, uint64_t row_stride,
                       uint32_t box_inner, uint32_t box_outer);

// Overrides of single tile-table entries, for measuring a choice against its alternatives
// (ffnk_tune_override; `python -m ffn_kernel_b200.tune`).  -1 = the table decides.  The library reads
// no environment variables: whoever wants an override sets it through the C ABI.
struct TuneOverrides {
  int pair = -1;            // 0/1: CTA pairs never / wherever the kernel variant exists
  int narrow = -1;          // 0: 256-column tiles only, 1: 64-column, 2: 128-column tiles
  int permute = -1;         // 0/1: FFN forward gathers rows in the gate/up GEMM / copies x to routed order first
  int epi_warps = -1;       // 4 or 8 epilogue warps
  int group_m = -1;         // row tiles per super-tile
  int wgrad_pair = -1;      // 0/1: weight gradients on single CTAs / CTA pairs
  int max_run_rows = -1;    // largest tiled TMA box for runs of consecutive tokens (0: gather4 only)
  int copy_threshold = -1;  // average run length below which MaskedLinear forward copies a to routed order
  int verbose = -1;         // 1: print the arguments of a tensor map the driver rejects
  int route_resident = -1;  // 0: long masks never take the one-launch resident routing kernel (count + scatter instead)
  int ksplit = -1;          // down projection of the FFN forward: 0/1 never split K, n > 1 split n ways wherever it can
  int early_start = -1;     // 0: the GEMMs of the single-call FFN forward never start beside their predecessor
};
TuneOverrides& tune_overrides();

// Diagnostics buffer installed by ffnk_debug_profile_buffer (null when off): 8 int64 per CTA.
long long* debug_profile_buffer();

// ffnk_ffn_down with an optional scratch buffer (16-byte aligned) for the fp32 partial tiles of its split-K
// variant, which it takes for few row tiles when ffn_down_scratch_bytes(M, d, h) > 0 bytes are given.
int64_t ffn_down_scratch_bytes(int64_t M, int64_t d, int64_t h);
// early != 0 (single-CTA tiles only): the kernel is launched so that it may start beside its predecessor in
// the stream (programmatic dependent launch) and ask its weights into L2 until the predecessor has finished.
int ffn_down_with_scratch(const void* inter, int64_t ldi, const void* w2, const void* u2, int64_t w_stride_k,
                          int64_t w_stride_n, const int32_t* perm, const int32_t* counts, void* y, int64_t ldy, int64_t M,
                          int64_t d, int64_t h, void* scratch, int64_t scratch_bytes, int early, int32_t* status,
                          void* stream);
int ffn_gateup_early(const void* x, int64_t ldx, const void* w1, const void* w3, const void* u1, const void* u3,
                     int64_t w_stride_k, int64_t w_stride_n, const int32_t* perm, const int32_t* counts, void* out,
                     int64_t ldo, int routed_in, int routed_out, int64_t M, int64_t d, int64_t h, int early,
                     int32_t* status, void* stream);

// permute_rows with an optional device-side gate: with only_if_scattered = T > 0 the kernel returns at
// once unless the mask's runs of same-modality tokens average fewer than T rows.
int permute_rows_launch(const void* x, int64_t ldx, const int32_t* perm, const int32_t* counts, void* out, int64_t ldo,
                        int64_t M, int64_t d, int only_if_scattered, void* stream);

}  // namespace ffnk
