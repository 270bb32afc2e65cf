// Host utilities of libffnk: device query, tensor-map construction, status word access,
// and the bounded-wait self test.
#include <cstdio>
#include <cstring>
#include <mutex>

#include "ffnk_internal.h"
#include "ptx.cuh"

namespace ffnk {

const DeviceInfo& device_info() {
  static DeviceInfo info[64];
  static std::mutex mu;
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  std::lock_guard<std::mutex> lock(mu);
  DeviceInfo& d = info[dev];
  if (d.sm_count == 0) {
    cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, dev);
    cudaDeviceGetAttribute(&d.cc_major, cudaDevAttrComputeCapabilityMajor, dev);
    cudaDeviceGetAttribute(&d.smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
  }
  return d;
}

TuneOverrides& tune_overrides() {
  static TuneOverrides t;
  return t;
}

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

int make_tensor_map_2d(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer, uint64_t row_stride,
                       uint32_t box_inner, uint32_t box_outer) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return FFNK_ERR_DRIVER;
  // The encoder is a driver-API call and needs the device's primary context current on the
  // calling thread; a thread that has only made query calls so far (autograd's backward
  // thread, for one) may not have it bound yet.  cudaFree(0) binds it.
  {
    thread_local int bound_device = -1;
    int dev = -1;
    cudaGetDevice(&dev);
    if (dev != bound_device) {
      cudaFree(0);
      bound_device = dev;
    }
  }
  if ((reinterpret_cast<uintptr_t>(base) & 15) || ((row_stride * 2) & 15)) return FFNK_ERR_ALIGN;
  if (inner == 0 || outer == 0) return FFNK_ERR_SHAPE;
  const cuuint64_t dims[2] = {inner, outer};
  const cuuint64_t strides[1] = {row_stride * 2};
  const cuuint32_t box[2] = {box_inner, box_outer};
  const cuuint32_t elem[2] = {1, 1};
  const CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS && tune_overrides().verbose > 0)
    fprintf(stderr, "ffnk: cuTensorMapEncodeTiled failed (CUresult %d): base %p dims {%llu, %llu} row stride %llu B box {%u, %u}\n",
            static_cast<int>(r), base, static_cast<unsigned long long>(inner), static_cast<unsigned long long>(outer),
            static_cast<unsigned long long>(row_stride * 2), box_inner, box_outer);
  return r == CUDA_SUCCESS ? 0 : FFNK_ERR_TENSORMAP;
}

// One CTA, one barrier that nobody arrives on.  The wait must return false after the budget,
// the status word must say so, and the kernel must exit normally.
__global__ void selftest_wait_kernel(int* status, uint64_t budget_ns) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(&bar, 1);
    fence_mbar_init();
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const bool ok = mbar_wait(&bar, 0, &abort_flag, budget_ns);
    if (!ok) atomicCAS(status, 0, ST_TIMEOUT_TEST);
  }
  __syncthreads();
}

}  // namespace ffnk

using namespace ffnk;

extern "C" int ffnk_version(void) { return 100; }

extern "C" int ffnk_read_status(int32_t* status, int clear, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (!status) return FFNK_ERR_NULL;
  int32_t host = 0;
  cudaError_t e = cudaMemcpyAsync(&host, status, sizeof(host), cudaMemcpyDeviceToHost, stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
  if (e != cudaSuccess) return cuda_status(e);
  if (clear && host != 0) {
    e = cudaMemsetAsync(status, 0, sizeof(host), stream);
    if (e != cudaSuccess) return cuda_status(e);
  }
  return host;
}

extern "C" int ffnk_selftest_bounded_wait(int32_t* status, int64_t budget_us, void* stream_) {
  if (!status) return FFNK_ERR_NULL;
  if (budget_us < 1 || budget_us > 2000000) return FFNK_ERR_SHAPE;
  selftest_wait_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream_)>>>(status, static_cast<uint64_t>(budget_us) * 1000);
  return cuda_status(cudaGetLastError());
}

extern "C" int ffnk_tune_override(const char* name, int value) {
  if (!name) return FFNK_ERR_NULL;
  TuneOverrides& t = tune_overrides();
  struct { const char* n; int* v; } table[] = {
      {"pair", &t.pair}, {"narrow", &t.narrow}, {"permute", &t.permute}, {"epi_warps", &t.epi_warps},
      {"group_m", &t.group_m}, {"wgrad_pair", &t.wgrad_pair}, {"max_run_rows", &t.max_run_rows},
      {"copy_threshold", &t.copy_threshold}, {"verbose", &t.verbose}, {"route_resident", &t.route_resident},
      {"ksplit", &t.ksplit}, {"early_start", &t.early_start}};
  for (auto& e : table)
    if (strcmp(e.n, name) == 0) {
      *e.v = value;
      return 0;
    }
  return FFNK_ERR_SHAPE;
}

extern "C" const char* ffnk_status_string(int code) {
  switch (code) {
    case 0: return "ok";
    case FFNK_ERR_NULL: return "null pointer argument";
    case FFNK_ERR_SHAPE: return "unsupported size (negative, too large, or not a multiple of 8)";
    case FFNK_ERR_ALIGN: return "pointer or row stride not 16-byte aligned";
    case FFNK_ERR_LAYOUT: return "weight must have stride_k == 1 or stride_n == 1";
    case FFNK_ERR_DRIVER: return "cuTensorMapEncodeTiled driver entry point unavailable";
    case FFNK_ERR_TENSORMAP: return "tensor map rejected by the driver";
    case FFNK_ERR_DEVICE: return "device is not compute capability 10.x";
    case FFNK_ERR_CAPACITY: return "problem exceeds the fixed capacity of the no-allocation entry point";
    case FFNK_ERR_CAPTURE: return "first call on this device must be made outside stream capture";
    case ST_TIMEOUT_PRODUCER: return "device: TMA producer wait expired";
    case ST_TIMEOUT_MMA_FULL: return "device: MMA wait for operands expired";
    case ST_TIMEOUT_MMA_TMEM: return "device: MMA wait for accumulator expired";
    case ST_TIMEOUT_EPILOGUE: return "device: epilogue wait expired";
    case ST_TIMEOUT_SCAN: return "device: routing scan look-back expired";
    case ST_TIMEOUT_TEST: return "device: self-test wait expired (expected)";
    case ST_TIMEOUT_PEER: return "device: wait on partner CTA expired";
    case ST_TIMEOUT_RANK: return "device: barrier wait for another rank expired";
    case ST_TIMEOUT_GRID: return "device: grid-wide wait of the small-M forward expired";
    default: return code <= -1000 ? "CUDA runtime error, code = -(1000 + cudaError_t)" : "unknown code";
  }
}
