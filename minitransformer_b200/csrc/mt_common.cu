// Host-side plumbing shared by every entry point: thread-local error text, the device
// status word, tensor-map construction through the driver entry point.
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include <cstdlib>
#include "mt_common.cuh"
#include "../../include/mt_b200_test.h"

namespace mt {

static thread_local char g_error[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
  return code;
}

// One status word per device that loads the library.
__device__ int g_device_status = 0;

static int g_launch_overlap = 1;

bool pdl_enabled() {
#ifdef MT_TIMING_KNOBS
  static int on = -1;
  if (on < 0) { const char* e = getenv("MT_PDL"); on = e ? atoi(e) : 1; }
  if (!on) return false;
#endif
  return g_launch_overlap != 0;
}

int set_launch_overlap(int enabled) {
  const int before = g_launch_overlap;
  g_launch_overlap = enabled ? 1 : 0;
  return before;
}

int* device_status_ptr() {
  static thread_local int cached_dev = -1;
  static thread_local int* cached_ptr = nullptr;
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess) return nullptr;
  if (dev == cached_dev && cached_ptr) return cached_ptr;
  void* p = nullptr;
  if (cudaGetSymbolAddress(&p, g_device_status) != cudaSuccess) return nullptr;
  cached_dev = dev;
  cached_ptr = static_cast<int*>(p);
  return cached_ptr;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn) return fn;
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
      q != cudaDriverEntryPointSuccess)
    return nullptr;
  fn = reinterpret_cast<EncodeTiledFn>(p);
  return fn;
}

int make_tensor_map_2d(CUtensorMap* map, CUtensorMapDataType dtype, int elem_bytes, const void* base,
                       uint64_t inner, uint64_t outer, uint64_t outer_stride_bytes, uint32_t box_inner,
                       uint32_t box_outer, CUtensorMapSwizzle swizzle) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return fail(MT_ERR_CUDA, "cuTensorMapEncodeTiled entry point not available");
  if (!aligned16(base) || (outer_stride_bytes & 15))
    return fail(MT_ERR_INVALID_ARG, "tensor map needs a 16-byte aligned base (%p) and row stride (%llu)", base,
                (unsigned long long)outer_stride_bytes);
  (void)elem_bytes;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {outer_stride_bytes};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, dtype, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(MT_ERR_CUDA, "cuTensorMapEncodeTiled failed (%d) dims=(%llu,%llu) stride=%llu box=(%u,%u)", (int)r,
                (unsigned long long)inner, (unsigned long long)outer, (unsigned long long)outer_stride_bytes,
                box_inner, box_outer);
  return MT_OK;
}

// One thread waits on a barrier that nothing signals; the bounded wait gives up after
// `timeout_ns`, raises the status bit and the kernel returns.
__global__ void bounded_wait_probe_kernel(int* status, uint64_t timeout_ns) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(&bar, 1);
    mbar_fence_init();
    mbar_wait_bounded(&bar, 0, &abort_flag, status, DS_TMA_WAIT, timeout_ns);
  }
}

}  // namespace mt

extern "C" {

int mt_test_bounded_wait(int64_t timeout_ns, mt_stream_t stream) {
  MT_REQUIRE(timeout_ns > 0 && timeout_ns <= 100000000, "mt_test_bounded_wait: limit must be within (0, 100 ms]");
  int* p = mt::device_status_ptr();
  if (!p) return mt::fail(MT_ERR_CUDA, "device status word not reachable");
  mt::bounded_wait_probe_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(p, (uint64_t)timeout_ns);
  MT_CUDA(cudaGetLastError());
  return MT_OK;
}

int mt_version(void) { return 200; }

int mt_set_launch_overlap(int enabled) { return mt::set_launch_overlap(enabled); }

const char* mt_last_error_string(void) { return mt::g_error; }

int64_t mt_swizzled_scale_bytes(int64_t rows, int64_t k_blocks) {
  if (rows < 0 || k_blocks < 0) return 0;
  int64_t rb = (rows + 127) / 128;
  int64_t kc = (k_blocks + 3) / 4;
  kc = (kc + 3) / 4 * 4;
  return rb * kc * 512;
}

int mt_read_device_status(int* status_out, mt_stream_t stream) {
  MT_REQUIRE(status_out != nullptr, "status_out is null");
  int* p = mt::device_status_ptr();
  if (!p) return mt::fail(MT_ERR_CUDA, "device status word not reachable");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  MT_CUDA(cudaMemcpyAsync(status_out, p, sizeof(int), cudaMemcpyDeviceToHost, s));
  MT_CUDA(cudaMemsetAsync(p, 0, sizeof(int), s));
  MT_CUDA(cudaStreamSynchronize(s));
  return MT_OK;
}

}  // extern "C"
