// Host runtime of the C ABI: thread-local error text, device status word,
// device attribute cache and TMA descriptor encoding through the driver entry
// point (resolved at run time, so the library does not link libcuda).
#include "host.h"

#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "../../include/mslk_b200.h"
#include "common.cuh"

namespace mslk_b200 {

static thread_local char g_err[512] = "";

int fail(int code, const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

void clear_error() { g_err[0] = 0; }

int check_cuda(cudaError_t e, const char *what) {
  if (e == cudaSuccess) return 0;
  return fail(2, "%s: %s", what, cudaGetErrorString(e));
}

__device__ int g_device_status = 0;

constexpr int kMaxDevices = 64;
static int *g_status_ptr[kMaxDevices];
static int g_sm_count[kMaxDevices];
static std::mutex g_mu;

int *device_status_ptr() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    fail(2, "cudaGetDevice failed or device index out of range");
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(g_mu);
  if (!g_status_ptr[dev]) {
    void *p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_device_status);
    if (e != cudaSuccess) {
      fail(2, "cudaGetSymbolAddress(status): %s (was the library built for sm_100a?)", cudaGetErrorString(e));
      return nullptr;
    }
    g_status_ptr[dev] = static_cast<int *>(p);
  }
  return g_status_ptr[dev];
}

int sm_count() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 148;
  std::lock_guard<std::mutex> lock(g_mu);
  if (!g_sm_count[dev]) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    g_sm_count[dev] = n;
  }
  return g_sm_count[dev];
}

int pdl_attribute(cudaLaunchAttribute *attr) {
  static const bool enabled = [] {
    const char *e = getenv("MSLK_B200_PDL");
    return !(e && e[0] == '0');
  }();
  if (!enabled) return 0;
  attr->id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr->val.programmaticStreamSerializationAllowed = 1;
  return 1;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void *p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

static int encode(CUtensorMap *out, CUtensorMapDataType dt, const void *base, uint64_t cols, uint64_t rows,
                  uint64_t pitch_bytes, uint32_t box_cols, uint32_t box_rows, CUtensorMapSwizzle swizzle) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fail(2, "cuTensorMapEncodeTiled is not available from the CUDA driver");
  if (reinterpret_cast<uintptr_t>(base) & 15u) return fail(1, "TMA operand base address must be 16-byte aligned");
  if (pitch_bytes & 15u) return fail(1, "TMA operand row pitch must be a multiple of 16 bytes");
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {pitch_bytes};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, dt, 2, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(2, "cuTensorMapEncodeTiled failed with CUresult %d (cols=%llu rows=%llu pitch=%llu box=%ux%u)",
                static_cast<int>(r), (unsigned long long)cols, (unsigned long long)rows,
                (unsigned long long)pitch_bytes, box_cols, box_rows);
  return 0;
}

int make_tmap_2d_bytes(CUtensorMap *out, const void *base, uint64_t cols_bytes, uint64_t rows,
                       uint64_t pitch_bytes, uint32_t box_cols_bytes, uint32_t box_rows,
                       CUtensorMapSwizzle swizzle) {
  return encode(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, base, cols_bytes, rows, pitch_bytes, box_cols_bytes, box_rows,
                swizzle);
}

int make_tmap_2d_u32(CUtensorMap *out, const void *base, uint64_t cols, uint64_t rows, uint64_t pitch_bytes,
                     uint32_t box_cols, uint32_t box_rows) {
  return encode(out, CU_TENSOR_MAP_DATA_TYPE_UINT32, base, cols, rows, pitch_bytes, box_cols, box_rows,
                CU_TENSOR_MAP_SWIZZLE_NONE);
}

int make_tmap_2d_bf16(CUtensorMap *out, const void *base, uint64_t cols, uint64_t rows, uint64_t pitch_bytes,
                      uint32_t box_cols, uint32_t box_rows, CUtensorMapSwizzle swizzle) {
  return encode(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, base, cols, rows, pitch_bytes, box_cols, box_rows, swizzle);
}

}  // namespace mslk_b200

namespace mslk_b200 {
namespace {
// One CTA waits on an mbarrier that nothing ever arrives on, with the caller's (short) limit: the bounded
// wait must give up, leave its code in the status word and let the kernel return normally.
__global__ void selftest_wait_timeout_kernel(unsigned long long limit_ns, int *status, int *returned) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    abort_flag = 0;
    fence_barrier_init();
  }
  __syncthreads();
  bool ok = true;
  if (threadIdx.x == 0) ok = mbar_wait_limit(&bar, 0, &abort_flag, status, kStatusEpilogueTimeout, limit_ns);
  __syncthreads();
  // the other threads see the abort flag, as the other roles of a GEMM CTA do
  if (threadIdx.x == 32 && returned) *returned = abort_flag ? 1 : (ok ? 0 : 1);
}
}  // namespace
}  // namespace mslk_b200

MSLK_API int mslk_b200_selftest_wait_timeout(uint64_t limit_ns, int *returned_flag, void *stream) {
  using namespace mslk_b200;
  clear_error();
  if (limit_ns == 0 || limit_ns > 100000000ull) return fail(1, "selftest_wait_timeout: limit must be 1 ns .. 100 ms");
  int *status = device_status_ptr();
  if (!status) return 2;
  selftest_wait_timeout_kernel<<<1, 64, 0, static_cast<cudaStream_t>(stream)>>>(limit_ns, status, returned_flag);
  return check_cuda(cudaGetLastError(), "selftest_wait_timeout launch");
}

MSLK_API int mslk_b200_abi_version(void) { return MSLK_B200_ABI_VERSION; }

MSLK_API const char *mslk_b200_last_error(void) { return mslk_b200::g_err; }

MSLK_API int mslk_b200_device_status(int *status_out) {
  using namespace mslk_b200;
  clear_error();
  int *p = device_status_ptr();
  if (!p) return 2;
  if (int rc = check_cuda(cudaDeviceSynchronize(), "cudaDeviceSynchronize")) return rc;
  int v = 0;
  if (int rc = check_cuda(cudaMemcpy(&v, p, sizeof(int), cudaMemcpyDeviceToHost), "read status")) return rc;
  if (v != 0) {
    int zero = 0;
    if (int rc = check_cuda(cudaMemcpy(p, &zero, sizeof(int), cudaMemcpyHostToDevice), "clear status")) return rc;
  }
  if (status_out) *status_out = v;
  return 0;
}
