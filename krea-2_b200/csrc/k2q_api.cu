// Host-side plumbing shared by every entry point: error strings, device checks, the
// cuTensorMapEncodeTiled lookup and the status block read-back.
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "k2q_common.cuh"

namespace k2q {

static thread_local char g_err[512] = "";

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

int check_cuda(cudaError_t e, const char* what) {
  if (e == cudaSuccess) return K2Q_OK;
  return fail(K2Q_ECUDA, "%s: %s (%s)", what, cudaGetErrorName(e), cudaGetErrorString(e));
}

namespace {
struct DevInfo {
  bool known = false;
  int major = 0, minor = 0, sms = 0;
};
std::mutex g_mu;
DevInfo g_dev[64];

int dev_info(DevInfo* out) {
  int dev = 0;
  if (int rc = check_cuda(cudaGetDevice(&dev), "cudaGetDevice")) return rc;
  if (dev < 0 || dev >= 64) return fail(K2Q_EINVAL, "device index %d out of range", dev);
  std::lock_guard<std::mutex> lock(g_mu);
  if (!g_dev[dev].known) {
    DevInfo d;
    if (int rc = check_cuda(cudaDeviceGetAttribute(&d.major, cudaDevAttrComputeCapabilityMajor, dev),
                            "cudaDeviceGetAttribute(major)"))
      return rc;
    if (int rc = check_cuda(cudaDeviceGetAttribute(&d.minor, cudaDevAttrComputeCapabilityMinor, dev),
                            "cudaDeviceGetAttribute(minor)"))
      return rc;
    if (int rc = check_cuda(cudaDeviceGetAttribute(&d.sms, cudaDevAttrMultiProcessorCount, dev),
                            "cudaDeviceGetAttribute(sms)"))
      return rc;
    d.known = true;
    g_dev[dev] = d;
  }
  *out = g_dev[dev];
  return K2Q_OK;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;

int get_encode(EncodeTiledFn* fn) {
  std::lock_guard<std::mutex> lock(g_mu);
  if (!g_encode) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (int rc = check_cuda(
            cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q),
            "cudaGetDriverEntryPoint(cuTensorMapEncodeTiled)"))
      return rc;
    if (q != cudaDriverEntryPointSuccess || !p)
      return fail(K2Q_ECUDA, "cuTensorMapEncodeTiled not available from this driver");
    g_encode = reinterpret_cast<EncodeTiledFn>(p);
  }
  *fn = g_encode;
  return K2Q_OK;
}
}  // namespace

int check_device_arch() {
  DevInfo d;
  if (int rc = dev_info(&d)) return rc;
  if (d.major != 10)
    return fail(K2Q_EARCH, "k2q kernels are built for sm_100a only; current device is sm_%d%d",
                d.major, d.minor);
  return K2Q_OK;
}

bool overlapped_launch_allowed(cudaStream_t stream) {
  static const bool disabled = getenv("K2Q_NO_PDL") != nullptr;
  if (disabled) return false;
  cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(stream, &st) != cudaSuccess) {
    (void)cudaGetLastError();
    return false;
  }
  return st == cudaStreamCaptureStatusNone;
}

int sm_count() {
  DevInfo d;
  if (dev_info(&d)) return 0;
  return d.sms;
}

int encode_tmap_2d_u8(CUtensorMap* map, const void* base, uint64_t inner_bytes, uint64_t rows,
                      uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_rows,
                      int swizzle) {
  EncodeTiledFn enc;
  if (int rc = get_encode(&enc)) return rc;
  if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0)
    return fail(K2Q_EINVAL, "TMA operand base %p is not 16-byte aligned", base);
  if ((row_stride_bytes & 15u) != 0)
    return fail(K2Q_EINVAL, "TMA operand row stride %llu is not a multiple of 16 bytes",
                (unsigned long long)row_stride_bytes);
  cuuint64_t dims[2] = {inner_bytes, rows};
  cuuint64_t strides[1] = {row_stride_bytes};
  cuuint32_t box[2] = {box_inner, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides,
                   box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   swizzle == 1 ? CU_TENSOR_MAP_SWIZZLE_128B
                   : swizzle == 2 ? CU_TENSOR_MAP_SWIZZLE_64B
                   : swizzle == 3 ? CU_TENSOR_MAP_SWIZZLE_32B
                                  : CU_TENSOR_MAP_SWIZZLE_NONE,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(K2Q_ECUDA, "cuTensorMapEncodeTiled failed with CUresult %d (inner=%llu rows=%llu)",
                (int)r, (unsigned long long)inner_bytes, (unsigned long long)rows);
  return K2Q_OK;
}

}  // namespace k2q

extern "C" {

int k2q_version(void) { return K2Q_VERSION; }

const char* k2q_last_error(void) { return k2q::g_err; }

int64_t k2q_status_bytes(void) { return (int64_t)sizeof(k2q::Status); }

int k2q_check_status(const void* status_dev, void* stream) {
  if (!status_dev) return k2q::fail(K2Q_EINVAL, "status block is NULL");
  k2q::Status h;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (int rc = k2q::check_cuda(
          cudaMemcpyAsync(&h, status_dev, sizeof(h), cudaMemcpyDeviceToHost, s),
          "cudaMemcpyAsync(status)"))
    return rc;
  if (int rc = k2q::check_cuda(cudaStreamSynchronize(s), "cudaStreamSynchronize(status)")) return rc;
  if (h.code != 0)
    return k2q::fail(K2Q_ETIMEOUT,
                     "a bounded device wait expired: wait id %d, CTA %d, detail %d "
                     "(results of that launch are invalid)",
                     h.code, h.block, h.detail);
  return K2Q_OK;
}

}  // extern "C"
