// Tensor-core int8 peak probe: every SM issues back-to-back tcgen05.mma kind::i8 (M128 N256 K32)
// on operands that stay in shared memory -- no loads, no epilogue.  The rate it reaches is the
// practical ceiling (clocks and power included) that the GEMM kernels are compared with.
#include "k2q_common.cuh"

namespace k2q {
namespace {

constexpr uint32_t kSmemBytes = (128 + 256) * 128 + 64;

__global__ void __launch_bounds__(128, 1) peak_i8_kernel(int iters, Status* status) {
  extern __shared__ __align__(1024) uint8_t smem[];
  const uint32_t base = smem_u32(smem);
  uint64_t* bar = reinterpret_cast<uint64_t*>(smem + (128 + 256) * 128);
  uint32_t* slot = reinterpret_cast<uint32_t*>(bar + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(slot + 1);
  if ((base & 1023u) != 0u) return;
  for (int i = threadIdx.x; i < (128 + 256) * 128 / 4; i += blockDim.x)
    reinterpret_cast<uint32_t*>(smem)[i] = 0x01010101u * (i & 3);
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(bar), 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  fence_proxy_async_smem();
  const int warp = threadIdx.x >> 5;
  if (warp == 0) {
    tmem_alloc(smem_u32(slot), 256);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *slot;
  if (threadIdx.x == 0) {
    constexpr uint32_t idesc = umma_idesc_i8(128, 256);
    const uint64_t a = umma_desc_k128(base), b = umma_desc_k128(base + 128 * 128);
    for (int it = 0; it < iters; ++it) {
#pragma unroll
      for (int k = 0; k < 4; ++k) umma_i8(tmem, a + 2u * k, b + 2u * k, idesc, (it | k) != 0 ? 1u : 0u);
    }
    tc_commit(smem_u32(bar));
    const WaitCtx ctx{abort_flag, status};
    mbar_wait(smem_u32(bar), 0, ctx, 301, iters);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem, 256);
  }
}

}  // namespace
}  // namespace k2q

using namespace k2q;

// Not part of the reference-facing surface: a calibration helper for benchmarks.
extern "C" int k2q_measure_i8_peak(int iters, void* status, double* tops_out, void* stream) {
  if (int rc = check_device_arch()) return rc;
  if (iters < 1 || iters > (1 << 20) || !status || !tops_out)
    return fail(K2Q_EINVAL, "k2q_measure_i8_peak: bad arguments");
  const int sms = sm_count();
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (int rc = check_cuda(cudaFuncSetAttribute(peak_i8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               (int)kSmemBytes),
                          "cudaFuncSetAttribute(peak_i8)"))
    return rc;
  cudaEvent_t e0, e1;
  if (int rc = check_cuda(cudaEventCreate(&e0), "cudaEventCreate")) return rc;
  if (int rc = check_cuda(cudaEventCreate(&e1), "cudaEventCreate")) return rc;
  peak_i8_kernel<<<sms, 128, kSmemBytes, s>>>(iters, static_cast<Status*>(status));  // warm-up
  cudaEventRecord(e0, s);
  peak_i8_kernel<<<sms, 128, kSmemBytes, s>>>(iters, static_cast<Status*>(status));
  cudaEventRecord(e1, s);
  int rc = check_cuda(cudaEventSynchronize(e1), "peak_i8 run");
  float ms = 0.f;
  if (!rc) rc = check_cuda(cudaEventElapsedTime(&ms, e0, e1), "cudaEventElapsedTime");
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  if (rc) return rc;
  const double ops = 2.0 * 128 * 256 * 32 * 4.0 * iters * sms;
  *tops_out = ops / (ms * 1e-3) / 1e12;
  return K2Q_OK;
}
