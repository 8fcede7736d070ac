// Self-test of the bounded-wait machinery: one warp waits on an mbarrier that nobody ever arrives at,
// with a limit of a few microseconds instead of the production kernels' two seconds.  The wait gives
// up, records where in the status block, the kernel returns normally and the context stays usable.
// Nothing here traps, asserts or touches memory it does not own.
#include "k2q_common.cuh"

namespace k2q {
namespace {

constexpr int kSelfTestWaitId = 901;

__global__ void __launch_bounds__(32, 1) selftest_wait_kernel(Status* status, int detail) {
  __shared__ __align__(8) uint64_t bar;
  __shared__ int abort_flag_s;
  volatile int* abort_flag = &abort_flag_s;
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&bar), 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  __syncwarp();
  const WaitCtx wctx{abort_flag, status};
  if (threadIdx.x == 0) {
    // parity 0 of a fresh barrier never completes without an arrival: 2 busy polls, then at most
    // 4 suspended polls of 1 microsecond
    (void)mbar_wait<2u, 4u, 1000u>(smem_u32(&bar), 0u, wctx, kSelfTestWaitId, detail);
  }
  __syncwarp();
}

}  // namespace
}  // namespace k2q

using namespace k2q;

extern "C" int k2q_selftest_wait_expiry(void* status, int detail, void* stream) {
  if (int rc = check_device_arch()) return rc;
  if (!status) return fail(K2Q_EINVAL, "k2q_selftest_wait_expiry: status block is NULL");
  selftest_wait_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<Status*>(status), detail);
  return check_cuda(cudaGetLastError(), "selftest_wait launch");
}
