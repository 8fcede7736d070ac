// Re-expression of a group-128 int4 base against ONE scale per output channel:
//     s_n      = max_g sw4[n, g] * (7 / 127)
//     w8[n, k] = rint(q4[n, k] * (sw4[n, k / 128] / s_n))          |w8| <= 127
// dX = Q8(dY * s) . W contracts over the output channels, and an int4 group scale sits on BOTH
// indices of that contraction, so the backward (and the optional int8-rate forward) of a 4-bit
// base runs on these codes.  HBM-bound: 0.5 byte read and 1 byte written per weight; one warp per
// row, 16 packed bytes (32 codes) per lane and step, 16-byte loads and two 16-byte stores.
// Arithmetic in fp32 with IEEE division, multiplication and round-half-even, so that a host
// restatement with the same three operations gives the same codes bit for bit.
#include "k2q_common.cuh"

namespace k2q {
namespace {

constexpr int kWarpsPerBlock = 8;

__global__ void __launch_bounds__(kWarpsPerBlock * 32)
requant_i4_kernel(const uint8_t* __restrict__ q4, const __nv_bfloat16* __restrict__ sw4, int64_t N, int64_t K,
                  int8_t* __restrict__ w8, int64_t ldw8, float* __restrict__ s_out) {
  const int lane = threadIdx.x & 31;
  const int64_t warp0 = static_cast<int64_t>(blockIdx.x) * kWarpsPerBlock + (threadIdx.x >> 5);
  const int64_t nwarps = static_cast<int64_t>(gridDim.x) * kWarpsPerBlock;
  const int groups = static_cast<int>(K / 128);
  for (int64_t n = warp0; n < N; n += nwarps) {
    const __nv_bfloat16* srow = sw4 + n * groups;
    float mx = 0.f;
    for (int g = lane; g < groups; g += 32) mx = fmaxf(mx, __bfloat162float(srow[g]));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    const float s_n = __fmul_rn(mx, 7.0f / 127.0f);
    if (lane == 0) s_out[n] = s_n;
    const uint8_t* qrow = q4 + n * (K / 2);
    int8_t* orow = w8 + n * ldw8;
    // a warp covers 1024 codes per step: lane l takes codes 32 l .. 32 l + 31 (one quarter of a group)
    for (int64_t k0 = static_cast<int64_t>(lane) * 32; k0 < K; k0 += 1024) {
      const float ratio = s_n > 0.f ? __fdiv_rn(__bfloat162float(srow[k0 >> 7]), s_n) : 0.f;
      const uint4 pk = *reinterpret_cast<const uint4*>(qrow + (k0 >> 1));
      const uint32_t w[4] = {pk.x, pk.y, pk.z, pk.w};
      uint32_t out[8];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        uint32_t lo4 = 0, hi4 = 0;
#pragma unroll
        for (int b = 0; b < 4; ++b) {
          const int byte = static_cast<int>((w[j] >> (8 * b)) & 0xFFu);
          const int c0 = ((byte & 0xF) ^ 8) - 8;          // sign-extended low nibble: code 2b
          const int c1 = ((byte >> 4) ^ 8) - 8;           // high nibble: code 2b + 1
          int v0 = __float2int_rn(__fmul_rn(static_cast<float>(c0), ratio));
          int v1 = __float2int_rn(__fmul_rn(static_cast<float>(c1), ratio));
          v0 = max(-127, min(127, v0));
          v1 = max(-127, min(127, v1));
          const uint32_t pair = (static_cast<uint32_t>(v0) & 0xFFu) | ((static_cast<uint32_t>(v1) & 0xFFu) << 8);
          if (b < 2) lo4 |= pair << (16 * b); else hi4 |= pair << (16 * (b - 2));
        }
        out[2 * j] = lo4;
        out[2 * j + 1] = hi4;
      }
      uint4* dst = reinterpret_cast<uint4*>(orow + k0);
      dst[0] = make_uint4(out[0], out[1], out[2], out[3]);
      dst[1] = make_uint4(out[4], out[5], out[6], out[7]);
    }
  }
}

}  // namespace
}  // namespace k2q

using namespace k2q;

extern "C" int k2q_requant_i4_to_i8(const uint8_t* q4, const void* scale4_bf16, int64_t N, int64_t K,
                                    int8_t* w8, int64_t ldw8, float* scale8, void* stream) {
  if (int rc = check_device_arch()) return rc;
  if (N < 0 || K <= 0 || K % 128 != 0)
    return fail(K2Q_EINVAL, "k2q_requant_i4_to_i8: bad shape N=%lld K=%lld (K must be a multiple of 128)",
                (long long)N, (long long)K);
  if (N == 0) return K2Q_OK;
  if (!q4 || !scale4_bf16 || !w8 || !scale8) return fail(K2Q_EINVAL, "k2q_requant_i4_to_i8: NULL operand");
  if (ldw8 < K || ldw8 % 16 != 0) return fail(K2Q_EINVAL, "k2q_requant_i4_to_i8: ldw8 must be >= K and a multiple of 16");
  if ((reinterpret_cast<uintptr_t>(q4) | reinterpret_cast<uintptr_t>(w8)) & 15)
    return fail(K2Q_EINVAL, "k2q_requant_i4_to_i8: q4 and w8 must be 16-byte aligned");
  const int sms = sm_count();
  if (sms <= 0) return fail(K2Q_ECUDA, "k2q_requant_i4_to_i8: could not read the SM count");
  const int64_t want = (N + kWarpsPerBlock - 1) / kWarpsPerBlock;
  const int grid = static_cast<int>(want < 8LL * sms ? want : 8LL * sms);
  requant_i4_kernel<<<grid, kWarpsPerBlock * 32, 0, static_cast<cudaStream_t>(stream)>>>(
      q4, static_cast<const __nv_bfloat16*>(scale4_bf16), N, K, w8, ldw8, scale8);
  return check_cuda(cudaGetLastError(), "requant_i4_kernel launch");
}
