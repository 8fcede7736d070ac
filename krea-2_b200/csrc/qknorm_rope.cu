// QK-RMSNorm + rotary embedding of the q and k projections, in place, one pass over their bf16
// outputs (mmdit.py:135-141 QKNorm, :25-31 ropeapply, called from Attention.forward :199-208).
// Head dimension 128.  Per (token, head) row of 128 values, with the reference's rounding points:
//     y  = bf16( (x * rsqrt(mean(x^2) + eps)) * (1 + w) )          fp32 statistics, RMSNorm.forward
//     o0 = bf16( cos * y0 - sin * y1 ),  o1 = bf16( sin * y0 + cos * y1 )   consecutive pairs, fp32
// The eager model code spends about twenty elementwise launches per block on this (two casts and a
// norm per tensor, the rotation as stack / multiply / add / cast); here q and k are read and written
// once.  HBM-bound: 2 bytes read and 2 written per value; one warp per token, a 128-value head row
// at a time, 8 bytes per lane.
//
// The tensors are the column blocks of the projections' GEMM output, [T, heads * 128] with a row
// stride (so the slices of one grouped [T, N_q + N_k + ...] result are taken as they are); attention
// then reads them through a [B, heads, S, 128] view of the same memory.
#include "k2q_common.cuh"

namespace k2q {
namespace {

constexpr int kHeadDim = 128;
constexpr int kWarps = 8;

struct QkSegment {
  __nv_bfloat16* x;     // [T, ld] rows, heads * 128 used columns
  int64_t ld;
  int heads;
  const float* w;       // [128]: the norm weight is 1 + w
};

struct QkParams {
  QkSegment seg[2];     // q, k
  int64_t T;
  const float* cosv;    // [T, 64] or NULL (norm only)
  const float* sinv;
  float eps;
};

__global__ void __launch_bounds__(kWarps * 32) qknorm_rope_kernel(const QkParams p) {
  const int lane = threadIdx.x & 31;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * kWarps;
  // one warp per token: its cos / sin pair serves every head of q and k, and no index is divided
  for (int64_t t = static_cast<int64_t>(blockIdx.x) * kWarps + (threadIdx.x >> 5); t < p.T; t += stride) {
    float2 c = make_float2(1.f, 1.f), sn = make_float2(0.f, 0.f);
    if (p.cosv != nullptr) {
      c = __ldg(reinterpret_cast<const float2*>(p.cosv + t * (kHeadDim / 2)) + lane);
      sn = __ldg(reinterpret_cast<const float2*>(p.sinv + t * (kHeadDim / 2)) + lane);
    }
#pragma unroll
    for (int s = 0; s < 2; ++s) {
      const QkSegment& sg = p.seg[s];
      if (sg.heads == 0) continue;
      const float4 w = __ldg(reinterpret_cast<const float4*>(sg.w) + lane);
      const float wv[4] = {w.x + 1.0f, w.y + 1.0f, w.z + 1.0f, w.w + 1.0f};
      // four head rows are requested before the first is worked on (loads in flight per warp)
      for (int h0 = 0; h0 < sg.heads; h0 += 4) {
        uint2 raws[4];
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (h0 + j < sg.heads) raws[j] = *reinterpret_cast<const uint2*>(sg.x + t * sg.ld + (h0 + j) * kHeadDim + lane * 4);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
        const int h = h0 + j;
        if (h >= sg.heads) break;
        __nv_bfloat16* row = sg.x + t * sg.ld + h * kHeadDim + lane * 4;
        const uint2 raw = raws[j];
        float v[4] = {__uint_as_float(raw.x << 16), __uint_as_float(raw.x & 0xFFFF0000u),
                      __uint_as_float(raw.y << 16), __uint_as_float(raw.y & 0xFFFF0000u)};
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) ss = __fmaf_rn(v[i], v[i], ss);
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        const float rstd = rsqrtf(ss / static_cast<float>(kHeadDim) + p.eps);
        float y[4];
#pragma unroll
        for (int i = 0; i < 4; ++i)
          y[i] = __bfloat162float(__float2bfloat16_rn(__fmul_rn(__fmul_rn(v[i], rstd), wv[i])));
        if (p.cosv != nullptr) {
          const float o0 = __fsub_rn(__fmul_rn(c.x, y[0]), __fmul_rn(sn.x, y[1]));
          const float o1 = __fadd_rn(__fmul_rn(sn.x, y[0]), __fmul_rn(c.x, y[1]));
          const float o2 = __fsub_rn(__fmul_rn(c.y, y[2]), __fmul_rn(sn.y, y[3]));
          const float o3 = __fadd_rn(__fmul_rn(sn.y, y[2]), __fmul_rn(c.y, y[3]));
          y[0] = o0; y[1] = o1; y[2] = o2; y[3] = o3;
        }
        uint2 out;
        out.x = pack_bf16x2(y[0], y[1]);
        out.y = pack_bf16x2(y[2], y[3]);
        *reinterpret_cast<uint2*>(row) = out;
        }
      }
    }
  }
}

}  // namespace
}  // namespace k2q

using namespace k2q;

extern "C" int k2q_qknorm_rope(void* q_bf16, int64_t ldq, int heads_q, const float* wq,
                               void* k_bf16, int64_t ldk, int heads_k, const float* wk, int64_t T,
                               const float* cos_t, const float* sin_t, float eps, void* stream) {
  if (int rc = check_device_arch()) return rc;
  if (T < 0 || heads_q < 0 || heads_k < 0 || heads_q + heads_k <= 0)
    return fail(K2Q_EINVAL, "k2q_qknorm_rope: bad shape T=%lld heads %d + %d", (long long)T, heads_q, heads_k);
  if (T == 0) return K2Q_OK;
  if ((heads_q > 0 && (!q_bf16 || !wq)) || (heads_k > 0 && (!k_bf16 || !wk)))
    return fail(K2Q_EINVAL, "k2q_qknorm_rope: NULL tensor or norm weight");
  if ((cos_t == nullptr) != (sin_t == nullptr))
    return fail(K2Q_EINVAL, "k2q_qknorm_rope: cos and sin tables must be given together");
  if ((heads_q > 0 && (ldq < static_cast<int64_t>(heads_q) * kHeadDim || ldq % 4 != 0)) ||
      (heads_k > 0 && (ldk < static_cast<int64_t>(heads_k) * kHeadDim || ldk % 4 != 0)))
    return fail(K2Q_EINVAL, "k2q_qknorm_rope: row strides must cover heads * 128 columns and be multiples of 4");
  const uintptr_t al = (heads_q > 0 ? reinterpret_cast<uintptr_t>(q_bf16) : 0) |
                       (heads_k > 0 ? reinterpret_cast<uintptr_t>(k_bf16) : 0);
  if (al & 7) return fail(K2Q_EINVAL, "k2q_qknorm_rope: q and k must be 8-byte aligned");
  if ((heads_q > 0 && (reinterpret_cast<uintptr_t>(wq) & 15)) || (heads_k > 0 && (reinterpret_cast<uintptr_t>(wk) & 15)) ||
      (cos_t && ((reinterpret_cast<uintptr_t>(cos_t) | reinterpret_cast<uintptr_t>(sin_t)) & 7)))
    return fail(K2Q_EINVAL, "k2q_qknorm_rope: norm weights must be 16-byte aligned, cos/sin tables 8-byte aligned");
  QkParams p{};
  p.seg[0] = QkSegment{static_cast<__nv_bfloat16*>(q_bf16), ldq, heads_q, wq};
  p.seg[1] = QkSegment{static_cast<__nv_bfloat16*>(k_bf16), ldk, heads_k, wk};
  p.T = T; p.cosv = cos_t; p.sinv = sin_t; p.eps = eps;
  const int sms = sm_count();
  if (sms <= 0) return fail(K2Q_ECUDA, "k2q_qknorm_rope: could not read the SM count");
  const int64_t want = (T + kWarps - 1) / kWarps;           // one warp per token
  const int64_t cap = static_cast<int64_t>(sms) * 8;       // 8 CTAs of 8 warps per SM: the SM's 64 warps
  const int grid = static_cast<int>(want < cap ? want : cap);
  qknorm_rope_kernel<<<grid, kWarps * 32, 0, static_cast<cudaStream_t>(stream)>>>(p);
  return check_cuda(cudaGetLastError(), "qknorm_rope_kernel launch");
}
