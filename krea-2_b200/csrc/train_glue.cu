// The elementwise steps of a DiT block between the quantised Linears, forward AND backward, one
// kernel each (the training-time companions of the fused quantisation prologues): in eager model
// code every step below is a chain of casts, norms, multiplies and adds with a bf16 rounding after
// each, and in a LoRA training step those chains cost more than the GEMMs.  HBM-bound kernels over
// bf16 rows; forward values keep the reference's bf16 rounding points, backward values are
// computed in fp32 from the saved inputs and rounded once.
//
//   norm_mod      y = (1 + sc_b) * rmsnorm(x) + sh_b      mmdit.py:158-160, 313-317 (fwd also returns rstd)
//   qk_norm_rope  per head: rmsnorm, rotate pairs          mmdit.py:135-141, 25-31 (qknorm_rope.cu holds the
//                                                          in-place inference form of the same forward)
//   swiglu        h = silu(g) * u                          mmdit.py:178
//   sigmoid_gate  y = a * sigmoid(g)                       mmdit.py:210
//   gate_residual out = x + gate_b * y                     mmdit.py:318-321 (x = NULL: gate_b * y, its backward)
#include "k2q_common.cuh"

namespace k2q {
namespace {

constexpr int kRowThreads = 256;
constexpr int kMaxVec = 4;              // 8-element vectors per thread: rows of up to 8192 columns
constexpr int kHeadDim = 128;

__device__ __forceinline__ float bf16r(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

__device__ __forceinline__ void unpack8(const uint4& r, float* v) {
  const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    v[2 * i] = __uint_as_float(w[i] << 16);
    v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
  }
}
__device__ __forceinline__ uint4 pack8(const float* v) {
  uint4 r;
  r.x = pack_bf16x2(v[0], v[1]); r.y = pack_bf16x2(v[2], v[3]);
  r.z = pack_bf16x2(v[4], v[5]); r.w = pack_bf16x2(v[6], v[7]);
  return r;
}
__device__ __forceinline__ void load8f(const float* p, float* v) {
  const float4 a = __ldg(reinterpret_cast<const float4*>(p));
  const float4 b = __ldg(reinterpret_cast<const float4*>(p) + 1);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}

// sum over the CTA's kRowThreads threads, the same value in every thread
__device__ __forceinline__ float cta_sum(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();                                   // the previous use of red[] has been read
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = 0.f;
#pragma unroll
  for (int w = 0; w < kRowThreads / 32; ++w) t += red[w];
  return t;
}

struct NormModParams {
  const __nv_bfloat16* x; int64_t ldx;
  const __nv_bfloat16* dy; int64_t lddy;       // backward only
  int64_t M; int K;
  const float* normw;
  const __nv_bfloat16* mscale; const __nv_bfloat16* mshift;
  int64_t rows_per_batch; float eps;
  __nv_bfloat16* out; int64_t ldo;             // forward: y, backward: dx
  float* rstd;                                 // forward: written, backward: read
};

template <bool BWD>
__global__ void __launch_bounds__(kRowThreads) norm_mod_kernel(const NormModParams p) {
  __shared__ float red[kRowThreads / 32];
  const int nvec = p.K >> 3;
  for (int64_t row = blockIdx.x; row < p.M; row += gridDim.x) {
    const int64_t b = row / p.rows_per_batch;
    float xv[kMaxVec][8];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < kMaxVec; ++i) {
      const int v = threadIdx.x + i * kRowThreads;
      if (v < nvec) {
        unpack8(__ldg(reinterpret_cast<const uint4*>(p.x + row * p.ldx) + v), xv[i]);
        if (!BWD) {
#pragma unroll
          for (int e = 0; e < 8; ++e) ss = __fmaf_rn(xv[i][e], xv[i][e], ss);
        }
      }
    }
    if (!BWD) {
      const float tot = cta_sum(ss, red);
      const float rstd = rsqrtf(tot / static_cast<float>(p.K) + p.eps);
      if (threadIdx.x == 0) p.rstd[row] = rstd;
#pragma unroll
      for (int i = 0; i < kMaxVec; ++i) {
        const int v = threadIdx.x + i * kRowThreads;
        if (v < nvec) {
          float w[8], o[8];
          load8f(p.normw + 8 * v, w);
#pragma unroll
          for (int e = 0; e < 8; ++e) o[e] = bf16r(__fmul_rn(__fmul_rn(xv[i][e], rstd), w[e] + 1.0f));
          if (p.mscale != nullptr) {
            float sc[8];
            unpack8(__ldg(reinterpret_cast<const uint4*>(p.mscale + b * p.K) + v), sc);
#pragma unroll
            for (int e = 0; e < 8; ++e) o[e] = bf16r(bf16r(1.0f + sc[e]) * o[e]);
          }
          if (p.mshift != nullptr) {
            float sh[8];
            unpack8(__ldg(reinterpret_cast<const uint4*>(p.mshift + b * p.K) + v), sh);
#pragma unroll
            for (int e = 0; e < 8; ++e) o[e] = bf16r(o[e] + sh[e]);
          }
          reinterpret_cast<uint4*>(p.out + row * p.ldo)[v] = pack8(o);
        }
      }
    } else {
      // dn = dy * (1 + sc);  gw = dn * (1 + w);  xh = x * rstd;  dx = rstd * (gw - xh * mean(gw * xh))
      const float rstd = p.rstd[row];
      float gw[kMaxVec][8];
      float dot = 0.f;
#pragma unroll
      for (int i = 0; i < kMaxVec; ++i) {
        const int v = threadIdx.x + i * kRowThreads;
        if (v < nvec) {
          float g[8], w[8];
          unpack8(__ldg(reinterpret_cast<const uint4*>(p.dy + row * p.lddy) + v), g);
          load8f(p.normw + 8 * v, w);
          if (p.mscale != nullptr) {
            float sc[8];
            unpack8(__ldg(reinterpret_cast<const uint4*>(p.mscale + b * p.K) + v), sc);
#pragma unroll
            for (int e = 0; e < 8; ++e) g[e] *= bf16r(1.0f + sc[e]);
          }
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            gw[i][e] = g[e] * (w[e] + 1.0f);
            xv[i][e] *= rstd;
            dot = __fmaf_rn(gw[i][e], xv[i][e], dot);
          }
        }
      }
      const float c = cta_sum(dot, red) / static_cast<float>(p.K);
#pragma unroll
      for (int i = 0; i < kMaxVec; ++i) {
        const int v = threadIdx.x + i * kRowThreads;
        if (v < nvec) {
          float o[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) o[e] = rstd * (gw[i][e] - xv[i][e] * c);
          reinterpret_cast<uint4*>(p.out + row * p.ldo)[v] = pack8(o);
        }
      }
    }
  }
}

// ---- QK norm + rotation, one warp per token, one 128-value head row at a time ------------------
struct QkTrainSeg {
  const __nv_bfloat16* x; int64_t ldx;      // projection output [T, ldx], heads * 128 used columns
  const __nv_bfloat16* dy;                  // backward: gradient of the rotated tensor, element
  int64_t dy_sb, dy_ss, dy_sh;              //   (b, s, h, d) at dy[b*sb + s*ss + h*sh + d]
  __nv_bfloat16* out; int64_t ldo;          // forward: rotated tensor [T, ldo]; backward: dx [T, ldo]
  int heads; const float* w;
};
struct QkTrainParams {
  QkTrainSeg seg[2];
  int64_t T; int64_t S;                     // S tokens per batch element (backward's dy indexing)
  const float* cosv; const float* sinv; float eps;
};

template <bool BWD>
__global__ void __launch_bounds__(256) qk_train_kernel(const QkTrainParams p) {
  const int lane = threadIdx.x & 31;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * 8;
  // one warp per token: its cos / sin pair serves every head of q and k, and no index is divided
  for (int64_t t = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5); t < p.T; t += stride) {
    float2 c = make_float2(1.f, 1.f), sn = make_float2(0.f, 0.f);
    if (p.cosv != nullptr) {
      c = __ldg(reinterpret_cast<const float2*>(p.cosv + t * (kHeadDim / 2)) + lane);
      sn = __ldg(reinterpret_cast<const float2*>(p.sinv + t * (kHeadDim / 2)) + lane);
    }
    int64_t bi = 0, si = t;
    if (BWD) { bi = t / p.S; si = t - bi * p.S; }
#pragma unroll
    for (int s = 0; s < 2; ++s) {
      const QkTrainSeg& sg = p.seg[s];
      const float4 w4 = __ldg(reinterpret_cast<const float4*>(sg.w) + lane);
      const float w[4] = {w4.x + 1.0f, w4.y + 1.0f, w4.z + 1.0f, w4.w + 1.0f};
      // four head rows are requested before the first is worked on (loads in flight per warp)
      for (int h0 = 0; h0 < sg.heads; h0 += 4) {
        uint2 raws[4];
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (h0 + j < sg.heads) raws[j] = __ldg(reinterpret_cast<const uint2*>(sg.x + t * sg.ldx + (h0 + j) * kHeadDim + lane * 4));
#pragma unroll
        for (int j = 0; j < 4; ++j) {
        const int h = h0 + j;
        if (h >= sg.heads) break;
        const uint2 raw = raws[j];
        float v[4] = {__uint_as_float(raw.x << 16), __uint_as_float(raw.x & 0xFFFF0000u),
                      __uint_as_float(raw.y << 16), __uint_as_float(raw.y & 0xFFFF0000u)};
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) ss = __fmaf_rn(v[i], v[i], ss);
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        const float rstd = rsqrtf(ss / static_cast<float>(kHeadDim) + p.eps);
        float o[4];
        if (!BWD) {
          float y[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) y[i] = bf16r(__fmul_rn(__fmul_rn(v[i], rstd), w[i]));
          if (p.cosv != nullptr) {
            o[0] = __fsub_rn(__fmul_rn(c.x, y[0]), __fmul_rn(sn.x, y[1]));
            o[1] = __fadd_rn(__fmul_rn(sn.x, y[0]), __fmul_rn(c.x, y[1]));
            o[2] = __fsub_rn(__fmul_rn(c.y, y[2]), __fmul_rn(sn.y, y[3]));
            o[3] = __fadd_rn(__fmul_rn(sn.y, y[2]), __fmul_rn(c.y, y[3]));
          } else {
#pragma unroll
            for (int i = 0; i < 4; ++i) o[i] = y[i];
          }
        } else {
          const uint2 graw = __ldg(reinterpret_cast<const uint2*>(sg.dy + bi * sg.dy_sb + si * sg.dy_ss + h * sg.dy_sh + lane * 4));
          const float g[4] = {__uint_as_float(graw.x << 16), __uint_as_float(graw.x & 0xFFFF0000u),
                              __uint_as_float(graw.y << 16), __uint_as_float(graw.y & 0xFFFF0000u)};
          // transpose of the rotation, then the norm's backward on the row
          float dyv[4] = {c.x * g[0] + sn.x * g[1], c.x * g[1] - sn.x * g[0],
                          c.y * g[2] + sn.y * g[3], c.y * g[3] - sn.y * g[2]};
          float dot = 0.f;
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            dyv[i] *= w[i];
            v[i] *= rstd;
            dot = __fmaf_rn(dyv[i], v[i], dot);
          }
#pragma unroll
          for (int o2 = 1; o2 < 32; o2 <<= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o2);
          const float cm = dot / static_cast<float>(kHeadDim);
#pragma unroll
          for (int i = 0; i < 4; ++i) o[i] = rstd * (dyv[i] - v[i] * cm);
        }
        uint2 outw;
        outw.x = pack_bf16x2(o[0], o[1]);
        outw.y = pack_bf16x2(o[2], o[3]);
        *reinterpret_cast<uint2*>(sg.out + t * sg.ldo + h * kHeadDim + lane * 4) = outw;
        }
      }
    }
  }
}

// ---- plain elementwise pairs ------------------------------------------------------------------
enum PairOp : int { SWIGLU_FWD, SWIGLU_BWD, SIGGATE_FWD, SIGGATE_BWD, GATE_RESIDUAL };

struct PairParams {
  const __nv_bfloat16* a; int64_t lda;      // g (swiglu) | a (sigmoid gate) | y (gate_residual)
  const __nv_bfloat16* b; int64_t ldb;      // u          | g                | x or NULL
  const __nv_bfloat16* d; int64_t ldd;      // backward: upstream gradient;  gate_residual: gate [B, K]
  __nv_bfloat16* o1; int64_t ldo1;          // h | y | out     ; backward: d(a operand)
  __nv_bfloat16* o2; int64_t ldo2;          // backward: d(b operand)
  int64_t M; int K; int64_t rows_per_batch;
};

template <int OP>
__global__ void __launch_bounds__(256) pair_kernel(const PairParams p) {
  const int nvec = p.K >> 3;
  // rows by CTA, 16-byte vectors of a row by thread: no index is ever divided
  for (int64_t row = blockIdx.x; row < p.M; row += gridDim.x) {
    const __nv_bfloat16* gate_row = OP == GATE_RESIDUAL ? p.d + (row / p.rows_per_batch) * p.K : nullptr;
    for (int v = threadIdx.x; v < nvec; v += 256) {
      float a[8], b[8], d[8], r1[8], r2[8];
      unpack8(__ldg(reinterpret_cast<const uint4*>(p.a + row * p.lda) + v), a);
      if (OP != GATE_RESIDUAL || p.b != nullptr) unpack8(__ldg(reinterpret_cast<const uint4*>(p.b + row * p.ldb) + v), b);
      if (OP == SWIGLU_BWD || OP == SIGGATE_BWD) unpack8(__ldg(reinterpret_cast<const uint4*>(p.d + row * p.ldd) + v), d);
      if (OP == GATE_RESIDUAL) unpack8(__ldg(reinterpret_cast<const uint4*>(gate_row) + v), d);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        if (OP == SWIGLU_FWD) {
          r1[e] = bf16r(bf16r(__fdividef(a[e], 1.0f + __expf(-a[e]))) * b[e]);           // F.silu then the product, bf16 ops
        } else if (OP == SWIGLU_BWD) {
          const float sig = __fdividef(1.0f, 1.0f + __expf(-a[e]));
          const float ds = bf16r(d[e] * b[e]);                                               // gradient of silu(g)
          r1[e] = ds * sig * (1.0f + a[e] * (1.0f - sig));                                   // dg
          r2[e] = d[e] * bf16r(a[e] * sig);                                                  // du = dh * silu(g)
        } else if (OP == SIGGATE_FWD) {
          r1[e] = bf16r(a[e] * bf16r(__fdividef(1.0f, 1.0f + __expf(-b[e]))));
        } else if (OP == SIGGATE_BWD) {
          const float sig = __fdividef(1.0f, 1.0f + __expf(-b[e]));
          r1[e] = d[e] * bf16r(sig);                                                         // da
          r2[e] = bf16r(d[e] * a[e]) * sig * (1.0f - sig);                                   // dg
        } else {
          const float gy = bf16r(d[e] * a[e]);                                               // gate * y
          r1[e] = p.b != nullptr ? gy + b[e] : gy;
        }
      }
      reinterpret_cast<uint4*>(p.o1 + row * p.ldo1)[v] = pack8(r1);
      if (OP == SWIGLU_BWD || OP == SIGGATE_BWD) reinterpret_cast<uint4*>(p.o2 + row * p.ldo2)[v] = pack8(r2);
    }
  }
}

bool bad_rows(const void* ptr, int64_t ld, int K) {
  return ptr == nullptr || ld < K || (ld & 7) != 0 || (reinterpret_cast<uintptr_t>(ptr) & 15) != 0;
}

int elementwise_grid(int64_t work_items, int threads) {
  const int sms = sm_count();
  if (sms <= 0) return -1;
  const int64_t want = (work_items + threads - 1) / threads;
  const int64_t cap = static_cast<int64_t>(sms) * 8;
  return static_cast<int>(want < cap ? (want > 0 ? want : 1) : cap);
}

template <int OP>
int run_pair(const char* name, PairParams p, bool has_b, bool has_d, bool has_o2, void* stream) {
  if (int rc = check_device_arch()) return rc;
  if (p.M < 0 || p.K <= 0 || (p.K & 7)) return fail(K2Q_EINVAL, "%s: bad shape M=%lld K=%d (K must be a multiple of 8)", name, (long long)p.M, p.K);
  if (p.M == 0) return K2Q_OK;
  if (bad_rows(p.a, p.lda, p.K) || (has_b && bad_rows(p.b, p.ldb, p.K)) || bad_rows(p.o1, p.ldo1, p.K) ||
      (has_o2 && bad_rows(p.o2, p.ldo2, p.K)))
    return fail(K2Q_EINVAL, "%s: tensors must be non-NULL, 16-byte aligned, with row strides >= K that are multiples of 8", name);
  if (has_d && OP != GATE_RESIDUAL && bad_rows(p.d, p.ldd, p.K)) return fail(K2Q_EINVAL, "%s: bad upstream gradient", name);
  if (OP == GATE_RESIDUAL && (p.d == nullptr || (reinterpret_cast<uintptr_t>(p.d) & 15) || p.rows_per_batch <= 0))
    return fail(K2Q_EINVAL, "%s: the gate [B, K] must be non-NULL and 16-byte aligned, rows_per_batch positive", name);
  const int grid = elementwise_grid(p.M * 256, 256);        // one CTA per row, at most 8 CTAs per SM
  if (grid < 0) return fail(K2Q_ECUDA, "%s: could not read the SM count", name);
  pair_kernel<OP><<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(p);
  return check_cuda(cudaGetLastError(), name);
}

}  // namespace
}  // namespace k2q

using namespace k2q;

extern "C" {

int k2q_norm_mod_fwd(const void* x_bf16, int64_t ldx, int64_t M, int64_t K, const float* norm_scale,
                     const void* mod_scale_bf16, const void* mod_shift_bf16, int64_t rows_per_batch, float eps,
                     void* y_bf16, int64_t ldy, float* rstd, void* stream) {
  if (int rc = check_device_arch()) return rc;
  if (M < 0 || K <= 0 || (K & 7) || K > 8 * kRowThreads * kMaxVec)
    return fail(K2Q_EINVAL, "k2q_norm_mod_fwd: bad shape M=%lld K=%lld (K a multiple of 8, at most %d)", (long long)M,
                (long long)K, 8 * kRowThreads * kMaxVec);
  if (M == 0) return K2Q_OK;
  if (bad_rows(x_bf16, ldx, (int)K) || bad_rows(y_bf16, ldy, (int)K) || !norm_scale || !rstd ||
      (reinterpret_cast<uintptr_t>(norm_scale) & 15) || (reinterpret_cast<uintptr_t>(mod_scale_bf16) & 15) ||
      (reinterpret_cast<uintptr_t>(mod_shift_bf16) & 15) || rows_per_batch <= 0)
    return fail(K2Q_EINVAL, "k2q_norm_mod_fwd: NULL or misaligned operand");
  NormModParams p{};
  p.x = static_cast<const __nv_bfloat16*>(x_bf16); p.ldx = ldx; p.M = M; p.K = (int)K; p.normw = norm_scale;
  p.mscale = static_cast<const __nv_bfloat16*>(mod_scale_bf16); p.mshift = static_cast<const __nv_bfloat16*>(mod_shift_bf16);
  p.rows_per_batch = rows_per_batch; p.eps = eps; p.out = static_cast<__nv_bfloat16*>(y_bf16); p.ldo = ldy; p.rstd = rstd;
  const int sms = sm_count();
  if (sms <= 0) return fail(K2Q_ECUDA, "k2q_norm_mod_fwd: could not read the SM count");
  const int grid = (int)(M < 8LL * sms ? M : 8LL * sms);
  norm_mod_kernel<false><<<grid, kRowThreads, 0, static_cast<cudaStream_t>(stream)>>>(p);
  return check_cuda(cudaGetLastError(), "k2q_norm_mod_fwd");
}

int k2q_norm_mod_bwd(const void* dy_bf16, int64_t lddy, const void* x_bf16, int64_t ldx, const float* rstd, int64_t M,
                     int64_t K, const float* norm_scale, const void* mod_scale_bf16, int64_t rows_per_batch,
                     void* dx_bf16, int64_t lddx, void* stream) {
  if (int rc = check_device_arch()) return rc;
  if (M < 0 || K <= 0 || (K & 7) || K > 8 * kRowThreads * kMaxVec)
    return fail(K2Q_EINVAL, "k2q_norm_mod_bwd: bad shape M=%lld K=%lld", (long long)M, (long long)K);
  if (M == 0) return K2Q_OK;
  if (bad_rows(x_bf16, ldx, (int)K) || bad_rows(dy_bf16, lddy, (int)K) || bad_rows(dx_bf16, lddx, (int)K) || !norm_scale ||
      !rstd || (reinterpret_cast<uintptr_t>(norm_scale) & 15) || (reinterpret_cast<uintptr_t>(mod_scale_bf16) & 15) ||
      rows_per_batch <= 0)
    return fail(K2Q_EINVAL, "k2q_norm_mod_bwd: NULL or misaligned operand");
  NormModParams p{};
  p.x = static_cast<const __nv_bfloat16*>(x_bf16); p.ldx = ldx; p.dy = static_cast<const __nv_bfloat16*>(dy_bf16); p.lddy = lddy;
  p.M = M; p.K = (int)K; p.normw = norm_scale; p.mscale = static_cast<const __nv_bfloat16*>(mod_scale_bf16);
  p.rows_per_batch = rows_per_batch; p.out = static_cast<__nv_bfloat16*>(dx_bf16); p.ldo = lddx;
  p.rstd = const_cast<float*>(rstd);
  const int sms = sm_count();
  if (sms <= 0) return fail(K2Q_ECUDA, "k2q_norm_mod_bwd: could not read the SM count");
  const int grid = (int)(M < 8LL * sms ? M : 8LL * sms);
  norm_mod_kernel<true><<<grid, kRowThreads, 0, static_cast<cudaStream_t>(stream)>>>(p);
  return check_cuda(cudaGetLastError(), "k2q_norm_mod_bwd");
}

int k2q_qknorm_rope_fwd(const void* q_bf16, int64_t ldq, int heads_q, const float* wq, void* qo_bf16, int64_t ldqo,
                        const void* k_bf16, int64_t ldk, int heads_k, const float* wk, void* ko_bf16, int64_t ldko,
                        int64_t T, const float* cos_t, const float* sin_t, float eps, void* stream) {
  if (int rc = check_device_arch()) return rc;
  if (T < 0 || heads_q <= 0 || heads_k <= 0) return fail(K2Q_EINVAL, "k2q_qknorm_rope_fwd: bad shape");
  if (T == 0) return K2Q_OK;
  if (bad_rows(q_bf16, ldq, heads_q * kHeadDim) || bad_rows(k_bf16, ldk, heads_k * kHeadDim) ||
      bad_rows(qo_bf16, ldqo, heads_q * kHeadDim) || bad_rows(ko_bf16, ldko, heads_k * kHeadDim) || !wq || !wk ||
      ((reinterpret_cast<uintptr_t>(wq) | reinterpret_cast<uintptr_t>(wk)) & 15) || (cos_t == nullptr) != (sin_t == nullptr) ||
      ((reinterpret_cast<uintptr_t>(cos_t) | reinterpret_cast<uintptr_t>(sin_t)) & 7))
    return fail(K2Q_EINVAL, "k2q_qknorm_rope_fwd: NULL or misaligned operand");
  QkTrainParams p{};
  p.seg[0] = QkTrainSeg{static_cast<const __nv_bfloat16*>(q_bf16), ldq, nullptr, 0, 0, 0,
                        static_cast<__nv_bfloat16*>(qo_bf16), ldqo, heads_q, wq};
  p.seg[1] = QkTrainSeg{static_cast<const __nv_bfloat16*>(k_bf16), ldk, nullptr, 0, 0, 0,
                        static_cast<__nv_bfloat16*>(ko_bf16), ldko, heads_k, wk};
  p.T = T; p.S = T; p.cosv = cos_t; p.sinv = sin_t; p.eps = eps;
  const int grid = elementwise_grid(T * 32, 256);           // one warp per token
  if (grid < 0) return fail(K2Q_ECUDA, "k2q_qknorm_rope_fwd: could not read the SM count");
  qk_train_kernel<false><<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(p);
  return check_cuda(cudaGetLastError(), "k2q_qknorm_rope_fwd");
}

int k2q_qknorm_rope_bwd(const void* q_bf16, int64_t ldq, int heads_q, const float* wq, const void* dqo_bf16,
                        int64_t dq_sb, int64_t dq_ss, int64_t dq_sh, void* dq_bf16, int64_t lddq,
                        const void* k_bf16, int64_t ldk, int heads_k, const float* wk, const void* dko_bf16,
                        int64_t dk_sb, int64_t dk_ss, int64_t dk_sh, void* dk_bf16, int64_t lddk,
                        int64_t B, int64_t S, const float* cos_t, const float* sin_t, float eps, void* stream) {
  if (int rc = check_device_arch()) return rc;
  if (B < 0 || S <= 0 || heads_q <= 0 || heads_k <= 0) return fail(K2Q_EINVAL, "k2q_qknorm_rope_bwd: bad shape");
  if (B == 0) return K2Q_OK;
  if (bad_rows(q_bf16, ldq, heads_q * kHeadDim) || bad_rows(k_bf16, ldk, heads_k * kHeadDim) ||
      bad_rows(dq_bf16, lddq, heads_q * kHeadDim) || bad_rows(dk_bf16, lddk, heads_k * kHeadDim) || !dqo_bf16 || !dko_bf16 ||
      !wq || !wk || ((reinterpret_cast<uintptr_t>(wq) | reinterpret_cast<uintptr_t>(wk)) & 15) ||
      (cos_t == nullptr) != (sin_t == nullptr) || ((reinterpret_cast<uintptr_t>(cos_t) | reinterpret_cast<uintptr_t>(sin_t)) & 7) ||
      ((reinterpret_cast<uintptr_t>(dqo_bf16) | reinterpret_cast<uintptr_t>(dko_bf16)) & 7) ||
      ((dq_sb | dq_ss | dq_sh | dk_sb | dk_ss | dk_sh) & 3))
    return fail(K2Q_EINVAL, "k2q_qknorm_rope_bwd: NULL or misaligned operand (gradient strides must be multiples of 4)");
  QkTrainParams p{};
  p.seg[0] = QkTrainSeg{static_cast<const __nv_bfloat16*>(q_bf16), ldq, static_cast<const __nv_bfloat16*>(dqo_bf16), dq_sb, dq_ss,
                        dq_sh, static_cast<__nv_bfloat16*>(dq_bf16), lddq, heads_q, wq};
  p.seg[1] = QkTrainSeg{static_cast<const __nv_bfloat16*>(k_bf16), ldk, static_cast<const __nv_bfloat16*>(dko_bf16), dk_sb, dk_ss,
                        dk_sh, static_cast<__nv_bfloat16*>(dk_bf16), lddk, heads_k, wk};
  p.T = B * S; p.S = S; p.cosv = cos_t; p.sinv = sin_t; p.eps = eps;
  const int grid = elementwise_grid(p.T * 32, 256);         // one warp per token
  if (grid < 0) return fail(K2Q_ECUDA, "k2q_qknorm_rope_bwd: could not read the SM count");
  qk_train_kernel<true><<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(p);
  return check_cuda(cudaGetLastError(), "k2q_qknorm_rope_bwd");
}

int k2q_swiglu_fwd(const void* g, int64_t ldg, const void* u, int64_t ldu, int64_t M, int64_t K, void* h, int64_t ldh,
                   void* stream) {
  PairParams p{};
  p.a = static_cast<const __nv_bfloat16*>(g); p.lda = ldg; p.b = static_cast<const __nv_bfloat16*>(u); p.ldb = ldu;
  p.o1 = static_cast<__nv_bfloat16*>(h); p.ldo1 = ldh; p.M = M; p.K = (int)(K > 0x7fffffff ? -1 : K);
  return run_pair<SWIGLU_FWD>("k2q_swiglu_fwd", p, true, false, false, stream);
}
int k2q_swiglu_bwd(const void* dh, int64_t lddh, const void* g, int64_t ldg, const void* u, int64_t ldu, int64_t M,
                   int64_t K, void* dg, int64_t lddg, void* du, int64_t lddu, void* stream) {
  PairParams p{};
  p.a = static_cast<const __nv_bfloat16*>(g); p.lda = ldg; p.b = static_cast<const __nv_bfloat16*>(u); p.ldb = ldu;
  p.d = static_cast<const __nv_bfloat16*>(dh); p.ldd = lddh; p.o1 = static_cast<__nv_bfloat16*>(dg); p.ldo1 = lddg;
  p.o2 = static_cast<__nv_bfloat16*>(du); p.ldo2 = lddu; p.M = M; p.K = (int)(K > 0x7fffffff ? -1 : K);
  return run_pair<SWIGLU_BWD>("k2q_swiglu_bwd", p, true, true, true, stream);
}
int k2q_sigmoid_gate_fwd(const void* a, int64_t lda, const void* g, int64_t ldg, int64_t M, int64_t K, void* y,
                         int64_t ldy, void* stream) {
  PairParams p{};
  p.a = static_cast<const __nv_bfloat16*>(a); p.lda = lda; p.b = static_cast<const __nv_bfloat16*>(g); p.ldb = ldg;
  p.o1 = static_cast<__nv_bfloat16*>(y); p.ldo1 = ldy; p.M = M; p.K = (int)(K > 0x7fffffff ? -1 : K);
  return run_pair<SIGGATE_FWD>("k2q_sigmoid_gate_fwd", p, true, false, false, stream);
}
int k2q_sigmoid_gate_bwd(const void* dy, int64_t lddy, const void* a, int64_t lda, const void* g, int64_t ldg, int64_t M,
                         int64_t K, void* da, int64_t ldda, void* dg, int64_t lddg, void* stream) {
  PairParams p{};
  p.a = static_cast<const __nv_bfloat16*>(a); p.lda = lda; p.b = static_cast<const __nv_bfloat16*>(g); p.ldb = ldg;
  p.d = static_cast<const __nv_bfloat16*>(dy); p.ldd = lddy; p.o1 = static_cast<__nv_bfloat16*>(da); p.ldo1 = ldda;
  p.o2 = static_cast<__nv_bfloat16*>(dg); p.ldo2 = lddg; p.M = M; p.K = (int)(K > 0x7fffffff ? -1 : K);
  return run_pair<SIGGATE_BWD>("k2q_sigmoid_gate_bwd", p, true, true, true, stream);
}
int k2q_gate_residual(const void* x_or_null, int64_t ldx, const void* y, int64_t ldy, const void* gate_bk,
                      int64_t rows_per_batch, int64_t M, int64_t K, void* out, int64_t ldo, void* stream) {
  PairParams p{};
  p.a = static_cast<const __nv_bfloat16*>(y); p.lda = ldy; p.b = static_cast<const __nv_bfloat16*>(x_or_null); p.ldb = ldx;
  p.d = static_cast<const __nv_bfloat16*>(gate_bk); p.rows_per_batch = rows_per_batch;
  p.o1 = static_cast<__nv_bfloat16*>(out); p.ldo1 = ldo; p.M = M; p.K = (int)(K > 0x7fffffff ? -1 : K);
  return run_pair<GATE_RESIDUAL>("k2q_gate_residual", p, x_or_null != nullptr, true, false, stream);
}

}  // extern "C"
