// K1 / K2 and friends: block-128 Walsh-Hadamard rotation of rows fused with quantisation.
//
// One kernel template covers
//   ROT_Q8   rotate + per-row int8        (activations K2, int8 weights K1)
//   ROT_Q4   rotate + per-(row,128-group) int4, packed two codes per byte (int4 weights K1)
//   ROT_ONLY rotate, write bf16 / f32     (de-rotation of dX, rotation of the LoRA A matrix)
//   Q8_ONLY  per-row int8 of g*colscale   (dY folded with the weight scales, backward)
//
// Work split: a row is cut into "tasks" of 16 elements; the 8 tasks of one 128-block sit in 8
// neighbouring lanes.  A task is two 8-element pieces 64 elements apart, so every 128-bit load
// of a warp instruction lands in fully used 128-byte segments.  Butterfly stages h=1,2,4 and
// h=64 run inside a thread, h=8,16,32 are lane exchanges (shfl.xor 1,2,4).  The stage order,
// the (a+b, a-b) pairing and the single final multiply are those of the CPU oracle, all in
// fp32 with explicitly rounded operations, so codes and scales come out bit-identical.
#include "k2q_common.cuh"

namespace k2q {
namespace {

enum Mode : int { ROT_Q8 = 0, ROT_Q4 = 1, ROT_ONLY = 2, Q8_ONLY = 3 };

constexpr int kThreads = 256;
constexpr float kHadNorm = 0.088388347648318440550f;  // fp32(2^-3.5)

struct RowsParams {
  const void* x;
  int64_t ldx;
  int64_t M;
  int K;
  int t_row;              // threads per row (8..256, power of two)
  const float* colscale;  // Q8_ONLY
  int8_t* q8;             // [M,K]
  float* s8;              // [M]
  uint8_t* q4;            // [M,K/2]
  __nv_bfloat16* s4;      // [M,K/128]
  void* y;                // ROT_ONLY output
  int64_t ldy;
  int y_f32;
};

__device__ __forceinline__ void load8(const __nv_bfloat16* p, float* v) {
  uint4 r = __ldg(reinterpret_cast<const uint4*>(p));
  const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    v[2 * i] = __uint_as_float(w[i] << 16);
    v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
  }
}
__device__ __forceinline__ void load8(const float* p, float* v) {
  float4 a = __ldg(reinterpret_cast<const float4*>(p));
  float4 b = __ldg(reinterpret_cast<const float4*>(p) + 1);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
  v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}

// stages h = 1, 2, 4 on one 8-element piece
__device__ __forceinline__ void butterfly8(float* v) {
#pragma unroll
  for (int h = 1; h < 8; h <<= 1) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if ((i & h) == 0) {
        const float a = v[i], b = v[i + h];
        v[i] = __fadd_rn(a, b);
        v[i + h] = __fsub_rn(a, b);
      }
    }
  }
}

// full 128-point transform of the block whose 16 values per lane are in v (8 lanes per block)
__device__ __forceinline__ void hadamard_task(float* v, int t8) {
  butterfly8(v);
  butterfly8(v + 8);
#pragma unroll
  for (int j = 0; j < 3; ++j) {  // h = 8, 16, 32: partner lane differs in bit j of t8
    const bool upper = (t8 >> j) & 1;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const float o = __shfl_xor_sync(0xffffffffu, v[i], 1 << j);
      v[i] = upper ? __fsub_rn(o, v[i]) : __fadd_rn(v[i], o);
    }
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) {  // h = 64
    const float a = v[i], b = v[i + 8];
    v[i] = __fadd_rn(a, b);
    v[i + 8] = __fsub_rn(a, b);
  }
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __fmul_rn(v[i], kHadNorm);
}

__device__ __forceinline__ int quant_code(float v, float s, float qmax) {
  float q = rintf(__fdiv_rn(v, s));
  q = fminf(fmaxf(q, -qmax), qmax);
  return static_cast<int>(q);
}

template <typename InT, int NCHUNK, int MODE>
__global__ void __launch_bounds__(kThreads) rows_kernel(const RowsParams p) {
  __shared__ float s_red[kThreads / 32];

  const int t_row = p.t_row;
  const int tr = threadIdx.x & (t_row - 1);
  const int64_t row = static_cast<int64_t>(blockIdx.x) * (kThreads / t_row) + threadIdx.x / t_row;
  const bool row_ok = row < p.M;
  const int ntasks = p.K >> 4;
  const InT* xrow = static_cast<const InT*>(p.x) + (row_ok ? row : 0) * p.ldx;

  float v[NCHUNK][16];
  float amax = 0.f;

#pragma unroll
  for (int c = 0; c < NCHUNK; ++c) {
    const int task = tr + c * t_row;
    const bool ok = row_ok && task < ntasks;
    const int t8 = task & 7;
    const int k0 = (task >> 3) * 128 + t8 * 8;
    if (ok) {
      load8(xrow + k0, v[c]);
      load8(xrow + k0 + 64, v[c] + 8);
    } else {
#pragma unroll
      for (int i = 0; i < 16; ++i) v[c][i] = 0.f;
    }
    if (MODE == Q8_ONLY) {
      if (ok && p.colscale != nullptr) {
        float cs[16];
        load8(p.colscale + k0, cs);
        load8(p.colscale + k0 + 64, cs + 8);
#pragma unroll
        for (int i = 0; i < 16; ++i) v[c][i] = __fmul_rn(v[c][i], cs[i]);
      }
    } else {
      hadamard_task(v[c], t8);
    }

    if (MODE == ROT_ONLY) {
      if (ok) {
        if (p.y_f32) {
          float* yrow = static_cast<float*>(p.y) + row * p.ldy;
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            float4* dst = reinterpret_cast<float4*>(yrow + k0 + 64 * h);
            dst[0] = make_float4(v[c][8 * h], v[c][8 * h + 1], v[c][8 * h + 2], v[c][8 * h + 3]);
            dst[1] = make_float4(v[c][8 * h + 4], v[c][8 * h + 5], v[c][8 * h + 6], v[c][8 * h + 7]);
          }
        } else {
          __nv_bfloat16* yrow = static_cast<__nv_bfloat16*>(p.y) + row * p.ldy;
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            uint4 o;
            o.x = pack_bf16x2(v[c][8 * h], v[c][8 * h + 1]);
            o.y = pack_bf16x2(v[c][8 * h + 2], v[c][8 * h + 3]);
            o.z = pack_bf16x2(v[c][8 * h + 4], v[c][8 * h + 5]);
            o.w = pack_bf16x2(v[c][8 * h + 6], v[c][8 * h + 7]);
            *reinterpret_cast<uint4*>(yrow + k0 + 64 * h) = o;
          }
        }
      }
    } else if (MODE == ROT_Q4) {
      float gmax = 0.f;
#pragma unroll
      for (int i = 0; i < 16; ++i) gmax = fmaxf(gmax, fabsf(v[c][i]));
      gmax = fmaxf(gmax, __shfl_xor_sync(0xffffffffu, gmax, 1));
      gmax = fmaxf(gmax, __shfl_xor_sync(0xffffffffu, gmax, 2));
      gmax = fmaxf(gmax, __shfl_xor_sync(0xffffffffu, gmax, 4));
      const float s = __fdiv_rn(fmaxf(gmax, 1e-8f), 7.0f);
      if (ok) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          uint32_t word = 0;
#pragma unroll
          for (int i = 0; i < 8; ++i)
            word |= static_cast<uint32_t>(quant_code(v[c][8 * h + i], s, 7.0f) & 0xF) << (4 * i);
          *reinterpret_cast<uint32_t*>(p.q4 + row * (p.K >> 1) + (k0 >> 1) + 32 * h) = word;
        }
        if (t8 == 0) p.s4[row * (p.K >> 7) + (task >> 3)] = __float2bfloat16_rn(s);
      }
    } else {
#pragma unroll
      for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(v[c][i]));
    }
  }

  if (MODE == ROT_Q8 || MODE == Q8_ONLY) {
    // row absmax: inside the warp, then across the warps that share the row
    const int span = t_row < 32 ? t_row : 32;
    for (int off = span >> 1; off > 0; off >>= 1)
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
    if (t_row > 32) {
      if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = amax;
      __syncthreads();
      const int w0 = (threadIdx.x / t_row) * (t_row >> 5);
      amax = 0.f;
      for (int w = 0; w < (t_row >> 5); ++w) amax = fmaxf(amax, s_red[w0 + w]);
    }
    const float s = __fdiv_rn(fmaxf(amax, 1e-8f), 127.0f);
    if (row_ok && tr == 0) p.s8[row] = s;
#pragma unroll
    for (int c = 0; c < NCHUNK; ++c) {
      const int task = tr + c * t_row;
      if (!(row_ok && task < ntasks)) continue;
      const int k0 = (task >> 3) * 128 + (task & 7) * 8;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        uint32_t w[2] = {0u, 0u};
#pragma unroll
        for (int i = 0; i < 8; ++i)
          w[i >> 2] |= static_cast<uint32_t>(quant_code(v[c][8 * h + i], s, 127.0f) & 0xFF)
                       << (8 * (i & 3));
        *reinterpret_cast<uint2*>(p.q8 + row * static_cast<int64_t>(p.K) + k0 + 64 * h) =
            make_uint2(w[0], w[1]);
      }
    }
  }
}

// Pick threads-per-row and chunks-per-thread: smallest padding, then chunks nearest to 3.
void pick_split(int K, int* t_row, int* nchunk) {
  static const int kChunks[] = {1, 2, 3, 4, 6, 8};
  const int ntasks = K / 16;
  int best_waste = 1 << 30, best_t = 0, best_c = 0, best_pref = 1 << 30;
  for (int t = 256; t >= 8; t >>= 1) {
    for (int c : kChunks) {
      const int cover = t * c;
      if (cover < ntasks) continue;
      const int waste = cover - ntasks;
      const int pref = (c > 3 ? c - 3 : 3 - c) * 4 + (t > 64 ? 1 : 0);
      if (waste < best_waste || (waste == best_waste && pref < best_pref)) {
        best_waste = waste; best_t = t; best_c = c; best_pref = pref;
      }
    }
  }
  *t_row = best_t;
  *nchunk = best_c;
}

template <typename InT, int MODE>
int launch_rows(const RowsParams& p, int nchunk, cudaStream_t stream) {
  const int rows_per_cta = kThreads / p.t_row;
  const int64_t grid64 = (p.M + rows_per_cta - 1) / rows_per_cta;
  if (grid64 > 0x7fffffffLL) return fail(K2Q_EINVAL, "too many rows (%lld)", (long long)p.M);
  const dim3 grid(static_cast<unsigned>(grid64));
  switch (nchunk) {
    case 1: rows_kernel<InT, 1, MODE><<<grid, kThreads, 0, stream>>>(p); break;
    case 2: rows_kernel<InT, 2, MODE><<<grid, kThreads, 0, stream>>>(p); break;
    case 3: rows_kernel<InT, 3, MODE><<<grid, kThreads, 0, stream>>>(p); break;
    case 4: rows_kernel<InT, 4, MODE><<<grid, kThreads, 0, stream>>>(p); break;
    case 6: rows_kernel<InT, 6, MODE><<<grid, kThreads, 0, stream>>>(p); break;
    case 8: rows_kernel<InT, 8, MODE><<<grid, kThreads, 0, stream>>>(p); break;
    default: return fail(K2Q_EINVAL, "internal: unsupported chunk count %d", nchunk);
  }
  return check_cuda(cudaGetLastError(), "rows_kernel launch");
}

template <int MODE>
int run_rows(RowsParams p, int dtype, const char* name, cudaStream_t stream) {
  if (int rc = check_device_arch()) return rc;
  if (p.M < 0 || p.K <= 0) return fail(K2Q_EINVAL, "%s: bad shape M=%lld K=%d", name, (long long)p.M, p.K);
  if (p.K % 128 != 0) return fail(K2Q_EINVAL, "%s: K=%d is not a multiple of 128", name, p.K);
  if (p.K > 32768) return fail(K2Q_EINVAL, "%s: K=%d exceeds the supported maximum 32768", name, p.K);
  if (dtype != K2Q_BF16 && dtype != K2Q_F32) return fail(K2Q_EINVAL, "%s: unknown dtype tag %d", name, dtype);
  if (p.M == 0) return K2Q_OK;
  if (!p.x) return fail(K2Q_EINVAL, "%s: input pointer is NULL", name);
  const int esz = dtype == K2Q_BF16 ? 2 : 4;
  if (p.ldx < p.K) return fail(K2Q_EINVAL, "%s: leading dimension %lld < K=%d", name, (long long)p.ldx, p.K);
  if ((reinterpret_cast<uintptr_t>(p.x) & 15u) || ((p.ldx * esz) & 15))
    return fail(K2Q_EINVAL, "%s: input rows must be 16-byte aligned (ptr %p, ld %lld)", name, p.x,
                (long long)p.ldx);
  int nchunk = 0;
  pick_split(p.K, &p.t_row, &nchunk);
  if (dtype == K2Q_BF16) return launch_rows<__nv_bfloat16, MODE>(p, nchunk, stream);
  return launch_rows<float, MODE>(p, nchunk, stream);
}

bool misaligned(const void* ptr, unsigned a) { return (reinterpret_cast<uintptr_t>(ptr) & (a - 1)) != 0; }

}  // namespace
}  // namespace k2q

using namespace k2q;

extern "C" {

int k2q_fwht_quant_act_i8(const void* x, int x_dtype, int64_t M, int64_t K, int64_t ldx, int8_t* xq,
                          float* sx, void* stream) {
  if (M > 0 && (!xq || !sx)) return fail(K2Q_EINVAL, "k2q_fwht_quant_act_i8: output pointer is NULL");
  if (misaligned(xq, 8)) return fail(K2Q_EINVAL, "k2q_fwht_quant_act_i8: xq must be 8-byte aligned");
  RowsParams p{};
  p.x = x; p.ldx = ldx; p.M = M; p.K = static_cast<int>(K > 0x7fffffff ? -1 : K);
  p.q8 = xq; p.s8 = sx;
  return run_rows<ROT_Q8>(p, x_dtype, "k2q_fwht_quant_act_i8", static_cast<cudaStream_t>(stream));
}

int k2q_quant_weight_i8(const void* w, int w_dtype, int64_t N, int64_t K, int64_t ldw, int8_t* q,
                        float* scale, void* stream) {
  if (N > 0 && (!q || !scale)) return fail(K2Q_EINVAL, "k2q_quant_weight_i8: output pointer is NULL");
  if (misaligned(q, 8)) return fail(K2Q_EINVAL, "k2q_quant_weight_i8: q must be 8-byte aligned");
  RowsParams p{};
  p.x = w; p.ldx = ldw; p.M = N; p.K = static_cast<int>(K > 0x7fffffff ? -1 : K);
  p.q8 = q; p.s8 = scale;
  return run_rows<ROT_Q8>(p, w_dtype, "k2q_quant_weight_i8", static_cast<cudaStream_t>(stream));
}

int k2q_quant_weight_i4(const void* w, int w_dtype, int64_t N, int64_t K, int64_t ldw, uint8_t* q4,
                        void* scale4_bf16, void* stream) {
  if (N > 0 && (!q4 || !scale4_bf16))
    return fail(K2Q_EINVAL, "k2q_quant_weight_i4: output pointer is NULL");
  if (misaligned(q4, 4)) return fail(K2Q_EINVAL, "k2q_quant_weight_i4: q4 must be 4-byte aligned");
  RowsParams p{};
  p.x = w; p.ldx = ldw; p.M = N; p.K = static_cast<int>(K > 0x7fffffff ? -1 : K);
  p.q4 = q4; p.s4 = static_cast<__nv_bfloat16*>(scale4_bf16);
  return run_rows<ROT_Q4>(p, w_dtype, "k2q_quant_weight_i4", static_cast<cudaStream_t>(stream));
}

int k2q_quant_rows_i8(const void* g, int g_dtype, int64_t M, int64_t N, int64_t ldg,
                      const float* colscale, int8_t* gq, float* sg, void* stream) {
  if (M > 0 && (!gq || !sg)) return fail(K2Q_EINVAL, "k2q_quant_rows_i8: output pointer is NULL");
  if (misaligned(gq, 8) || misaligned(colscale, 16))
    return fail(K2Q_EINVAL, "k2q_quant_rows_i8: gq must be 8-byte and colscale 16-byte aligned");
  RowsParams p{};
  p.x = g; p.ldx = ldg; p.M = M; p.K = static_cast<int>(N > 0x7fffffff ? -1 : N);
  p.colscale = colscale; p.q8 = gq; p.s8 = sg;
  return run_rows<Q8_ONLY>(p, g_dtype, "k2q_quant_rows_i8", static_cast<cudaStream_t>(stream));
}

int k2q_fwht_rows(const void* x, int x_dtype, int64_t M, int64_t K, int64_t ldx, void* y, int y_dtype,
                  int64_t ldy, void* stream) {
  if (M > 0 && !y) return fail(K2Q_EINVAL, "k2q_fwht_rows: output pointer is NULL");
  if (y_dtype != K2Q_BF16 && y_dtype != K2Q_F32)
    return fail(K2Q_EINVAL, "k2q_fwht_rows: unknown output dtype tag %d", y_dtype);
  const int esz = y_dtype == K2Q_BF16 ? 2 : 4;
  if (ldy < K || misaligned(y, 16) || ((ldy * esz) & 15))
    return fail(K2Q_EINVAL, "k2q_fwht_rows: output rows must be 16-byte aligned and ldy >= K");
  RowsParams p{};
  p.x = x; p.ldx = ldx; p.M = M; p.K = static_cast<int>(K > 0x7fffffff ? -1 : K);
  p.y = y; p.ldy = ldy; p.y_f32 = (y_dtype == K2Q_F32);
  return run_rows<ROT_ONLY>(p, x_dtype, "k2q_fwht_rows", static_cast<cudaStream_t>(stream));
}

}  // extern "C"
