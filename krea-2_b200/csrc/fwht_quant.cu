// K1 / K2 and friends: block-128 Walsh-Hadamard rotation of rows fused with quantisation.
//
// One kernel template covers
//   ROT_Q8   rotate + per-row int8        (activations K2, int8 weights K1)
//   ROT_Q4   rotate + per-(row,128-group) int4, packed two codes per byte (int4 weights K1)
//   ROT_ONLY rotate, write bf16 / f32     (de-rotation of dX, rotation of the LoRA A matrix)
//   Q8_ONLY  per-row int8 of g*colscale   (dY folded with the weight scales, backward)
//
// Work split: four neighbouring lanes own one 128-block, 32 consecutive elements each.  Butterfly
// stages h = 1..16 run inside the thread, stages h = 32 and h = 64 are lane exchanges (shfl.xor 1
// and 2): one shuffle per element, far below the shuffle unit's rate, and few enough registers
// for four resident CTAs per SM, so loads of one CTA overlap the arithmetic of the others.  Global
// traffic is coalesced: the threads of a row copy the row to shared memory with 128-bit loads
// (consecutive lanes, consecutive 16-byte chunks), each thread then reads its own 32 elements from
// a padded, bank-conflict-free layout; results go back the same way.  Stage order, the (a+b, a-b) pairing and the single
// final multiply are those of the CPU oracle, in fp32 with explicitly rounded operations, so
// codes and scales come out bit-identical.
//
// Quantisation  q = rint(v / s)  avoids a division per element: y = v * (1/s) is within 2e-5 of
// the true quotient, so unless y lies within 3e-5 of a half-integer rint(y) equals the oracle's
// rint(RN(v/s)); a group of 4 or 8 elements that contains such a one is redone with the exact IEEE division.
#include "k2q_common.cuh"
#include "rows_math.cuh"

namespace k2q {
namespace {

enum Mode : int { ROT_Q8 = 0, ROT_Q4 = 1, ROT_ONLY = 2, Q8_ONLY = 3 };
// Elementwise work of the step BEFORE the quantised Linear, applied to the row on its way in (ROT_Q8,
// bf16 input), with the reference's bf16 rounding points (every torch op on a bf16 tensor rounds):
//   PRO_SWIGLU   v = silu(g) * u                         (mmdit.py:178, the input of mlp.down)
//   PRO_GATE     v = attention * sigmoid(gate)           (mmdit.py:210, the input of attn.wo)
//   PRO_NORMMOD  v = (1 + scale_b) * rmsnorm(x) + shift_b  with weight (1 + norm.scale), fp32 statistics
//                (mmdit.py:158-160, 313-317, the input of wq / wk / wv / gate and of mlp.gate / mlp.up;
//                scale_b / shift_b = NULL: the plain norm of the text-fusion blocks, mmdit.py:237-246)
enum Prologue : int { PRO_NONE = 0, PRO_SWIGLU = 1, PRO_GATE = 2, PRO_NORMMOD = 3 };

constexpr int kMaxRowsPerCta = 32;

struct RowsParams {
  const void* x;
  int64_t ldx;
  int64_t M;
  int K;
  int tpr;                // threads per row = K / EPT
  int warp_stage_bytes;   // shared-memory staging per warp
  int rows_per_cta;
  int row_iters;          // consecutive row groups handled by one CTA
  const float* colscale;  // Q8_ONLY
  int8_t* q8;             // [M,K]
  float* s8;              // [M]
  uint8_t* q4;            // [M,K/2]
  __nv_bfloat16* s4;      // [M,K/128]
  void* y;                // ROT_ONLY output
  int64_t ldy;
  int y_f32;
  // prologues
  const __nv_bfloat16* x2;       // PRO_SWIGLU: u;  PRO_GATE: gate      [M, ldx2]
  int64_t ldx2;
  const float* normw;            // PRO_NORMMOD: norm.scale [K] (the weight is 1 + this)
  const __nv_bfloat16* mscale;   // [B, K] or NULL
  const __nv_bfloat16* mshift;   // [B, K] or NULL
  int64_t rows_per_batch;        // row -> b = row / rows_per_batch
  float eps;
};

__device__ __forceinline__ float bf16r(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

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

// the same from shared memory (plain loads)
__device__ __forceinline__ void load8s(const __nv_bfloat16* p, float* v) {
  const uint4 r = *reinterpret_cast<const uint4*>(p);
  const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    v[2 * i] = __uint_as_float(w[i] << 16);
    v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
  }
}
__device__ __forceinline__ void load8s(const float* p, float* v) {
  const float4 a = *reinterpret_cast<const float4*>(p);
  const float4 b = *(reinterpret_cast<const float4*>(p) + 1);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
  v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}

// Where a warp's 32 threads sit in the CTA's rows.  Threads are numbered row by row (tpr threads per
// row, 32 consecutive elements each), so a warp covers 1024 consecutive elements of one row, or, when
// tpr is not a multiple of 32, the end of one row and the start of the next.
struct WarpSpan {
  int t0;          // first thread of the warp
  bool uniform;    // all 32 threads in one row
  bool row_ok;     // uniform: that row exists
  int64_t row;     // uniform: global row
  int tr0;         // uniform: first thread's index inside the row
};

// Global <-> shared staging is private to a warp: lane l moves the 16-byte chunks l, l + 32, ... of the
// warp's contiguous 32 * PER chunks (coalesced 512-byte requests), thread-local chunks sit at
// [thread * (PER + 1) + j] (one pad chunk per thread: both phases are free of bank conflicts), and
// __syncwarp is the only synchronisation.  Results leave the same way.
template <int OC>
__device__ __forceinline__ void store_warp_coalesced(uint8_t* wreg, const WarpSpan& w, const RowsParams& p, int lane,
                                                     const uint4 (&mine)[OC], uint8_t* out, int64_t out_row_bytes,
                                                     int64_t row0) {
  __syncwarp();  // every lane has finished reading the input chunks
#pragma unroll
  for (int j = 0; j < OC; ++j) *reinterpret_cast<uint4*>(wreg + (lane * (OC + 1) + j) * 16) = mine[j];
  __syncwarp();
  if (w.uniform) {
    if (w.row_ok) {
      uint8_t* dst = out + w.row * out_row_bytes + static_cast<int64_t>(w.tr0) * (OC * 16);
#pragma unroll
      for (int i = 0; i < OC; ++i) {
        const int c = i * 32 + lane;
        *reinterpret_cast<uint4*>(dst + c * 16) = *reinterpret_cast<const uint4*>(wreg + (c + c / OC) * 16);
      }
    }
  } else {
#pragma unroll
    for (int i = 0; i < OC; ++i) {
      const int c = i * 32 + lane;
      const int t = w.t0 + c / OC, j = c % OC;
      const int rr = t / p.tpr, tt = t - rr * p.tpr;
      const int64_t grow = row0 + rr;
      if (rr < p.rows_per_cta && grow < p.M)
        *reinterpret_cast<uint4*>(out + grow * out_row_bytes + static_cast<int64_t>(tt) * (OC * 16) + j * 16) =
            *reinterpret_cast<const uint4*>(wreg + (c + c / OC) * 16);
    }
  }
}

template <typename InT, int MODE, int PRO = PRO_NONE>
__device__ __forceinline__ void rows_body(const RowsParams& p) {
  __shared__ int s_amax[3][kMaxRowsPerCta];   // row absmax slots, rotated over the row groups (see below)
  __shared__ float s_part[PRO == PRO_NORMMOD ? 128 : 1];   // sum of squares per 128-block of the CTA's rows   // by parity of the row group: a group never waits for the next one's reset

  pdl_wait();   // nothing to set up: an overlapped launch only hides the launch latency behind the kernel in front
  const int row_in_cta = threadIdx.x / p.tpr;
  const int tr = threadIdx.x - row_in_cta * p.tpr;   // half-block index inside the row
  const int k0 = tr * EPT;   // tpr is a multiple of 4, so a block's four lanes sit in one warp

  // Q8_ONLY: the thread's 32 column scales, the same for every row; requested first so that their
  // latency hides behind the first row copy
  float cs[MODE == Q8_ONLY ? EPT : 1];
  if (MODE == Q8_ONLY) {
    if (row_in_cta < p.rows_per_cta && p.colscale != nullptr) {
#pragma unroll
      for (int i = 0; i < EPT / 8; ++i) load8(p.colscale + k0 + 8 * i, cs + 8 * i);
    }
  }

  // ---- coalesced global -> shared copy of the warp's elements, then each thread takes its 32.
  // A CTA works through row_iters consecutive groups of rows_per_cta rows; the chunks of the next
  // group are requested (into registers) before the current group is computed.
  extern __shared__ __align__(16) uint8_t stage[];
  constexpr int CPT = EPT * sizeof(InT) / 16;                // 16-byte chunks per thread (4 or 8)
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  uint8_t* wreg = stage + warp * p.warp_stage_bytes;
  WarpSpan ws;
  ws.t0 = warp << 5;
  const int span_r0 = ws.t0 / p.tpr;
  ws.uniform = span_r0 == (ws.t0 + 31) / p.tpr;
  ws.tr0 = ws.t0 - span_r0 * p.tpr;

  uint4 tmp[CPT];
  auto fetch = [&](int64_t row0) {   // row0: first row of the group
    if (ws.uniform) {
      const int64_t grow = row0 + span_r0;
      const bool in = span_r0 < p.rows_per_cta && grow < p.M;
      const uint4* src = reinterpret_cast<const uint4*>(static_cast<const InT*>(p.x) + (in ? grow : 0) * p.ldx + ws.tr0 * EPT);
#pragma unroll
      for (int i = 0; i < CPT; ++i) tmp[i] = in ? __ldg(src + i * 32 + lane) : make_uint4(0u, 0u, 0u, 0u);
    } else {
#pragma unroll
      for (int i = 0; i < CPT; ++i) {
        const int c = i * 32 + lane;
        const int t = ws.t0 + c / CPT, j = c % CPT;
        const int rr = t / p.tpr, tt = t - rr * p.tpr;
        const int64_t grow = row0 + rr;
        const bool in = rr < p.rows_per_cta && grow < p.M;
        const InT* src = static_cast<const InT*>(p.x) + (in ? grow : 0) * p.ldx + tt * EPT + j * (16 / static_cast<int>(sizeof(InT)));
        tmp[i] = in ? __ldg(reinterpret_cast<const uint4*>(src)) : make_uint4(0u, 0u, 0u, 0u);
      }
    }
  };

  const int64_t first_row = static_cast<int64_t>(blockIdx.x) * p.row_iters * p.rows_per_cta;
  fetch(first_row);
  if (MODE == ROT_Q8 || MODE == Q8_ONLY) {
    for (int i = threadIdx.x; i < 3 * kMaxRowsPerCta; i += blockDim.x) (&s_amax[0][0])[i] = 0;
    __syncthreads();
  }
  for (int it = 0; it < p.row_iters; ++it) {
  const int64_t row0 = first_row + static_cast<int64_t>(it) * p.rows_per_cta;
  const int64_t row = row0 + row_in_cta;
  const bool ok = row_in_cta < p.rows_per_cta && row < p.M;
  ws.row = row0 + span_r0;
  ws.row_ok = span_r0 < p.rows_per_cta && ws.row < p.M;
  int* amax_s = s_amax[it % 3];

  __syncwarp();   // the previous group's results have left the staging region
#pragma unroll
  for (int i = 0; i < CPT; ++i) {
    const int c = i * 32 + lane;
    *reinterpret_cast<uint4*>(wreg + (c + c / CPT) * 16) = tmp[i];
  }
  __syncwarp();
  float v[EPT];   // rows that do not exist were staged as zeros
  {
    const uint8_t* mine = wreg + lane * (CPT + 1) * 16;
#pragma unroll
    for (int i = 0; i < EPT / 8; ++i) load8s(reinterpret_cast<const InT*>(mine) + 8 * i, v + 8 * i);
  }
  if (it + 1 < p.row_iters) fetch(row0 + p.rows_per_cta);   // in flight while this group is computed

  if (PRO == PRO_SWIGLU || PRO == PRO_GATE) {
    // the second operand: this thread's 32 elements straight from global memory (four 16-byte loads)
    float w2[EPT];
    const __nv_bfloat16* src2 = p.x2 + (ok ? row : 0) * p.ldx2 + k0;
#pragma unroll
    for (int i = 0; i < EPT / 8; ++i) load8(src2 + 8 * i, w2 + 8 * i);
#pragma unroll
    for (int i = 0; i < EPT; ++i) {
      if (PRO == PRO_SWIGLU) {
        const float sg = bf16r(__fdividef(v[i], 1.0f + __expf(-v[i])));     // F.silu on a bf16 tensor
        v[i] = bf16r(sg * w2[i]);
      } else {
        const float sig = bf16r(__fdividef(1.0f, 1.0f + __expf(-w2[i])));   // torch.sigmoid on a bf16 tensor
        v[i] = bf16r(v[i] * sig);
      }
    }
    if (!ok) {
#pragma unroll
      for (int i = 0; i < EPT; ++i) v[i] = 0.f;
    }
  }
  if (PRO == PRO_NORMMOD) {
    // fp32 mean of squares over the row, in a fixed order: 32 elements per thread, the four lanes of a
    // 128-block by shuffles, the row's blocks one after the other out of shared memory
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < EPT; ++i) ss = __fmaf_rn(v[i], v[i], ss);
    ss += __shfl_xor_sync(0xffffffffu, ss, 1);
    ss += __shfl_xor_sync(0xffffffffu, ss, 2);
    const int blocks_per_row = p.tpr >> 2;
    __syncthreads();   // the previous group's partial sums have been read
    if ((tr & 3) == 0 && row_in_cta < p.rows_per_cta) s_part[row_in_cta * blocks_per_row + (tr >> 2)] = ss;
    __syncthreads();
    float tot = 0.f;
    if (row_in_cta < p.rows_per_cta) {
      for (int j = 0; j < blocks_per_row; ++j) tot += s_part[row_in_cta * blocks_per_row + j];
    }
    const float rstd = rsqrtf(tot / static_cast<float>(p.K) + p.eps);
    const int64_t b = (ok ? row : 0) / p.rows_per_batch;
    float wn[EPT];
#pragma unroll
    for (int i = 0; i < EPT / 8; ++i) load8(p.normw + k0 + 8 * i, wn + 8 * i);
#pragma unroll
    for (int i = 0; i < EPT; ++i) v[i] = bf16r(__fmul_rn(__fmul_rn(v[i], rstd), wn[i] + 1.0f));   // RMSNorm.forward: .to(bf16)
    if (p.mscale != nullptr) {
      float sc[EPT];
#pragma unroll
      for (int i = 0; i < EPT / 8; ++i) load8(p.mscale + b * p.K + k0 + 8 * i, sc + 8 * i);
#pragma unroll
      for (int i = 0; i < EPT; ++i) v[i] = bf16r(bf16r(1.0f + sc[i]) * v[i]);                 // (1 + scale) * norm, bf16 ops
    }
    if (p.mshift != nullptr) {
      float sh[EPT];
#pragma unroll
      for (int i = 0; i < EPT / 8; ++i) load8(p.mshift + b * p.K + k0 + 8 * i, sh + 8 * i);
#pragma unroll
      for (int i = 0; i < EPT; ++i) v[i] = bf16r(v[i] + sh[i]);
    }
    if (!ok) {
#pragma unroll
      for (int i = 0; i < EPT; ++i) v[i] = 0.f;
    }
  }

  if (MODE == Q8_ONLY) {
    if (ok && p.colscale != nullptr) {
#pragma unroll
      for (int i = 0; i < EPT; ++i) v[i] = __fmul_rn(v[i], cs[i]);
    }
  } else {
    fwht128_thread(v, tr);
  }

  if (MODE == ROT_ONLY) {
    if (p.y_f32) {
      uint4 o[EPT / 4];
#pragma unroll
      for (int i = 0; i < EPT / 4; ++i)
        o[i] = make_uint4(__float_as_uint(v[4 * i]), __float_as_uint(v[4 * i + 1]), __float_as_uint(v[4 * i + 2]),
                          __float_as_uint(v[4 * i + 3]));
      store_warp_coalesced<EPT / 4>(wreg, ws, p, lane, o, static_cast<uint8_t*>(p.y), p.ldy * 4, row0);
    } else {
      uint4 o[EPT / 8];
#pragma unroll
      for (int i = 0; i < EPT / 8; ++i) {
        o[i].x = pack_bf16x2(v[8 * i], v[8 * i + 1]);
        o[i].y = pack_bf16x2(v[8 * i + 2], v[8 * i + 3]);
        o[i].z = pack_bf16x2(v[8 * i + 4], v[8 * i + 5]);
        o[i].w = pack_bf16x2(v[8 * i + 6], v[8 * i + 7]);
      }
      store_warp_coalesced<EPT / 8>(wreg, ws, p, lane, o, static_cast<uint8_t*>(p.y), p.ldy * 2, row0);
    }
    continue;
  }

  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < EPT; ++i) amax = fmaxf(amax, fabsf(v[i]));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));  // the 128-block's absmax

  if (MODE == ROT_Q4) {
    const float s = __fdiv_rn(fmaxf(amax, 1e-8f), 7.0f);
    const float inv = __frcp_rn(s);
    uint4 o[1];
    {
      uint32_t words[EPT / 8];
#pragma unroll
      for (int w = 0; w < EPT / 8; ++w) {
        uint32_t code[8];
        quant_codes<8>(v + 8 * w, s, inv, code);
        uint32_t word = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) word |= (code[i] & 0xFu) << (4 * i);
        words[w] = word;
      }
      o[0] = make_uint4(words[0], words[1], words[2], words[3]);
    }
    if (ok && (tr & 3) == 0) p.s4[row * (p.K >> 7) + (tr >> 2)] = __float2bfloat16_rn(s);
    store_warp_coalesced<1>(wreg, ws, p, lane, o, p.q4, p.K >> 1, row0);
    continue;
  }

  // ROT_Q8 / Q8_ONLY: absmax of the whole row through shared memory (floats >= 0 order as ints).  One
  // barrier per row group: group `it` collects in slot it % 3 while the next group's slot is cleared --
  // its last readers (group it - 2) are behind the barrier of group it - 1, which every thread here has
  // passed, and its next writers come after this group's barrier.
  if (ok && (tr & 3) == 0) atomicMax(&amax_s[row_in_cta], __float_as_int(amax));
  if (threadIdx.x < kMaxRowsPerCta) s_amax[(it + 1) % 3][threadIdx.x] = 0;
  __syncthreads();
  const float s = __fdiv_rn(fmaxf(__int_as_float(amax_s[ok ? row_in_cta : 0]), 1e-8f), 127.0f);
  const float inv = __frcp_rn(s);
  if (ok && tr == 0) p.s8[row] = s;
  uint4 o[EPT / 16];
  {
    uint32_t words[EPT / 4];
    quant_row32_i8(v, s, inv, words);
#pragma unroll
    for (int w4 = 0; w4 < EPT / 16; ++w4) o[w4] = make_uint4(words[4 * w4], words[4 * w4 + 1], words[4 * w4 + 2], words[4 * w4 + 3]);
  }
  store_warp_coalesced<EPT / 16>(wreg, ws, p, lane, o, reinterpret_cast<uint8_t*>(p.q8), p.K, row0);
  }   // row groups
}

// Register budgets (blocks of up to 512 threads): 80 keeps two 384-thread CTAs (K = 12288) on an SM,
// which the rotating modes need more than registers; the dY quantiser holds its 32 column scales
// across the row groups and runs faster with the full 128.
template <typename InT, int MODE>
__global__ void __maxnreg__(80) rows_kernel(const RowsParams p) { rows_body<InT, MODE>(p); }
template <typename InT, int MODE>
__global__ void __maxnreg__(128) rows_kernel_wide(const RowsParams p) { rows_body<InT, MODE>(p); }
template <int PRO>
__global__ void __maxnreg__(128) rows_kernel_pro(const RowsParams p) { rows_body<__nv_bfloat16, ROT_Q8, PRO>(p); }

template <typename InT, int MODE, int PRO = PRO_NONE>
int launch_rows(RowsParams& p, cudaStream_t stream) {
  p.tpr = p.K / EPT;
  int rows = 128 / p.tpr;   // small CTAs: the CTA-wide barriers of the staging phases cost less (measured)
  if (rows < 1) rows = 1;
  if (rows > kMaxRowsPerCta) rows = kMaxRowsPerCta;
  p.rows_per_cta = rows;
  const int threads = (rows * p.tpr + 31) / 32 * 32;
  const int64_t groups = (p.M + rows - 1) / rows;
  // several row groups per CTA once every SM has 8 CTAs: two for the rotating modes on short rows, four on long
  // rows and for the dY quantiser, which re-uses its column scales (all measured)
  const int sms = sm_count() > 0 ? sm_count() : 148;
  const int64_t iters = groups / (static_cast<int64_t>(sms) * 8), cap = (MODE == Q8_ONLY || p.K >= 8192) ? 4 : 2;
  p.row_iters = iters > cap ? static_cast<int>(cap) : (iters < 1 ? 1 : static_cast<int>(iters));
  const int64_t grid64 = (groups + p.row_iters - 1) / p.row_iters;
  if (grid64 > 0x7fffffffLL) return fail(K2Q_EINVAL, "too many rows (%lld)", (long long)p.M);
  constexpr int CPT = EPT * sizeof(InT) / 16;                  // 16-byte chunks per thread coming in
  int out_chunks = 2;                                          // int8 codes going out
  if (MODE == ROT_Q4) out_chunks = 1;
  if (MODE == ROT_ONLY) out_chunks = p.y_f32 ? EPT / 4 : EPT / 8;
  const int chunks = CPT > out_chunks ? CPT : out_chunks;      // the staging area serves both directions
  p.warp_stage_bytes = 32 * (chunks + 1) * 16;
  const size_t smem = static_cast<size_t>(threads / 32) * p.warp_stage_bytes;
  auto kern = PRO != PRO_NONE ? rows_kernel_pro<PRO>
                              : (MODE == Q8_ONLY ? rows_kernel_wide<InT, MODE> : rows_kernel<InT, MODE>);
  if (smem > 48 * 1024) {
    if (int rc = check_cuda(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem),
                            "cudaFuncSetAttribute(rows_kernel)"))
      return rc;
  }
  return launch_overlapped(kern, static_cast<unsigned>(grid64), static_cast<unsigned>(threads), smem, stream, 1,
                           "rows_kernel launch", p);
}

bool misaligned(const void* ptr, unsigned a) { return (reinterpret_cast<uintptr_t>(ptr) & (a - 1)) != 0; }

template <int MODE>
int run_rows(RowsParams p, int dtype, const char* name, cudaStream_t stream) {
  if (int rc = check_device_arch()) return rc;
  if (p.M < 0 || p.K <= 0) return fail(K2Q_EINVAL, "%s: bad shape M=%lld K=%d", name, (long long)p.M, p.K);
  if (p.K % 128 != 0) return fail(K2Q_EINVAL, "%s: K=%d is not a multiple of 128", name, p.K);
  if (p.K > 512 * EPT) return fail(K2Q_EINVAL, "%s: K=%d exceeds the supported maximum %d", name, p.K, 512 * EPT);
  if (dtype != K2Q_BF16 && dtype != K2Q_F32) return fail(K2Q_EINVAL, "%s: unknown dtype tag %d", name, dtype);
  if (p.M == 0) return K2Q_OK;
  if (!p.x) return fail(K2Q_EINVAL, "%s: input pointer is NULL", name);
  const int esz = dtype == K2Q_BF16 ? 2 : 4;
  if (p.ldx < p.K) return fail(K2Q_EINVAL, "%s: leading dimension %lld < K=%d", name, (long long)p.ldx, p.K);
  if (misaligned(p.x, 16) || ((p.ldx * esz) & 15))
    return fail(K2Q_EINVAL, "%s: input rows must be 16-byte aligned (ptr %p, ld %lld)", name, p.x,
                (long long)p.ldx);
  if (dtype == K2Q_BF16) return launch_rows<__nv_bfloat16, MODE>(p, stream);
  return launch_rows<float, MODE>(p, stream);
}

template <int PRO>
int run_prologue(RowsParams p, const char* name, cudaStream_t stream) {
  if (int rc = check_device_arch()) return rc;
  if (p.M < 0 || p.K <= 0) return fail(K2Q_EINVAL, "%s: bad shape M=%lld K=%d", name, (long long)p.M, p.K);
  if (p.K % 128 != 0) return fail(K2Q_EINVAL, "%s: K=%d is not a multiple of 128", name, p.K);
  if (p.K > 512 * EPT) return fail(K2Q_EINVAL, "%s: K=%d exceeds the supported maximum %d", name, p.K, 512 * EPT);
  if (p.M == 0) return K2Q_OK;
  if (!p.x || !p.q8 || !p.s8) return fail(K2Q_EINVAL, "%s: NULL operand", name);
  if (p.ldx < p.K || misaligned(p.x, 16) || ((p.ldx * 2) & 15) || misaligned(p.q8, 16))
    return fail(K2Q_EINVAL, "%s: rows must be 16-byte aligned with ld >= K", name);
  if (PRO == PRO_SWIGLU || PRO == PRO_GATE) {
    if (!p.x2 || p.ldx2 < p.K || misaligned(p.x2, 16) || ((p.ldx2 * 2) & 15))
      return fail(K2Q_EINVAL, "%s: the second operand must be 16-byte aligned with ld >= K", name);
  }
  if (PRO == PRO_NORMMOD) {
    if (!p.normw || misaligned(p.normw, 16) || misaligned(p.mscale, 16) || misaligned(p.mshift, 16))
      return fail(K2Q_EINVAL, "%s: norm weight / modulation vectors must be non-NULL (weight) and 16-byte aligned", name);
    if (p.rows_per_batch <= 0) return fail(K2Q_EINVAL, "%s: rows_per_batch must be positive", name);
  }
  return launch_rows<__nv_bfloat16, ROT_Q8, PRO>(p, stream);
}

}  // namespace
}  // namespace k2q

using namespace k2q;

extern "C" {

int k2q_swiglu_fwht_quant(const void* g_bf16, int64_t ldg, const void* u_bf16, int64_t ldu, int64_t M, int64_t K,
                          int8_t* xq, float* sx, void* stream) {
  RowsParams p{};
  p.x = g_bf16; p.ldx = ldg; p.x2 = static_cast<const __nv_bfloat16*>(u_bf16); p.ldx2 = ldu;
  p.M = M; p.K = static_cast<int>(K > 0x7fffffff ? -1 : K); p.q8 = xq; p.s8 = sx;
  return run_prologue<PRO_SWIGLU>(p, "k2q_swiglu_fwht_quant", static_cast<cudaStream_t>(stream));
}

int k2q_gate_fwht_quant(const void* attn_bf16, int64_t lda, const void* gate_bf16, int64_t ldg, int64_t M, int64_t K,
                        int8_t* xq, float* sx, void* stream) {
  RowsParams p{};
  p.x = attn_bf16; p.ldx = lda; p.x2 = static_cast<const __nv_bfloat16*>(gate_bf16); p.ldx2 = ldg;
  p.M = M; p.K = static_cast<int>(K > 0x7fffffff ? -1 : K); p.q8 = xq; p.s8 = sx;
  return run_prologue<PRO_GATE>(p, "k2q_gate_fwht_quant", static_cast<cudaStream_t>(stream));
}

int k2q_norm_mod_fwht_quant(const void* x_bf16, int64_t ldx, int64_t M, int64_t K, const float* norm_scale,
                            const void* mod_scale_bf16, const void* mod_shift_bf16, int64_t rows_per_batch,
                            float eps, int8_t* xq, float* sx, void* stream) {
  RowsParams p{};
  p.x = x_bf16; p.ldx = ldx; p.M = M; p.K = static_cast<int>(K > 0x7fffffff ? -1 : K); p.q8 = xq; p.s8 = sx;
  p.normw = norm_scale; p.mscale = static_cast<const __nv_bfloat16*>(mod_scale_bf16);
  p.mshift = static_cast<const __nv_bfloat16*>(mod_shift_bf16); p.rows_per_batch = rows_per_batch; p.eps = eps;
  return run_prologue<PRO_NORMMOD>(p, "k2q_norm_mod_fwht_quant", static_cast<cudaStream_t>(stream));
}

int k2q_fwht_quant_act_i8(const void* x, int x_dtype, int64_t M, int64_t K, int64_t ldx, int8_t* xq,
                          float* sx, void* stream) {
  if (M > 0 && (!xq || !sx)) return fail(K2Q_EINVAL, "k2q_fwht_quant_act_i8: output pointer is NULL");
  if (misaligned(xq, 16)) return fail(K2Q_EINVAL, "k2q_fwht_quant_act_i8: xq must be 16-byte aligned");
  RowsParams p{};
  p.x = x; p.ldx = ldx; p.M = M; p.K = static_cast<int>(K > 0x7fffffff ? -1 : K);
  p.q8 = xq; p.s8 = sx;
  return run_rows<ROT_Q8>(p, x_dtype, "k2q_fwht_quant_act_i8", static_cast<cudaStream_t>(stream));
}

int k2q_quant_weight_i8(const void* w, int w_dtype, int64_t N, int64_t K, int64_t ldw, int8_t* q,
                        float* scale, void* stream) {
  if (N > 0 && (!q || !scale)) return fail(K2Q_EINVAL, "k2q_quant_weight_i8: output pointer is NULL");
  if (misaligned(q, 16)) return fail(K2Q_EINVAL, "k2q_quant_weight_i8: q must be 16-byte aligned");
  RowsParams p{};
  p.x = w; p.ldx = ldw; p.M = N; p.K = static_cast<int>(K > 0x7fffffff ? -1 : K);
  p.q8 = q; p.s8 = scale;
  return run_rows<ROT_Q8>(p, w_dtype, "k2q_quant_weight_i8", static_cast<cudaStream_t>(stream));
}

int k2q_quant_weight_i4(const void* w, int w_dtype, int64_t N, int64_t K, int64_t ldw, uint8_t* q4,
                        void* scale4_bf16, void* stream) {
  if (N > 0 && (!q4 || !scale4_bf16))
    return fail(K2Q_EINVAL, "k2q_quant_weight_i4: output pointer is NULL");
  if (misaligned(q4, 16)) return fail(K2Q_EINVAL, "k2q_quant_weight_i4: q4 must be 16-byte aligned");
  RowsParams p{};
  p.x = w; p.ldx = ldw; p.M = N; p.K = static_cast<int>(K > 0x7fffffff ? -1 : K);
  p.q4 = q4; p.s4 = static_cast<__nv_bfloat16*>(scale4_bf16);
  return run_rows<ROT_Q4>(p, w_dtype, "k2q_quant_weight_i4", static_cast<cudaStream_t>(stream));
}

int k2q_quant_rows_i8(const void* g, int g_dtype, int64_t M, int64_t N, int64_t ldg,
                      const float* colscale, int8_t* gq, float* sg, void* stream) {
  if (M > 0 && (!gq || !sg)) return fail(K2Q_EINVAL, "k2q_quant_rows_i8: output pointer is NULL");
  if (misaligned(gq, 16) || misaligned(colscale, 16))
    return fail(K2Q_EINVAL, "k2q_quant_rows_i8: gq and colscale must be 16-byte aligned");
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
