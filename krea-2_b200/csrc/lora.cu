// K5 / K7: the skinny LoRA GEMMs, plus the one-off int8 transpose.
//
// These are memory-bound (one pass over a [T, K] bf16 matrix against a rank<=64 factor), so they
// use warp-level mma.sync m16n8k16 bf16 with fp32 accumulation rather than tcgen05.  The fp32
// factor is split into bf16 high and low parts (two MMAs) so that the result carries ~16 bits
// of the factor's mantissa, better than the TF32 product the reference trainer runs
// (lora.py:47 under runtime.tf32).  All reductions run in a fixed order: results are
// run-to-run identical, which gradient-checkpoint recomputation relies on.
#include <mutex>

#include "k2q_common.cuh"

namespace k2q {
namespace {

// ------------------------------------------------------------------------------------------
// K5: out[M, r] = scale * X[M, K] . A[r, K]^T
// CTA = 8 warps; the CTA owns MT*16 rows and one K range, the warps split that range in 32-wide
// chunks (warp w takes chunks w, w+8, ...).  Every CTA streams the factor's K range from L2, so
// rows per CTA (MT*16) set the L2 traffic; when that leaves fewer CTAs than SMs, the CTAs of a
// thread-block cluster split K between them and rank 0 adds the partial sums out of the others'
// shared memory, in rank order (no workspace, no atomics: results are run-to-run identical).
// Within a chunk a lane reads 16 contiguous bytes of a row; the MMA's contraction index is a
// permutation of k, applied identically to both operands.
// Two kernels share this scheme.  lora_down_kernel (first below) stages through registers: all
// loads of a chunk are unconditional (addresses clamped, values zeroed by selects) and the next
// chunk is fetched into a second register set before the current one is multiplied.  It accepts a
// factor of any stride and is the fallback.  lora_down_async_kernel stages through shared
// memory with cp.async and serves the usual unit-stride factor.
// ------------------------------------------------------------------------------------------
struct DownParams {
  const __nv_bfloat16* x;
  int64_t ldx;
  int64_t M;
  int K;
  const float* a;
  int64_t a_rs, a_cs;
  int r;
  float scale;
  float* out;
  int64_t ldo;
};

constexpr int kDownWarps = 8;

template <int MT, int NT>
__global__ void __launch_bounds__(kDownWarps * 32) lora_down_kernel(const DownParams p) {
  extern __shared__ float red[];  // [MT*16][NT*8]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, q = lane & 3;
  const uint32_t ksplit = cluster_nctarank(), krank = cluster_ctarank();
  const int64_t m0 = static_cast<int64_t>(blockIdx.x / ksplit) * (MT * 16);

  float acc[MT][NT][4];
#pragma unroll
  for (int i = 0; i < MT; ++i)
#pragma unroll
    for (int t = 0; t < NT; ++t)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[i][t][e] = 0.f;

  const int all_chunks = (p.K + 31) >> 5;
  const int per_rank = (all_chunks + static_cast<int>(ksplit) - 1) / static_cast<int>(ksplit);
  const int chunk_lo = static_cast<int>(krank) * per_rank;
  const int nchunks = chunk_lo + per_rank < all_chunks ? chunk_lo + per_rank : all_chunks;   // end of this CTA's range

  // rows of X (clamped: rows past M only feed accumulators that are never written) and of the factor
  const __nv_bfloat16* xrow[MT][2];
#pragma unroll
  for (int i = 0; i < MT; ++i)
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      int64_t row = m0 + i * 16 + g + 8 * h;
      if (row > p.M - 1) row = p.M - 1;
      xrow[i][h] = p.x + row * p.ldx;
    }
  const float* arow[NT];
  bool j_ok[NT];
#pragma unroll
  for (int t = 0; t < NT; ++t) {
    const int j = t * 8 + g;
    j_ok[t] = j < p.r;
    arow[t] = p.a + (j_ok[t] ? j : 0) * p.a_rs;
  }

  auto fetch = [&](int c, uint4 (&xa)[MT][2], float (&av)[NT][8]) {
    const int k0 = c * 32 + q * 8;
    const bool k_ok = k0 < p.K;   // K is a multiple of 8: a lane's 8-element piece is all in or all out
    const int kc = k_ok ? k0 : 0;
#pragma unroll
    for (int i = 0; i < MT; ++i)
#pragma unroll
      for (int h = 0; h < 2; ++h) xa[i][h] = __ldg(reinterpret_cast<const uint4*>(xrow[i][h] + kc));
#pragma unroll
    for (int t = 0; t < NT; ++t) {
#pragma unroll
      for (int e = 0; e < 8; ++e) av[t][e] = __ldg(arow[t] + static_cast<int64_t>(kc + e) * p.a_cs);
    }
    if (!k_ok) {   // K tail: this lane's piece lies past the end
#pragma unroll
      for (int i = 0; i < MT; ++i)
#pragma unroll
        for (int h = 0; h < 2; ++h) xa[i][h] = make_uint4(0u, 0u, 0u, 0u);
    }
#pragma unroll
    for (int t = 0; t < NT; ++t)
#pragma unroll
      for (int e = 0; e < 8; ++e) av[t][e] = (k_ok && j_ok[t]) ? av[t][e] : 0.f;
  };

  auto multiply = [&](const uint4 (&xa)[MT][2], const float (&av)[NT][8]) {
#pragma unroll
    for (int t = 0; t < NT; ++t) {
      uint32_t bh[4], bl[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) split2(av[t][2 * e], av[t][2 * e + 1], bh[e], bl[e]);
#pragma unroll
      for (int i = 0; i < MT; ++i) {
        // first k16: elements (0,1) and (2,3) of each 8-wide piece; second k16: (4,5) and (6,7)
        const uint32_t a1[4] = {xa[i][0].x, xa[i][1].x, xa[i][0].y, xa[i][1].y};
        const uint32_t a2[4] = {xa[i][0].z, xa[i][1].z, xa[i][0].w, xa[i][1].w};
        mma_bf16_16816(acc[i][t], a1, bh[0], bh[1]);
        mma_bf16_16816(acc[i][t], a1, bl[0], bl[1]);
        mma_bf16_16816(acc[i][t], a2, bh[2], bh[3]);
        mma_bf16_16816(acc[i][t], a2, bl[2], bl[3]);
      }
    }
  };

  uint4 xa0[MT][2], xa1[MT][2];
  float av0[NT][8], av1[NT][8];
  if (chunk_lo + warp < nchunks) fetch(chunk_lo + warp, xa0, av0);
  for (int c = chunk_lo + warp; c < nchunks; c += 2 * kDownWarps) {
    const bool more1 = c + kDownWarps < nchunks;
    if (more1) fetch(c + kDownWarps, xa1, av1);
    multiply(xa0, av0);
    if (c + 2 * kDownWarps < nchunks) fetch(c + 2 * kDownWarps, xa0, av0);
    if (more1) multiply(xa1, av1);
  }

  // fixed-order reduction over the warps
  constexpr int RP = NT * 8;
  for (int w = 0; w < kDownWarps; ++w) {
    if (warp == w) {
#pragma unroll
      for (int i = 0; i < MT; ++i)
#pragma unroll
        for (int t = 0; t < NT; ++t)
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int row = i * 16 + g + 8 * (e >> 1);
            const int col = t * 8 + 2 * q + (e & 1);
            float* dst = red + row * RP + col;
            *dst = (w == 0) ? acc[i][t][e] : *dst + acc[i][t][e];
          }
    }
    __syncthreads();
  }
  if (ksplit > 1) cluster_sync_all();   // every rank's partial sums are in its shared memory
  if (krank == 0) {
    const uint32_t red_addr = smem_u32(red);
    for (int idx = threadIdx.x; idx < MT * 16 * RP; idx += kDownWarps * 32) {
      const int row = idx / RP, col = idx % RP;
      float sum = red[idx];
      for (uint32_t k = 1; k < ksplit; ++k) sum += ld_cluster_f32(map_to_cta(red_addr + 4u * idx, k));
      if (m0 + row < p.M && col < p.r) p.out[(m0 + row) * p.ldo + col] = p.scale * sum;
    }
  }
  if (ksplit > 1) cluster_sync_all();   // nobody leaves while rank 0 still reads its shared memory
}

// The same product with the loads taken off the register file: every lane copies the 16-byte
// pieces it will itself consume (8 of X, 2 per n8 tile of the factor) into a lane-private slot of
// shared memory with cp.async, two (or one) chunks ahead.  A lane only ever reads what it copied, so
// cp.async.wait_group is the only synchronisation, the slots [piece][lane] are free of bank
// conflicts, and a warp keeps up to two chunks (16 KB) in flight at a cost of no registers.
// Needs a unit-stride, 16-byte aligned factor.
__host__ __device__ constexpr int down_stages(int mt, int nt) { return 2 * mt + 2 * nt <= 16 ? 3 : 2; }   // ring <= 192 KB per CTA

template <int MT, int NT>
__global__ void __launch_bounds__(kDownWarps * 32) lora_down_async_kernel(const DownParams p) {
  extern __shared__ __align__(16) uint8_t dsm[];
  constexpr int kDownStages = down_stages(MT, NT);
  constexpr int PIECES = 2 * MT + 2 * NT;                 // 16-byte pieces per lane per chunk
  constexpr int STAGE_BYTES = PIECES * 32 * 16;           // per warp
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, q = lane & 3;
  const uint32_t ksplit = cluster_nctarank(), krank = cluster_ctarank();
  const int64_t m0 = static_cast<int64_t>(blockIdx.x / ksplit) * (MT * 16);
  float* red = reinterpret_cast<float*>(dsm);             // [MT*16][NT*8], first in the buffer
  const uint32_t ring = smem_u32(dsm) + MT * 16 * NT * 8 * 4 + warp * (kDownStages * STAGE_BYTES) + lane * 16;

  float acc[MT][NT][4];
#pragma unroll
  for (int i = 0; i < MT; ++i)
#pragma unroll
    for (int t = 0; t < NT; ++t)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[i][t][e] = 0.f;

  const int all_chunks = (p.K + 31) >> 5;
  const int per_rank = (all_chunks + static_cast<int>(ksplit) - 1) / static_cast<int>(ksplit);
  const int chunk_lo = static_cast<int>(krank) * per_rank;
  const int chunk_hi = chunk_lo + per_rank < all_chunks ? chunk_lo + per_rank : all_chunks;

  const __nv_bfloat16* xrow[MT][2];
#pragma unroll
  for (int i = 0; i < MT; ++i)
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      int64_t row = m0 + i * 16 + g + 8 * h;
      if (row > p.M - 1) row = p.M - 1;   // rows past M only feed accumulators that are never written
      xrow[i][h] = p.x + row * p.ldx;
    }
  const float* arow[NT];
  bool j_ok[NT];
#pragma unroll
  for (int t = 0; t < NT; ++t) {
    const int j = t * 8 + g;
    j_ok[t] = j < p.r;
    arow[t] = p.a + (j_ok[t] ? j : 0) * p.a_rs;
  }

  auto issue = [&](int c, int stage) {
    if (c < chunk_hi) {
      const int k0 = c * 32 + q * 8;
      const bool k_ok = k0 < p.K;   // K is a multiple of 8: a lane's 8-element piece is all in or all out
      const int kc = k_ok ? k0 : 0;
      const uint32_t dst = ring + stage * STAGE_BYTES;
#pragma unroll
      for (int i = 0; i < MT; ++i)
#pragma unroll
        for (int h = 0; h < 2; ++h) cp_async16(dst + (2 * i + h) * 512, xrow[i][h] + kc, k_ok ? 16u : 0u);
#pragma unroll
      for (int t = 0; t < NT; ++t) {
        const uint32_t nbytes = (k_ok && j_ok[t]) ? 16u : 0u;
        cp_async16(dst + (2 * MT + 2 * t) * 512, arow[t] + kc, nbytes);
        cp_async16(dst + (2 * MT + 2 * t + 1) * 512, arow[t] + kc + 4, nbytes);
      }
    }
    cp_async_commit();   // one group per call, empty past the end, so the wait counts stay uniform
  };

  int c = chunk_lo + warp;
#pragma unroll
  for (int s = 0; s < kDownStages - 1; ++s) issue(c + s * kDownWarps, s);
  int stage = 0;
  for (; c < chunk_hi; c += kDownWarps) {
    {
      int nstage = stage + kDownStages - 1;
      if (nstage >= kDownStages) nstage -= kDownStages;
      issue(c + (kDownStages - 1) * kDownWarps, nstage);
    }
    cp_async_wait<kDownStages - 1>();   // this chunk's group has landed (the lane reads only its own pieces)
    const uint32_t src = ring + stage * STAGE_BYTES;
    uint4 xa[MT][2];
#pragma unroll
    for (int i = 0; i < MT; ++i)
#pragma unroll
      for (int h = 0; h < 2; ++h)
        asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                     : "=r"(xa[i][h].x), "=r"(xa[i][h].y), "=r"(xa[i][h].z), "=r"(xa[i][h].w)
                     : "r"(src + (2 * i + h) * 512));
    uint32_t bh[NT][4], bl[NT][4];
#pragma unroll
    for (int t = 0; t < NT; ++t) {
      float av[8];
      asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];"
                   : "=f"(av[0]), "=f"(av[1]), "=f"(av[2]), "=f"(av[3])
                   : "r"(src + (2 * MT + 2 * t) * 512));
      asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];"
                   : "=f"(av[4]), "=f"(av[5]), "=f"(av[6]), "=f"(av[7])
                   : "r"(src + (2 * MT + 2 * t + 1) * 512));
#pragma unroll
      for (int e = 0; e < 4; ++e) split2(av[2 * e], av[2 * e + 1], bh[t][e], bl[t][e]);
    }
    // four passes over all MT x NT accumulators: consecutive MMAs never touch the same accumulator.
    // first k16: elements (0,1) and (2,3) of each 8-wide piece; second k16: (4,5) and (6,7)
#pragma unroll
    for (int pass = 0; pass < 4; ++pass) {
#pragma unroll
      for (int t = 0; t < NT; ++t) {
#pragma unroll
        for (int i = 0; i < MT; ++i) {
          const uint32_t a1[4] = {xa[i][0].x, xa[i][1].x, xa[i][0].y, xa[i][1].y};
          const uint32_t a2[4] = {xa[i][0].z, xa[i][1].z, xa[i][0].w, xa[i][1].w};
          if (pass == 0) mma_bf16_16816(acc[i][t], a1, bh[t][0], bh[t][1]);
          if (pass == 1) mma_bf16_16816(acc[i][t], a2, bh[t][2], bh[t][3]);
          if (pass == 2) mma_bf16_16816(acc[i][t], a1, bl[t][0], bl[t][1]);
          if (pass == 3) mma_bf16_16816(acc[i][t], a2, bl[t][2], bl[t][3]);
        }
      }
    }
    if (++stage == kDownStages) stage = 0;
  }
  cp_async_wait<0>();
  __syncthreads();   // every warp is done with its ring: the memory is reused for the reduction

  // Reduction in a fixed order.  Every warp parks its accumulators in its own slab, laid out
  // [value index][lane] (conflict-free to write and to read back); each thread then adds the
  // eight slabs for its share of the tile, and rank 0 adds the other K ranges of the cluster.
  constexpr int VALS = MT * NT * 4;                       // accumulator values per lane
  float* slab = reinterpret_cast<float*>(dsm + MT * 16 * NT * 8 * 4);
#pragma unroll
  for (int i = 0; i < MT; ++i)
#pragma unroll
    for (int t = 0; t < NT; ++t)
#pragma unroll
      for (int e = 0; e < 4; ++e) slab[(warp * VALS + (i * NT + t) * 4 + e) * 32 + lane] = acc[i][t][e];
  __syncthreads();
  constexpr int PER = VALS * 32 / (kDownWarps * 32);      // tile values per thread
  float part[PER];
#pragma unroll
  for (int k = 0; k < PER; ++k) {
    const int pos = (k * kDownWarps + warp) * 32 + lane;  // [value index][lane], value index = k * 8 + warp
    float sum = slab[pos];
#pragma unroll
    for (int w = 1; w < kDownWarps; ++w) sum += slab[w * VALS * 32 + pos];
    part[k] = sum;
    red[pos] = sum;
  }
  if (ksplit > 1) {
    cluster_sync_all();   // every rank's partial tile is in its `red`
    if (krank == 0) {
      const uint32_t red_addr = smem_u32(red);
#pragma unroll
      for (int k = 0; k < PER; ++k) {
        const int pos = (k * kDownWarps + warp) * 32 + lane;
        for (uint32_t kr = 1; kr < ksplit; ++kr) part[k] += ld_cluster_f32(map_to_cta(red_addr + 4u * pos, kr));
      }
    }
  }
  if (krank == 0) {
#pragma unroll
    for (int k = 0; k < PER; ++k) {
      const int idx = k * kDownWarps + warp;              // (i * NT + t) * 4 + e
      const int e = idx & 3, t = (idx >> 2) % NT, i = (idx >> 2) / NT;
      const int row = i * 16 + g + 8 * (e >> 1), col = t * 8 + 2 * q + (e & 1);
      if (m0 + row < p.M && col < p.r) p.out[(m0 + row) * p.ldo + col] = p.scale * part[k];
    }
  }
  if (ksplit > 1) cluster_sync_all();   // nobody leaves while rank 0 still reads its shared memory
}

// ------------------------------------------------------------------------------------------
// K7: out[r, C] = scale * P[T, r]^T . Q[T, C]      (split over T, partials reduced in order)
// CTA = 4 warps, 128 columns of C (32 per warp), one T-range.  Tiles of 64 rows of Q (bf16) and
// of P (fp32, split once per CTA into bf16 high and low parts) are staged in shared memory; both
// MMA operands are read back transposed with ldmatrix.trans.  The next tile's global loads are
// issued before the current tile is multiplied.
// ------------------------------------------------------------------------------------------
constexpr int kTnCols = 128;
constexpr int kTnPad = 8;
constexpr int kTnRows = 64;   // rows of T staged per step (four k16 MMA steps per barrier pair)

struct TnParams {
  const float* pmat;
  int64_t ldp;
  const __nv_bfloat16* q;
  int64_t ldq;
  int64_t T;
  int r;
  int64_t C;
  int64_t t_chunk;  // rows of T per split (multiple of 16)
  float* ws;        // [nsplit][r][C]
};

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}

template <int RT>  // r-tiles of 16
__global__ void __launch_bounds__(128) lora_tn_kernel(const TnParams p) {
  constexpr int RW = RT * 16;          // staged width of P
  constexpr int PV = kTnRows * RW / 128;   // P elements per thread per tile (8, 16 or 32)
  __shared__ __align__(16) __nv_bfloat16 qs[kTnRows][kTnCols + kTnPad];
  __shared__ __align__(16) __nv_bfloat16 phs[kTnRows][RW + kTnPad];
  __shared__ __align__(16) __nv_bfloat16 pls[kTnRows][RW + kTnPad];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, q = lane & 3;
  const int64_t c0 = static_cast<int64_t>(blockIdx.x) * kTnCols;
  const int64_t t_begin = static_cast<int64_t>(blockIdx.y) * p.t_chunk;
  const int64_t t_end = t_begin + p.t_chunk < p.T ? t_begin + p.t_chunk : p.T;

  float acc[RT][4][4];
#pragma unroll
  for (int i = 0; i < RT; ++i)
#pragma unroll
    for (int t = 0; t < 4; ++t)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[i][t][e] = 0.f;

  // staging of Q: 64 rows x 128 cols bf16 = 1024 x 16 bytes, eight per thread (row = idx / 16);
  // of P: thread owns PV consecutive j of one row (row = (tid * PV) / RW)
  const int prow = (threadIdx.x * PV) / RW, pcol = (threadIdx.x * PV) % RW;
  auto fetch = [&](int64_t t0, uint4 (&v)[8], float (&pv)[PV]) {
#pragma unroll
    for (int h = 0; h < 8; ++h) {
      const int idx = h * 128 + threadIdx.x;
      const int64_t t = t0 + (idx >> 4);
      const int64_t c = c0 + (idx & 15) * 8;
      v[h] = (t < t_end && c < p.C) ? __ldg(reinterpret_cast<const uint4*>(p.q + t * p.ldq + c))
                                    : make_uint4(0u, 0u, 0u, 0u);
    }
    const int64_t t = t0 + prow;
    const float* src = p.pmat + (t < t_end ? t : 0) * p.ldp;   // row 0 always exists; a split past the end has t_begin >= T
#pragma unroll
    for (int e = 0; e < PV; ++e) {
      const int j = pcol + e;
      const float x = __ldg(src + (j < p.r ? j : 0));
      pv[e] = (t < t_end && j < p.r) ? x : 0.f;
    }
  };

  uint4 nxt[8];
  float pnx[PV];
  fetch(t_begin, nxt, pnx);
  for (int64_t t0 = t_begin; t0 < t_end; t0 += kTnRows) {
    __syncthreads();  // previous tile fully consumed
#pragma unroll
    for (int h = 0; h < 8; ++h) {
      const int idx = h * 128 + threadIdx.x;
      *reinterpret_cast<uint4*>(&qs[idx >> 4][(idx & 15) * 8]) = nxt[h];
    }
#pragma unroll
    for (int e = 0; e < PV; e += 2) {
      uint32_t hi, lo;
      split2(pnx[e], pnx[e + 1], hi, lo);
      *reinterpret_cast<uint32_t*>(&phs[prow][pcol + e]) = hi;
      *reinterpret_cast<uint32_t*>(&pls[prow][pcol + e]) = lo;
    }
    __syncthreads();
    if (t0 + kTnRows < t_end) fetch(t0 + kTnRows, nxt, pnx);

    const int mat = lane >> 3;   // which 8x8 matrix of an ldmatrix.x4 this lane addresses
#pragma unroll
    for (int ks = 0; ks < kTnRows / 16; ++ks) {
      if (t0 + ks * 16 >= t_end) break;
      // A fragments: P^T, element (m=j, k=t) = P[t][j]; matrices (j 0-7,t 0-7) (j 8-15,t 0-7) (j 0-7,t 8-15) (j 8-15,t 8-15)
      uint32_t ah[RT][4], al[RT][4];
#pragma unroll
      for (int i = 0; i < RT; ++i) {
        const int row = ks * 16 + (lane & 7) + 8 * (mat >> 1);
        const int col = i * 16 + 8 * (mat & 1);
        ldmatrix_x4_trans(ah[i], smem_u32(&phs[row][col]));
        ldmatrix_x4_trans(al[i], smem_u32(&pls[row][col]));
      }
      // B fragments for the warp's 32 columns: two ldmatrix.x4.trans (two n8 tiles each)
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        uint32_t b[4];   // 0: k 0-7 / tile A, 1: k 8-15 / tile A, 2, 3: tile B
        const int row = ks * 16 + (lane & 7) + 8 * (mat & 1);
        const int col = warp * 32 + half * 16 + 8 * (mat >> 1);
        ldmatrix_x4_trans(b, smem_u32(&qs[row][col]));
#pragma unroll
        for (int i = 0; i < RT; ++i) {
          mma_bf16_16816(acc[i][half * 2], ah[i], b[0], b[1]);
          mma_bf16_16816(acc[i][half * 2], al[i], b[0], b[1]);
          mma_bf16_16816(acc[i][half * 2 + 1], ah[i], b[2], b[3]);
          mma_bf16_16816(acc[i][half * 2 + 1], al[i], b[2], b[3]);
        }
      }
    }
  }

  float* ws = p.ws + static_cast<int64_t>(blockIdx.y) * p.r * p.C;
#pragma unroll
  for (int i = 0; i < RT; ++i)
#pragma unroll
    for (int t = 0; t < 4; ++t)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int j = i * 16 + g + 8 * (e >> 1);
        const int64_t c = c0 + warp * 32 + t * 8 + 2 * q + (e & 1);
        if (j < p.r && c < p.C) ws[j * p.C + c] = acc[i][t][e];
      }
}

// The same product with a three-deep cp.async ring: the 64-row tiles of Q land directly in their
// padded shared-memory layout, the fp32 rows of P in a raw buffer from which every thread splits
// the pieces it copied itself into the bf16 high / low tiles.  Two tiles (50 KB) are in flight per
// CTA while one is multiplied.  Needs 16-byte aligned P rows and a rank that is a multiple of 4.
constexpr int kTnStages = 3;

template <int RT>
struct TnSmem {
  static constexpr int RW = RT * 16;
  static constexpr int kQ = kTnRows * (kTnCols + kTnPad) * 2;    // 17408
  static constexpr int kP = kTnRows * RW * 4;
  static constexpr int kStage = kQ + kP;
  static constexpr int kSplitOff = kTnStages * kStage;           // phs, pls
  static constexpr int kSplit = kTnRows * (RW + kTnPad) * 2;
  static constexpr int kBytes = kSplitOff + 2 * kSplit;
};

template <int RT>
__global__ void __launch_bounds__(128) lora_tn_async_kernel(const TnParams p) {
  using L = TnSmem<RT>;
  constexpr int RW = L::RW;
  constexpr int PP = kTnRows * RW / 4 / 128;   // 16-byte pieces of P per thread per tile (2, 4 or 8)
  constexpr int QROW = (kTnCols + kTnPad) * 2; // bytes
  constexpr int SROW = (RW + kTnPad) * 2;
  extern __shared__ __align__(16) uint8_t tsm[];
  const uint32_t base = smem_u32(tsm);
  const uint32_t phs = base + L::kSplitOff, pls = phs + L::kSplit;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, q = lane & 3;
  const int64_t c0 = static_cast<int64_t>(blockIdx.x) * kTnCols;
  const int64_t t_begin = static_cast<int64_t>(blockIdx.y) * p.t_chunk;
  const int64_t t_end = t_begin + p.t_chunk < p.T ? t_begin + p.t_chunk : p.T;

  float acc[RT][4][4];
#pragma unroll
  for (int i = 0; i < RT; ++i)
#pragma unroll
    for (int t = 0; t < 4; ++t)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[i][t][e] = 0.f;

  auto issue = [&](int64_t t0, int stage) {
    if (t0 < t_end) {
      const uint32_t qdst = base + stage * L::kStage, pdst = qdst + L::kQ;
#pragma unroll
      for (int h = 0; h < 8; ++h) {
        const int idx = h * 128 + threadIdx.x;
        const int row = idx >> 4, piece = idx & 15;
        const int64_t t = t0 + row, c = c0 + piece * 8;
        const bool in = t < t_end && c < p.C;
        cp_async16(qdst + row * QROW + piece * 16, p.q + (in ? t * p.ldq + c : 0), in ? 16u : 0u);
      }
#pragma unroll
      for (int h = 0; h < PP; ++h) {
        const int idx = h * 128 + threadIdx.x;
        const int row = idx / (RW / 4), piece = idx % (RW / 4);
        const int64_t t = t0 + row;
        const bool in = t < t_end && piece * 4 < p.r;
        cp_async16(pdst + idx * 16, p.pmat + (in ? t * p.ldp + piece * 4 : 0), in ? 16u : 0u);
      }
    }
    cp_async_commit();
  };

#pragma unroll
  for (int s = 0; s < kTnStages - 1; ++s) issue(t_begin + s * kTnRows, s);
  int stage = 0;
  const int mat = lane >> 3;   // which 8x8 matrix of an ldmatrix.x4 this lane addresses
  for (int64_t t0 = t_begin; t0 < t_end; t0 += kTnRows) {
    {
      int nstage = stage + kTnStages - 1;
      if (nstage >= kTnStages) nstage -= kTnStages;
      issue(t0 + (kTnStages - 1) * kTnRows, nstage);   // that slot was released by the barrier ending the last step
    }
    cp_async_wait<kTnStages - 1>();
    // own pieces of P: fp32 -> bf16 high / low
    const uint32_t qsrc = base + stage * L::kStage, psrc = qsrc + L::kQ;
#pragma unroll
    for (int h = 0; h < PP; ++h) {
      const int idx = h * 128 + threadIdx.x;
      const int row = idx / (RW / 4), piece = idx % (RW / 4);
      float v0, v1, v2, v3;
      asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v0), "=f"(v1), "=f"(v2), "=f"(v3) : "r"(psrc + idx * 16));
      uint32_t h0, l0, h1, l1;
      split2(v0, v1, h0, l0);
      split2(v2, v3, h1, l1);
      const uint32_t off = row * SROW + piece * 8;
      asm volatile("st.shared.v2.u32 [%0], {%1,%2};" ::"r"(phs + off), "r"(h0), "r"(h1) : "memory");
      asm volatile("st.shared.v2.u32 [%0], {%1,%2};" ::"r"(pls + off), "r"(l0), "r"(l1) : "memory");
    }
    __syncthreads();   // everybody's copies of this tile have landed and the split tiles are written

#pragma unroll
    for (int ks = 0; ks < kTnRows / 16; ++ks) {
      if (t0 + ks * 16 >= t_end) break;
      uint32_t ah[RT][4], al[RT][4];
#pragma unroll
      for (int i = 0; i < RT; ++i) {
        const int row = ks * 16 + (lane & 7) + 8 * (mat >> 1);
        const int col = i * 16 + 8 * (mat & 1);
        ldmatrix_x4_trans(ah[i], phs + row * SROW + col * 2);
        ldmatrix_x4_trans(al[i], pls + row * SROW + col * 2);
      }
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        uint32_t b[4];
        const int row = ks * 16 + (lane & 7) + 8 * (mat & 1);
        const int col = warp * 32 + half * 16 + 8 * (mat >> 1);
        ldmatrix_x4_trans(b, qsrc + row * QROW + col * 2);
#pragma unroll
        for (int i = 0; i < RT; ++i) {
          mma_bf16_16816(acc[i][half * 2], ah[i], b[0], b[1]);
          mma_bf16_16816(acc[i][half * 2 + 1], ah[i], b[2], b[3]);
        }
#pragma unroll
        for (int i = 0; i < RT; ++i) {
          mma_bf16_16816(acc[i][half * 2], al[i], b[0], b[1]);
          mma_bf16_16816(acc[i][half * 2 + 1], al[i], b[2], b[3]);
        }
      }
    }
    __syncthreads();   // tile consumed: its slot and the split tiles may be overwritten
    if (++stage == kTnStages) stage = 0;
  }
  cp_async_wait<0>();

  float* ws = p.ws + static_cast<int64_t>(blockIdx.y) * p.r * p.C;
#pragma unroll
  for (int i = 0; i < RT; ++i)
#pragma unroll
    for (int t = 0; t < 4; ++t)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int j = i * 16 + g + 8 * (e >> 1);
        const int64_t c = c0 + warp * 32 + t * 8 + 2 * q + (e & 1);
        if (j < p.r && c < p.C) ws[j * p.C + c] = acc[i][t][e];
      }
}

__global__ void lora_tn_reduce_kernel(const float* ws, int nsplit, int64_t rc, int64_t C, float scale,
                                      float* out, int64_t ldo) {
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= rc) return;
  float s = 0.f;
  for (int k = 0; k < nsplit; ++k) s += ws[k * rc + idx];
  out[(idx / C) * ldo + (idx % C)] = scale * s;
}

int tn_splits(int64_t T, int64_t C) {
  const int64_t col_ctas = (C + kTnCols - 1) / kTnCols;
  const int sms = sm_count() > 0 ? sm_count() : 148;   // of the current device (148 on B200)
  int64_t n = 2 * sms / col_ctas;   // at most two CTAs per SM (one wave), each with several 64-row steps
  const int64_t max_n = (T + 63) / 64;
  if (n > max_n) n = max_n;
  if (n < 1) n = 1;
  return static_cast<int>(n);
}

// ------------------------------------------------------------------------------------------
// Built-in scratch for k2q_lora_tn_static: split-T partial sums live in this file-scope device
// array instead of a caller-supplied workspace.  Every GPU that loads the library carries the
// array until the process exits.  In host code the array's name is only a handle; the device
// address is looked up once per device with cudaGetSymbolAddress while that device is current.
// ------------------------------------------------------------------------------------------
constexpr int64_t kStaticScratchFloats = 4ll << 20;   // 16 MiB
static __device__ __align__(256) float g_tn_scratch[kStaticScratchFloats];

std::mutex g_scratch_mu;
float* g_scratch_addr[64] = {nullptr};

int static_scratch(float** out) {
  int dev = 0;
  if (int rc = check_cuda(cudaGetDevice(&dev), "cudaGetDevice")) return rc;
  if (dev < 0 || dev >= 64) return fail(K2Q_EINVAL, "device index %d out of range", dev);
  std::lock_guard<std::mutex> lock(g_scratch_mu);
  if (g_scratch_addr[dev] == nullptr) {
    void* ptr = nullptr;
    if (int rc = check_cuda(cudaGetSymbolAddress(&ptr, g_tn_scratch), "cudaGetSymbolAddress(g_tn_scratch)"))
      return rc;
    if (ptr == nullptr) return fail(K2Q_ECUDA, "cudaGetSymbolAddress returned a null address");
    g_scratch_addr[dev] = static_cast<float*>(ptr);
  }
  *out = g_scratch_addr[dev];
  return K2Q_OK;
}

// ------------------------------------------------------------------------------------------
// int8 transpose, 64x64 tiles through shared memory
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) transpose_i8_kernel(const int8_t* src, int64_t R, int64_t C, int8_t* dst) {
  __shared__ int8_t tile[64][68];
  const int64_t r0 = static_cast<int64_t>(blockIdx.y) * 64, c0 = static_cast<int64_t>(blockIdx.x) * 64;
#pragma unroll
  for (int it = 0; it < 4; ++it) {
    const int idx = it * 256 + threadIdx.x;
    const int r = idx >> 4, c4 = (idx & 15) * 4;
    uint32_t w = 0;
    if (r0 + r < R && c0 + c4 < C) w = *reinterpret_cast<const uint32_t*>(src + (r0 + r) * C + c0 + c4);
    *reinterpret_cast<uint32_t*>(&tile[r][c4]) = w;
  }
  __syncthreads();
#pragma unroll
  for (int it = 0; it < 4; ++it) {
    const int idx = it * 256 + threadIdx.x;
    const int c = idx >> 4, r4 = (idx & 15) * 4;
    if (c0 + c < C && r0 + r4 < R) {
      const uint32_t w = static_cast<uint32_t>(static_cast<uint8_t>(tile[r4][c])) |
                         static_cast<uint32_t>(static_cast<uint8_t>(tile[r4 + 1][c])) << 8 |
                         static_cast<uint32_t>(static_cast<uint8_t>(tile[r4 + 2][c])) << 16 |
                         static_cast<uint32_t>(static_cast<uint8_t>(tile[r4 + 3][c])) << 24;
      *reinterpret_cast<uint32_t*>(dst + (c0 + c) * R + r0 + r4) = w;
    }
  }
}

template <int MT, int NT>
int launch_down(const DownParams& p, bool a_vec, cudaStream_t s) {
  const int64_t tiles = (p.M + MT * 16 - 1) / (MT * 16);
  // K split over a cluster while that does not exceed one CTA per SM and leaves every warp a chunk
  const int sms = sm_count() > 0 ? sm_count() : 148;
  const int chunks = (p.K + 31) / 32;
  int ksplit = 1;
  while (ksplit < 8 && tiles * (2 * ksplit) <= sms && chunks / (2 * ksplit) >= kDownWarps) ksplit *= 2;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(static_cast<unsigned>(tiles * ksplit));
  cfg.blockDim = dim3(kDownWarps * 32);
  cfg.dynamicSmemBytes = sizeof(float) * MT * 16 * NT * 8;   // at most 16 KB
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = static_cast<unsigned>(ksplit);
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (a_vec) {
    auto kern = lora_down_async_kernel<MT, NT>;
    const int smem = MT * 16 * NT * 8 * 4 + kDownWarps * down_stages(MT, NT) * (2 * MT + 2 * NT) * 512;
    if (int rc = check_cuda(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem),
                            "cudaFuncSetAttribute(lora_down)"))
      return rc;
    cfg.dynamicSmemBytes = smem;
    return check_cuda(cudaLaunchKernelEx(&cfg, kern, p), "lora_down launch");
  }
  return check_cuda(cudaLaunchKernelEx(&cfg, lora_down_kernel<MT, NT>, p), "lora_down launch");
}

// the most rows per CTA (least re-reading of the factor) that still yields a CTA per SM at the
// largest K split
template <int NT>
int dispatch_down(const DownParams& p, bool a_vec, cudaStream_t s) {
  const int sms = sm_count() > 0 ? sm_count() : 148;
  if (NT <= 4) {
    if ((p.M + 63) / 64 * 8 >= sms) return launch_down<(NT <= 4 ? 4 : 1), NT>(p, a_vec, s);
  }
  if ((p.M + 31) / 32 * 8 >= sms && (NT <= 4 || a_vec)) return launch_down<2, NT>(p, a_vec, s);
  return launch_down<1, NT>(p, a_vec, s);
}

template <int RT>
int launch_tn_rt(const TnParams& p, dim3 grid, bool async_ok, cudaStream_t s) {
  if (async_ok) {
    auto kern = lora_tn_async_kernel<RT>;
    if (int rc = check_cuda(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, TnSmem<RT>::kBytes),
                            "cudaFuncSetAttribute(lora_tn)"))
      return rc;
    kern<<<grid, 128, TnSmem<RT>::kBytes, s>>>(p);
  } else {
    lora_tn_kernel<RT><<<grid, 128, 0, s>>>(p);
  }
  return check_cuda(cudaGetLastError(), "lora_tn launch");
}

int launch_tn(const TnParams& p, int nsplit, cudaStream_t s) {
  const dim3 grid(static_cast<unsigned>((p.C + kTnCols - 1) / kTnCols), static_cast<unsigned>(nsplit));
  const bool async_ok = (p.ldp % 4) == 0 && (p.r % 4) == 0 && (reinterpret_cast<uintptr_t>(p.pmat) & 15u) == 0;
  if (p.r <= 16) return launch_tn_rt<1>(p, grid, async_ok, s);
  if (p.r <= 32) return launch_tn_rt<2>(p, grid, async_ok, s);
  return launch_tn_rt<4>(p, grid, async_ok, s);
}

}  // namespace
}  // namespace k2q

using namespace k2q;

extern "C" {

int k2q_lora_down(const void* x_bf16, int64_t M, int64_t K, int64_t ldx, const float* a, int64_t a_rs,
                  int64_t a_cs, int32_t r, float scale, float* out, int64_t ldo, void* stream) {
  if (int rc = check_device_arch()) return rc;
  if (M < 0 || K <= 0 || K % 8 != 0 || K > 0x7fffff00LL)
    return fail(K2Q_EINVAL, "k2q_lora_down: bad shape M=%lld K=%lld (K must be a multiple of 8)", (long long)M,
                (long long)K);
  if (r < 1 || r > 64) return fail(K2Q_EINVAL, "k2q_lora_down: rank %d not in [1,64]", r);
  if (M == 0) return K2Q_OK;
  if (!x_bf16 || !a || !out) return fail(K2Q_EINVAL, "k2q_lora_down: NULL operand");
  if (ldx < K || (ldx % 8) != 0 || (reinterpret_cast<uintptr_t>(x_bf16) & 15u))
    return fail(K2Q_EINVAL, "k2q_lora_down: x rows must be 16-byte aligned with ldx >= K");
  if (ldo < r) return fail(K2Q_EINVAL, "k2q_lora_down: ldo < rank");
  if (M / 16 > 0x7fffffffLL) return fail(K2Q_EINVAL, "k2q_lora_down: M too large");
  const bool a_vec = a_cs == 1 && (a_rs % 4) == 0 && (reinterpret_cast<uintptr_t>(a) & 15u) == 0;
  DownParams p{static_cast<const __nv_bfloat16*>(x_bf16), ldx, M, (int)K, a, a_rs, a_cs, r, scale, out, ldo};
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (r <= 16) return dispatch_down<2>(p, a_vec, s);
  if (r <= 32) return dispatch_down<4>(p, a_vec, s);
  return dispatch_down<8>(p, a_vec, s);
}

int64_t k2q_lora_tn_workspace_bytes(int64_t T, int32_t r, int64_t C) {
  if (T <= 0 || r <= 0 || C <= 0) return 0;
  return static_cast<int64_t>(tn_splits(T, C)) * r * C * (int64_t)sizeof(float);
}

int k2q_lora_tn(const float* pmat, int64_t ldp, const void* q_bf16, int64_t ldq, int64_t T, int32_t r,
                int64_t C, float scale, float* out, int64_t ldo, void* ws, int64_t ws_bytes, void* stream) {
  if (int rc = check_device_arch()) return rc;
  if (T < 0 || C <= 0 || (C % 8) != 0) return fail(K2Q_EINVAL, "k2q_lora_tn: bad shape T=%lld C=%lld", (long long)T, (long long)C);
  if (r < 1 || r > 64) return fail(K2Q_EINVAL, "k2q_lora_tn: rank %d not in [1,64]", r);
  if (!out || ldo < C) return fail(K2Q_EINVAL, "k2q_lora_tn: bad output");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (T == 0) {
    return check_cuda(cudaMemset2DAsync(out, ldo * sizeof(float), 0, C * sizeof(float), r, s), "cudaMemset2DAsync");
  }
  if (!pmat || !q_bf16 || !ws) return fail(K2Q_EINVAL, "k2q_lora_tn: NULL operand");
  if (ldp < r) return fail(K2Q_EINVAL, "k2q_lora_tn: ldp < rank");
  if (ldq < C || (ldq % 8) != 0 || (reinterpret_cast<uintptr_t>(q_bf16) & 15u))
    return fail(K2Q_EINVAL, "k2q_lora_tn: q rows must be 16-byte aligned with ldq >= C");
  const int nsplit = tn_splits(T, C);
  const int64_t need = static_cast<int64_t>(nsplit) * r * C * (int64_t)sizeof(float);
  if (ws_bytes < need)
    return fail(K2Q_EINVAL, "k2q_lora_tn: workspace of %lld bytes given, %lld needed", (long long)ws_bytes,
                (long long)need);
  TnParams p{};
  p.pmat = pmat; p.ldp = ldp; p.q = static_cast<const __nv_bfloat16*>(q_bf16); p.ldq = ldq;
  p.T = T; p.r = r; p.C = C;
  p.t_chunk = ((T + nsplit - 1) / nsplit + 15) / 16 * 16;   // multiple of 16: k16 steps never straddle splits
  p.ws = static_cast<float*>(ws);
  if (int rc = launch_tn(p, nsplit, s)) return rc;
  const int64_t rc_elems = static_cast<int64_t>(r) * C;
  lora_tn_reduce_kernel<<<static_cast<unsigned>((rc_elems + 255) / 256), 256, 0, s>>>(
      p.ws, nsplit, rc_elems, C, scale, out, ldo);
  return check_cuda(cudaGetLastError(), "lora_tn_reduce launch");
}

int64_t k2q_lora_tn_static_max_bytes(void) { return kStaticScratchFloats * (int64_t)sizeof(float); }

int k2q_lora_tn_static(const float* pmat, int64_t ldp, const void* q_bf16, int64_t ldq, int64_t T, int32_t r,
                       int64_t C, float scale, float* out, int64_t ldo, void* stream) {
  if (int rc = check_device_arch()) return rc;
  if (T < 0 || C <= 0 || (C % 8) != 0)
    return fail(K2Q_EINVAL, "k2q_lora_tn_static: bad shape T=%lld C=%lld", (long long)T, (long long)C);
  if (r < 1 || r > 64) return fail(K2Q_EINVAL, "k2q_lora_tn_static: rank %d not in [1,64]", r);
  if (!out || ldo < C) return fail(K2Q_EINVAL, "k2q_lora_tn_static: bad output");
  if (T == 0) {   // an empty sum, as k2q_lora_tn gives it: zeros, no kernel, no scratch
    return check_cuda(cudaMemset2DAsync(out, ldo * sizeof(float), 0, C * sizeof(float), r,
                                        static_cast<cudaStream_t>(stream)),
                      "cudaMemset2DAsync");
  }
  if (!pmat || !q_bf16) return fail(K2Q_EINVAL, "k2q_lora_tn_static: NULL operand");
  if (ldp < r) return fail(K2Q_EINVAL, "k2q_lora_tn_static: leading dimension too small");
  if (ldq < C || (ldq % 8) != 0 || (reinterpret_cast<uintptr_t>(q_bf16) & 15u))
    return fail(K2Q_EINVAL, "k2q_lora_tn_static: q rows must be 16-byte aligned with ldq >= C");
  const int nsplit = tn_splits(T, C);
  const int64_t need = static_cast<int64_t>(nsplit) * r * C * (int64_t)sizeof(float);
  if (need > k2q_lora_tn_static_max_bytes())
    return fail(K2Q_EINVAL,
                "k2q_lora_tn_static: this problem needs %lld bytes of scratch, the built-in array holds %lld; "
                "use k2q_lora_tn with a caller-provided workspace",
                (long long)need, (long long)k2q_lora_tn_static_max_bytes());
  float* scratch = nullptr;
  if (int rc = static_scratch(&scratch)) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  TnParams p{};
  p.pmat = pmat; p.ldp = ldp; p.q = static_cast<const __nv_bfloat16*>(q_bf16); p.ldq = ldq;
  p.T = T; p.r = r; p.C = C;
  p.t_chunk = ((T + nsplit - 1) / nsplit + 15) / 16 * 16;   // multiple of 16: k16 steps never straddle splits
  p.ws = scratch;   // every partial sum the reduction reads is written by this launch: nothing to clear
  if (int rc = launch_tn(p, nsplit, s)) return rc;
  const int64_t rc_elems = static_cast<int64_t>(r) * C;
  lora_tn_reduce_kernel<<<static_cast<unsigned>((rc_elems + 255) / 256), 256, 0, s>>>(scratch, nsplit, rc_elems, C,
                                                                                      scale, out, ldo);
  return check_cuda(cudaGetLastError(), "lora_tn_reduce launch");
}

int k2q_transpose_i8(const int8_t* src, int64_t R, int64_t C, int8_t* dst, void* stream) {
  if (int rc = check_device_arch()) return rc;
  if (R <= 0 || C <= 0 || (R % 4) != 0 || (C % 4) != 0)
    return fail(K2Q_EINVAL, "k2q_transpose_i8: R=%lld and C=%lld must be positive multiples of 4", (long long)R,
                (long long)C);
  if (!src || !dst || (reinterpret_cast<uintptr_t>(src) & 3u) || (reinterpret_cast<uintptr_t>(dst) & 3u))
    return fail(K2Q_EINVAL, "k2q_transpose_i8: operands must be non-NULL and 4-byte aligned");
  const dim3 grid(static_cast<unsigned>((C + 63) / 64), static_cast<unsigned>((R + 63) / 64));
  transpose_i8_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(src, R, C, dst);
  return check_cuda(cudaGetLastError(), "transpose_i8 launch");
}

}  // extern "C"
