// K3: W8A8 GEMM on tcgen05 int8 tensor cores, with the dequant / bias / activation / LoRA
// epilogue fused.  Also serves the backward dX GEMM (codes transposed to [K,N], sw folded into
// the quantised dY, the LoRA operand being du and the rotated A).
//
// Persistent kernel, one CTA per SM, 384 threads in three warpgroups (setmaxnreg hands the
// registers of the data-movement warpgroup to the two epilogue warpgroups):
//   warp 0 lane 0   TMA producer: xq tile [128 x 128B] + wq tile [256 x 128B] per K-block into
//                   a ring of STAGES shared-memory slots (SWIZZLE_128B boxes, every CTA loads for itself)
//   warp 1 lane 0   MMA issuer: per K-block four tcgen05.mma kind::i8 (M128 N256 K32) into one
//                   of two 256-column TMEM accumulators; tcgen05.commit frees the slot / hands
//                   the accumulator to the epilogue
//   warps 4..11     epilogue: warps 4..7 take columns 0..127 of the tile, warps 8..11 columns
//                   128..255; each reads its 32-lane TMEM quarter 32 columns at a time (tcgen05.ld),
//                   fp32 dequant (+bias, +GELU, +LoRA u.B^T), bf16 pack, 16-byte global stores.
//                   The second accumulator lets tile i+1's MMAs run under tile i's epilogue.
// PAIR mode (the default for all but tiny problems): two CTAs of a cluster work on one 256 x 256
// tile with tcgen05.mma.cta_group::2.  Each CTA stages its own 128 rows of A and HALF of the B
// tile, so per CTA both the TMA writes into shared memory and the tensor core's operand reads
// drop by a third; the single-CTA kernel is bound by exactly that shared-memory traffic.  CTA 0
// issues the MMAs for both; completion is committed to the barriers of both CTAs (two plain
// commits, one per CTA), the partner's TMA reports to CTA 0's "full" barrier, and the partner's
// epilogue warps release the accumulator on CTA 0's barrier.
// Every mbarrier wait is bounded (see k2q_common.cuh); on expiry the CTA drains and exits.
#include "k2q_common.cuh"

namespace k2q {
namespace {

constexpr int BM = 128;         // tokens per tile   (UMMA M)
constexpr int BN = 256;         // channels per tile (UMMA N)
constexpr int BK = 128;         // int8 elements (= bytes) per K-block: one 128B swizzle row
constexpr int UMMA_K = 32;      // K of one kind::i8 instruction
constexpr int kThreads = 384;
constexpr int kEpiThreads = 256;
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kStageBytesSingle = (BM + BN) * BK;      // 49152: A 128 rows + B 256 rows
constexpr uint32_t kStageBytesPair = (BM + BN / 2) * BK;    // 32768: A 128 rows + B 128 rows per CTA

enum WaitId : int {
  W_EMPTY = 101,       // producer waiting for a free slot
  W_FULL = 102,        // MMA issuer waiting for TMA data
  W_TMEM_EMPTY = 103,  // MMA issuer waiting for the epilogue to release an accumulator
  W_TMEM_FULL = 104,   // epilogue waiting for the accumulator
  W_SMEM_ALIGN = 105   // dynamic shared memory base not 1024-byte aligned
};

struct GemmParams {
  int M, N, K;
  int tiles_m, tiles_n;
  const float* sx;
  const float* sw;
  const float* bias;
  const float* u;
  const float* Bm;
  int64_t ldu, ldb;
  int rank;
  float lora_scale;
  int act;
  __nv_bfloat16* y;
  int64_t ldy;
  Status* status;
};

template <int STAGES, int RMAX, bool PAIR>
struct Smem {
  static constexpr uint32_t kStageBytes = PAIR ? kStageBytesPair : kStageBytesSingle;
  static constexpr uint32_t kRing = STAGES * kStageBytes;
  static constexpr uint32_t kColOff = kRing;                             // sw_s[256], bias_s[256]
  static constexpr uint32_t kLoraOff = kColOff + 2 * BN * 4;             // Bs[256][RMAX]
  static constexpr uint32_t kBarOff = kLoraOff + BN * RMAX * 4;          // mbarriers
  static constexpr uint32_t kBytes = kBarOff + (2 * STAGES + 4) * 8 + 16;
};

__device__ __forceinline__ float gelu_tanh_f(float v) {
  // 0.5 v (1 + tanh(sqrt(2/pi) (v + 0.044715 v^3))) with the hardware tanh (|error| < 6e-4, far below
  // the bf16 resolution of the output)
  const float z = v * fmaf(0.0356774081f, v * v, 0.7978845608f);
  float th;
  asm("tanh.approx.f32 %0, %1;" : "=f"(th) : "f"(z));
  const float hv = 0.5f * v;
  return fmaf(hv, th, hv);
}

template <int STAGES, int RMAX, bool PAIR>
__global__ void __launch_bounds__(kThreads, 1)
gemm_w8a8_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w,
                 const GemmParams p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  using L = Smem<STAGES, RMAX, PAIR>;
  constexpr uint32_t kStageBytes = L::kStageBytes;
  const uint32_t cta_rank = PAIR ? cluster_ctarank() : 0u;         // 0 = the CTA that issues the MMAs
  const int worker = PAIR ? static_cast<int>(blockIdx.x >> 1) : static_cast<int>(blockIdx.x);
  const int num_workers = PAIR ? static_cast<int>(gridDim.x >> 1) : static_cast<int>(gridDim.x);
  constexpr int TILE_M = PAIR ? 2 * BM : BM;                        // rows of one tile (both CTAs)

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t smem_base = smem_u32(smem);

  float* sw_s = reinterpret_cast<float*>(smem + L::kColOff);
  float* bias_s = sw_s + BN;
  float* lora_s = reinterpret_cast<float*>(smem + L::kLoraOff);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBarOff);
  const uint32_t bar_full = smem_u32(bars);                 // [STAGES]
  const uint32_t bar_empty = bar_full + 8 * STAGES;         // [STAGES]
  const uint32_t bar_tfull = bar_empty + 8 * STAGES;        // [2]
  const uint32_t bar_tempty = bar_tfull + 16;               // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  if ((smem_base & 1023u) != 0u) {  // uniform over the CTA: nothing has been set up yet
    if (threadIdx.x == 0 && atomicCAS(&p.status->code, 0, W_SMEM_ALIGN) == 0) {
      p.status->block = static_cast<int>(blockIdx.x);
      p.status->detail = static_cast<int>(smem_base & 1023u);
    }
    return;
  }

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar_tfull + 8 * b, 1);
      mbar_init(bar_tempty + 8 * b, (PAIR ? 2 : 1) * kEpiThreads / 32);   // one arrival per epilogue warp (of both CTAs)
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap_x);
    tma_prefetch_desc(&tmap_w);
  }
  if (warp == 1) {
    if (PAIR) {
      tmem_alloc_pair(smem_u32(tmem_slot), kTmemCols);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(smem_u32(tmem_slot), kTmemCols);
      tmem_relinquish();
    }
  }
  tc_fence_before();
  __syncthreads();
  if (PAIR) cluster_sync_all();   // both CTAs' barriers are initialised before anyone signals them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const WaitCtx wctx{abort_flag, p.status};
  const int num_tiles = p.tiles_m * p.tiles_n;
  const int kblocks = p.K / BK;

  if (warp < 4) {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = worker; ok && tile < num_tiles; tile += num_workers) {
        const int m0 = (tile / p.tiles_n) * TILE_M + static_cast<int>(cta_rank) * BM;
        const int n0 = (tile % p.tiles_n) * BN + (PAIR ? static_cast<int>(cta_rank) * (BN / 2) : 0);
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!mbar_wait(bar_empty + 8 * stage, phase ^ 1u, wctx, W_EMPTY, kb)) { ok = false; break; }
          const uint32_t a_dst = smem_base + stage * kStageBytes;
          if (PAIR) {
            // both CTAs' copies report to CTA 0's barrier, which expects the bytes of both
            const uint32_t full0 = map_to_cta(bar_full + 8 * stage, 0u);
            if (cta_rank == 0) mbar_expect_tx(bar_full + 8 * stage, 2u * kStageBytes);
            tma_load_2d_pair(a_dst, &tmap_x, kb * BK, m0, full0);
            tma_load_2d_pair(a_dst + BM * BK, &tmap_w, kb * BK, n0, full0);
          } else {
            const uint32_t full = bar_full + 8 * stage;
            mbar_expect_tx(full, kStageBytes);
            tma_load_2d(a_dst, &tmap_x, kb * BK, m0, full);
            tma_load_2d(a_dst + BM * BK, &tmap_w, kb * BK, n0, full);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0 && cta_rank == 0) {
      constexpr uint32_t idesc = umma_idesc_i8(TILE_M, BN);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int it = 0;
      for (int tile = worker; ok && tile < num_tiles; tile += num_workers, ++it) {
        const int buf = it & 1;
        const uint32_t use_parity = static_cast<uint32_t>(it >> 1) & 1u;
        if (!mbar_wait(bar_tempty + 8 * buf, use_parity ^ 1u, wctx, W_TMEM_EMPTY, it)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(buf * BN);
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!mbar_wait(bar_full + 8 * stage, phase, wctx, W_FULL, kb)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = smem_base + stage * kStageBytes;
          const uint64_t a_desc = umma_desc_k128(a_addr);
          const uint64_t b_desc = umma_desc_k128(a_addr + BM * BK);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            // advancing K by 32 bytes inside the 128B swizzle row = +2 in the address field
            if (PAIR) umma_i8_pair(d_tmem, a_desc + 2u * k, b_desc + 2u * k, idesc, (kb | k) != 0 ? 1u : 0u);
            else umma_i8(d_tmem, a_desc + 2u * k, b_desc + 2u * k, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          // slot reusable once these MMAs have read it (in both CTAs)
          if (PAIR) {
            tc_commit_pair(bar_empty + 8 * stage);
            tc_commit_pair(map_to_cta(bar_empty + 8 * stage, 1u));
          } else {
            tc_commit(bar_empty + 8 * stage);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (ok) {  // accumulator complete -> epilogue (of both CTAs)
          if (PAIR) {
            tc_commit_pair(bar_tfull + 8 * buf);
            tc_commit_pair(map_to_cta(bar_tfull + 8 * buf, 1u));
          } else {
            tc_commit(bar_tfull + 8 * buf);
          }
        }
      }
    }
  }
  } else {
    // ------------------------------------------------------------------ epilogue
    asm volatile("setmaxnreg.inc.sync.aligned.u32 232;");
    const int et = threadIdx.x - 128;         // 0..255
    const int quarter = warp & 3;             // TMEM lane quarter this warp may read
    const int chunk0 = ((warp - 4) >> 2) * (BN / 64);   // first 32-column chunk of this warp's half
    // After an expired wait a thread keeps walking the tile loop (so the named barriers below
    // still see all 128 threads) but touches neither TMEM nor memory any more.
    bool ok = true;
    int it = 0;
    const uint32_t tempty0 = PAIR ? map_to_cta(bar_tempty, 0u) : bar_tempty;   // CTA 0 owns the MMA issue
    for (int tile = worker; tile < num_tiles; tile += num_workers, ++it) {
      const int m0 = (tile / p.tiles_n) * TILE_M + static_cast<int>(cta_rank) * BM;
      const int n0 = (tile % p.tiles_n) * BN;
      const int buf = it & 1;
      const uint32_t use_parity = static_cast<uint32_t>(it >> 1) & 1u;

      // per-column operands of this tile (the previous tile's readers have passed this barrier)
      named_bar_sync(1, kEpiThreads);
      if (ok) {
        for (int i = et; i < BN; i += kEpiThreads) {
          const int col = n0 + i;
          const bool in = col < p.N;
          sw_s[i] = in ? (p.sw ? __ldg(p.sw + col) : 1.0f) : 0.0f;
          bias_s[i] = (in && p.bias) ? __ldg(p.bias + col) : 0.0f;
        }
        if (RMAX > 0) {
          constexpr int RD = RMAX > 0 ? RMAX : 1;
          for (int i = et; i < BN * RMAX; i += kEpiThreads) {
            const int n = i / RD, j = i % RD;
            const int col = n0 + n;
            lora_s[i] = (col < p.N && j < p.rank) ? p.lora_scale * __ldg(p.Bm + col * p.ldb + j) : 0.0f;
          }
        }
      }
      named_bar_sync(1, kEpiThreads);

      const int row = m0 + quarter * 32 + lane;
      const bool row_ok = row < p.M;
      const float sxr = (row_ok && p.sx) ? __ldg(p.sx + row) : 1.0f;
      float ur[RMAX > 0 ? RMAX : 1];
      if (RMAX > 0) {
#pragma unroll
        for (int j = 0; j < RMAX; ++j)
          ur[j] = (row_ok && j < p.rank) ? __ldg(p.u + row * p.ldu + j) : 0.0f;
      }

      // one waiter per warp (waking many threads off one mbarrier is slow); tcgen05.ld is
      // warp-collective, so the outcome is shared by the whole warp
      if (ok && lane == 0) ok = mbar_wait(bar_tfull + 8 * buf, use_parity, wctx, W_TMEM_FULL, it);
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) continue;
      tc_fence_after();
      const uint32_t t_addr = tmem_base + static_cast<uint32_t>(buf * BN) +
                              (static_cast<uint32_t>(quarter * 32) << 16);
      __nv_bfloat16* yrow = p.y + static_cast<int64_t>(row_ok ? row : 0) * p.ldy + n0;

#pragma unroll 1
      for (int c = chunk0; c < chunk0 + BN / 64; ++c) {
        uint32_t acc[32];
        tmem_ld32(t_addr + c * 32, acc);
        tmem_ld_wait();
        if (c == chunk0 + BN / 64 - 1) {  // this warp has read its half of the accumulator
          tc_fence_before();
          __syncwarp();
          if (lane == 0) {
            if (PAIR) mbar_arrive_cluster(tempty0 + 8 * buf);
            else mbar_arrive(bar_tempty + 8 * buf);
          }
        }
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const int cj = c * 32 + j;
          float t = __fmul_rn(static_cast<float>(static_cast<int32_t>(acc[j])), sxr);
          t = __fmul_rn(t, sw_s[cj]);
          t = __fadd_rn(t, bias_s[cj]);
          if (p.act == K2Q_ACT_GELU_TANH) t = gelu_tanh_f(t);
          if (RMAX > 0) {
            const float4* b4 = reinterpret_cast<const float4*>(lora_s + cj * RMAX);
            float d = 0.f;
#pragma unroll
            for (int j4 = 0; j4 < RMAX / 4; ++j4) {
              const float4 b = b4[j4];
              d = fmaf(ur[4 * j4], b.x, d);
              d = fmaf(ur[4 * j4 + 1], b.y, d);
              d = fmaf(ur[4 * j4 + 2], b.z, d);
              d = fmaf(ur[4 * j4 + 3], b.w, d);
            }
            t += d;
          }
          v[j] = t;
        }
        if (row_ok) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            if (n0 + c * 32 + g * 8 + 8 <= p.N) {
              uint4 o;
              o.x = pack_bf16x2(v[8 * g], v[8 * g + 1]);
              o.y = pack_bf16x2(v[8 * g + 2], v[8 * g + 3]);
              o.z = pack_bf16x2(v[8 * g + 4], v[8 * g + 5]);
              o.w = pack_bf16x2(v[8 * g + 6], v[8 * g + 7]);
              *reinterpret_cast<uint4*>(yrow + c * 32 + g * 8) = o;
            }
          }
        }
      }
    }
  }

  // ---------------------------------------------------------------------- teardown
  if (*abort_flag) {
    // a wait expired somewhere: give copies and MMAs still in flight time to land
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (PAIR) cluster_sync_all();   // the partner may still read this CTA's operands / signal its barriers
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    if (PAIR) tmem_dealloc_pair(tmem_base, kTmemCols);
    else tmem_dealloc(tmem_base, kTmemCols);
  }
}

template <int STAGES, int RMAX, bool PAIR>
int launch(const CUtensorMap& tx, const CUtensorMap& tw, const GemmParams& p, int grid, cudaStream_t stream) {
  using L = Smem<STAGES, RMAX, PAIR>;
  static_assert(L::kBytes <= 232448, "shared memory budget exceeded");
  auto kern = gemm_w8a8_kernel<STAGES, RMAX, PAIR>;
  if (int rc = check_cuda(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kBytes),
                          "cudaFuncSetAttribute(gemm_w8a8)"))
    return rc;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(static_cast<unsigned>(grid));
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = L::kBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = PAIR ? 2 : 1;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return check_cuda(cudaLaunchKernelEx(&cfg, kern, tx, tw, p), "gemm_w8a8 launch");
}

}  // namespace
}  // namespace k2q

using namespace k2q;

extern "C" int k2q_gemm_w8a8(const int8_t* xq, const int8_t* wq, const float* sw, int64_t M, int64_t N,
                             int64_t K, const k2q_epilogue* ep, void* y_bf16, int64_t ldy, void* status,
                             void* stream) {
  if (int rc = check_device_arch()) return rc;
  if (M < 0 || N <= 0 || K <= 0 || M > 0x7fffff00LL || N > 0x7fffff00LL || K > 0x7fffff00LL)
    return fail(K2Q_EINVAL, "k2q_gemm_w8a8: bad shape M=%lld N=%lld K=%lld", (long long)M, (long long)N,
                (long long)K);
  if (K % 128 != 0) return fail(K2Q_EINVAL, "k2q_gemm_w8a8: K=%lld is not a multiple of 128", (long long)K);
  if (N % 16 != 0) return fail(K2Q_EINVAL, "k2q_gemm_w8a8: N=%lld is not a multiple of 16", (long long)N);
  if (M == 0) return K2Q_OK;
  if (!xq || !wq || !y_bf16 || !status) return fail(K2Q_EINVAL, "k2q_gemm_w8a8: NULL operand");
  if (ldy < N || (ldy % 8) != 0 || (reinterpret_cast<uintptr_t>(y_bf16) & 15u))
    return fail(K2Q_EINVAL, "k2q_gemm_w8a8: y must be 16-byte aligned with ldy >= N and ldy %% 8 == 0");
  k2q_epilogue e{};
  if (ep) e = *ep;
  if (e.rank < 0 || e.rank > 64) return fail(K2Q_EINVAL, "k2q_gemm_w8a8: LoRA rank %d not in [0,64]", e.rank);
  if ((e.u == nullptr) != (e.Bm == nullptr) || ((e.u != nullptr) != (e.rank > 0)))
    return fail(K2Q_EINVAL, "k2q_gemm_w8a8: u, Bm and rank must be given together");
  if (e.rank > 0 && (e.ldu < e.rank || e.ldb < e.rank))
    return fail(K2Q_EINVAL, "k2q_gemm_w8a8: ldu/ldb smaller than rank");
  if (e.act != K2Q_ACT_NONE && e.act != K2Q_ACT_GELU_TANH)
    return fail(K2Q_EINVAL, "k2q_gemm_w8a8: unknown activation %d", e.act);

  // CTA pairs (256 x 256 tiles) unless the problem has too few rows to fill them
  const bool pair = M > BM;
  const int tile_m = pair ? 2 * BM : BM;
  GemmParams p{};
  p.M = (int)M; p.N = (int)N; p.K = (int)K;
  p.tiles_m = (int)((M + tile_m - 1) / tile_m);
  p.tiles_n = (int)((N + BN - 1) / BN);
  p.sx = e.sx; p.sw = sw; p.bias = e.bias;
  p.u = e.u; p.Bm = e.Bm; p.ldu = e.ldu; p.ldb = e.ldb; p.rank = e.rank;
  p.lora_scale = e.lora_scale; p.act = e.act;
  p.y = static_cast<__nv_bfloat16*>(y_bf16); p.ldy = ldy;
  p.status = static_cast<Status*>(status);

  CUtensorMap tx, tw;
  if (int rc = encode_tmap_2d_u8(&tx, xq, (uint64_t)K, (uint64_t)M, (uint64_t)K, BK, BM, 1)) return rc;
  if (int rc = encode_tmap_2d_u8(&tw, wq, (uint64_t)K, (uint64_t)N, (uint64_t)K, BK, pair ? BN / 2 : BN, 1)) return rc;

  const int sms = sm_count();
  if (sms <= 0) return fail(K2Q_ECUDA, "k2q_gemm_w8a8: could not read the SM count");
  const int64_t tiles = (int64_t)p.tiles_m * p.tiles_n;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (pair) {
    const int64_t pairs = tiles < sms / 2 ? tiles : sms / 2;
    const int grid = (int)(2 * pairs);
    if (e.rank == 0) return launch<6, 0, true>(tx, tw, p, grid, s);
    if (e.rank <= 16) return launch<6, 16, true>(tx, tw, p, grid, s);
    if (e.rank <= 32) return launch<5, 32, true>(tx, tw, p, grid, s);
    return launch<4, 64, true>(tx, tw, p, grid, s);
  }
  const int grid = (int)(tiles < sms ? tiles : sms);
  if (e.rank == 0) return launch<4, 0, false>(tx, tw, p, grid, s);
  if (e.rank <= 16) return launch<4, 16, false>(tx, tw, p, grid, s);
  if (e.rank <= 32) return launch<4, 32, false>(tx, tw, p, grid, s);
  return launch<3, 64, false>(tx, tw, p, grid, s);
}
