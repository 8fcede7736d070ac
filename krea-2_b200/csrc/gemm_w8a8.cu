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
//                   fp32 dequant (+bias, +GELU), bf16 pack, 16-byte global stores.  With a LoRA
//                   term the accumulator is read in MMA-fragment layout instead and u.B^T is added
//                   by warp-level bf16 MMAs on split-precision operands (see the epilogue).
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

template <int STAGES, int RMAX, bool PAIR, bool FMA>
struct Smem {
  static constexpr uint32_t kStageBytes = PAIR ? kStageBytesPair : kStageBytesSingle;
  static constexpr uint32_t kRing = STAGES * kStageBytes;
  static constexpr uint32_t kColOff = kRing;                             // sw_s[256], bias_s[256]
  // LoRA factor of the tile as bf16 high and low parts, rows padded by 8 elements so that the
  // MMA fragment reads (8 rows x 4 words per warp) hit 32 different banks
  static constexpr uint32_t kLoraRow = RMAX + 8;                         // bf16 elements per row
  static constexpr uint32_t kLoraOff = kColOff + 2 * BN * 4;             // hi[256][RMAX+8], lo[256][RMAX+8]
  // ranks up to 32 take the adapter term on the fp32 pipe instead: the factor of the tile, scaled, as
  // fp32 [RMAX][256] (rank-major, so that a warp reads four neighbouring columns of one rank with one
  // broadcast 16-byte load)
  static constexpr bool kFmaLora = FMA;
  static_assert(!FMA || (RMAX > 0 && RMAX <= 32), "the fp32-pipe adapter epilogue covers ranks up to 32");
  static constexpr uint32_t kLoraBytes = RMAX == 0 ? 0 : (kFmaLora ? RMAX * BN * 4 : 2 * BN * kLoraRow * 2);
  static constexpr uint32_t kBarOff = kLoraOff + kLoraBytes;             // mbarriers
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

template <int STAGES, int RMAX, bool PAIR, bool BMN, bool FMA>
__global__ void __launch_bounds__(kThreads, 1)
gemm_w8a8_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w,
                 const GemmParams p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  using L = Smem<STAGES, RMAX, PAIR, FMA>;
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
  __nv_bfloat16* lora_h = reinterpret_cast<__nv_bfloat16*>(smem + L::kLoraOff);
  __nv_bfloat16* lora_l = lora_h + BN * L::kLoraRow;
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
          if (!mbar_wait<4>(bar_empty + 8 * stage, phase ^ 1u, wctx, W_EMPTY, kb)) { ok = false; break; }
          const uint32_t a_dst = smem_base + stage * kStageBytes;
          // BMN: the weight operand is read from its [contraction, output] layout (dX = dYq . Wq with Wq
          // [N, K] as stored): boxes of 128 contraction rows x 128 output bytes, coordinates swapped
          if (PAIR) {
            // both CTAs' copies report to CTA 0's barrier, which expects the bytes of both
            const uint32_t full0 = map_to_cta(bar_full + 8 * stage, 0u);
            if (cta_rank == 0) mbar_expect_tx(bar_full + 8 * stage, 2u * kStageBytes);
            tma_load_2d_pair(a_dst, &tmap_x, kb * BK, m0, full0);
            if (BMN) tma_load_2d_pair(a_dst + BM * BK, &tmap_w, n0, kb * BK, full0);
            else tma_load_2d_pair(a_dst + BM * BK, &tmap_w, kb * BK, n0, full0);
          } else {
            const uint32_t full = bar_full + 8 * stage;
            mbar_expect_tx(full, kStageBytes);
            tma_load_2d(a_dst, &tmap_x, kb * BK, m0, full);
            if (BMN) {
              tma_load_2d(a_dst + BM * BK, &tmap_w, n0, kb * BK, full);
              tma_load_2d(a_dst + BM * BK + 128 * BK, &tmap_w, n0 + 128, kb * BK, full);
            } else {
              tma_load_2d(a_dst + BM * BK, &tmap_w, kb * BK, n0, full);
            }
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0 && cta_rank == 0) {
      constexpr uint32_t idesc = umma_idesc_i8(TILE_M, BN) | (BMN ? (1u << 16) : 0u);   // bit 16: B is MN-major
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int it = 0;
      for (int tile = worker; ok && tile < num_tiles; tile += num_workers, ++it) {
        const int buf = it & 1;
        const uint32_t use_parity = static_cast<uint32_t>(it >> 1) & 1u;
        if (!mbar_wait<4>(bar_tempty + 8 * buf, use_parity ^ 1u, wctx, W_TMEM_EMPTY, it)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(buf * BN);
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!mbar_wait<8>(bar_full + 8 * stage, phase, wctx, W_FULL, kb)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = smem_base + stage * kStageBytes;
          const uint64_t a_desc = umma_desc_k128(a_addr);
          const uint64_t b_desc = BMN ? umma_desc_mn128(a_addr + BM * BK, 128u * BK) : umma_desc_k128(a_addr + BM * BK);
          // advancing K by 32: +32 bytes inside the 128B swizzle row of a K-major operand (+2 in the
          // address field); four 8-row groups = 4096 bytes further in an MN-major one (+256)
          constexpr uint32_t kb_step = BMN ? 256u : 2u;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            if (PAIR) umma_i8_pair(d_tmem, a_desc + 2u * k, b_desc + kb_step * k, idesc, (kb | k) != 0 ? 1u : 0u);
            else umma_i8(d_tmem, a_desc + 2u * k, b_desc + kb_step * k, idesc, (kb | k) != 0 ? 1u : 0u);
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
    // column operands of a tile: this thread's column scale and bias (BN = one column per epilogue
    // thread) and its RMAX elements of the scaled LoRA factor, element i = e * 256 + et of the
    // [256][RMAX] tile
    constexpr int RD = RMAX > 0 ? RMAX : 1;
    constexpr int PER = RMAX > 0 ? BN * RD / kEpiThreads : 1;
    constexpr bool FMA_LORA = L::kFmaLora;
    static_assert(BN == kEpiThreads, "one column per epilogue thread");
    float sw_pre = 0.f, bias_pre = 0.f;
    float b_pre[PER];
    auto load_cols = [&](int tile_) {
      const int n0_ = (tile_ % p.tiles_n) * BN;
      const int col = n0_ + et;
      const bool in = col < p.N;
      sw_pre = in ? (p.sw ? __ldg(p.sw + col) : 1.0f) : 0.0f;
      bias_pre = (in && p.bias) ? __ldg(p.bias + col) : 0.0f;
      if constexpr (FMA_LORA) {
        // this thread's column of the factor: RMAX consecutive floats of row `col`
        const float* brow = p.Bm + static_cast<int64_t>(in ? col : 0) * p.ldb;
#pragma unroll
        for (int j = 0; j < RD; ++j) {
          const bool inb = in && j < p.rank;
          const float b = __ldg(brow + (inb ? j : 0));
          b_pre[j] = inb ? p.lora_scale * b : 0.0f;
        }
      } else if (RMAX > 0) {
#pragma unroll
        for (int e = 0; e < PER; ++e) {
          const int i = e * kEpiThreads + et;
          const int n = i / RD, j = i % RD;
          const bool inb = n0_ + n < p.N && j < p.rank;
          const float b = __ldg(p.Bm + static_cast<int64_t>(inb ? n0_ + n : 0) * p.ldb + (inb ? j : 0));
          b_pre[e] = inb ? p.lora_scale * b : 0.0f;
        }
      }
    };
    if (worker < num_tiles) load_cols(worker);
    // rows of u for the LoRA epilogue, raw fp32 in MMA A-fragment order [mt][k-step][(row g, k lo) (row g+8, k lo)
    // (row g, k hi) (row g+8, k hi)] x 2 consecutive k
    constexpr int KSU = RMAX > 0 ? RMAX / 16 : 1;
    constexpr bool PF_U = RMAX > 0 && RMAX <= 32;      // beyond rank 32 the registers do not allow the look-ahead
    float u_pre[PF_U ? 2 * KSU * 8 : 1];               // (FMA form: RMAX values of this lane's row)
    auto load_u_row = [&](int tile_, float* f) {
      const int m0_ = (tile_ / p.tiles_n) * TILE_M + static_cast<int>(cta_rank) * BM;
      const int r = m0_ + quarter * 32 + lane;
      const bool okr = r < p.M;
      const float* ur = p.u + static_cast<int64_t>(okr ? r : 0) * p.ldu;
#pragma unroll
      for (int j = 0; j < RD; ++j) {
        const bool inj = okr && j < p.rank;
        const float x = __ldg(ur + (inj ? j : 0));
        f[j] = inj ? x : 0.0f;
      }
    };
    auto load_u = [&](int tile_, float* f) {
      const int m0_ = (tile_ / p.tiles_n) * TILE_M + static_cast<int>(cta_rank) * BM;
      const int rb = m0_ + quarter * 32 + (lane >> 2);
      const int q2 = 2 * (lane & 3);
#pragma unroll
      for (int mt = 0; mt < 2; ++mt) {
        const bool ok0 = rb + 16 * mt < p.M, ok1 = rb + 16 * mt + 8 < p.M;
        const float* u0 = p.u + static_cast<int64_t>(ok0 ? rb + 16 * mt : 0) * p.ldu;
        const float* u1 = p.u + static_cast<int64_t>(ok1 ? rb + 16 * mt + 8 : 0) * p.ldu;
#pragma unroll
        for (int ks = 0; ks < KSU; ++ks) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int cc = 16 * ks + q2 + (e >> 1) * 8;
            const bool okr = (e & 1) ? ok1 : ok0;
            const float* ur = (e & 1) ? u1 : u0;
            const float x0 = __ldg(ur + (cc < p.rank ? cc : 0));
            const float x1 = __ldg(ur + (cc + 1 < p.rank ? cc + 1 : 0));
            f[(mt * KSU + ks) * 8 + 2 * e] = (okr && cc < p.rank) ? x0 : 0.0f;
            f[(mt * KSU + ks) * 8 + 2 * e + 1] = (okr && cc + 1 < p.rank) ? x1 : 0.0f;
          }
        }
      }
    };
    if (PF_U && worker < num_tiles) {
      if constexpr (FMA_LORA) load_u_row(worker, u_pre);
      else load_u(worker, u_pre);
    }
    for (int tile = worker; tile < num_tiles; tile += num_workers, ++it) {
      const int m0 = (tile / p.tiles_n) * TILE_M + static_cast<int>(cta_rank) * BM;
      const int n0 = (tile % p.tiles_n) * BN;
      const int buf = it & 1;
      const uint32_t use_parity = static_cast<uint32_t>(it >> 1) & 1u;

      // Per-column operands of this tile.  They were requested one tile ahead (below, and before
      // the loop for the first tile), so only the conversion and the shared-memory stores sit
      // between the two barriers; the previous tile's readers have passed the first one.
      named_bar_sync(1, kEpiThreads);
      if (ok) {
        sw_s[et] = sw_pre;
        bias_s[et] = bias_pre;
        if constexpr (FMA_LORA) {
          float* bt = reinterpret_cast<float*>(lora_h);
#pragma unroll
          for (int j = 0; j < RD; ++j) bt[j * BN + et] = b_pre[j];      // consecutive threads, consecutive banks
        } else if (RMAX > 0) {
#pragma unroll
          for (int e = 0; e < PER; ++e) {
            const int i = e * kEpiThreads + et;
            const int n = i / RD, j = i % RD;
            const __nv_bfloat16 bh = __float2bfloat16_rn(b_pre[e]);
            lora_h[n * L::kLoraRow + j] = bh;
            lora_l[n * L::kLoraRow + j] = __float2bfloat16_rn(b_pre[e] - __bfloat162float(bh));
          }
        }
      }
      named_bar_sync(1, kEpiThreads);
      if (tile + num_workers < num_tiles) load_cols(tile + num_workers);

      if constexpr (RMAX == 0) {
        // ---------------- plain epilogue: one accumulator row per lane, 32 columns at a time
        const int row = m0 + quarter * 32 + lane;
        const bool row_ok = row < p.M;
        const float sxr = (row_ok && p.sx) ? __ldg(p.sx + row) : 1.0f;

        // one waiter per warp (waking many threads off one mbarrier is slow); tcgen05.ld is
        // warp-collective, so the outcome is shared by the whole warp
        if (ok && lane == 0) ok = mbar_wait<4>(bar_tfull + 8 * buf, use_parity, wctx, W_TMEM_FULL, it);
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
      } else if constexpr (FMA_LORA) {
        // ---------------- adapter epilogue for ranks up to 32: the plain epilogue's layout (one accumulator row
        // per lane, 32 columns at a time, 16-byte stores) with the adapter term u . (scale B)^T added on the
        // fp32 pipe: per rank j one packed fma per pair of columns, the factor's four neighbouring columns by
        // one broadcast shared-memory load.  Exact fp32 products; the tensor pipe is left to the main loop
        // (legacy warp-level MMAs here slowed it down: they share the pipe with tcgen05.mma).
        const int row = m0 + quarter * 32 + lane;
        const bool row_ok = row < p.M;
        const float sxr = (row_ok && p.sx) ? __ldg(p.sx + row) : 1.0f;
        float u_row[RD];
#pragma unroll
        for (int j = 0; j < RD; ++j) u_row[j] = u_pre[j];
        if (tile + num_workers < num_tiles) load_u_row(tile + num_workers, u_pre);

        if (ok && lane == 0) ok = mbar_wait<4>(bar_tfull + 8 * buf, use_parity, wctx, W_TMEM_FULL, it);
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) continue;
        tc_fence_after();
        const uint32_t t_addr = tmem_base + static_cast<uint32_t>(buf * BN) +
                                (static_cast<uint32_t>(quarter * 32) << 16);
        __nv_bfloat16* yrow = p.y + static_cast<int64_t>(row_ok ? row : 0) * p.ldy + n0;
        const float* bt = reinterpret_cast<const float*>(lora_h);

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
          uint64_t t2[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            float tv[2];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              const int cj = c * 32 + 2 * j + h;
              float t = __fmul_rn(static_cast<float>(static_cast<int32_t>(acc[2 * j + h])), sxr);
              t = __fmul_rn(t, sw_s[cj]);
              t = __fadd_rn(t, bias_s[cj]);
              if (p.act == K2Q_ACT_GELU_TANH) t = gelu_tanh_f(t);
              tv[h] = t;
            }
            t2[j] = pack_f32x2(tv[0], tv[1]);
          }
#pragma unroll
          for (int j = 0; j < RD; ++j) {
            const uint64_t uj = pack_f32x2(u_row[j], u_row[j]);
            const float4* bj = reinterpret_cast<const float4*>(bt + j * BN + c * 32);
#pragma unroll
            for (int g = 0; g < 8; ++g) {
              const float4 b = bj[g];
              t2[2 * g] = fma_f32x2(uj, pack_f32x2(b.x, b.y), t2[2 * g]);
              t2[2 * g + 1] = fma_f32x2(uj, pack_f32x2(b.z, b.w), t2[2 * g + 1]);
            }
          }
          if (row_ok) {
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              if (n0 + c * 32 + g * 8 + 8 <= p.N) {
                float v[8];
#pragma unroll
                for (int q = 0; q < 4; ++q) unpack_f32x2(t2[4 * g + q], v[2 * q], v[2 * q + 1]);
                uint4 o;
                o.x = pack_bf16x2(v[0], v[1]);
                o.y = pack_bf16x2(v[2], v[3]);
                o.z = pack_bf16x2(v[4], v[5]);
                o.w = pack_bf16x2(v[6], v[7]);
                *reinterpret_cast<uint4*>(yrow + c * 32 + g * 8) = o;
              }
            }
          }
        }
      } else {
        // ---------------- LoRA epilogue: everything in the register layout of an m16n8 MMA
        // accumulator (lane = 4 g + q holds rows g and g + 8, columns 2q and 2q + 1 of every n8
        // tile).  The int32 accumulator is read from TMEM in that layout (16x256b loads), the
        // adapter term u.B^T is computed in it by warp-level bf16 MMAs on split-precision operands
        // (hi.hi + hi.lo + lo.hi, error ~2^-16 relative), and the sum is stored from it: nothing
        // is transposed through shared memory.
        constexpr int KS = RMAX / 16;
        const int fg = lane >> 2, fq = lane & 3;
        const int rbase = m0 + quarter * 32 + fg;          // rows rbase + 16 mt + 8 h
        float sxf[2][2];
        bool rok[2][2];
#pragma unroll
        for (int mt = 0; mt < 2; ++mt)
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const int r = rbase + 16 * mt + 8 * h;
            rok[mt][h] = r < p.M;
            sxf[mt][h] = (rok[mt][h] && p.sx) ? __ldg(p.sx + r) : 1.0f;
          }
        // the warp's 32 rows of u as A fragments (two 16-row tiles, RMAX/16 k-steps), high and low parts;
        // for ranks up to 32 the raw values were requested one tile ahead
        uint32_t ah[2][KS][4], al[2][KS][4];
        {
          float u_now[PF_U ? 1 : 2 * KSU * 8];
          if (!PF_U) load_u(tile, u_now);
          const float* f = PF_U ? u_pre : u_now;
#pragma unroll
          for (int mt = 0; mt < 2; ++mt)
#pragma unroll
            for (int ks = 0; ks < KS; ++ks)
#pragma unroll
              for (int e = 0; e < 4; ++e)
                split2(f[(mt * KSU + ks) * 8 + 2 * e], f[(mt * KSU + ks) * 8 + 2 * e + 1], ah[mt][ks][e], al[mt][ks][e]);
          if (PF_U && tile + num_workers < num_tiles) load_u(tile + num_workers, u_pre);
        }

        if (ok && lane == 0) ok = mbar_wait<4>(bar_tfull + 8 * buf, use_parity, wctx, W_TMEM_FULL, it);
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) continue;
        tc_fence_after();
        const uint32_t t_addr = tmem_base + static_cast<uint32_t>(buf * BN) +
                                (static_cast<uint32_t>(quarter * 32) << 16);
        // even q stores row g, odd q row g + 8 (after the pair exchange below): 4 columns = 8 bytes
        const int srow = rbase + 8 * (fq & 1);
        __nv_bfloat16* ybase = p.y + n0 + 2 * (fq & 2);

#pragma unroll 1
        for (int c = chunk0; c < chunk0 + BN / 64; ++c) {
          uint32_t accf[2][16];
          tmem_ld_frag16x32(t_addr + c * 32, accf[0]);
          tmem_ld_frag16x32(t_addr + (16u << 16) + c * 32, accf[1]);
          // delta[32 rows][32 columns] while the accumulator loads are in flight; consecutive MMAs
          // go to different accumulators
          float cf[2][4][4];
#pragma unroll
          for (int mt = 0; mt < 2; ++mt)
#pragma unroll
            for (int nt = 0; nt < 4; ++nt)
#pragma unroll
              for (int e = 0; e < 4; ++e) cf[mt][nt][e] = 0.0f;
#pragma unroll
          for (int ks = 0; ks < KS; ++ks) {
            uint32_t bh[4][2], bl[4][2];
#pragma unroll
            for (int nt = 0; nt < 4; ++nt) {
              const int boff = (c * 32 + 8 * nt + fg) * static_cast<int>(L::kLoraRow) + 2 * fq + 16 * ks;
              const uint32_t* ph = reinterpret_cast<const uint32_t*>(lora_h + boff);
              const uint32_t* pl = reinterpret_cast<const uint32_t*>(lora_l + boff);
              bh[nt][0] = ph[0]; bh[nt][1] = ph[4];
              bl[nt][0] = pl[0]; bl[nt][1] = pl[4];
            }
#pragma unroll
            for (int nt = 0; nt < 4; ++nt)
#pragma unroll
              for (int mt = 0; mt < 2; ++mt) mma_bf16_16816(cf[mt][nt], ah[mt][ks], bh[nt][0], bh[nt][1]);
#pragma unroll
            for (int nt = 0; nt < 4; ++nt)
#pragma unroll
              for (int mt = 0; mt < 2; ++mt) mma_bf16_16816(cf[mt][nt], ah[mt][ks], bl[nt][0], bl[nt][1]);
#pragma unroll
            for (int nt = 0; nt < 4; ++nt)
#pragma unroll
              for (int mt = 0; mt < 2; ++mt) mma_bf16_16816(cf[mt][nt], al[mt][ks], bh[nt][0], bh[nt][1]);
          }
          tmem_ld_wait();
          if (c == chunk0 + BN / 64 - 1) {  // this warp has read its half of the accumulator
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
              if (PAIR) mbar_arrive_cluster(tempty0 + 8 * buf);
              else mbar_arrive(bar_tempty + 8 * buf);
            }
          }
#pragma unroll
          for (int nt = 0; nt < 4; ++nt) {
            const int cj = c * 32 + 8 * nt + 2 * fq;
            const float2 sw2 = *reinterpret_cast<const float2*>(sw_s + cj);
            const float2 bi2 = *reinterpret_cast<const float2*>(bias_s + cj);
#pragma unroll
            for (int mt = 0; mt < 2; ++mt) {
              uint32_t pk[2];
#pragma unroll
              for (int h = 0; h < 2; ++h) {
                float t0 = __fmul_rn(static_cast<float>(static_cast<int32_t>(accf[mt][4 * nt + 2 * h])), sxf[mt][h]);
                float t1 = __fmul_rn(static_cast<float>(static_cast<int32_t>(accf[mt][4 * nt + 2 * h + 1])), sxf[mt][h]);
                t0 = __fadd_rn(__fmul_rn(t0, sw2.x), bi2.x);
                t1 = __fadd_rn(__fmul_rn(t1, sw2.y), bi2.y);
                if (p.act == K2Q_ACT_GELU_TANH) {
                  t0 = gelu_tanh_f(t0);
                  t1 = gelu_tanh_f(t1);
                }
                pk[h] = pack_bf16x2(t0 + cf[mt][nt][2 * h], t1 + cf[mt][nt][2 * h + 1]);
              }
              // lanes q and q^1 swap one pair: the even lane ends up with four consecutive columns of
              // row g, the odd lane with the same four columns of row g + 8
              const uint32_t got = __shfl_xor_sync(0xffffffffu, (fq & 1) ? pk[0] : pk[1], 1);
              const uint2 o = (fq & 1) ? make_uint2(got, pk[1]) : make_uint2(pk[0], got);
              const int r = srow + 16 * mt;
              if (r < p.M && n0 + c * 32 + 8 * nt < p.N)
                *reinterpret_cast<uint2*>(ybase + static_cast<int64_t>(r) * p.ldy + c * 32 + 8 * nt) = o;
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

// FMA: the adapter term on the fp32 pipe (ranks up to 32) instead of warp-level MMAs.  Measured with the
// main loop running beside it (CTA pairs): for rank <= 16 it wins on large problems (M = 36864: 1.08x the
// plain GEMM against 1.19x at N = K = 6144) and loses a little on small ones (M = 4096, N = K = 3072: 1.37x
// against 1.30x); for ranks 17..32 it wins only when the contraction is long enough (K >= 12288) to hide twice
// the fp32 work per tile.  The host picks accordingly.
template <int STAGES, int RMAX, bool PAIR, bool BMN = false, bool FMA = false>
int launch(const CUtensorMap& tx, const CUtensorMap& tw, const GemmParams& p, int grid, cudaStream_t stream) {
  using L = Smem<STAGES, RMAX, PAIR, FMA>;
  static_assert(L::kBytes <= 232448, "shared memory budget exceeded");
  auto kern = gemm_w8a8_kernel<STAGES, RMAX, PAIR, BMN, FMA>;
  if (int rc = check_cuda(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kBytes),
                          "cudaFuncSetAttribute(gemm_w8a8)"))
    return rc;
  // ordinary stream order: an overlapped start (launch_overlapped) measured slower for this kernel in the
  // host-buffer pipeline (1.32 -> 1.48 ms per call) and no faster device-resident
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

namespace {

// Shared host side of the two entry points.  bmn = false: wq is [N, K] with the contraction index K
// contiguous (forward).  bmn = true: wq is [K, N], contraction index first (dX through the stored
// [out, in] codes): the kernel reads it as an MN-major operand.
int gemm_w8a8_impl(const char* who, const int8_t* xq, const int8_t* wq, const float* sw, int64_t M, int64_t N,
                   int64_t K, const k2q_epilogue* ep, void* y_bf16, int64_t ldy, void* status, void* stream,
                   bool bmn) {
  if (int rc = check_device_arch()) return rc;
  if (M < 0 || N <= 0 || K <= 0 || M > 0x7fffff00LL || N > 0x7fffff00LL || K > 0x7fffff00LL)
    return fail(K2Q_EINVAL, "%s: bad shape M=%lld N=%lld K=%lld", who, (long long)M, (long long)N, (long long)K);
  if (K % 128 != 0) return fail(K2Q_EINVAL, "%s: contraction length %lld is not a multiple of 128", who, (long long)K);
  if (N % 16 != 0) return fail(K2Q_EINVAL, "%s: N=%lld is not a multiple of 16", who, (long long)N);
  if (M == 0) return K2Q_OK;
  if (!xq || !wq || !y_bf16 || !status) return fail(K2Q_EINVAL, "%s: NULL operand", who);
  if (ldy < N || (ldy % 8) != 0 || (reinterpret_cast<uintptr_t>(y_bf16) & 15u))
    return fail(K2Q_EINVAL, "%s: y must be 16-byte aligned with ldy >= N and ldy %% 8 == 0", who);
  k2q_epilogue e{};
  if (ep) e = *ep;
  if (e.rank < 0 || e.rank > 64) return fail(K2Q_EINVAL, "%s: LoRA rank %d not in [0,64]", who, e.rank);
  if ((e.u == nullptr) != (e.Bm == nullptr) || ((e.u != nullptr) != (e.rank > 0)))
    return fail(K2Q_EINVAL, "%s: u, Bm and rank must be given together", who);
  if (e.rank > 0 && (e.ldu < e.rank || e.ldb < e.rank)) return fail(K2Q_EINVAL, "%s: ldu/ldb smaller than rank", who);
  if (e.act != K2Q_ACT_NONE && e.act != K2Q_ACT_GELU_TANH) return fail(K2Q_EINVAL, "%s: unknown activation %d", who, e.act);

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
  if (bmn) {
    if (int rc = encode_tmap_2d_u8(&tw, wq, (uint64_t)N, (uint64_t)K, (uint64_t)N, 128, BK, 1)) return rc;
  } else {
    if (int rc = encode_tmap_2d_u8(&tw, wq, (uint64_t)K, (uint64_t)N, (uint64_t)K, BK, pair ? BN / 2 : BN, 1)) return rc;
  }

  const int sms = sm_count();
  if (sms <= 0) return fail(K2Q_ECUDA, "%s: could not read the SM count", who);
  const int64_t tiles = (int64_t)p.tiles_m * p.tiles_n;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (pair) {
    const int64_t pairs = tiles < sms / 2 ? tiles : sms / 2;
    const int grid = (int)(2 * pairs);
    if (bmn) {
      if (e.rank == 0) return launch<6, 0, true, true>(tx, tw, p, grid, s);
      if (e.rank <= 16) return M >= 8192 ? launch<6, 16, true, true, true>(tx, tw, p, grid, s)
                                         : launch<6, 16, true, true>(tx, tw, p, grid, s);
      if (e.rank <= 32) return K >= 12288 ? launch<5, 32, true, true, true>(tx, tw, p, grid, s)
                                          : launch<5, 32, true, true>(tx, tw, p, grid, s);
      return launch<4, 64, true, true>(tx, tw, p, grid, s);
    }
    if (e.rank == 0) return launch<6, 0, true>(tx, tw, p, grid, s);
    if (e.rank <= 16) return M >= 8192 ? launch<6, 16, true, false, true>(tx, tw, p, grid, s)
                                       : launch<6, 16, true>(tx, tw, p, grid, s);
    if (e.rank <= 32) return K >= 12288 ? launch<5, 32, true, false, true>(tx, tw, p, grid, s)
                                        : launch<5, 32, true>(tx, tw, p, grid, s);
    return launch<4, 64, true>(tx, tw, p, grid, s);
  }
  const int grid = (int)(tiles < sms ? tiles : sms);
  if (bmn) {
    if (e.rank == 0) return launch<4, 0, false, true>(tx, tw, p, grid, s);
    if (e.rank <= 16) return launch<4, 16, false, true>(tx, tw, p, grid, s);
    if (e.rank <= 32) return launch<3, 32, false, true>(tx, tw, p, grid, s);
    return launch<3, 64, false, true>(tx, tw, p, grid, s);
  }
  if (e.rank == 0) return launch<4, 0, false>(tx, tw, p, grid, s);
  if (e.rank <= 16) return launch<4, 16, false>(tx, tw, p, grid, s);
  if (e.rank <= 32) return launch<3, 32, false>(tx, tw, p, grid, s);
  return launch<3, 64, false>(tx, tw, p, grid, s);
}

}  // namespace

extern "C" int k2q_gemm_w8a8(const int8_t* xq, const int8_t* wq, const float* sw, int64_t M, int64_t N,
                             int64_t K, const k2q_epilogue* ep, void* y_bf16, int64_t ldy, void* status,
                             void* stream) {
  return gemm_w8a8_impl("k2q_gemm_w8a8", xq, wq, sw, M, N, K, ep, y_bf16, ldy, status, stream, false);
}

extern "C" int k2q_gemm_dx_w8(const int8_t* gq, const int8_t* wq, int64_t M, int64_t N, int64_t K,
                              const k2q_epilogue* ep, void* dx_bf16, int64_t lddx, void* status, void* stream) {
  // dX[M, K] = epilogue(gq[M, N] . wq[N, K]): contraction over N (a multiple of 128), output columns K
  if (N % 128 != 0)
    return fail(K2Q_EINVAL, "k2q_gemm_dx_w8: N=%lld (the contraction) is not a multiple of 128", (long long)N);
  return gemm_w8a8_impl("k2q_gemm_dx_w8", gq, wq, nullptr, M, /*output columns*/ K, /*contraction*/ N, ep, dx_bf16,
                        lddx, status, stream, true);
}
