// K4: W4A8 GEMM (group-128 int4 weights x per-token int8 activations) on tcgen05 int8 tensor
// cores.  The scale of a weight group varies along K, so each 128-wide K-block ("slab") is
// accumulated on its own in TMEM and folded into fp32 running sums by the epilogue warps:
//     run[n,m] += float(acc_g[n,m]) * sw4[n,g]            (g ascending, fp32 mul then fp32 add)
//     y[m,n]    = act(run*sx[m] + bias[n]) + lora
// The product is computed TRANSPOSED (D = W_tile . X_tile^T: TMEM lane = output channel n,
// TMEM column = token m) so that the group scale is one scalar per epilogue thread.
//
// int32 -> fp32 without a conversion instruction: the converters emit code*16 (the nibble moved
// to the high half of the byte) and every slab accumulator starts from the bit pattern of
// 1.5*2^19, whose ulp is 1/16.  The finished accumulator, read as a float, is then exactly
// 786432 + acc, and  fma(v, s, -786432*s)  yields round(acc*s), the same value a convert and a
// multiply would give (786432*s is exact for a bf16 s).  The epilogue uses packed fp32 pairs.
//
// 512 threads (four warpgroups) per CTA, one CTA per SM, persistent over 128(n) x 128(m) tiles;
// setmaxnreg moves registers from the data-movement warpgroups to the two epilogue warpgroups.
// One mbarrier hand-off costs a few hundred cycles, about as long as a slab's MMAs, so the
// pipeline is deep: six load slots, four unpacked-operand buffers, four TMEM accumulators.
//   warp 0 lane 0   TMA producer: packed int4 tile [128 n x 64 B] (no swizzle) + xq tile
//                   [128 m x 128 B] (SWIZZLE_128B) per slab into a ring of 6 slots
//   warp 1 lane 0   MMA issuer: per slab four tcgen05.mma kind::i8 (M128 N128 K32) into one of
//                   four 128-column TMEM accumulators
//   warps 4..7      converters: unpack the int4 tile into one of four 128B-swizzled int8 buffers;
//                   fence.proxy.async; signal the MMA issuer
//   warps 8..15     epilogue: warps 8..11 own token columns 0..63 of the tile, warps 12..15 columns
//                   64..127; tcgen05.ld, running sums in registers, accumulator reset (tcgen05.st),
//                   final scale/bias/act/LoRA, bf16 stores
// Every mbarrier wait is bounded; on expiry the CTA drains and exits (k2q_common.cuh).
#include "k2q_common.cuh"

namespace k2q {
namespace {

constexpr int TN = 128;   // output channels per tile (UMMA M, TMEM lanes)
constexpr int TM = 128;   // tokens per tile (UMMA N, TMEM columns)
constexpr int BK = 128;   // one weight group per slab
constexpr int UMMA_K = 32;
constexpr int kThreads = 512;
constexpr int kConvThreads = 128;
constexpr int kConvWarps = kConvThreads / 32;
constexpr int kEpiThreads = 256;
constexpr int kEpiWarps = kEpiThreads / 32;
constexpr int NBUF = 4;          // TMEM accumulators of TM columns
constexpr int LSTAGES = 6;       // load ring (packed W + xq)
constexpr int CSTAGES = 4;       // unpacked-W ring
constexpr uint32_t kTmemCols = NBUF * TM;                     // 512
constexpr uint32_t kPackedBytes = TN * BK / 2;                // 8192
constexpr uint32_t kXBytes = TM * BK;                         // 16384
constexpr uint32_t kLoadStage = kPackedBytes + kXBytes;       // 24576
constexpr uint32_t kWBytes = TN * BK;                         // 16384 unpacked
constexpr uint32_t kAccInit = 0x49400000u;                    // bits of 786432.0f = 1.5 * 2^19
constexpr float kAccBias = 786432.0f;

enum WaitId : int {
  W_EMPTY = 201,       // producer: load slot free
  W_FULL_CONV = 202,   // converter: TMA data landed
  W_CONV_EMPTY = 203,  // converter: unpacked buffer free
  W_FULL_MMA = 204,    // MMA issuer: TMA data landed
  W_CONV_FULL = 205,   // MMA issuer: unpacked tile ready
  W_ACC_EMPTY = 206,   // MMA issuer: accumulator set released (and reset)
  W_ACC_FULL = 207,    // epilogue: slab accumulated
  W_SMEM_ALIGN = 208
};

struct Gemm4Params {
  int M, N, K;
  int tiles_m, tiles_n;
  const __nv_bfloat16* sw4;  // [N, K/128]
  const float* sx;
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

template <int RMAX>
struct Smem4 {
  static constexpr uint32_t kLoadOff = 0;                                  // LSTAGES x [xq | packed]
  static constexpr uint32_t kConvOff = LSTAGES * kLoadStage;               // CSTAGES x unpacked W
  static constexpr uint32_t kSxOff = kConvOff + CSTAGES * kWBytes;         // sx_s[TM]
  static constexpr uint32_t kUOff = kSxOff + TM * 4;                       // u_s[TM][RMAX]
  static constexpr uint32_t kBarOff = kUOff + TM * RMAX * 4;
  static constexpr uint32_t kNumBars = 2 * LSTAGES + 2 * CSTAGES + 2 * NBUF;
  static constexpr uint32_t kBytes = kBarOff + kNumBars * 8 + 16;
};

__device__ __forceinline__ float gelu_tanh4(float v) {
  // 0.5 v (1 + tanh(sqrt(2/pi) (v + 0.044715 v^3))) with the hardware tanh (|error| < 6e-4, far below
  // the bf16 resolution of the output)
  const float z = v * fmaf(0.0356774081f, v * v, 0.7978845608f);
  float th;
  asm("tanh.approx.f32 %0, %1;" : "=f"(th) : "f"(z));
  const float hv = 0.5f * v;
  return fmaf(hv, th, hv);
}

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t r;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
  return r;
}

template <int RMAX>
__global__ void __launch_bounds__(kThreads, 1)
gemm_w4a8_kernel(const __grid_constant__ CUtensorMap tmap_w4, const __grid_constant__ CUtensorMap tmap_x,
                 const Gemm4Params p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  using L = Smem4<RMAX>;
  constexpr int RD = RMAX > 0 ? RMAX : 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t smem_base = smem_u32(smem);

  float* sx_s = reinterpret_cast<float*>(smem + L::kSxOff);
  float* u_s = reinterpret_cast<float*>(smem + L::kUOff);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBarOff);
  const uint32_t bar_full = smem_u32(bars);                  // [LSTAGES] TMA landed
  const uint32_t bar_empty = bar_full + 8 * LSTAGES;         // [LSTAGES] MMAs have read the slot
  const uint32_t bar_cfull = bar_empty + 8 * LSTAGES;        // [CSTAGES] unpacked tile written
  const uint32_t bar_cempty = bar_cfull + 8 * CSTAGES;       // [CSTAGES] MMAs have read it
  const uint32_t bar_afull = bar_cempty + 8 * CSTAGES;       // [NBUF]
  const uint32_t bar_aempty = bar_afull + 8 * NBUF;          // [NBUF]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + L::kNumBars);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  if ((smem_base & 1023u) != 0u) {
    if (threadIdx.x == 0 && atomicCAS(&p.status->code, 0, W_SMEM_ALIGN) == 0) {
      p.status->block = static_cast<int>(blockIdx.x);
      p.status->detail = static_cast<int>(smem_base & 1023u);
    }
    return;
  }

  if (threadIdx.x == 0) {
    for (int s = 0; s < LSTAGES; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int s = 0; s < CSTAGES; ++s) {
      mbar_init(bar_cfull + 8 * s, kConvWarps);   // one arrival per warp
      mbar_init(bar_cempty + 8 * s, 1);
    }
    for (int b = 0; b < NBUF; ++b) {
      mbar_init(bar_afull + 8 * b, 1);
      mbar_init(bar_aempty + 8 * b, kEpiWarps);
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap_w4);
    tma_prefetch_desc(&tmap_x);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const WaitCtx wctx{abort_flag, p.status};
  const int num_tiles = p.tiles_m * p.tiles_n;
  const int slabs = p.K / BK;

  auto slot_x = [&](int s) { return smem_base + L::kLoadOff + s * kLoadStage; };
  auto slot_p = [&](int s) { return smem_base + L::kLoadOff + s * kLoadStage + kXBytes; };
  auto slot_w = [&](int c) { return smem_base + L::kConvOff + c * kWBytes; };

  // Register re-partition (warpgroup-collective, first statement of each role branch):
  // 40 per thread for the TMA/MMA warpgroup, 72 for the converters, 200 for the epilogue.
  if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
    if (warp == 0) {
      // ---------------------------------------------------------------- TMA producer
      if (lane == 0) {
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
          const int n0 = (tile % p.tiles_n) * TN;
          const int m0 = (tile / p.tiles_n) * TM;
          for (int g = 0; g < slabs; ++g) {
            if (!mbar_wait(bar_empty + 8 * stage, phase ^ 1u, wctx, W_EMPTY, g)) { ok = false; break; }
            const uint32_t full = bar_full + 8 * stage;
            mbar_expect_tx(full, kLoadStage);
            tma_load_2d(slot_x(stage), &tmap_x, g * BK, m0, full);
            tma_load_2d(slot_p(stage), &tmap_w4, g * (BK / 2), n0, full);
            if (++stage == LSTAGES) { stage = 0; phase ^= 1u; }
          }
        }
      }
    } else if (warp == 1) {
      // ---------------------------------------------------------------- MMA issuer
      if (lane == 0) {
        constexpr uint32_t idesc = umma_idesc_i8(128, TM);
        int stage = 0, cst = 0;
        uint32_t phase = 0, cphase = 0;
        uint32_t slab = 0;  // running slab count of this CTA -> accumulator set
        bool ok = true;
        for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
          for (int g = 0; g < slabs; ++g, ++slab) {
            const uint32_t buf = slab % NBUF;
            const uint32_t use_parity = (slab / NBUF) & 1u;
            // the accumulator must have been drained AND reset to the bias pattern by the epilogue
            if (!mbar_wait(bar_aempty + 8 * buf, use_parity, wctx, W_ACC_EMPTY, g)) { ok = false; break; }
            if (!mbar_wait(bar_full + 8 * stage, phase, wctx, W_FULL_MMA, g)) { ok = false; break; }
            if (!mbar_wait(bar_cfull + 8 * cst, cphase, wctx, W_CONV_FULL, g)) { ok = false; break; }
            tc_fence_after();
            const uint64_t a_desc = umma_desc_k128(slot_w(cst));
            const uint64_t b_desc = umma_desc_k128(slot_x(stage));
            const uint32_t d_tmem = tmem_base + buf * TM;
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k)
              umma_i8(d_tmem, a_desc + 2u * k, b_desc + 2u * k, idesc, 1u);
            tc_commit(bar_empty + 8 * stage);
            tc_commit(bar_cempty + 8 * cst);
            tc_commit(bar_afull + 8 * buf);
            if (++stage == LSTAGES) { stage = 0; phase ^= 1u; }
            if (++cst == CSTAGES) { cst = 0; cphase ^= 1u; }
          }
        }
      }
    }
  } else if (warp < 8) {
    // ------------------------------------------------------------------ int4 -> int8 converters
    asm volatile("setmaxnreg.dec.sync.aligned.u32 72;");
    const int cw = warp - 4;  // rows 32*cw .. 32*cw+31 of the tile
    int stage = 0, cst = 0;
    uint32_t phase = 0, cphase = 0;
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
      for (int g = 0; g < slabs; ++g) {
        if (lane == 0) {  // one waiter per warp, outcome shared below
          ok = mbar_wait(bar_full + 8 * stage, phase, wctx, W_FULL_CONV, g);
          if (ok) ok = mbar_wait(bar_cempty + 8 * cst, cphase ^ 1u, wctx, W_CONV_EMPTY, g);
        }
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) break;
        const uint8_t* src = smem + (slot_p(stage) - smem_base);
        uint8_t* dst = smem + (slot_w(cst) - smem_base);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int r = cw * 32 + i * 8 + (lane >> 2);  // row of the tile
          const int c = lane & 3;                       // 16-byte packed chunk = codes 32c..32c+31
          const uint4 pk = *reinterpret_cast<const uint4*>(src + r * 64 + c * 16);
          const uint32_t w[4] = {pk.x, pk.y, pk.z, pk.w};
          uint32_t o[8];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const uint32_t lo = (w[j] << 4) & 0xF0F0F0F0u;  // even codes, value*16 as int8
            const uint32_t hi = w[j] & 0xF0F0F0F0u;         // odd codes
            o[2 * j] = prmt(lo, hi, 0x5140u);
            o[2 * j + 1] = prmt(lo, hi, 0x7362u);
          }
          // 128B swizzle: 16-byte chunk index XOR (row mod 8)
          const int ch0 = (2 * c) ^ (r & 7), ch1 = (2 * c + 1) ^ (r & 7);
          *reinterpret_cast<uint4*>(dst + r * 128 + ch0 * 16) = make_uint4(o[0], o[1], o[2], o[3]);
          *reinterpret_cast<uint4*>(dst + r * 128 + ch1 * 16) = make_uint4(o[4], o[5], o[6], o[7]);
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_cfull + 8 * cst);
        if (++stage == LSTAGES) { stage = 0; phase ^= 1u; }
        if (++cst == CSTAGES) { cst = 0; cphase ^= 1u; }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue
    asm volatile("setmaxnreg.inc.sync.aligned.u32 200;");
    constexpr int CW = TM / 2;              // token columns per epilogue thread
    const int et = threadIdx.x - 256;       // 0..255
    const int ch = (warp - 8) >> 2;         // which half of the token columns this warp owns
    const int quarter = warp & 3;           // TMEM lane quarter this warp may access
    const int nl = quarter * 32 + lane;
    const uint32_t lane_sel = (static_cast<uint32_t>(quarter * 32) << 16) + ch * CW;

    // all accumulators start from the bias pattern; the first "released" signal carries it
#pragma unroll
    for (int b = 0; b < NBUF; ++b) {
#pragma unroll
      for (int c = 0; c < CW / 32; ++c) tmem_st32_fill(tmem_base + lane_sel + b * TM + c * 32, kAccInit);
    }
    tmem_st_wait();
    tc_fence_before();
    __syncwarp();
    if (lane == 0) {
#pragma unroll
      for (int b = 0; b < NBUF; ++b) mbar_arrive(bar_aempty + 8 * b);
    }

    uint32_t slab = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
      const int n0 = (tile % p.tiles_n) * TN;
      const int m0 = (tile / p.tiles_n) * TM;
      const int n = n0 + nl;
      const bool n_ok = n < p.N;

      named_bar_sync(1, kEpiThreads);
      if (ok) {
        if (et < TM) {
          const int m = m0 + et;
          sx_s[et] = (m < p.M) ? (p.sx ? __ldg(p.sx + m) : 1.0f) : 0.0f;
        }
        if (RMAX > 0) {
          for (int i = et; i < TM * RMAX; i += kEpiThreads) {
            const int mm = i / RD, j = i % RD;
            u_s[i] = (m0 + mm < p.M && j < p.rank) ? __ldg(p.u + (m0 + mm) * p.ldu + j) : 0.0f;
          }
        }
      }
      named_bar_sync(1, kEpiThreads);

      const float bias_n = (n_ok && p.bias) ? __ldg(p.bias + n) : 0.0f;
      const __nv_bfloat16* swrow = p.sw4 + static_cast<int64_t>(n_ok ? n : 0) * slabs;

      uint64_t run2[CW / 2];
#pragma unroll
      for (int j = 0; j < CW / 2; ++j) run2[j] = 0ull;

      float s_next = n_ok ? __bfloat162float(swrow[0]) : 0.f;
      for (int g = 0; g < slabs; ++g, ++slab) {
        const float s_g = s_next;
        if (g + 1 < slabs) s_next = n_ok ? __bfloat162float(swrow[g + 1]) : 0.f;
        const uint32_t buf = slab % NBUF;
        const uint32_t use_parity = (slab / NBUF) & 1u;
        if (ok && lane == 0) ok = mbar_wait(bar_afull + 8 * buf, use_parity, wctx, W_ACC_FULL, g);
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) continue;
        tc_fence_after();
        const uint32_t s_bits = __float_as_uint(s_g);
        const uint32_t c_bits = __float_as_uint(-__fmul_rn(kAccBias, s_g));   // exact
        const uint64_t s2 = pack_f32x2(s_bits, s_bits), c2 = pack_f32x2(c_bits, c_bits);
        const uint32_t t_addr = tmem_base + lane_sel + buf * TM;
#pragma unroll
        for (int c = 0; c < CW / 32; ++c) {
          uint32_t acc[32];
          tmem_ld32(t_addr + c * 32, acc);
          tmem_ld_wait();
          tmem_st32_fill(t_addr + c * 32, kAccInit);   // reset for the slab after next
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const uint64_t t2 = fma_f32x2(pack_f32x2(acc[2 * j], acc[2 * j + 1]), s2, c2);
            run2[c * 16 + j] = add_f32x2(run2[c * 16 + j], t2);
          }
        }
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_aempty + 8 * buf);
      }
      if (!ok) continue;

      float br[RD];
      if (RMAX > 0) {
#pragma unroll
        for (int j = 0; j < RMAX; ++j)
          br[j] = (n_ok && j < p.rank) ? p.lora_scale * __ldg(p.Bm + n * p.ldb + j) : 0.0f;
      }
      // final scale, bias, activation, adapter term; y is [M, ldy]: a warp writes 32
      // neighbouring channels of one token per store instruction
#pragma unroll
      for (int j2 = 0; j2 < CW / 2; ++j2) {
        float rv[2];
        unpack_f32x2(run2[j2], rv[0], rv[1]);
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int j = ch * CW + 2 * j2 + e;
          float t = __fmul_rn(rv[e], sx_s[j]);
          t = __fadd_rn(t, bias_n);
          if (p.act == K2Q_ACT_GELU_TANH) t = gelu_tanh4(t);
          if (RMAX > 0) {
            const float4* u4 = reinterpret_cast<const float4*>(u_s + j * RD);
            float d = 0.f;
#pragma unroll
            for (int j4 = 0; j4 < RMAX / 4; ++j4) {
              const float4 uu = u4[j4];
              d = fmaf(uu.x, br[4 * j4], d);
              d = fmaf(uu.y, br[4 * j4 + 1], d);
              d = fmaf(uu.z, br[4 * j4 + 2], d);
              d = fmaf(uu.w, br[4 * j4 + 3], d);
            }
            t += d;
          }
          const int m = m0 + j;
          if (n_ok && m < p.M) p.y[static_cast<int64_t>(m) * p.ldy + n] = __float2bfloat16_rn(t);
        }
      }
    }
  }

  // ---------------------------------------------------------------------- teardown
  if (*abort_flag) {
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

template <int RMAX>
int launch4(const CUtensorMap& tw, const CUtensorMap& tx, const Gemm4Params& p, int grid, cudaStream_t stream) {
  using L = Smem4<RMAX>;
  static_assert(L::kBytes <= 232448, "shared memory budget exceeded");
  auto kern = gemm_w4a8_kernel<RMAX>;
  if (int rc = check_cuda(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kBytes),
                          "cudaFuncSetAttribute(gemm_w4a8)"))
    return rc;
  kern<<<grid, kThreads, L::kBytes, stream>>>(tw, tx, p);
  return check_cuda(cudaGetLastError(), "gemm_w4a8 launch");
}

}  // namespace
}  // namespace k2q

using namespace k2q;

extern "C" int k2q_gemm_w4a8(const int8_t* xq, const uint8_t* wq4, const void* sw4_bf16, int64_t M,
                             int64_t N, int64_t K, const k2q_epilogue* ep, void* y_bf16, int64_t ldy,
                             void* status, void* stream) {
  if (int rc = check_device_arch()) return rc;
  if (M < 0 || N <= 0 || K <= 0 || M > 0x7fffff00LL || N > 0x7fffff00LL || K > 0x7fffff00LL)
    return fail(K2Q_EINVAL, "k2q_gemm_w4a8: bad shape M=%lld N=%lld K=%lld", (long long)M, (long long)N,
                (long long)K);
  if (K % 128 != 0) return fail(K2Q_EINVAL, "k2q_gemm_w4a8: K=%lld is not a multiple of 128", (long long)K);
  if (N % 16 != 0) return fail(K2Q_EINVAL, "k2q_gemm_w4a8: N=%lld is not a multiple of 16", (long long)N);
  if (M == 0) return K2Q_OK;
  if (!xq || !wq4 || !sw4_bf16 || !y_bf16 || !status) return fail(K2Q_EINVAL, "k2q_gemm_w4a8: NULL operand");
  if (ldy < N) return fail(K2Q_EINVAL, "k2q_gemm_w4a8: ldy < N");
  k2q_epilogue e{};
  if (ep) e = *ep;
  if (e.rank < 0 || e.rank > 32) return fail(K2Q_EINVAL, "k2q_gemm_w4a8: LoRA rank %d not in [0,32]", e.rank);
  if ((e.u == nullptr) != (e.Bm == nullptr) || ((e.u != nullptr) != (e.rank > 0)))
    return fail(K2Q_EINVAL, "k2q_gemm_w4a8: u, Bm and rank must be given together");
  if (e.rank > 0 && (e.ldu < e.rank || e.ldb < e.rank))
    return fail(K2Q_EINVAL, "k2q_gemm_w4a8: ldu/ldb smaller than rank");
  if (e.act != K2Q_ACT_NONE && e.act != K2Q_ACT_GELU_TANH)
    return fail(K2Q_EINVAL, "k2q_gemm_w4a8: unknown activation %d", e.act);

  Gemm4Params p{};
  p.M = (int)M; p.N = (int)N; p.K = (int)K;
  p.tiles_m = (int)((M + TM - 1) / TM);
  p.tiles_n = (int)((N + TN - 1) / TN);
  p.sw4 = static_cast<const __nv_bfloat16*>(sw4_bf16);
  p.sx = e.sx; p.bias = e.bias;
  p.u = e.u; p.Bm = e.Bm; p.ldu = e.ldu; p.ldb = e.ldb; p.rank = e.rank;
  p.lora_scale = e.lora_scale; p.act = e.act;
  p.y = static_cast<__nv_bfloat16*>(y_bf16); p.ldy = ldy;
  p.status = static_cast<Status*>(status);

  CUtensorMap tw, tx;
  if (int rc = encode_tmap_2d_u8(&tw, wq4, (uint64_t)K / 2, (uint64_t)N, (uint64_t)K / 2, BK / 2, TN, 0)) return rc;
  if (int rc = encode_tmap_2d_u8(&tx, xq, (uint64_t)K, (uint64_t)M, (uint64_t)K, BK, TM, 1)) return rc;

  const int sms = sm_count();
  if (sms <= 0) return fail(K2Q_ECUDA, "k2q_gemm_w4a8: could not read the SM count");
  const int64_t tiles = (int64_t)p.tiles_m * p.tiles_n;
  const int grid = (int)(tiles < sms ? tiles : sms);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (e.rank == 0) return launch4<0>(tw, tx, p, grid, s);
  if (e.rank <= 16) return launch4<16>(tw, tx, p, grid, s);
  return launch4<32>(tw, tx, p, grid, s);
}
