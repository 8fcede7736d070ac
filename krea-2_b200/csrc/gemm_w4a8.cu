// K4: W4A8 GEMM (group-128 int4 weights x per-token int8 activations) on tcgen05 int8 tensor
// cores.  The scale of a weight group varies along K, so each 128-wide K-block ("slab") is
// accumulated on its own in TMEM and folded into fp32 running sums by the epilogue warps:
//     run[n,m] += float(acc_g[n,m]) * sw4[n,g]                   (g ascending)
//     y[m,n]    = act(run*sx[m] + bias[n]) + lora
// The product is computed TRANSPOSED (D = W_tile . X_tile^T: TMEM lane = output channel n,
// TMEM column = token m) so that the group scale is one scalar per epilogue thread, and the weight
// operand is fed to the tensor core FROM TENSOR MEMORY: converter thread r owns channel r of the
// tile, reads its 64 packed bytes of the slab from shared memory, expands them to 128 int8 values
// (code * 16: the nibble moved to the high half of the byte) and writes them to its TMEM lane with
// one tcgen05.st.  Shared memory then carries only the TMA writes, one read of the packed weights
// and the tensor core's reads of the activation tile.
//
// Per tile 128 channels x 192 tokens; TMEM holds four 32-column operand buffers and two 192-column
// accumulators (128 + 384 = 512 columns).
//
// Per slab an epilogue thread folds its 96 accumulator columns as run = fma(float(16 * acc), s / 16,
// run): a cvt and one packed fma per pair of values, one fp32 rounding per slab -- the CPU oracle's
// definition, reproduced bit for bit.  The three 32-column chunks of a slab sit in three register
// buffers; as soon as a chunk has been folded its buffer is refilled with the same chunk of the next
// slab (a non-blocking probe of that slab's barrier was issued one fold earlier), so the barrier
// probe, the tensor-memory reads and the release of the next accumulator overlap the folds.
//
// What bounds the kernel (B200, measured): one conversion per accumulator value and slab on the 16-lane
// ALU pipe, next to the converters' logic and byte permutes and every integer instruction of the
// hand-off sequences: that pipe is 71-76 % busy at 35-42 % tensor activity.  It got there by taking
// instructions OUT of the hot loops: with per-slab index arithmetic (ring index and parity by division,
// buffer addresses by multiplication, a conditional around every request of the next slab) the same
// kernel needed 1290 cycles per slab; rolling addresses, a peeled last slab, one tcgen05.wait::ld
// per slab, a converter loop that runs over all slabs of the CTA, and a last step of the tile without
// per-value address arithmetic or activation tests brought it to 955 (384 cycles of MMAs).  Every
// variant that moved work between pipes at the price of more instructions was slower and is not
// kept: accumulators seeded by a kind::f16 MMA with the bit pattern of 1.53125 * 2^23 so that a packed
// subtraction on the FMA pipe replaces the cvt; the same conversion as an integer multiply-add plus a
// packed subtraction; each slab issued as two N = 96 halves with barriers of their own; the slab loop
// unrolled by two (instruction cache).  All of them were verified bit-exact first.  tcgen05.mma
// kind::i8 rejects the instruction descriptor's negate bits (illegal instruction on B200), which
// rules out cancelling offsets between slabs.
//
// 512 threads (four warpgroups) per CTA, one CTA per SM, persistent; setmaxnreg moves registers to
// the two epilogue warpgroups.
//   warp 0 lane 0   TMA producer: packed int4 tile [128 n x 64 B] (SWIZZLE_64B: conflict-free
//                   row-per-thread reads) + xq tile [192 m x 128 B] (SWIZZLE_128B) per slab
//   warp 1 lane 0   MMA issuer: per slab four tcgen05.mma kind::i8 (M128 N192 K32), A from TMEM, and
//                   ONE tcgen05.commit to the slab's "done" barrier, which the producer (load slot),
//                   the converters (operand buffer) and the epilogue (accumulator) all wait on
//   warps 4..7      converters (warp q owns TMEM lanes 32q..32q+31)
//   warps 8..15     epilogue: warps 8..11 own token columns 0..95 of the tile, warps 12..15 columns
//                   96..191; tcgen05.ld, running sums in registers, final scale/bias/act/LoRA
// Every mbarrier wait is bounded; on expiry the CTA drains and exits (k2q_common.cuh).
#include "k2q_common.cuh"

namespace k2q {
namespace {

constexpr int TN = 128;   // output channels per tile (UMMA M, TMEM lanes)
constexpr int TM = 192;   // tokens per tile (UMMA N, TMEM columns)
constexpr int BK = 128;   // one weight group per slab
constexpr int UMMA_K = 32;
constexpr int kThreads = 512;
constexpr int kConvWarps = 4;
constexpr int kEpiThreads = 256;
constexpr int kEpiWarps = kEpiThreads / 32;
constexpr int NBUF = 2;           // TMEM accumulators of TM columns
constexpr int ABUF = 4;           // TMEM operand buffers of 32 columns (128 int8 per lane)
static_assert((ABUF & (ABUF - 1)) == 0, "the operand buffer index wraps with a mask");
constexpr uint32_t kACols = BK / 4;
constexpr uint32_t kAccCol0 = ABUF * kACols;                  // 128
constexpr uint32_t kTmemCols = 512;
static_assert(kAccCol0 + NBUF * TM <= kTmemCols, "tensor memory budget");
constexpr uint32_t kXBytes = TM * BK;                         // 24576
constexpr uint32_t kPackedBytes = TN * BK / 2;                // 8192
constexpr uint32_t kLoadStage = kXBytes + kPackedBytes;       // 32768
constexpr int kDone = 8;          // ring of "the MMAs of slab s have completed" barriers (one commit per slab)
static_assert((kDone & (kDone - 1)) == 0, "the ring index wraps with a mask");
constexpr int CW = TM / 2;        // 96 token columns per epilogue thread: three chunks of 32
// Waits that run several slabs ahead of their producer (load slots, operand buffers) go straight to
// the suspended poll: a spinning waiter costs the schedulers issue slots that the epilogue needs.
constexpr uint32_t kLazySpin = 0;

enum WaitId : int {
  W_EMPTY = 201,       // producer: load slot free
  W_FULL_CONV = 202,   // converter: TMA data landed
  W_CONV_EMPTY = 203,  // converter: operand buffer free
  W_FULL_MMA = 204,    // MMA issuer: TMA data landed
  W_CONV_FULL = 205,   // MMA issuer: operand buffer written
  W_ACC_EMPTY = 206,   // MMA issuer: accumulator released
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

template <int RMAX, int LSTAGES>
struct Smem4 {
  static constexpr uint32_t kLoadOff = 0;                                  // LSTAGES x [xq | packed]
  static constexpr uint32_t kSxOff = LSTAGES * kLoadStage;                 // sx_s[TM] (1 KB reserved)
  static constexpr uint32_t kUOff = kSxOff + 1024;                         // u_s[TM][RMAX]
  static constexpr uint32_t kBarOff = kUOff + TM * RMAX * 4;
  static constexpr uint32_t kNumBars = LSTAGES + ABUF + NBUF + kDone;
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

// One 32-column chunk (16 packed pairs) folded into the running sums: raw = int32 accumulators
// (16 * acc), run = fma(float(raw), s / 16, run) with s2 = {s/16, s/16}.
__device__ __forceinline__ void fold_chunk(const uint32_t* raw, uint64_t* run2, uint64_t s2) {
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    const float f0 = static_cast<float>(static_cast<int32_t>(raw[2 * j]));
    const float f1 = static_cast<float>(static_cast<int32_t>(raw[2 * j + 1]));
    run2[j] = fma_f32x2(pack_f32x2(__float_as_uint(f0), __float_as_uint(f1)), s2, run2[j]);
  }
}

// The tile's last step of an epilogue thread without an adapter (one channel, CW tokens):
// y = act(run * sx + bias).  y is [M, ldy]: a warp writes 32 neighbouring channels of one token per store
// instruction; the row pointer advances by ldy per token, the tail of the last token tile is cut by one
// count, and the activation is a compile-time choice made once per tile.
template <bool GELU>
__device__ __forceinline__ void finish_tile(const uint64_t* run2, const float* sxp, float bias_n, int valid,
                                            __nv_bfloat16* yp, int64_t ldy) {
#pragma unroll
  for (int j2 = 0; j2 < CW / 2; ++j2) {
    float rv[2];
    unpack_f32x2(run2[j2], rv[0], rv[1]);
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int jl = 2 * j2 + e;
      float tv = __fadd_rn(__fmul_rn(rv[e], sxp[jl]), bias_n);
      if (GELU) tv = gelu_tanh4(tv);
      if (jl < valid) *yp = __float2bfloat16_rn(tv);
      yp += ldy;
    }
  }
}

template <int RMAX, int LSTAGES>
__global__ void __launch_bounds__(kThreads, 1)
gemm_w4a8_kernel(const __grid_constant__ CUtensorMap tmap_w4, const __grid_constant__ CUtensorMap tmap_x,
                 const Gemm4Params p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  using L = Smem4<RMAX, LSTAGES>;
  constexpr int RD = RMAX > 0 ? RMAX : 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t smem_base = smem_u32(smem);

  float* sx_s = reinterpret_cast<float*>(smem + L::kSxOff);
  float* u_s = reinterpret_cast<float*>(smem + L::kUOff);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBarOff);
  const uint32_t bar_full = smem_u32(bars);                  // [LSTAGES] TMA landed
  const uint32_t bar_cfull = bar_full + 8 * LSTAGES;         // [ABUF] operand buffer written
  const uint32_t bar_aempty = bar_cfull + 8 * ABUF;          // [NBUF] accumulator drained
  // [kDone] the MMAs of slab s (running count per CTA) have completed: barrier s % kDone, parity
  // (s / kDone) & 1.  One commit per slab serves the three parties that wait for it: the producer
  // (load slot of slab s - LSTAGES), the converters (operand buffer of slab s - ABUF) and the epilogue.
  const uint32_t bar_done = bar_aempty + 8 * NBUF;
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
    for (int s = 0; s < LSTAGES; ++s) mbar_init(bar_full + 8 * s, 1);
    for (int s = 0; s < ABUF; ++s) mbar_init(bar_cfull + 8 * s, kConvWarps);   // one arrival per converter warp
    for (int b = 0; b < NBUF; ++b) mbar_init(bar_aempty + 8 * b, kEpiWarps);
    for (int d = 0; d < kDone; ++d) mbar_init(bar_done + 8 * d, 1);
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
  // set-up done: from here on global memory is touched, so the kernels in front must have completed
  pdl_wait();
  pdl_launch_dependents();

  const WaitCtx wctx{abort_flag, p.status};
  const int num_tiles = p.tiles_m * p.tiles_n;
  const int slabs = p.K / BK;

  auto slot_x = [&](int s) { return smem_base + L::kLoadOff + s * kLoadStage; };
  auto slot_p = [&](int s) { return smem_base + L::kLoadOff + s * kLoadStage + kXBytes; };

  // Register re-partition (warpgroup-collective, first statement of each role branch):
  // 24 per thread for the TMA/MMA warpgroup, 56 for the converters, 216 for the epilogue
  // (4 x 24 + 4 x 56 + 8 x 216 = 2048 registers per lane: the whole register file).
  if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 24;");
    if (warp == 0) {
      // ---------------------------------------------------------------- TMA producer
      if (lane == 0) {
        int stage = 0;
        uint32_t slab = 0;
        bool ok = true;
        for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
          const int n0 = (tile % p.tiles_n) * TN;
          const int m0 = (tile / p.tiles_n) * TM;
          for (int g = 0; g < slabs; ++g, ++slab) {
            if (slab >= LSTAGES) {
              const uint32_t prev = slab - LSTAGES;
              if (!mbar_wait<kLazySpin>(bar_done + 8 * (prev % kDone), (prev / kDone) & 1u, wctx, W_EMPTY, g)) { ok = false; break; }
            }
            const uint32_t full = bar_full + 8 * stage;
            mbar_expect_tx(full, kLoadStage);
            tma_load_2d(slot_p(stage), &tmap_w4, g * (BK / 2), n0, full);
            tma_load_2d(slot_x(stage), &tmap_x, g * BK, m0, full);
            if (++stage == LSTAGES) stage = 0;
          }
        }
      }
    } else if (warp == 1) {
      // ---------------------------------------------------------------- MMA issuer
      if (lane == 0) {
        constexpr uint32_t idesc = umma_idesc_i8(TN, TM);
        int stage = 0;
        uint32_t slab = 0;  // running slab count of this CTA -> accumulator / operand buffer
        bool ok = true;
        for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
          for (int g = 0; g < slabs; ++g, ++slab) {
            const uint32_t buf = slab % NBUF;
            const uint32_t ab = slab % ABUF;
            // the accumulator must have been drained (and reset) by the epilogue; the converters'
            // signal also covers the TMA data (they waited for it before they read the packed tile)
            const bool acc_free = mbar_test(bar_aempty + 8 * buf, (slab / NBUF) & 1u);
            const bool op_ready = mbar_test(bar_cfull + 8 * ab, (slab / ABUF) & 1u);
            if (!acc_free && !mbar_wait(bar_aempty + 8 * buf, (slab / NBUF) & 1u, wctx, W_ACC_EMPTY, g)) { ok = false; break; }
            if (!op_ready && !mbar_wait(bar_cfull + 8 * ab, (slab / ABUF) & 1u, wctx, W_CONV_FULL, g)) { ok = false; break; }
            tc_fence_after();
            const uint64_t b_desc = umma_desc_k128(slot_x(stage));
            const uint32_t d_tmem = tmem_base + kAccCol0 + buf * TM;
            const uint32_t a_tmem = tmem_base + ab * kACols;
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k)   // the slab's first MMA overwrites the accumulator
              umma_i8_ts(d_tmem, a_tmem + 8u * k, b_desc + 2u * k, idesc, k > 0 ? 1u : 0u);
            tc_commit(bar_done + 8 * (slab % kDone));
            if (++stage == LSTAGES) stage = 0;
          }
        }
      }
    }
  } else if (warp < 8) {
    // ------------------------------------------------------------------ int4 -> int8 converters
    asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;            // channel of the tile = TMEM lane
    const uint32_t lane_sel = static_cast<uint32_t>(quarter * 32) << 16;
    const int swz = (row >> 1) & 3;                 // SWIZZLE_64B: 16-byte chunk index XOR address bits 7..8
    // The converters do not care about tiles: one loop over all slabs of this CTA, every address and
    // barrier advanced by a rolling register (no division, no multiply per slab).
    const int my_tiles = (num_tiles - static_cast<int>(blockIdx.x) + static_cast<int>(gridDim.x) - 1) / static_cast<int>(gridDim.x);
    const uint32_t total = static_cast<uint32_t>(my_tiles) * static_cast<uint32_t>(slabs);
    const uint8_t* const src0 = smem + L::kLoadOff + kXBytes + row * 64;     // this thread's 64 packed bytes in slot 0
    const uint8_t* src = src0;
    uint32_t full = bar_full, phase = 0;
    int stage = 0;
    uint32_t ab = 0;                                  // operand buffer of this slab
    uint32_t didx = 0, dpar = 0;                      // "done" barrier + parity of slab - ABUF (valid from slab ABUF on)
    bool ok = true;
    for (uint32_t slab = 0; slab < total; ++slab) {
      // probe first (all lanes, no hand-off inside the warp); only an incomplete phase takes the
      // bounded wait of lane 0
      if (!__all_sync(0xffffffffu, mbar_test(full, phase))) {
        if (lane == 0) ok = mbar_wait<kLazySpin>(full, phase, wctx, W_FULL_CONV, static_cast<int>(slab));
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) break;
      }
      uint32_t o[32];
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const uint4 pk = *reinterpret_cast<const uint4*>(src + ((c ^ swz) << 4));   // codes 32c .. 32c+31
        const uint32_t w[4] = {pk.x, pk.y, pk.z, pk.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const uint32_t lo = (w[j] << 4) & 0xF0F0F0F0u;  // even codes, value*16 as int8
          const uint32_t hi = w[j] & 0xF0F0F0F0u;         // odd codes
          o[8 * c + 2 * j] = prmt(lo, hi, 0x5140u);
          o[8 * c + 2 * j + 1] = prmt(lo, hi, 0x7362u);
        }
      }
      // the operand buffer is free once the MMAs of the slab that used it last have completed;
      // unpacking above did not need it
      if (slab >= ABUF) {
        if (!__all_sync(0xffffffffu, mbar_test(bar_done + 8 * didx, dpar))) {
          if (lane == 0) ok = mbar_wait<kLazySpin>(bar_done + 8 * didx, dpar, wctx, W_CONV_EMPTY, static_cast<int>(slab));
          ok = __shfl_sync(0xffffffffu, ok, 0);
          if (!ok) break;
        }
        didx = (didx + 1u) & (kDone - 1);
        dpar ^= (didx == 0u) ? 1u : 0u;
      }
      tc_fence_after();
      tmem_st32(tmem_base + lane_sel + ab * kACols, o);
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_cfull + 8 * ab);
      ab = (ab + 1u) & (ABUF - 1);
      src += kLoadStage;
      full += 8;
      if (++stage == LSTAGES) { stage = 0; phase ^= 1u; src = src0; full = bar_full; }
    }
  } else {
    // ------------------------------------------------------------------ epilogue
    asm volatile("setmaxnreg.inc.sync.aligned.u32 216;");
    const int et = threadIdx.x - 256;       // 0..255
    const int ch = (warp - 8) >> 2;         // which half of the token columns this warp owns
    const int quarter = warp & 3;           // TMEM lane quarter this warp may access
    const int nl = quarter * 32 + lane;
    const uint32_t lane_sel = (static_cast<uint32_t>(quarter * 32) << 16) + kAccCol0 + ch * CW;
    tc_fence_before();
    __syncwarp();
    if (lane == 0) {
#pragma unroll
      for (int b = 0; b < NBUF; ++b) mbar_arrive(bar_aempty + 8 * b);
    }

    uint32_t slab = 0;
    bool ok = true;
    uint32_t r0[32], r1[32], r2[32];
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

      // rows past N read the scales of row 0 and multiply zero accumulators (TMA fills them with zeros)
      const __nv_bfloat16* swrow = p.sw4 + static_cast<int64_t>(n_ok ? n : 0) * slabs;

      uint64_t run2[CW / 2];
#pragma unroll
      for (int j = 0; j < CW / 2; ++j) run2[j] = 0ull;

      // Rolling pipeline over the slabs of the tile: the three 32-column chunks of slab g are in
      // flight or in r0..r2 when iteration g starts; as soon as a chunk has been folded its
      // registers are refilled with the same chunk of slab g + 1, so the barrier probe, the
      // tensor-memory reads and the release of the next accumulator hide behind the folds.
      const uint32_t tacc = tmem_base + lane_sel;
      if (ok) {
        if (lane == 0) ok = mbar_wait(bar_done + 8 * (slab % kDone), (slab / kDone) & 1u, wctx, W_ACC_FULL, 0);
        ok = __shfl_sync(0xffffffffu, ok, 0);
      }
      if (ok) {
        tc_fence_after();
        const uint32_t t = tacc + (slab % NBUF) * TM;
        tmem_ld32(t, r0);
        tmem_ld32(t + 32, r1);
        tmem_ld32(t + 64, r2);
      } else {   // aborted: nothing is read; the assignment only ends the registers' live range here
#pragma unroll
        for (int j = 0; j < 32; ++j) r0[j] = r1[j] = r2[j] = 0u;
      }
      float s_next = __bfloat162float(swrow[0]);
      if (ok) {
        // rolling state, advanced without divisions: barrier + parity of the NEXT slab, accumulator of this one
        uint32_t nidx = (slab + 1) % kDone, npar = ((slab + 1) / kDone) & 1u;
        uint32_t rel = bar_aempty + 8 * (slab % NBUF), rel_other = bar_aempty + 8 * ((slab + 1) % NBUF);
        uint32_t tn = tacc + ((slab + 1) % NBUF) * TM, tn_other = tacc + (slab % NBUF) * TM;
        for (int g = 0; g + 1 < slabs; ++g) {       // every slab but the tile's last: slab g + 1 exists
          const uint32_t sb = __float_as_uint(s_next * 0.0625f);   // the accumulators hold 16 * acc
          const uint64_t s2 = pack_f32x2(sb, sb);
          s_next = __bfloat162float(swrow[g + 1]);
          const bool ready = mbar_test(bar_done + 8 * nidx, npar);
          tmem_ld_wait_dep(r0);       // one wait covers the three loads in flight
          tmem_ld_ready(r1);
          tmem_ld_ready(r2);
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(rel);   // slab g is in registers: release its accumulator
          fold_chunk(r0, run2, s2);
          if (!__all_sync(0xffffffffu, ready)) {
            if (lane == 0) ok = mbar_wait(bar_done + 8 * nidx, npar, wctx, W_ACC_FULL, g);
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) break;                           // aborted: every role leaves its loops
          }
          tc_fence_after();
          tmem_ld32(tn, r0);
          fold_chunk(r1, run2 + 16, s2);
          tmem_ld32(tn + 32, r1);
          fold_chunk(r2, run2 + 32, s2);
          tmem_ld32(tn + 64, r2);
          nidx = (nidx + 1u) & (kDone - 1);
          npar ^= (nidx == 0u) ? 1u : 0u;
          { const uint32_t t = rel; rel = rel_other; rel_other = t; }
          { const uint32_t t = tn; tn = tn_other; tn_other = t; }
        }
        if (ok) {                                     // the tile's last slab: nothing to request behind it
          const uint32_t sb = __float_as_uint(s_next * 0.0625f);
          const uint64_t s2 = pack_f32x2(sb, sb);
          tmem_ld_wait_dep(r0);       // one wait covers the three loads in flight
          tmem_ld_ready(r1);
          tmem_ld_ready(r2);
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(rel);
          fold_chunk(r0, run2, s2);
          fold_chunk(r1, run2 + 16, s2);
          fold_chunk(r2, run2 + 32, s2);
          slab += static_cast<uint32_t>(slabs);
        }
      }
      if (!ok) continue;

      const float bias_n = (n_ok && p.bias) ? __ldg(p.bias + n) : 0.0f;
      float br[RD];
      if (RMAX > 0) {
#pragma unroll
        for (int j = 0; j < RMAX; ++j)
          br[j] = (n_ok && j < p.rank) ? p.lora_scale * __ldg(p.Bm + n * p.ldb + j) : 0.0f;
      }
      // final scale, bias, activation, adapter term; y is [M, ldy]: a warp writes 32 neighbouring
      // channels of one token per store instruction.  The row pointer advances by ldy per token, the
      // tail of the last token tile is cut by one count, and the activation is chosen once per tile.
      if (RMAX == 0) {
        if (n_ok) {
          const int valid = min(CW, p.M - m0 - ch * CW);                 // tokens of this thread's half that exist
          __nv_bfloat16* yp = p.y + n + static_cast<int64_t>(m0 + ch * CW) * p.ldy;
          if (p.act == K2Q_ACT_GELU_TANH) finish_tile<true>(run2, sx_s + ch * CW, bias_n, valid, yp, p.ldy);
          else finish_tile<false>(run2, sx_s + ch * CW, bias_n, valid, yp, p.ldy);
        }
      } else {
        // adapter epilogue (short of registers: address and activation per value)
        __nv_bfloat16* ycol = p.y + n;
#pragma unroll
        for (int j2 = 0; j2 < CW / 2; ++j2) {
          float rv[2];
          unpack_f32x2(run2[j2], rv[0], rv[1]);
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int j = ch * CW + 2 * j2 + e;
            float tv = __fmul_rn(rv[e], sx_s[j]);
            tv = __fadd_rn(tv, bias_n);
            if (p.act == K2Q_ACT_GELU_TANH) tv = gelu_tanh4(tv);
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
            tv += d;
            const int m = m0 + j;
            if (n_ok && m < p.M) ycol[static_cast<int64_t>(m) * p.ldy] = __float2bfloat16_rn(tv);
          }
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

template <int RMAX, int LSTAGES>
int launch4(const CUtensorMap& tw, const CUtensorMap& tx, const Gemm4Params& p, int grid, cudaStream_t stream) {
  using L = Smem4<RMAX, LSTAGES>;
  static_assert(L::kBytes <= 232448, "shared memory budget exceeded");
  auto kern = gemm_w4a8_kernel<RMAX, LSTAGES>;
  if (int rc = check_cuda(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kBytes),
                          "cudaFuncSetAttribute(gemm_w4a8)"))
    return rc;
  return launch_overlapped(kern, static_cast<unsigned>(grid), kThreads, L::kBytes, stream, 1, "gemm_w4a8 launch", tw, tx, p);
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
  if (int rc = encode_tmap_2d_u8(&tw, wq4, (uint64_t)K / 2, (uint64_t)N, (uint64_t)K / 2, BK / 2, TN, 2)) return rc;
  if (int rc = encode_tmap_2d_u8(&tx, xq, (uint64_t)K, (uint64_t)M, (uint64_t)K, BK, TM, 1)) return rc;

  const int sms = sm_count();
  if (sms <= 0) return fail(K2Q_ECUDA, "k2q_gemm_w4a8: could not read the SM count");
  const int64_t tiles = (int64_t)p.tiles_m * p.tiles_n;
  const int grid = (int)(tiles < sms ? tiles : sms);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (e.rank == 0) return launch4<0, 6>(tw, tx, p, grid, s);
  if (e.rank <= 16) return launch4<16, 6>(tw, tx, p, grid, s);
  return launch4<32, 6>(tw, tx, p, grid, s);
}
