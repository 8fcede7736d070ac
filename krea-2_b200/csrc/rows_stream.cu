// K2 as a streaming kernel: block-128 rotation + per-token int8 of contiguous bf16 rows whose length is a
// multiple of 1024, with every byte moved by TMA.
//
// One persistent CTA per SM.  A producer thread requests whole rows with tiled TMA loads (2 KB boxes of
// 32 x 64 bytes, SWIZZLE_64B, landing in a ring of row slots; completion on an mbarrier), so the loads run
// as far ahead as the ring allows and cost the arithmetic warps no instructions and no registers.  A row
// is worked on by a TEAM of K / 1024 warps (a CTA holds up to 24 such warps = several teams, each on its
// own rows): every thread reads its 32 consecutive elements (four 16-byte shared-memory loads, free of bank
// conflicts thanks to the swizzle), the slot is handed back at once, the rotation and the thread / warp
// maxima follow in registers, the row maximum goes through one shared-memory word and ONE named barrier
// of the team (three rotating words: the next row's word is cleared before this row's barrier), codes are
// packed, written to the warp's own 1 KB staging tile (SWIZZLE_32B pattern) and leave with a TMA store.
// The arithmetic is that of rows_math.cuh, so codes and scales equal the other row kernels' bit for bit.
//
// Every wait is bounded.  A thread whose wait expired keeps walking its rows without touching memory, so
// that its team's barriers still see every warp; the CTA gives copies in flight time to land and leaves.
#include "k2q_common.cuh"
#include "rows_math.cuh"

namespace k2q {
namespace {

constexpr int kMaxTeamWarps = 24;       // consumer warps per CTA
constexpr int kMaxRowWarps = 16;         // K <= 16384: a row is one TMA box of at most 256 lines
constexpr int kMaxTeams = 8;            // named barriers 1..8
constexpr int kStages = 3;              // row slots per team
constexpr int kTileBytes = 2048;        // one warp's 1024 bf16 elements
constexpr int kOutTile = 1024;          // one warp's 1024 codes
constexpr int W_ROW_FULL = 501, W_ROW_EMPTY = 502;

struct StreamParams {
  float* sx;
  int64_t M;
  int tw;        // warps per row = K / 1024
  int nt;        // teams per CTA
  Status* status;
};

__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, int32_t c0, int32_t c1, uint32_t src_smem) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(map), "r"(src_smem), "r"(c0), "r"(c1)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void bulk_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

__global__ void __launch_bounds__((kMaxTeamWarps + 1) * 32, 1)
k2_stream_kernel(const __grid_constant__ CUtensorMap in_map, const __grid_constant__ CUtensorMap out_map,
                 const StreamParams p) {
  extern __shared__ uint8_t smem_raw[];
  // swizzled TMA tiles want their base on a 1024-byte boundary: the launch asks for 1 KB of slack
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  __shared__ __align__(8) uint64_t bars[2 * kMaxTeams * kStages];
  __shared__ int amax_slot[kMaxTeams][3];
  __shared__ int abort_flag_s;
  volatile int* abort_flag = &abort_flag_s;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nt = p.nt, tw = p.tw;
  uint8_t* ring = smem;                                                        // [nt][kStages][tw][2 KB]
  uint8_t* outs = smem + static_cast<size_t>(nt) * kStages * tw * kTileBytes;  // [nt * tw][2][1 KB]
  const uint32_t bar_full = smem_u32(bars), bar_empty = bar_full + 8u * kMaxTeams * kStages;

  if (threadIdx.x == 0) {
    for (int i = 0; i < nt * kStages; ++i) {
      mbar_init(bar_full + 8u * i, 1);
      mbar_init(bar_empty + 8u * i, static_cast<uint32_t>(tw));
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (threadIdx.x < kMaxTeams * 3) (&amax_slot[0][0])[threadIdx.x] = 0;
  __syncthreads();
  // set-up done: from here on global memory is touched, so the kernels in front must have completed
  pdl_wait();
  pdl_launch_dependents();
  const WaitCtx wctx{abort_flag, p.status};

  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    if (lane == 0) {
      tma_prefetch_desc(&in_map);
      bool ok = true;
      const uint32_t slot_bytes = static_cast<uint32_t>(tw) * kTileBytes;
      const int64_t row_step = static_cast<int64_t>(gridDim.x) * nt;
      int stage = 0;
      uint32_t use = 0;                      // how often the ring has wrapped
      for (int64_t row0 = static_cast<int64_t>(blockIdx.x) * nt; ok && row0 < p.M; row0 += row_step) {
        for (int t = 0; t < nt && row0 + t < p.M; ++t) {
          const uint32_t slot = static_cast<uint32_t>(t * kStages + stage);
          if (use > 0) ok = mbar_wait<8>(bar_empty + 8u * slot, (use - 1u) & 1u, wctx, W_ROW_EMPTY, stage);
          if (!ok) break;
          mbar_expect_tx(bar_full + 8u * slot, slot_bytes);
          // the whole row as one box of K / 64 lines of 128 bytes
          tma_load_2d(smem_u32(ring) + slot * slot_bytes, &in_map, 0, static_cast<int32_t>((row0 + t) * (tw * 16)),
                      bar_full + 8u * slot);
        }
        if (++stage == kStages) {
          stage = 0;
          ++use;
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ consumers
    const int cw = warp - 1;               // consumer warp index
    const int t = cw / tw, w = cw - t * tw;
    if (t < nt) {
      if (lane == 0) tma_prefetch_desc(&out_map);
      const int tr = w * 32 + lane;
      // SWIZZLE_128B: the 16-byte chunk index inside a 128-byte line XOR the line's index modulo 8.  A thread's
      // 64 input bytes are half of line tr / 2, its 32 output bytes a quarter of line lane / 4 of the warp's tile.
      const int in_line = tr >> 1, in_c0 = (tr & 1) * 4, in_swz = in_line & 7;
      const int out_line = lane >> 2, out_c0 = (lane & 3) * 2, out_swz = out_line & 7;
      // everything that changes from row to row is carried along instead of being recomputed: the ring slot
      // (= the row-maximum word: both rotate over three), its barriers' parity, the staging tile, the
      // coordinate of the store, the address of the scale
      const uint32_t slot_bytes = static_cast<uint32_t>(tw) * kTileBytes;
      const uint8_t* in0 = ring + static_cast<size_t>(t) * kStages * slot_bytes + in_line * 128;
      uint32_t in_off[4];
#pragma unroll
      for (int c = 0; c < 4; ++c) in_off[c] = static_cast<uint32_t>(((in_c0 + c) ^ in_swz) << 4);
      uint8_t* ob = outs + static_cast<size_t>(cw) * 2 * kOutTile;           // 2 KB aligned pair of tiles
      const uint32_t o_off0 = static_cast<uint32_t>(out_line * 128 + (((out_c0 + 0) ^ out_swz) << 4));
      const uint32_t o_off1 = static_cast<uint32_t>(out_line * 128 + (((out_c0 + 1) ^ out_swz) << 4));
      const uint32_t full0 = bar_full + 8u * static_cast<uint32_t>(t * kStages);
      const uint32_t empty0 = bar_empty + 8u * static_cast<uint32_t>(t * kStages);
      int* const slot_word = amax_slot[t];
      const int64_t row_step = static_cast<int64_t>(gridDim.x) * nt;
      int64_t row = static_cast<int64_t>(blockIdx.x) * nt + t;
      float* sx_p = p.sx + row;
      int32_t oc = static_cast<int32_t>(row * (tw * 8) + w * 8);
      const int32_t oc_step = static_cast<int32_t>(row_step * (tw * 8));
      int stage = 0;
      uint32_t parity = 0;
      bool ok = true;
      for (; row < p.M; row += row_step, sx_p += row_step, oc += oc_step) {
        const int nxt = stage == kStages - 1 ? 0 : stage + 1;
        float v[EPT];
        float amax = 0.f;
        if (ok && *abort_flag) ok = false;
        if (ok) ok = mbar_wait<32>(full0 + 8u * stage, parity, wctx, W_ROW_FULL, stage);
        ok = __all_sync(0xffffffffu, ok);
        if (ok) {
          const uint8_t* line = in0 + stage * slot_bytes;
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const uint4 r = *reinterpret_cast<const uint4*>(line + in_off[c]);
            const uint32_t wd[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              v[8 * c + 2 * j] = __uint_as_float(wd[j] << 16);
              v[8 * c + 2 * j + 1] = __uint_as_float(wd[j] & 0xFFFF0000u);
            }
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(empty0 + 8u * stage);      // the slot may be refilled
          fwht128_thread(v, tr);
          // thread maximum as four independent chains, warp maximum by one integer reduction (floats >= 0
          // order as unsigned integers)
          float a4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
          for (int j = 0; j < EPT; j += 4) {
#pragma unroll
            for (int q = 0; q < 4; ++q) a4[q] = fmaxf(a4[q], fabsf(v[j + q]));
          }
          amax = fmaxf(fmaxf(a4[0], a4[1]), fmaxf(a4[2], a4[3]));
          const uint32_t wmax = __reduce_max_sync(0xffffffffu, __float_as_uint(amax));
          if (lane == 0) atomicMax(slot_word + stage, static_cast<int>(wmax));
        }
        // the next row's word: its last readers (two rows back) are behind the previous row's barrier, which
        // this thread has passed; its next writers come after this row's barrier
        if (w == 0 && lane == 0) slot_word[nxt] = 0;
        named_bar_sync(1 + t, tw * 32);
        const int cur = stage;
        stage = nxt;
        if (nxt == 0) parity ^= 1u;
        if (!ok) continue;
        const float s = __fdiv_rn(fmaxf(__int_as_float(slot_word[cur]), 1e-8f), 127.0f);
        const float inv = __frcp_rn(s);
        if (w == 0 && lane == 0) *sx_p = s;
        uint32_t words[EPT / 4];
        quant_row32_i8(v, s, inv, words);
        if (lane == 0) bulk_wait_read<1>();      // the store that last read this tile (two rows back) has done so
        __syncwarp();
        *reinterpret_cast<uint4*>(ob + o_off0) = make_uint4(words[0], words[1], words[2], words[3]);
        *reinterpret_cast<uint4*>(ob + o_off1) = make_uint4(words[4], words[5], words[6], words[7]);
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          tma_store_2d(&out_map, 0, oc, smem_u32(ob));
          bulk_commit();
        }
        ob = reinterpret_cast<uint8_t*>(reinterpret_cast<uintptr_t>(ob) ^ static_cast<uintptr_t>(kOutTile));
      }
      if (lane == 0) bulk_wait_all();
    }
  }
  __syncthreads();
  if (*abort_flag) {
    // a wait expired somewhere: give loads still in flight time to land in this CTA's shared memory
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
  }
}

}  // namespace
}  // namespace k2q

using namespace k2q;

extern "C" int k2q_fwht_quant_act_i8_stream_ok(int x_dtype, int64_t M, int64_t K, int64_t ldx) {
  return x_dtype == K2Q_BF16 && M > 0 && K >= 1024 && K % 1024 == 0 && K / 1024 <= kMaxRowWarps && ldx == K &&
                 M * (K / 64) < (int64_t(1) << 31)
             ? 1
             : 0;
}

extern "C" int k2q_fwht_quant_act_i8_stream(const void* x_bf16, int64_t M, int64_t K, int8_t* xq, float* sx, void* status,
                                            void* stream) {
  if (int rc = check_device_arch()) return rc;
  if (M == 0) return K2Q_OK;
  if (!k2q_fwht_quant_act_i8_stream_ok(K2Q_BF16, M, K, K))
    return fail(K2Q_EINVAL, "k2q_fwht_quant_act_i8_stream: contiguous bf16 rows with K a multiple of 1024 (<= %d) expected, got M=%lld K=%lld",
                kMaxRowWarps * 1024, (long long)M, (long long)K);
  if (!x_bf16 || !xq || !sx || !status) return fail(K2Q_EINVAL, "k2q_fwht_quant_act_i8_stream: NULL pointer");
  if ((reinterpret_cast<uintptr_t>(x_bf16) & 15u) || (reinterpret_cast<uintptr_t>(xq) & 15u))
    return fail(K2Q_EINVAL, "k2q_fwht_quant_act_i8_stream: x and xq must be 16-byte aligned");
  StreamParams p;
  p.sx = sx;
  p.M = M;
  p.tw = static_cast<int>(K / 1024);
  p.nt = kMaxTeamWarps / p.tw < kMaxTeams ? kMaxTeamWarps / p.tw : kMaxTeams;
  p.status = static_cast<Status*>(status);
  // both tensors as lines of 128 bytes: a row is K / 64 input lines (one box) and K / 128 output lines (8 per warp)
  CUtensorMap in_map, out_map;
  if (int rc = encode_tmap_2d_u8(&in_map, x_bf16, 128, static_cast<uint64_t>(M) * (K / 64), 128, 128,
                                 static_cast<uint32_t>(K / 64), 1))
    return rc;
  if (int rc = encode_tmap_2d_u8(&out_map, xq, 128, static_cast<uint64_t>(M) * (K / 128), 128, 128, 8, 1)) return rc;
  const int sms = sm_count();
  if (sms <= 0) return fail(K2Q_ECUDA, "k2q_fwht_quant_act_i8_stream: SM count unknown");
  const int64_t rounds_all = (M + p.nt - 1) / p.nt;       // CTAs that would each take one round
  const int grid = static_cast<int>(rounds_all < sms ? rounds_all : sms);
  const size_t smem = static_cast<size_t>(p.nt) * p.tw * (kStages * kTileBytes + 2 * kOutTile) + 1024;
  static bool attr_set[64] = {};
  int dev = 0;
  if (int rc = check_cuda(cudaGetDevice(&dev), "cudaGetDevice")) return rc;
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    if (int rc = check_cuda(cudaFuncSetAttribute(k2_stream_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                 kMaxTeamWarps * (kStages * kTileBytes + 2 * kOutTile) + 1024),
                            "cudaFuncSetAttribute(k2_stream_kernel)"))
      return rc;
    attr_set[dev] = true;
  }
  return launch_overlapped(k2_stream_kernel, static_cast<unsigned>(grid), static_cast<unsigned>((p.nt * p.tw + 1) * 32), smem,
                           static_cast<cudaStream_t>(stream), 1, "k2_stream_kernel launch", in_map, out_map, p);
}
