// Arithmetic shared by the row kernels: the block-128 Walsh-Hadamard rotation of the 32 elements a
// thread holds and the division-free exact quantiser.  Four neighbouring lanes own one 128-block, 32
// consecutive elements each; stage order, the (a+b, a-b) pairing and the single final multiply are those of
// the CPU restatement, in fp32 with explicitly rounded operations, so every kernel that goes through
// these functions produces the same bits.
#pragma once

#include "k2q_common.cuh"

namespace k2q {

constexpr float kHadNorm = 0.088388347648318440550f;  // fp32(2^-3.5)
constexpr float kRoundMagic = 12582912.0f;            // 1.5 * 2^23: x + magic rounds x to nearest-even
constexpr int EPT = 32;                               // elements per thread

// rint(v / s) as an integer-valued float; inv ~ 1/s.  Bit-identical with rintf(__fdiv_rn(v, s)).
__device__ __forceinline__ float quant_round(float v, float s, float inv) {
  const float y = __fmul_rn(v, inv);
  float q = __fsub_rn(__fadd_rn(y, kRoundMagic), kRoundMagic);
  if (fabsf(__fsub_rn(y, q)) > 0.499f) q = rintf(__fdiv_rn(v, s));
  return q;
}
// low byte of the two's complement integer held by an integer-valued float |q| < 2^22
__device__ __forceinline__ uint32_t code_bits(float q) { return __float_as_uint(__fadd_rn(q, kRoundMagic)); }

// Codes of N consecutive elements: word i holds rint(v[i] / s) as a two's complement integer in
// its low bits.  t = v * (1/s) + 1.5 * 2^23 carries rint(v * (1/s)) in its low mantissa bits, and
// v * (1/s) is within 2e-5 of the quotient the oracle rounds; dev tracks how close any of the N
// came to a rounding tie, and only then (rarely) they are redone with the exact IEEE division.
// One rarely taken branch per N elements, no second rounding add per element.
template <int N>
__device__ __forceinline__ void quant_codes(const float* v, float s, float inv, uint32_t (&code)[N]) {
  static_assert(N % 2 == 0, "codes are formed two at a time");
  // two elements per instruction (packed fp32 pairs, each half rounded as the scalar operation would be)
  const uint64_t inv2 = pack_f32x2(inv, inv), magic2 = pack_f32x2(kRoundMagic, kRoundMagic);
  const uint64_t nmagic2 = pack_f32x2(-kRoundMagic, -kRoundMagic), neg2 = pack_f32x2(-1.0f, -1.0f);
  float dev = 0.f;
#pragma unroll
  for (int i = 0; i < N; i += 2) {
    const uint64_t y = mul_f32x2(pack_f32x2(v[i], v[i + 1]), inv2);
    const uint64_t t = add_f32x2(y, magic2);
    const uint64_t d = fma_f32x2(add_f32x2(t, nmagic2), neg2, y);     // y - (t - magic)
    float d0, d1, t0, t1;
    unpack_f32x2(d, d0, d1);
    unpack_f32x2(t, t0, t1);
    dev = fmaxf(fmaxf(dev, fabsf(d0)), fabsf(d1));
    code[i] = __float_as_uint(t0);
    code[i + 1] = __float_as_uint(t1);
  }
  if (dev > 0.49997f) {
#pragma unroll
    for (int i = 0; i < N; ++i) code[i] = code_bits(quant_round(v[i], s, inv));
  }
}

__device__ __forceinline__ uint32_t prmt_b(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t r;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
  return r;
}

// int8 codes of a thread's 32 elements, packed four to a word (element 4q + j in byte j of word q), with ONE
// test for the whole thread: the packed path forms every code from t = v * (1/s) + magic and tracks how close
// any of the 32 products came to a rounding tie; only then (about one thread in a thousand) all 32 are redone
// with the exact IEEE division.  Same codes as quant_codes.
__device__ __forceinline__ void quant_row32_i8(const float (&v)[EPT], float s, float inv, uint32_t (&words)[EPT / 4]) {
  const uint64_t inv2 = pack_f32x2(inv, inv), magic2 = pack_f32x2(kRoundMagic, kRoundMagic);
  const uint64_t nmagic2 = pack_f32x2(-kRoundMagic, -kRoundMagic), neg2 = pack_f32x2(-1.0f, -1.0f);
  float dev0 = 0.f, dev1 = 0.f;
#pragma unroll
  for (int q = 0; q < EPT / 4; ++q) {
    uint32_t code[4];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const uint64_t y = mul_f32x2(pack_f32x2(v[4 * q + 2 * h], v[4 * q + 2 * h + 1]), inv2);
      const uint64_t t = add_f32x2(y, magic2);
      const uint64_t d = fma_f32x2(add_f32x2(t, nmagic2), neg2, y);     // y - (t - magic)
      float d0, d1, t0, t1;
      unpack_f32x2(d, d0, d1);
      unpack_f32x2(t, t0, t1);
      if (h == 0) dev0 = fmaxf(fmaxf(dev0, fabsf(d0)), fabsf(d1));
      else dev1 = fmaxf(fmaxf(dev1, fabsf(d0)), fabsf(d1));
      code[2 * h] = __float_as_uint(t0);
      code[2 * h + 1] = __float_as_uint(t1);
    }
    words[q] = prmt_b(prmt_b(code[0], code[1], 0x0040u), prmt_b(code[2], code[3], 0x0040u), 0x5410u);
  }
  if (fmaxf(dev0, dev1) > 0.49997f) {
#pragma unroll
    for (int q = 0; q < EPT / 4; ++q) {
      uint32_t code[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) code[j] = code_bits(quant_round(v[4 * q + j], s, inv));
      words[q] = prmt_b(prmt_b(code[0], code[1], 0x0040u), prmt_b(code[2], code[3], 0x0040u), 0x5410u);
    }
  }
}

// Rotation of a thread's 32 elements of a 128-block; tr = the thread's index inside its row (its low two
// bits = which quarter of the block it owns).  All 32 lanes of the warp must call it together.
__device__ __forceinline__ void fwht128_thread(float (&v)[EPT], int tr) {
  // stage h = 1 inside each pair of neighbours, stages h = 2, 4, 8, 16 on packed pairs (two butterflies per
  // instruction pair; a - b as fma(b, -1, a): one rounding, the same as the subtraction)
  const uint64_t neg2 = pack_f32x2(-1.0f, -1.0f);
#pragma unroll
  for (int i = 0; i < EPT; i += 2) {
    const float a = v[i], b = v[i + 1];
    v[i] = __fadd_rn(a, b);
    v[i + 1] = __fsub_rn(a, b);
  }
#pragma unroll
  for (int h = 2; h < EPT; h <<= 1) {
#pragma unroll
    for (int i = 0; i < EPT; i += 2) {
      if ((i & h) == 0) {
        const uint64_t a = pack_f32x2(v[i], v[i + 1]), b = pack_f32x2(v[i + h], v[i + h + 1]);
        unpack_f32x2(add_f32x2(a, b), v[i], v[i + 1]);
        unpack_f32x2(fma_f32x2(b, neg2, a), v[i + h], v[i + h + 1]);
      }
    }
  }
#pragma unroll
  for (int j = 0; j < 2; ++j) {        // stages h = 32, 64: the partner lane differs in bit j of tr
    const float sgn = ((tr >> j) & 1) ? -1.0f : 1.0f;   // lower lane a+b, upper lane a-b
    const uint64_t sgn2 = pack_f32x2(sgn, sgn);
#pragma unroll
    for (int i = 0; i < EPT; i += 2) {
      const float o0 = __shfl_xor_sync(0xffffffffu, v[i], 1 << j);
      const float o1 = __shfl_xor_sync(0xffffffffu, v[i + 1], 1 << j);
      // o + v or o - v, one rounding like the plain add
      unpack_f32x2(fma_f32x2(pack_f32x2(v[i], v[i + 1]), sgn2, pack_f32x2(o0, o1)), v[i], v[i + 1]);
    }
  }
  const uint64_t norm2 = pack_f32x2(kHadNorm, kHadNorm);
#pragma unroll
  for (int i = 0; i < EPT; i += 2) unpack_f32x2(mul_f32x2(pack_f32x2(v[i], v[i + 1]), norm2), v[i], v[i + 1]);
}

}  // namespace k2q
