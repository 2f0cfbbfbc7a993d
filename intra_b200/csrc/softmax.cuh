// Register-level pieces of the online softmax a thread runs over its share of a query row: 32 or 64
// score columns live in registers (read from tensor memory) and are turned into packed bf16
// probabilities.
//
// The work is arranged so that a warp depends as little as possible on others to hide its latencies:
//   * row maximum: four independent chains of three-input max instead of one 127-deep chain;
//   * the row sum uses the packed two-lane add (add.f32x2); multiply-adds stay scalar, which is the
//     cheaper form on this part (see ex2_fma_pipe);
//   * exponentials are split between the two pipes that can produce them: most go to the MUFU
//     (ex2.approx, 16 results per clock per SM), a fixed share is computed on the FMA pipe with a
//     floor / degree-3-polynomial / exponent-add evaluation of 2^x whose relative error (8.6e-5) is far
//     below the bf16 rounding applied to P right after.
// Replaces the reference's softmax.h:66-166 (exp2f with folded scale, quad-shuffle row reductions),
// which has four threads per row; here a row is one thread, so there are no shuffles at all.
#pragma once
#include <math_constants.h>
#include <stdint.h>

#include "ptx.cuh"

namespace intra {
namespace sm {

using f2 = unsigned long long;   // two packed fp32 lanes

__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
__device__ __forceinline__ f2 pack2(float lo, float hi) {
  f2 r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack2(f2 v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ f2 fma2(f2 a, f2 b, f2 c) {
  f2 d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ f2 add2(f2 a, f2 b) {
  f2 d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ f2 add2_rm(f2 a, f2 b) {   // round towards minus infinity
  f2 d;
  asm("add.rm.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ f2 sub2(f2 a, f2 b) {
  f2 d;
  asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}

// Maximum of N scores held in registers (N = 64 or 128): four chains of three-input max.
template <int N>
__device__ __forceinline__ float row_max(const float (&s)[N]) {
  static_assert(N % 8 == 4 || N % 8 == 0, "N must be a multiple of 4");
  float a0 = max3(s[0], s[1], s[2]), a1 = max3(s[3], s[4], s[5]);
  float a2 = max3(s[6], s[7], s[8]), a3 = max3(s[9], s[10], s[11]);
  constexpr int kLoopEnd = 12 + ((N - 12) / 8) * 8;
#pragma unroll
  for (int c = 12; c < kLoopEnd; c += 8) {
    a0 = max3(a0, s[c], s[c + 1]);
    a1 = max3(a1, s[c + 2], s[c + 3]);
    a2 = max3(a2, s[c + 4], s[c + 5]);
    a3 = max3(a3, s[c + 6], s[c + 7]);
  }
  a0 = max3(a0, s[N - 4], s[N - 3]);        // N - 12 is 4 mod 8: four scores left
  a1 = max3(a1, s[N - 2], s[N - 1]);
  return max3(a0, a1, fmaxf(a2, a3));
}

// 2^x for two values on the FMA pipe, for x <= 127: floor(x) by a round-down add of 1.5 * 2^23, the
// fraction f = x - floor(x) in [0, 1) through a cubic fitted to 2^f (max relative error 8.6e-5), and
// floor(x) added straight into the exponent field. Inputs below -126 (masked scores are -inf) are
// clamped, which yields 2^-126, i.e. zero for every purpose here.
// Measured on B200 (clocks per warp instruction per scheduler): fma.rn.f32x2 3.0 against 0.75 for a
// scalar fma, add/sub.f32x2 2.0, 3-input max 2.0, ex2.approx 8.0. So the packed form is used where it
// saves issue slots cheaply (the three add/subs) and the multiply-adds stay scalar.
__device__ __forceinline__ void ex2_fma_pipe(float x0, float x1, float& r0, float& r1) {
  constexpr float kMagic = 12582912.f;
  const f2 xc = pack2(fmaxf(x0, -126.f), fmaxf(x1, -126.f));
  const f2 magic = pack2(kMagic, kMagic);
  const f2 t = add2_rm(xc, magic);
  const f2 f = sub2(xc, sub2(t, magic));
  float f0, f1, t0, t1;
  unpack2(f, f0, f1);
  unpack2(t, t0, t1);
  float p0 = fmaf(f0, 0.07706704f, 0.22764499f), p1 = fmaf(f1, 0.07706704f, 0.22764499f);
  p0 = fmaf(p0, f0, 0.69511676f);
  p1 = fmaf(p1, f1, 0.69511676f);
  p0 = fmaf(p0, f0, 1.f);
  p1 = fmaf(p1, f1, 1.f);
  r0 = __int_as_float(__float_as_int(p0) + (__float_as_int(t0) << 23));
  r1 = __int_as_float(__float_as_int(p1) + (__float_as_int(t1) << 23));
}

// Which of every 8 consecutive score pairs take the FMA-pipe exponential (bit i = pair i). The split
// forms of the kernel, whose softmax warps all work on one tile in lockstep, are bound by the MUFU and
// gain from moving two pairs of eight; the row-owner form is bound by issue slots and keeps them all
// on the MUFU.
constexpr uint32_t EX2_FMA_PAIRS_2_OF_8 = 0x88u;   // pairs 3 and 7
constexpr uint32_t EX2_FMA_PAIRS_NONE = 0x00u;

// p[c] = 2^(s[c] * scale_log2 - base) for 32 scores starting at s[first]; returns their 16 packed
// bf16 pairs in pk and adds the fp32 values into the four packed partial sums.
template <uint32_t FMA_PAIRS, int N>
__device__ __forceinline__ void exp_chunk(const float (&s)[N], int first, float scale_log2, float base,
                                          uint32_t (&pk)[16], f2 (&sum)[4]) {
  const float nbase = -base;
#pragma unroll
  for (int c = 0; c < 16; ++c) {
    const float x0 = fmaf(s[first + 2 * c], scale_log2, nbase);
    const float x1 = fmaf(s[first + 2 * c + 1], scale_log2, nbase);
    float p0, p1;
    if ((FMA_PAIRS >> (c & 7)) & 1u) {
      ex2_fma_pipe(x0, x1, p0, p1);
    } else {
      p0 = ptx::ex2(x0);
      p1 = ptx::ex2(x1);
    }
    sum[c & 3] = add2(sum[c & 3], pack2(p0, p1));
    pk[c] = ptx::pack_bf16(p0, p1);
  }
}

__device__ __forceinline__ float sum4(const f2 (&sum)[4]) {
  float a, b, c, d, e, f, g, h;
  unpack2(sum[0], a, b);
  unpack2(sum[1], c, d);
  unpack2(sum[2], e, f);
  unpack2(sum[3], g, h);
  return ((a + b) + (c + d)) + ((e + f) + (g + h));
}

}  // namespace sm
}  // namespace intra
