// Definitions shared by the attention kernel (attn_kernel_dual.cuh) and the device self-tests
// (selftest.cuh): tile geometry, the parameter block, the shared-memory tile layout and the two
// tensor-core contractions of flash attention on sm_100a,
//
//   S = Q K^T    both operands 128-byte-swizzled shared-memory tiles, accumulator in tensor memory
//   O += P V     P read from tensor memory (bf16, written over S by the softmax), V from shared memory
//
// each a chain of eight tcgen05.mma of K = 16. They replace flash::gemm / flash::gemm_rs of the
// reference (csrc/flash_attn/src/utils.h:133-181) and its tile traits (src/kernel_traits.h:52-404).
//
// Abort protocol of every kernel in this directory: all waits are bounded (ptx::mbar_wait). A wait
// that runs out raises the CTA's shared abort flag with the id of the wait site; every other role
// sees the flag in its own next wait and leaves its loop; the CTA then lets tensor-core work in flight
// finish, frees its tensor memory and records STATUS_WAIT_BASE + id in the status word with an
// atomicCAS from 0, so the word keeps the first failure until the host resets it. Kernels never read
// the word: a recorded failure does not turn later launches into no-ops.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math_constants.h>
#include <stdint.h>

#include "intra_index.h"
#include "ptx.cuh"

namespace intra {

constexpr int HEAD_DIM = 128;
constexpr int TILE_BYTES = TILE_M * HEAD_DIM * 2;       // 32 KiB: 128 rows x 256 B
constexpr int HALF_BYTES = TILE_BYTES / 2;              // one 64-element half of the head dim
constexpr int SELFTEST_SMEM_BYTES = 3 * TILE_BYTES + 1024;   // one tile each for A, B, V + alignment slack
constexpr int TMEM_COLS = 256;                          // the single-tile self-test's allocation
constexpr int TMEM_S = 0;                               // S (fp32, 128 cols); P (bf16 pairs) over cols 0..63
constexpr int TMEM_O = 128;                             // O (fp32, 128 cols)
constexpr float RESCALE_THRESHOLD = 8.0f;               // in log2 units: p stays below 2^8

// Status codes written to FwdParams::status by a CTA that gave up.
constexpr int STATUS_WAIT_BASE = 100;                   // + id of the wait site that ran out

struct TensorView {      // (batch, token, head, 128) view, strides in elements
  int64_t sb, ss, sh;
};

struct FwdParams {
  const __nv_bfloat16* q;
  const __nv_bfloat16* k;
  const __nv_bfloat16* v;
  __nv_bfloat16* o;
  TensorView qs, ks, vs, os;
  int B, H, Hkv;
  Problem prob;
  float scale_log2;      // softmax_scale * log2(e)
  int* status;           // device word: 0 = ok
  float* lse;            // optional (B, H, S) fp32: natural log of each row's softmax denominator; null = not wanted
};

// log(sum_j exp(scale * s_j)) of a row from the running maximum its probabilities were taken against
// (in raw score units, possibly stale: the lazy rescale keeps p = 2^(s * scale_log2 - m * scale_log2)
// consistent with it) and their sum. The reference computes the same quantity and drops it
// (csrc/flash_attn/src/flash_fwd_kernel.h:5675).
__device__ __forceinline__ float row_lse(float m_run, float l_sum, float scale_log2) {
  return l_sum > 0.f ? (m_run * scale_log2 + log2f(l_sum)) * 0.6931471805599453f : -CUDART_INF_F;
}

// Byte offset of 16-byte chunk `chunk` (0..15) of row `row` inside a swizzled tile: two 64-element
// halves, 128-byte rows, chunk index xor-ed with (row mod 8) as the 128-byte swizzle prescribes.
__device__ __forceinline__ uint32_t tile_offset(int row, int chunk) {
  return (chunk >> 3) * HALF_BYTES + row * 128 + (((chunk & 7) ^ (row & 7)) << 4);
}

// Descriptor of a whole swizzled tile as a K-major operand (Q, or K for QK^T) and as an MN-major one
// (V for PV). The per-MMA descriptors differ from these only in the start-address field, so the issuing
// thread adds a constant per step instead of rebuilding them.
__device__ __forceinline__ uint64_t tile_desc_kmajor(uint32_t smem) { return ptx::smem_desc_sw128(smem, 16, 1024); }
__device__ __forceinline__ uint64_t tile_desc_mnmajor(uint32_t smem) { return ptx::smem_desc_sw128(smem, HALF_BYTES, 1024); }

// S[128 x 128] = A[128 x 128] * B[128 x 128]^T, both K-major tiles: 8 MMAs of K = 16. Step s reads the
// 32-byte slice s % 4 of half s / 4 of each row; descriptor addresses count 16-byte units.
__device__ __forceinline__ void issue_qk_desc(uint64_t q_desc, uint64_t k_desc, uint32_t s_tmem) {
  constexpr uint32_t idesc = ptx::idesc_bf16_f32(TILE_M, TILE_N, 0, 0);
#pragma unroll
  for (int s = 0; s < HEAD_DIM / 16; ++s) {
    const uint64_t off = uint64_t(((s >> 2) * HALF_BYTES + (s & 3) * 32) >> 4);
    if (s == 0) ptx::mma_ss_first(s_tmem, q_desc + off, k_desc + off, idesc);
    else ptx::mma_ss_acc(s_tmem, q_desc + off, k_desc + off, idesc);
  }
}
__device__ __forceinline__ void issue_qk(uint32_t q_smem, uint32_t k_smem, uint32_t s_tmem) {
  issue_qk_desc(tile_desc_kmajor(q_smem), tile_desc_kmajor(k_smem), s_tmem);
}
// O[128 x 128] (+)= P[128 x 128 keys] * V[128 keys x 128]: A from tensor memory (bf16 pairs, 8
// columns per 16 keys), B = V tile read MN-major (head dim contiguous): 8 MMAs of K = 16 keys, each
// 16 keys = 2048 bytes further into the tile.
__device__ __forceinline__ void issue_pv_desc(uint32_t p_tmem, uint64_t v_desc, uint32_t o_tmem, bool accumulate) {
  constexpr uint32_t idesc = ptx::idesc_bf16_f32(TILE_M, HEAD_DIM, 0, 1);
  if (accumulate) ptx::mma_ts_acc(o_tmem, p_tmem, v_desc, idesc);
  else ptx::mma_ts_first(o_tmem, p_tmem, v_desc, idesc);
#pragma unroll
  for (int s = 1; s < TILE_N / 16; ++s) ptx::mma_ts_acc(o_tmem, p_tmem + s * 8, v_desc + uint64_t(s * (2048 >> 4)), idesc);
}
__device__ __forceinline__ void issue_pv(uint32_t p_tmem, uint32_t v_smem, uint32_t o_tmem, bool accumulate) {
  issue_pv_desc(p_tmem, tile_desc_mnmajor(v_smem), o_tmem, accumulate);
}

}  // namespace intra
