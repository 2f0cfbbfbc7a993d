// Forward sparse attention for the five INTRA patterns on sm_100a.
//
// One CTA computes one tile of intra_index.h: up to 128 query rows of one head against the tile's
// ordered key slots, 128 slots at a time, flash-attention style:
//
//   loader warps   evaluate the index maps and gather the (non-contiguous) Q / K / V token rows
//                  with 16-byte cp.async copies into 128-byte-swizzled shared-memory tiles
//   MMA warp       one thread issues tcgen05.mma:  S = Q K^T  (both operands in shared memory) and
//                  O += P V  (P read from tensor memory, V from shared memory)
//   softmax warps  one thread per query row: read S from tensor memory, apply the row's key-slot
//                  interval [lo, hi] (only on tiles the interval does not cover), online softmax
//                  in fp32 with a lazily updated running maximum, write P as bf16 back to tensor
//                  memory over S, rescale O when the maximum moved, and finally normalise O and
//                  store the rows to their token positions
//
// Tensor memory per CTA: 128 columns for S/P and 128 for O, so two CTAs share an SM and one CTA's
// softmax overlaps the other's MMAs. Every wait is bounded; a wait that gives up raises the CTA's
// abort flag, every role leaves its loop, and the kernel reports a status instead of hanging.
//
// It replaces the reference's mma.sync kernels compute_attn_1rowblock_sparse_16group_llm,
// compute_attn_1rowblock_sw_llm, ..._mask0_8group_text_front and ..._masksw_text_front
// (csrc/flash_attn/src/flash_fwd_kernel.h:5294-5707, 5712-6158, 4852-5293, 3970-4851).
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
constexpr int FWD_THREADS = 384;                        // softmax WG | loader WG | MMA warp (+3 idle)
constexpr int FWD_SMEM_BYTES = 3 * TILE_BYTES + 1024;   // Q, K, V + alignment slack
constexpr int TMEM_COLS = 256;
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

__global__ void __launch_bounds__(FWD_THREADS, 2) intra_fwd_kernel(const FwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t bars[9];
  __shared__ uint32_t tmem_base_smem;
  __shared__ int abort_flag;

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;

  // ---- which tile --------------------------------------------------------------------------
  const int heads_total = p.B * p.H;
  const int idx = blockIdx.x / heads_total;
  const int bh = blockIdx.x % heads_total;
  const int b = bh / p.H;
  const int h = bh % p.H;
  const int hk = h / (p.H / p.Hkv);
  const Tile t = make_tile(p.prob, idx);
  if (t.n_kv_tiles == 0) return;                       // group shorter than this tile's first row
  if (tid == 0) abort_flag = *reinterpret_cast<volatile int*>(p.status);
  __syncthreads();
  if (abort_flag != 0) return;                         // an earlier CTA already failed (CTA-uniform)
  __syncthreads();

  uint64_t* q_full = &bars[0];
  uint64_t* k_full = &bars[1];
  uint64_t* k_empty = &bars[2];
  uint64_t* v_full = &bars[3];
  uint64_t* v_empty = &bars[4];
  uint64_t* s_full = &bars[5];
  uint64_t* p_full = &bars[6];
  uint64_t* o_done = &bars[7];
  uint64_t* drain = &bars[8];

  const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t q_smem = smem_base;
  const uint32_t k_smem = smem_base + TILE_BYTES;
  const uint32_t v_smem = smem_base + 2 * TILE_BYTES;

  if (tid == 0) {
    abort_flag = 0;
    ptx::mbar_init(q_full, 128);
    ptx::mbar_init(k_full, 128);
    ptx::mbar_init(k_empty, 1);
    ptx::mbar_init(v_full, 128);
    ptx::mbar_init(v_empty, 1);
    ptx::mbar_init(s_full, 1);
    ptx::mbar_init(p_full, 128);
    ptx::mbar_init(o_done, 1);
    ptx::mbar_init(drain, 1);
    ptx::fence_mbar_init();
  }
  if (warp == 0) {
    ptx::tmem_alloc(&tmem_base_smem, TMEM_COLS);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem = tmem_base_smem;
  const int n_kv = t.n_kv_tiles;
  volatile int* abort_p = &abort_flag;

  if (warp < 4) {
    // ================================ softmax / correction / epilogue ==========================
    ptx::setmaxnreg_inc<160>();
    const int row = tid;                                  // TMEM lane == query row
    const uint32_t lane_addr = tmem + (uint32_t(warp * 32) << 16);
    int token, lo, hi;
    q_row(p.prob, t, row, &token, &lo, &hi);
    float m_run = -CUDART_INF_F;                          // running maximum of raw scores
    float l_run = 0.f;                                    // running sum of p
    bool ok = true;

    for (int n = 0; n < n_kv && ok; ++n) {
      ok = ptx::mbar_wait(s_full, n & 1, abort_p);
      if (!ok) { if (*abort_p == 1) *abort_p = 11; break; }
      if (n > 0) {
        ok = ptx::mbar_wait(o_done, (n - 1) & 1, abort_p);
        if (!ok) { if (*abort_p == 1) *abort_p = 12; break; }
      }
      ptx::tc_fence_after();

      float s[TILE_N];
#pragma unroll
      for (int c = 0; c < 4; ++c) ptx::tmem_ld32(lane_addr + TMEM_S + c * 32, reinterpret_cast<uint32_t*>(s) + c * 32);
      ptx::tmem_wait_ld();

      const int u0 = n * TILE_N;
      if (lo > u0 || hi < u0 + TILE_N - 1) {              // this row's interval does not cover the tile
#pragma unroll
        for (int c = 0; c < TILE_N; ++c) {
          const int u = u0 + c;
          if (u < lo || u > hi) s[c] = -CUDART_INF_F;
        }
      }
      float tmax = s[0];
#pragma unroll
      for (int c = 1; c < TILE_N; ++c) tmax = fmaxf(tmax, s[c]);
      const float m_new = fmaxf(m_run, tmax);
      // Move the running maximum only when the scores outgrow it by 2^8; until then p is merely
      // scaled by a constant that the final division by the row sum removes.
      const bool grow = (m_new - m_run) * p.scale_log2 > RESCALE_THRESHOLD;
      float alpha = 1.f;
      if (grow) {
        alpha = ptx::ex2((m_run - m_new) * p.scale_log2);  // 0 when m_run is still -inf
        l_run *= alpha;
        m_run = m_new;
      }
      if (n > 0 && __any_sync(0xffffffffu, grow)) {       // rare once the maximum has settled
#pragma unroll 1
        for (int c = 0; c < HEAD_DIM / 8; ++c) {
          uint32_t o[8];
          ptx::tmem_ld8(lane_addr + TMEM_O + c * 8, o);
          ptx::tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 8; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
          ptx::tmem_st8(lane_addr + TMEM_O + c * 8, o);
        }
      }
      const float base = (m_run == -CUDART_INF_F) ? 0.f : m_run * p.scale_log2;
      float lsum = 0.f;
#pragma unroll
      for (int c4 = 0; c4 < 4; ++c4) {                    // 32 scores -> 16 packed columns of P
        uint32_t pk[16];
#pragma unroll
        for (int c = 0; c < 16; ++c) {
          const float p0 = ptx::ex2(fmaf(s[c4 * 32 + 2 * c], p.scale_log2, -base));
          const float p1 = ptx::ex2(fmaf(s[c4 * 32 + 2 * c + 1], p.scale_log2, -base));
          lsum += p0 + p1;
          pk[c] = ptx::pack_bf16(p0, p1);
        }
        ptx::tmem_st16(lane_addr + TMEM_S + c4 * 16, pk);
      }
      l_run += lsum;
      ptx::tmem_wait_st();
      ptx::tc_fence_before();
      ptx::mbar_arrive(p_full);
    }

    if (ok) {
      ok = ptx::mbar_wait(o_done, (n_kv - 1) & 1, abort_p);
      if (!ok && *abort_p == 1) *abort_p = 13;
    }
    if (ok) {
      ptx::tc_fence_after();
      const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
      if (p.lse != nullptr && token >= 0) p.lse[(int64_t(b) * p.H + h) * p.prob.S + token] = row_lse(m_run, l_run, p.scale_log2);
      __nv_bfloat16* dst = p.o + b * p.os.sb + int64_t(token < 0 ? 0 : token) * p.os.ss + h * p.os.sh;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t o[32];
        ptx::tmem_ld32(lane_addr + TMEM_O + c * 32, o);
        ptx::tmem_wait_ld();
        if (token >= 0) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint4 w;
            w.x = ptx::pack_bf16(__uint_as_float(o[8 * i + 0]) * inv, __uint_as_float(o[8 * i + 1]) * inv);
            w.y = ptx::pack_bf16(__uint_as_float(o[8 * i + 2]) * inv, __uint_as_float(o[8 * i + 3]) * inv);
            w.z = ptx::pack_bf16(__uint_as_float(o[8 * i + 4]) * inv, __uint_as_float(o[8 * i + 5]) * inv);
            w.w = ptx::pack_bf16(__uint_as_float(o[8 * i + 6]) * inv, __uint_as_float(o[8 * i + 7]) * inv);
            *reinterpret_cast<uint4*>(dst + c * 32 + i * 8) = w;
          }
        }
      }
    }
  } else if (warp < 8) {
    // ================================ loaders ===================================================
    ptx::setmaxnreg_dec<40>();
    const int lt = tid - 128;
    const int chunk = lt & 15;                            // 16-byte chunk of the 256-byte row
    const int rsub = lt >> 4;                             // row within a pass of 8 rows
    bool ok = true;
    {
      const __nv_bfloat16* qb = p.q + b * p.qs.sb + h * p.qs.sh + chunk * 8;
#pragma unroll 4
      for (int ps = 0; ps < TILE_M / 8; ++ps) {
        const int row = ps * 8 + rsub;
        int token, lo, hi;
        q_row(p.prob, t, row, &token, &lo, &hi);
        const void* src = token >= 0 ? static_cast<const void*>(qb + int64_t(token) * p.qs.ss) : static_cast<const void*>(p.q);
        ptx::cp_async_16(q_smem + tile_offset(row, chunk), src, token >= 0 ? 16u : 0u);
      }
      ptx::cp_async_commit();
    }
    const __nv_bfloat16* kb = p.k + b * p.ks.sb + hk * p.ks.sh + chunk * 8;
    const __nv_bfloat16* vb = p.v + b * p.vs.sb + hk * p.vs.sh + chunk * 8;
    for (int n = 0; n < n_kv && ok; ++n) {
      if (n > 0) {
        ok = ptx::mbar_wait(k_empty, (n - 1) & 1, abort_p);
        if (!ok) { if (*abort_p == 1) *abort_p = 21; break; }
      }
#pragma unroll 4
      for (int ps = 0; ps < TILE_N / 8; ++ps) {
        const int row = ps * 8 + rsub;
        const int token = key_token(p.prob, t, n * TILE_N + row);
        const void* src = token >= 0 ? static_cast<const void*>(kb + int64_t(token) * p.ks.ss) : static_cast<const void*>(p.k);
        ptx::cp_async_16(k_smem + tile_offset(row, chunk), src, token >= 0 ? 16u : 0u);
      }
      ptx::cp_async_commit();
      if (n > 0) {
        ok = ptx::mbar_wait(v_empty, (n - 1) & 1, abort_p);
        if (!ok) { if (*abort_p == 1) *abort_p = 22; break; }
      }
#pragma unroll 4
      for (int ps = 0; ps < TILE_N / 8; ++ps) {
        const int row = ps * 8 + rsub;
        const int token = key_token(p.prob, t, n * TILE_N + row);
        const void* src = token >= 0 ? static_cast<const void*>(vb + int64_t(token) * p.vs.ss) : static_cast<const void*>(p.v);
        ptx::cp_async_16(v_smem + tile_offset(row, chunk), src, token >= 0 ? 16u : 0u);
      }
      ptx::cp_async_commit();
      if (n == 0) {                                       // Q landed (oldest of three groups)
        ptx::cp_async_wait<2>();
        ptx::fence_proxy_async_smem();
        ptx::mbar_arrive(q_full);
      }
      ptx::cp_async_wait<1>();                            // K(n) landed
      ptx::fence_proxy_async_smem();
      ptx::mbar_arrive(k_full);
      ptx::cp_async_wait<0>();                            // V(n) landed
      ptx::fence_proxy_async_smem();
      ptx::mbar_arrive(v_full);
    }
    ptx::cp_async_wait<0>();
  } else {
    // ================================ MMA issue ==================================================
    ptx::setmaxnreg_dec<40>();
    if (warp == 8) {
      bool ok = ptx::mbar_wait(q_full, 0, abort_p);
      if (!ok && *abort_p == 1) *abort_p = 31;
      for (int n = 0; n < n_kv && ok; ++n) {
        ok = ptx::mbar_wait(k_full, n & 1, abort_p);
        if (!ok) { if (*abort_p == 1) *abort_p = 32; break; }
        ptx::tc_fence_after();
        if (ptx::elect_one()) {
          issue_qk(q_smem, k_smem, tmem + TMEM_S);
          ptx::mma_commit(k_empty);
          ptx::mma_commit(s_full);
        }
        __syncwarp();
        ok = ptx::mbar_wait(p_full, n & 1, abort_p);
        if (!ok) { if (*abort_p == 1) *abort_p = 33; break; }
        ok = ptx::mbar_wait(v_full, n & 1, abort_p);
        if (!ok) { if (*abort_p == 1) *abort_p = 34; break; }
        ptx::tc_fence_after();
        if (ptx::elect_one()) {
          issue_pv(tmem + TMEM_S, v_smem, tmem + TMEM_O, n > 0);
          ptx::mma_commit(v_empty);
          ptx::mma_commit(o_done);
        }
        __syncwarp();
      }
      if (!ok) {                                          // let MMAs in flight finish before TMEM is freed
        if (ptx::elect_one()) ptx::mma_commit(drain);
        __syncwarp();
        int dummy = 0;
        ptx::mbar_wait(drain, 0, &dummy, 100);
      }
    }
  }

  // ---- teardown --------------------------------------------------------------------------------
  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem, TMEM_COLS);
  }
  if (tid == 0 && abort_flag != 0) atomicCAS(p.status, 0, STATUS_WAIT_BASE + abort_flag);
}

}  // namespace intra
