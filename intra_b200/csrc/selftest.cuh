// Diagnostics that run on the device: a single-tile check of the two tensor-core contractions
// through the same tile layout, descriptors and TMEM paths as the attention kernel, and a kernel
// that enumerates the (query, key) pairs the device-side index maps visit.
#pragma once
#include "attn_kernel.cuh"

namespace intra {

// a, b, v: contiguous [128][128] bf16.  s_out = a * b^T (fp32, [128][128]);
// o_out = bf16(s_out * p_scale) * v (fp32, [128][128]).  One CTA of 128 threads.
__global__ void __launch_bounds__(128, 1)
umma_selftest_kernel(const __nv_bfloat16* a, const __nv_bfloat16* b, const __nv_bfloat16* v, float p_scale,
                     float* s_out, float* o_out, int* status) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t bar;
  __shared__ uint32_t tmem_base_smem;
  __shared__ int abort_flag;
  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t a_smem = smem_base, b_smem = smem_base + TILE_BYTES, v_smem = smem_base + 2 * TILE_BYTES;
  if (tid == 0) {
    abort_flag = 0;
    ptx::mbar_init(&bar, 1);
    ptx::fence_mbar_init();
  }
  if (warp == 0) {
    ptx::tmem_alloc(&tmem_base_smem, TMEM_COLS);
    ptx::tmem_relinquish();
  }
  const int chunk = tid & 15, rsub = tid >> 4;
  for (int ps = 0; ps < TILE_M / 8; ++ps) {
    const int row = ps * 8 + rsub;
    const size_t off = size_t(row) * HEAD_DIM + chunk * 8;
    ptx::cp_async_16(a_smem + tile_offset(row, chunk), a + off, 16);
    ptx::cp_async_16(b_smem + tile_offset(row, chunk), b + off, 16);
    ptx::cp_async_16(v_smem + tile_offset(row, chunk), v + off, 16);
  }
  ptx::cp_async_commit();
  ptx::cp_async_wait<0>();
  ptx::fence_proxy_async_smem();
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem = tmem_base_smem;
  const uint32_t lane_addr = tmem + (uint32_t(warp * 32) << 16);

  if (tid == 0) {
    issue_qk(a_smem, b_smem, tmem + TMEM_S);
    ptx::mma_commit(&bar);
  }
  bool ok = ptx::mbar_wait(&bar, 0, &abort_flag, 1000);
  ptx::tc_fence_after();
  float s[TILE_N];
  if (ok) {
#pragma unroll
    for (int c = 0; c < 4; ++c) ptx::tmem_ld32(lane_addr + TMEM_S + c * 32, reinterpret_cast<uint32_t*>(s) + c * 32);
    ptx::tmem_wait_ld();
#pragma unroll
    for (int c = 0; c < TILE_N; ++c) s_out[tid * TILE_N + c] = s[c];
    uint32_t pk[TILE_N / 2];
#pragma unroll
    for (int c = 0; c < TILE_N / 2; ++c) pk[c] = ptx::pack_bf16(s[2 * c] * p_scale, s[2 * c + 1] * p_scale);
    ptx::tmem_st32(lane_addr + TMEM_S, pk);
    ptx::tmem_st32(lane_addr + TMEM_S + 32, pk + 32);
    ptx::tmem_wait_st();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  if (tid == 0 && ok) {
    issue_pv(tmem + TMEM_S, v_smem, tmem + TMEM_O, false);
    ptx::mma_commit(&bar);
  }
  if (ok) ok = ptx::mbar_wait(&bar, 1, &abort_flag, 1000);
  ptx::tc_fence_after();
  if (ok) {
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      uint32_t o[32];
      ptx::tmem_ld32(lane_addr + TMEM_O + c * 32, o);
      ptx::tmem_wait_ld();
#pragma unroll
      for (int i = 0; i < 32; ++i) o_out[tid * HEAD_DIM + c * 32 + i] = __uint_as_float(o[i]);
    }
  }
  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem, TMEM_COLS);
  }
  if (tid == 0 && abort_flag != 0) atomicCAS(status, 0, STATUS_WAIT_BASE + 90);
}

// counts[q * S + k] += 1 for every (query token, key token) pair the tiles of `prob` visit.
// One block per tile, one thread per query row.
__global__ void visited_kernel(Problem prob, uint8_t* counts) {
  const Tile t = make_tile(prob, blockIdx.x);
  if (t.n_kv_tiles == 0) return;
  int token, lo, hi;
  q_row(prob, t, threadIdx.x, &token, &lo, &hi);
  if (token < 0) return;
  for (int u = lo; u <= hi; ++u) {
    const int kt = key_token(prob, t, u);
    if (kt >= 0) {
      uint8_t* c = counts + size_t(token) * prob.S + kt;   // each (q, k) belongs to one row of one tile
      *c = static_cast<uint8_t>(*c + 1);
    }
  }
}

}  // namespace intra
