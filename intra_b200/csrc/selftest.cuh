// Diagnostics that run on the device: a single-tile check of the two tensor-core contractions
// through the same tile layout, descriptors and TMEM paths as the attention kernel; a kernel that
// enumerates the (query, key) pairs the device-side index maps visit; a kernel that fetches every
// query and key tile of a problem through the attention kernel's own TMA code and reports which token
// rows arrived; and a kernel whose wait is never satisfied, to exercise the abort protocol.
#pragma once
#include "attn_kernel.cuh"
#include "attn_kernel_dual.cuh"

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

// ---- TMA rows ---------------------------------------------------------------------------------------
// One CTA per item of the attention kernel's item list. Thread 0 plans the item exactly as the planner
// warp does and requests its tiles with the attention kernel's own fetch functions; the 128 threads
// then read row r's first 16 bytes of both 64-element halves out of the swizzled tile and decode the
// token id the test encoded there: elements 0..2 of each half hold (token + 1) in base 256, so a
// zero-filled row decodes to -1; elements 3..5 hold the head, the batch and which tensor it is (0 q,
// 1 k, 2 v). A row whose two halves disagree reports -2, one from the wrong head or batch -4, one from
// the wrong tensor -5.
//   q_out[item][s][r]                    sub-tile s, query row r
//   k_out[item][s][n][r], v_out likewise key tile n (s = 0 only, unless the sub-tiles keep their own keys)
__device__ __forceinline__ int decode_row_token(const uint8_t* tile, int row, int head, int batch, int tensor_id) {
  int tok[2];
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(tile + tile_offset(row, half * 8));
    tok[half] = int(__bfloat162float(e[0])) + 256 * int(__bfloat162float(e[1])) + 65536 * int(__bfloat162float(e[2])) - 1;
    if (tok[half] >= 0 && (int(__bfloat162float(e[3])) != head || int(__bfloat162float(e[4])) != batch)) return -4;
    if (tok[half] >= 0 && int(__bfloat162float(e[5])) != tensor_id) return -5;
  }
  return tok[0] == tok[1] ? tok[0] : -2;
}

template <bool kSplitKV>
__global__ void __launch_bounds__(128, 1)
tma_rows_selftest_kernel(const __grid_constant__ DualParams p, int* q_out, int* k_out, int* v_out, int max_kv) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  __shared__ ItemSlot sl;
  const int tid = threadIdx.x;
  const int item = blockIdx.x;
  const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint8_t* tile = smem_raw + (smem_base - ptx::smem_u32(smem_raw));
  const DualItem di = dual_decode(p, item);
  const int n_kv = di.pt.kv.n_kv_tiles;
  if (n_kv == 0) return;                                   // CTA-uniform
  if (tid == 0) {
    abort_flag = 0;
    ptx::mbar_init(&bar, 1);
    ptx::fence_mbar_init();
    sl.pt = di.pt;
    sl.b = di.b; sl.h0 = di.h0; sl.h1 = di.h1; sl.hk = di.hk;
    if (!kSplitKV) plan_slot_boxes(p, di, sl);
  }
  __syncthreads();
  const TmaOperand q_op = {&p.maps.q_main, &p.maps.q_text, &p.maps.q_main};
  const TmaOperand k_op = {&p.maps.k_main, &p.maps.k_text, &p.maps.k_aux};
  const TmaOperand v_op = {&p.maps.v_main, &p.maps.v_text, &p.maps.v_aux};
  const CUtensorMap* k_main = p.f.prob.kind == KIND_IMG_GATHER0 ? k_op.aux_map : k_op.main_map;
  const CUtensorMap* v_main = p.f.prob.kind == KIND_IMG_GATHER0 ? v_op.aux_map : v_op.main_map;
  uint32_t phase = 0;
  bool ok = true;
  // fetch(): thread 0 has issued one tile's loads onto `bar`; everyone waits for them and reads a row.
  auto collect = [&](int* dst, int head, int tensor_id) {
    ok = ok && ptx::mbar_wait(&bar, phase & 1, &abort_flag, 1000);
    ++phase;
    if (ok) dst[tid] = decode_row_token(tile, tid, head, sl.b, tensor_id);
    __syncthreads();                                       // the buffer is reused by the next fetch
  };
  for (int sx = 0; sx < 2; ++sx) {
    if (tid == 0 && abort_flag == 0) {
      ptx::mbar_arrive_expect_tx(&bar, TILE_BYTES);
      if (kSplitKV) tma_fetch_q(p.f.prob, pair_kv_map(sl.pt, 1, sx), sx ? sl.h1 : sl.h0, sl.b, q_op, smem_base, &bar);
      else if (sx == 0) tma_fetch_box(sl.q0, sl.q0_rank4, sl.q0_text ? q_op.text_map : q_op.main_map, smem_base, &bar);
      else tma_fetch_box(sl.q1, sl.q1_rank4, sl.q1_text ? q_op.text_map : q_op.main_map, smem_base, &bar);
    }
    collect(q_out + (size_t(item) * 2 + sx) * TILE_M, sx ? sl.h1 : sl.h0, 0);
  }
  for (int is_v = 0; is_v < 2; ++is_v) {
    int* out = is_v ? v_out : k_out;
    for (int sx = 0; sx < (kSplitKV ? 2 : 1); ++sx) {
      for (int n = 0; n < n_kv; ++n) {
        if (tid == 0 && abort_flag == 0) {
          ptx::mbar_arrive_expect_tx(&bar, TILE_BYTES);
          if (kSplitKV) {
            tma_fetch_kv(p.f.prob, pair_kv_map(sl.pt, 1, sx), n, sl.hk, sl.b, is_v ? v_op : k_op, smem_base, &bar);
          } else {
            const KvSegment& sg = n < sl.n_text ? sl.seg0 : sl.seg1;
            const CUtensorMap* m = is_v ? (sg.text ? v_op.text_map : v_main) : (sg.text ? k_op.text_map : k_main);
            tma_fetch_planned(sg, n, m, smem_base, &bar);
          }
        }
        collect(out + ((size_t(item) * 2 + sx) * max_kv + n) * TILE_N, sl.hk, 1 + is_v);
      }
    }
  }
  if (tid == 0 && abort_flag != 0) atomicCAS(p.f.status, 0, STATUS_WAIT_BASE + 91);
}

// ---- abort protocol ---------------------------------------------------------------------------------
// Two warps of one CTA, tensor memory allocated as in the attention kernel. Warp 1 waits on a barrier
// that nothing ever arrives at, with a limit of `limit_ms`; warp 0 waits on a second such barrier with
// the attention kernel's long limit and must be released by the abort flag warp 1 raises, not by its
// own clock. The CTA then tears down as the attention kernel does: tensor memory freed, status recorded.
// The kernel returns normally; nothing traps and no wait is unbounded.
__global__ void __launch_bounds__(64, 1) abort_selftest_kernel(int limit_ms, int* status, long long* waited_ns) {
  __shared__ uint64_t bars[2];
  __shared__ uint32_t tmem_base_smem;
  __shared__ int abort_flag;
  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  if (tid == 0) {
    abort_flag = 0;
    ptx::mbar_init(&bars[0], 1);
    ptx::mbar_init(&bars[1], 1);
    ptx::fence_mbar_init();
  }
  if (warp == 0) {
    ptx::tmem_alloc(&tmem_base_smem, 32);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem = tmem_base_smem;
  volatile int* abort_p = &abort_flag;
  const uint64_t t0 = ptx::globaltimer_ns();
  if (warp == 1) {
    if (!ptx::mbar_wait(&bars[1], 0, abort_p, uint32_t(limit_ms)) && *abort_p == 1) *abort_p = 92;
  } else {
    if (!ptx::mbar_wait(&bars[0], 0, abort_p) && *abort_p == 1) *abort_p = 93;
  }
  if (tid == 0) *waited_ns = static_cast<long long>(ptx::globaltimer_ns() - t0);
  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem, 32);
  }
  if (tid == 0 && abort_flag != 0) atomicCAS(status, 0, STATUS_WAIT_BASE + abort_flag);
}

}  // namespace intra
