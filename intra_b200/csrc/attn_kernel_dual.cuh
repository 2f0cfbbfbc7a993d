// Persistent, ping-pong forward kernel: each CTA owns one SM and walks a static list of pair tiles
// (intra_index.h): two 128-row query sub-tiles that share every K / V tile brought into shared
// memory (or, for Gather-0, keep a K / V buffer each). While one sub-tile's softmax runs on the CUDA
// cores, the tensor core works on the other's QK^T and PV, so the two pipes overlap inside one CTA.
//
// Warp roles (N = softmax column split, 2 or 4):
//   warps [0, 4N)      softmax / correction, all on one sub-tile at a time, alternating between the two:
//                      warp w owns rows 32 (w % 4) .. +31 and score columns [(w / 4) * 128 / N, +128 / N)
//                      (TMEM: S0 cols 0-127, S1 cols 128-255, O0 cols 256-383, O1 cols 384-511; P overlays S)
//   warps [4N, 4N+4)   with TMA loads: epilogue (O of a finished item -> bf16 -> global while the softmax
//                      warps are already on the next item); otherwise loaders: index maps + cp.async row
//                      gathers whose completion the copies signal themselves
//   warp 4N+4          an elected thread issues tcgen05.mma in the order QK0(n) PV1(n-1) QK1(n) PV0(n),
//                      carried across item boundaries so that the next item's first QK^T overlaps this
//                      item's last softmax
//   warp 4N+5          one thread issues the TMA loads: Q0, Q1 and a 2-stage ring each for K and V
//   warp 4N+6          planner: decodes the CTA's items a few ahead into a ring in shared memory (key-tile
//                      count, per-row token and key interval, TMA box coordinates) for all other roles
//
// Items are dealt to CTAs heaviest first in boustrophedon order, which needs no counters in global
// memory. Every wait is bounded; see attn_kernel.cuh for the abort protocol, which is the same.
//
// A tcgen05.commit costs the tensor pipe about as much as one MMA, so only two are issued per key tile:
// after QK0 (S0 ready) and after QK1 (S1 ready). Because the pipe completes in issue order the second
// one also tells the loaders that the K stage of that tile, the V stage of the tile before it and - on
// an item's last key tile - the Q buffers may be overwritten; it alternates between two barriers so
// that waiters a tile ahead or behind can never confuse phases. O is signalled once per item.
//
// Replaces, like attn_kernel.cuh, the reference's compute_attn_1rowblock_* kernels
// (csrc/flash_attn/src/flash_fwd_kernel.h:3970-6158) for every pattern.
#pragma once
#include "attn_kernel.cuh"
#include "softmax.cuh"
#include "tma_maps.h"

namespace intra {

// Softmax column split: each query row of a sub-tile is shared by NSPLIT threads (one per softmax
// warpgroup), 128 / NSPLIT score columns each. Two instantiations: NSPLIT = 4 (768 threads) hides more
// latency and wins on short items, NSPLIT = 2 (512 threads) leaves the MMA-issuing warp's scheduler
// less crowded and wins on long ones; the host picks by the key tiles per item.
//
// NSPLIT = 1 is a different pipeline for long items (the "row-owner" form): the softmax warps form two
// sets of four, one per sub-tile, a thread owning its query row alone (no exchange of maxima). Both
// sub-tiles' QK^T go to ONE score buffer in tensor memory, which a set copies to registers and hands
// back at once, while P has a buffer of its own per sub-tile. The tensor core then never waits for a
// softmax phase, only for the copy, and a set has a whole key-tile period for its phase while the
// other set's phase runs beside it and fills its latencies.
template <int NSPLIT>
struct DualCfg {
  static_assert(NSPLIT == 1 || NSPLIT == 2 || NSPLIT == 4, "softmax column split must be 1 (row-owner form), 2 or 4");
  static constexpr int COLS = TILE_N / NSPLIT;            // score columns per softmax thread
  static constexpr int SM_WARPS = NSPLIT == 1 ? 8 : 4 * NSPLIT;   // softmax warps
  static constexpr int SM_THREADS = 32 * SM_WARPS;
  static constexpr int THREADS = SM_THREADS + 256;        // + epilogue / loader warpgroup + MMA / TMA warpgroup
  // setmaxnreg budgets: softmax, epilogue / loaders, MMA / TMA / planner. The last group must not spill:
  // a local-memory access in the MMA-issuing thread's loop stalls the tensor pipe. Sums: 512 threads
  // start with 128 registers each (65536), 768 threads with 80 (61440).
  static constexpr int SM_REGS = NSPLIT == 1 ? 184 : NSPLIT == 2 ? 176 : 88;
  static constexpr int EP_REGS = NSPLIT == 1 ? 48 : 64;
  static constexpr int MMA_REGS = NSPLIT == 1 ? 96 : NSPLIT == 2 ? 96 : 64;
  static_assert(SM_THREADS * SM_REGS + 128 * (EP_REGS + MMA_REGS) <= (NSPLIT == 4 ? 61440 : 65536),
                "register budgets exceed what the CTA was launched with: setmaxnreg.inc would never return");
};
constexpr int KV_STAGES = 2;
constexpr int DUAL_SMEM_BYTES = (2 + 2 * KV_STAGES) * TILE_BYTES + 1024;   // Q0 Q1 | K ring | V ring
constexpr int DUAL_TMEM_COLS = 512;

struct DualParams {
  FwdParams f;
  int row_pairs;        // 0: sub-tiles are two heads of one KV group; 1: two row tiles of one head
  int n_pair_tiles;     // pair tiles per (batch, head or head pair)
  int heads_per_item;   // row_pairs ? H : H / 2  (number of items per pair tile and batch)
  int n_items;          // n_pair_tiles * B * heads_per_item
  int split_kv;         // the two sub-tiles keep their own key lists (Gather-0): K / V buffer s belongs to sub-tile s
  int use_tma;          // tiles are fetched as TMA boxes (tma_maps.h) instead of cp.async row gathers; selects kTma
  int wide_stores;      // every output row is 32-byte aligned: 256-bit global stores
  TmaMaps maps;
};

// The tensor maps of one operand (Q, K or V).
struct TmaOperand {
  const CUtensorMap* main_map;
  const CUtensorMap* text_map;
  const CUtensorMap* aux_map;
};

// Fetch the 128 rows starting at `start` of tile `t` into the swizzled tile at `dst` (two boxes, one
// per half of the head dim), completion counted on `bar`.
__device__ __forceinline__ void tma_fetch_tile(const Problem& prob, const Tile& t, int start, bool text, int head,
                                               int batch, const TmaOperand& op, uint32_t dst, uint64_t* bar) {
  int c[5];
  const int is_text = tma_box_coords(prob, t, start, text, head, batch, c);
  const bool rank4 = is_text || t.kind == KIND_LLM_WINDOW;
  // a Gather-0 problem's text tiles are image-Scatter tiles whose image keys come through the aux view
  const CUtensorMap* m = is_text ? op.text_map : (prob.kind == KIND_IMG_GATHER0 ? op.aux_map : op.main_map);
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    if (rank4) ptx::tma_load_4d(dst + half * HALF_BYTES, m, bar, half * 64, c[1], c[2], c[3]);
    else ptx::tma_load_5d(dst + half * HALF_BYTES, m, bar, half * 64, c[1], c[2], c[3], c[4]);
  }
}

// Query rows of sub-tile `t` (TILE_BYTES in all).
__device__ __forceinline__ void tma_fetch_q(const Problem& prob, const Tile& t, int head, int batch, const TmaOperand& op,
                                            uint32_t dst, uint64_t* bar) {
  if (t.kind == KIND_IMG_GATHER0) {                       // two 8x8 patches, 64 rows each
#pragma unroll
    for (int patch = 0; patch < 2; ++patch) {
      const int pc = t.pcol + (patch == 1 && t.nq > PATCH * PATCH ? 1 : 0);   // no right patch: the left one again
#pragma unroll
      for (int half = 0; half < 2; ++half)
        ptx::tma_load_5d(dst + half * HALF_BYTES + patch * (64 * 128), op.main_map, bar, half * 64, PATCH * pc,
                         PATCH * t.prow, head, batch);
    }
    return;
  }
  int start; bool text;
  tma_q_start(t, &start, &text);
  tma_fetch_tile(prob, t, start, text, head, batch, op, dst, bar);
}

// Key tile n of key-slot map `kv` (TILE_BYTES).
__device__ __forceinline__ void tma_fetch_kv(const Problem& prob, const Tile& kv, int n, int head, int batch,
                                             const TmaOperand& op, uint32_t dst, uint64_t* bar) {
  if (kv.kind == KIND_IMG_GATHER0) {
    // slots: 16 window columns (2 tiles) | 512 text (4 tiles) | the right patch's extra columns (1 tile)
    if (n >= 2 && n < 6) {
#pragma unroll
      for (int half = 0; half < 2; ++half)
        ptx::tma_load_4d(dst + half * HALF_BYTES, op.text_map, bar, half * 64, TILE_N * (n - 2), head, batch);
    } else {
      const int wc0 = n < 2 ? 8 * n : WIN + 8 * (n - 6);
#pragma unroll
      for (int half = 0; half < 2; ++half)
        ptx::tma_load_5d(dst + half * HALF_BYTES, op.main_map, bar, half * 64, kv.r0, kv.c0 + wc0, head, batch);
    }
    return;
  }
  int start; bool text;
  tma_kv_start(kv, n, &start, &text);
  tma_fetch_tile(prob, kv, start, text, head, batch, op, dst, bar);
}

struct DualItem {
  PairTile pt;
  int b, h0, h1, hk;
};

// Item number `seq` of this CTA: heaviest-first list dealt round by round, every other round reversed.
INTRA_HD int dual_item_index(int seq, int cta, int n_cta) {
  return seq * n_cta + ((seq & 1) ? (n_cta - 1 - cta) : cta);
}

INTRA_HD DualItem dual_decode(const DualParams& p, int item) {
  DualItem it;
  const int per_tile = p.f.B * p.heads_per_item;
  const int idx = item / per_tile;
  const int rem = item % per_tile;
  it.b = rem / p.heads_per_item;
  const int hh = rem % p.heads_per_item;
  if (p.row_pairs) { it.h0 = it.h1 = hh; } else { it.h0 = 2 * hh; it.h1 = 2 * hh + 1; }
  it.hk = it.h0 / (p.f.H / p.f.Hkv);
  it.pt = make_pair(p.f.prob, p.row_pairs, idx);
  return it;
}

// Normalise `ncols` (a multiple of 32) accumulator columns of this thread's TMEM lane by `inv` and store
// them as bf16 to `dst` (this row's position in the output). `wide` selects 32-byte stores, which need
// 32-byte aligned rows; tensor-memory loads are finished when the function returns.
__device__ __forceinline__ void store_o_row(uint32_t o_addr, int ncols, float inv, __nv_bfloat16* dst, bool valid,
                                            bool wide) {
  for (int c = 0; c < ncols / 32; ++c) {
    uint32_t o[32];
    ptx::tmem_ld32(o_addr + c * 32, o);
    ptx::tmem_wait_ld();
    if (valid) {
      uint32_t w[16];
#pragma unroll
      for (int i = 0; i < 16; ++i)
        w[i] = ptx::pack_bf16(__uint_as_float(o[2 * i]) * inv, __uint_as_float(o[2 * i + 1]) * inv);
      __nv_bfloat16* d = dst + c * 32;
      if (wide) {
        ptx::st_global_v8(d, w);
        ptx::st_global_v8(d + 16, w + 8);
      } else {
#pragma unroll
        for (int i = 0; i < 4; ++i)
          *reinterpret_cast<uint4*>(d + i * 8) = make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]);
      }
    }
  }
}

// Box coordinates of an item's key tiles are affine in the tile number within at most two segments
// (image kinds: the 512 text keys, then the image keys). The TMA thread works them out once per item
// and afterwards only adds a constant per tile: it shares a scheduler with softmax warps, and every
// instruction it spends per tile slows those down.
struct KvSegment {
  int c[5];          // coordinates of the segment's first tile (c[0] unused)
  int d[5];          // increment per tile
  int first;         // first tile of the segment
  int text;          // 1: text map (rank 4), 0: main / aux map
  int rank4;
};
__device__ __forceinline__ void kv_segment(const Problem& prob, const Tile& kv, int first, int n_kv, int head, int batch,
                                           KvSegment* sg) {
  int start; bool text;
  tma_kv_start(kv, first, &start, &text);
  sg->first = first;
  sg->text = tma_box_coords(prob, kv, start, text, head, batch, sg->c);
  sg->rank4 = sg->text || kv.kind == KIND_LLM_WINDOW;
  int c1[5];
  if (first + 1 < n_kv) {
    tma_kv_start(kv, first + 1, &start, &text);
    tma_box_coords(prob, kv, start, text, head, batch, c1);
  } else {
#pragma unroll
    for (int i = 0; i < 5; ++i) c1[i] = sg->c[i];
  }
#pragma unroll
  for (int i = 0; i < 5; ++i) sg->d[i] = c1[i] - sg->c[i];
}
__device__ __forceinline__ void tma_fetch_planned(const KvSegment& sg, int n, const CUtensorMap* m, uint32_t dst,
                                                  uint64_t* bar) {
  const int k = n - sg.first;
  const int c1 = sg.c[1] + k * sg.d[1], c2 = sg.c[2] + k * sg.d[2], c3 = sg.c[3] + k * sg.d[3];
  if (sg.rank4) {
    ptx::tma_load_4d(dst, m, bar, 0, c1, c2, c3);
    ptx::tma_load_4d(dst + HALF_BYTES, m, bar, 64, c1, c2, c3);
  } else {
    const int c4 = sg.c[4] + k * sg.d[4];
    ptx::tma_load_5d(dst, m, bar, 0, c1, c2, c3, c4);
    ptx::tma_load_5d(dst + HALF_BYTES, m, bar, 64, c1, c2, c3, c4);
  }
}

// One entry of the CTA's item ring: everything any role needs to know about an item, worked out once
// by the planner warp a few items ahead instead of by every warp at every item boundary (the index
// arithmetic has divisions in it, and softmax warps have no issue slots to spare).
constexpr int ITEM_RING = 4;
struct ItemSlot {
  int valid;                     // 0: end of this CTA's list
  int n_kv;                      // key tiles of the item (> 0)
  int b, h0, h1, hk;
  // shared-key modes: what the TMA thread needs to request the tiles
  int n_text;                    // tiles of the first key segment (== n_kv unless text + image keys)
  int q0_text, q1_text, q0_rank4, q1_rank4;
  KvSegment seg0, seg1;
  int q0[5], q1[5];              // box coordinates of the two query sub-tiles
  PairTile pt;                   // for the cp.async loaders (key slots -> tokens)
  int token[2][TILE_M];          // per sub-tile and query row: token (-1: padding row) and its inclusive
  int lo[2][TILE_M];             // interval of key slots
  int hi[2][TILE_M];
};
__device__ __forceinline__ void plan_query(const Problem& prob, const Tile& t, int head, int batch, int c[5], int* is_text,
                                           int* rank4) {
  int start; bool text;
  tma_q_start(t, &start, &text);
  *is_text = tma_box_coords(prob, t, start, text, head, batch, c);
  *rank4 = *is_text || t.kind == KIND_LLM_WINDOW;
}
// TMA box coordinates of an item's two query tiles and of its key tiles (shared-key modes), for the
// thread that issues the loads.
__device__ __forceinline__ void plan_slot_boxes(const DualParams& p, const DualItem& di, ItemSlot& sl) {
  const int n_kv = di.pt.kv.n_kv_tiles;
  const bool image_kind = di.pt.kv.kind == KIND_IMG_SCATTER;
  const int n_text = image_kind && TEXT_LEN / TILE_N < n_kv ? TEXT_LEN / TILE_N : n_kv;
  sl.n_text = n_text;
  kv_segment(p.f.prob, di.pt.kv, 0, n_text, di.hk, di.b, &sl.seg0);
  if (n_text < n_kv) kv_segment(p.f.prob, di.pt.kv, n_text, n_kv, di.hk, di.b, &sl.seg1);
  // an absent sub-tile (odd tile count) is fed the other one's rows; its results are dropped
  const Tile& t0 = di.pt.sub[0].n_kv_tiles > 0 ? di.pt.sub[0] : di.pt.sub[1];
  const Tile& t1 = di.pt.sub[1].n_kv_tiles > 0 ? di.pt.sub[1] : di.pt.sub[0];
  plan_query(p.f.prob, t0, di.h0, di.b, sl.q0, &sl.q0_text, &sl.q0_rank4);
  plan_query(p.f.prob, t1, di.h1, di.b, sl.q1, &sl.q1_text, &sl.q1_rank4);
}
// Planner warp: fills ring slot after ring slot with the CTA's non-empty items, then one end marker.
// slot_ready[r] completes once per fill of slot r; slot_free[r] once all consumers have let go of it.
__device__ __forceinline__ void plan_items(const DualParams& p, ItemSlot* ring, uint64_t* slot_ready, uint64_t* slot_free,
                                           int cta, int n_cta, int lane, bool plan_boxes, volatile int* abort_p) {
  int seq = 0;
  for (int i = 0;; ++i) {
    DualItem di;
    bool valid = false;
    for (;; ++seq) {
      const int item = dual_item_index(seq, cta, n_cta);
      if (item >= p.n_items) break;
      di = dual_decode(p, item);
      if (di.pt.kv.n_kv_tiles > 0) { valid = true; ++seq; break; }
    }
    const int r = i % ITEM_RING;
    if (i >= ITEM_RING && !ptx::mbar_wait(&slot_free[r], ((i / ITEM_RING) - 1) & 1, abort_p)) {
      if (*abort_p == 1) *abort_p = 51;
      return;
    }
    ItemSlot& sl = ring[r];
    if (valid) {
#pragma unroll 1
      for (int row = lane; row < TILE_M; row += 32) {
#pragma unroll
        for (int sx = 0; sx < 2; ++sx) {
          int token, lo, hi;
          pair_q_row(p.f.prob, di.pt, sx, row, &token, &lo, &hi);
          sl.token[sx][row] = token;
          sl.lo[sx][row] = lo;
          sl.hi[sx][row] = hi;
        }
      }
    }
    if (lane == 0) {
      sl.valid = valid;
      if (valid) {
        const int n_kv = di.pt.kv.n_kv_tiles;
        sl.n_kv = n_kv;
        sl.b = di.b; sl.h0 = di.h0; sl.h1 = di.h1; sl.hk = di.hk;
        sl.pt = di.pt;
        if (plan_boxes) plan_slot_boxes(p, di, sl);
      }
    }
    __syncwarp();
    if (lane == 0) ptx::mbar_arrive(&slot_ready[r]);
    if (!valid) return;
  }
}
__device__ __forceinline__ void tma_fetch_box(const int c[5], int rank4, const CUtensorMap* m, uint32_t dst, uint64_t* bar) {
  if (rank4) {
    ptx::tma_load_4d(dst, m, bar, 0, c[1], c[2], c[3]);
    ptx::tma_load_4d(dst + HALF_BYTES, m, bar, 64, c[1], c[2], c[3]);
  } else {
    ptx::tma_load_5d(dst, m, bar, 0, c[1], c[2], c[3], c[4]);
    ptx::tma_load_5d(dst + HALF_BYTES, m, bar, 64, c[1], c[2], c[3], c[4]);
  }
}

// Shared-memory layout and barriers the loaders of the split-K/V mode need.
struct SplitLoaderCtx {
  uint32_t q_smem0, k_smem0, v_smem0;
  uint64_t *q_full, *q1_full, *k_full, *v_full, *s0_full, *s1_full;
  const ItemSlot* ring;
  uint64_t *slot_ready, *slot_free;
  volatile int* abort_p;
};

// Loader of the split-K/V mode (Gather-0): sub-tile s has its own key list and its own single K and V
// buffer, refilled as soon as the MMA that read it has completed. Event driven: when QK0 of key tile
// j is done (which, the pipe being in order, also means PV0 of tile j-1 is done) V0(j) and K0(j+1)
// are requested; likewise for sub-tile 1, whose event also frees the Q buffers at an item's end.
// kTma: one thread issues TMA boxes; otherwise all 128 loader threads gather rows with cp.async.
template <bool kTma>
__device__ __forceinline__ void split_loader(const DualParams& p, const SplitLoaderCtx& cx, int lt) {
  const int chunk = lt & 15, rsub = lt >> 4;
  const TmaOperand q_op = {&p.maps.q_main, &p.maps.q_text, &p.maps.q_main};
  const TmaOperand k_op = {&p.maps.k_main, &p.maps.k_text, &p.maps.k_aux};
  const TmaOperand v_op = {&p.maps.v_main, &p.maps.v_text, &p.maps.v_aux};

  auto fetch_q = [&](const ItemSlot& sl) {
    if (kTma) {
      ptx::mbar_arrive_expect_tx(cx.q_full, TILE_BYTES);
      ptx::mbar_arrive_expect_tx(cx.q1_full, TILE_BYTES);
      tma_fetch_q(p.f.prob, pair_kv_map(sl.pt, 1, 0), sl.h0, sl.b, q_op, cx.q_smem0, cx.q_full);
      tma_fetch_q(p.f.prob, pair_kv_map(sl.pt, 1, 1), sl.h1, sl.b, q_op, cx.q_smem0 + TILE_BYTES, cx.q1_full);
    } else {
#pragma unroll 1
      for (int sx = 0; sx < 2; ++sx) {
        const __nv_bfloat16* qb = p.f.q + sl.b * p.f.qs.sb + (sx ? sl.h1 : sl.h0) * p.f.qs.sh + chunk * 8;
#pragma unroll 4
        for (int ps = 0; ps < TILE_M / 8; ++ps) {
          const int row = ps * 8 + rsub;
          const int token = sl.token[sx][row];
          const void* src = token >= 0 ? static_cast<const void*>(qb + int64_t(token) * p.f.qs.ss) : static_cast<const void*>(p.f.q);
          ptx::cp_async_16(cx.q_smem0 + sx * TILE_BYTES + tile_offset(row, chunk), src, token >= 0 ? 16u : 0u);
        }
      }
      ptx::cp_async_mbar_arrive_noinc(cx.q_full);
      ptx::cp_async_mbar_arrive_noinc(cx.q1_full);
    }
  };
  auto fetch_kv = [&](bool is_v, int sx, const ItemSlot& sl, int n) {
    const Tile& map = pair_kv_map(sl.pt, 1, sx);
    const uint32_t dst = (is_v ? cx.v_smem0 : cx.k_smem0) + sx * TILE_BYTES;
    uint64_t* bar = is_v ? &cx.v_full[sx] : &cx.k_full[sx];
    if (kTma) {
      ptx::mbar_arrive_expect_tx(bar, TILE_BYTES);
      tma_fetch_kv(p.f.prob, map, n, sl.hk, sl.b, is_v ? v_op : k_op, dst, bar);
    } else {
      const __nv_bfloat16* base = is_v ? p.f.v + sl.b * p.f.vs.sb + sl.hk * p.f.vs.sh + chunk * 8
                                       : p.f.k + sl.b * p.f.ks.sb + sl.hk * p.f.ks.sh + chunk * 8;
      const int64_t ss = is_v ? p.f.vs.ss : p.f.ks.ss;
#pragma unroll 4
      for (int ps = 0; ps < TILE_N / 8; ++ps) {
        const int row = ps * 8 + rsub;
        const int token = key_token(p.f.prob, map, n * TILE_N + row);
        const void* src = token >= 0 ? static_cast<const void*>(base + int64_t(token) * ss) : static_cast<const void*>(p.f.k);
        ptx::cp_async_16(dst + tile_offset(row, chunk), src, token >= 0 ? 16u : 0u);
      }
      ptx::cp_async_mbar_arrive_noinc(bar);
    }
  };
  // one arrival per consumer warp; the TMA loader is a single thread
  auto release = [&](int seq) {
    if (kTma) { ptx::mbar_arrive(&cx.slot_free[seq % ITEM_RING]); return; }
    __syncwarp();
    if ((lt & 31) == 0) ptx::mbar_arrive(&cx.slot_free[seq % ITEM_RING]);
  };
  auto acquire = [&](int seq) -> const ItemSlot* {
    if (!ptx::mbar_wait(&cx.slot_ready[seq % ITEM_RING], (seq / ITEM_RING) & 1, cx.abort_p)) {
      if (*cx.abort_p == 1) *cx.abort_p = 57;
      return nullptr;
    }
    const ItemSlot* sl = &cx.ring[seq % ITEM_RING];
    return sl->valid ? sl : nullptr;
  };

  int seq = 0, n = 0;                                      // the key tile being fed: tile n of item seq
  const ItemSlot* cur = acquire(0);
  if (cur == nullptr) { if (!kTma) { ptx::cp_async_commit(); ptx::cp_async_wait<0>(); } return; }
  fetch_q(*cur);
  fetch_kv(false, 0, *cur, 0);
  fetch_kv(false, 1, *cur, 0);
  for (uint32_t j = 0;; ++j) {                            // j: key tiles of this CTA so far
    const bool last_of_item = n + 1 >= cur->n_kv;
    const ItemSlot* nxt = last_of_item ? acquire(seq + 1) : cur;     // nullptr: the list ends (or a wait gave up)
    const int nn = last_of_item ? 0 : n + 1;
    if (!ptx::mbar_wait(cx.s0_full, j & 1, cx.abort_p)) { if (*cx.abort_p == 1) *cx.abort_p = 24; break; }
    fetch_kv(true, 0, *cur, n);
    if (nxt != nullptr) fetch_kv(false, 0, *nxt, nn);
    if (!ptx::mbar_wait(&cx.s1_full[j & 1], (j >> 1) & 1, cx.abort_p)) { if (*cx.abort_p == 1) *cx.abort_p = 25; break; }
    fetch_kv(true, 1, *cur, n);
    if (nxt == nullptr) break;
    if (last_of_item) fetch_q(*nxt);
    fetch_kv(false, 1, *nxt, nn);
    if (last_of_item) { release(seq); ++seq; }
    cur = nxt;
    n = nn;
  }
  if (!kTma) { ptx::cp_async_commit(); ptx::cp_async_wait<0>(); }
}

template <int NSPLIT, bool kSplitKV, bool kTma>
__global__ void __launch_bounds__(DualCfg<NSPLIT>::THREADS, 1) intra_fwd_dual_kernel(const __grid_constant__ DualParams p) {
  using Cfg = DualCfg<NSPLIT>;
  constexpr int COLS = Cfg::COLS, SM_WARPS = Cfg::SM_WARPS, SM_THREADS = Cfg::SM_THREADS;
  constexpr int SM_REGS = Cfg::SM_REGS, EP_REGS = Cfg::EP_REGS, MMA_REGS = Cfg::MMA_REGS;
  extern __shared__ uint8_t smem_raw[];
  // barriers: 0 q_full, 1-2 k_full, 3-4 v_full, 5 s0_full, 6-7 s1_full[stage], 8-9 p_full[s],
  //           10-11 o_done[s], 12 drain, 13 xbar (softmax threads' exchange rendezvous),
  //           14 l_ready (row sums of an item published), 15-16 o_free[s] (O of an item has been read),
  //           17 q1_full (barrier 0 is Q0's)
  //           18-21 slot_ready[r], 22-25 slot_free[r] (item ring)
  //           row-owner form only: 26-27 s_taken[s] (the set has copied its scores out of the shared buffer),
  //           28 pv0_done (a PV of sub-tile 0 has completed), 29-30 v_done[key tile & 1] (PV1 of that key tile
  //           and everything its warp issued before), 31 l_ready of sub-tile 1, 32 the PV warp's drain
  __shared__ uint64_t bars[18 + 2 * ITEM_RING + 7];
  __shared__ ItemSlot ring[ITEM_RING];
  __shared__ uint32_t tmem_base_smem;
  __shared__ int abort_flag;
  __shared__ float xch_max[2][NSPLIT][TILE_M];      // [phase parity][column part][row]: partial row maxima
  __shared__ float xch_sum[2][2][NSPLIT][TILE_M];   // [item parity][sub-tile][column part][row]: partial row sums
  __shared__ float xch_m[2][2][TILE_M];             // [item parity][sub-tile][row]: the running maximum they refer to

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;

  uint64_t* q_full = &bars[0];       // Q of sub-tile 0 has landed
  uint64_t* q1_full = &bars[17];     // Q of sub-tile 1 has landed
  uint64_t* k_full = &bars[1];
  uint64_t* v_full = &bars[3];
  uint64_t* s0_full = &bars[5];     // QK0 of a key tile has completed
  uint64_t* s1_full = &bars[6];     // [key tile & 1]: QK1 of that key tile (and everything issued before it)
  uint64_t* p_full = &bars[8];
  uint64_t* o_done = &bars[10];     // last PV of an item, per sub-tile
  uint64_t* drain = &bars[12];
  uint64_t* xbar = &bars[13];
  uint64_t* l_ready = &bars[14];
  uint64_t* o_free = &bars[15];
  uint64_t* slot_ready = &bars[18];
  uint64_t* slot_free = &bars[18 + ITEM_RING];
  uint64_t* s_taken = &bars[18 + 2 * ITEM_RING];
  uint64_t* pv0_done = &bars[18 + 2 * ITEM_RING + 2];
  uint64_t* v_done = &bars[18 + 2 * ITEM_RING + 3];
  uint64_t* l_ready1 = &bars[18 + 2 * ITEM_RING + 5];
  uint64_t* drain2 = &bars[18 + 2 * ITEM_RING + 6];

  const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t q_smem0 = smem_base;                                 // Q sub-tile s at + s * TILE_BYTES
  const uint32_t k_smem0 = smem_base + 2 * TILE_BYTES;                // K stage j at + j * TILE_BYTES
  const uint32_t v_smem0 = smem_base + (2 + KV_STAGES) * TILE_BYTES;

  if (tid == 0) {
    abort_flag = 0;
    const uint32_t producers = kTma ? 1 : 128;       // one TMA-issuing thread, or every loader thread
    ptx::mbar_init(q_full, producers);
    ptx::mbar_init(q1_full, producers);
    for (int j = 0; j < KV_STAGES; ++j) {
      ptx::mbar_init(&k_full[j], producers);
      ptx::mbar_init(&v_full[j], producers);
    }
    ptx::mbar_init(s0_full, 1);
    for (int s = 0; s < 2; ++s) {
      ptx::mbar_init(&s1_full[s], 1);
      ptx::mbar_init(&p_full[s], NSPLIT == 1 ? 4 : SM_WARPS);   // one arrival per softmax warp (of the sub-tile's set)
      ptx::mbar_init(&s_taken[s], 4);
      ptx::mbar_init(&v_done[s], 1);
      ptx::mbar_init(&o_done[s], 1);
    }
    ptx::mbar_init(drain, 1);
    ptx::mbar_init(xbar, SM_WARPS);                       // one arrival per softmax warp
    ptx::mbar_init(l_ready, NSPLIT == 1 ? 4 : SM_WARPS);
    ptx::mbar_init(l_ready1, 4);
    ptx::mbar_init(pv0_done, 1);
    ptx::mbar_init(drain2, 1);
    ptx::mbar_init(&o_free[0], (kTma || NSPLIT == 1) ? 128 : SM_THREADS);   // whoever runs the epilogue
    ptx::mbar_init(&o_free[1], (kTma || NSPLIT == 1) ? 128 : SM_THREADS);
    // ring consumers, one arrival per warp: softmax warps, the MMA warp, and either the four epilogue warps
    // plus the TMA thread, or the four cp.async loader warps
    const uint32_t consumers = SM_WARPS + (NSPLIT == 1 ? 2 : 1) + (kTma ? 5 : 4);
    for (int r = 0; r < ITEM_RING; ++r) {
      ptx::mbar_init(&slot_ready[r], 1);
      ptx::mbar_init(&slot_free[r], consumers);
    }
    ptx::fence_mbar_init();
  }
  if (warp == 0) {
    ptx::tmem_alloc(&tmem_base_smem, DUAL_TMEM_COLS);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem = tmem_base_smem;
  volatile int* abort_p = &abort_flag;
  const int n_cta = gridDim.x;
  const int cta = blockIdx.x;

  // Loader-side waits on the MMA warp's progress (see the note on commits at the top of the file).
  // Key tile j (counted over the whole CTA) signals s1_full[j & 1]; its phase there has parity (j / 2) & 1.
#define INTRA_WAIT_TILE_DONE(j, code)                                               \
  do {                                                                              \
    ok = ptx::mbar_wait(&s1_full[(j) & 1], ((j) >> 1) & 1, abort_p);                \
    if (!ok) { if (*abort_p == 1) *abort_p = (code); }                              \
  } while (0)
  // The V stage key tile j is to be loaded into is free: in the split forms PV1 of key tile j-2 was
  // issued before QK1 of key tile j-1, whose signal the loaders use; in the row-owner form the PV warp
  // signals for itself.
#define INTRA_WAIT_V_STAGE(j, code)                                                  \
  do {                                                                              \
    if (NSPLIT == 1) ok = ptx::mbar_wait(&v_done[(j) & 1], (((j) - 2) >> 1) & 1, abort_p);   \
    else ok = ptx::mbar_wait(&s1_full[((j) - 1) & 1], (((j) - 1) >> 1) & 1, abort_p); \
    if (!ok) { if (*abort_p == 1) *abort_p = (code); }                              \
  } while (0)

  // Item `seq` of this CTA's list, from the ring; leaves the loop at the end marker.
#define INTRA_RING_ACQUIRE(sl, code)                                                 \
  const ItemSlot& sl = ring[seq % ITEM_RING];                                        \
  ok = ptx::mbar_wait(&slot_ready[seq % ITEM_RING], (seq / ITEM_RING) & 1, abort_p); \
  if (!ok) { if (*abort_p == 1) *abort_p = (code); break; }                          \
  if (!sl.valid) break
#define INTRA_RING_RELEASE_WARP()                                                    \
  do { __syncwarp(); if (lane == 0) ptx::mbar_arrive(&slot_free[seq % ITEM_RING]); } while (0)

  if (warp < SM_WARPS) {
    // ================================ softmax / correction / epilogue ==========================
    // All softmax warps work on ONE sub-tile at a time, alternating between the two: thread (part, row)
    // owns the COLS score columns `part` of query row `row` of both sub-tiles. NSPLIT warps per
    // scheduler then hide each other's latencies while the tensor core works on the other sub-tile.
    // The parts of a row agree on the row maximum through shared memory and a bounded mbarrier.
    ptx::setmaxnreg_inc<SM_REGS>();
    if constexpr (NSPLIT == 1) {
      // ---- row-owner form: warps 0-3 own sub-tile 0, warps 4-7 sub-tile 1; thread = query row. Each set
      //      runs its own loop, paced only by its own barriers. TMEM: shared score buffer cols 0-127,
      //      P0 cols 128-191, P1 cols 192-255, O0 / O1 as in the split forms. -----------------------------
      const int sx = warp >> 2;
      const int row = tid & 127;
      const uint32_t lane_addr = tmem + (uint32_t((warp & 3) * 32) << 16);
      const uint32_t p_addr = lane_addr + 128 + sx * 64;
      const uint32_t o_addr = lane_addr + 256 + sx * 128;
      const float scale_log2 = p.f.scale_log2;
      uint32_t kt = 0;                                    // key tiles processed so far by this CTA
      uint32_t n_done = 0;                                // items finished
      bool ok = true;
      for (int seq = 0; ok; ++seq) {
        INTRA_RING_ACQUIRE(sl, 52);
        const int n_kv = sl.n_kv;
        const int lo = sl.lo[sx][row], hi = sl.hi[sx][row];
        const int tk = sl.token[sx][row];
        const int item_b = sl.b, item_h = sx ? sl.h1 : sl.h0;
        INTRA_RING_RELEASE_WARP();
        float m_run = -CUDART_INF_F, l_run = 0.f;
        for (int n = 0; n < n_kv && ok; ++n, ++kt) {
          // QK^T of this sub-tile: sub-tile 0's has a barrier of its own, sub-tile 1's is the key tile's last
          ok = sx ? ptx::mbar_wait(&s1_full[kt & 1], (kt >> 1) & 1, abort_p) : ptx::mbar_wait(s0_full, kt & 1, abort_p);
          if (!ok) { if (*abort_p == 1) *abort_p = 11 + sx; break; }
          ptx::tc_fence_after();
          float s[TILE_N];
          uint32_t* const su = reinterpret_cast<uint32_t*>(s);
          const int u0 = n * TILE_N;
          float tile_max;
          if (!__any_sync(0xffffffffu, lo > u0 || hi < u0 + TILE_N - 1)) {
            // the row maximum of one 32-column chunk is worked out while the next chunk is on its way
            ptx::tmem_ld32(lane_addr, su);
            ptx::tmem_wait_ld();
            ptx::tmem_ld32(lane_addr + 32, su + 32);
            tile_max = sm::row_max(*reinterpret_cast<const float(*)[32]>(&s[0]));
            ptx::tmem_wait_ld();
            ptx::tmem_ld32(lane_addr + 64, su + 64);
            tile_max = fmaxf(tile_max, sm::row_max(*reinterpret_cast<const float(*)[32]>(&s[32])));
            ptx::tmem_wait_ld();
            ptx::tmem_ld32(lane_addr + 96, su + 96);
            tile_max = fmaxf(tile_max, sm::row_max(*reinterpret_cast<const float(*)[32]>(&s[64])));
            ptx::tmem_wait_ld();
            ptx::tc_fence_before();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(&s_taken[sx]);   // the other sub-tile's QK^T may overwrite the buffer
            tile_max = fmaxf(tile_max, sm::row_max(*reinterpret_cast<const float(*)[32]>(&s[96])));
          } else {
#pragma unroll
            for (int c = 0; c < TILE_N / 32; ++c) ptx::tmem_ld32(lane_addr + c * 32, su + c * 32);
            ptx::tmem_wait_ld();
            ptx::tc_fence_before();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(&s_taken[sx]);
            // Diagonal and window-edge tiles: rows whose key interval does not cover the whole tile mask the
            // scores outside it, one unsigned compare and a select per score (with || on two signed compares
            // it compiles to a divergent branch per score, thousands of clocks a tile). Kept apart from the
            // common path above, which predicated selects would slow down.
            const int first = lo - u0;
            const unsigned span = unsigned(hi - lo);
#pragma unroll
            for (int c = 0; c < TILE_N; ++c) s[c] = unsigned(c - first) > span ? -CUDART_INF_F : s[c];
            tile_max = sm::row_max(s);
          }
          const float m_new = fmaxf(m_run, tile_max);
          // The running maximum moves only when the scores outgrow it by 2^8 (see the split forms below).
          const bool grow = (m_new - m_run) * scale_log2 > RESCALE_THRESHOLD;
          float alpha = 1.f;
          if (grow) {
            alpha = ptx::ex2((m_run - m_new) * scale_log2);
            l_run *= alpha;
            m_run = m_new;
          }
          // The PV of this sub-tile's previous key tile (of this item or the one before) reads the P buffer
          // and writes O: both may be touched only once it has completed.
          if (kt > 0) {
            ok = sx ? ptx::mbar_wait(&v_done[(kt - 1) & 1], ((kt - 1) >> 1) & 1, abort_p)
                    : ptx::mbar_wait(pv0_done, (kt - 1) & 1, abort_p);
            if (!ok) { if (*abort_p == 1) *abort_p = 13 + sx; break; }
            ptx::tc_fence_after();
          }
          if (n > 0 && __any_sync(0xffffffffu, grow)) {   // rare once the maximum has settled
#pragma unroll 1
            for (int c = 0; c < HEAD_DIM / 16; ++c) {
              uint32_t o[16];
              ptx::tmem_ld16(o_addr + c * 16, o);
              ptx::tmem_wait_ld();
#pragma unroll
              for (int i = 0; i < 16; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
              ptx::tmem_st16(o_addr + c * 16, o);
            }
          }
          const float base = (m_run == -CUDART_INF_F) ? 0.f : m_run * scale_log2;
          sm::f2 sum[4] = {0ull, 0ull, 0ull, 0ull};
#pragma unroll
          for (int c2 = 0; c2 < TILE_N / 32; ++c2) {
            uint32_t pk[16];
            sm::exp_chunk<sm::EX2_FMA_PAIRS_NONE>(s, c2 * 32, scale_log2, base, pk, sum);
            ptx::tmem_st16(p_addr + c2 * 16, pk);
          }
          l_run += sm::sum4(sum);
          ptx::tmem_wait_st();
          ptx::tc_fence_before();
          __syncwarp();
          if (lane == 0) ptx::mbar_arrive(&p_full[sx]);
        }
        if (!ok) break;
        const int ipar = n_done & 1;
        if (kTma) {                                       // the epilogue warps take it from here
          // ... once they are done with this sub-tile of the item before: a set is not held back by the
          // other set or by the PVs of an item of one key tile, so without this wait it could report two
          // items before the epilogue warps have looked at the barrier once (and overwrite the sums of the
          // item before the last, which they may still be reading).
          if (n_done > 0) {
            ok = ptx::mbar_wait(&o_free[sx], (n_done - 1) & 1, abort_p);
            if (!ok) { if (*abort_p == 1) *abort_p = 19; break; }
          }
          xch_sum[ipar][sx][0][row] = l_run;
          if (p.f.lse != nullptr) xch_m[ipar][sx][row] = m_run;
          __syncwarp();
          if (lane == 0) ptx::mbar_arrive(sx ? l_ready1 : l_ready);
          ++n_done;
          continue;
        }
        ok = ptx::mbar_wait(&o_done[sx], n_done & 1, abort_p);       // last PV of this item
        if (!ok) { if (*abort_p == 1) *abort_p = 15 + sx; break; }
        ptx::tc_fence_after();
        const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
        if (p.f.lse != nullptr && tk >= 0)
          p.f.lse[(int64_t(item_b) * p.f.H + item_h) * p.f.prob.S + tk] = row_lse(m_run, l_run, p.f.scale_log2);
        __nv_bfloat16* dst = p.f.o + item_b * p.f.os.sb + int64_t(tk < 0 ? 0 : tk) * p.f.os.ss + item_h * p.f.os.sh;
        store_o_row(o_addr, HEAD_DIM, inv, dst, tk >= 0, p.wide_stores != 0);
        ptx::tc_fence_before();
        ptx::mbar_arrive(&o_free[sx]);
        ++n_done;
      }
    } else {
    const int half = warp >> 2;                           // which COLS columns of every score tile
    const int row = tid & 127;                            // TMEM lane == query row
    const uint32_t lane_addr = tmem + (uint32_t((warp & 3) * 32) << 16);
    const float scale_log2 = p.f.scale_log2;
    uint32_t it = 0;                                      // key tiles processed so far by this CTA
    uint32_t ph = 0;                                      // exchange phases so far (double-buffer index)
    uint32_t n_done = 0;                                  // items finished
    bool ok = true;

    for (int seq = 0; ok; ++seq) {
      INTRA_RING_ACQUIRE(sl, 52);
      const int n_kv = sl.n_kv;
      const int lo[2] = {sl.lo[0][row], sl.lo[1][row]}, hi[2] = {sl.hi[0][row], sl.hi[1][row]};
      const int token[2] = {sl.token[0][row], sl.token[1][row]};
      const int item_b = sl.b, item_h[2] = {sl.h0, sl.h1};
      INTRA_RING_RELEASE_WARP();
      float m_run[2] = {-CUDART_INF_F, -CUDART_INF_F};    // running maxima (identical in both halves)
      float l_part[2] = {0.f, 0.f};                       // this half's share of the row sums

      for (int n = 0; n < n_kv && ok; ++n, ++it) {
#pragma unroll
        for (int sx = 0; sx < 2; ++sx) {
          if (sx == 0) ok = ptx::mbar_wait(s0_full, it & 1, abort_p);
          else ok = ptx::mbar_wait(&s1_full[it & 1], (it >> 1) & 1, abort_p);
          if (!ok) { if (*abort_p == 1) *abort_p = 11 + sx; break; }
          ptx::tc_fence_after();
          const uint32_t s_addr = lane_addr + sx * 128;
          const uint32_t o_addr = lane_addr + 256 + sx * 128 + half * COLS;

          float s[COLS];
#pragma unroll
          for (int c = 0; c < COLS / 32; ++c)
            ptx::tmem_ld32(s_addr + half * COLS + c * 32, reinterpret_cast<uint32_t*>(s) + c * 32);
          ptx::tmem_wait_ld();

          const int u0 = n * TILE_N + half * COLS;
          // Rows whose key interval does not cover these columns (diagonal and window-edge tiles) mask
          // the scores outside it. Short items (the 4-way instantiation) meet such tiles often: there the
          // test is one unsigned compare and a select per score - with || on two signed compares it
          // compiles to a divergent branch per score, 1300 clocks a phase - behind a warp-wide vote, which
          // keeps the selects out of the other tiles' instruction stream. Long items keep the plain form,
          // which the compiler schedules better around their rarely taken branch.
          if constexpr (NSPLIT == 4) {
            if (__any_sync(0xffffffffu, lo[sx] > u0 || hi[sx] < u0 + COLS - 1)) {
              const int first = lo[sx] - u0;
              const unsigned span = unsigned(hi[sx] - lo[sx]);
#pragma unroll
              for (int c = 0; c < COLS; ++c) s[c] = unsigned(c - first) > span ? -CUDART_INF_F : s[c];
            }
          } else {
            if (lo[sx] > u0 || hi[sx] < u0 + COLS - 1) {
#pragma unroll
              for (int c = 0; c < COLS; ++c) {
                const int u = u0 + c;
                if (u < lo[sx] || u > hi[sx]) s[c] = -CUDART_INF_F;
              }
            }
          }
          const float my_max = sm::row_max(s);
          xch_max[ph & 1][half][row] = my_max;
          __syncwarp();                                   // rendezvous of all 8 softmax warps (bounded, unlike
          if (lane == 0) ptx::mbar_arrive(xbar);          // bar.sync): one arrival per warp
          ok = ptx::mbar_wait(xbar, ph & 1, abort_p);     // also: everyone has finished reading S
          if (!ok) { if (*abort_p == 1) *abort_p = 17; break; }
          float tile_max = my_max;
#pragma unroll
          for (int o = 1; o < NSPLIT; ++o) tile_max = fmaxf(tile_max, xch_max[ph & 1][(half + o) % NSPLIT][row]);
          ++ph;
          const float m_new = fmaxf(m_run[sx], tile_max);
          // Move the running maximum only when the scores outgrow it by 2^8; until then p is merely
          // scaled by a constant that the final division by the row sum removes.
          const bool grow = (m_new - m_run[sx]) * scale_log2 > RESCALE_THRESHOLD;
          float alpha = 1.f;
          if (grow) {
            alpha = ptx::ex2((m_run[sx] - m_new) * scale_log2);    // 0 when the maximum is still -inf
            l_part[sx] *= alpha;
            m_run[sx] = m_new;
          }
          if (n > 0 && __any_sync(0xffffffffu, grow)) {   // rare once the maximum has settled
            // The previous key tile's PV was issued before the QK^T whose completion was just waited
            // for, and the tensor pipe completes in order: O is quiescent here.
#pragma unroll 1
            for (int c = 0; c < COLS / 16; ++c) {
              uint32_t o[16];
              ptx::tmem_ld16(o_addr + c * 16, o);
              ptx::tmem_wait_ld();
#pragma unroll
              for (int i = 0; i < 16; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
              ptx::tmem_st16(o_addr + c * 16, o);
            }
          }
          const float base = (m_run[sx] == -CUDART_INF_F) ? 0.f : m_run[sx] * scale_log2;
          sm::f2 sum[4] = {0ull, 0ull, 0ull, 0ull};
#pragma unroll
          for (int c2 = 0; c2 < COLS / 32; ++c2) {        // 32 scores -> 16 packed columns of P
            uint32_t pk[16];
            sm::exp_chunk<sm::EX2_FMA_PAIRS_2_OF_8>(s, c2 * 32, scale_log2, base, pk, sum);
            ptx::tmem_st16(s_addr + half * (COLS / 2) + c2 * 16, pk);
          }
          l_part[sx] += sm::sum4(sum);
          ptx::tmem_wait_st();
          ptx::tc_fence_before();
          __syncwarp();
          if (lane == 0) ptx::mbar_arrive(&p_full[sx]);
        }
      }
      if (!ok) break;

      // ---- row sums: publish this half's share; whoever stores O adds the two halves ----------
      const int ipar = n_done & 1;
      if (kTma && n_done > 0) {
        // The epilogue warps must have taken the report of the item before (they have once they hand its
        // first accumulator back) before the barrier may complete again. The order of the MMAs makes
        // this wait return at once in practice; it turns that timing into a guarantee.
        ok = ptx::mbar_wait(&o_free[0], (n_done - 1) & 1, abort_p);
        if (!ok) { if (*abort_p == 1) *abort_p = 19; break; }
      }
      xch_sum[ipar][0][half][row] = l_part[0];
      xch_sum[ipar][1][half][row] = l_part[1];
      if (half == 0 && p.f.lse != nullptr) {              // every part of a row holds the same maximum
        xch_m[ipar][0][row] = m_run[0];
        xch_m[ipar][1][row] = m_run[1];
      }
      if (kTma) {
        // the epilogue warps take it from here; go straight on to the next item
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(l_ready);
        ++n_done;
        continue;
      }
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(xbar);
      ok = ptx::mbar_wait(xbar, ph & 1, abort_p);
      if (!ok) { if (*abort_p == 1) *abort_p = 18; break; }
      ++ph;
#pragma unroll
      for (int sx = 0; sx < 2; ++sx) {
        ok = ptx::mbar_wait(&o_done[sx], n_done & 1, abort_p);     // last PV of this item
        if (!ok) { if (*abort_p == 1) *abort_p = 15 + sx; break; }
        ptx::tc_fence_after();
        float l_tot = l_part[sx];
#pragma unroll
        for (int o = 1; o < NSPLIT; ++o) l_tot += xch_sum[ipar][sx][(half + o) % NSPLIT][row];
        const float inv = l_tot > 0.f ? 1.f / l_tot : 0.f;
        const int h = item_h[sx];
        const int tk = token[sx];
        if (half == 0 && p.f.lse != nullptr && tk >= 0)
          p.f.lse[(int64_t(item_b) * p.f.H + h) * p.f.prob.S + tk] = row_lse(m_run[sx], l_tot, p.f.scale_log2);
        __nv_bfloat16* dst = p.f.o + item_b * p.f.os.sb + int64_t(tk < 0 ? 0 : tk) * p.f.os.ss + h * p.f.os.sh + half * COLS;
        store_o_row(lane_addr + 256 + sx * 128 + half * COLS, COLS, inv, dst, tk >= 0, p.wide_stores != 0);
        ptx::tc_fence_before();
        ptx::mbar_arrive(&o_free[sx]);
      }
      if (!ok) break;
      ++n_done;
    }
    }  // NSPLIT > 1
  } else if (warp < SM_WARPS + 4) {
    // ================================ epilogue warps / loaders =====================================
    ptx::setmaxnreg_dec<EP_REGS>();
    const int lt = tid - SM_THREADS;
    uint32_t kc = 0;                                      // K / V tiles loaded so far (ring position)
    bool ok = true;
    int n_done = 0;

    if (kTma) {
      // ---- epilogue warps: O of a finished item -> global, while the softmax warps are already on
      //      the next item. Thread = query row (all 128 columns). ------------------------------------
      const int row = tid & 127;
      const uint32_t lane_addr = tmem + (uint32_t((warp & 3) * 32) << 16);
      for (int seq = 0; ok; ++seq) {
        INTRA_RING_ACQUIRE(sl, 53);
        const int token[2] = {sl.token[0][row], sl.token[1][row]};
        const int item_b = sl.b, item_h[2] = {sl.h0, sl.h1};
        INTRA_RING_RELEASE_WARP();
        const int ipar = n_done & 1;
        if (NSPLIT > 1) {
          ok = ptx::mbar_wait(l_ready, ipar, abort_p);
          if (!ok) { if (*abort_p == 1) *abort_p = 41; break; }
        }
#pragma unroll
        for (int sx = 0; sx < 2; ++sx) {
          if (NSPLIT == 1) {                                       // each sub-tile's warp set reports for itself
            ok = ptx::mbar_wait(sx ? l_ready1 : l_ready, ipar, abort_p);
            if (!ok) { if (*abort_p == 1) *abort_p = 41; break; }
          }
          ok = ptx::mbar_wait(&o_done[sx], ipar, abort_p);         // last PV of this item
          if (!ok) { if (*abort_p == 1) *abort_p = 42 + sx; break; }
          ptx::tc_fence_after();
          float l_tot = 0.f;
#pragma unroll
          for (int o = 0; o < NSPLIT; ++o) l_tot += xch_sum[ipar][sx][o][row];
          const float inv = l_tot > 0.f ? 1.f / l_tot : 0.f;
          const int h = item_h[sx];
          const int tk = token[sx];
          if (p.f.lse != nullptr && tk >= 0)
            p.f.lse[(int64_t(item_b) * p.f.H + h) * p.f.prob.S + tk] = row_lse(xch_m[ipar][sx][row], l_tot, p.f.scale_log2);
          __nv_bfloat16* dst = p.f.o + item_b * p.f.os.sb + int64_t(tk < 0 ? 0 : tk) * p.f.os.ss + h * p.f.os.sh;
          store_o_row(lane_addr + 256 + sx * 128, 128, inv, dst, tk >= 0, p.wide_stores != 0);
          ptx::tc_fence_before();
          ptx::mbar_arrive(&o_free[sx]);                           // the next item's first PV may overwrite O
        }
        ++n_done;
      }
    } else if (kSplitKV) {
      const SplitLoaderCtx cx = {q_smem0, k_smem0, v_smem0, q_full, q1_full, k_full, v_full, s0_full, s1_full,
                                 ring, slot_ready, slot_free, abort_p};
      split_loader<false>(p, cx, lt);
    } else {
      // ---- cp.async row gathers by all 128 loader threads (ragged shapes) ------------------------
      const int chunk = lt & 15;                          // 16-byte chunk of the 256-byte row
      const int rsub = lt >> 4;                           // row within a pass of 8 rows
      for (int seq = 0; ok; ++seq) {
        INTRA_RING_ACQUIRE(sl, 54);
        const int n_kv = sl.n_kv;
        if (n_done > 0) {
          INTRA_WAIT_TILE_DONE(kc - 1, 21);
          if (!ok) break;
        }
        {
          const __nv_bfloat16* qb0 = p.f.q + sl.b * p.f.qs.sb + sl.h0 * p.f.qs.sh + chunk * 8;
          const __nv_bfloat16* qb1 = p.f.q + sl.b * p.f.qs.sb + sl.h1 * p.f.qs.sh + chunk * 8;
#pragma unroll 4
          for (int ps = 0; ps < TILE_M / 8; ++ps) {
            const int row = ps * 8 + rsub;
            int token = sl.token[0][row];
            const void* src = token >= 0 ? static_cast<const void*>(qb0 + int64_t(token) * p.f.qs.ss) : static_cast<const void*>(p.f.q);
            ptx::cp_async_16(q_smem0 + tile_offset(row, chunk), src, token >= 0 ? 16u : 0u);
            token = sl.token[1][row];
            src = token >= 0 ? static_cast<const void*>(qb1 + int64_t(token) * p.f.qs.ss) : static_cast<const void*>(p.f.q);
            ptx::cp_async_16(q_smem0 + TILE_BYTES + tile_offset(row, chunk), src, token >= 0 ? 16u : 0u);
          }
          ptx::cp_async_mbar_arrive_noinc(q_full);
          ptx::cp_async_mbar_arrive_noinc(q1_full);
        }
        const __nv_bfloat16* kb = p.f.k + sl.b * p.f.ks.sb + sl.hk * p.f.ks.sh + chunk * 8;
        const __nv_bfloat16* vb = p.f.v + sl.b * p.f.vs.sb + sl.hk * p.f.vs.sh + chunk * 8;
        const Tile kv = sl.pt.kv;
        INTRA_RING_RELEASE_WARP();
        for (int n = 0; n < n_kv && ok; ++n, ++kc) {
          const int stage = kc % KV_STAGES;
          int tokens[TILE_N / 8];
#pragma unroll
          for (int ps = 0; ps < TILE_N / 8; ++ps) tokens[ps] = key_token(p.f.prob, kv, n * TILE_N + ps * 8 + rsub);
          if (kc >= 2) {
            INTRA_WAIT_TILE_DONE(kc - 2, 22);
            if (!ok) break;
          }
          const uint32_t kdst = k_smem0 + stage * TILE_BYTES;
#pragma unroll
          for (int ps = 0; ps < TILE_N / 8; ++ps) {
            const int row = ps * 8 + rsub;
            const int token = tokens[ps];
            const void* src = token >= 0 ? static_cast<const void*>(kb + int64_t(token) * p.f.ks.ss) : static_cast<const void*>(p.f.k);
            ptx::cp_async_16(kdst + tile_offset(row, chunk), src, token >= 0 ? 16u : 0u);
          }
          ptx::cp_async_mbar_arrive_noinc(&k_full[stage]);
          if (kc >= 2) {
            INTRA_WAIT_V_STAGE(kc, 23);
            if (!ok) break;
          }
          const uint32_t vdst = v_smem0 + stage * TILE_BYTES;
#pragma unroll
          for (int ps = 0; ps < TILE_N / 8; ++ps) {
            const int row = ps * 8 + rsub;
            const int token = tokens[ps];
            const void* src = token >= 0 ? static_cast<const void*>(vb + int64_t(token) * p.f.vs.ss) : static_cast<const void*>(p.f.v);
            ptx::cp_async_16(vdst + tile_offset(row, chunk), src, token >= 0 ? 16u : 0u);
          }
          ptx::cp_async_mbar_arrive_noinc(&v_full[stage]);
        }
        ++n_done;
      }
      ptx::cp_async_commit();
      ptx::cp_async_wait<0>();
    }
  } else {
    // ================================ MMA issue ==================================================
    ptx::setmaxnreg_dec<MMA_REGS>();
    if (kSplitKV && warp == SM_WARPS + 5 && kTma && lane == 0) {
      const SplitLoaderCtx cx = {q_smem0, k_smem0, v_smem0, q_full, q1_full, k_full, v_full, s0_full, s1_full,
                                 ring, slot_ready, slot_free, abort_p};
      split_loader<true>(p, cx, 0);
    } else if (warp == SM_WARPS + 5 && kTma && lane == 0) {
      // ---- one thread drives the TMA unit ------------------------------------------------------------
      uint32_t kc = 0;                                    // K / V tiles requested so far (ring position)
      bool ok = true;
      int n_done = 0;
      ptx::prefetch_tensormap(&p.maps.q_main);
      ptx::prefetch_tensormap(&p.maps.k_main);
      ptx::prefetch_tensormap(&p.maps.v_main);
      const TmaOperand q_op = {&p.maps.q_main, &p.maps.q_text, &p.maps.q_main};
      const TmaOperand k_op = {&p.maps.k_main, &p.maps.k_text, &p.maps.k_aux};
      const TmaOperand v_op = {&p.maps.v_main, &p.maps.v_text, &p.maps.v_aux};
      const CUtensorMap* k_main = p.f.prob.kind == KIND_IMG_GATHER0 ? k_op.aux_map : k_op.main_map;
      const CUtensorMap* v_main = p.f.prob.kind == KIND_IMG_GATHER0 ? v_op.aux_map : v_op.main_map;
      for (int seq = 0; ok; ++seq) {
        INTRA_RING_ACQUIRE(sl, 55);
        const int n_kv = sl.n_kv, n_text = sl.n_text;
        for (int n = 0; n < n_kv && ok; ++n, ++kc) {
          const int stage = kc % KV_STAGES;
          const KvSegment& sg = n < n_text ? sl.seg0 : sl.seg1;
          const CUtensorMap* kmap = sg.text ? k_op.text_map : k_main;
          const CUtensorMap* vmap = sg.text ? v_op.text_map : v_main;
          if (kc >= 2) {                                // K stage: QK1 of key tile kc-2
            INTRA_WAIT_TILE_DONE(kc - 2, 22);
            if (!ok) break;
          }
          ptx::mbar_arrive_expect_tx(&k_full[stage], TILE_BYTES);
          tma_fetch_planned(sg, n, kmap, k_smem0 + stage * TILE_BYTES, &k_full[stage]);
          if (n == 0) {
            // The item's queries go in between its first K and V tiles, each as early as its buffer
            // frees: Q0 after QK0 of the previous item's last key tile, Q1 after that tile's QK1.
            if (n_done > 0) {
              ok = ptx::mbar_wait(s0_full, (kc - 1) & 1, abort_p);
              if (!ok) { if (*abort_p == 1) *abort_p = 21; break; }
            }
            ptx::mbar_arrive_expect_tx(q_full, TILE_BYTES);
            tma_fetch_box(sl.q0, sl.q0_rank4, sl.q0_text ? q_op.text_map : q_op.main_map, q_smem0, q_full);
          }
          if (NSPLIT == 1) {                            // Q1: QK1 of the previous item's last key tile; V stage: PV1 of kc-2
            if (n == 0 && n_done > 0) {
              INTRA_WAIT_TILE_DONE(kc - 1, 23);
              if (!ok) break;
            }
            if (kc >= 2) {
              INTRA_WAIT_V_STAGE(kc, 26);
              if (!ok) break;
            }
          } else if (kc >= 2 || (n == 0 && n_done > 0)) {   // V stage: PV1 of key tile kc-2, issued before QK1 of kc-1
            INTRA_WAIT_TILE_DONE(kc - 1, 23);
            if (!ok) break;
          }
          if (n == 0) {
            ptx::mbar_arrive_expect_tx(q1_full, TILE_BYTES);
            tma_fetch_box(sl.q1, sl.q1_rank4, sl.q1_text ? q_op.text_map : q_op.main_map, q_smem0 + TILE_BYTES, q1_full);
          }
          ptx::mbar_arrive_expect_tx(&v_full[stage], TILE_BYTES);
          tma_fetch_planned(sg, n, vmap, v_smem0 + stage * TILE_BYTES, &v_full[stage]);
        }
        if (!ok) break;
        ptx::mbar_arrive(&slot_free[seq % ITEM_RING]);
        ++n_done;
      }
    } else if (warp == SM_WARPS + 6) {
      // ---- planner: keeps the item ring filled -------------------------------------------------------
      plan_items(p, ring, slot_ready, slot_free, cta, n_cta, lane, kTma && !kSplitKV, abort_p);
    }
    if ((warp == SM_WARPS + 4 || warp == SM_WARPS + 7) && NSPLIT == 1) {
      // ---- row-owner form: two issuing warps, so that neither kind of product waits for the other's
      //      operands. Warp 4N+4 issues QK0(j) QK1(j) over the CTA's key tiles j, each into the shared
      //      score buffer as soon as the other set has copied its scores out; warp 4N+7 issues
      //      PV0(j) PV1(j) as the sets deliver P. Each thread's commits cover its own MMAs only. ---------
      const uint64_t k_desc0 = tile_desc_kmajor(k_smem0), v_desc0 = tile_desc_mnmajor(v_smem0);
      constexpr uint64_t kStageStep = TILE_BYTES >> 4;    // descriptor distance between ring stages
      const bool qk_role = warp == SM_WARPS + 4;
      bool ok = true;
      uint32_t j = 0;                                     // key tiles so far, counted over the CTA
      for (int seq = 0; ok; ++seq) {
        INTRA_RING_ACQUIRE(sl, 56);
        const int n_kv = sl.n_kv;
        INTRA_RING_RELEASE_WARP();
        if (qk_role) {
          const uint64_t q0_desc = tile_desc_kmajor(q_smem0), q1_desc = tile_desc_kmajor(q_smem0 + TILE_BYTES);
          for (int n = 0; n < n_kv; ++n, ++j) {
            const int stage = j % KV_STAGES;
            if (n == 0) {
              ok = ptx::mbar_wait(q_full, seq & 1, abort_p);
              if (!ok) { if (*abort_p == 1) *abort_p = 31; break; }
            }
            ok = ptx::mbar_wait(&k_full[stage], (j / KV_STAGES) & 1, abort_p);
            if (!ok) { if (*abort_p == 1) *abort_p = 32; break; }
            ptx::fence_proxy_async_smem();
            if (j > 0) {                                  // set 1 has copied the previous key tile's scores out
              ok = ptx::mbar_wait(&s_taken[1], (j - 1) & 1, abort_p);
              if (!ok) { if (*abort_p == 1) *abort_p = 33; break; }
            }
            ptx::tc_fence_after();
            if (ptx::elect_one()) {
              issue_qk_desc(q0_desc, k_desc0 + stage * kStageStep, tmem);
              ptx::mma_commit(s0_full);
            }
            __syncwarp();
            if (n == 0) {
              ok = ptx::mbar_wait(q1_full, seq & 1, abort_p);
              if (!ok) { if (*abort_p == 1) *abort_p = 42; break; }
              ptx::fence_proxy_async_smem();
            }
            ok = ptx::mbar_wait(&s_taken[0], j & 1, abort_p);
            if (!ok) { if (*abort_p == 1) *abort_p = 34; break; }
            ptx::tc_fence_after();
            if (ptx::elect_one()) {
              issue_qk_desc(q1_desc, k_desc0 + stage * kStageStep, tmem);
              // set 1's scores; also: the K stage and (an item's last key tile) the Q buffers are free
              ptx::mma_commit(&s1_full[j & 1]);
            }
            __syncwarp();
          }
        } else {
          for (int n = 0; n < n_kv; ++n, ++j) {
            const int stage = j % KV_STAGES;
            ok = ptx::mbar_wait(&p_full[0], j & 1, abort_p);
            if (!ok) { if (*abort_p == 1) *abort_p = 35; break; }
            ok = ptx::mbar_wait(&v_full[stage], (j / KV_STAGES) & 1, abort_p);
            if (!ok) { if (*abort_p == 1) *abort_p = 40; break; }
            ptx::fence_proxy_async_smem();
            if (n == 0 && seq > 0) {                      // O0 of the previous item must have been read
              ok = ptx::mbar_wait(&o_free[0], (seq - 1) & 1, abort_p);
              if (!ok) { if (*abort_p == 1) *abort_p = 37; break; }
            }
            ptx::tc_fence_after();
            if (ptx::elect_one()) {
              issue_pv_desc(tmem + 128, v_desc0 + stage * kStageStep, tmem + 256, n > 0);
              ptx::mma_commit(pv0_done);
              if (n == n_kv - 1) ptx::mma_commit(&o_done[0]);
            }
            __syncwarp();
            ok = ptx::mbar_wait(&p_full[1], j & 1, abort_p);
            if (!ok) { if (*abort_p == 1) *abort_p = 36; break; }
            if (n == 0 && seq > 0) {
              ok = ptx::mbar_wait(&o_free[1], (seq - 1) & 1, abort_p);
              if (!ok) { if (*abort_p == 1) *abort_p = 38; break; }
            }
            ptx::tc_fence_after();
            if (ptx::elect_one()) {
              issue_pv_desc(tmem + 192, v_desc0 + stage * kStageStep, tmem + 384, n > 0);
              if (n == n_kv - 1) ptx::mma_commit(&o_done[1]);
              ptx::mma_commit(&v_done[j & 1]);            // set 1's P buffer and O1, and the V stage, are free
            }
            __syncwarp();
          }
        }
      }
      if (!ok) {                                          // let MMAs in flight finish before TMEM is freed
        uint64_t* const my_drain = qk_role ? drain : drain2;
        if (ptx::elect_one()) ptx::mma_commit(my_drain);
        __syncwarp();
        int dummy = 0;
        ptx::mbar_wait(my_drain, 0, &dummy, 100);
      }
    } else if (warp == SM_WARPS + 4) {
      uint32_t kc = 0;                                    // key tiles issued so far
      uint32_t it0 = 0, it1 = 0;                          // PVs issued per sub-tile (p_full phases)
      const uint64_t q0_desc = tile_desc_kmajor(q_smem0), q1_desc = tile_desc_kmajor(q_smem0 + TILE_BYTES);
      const uint64_t k_desc0 = tile_desc_kmajor(k_smem0), v_desc0 = tile_desc_mnmajor(v_smem0);
      constexpr uint64_t kStageStep = TILE_BYTES >> 4;    // descriptor distance between ring stages
      bool pend = false;                                  // PV1 of the previous key tile not yet issued
      bool pend_last = false;                             // ... and it is the last one of its item
      uint32_t pend_acc = 0, pend_stage = 0;
      int pend_item = 0;                                  // items finished before the pending PV1's item
      int n_done = 0;
      bool ok = true;

      for (int seq = 0; ok; ++seq) {
        INTRA_RING_ACQUIRE(sl, 56);
        const int n_kv = sl.n_kv;
        INTRA_RING_RELEASE_WARP();
        ok = ptx::mbar_wait(q_full, n_done & 1, abort_p);
        if (!ok) { if (*abort_p == 1) *abort_p = 31; break; }
        for (int n = 0; n < n_kv; ++n, ++kc) {
          // shared keys: both sub-tiles read ring stage kc % 2; split keys: sub-tile s reads buffer s
          const int stage = kSplitKV ? 0 : kc % KV_STAGES;
          const uint32_t par = kSplitKV ? (kc & 1) : (kc / KV_STAGES) & 1;
          ok = ptx::mbar_wait(&k_full[stage], par, abort_p);
          if (!ok) { if (*abort_p == 1) *abort_p = 32; break; }
          ptx::fence_proxy_async_smem();
          ptx::tc_fence_after();
          const uint64_t k_desc = k_desc0 + stage * kStageStep;
          if (ptx::elect_one()) {
            issue_qk_desc(q0_desc, k_desc, tmem + 0);
            ptx::mma_commit(s0_full);
          }
          __syncwarp();
          if (pend) {
            ok = ptx::mbar_wait(&p_full[1], it1 & 1, abort_p);
            if (!ok) { if (*abort_p == 1) *abort_p = 33; break; }
            if (pend_acc == 0 && pend_item > 0) {         // first PV1 of an item: O1 of the item before it
              ok = ptx::mbar_wait(&o_free[1], (pend_item - 1) & 1, abort_p);
              if (!ok) { if (*abort_p == 1) *abort_p = 38; break; }
            }
            if (kSplitKV) {                               // sub-tile 1's own V buffer
              ok = ptx::mbar_wait(&v_full[1], (kc - 1) & 1, abort_p);
              if (!ok) { if (*abort_p == 1) *abort_p = 40; break; }
              ptx::fence_proxy_async_smem();
            }
            ptx::tc_fence_after();
            if (ptx::elect_one()) {
              issue_pv_desc(tmem + 128, v_desc0 + pend_stage * kStageStep, tmem + 384, pend_acc != 0);
              if (pend_last) ptx::mma_commit(&o_done[1]);
            }
            __syncwarp();
            ++it1;
            pend = false;
          }
          if (n == 0) {                                   // the item's second query tile
            ok = ptx::mbar_wait(q1_full, n_done & 1, abort_p);
            if (!ok) { if (*abort_p == 1) *abort_p = 42; break; }
            ptx::fence_proxy_async_smem();
            ptx::tc_fence_after();
          }
          if (kSplitKV) {                                 // sub-tile 1's own K buffer
            ok = ptx::mbar_wait(&k_full[1], par, abort_p);
            if (!ok) { if (*abort_p == 1) *abort_p = 41; break; }
            ptx::fence_proxy_async_smem();
            ptx::tc_fence_after();
          }
          if (ptx::elect_one()) {
            issue_qk_desc(q1_desc, kSplitKV ? k_desc0 + kStageStep : k_desc, tmem + 128);
            ptx::mma_commit(&s1_full[kc & 1]);
          }
          __syncwarp();
          ok = ptx::mbar_wait(&v_full[stage], par, abort_p);
          if (!ok) { if (*abort_p == 1) *abort_p = 34; break; }
          ptx::fence_proxy_async_smem();
          ok = ptx::mbar_wait(&p_full[0], it0 & 1, abort_p);
          if (!ok) { if (*abort_p == 1) *abort_p = 35; break; }
          if (n == 0 && n_done > 0) {                     // O0 of the previous item must have been read
            ok = ptx::mbar_wait(&o_free[0], (n_done - 1) & 1, abort_p);
            if (!ok) { if (*abort_p == 1) *abort_p = 37; break; }
          }
          ptx::tc_fence_after();
          if (ptx::elect_one()) {
            issue_pv_desc(tmem + 0, v_desc0 + stage * kStageStep, tmem + 256, n > 0);
            if (n == n_kv - 1) ptx::mma_commit(&o_done[0]);
          }
          __syncwarp();
          ++it0;
          pend = true;
          pend_last = (n == n_kv - 1);
          pend_acc = n > 0 ? 1u : 0u;
          pend_stage = kSplitKV ? 1 : stage;
          pend_item = n_done;
        }
        ++n_done;
      }
      if (ok && pend) {
        ok = ptx::mbar_wait(&p_full[1], it1 & 1, abort_p);
        if (!ok && *abort_p == 1) *abort_p = 36;
        if (ok && pend_acc == 0 && pend_item > 0) {
          ok = ptx::mbar_wait(&o_free[1], (pend_item - 1) & 1, abort_p);
          if (!ok && *abort_p == 1) *abort_p = 39;
        }
        if (ok && kSplitKV) {
          ok = ptx::mbar_wait(&v_full[1], (kc - 1) & 1, abort_p);
          if (!ok && *abort_p == 1) *abort_p = 40;
          ptx::fence_proxy_async_smem();
        }
        if (ok) {
          ptx::tc_fence_after();
          if (ptx::elect_one()) {
            issue_pv_desc(tmem + 128, v_desc0 + pend_stage * kStageStep, tmem + 384, pend_acc != 0);
            ptx::mma_commit(&o_done[1]);
          }
          __syncwarp();
        }
      }
      if (!ok) {                                          // let MMAs in flight finish before TMEM is freed
        if (ptx::elect_one()) ptx::mma_commit(drain);
        __syncwarp();
        int dummy = 0;
        ptx::mbar_wait(drain, 0, &dummy, 100);
      }
    }
  }
#undef INTRA_WAIT_TILE_DONE
#undef INTRA_WAIT_V_STAGE
#undef INTRA_RING_ACQUIRE
#undef INTRA_RING_RELEASE_WARP

  // ---- teardown --------------------------------------------------------------------------------
  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem, DUAL_TMEM_COLS);
  }
  if (tid == 0 && abort_flag != 0) atomicCAS(p.f.status, 0, STATUS_WAIT_BASE + abort_flag);
}

}  // namespace intra
