// Computational-Query-Set index maps of the five INTRA attention patterns, in closed form.
//
// Every pattern is decomposed into independent "tiles": up to TILE_M query rows that share one
// ordered list of key slots. A tile is described by three integer functions
//
//     q_row(r)      -> (token id of query row r or -1, lo, hi)   row r attends key slots lo..hi
//     key_token(u)  -> token id of key slot u (or -1 for a padding slot)
//     n_kv_tiles    -> number of TILE_N-wide key tiles that cover the slots
//
// so that the set of attended (query token, key token) pairs of the whole problem is exactly
//     { (q_row(r).token, key_token(u)) : tile, valid r, lo <= u <= hi }.
// The same header is compiled for the host (visited-set tests, launch geometry) and for the
// device (row gathers, masks), so the sets the kernels visit are the sets the tests enumerate.
//
// Patterns follow the dense-mask specification of the reference (intra_attn/reference.py:14-74);
// the closed forms replace the reference's per-pattern loader structs (csrc/flash_attn/src/
// gmem_tile.h:270-1426) and block bookkeeping (csrc/flash_attn/src/block_info.h:51-108).
#pragma once
#include <stdint.h>

#if defined(__CUDACC__)
#define INTRA_HD __host__ __device__ __forceinline__
#else
#define INTRA_HD inline
#endif

namespace intra {

constexpr int TILE_M = 128;      // query rows per tile
constexpr int TILE_N = 128;      // key slots per key tile
constexpr int TEXT_LEN = 512;    // FLUX text tokens placed before the image grid (interface.py:14)
constexpr int TEXT_CHUNK = 64;   // text tokens riding with one image group
constexpr int IMG_GROUPS = 8;    // 2 x 4 sub-lattice
constexpr int PATCH = 8;         // Gather-0 query patch edge
constexpr int WIN = 16;          // Gather-0 key window edge

enum Kind : int {
  KIND_LLM_SCATTER = 0,   // token i in group i % G, causal inside the group
  KIND_LLM_GATHER1 = 1,   // segments of G tokens, segment s in group s % G, causal inside the group
  KIND_LLM_WINDOW = 2,    // 64-query blocks see themselves plus the preceding W-64 tokens, causal
  KIND_IMG_SCATTER = 3,   // 8 groups on a 2x4 sub-lattice + dense text keys, bidirectional
  KIND_IMG_GATHER0 = 4,   // 8x8 query patches see a 16x16 window + dense text keys
};

INTRA_HD int ceil_div(int a, int b) { return (a + b - 1) / b; }
INTRA_HD int imin(int a, int b) { return a < b ? a : b; }
INTRA_HD int imax(int a, int b) { return a > b ? a : b; }

struct Problem {
  int kind;
  int S;        // tokens per sequence
  int G;        // group count (LLM scatter / gather1); IMG_GROUPS for the image kinds
  int W;        // window length (LLM window) or grid width (image kinds)
  int n_tiles;  // tiles per (batch, head)
  int tiles_m;  // scatter / gather1: tiles per group;  image scatter: tiles per group
  int n_img;    // image kinds: image tokens per group = W*W/8
  int pairs_per_row;  // gather0: patch pairs per patch row
};

// Length of group g's packed token list for the two grouped LLM patterns.
INTRA_HD int llm_group_len(int kind, int S, int G, int g) {
  if (kind == KIND_LLM_SCATTER) return S / G + (g < S % G ? 1 : 0);
  const int span = G * G;                  // one segment of every group
  const int rem = S % span;
  return (S / span) * G + imin(imax(rem - g * G, 0), G);
}

// Token id of packed index t in group g.
INTRA_HD int llm_group_token(int kind, int G, int g, int t) {
  if (kind == KIND_LLM_SCATTER) return t * G + g;
  return (t / G) * G * G + g * G + t % G;
}

// First row / column of the 16-wide Gather-0 window of patch index x (of np patches per edge):
// centred on the patch, shifted inwards at the borders (reference.py:65-68).
INTRA_HD int gather0_start(int x, int np) {
  if (x == 0) return 0;
  if (x == np - 1) return x * PATCH - (WIN - PATCH);
  return x * PATCH - (WIN - PATCH) / 2;
}

// Returns 0 on success; negative if the shape is not supported.
INTRA_HD int make_problem(int kind, int S, int G, int W, Problem* out) {
  Problem p;
  p.kind = kind; p.S = S; p.G = G; p.W = W;
  p.n_tiles = 0; p.tiles_m = 0; p.n_img = 0; p.pairs_per_row = 0;
  if (S <= 0) return -1;
  switch (kind) {
    case KIND_LLM_SCATTER:
    case KIND_LLM_GATHER1: {
      if (G <= 0 || G > S) return -1;
      int nmax = 0;
      for (int g = 0; g < G; ++g) nmax = imax(nmax, llm_group_len(kind, S, G, g));
      p.tiles_m = ceil_div(nmax, TILE_M);
      p.n_tiles = p.tiles_m * G;
      break;
    }
    case KIND_LLM_WINDOW:
      if (W < 64) return -1;      // below one query block some rows would see no key at all
      p.n_tiles = ceil_div(S, TILE_M);
      break;
    case KIND_IMG_SCATTER:
    case KIND_IMG_GATHER0:
      if (W < 16 || W % 8 != 0 || S != TEXT_LEN + W * W) return -1;
      p.G = IMG_GROUPS;
      p.n_img = W * W / IMG_GROUPS;
      p.tiles_m = 1 + ceil_div(p.n_img, TILE_M);
      if (kind == KIND_IMG_SCATTER) {
        p.n_tiles = p.tiles_m * IMG_GROUPS;
      } else {
        p.pairs_per_row = ceil_div(W / PATCH, 2);
        p.n_tiles = IMG_GROUPS + (W / PATCH) * p.pairs_per_row;
      }
      break;
    default:
      return -1;
  }
  *out = p;
  return 0;
}

struct Tile {
  int kind;        // how rows / slots are mapped (a Gather-0 text tile maps like image scatter)
  int g;           // group id (LLM groups; image group / text chunk id)
  int t0;          // packed index of row 0 (grouped kinds), first token (window)
  int nq;          // rows r with t0 + r < nq are valid (see q_row for the image kinds)
  int nk;          // number of key slots (slots >= nk are padding)
  int n_kv_tiles;  // ceil(nk / TILE_N); 0 for an empty tile
  int kbase;       // window: token id of key slot 0
  int is_text;     // image kinds: tile holds a 64-token text chunk
  // gather0 patch-pair tile
  int r0, c0;      // first row / column of the union key window
  int off;         // column offset of the right patch's window inside the union (0: no right patch)
  int prow, pcol;  // patch row, left patch column
};

// Tile `idx` of the problem, idx in [0, n_tiles). Ordered so that tiles with more key tiles come
// first (longest-processing-time-first across the grid).
INTRA_HD Tile make_tile(const Problem& p, int idx) {
  Tile t;
  t.kind = p.kind; t.g = 0; t.t0 = 0; t.nq = 0; t.nk = 0; t.n_kv_tiles = 0; t.kbase = 0;
  t.is_text = 0; t.r0 = 0; t.c0 = 0; t.off = 0; t.prow = 0; t.pcol = 0;
  switch (p.kind) {
    case KIND_LLM_SCATTER:
    case KIND_LLM_GATHER1: {
      const int m = p.tiles_m - 1 - idx / p.G;
      t.g = idx % p.G;
      t.t0 = m * TILE_M;
      t.nq = llm_group_len(p.kind, p.S, p.G, t.g);
      if (t.t0 < t.nq) {
        t.nk = imin(t.t0 + TILE_M, t.nq);     // causal: no key beyond the tile's last query
        t.n_kv_tiles = ceil_div(t.nk, TILE_N);
      }
      break;
    }
    case KIND_LLM_WINDOW: {
      const int m = p.n_tiles - 1 - idx;
      t.t0 = m * TILE_M;
      t.nq = p.S;
      t.kbase = imax(t.t0 - (p.W - 64), 0);
      t.nk = imin(t.t0 + TILE_M, p.S) - t.kbase;
      t.n_kv_tiles = ceil_div(t.nk, TILE_N);
      break;
    }
    case KIND_IMG_SCATTER: {
      const int m = idx / IMG_GROUPS;
      t.g = idx % IMG_GROUPS;
      t.is_text = (m == 0);
      t.t0 = t.is_text ? 0 : (m - 1) * TILE_M;
      t.nq = t.is_text ? TEXT_CHUNK : p.n_img;
      t.nk = TEXT_LEN + p.n_img;
      t.n_kv_tiles = ceil_div(t.nk, TILE_N);
      break;
    }
    case KIND_IMG_GATHER0: {
      if (idx < IMG_GROUPS) {            // text chunk: same rows and keys as image scatter
        t.kind = KIND_IMG_SCATTER;
        t.g = idx; t.is_text = 1; t.t0 = 0; t.nq = TEXT_CHUNK;
        t.nk = TEXT_LEN + p.n_img;
        t.n_kv_tiles = ceil_div(t.nk, TILE_N);
        break;
      }
      const int pp = idx - IMG_GROUPS;
      const int np = p.W / PATCH;
      t.prow = pp / p.pairs_per_row;
      t.pcol = 2 * (pp % p.pairs_per_row);
      t.r0 = gather0_start(t.prow, np);
      t.c0 = gather0_start(t.pcol, np);
      const bool has_right = t.pcol + 1 < np;
      t.off = has_right ? gather0_start(t.pcol + 1, np) - t.c0 : 0;
      t.nq = has_right ? 2 * PATCH * PATCH : PATCH * PATCH;
      t.nk = TEXT_LEN + WIN * WIN + WIN * t.off;
      t.n_kv_tiles = ceil_div(t.nk, TILE_N);
      break;
    }
    default: break;
  }
  return t;
}

// Token id of image-scatter group member u (u-th image token of group g in raster order).
INTRA_HD int img_scatter_token(int W, int g, int u) {
  const int quads = W / 4;                       // group members per grid row
  const int a = g / 4, b = g % 4;                // (row parity, column mod 4)
  return TEXT_LEN + (u / quads) * 2 * W + (u % quads) * 4 + a * W + b;
}

// Query row r of tile t: token id (or -1 if the row is padding) and the inclusive key-slot
// interval [lo, hi] the row attends. Padding rows get the full interval so that their (discarded)
// softmax stays finite.
INTRA_HD void q_row(const Problem& p, const Tile& t, int r, int* token, int* lo, int* hi) {
  *lo = 0; *hi = t.nk - 1; *token = -1;
  switch (t.kind) {
    case KIND_LLM_SCATTER:
    case KIND_LLM_GATHER1: {
      const int q = t.t0 + r;
      if (q < t.nq) { *token = llm_group_token(t.kind, p.G, t.g, q); *hi = q; }
      break;
    }
    case KIND_LLM_WINDOW: {
      const int i = t.t0 + r;
      if (i < t.nq) {
        *token = i;
        *lo = imax((i / 64) * 64 - (p.W - 64), 0) - t.kbase;
        *hi = i - t.kbase;
      }
      break;
    }
    case KIND_IMG_SCATTER: {
      const int u = t.t0 + r;
      if (t.is_text) { if (r < TEXT_CHUNK) *token = t.g * TEXT_CHUNK + r; }
      else if (u < t.nq) *token = img_scatter_token(p.W, t.g, u);
      break;
    }
    case KIND_IMG_GATHER0: {
      if (r < t.nq) {
        const int side = r / (PATCH * PATCH);      // 0: left patch, 1: right patch
        const int i = r % (PATCH * PATCH);
        *token = TEXT_LEN + (t.prow * PATCH + i / PATCH) * p.W + (t.pcol + side) * PATCH + i % PATCH;
        *lo = side ? WIN * t.off : 0;
        *hi = *lo + TEXT_LEN + WIN * WIN - 1;
      }
      break;
    }
    default: break;
  }
}

// Token id held by key slot u of tile t, or -1 for a padding slot.
//
// Gather-0 patch-pair tiles order their slots so that each patch's keys are one contiguous
// interval: [columns only the left patch sees | shared columns | 512 text | columns only the
// right patch sees], image columns stored column-major (16 window rows per column).
INTRA_HD int key_token(const Problem& p, const Tile& t, int u) {
  if (u < 0 || u >= t.nk) return -1;
  switch (t.kind) {
    case KIND_LLM_SCATTER:
    case KIND_LLM_GATHER1:
      return llm_group_token(t.kind, p.G, t.g, u);
    case KIND_LLM_WINDOW:
      return t.kbase + u;
    case KIND_IMG_SCATTER:
      return u < TEXT_LEN ? u : img_scatter_token(p.W, t.g, u - TEXT_LEN);
    case KIND_IMG_GATHER0: {
      int v;
      if (u < WIN * WIN) v = u;
      else if (u < WIN * WIN + TEXT_LEN) return u - WIN * WIN;
      else v = u - TEXT_LEN;
      return TEXT_LEN + (t.r0 + v % WIN) * p.W + t.c0 + v / WIN;
    }
    default: return -1;
  }
}

// ----------------------------------------------------------------------------------------------
// Pair tiles: two query sub-tiles that share one key-slot list, so that one K / V tile in shared
// memory feeds 256 query rows.
//
//   head pairs (row_pairs == 0): both sub-tiles are the same Tile; the caller gives them two query
//       heads of one KV-head group (grouped-query attention).
//   row pairs  (row_pairs == 1): the sub-tiles are two different Tiles of one head whose keys
//       coincide or nest: consecutive tiles of a Scatter / Gather-1 group, of the window sequence,
//       or of an image-Scatter group. The shared key list is the union; each sub-tile's [lo, hi]
//       is shifted into the union's slot numbering (only the window pattern needs a shift).
//       Gather-0 has no two tiles with nested keys: its pairs are two tiles with the same number of
//       key tiles, each keeping its own key list (sub[s] is then also sub-tile s's key-slot map).
struct PairTile {
  Tile sub[2];     // sub-tile with n_kv_tiles == 0 is absent (all its rows are padding)
  Tile kv;         // key-slot map of the pair; kv.n_kv_tiles key tiles are processed
  int shift[2];    // added to sub[s]'s lo / hi to express them in kv's slot numbering
};

INTRA_HD int n_pair_tiles(const Problem& p, int row_pairs) {
  if (!row_pairs) return p.n_tiles;
  switch (p.kind) {
    case KIND_LLM_SCATTER:
    case KIND_LLM_GATHER1: return ceil_div(p.tiles_m, 2) * p.G;
    case KIND_LLM_WINDOW: return ceil_div(p.n_tiles, 2);
    case KIND_IMG_SCATTER: return ceil_div(p.tiles_m, 2) * IMG_GROUPS;
    case KIND_IMG_GATHER0: return IMG_GROUPS / 2 + ceil_div(p.n_tiles - IMG_GROUPS, 2);
    default: return 0;
  }
}

// Pair tile `idx` in [0, n_pair_tiles), heaviest first.
INTRA_HD PairTile make_pair(const Problem& p, int row_pairs, int idx) {
  PairTile pt;
  pt.shift[0] = pt.shift[1] = 0;
  if (!row_pairs) {
    pt.sub[0] = pt.sub[1] = pt.kv = make_tile(p, idx);
    return pt;
  }
  int idx_first = -1, idx_second = -1;     // first = earlier rows / fewer keys
  switch (p.kind) {
    case KIND_LLM_SCATTER:
    case KIND_LLM_GATHER1: {
      const int g = idx % p.G, mp = idx / p.G;
      idx_second = (2 * mp) * p.G + g;
      if (2 * mp + 1 < p.tiles_m) idx_first = (2 * mp + 1) * p.G + g;
      break;
    }
    case KIND_LLM_WINDOW:
      idx_second = 2 * idx;
      if (2 * idx + 1 < p.n_tiles) idx_first = 2 * idx + 1;
      break;
    case KIND_IMG_SCATTER: {
      // All pairs weigh the same, so the order is free: group-major, so that the pairs in flight at any
      // moment are the row pairs of a few (head, group) key sets that stay in L2, instead of one row
      // pair of every group, which re-reads every key set from DRAM once per row pair.
      const int n_mp = ceil_div(p.tiles_m, 2);
      const int g = idx / n_mp, mp = idx % n_mp;
      idx_first = (2 * mp) * IMG_GROUPS + g;
      if (2 * mp + 1 < p.tiles_m) idx_second = (2 * mp + 1) * IMG_GROUPS + g;
      break;
    }
    case KIND_IMG_GATHER0: {
      // Gather-0 tiles share no keys: a "pair" is two tiles of equal length (two text chunks, or two
      // patch pairs) that keep their own key lists; the caller gives each its own K / V buffers. A
      // last tile without a partner is doubled.
      PairTile sp;
      sp.shift[0] = sp.shift[1] = 0;
      const int first = idx < IMG_GROUPS / 2 ? 2 * idx : IMG_GROUPS + 2 * (idx - IMG_GROUPS / 2);
      sp.sub[0] = make_tile(p, first);
      sp.sub[1] = make_tile(p, first + 1 < p.n_tiles ? first + 1 : first);
      if (first + 1 >= p.n_tiles) { sp.sub[1].n_kv_tiles = 0; sp.sub[1].nq = 0; }   // absent
      sp.kv = sp.sub[0];                                   // only its n_kv_tiles is used in this mode:
      sp.kv.n_kv_tiles = imax(sp.sub[0].n_kv_tiles, sp.sub[1].n_kv_tiles);   // shorter list is padded
      sp.kv.nk = sp.kv.n_kv_tiles * TILE_N;
      return sp;
    }
    default: break;
  }
  Tile none = make_tile(p, 0);
  none.n_kv_tiles = 0; none.nq = 0; none.nk = 0;
  pt.sub[0] = idx_first >= 0 ? make_tile(p, idx_first) : none;
  pt.sub[1] = idx_second >= 0 ? make_tile(p, idx_second) : none;
  const bool has0 = pt.sub[0].n_kv_tiles > 0, has1 = pt.sub[1].n_kv_tiles > 0;
  pt.kv = has1 ? pt.sub[1] : pt.sub[0];
  if (p.kind == KIND_LLM_WINDOW && has0 && has1) {
    pt.kv.kbase = pt.sub[0].kbase;                                  // earlier rows start earlier
    pt.kv.nk = pt.sub[1].kbase + pt.sub[1].nk - pt.kv.kbase;
    pt.kv.n_kv_tiles = ceil_div(pt.kv.nk, TILE_N);
    pt.shift[1] = pt.sub[1].kbase - pt.kv.kbase;
  }
  if (!has0 && !has1) pt.kv.n_kv_tiles = 0;
  return pt;
}

// Key-slot map of sub-tile s: the pair's shared map, or the sub-tile's own when the pair does not share
// keys (an absent sub-tile borrows the other one's so that loads stay in bounds).
INTRA_HD const Tile& pair_kv_map(const PairTile& pt, int split_kv, int s) {
  if (!split_kv) return pt.kv;
  return pt.sub[s].n_kv_tiles > 0 ? pt.sub[s] : pt.sub[s ^ 1];
}

// q_row of sub-tile s of a pair, with lo / hi in the pair's slot numbering.
INTRA_HD void pair_q_row(const Problem& p, const PairTile& pt, int s, int r, int* token, int* lo, int* hi) {
  if (pt.sub[s].n_kv_tiles == 0) { *token = -1; *lo = 0; *hi = pt.kv.nk - 1; return; }
  q_row(p, pt.sub[s], r, token, lo, hi);
  if (*token < 0) { *lo = 0; *hi = pt.kv.nk - 1; return; }
  *lo += pt.shift[s];
  *hi += pt.shift[s];
}

}  // namespace intra
