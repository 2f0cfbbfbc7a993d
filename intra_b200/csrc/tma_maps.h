// Tensor-map (TMA) views of the Q / K / V tensors for the patterns whose row gathers are affine:
// a 128-row tile of any such pattern is one box of a <= 5-dimensional strided view of the caller's
// (batch, token, head, 128) tensor, so a single thread can fetch it with two bulk-tensor copies (one
// per 64-element half of the head dim) that land in shared memory already 128-byte swizzled.
//
//   Scatter  (S % G == 0)        dims (d, g, t, head, batch)       box (64, 1, 128)      token = t*G + g
//   Gather-1 (S % G^2 == 0, G|128) dims (d, w, seg, head, batch)   box (64, G, 128/G)    token = seg*G^2 + w, w = g*G + j
//   window                       dims (d, token, head, batch)      box (64, 128)
//   image Scatter, image part    dims (d, c, r, head, batch), traversal strides (1, 4, 2), base at token 512
//                                box (64, W, 2*128/(W/4)): every 4th column from c = b, every 2nd row from r = a
//                text part       dims (d, token, head, batch), 512 tokens, box (64, 128)
//   Gather-0 patch pairs  keys   dims (d, r, c, head, batch), box (64, 16, 8): 8 window columns, 16 rows each
//                        queries dims (d, c, r, head, batch), box (64, 8, 8): one 8x8 patch, two boxes per tile
//            text chunks         as image Scatter (the "aux" map) + the text map
//
// Shapes outside these conditions (ragged groups, odd widths) use the cp.async gathers.
// This replaces the per-thread address arithmetic of the reference's loaders
// (csrc/flash_attn/src/gmem_tile.h:481-1426, csrc/flash_attn/src/intra_copy.h:13-101).
#pragma once
#include <cuda.h>

#include "intra_index.h"

namespace intra {

struct alignas(64) TmaMaps {
  CUtensorMap q_main, k_main, v_main;   // the pattern's strided view
  CUtensorMap q_text, k_text, v_text;   // image kinds: the 512 text tokens
  CUtensorMap k_aux, v_aux;             // Gather-0: image-Scatter view for the keys of its text tiles
};

// Can the problem's tiles be fetched as TMA boxes?
INTRA_HD bool tma_supported(const Problem& p) {
  switch (p.kind) {
    case KIND_LLM_SCATTER: return p.S % p.G == 0;
    case KIND_LLM_GATHER1: return p.S % (p.G * p.G) == 0 && TILE_M % p.G == 0 && p.G * p.G <= 65536;
    case KIND_LLM_WINDOW: return true;
    case KIND_IMG_SCATTER:
    case KIND_IMG_GATHER0:
      return p.W % 8 == 0 && p.W <= 256 && TILE_M % (p.W / 4) == 0 && 2 * (TILE_M / (p.W / 4)) <= 256;
    default: return false;
  }
}

// Box coordinates (innermost first; c[0] is filled by the caller with 0 or 64) of the 128 rows that
// start at `start` in the tile's own numbering: packed index for Scatter / Gather-1 and image
// Scatter image rows, token id for the window and for text rows. Returns 1 if the text map is meant.
INTRA_HD int tma_box_coords(const Problem& p, const Tile& t, int start, bool text, int head, int batch, int c[5]) {
  c[0] = 0; c[1] = 0; c[2] = 0; c[3] = 0; c[4] = 0;
  switch (t.kind) {
    case KIND_LLM_SCATTER:
      c[1] = t.g; c[2] = start; c[3] = head; c[4] = batch;
      return 0;
    case KIND_LLM_GATHER1:
      c[1] = t.g * p.G; c[2] = start / p.G; c[3] = head; c[4] = batch;
      return 0;
    case KIND_LLM_WINDOW:
      c[1] = start; c[2] = head; c[3] = batch;
      return 0;
    case KIND_IMG_SCATTER:
      if (text) { c[1] = start; c[2] = head; c[3] = batch; return 1; }
      c[1] = t.g % 4; c[2] = t.g / 4 + 2 * (start / (p.W / 4)); c[3] = head; c[4] = batch;
      return 0;
    default:
      return 0;
  }
}

// Query sub-tile `t`: where its 128 rows start and whether they are text rows.
INTRA_HD void tma_q_start(const Tile& t, int* start, bool* text) {
  *text = false;
  *start = t.t0;
  if (t.kind == KIND_IMG_SCATTER && t.is_text) { *text = true; *start = t.g * TEXT_CHUNK; }
}
// Key tile n of key-slot map `kv`.
INTRA_HD void tma_kv_start(const Tile& kv, int n, int* start, bool* text) {
  *text = false;
  *start = n * TILE_N;
  if (kv.kind == KIND_LLM_WINDOW) *start += kv.kbase;
  if (kv.kind == KIND_IMG_SCATTER) {
    if (*start < TEXT_LEN) *text = true; else *start -= TEXT_LEN;
  }
}

}  // namespace intra
