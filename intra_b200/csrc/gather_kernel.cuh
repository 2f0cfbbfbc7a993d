// Head interleave for the multi-GPU launcher: an all-gather of head-sharded outputs lands rank-major,
// parts[w][row][block], and callers want (batch, token, head, 128) order, out[row][w][block], where a
// row is one (batch, token) and a block is one rank's heads of that row (heads/world * 256 bytes).
// A pure copy, bound by HBM bandwidth: every 16-byte unit is read once and written once, consecutive
// threads move consecutive units of a block, and the grid is a multiple of the SM count walking the
// units with a grid stride. The reference has no multi-GPU path and so no counterpart.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace intra {

constexpr int INTERLEAVE_THREADS = 256;
constexpr int INTERLEAVE_UNROLL = 4;     // independent 16-byte loads in flight per thread

// units16: 16-byte units per block; total = world * rows * units16.
__global__ void __launch_bounds__(INTERLEAVE_THREADS)
interleave_heads_kernel(const uint4* __restrict__ parts, uint4* __restrict__ out, int world, int64_t rows, int units16) {
  const int64_t total = int64_t(world) * rows * units16;
  const int64_t stride = int64_t(gridDim.x) * INTERLEAVE_THREADS;
  for (int64_t i0 = int64_t(blockIdx.x) * INTERLEAVE_THREADS + threadIdx.x; i0 < total; i0 += stride * INTERLEAVE_UNROLL) {
    uint4 val[INTERLEAVE_UNROLL];
    int64_t dst[INTERLEAVE_UNROLL];
#pragma unroll
    for (int j = 0; j < INTERLEAVE_UNROLL; ++j) {
      const int64_t i = i0 + j * stride;                 // index into out: (row, w, unit)
      dst[j] = -1;
      if (i < total) {
        const int unit = int(i % units16);
        const int64_t rw = i / units16;
        const int w = int(rw % world);
        const int64_t row = rw / world;
        val[j] = __ldcs(parts + (int64_t(w) * rows + row) * units16 + unit);
        dst[j] = i;
      }
    }
#pragma unroll
    for (int j = 0; j < INTERLEAVE_UNROLL; ++j)
      if (dst[j] >= 0) __stcs(out + dst[j], val[j]);
  }
}

}  // namespace intra
