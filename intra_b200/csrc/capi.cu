// Host side of libintra_b200: argument checks, per-pattern problem set-up and kernel launches
// behind the C ABI of include/intra_b200.h. Mirrors what the reference's ATen host code does
// (csrc/flash_attn/flash_api.cpp:355-552 `mha_fwd`, :556-763 `mha_fwd_llm`) without ATen: the caller
// owns every tensor, this file only validates, fills the parameter block and launches.
#include "../../include/intra_b200.h"

#include <cuda.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cmath>
#include <cstdlib>
#include <mutex>
#include <vector>

#include "attn_kernel.cuh"
#include "attn_kernel_dual.cuh"
#include "gather_kernel.cuh"
#include "selftest.cuh"

namespace {

using namespace intra;

thread_local int g_last_cuda_error = 0;

constexpr int MAX_DEVICES = 64;
struct DeviceState {
  std::once_flag once;
  int init_status = INTRA_OK;
  int* status_word = nullptr;     // device memory, one int
  int sm_count = 0;
};
DeviceState g_dev[MAX_DEVICES];

// Test hook (intra_b200_test_force_path): overrides of the launcher's own choice of kernel variant.
std::atomic<int> g_force_no_tma{0};      // 1: cp.async row gathers even where TMA boxes would do
// Items with at least this many key tiles on average go to the row-owner form of the kernel
// (attn_kernel_dual.cuh); below it the 4-way column split is faster (measured: equal at 8.5 key tiles
// per item, 18-22 % behind on window patterns with their 5 key tiles, most of them masked at an edge).
#ifndef INTRA_ROW_OWNER_MIN_TILES
#define INTRA_ROW_OWNER_MIN_TILES 8
#endif
constexpr int ROW_OWNER_MIN_TILES = INTRA_ROW_OWNER_MIN_TILES;
std::atomic<int> g_force_split{0};       // 1 (row-owner form), 2 or 4: softmax column split; 0: the launcher decides

int cuda_fail(cudaError_t e) {
  g_last_cuda_error = static_cast<int>(e);
  return INTRA_ERR_CUDA;
}

struct DeviceGuard {
  int prev = -1;
  bool ok = true;
  explicit DeviceGuard(int device) {
    if (cudaGetDevice(&prev) != cudaSuccess) { ok = false; return; }
    if (prev != device && cudaSetDevice(device) != cudaSuccess) ok = false;
  }
  ~DeviceGuard() {
    int cur = -1;
    if (prev >= 0 && cudaGetDevice(&cur) == cudaSuccess && cur != prev) cudaSetDevice(prev);
  }
};

// Shared-memory opt-in of every kernel variant, on the current device. Allocates nothing.
template <typename K>
cudaError_t opt_in_smem(K kernel, int bytes) {
  return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
}
cudaError_t set_kernel_attributes() {
  cudaError_t e = opt_in_smem(umma_selftest_kernel, SELFTEST_SMEM_BYTES);
  if (e == cudaSuccess) e = opt_in_smem(intra_fwd_dual_kernel<1, false, true>, DUAL_SMEM_BYTES);
  if (e == cudaSuccess) e = opt_in_smem(intra_fwd_dual_kernel<1, false, false>, DUAL_SMEM_BYTES);
  if (e == cudaSuccess) e = opt_in_smem(intra_fwd_dual_kernel<2, false, true>, DUAL_SMEM_BYTES);
  if (e == cudaSuccess) e = opt_in_smem(intra_fwd_dual_kernel<2, false, false>, DUAL_SMEM_BYTES);
  if (e == cudaSuccess) e = opt_in_smem(intra_fwd_dual_kernel<4, false, true>, DUAL_SMEM_BYTES);
  if (e == cudaSuccess) e = opt_in_smem(intra_fwd_dual_kernel<4, false, false>, DUAL_SMEM_BYTES);
  if (e == cudaSuccess) e = opt_in_smem(intra_fwd_dual_kernel<2, true, true>, DUAL_SMEM_BYTES);
  if (e == cudaSuccess) e = opt_in_smem(intra_fwd_dual_kernel<2, true, false>, DUAL_SMEM_BYTES);
  if (e == cudaSuccess) e = opt_in_smem(intra_fwd_dual_kernel<4, true, true>, DUAL_SMEM_BYTES);
  if (e == cudaSuccess) e = opt_in_smem(intra_fwd_dual_kernel<4, true, false>, DUAL_SMEM_BYTES);
  return e;
}

// One-time set-up of a device (current when called): architecture check, shared-memory opt-in of the
// kernels, and the status word the kernels report to.
void init_device(int device) {
  DeviceState& st = g_dev[device];
  cudaDeviceProp prop;
  cudaError_t e = cudaGetDeviceProperties(&prop, device);
  if (e != cudaSuccess) { st.init_status = cuda_fail(e); return; }
  if (prop.major != 10) { st.init_status = INTRA_ERR_DEVICE; return; }
  e = set_kernel_attributes();
  st.sm_count = prop.multiProcessorCount;
  if (e == cudaSuccess) e = cudaMalloc(&st.status_word, sizeof(int));
  if (e == cudaSuccess) e = cudaMemset(st.status_word, 0, sizeof(int));
  if (e != cudaSuccess) st.init_status = cuda_fail(e);
}

int ensure_device(int device) {
  if (device < 0 || device >= MAX_DEVICES) return INTRA_ERR_BAD_ARG;
  DeviceState& st = g_dev[device];
  std::call_once(st.once, init_device, device);
  return st.init_status;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
bool strides_ok(const int64_t s[3]) { return s && s[0] % 8 == 0 && s[1] % 8 == 0 && s[2] % 8 == 0; }

int map_kind(int family, int pattern) {
  if (family == 0) {
    if (pattern == INTRA_LLM_SCATTER) return KIND_LLM_SCATTER;
    if (pattern == INTRA_LLM_GATHER1) return KIND_LLM_GATHER1;
    if (pattern == INTRA_LLM_WINDOW) return KIND_LLM_WINDOW;
  } else if (family == 1) {
    if (pattern == INTRA_IMAGE_SCATTER) return KIND_IMG_SCATTER;
    if (pattern == INTRA_IMAGE_GATHER0) return KIND_IMG_GATHER0;
  }
  return -1;
}

// `param` is group_num for scatter / gather1 and window / width otherwise.
int problem_from(int family, int pattern, int S, int param, Problem* prob) {
  const int kind = map_kind(family, pattern);
  if (kind < 0) return INTRA_ERR_UNSUPPORTED;
  const bool grouped = kind == KIND_LLM_SCATTER || kind == KIND_LLM_GATHER1;
  if (make_problem(kind, S, grouped ? param : 0, grouped ? 0 : param, prob) != 0) return INTRA_ERR_UNSUPPORTED;
  return INTRA_OK;
}

// ---- tensor maps ------------------------------------------------------------------------------------
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// cuTensorMapEncodeTiled through the runtime, so the library does not link against libcuda.
EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = [] {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult r;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &r) != cudaSuccess ||
        r != cudaDriverEntryPointSuccess)
      f = nullptr;
    return reinterpret_cast<EncodeTiledFn>(f);
  }();
  return fn;
}

bool encode_map(CUtensorMap* m, const void* base, int rank, const cuuint64_t* dims, const cuuint64_t* strides_bytes,
                const cuuint32_t* box, const cuuint32_t* estr) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return false;
  for (int i = 0; i < rank; ++i)
    if (dims[i] == 0 || dims[i] > 0xffffffffull || box[i] == 0 || box[i] > 256) return false;
  for (int i = 0; i + 1 < rank; ++i)
    if (strides_bytes[i] == 0 || strides_bytes[i] % 16 != 0 || strides_bytes[i] >= (1ull << 40)) return false;
  return fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, rank, const_cast<void*>(base), dims, strides_bytes, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// The views of tma_maps.h for one (batch, token, head, 128) tensor with `heads` heads.
bool build_maps(const Problem& p, const __nv_bfloat16* ptr, const TensorView& tv, int heads, int B, bool is_query,
                CUtensorMap* main_map, CUtensorMap* text_map, CUtensorMap* aux_map) {
  const cuuint64_t ss = cuuint64_t(tv.ss) * 2, sh = cuuint64_t(tv.sh) * 2, sb = cuuint64_t(tv.sb) * 2;
  if (tv.ss <= 0 || tv.sh <= 0 || tv.sb <= 0) return false;
  const cuuint32_t ones[5] = {1, 1, 1, 1, 1};
  switch (p.kind) {
    case KIND_LLM_SCATTER: {
      const cuuint64_t dims[5] = {128, cuuint64_t(p.G), cuuint64_t(p.S / p.G), cuuint64_t(heads), cuuint64_t(B)};
      const cuuint64_t str[4] = {ss, ss * p.G, sh, sb};
      const cuuint32_t box[5] = {64, 1, 128, 1, 1};
      return encode_map(main_map, ptr, 5, dims, str, box, ones);
    }
    case KIND_LLM_GATHER1: {
      const cuuint64_t span = cuuint64_t(p.G) * p.G;
      const cuuint64_t dims[5] = {128, span, cuuint64_t(p.S) / span, cuuint64_t(heads), cuuint64_t(B)};
      const cuuint64_t str[4] = {ss, ss * span, sh, sb};
      const cuuint32_t box[5] = {64, cuuint32_t(p.G), cuuint32_t(TILE_M / p.G), 1, 1};
      return encode_map(main_map, ptr, 5, dims, str, box, ones);
    }
    case KIND_LLM_WINDOW: {
      const cuuint64_t dims[4] = {128, cuuint64_t(p.S), cuuint64_t(heads), cuuint64_t(B)};
      const cuuint64_t str[3] = {ss, sh, sb};
      const cuuint32_t box[4] = {64, 128, 1, 1};
      return encode_map(main_map, ptr, 4, dims, str, box, ones);
    }
    case KIND_IMG_SCATTER: {
      const cuuint64_t dims[5] = {128, cuuint64_t(p.W), cuuint64_t(p.W), cuuint64_t(heads), cuuint64_t(B)};
      const cuuint64_t str[4] = {ss, ss * p.W, sh, sb};
      const cuuint32_t box[5] = {64, cuuint32_t(p.W), cuuint32_t(2 * (TILE_M / (p.W / 4))), 1, 1};
      const cuuint32_t estr[5] = {1, 4, 2, 1, 1};
      if (!encode_map(main_map, ptr + int64_t(TEXT_LEN) * tv.ss, 5, dims, str, box, estr)) return false;
      const cuuint64_t tdims[4] = {128, TEXT_LEN, cuuint64_t(heads), cuuint64_t(B)};
      const cuuint64_t tstr[3] = {ss, sh, sb};
      const cuuint32_t tbox[4] = {64, 128, 1, 1};
      return encode_map(text_map, ptr, 4, tdims, tstr, tbox, ones);
    }
    case KIND_IMG_GATHER0: {
      // patch-pair tiles: keys as 16-row x 8-column boxes (row index fastest), queries as 8x8 patches
      const __nv_bfloat16* img = ptr + int64_t(TEXT_LEN) * tv.ss;
      const cuuint64_t dims[5] = {128, cuuint64_t(p.W), cuuint64_t(p.W), cuuint64_t(heads), cuuint64_t(B)};
      if (is_query) {
        const cuuint64_t str[4] = {ss, ss * p.W, sh, sb};            // (d, c, r, head, batch)
        const cuuint32_t box[5] = {64, PATCH, PATCH, 1, 1};
        if (!encode_map(main_map, img, 5, dims, str, box, ones)) return false;
      } else {
        const cuuint64_t str[4] = {ss * p.W, ss, sh, sb};            // (d, r, c, head, batch)
        const cuuint32_t box[5] = {64, WIN, 8, 1, 1};
        if (!encode_map(main_map, img, 5, dims, str, box, ones)) return false;
        // text tiles: image-Scatter view of the keys
        const cuuint64_t astr[4] = {ss, ss * p.W, sh, sb};
        const cuuint32_t abox[5] = {64, cuuint32_t(p.W), cuuint32_t(2 * (TILE_M / (p.W / 4))), 1, 1};
        const cuuint32_t aestr[5] = {1, 4, 2, 1, 1};
        if (!encode_map(aux_map, img, 5, dims, astr, abox, aestr)) return false;
      }
      const cuuint64_t tdims[4] = {128, TEXT_LEN, cuuint64_t(heads), cuuint64_t(B)};
      const cuuint64_t tstr[3] = {ss, sh, sb};
      const cuuint32_t tbox[4] = {64, 128, 1, 1};
      return encode_map(text_map, ptr, 4, tdims, tstr, tbox, ones);
    }
    default:
      return false;
  }
}

// ---- scratch for intra_b200_fwd_llm_noalloc -------------------------------------------------------
// The attention kernel's only scratch is the status word it reports to. For callers that must not
// allocate, that word lives in this fixed array, which every GPU that loads the library holds until
// the process exits. Host code sees only a stand-in for the array under this name; its device
// address is fetched once per device with cudaGetSymbolAddress and handed to the kernel.
constexpr size_t NOALLOC_SCRATCH_BYTES = 256;
static __device__ __align__(256) unsigned char g_noalloc_scratch[NOALLOC_SCRATCH_BYTES];

struct NoAllocState {
  std::once_flag once;
  int init_status = INTRA_OK;
  int* scratch = nullptr;         // device address of g_noalloc_scratch on this device
  int sm_count = 0;
};
NoAllocState g_noalloc[MAX_DEVICES];

// Runs once per device with that device current. Allocates nothing.
void init_noalloc(int device) {
  NoAllocState& st = g_noalloc[device];
  int major = 0;
  cudaError_t e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device);
  if (e != cudaSuccess) { st.init_status = cuda_fail(e); return; }
  if (major != 10) { st.init_status = INTRA_ERR_DEVICE; return; }
  e = cudaDeviceGetAttribute(&st.sm_count, cudaDevAttrMultiProcessorCount, device);
  if (e == cudaSuccess) e = set_kernel_attributes();
  void* ptr = nullptr;
  if (e == cudaSuccess) e = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
  if (e != cudaSuccess) { st.init_status = cuda_fail(e); return; }
  st.scratch = static_cast<int*>(ptr);
}

// Bytes of scratch one launch of the attention kernel needs: its status word.
size_t fwd_scratch_bytes(const Problem&) { return sizeof(int); }

// Checks that need no device: pointers, sizes, alignment, and the pattern's problem description.
int check_args(const void* q, const void* k, const void* v, void* out, int B, int S, int H, int Hkv,
               const int64_t* qs, const int64_t* ks, const int64_t* vs, const int64_t* os, int family, int pattern,
               int param, float softmax_scale, Problem* prob) {
  if (!q || !k || !v || !out || B <= 0 || S <= 0 || H <= 0 || Hkv <= 0 || H % Hkv != 0) return INTRA_ERR_BAD_ARG;
  if (!qs || !ks || !vs || !os) return INTRA_ERR_BAD_ARG;
  if (!(softmax_scale > 0.f) || !std::isfinite(softmax_scale)) return INTRA_ERR_BAD_ARG;
  // every head, token and batch of the output must be a distinct row: a zero or negative stride (an
  // expanded tensor) would make different tiles write the same memory
  if (os[0] <= 0 || os[1] <= 0 || os[2] <= 0) return INTRA_ERR_BAD_ARG;
  if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(out) || !strides_ok(qs) || !strides_ok(ks) ||
      !strides_ok(vs) || !strides_ok(os))
    return INTRA_ERR_ALIGNMENT;
  int rc = problem_from(family, pattern, S, param, prob);
  if (rc != INTRA_OK) return rc;
  const int64_t blocks = int64_t(prob->n_tiles) * B * H;
  if (blocks <= 0 || blocks > 0x7fffffffLL) return INTRA_ERR_UNSUPPORTED;
  return INTRA_OK;
}

// How the launcher splits a problem into the persistent kernel's items, and which kernel variant it
// picks (the counterpart of the reference's MASK_SWITCH / launch templates,
// csrc/flash_attn/src/flash_fwd_launch_template.h:401-565, :720-776).
// Softmax arrangement (attn_kernel_dual.cuh) for a problem: 4 = 4-way column split (short items),
// 1 = row-owner form (long items that share their key tiles), 2 = 2-way split (long items with split
// key lists). Host arithmetic only.
int pick_form(const Problem& prob, int row_pairs, int split_kv) {
  const int n_pairs = n_pair_tiles(prob, row_pairs);
  int64_t n_tiles = 0, n_kv = 0;
  for (int idx = 0; idx < n_pairs; ++idx) {
    const int t = make_pair(prob, row_pairs, idx).kv.n_kv_tiles;
    if (t > 0) { ++n_tiles; n_kv += t; }
  }
  const int force_split = g_force_split.load();
  int form = force_split ? force_split : (n_tiles > 0 && n_kv < int64_t(ROW_OWNER_MIN_TILES) * n_tiles) ? 4 : 1;
  if (form == 1 && split_kv) form = 2;
  return form;
}

int plan_launch(const FwdParams& p, DualParams* d, int* split) {
  d->f = p;
  d->split_kv = p.prob.kind == KIND_IMG_GATHER0 ? 1 : 0;
  d->row_pairs = (d->split_kv || (p.H / p.Hkv) % 2 != 0) ? 1 : 0;
  d->n_pair_tiles = n_pair_tiles(p.prob, d->row_pairs);
  d->heads_per_item = d->row_pairs ? p.H : p.H / 2;
  const int64_t items = int64_t(d->n_pair_tiles) * p.B * d->heads_per_item;
  if (items <= 0 || items > 0x7fffffffLL) return INTRA_ERR_UNSUPPORTED;
  d->n_items = static_cast<int>(items);
  d->wide_stores = (reinterpret_cast<uintptr_t>(p.o) % 32 == 0 && p.os.sb % 16 == 0 && p.os.ss % 16 == 0 && p.os.sh % 16 == 0) ? 1 : 0;
  d->use_tma = !g_force_no_tma.load() && tma_supported(p.prob) &&
               build_maps(p.prob, p.q, p.qs, p.H, p.B, true, &d->maps.q_main, &d->maps.q_text, &d->maps.k_aux) &&
               build_maps(p.prob, p.k, p.ks, p.Hkv, p.B, false, &d->maps.k_main, &d->maps.k_text, &d->maps.k_aux) &&
               build_maps(p.prob, p.v, p.vs, p.Hkv, p.B, false, &d->maps.v_main, &d->maps.v_text, &d->maps.v_aux);
  *split = pick_form(p.prob, d->row_pairs, d->split_kv);
  return INTRA_OK;
}

// Fills the parameter block and launches the attention kernel on `stream` of the current device.
// `status_word` is where the kernel records a bounded wait that ran out; nothing here allocates.
int launch_fwd(const void* q, const void* k, const void* v, void* out, int B, int H, int Hkv, const int64_t* qs,
               const int64_t* ks, const int64_t* vs, const int64_t* os, const Problem& prob, float softmax_scale,
               int* status_word, int sm_count, cudaStream_t st, float* lse) {
  FwdParams p;
  p.prob = prob;
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.k = static_cast<const __nv_bfloat16*>(k);
  p.v = static_cast<const __nv_bfloat16*>(v);
  p.o = static_cast<__nv_bfloat16*>(out);
  p.qs = {qs[0], qs[1], qs[2]};
  p.ks = {ks[0], ks[1], ks[2]};
  p.vs = {vs[0], vs[1], vs[2]};
  p.os = {os[0], os[1], os[2]};
  p.B = B; p.H = H; p.Hkv = Hkv;
  p.scale_log2 = softmax_scale * 1.4426950408889634f;
  p.status = status_word;
  p.lse = lse;
  DualParams d;
  int split = 0;
  int rc = plan_launch(p, &d, &split);
  if (rc != INTRA_OK) return rc;
  const int grid = d.n_items < sm_count ? d.n_items : sm_count;     // persistent: one CTA per SM
#define INTRA_LAUNCH_DUAL(N, SPLIT) \
  do { \
    if (d.use_tma) intra_fwd_dual_kernel<N, SPLIT, true><<<grid, DualCfg<N>::THREADS, DUAL_SMEM_BYTES, st>>>(d); \
    else intra_fwd_dual_kernel<N, SPLIT, false><<<grid, DualCfg<N>::THREADS, DUAL_SMEM_BYTES, st>>>(d); \
  } while (0)
  if (split == 4 && d.split_kv) INTRA_LAUNCH_DUAL(4, true);
  else if (split == 4) INTRA_LAUNCH_DUAL(4, false);
  else if (d.split_kv) INTRA_LAUNCH_DUAL(2, true);
  else if (split == 2) INTRA_LAUNCH_DUAL(2, false);
  else INTRA_LAUNCH_DUAL(1, false);
#undef INTRA_LAUNCH_DUAL
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e);
  return INTRA_OK;
}

// The regular entry points: per-device state (with its one allocation, the status word) on first use.
int run_fwd(const void* q, const void* k, const void* v, void* out, int B, int S, int H, int Hkv,
            const int64_t* qs, const int64_t* ks, const int64_t* vs, const int64_t* os, int family, int pattern,
            int param, float softmax_scale, int device, void* stream, float* lse = nullptr) {
  Problem prob;
  int rc = check_args(q, k, v, out, B, S, H, Hkv, qs, ks, vs, os, family, pattern, param, softmax_scale, &prob);
  if (rc != INTRA_OK) return rc;
  DeviceGuard guard(device);
  if (!guard.ok) return cuda_fail(cudaGetLastError());
  rc = ensure_device(device);
  if (rc != INTRA_OK) return rc;
  return launch_fwd(q, k, v, out, B, H, Hkv, qs, ks, vs, os, prob, softmax_scale, g_dev[device].status_word,
                    g_dev[device].sm_count, static_cast<cudaStream_t>(stream), lse);
}

}  // namespace

extern "C" {

int intra_b200_fwd_llm(const void* q, const void* k, const void* v, void* out, int B, int S, int H, int Hkv,
                       const int64_t q_strides[3], const int64_t k_strides[3], const int64_t v_strides[3],
                       const int64_t out_strides[3], int pattern, int group_num, int window, float softmax_scale,
                       int device, void* cuda_stream) {
  const int param = pattern == INTRA_LLM_WINDOW ? window : group_num;
  return run_fwd(q, k, v, out, B, S, H, Hkv, q_strides, k_strides, v_strides, out_strides, 0, pattern, param,
                    softmax_scale, device, cuda_stream);
}

int intra_b200_fwd_image(const void* q, const void* k, const void* v, void* out, int B, int S, int H,
                         const int64_t q_strides[3], const int64_t k_strides[3], const int64_t v_strides[3],
                         const int64_t out_strides[3], int pattern, int width, float softmax_scale, int device,
                         void* cuda_stream) {
  return run_fwd(q, k, v, out, B, S, H, H, q_strides, k_strides, v_strides, out_strides, 1, pattern, width,
                    softmax_scale, device, cuda_stream);
}

int intra_b200_fwd_llm_lse(const void* q, const void* k, const void* v, void* out, float* lse, int B, int S, int H,
                           int Hkv, const int64_t q_strides[3], const int64_t k_strides[3],
                           const int64_t v_strides[3], const int64_t out_strides[3], int pattern, int group_num,
                           int window, float softmax_scale, int device, void* cuda_stream) {
  if (!lse || reinterpret_cast<uintptr_t>(lse) % 4 != 0) return INTRA_ERR_BAD_ARG;
  const int param = pattern == INTRA_LLM_WINDOW ? window : group_num;
  return run_fwd(q, k, v, out, B, S, H, Hkv, q_strides, k_strides, v_strides, out_strides, 0, pattern, param,
                    softmax_scale, device, cuda_stream, lse);
}

int intra_b200_fwd_image_lse(const void* q, const void* k, const void* v, void* out, float* lse, int B, int S, int H,
                             const int64_t q_strides[3], const int64_t k_strides[3], const int64_t v_strides[3],
                             const int64_t out_strides[3], int pattern, int width, float softmax_scale, int device,
                             void* cuda_stream) {
  if (!lse || reinterpret_cast<uintptr_t>(lse) % 4 != 0) return INTRA_ERR_BAD_ARG;
  return run_fwd(q, k, v, out, B, S, H, H, q_strides, k_strides, v_strides, out_strides, 1, pattern, width,
                    softmax_scale, device, cuda_stream, lse);
}

const char* intra_b200_strerror(int status) {
  switch (status) {
    case INTRA_OK: return "ok";
    case INTRA_ERR_BAD_ARG: return "bad argument: null pointer, non-positive size, heads not divisible, or softmax scale not positive";
    case INTRA_ERR_UNSUPPORTED: return "unsupported pattern / group_num / window / width / sequence length";
    case INTRA_ERR_ALIGNMENT: return "pointers and strides must keep every 128-element bf16 row 16-byte aligned";
    case INTRA_ERR_CUDA: return "a CUDA runtime call failed (see intra_b200_last_cuda_error)";
    case INTRA_ERR_DEVICE: return "device is not an sm_100 (B200) GPU";
    case INTRA_ERR_KERNEL: return "a kernel gave up on a bounded wait (see intra_b200_device_status)";
    default: return "unknown status";
  }
}

int intra_b200_last_cuda_error(void) { return g_last_cuda_error; }

int intra_b200_device_status(int device, int* status_word, int reset) {
  if (!status_word) return INTRA_ERR_BAD_ARG;
  DeviceGuard guard(device);
  if (!guard.ok) return cuda_fail(cudaGetLastError());
  int rc = ensure_device(device);
  if (rc != INTRA_OK) return rc;
  cudaError_t e = cudaDeviceSynchronize();
  if (e == cudaSuccess) e = cudaMemcpy(status_word, g_dev[device].status_word, sizeof(int), cudaMemcpyDeviceToHost);
  if (e == cudaSuccess && reset && *status_word != 0) e = cudaMemset(g_dev[device].status_word, 0, sizeof(int));
  if (e != cudaSuccess) return cuda_fail(e);
  return *status_word == 0 ? INTRA_OK : INTRA_ERR_KERNEL;
}

int intra_b200_visited_host(int family, int pattern, int S, int param, uint8_t* counts) {
  if (!counts) return INTRA_ERR_BAD_ARG;
  Problem prob;
  int rc = problem_from(family, pattern, S, param, &prob);
  if (rc != INTRA_OK) return rc;
  for (int idx = 0; idx < prob.n_tiles; ++idx) {
    const Tile t = make_tile(prob, idx);
    if (t.n_kv_tiles == 0) continue;
    for (int r = 0; r < TILE_M; ++r) {
      int token, lo, hi;
      q_row(prob, t, r, &token, &lo, &hi);
      if (token < 0) continue;
      if (token >= S || lo < 0 || hi >= t.n_kv_tiles * TILE_N) return INTRA_ERR_KERNEL;   // map out of range
      for (int u = lo; u <= hi; ++u) {
        const int kt = key_token(prob, t, u);
        if (kt < 0) continue;
        if (kt >= S) return INTRA_ERR_KERNEL;
        uint8_t* c = counts + size_t(token) * S + kt;
        if (*c < 255) ++*c;
      }
    }
  }
  return INTRA_OK;
}

int intra_b200_visited_pairs_host(int family, int pattern, int S, int param, uint8_t* counts) {
  if (!counts) return INTRA_ERR_BAD_ARG;
  Problem prob;
  int rc = problem_from(family, pattern, S, param, &prob);
  if (rc != INTRA_OK) return rc;
  const int n = n_pair_tiles(prob, 1);
  if (n <= 0) return INTRA_ERR_UNSUPPORTED;
  for (int idx = 0; idx < n; ++idx) {
    const PairTile pt = make_pair(prob, 1, idx);
    const int split = prob.kind == KIND_IMG_GATHER0;
    for (int s = 0; s < 2; ++s) {
      const Tile& kvmap = pair_kv_map(pt, split, s);
      for (int r = 0; r < TILE_M; ++r) {
        int token, lo, hi;
        pair_q_row(prob, pt, s, r, &token, &lo, &hi);
        if (token < 0) continue;
        if (token >= S || lo < 0 || hi >= pt.kv.n_kv_tiles * TILE_N) return INTRA_ERR_KERNEL;
        for (int u = lo; u <= hi; ++u) {
          const int kt = key_token(prob, kvmap, u);
          if (kt < 0) continue;
          if (kt >= S) return INTRA_ERR_KERNEL;
          uint8_t* c = counts + size_t(token) * S + kt;
          if (*c < 255) ++*c;
        }
      }
    }
  }
  return INTRA_OK;
}

int intra_b200_visited_device(int family, int pattern, int S, int param, uint8_t* counts_dev, int device,
                              void* cuda_stream) {
  if (!counts_dev) return INTRA_ERR_BAD_ARG;
  Problem prob;
  int rc = problem_from(family, pattern, S, param, &prob);
  if (rc != INTRA_OK) return rc;
  DeviceGuard guard(device);
  if (!guard.ok) return cuda_fail(cudaGetLastError());
  rc = ensure_device(device);
  if (rc != INTRA_OK) return rc;
  visited_kernel<<<prob.n_tiles, TILE_M, 0, static_cast<cudaStream_t>(cuda_stream)>>>(prob, counts_dev);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? INTRA_OK : cuda_fail(e);
}

int intra_b200_tile_counts(int family, int pattern, int S, int param, int64_t* n_tiles, int64_t* n_kv_tiles) {
  if (!n_tiles || !n_kv_tiles) return INTRA_ERR_BAD_ARG;
  Problem prob;
  int rc = problem_from(family, pattern, S, param, &prob);
  if (rc != INTRA_OK) return rc;
  int64_t nt = 0, nkv = 0;
  for (int idx = 0; idx < prob.n_tiles; ++idx) {
    const Tile t = make_tile(prob, idx);
    if (t.n_kv_tiles == 0) continue;
    ++nt;
    nkv += t.n_kv_tiles;
  }
  *n_tiles = nt;
  *n_kv_tiles = nkv;
  return INTRA_OK;
}

int intra_b200_selftest_umma(const void* a, const void* b, const void* v, float p_scale, float* s_out, float* o_out,
                             int device, void* cuda_stream) {
  if (!a || !b || !v || !s_out || !o_out) return INTRA_ERR_BAD_ARG;
  DeviceGuard guard(device);
  if (!guard.ok) return cuda_fail(cudaGetLastError());
  int rc = ensure_device(device);
  if (rc != INTRA_OK) return rc;
  umma_selftest_kernel<<<1, 128, SELFTEST_SMEM_BYTES, static_cast<cudaStream_t>(cuda_stream)>>>(
      static_cast<const __nv_bfloat16*>(a), static_cast<const __nv_bfloat16*>(b),
      static_cast<const __nv_bfloat16*>(v), p_scale, s_out, o_out, g_dev[device].status_word);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? INTRA_OK : cuda_fail(e);
}

int intra_b200_interleave_heads(const void* parts, void* out, int world, int64_t rows, int64_t block_bytes,
                                int device, void* cuda_stream) {
  if (!parts || !out || world <= 0 || rows <= 0 || block_bytes <= 0) return INTRA_ERR_BAD_ARG;
  if (!aligned16(parts) || !aligned16(out) || block_bytes % 16 != 0) return INTRA_ERR_ALIGNMENT;
  if (block_bytes / 16 > 0x7fffffffLL) return INTRA_ERR_UNSUPPORTED;
  DeviceGuard guard(device);
  if (!guard.ok) return cuda_fail(cudaGetLastError());
  int rc = ensure_device(device);
  if (rc != INTRA_OK) return rc;
  const int64_t total = int64_t(world) * rows * (block_bytes / 16);
  const int64_t per_cta = int64_t(INTERLEAVE_THREADS) * INTERLEAVE_UNROLL;
  const int64_t want = (total + per_cta - 1) / per_cta;
  const int64_t cap = int64_t(g_dev[device].sm_count) * 8;           // 8 resident CTAs of 256 threads per SM
  const int grid = static_cast<int>(want < cap ? want : cap);
  interleave_heads_kernel<<<grid, INTERLEAVE_THREADS, 0, static_cast<cudaStream_t>(cuda_stream)>>>(
      static_cast<const uint4*>(parts), static_cast<uint4*>(out), world, rows, static_cast<int>(block_bytes / 16));
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? INTRA_OK : cuda_fail(e);
}

int intra_b200_test_kernel_form(int family, int pattern, int S, int param, int H, int Hkv) {
  if (S <= 0 || H <= 0 || Hkv <= 0 || H % Hkv != 0) return INTRA_ERR_BAD_ARG;
  Problem prob;
  const int rc = problem_from(family, pattern, S, param, &prob);
  if (rc != INTRA_OK) return rc;
  const int split_kv = prob.kind == KIND_IMG_GATHER0 ? 1 : 0;
  const int row_pairs = (split_kv || (H / Hkv) % 2 != 0) ? 1 : 0;
  return pick_form(prob, row_pairs, split_kv);
}

int intra_b200_test_force_path(int no_tma, int softmax_split) {
  if (softmax_split != 0 && softmax_split != 1 && softmax_split != 2 && softmax_split != 4) return INTRA_ERR_BAD_ARG;
  g_force_no_tma.store(no_tma ? 1 : 0);
  g_force_split.store(softmax_split);
  return INTRA_OK;
}

int intra_b200_test_poke_status(int device, int value) {
  DeviceGuard guard(device);
  if (!guard.ok) return cuda_fail(cudaGetLastError());
  int rc = ensure_device(device);
  if (rc != INTRA_OK) return rc;
  cudaError_t e = cudaDeviceSynchronize();
  if (e == cudaSuccess) e = cudaMemcpy(g_dev[device].status_word, &value, sizeof(int), cudaMemcpyHostToDevice);
  return e == cudaSuccess ? INTRA_OK : cuda_fail(e);
}

int intra_b200_test_wait_timeout(int limit_ms, long long* waited_ns_dev, int device, void* cuda_stream) {
  if (limit_ms <= 0 || limit_ms > 1000 || !waited_ns_dev) return INTRA_ERR_BAD_ARG;
  DeviceGuard guard(device);
  if (!guard.ok) return cuda_fail(cudaGetLastError());
  int rc = ensure_device(device);
  if (rc != INTRA_OK) return rc;
  abort_selftest_kernel<<<1, 64, 0, static_cast<cudaStream_t>(cuda_stream)>>>(limit_ms, g_dev[device].status_word,
                                                                             waited_ns_dev);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? INTRA_OK : cuda_fail(e);
}

int intra_b200_test_tma_rows(const void* q, const void* k, const void* v, int B, int S, int H, int Hkv,
                             const int64_t q_strides[3], const int64_t k_strides[3], const int64_t v_strides[3],
                             int family, int pattern, int param, int32_t* q_got_dev, int32_t* k_got_dev,
                             int32_t* v_got_dev, int32_t* q_want, int32_t* k_want, int64_t* n_items, int64_t* max_kv,
                             int device, void* cuda_stream) {
  if (!n_items || !max_kv) return INTRA_ERR_BAD_ARG;
  Problem prob;
  // q doubles as the (unused) output pointer so that the common argument checks apply
  int rc = check_args(q, k, v, const_cast<void*>(q), B, S, H, Hkv, q_strides, k_strides, v_strides, q_strides, family,
                      pattern, param, 1.f, &prob);
  if (rc != INTRA_OK) return rc;
  if (!tma_supported(prob)) return INTRA_ERR_UNSUPPORTED;
  DeviceGuard guard(device);
  if (!guard.ok) return cuda_fail(cudaGetLastError());
  rc = ensure_device(device);
  if (rc != INTRA_OK) return rc;
  FwdParams p;
  p.prob = prob;
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.k = static_cast<const __nv_bfloat16*>(k);
  p.v = static_cast<const __nv_bfloat16*>(v);
  p.o = nullptr;
  p.qs = {q_strides[0], q_strides[1], q_strides[2]};
  p.ks = {k_strides[0], k_strides[1], k_strides[2]};
  p.vs = {v_strides[0], v_strides[1], v_strides[2]};
  p.os = p.qs;
  p.B = B; p.H = H; p.Hkv = Hkv;
  p.scale_log2 = 1.f;
  p.status = g_dev[device].status_word;
  p.lse = nullptr;
  DualParams d;
  int split = 0;
  const int forced = g_force_no_tma.exchange(0);           // the maps are wanted whatever the override says
  rc = plan_launch(p, &d, &split);
  g_force_no_tma.store(forced);
  if (rc != INTRA_OK) return rc;
  if (!d.use_tma) return INTRA_ERR_UNSUPPORTED;
  int mk = 0;
  for (int idx = 0; idx < d.n_pair_tiles; ++idx) mk = imax(mk, make_pair(prob, d.row_pairs, idx).kv.n_kv_tiles);
  *n_items = d.n_items;
  *max_kv = mk;
  if (!q_got_dev || !k_got_dev || !v_got_dev || !q_want || !k_want) return INTRA_OK;     // sizes only

  // what should arrive: -9 = any row will do (padding rows, slots no query attends)
  for (int item = 0; item < d.n_items; ++item) {
    const DualItem di = dual_decode(d, item);
    for (int sx = 0; sx < 2; ++sx) {
      int32_t* qw = q_want + (size_t(item) * 2 + sx) * TILE_M;
      int32_t* kw = k_want + (size_t(item) * 2 + sx) * mk * TILE_N;
      for (int i = 0; i < mk * TILE_N; ++i) kw[i] = -9;
      for (int r = 0; r < TILE_M; ++r) qw[r] = -9;
      if (di.pt.kv.n_kv_tiles == 0) continue;
      const Tile& map = pair_kv_map(di.pt, d.split_kv, sx);
      if (d.split_kv || sx == 0)
        for (int u = 0; u < di.pt.kv.n_kv_tiles * TILE_N; ++u) {
          const int kt = key_token(prob, map, u);
          if (kt >= 0) kw[u] = kt;
        }
      for (int r = 0; r < TILE_M; ++r) {
        int token, lo, hi;
        pair_q_row(prob, di.pt, sx, r, &token, &lo, &hi);
        if (token < 0) continue;
        qw[r] = token;
        // every attended slot must hold a real key: slots [0, nk) do, by key_token's first line
        if (lo < 0 || hi >= map.nk || key_token(prob, map, lo) < 0 || key_token(prob, map, hi) < 0) return INTRA_ERR_KERNEL;
      }
    }
  }
  cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
  const int smem = TILE_BYTES + 1024;
  if (d.split_kv) tma_rows_selftest_kernel<true><<<d.n_items, 128, smem, st>>>(d, q_got_dev, k_got_dev, v_got_dev, mk);
  else tma_rows_selftest_kernel<false><<<d.n_items, 128, smem, st>>>(d, q_got_dev, k_got_dev, v_got_dev, mk);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? INTRA_OK : cuda_fail(e);
}

int intra_b200_fwd_llm_noalloc(const void* q, const void* k, const void* v, void* out, int B, int S, int H, int Hkv,
                               const int64_t q_strides[3], const int64_t k_strides[3], const int64_t v_strides[3],
                               const int64_t out_strides[3], int pattern, int group_num, int window,
                               float softmax_scale, int device, void* cuda_stream, int* prev_status) {
  Problem prob;
  int rc = check_args(q, k, v, out, B, S, H, Hkv, q_strides, k_strides, v_strides, out_strides, 0, pattern,
                      pattern == INTRA_LLM_WINDOW ? window : group_num, softmax_scale, &prob);
  if (rc != INTRA_OK) return rc;
  if (device < 0 || device >= MAX_DEVICES) return INTRA_ERR_BAD_ARG;
  // The launch's scratch has to fit the fixed array; a shape that needed more is turned away here.
  if (fwd_scratch_bytes(prob) > NOALLOC_SCRATCH_BYTES) return INTRA_ERR_UNSUPPORTED;

  DeviceGuard guard(device);
  if (!guard.ok) return cuda_fail(cudaGetLastError());
  NoAllocState& st = g_noalloc[device];
  std::call_once(st.once, init_noalloc, device);
  if (st.init_status != INTRA_OK) return st.init_status;

  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  cudaError_t e;
  if (prev_status) {      // what the previous call on this device left behind (0 before the first call)
    e = cudaStreamSynchronize(stream);
    if (e == cudaSuccess) e = cudaMemcpy(prev_status, st.scratch, sizeof(int), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return cuda_fail(e);
  }
  e = cudaMemsetAsync(st.scratch, 0, sizeof(int), stream);   // the status word must start at zero
  if (e != cudaSuccess) return cuda_fail(e);
  return launch_fwd(q, k, v, out, B, H, Hkv, q_strides, k_strides, v_strides, out_strides, prob, softmax_scale,
                    st.scratch, st.sm_count, stream, nullptr);
}

}  // extern "C"
