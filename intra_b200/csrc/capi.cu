// Host side of libintra_b200: argument checks, per-pattern problem set-up and kernel launches
// behind the C ABI of include/intra_b200.h. Mirrors what the reference's ATen host code does
// (csrc/flash_attn/flash_api.cpp:355-552 `mha_fwd`, :556-763 `mha_fwd_llm`) without ATen: the caller
// owns every tensor, this file only validates, fills the parameter block and launches.
#include "../../include/intra_b200.h"

#include <cuda.h>
#include <cuda_runtime.h>

#include <cmath>
#include <cstdlib>
#include <mutex>
#include <vector>

#include "attn_kernel.cuh"
#include "attn_kernel_dual.cuh"
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

// One-time set-up of a device (current when called): architecture check, shared-memory opt-in of the
// kernels, and the status word the kernels report to.
void init_device(int device) {
  DeviceState& st = g_dev[device];
  cudaDeviceProp prop;
  cudaError_t e = cudaGetDeviceProperties(&prop, device);
  if (e != cudaSuccess) { st.init_status = cuda_fail(e); return; }
  if (prop.major != 10) { st.init_status = INTRA_ERR_DEVICE; return; }
  e = cudaFuncSetAttribute(intra_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FWD_SMEM_BYTES);
  if (e == cudaSuccess)
    e = cudaFuncSetAttribute(intra_fwd_kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                             cudaSharedmemCarveoutMaxShared);
  if (e == cudaSuccess)
    e = cudaFuncSetAttribute(umma_selftest_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FWD_SMEM_BYTES);
  if (e == cudaSuccess)
    e = cudaFuncSetAttribute(intra_fwd_dual_kernel<2, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, DUAL_SMEM_BYTES);
  if (e == cudaSuccess)
    e = cudaFuncSetAttribute(intra_fwd_dual_kernel<2, false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, DUAL_SMEM_BYTES);
  if (e == cudaSuccess)
    e = cudaFuncSetAttribute(intra_fwd_dual_kernel<4, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, DUAL_SMEM_BYTES);
  if (e == cudaSuccess)
    e = cudaFuncSetAttribute(intra_fwd_dual_kernel<4, false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, DUAL_SMEM_BYTES);
  if (e == cudaSuccess)
    e = cudaFuncSetAttribute(intra_fwd_dual_kernel<2, true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, DUAL_SMEM_BYTES);
  if (e == cudaSuccess)
    e = cudaFuncSetAttribute(intra_fwd_dual_kernel<2, true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, DUAL_SMEM_BYTES);
  if (e == cudaSuccess)
    e = cudaFuncSetAttribute(intra_fwd_dual_kernel<4, true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, DUAL_SMEM_BYTES);
  if (e == cudaSuccess)
    e = cudaFuncSetAttribute(intra_fwd_dual_kernel<4, true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, DUAL_SMEM_BYTES);
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
};
NoAllocState g_noalloc[MAX_DEVICES];

// Runs once per device with that device current. Allocates nothing.
void init_noalloc(int device) {
  NoAllocState& st = g_noalloc[device];
  int major = 0;
  cudaError_t e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device);
  if (e != cudaSuccess) { st.init_status = cuda_fail(e); return; }
  if (major != 10) { st.init_status = INTRA_ERR_DEVICE; return; }
  e = cudaFuncSetAttribute(intra_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FWD_SMEM_BYTES);
  if (e == cudaSuccess)
    e = cudaFuncSetAttribute(intra_fwd_kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                             cudaSharedmemCarveoutMaxShared);
  void* ptr = nullptr;
  if (e == cudaSuccess) e = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
  if (e != cudaSuccess) { st.init_status = cuda_fail(e); return; }
  st.scratch = static_cast<int*>(ptr);
}

// Bytes of scratch one launch of the attention kernel needs: its status word.
size_t fwd_scratch_bytes(const Problem&) { return sizeof(int); }

int launch_fwd(const void* q, const void* k, const void* v, void* out, int B, int S, int H, int Hkv,
               const int64_t* qs, const int64_t* ks, const int64_t* vs, const int64_t* os, int family, int pattern,
               int param, float softmax_scale, int device, void* stream, float* lse = nullptr) {
  if (!q || !k || !v || !out || B <= 0 || S <= 0 || H <= 0 || Hkv <= 0 || H % Hkv != 0) return INTRA_ERR_BAD_ARG;
  if (!qs || !ks || !vs || !os) return INTRA_ERR_BAD_ARG;
  if (!(softmax_scale > 0.f) || !std::isfinite(softmax_scale)) return INTRA_ERR_BAD_ARG;
  if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(out) || !strides_ok(qs) || !strides_ok(ks) ||
      !strides_ok(vs) || !strides_ok(os))
    return INTRA_ERR_ALIGNMENT;
  FwdParams p;
  int rc = problem_from(family, pattern, S, param, &p.prob);
  if (rc != INTRA_OK) return rc;
  const int64_t blocks = int64_t(p.prob.n_tiles) * B * H;
  if (blocks <= 0 || blocks > 0x7fffffffLL) return INTRA_ERR_UNSUPPORTED;

  DeviceGuard guard(device);
  if (!guard.ok) return cuda_fail(cudaGetLastError());
  rc = ensure_device(device);
  if (rc != INTRA_OK) return rc;

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
  p.status = g_dev[device].status_word;
  p.lse = lse;
  // Everything runs on the persistent two-sub-tile kernel (Gather-0, whose tiles share no keys, with one
  // K / V buffer per sub-tile); INTRA_B200_SINGLE_TILE=1 forces the one-tile kernel, for A/B runs.
  static const bool force_single = [] { const char* v = std::getenv("INTRA_B200_SINGLE_TILE"); return v && v[0] == '1'; }();
  if (!force_single) {
    DualParams d;
    d.f = p;
    d.split_kv = p.prob.kind == KIND_IMG_GATHER0 ? 1 : 0;
    d.row_pairs = (d.split_kv || (H / Hkv) % 2 != 0) ? 1 : 0;
    d.n_pair_tiles = n_pair_tiles(p.prob, d.row_pairs);
    d.heads_per_item = d.row_pairs ? H : H / 2;
    const int64_t items = int64_t(d.n_pair_tiles) * B * d.heads_per_item;
    if (items <= 0 || items > 0x7fffffffLL) return INTRA_ERR_UNSUPPORTED;
    d.n_items = static_cast<int>(items);
    static const bool no_tma = [] { const char* v = std::getenv("INTRA_B200_NO_TMA"); return v && v[0] == '1'; }();
    d.wide_stores = (reinterpret_cast<uintptr_t>(out) % 32 == 0 && os[0] % 16 == 0 && os[1] % 16 == 0 && os[2] % 16 == 0) ? 1 : 0;
    d.use_tma = !no_tma && tma_supported(p.prob) &&
                build_maps(p.prob, p.q, p.qs, H, B, true, &d.maps.q_main, &d.maps.q_text, &d.maps.k_aux) &&
                build_maps(p.prob, p.k, p.ks, Hkv, B, false, &d.maps.k_main, &d.maps.k_text, &d.maps.k_aux) &&
                build_maps(p.prob, p.v, p.vs, Hkv, B, false, &d.maps.v_main, &d.maps.v_text, &d.maps.v_aux);
    const int grid = static_cast<int>(items < g_dev[device].sm_count ? items : g_dev[device].sm_count);
    // Softmax column split (attn_kernel_dual.cuh): 4-way for short items, 2-way for long ones.
    int64_t n_tiles = 0, n_kv = 0;
    for (int idx = 0; idx < d.n_pair_tiles; ++idx) {
      const int t = make_pair(p.prob, d.row_pairs, idx).kv.n_kv_tiles;
      if (t > 0) { ++n_tiles; n_kv += t; }
    }
    static const int force_split = [] { const char* v = std::getenv("INTRA_B200_SOFTMAX_SPLIT"); return v ? std::atoi(v) : 0; }();
    const bool four = force_split ? force_split == 4 : (n_tiles > 0 && n_kv < 24 * n_tiles);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
#define INTRA_LAUNCH_DUAL(N, SPLIT) \
    do { \
      if (d.use_tma) intra_fwd_dual_kernel<N, SPLIT, true><<<grid, DualCfg<N>::THREADS, DUAL_SMEM_BYTES, st>>>(d); \
      else intra_fwd_dual_kernel<N, SPLIT, false><<<grid, DualCfg<N>::THREADS, DUAL_SMEM_BYTES, st>>>(d); \
    } while (0)
    if (four && d.split_kv) INTRA_LAUNCH_DUAL(4, true);
    else if (four) INTRA_LAUNCH_DUAL(4, false);
    else if (d.split_kv) INTRA_LAUNCH_DUAL(2, true);
    else INTRA_LAUNCH_DUAL(2, false);
#undef INTRA_LAUNCH_DUAL
  } else {
    intra_fwd_kernel<<<static_cast<unsigned>(blocks), FWD_THREADS, FWD_SMEM_BYTES, static_cast<cudaStream_t>(stream)>>>(p);
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e);
  return INTRA_OK;
}

}  // namespace

extern "C" {

int intra_b200_fwd_llm(const void* q, const void* k, const void* v, void* out, int B, int S, int H, int Hkv,
                       const int64_t q_strides[3], const int64_t k_strides[3], const int64_t v_strides[3],
                       const int64_t out_strides[3], int pattern, int group_num, int window, float softmax_scale,
                       int device, void* cuda_stream) {
  const int param = pattern == INTRA_LLM_WINDOW ? window : group_num;
  return launch_fwd(q, k, v, out, B, S, H, Hkv, q_strides, k_strides, v_strides, out_strides, 0, pattern, param,
                    softmax_scale, device, cuda_stream);
}

int intra_b200_fwd_image(const void* q, const void* k, const void* v, void* out, int B, int S, int H,
                         const int64_t q_strides[3], const int64_t k_strides[3], const int64_t v_strides[3],
                         const int64_t out_strides[3], int pattern, int width, float softmax_scale, int device,
                         void* cuda_stream) {
  return launch_fwd(q, k, v, out, B, S, H, H, q_strides, k_strides, v_strides, out_strides, 1, pattern, width,
                    softmax_scale, device, cuda_stream);
}

int intra_b200_fwd_llm_lse(const void* q, const void* k, const void* v, void* out, float* lse, int B, int S, int H,
                           int Hkv, const int64_t q_strides[3], const int64_t k_strides[3],
                           const int64_t v_strides[3], const int64_t out_strides[3], int pattern, int group_num,
                           int window, float softmax_scale, int device, void* cuda_stream) {
  if (!lse || reinterpret_cast<uintptr_t>(lse) % 4 != 0) return INTRA_ERR_BAD_ARG;
  const int param = pattern == INTRA_LLM_WINDOW ? window : group_num;
  return launch_fwd(q, k, v, out, B, S, H, Hkv, q_strides, k_strides, v_strides, out_strides, 0, pattern, param,
                    softmax_scale, device, cuda_stream, lse);
}

int intra_b200_fwd_image_lse(const void* q, const void* k, const void* v, void* out, float* lse, int B, int S, int H,
                             const int64_t q_strides[3], const int64_t k_strides[3], const int64_t v_strides[3],
                             const int64_t out_strides[3], int pattern, int width, float softmax_scale, int device,
                             void* cuda_stream) {
  if (!lse || reinterpret_cast<uintptr_t>(lse) % 4 != 0) return INTRA_ERR_BAD_ARG;
  return launch_fwd(q, k, v, out, B, S, H, H, q_strides, k_strides, v_strides, out_strides, 1, pattern, width,
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
  umma_selftest_kernel<<<1, 128, FWD_SMEM_BYTES, static_cast<cudaStream_t>(cuda_stream)>>>(
      static_cast<const __nv_bfloat16*>(a), static_cast<const __nv_bfloat16*>(b),
      static_cast<const __nv_bfloat16*>(v), p_scale, s_out, o_out, g_dev[device].status_word);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? INTRA_OK : cuda_fail(e);
}

int intra_b200_fwd_llm_noalloc(const void* q, const void* k, const void* v, void* out, int B, int S, int H, int Hkv,
                               const int64_t q_strides[3], const int64_t k_strides[3], const int64_t v_strides[3],
                               const int64_t out_strides[3], int pattern, int group_num, int window,
                               float softmax_scale, int device, void* cuda_stream, int* prev_status) {
  if (!q || !k || !v || !out || B <= 0 || S <= 0 || H <= 0 || Hkv <= 0 || H % Hkv != 0) return INTRA_ERR_BAD_ARG;
  if (!q_strides || !k_strides || !v_strides || !out_strides) return INTRA_ERR_BAD_ARG;
  if (!(softmax_scale > 0.f) || !std::isfinite(softmax_scale)) return INTRA_ERR_BAD_ARG;
  if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(out) || !strides_ok(q_strides) ||
      !strides_ok(k_strides) || !strides_ok(v_strides) || !strides_ok(out_strides))
    return INTRA_ERR_ALIGNMENT;
  if (device < 0 || device >= MAX_DEVICES) return INTRA_ERR_BAD_ARG;
  FwdParams p;
  int rc = problem_from(0, pattern, S, pattern == INTRA_LLM_WINDOW ? window : group_num, &p.prob);
  if (rc != INTRA_OK) return rc;
  const int64_t blocks = int64_t(p.prob.n_tiles) * B * H;
  if (blocks <= 0 || blocks > 0x7fffffffLL) return INTRA_ERR_UNSUPPORTED;
  // The launch's scratch has to fit the fixed array; a shape that needed more is turned away here.
  if (fwd_scratch_bytes(p.prob) > NOALLOC_SCRATCH_BYTES) return INTRA_ERR_UNSUPPORTED;

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

  p.q = static_cast<const __nv_bfloat16*>(q);
  p.k = static_cast<const __nv_bfloat16*>(k);
  p.v = static_cast<const __nv_bfloat16*>(v);
  p.o = static_cast<__nv_bfloat16*>(out);
  p.qs = {q_strides[0], q_strides[1], q_strides[2]};
  p.ks = {k_strides[0], k_strides[1], k_strides[2]};
  p.vs = {v_strides[0], v_strides[1], v_strides[2]};
  p.os = {out_strides[0], out_strides[1], out_strides[2]};
  p.B = B; p.H = H; p.Hkv = Hkv;
  p.scale_log2 = softmax_scale * 1.4426950408889634f;
  p.status = st.scratch;
  p.lse = nullptr;
  intra_fwd_kernel<<<static_cast<unsigned>(blocks), FWD_THREADS, FWD_SMEM_BYTES, stream>>>(p);
  e = cudaGetLastError();
  return e == cudaSuccess ? INTRA_OK : cuda_fail(e);
}

}  // extern "C"
