/* C ABI of libintra_b200: INTRA forward sparse attention on NVIDIA B200 (sm_100a).
 *
 * Plain pointers and sizes only; no PyTorch or C++ types cross this boundary. Every function
 * returns an int status (0 = INTRA_OK, negative = rejected before anything was launched, see
 * intra_b200_strerror) and never throws. Launches are asynchronous on the given CUDA stream.
 *
 * Tensors are bf16 with head dim 128, addressed as (batch, token, head, 128) through three element
 * strides {batch, token, head}; the innermost stride is 1. Base pointers and all strides must keep
 * every 128-element row 16-byte aligned. q/out have H heads, k/v have Hkv heads, H % Hkv == 0.
 */
#ifndef INTRA_B200_H_
#define INTRA_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define INTRA_OK 0
#define INTRA_ERR_BAD_ARG (-1)      /* null pointer, non-positive size, H % Hkv != 0, bad scale */
#define INTRA_ERR_UNSUPPORTED (-2)  /* pattern id / group_num / window / width / seqlen combination */
#define INTRA_ERR_ALIGNMENT (-3)    /* a pointer or stride breaks the 16-byte row alignment */
#define INTRA_ERR_CUDA (-4)         /* a CUDA runtime call failed; see intra_b200_last_cuda_error */
#define INTRA_ERR_DEVICE (-5)       /* the device is not an sm_100 part */
#define INTRA_ERR_KERNEL (-6)       /* a kernel gave up on a bounded wait; see intra_b200_device_status */

/* Pattern ids, identical to the reference's (intra_attn/interface.py:12-13). */
#define INTRA_LLM_SCATTER 0
#define INTRA_LLM_GATHER1 1
#define INTRA_LLM_WINDOW 4
#define INTRA_IMAGE_SCATTER 0
#define INTRA_IMAGE_GATHER0 4

/* Causal prefill attention for language models; replaces the reference's `fwd_llm` binding
 * (csrc/flash_attn/flash_api.cpp:556-763, bound at :1769). `pattern` is INTRA_LLM_*:
 *   scatter: token i attends j <= i with j % group_num == i % group_num (any S, any group_num <= S)
 *   gather1: segments of group_num tokens, segment s in group s % group_num (any S, any group_num)
 *   window:  each 64-query block attends itself and the preceding window-64 tokens (window >= 64)
 * `window` is ignored by scatter/gather1, `group_num` by window. `out` must not alias q, k or v. */
int intra_b200_fwd_llm(const void* q, const void* k, const void* v, void* out,
                       int B, int S, int H, int Hkv,
                       const int64_t q_strides[3], const int64_t k_strides[3],
                       const int64_t v_strides[3], const int64_t out_strides[3],
                       int pattern, int group_num, int window, float softmax_scale,
                       int device, void* cuda_stream);

/* Bidirectional attention over 512 text tokens followed by a width x width image grid
 * (S == 512 + width * width, width a multiple of 8, >= 16); replaces the reference's `fwd` binding
 * (csrc/flash_attn/flash_api.cpp:355-552, bound at :1768). `pattern` is INTRA_IMAGE_*. */
int intra_b200_fwd_image(const void* q, const void* k, const void* v, void* out,
                         int B, int S, int H,
                         const int64_t q_strides[3], const int64_t k_strides[3],
                         const int64_t v_strides[3], const int64_t out_strides[3],
                         int pattern, int width, float softmax_scale,
                         int device, void* cuda_stream);

/* The two functions above with one more output: lse, (B, H, S) fp32 contiguous, lse[b][h][i] = the
 * natural log of sum_j exp(softmax_scale * q_i . k_j) over the keys j token i attends. It is what merging
 * partial attention results over disjoint key sets needs (split KV, ring attention). The reference's
 * bindings return this tensor as `softmax_lse` (csrc/flash_attn/flash_api.cpp:470, 551, 670) although its
 * INTRA kernels compute it and then drop it (csrc/flash_attn/src/flash_fwd_kernel.h:5675); here it is
 * written. `lse` must be 4-byte aligned device memory; every element is written. */
int intra_b200_fwd_llm_lse(const void* q, const void* k, const void* v, void* out, float* lse,
                           int B, int S, int H, int Hkv,
                           const int64_t q_strides[3], const int64_t k_strides[3],
                           const int64_t v_strides[3], const int64_t out_strides[3],
                           int pattern, int group_num, int window, float softmax_scale,
                           int device, void* cuda_stream);
int intra_b200_fwd_image_lse(const void* q, const void* k, const void* v, void* out, float* lse,
                             int B, int S, int H,
                             const int64_t q_strides[3], const int64_t k_strides[3],
                             const int64_t v_strides[3], const int64_t out_strides[3],
                             int pattern, int width, float softmax_scale,
                             int device, void* cuda_stream);

/* Text for a status code; replaces the reference's TORCH_CHECK messages
 * (csrc/flash_attn/flash_api.cpp:377-394, 576-597). */
const char* intra_b200_strerror(int status);

/* cudaError_t of the most recent failed CUDA call made by this library on the calling thread
 * (0 if none); the counterpart of C10_CUDA_KERNEL_LAUNCH_CHECK
 * (csrc/flash_attn/src/flash_fwd_launch_template.h:516). */
int intra_b200_last_cuda_error(void);

/* Synchronises `device` and reads the word its kernels write when a bounded wait runs out
 * (0 = no kernel has given up since the last reset). `reset` != 0 clears it afterwards. Returns
 * INTRA_ERR_KERNEL when the word is non-zero. The word keeps the FIRST failure (100 + the id of the
 * wait site) until it is reset; kernels only ever write it, so a recorded failure does not change what
 * later launches do: they run normally, and their outputs are valid if the word is still unchanged
 * after them. The launch whose kernel gave up left some output rows unwritten. The entry points do
 * not poll the word (that would need a host synchronisation per call); a caller that wants to know
 * calls this function, e.g. once per step. It covers the regular entry points only:
 * intra_b200_fwd_llm_noalloc reports through its own `prev_status` argument. No counterpart in the
 * reference, whose kernels have no waits that can fail. */
int intra_b200_device_status(int device, int* status_word, int reset);

/* For the multi-GPU launcher (no counterpart in the reference, which runs on one GPU): reorders the
 * result of an all-gather of head-sharded outputs, parts[world][rows][block_bytes] (rank-major), into
 * out[rows][world][block_bytes], i.e. (batch, token, head, 128) order with rows = batch * tokens and
 * block_bytes = heads per rank * 256. Device pointers, 16-byte aligned; block_bytes a multiple of 16;
 * parts and out must not overlap. Asynchronous on `cuda_stream`. */
int intra_b200_interleave_heads(const void* parts, void* out, int world, int64_t rows, int64_t block_bytes,
                                int device, void* cuda_stream);

/* Test hooks (the reference has no counterpart): the (query, key) pairs the index maps visit.
 * `family` 0 = llm, 1 = image; `param` = group_num (scatter, gather1), window, or width.
 * counts is S*S bytes; counts[q*S + k] is incremented once per visit. The host variant evaluates
 * the maps on the CPU into host memory; the device variant evaluates them in a kernel into device
 * memory that the caller has zeroed. */
int intra_b200_visited_host(int family, int pattern, int S, int param, uint8_t* counts);
int intra_b200_visited_device(int family, int pattern, int S, int param, uint8_t* counts_dev,
                              int device, void* cuda_stream);
/* Same as intra_b200_visited_host for the decomposition into pairs of row tiles that share their
 * key tiles (used when the query heads of a KV group cannot be paired) or, for Gather-0, pairs of
 * equally long tiles that keep their own key lists. */
int intra_b200_visited_pairs_host(int family, int pattern, int S, int param, uint8_t* counts);

/* Test hook: number of tiles (CTAs per batch and head) and key tiles summed over them, i.e. the
 * tensor-core work the launch does in units of 128 x 128 score tiles. */
int intra_b200_tile_counts(int family, int pattern, int S, int param, int64_t* n_tiles, int64_t* n_kv_tiles);

/* Test hook: one 128x128x128 tile through both tensor-core contractions with the attention
 * kernel's operand layouts. a, b, v: device [128][128] bf16; s_out = a b^T and
 * o_out = bf16(s_out * p_scale) v, device [128][128] fp32. */
int intra_b200_selftest_umma(const void* a, const void* b, const void* v, float p_scale,
                             float* s_out, float* o_out, int device, void* cuda_stream);

/* Test hook: fetches every query tile and every key / value tile of a problem through the attention
 * kernel's own TMA planning and load code (the counterpart of the reference's per-thread gather
 * loaders, csrc/flash_attn/src/gmem_tile.h:270-1426) and reports which token row landed in which
 * shared-memory row. q, k, v are device tensors as for the forward call whose rows encode their token
 * id: elements 0..5 and 64..69 of token t's row hold (t + 1) % 256, (t + 1) / 256 % 256, (t + 1) / 65536,
 * the head, the batch, and 0 / 1 / 2 for q / k / v.
 * Call once with the five array pointers NULL to learn the sizes: *n_items items and *max_kv key tiles
 * per item at most. Then pass device arrays q_got (n_items*2*128 int32), k_got and v_got
 * (n_items*2*max_kv*128 int32 each) and host arrays q_want, k_want of the same sizes: the kernel
 * writes the token ids it found (-1: a zero row, -2: the two halves of a row disagree, -4: wrong head
 * or batch, -5: wrong tensor), the host side
 * the ids the index maps of intra_index.h prescribe (-9: the row is never used). Returns
 * INTRA_ERR_UNSUPPORTED for shapes the TMA path does not take, INTRA_ERR_KERNEL if a query row's key
 * interval reaches a slot without a key. */
int intra_b200_test_tma_rows(const void* q, const void* k, const void* v, int B, int S, int H, int Hkv,
                             const int64_t q_strides[3], const int64_t k_strides[3],
                             const int64_t v_strides[3], int family, int pattern, int param,
                             int32_t* q_got_dev, int32_t* k_got_dev, int32_t* v_got_dev,
                             int32_t* q_want, int32_t* k_want, int64_t* n_items, int64_t* max_kv,
                             int device, void* cuda_stream);

/* Test hook: overrides the launcher's choice of kernel variant for all later launches of the process:
 * no_tma != 0 forces the cp.async row gathers; softmax_split 1 forces the row-owner form (patterns
 * with split key lists, i.e. Gather-0, get the 2-way split instead), 2 or 4 that column split;
 * (0, 0) restores the launcher's own choice. Replaces nothing in the reference. */
int intra_b200_test_force_path(int no_tma, int softmax_split);

/* Test hook, host arithmetic only (no GPU needed): which form of the attention kernel the launcher
 * picks for a problem: 1 = row-owner form (items of at least 8 key tiles on average that share their
 * key tiles), 4 = 4-way column split (shorter items), 2 = 2-way split (long items with split key
 * lists); a negative status for arguments the entry points would refuse. The counterpart of the
 * reference's MASK_SWITCH / launch-template choice (flash_fwd_launch_template.h:401-565). */
int intra_b200_test_kernel_form(int family, int pattern, int S, int param, int H, int Hkv);

/* Test hooks for the failure path (the reference has none). _poke_status synchronises the device and
 * overwrites its status word from the host. _wait_timeout launches a two-warp kernel in which one
 * warp's wait is never satisfied and runs out after limit_ms (1..1000); it returns normally, leaves
 * 100 + 92 in the status word, and writes to *waited_ns_dev how long the OTHER warp, whose own limit
 * is the attention kernel's two seconds, waited before the first warp's give-up released it. */
int intra_b200_test_poke_status(int device, int value);
int intra_b200_test_wait_timeout(int limit_ms, long long* waited_ns_dev, int device, void* cuda_stream);

/* intra_b200_fwd_llm for hosts that cannot let a library allocate device memory. It has no
 * counterpart in the reference.
 *
 * Who needs it: a serving engine or trainer that reserves (nearly) all of HBM for its own arena at
 * start-up leaves nothing for a cudaMalloc made later from inside a library, and a latency-bound
 * serving thread cannot afford the device-wide synchronisation a cudaMalloc implies. The regular
 * entry points allocate once per device (a status word the kernel reports to); this one never calls
 * cudaMalloc, cudaFree or any other allocating routine, and runs the same kernel. The caller still
 * passes q, k, v and out.
 *
 * The kernel's scratch - today that one status word - lives in a fixed 256-byte array that is part of
 * the library image, so every GPU that loads the library carries those 256 bytes until the process
 * exits. A launch whose scratch would not fit in the array is refused with INTRA_ERR_UNSUPPORTED;
 * with the present kernel the scratch does not grow with the problem, so no attention shape is
 * refused for that reason. All other argument rules and status codes are those of
 * intra_b200_fwd_llm.
 *
 * The first call on a device looks up the array's device address (with that device made current)
 * and opts the kernels into their shared-memory size; make that first call before any stream capture.
 * Every call on a device shares the array: the call clears the status word on `cuda_stream` before
 * its launch, so calls whose GPU work overlaps (different streams, or threads racing on one device)
 * race on that word - serialise them on one stream. The array keeps what the last call left, and that
 * is the only way to learn whether a call's kernel gave up: pass a non-null `prev_status` to have the
 * NEXT call first synchronise `cuda_stream` and copy out the word the previous call left (0 = healthy,
 * also before the first call); with NULL the call stays asynchronous and the previous call's word is
 * cleared unread. `prev_status` is written only when the arguments pass validation; on an argument
 * error it is left untouched. intra_b200_device_status does not see this array (and would allocate). */
int intra_b200_fwd_llm_noalloc(const void* q, const void* k, const void* v, void* out,
                               int B, int S, int H, int Hkv,
                               const int64_t q_strides[3], const int64_t k_strides[3],
                               const int64_t v_strides[3], const int64_t out_strides[3],
                               int pattern, int group_num, int window, float softmax_scale,
                               int device, void* cuda_stream, int* prev_status);

#ifdef __cplusplus
}
#endif
#endif /* INTRA_B200_H_ */
