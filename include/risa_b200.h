/*
 * C-ABI of the B200-native RISA quantised-attention library (librisa_b200.so).
 *
 * Every entry point takes plain pointers to DEVICE memory, sizes, element strides and the
 * caller's CUDA stream (as void*), enqueues work on that stream without synchronising the host,
 * allocates nothing unless stated, and returns 0 on success or a non-zero status whose text is
 * available from risa_b200_last_error() (thread-local).  The reference project's own launchers
 * throw C++ exceptions through their extern "C" signatures; a status code is what a cgo / JNI /
 * ctypes / nanobind caller can actually consume.
 *
 * Each declaration names the reference interface it replaces (path inside the reference project).
 * Data layouts are the reference's public packed formats:
 *   q/k codes  int8 [B,H,L,D] contiguous, D in {64,128,256}
 *   q scales   f32  [B,Hq,ceil(Lq/128)*(D==256?64:32)],  k scales f32 [B,Hkv,ceil(Lk/cta_k)*4]
 *   v codes    int8 [B*Hkv*D, padded_Lk] with the 16-token storage order
 *              {0,1,8,9,2,3,10,11,4,5,12,13,6,7,14,15}, v scale / centre f32 [B*Hkv*D]
 * dtype codes: 0 = float32, 1 = float16, 2 = bfloat16, 3 = bool (masks only).
 */
#ifndef RISA_B200_H
#define RISA_B200_H
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define RISA_B200_OK 0
#define RISA_B200_INVALID 1 /* contract violation: shapes, strides, alignment, null pointers */
#define RISA_B200_CUDA 2    /* CUDA runtime / launch error                                     */
#define RISA_B200_DEVICE 3  /* kernel reported a device-side failure (bounded wait ran out)    */

/* Text of the last failure on the calling thread ("" if none). */
const char* risa_b200_last_error(void);
/* Library ABI version; bumped when a signature changes. */
int risa_b200_abi_version(void);

/* K anchor detection + rotation + INT8 quantisation of Q and K.
 * Replaces launch_quantize_qk / launch_quantize_qk_gather (csrc/launchers.h:14-31; kernels
 * csrc/kernels/quantize_qk_impl.cuh:442-826).  q_perm / k_perm: optional int32 [B,H,L] gather
 * tables (NULL = identity), the reference's risa::QuantInput.  anchors: int32 [B,Hkv] scratch that
 * receives the chosen anchor row (or -1). */
int risa_b200_quantize_qk(const void* q, void* q_codes, float* q_scale, const void* k,
                          void* k_codes, float* k_scale, int batch, int q_heads, int q_len,
                          int kv_heads, int k_len, int head_dim, int cta_k, int64_t q_stride_b,
                          int64_t q_stride_h, int64_t q_stride_n, int64_t k_stride_b,
                          int64_t k_stride_h, int64_t k_stride_n, int dtype_code, int32_t* anchors,
                          const int32_t* q_perm, const int32_t* k_perm, void* stream);

/* Per-channel INT8 quantisation of V (absmax or residual-corrected midpoint-affine) into the
 * transposed, token-permuted packed layout.  Replaces launch_quantize_v / launch_quantize_v_gather
 * (csrc/launchers.h:33-43; kernel csrc/kernels/quantize_v_impl.cuh:83-409).  workspace: device
 * scratch of at least risa_b200_quantize_v_workspace_size() bytes (the reference kernel needs
 * none because it uses one CTA per 8 channels; this one spreads a channel over many CTAs). */
size_t risa_b200_quantize_v_workspace_size(int batch, int kv_heads, int k_len, int head_dim);
int risa_b200_quantize_v(const void* v, void* v_codes, float* v_scale, float* v_center, int batch,
                         int kv_heads, int k_len, int head_dim, int padded_len, int64_t stride_b,
                         int64_t stride_h, int64_t stride_n, int dtype_code, int midpoint_affine,
                         const int32_t* perm, void* workspace, size_t workspace_bytes,
                         void* stream);

/* Q, K and V of one call: what the reference's binding risa_sdpa_quantize does with its two
 * launcher calls (csrc/bindings.cpp:195-272: launch_quantize_qk[_gather] then launch_quantize_v[_gather]).
 * Same results as risa_b200_quantize_qk followed by risa_b200_quantize_v with the same arguments
 * (kv_perm is the gather table of both K and V) in two launches: the steps that depend on nothing
 * (K anchor detection, V range pass, Q quantiser), then the steps that depend on those (K quantiser,
 * V code pass; key lengths that are not a multiple of 16 keep a separate V launch). */
int risa_b200_quantize_qkv(const void* q, void* q_codes, float* q_scale, const void* k,
                           void* k_codes, float* k_scale, const void* v, void* v_codes,
                           float* v_scale, float* v_center, int batch, int q_heads, int q_len,
                           int kv_heads, int k_len, int head_dim, int cta_k, int padded_len,
                           int64_t q_stride_b, int64_t q_stride_h, int64_t q_stride_n,
                           int64_t k_stride_b, int64_t k_stride_h, int64_t k_stride_n,
                           int64_t v_stride_b, int64_t v_stride_h, int64_t v_stride_n,
                           int dtype_code, int midpoint_affine, int32_t* anchors,
                           const int32_t* q_perm, const int32_t* kv_perm, void* workspace,
                           size_t workspace_bytes, void* stream);

/* The rule by which dense unmasked calls cut the CTAs of their last, partial wave into key-range
 * parts: number of parts per CTA (2..4), or 0 when a launch of `ctas` CTAs (query blocks x heads x
 * batch, x 2 for head_dim 256) over `key_tiles` tiles of `cta_k` keys on a GPU with `sms` SMs runs
 * whole CTAs only.  R = ctas mod sms CTAs in p parts each take ceil(R * p / sms) rounds of 1 / p of
 * a CTA's time; the best p is taken if it saves at least a fifth of a CTA's time and 2048 keys.  A
 * non-zero answer means one more launch (the merge).  Pure function; no counterpart in the
 * reference. */
int risa_b200_split_last_wave_parts(int ctas, int key_tiles, int cta_k, int sms);

/* V quantisation for callers that must not allocate.  Some users of this library cannot obtain
 * device memory at call time: a serving process that fixes its memory budget at start-up and
 * forbids cudaMalloc afterwards (it stalls every stream of the device and can fail once memory is
 * fragmented), or a host runtime bound through cgo / JNI / ctypes that owns no device allocator at
 * all.  For them the scratch of risa_b200_quantize_v lives inside the library, in a fixed device
 * array of risa_b200_quantize_v_static_limit() bytes (4 MiB) that every GPU loading the library
 * keeps until the process exits.  The caller passes inputs and outputs only; the call allocates
 * nothing and frees nothing.  Problems whose risa_b200_quantize_v_workspace_size() exceeds the limit
 * are refused with RISA_B200_INVALID (B*Hkv*D = 512 channels at 32768 keys need 1.25 MiB).
 * The first call on each device looks up the array's device address (with that device current);
 * make that first call before any stream capture starts.  All calls on a device share the one
 * array: it keeps the previous call's contents (nothing needs clearing, every word read is written
 * earlier in the same call), and two calls that overlap on the GPU -- different streams without
 * ordering -- race on it.  Results are identical to risa_b200_quantize_v.  No counterpart in the
 * reference, whose V kernel needs no scratch. */
size_t risa_b200_quantize_v_static_limit(void);
int risa_b200_quantize_v_static(const void* v, void* v_codes, float* v_scale, float* v_center,
                                int batch, int kv_heads, int k_len, int head_dim, int padded_len,
                                int64_t stride_b, int64_t stride_h, int64_t stride_n,
                                int dtype_code, int midpoint_affine, const int32_t* perm,
                                void* stream);

/* Fused INT8 attention over packed operands: dense, masked, causal, CSR sparse reuse, block-mass
 * capture, optional LSE.  Replaces launch_attention (csrc/launchers.h:49-60; kernels
 * csrc/kernels/attention_int8.cuh:145-1088, attention_dispatch.cu:113-296).  Same argument
 * meaning; block_mass is the reference's capture workspace (masses, per-tile statistics, final
 * softmax state) in the same layout. */
int risa_b200_attention(const void* q, const void* k, const void* v, void* o, const float* q_scale,
                        const float* k_scale, const float* v_scale, const float* v_center,
                        const void* mask, int64_t mask_stride_b, int64_t mask_stride_h,
                        int64_t mask_stride_q, int64_t mask_stride_k, int mask_dtype_code,
                        int cta_k, int batch, int q_len, int k_len, int q_heads, int kv_heads,
                        int head_dim, int64_t o_stride_b, int64_t o_stride_n, int64_t o_stride_h,
                        float sm_scale, int out_dtype_code, const int32_t* sparse_row_offsets,
                        const int32_t* sparse_block_indices, float* block_mass, int is_causal,
                        float* lse, const int32_t* key_mask_tiles, void* stream);

/* risa_b200_attention with room for the split last wave (see risa_b200_split_last_wave_parts): a
 * dense, unmasked, non-causal call without tile lists may leave key-range parts of its last CTAs
 * in `scratch` (16-byte aligned) and finish them with a merge launch; every other call, and
 * scratch == NULL, behaves exactly as risa_b200_attention.  risa_b200_attention_scratch_size()
 * gives the bytes to provide for a shape on the current device, 0 when the shape would not be
 * split there.  Outputs of split rows can differ from the unsplit ones by FP32 summation order. */
size_t risa_b200_attention_scratch_size(int batch, int q_heads, int q_len, int k_len, int head_dim,
                                        int cta_k);
int risa_b200_attention_scratch(const void* q, const void* k, const void* v, void* o,
                                const float* q_scale, const float* k_scale, const float* v_scale,
                                const float* v_center, const void* mask, int64_t mask_stride_b,
                                int64_t mask_stride_h, int64_t mask_stride_q, int64_t mask_stride_k,
                                int mask_dtype_code, int cta_k, int batch, int q_len, int k_len,
                                int q_heads, int kv_heads, int head_dim, int64_t o_stride_b,
                                int64_t o_stride_n, int64_t o_stride_h, float sm_scale,
                                int out_dtype_code, const int32_t* sparse_row_offsets,
                                const int32_t* sparse_block_indices, float* block_mass,
                                int is_causal, float* lse, const int32_t* key_mask_tiles,
                                void* scratch, size_t scratch_bytes, void* stream);

/* Pattern construction inside the dense pass.  Same attention as risa_b200_attention with a
 * block-mass workspace (same outputs, bit for bit), but instead of writing 8 bytes per (query, key
 * tile) to a workspace of the reference's layout, sorting the block masses with a library sort and
 * running a separate selection kernel, every CTA keeps the statistics of its 128 queries in a slot
 * of `scratch` (one slot per CTA resident at once: 148 x n_k KiB instead of B*Hq*Lq*(2 n_k + 2)
 * floats), reduces them to the block masses of its query block after its last key tile, orders
 * them (descending, equal masses by ascending tile id) and closes the retained-mass prefix at
 * `theta` in the reference's FP64 order.  Replaces, as one launch: launch_attention in capture mode
 * + the block-mass kernel (csrc/kernels/attention_int8.cuh:51-143,1028-1088), torch.sort and
 * stage 1 of launch_select_retained_mass (src/risa_attention/sparse.py:18-52,
 * csrc/kernels/sparse_selection.cu:9-67).  Outputs per CSR row r = (batch, head, query block):
 * counts[r] kept tiles, bitmaps[r, ceil(n_k/32)] kept tiles as bits, row_totals[r, 2] = kept and
 * total mass (doubles); block_masses (optional, may be NULL) = f32 [rows, n_k].
 * risa_b200_pack_selected then turns counts + bitmaps into CSR row offsets and ascending tile ids
 * and writes summary = {kept mass, total mass, kept tiles} (stages 2-3 of the reference selector,
 * sparse_selection.cu:69-127).  Limits: tensor-core kernel shapes only, n_k <=
 * risa_b200_select_max_key_tiles(cta_k); scratch 256-byte aligned, at least
 * risa_b200_select_scratch_size() bytes; its slot flags are cleared on `stream` by the call. */
size_t risa_b200_select_scratch_size(int k_len, int cta_k);
int risa_b200_select_max_key_tiles(int cta_k);
int risa_b200_attention_select(const void* q, const void* k, const void* v, void* o,
                               const float* q_scale, const float* k_scale, const float* v_scale,
                               const float* v_center, const void* mask, int64_t mask_stride_b,
                               int64_t mask_stride_h, int64_t mask_stride_q, int64_t mask_stride_k,
                               int mask_dtype_code, int cta_k, int batch, int q_len, int k_len,
                               int q_heads, int kv_heads, int head_dim, int64_t o_stride_b,
                               int64_t o_stride_n, int64_t o_stride_h, float sm_scale,
                               int out_dtype_code, int is_causal, double theta, void* scratch,
                               size_t scratch_bytes, float* block_masses, int32_t* counts,
                               uint32_t* bitmaps, double* row_totals, void* stream);
int risa_b200_pack_selected(const int32_t* counts, const uint32_t* bitmaps,
                            const double* row_totals, int32_t* row_offsets, int32_t* block_indices,
                            double* summary, int row_count, int key_blocks, void* stream);

/* One call for the unmasked dense path: quantise Q, K and V into caller-provided scratch and run
 * the attention kernel on it.  Same kernels, same results as risa_b200_quantize_qk +
 * risa_b200_quantize_v + risa_b200_attention issued one after the other on `stream`; it exists so a
 * host runtime pays one foreign-function call and one scratch allocation per attention call instead
 * of three calls and nine buffers, which is what bounds short sequences.  The reference's FFI has no
 * fused entry point (csrc/bindings.cpp:195-461 exposes the two steps separately); its Python
 * execute_dense_attention (src/risa_attention/_execution.py:28-66) is the caller this serves.
 * scratch: device memory of at least risa_b200_dense_scratch_size() bytes, 256-byte aligned. */
size_t risa_b200_dense_scratch_size(int batch, int q_heads, int q_len, int kv_heads, int k_len,
                                    int head_dim, int cta_k);
int risa_b200_dense_attention(const void* q, const void* k, const void* v, void* o, void* scratch,
                              size_t scratch_bytes, int batch, int q_heads, int q_len,
                              int kv_heads, int k_len, int head_dim, int cta_k,
                              int64_t q_stride_b, int64_t q_stride_h, int64_t q_stride_n,
                              int64_t k_stride_b, int64_t k_stride_h, int64_t k_stride_n,
                              int64_t v_stride_b, int64_t v_stride_h, int64_t v_stride_n,
                              int dtype_code, int midpoint_affine, float sm_scale,
                              int out_dtype_code, int64_t o_stride_b, int64_t o_stride_n,
                              int64_t o_stride_h, int is_causal, void* stream);

/* Selects which attention kernel family calls made BY THE CALLING THREAD may use: 0 = automatic
 * (tensor-core kernel where it applies, in the instantiation for the call's class: no mask / causal
 * / boolean rows / other per-query masks / masks broadcast over queries), 1 = force the
 * row-per-thread integer kernel, whose FP32 operation order equals the reference's (the on-device
 * cross-check of the tensor-core kernel), 2 = the tensor-core kernel with every softmax path
 * compiled in, whose bits the class-specific instantiations must reproduce (a diagnostic).
 * Thread-local: other threads of the process are not affected.  Returns the previous value. */
int risa_b200_set_attention_path(int path);

/* Reads (and clears) the device status word of the tensor-core attention kernel.  Every wait inside
 * that kernel is bounded; if one expires the CTA records where, writes NaN into the output rows
 * (and LSE entries) it owns, drains and exits, and this call returns RISA_B200_DEVICE with the site
 * in risa_b200_last_error().  The record is per process and only reports: later launches are not
 * affected by an earlier expiry.  Synchronises the device.  No counterpart in the reference, whose
 * kernels have no waits that can expire. */
int risa_b200_device_status(void);

/* Health check of the bounded-wait machinery on this GPU and driver: one warp waits, for at most
 * limit_ns nanoseconds (0 < limit_ns <= 1e9), on a barrier that nothing ever completes, then
 * returns.  Afterwards risa_b200_device_status() reports RISA_B200_DEVICE with site 900 and the
 * context stays usable.  Nothing faults, traps or spins past the limit.  No counterpart in the
 * reference. */
int risa_b200_bounded_wait_self_test(uint64_t limit_ns, void* stream);

/* Retained-mass prefix selection over descending-sorted block masses and CSR packing.  Replaces
 * launch_select_retained_mass + retained_mass_selector_workspace_size (csrc/launchers.h:61-67;
 * csrc/kernels/sparse_selection.cu:9-159).  summary receives {selected mass, total mass, number of
 * selected blocks} as doubles. */
size_t risa_b200_selector_workspace_size(int row_count);
int risa_b200_select_retained_mass(const float* sorted_mass, const int64_t* descending_indices,
                                   int32_t* counts, uint8_t* support, double* row_totals,
                                   int32_t* row_offsets, int32_t* block_indices, double* summary,
                                   void* scan_workspace, size_t scan_workspace_bytes,
                                   int row_count, int key_blocks, double theta, void* stream);

/* Visible-tile list of a mask broadcast over queries.  Replaces launch_prepare_key_mask_tiles
 * (csrc/launchers.h:45-48; csrc/kernels/key_mask_tiles.cu:10-61). */
int risa_b200_prepare_key_mask_tiles(const void* mask, int32_t* tiles, int batch, int q_heads,
                                     int k_len, int tile_size, int64_t stride_b, int64_t stride_h,
                                     int64_t stride_k, int dtype_code, void* stream);

/* Row-wise logit shift scale * <q_i, k_anchor> removed by the K anchor translation.  Replaces
 * launch_correct_lse (csrc/launchers.h:9-13; csrc/kernels/lse_correction.cu:4-44). */
int risa_b200_correct_lse(const void* q, const void* k, const int32_t* anchors, float* out,
                          int batch, int q_heads, int kv_heads, int q_len, int head_dim,
                          int64_t q_stride_b, int64_t q_stride_h, int64_t q_stride_n,
                          int64_t k_stride_b, int64_t k_stride_h, int64_t k_stride_n, float scale,
                          int dtype_code, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* RISA_B200_H */
