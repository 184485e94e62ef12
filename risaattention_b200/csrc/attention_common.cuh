// Argument block, capture-workspace layout and per-element helpers shared by the attention kernels.
#pragma once
#include "softmax_row.cuh"

namespace risa_b200 {

struct AttentionArgs {
  const int8_t* q;
  const int8_t* k;
  const int8_t* v;
  void* o;
  const float* q_scale;
  const float* k_scale;
  const float* v_scale;
  const float* v_center;
  const void* mask;
  int64_t mask_stride_b, mask_stride_h, mask_stride_q, mask_stride_k;
  int mask_dtype_code;
  int cta_k, batch, q_len, k_len, q_heads, kv_heads, head_dim;
  int64_t o_stride_b, o_stride_n, o_stride_h;  // in elements
  float sm_scale;
  int out_dtype_code;  // 1 = fp16, 2 = bf16
  const int32_t* row_offsets;
  const int32_t* block_indices;
  float* block_mass;
  int is_causal;
  float* lse;
  const int32_t* key_mask_tiles;
  // In-pass pattern construction (tensor-core kernel only; all null / zero otherwise): the CTA keeps
  // its per-(query, tile) statistics in a slot of `select_scratch`, reduces them to block masses
  // after its last tile and closes the retained-mass prefix itself.
  void* select_scratch;      // [slots] int32 claim flags (256-byte aligned block), then the slots
  int select_slots;          // number of slots (>= CTAs resident at once)
  double select_theta;
  float* select_masses;      // optional [B*Hq*n_q, n_k] block masses
  int32_t* select_counts;    // [B*Hq*n_q] tiles kept per row
  uint32_t* select_bitmaps;  // [B*Hq*n_q, ceil(n_k / 32)] kept tiles as bits
  double* select_totals;     // [B*Hq*n_q, 2] kept mass, total mass
  // Key-range split of the last, partial wave of CTAs (tensor-core kernel, dense unmasked calls):
  // CTAs from linear index tail_begin on are replaced by tail_splits CTAs each, every one taking a
  // contiguous share of the key tiles and leaving its unnormalised output rows, maximum and
  // denominator in tail_scratch ([tail CTA][part][130][128] floats); a merge launch combines them.
  // tail_splits <= 1: off.
  int tail_begin, tail_splits;
  float* tail_scratch;
  size_t tail_scratch_bytes;  // what the caller provided (host side only)
  // 2^8 and 2^16 as run-time values for the multiply-add packing of probability codes
  // (softmax_row.cuh, MAD_PACK)
  uint32_t pack_by256, pack_by65536;
};

// One part of AttentionArgs::tail_scratch: 128 rows x (128 channels, maximum, denominator).
constexpr size_t kTailPartBytes = size_t(130) * 128 * sizeof(float);

// Capture workspace (FP32 words), identical to the reference's (attention_int8.cuh:58-60,
// 770-797, 871-895): block masses [B*Hq*n_q, n_k]; then for every query row and every visited tile
// but the last a pair (u32 probability sum, f32 tile maximum); then per row the last tile's pair
// (f32 sum, f32 maximum); then per row (final maximum, final denominator).
struct CaptureLayout {
  uint32_t* full;
  float* last;
  float* state;
};

__host__ __device__ inline CaptureLayout capture_layout(const AttentionArgs& a, int n_q, int n_k) {
  const int64_t rows = int64_t(a.batch) * a.q_heads * a.q_len;
  const int64_t masses = int64_t(a.batch) * a.q_heads * n_q * n_k;
  CaptureLayout c;
  c.full = reinterpret_cast<uint32_t*>(a.block_mass + masses);
  c.last = a.block_mass + masses + rows * (n_k - 1) * 2;
  c.state = c.last + rows * 2;
  return c;
}

#ifdef __CUDACC__
// Score of (row, key) after the attention mask: kept -> s + bias * log2(e); masked -> -inf.
// Boolean masks keep where true; additive masks keep where the bias is finite
// (reference attention_masks.cuh:45-89).
__device__ __forceinline__ float apply_mask(const AttentionArgs& a, int batch, int head, int row,
                                            int key, bool row_ok, float x, float sc) {
  bool keep = row_ok && key < a.k_len;
  float bias = 0.0f;
  if (keep) {
    const int64_t off = int64_t(batch) * a.mask_stride_b + int64_t(head) * a.mask_stride_h +
                        int64_t(row) * a.mask_stride_q + int64_t(key) * a.mask_stride_k;
    if (a.mask_dtype_code == 3) {
      keep = static_cast<const uint8_t*>(a.mask)[off] != 0;
    } else {
      if (a.mask_dtype_code == 0)
        bias = static_cast<const float*>(a.mask)[off];
      else if (a.mask_dtype_code == 1)
        bias = __half2float(static_cast<const __half*>(a.mask)[off]);
      else
        bias = __bfloat162float(static_cast<const __nv_bfloat16*>(a.mask)[off]);
      keep = isfinite(bias);
    }
  }
  if (!keep) return -INFINITY;
  // score * scale and + bias are separate roundings.  (The reference writes the same two steps and
  // leaves fusing them to its compiler, which decides differently per kernel instantiation; masked
  // outputs therefore agree with it to the last FP32 bit in most but not all configurations.)
  return __fadd_rn(__fmul_rn(x, sc), bias * kLog2e);
}

__device__ __forceinline__ void store_pair(void* p, float a, float b, int out_dtype_code) {
  if (out_dtype_code == 1) {
    *reinterpret_cast<__half2*>(p) = __floats2half2_rn(a, b);
  } else {
    *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(a, b);
  }
}
#endif

// Kernel families (defined in attention_rows.cu / attention_tc.cu).
int attention_rows(const AttentionArgs& a, cudaStream_t stream);
bool attention_tc_supported(const AttentionArgs& a);
// every_path: run the instantiation with all softmax paths compiled in instead of the one for the
// call's class (the results are the same bits; a diagnostic).
int attention_tc(const AttentionArgs& a, cudaStream_t stream, bool every_path = false);
int attention_tc_select_max_tiles(int cta_k);
// Parts per CTA of the last wave (0: whole CTAs) for a dense unmasked launch; attention_tc.cu.
int attention_tc_split_parts(int ctas, int n_k, int cta_k, int sms);

}  // namespace risa_b200
