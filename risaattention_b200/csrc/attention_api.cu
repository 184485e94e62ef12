// C-ABI entry of the fused INT8 attention call: validation, kernel-family selection and the
// block-mass reduction that follows a capture pass.
#include "attention_common.cuh"
#include <cstdint>

namespace risa_b200 {
namespace {

// Kernel family the calling thread asked for (0 = automatic, 1 = row-per-thread kernel, 2 = the
// tensor-core kernel with every path compiled in); per thread, so that a parity check forcing a
// kernel cannot change what other threads of the process run.
thread_local int g_attention_path = 0;

// Block mass of (query block, key tile): sum over the block's queries of
// numerator * 2^(tile_max - m_final) / d_final.  One CTA per (query block, head, batch), thread =
// query; the sum uses the reference's tree (shfl_down inside each warp, then across the four warp
// sums; attention_int8.cuh:1067-1086) because the masses feed an exact selection.
__global__ __launch_bounds__(128) void block_mass_kernel(const AttentionArgs a, int n_q, int n_k) {
  __shared__ float warp_sums[4];
  const CaptureLayout cap = capture_layout(a, n_q, n_k);
  const int q_block = blockIdx.x, head = blockIdx.y, batch = blockIdx.z;
  const int row = q_block * 128 + threadIdx.x;
  const bool ok = row < a.q_len;
  const int64_t bh = int64_t(batch) * a.q_heads + head;
  const int64_t grow = bh * a.q_len + row;
  float m_final = 0.f, d_final = 0.f;
  if (ok) {
    m_final = cap.state[grow * 2];
    d_final = cap.state[grow * 2 + 1];
  }
  float* out = a.block_mass + (bh * n_q + q_block) * n_k;
  for (int t = 0; t < n_k; ++t) {
    float mass = 0.0f;
    if (ok) {
      float numer, tmax;
      if (t + 1 < n_k) {
        const uint32_t* slot = cap.full + (grow * (n_k - 1) + t) * 2;
        numer = __uint2float_rn(slot[0]);
        tmax = __uint_as_float(slot[1]);
      } else {
        numer = cap.last[grow * 2];
        tmax = cap.last[grow * 2 + 1];
      }
      mass = d_final > 0.0f ? numer * ex2_approx(tmax - m_final) / d_final : 0.0f;
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) mass += __shfl_down_sync(0xffffffffu, mass, off);
    __syncthreads();  // warp_sums of the previous tile consumed
    if ((threadIdx.x & 31) == 0) warp_sums[threadIdx.x >> 5] = mass;
    __syncthreads();
    if (threadIdx.x < 32) {
      float total = threadIdx.x < 4 ? warp_sums[threadIdx.x] : 0.0f;
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) total += __shfl_down_sync(0xffffffffu, total, off);
      if (threadIdx.x == 0) out[t] = total;
    }
  }
}

}  // namespace
}  // namespace risa_b200

using namespace risa_b200;

extern "C" int risa_b200_set_attention_path(int path) {
  const int previous = g_attention_path;
  g_attention_path = path == 1 || path == 2 ? path : 0;
  return previous;
}

namespace {

// Outputs and scratch of the in-pass pattern construction (risa_b200_attention_select).
struct SelectRequest {
  double theta;
  void* scratch;
  int slots;
  float* masses;
  int32_t* counts;
  uint32_t* bitmaps;
  double* totals;
};

int run_attention(
    const void* q, const void* k, const void* v, void* o, const float* q_scale,
    const float* k_scale, const float* v_scale, const float* v_center, const void* mask,
    int64_t mask_stride_b, int64_t mask_stride_h, int64_t mask_stride_q, int64_t mask_stride_k,
    int mask_dtype_code, int cta_k, int batch, int q_len, int k_len, int q_heads, int kv_heads,
    int head_dim, int64_t o_stride_b, int64_t o_stride_n, int64_t o_stride_h, float sm_scale,
    int out_dtype_code, const int32_t* sparse_row_offsets, const int32_t* sparse_block_indices,
    float* block_mass, int is_causal, float* lse, const int32_t* key_mask_tiles,
    void* stream_ptr, const SelectRequest* select, float* tail_scratch = nullptr,
    size_t tail_scratch_bytes = 0) {
  RISA_REQUIRE(cta_k == 64 || cta_k == 128, "risa_attention: cta_k must be 64 or 128");
  RISA_REQUIRE(head_dim == 64 || head_dim == 128 || head_dim == 256,
               "risa_attention: unsupported head_dim");
  RISA_REQUIRE(!(cta_k == 128 && head_dim == 64),
               "risa_attention: cta_k 128 requires head_dim 128 or 256");
  RISA_REQUIRE((sparse_row_offsets == nullptr) == (sparse_block_indices == nullptr),
               "risa_attention: sparse row offsets and block indices must be provided together");
  RISA_REQUIRE(!(block_mass && sparse_row_offsets),
               "risa_attention: block mass requires dense attention");
  RISA_REQUIRE(q && k && v && o && q_scale && k_scale && v_scale && v_center,
               "risa_attention: null tensor");
  RISA_REQUIRE(batch > 0 && q_len > 0 && k_len > 0 && q_heads > 0 && kv_heads > 0 &&
                   q_heads % kv_heads == 0,
               "risa_attention: sizes must be positive and q heads divisible by kv heads");
  RISA_REQUIRE(out_dtype_code == 1 || out_dtype_code == 2,
               "risa_attention: output_dtype_code must be 1 (fp16) or 2 (bf16)");
  RISA_REQUIRE(mask == nullptr || (mask_dtype_code >= 0 && mask_dtype_code <= 3),
               "risa_attention: attention mask must be bool, float16, bfloat16, or float32");
  RISA_REQUIRE(reinterpret_cast<uintptr_t>(q) % 16 == 0 && reinterpret_cast<uintptr_t>(k) % 16 == 0 &&
                   reinterpret_cast<uintptr_t>(v) % 16 == 0 && reinterpret_cast<uintptr_t>(o) % 4 == 0 &&
                   o_stride_b % 2 == 0 && o_stride_n % 2 == 0 && o_stride_h % 2 == 0,
               "risa_attention: packed operands must be 16-byte aligned and output strides even");
  AttentionArgs a{};
  a.pack_by256 = 256u;
  a.pack_by65536 = 65536u;
  a.q = static_cast<const int8_t*>(q);
  a.k = static_cast<const int8_t*>(k);
  a.v = static_cast<const int8_t*>(v);
  a.o = o;
  a.q_scale = q_scale;
  a.k_scale = k_scale;
  a.v_scale = v_scale;
  a.v_center = v_center;
  a.mask = mask;
  a.mask_stride_b = mask_stride_b;
  a.mask_stride_h = mask_stride_h;
  a.mask_stride_q = mask_stride_q;
  a.mask_stride_k = mask_stride_k;
  a.mask_dtype_code = mask_dtype_code;
  a.cta_k = cta_k;
  a.batch = batch;
  a.q_len = q_len;
  a.k_len = k_len;
  a.q_heads = q_heads;
  a.kv_heads = kv_heads;
  a.head_dim = head_dim;
  a.o_stride_b = o_stride_b;
  a.o_stride_n = o_stride_n;
  a.o_stride_h = o_stride_h;
  a.sm_scale = sm_scale;
  a.out_dtype_code = out_dtype_code;
  a.row_offsets = sparse_row_offsets;
  a.block_indices = sparse_block_indices;
  a.block_mass = block_mass;
  a.is_causal = is_causal != 0;
  a.lse = lse;
  a.tail_scratch = tail_scratch;  // room for the parts of a split last wave, or null
  a.tail_scratch_bytes = tail_scratch_bytes;
  a.key_mask_tiles = (mask != nullptr && mask_stride_q == 0 && !sparse_row_offsets &&
                      !block_mass && !is_causal)
                         ? key_mask_tiles
                         : nullptr;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  if (select) {
    RISA_REQUIRE(attention_tc_supported(a),
                 "attention_select: shape or alignment outside the tensor-core kernel");
    const int n_k = (k_len + cta_k - 1) / cta_k;
    RISA_REQUIRE(n_k <= attention_tc_select_max_tiles(cta_k),
                 "attention_select: at most %d key tiles of %d keys",
                 attention_tc_select_max_tiles(cta_k), cta_k);
    a.select_scratch = select->scratch;
    a.select_slots = select->slots;
    a.select_theta = select->theta;
    a.select_masses = select->masses;
    a.select_counts = select->counts;
    a.select_bitmaps = select->bitmaps;
    a.select_totals = select->totals;
    return attention_tc(a, stream, g_attention_path == 2);
  }
  int status;
  if (g_attention_path != 1 && attention_tc_supported(a))
    status = attention_tc(a, stream, g_attention_path == 2);
  else
    status = attention_rows(a, stream);
  if (status != RISA_B200_OK) return status;
  if (block_mass) {
    const int n_q = (q_len + 127) / 128, n_k = (k_len + cta_k - 1) / cta_k;
    block_mass_kernel<<<dim3(n_q, q_heads, batch), 128, 0, stream>>>(a, n_q, n_k);
    return check_launch("attention (block mass)");
  }
  return RISA_B200_OK;
}

// Slots of the selection scratch: one per CTA that can be resident at once (the kernel's shared
// memory allows one CTA per SM).
int select_slot_count() {
  static thread_local int cached_device = -1, cached = 0;
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess) return 0;
  if (device != cached_device) {
    int sms = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess)
      return 0;
    cached = sms;
    cached_device = device;
  }
  return cached;
}

size_t select_flag_bytes(int slots) { return (size_t(slots) * 4 + 255) / 256 * 256; }

}  // namespace

extern "C" int risa_b200_attention(
    const void* q, const void* k, const void* v, void* o, const float* q_scale,
    const float* k_scale, const float* v_scale, const float* v_center, const void* mask,
    int64_t mask_stride_b, int64_t mask_stride_h, int64_t mask_stride_q, int64_t mask_stride_k,
    int mask_dtype_code, int cta_k, int batch, int q_len, int k_len, int q_heads, int kv_heads,
    int head_dim, int64_t o_stride_b, int64_t o_stride_n, int64_t o_stride_h, float sm_scale,
    int out_dtype_code, const int32_t* sparse_row_offsets, const int32_t* sparse_block_indices,
    float* block_mass, int is_causal, float* lse, const int32_t* key_mask_tiles,
    void* stream_ptr) {
  return run_attention(q, k, v, o, q_scale, k_scale, v_scale, v_center, mask, mask_stride_b,
                       mask_stride_h, mask_stride_q, mask_stride_k, mask_dtype_code, cta_k, batch,
                       q_len, k_len, q_heads, kv_heads, head_dim, o_stride_b, o_stride_n,
                       o_stride_h, sm_scale, out_dtype_code, sparse_row_offsets,
                       sparse_block_indices, block_mass, is_causal, lse, key_mask_tiles, stream_ptr,
                       nullptr);
}

extern "C" int risa_b200_split_last_wave_parts(int ctas, int key_tiles, int cta_k, int sms) {
  return risa_b200::attention_tc_split_parts(ctas, key_tiles, cta_k, sms);
}

extern "C" size_t risa_b200_attention_scratch_size(int batch, int q_heads, int q_len, int k_len,
                                                   int head_dim, int cta_k) {
  if (batch <= 0 || q_heads <= 0 || q_len <= 0 || k_len <= 0 || (cta_k != 64 && cta_k != 128))
    return 0;
  const int halves = head_dim == 256 ? 2 : 1, sms = select_slot_count();
  const int64_t ctas = int64_t((q_len + 127) / 128) * q_heads * halves * batch;
  if (ctas > INT32_MAX || sms <= 0) return 0;
  const int parts =
      risa_b200::attention_tc_split_parts(int(ctas), (k_len + cta_k - 1) / cta_k, cta_k, sms);
  return size_t(ctas % sms) * parts * risa_b200::kTailPartBytes;
}

extern "C" int risa_b200_attention_scratch(
    const void* q, const void* k, const void* v, void* o, const float* q_scale,
    const float* k_scale, const float* v_scale, const float* v_center, const void* mask,
    int64_t mask_stride_b, int64_t mask_stride_h, int64_t mask_stride_q, int64_t mask_stride_k,
    int mask_dtype_code, int cta_k, int batch, int q_len, int k_len, int q_heads, int kv_heads,
    int head_dim, int64_t o_stride_b, int64_t o_stride_n, int64_t o_stride_h, float sm_scale,
    int out_dtype_code, const int32_t* sparse_row_offsets, const int32_t* sparse_block_indices,
    float* block_mass, int is_causal, float* lse, const int32_t* key_mask_tiles, void* scratch,
    size_t scratch_bytes, void* stream_ptr) {
  RISA_REQUIRE(scratch == nullptr || reinterpret_cast<uintptr_t>(scratch) % 16 == 0,
               "risa_attention: scratch must be 16-byte aligned device memory, or null");
  return run_attention(q, k, v, o, q_scale, k_scale, v_scale, v_center, mask, mask_stride_b,
                       mask_stride_h, mask_stride_q, mask_stride_k, mask_dtype_code, cta_k, batch,
                       q_len, k_len, q_heads, kv_heads, head_dim, o_stride_b, o_stride_n,
                       o_stride_h, sm_scale, out_dtype_code, sparse_row_offsets,
                       sparse_block_indices, block_mass, is_causal, lse, key_mask_tiles, stream_ptr,
                       nullptr, static_cast<float*>(scratch), scratch_bytes);
}

extern "C" size_t risa_b200_select_scratch_size(int k_len, int cta_k) {
  if (k_len <= 0 || (cta_k != 64 && cta_k != 128)) return 0;
  const int slots = select_slot_count();
  const size_t n_k = (size_t(k_len) + cta_k - 1) / cta_k;
  return slots == 0 ? 0 : select_flag_bytes(slots) + size_t(slots) * n_k * 128 * 8;
}

extern "C" int risa_b200_select_max_key_tiles(int cta_k) {
  return (cta_k == 64 || cta_k == 128) ? attention_tc_select_max_tiles(cta_k) : 0;
}

extern "C" int risa_b200_attention_select(
    const void* q, const void* k, const void* v, void* o, const float* q_scale,
    const float* k_scale, const float* v_scale, const float* v_center, const void* mask,
    int64_t mask_stride_b, int64_t mask_stride_h, int64_t mask_stride_q, int64_t mask_stride_k,
    int mask_dtype_code, int cta_k, int batch, int q_len, int k_len, int q_heads, int kv_heads,
    int head_dim, int64_t o_stride_b, int64_t o_stride_n, int64_t o_stride_h, float sm_scale,
    int out_dtype_code, int is_causal, double theta, void* scratch, size_t scratch_bytes,
    float* block_masses, int32_t* counts, uint32_t* bitmaps, double* row_totals,
    void* stream_ptr) {
  RISA_REQUIRE(theta > 0.0 && theta <= 1.0, "theta must be finite and in (0, 1]");
  RISA_REQUIRE(counts && bitmaps && row_totals, "attention_select: null output");
  const size_t need = risa_b200_select_scratch_size(k_len, cta_k);
  RISA_REQUIRE(need != 0 && scratch != nullptr && scratch_bytes >= need &&
                   reinterpret_cast<uintptr_t>(scratch) % 256 == 0,
               "attention_select: scratch must be 256-byte aligned device memory of at least "
               "risa_b200_select_scratch_size() = %zu bytes", need);
  const int slots = select_slot_count();
  // every slot starts unclaimed (stream-ordered; nothing else of the scratch needs a defined start)
  cudaError_t e = cudaMemsetAsync(scratch, 0, select_flag_bytes(slots),
                                  static_cast<cudaStream_t>(stream_ptr));
  if (e != cudaSuccess)
    return fail(RISA_B200_CUDA, "attention_select: cudaMemsetAsync: %s", cudaGetErrorString(e));
  const SelectRequest request{theta, scratch, slots, block_masses, counts, bitmaps, row_totals};
  return run_attention(q, k, v, o, q_scale, k_scale, v_scale, v_center, mask, mask_stride_b,
                       mask_stride_h, mask_stride_q, mask_stride_k, mask_dtype_code, cta_k, batch,
                       q_len, k_len, q_heads, kv_heads, head_dim, o_stride_b, o_stride_n,
                       o_stride_h, sm_scale, out_dtype_code, nullptr, nullptr, nullptr, is_causal,
                       nullptr, nullptr, stream_ptr, &request);
}

// ---- fused dense call: quantise into caller scratch, then attend --------------------------------
namespace {

struct DenseScratch {
  size_t q_codes, k_codes, v_codes, q_scale, k_scale, v_scale, v_center, anchors, v_work, tail,
      total;
};

constexpr size_t align256(size_t n) { return (n + 255) & ~size_t(255); }

DenseScratch dense_scratch_layout(int batch, int q_heads, int q_len, int kv_heads, int k_len,
                                  int head_dim, int cta_k) {
  const size_t n_q = (size_t(q_len) + 127) / 128, n_k = (size_t(k_len) + cta_k - 1) / cta_k;
  const size_t channels = size_t(batch) * kv_heads * head_dim;
  DenseScratch s;
  size_t at = 0;
  auto take = [&at](size_t bytes) { const size_t here = at; at += align256(bytes); return here; };
  s.q_codes = take(size_t(batch) * q_heads * q_len * head_dim);
  s.k_codes = take(size_t(batch) * kv_heads * k_len * head_dim);
  s.v_codes = take(channels * n_k * cta_k);
  s.q_scale = take(size_t(batch) * q_heads * n_q * (head_dim == 256 ? 64 : 32) * sizeof(float));
  s.k_scale = take(size_t(batch) * kv_heads * n_k * 4 * sizeof(float));
  s.v_scale = take(channels * sizeof(float));
  s.v_center = take(channels * sizeof(float));
  s.anchors = take(size_t(batch) * kv_heads * sizeof(int32_t));
  s.v_work = take(risa_b200_quantize_v_workspace_size(batch, kv_heads, k_len, head_dim));
  // parts of a split last wave (attention_tc.cu); nothing for shapes the rule leaves whole
  s.tail = take(risa_b200_attention_scratch_size(batch, q_heads, q_len, k_len, head_dim, cta_k));
  s.total = at;
  return s;
}

}  // namespace

extern "C" size_t risa_b200_dense_scratch_size(int batch, int q_heads, int q_len, int kv_heads,
                                               int k_len, int head_dim, int cta_k) {
  if (batch <= 0 || q_heads <= 0 || q_len <= 0 || kv_heads <= 0 || k_len <= 0 ||
      (cta_k != 64 && cta_k != 128) || (head_dim != 64 && head_dim != 128 && head_dim != 256))
    return 0;
  return dense_scratch_layout(batch, q_heads, q_len, kv_heads, k_len, head_dim, cta_k).total;
}

extern "C" int risa_b200_dense_attention(
    const void* q, const void* k, const void* v, void* o, void* scratch, size_t scratch_bytes,
    int batch, int q_heads, int q_len, int kv_heads, int k_len, int head_dim, int cta_k,
    int64_t q_stride_b, int64_t q_stride_h, int64_t q_stride_n, int64_t k_stride_b,
    int64_t k_stride_h, int64_t k_stride_n, int64_t v_stride_b, int64_t v_stride_h,
    int64_t v_stride_n, int dtype_code, int midpoint_affine, float sm_scale, int out_dtype_code,
    int64_t o_stride_b, int64_t o_stride_n, int64_t o_stride_h, int is_causal, void* stream) {
  using namespace risa_b200;
  const size_t need =
      risa_b200_dense_scratch_size(batch, q_heads, q_len, kv_heads, k_len, head_dim, cta_k);
  RISA_REQUIRE(need != 0, "risa_dense_attention: unsupported shape");
  RISA_REQUIRE(scratch != nullptr && scratch_bytes >= need &&
                   reinterpret_cast<uintptr_t>(scratch) % 256 == 0,
               "risa_dense_attention: scratch must be 256-byte aligned device memory of at least "
               "risa_b200_dense_scratch_size() bytes");
  const DenseScratch s =
      dense_scratch_layout(batch, q_heads, q_len, kv_heads, k_len, head_dim, cta_k);
  char* base = static_cast<char*>(scratch);
  const int padded = (k_len + cta_k - 1) / cta_k * cta_k;
  float* q_scale = reinterpret_cast<float*>(base + s.q_scale);
  float* k_scale = reinterpret_cast<float*>(base + s.k_scale);
  float* v_scale = reinterpret_cast<float*>(base + s.v_scale);
  float* v_center = reinterpret_cast<float*>(base + s.v_center);
  const int status = risa_b200_quantize_qkv(
      q, base + s.q_codes, q_scale, k, base + s.k_codes, k_scale, v, base + s.v_codes, v_scale,
      v_center, batch, q_heads, q_len, kv_heads, k_len, head_dim, cta_k, padded, q_stride_b,
      q_stride_h, q_stride_n, k_stride_b, k_stride_h, k_stride_n, v_stride_b, v_stride_h,
      v_stride_n, dtype_code, midpoint_affine, reinterpret_cast<int32_t*>(base + s.anchors),
      nullptr, nullptr, base + s.v_work, s.tail - s.v_work, stream);
  if (status != RISA_B200_OK) return status;
  return run_attention(base + s.q_codes, base + s.k_codes, base + s.v_codes, o, q_scale, k_scale,
                       v_scale, v_center, nullptr, 0, 0, 0, 0, -1, cta_k, batch, q_len, k_len,
                       q_heads, kv_heads, head_dim, o_stride_b, o_stride_n, o_stride_h, sm_scale,
                       out_dtype_code, nullptr, nullptr, nullptr, is_causal, nullptr, nullptr,
                       stream, nullptr, reinterpret_cast<float*>(base + s.tail), s.total - s.tail);
}
