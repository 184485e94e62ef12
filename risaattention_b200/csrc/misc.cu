// Small kernels around the attention call: LSE shift of the K anchor, visible-tile lists of
// broadcast key masks, retained-mass selection with CSR packing, plus the library's error text.
#include "common.cuh"
#include "select.cuh"

namespace risa_b200 {

char* error_buffer() {
  static thread_local char buffer[512] = {0};
  return buffer;
}

namespace {

// ---- LSE shift: out[b,h,i] = scale * <q_i, k_anchor>, 0 when the head has no anchor -----------
// The K anchor translation removes scale * <q_i, k_anchor> from every logit of row i; this puts it
// back into the LSE.  A CTA covers kShiftRows query rows of one (batch, head): the anchor key row
// is converted to FP32 once into shared memory, then every warp walks its share of the rows.  The
// value must equal the reference's bit for bit (lse_correction.cu:4-28), which fixes the order of
// the FP32 operations: lane l accumulates channels l, l + 32, ... in increasing order with the
// product and the sum rounded separately, the 32 partials are combined by a shift-down tree, and
// the scale multiplies the finished sum.
constexpr int kShiftRows = 64, kShiftThreads = 256;

template <typename T>
__global__ __launch_bounds__(kShiftThreads) void lse_shift_rows_kernel(
    const T* __restrict__ q, const T* __restrict__ k, const int32_t* __restrict__ anchors,
    float* __restrict__ out, int q_heads, int kv_heads, int q_len, int head_dim, int64_t q_stride_b,
    int64_t q_stride_h, int64_t q_stride_n, int64_t k_stride_b, int64_t k_stride_h,
    int64_t k_stride_n, float scale) {
  __shared__ float anchor_row[256];
  const int head = blockIdx.y, batch = blockIdx.z;
  const int kv_head = head / (q_heads / kv_heads);
  const int anchor = anchors[batch * kv_heads + kv_head];
  const int first = blockIdx.x * kShiftRows;
  const int rows = min(kShiftRows, q_len - first);
  float* dst = out + (int64_t(batch) * q_heads + head) * q_len + first;
  if (anchor < 0) {  // no translation happened for this KV head
    for (int i = threadIdx.x; i < rows; i += kShiftThreads) dst[i] = 0.0f * scale;
    return;
  }
  const T* key = k + batch * k_stride_b + kv_head * k_stride_h + int64_t(anchor) * k_stride_n;
  for (int d = threadIdx.x; d < head_dim; d += kShiftThreads)
    anchor_row[d] = static_cast<float>(key[d]);
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const T* q_head = q + batch * q_stride_b + head * q_stride_h;
  for (int i = warp; i < rows; i += kShiftThreads / 32) {
    const T* q_row = q_head + int64_t(first + i) * q_stride_n;
    float partial = 0.0f;
    for (int d = lane; d < head_dim; d += 32)
      partial = __fadd_rn(partial, __fmul_rn(static_cast<float>(q_row[d]), anchor_row[d]));
#pragma unroll
    for (int off = 16; off > 0; off >>= 1)
      partial += __shfl_down_sync(0xffffffffu, partial, off);
    if (lane == 0) dst[i] = partial * scale;
  }
}

// ---- key-mask tiles ---------------------------------------------------------------------------
// A mask broadcast over queries hides the same keys from every row, so key tiles without a single
// visible key can be skipped by the whole attention call.  Output per (batch, head): the visible
// tile ids in ascending order followed, at index `tiles`, by their number (same layout as the
// reference's key_mask_tiles.cu).  One CTA per (batch, head): the warps mark visible tiles in a
// shared-memory bitmap -- a lane looks at four keys per step, as one 32-bit load when the mask is
// a dense boolean row -- and warp 0 then expands the bitmap into the list.
constexpr int kTileListThreads = 256;
constexpr int kTileListMaxWords = 1024;  // 32768 tiles per (batch, head)

__device__ __forceinline__ bool key_visible(const void* mask, int64_t index, int dtype_code) {
  if (dtype_code == 3) return static_cast<const uint8_t*>(mask)[index] != 0;
  float bias;
  if (dtype_code == 0) bias = static_cast<const float*>(mask)[index];
  else if (dtype_code == 1) bias = __half2float(static_cast<const __half*>(mask)[index]);
  else bias = __bfloat162float(static_cast<const __nv_bfloat16*>(mask)[index]);
  return isfinite(bias);
}

__global__ __launch_bounds__(kTileListThreads) void visible_tile_list_kernel(
    const void* __restrict__ mask, int32_t* __restrict__ output, int heads, int length,
    int tile_size, int64_t stride_b, int64_t stride_h, int64_t stride_k, int dtype_code) {
  __shared__ uint32_t visible_bits[kTileListMaxWords];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int tiles = (length + tile_size - 1) / tile_size;
  const int words = (tiles + 31) / 32;
  for (int w = threadIdx.x; w < words; w += kTileListThreads) visible_bits[w] = 0u;
  __syncthreads();
  const int64_t row_base = int64_t(blockIdx.x) * stride_b + int64_t(blockIdx.y) * stride_h;
  const bool packed_bool = dtype_code == 3 && stride_k == 1 &&
                           (reinterpret_cast<uintptr_t>(mask) + row_base) % 4 == 0;
  for (int tile = warp; tile < tiles; tile += kTileListThreads / 32) {
    bool any = false;
    const int begin = tile * tile_size, end = min(length, begin + tile_size);
    for (int key = begin + 4 * lane; key < end; key += 128) {
      if (packed_bool && key + 4 <= end) {
        any |= *reinterpret_cast<const uint32_t*>(static_cast<const uint8_t*>(mask) + row_base +
                                                  key) != 0u;
      } else {
        for (int j = key; j < min(end, key + 4); ++j)
          any |= key_visible(mask, row_base + int64_t(j) * stride_k, dtype_code);
      }
    }
    if (__any_sync(0xffffffffu, any) && lane == 0)
      atomicOr(&visible_bits[tile >> 5], 1u << (tile & 31));
  }
  __syncthreads();
  if (warp != 0) return;
  int32_t* list = output + (int64_t(blockIdx.x) * heads + blockIdx.y) * (tiles + 1);
  int listed = 0;
  for (int w = 0; w < words; ++w) {
    const uint32_t word = visible_bits[w];
    if (word >> lane & 1u) list[listed + __popc(word & ((1u << lane) - 1u))] = 32 * w + lane;
    listed += __popc(word);
  }
  if (lane == 0) list[tiles] = listed;
}

// ---- retained-mass selection ---------------------------------------------------------------------
// Stage 1, one warp per CSR row (eight rows per CTA): closes the descending prefix (select.cuh) and
// records the kept tiles as a bitmap -- the tile ids of ranks 0 .. count-1, scattered as bits -- in
// `support`, ceil(key_blocks / 32) words per row, rows back to back.
constexpr int kSelectRowsPerCta = 8;

__global__ __launch_bounds__(32 * kSelectRowsPerCta) void close_prefix_kernel(
    const float* __restrict__ sorted_mass, const int64_t* __restrict__ order,
    int32_t* __restrict__ counts, uint8_t* __restrict__ support, double* __restrict__ row_totals,
    uint32_t row_count, uint32_t key_blocks, double theta) {
  __shared__ uint32_t bitmaps[kSelectRowsPerCta][kTileListMaxWords / 8];
  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t row = blockIdx.x * kSelectRowsPerCta + warp;
  if (row >= row_count) return;
  const uint64_t base = uint64_t(row) * key_blocks;
  const RetainedPrefix kept = retained_prefix(sorted_mass + base, key_blocks, theta);
  const uint32_t words = bitmap_words(key_blocks);
  uint32_t* bits = bitmaps[warp];
  for (uint32_t w = lane; w < words; w += 32) bits[w] = 0u;
  __syncwarp();
  for (uint32_t rank = lane; rank < kept.count; rank += 32) {
    const uint32_t tile = static_cast<uint32_t>(order[base + rank]);
    atomicOr(&bits[tile >> 5], 1u << (tile & 31));
  }
  __syncwarp();
  uint32_t* out = reinterpret_cast<uint32_t*>(support) + uint64_t(row) * words;
  for (uint32_t w = lane; w < words; w += 32) out[w] = bits[w];
  if (lane == 0) {
    counts[row] = static_cast<int32_t>(kept.count);
    row_totals[row * 2] = kept.selected;
    row_totals[row * 2 + 1] = kept.total;
  }
}

// Stage 2, single CTA: exclusive scan of the row counts (integer, order-free) and the FP64 summary,
// whose 256 strided partials and halving tree follow reference sparse_selection.cu:69-101.
__global__ __launch_bounds__(256) void offsets_and_summary_kernel(
    const int32_t* __restrict__ counts, const double* __restrict__ row_totals,
    int32_t* __restrict__ row_offsets, double* __restrict__ summary, uint32_t row_count) {
  __shared__ double s_sel[256], s_tot[256];
  __shared__ int32_t s_scan[256];
  const uint32_t tid = threadIdx.x;
  double selected = 0.0, total = 0.0;
  for (uint32_t row = tid; row < row_count; row += 256) {
    selected += row_totals[row * 2];
    total += row_totals[row * 2 + 1];
  }
  s_sel[tid] = selected;
  s_tot[tid] = total;
  // contiguous slice per thread for the scan
  const uint32_t per = (row_count + 255) / 256;
  const uint32_t begin = min(row_count, tid * per), end = min(row_count, begin + per);
  int32_t local = 0;
  for (uint32_t r = begin; r < end; ++r) local += counts[r];
  s_scan[tid] = local;
  __syncthreads();
  for (uint32_t stride = 128; stride > 0; stride >>= 1) {
    if (tid < stride) {
      s_sel[tid] += s_sel[tid + stride];
      s_tot[tid] += s_tot[tid + stride];
    }
    __syncthreads();
  }
  if (tid == 0) {
    int32_t running = 0;
    for (int i = 0; i < 256; ++i) {
      const int32_t c = s_scan[i];
      s_scan[i] = running;
      running += c;
    }
    row_offsets[row_count] = running;
    summary[0] = s_sel[0];
    summary[1] = s_tot[0];
    summary[2] = static_cast<double>(running);
  }
  __syncthreads();
  int32_t running = s_scan[tid];
  for (uint32_t r = begin; r < end; ++r) {
    row_offsets[r] = running;
    running += counts[r];
  }
}

// Stage 3, one warp per row: expands the row's bitmap into ascending tile ids at its CSR offset.
// `stride_bytes`: distance between the bitmaps of consecutive rows.
__global__ __launch_bounds__(256) void expand_bitmaps_kernel(const uint8_t* __restrict__ support,
                                                             const int32_t* __restrict__ row_offsets,
                                                             int32_t* __restrict__ block_indices,
                                                             uint32_t row_count,
                                                             uint32_t key_blocks,
                                                             uint64_t stride_bytes) {
  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t row = blockIdx.x * 8 + warp;
  if (row >= row_count) return;
  const uint32_t* bits = reinterpret_cast<const uint32_t*>(support + uint64_t(row) * stride_bytes);
  int32_t* out = block_indices + row_offsets[row];
  uint32_t written = 0;
  for (uint32_t w = 0; w < bitmap_words(key_blocks); ++w) {
    const uint32_t word = bits[w];
    if (word >> lane & 1u) out[written + __popc(word & ((1u << lane) - 1u))] = int32_t(32 * w + lane);
    written += __popc(word);
  }
}

}  // namespace
}  // namespace risa_b200

using namespace risa_b200;

extern "C" const char* risa_b200_last_error(void) { return error_buffer(); }
extern "C" int risa_b200_abi_version(void) { return 1; }

extern "C" int risa_b200_correct_lse(const void* q, const void* k, const int32_t* anchors,
                                     float* out, int batch, int q_heads, int kv_heads, int q_len,
                                     int head_dim, int64_t qb, int64_t qh, int64_t qn, int64_t kb,
                                     int64_t kh, int64_t kn, float scale, int dtype_code,
                                     void* stream_ptr) {
  RISA_REQUIRE(q && k && anchors && out, "lse_shift: null tensor");
  RISA_REQUIRE(batch > 0 && q_heads > 0 && kv_heads > 0 && q_len > 0 && head_dim > 0 &&
                   q_heads % kv_heads == 0,
               "lse_shift: invalid sizes");
  RISA_REQUIRE(dtype_code >= 0 && dtype_code <= 2, "lse_shift: dtype code must be 0, 1 or 2");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  RISA_REQUIRE(head_dim <= 256, "lse_shift: head_dim must not exceed 256");
  const dim3 grid((q_len + kShiftRows - 1) / kShiftRows, q_heads, batch);
  RISA_DISPATCH_FLOAT(dtype_code, T, {
    lse_shift_rows_kernel<T><<<grid, kShiftThreads, 0, stream>>>(
        static_cast<const T*>(q), static_cast<const T*>(k), anchors, out, q_heads, kv_heads, q_len,
        head_dim, qb, qh, qn, kb, kh, kn, scale);
  });
  return check_launch("lse_shift");
}

extern "C" int risa_b200_prepare_key_mask_tiles(const void* mask, int32_t* tiles, int batch,
                                                int q_heads, int k_len, int tile_size,
                                                int64_t stride_b, int64_t stride_h,
                                                int64_t stride_k, int dtype_code,
                                                void* stream_ptr) {
  RISA_REQUIRE(mask && tiles, "prepare_key_mask_tiles: null tensor");
  RISA_REQUIRE(tile_size == 64 || tile_size == 128,
               "prepare_key_mask_tiles requires an expanded broadcast key mask");
  RISA_REQUIRE(dtype_code >= 0 && dtype_code <= 3 && batch > 0 && q_heads > 0 && k_len > 0,
               "prepare_key_mask_tiles: invalid arguments");
  RISA_REQUIRE((k_len + tile_size - 1) / tile_size <= 32 * kTileListMaxWords,
               "prepare_key_mask_tiles: more than %d key tiles", 32 * kTileListMaxWords);
  visible_tile_list_kernel<<<dim3(batch, q_heads), kTileListThreads, 0,
                             static_cast<cudaStream_t>(stream_ptr)>>>(
      mask, tiles, q_heads, k_len, tile_size, stride_b, stride_h, stride_k, dtype_code);
  return check_launch("prepare_key_mask_tiles");
}

// Scratch for rows too short to hold their own bitmap word (see risa_b200_select_retained_mass).
extern "C" size_t risa_b200_selector_workspace_size(int row_count) {
  return 16 + (row_count > 0 ? size_t(row_count) * 4 : 0);
}

extern "C" int risa_b200_select_retained_mass(const float* sorted_mass, const int64_t* order,
                                              int32_t* counts, uint8_t* support,
                                              double* row_totals, int32_t* row_offsets,
                                              int32_t* block_indices, double* summary,
                                              void* scan_workspace, size_t scan_workspace_bytes,
                                              int row_count, int key_blocks, double theta,
                                              void* stream_ptr) {
  RISA_REQUIRE(sorted_mass && order && counts && support && row_totals && row_offsets &&
                   block_indices && summary,
               "select_retained_mass: null tensor");
  RISA_REQUIRE(row_count > 0 && key_blocks > 0, "select_retained_mass: empty problem");
  RISA_REQUIRE(theta > 0.0 && theta <= 1.0, "theta must be finite and in (0, 1]");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  // The per-row bitmaps (ceil(key_blocks / 32) words each) live in the caller's support scratch,
  // packed back to back from its start; rows of fewer than four key blocks are too short for a
  // word each, their bitmaps go to the scan workspace (sized for that by
  // risa_b200_selector_workspace_size).
  const uint32_t words = bitmap_words(uint32_t(key_blocks));
  uint8_t* bitmaps = support;
  if (uint32_t(key_blocks) < 4 * words) {
    RISA_REQUIRE(scan_workspace != nullptr && scan_workspace_bytes >= size_t(row_count) * 4,
                 "select_retained_mass: scan workspace of %zu bytes required",
                 size_t(row_count) * 4);
    bitmaps = static_cast<uint8_t*>(scan_workspace);
  }
  RISA_REQUIRE(reinterpret_cast<uintptr_t>(bitmaps) % 4 == 0,
               "select_retained_mass: scratch buffers must be 4-byte aligned");
  RISA_REQUIRE(words <= kTileListMaxWords / 8,
               "select_retained_mass: more than %d key blocks per row", 4 * kTileListMaxWords);
  close_prefix_kernel<<<(row_count + kSelectRowsPerCta - 1) / kSelectRowsPerCta,
                        32 * kSelectRowsPerCta, 0, stream>>>(
      sorted_mass, order, counts, bitmaps, row_totals, uint32_t(row_count), uint32_t(key_blocks),
      theta);
  offsets_and_summary_kernel<<<1, 256, 0, stream>>>(counts, row_totals, row_offsets, summary,
                                                    uint32_t(row_count));
  expand_bitmaps_kernel<<<(row_count + 7) / 8, 256, 0, stream>>>(
      bitmaps, row_offsets, block_indices, uint32_t(row_count), uint32_t(key_blocks),
      uint64_t(words) * 4);
  return check_launch("select_retained_mass");
}

extern "C" int risa_b200_pack_selected(const int32_t* counts, const uint32_t* bitmaps,
                                       const double* row_totals, int32_t* row_offsets,
                                       int32_t* block_indices, double* summary, int row_count,
                                       int key_blocks, void* stream_ptr) {
  RISA_REQUIRE(counts && bitmaps && row_totals && row_offsets && block_indices && summary,
               "pack_selected: null tensor");
  RISA_REQUIRE(row_count > 0 && key_blocks > 0, "pack_selected: empty problem");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  offsets_and_summary_kernel<<<1, 256, 0, stream>>>(counts, row_totals, row_offsets, summary,
                                                    uint32_t(row_count));
  expand_bitmaps_kernel<<<(row_count + 7) / 8, 256, 0, stream>>>(
      reinterpret_cast<const uint8_t*>(bitmaps), row_offsets, block_indices, uint32_t(row_count),
      uint32_t(key_blocks), uint64_t(bitmap_words(uint32_t(key_blocks))) * 4);
  return check_launch("pack_selected");
}
