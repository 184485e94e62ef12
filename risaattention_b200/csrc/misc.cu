// Small kernels around the attention call: LSE shift of the K anchor, visible-tile lists of
// broadcast key masks, retained-mass selection with CSR packing, plus the library's error text.
#include "common.cuh"

namespace risa_b200 {

char* error_buffer() {
  static thread_local char buffer[512] = {0};
  return buffer;
}

namespace {

// ---- LSE shift: out[b,h,i] = scale * <q_i, k_anchor>, 0 when the head has no anchor -----------
// One warp per query row; products and sums are separate roundings (no FMA), lanes stride the
// channels by 32 and combine with a shfl_down tree (reference lse_correction.cu:4-28).
template <typename T>
__global__ __launch_bounds__(128) void lse_shift_kernel(const T* q, const T* k,
                                                        const int32_t* anchors, float* out, int hq,
                                                        int hk, int nq, int head_dim, int64_t qb,
                                                        int64_t qh, int64_t qn, int64_t kb,
                                                        int64_t kh, int64_t kn, float scale) {
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * 4 + (threadIdx.x >> 5);
  const int head = blockIdx.y, batch = blockIdx.z;
  if (row >= nq) return;
  const int kv_head = head / (hq / hk);
  const int anchor = anchors[batch * hk + kv_head];
  float sum = 0.0f;
  if (anchor >= 0) {
    const T* qr = q + batch * qb + head * qh + int64_t(row) * qn;
    const T* kr = k + batch * kb + kv_head * kh + int64_t(anchor) * kn;
    for (int d = lane; d < head_dim; d += 32)
      sum = __fadd_rn(sum, __fmul_rn(static_cast<float>(qr[d]), static_cast<float>(kr[d])));
    for (int step = 16; step; step >>= 1) sum += __shfl_down_sync(0xffffffffu, sum, step);
  }
  if (lane == 0) out[(int64_t(batch) * hq + head) * nq + row] = sum * scale;
}

// ---- key-mask tiles ---------------------------------------------------------------------------
__device__ __forceinline__ bool mask_visible(const void* mask, int64_t index, int dtype_code) {
  if (dtype_code == 3) return static_cast<const uint8_t*>(mask)[index] != 0;
  const float bias = dtype_code == 0   ? static_cast<const float*>(mask)[index]
                     : dtype_code == 1 ? __half2float(static_cast<const __half*>(mask)[index])
                                       : __bfloat162float(
                                             static_cast<const __nv_bfloat16*>(mask)[index]);
  return isfinite(bias);
}

// One CTA (4 warps) per (batch, head): flag tiles with no visible key, then warp 0 compacts the
// visible tile ids to the front and appends their count (reference key_mask_tiles.cu:10-43).
__global__ __launch_bounds__(128) void key_mask_tiles_kernel(const void* mask, int32_t* output,
                                                             int heads, int length, int tile_size,
                                                             int64_t stride_b, int64_t stride_h,
                                                             int64_t stride_k, int dtype_code) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int tiles = (length + tile_size - 1) / tile_size;
  const int64_t row = int64_t(blockIdx.x) * heads + blockIdx.y;
  const int64_t mask_row = int64_t(blockIdx.x) * stride_b + int64_t(blockIdx.y) * stride_h;
  int32_t* flags = output + row * (tiles + 1);
  for (int tile = warp; tile < tiles; tile += 4) {
    bool visible = false;
    for (int off = lane; off < tile_size; off += 32) {
      const int key = tile * tile_size + off;
      if (key < length) visible |= mask_visible(mask, mask_row + int64_t(key) * stride_k, dtype_code);
    }
    const bool excluded = __ballot_sync(0xffffffffu, visible) == 0;
    if (lane == 0) flags[tile] = excluded;
  }
  __syncthreads();
  if (warp == 0) {
    int active_count = 0;
    for (int base = 0; base < tiles; base += 32) {
      const int tile = base + lane;
      const bool active = tile < tiles && flags[tile] == 0;
      const unsigned votes = __ballot_sync(0xffffffffu, active);
      const int rank = __popc(votes & ((1u << lane) - 1));
      __syncwarp();
      if (active) flags[active_count + rank] = tile;
      __syncwarp();
      active_count += __popc(votes);
    }
    if (lane == 0) flags[tiles] = active_count;
  }
}

// ---- retained-mass selection ---------------------------------------------------------------------
// One warp per CSR row over the descending-sorted masses: FP64 total (lane-strided, shfl_down
// tree), then 32-rank chunks with an inclusive Hillis-Steele FP64 scan; the first rank whose
// cumulative mass reaches theta * total closes the prefix (reference sparse_selection.cu:9-67; the
// FP64 operation order decides which rank that is).
__global__ __launch_bounds__(32) void select_rows_kernel(const float* __restrict__ sorted_mass,
                                                         const int64_t* __restrict__ order,
                                                         int32_t* __restrict__ counts,
                                                         uint8_t* __restrict__ support,
                                                         double* __restrict__ row_totals,
                                                         uint32_t key_blocks, double theta) {
  const uint32_t row = blockIdx.x, lane = threadIdx.x;
  const uint64_t base = uint64_t(row) * key_blocks;
  double lane_total = 0.0;
  for (uint32_t rank = lane; rank < key_blocks; rank += 32) {
    lane_total += static_cast<double>(sorted_mass[base + rank]);
    support[base + rank] = 0;
  }
  double total = lane_total;
#pragma unroll
  for (uint32_t off = 16; off > 0; off >>= 1) total += __shfl_down_sync(0xffffffffu, total, off);
  total = __shfl_sync(0xffffffffu, total, 0);
  const double target = theta * total;
  double cumulative = 0.0, selected = total;
  uint32_t count = key_blocks;
  for (uint32_t chunk = 0; chunk < key_blocks; chunk += 32) {
    const uint32_t rank = chunk + lane;
    double prefix = rank < key_blocks ? static_cast<double>(sorted_mass[base + rank]) : 0.0;
#pragma unroll
    for (uint32_t off = 1; off < 32; off <<= 1) {
      const double previous = __shfl_up_sync(0xffffffffu, prefix, off);
      if (lane >= off) prefix += previous;
    }
    const bool reaches = rank < key_blocks && cumulative + prefix >= target;
    const uint32_t candidates = __ballot_sync(0xffffffffu, reaches);
    if (candidates != 0) {
      const uint32_t first = __ffs(candidates) - 1;
      count = chunk + first + 1;
      selected = cumulative + __shfl_sync(0xffffffffu, prefix, first);
      break;
    }
    cumulative += __shfl_sync(0xffffffffu, prefix, 31);
  }
  __syncwarp();
  for (uint32_t rank = lane; rank < count; rank += 32)
    support[base + static_cast<uint32_t>(order[base + rank])] = 1;
  if (lane == 0) {
    counts[row] = static_cast<int32_t>(count);
    row_totals[row * 2] = selected;
    row_totals[row * 2 + 1] = total;
  }
}

// Single CTA: exclusive scan of the row counts (integer, order-free) and the FP64 summary, whose
// 256 strided partials and halving tree follow reference sparse_selection.cu:69-101.
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

// One warp per row: ballot compaction of the support flags into ascending tile ids.
__global__ __launch_bounds__(256) void compact_csr_kernel(const uint8_t* __restrict__ support,
                                                          const int32_t* __restrict__ row_offsets,
                                                          int32_t* __restrict__ block_indices,
                                                          uint32_t row_count, uint32_t key_blocks) {
  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t row = blockIdx.x * 8 + warp;
  if (row >= row_count) return;
  const uint64_t base = uint64_t(row) * key_blocks;
  const uint32_t out = row_offsets[row];
  uint32_t before = 0;
  for (uint32_t chunk = 0; chunk < key_blocks; chunk += 32) {
    const uint32_t key = chunk + lane;
    const bool keep = key < key_blocks && support[base + key] != 0;
    const uint32_t votes = __ballot_sync(0xffffffffu, keep);
    if (keep) block_indices[out + before + __popc(votes & ((1u << lane) - 1u))] = int32_t(key);
    before += __popc(votes);
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
  const dim3 grid((q_len + 3) / 4, q_heads, batch);
  RISA_DISPATCH_FLOAT(dtype_code, T, {
    lse_shift_kernel<T><<<grid, 128, 0, stream>>>(static_cast<const T*>(q),
                                                  static_cast<const T*>(k), anchors, out, q_heads,
                                                  kv_heads, q_len, head_dim, qb, qh, qn, kb, kh, kn,
                                                  scale);
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
  key_mask_tiles_kernel<<<dim3(batch, q_heads), 128, 0, static_cast<cudaStream_t>(stream_ptr)>>>(
      mask, tiles, q_heads, k_len, tile_size, stride_b, stride_h, stride_k, dtype_code);
  return check_launch("prepare_key_mask_tiles");
}

extern "C" size_t risa_b200_selector_workspace_size(int) { return 16; }

extern "C" int risa_b200_select_retained_mass(const float* sorted_mass, const int64_t* order,
                                              int32_t* counts, uint8_t* support,
                                              double* row_totals, int32_t* row_offsets,
                                              int32_t* block_indices, double* summary, void*,
                                              size_t, int row_count, int key_blocks, double theta,
                                              void* stream_ptr) {
  RISA_REQUIRE(sorted_mass && order && counts && support && row_totals && row_offsets &&
                   block_indices && summary,
               "select_retained_mass: null tensor");
  RISA_REQUIRE(row_count > 0 && key_blocks > 0, "select_retained_mass: empty problem");
  RISA_REQUIRE(theta > 0.0 && theta <= 1.0, "theta must be finite and in (0, 1]");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  select_rows_kernel<<<row_count, 32, 0, stream>>>(sorted_mass, order, counts, support, row_totals,
                                                   uint32_t(key_blocks), theta);
  offsets_and_summary_kernel<<<1, 256, 0, stream>>>(counts, row_totals, row_offsets, summary,
                                                    uint32_t(row_count));
  compact_csr_kernel<<<(row_count + 7) / 8, 256, 0, stream>>>(support, row_offsets, block_indices,
                                                              uint32_t(row_count),
                                                              uint32_t(key_blocks));
  return check_launch("select_retained_mass");
}
