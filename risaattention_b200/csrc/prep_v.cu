// V preparation for INT8 attention on B200: per-channel range, INT8 codes written transposed
// ([B*Hkv*D, padded_Lk]) in the packed 16-token storage order, and the residual-corrected centre
// of the midpoint-affine mode.
//
// Behaviour follows the reference project's csrc/kernels/quantize_v_impl.cuh:83-292 bit for bit
// (scale = max(radius * (1/127), 1e-12), code = rni((v - centre) * (1/scale)), residual summed in
// the order "slot t of 512 visits tokens Lk-1-t, Lk-1-t-512, ...; xor butterfly inside each group
// of 32 slots; groups added in index order").  The organisation differs: the reference gives one
// CTA all tokens of 8 channels, which leaves B*Hkv*D/8 CTAs (64 at B=1, Hkv=4, D=128) for 148 SMs.
// Here three small kernels spread every channel over many CTAs:
//   1. range:    coalesced row reads, per-(chunk, channel) min/max into scratch;
//   2. quantise: each CTA owns 8 channels x a 128-slot slice of the residual order, reduces the
//                chunk ranges itself, writes codes and its slots' residual sums;
//   3. finish:   (midpoint-affine only) combines the residual sums in the reference order.
// Compiled with --use_fast_math like the reference so 1.f / x and x / float(L) lower identically.
#include "prep_v_steps.cuh"
#include <mutex>

namespace risa_b200 {
namespace {

constexpr int kSlotsPerCta = 128;  // residual-order slots per quantise CTA

// grid (chunks, Hkv, B), 256 threads.
template <typename T>
__global__ __launch_bounds__(kRangeThreads) void v_range_kernel(const VRangeJob job) {
  chain_wait();
  chain_release();
  v_range_block<T>(job, blockIdx.x, blockIdx.y, blockIdx.z);
}

// grid (slot slices, B*Hkv*D/8), 128 threads.
template <typename T, bool AFFINE>
__global__ __launch_bounds__(kSlotsPerCta) void v_quantize_kernel(
    const T* __restrict__ v, int8_t* __restrict__ out, float* __restrict__ scale_out,
    float* __restrict__ center_out, const float2* __restrict__ ranges,
    float* __restrict__ residuals, int k_len, int padded_len, int kv_heads, int head_dim,
    int chunks, int slots, int64_t stride_b, int64_t stride_h, int64_t stride_n,
    const int32_t* __restrict__ perm) {
  chain_wait();
  chain_release();
  __shared__ float s_inv[8], s_center[8];
  const int d_tiles = head_dim / 8;
  const int d_tile = blockIdx.y % d_tiles, bh = blockIdx.y / d_tiles;
  const int h = bh % kv_heads, b = bh / kv_heads;
  const int d0 = d_tile * 8;
  const int slot = blockIdx.x * kSlotsPerCta + threadIdx.x;
  const T* in = v + b * stride_b + h * stride_h + d0;
  const int32_t* row_map = perm ? perm + static_cast<int64_t>(bh) * k_len : nullptr;
  const int64_t out_row = static_cast<int64_t>(bh) * head_dim + d0;

  if (threadIdx.x < 8) {
    float lo = FLT_MAX, hi = -FLT_MAX;
    const float2* r = ranges + static_cast<int64_t>(bh) * chunks * head_dim + d0 + threadIdx.x;
    for (int c = 0; c < chunks; ++c) {
      const float2 x = __ldg(r + static_cast<int64_t>(c) * head_dim);
      lo = fminf(lo, x.x);
      hi = fmaxf(hi, x.y);
    }
    float center, radius;
    if constexpr (AFFINE) {
      center = 0.5f * (lo + hi);
      radius = 0.5f * (hi - lo);
    } else {
      center = 0.0f;
      radius = fmaxf(fabsf(lo), fabsf(hi));
    }
    const float sc = fmaxf(radius * (1.f / 127.f), 1e-12f);
    s_inv[threadIdx.x] = 1.f / sc;
    s_center[threadIdx.x] = center;
    if (blockIdx.x == 0) {
      scale_out[out_row + threadIdx.x] = sc;
      if constexpr (!AFFINE) center_out[out_row + threadIdx.x] = 0.0f;
    }
  }
  __syncthreads();
  float inv[8], center[8], residual[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    inv[i] = s_inv[i];
    center[i] = s_center[i];
    residual[i] = 0.f;
  }
  if (slot < slots) {
    for (int src = k_len - 1 - slot; src >= 0; src -= slots) {
      float t[8];
      const int64_t row = row_map ? __ldg(row_map + src) : src;
      load8(in + row * stride_n, t);
      const int dst = storage_position(src);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float normalized = (t[i] - center[i]) * inv[i];
        const uint32_t code = to_s8(normalized);
        out[(out_row + i) * padded_len + dst] = static_cast<int8_t>(code);
        if constexpr (AFFINE)
          residual[i] += normalized - static_cast<float>(static_cast<int8_t>(code));
      }
    }
    if constexpr (AFFINE) {
#pragma unroll
      for (int i = 0; i < 8; ++i)
        residuals[(out_row + i) * slots + slot] = residual[i];
    }
    // zero tail [k_len, padded_len): the permutation stays inside aligned 16-token groups
    for (int src = k_len + slot; src < padded_len; src += slots) {
      const int dst = storage_position(src);
#pragma unroll
      for (int i = 0; i < 8; ++i) out[(out_row + i) * padded_len + dst] = 0;
    }
  }
}

// grid (slots / 32, B*Hkv*D / 64), 512 threads.
template <typename T, bool AFFINE>
__global__ __launch_bounds__(kTiledThreads) void v_quantize_tiled_kernel(const VCodesJob job) {
  chain_wait();
  chain_release();
  v_codes_tiled_block<T, AFFINE>(job, blockIdx.x, blockIdx.y);
}

// grid (B*Hkv*D), `slots` threads: xor butterfly per warp, warps added in order by thread 0.
__global__ void v_center_kernel(const float* __restrict__ residuals,
                                const float2* __restrict__ ranges, float* __restrict__ center_out,
                                int k_len, int head_dim, int chunks, int slots) {
  chain_wait();
  chain_release();
  __shared__ float warp_sum[16];
  const int channel = blockIdx.x;
  float r = residuals[static_cast<int64_t>(channel) * slots + threadIdx.x];
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) r += __shfl_xor_sync(0xffffffffu, r, off);
  if ((threadIdx.x & 31) == 0) warp_sum[threadIdx.x >> 5] = r;
  __syncthreads();
  if (threadIdx.x == 0) {
    float total = 0.0f;
    for (int w = 0; w < slots / 32; ++w) total += warp_sum[w];
    const int bh = channel / head_dim, c = channel % head_dim;
    float lo = FLT_MAX, hi = -FLT_MAX;
    const float2* rg = ranges + static_cast<int64_t>(bh) * chunks * head_dim + c;
    for (int i = 0; i < chunks; ++i) {
      const float2 x = __ldg(rg + static_cast<int64_t>(i) * head_dim);
      lo = fminf(lo, x.x);
      hi = fmaxf(hi, x.y);
    }
    const float center = 0.5f * (lo + hi);
    const float radius = 0.5f * (hi - lo);
    const float sc = fmaxf(radius * (1.f / 127.f), 1e-12f);
    // reciprocal of the stored reciprocal, both approximate: not the same bits as sc itself
    const float inv = rcp_approx(sc);
    const float scale = rcp_approx(inv);
    // one FMA: centre + scale * mean.  Against the reference's compiled kernel this is bit-identical
    // in more than 99 % of channels and one ulp away in the rest (approximate division feeding a
    // sum that cancels against a small centre).
    center_out[channel] = fmaf(scale, total / static_cast<float>(k_len), center);
  }
}

struct VPlan {
  int chunks, slots;
  size_t range_bytes, residual_bytes;
};

VPlan plan(int batch, int kv_heads, int k_len, int head_dim) {
  VPlan p;
  p.chunks = (k_len + kRangeChunk - 1) / kRangeChunk;
  p.slots = k_len <= 256 ? 128 : 512;
  const size_t channels = static_cast<size_t>(batch) * kv_heads * head_dim;
  p.range_bytes = (channels * p.chunks * sizeof(float2) + 255) / 256 * 256;
  p.residual_bytes = channels * p.slots * sizeof(float);
  return p;
}

}  // namespace
}  // namespace risa_b200

using namespace risa_b200;

extern "C" size_t risa_b200_quantize_v_workspace_size(int batch, int kv_heads, int k_len,
                                                      int head_dim) {
  if (batch <= 0 || kv_heads <= 0 || k_len <= 0 || head_dim <= 0) return 0;
  const VPlan p = plan(batch, kv_heads, k_len, head_dim);
  return p.range_bytes + p.residual_bytes;
}

namespace {
// 16-byte code stores need whole storage groups and an aligned destination; a CTA of the tiled
// kernel owns kTiledChannels channels of one head, so the head must split into whole groups.
bool tiled_form(const void* v_codes, int k_len, int head_dim) {
  return k_len % 16 == 0 && reinterpret_cast<uintptr_t>(v_codes) % 16 == 0 &&
         head_dim % kTiledChannels == 0;
}
}  // namespace

int risa_b200::v_quantize_jobs(const void* v, void* v_codes, float* v_scale, float* v_center,
                               int batch, int kv_heads, int k_len, int head_dim, int padded_len,
                               int64_t stride_b, int64_t stride_h, int64_t stride_n,
                               int dtype_code, int midpoint_affine, const int32_t* perm,
                               void* workspace, size_t workspace_bytes, VRangeJob* range,
                               VCodesJob* codes) {
  RISA_REQUIRE(v && v_codes && v_scale && v_center, "quantize_v: null tensor");
  RISA_REQUIRE(batch > 0 && kv_heads > 0 && k_len > 0, "quantize_v: sizes must be positive");
  RISA_REQUIRE(head_dim > 0 && head_dim % 8 == 0 && head_dim <= 256,
               "quantize_v: head_dim must be a positive multiple of 8 (at most 256)");
  RISA_REQUIRE(padded_len >= k_len && padded_len % 16 == 0,
               "quantize_v: padded length must cover the keys and be a multiple of 16");
  RISA_REQUIRE(dtype_code >= 0 && dtype_code <= 2, "quantize_v: dtype code must be 0, 1 or 2");
  const size_t esize = dtype_code == 0 ? 4 : 2;
  auto stride_ok = [esize](int64_t stride, int extent) {
    return extent < 2 || (static_cast<size_t>(stride) * esize) % 16 == 0;
  };
  RISA_REQUIRE(reinterpret_cast<uintptr_t>(v) % 16 == 0 && stride_ok(stride_b, batch) &&
                   stride_ok(stride_h, kv_heads) && stride_ok(stride_n, k_len),
               "quantize_v: V base pointer and batch/head/sequence strides must be 16-byte "
               "aligned");
  const VPlan p = plan(batch, kv_heads, k_len, head_dim);
  RISA_REQUIRE(workspace != nullptr && workspace_bytes >= p.range_bytes + p.residual_bytes,
               "quantize_v: workspace of %zu bytes required", p.range_bytes + p.residual_bytes);
  RISA_REQUIRE(reinterpret_cast<uintptr_t>(workspace) % 16 == 0,
               "quantize_v: workspace must be 16-byte aligned");
  range->v = v;
  range->ranges = static_cast<float2*>(workspace);
  range->k_len = k_len;
  range->head_dim = head_dim;
  range->kv_heads = kv_heads;
  range->batch = batch;
  range->chunks = p.chunks;
  range->stride_b = stride_b;
  range->stride_h = stride_h;
  range->stride_n = stride_n;
  range->perm = perm;
  codes->v = nullptr;
  if (tiled_form(v_codes, k_len, head_dim)) {
    codes->v = v;
    codes->out = static_cast<int8_t*>(v_codes);
    codes->scale_out = v_scale;
    codes->center_out = v_center;
    codes->ranges = range->ranges;
    codes->residuals = reinterpret_cast<float*>(static_cast<char*>(workspace) + p.range_bytes);
    codes->k_len = k_len;
    codes->padded_len = padded_len;
    codes->kv_heads = kv_heads;
    codes->head_dim = head_dim;
    codes->batch = batch;
    codes->chunks = p.chunks;
    codes->slots = p.slots;
    codes->stride_b = stride_b;
    codes->stride_h = stride_h;
    codes->stride_n = stride_n;
    codes->perm = perm;
    codes->midpoint_affine = midpoint_affine;
  }
  return RISA_B200_OK;
}

// Everything after the range step; the arguments were checked by v_quantize_jobs().
int risa_b200::quantize_v_after_range(const void* v, void* v_codes, float* v_scale,
                                      float* v_center, int batch, int kv_heads, int k_len,
                                      int head_dim, int padded_len, int64_t stride_b,
                                      int64_t stride_h, int64_t stride_n, int dtype_code,
                                      int midpoint_affine, const int32_t* perm, void* workspace,
                                      bool codes_done, void* stream_ptr) {
  const VPlan p = plan(batch, kv_heads, k_len, head_dim);
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  float2* ranges = static_cast<float2*>(workspace);
  float* residuals = reinterpret_cast<float*>(static_cast<char*>(workspace) + p.range_bytes);
  const int channels = batch * kv_heads * head_dim;
  RISA_DISPATCH_FLOAT(dtype_code, T, {
    if (codes_done) {
      // the code step has run next to the K quantiser
    } else if (tiled_form(v_codes, k_len, head_dim)) {
      VRangeJob range;
      VCodesJob codes;
      v_quantize_jobs(v, v_codes, v_scale, v_center, batch, kv_heads, k_len, head_dim, padded_len,
                      stride_b, stride_h, stride_n, dtype_code, midpoint_affine, perm, workspace,
                      p.range_bytes + p.residual_bytes, &range, &codes);
      const dim3 tiled_grid(p.slots / kTiledSlots, channels / kTiledChannels);
      if (midpoint_affine)
        launch_chained(v_quantize_tiled_kernel<T, true>, tiled_grid, dim3(kTiledThreads), 0, stream,
                       codes);
      else
        launch_chained(v_quantize_tiled_kernel<T, false>, tiled_grid, dim3(kTiledThreads), 0,
                       stream, codes);
    } else {
      const dim3 grid(p.slots / kSlotsPerCta, channels / 8);
      if (midpoint_affine)
        launch_chained(v_quantize_kernel<T, true>, grid, dim3(kSlotsPerCta), 0, stream,
            static_cast<const T*>(v), static_cast<int8_t*>(v_codes), v_scale, v_center, ranges,
            residuals, k_len, padded_len, kv_heads, head_dim, p.chunks, p.slots, stride_b,
            stride_h, stride_n, perm);
      else
        launch_chained(v_quantize_kernel<T, false>, grid, dim3(kSlotsPerCta), 0, stream,
            static_cast<const T*>(v), static_cast<int8_t*>(v_codes), v_scale, v_center, ranges,
            residuals, k_len, padded_len, kv_heads, head_dim, p.chunks, p.slots, stride_b,
            stride_h, stride_n, perm);
    }
    if (midpoint_affine)
      launch_chained(v_center_kernel, dim3(channels), dim3(p.slots), 0, stream, residuals, ranges,
                     v_center, k_len, head_dim, p.chunks, p.slots);
  });
  return check_launch("quantize_v");
}

extern "C" int risa_b200_quantize_v(const void* v, void* v_codes, float* v_scale, float* v_center,
                                    int batch, int kv_heads, int k_len, int head_dim,
                                    int padded_len, int64_t stride_b, int64_t stride_h,
                                    int64_t stride_n, int dtype_code, int midpoint_affine,
                                    const int32_t* perm, void* workspace, size_t workspace_bytes,
                                    void* stream_ptr) {
  VRangeJob range;
  VCodesJob codes;
  const int status = v_quantize_jobs(v, v_codes, v_scale, v_center, batch, kv_heads, k_len,
                                     head_dim, padded_len, stride_b, stride_h, stride_n,
                                     dtype_code, midpoint_affine, perm, workspace, workspace_bytes,
                                     &range, &codes);
  if (status != RISA_B200_OK) return status;
  RISA_DISPATCH_FLOAT(dtype_code, T, {
    launch_chained(v_range_kernel<T>, dim3(range.chunks, kv_heads, batch), dim3(kRangeThreads), 0,
                   static_cast<cudaStream_t>(stream_ptr), range);
  });
  return quantize_v_after_range(v, v_codes, v_scale, v_center, batch, kv_heads, k_len, head_dim,
                                padded_len, stride_b, stride_h, stride_n, dtype_code,
                                midpoint_affine, perm, workspace, false, stream_ptr);
}

// ---- allocation-free variant --------------------------------------------------------------------
// Scratch for callers that cannot hand over device memory of their own.  The array lives in the
// library's device image: every GPU that loads the library carries these bytes until the process
// exits, which is why the ceiling is kept modest.
namespace {
constexpr size_t kStaticScratchBytes = size_t(4) << 20;  // 4 MiB
static __device__ __align__(256) unsigned char g_v_static_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
std::mutex g_static_scratch_mutex;
void* g_static_scratch_ptr[kMaxDevices] = {nullptr};

// In host code `g_v_static_scratch` is only a handle for the runtime, not a device address; the
// address a kernel can use has to be asked for, per device, with that device current.
int static_scratch_for_current_device(void** out) {
  int device = -1;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess) return fail(RISA_B200_CUDA, "quantize_v_static: %s", cudaGetErrorString(e));
  if (device < 0 || device >= kMaxDevices)
    return fail(RISA_B200_INVALID, "quantize_v_static: device index %d not supported", device);
  std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
  if (g_static_scratch_ptr[device] == nullptr) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_v_static_scratch);
    if (e != cudaSuccess || ptr == nullptr)
      return fail(RISA_B200_CUDA, "quantize_v_static: cannot resolve the scratch array: %s",
                  cudaGetErrorString(e));
    g_static_scratch_ptr[device] = ptr;
  }
  *out = g_static_scratch_ptr[device];
  return RISA_B200_OK;
}
}  // namespace

extern "C" size_t risa_b200_quantize_v_static_limit(void) { return kStaticScratchBytes; }

extern "C" int risa_b200_quantize_v_static(const void* v, void* v_codes, float* v_scale,
                                           float* v_center, int batch, int kv_heads, int k_len,
                                           int head_dim, int padded_len, int64_t stride_b,
                                           int64_t stride_h, int64_t stride_n, int dtype_code,
                                           int midpoint_affine, const int32_t* perm,
                                           void* stream_ptr) {
  const size_t need = risa_b200_quantize_v_workspace_size(batch, kv_heads, k_len, head_dim);
  RISA_REQUIRE(need != 0, "quantize_v_static: sizes must be positive");
  RISA_REQUIRE(need <= kStaticScratchBytes,
               "quantize_v_static: this problem needs %zu bytes of scratch but the built-in "
               "scratch holds %zu; use risa_b200_quantize_v with a caller workspace",
               need, kStaticScratchBytes);
  void* scratch = nullptr;
  const int status = static_scratch_for_current_device(&scratch);
  if (status != RISA_B200_OK) return status;
  // Nothing in the scratch has to start at zero: the range and residual partials a call reads are
  // all written earlier in the same call.  Whatever the previous call left is simply overwritten.
  return risa_b200_quantize_v(v, v_codes, v_scale, v_center, batch, kv_heads, k_len, head_dim,
                              padded_len, stride_b, stride_h, stride_n, dtype_code,
                              midpoint_affine, perm, scratch, kStaticScratchBytes, stream_ptr);
}
