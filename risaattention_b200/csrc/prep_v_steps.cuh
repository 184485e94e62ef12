// The range step and the (tiled) code step of the V quantiser as CTA bodies, shared by their
// stand-alone kernels (prep_v.cu) and by the launches that run them next to the Q / K quantisers
// (prep_qk.cu).  Reference: csrc/kernels/quantize_v_impl.cuh:83-292.
#pragma once
#include "common.cuh"
#include <cfloat>

namespace risa_b200 {

constexpr int kRangeChunk = 512;   // tokens per range CTA
constexpr int kRangeThreads = 256;

// What the range step of one risa_b200_quantize_v call reads and writes.
struct VRangeJob {
  const void* v;
  float2* ranges;  // [B*Hkv][chunks][head_dim] (min, max)
  int k_len, head_dim, kv_heads, batch, chunks;
  int64_t stride_b, stride_h, stride_n;
  const int32_t* perm;
};

template <typename T>
__device__ __forceinline__ void load8(const T* p, float* v) {
  Load4<T>::load(p, v);
  Load4<T>::load(p + 4, v + 4);
}

// One CTA of 256 threads = one 512-token chunk of one (batch, kv head): thread = (token lane,
// 8-channel group).
template <typename T>
__device__ __forceinline__ void v_range_block(const VRangeJob& job, int chunk, int h, int b) {
  __shared__ float s_mn[256][9], s_mx[256][9];
  const int head_dim = job.head_dim, k_len = job.k_len;
  const int groups = head_dim / 8;            // 8, 16 or 32 threads per token row
  const int tokens_per_step = 256 / groups;
  const int g = threadIdx.x % groups, tl = threadIdx.x / groups;
  const int64_t bh = static_cast<int64_t>(b) * job.kv_heads + h;
  const T* in = static_cast<const T*>(job.v) + b * job.stride_b + h * job.stride_h + g * 8;
  const int32_t* row_map = job.perm ? job.perm + bh * k_len : nullptr;
  float mn[8], mx[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    mn[i] = FLT_MAX;
    mx[i] = -FLT_MAX;
  }
  const int begin = chunk * kRangeChunk;
  const int end = min(k_len, begin + kRangeChunk);
  for (int n = begin + tl; n < end; n += tokens_per_step) {
    float t[8];
    const int64_t src = row_map ? __ldg(row_map + n) : n;
    load8(in + src * job.stride_n, t);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      mn[i] = fminf(mn[i], t[i]);
      mx[i] = fmaxf(mx[i], t[i]);
    }
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    s_mn[threadIdx.x][i] = mn[i];
    s_mx[threadIdx.x][i] = mx[i];
  }
  __syncthreads();
  if (threadIdx.x < head_dim) {
    const int c = threadIdx.x, cg = c / 8, ci = c % 8;
    float lo = FLT_MAX, hi = -FLT_MAX;
    for (int t = 0; t < tokens_per_step; ++t) {
      lo = fminf(lo, s_mn[t * groups + cg][ci]);
      hi = fmaxf(hi, s_mx[t * groups + cg][ci]);
    }
    job.ranges[(bh * job.chunks + chunk) * head_dim + c] = make_float2(lo, hi);
  }
}

__device__ __forceinline__ int storage_position(int token) {
  // token bits {b3,b2,b1,b0} -> storage bits {b2,b0,b3,b1}: order 0,1,8,9,2,3,10,11,...
  const int w = token & 15;
  return (token & ~15) | (w & 1) | (((w >> 3) & 1) << 1) | (((w >> 1) & 1) << 2) |
         (((w >> 2) & 1) << 3);
}

// Same work as v_quantize_kernel for key lengths that are a multiple of 16, organised for the memory
// system: a CTA owns 32 consecutive slots x 64 channels (thread = one slot, four channels), so a
// half-warp reads one token's 64 channels as one contiguous segment, and the codes of a 32-token
// window go through shared memory to leave as 16-byte stores (one aligned 16-token storage group
// of one channel each) instead of single bytes.  Each (slot, channel) residual is still summed by
// one thread over tokens Lk-1-slot, Lk-1-slot-slots, ... in that order.
// CTA (bx, by) of a (slots / 32) x (B*Hkv*D / 64) grid, 512 threads.
constexpr int kTiledSlots = 32, kTiledChannels = 64, kTiledThreads = 512;

// What the code step of one risa_b200_quantize_v call reads and writes (tiled form).
struct VCodesJob {
  const void* v;
  int8_t* out;
  float* scale_out;
  float* center_out;
  const float2* ranges;
  float* residuals;
  int k_len, padded_len, kv_heads, head_dim, batch, chunks, slots;
  int64_t stride_b, stride_h, stride_n;
  const int32_t* perm;
  int midpoint_affine;
};

template <typename T, bool AFFINE>
__device__ __forceinline__ void v_codes_tiled_block(const VCodesJob& job, int bx, int by) {
  const T* __restrict__ v = static_cast<const T*>(job.v);
  int8_t* __restrict__ out = job.out;
  float* __restrict__ scale_out = job.scale_out;
  float* __restrict__ center_out = job.center_out;
  const float2* __restrict__ ranges = job.ranges;
  float* __restrict__ residuals = job.residuals;
  const int k_len = job.k_len, padded_len = job.padded_len, kv_heads = job.kv_heads;
  const int head_dim = job.head_dim, chunks = job.chunks, slots = job.slots;
  const int64_t stride_b = job.stride_b, stride_h = job.stride_h, stride_n = job.stride_n;
  const int32_t* __restrict__ perm = job.perm;
  __shared__ float s_inv[kTiledChannels], s_center[kTiledChannels];
  // 32 positions per channel; a row pitch of 36 bytes (9 words) spreads the 16 channel quads of a
  // half-warp over 8 banks (any pitch that is a multiple of 16 bytes would put them on 2)
  __shared__ __align__(4) unsigned char s_tile[2][kTiledChannels][36];
  const int d_tiles = head_dim / kTiledChannels;
  const int d_tile = by % d_tiles, bh = by / d_tiles;
  const int h = bh % kv_heads, b = bh / kv_heads;
  const int d0 = d_tile * kTiledChannels;
  const int sl = threadIdx.x >> 4, quad = threadIdx.x & 15;
  const int slot = bx * kTiledSlots + sl;
  const T* in = v + b * stride_b + h * stride_h + d0 + 4 * quad;
  const int32_t* row_map = perm ? perm + static_cast<int64_t>(bh) * k_len : nullptr;
  const int64_t out_row = static_cast<int64_t>(bh) * head_dim + d0;

  // channel range = min / max over the per-chunk partials: spread over the whole CTA (eight chunk
  // subsets per channel) so that the loads overlap instead of forming one long dependent loop
  __shared__ float s_lo[kTiledThreads / kTiledChannels][kTiledChannels];
  __shared__ float s_hi[kTiledThreads / kTiledChannels][kTiledChannels];
  {
    const int channel = threadIdx.x % kTiledChannels, part = threadIdx.x / kTiledChannels;
    float lo = FLT_MAX, hi = -FLT_MAX;
    const float2* r = ranges + static_cast<int64_t>(bh) * chunks * head_dim + d0 + channel;
    for (int c = part; c < chunks; c += kTiledThreads / kTiledChannels) {
      const float2 x = __ldg(r + static_cast<int64_t>(c) * head_dim);
      lo = fminf(lo, x.x);
      hi = fmaxf(hi, x.y);
    }
    s_lo[part][channel] = lo;
    s_hi[part][channel] = hi;
  }
  __syncthreads();
  if (threadIdx.x < kTiledChannels) {
    float lo = FLT_MAX, hi = -FLT_MAX;
#pragma unroll
    for (int part = 0; part < kTiledThreads / kTiledChannels; ++part) {
      lo = fminf(lo, s_lo[part][threadIdx.x]);
      hi = fmaxf(hi, s_hi[part][threadIdx.x]);
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
    if (bx == 0) {
      scale_out[out_row + threadIdx.x] = sc;
      if constexpr (!AFFINE) center_out[out_row + threadIdx.x] = 0.0f;
    }
  }
  __syncthreads();
  float inv[4], center[4], residual[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    inv[i] = s_inv[4 * quad + i];
    center[i] = s_center[4 * quad + i];
    residual[i] = 0.f;
  }
  // Window of iteration `it`: tokens [hi - 31, hi], hi = k_len - 1 - 32 * bx - slots * it;
  // with k_len a multiple of 16 the window is two aligned 16-token storage groups.
  const int first_hi = k_len - 1 - bx * kTiledSlots;
  int buffer = 0;
  // The loads of kBatch consecutive windows are issued together (a token's row is only read once,
  // so nothing but the number of loads in flight hides the memory latency), then the windows are
  // converted and written one after the other.
  constexpr int kBatch = 8;
  for (int batch_hi = first_hi; batch_hi >= 0; batch_hi -= kBatch * slots) {
    float t[kBatch][4];
#pragma unroll
    for (int u = 0; u < kBatch; ++u) {
      const int src = batch_hi - u * slots - sl;
      if (src >= 0) {
        const int64_t row = row_map ? __ldg(row_map + src) : src;
        Load4<T>::load(in + row * stride_n, t[u]);
      }
    }
#pragma unroll
    for (int u = 0; u < kBatch; ++u) {
      const int hi = batch_hi - u * slots;
      if (hi < 0) break;  // uniform over the CTA
      const int lo = hi - (kTiledSlots - 1);
      const int src = hi - sl;
      if (src >= 0) {
        const int position = storage_position(src) - lo;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float normalized = (t[u][i] - center[i]) * inv[i];
          const uint32_t code = to_s8(normalized);
          s_tile[buffer][4 * quad + i][position] = static_cast<unsigned char>(code);
          if constexpr (AFFINE)
            residual[i] += normalized - static_cast<float>(static_cast<int8_t>(code));
        }
      }
      __syncthreads();  // the other buffer was read before the previous barrier: safe to refill
      if (threadIdx.x < 2 * kTiledChannels) {
        const int channel = threadIdx.x >> 1, group = threadIdx.x & 1;
        const int base = lo + 16 * group;
        if (base >= 0) {
          const uint32_t* w = reinterpret_cast<const uint32_t*>(&s_tile[buffer][channel][16 * group]);
          *reinterpret_cast<uint4*>(out + (out_row + channel) * padded_len + base) =
              make_uint4(w[0], w[1], w[2], w[3]);
        }
      }
      buffer ^= 1;
    }
  }
  if constexpr (AFFINE) {
#pragma unroll
    for (int i = 0; i < 4; ++i)
      residuals[(out_row + 4 * quad + i) * slots + slot] = residual[i];
  }
  // zero tail [k_len, padded_len): whole 16-byte groups because k_len is a multiple of 16
  for (int idx = bx * kTiledThreads + threadIdx.x;
       idx < kTiledChannels * ((padded_len - k_len) / 16); idx += job.slots / kTiledSlots * kTiledThreads) {
    const int channel = idx % kTiledChannels, group = idx / kTiledChannels;
    *reinterpret_cast<uint4*>(out + (out_row + channel) * padded_len + k_len + 16 * group) =
        make_uint4(0u, 0u, 0u, 0u);
  }
}

// Host side of the V quantiser split into its steps (prep_v.cu): v_quantize_jobs() checks the
// arguments of a risa_b200_quantize_v call and describes its range step and -- when the tiled form
// applies, else codes->v stays null -- its code step, launching nothing;
// quantize_v_after_range() launches what follows the range step, without the code step if that has
// been run by somebody else.
int v_quantize_jobs(const void* v, void* v_codes, float* v_scale, float* v_center, int batch,
                    int kv_heads, int k_len, int head_dim, int padded_len, int64_t stride_b,
                    int64_t stride_h, int64_t stride_n, int dtype_code, int midpoint_affine,
                    const int32_t* perm, void* workspace, size_t workspace_bytes, VRangeJob* range,
                    VCodesJob* codes);
int quantize_v_after_range(const void* v, void* v_codes, float* v_scale, float* v_center, int batch,
                           int kv_heads, int k_len, int head_dim, int padded_len, int64_t stride_b,
                           int64_t stride_h, int64_t stride_n, int dtype_code, int midpoint_affine,
                           const int32_t* perm, void* workspace, bool codes_done, void* stream_ptr);
// Q and K quantisation (prep_qk.cu).  With a range job the V range step runs inside the first
// launch (next to the anchor detector and the Q quantiser); with a codes job the V code step runs
// inside the second (next to the K quantiser).
int quantize_qk_with_v_steps(const void* q, void* q_codes, float* q_scale, const void* k,
                             void* k_codes, float* k_scale, int batch, int q_heads, int q_len,
                             int kv_heads, int k_len, int head_dim, int cta_k, int64_t q_stride_b,
                             int64_t q_stride_h, int64_t q_stride_n, int64_t k_stride_b,
                             int64_t k_stride_h, int64_t k_stride_n, int dtype_code,
                             int32_t* anchors, const int32_t* q_perm, const int32_t* k_perm,
                             const VRangeJob* range_job, const VCodesJob* codes_job,
                             void* stream_ptr);

}  // namespace risa_b200
