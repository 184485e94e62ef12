// Per-channel value range of V, first step of its quantisation: shared by the stand-alone range
// kernel and by the kernel that runs it next to the Q quantiser and the K anchor detector.
// Reference: csrc/kernels/quantize_v_impl.cuh:83-160 (the min / max part of the per-channel pass).
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

// Host side of the V quantiser split at the range step (prep_v.cu): v_range_job() checks the
// arguments of a risa_b200_quantize_v call and describes its range step without launching it;
// quantize_v_after_range() launches everything that follows the range step.
int v_range_job(const void* v, void* v_codes, float* v_scale, float* v_center, int batch,
                int kv_heads, int k_len, int head_dim, int padded_len, int64_t stride_b,
                int64_t stride_h, int64_t stride_n, int dtype_code, const int32_t* perm,
                void* workspace, size_t workspace_bytes, VRangeJob* job);
int quantize_v_after_range(const void* v, void* v_codes, float* v_scale, float* v_center, int batch,
                           int kv_heads, int k_len, int head_dim, int padded_len, int64_t stride_b,
                           int64_t stride_h, int64_t stride_n, int dtype_code, int midpoint_affine,
                           const int32_t* perm, void* workspace, void* stream_ptr);
// Q and K quantisation (prep_qk.cu); with a range job the V range step runs inside the first launch.
int quantize_qk_with_range(const void* q, void* q_codes, float* q_scale, const void* k,
                           void* k_codes, float* k_scale, int batch, int q_heads, int q_len,
                           int kv_heads, int k_len, int head_dim, int cta_k, int64_t q_stride_b,
                           int64_t q_stride_h, int64_t q_stride_n, int64_t k_stride_b,
                           int64_t k_stride_h, int64_t k_stride_n, int dtype_code, int32_t* anchors,
                           const int32_t* q_perm, const int32_t* k_perm, const VRangeJob* range_job,
                           void* stream_ptr);

}  // namespace risa_b200
