// Q/K preparation for INT8 attention on B200: K anchor detection, block Hadamard rotation and
// symmetric INT8 quantisation with FP32 group scales.
//
// Behaviour follows the reference project's csrc/kernels/quantize_qk_impl.cuh (anchor :442-577,
// rotations :69-147, Q groups :153-269, K groups :278-426) so that codes and scales are
// bit-identical; the kernel organisation is different:
//   * a lane owns 16 contiguous channels of a row (four vector loads, one 16-byte code store),
//     so only the three highest Hadamard stages need warp shuffles;
//   * one CTA quantises a whole 128-row query block or a whole key tile, with the four key scale
//     groups of the tile spread over its warps, so no lane holds more than 64 values.
// This file is compiled with --use_fast_math on purpose: the reference's scale arithmetic
// (x / 127.f, 1.f / x) is defined by that mode's approximate division and reciprocal.
#include "prep_v_steps.cuh"

namespace risa_b200 {
namespace {

constexpr int kRotH4 = 4, kRotH64 = 64, kRotSigned128 = 128, kRotPlain128 = 129;

// In-lane H4 on 4 adjacent channels (channel bits 1 and 2), with the 0.5 normalisation.
__device__ __forceinline__ void h4(float* v) {
  const float a0 = v[0] + v[1], a1 = v[0] - v[1], a2 = v[2] + v[3], a3 = v[2] - v[3];
  v[0] = (a0 + a2) * 0.5f;
  v[1] = (a1 + a3) * 0.5f;
  v[2] = (a0 - a2) * 0.5f;
  v[3] = (a1 - a3) * 0.5f;
}

// Rotates the 16 channels [16*chunk, 16*chunk+16) held by this lane.  Lanes holding one row's
// (or one 128-channel tile's) chunks are consecutive, so span 16/32/64 pair lane ^ 1/2/4.
template <int ROT>
__device__ __forceinline__ void rotate16(float* v, int chunk) {
  if constexpr (ROT == kRotSigned128) {
    constexpr uint32_t kSigns[4] = {0x1035997bu, 0x8087f5eeu, 0xee2e4e1au, 0x71132418u};
    const uint32_t word = chunk < 2 ? kSigns[0] : chunk < 4 ? kSigns[1] : chunk < 6 ? kSigns[2]
                                                                                   : kSigns[3];
    const uint32_t bits = word >> ((chunk & 1) * 16);
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const uint32_t flip = ((bits >> i) & 1u) ^ 1u;
      v[i] = __uint_as_float(__float_as_uint(v[i]) ^ (flip << 31));
    }
  }
#pragma unroll
  for (int i = 0; i < 16; i += 4) h4(v + i);
  if constexpr (ROT == kRotH4) return;
  // spans 4 and 8 stay inside the lane
#pragma unroll
  for (int span = 4; span <= 8; span <<= 1) {
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      if ((i & span) == 0) {
        const float lo = v[i], hi = v[i + span];
        v[i] = lo + hi;
        v[i + span] = lo - hi;
      }
    }
  }
  constexpr int kLaneStages = ROT == kRotH64 ? 2 : 3;  // spans 16,32 (,64)
#pragma unroll
  for (int s = 0; s < kLaneStages; ++s) {
    const int bit = 1 << s;
    // other - v in the upper lane of a pair, v + other in the lower one: one FMA with a lane sign
    const float sign = (chunk & bit) != 0 ? -1.0f : 1.0f;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const float other = __shfl_xor_sync(0xffffffffu, v[i], bit);
      v[i] = fmaf(v[i], sign, other);
    }
  }
  constexpr float kNorm = ROT == kRotH64 ? 0.25f : 0.1767766952966369f;
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] *= kNorm;
}

template <typename T>
__device__ __forceinline__ void load16(const T* p, float* v) {
#pragma unroll
  for (int i = 0; i < 4; ++i) Load4<T>::load(p + 4 * i, v + 4 * i);
}

__device__ __forceinline__ float absmax16(const float* v) {
  float mx = 0.f;
#pragma unroll
  for (int i = 0; i < 16; ++i) mx = fmaxf(mx, fabsf(v[i]));
  return mx;
}

__device__ __forceinline__ void store16_codes(int8_t* p, const float* v, float inv) {
  uint4 w;
  w.x = pack4_s8(v[0] * inv, v[1] * inv, v[2] * inv, v[3] * inv);
  w.y = pack4_s8(v[4] * inv, v[5] * inv, v[6] * inv, v[7] * inv);
  w.z = pack4_s8(v[8] * inv, v[9] * inv, v[10] * inv, v[11] * inv);
  w.w = pack4_s8(v[12] * inv, v[13] * inv, v[14] * inv, v[15] * inv);
  *reinterpret_cast<uint4*>(p) = w;
}

// ------------------------------------------------------------------------------------------
// Q: one CTA per (128-row block, head, batch).  A scale group is 4 rows {r, r+8, r+16, r+24} of a
// 32-row tile (D <= 128) or 2 rows {r, r+8} of a 16-row tile (D = 256), times all channels.
// ------------------------------------------------------------------------------------------
struct QJob {
  const void* q;
  int8_t* codes;
  float* scales;
  int q_len, q_heads, batch, blocks, scales_per_head;
  int64_t stride_b, stride_h, stride_n;
  const int32_t* perm;
};

template <typename T, int D, int ROT>
__device__ __forceinline__ void quantize_q_block(const QJob& job, int blk, int h, int b) {
  const T* __restrict__ q = static_cast<const T*>(job.q);
  int8_t* __restrict__ codes = job.codes;
  float* __restrict__ scales = job.scales;
  const int q_len = job.q_len, q_heads = job.q_heads, scales_per_head = job.scales_per_head;
  const int64_t stride_b = job.stride_b, stride_h = job.stride_h, stride_n = job.stride_n;
  const int32_t* __restrict__ perm = job.perm;
  constexpr int LPR = D / 16;                       // lanes per row
  constexpr int GROUP_ROWS = D == 256 ? 2 : 4;      // rows per scale group
  constexpr int GLANES = GROUP_ROWS * LPR;          // lanes per group (16 or 32)
  constexpr int GPP = 32 / GLANES;                  // groups per warp pass
  constexpr int TILE_ROWS = D == 256 ? 16 : 32;     // rows sharing one set of 8 groups
  constexpr int GROUPS = 128 / GROUP_ROWS;          // groups per 128-row block
  constexpr int PASSES = GROUPS / GPP / 8;          // passes per warp (8 warps)
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const T* in = q + b * stride_b + h * stride_h;
  const int64_t bh = static_cast<int64_t>(b) * q_heads + h;
  int8_t* out = codes + bh * q_len * D;
  float* sc_out = scales + bh * scales_per_head + blk * (GROUPS);
  const int32_t* row_map = perm ? perm + bh * q_len : nullptr;

  const int slot = lane / GLANES;           // which group of the pass
  const int j = (lane % GLANES) / LPR;      // row inside the group
  const int chunk = lane % LPR;             // 16-channel chunk inside the row

  // Passes are independent (a scale group lives inside one pass); they are taken kBatch at a time so
  // that a thread holds kBatch * 16 values instead of all of them: fewer registers, more resident
  // CTAs whose load and arithmetic phases overlap one another.
  constexpr int kBatch = 2;
  static_assert(PASSES % kBatch == 0, "pass batching");
#pragma unroll 1
  for (int p0 = 0; p0 < PASSES; p0 += kBatch) {
    float v[kBatch][16];
    int rows[kBatch];
#pragma unroll
    for (int p = 0; p < kBatch; ++p) {
      const int group = (warp * PASSES + p0 + p) * GPP + slot;  // 0..GROUPS-1 == tile*8 + o
      const int row = blk * 128 + (group >> 3) * TILE_ROWS + (group & 7) + 8 * j;
      rows[p] = row;
#pragma unroll
      for (int i = 0; i < 16; ++i) v[p][i] = 0.f;
      if (row < q_len) {
        const int64_t src = row_map ? __ldg(row_map + row) : row;
        load16(in + src * stride_n + chunk * 16, v[p]);
      }
    }
#pragma unroll
    for (int p = 0; p < kBatch; ++p) {
      rotate16<ROT>(v[p], D == 256 ? (chunk & 7) : chunk);
      float mx = absmax16(v[p]);
#pragma unroll
      for (int off = GLANES / 2; off > 0; off >>= 1)
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
      const float sc = mx / 127.f + 1e-7f;
      const float inv = 1.f / sc;
      const int group = (warp * PASSES + p0 + p) * GPP + slot;
      if ((lane % GLANES) == 0) sc_out[group] = sc;
      if (rows[p] < q_len)
        store16_codes(out + static_cast<int64_t>(rows[p]) * D + chunk * 16, v[p], inv);
    }
  }
}

template <typename T, int D, int ROT>
__global__ __launch_bounds__(256) void quantize_q_kernel(const QJob job) {
  chain_wait();
  chain_release();
  quantize_q_block<T, D, ROT>(job, blockIdx.x, blockIdx.y, blockIdx.z);
}

// ------------------------------------------------------------------------------------------
// K: one CTA per (key tile, kv head, batch).  Scale group w of a tile = rows with (n % 8) / 2 == w.
// Warp (w, s) takes a contiguous share of group w's rows; groups spanning several warps combine
// their maxima through shared memory.
// ------------------------------------------------------------------------------------------
constexpr int k_threads(int d, int cta_k) { return d * cta_k / 64 < 128 ? 128 : d * cta_k / 64; }

struct KJob {
  const void* k;
  int8_t* codes;
  float* scales;
  const int32_t* anchors;
  int k_len, kv_heads, batch, tiles;
  int64_t stride_b, stride_h, stride_n;
  const int32_t* perm;
};

// One key tile by k_threads(D, CTA_K) consecutive threads.  `sub` is the index of that thread group
// inside the CTA (0 when the CTA is exactly one group) and `tid` the thread's index inside the
// group; groups of a CTA meet only at their own named barrier.
template <typename T, int D, int CTA_K, int ROT>
__device__ __forceinline__ void quantize_k_tile(const KJob& job, int tile, int h, int b, int sub,
                                                int tid) {
  const T* __restrict__ k = static_cast<const T*>(job.k);
  int8_t* __restrict__ codes = job.codes;
  float* __restrict__ scales = job.scales;
  const int k_len = job.k_len, kv_heads = job.kv_heads, scales_per_head = job.tiles * 4;
  const int64_t stride_b = job.stride_b, stride_h = job.stride_h, stride_n = job.stride_n;
  const int32_t* __restrict__ perm = job.perm;
  constexpr int LPR = D / 16;
  constexpr int RPP = 32 / LPR;                 // rows per warp pass
  constexpr int THREADS = k_threads(D, CTA_K);  // at most 64 values per lane
  constexpr int NW = THREADS / 128;             // warps per scale group (>= 1 except D64)
  constexpr int WPG = NW < 1 ? 1 : NW;
  constexpr int GROUP_ROWS = CTA_K / 4;
  constexpr int RW = GROUP_ROWS / WPG;          // rows per warp
  constexpr int PASSES = RW / RPP;
  static_assert(PASSES >= 1 && PASSES * RPP == RW, "tile geometry");
  __shared__ float warp_max[512 / THREADS][4][WPG];
  const int lane = tid & 31, warp = tid >> 5;
  const int w = warp % 4, s = warp / 4;
  const T* in = k + b * stride_b + h * stride_h;
  const int64_t bh = static_cast<int64_t>(b) * kv_heads + h;
  int8_t* out = codes + bh * k_len * D;
  const int32_t* row_map = perm ? perm + bh * k_len : nullptr;
  const int jr = lane / LPR, chunk = lane % LPR;

  float bias[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) bias[i] = 0.f;
  const int anchor = __ldg(job.anchors + bh);
  if (anchor >= 0) {
    const int64_t src = row_map ? __ldg(row_map + anchor) : anchor;
    load16(in + src * stride_n + chunk * 16, bias);
  }

  float v[PASSES][16];
  int rows[PASSES];
  float mx = 0.f;
#pragma unroll
  for (int p = 0; p < PASSES; ++p) {
    const int i = s * RW + p * RPP + jr;  // index inside the group's row list
    const int row = tile * CTA_K + 8 * (i >> 1) + 2 * w + (i & 1);
    rows[p] = row;
#pragma unroll
    for (int c = 0; c < 16; ++c) v[p][c] = 0.f;
    if (row < k_len) {
      const int64_t src = row_map ? __ldg(row_map + row) : row;
      load16(in + src * stride_n + chunk * 16, v[p]);
#pragma unroll
      for (int c = 0; c < 16; ++c) v[p][c] -= bias[c];
    }
  }
#pragma unroll
  for (int p = 0; p < PASSES; ++p) {
    rotate16<ROT>(v[p], D == 256 ? (chunk & 7) : chunk);
    mx = fmaxf(mx, absmax16(v[p]));
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
  if constexpr (WPG > 1) {
    if (lane == 0) warp_max[sub][w][s] = mx;
    asm volatile("bar.sync %0, %1;" ::"r"(1 + sub), "r"(THREADS) : "memory");
#pragma unroll
    for (int i = 0; i < WPG; ++i) mx = fmaxf(mx, warp_max[sub][w][i]);
  }
  const float sc = mx / 127.f + 1e-7f;
  const float inv = 1.f / sc;
  if (s == 0 && lane == 0) scales[bh * scales_per_head + tile * 4 + w] = sc;
#pragma unroll
  for (int p = 0; p < PASSES; ++p)
    if (rows[p] < k_len)
      store16_codes(out + static_cast<int64_t>(rows[p]) * D + chunk * 16, v[p], inv);
}

// grid (key tiles, kv heads, batch), k_threads(D, CTA_K) threads.
template <typename T, int D, int CTA_K, int ROT>
__global__ __launch_bounds__(k_threads(D, CTA_K)) void quantize_k_kernel(const KJob job) {
  chain_wait();
  chain_release();
  quantize_k_tile<T, D, CTA_K, ROT>(job, blockIdx.x, blockIdx.y, blockIdx.z, 0, threadIdx.x);
}

// The two steps that need the results of the first launch -- K quantisation (anchors) and the V
// code step (ranges) -- as one launch of 512-thread CTAs: CTAs [0, V CTAs) are CTAs of the tiled V
// code step (they run longest), each of the rest holds 512 / k_threads key tiles, one per thread
// group.
template <typename T, int D, int CTA_K, int ROT, bool AFFINE>
__global__ __launch_bounds__(kTiledThreads) void quantize_k_v_codes_kernel(const KJob k_job,
                                                                            const VCodesJob v_job) {
  chain_wait();
  chain_release();
  const int v_columns = v_job.slots / kTiledSlots;
  const int v_blocks = v_columns * (v_job.batch * v_job.kv_heads * v_job.head_dim / kTiledChannels);
  int block = blockIdx.x;
  if (block < v_blocks) {
    v_codes_tiled_block<T, AFFINE>(v_job, block % v_columns, block / v_columns);
    return;
  }
  block -= v_blocks;
  constexpr int THREADS = k_threads(D, CTA_K);
  constexpr int SUBS = kTiledThreads / THREADS;
  const int sub = threadIdx.x / THREADS, tid = threadIdx.x % THREADS;
  const int item = block * SUBS + sub;  // (batch, head, tile), tile fastest
  if (item >= k_job.tiles * k_job.kv_heads * k_job.batch) return;
  const int tile = item % k_job.tiles, bh = item / k_job.tiles;
  quantize_k_tile<T, D, CTA_K, ROT>(k_job, tile, bh % k_job.kv_heads, bh / k_job.kv_heads, sub, tid);
}

// ------------------------------------------------------------------------------------------
// K anchor detector: nine evenly spaced keys per (batch, kv head); the candidate minimising the
// summed squared distance to the others becomes the anchor if it lowers the sampled energy without
// raising the sampled absmax by more than 12.5 %.  The FP32 reduction shape (thread t owns
// channels t and t+128, shfl_down tree, warps added 0..3) decides borderline cases and is kept.
// ------------------------------------------------------------------------------------------
struct AnchorJob {
  const void* k;
  int32_t* anchors;
  int k_len, head_dim, kv_heads, batch;
  int64_t stride_b, stride_h, stride_n;
  const int32_t* perm;
};

// Threads 0..127 of the CTA do the work; a CTA may be larger (every thread takes the barriers).
template <typename T>
__device__ __forceinline__ void detect_anchor_block(const AnchorJob& job, int h, int b) {
  constexpr int S = 9;
  __shared__ float smp[S * 256];
  __shared__ float w_energy[4], w_max[4], w_dist[S][4], w_benergy[4], w_bmax[4];
  __shared__ int chosen;
  const int k_len = job.k_len, head_dim = job.head_dim;
  const int tid = threadIdx.x;
  const bool active = tid < 128;
  const int lane = tid & 31, warp = tid >> 5;
  const int64_t bh = static_cast<int64_t>(b) * job.kv_heads + h;
  const T* in = static_cast<const T*>(job.k) + b * job.stride_b + h * job.stride_h;
  const int32_t* row_map = job.perm ? job.perm + bh * k_len : nullptr;
  if (active) {
    for (int idx = tid; idx < S * head_dim; idx += 128) {
      const int sample = idx / head_dim, channel = idx - sample * head_dim;
      const int row = sample * (k_len - 1) / (S - 1);
      const int64_t src = row_map ? __ldg(row_map + row) : row;
      smp[idx] = load_scalar(in + src * job.stride_n + channel);
    }
  }
  __syncthreads();
  if (active) {
    float energy = 0.f, vmax = 0.f, dist[S];
#pragma unroll
    for (int c = 0; c < S; ++c) dist[c] = 0.f;
    for (int channel = tid; channel < head_dim; channel += 128) {
      float sum = 0.f;
#pragma unroll
      for (int sidx = 0; sidx < S; ++sidx) {
        const float x = smp[sidx * head_dim + channel];
        energy = fmaf(x, x, energy);
        vmax = fmaxf(vmax, fabsf(x));
        sum += x;
      }
#pragma unroll
      for (int c = 0; c < S; ++c) {
        const float dd = S * smp[c * head_dim + channel] - sum;
        dist[c] = fmaf(dd, dd, dist[c]);
      }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      energy += __shfl_down_sync(0xffffffffu, energy, off);
      vmax = fmaxf(vmax, __shfl_down_sync(0xffffffffu, vmax, off));
#pragma unroll
      for (int c = 0; c < S; ++c) dist[c] += __shfl_down_sync(0xffffffffu, dist[c], off);
    }
    if (lane == 0) {
      w_energy[warp] = energy;
      w_max[warp] = vmax;
#pragma unroll
      for (int c = 0; c < S; ++c) w_dist[c][warp] = dist[c];
    }
  }
  __syncthreads();
  if (tid == 0) {
    int best = 0;
    float best_d = 3.402823466e+38F;
#pragma unroll
    for (int c = 0; c < S; ++c) {
      float dsum = 0.f;
#pragma unroll
      for (int i = 0; i < 4; ++i) dsum += w_dist[c][i];
      if (dsum < best_d) {
        best = c;
        best_d = dsum;
      }
    }
    chosen = best;
  }
  __syncthreads();
  if (active) {
    float benergy = 0.f, bmax = 0.f;
    for (int channel = tid; channel < head_dim; channel += 128) {
      const float a = smp[chosen * head_dim + channel];
#pragma unroll
      for (int sidx = 0; sidx < S; ++sidx) {
        const float r = smp[sidx * head_dim + channel] - a;
        benergy = fmaf(r, r, benergy);
        bmax = fmaxf(bmax, fabsf(r));
      }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      benergy += __shfl_down_sync(0xffffffffu, benergy, off);
      bmax = fmaxf(bmax, __shfl_down_sync(0xffffffffu, bmax, off));
    }
    if (lane == 0) {
      w_benergy[warp] = benergy;
      w_bmax[warp] = bmax;
    }
  }
  __syncthreads();
  if (tid == 0) {
    float te = 0.f, tm = 0.f, be = 0.f, bm = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      te += w_energy[i];
      tm = fmaxf(tm, w_max[i]);
      be += w_benergy[i];
      bm = fmaxf(bm, w_bmax[i]);
    }
    const bool improves = be < te && bm <= tm * 1.125f;
    job.anchors[bh] = improves ? chosen * (k_len - 1) / (S - 1) : -1;
  }
}

template <typename T>
__global__ __launch_bounds__(128) void detect_anchor_kernel(const AnchorJob job) {
  chain_wait();
  chain_release();
  detect_anchor_block<T>(job, blockIdx.x, blockIdx.y);
}

// The three steps of a call's preparation that need nothing from one another -- the K anchor
// detector, the V range step and the Q quantiser -- as one launch: CTAs [0, anchor CTAs) detect,
// the next ones take V range chunks, the rest quantise Q blocks.  The detector comes first because
// it is one long dependent chain per head; the Q blocks fill the GPU behind it.
template <typename T, int D, int ROT>
__global__ __launch_bounds__(256, 4) void quantize_q_scan_kernel(const QJob q_job,
                                                              const AnchorJob anchor_job,
                                                              const VRangeJob range_job) {
  chain_wait();
  chain_release();
  const int n_anchor = anchor_job.kv_heads * anchor_job.batch;
  const int n_range = range_job.chunks * range_job.kv_heads * range_job.batch;
  int block = blockIdx.x;
  if (block < n_anchor) {
    detect_anchor_block<T>(anchor_job, block % anchor_job.kv_heads, block / anchor_job.kv_heads);
    return;
  }
  block -= n_anchor;
  if (block < n_range) {
    const int chunk = block % range_job.chunks, bh = block / range_job.chunks;
    v_range_block<T>(range_job, chunk, bh % range_job.kv_heads, bh / range_job.kv_heads);
    return;
  }
  block -= n_range;
  const int blk = block % q_job.blocks, bh = block / q_job.blocks;
  quantize_q_block<T, D, ROT>(q_job, blk, bh % q_job.q_heads, bh / q_job.q_heads);
}

// First launch of the preparation: the Q quantiser, and in front of it either the anchor detector
// as a launch of its own or -- when the V range step of the same call is handed in -- the anchor
// detector and the range step inside the same grid.
template <typename T, int D, int ROT>
void launch_q(const QJob& q_job, const AnchorJob& anchor_job, const VRangeJob* range_job,
              cudaStream_t stream) {
  if (range_job) {
    const int blocks = anchor_job.kv_heads * anchor_job.batch +
                       range_job->chunks * range_job->kv_heads * range_job->batch +
                       q_job.blocks * q_job.q_heads * q_job.batch;
    launch_chained(quantize_q_scan_kernel<T, D, ROT>, dim3(blocks), dim3(256), 0, stream, q_job,
                   anchor_job, *range_job);
  } else {
    launch_chained(detect_anchor_kernel<T>, dim3(anchor_job.kv_heads, anchor_job.batch), dim3(128),
                   0, stream, anchor_job);
    launch_chained(quantize_q_kernel<T, D, ROT>, dim3(q_job.blocks, q_job.q_heads, q_job.batch),
                   dim3(256), 0, stream, q_job);
  }
}

// Second launch: the K quantiser, together with the V code step when one is handed in.
template <typename T, int D, int CTA_K, int ROT>
void launch_k(KJob k_job, const VCodesJob* codes_job, cudaStream_t stream) {
  k_job.tiles = (k_job.k_len + CTA_K - 1) / CTA_K;
  if (codes_job) {
    constexpr int SUBS = kTiledThreads / k_threads(D, CTA_K);
    const int k_items = k_job.tiles * k_job.kv_heads * k_job.batch;
    const int v_blocks = codes_job->slots / kTiledSlots *
                         (codes_job->batch * codes_job->kv_heads * codes_job->head_dim /
                          kTiledChannels);
    const dim3 grid(v_blocks + (k_items + SUBS - 1) / SUBS);
    if (codes_job->midpoint_affine)
      launch_chained(quantize_k_v_codes_kernel<T, D, CTA_K, ROT, true>, grid, dim3(kTiledThreads), 0,
                     stream, k_job, *codes_job);
    else
      launch_chained(quantize_k_v_codes_kernel<T, D, CTA_K, ROT, false>, grid, dim3(kTiledThreads),
                     0, stream, k_job, *codes_job);
  } else {
    launch_chained(quantize_k_kernel<T, D, CTA_K, ROT>, dim3(k_job.tiles, k_job.kv_heads, k_job.batch),
                   dim3(k_threads(D, CTA_K)), 0, stream, k_job);
  }
}

template <typename T, int D, int ROT>
void launch_qk(QJob q_job, const AnchorJob& anchor_job, const VRangeJob* range_job,
               const KJob& k_job, const VCodesJob* codes_job, int cta_k, cudaStream_t stream) {
  q_job.scales_per_head = q_job.blocks * (D == 256 ? 64 : 32);
  launch_q<T, D, ROT>(q_job, anchor_job, range_job, stream);
  if constexpr (D == 64) {
    launch_k<T, D, 64, ROT>(k_job, codes_job, stream);
  } else {
    if (cta_k == 128) launch_k<T, D, 128, ROT>(k_job, codes_job, stream);
    else launch_k<T, D, 64, ROT>(k_job, codes_job, stream);
  }
}

}  // namespace
}  // namespace risa_b200

using namespace risa_b200;

int risa_b200::quantize_qk_with_v_steps(const void* q, void* q_codes, float* q_scale, const void* k,
                                      void* k_codes, float* k_scale, int batch, int q_heads,
                                      int q_len, int kv_heads, int k_len, int head_dim, int cta_k,
                                      int64_t q_stride_b, int64_t q_stride_h, int64_t q_stride_n,
                                      int64_t k_stride_b, int64_t k_stride_h, int64_t k_stride_n,
                                      int dtype_code, int32_t* anchors, const int32_t* q_perm,
                                      const int32_t* k_perm, const VRangeJob* range_job,
                                      const VCodesJob* codes_job, void* stream_ptr) {
  RISA_REQUIRE(head_dim == 64 || head_dim == 128 || head_dim == 256,
               "quantize_qk: padded head_dim must be 64, 128, or 256");
  RISA_REQUIRE((cta_k == 64 || cta_k == 128) && !(head_dim == 64 && cta_k != 64),
               "quantize_qk: unsupported key tile %d for head_dim %d", cta_k, head_dim);
  RISA_REQUIRE(q && q_codes && q_scale && k && k_codes && k_scale, "quantize_qk: null tensor");
  RISA_REQUIRE(anchors != nullptr, "quantize_qk: anchor_indices scratch is required");
  RISA_REQUIRE(dtype_code >= 0 && dtype_code <= 2, "quantize_qk: dtype code must be 0, 1 or 2");
  RISA_REQUIRE(batch > 0 && q_heads > 0 && kv_heads > 0 && q_len > 0 && k_len > 0,
               "quantize_qk: sizes must be positive");
  const size_t vec = 4 * (dtype_code == 0 ? 4 : 2);
  auto stride_ok = [](int64_t stride, int extent) {
    return extent < 2 || (stride > 0 && stride % 4 == 0);
  };
  RISA_REQUIRE(reinterpret_cast<uintptr_t>(q) % vec == 0 && stride_ok(q_stride_b, batch) &&
                   stride_ok(q_stride_h, q_heads) && stride_ok(q_stride_n, q_len) &&
                   reinterpret_cast<uintptr_t>(k) % vec == 0 && stride_ok(k_stride_b, batch) &&
                   stride_ok(k_stride_h, kv_heads) && stride_ok(k_stride_n, k_len),
               "quantize_qk: Q/K base pointers and batch/head/sequence strides must preserve "
               "4-element alignment");
  RISA_REQUIRE(reinterpret_cast<uintptr_t>(q_codes) % 16 == 0 &&
                   reinterpret_cast<uintptr_t>(k_codes) % 16 == 0,
               "quantize_qk: code buffers must be 16-byte aligned");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  QJob q_job;
  q_job.q = q;
  q_job.codes = static_cast<int8_t*>(q_codes);
  q_job.scales = q_scale;
  q_job.q_len = q_len;
  q_job.q_heads = q_heads;
  q_job.batch = batch;
  q_job.blocks = (q_len + 127) / 128;
  q_job.scales_per_head = 0;  // set per head_dim below
  q_job.stride_b = q_stride_b;
  q_job.stride_h = q_stride_h;
  q_job.stride_n = q_stride_n;
  q_job.perm = q_perm;
  AnchorJob anchor_job;
  anchor_job.k = k;
  anchor_job.anchors = anchors;
  anchor_job.k_len = k_len;
  anchor_job.head_dim = head_dim;
  anchor_job.kv_heads = kv_heads;
  anchor_job.batch = batch;
  anchor_job.stride_b = k_stride_b;
  anchor_job.stride_h = k_stride_h;
  anchor_job.stride_n = k_stride_n;
  anchor_job.perm = k_perm;
  KJob k_job;
  k_job.k = k;
  k_job.codes = static_cast<int8_t*>(k_codes);
  k_job.scales = k_scale;
  k_job.anchors = anchors;
  k_job.k_len = k_len;
  k_job.kv_heads = kv_heads;
  k_job.batch = batch;
  k_job.tiles = 0;  // set per key-tile width by launch_k
  k_job.stride_b = k_stride_b;
  k_job.stride_h = k_stride_h;
  k_job.stride_n = k_stride_n;
  k_job.perm = k_perm;
#define RISA_QK(D, ROT) \
  launch_qk<T, D, ROT>(q_job, anchor_job, range_job, k_job, codes_job, cta_k, stream)
  const bool h4_only = k_len <= 256;
  RISA_DISPATCH_FLOAT(dtype_code, T, {
    if (head_dim == 64) {
      if (h4_only) RISA_QK(64, kRotH4); else RISA_QK(64, kRotH64);
    } else if (head_dim == 128) {
      if (h4_only) RISA_QK(128, kRotH4); else RISA_QK(128, kRotSigned128);
    } else {
      if (h4_only) RISA_QK(256, kRotH4); else RISA_QK(256, kRotPlain128);
    }
  });
#undef RISA_QK
  return check_launch("quantize_qk");
}

extern "C" int risa_b200_quantize_qk(const void* q, void* q_codes, float* q_scale, const void* k,
                                     void* k_codes, float* k_scale, int batch, int q_heads,
                                     int q_len, int kv_heads, int k_len, int head_dim, int cta_k,
                                     int64_t q_stride_b, int64_t q_stride_h, int64_t q_stride_n,
                                     int64_t k_stride_b, int64_t k_stride_h, int64_t k_stride_n,
                                     int dtype_code, int32_t* anchors, const int32_t* q_perm,
                                     const int32_t* k_perm, void* stream_ptr) {
  return quantize_qk_with_v_steps(q, q_codes, q_scale, k, k_codes, k_scale, batch, q_heads, q_len,
                                  kv_heads, k_len, head_dim, cta_k, q_stride_b, q_stride_h,
                                  q_stride_n, k_stride_b, k_stride_h, k_stride_n, dtype_code,
                                  anchors, q_perm, k_perm, nullptr, nullptr, stream_ptr);
}

// Q, K and V of one call.  Same results as risa_b200_quantize_qk followed by risa_b200_quantize_v;
// the V range step travels in the first launch (quantize_q_scan_kernel) and, for key lengths and
// buffers the tiled code step accepts, the V code step in the second (quantize_k_v_codes_kernel).
extern "C" int risa_b200_quantize_qkv(
    const void* q, void* q_codes, float* q_scale, const void* k, void* k_codes, float* k_scale,
    const void* v, void* v_codes, float* v_scale, float* v_center, int batch, int q_heads,
    int q_len, int kv_heads, int k_len, int head_dim, int cta_k, int padded_len,
    int64_t q_stride_b, int64_t q_stride_h, int64_t q_stride_n, int64_t k_stride_b,
    int64_t k_stride_h, int64_t k_stride_n, int64_t v_stride_b, int64_t v_stride_h,
    int64_t v_stride_n, int dtype_code, int midpoint_affine, int32_t* anchors,
    const int32_t* q_perm, const int32_t* kv_perm, void* workspace, size_t workspace_bytes,
    void* stream_ptr) {
  VRangeJob range_job;
  VCodesJob codes_job;
  int status = v_quantize_jobs(v, v_codes, v_scale, v_center, batch, kv_heads, k_len, head_dim,
                               padded_len, v_stride_b, v_stride_h, v_stride_n, dtype_code,
                               midpoint_affine, kv_perm, workspace, workspace_bytes, &range_job,
                               &codes_job);
  if (status != RISA_B200_OK) return status;
  const bool codes_fused = codes_job.v != nullptr;
  status = quantize_qk_with_v_steps(q, q_codes, q_scale, k, k_codes, k_scale, batch, q_heads, q_len,
                                    kv_heads, k_len, head_dim, cta_k, q_stride_b, q_stride_h,
                                    q_stride_n, k_stride_b, k_stride_h, k_stride_n, dtype_code,
                                    anchors, q_perm, kv_perm, &range_job,
                                    codes_fused ? &codes_job : nullptr, stream_ptr);
  if (status != RISA_B200_OK) return status;
  return quantize_v_after_range(v, v_codes, v_scale, v_center, batch, kv_heads, k_len, head_dim,
                                padded_len, v_stride_b, v_stride_h, v_stride_n, dtype_code,
                                midpoint_affine, kv_perm, workspace, codes_fused, stream_ptr);
}
