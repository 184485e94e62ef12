// Row-per-thread INT8 attention kernel: every variant of the fused attention call (dense, additive
// or boolean masks, broadcast key masks with tile lists, causal, CSR sparse reuse, block-mass
// capture, LSE, head_dim 64/128/256, key tiles of 64/128) on plain integer dot-product
// instructions.  It is the complete-coverage path and the on-device cross-check of the tensor-core
// kernel, which takes over the shapes it supports.
//
// One CTA = 128 query rows of one (batch, head); thread r owns row r: its scores of the current key
// tile, its softmax state and (in shared memory, channel-major) its output accumulators.  Q, K and
// V tiles are staged in shared memory; K/V words are read warp-uniformly (broadcast).
// Semantics: reference csrc/kernels/attention_int8.cuh:145-1088 (tile loop, first/last tile rules,
// capture statistics, epilogue, LSE) and attention_masks.cuh:27-164.
#include "attention_common.cuh"

namespace risa_b200 {
namespace {

// unsigned probabilities x signed values
__device__ __forceinline__ int dp4a_u8s8(uint32_t p, uint32_t v, int acc) {
  int out;
  asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(out) : "r"(p), "r"(v), "r"(acc));
  return out;
}

template <int D, int CTA_K>
constexpr size_t rows_smem_bytes() {
  return size_t(128) * D            // Q codes, word-major [D/4][128]
         + size_t(CTA_K) * D        // K tile [CTA_K][D]
         + size_t(D) * CTA_K        // V tile [D][CTA_K]
         + size_t(D) * 128 * 4;     // output accumulators [D][128] f32
}

template <int D, int CTA_K, bool MASKED, bool CAPTURE>
__global__ __launch_bounds__(128) void attention_rows_kernel(const AttentionArgs a) {
  extern __shared__ __align__(16) unsigned char smem[];
  uint32_t* q_s = reinterpret_cast<uint32_t*>(smem);                    // [D/4][128]
  uint32_t* k_s = q_s + 32 * D;                                         // [CTA_K][D/4]
  uint32_t* v_s = k_s + CTA_K * D / 4;                                  // [D][CTA_K/4]
  float* o_s = reinterpret_cast<float*>(v_s + D * CTA_K / 4);           // [D][128]
  constexpr int DW = D / 4, KW = CTA_K / 4;

  const int tid = threadIdx.x;
  const int bx = blockIdx.x, head = blockIdx.y, batch = blockIdx.z;
  const int kv_head = head / (a.q_heads / a.kv_heads);
  const int n_k = (a.k_len + CTA_K - 1) / CTA_K;
  const int n_q = gridDim.x;
  const int padded = n_k * CTA_K;
  const int row = bx * 128 + tid;
  const bool row_ok = row < a.q_len;
  const int64_t bh = static_cast<int64_t>(batch) * a.q_heads + head;
  const int64_t kvh = static_cast<int64_t>(batch) * a.kv_heads + kv_head;
  const int8_t* q_g = a.q + (bh * a.q_len) * D;
  const int8_t* k_g = a.k + (kvh * a.k_len) * D;
  const int8_t* v_g = a.v + (kvh * D) * padded;

  // ---- stage Q (zero rows past the end) and clear the accumulators -------------------------
  for (int idx = tid; idx < 128 * DW; idx += 128) {
    const int r = idx / DW, wd = idx % DW;
    const int gr = bx * 128 + r;
    q_s[wd * 128 + r] =
        gr < a.q_len ? __ldg(reinterpret_cast<const uint32_t*>(q_g + int64_t(gr) * D) + wd) : 0u;
  }
  for (int idx = tid; idx < D * 128; idx += 128) o_s[idx] = 0.0f;

  // ---- tile list -----------------------------------------------------------------------------
  int n_iter;
  const int32_t* tile_ids = nullptr;
  bool key_list = false;
  if (a.row_offsets) {
    const int64_t r = bh * n_q + bx;
    const int start = a.row_offsets[r];
    n_iter = a.row_offsets[r + 1] - start;
    tile_ids = a.block_indices + start;
  } else if (a.key_mask_tiles) {
    tile_ids = a.key_mask_tiles + bh * (n_k + 1);
    n_iter = tile_ids[n_k];
    key_list = true;
  } else if (a.is_causal && !CAPTURE) {
    n_iter = (min(a.k_len, (bx + 1) * 128) + CTA_K - 1) / CTA_K;
  } else {
    n_iter = n_k;
  }

  const bool int_scores = !MASKED && !a.is_causal && a.sm_scale > 0.0f;
  const float scale2 = a.sm_scale * kLog2e;
  const int q_tile_rows = D == 256 ? 16 : 32;
  const int q_groups_per_head = n_q * (128 / q_tile_rows) * 8;
  const int q_group = (min(row, n_q * 128 - 1) / q_tile_rows) * 8 + (row & 7);
  const float q_scale = __ldg(a.q_scale + bh * q_groups_per_head + q_group);
  const float* k_scale = a.k_scale + kvh * (n_k * 4);

  RowState st;
  row_state_init(st);

  CaptureLayout cap;
  if constexpr (CAPTURE) cap = capture_layout(a, n_q, n_k);
  const int64_t grow = bh * a.q_len + row;

  for (int it = 0; it < n_iter; ++it) {
    const int tile = tile_ids ? tile_ids[it] : it;
    const bool last_iter = it == n_iter - 1;
    const bool last_rules = last_iter && !(key_list && tile + 1 < n_k);
    const int c0 = tile * CTA_K;
    __syncthreads();  // previous tile's K/V no longer in use (also orders the Q staging)
    for (int idx = tid; idx < CTA_K * DW; idx += 128) {
      const int r = idx / DW, wd = idx % DW;
      k_s[idx] = c0 + r < a.k_len
                     ? __ldg(reinterpret_cast<const uint32_t*>(k_g + int64_t(c0 + r) * D) + wd)
                     : 0u;
    }
    for (int idx = tid; idx < D * KW; idx += 128) {
      const int ch = idx / KW, wd = idx % KW;
      v_s[idx] = __ldg(reinterpret_cast<const uint32_t*>(v_g + int64_t(ch) * padded + c0) + wd);
    }
    __syncthreads();

    // ---- S = q . k^T for this row -------------------------------------------------------------
    float x[CTA_K];
    {
      int acc[CTA_K];
#pragma unroll
      for (int c = 0; c < CTA_K; ++c) acc[c] = 0;
      for (int w0 = 0; w0 < DW; w0 += 8) {
        uint32_t qw[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) qw[i] = q_s[(w0 + i) * 128 + tid];
#pragma unroll
        for (int c = 0; c < CTA_K; ++c) {
          const uint4 k0 = *reinterpret_cast<const uint4*>(k_s + c * DW + w0);
          const uint4 k1 = *reinterpret_cast<const uint4*>(k_s + c * DW + w0 + 4);
          int s = acc[c];
          s = __dp4a(int(qw[0]), int(k0.x), s);
          s = __dp4a(int(qw[1]), int(k0.y), s);
          s = __dp4a(int(qw[2]), int(k0.z), s);
          s = __dp4a(int(qw[3]), int(k0.w), s);
          s = __dp4a(int(qw[4]), int(k1.x), s);
          s = __dp4a(int(qw[5]), int(k1.y), s);
          s = __dp4a(int(qw[6]), int(k1.z), s);
          s = __dp4a(int(qw[7]), int(k1.w), s);
          acc[c] = s;
        }
      }
#pragma unroll
      for (int c = 0; c < CTA_K; ++c) x[c] = static_cast<float>(acc[c]);
    }

    float sc[4];
#pragma unroll
    for (int g = 0; g < 4; ++g) sc[g] = scale2 * (q_scale * __ldg(k_scale + tile * 4 + g));

    uint32_t P[KW];
    TileResult tr;
    if (int_scores) {
      if (last_rules) {
#pragma unroll
        for (int c = 0; c < CTA_K; ++c)
          if (c0 + c >= a.k_len) x[c] = -1.0e30f;
        tr = softmax_tile<CTA_K, kScoresInt, true, true>(x, sc, st, P);
      } else {
        tr = softmax_tile<CTA_K, kScoresInt, false, true>(x, sc, st, P);
      }
    } else {
#pragma unroll
      for (int c = 0; c < CTA_K; ++c) {
        const int g = (c & 7) >> 1;
        const int kv = c0 + c;
        float s;
        if constexpr (MASKED) s = apply_mask(a, batch, head, row, kv, row_ok, x[c], sc[g]);
        else s = x[c] * sc[g];
        if (a.is_causal && kv > row) s = -INFINITY;
        if (last_rules && kv >= a.k_len) s = -INFINITY;
        x[c] = s;
      }
      tr = last_rules ? softmax_tile<CTA_K, kScoresScaled, true, true>(x, sc, st, P)
                      : softmax_tile<CTA_K, kScoresScaled, false, true>(x, sc, st, P);
    }

    if constexpr (CAPTURE) {
      if (row_ok) {
        if (last_iter) {
          float* slot = cap.last + grow * 2;
          slot[0] = static_cast<float>(tr.numer);
          slot[1] = tr.tile_m;
        } else {
          uint32_t* slot = cap.full + (grow * (n_k - 1) + it) * 2;
          slot[0] = tr.numer;
          slot[1] = __float_as_uint(tr.tile_m);
        }
      }
    }

    // ---- O = O * o_scale + (P . V) * w ----------------------------------------------------------
    for (int ch = 0; ch < D; ++ch) {
      int accv = 0;
#pragma unroll
      for (int wd = 0; wd < KW; wd += 4) {
        const uint4 vv = *reinterpret_cast<const uint4*>(v_s + ch * KW + wd);
        accv = dp4a_u8s8(P[wd], vv.x, accv);
        accv = dp4a_u8s8(P[wd + 1], vv.y, accv);
        accv = dp4a_u8s8(P[wd + 2], vv.z, accv);
        accv = dp4a_u8s8(P[wd + 3], vv.w, accv);
      }
      float o = o_s[ch * 128 + tid];
      o *= tr.o_scale;
      o_s[ch * 128 + tid] = fmaf(static_cast<float>(accv), tr.w, o);
    }
  }

  // ---- epilogue ---------------------------------------------------------------------------------
  const float denom = row_denominator(st);
  if constexpr (CAPTURE) {
    if (row_ok) {
      cap.state[grow * 2] = st.m;
      cap.state[grow * 2 + 1] = denom;
    }
  }
  if (row_ok) {
    const float inv = rcp_approx(denom);
    const bool check_valid = MASKED || a.is_causal;
    const bool valid = denom > 0.0f;
    const float* vs = a.v_scale + kvh * D;
    const float* vc = a.v_center + kvh * D;
    char* o_row = static_cast<char*>(a.o) +
                  2 * (batch * a.o_stride_b + head * a.o_stride_h + int64_t(row) * a.o_stride_n);
    for (int ch = 0; ch < D; ch += 2) {
      float r0 = fmaf(o_s[ch * 128 + tid] * inv, __ldg(vs + ch), __ldg(vc + ch));
      float r1 = fmaf(o_s[(ch + 1) * 128 + tid] * inv, __ldg(vs + ch + 1), __ldg(vc + ch + 1));
      if (check_valid && !valid) r0 = r1 = 0.0f;
      store_pair(o_row + 2 * ch, r0, r1, a.out_dtype_code);
    }
    if (a.lse) a.lse[grow] = row_lse(denom, st.m);
  }
}

template <int D, int CTA_K, bool MASKED, bool CAPTURE>
int launch_rows(const AttentionArgs& a, cudaStream_t stream) {
  constexpr size_t bytes = rows_smem_bytes<D, CTA_K>();
  auto kernel = attention_rows_kernel<D, CTA_K, MASKED, CAPTURE>;
  // The attribute is per kernel and device; set it once per (thread, device).
  static thread_local int configured_device = -1;
  int device = -1;
  cudaGetDevice(&device);
  if (device != configured_device) {
    cudaError_t e =
        cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(bytes));
    if (e != cudaSuccess)
      return fail(RISA_B200_CUDA, "attention: cannot reserve %zu bytes of shared memory: %s",
                  bytes, cudaGetErrorString(e));
    configured_device = device;
  }
  const dim3 grid((a.q_len + 127) / 128, a.q_heads, a.batch);
  kernel<<<grid, 128, bytes, stream>>>(a);
  return check_launch("attention (row kernel)");
}

}  // namespace

int attention_rows(const AttentionArgs& a, cudaStream_t stream) {
  const bool masked = a.mask != nullptr;
  const bool capture = a.block_mass != nullptr;
#define RISA_ROWS(D, CK)                                                              \
  (masked ? (capture ? launch_rows<D, CK, true, true>(a, stream)                      \
                     : launch_rows<D, CK, true, false>(a, stream))                    \
          : (capture ? launch_rows<D, CK, false, true>(a, stream)                     \
                     : launch_rows<D, CK, false, false>(a, stream)))
  if (a.head_dim == 64) return RISA_ROWS(64, 64);
  if (a.head_dim == 128) return a.cta_k == 128 ? RISA_ROWS(128, 128) : RISA_ROWS(128, 64);
  return a.cta_k == 128 ? RISA_ROWS(256, 128) : RISA_ROWS(256, 64);
#undef RISA_ROWS
}

}  // namespace risa_b200
