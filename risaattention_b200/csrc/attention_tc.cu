// Tensor-core INT8 attention for B200 (sm_100a): S = Q.K^T (S8 x S8) and P.V (U8 x S8) run as
// tcgen05 kind::i8 MMAs whose INT32 accumulators live in tensor memory; Q, K and V tiles arrive by
// TMA into 128-byte-swizzled shared memory; the FP32 online softmax, the per-tile FP32 rescale of
// the output and the epilogue run on ordinary warps that read the accumulators with tcgen05.ld.
//
// One CTA = 128 queries of one (batch, head), key tiles of 128, head_dim 128.  Warp roles:
//   warps 0-3  softmax:    thread r owns query row r (tensor-memory lane r): two passes over the
//                          128 scores of a tile (maxima, then U8 probabilities written to shared
//                          memory as the A operand of P.V, bytes placed in the packed V order);
//   warps 4-7  correction: thread r owns the FP32 output row r in registers; per tile
//                          O = O * o_scale + float(P.V) * w, then the epilogue and the store;
//   warp 8     producer:   TMA loads of Q and of the K / V tile ring;
//   warp 9     MMA issue:  one thread issues the MMAs; QK^T of tile t+1 is issued before P.V of
//                          tile t so the tensor pipe works while the softmax of tile t runs.
// Tensor memory (512 columns): S double-buffered (2 x 128), P.V accumulator double-buffered
// (2 x 128).  The U8 probabilities are scaled to the TILE maximum (full 8-bit resolution per tile),
// so every tile's integer P.V has its own weight and must be folded into FP32 by the correction
// warps; nothing accumulates across tiles inside tensor memory.
// Numerics: reference csrc/kernels/attention_int8.cuh:427-1026 via softmax_row.cuh; the integer
// products are exact, so probabilities, capture statistics and block masses are bit-identical to the
// row-per-thread kernel; without capture the denominator is kept in one partial instead of four.
// Every mbarrier wait is bounded (tc_ptx.cuh): a protocol error sets a device status word and the
// CTA drains and exits instead of spinning.
#include "attention_common.cuh"
#include "tc_ptx.cuh"

#include <cuda.h>
#include <mutex>

namespace risa_b200 {
namespace {

using namespace tc;

constexpr int kStages = 3;            // K / V ring depth
constexpr int kTile = 128 * 128;      // bytes of one 128 x 128 INT8 tile
constexpr int kThreads = 320;

__device__ unsigned int g_tc_status;  // first failing wait site since the last status query

struct SmemLayout {
  static constexpr int q = 0;
  static constexpr int k = q + kTile;
  static constexpr int v = k + kStages * kTile;
  static constexpr int p = v + kStages * kTile;
  static constexpr int scales = p + 2 * kTile;          // float2 [2][128]
  static constexpr int fin = scales + 2 * 128 * 8;      // float2 [128]
  static constexpr int bars = fin + 128 * 8;            // 8-byte mbarriers
  static constexpr int n_bars = 2 + 4 * kStages + 10;
  static constexpr int tmem_slot = bars + n_bars * 8;
  static constexpr int total = tmem_slot + 16;
};
constexpr size_t kSmemBytes = SmemLayout::total + 1024;  // room to align the base to 1024

struct TileSeq {
  int n_iter;
  const int32_t* ids;
  __device__ __forceinline__ int tile(int it) const { return ids ? __ldg(ids + it) : it; }
};

__device__ __forceinline__ TileSeq tile_sequence(const AttentionArgs& a, int64_t bh, int bx,
                                                 int n_q, int n_k, bool capture) {
  TileSeq s;
  s.ids = nullptr;
  if (a.row_offsets) {
    const int64_t r = bh * n_q + bx;
    const int start = __ldg(a.row_offsets + r);
    s.n_iter = __ldg(a.row_offsets + r + 1) - start;
    s.ids = a.block_indices + start;
  } else if (a.is_causal && !capture) {
    s.n_iter = (min(a.k_len, (bx + 1) * 128) + 127) / 128;
  } else {
    s.n_iter = n_k;
  }
  return s;
}

template <bool CAPTURE>
__global__ __launch_bounds__(kThreads, 1) void attention_tc_kernel(
    const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
    const __grid_constant__ CUtensorMap map_v, const AttentionArgs a) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t sbase = smem_u32(smem);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int bx = blockIdx.x, head = blockIdx.y, batch = blockIdx.z;
  const int kv_head = head / (a.q_heads / a.kv_heads);
  const int n_k = (a.k_len + 127) / 128, n_q = gridDim.x;
  const int64_t bh = int64_t(batch) * a.q_heads + head;
  const int64_t kvh = int64_t(batch) * a.kv_heads + kv_head;
  unsigned int* error = &g_tc_status;

  // barrier addresses
  const uint32_t bar0 = sbase + SmemLayout::bars;
  auto bar = [&](int i) { return bar0 + 8u * i; };
  const int B_QFULL = 0, B_FIN = 1, B_KFULL = 2, B_KEMPTY = B_KFULL + kStages,
            B_VFULL = B_KEMPTY + kStages, B_VEMPTY = B_VFULL + kStages,
            B_SFULL = B_VEMPTY + kStages, B_SFREE = B_SFULL + 2, B_PFULL = B_SFREE + 2,
            B_PFREE = B_PFULL + 2, B_OFULL = B_PFREE + 2, B_OFREE = B_OFULL + 2;

  if (threadIdx.x == 0) {
    mbar_init(bar(B_QFULL), 1);
    mbar_init(bar(B_FIN), 128);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(bar(B_KFULL + s), 1);
      mbar_init(bar(B_KEMPTY + s), 1);
      mbar_init(bar(B_VFULL + s), 1);
      mbar_init(bar(B_VEMPTY + s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar(B_SFULL + b), 1);
      mbar_init(bar(B_SFREE + b), 128);
      mbar_init(bar(B_PFULL + b), 128);
      mbar_init(bar(B_PFREE + b), 1);
      mbar_init(bar(B_OFULL + b), 1);
      mbar_init(bar(B_OFREE + b), 128);
    }
    mbar_init_fence();
  }
  if (warp == 9) tmem_alloc(sbase + SmemLayout::tmem_slot, 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(smem + SmemLayout::tmem_slot);
  const uint32_t tmem_s[2] = {tmem, tmem + 128};
  const uint32_t tmem_o[2] = {tmem + 256, tmem + 384};

  const TileSeq seq = tile_sequence(a, bh, bx, n_q, n_k, CAPTURE);
  float2* scales = reinterpret_cast<float2*>(smem + SmemLayout::scales);
  float2* fin = reinterpret_cast<float2*>(smem + SmemLayout::fin);

  if (warp == 8) {
    // ------------------------------------------------------------------ producer
    if (lane == 0) {
      tma_prefetch_descriptor(&map_q);
      tma_prefetch_descriptor(&map_k);
      tma_prefetch_descriptor(&map_v);
      mbar_expect_tx(bar(B_QFULL), kTile);
      tma_load_3d(sbase + SmemLayout::q, &map_q, bar(B_QFULL), 0, bx * 128, int(bh));
      bool ok = true;
      int issued = 0;
      for (int it = 0; it < seq.n_iter && ok; ++it) {
        const int s = it % kStages, r = it / kStages;
        const int tile = seq.tile(it);
        ok = mbar_wait(bar(B_KEMPTY + s), (r & 1) ^ 1, error, 101);
        if (!ok) break;
        mbar_expect_tx(bar(B_KFULL + s), kTile);
        tma_load_3d(sbase + SmemLayout::k + s * kTile, &map_k, bar(B_KFULL + s), 0, tile * 128,
                    int(kvh));
        ok = mbar_wait(bar(B_VEMPTY + s), (r & 1) ^ 1, error, 102);
        if (!ok) {
          // the K load of this stage is in flight: let it land before the CTA can exit
          mbar_wait(bar(B_KFULL + s), r & 1, error, 103);
          break;
        }
        mbar_expect_tx(bar(B_VFULL + s), kTile);
        tma_load_3d(sbase + SmemLayout::v + s * kTile, &map_v, bar(B_VFULL + s), tile * 128, 0,
                    int(kvh));
        issued = it + 1;
      }
      if (!ok) {
        // drain: every issued load must have completed before shared memory is released
        mbar_wait(bar(B_QFULL), 0, error, 104);
        for (int it = max(0, issued - kStages); it < issued; ++it) {
          const int s = it % kStages, r = it / kStages;
          mbar_wait(bar(B_KFULL + s), r & 1, error, 105);
          mbar_wait(bar(B_VFULL + s), r & 1, error, 106);
        }
      }
    }
  } else if (warp == 9) {
    // ------------------------------------------------------------------ MMA issue
    if (lane == 0) {
      constexpr uint32_t idesc_qk = idesc_i8(true, true, 128);
      constexpr uint32_t idesc_pv = idesc_i8(false, true, 128);
      const uint64_t desc_q = smem_desc_k128(sbase + SmemLayout::q);
      bool ok = mbar_wait(bar(B_QFULL), 0, error, 201);
      auto issue_qk = [&](int it) -> bool {
        const int b = it & 1, u = it >> 1, s = it % kStages, r = it / kStages;
        if (!mbar_wait(bar(B_KFULL + s), r & 1, error, 202)) return false;
        if (!mbar_wait(bar(B_SFREE + b), (u & 1) ^ 1, error, 203)) return false;
        tc_fence_after();
        const uint64_t desc_k = smem_desc_k128(sbase + SmemLayout::k + s * kTile);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          mma_i8(tmem_s[b], desc_q + 2 * kk, desc_k + 2 * kk, idesc_qk, kk > 0);
        mma_commit(bar(B_SFULL + b));
        mma_commit(bar(B_KEMPTY + s));
        return true;
      };
      if (ok && seq.n_iter > 0) ok = issue_qk(0);
      for (int it = 0; it < seq.n_iter && ok; ++it) {
        if (it + 1 < seq.n_iter) {
          ok = issue_qk(it + 1);
          if (!ok) break;
        }
        const int b = it & 1, u = it >> 1, s = it % kStages, r = it / kStages;
        ok = mbar_wait(bar(B_PFULL + b), u & 1, error, 204) &&
             mbar_wait(bar(B_VFULL + s), r & 1, error, 205) &&
             mbar_wait(bar(B_OFREE + b), (u & 1) ^ 1, error, 206);
        if (!ok) break;
        tc_fence_after();
        const uint64_t desc_p = smem_desc_k128(sbase + SmemLayout::p + b * kTile);
        const uint64_t desc_v = smem_desc_k128(sbase + SmemLayout::v + s * kTile);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          mma_i8(tmem_o[b], desc_p + 2 * kk, desc_v + 2 * kk, idesc_pv, kk > 0);
        mma_commit(bar(B_OFULL + b));
        mma_commit(bar(B_VEMPTY + s));
        mma_commit(bar(B_PFREE + b));
      }
    }
  } else if (warp < 4) {
    // ------------------------------------------------------------------ softmax
    const int row_in = threadIdx.x;  // 0..127 == tensor-memory lane
    const int row = bx * 128 + row_in;
    const bool row_ok = row < a.q_len;
    const uint32_t lane_base = uint32_t(warp * 32) << 16;
    const bool int_scores = !a.is_causal && a.sm_scale > 0.0f;
    const float scale2 = a.sm_scale * kLog2e;
    const int q_groups_per_head = n_q * 32;
    const float q_scale = __ldg(a.q_scale + bh * q_groups_per_head + (row / 32) * 8 + (row & 7));
    const float* k_scale = a.k_scale + kvh * (n_k * 4);
    CaptureLayout cap;
    if constexpr (CAPTURE) cap = capture_layout(a, n_q, n_k);
    const int64_t grow = bh * a.q_len + row;
    unsigned char* p_row[2] = {smem + SmemLayout::p + row_in * 128,
                               smem + SmemLayout::p + kTile + row_in * 128};
    RowState st;
    row_state_init(st);
    bool ok = true;

    for (int it = 0; it < seq.n_iter && ok; ++it) {
      const int b = it & 1, u = it >> 1;
      const int tile = seq.tile(it);
      const bool last = it == seq.n_iter - 1;
      const int c0 = tile * 128;
      float sc[4];
#pragma unroll
      for (int g = 0; g < 4; ++g) sc[g] = scale2 * (q_scale * __ldg(k_scale + tile * 4 + g));
      ok = mbar_wait(bar(B_SFULL + b), u & 1, error, 301);
      if (!ok) break;
      tc_fence_after();

      // scores of one 32-column chunk as the floats the softmax consumes
      auto load_chunk = [&](int c, float* x) {
        uint32_t raw[32];
        tmem_load32(tmem_s[b] + lane_base + 32 * c, raw);
        tmem_load_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const int kv = c0 + 32 * c + i;
          float s = static_cast<float>(static_cast<int>(raw[i]));
          if (int_scores) {
            if (last && kv >= a.k_len) s = -1.0e30f;
          } else {
            s *= sc[(i & 7) >> 1];
            if (a.is_causal && kv > row) s = -INFINITY;
            if (last && kv >= a.k_len) s = -INFINITY;
          }
          x[i] = s;
        }
      };

      // pass 1: tile maximum
      TileMax tm;
      if (int_scores && !last) tile_max_init<kScoresInt, false>(tm);
      else tile_max_init<kScoresScaled, true>(tm);  // -50000 start (every other case)
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        float x[32];
        load_chunk(c, x);
        tile_max_chunk(x, tm);
      }
      const float tile_m = int_scores ? tile_max_finish<kScoresInt>(tm, sc)
                                      : tile_max_finish<kScoresScaled>(tm, sc);
      const TileScales ts = tile_begin(st, tile_m);

      // hand (o_scale, w) to the correction warps once they are done with this buffer's last use
      ok = mbar_wait(bar(B_OFREE + b), (u & 1) ^ 1, error, 302) &&
           mbar_wait(bar(B_PFREE + b), (u & 1) ^ 1, error, 303);
      if (!ok) break;
      scales[b * 128 + row_in] = make_float2(ts.o_scale, ts.w);

      // pass 2: probabilities -> shared memory (128-byte swizzle: 16-byte chunk index ^ row % 8)
      uint32_t numer = 0;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        float x[32];
        uint32_t P[8];
        load_chunk(c, x);
        if (int_scores) {
          if (last) tile_exp_chunk<kScoresInt, true, CAPTURE>(x, sc, ts, c == 0, st, P, numer);
          else tile_exp_chunk<kScoresInt, false, CAPTURE>(x, sc, ts, c == 0, st, P, numer);
        } else {
          if (last) tile_exp_chunk<kScoresScaled, true, CAPTURE>(x, sc, ts, c == 0, st, P, numer);
          else tile_exp_chunk<kScoresScaled, false, CAPTURE>(x, sc, ts, c == 0, st, P, numer);
        }
        const int sw = row_in & 7;
        *reinterpret_cast<uint4*>(p_row[b] + (((2 * c) ^ sw) << 4)) =
            make_uint4(P[0], P[1], P[2], P[3]);
        *reinterpret_cast<uint4*>(p_row[b] + (((2 * c + 1) ^ sw) << 4)) =
            make_uint4(P[4], P[5], P[6], P[7]);
      }
      tile_end<CAPTURE>(st, ts, numer);
      tc_fence_before();
      mbar_arrive(bar(B_SFREE + b));
      fence_async_smem();
      mbar_arrive(bar(B_PFULL + b));

      if constexpr (CAPTURE) {
        if (row_ok) {
          if (last) {
            float* slot = cap.last + grow * 2;
            slot[0] = static_cast<float>(numer);
            slot[1] = ts.tile_m;
          } else {
            uint32_t* slot = cap.full + (grow * (n_k - 1) + it) * 2;
            slot[0] = numer;
            slot[1] = __float_as_uint(ts.tile_m);
          }
        }
      }
    }
    const float denom = CAPTURE ? row_denominator(st) : st.d[0];
    fin[row_in] = make_float2(denom, st.m);
    mbar_arrive(bar(B_FIN));
    if constexpr (CAPTURE) {
      if (row_ok && ok) {
        cap.state[grow * 2] = st.m;
        cap.state[grow * 2 + 1] = denom;
      }
    }
  } else {
    // ------------------------------------------------------------------ correction + epilogue
    const int row_in = threadIdx.x - 128;
    const int row = bx * 128 + row_in;
    const uint32_t lane_base = uint32_t((warp - 4) * 32) << 16;
    float O[128];
#pragma unroll
    for (int i = 0; i < 128; ++i) O[i] = 0.0f;
    bool ok = true;
    for (int it = 0; it < seq.n_iter && ok; ++it) {
      const int b = it & 1, u = it >> 1;
      ok = mbar_wait(bar(B_PFULL + b), u & 1, error, 401);
      if (!ok) break;
      const float2 sw = scales[b * 128 + row_in];
      ok = mbar_wait(bar(B_OFULL + b), u & 1, error, 402);
      if (!ok) break;
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t acc[32];
        tmem_load32(tmem_o[b] + lane_base + 32 * c, acc);
        tmem_load_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float o = O[32 * c + i];
          o *= sw.x;
          O[32 * c + i] = fmaf(static_cast<float>(static_cast<int>(acc[i])), sw.y, o);
        }
      }
      tc_fence_before();
      mbar_arrive(bar(B_OFREE + b));
    }
    if (ok) ok = mbar_wait(bar(B_FIN), 0, error, 403);
    if (ok && row < a.q_len) {
      const float2 f = fin[row_in];
      const float denom = f.x;
      const float inv = rcp_approx(denom);
      const bool zero = a.is_causal && !(denom > 0.0f);
      const float* vs = a.v_scale + kvh * 128;
      const float* vc = a.v_center + kvh * 128;
      char* o_row = static_cast<char*>(a.o) +
                    2 * (batch * a.o_stride_b + head * a.o_stride_h + int64_t(row) * a.o_stride_n);
#pragma unroll
      for (int ch = 0; ch < 128; ch += 8) {
        uint32_t packed[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          float r0 = fmaf(O[ch + 2 * i] * inv, __ldg(vs + ch + 2 * i), __ldg(vc + ch + 2 * i));
          float r1 = fmaf(O[ch + 2 * i + 1] * inv, __ldg(vs + ch + 2 * i + 1),
                          __ldg(vc + ch + 2 * i + 1));
          if (zero) r0 = r1 = 0.0f;
          if (a.out_dtype_code == 1) {
            const __half2 h = __floats2half2_rn(r0, r1);
            packed[i] = *reinterpret_cast<const uint32_t*>(&h);
          } else {
            const __nv_bfloat162 h = __floats2bfloat162_rn(r0, r1);
            packed[i] = *reinterpret_cast<const uint32_t*>(&h);
          }
        }
        *reinterpret_cast<uint4*>(o_row + 2 * ch) =
            make_uint4(packed[0], packed[1], packed[2], packed[3]);
      }
      if (a.lse) a.lse[bh * a.q_len + row] = row_lse(denom, f.y);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 9) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

// ---- host side ---------------------------------------------------------------------------------
using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                              const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                              const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn encode_fn() {
  static EncodeFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult result;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &result) ==
            cudaSuccess &&
        result == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeFn>(ptr);
  });
  return fn;
}

// 3-D byte tensor {inner, rows, slabs} with a {128, 128, 1} box and the 128-byte swizzle.
bool make_map(CUtensorMap* map, const void* base, uint64_t inner, uint64_t rows, uint64_t slabs) {
  const cuuint64_t dims[3] = {inner, rows, slabs};
  const cuuint64_t strides[2] = {inner, inner * rows};
  const cuuint32_t box[3] = {128, 128, 1};
  const cuuint32_t elem[3] = {1, 1, 1};
  return encode_fn()(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(base), dims, strides,
                     box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                     CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

bool attention_tc_supported(const AttentionArgs& a) {
  return a.head_dim == 128 && a.cta_k == 128 && a.mask == nullptr && a.key_mask_tiles == nullptr &&
         encode_fn() != nullptr && reinterpret_cast<uintptr_t>(a.o) % 16 == 0 &&
         a.o_stride_b % 8 == 0 && a.o_stride_h % 8 == 0 && a.o_stride_n % 8 == 0;
}

int attention_tc(const AttentionArgs& a, cudaStream_t stream) {
  const int n_k = (a.k_len + 127) / 128;
  CUtensorMap map_q, map_k, map_v;
  if (!make_map(&map_q, a.q, 128, uint64_t(a.q_len), uint64_t(a.batch) * a.q_heads) ||
      !make_map(&map_k, a.k, 128, uint64_t(a.k_len), uint64_t(a.batch) * a.kv_heads) ||
      !make_map(&map_v, a.v, uint64_t(n_k) * 128, 128, uint64_t(a.batch) * a.kv_heads))
    return fail(RISA_B200_CUDA, "attention: tensor map creation failed");
  const bool capture = a.block_mass != nullptr;
  auto kernel = capture ? attention_tc_kernel<true> : attention_tc_kernel<false>;
  static thread_local int configured[2] = {-1, -1};
  int device = -1;
  cudaGetDevice(&device);
  if (configured[capture] != device) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         int(kSmemBytes));
    if (e != cudaSuccess)
      return fail(RISA_B200_CUDA, "attention: cannot reserve %zu bytes of shared memory: %s",
                  kSmemBytes, cudaGetErrorString(e));
    configured[capture] = device;
  }
  const dim3 grid((a.q_len + 127) / 128, a.q_heads, a.batch);
  kernel<<<grid, kThreads, kSmemBytes, stream>>>(map_q, map_k, map_v, a);
  return check_launch("attention (tensor-core kernel)");
}

}  // namespace risa_b200

extern "C" int risa_b200_device_status(void) {
  unsigned int status = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&status, risa_b200::g_tc_status, sizeof(status)) != cudaSuccess)
    return risa_b200::fail(RISA_B200_CUDA, "device status: %s",
                           cudaGetErrorString(cudaGetLastError()));
  if (status != 0) {
    cudaMemcpyToSymbol(risa_b200::g_tc_status, &zero, sizeof(zero));
    return risa_b200::fail(RISA_B200_DEVICE,
                           "attention kernel gave up waiting at site %u (bounded wait expired)",
                           status);
  }
  return RISA_B200_OK;
}
