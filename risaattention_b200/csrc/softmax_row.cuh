// One query row of the U8 online softmax, written for a thread that owns the whole row of integer
// scores of one key tile (the natural ownership when the accumulator lives in tensor memory, where
// lane == row; the row-per-thread integer kernel uses the same code).
//
// Numerics follow the reference project's csrc/kernels/attention_softmax.cuh:27-293 and
// attention_int8.cuh:456-865.  That code is organised around mma.sync fragments: four lanes share a
// row, lane g of the four owns key columns {2g, 2g+1, 2g+8, 2g+9} + 16j, has its own K scale group
// g = (column % 8) / 2, its own running denominator partial, and the row maximum is the maximum of
// the four lanes' scaled maxima.  A row-owning thread reproduces that by keeping four "virtual
// lanes".  The probability bytes of virtual lane g inside 16-key group j are exactly storage bytes
// 4g..4g+3 of that group in the packed V order {0,1,8,9,2,3,10,11,4,5,12,13,6,7,14,15}, so the
// packed word P[4j+g] is both the MMA operand word and the lane's four-probability sum operand.
#pragma once
#include "common.cuh"

namespace risa_b200 {

constexpr float kLog2e = 1.44269504088896340736f;
constexpr float kU8Offset = 7.9943534f;

enum ScoreKind : int {
  kScoresInt = 0,     // unmasked, non-causal, scale > 0: exact integer scores, scale fused in
  kScoresScaled = 1,  // scores pre-multiplied by the scale (masks, causal, scale <= 0)
};

struct RowState {
  float m;     // running maximum (log2 domain, includes the U8 offset)
  float d[4];  // denominator partials of the four virtual lanes
};

__device__ __forceinline__ void row_state_init(RowState& s) {
  s.m = -50000.0f;
  s.d[0] = s.d[1] = s.d[2] = s.d[3] = 0.0f;
}

__device__ __forceinline__ uint32_t to_u8(float p) {
  uint32_t q;
  asm("cvt.rni.sat.u8.f32 %0, %1;" : "=r"(q) : "f"(p));
  return q;
}

// Column of virtual lane g, 16-key group j, element e (0..3).
__device__ __forceinline__ constexpr int lane_column(int j, int g, int e) {
  return 16 * j + 2 * g + (e & 1) + 8 * (e >> 1);
}

struct TileResult {
  float tile_m;    // tile maximum (log2 domain, offset included)
  float o_scale;   // factor for the running output / denominator
  float w;         // weight of this tile's integer products
  uint32_t numer;  // sum of the tile's U8 probabilities
};

// x: scores of the tile as floats; for kScoresInt they are exact integers (tail keys already
// replaced by -1e30 in the last tile), for kScoresScaled they are already in the log2 domain with
// masked entries at -inf.  sc: per virtual lane scale (unused for kScoresScaled).  LAST selects the
// reference's generic last-visited-tile arithmetic: lane maxima start at -50000 and the
// denominator takes one FMA per pair of 16-key groups.  P receives CTA_K/4 packed words in storage
// order.  When EXACT_D is false the denominator is kept as a single partial (d[0]); outputs then
// agree with the reference to rounding, not bit for bit.
template <int CTA_K, int KIND, bool LAST, bool EXACT_D>
__device__ __forceinline__ TileResult softmax_tile(const float (&x)[CTA_K], const float (&sc)[4],
                                                   RowState& st, uint32_t (&P)[CTA_K / 4]) {
  constexpr int G16 = CTA_K / 16;
  float gmax[4];
#pragma unroll
  for (int g = 0; g < 4; ++g) {
    float mx = (KIND == kScoresInt && !LAST) ? -3.0e38f : -50000.0f;
#pragma unroll
    for (int j = 0; j < G16; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) mx = fmaxf(mx, x[lane_column(j, g, e)]);
    gmax[g] = KIND == kScoresScaled ? mx - kU8Offset : fmaf(mx, sc[g], -kU8Offset);
  }
  TileResult r;
  r.tile_m = fmaxf(fmaxf(gmax[0], gmax[1]), fmaxf(gmax[2], gmax[3]));
  const float neg_m = -r.tile_m;
  const float m_prev = st.m;
  st.m = fmaxf(m_prev, r.tile_m);
  const float smaller = ex2_approx(-fabsf(m_prev - r.tile_m));
  r.o_scale = m_prev < r.tile_m ? smaller : 1.0f;
  r.w = r.tile_m < m_prev ? smaller : 1.0f;
  r.numer = 0;
  float dprev[4];
#pragma unroll
  for (int g = 0; g < 4; ++g) { dprev[g] = st.d[g]; st.d[g] *= r.o_scale; }
#pragma unroll
  for (int j = 0; j < G16; ++j) {
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      uint32_t word = 0;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float s = x[lane_column(j, g, e)];
        const float p = KIND == kScoresScaled ? ex2_approx(s + neg_m)
                                            : ex2_approx(fmaf(s, sc[g], neg_m));
        word |= to_u8(p) << (8 * e);
      }
      P[4 * j + g] = word;
    }
  }
#pragma unroll
  for (int g = 0; g < 4; ++g) {
    if constexpr (LAST) {
      // generic path of the last visited tile: one FMA per pair of 16-key groups
#pragma unroll
      for (int j = 0; j < G16; j += 2) {
        const uint32_t s8 = __dp4a(P[4 * j + 4 + g], 0x01010101u, __dp4a(P[4 * j + g], 0x01010101u, 0u));
        r.numer += s8;
        if constexpr (EXACT_D) {
          // The reference's compiler fuses the rescale of the running denominator with the first
          // addend of this tile (d * o_scale + round(s * w) in one FMA); later addends fuse the
          // other way.  Found by comparing final denominators bit for bit on the GPU.
          if (j == 0) st.d[g] = fmaf(dprev[g], r.o_scale, __fmul_rn(static_cast<float>(s8), r.w));
          else st.d[g] = fmaf(static_cast<float>(s8), r.w, st.d[g]);
        }
      }
    } else {
#pragma unroll
      for (int j = 0; j < G16; ++j) {
        const uint32_t s4 = __dp4a(P[4 * j + g], 0x01010101u, 0u);
        r.numer += s4;
        if constexpr (EXACT_D) st.d[g] = fmaf(static_cast<float>(s4), r.w, st.d[g]);
      }
    }
  }
  if constexpr (!EXACT_D) st.d[0] = fmaf(static_cast<float>(r.numer), r.w, st.d[0]);
  return r;
}

__device__ __forceinline__ float row_denominator(const RowState& st) {
  return (st.d[0] + st.d[1]) + (st.d[2] + st.d[3]);
}

__device__ __forceinline__ float row_lse(float denom, float m) {
  return denom > 0.0f ? __fdividef(lg2_approx(denom) + m, kLog2e) : -INFINITY;
}

}  // namespace risa_b200
