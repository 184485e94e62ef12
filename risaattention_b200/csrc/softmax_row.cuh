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
//
// The tile is processed in chunks of 32 key columns (two 16-key groups) in two passes -- maxima,
// then exponentials -- so a thread never needs more than one chunk of scores in registers.
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

// Column (inside a 32-key chunk) of virtual lane g, 16-key group j (0/1), element e (0..3).
__device__ __forceinline__ constexpr int lane_column(int j, int g, int e) {
  return 16 * j + 2 * g + (e & 1) + 8 * (e >> 1);
}

struct TileMax {
  float g[4];
};

// LAST selects the reference's generic last-visited-tile arithmetic: lane maxima start at -50000
// (as they always do for pre-scaled scores) instead of being unbounded below.
template <int KIND, bool LAST>
__device__ __forceinline__ void tile_max_init(TileMax& t) {
  const float init = (KIND == kScoresInt && !LAST) ? -3.0e38f : -50000.0f;
  t.g[0] = t.g[1] = t.g[2] = t.g[3] = init;
}

// x: NCOL (32 or 16) consecutive key columns starting at a multiple of NCOL.  For kScoresInt they
// are exact integers (tail keys already replaced by -1e30 in the last tile), for kScoresScaled they
// are in the log2 domain with masked entries at -inf.
template <int NCOL = 32>
__device__ __forceinline__ void tile_max_chunk(const float* x, TileMax& t) {
#pragma unroll
  for (int g = 0; g < 4; ++g)
#pragma unroll
    for (int j = 0; j < NCOL / 16; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) t.g[g] = fmaxf(t.g[g], x[lane_column(j, g, e)]);
}

// Tile maximum in the log2 domain, U8 offset included.  sc: per virtual lane score scale.
template <int KIND>
__device__ __forceinline__ float tile_max_finish(const TileMax& t, const float (&sc)[4]) {
  float v[4];
#pragma unroll
  for (int g = 0; g < 4; ++g)
    v[g] = KIND == kScoresScaled ? t.g[g] - kU8Offset : fmaf(t.g[g], sc[g], -kU8Offset);
  return fmaxf(fmaxf(v[0], v[1]), fmaxf(v[2], v[3]));
}

struct TileScales {
  float tile_m;    // tile maximum
  float o_scale;   // factor for the running output / denominator
  float w;         // weight of this tile's integer products
  float dprev[4];  // denominator partials before rescaling (first addend of the last tile)
};

__device__ __forceinline__ TileScales tile_begin(RowState& st, float tile_m) {
  TileScales s;
  s.tile_m = tile_m;
  const float m_prev = st.m;
  st.m = fmaxf(m_prev, tile_m);
  const float smaller = ex2_approx(-fabsf(m_prev - tile_m));
  s.o_scale = m_prev < tile_m ? smaller : 1.0f;
  s.w = tile_m < m_prev ? smaller : 1.0f;
#pragma unroll
  for (int g = 0; g < 4; ++g) {
    s.dprev[g] = st.d[g];
    st.d[g] *= s.o_scale;
  }
  return s;
}

// Probabilities of one chunk of NCOL (32 or 16) keys.  P receives NCOL / 4 packed words in storage
// order (word 4j+g = lane g of 16-key group j), numer accumulates their U8 sum, s4 (optional)
// receives the sum of each word.
// U8 codes: adding 2^23 to a probability in [0, 255.5) rounds it to nearest-even into the low
// mantissa byte (the same integers cvt.rni.sat.u8 gives on this range) and three byte permutes pack
// four of them, which keeps the conversion off the half-rate conversion pipe.  The work is written
// stage by stage over all 32 columns (scale, exponential, round, pack) so that 32 independent
// operations are in flight per stage instead of one dependent chain per word.
// MAD_PACK: the four rounded values of a word are combined by three integer multiply-adds
// (u1 * 2^8 + u0, u3 * 2^8 + u2, hi * 2^16 + lo) instead of three byte permutes, which moves the
// packing from the ALU pipe, the busiest one of the tensor-core kernel, to the FMA pipe.  The float
// bit patterns are 0x4B000000 + e + code with e the amount by which the rounding constant exceeds
// 2^23; everything above bit 31 falls away, so the word comes out as the four codes plus
// 0x4B000000 + e0 + e1 * 2^8 + e2 * 2^16 + e3 * 2^24, which is 0 mod 2^32 for e = (0, 0, 256, 180).
// All four constants are even integers, so ties still round to the same (even) code.  The
// multipliers 2^8 and 2^16 arrive as run-time values (kernel arguments): written as literals they
// would be turned back into shifts on the ALU pipe.
struct PackMultipliers {
  uint32_t by256, by65536;
};

template <int KIND, bool WANT_SUMS, int NCOL = 32, bool MAD_PACK = false>
__device__ __forceinline__ void tile_exp_chunk(const float* x, const float (&sc)[4], float neg_m,
                                               uint32_t* P, uint32_t& numer, uint32_t* s4,
                                               PackMultipliers mul = PackMultipliers{0u, 0u}) {
  // Columns 2k and 2k + 1 share a K scale group, so scale and magic add run as packed FP32 pairs
  // (one instruction for two columns, same per-lane rounding as the scalar form).
  float p[NCOL];
  const uint64_t nm2 = pack_f32x2(neg_m, neg_m);
#pragma unroll
  for (int i = 0; i < NCOL; i += 2) {
    const uint64_t x2 = pack_f32x2(x[i], x[i + 1]);
    uint64_t r;
    if (KIND == kScoresScaled) {
      r = add_f32x2(x2, nm2);
    } else {
      const float s = sc[(i & 7) >> 1];
      r = fma_f32x2(x2, pack_f32x2(s, s), nm2);
    }
    unpack_f32x2(r, p[i], p[i + 1]);
  }
#pragma unroll
  for (int i = 0; i < NCOL; i += 2) {
    p[i] = ex2_approx(p[i]);
    p[i + 1] = ex2_approx(p[i + 1]);
  }
  uint32_t u[NCOL];
  const uint64_t magic2 = pack_f32x2(8388608.0f, 8388608.0f);
  // columns 8..15 of a 16-key group are bytes 2 and 3 of their words
  const uint64_t magic2_upper =
      MAD_PACK ? pack_f32x2(8388608.0f + 256.0f, 8388608.0f + 180.0f) : magic2;
#pragma unroll
  for (int i = 0; i < NCOL; i += 2) {
    float a, b;
    unpack_f32x2(add_f32x2(pack_f32x2(p[i], p[i + 1]), (i & 8) ? magic2_upper : magic2), a, b);
    u[i] = __float_as_uint(a);
    u[i + 1] = __float_as_uint(b);
  }
#pragma unroll
  for (int j = 0; j < NCOL / 16; ++j) {
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      if constexpr (MAD_PACK) {
        uint32_t lo, hi, w;
        asm("mad.lo.u32 %0, %1, %2, %3;"
            : "=r"(lo) : "r"(u[lane_column(j, g, 1)]), "r"(mul.by256), "r"(u[lane_column(j, g, 0)]));
        asm("mad.lo.u32 %0, %1, %2, %3;"
            : "=r"(hi) : "r"(u[lane_column(j, g, 3)]), "r"(mul.by256), "r"(u[lane_column(j, g, 2)]));
        asm("mad.lo.u32 %0, %1, %2, %3;" : "=r"(w) : "r"(hi), "r"(mul.by65536), "r"(lo));
        P[4 * j + g] = w;
      } else {
        const uint32_t lo = __byte_perm(u[lane_column(j, g, 0)], u[lane_column(j, g, 1)], 0x0040);
        const uint32_t hi = __byte_perm(u[lane_column(j, g, 2)], u[lane_column(j, g, 3)], 0x0040);
        P[4 * j + g] = __byte_perm(lo, hi, 0x5410);
      }
    }
  }
  uint32_t odd = 0;  // second partial sum: two short dependent chains instead of one
#pragma unroll
  for (int w = 0; w < NCOL / 4; ++w) {
    if constexpr (WANT_SUMS) {
      s4[w] = __dp4a(P[w], 0x01010101u, 0u);
      numer += s4[w];
    } else {
      if (w & 1) odd = __dp4a(P[w], 0x01010101u, odd);
      else numer = __dp4a(P[w], 0x01010101u, numer);
    }
  }
  numer += odd;
}

// Advances the four denominator partials over one chunk in the reference's order: one FMA per
// 16-key group; in the last visited tile one FMA per pair of groups, the very first fused with the
// rescale of the running partial -- d * o_scale + round(s * w) in a single FMA -- which is how the
// reference's compiled code rounds (found by comparing final denominators bit for bit on the GPU).
template <bool LAST, typename SumT>
__device__ __forceinline__ void denominator_chunk(RowState& st, const TileScales& ts,
                                                  bool first_chunk, const SumT* s4) {
#pragma unroll
  for (int g = 0; g < 4; ++g) {
    if constexpr (LAST) {
      const float s8 = static_cast<float>(uint32_t(s4[g]) + uint32_t(s4[4 + g]));
      if (first_chunk) st.d[g] = fmaf(ts.dprev[g], ts.o_scale, __fmul_rn(s8, ts.w));
      else st.d[g] = fmaf(s8, ts.w, st.d[g]);
    } else {
      st.d[g] = fmaf(static_cast<float>(uint32_t(s4[g])), ts.w, st.d[g]);
      st.d[g] = fmaf(static_cast<float>(uint32_t(s4[4 + g])), ts.w, st.d[g]);
    }
  }
}

// Single-partial denominator for paths that only need the output tolerance, not the reference's
// bits: d = d * o_scale + numer * w.
__device__ __forceinline__ void denominator_single(RowState& st, const TileScales& ts,
                                                   uint32_t numer) {
  st.d[0] = fmaf(static_cast<float>(numer), ts.w, st.d[0]);
}

struct TileResult {
  float tile_m, o_scale, w;
  uint32_t numer;
};

// Whole tile from a register array (row-per-thread kernel).
template <int CTA_K, int KIND, bool LAST, bool EXACT_D>
__device__ __forceinline__ TileResult softmax_tile(const float (&x)[CTA_K], const float (&sc)[4],
                                                   RowState& st, uint32_t (&P)[CTA_K / 4]) {
  TileMax tm;
  tile_max_init<KIND, LAST>(tm);
#pragma unroll
  for (int c = 0; c < CTA_K / 32; ++c) tile_max_chunk(&x[32 * c], tm);
  const TileScales ts = tile_begin(st, tile_max_finish<KIND>(tm, sc));
  uint32_t numer = 0;
#pragma unroll
  for (int c = 0; c < CTA_K / 32; ++c) {
    uint32_t s4[8];
    tile_exp_chunk<KIND, EXACT_D>(&x[32 * c], sc, -ts.tile_m, &P[8 * c], numer, s4);
    if constexpr (EXACT_D) denominator_chunk<LAST>(st, ts, c == 0, s4);
  }
  if constexpr (!EXACT_D) denominator_single(st, ts, numer);
  return {ts.tile_m, ts.o_scale, ts.w, numer};
}

__device__ __forceinline__ float row_denominator(const RowState& st) {
  return (st.d[0] + st.d[1]) + (st.d[2] + st.d[3]);
}

__device__ __forceinline__ float row_lse(float denom, float m) {
  return denom > 0.0f ? __fdividef(lg2_approx(denom) + m, kLog2e) : -INFINITY;
}

}  // namespace risa_b200
