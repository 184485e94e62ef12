// Tensor-core INT8 attention for B200 (sm_100a): S = Q.K^T (S8 x S8) and P.V (U8 x S8) run as
// tcgen05 kind::i8 MMAs whose INT32 accumulators live in tensor memory; Q, K and V tiles arrive by
// TMA into 128-byte-swizzled shared memory; the FP32 online softmax, the per-tile FP32 rescale of
// the output and the epilogue run on ordinary warps that read the accumulators with tcgen05.ld.
//
// One CTA = 128 queries of one (batch, head); key tiles of 64 or 128 and head_dim 64 or 128 are
// template parameters (the description below uses 128 / 128).  Five warpgroups:
//   WG0-WG2    softmax of tiles it % 3 == 0 / 1 / 2.  Thread r owns query row r (tensor-memory lane
//              r) and makes two passes over the tile's 128 scores: maxima on the raw integers, then
//              U8 probabilities written to shared memory as the A operand of P.V (bytes placed in
//              the packed V order).  The U8 codes depend only on the TILE maximum, so the groups
//              work on different tiles at the same time with no state shared between them.
//   WG3        correction.  Thread r owns the FP32 output row r in registers (as packed FP32 pairs)
//              and everything that is sequential over tiles: running maximum, denominator, per-tile
//              weights, O = O * o_scale + float(P.V) * w, capture statistics, epilogue and store.
//   WG4        warp 16: TMA producer (Q, K ring, V ring); warp 17: one thread issues the QK^T MMAs,
//              up to four tiles ahead of the read-back; warp 18: one thread issues the P.V MMAs.
// Tensor memory (512 columns) is four accumulator buffers of 128 columns.  Tile it owns buffer
// it % 4 from its Q.K^T until its P.V result has been read back: the scores are written there, the
// softmax group reads them, P.V overwrites the same columns and the correction group takes the
// result into registers.  Probabilities are scaled to the tile maximum (full 8-bit resolution in
// every tile), so each tile's integer P.V has its own weight and is folded into FP32 by the
// correction group; nothing accumulates across tiles inside tensor memory.
// Numerics: reference csrc/kernels/attention_int8.cuh:427-1026 via softmax_row.cuh.  The integer
// products are exact, so probabilities, capture statistics and block masses are bit-identical to
// the row-per-thread kernel; without capture the denominator is kept in one partial instead of four.
// Dense unmasked launches may cut the CTAs of their last, partial wave into key-range parts (see
// split_parts below): a part runs the same loop over its share of the key tiles and leaves its
// unnormalised rows, maximum and denominator in scratch for tail_merge_kernel.
// Every mbarrier wait is bounded (tc_ptx.cuh): when one expires the CTA's waiters leave, the producer
// waits for its loads in flight, the rows of the CTA are written as NaN and a device status word
// records the site; the CTA then exits instead of spinning.
#include "attention_common.cuh"
#include "select.cuh"
#include "tc_ptx.cuh"

#include <algorithm>
#include <climits>
#include <cuda.h>
#include <mutex>
#include <type_traits>

namespace risa_b200 {
namespace {

using namespace tc;

constexpr int kKStages = 3;           // K ring depth (K runs two tiles ahead of V)
constexpr int kVStages = 3;           // V ring depth
constexpr int kTile = 128 * 128;      // bytes of one 128 x 128 INT8 tile
constexpr int kThreads = 640;
constexpr int kSoftmaxGroups = 3;     // softmax warpgroups; tile it is handled by group it % 3
constexpr int kBuffers = 4;           // tensor-memory accumulator buffers; tile it uses it % 4
// What a launch produces besides the output: nothing, the reference's capture workspace, or the
// retained-mass selection of every query block.
enum Mode : int { kDense = 0, kCapture = 1, kSelect = 2 };
constexpr int kRegsLaunch = 96;        // what ptxas gives 640 threads (65536 / 640, multiple of 8)
constexpr int kRegsSoftmax = 96, kRegsCorrection = 168, kRegsIssue = 24;
// setmaxnreg redistributes the registers the CTA was launched with (threads x launch count); a
// request beyond that pool would block forever, outside the reach of the bounded barrier waits.
static_assert(128 * (kSoftmaxGroups * kRegsSoftmax + kRegsCorrection + kRegsIssue) <=
                  kThreads * kRegsLaunch,
              "register budget exceeds the launch pool");

// Unroll factor of the exponent pass over a tile's 32-column chunks: two copies of the chunk body
// measured fastest (one copy leaves the loads too little to hide behind, four copies fall out of the
// instruction cache next to the other roles' code).
constexpr int kExpUnroll = 2;
constexpr unsigned int kSelfTestSite = 900;  // site number reported by the bounded-wait self test

// Per head_dim and key-tile width: what one CTA holds and how deep its rings are.  head_dim 256 is
// run as two CTAs per (query block, head), each contracting Q.K^T over all 256 channels (two
// 128-byte column panels of the Q and K tiles) but producing 128 of the output channels, so that
// the accumulator, the output registers of the correction group and tensor memory stay exactly as
// for head_dim 128; the price is that both CTAs do the softmax.  Its larger Q / K tiles are paid
// for with shallower rings.  Kernels with 64-key tiles (per-query masks, short sequences,
// head_dim 64) have smaller K stages and spend the difference on a per-warp staging area through
// which mask values are loaded with coalesced accesses and handed to the row-owning threads.
template <int D, int CTA_K>
struct SmemLayout {
  static constexpr int kOut = D == 256 ? 128 : D;          // output channels per CTA
  static constexpr int kHalves = D == 256 ? 2 : 1;         // CTAs per (query block, head)
  static constexpr int kPanels = D == 256 ? 2 : 1;         // column panels of a Q / K tile
  static constexpr int kPanelBytes = D == 64 ? 64 : 128;   // bytes per row of a panel
  static constexpr int kKSt = D == 256 ? 2 : kKStages;     // K ring depth
  static constexpr int kVSt = D == 256 ? 2 : kVStages;     // V ring depth
  static constexpr int kSlots = D == 256 ? 3 : 4;          // P tiles and per-row statistics
  static constexpr int kQBytes = kPanels * kTile;          // the Q tile
  static constexpr int kKPanel = CTA_K * 128;              // one column panel of a K stage
  static constexpr int kKStage = kPanels * kKPanel;        // one K stage
  static constexpr int kMaskStageWords = 32 * 33;          // 32 x 32 values, rows padded to 33
  static constexpr int kMaskStageBytes =
      CTA_K == 64 ? kSoftmaxGroups * 4 * kMaskStageWords * 4 : 0;  // one area per softmax warp
  static constexpr int q = 0;
  static constexpr int k = q + kQBytes;
  static constexpr int v = k + kKSt * kKStage;
  static constexpr int p = v + kVSt * kTile;
  static constexpr int stats = p + kSlots * kTile;         // float2 [slots][128]: tile max, U8 sum
  static constexpr int sums = stats + 4 * 128 * 8;         // uint16 [slots][128][CTA_K / 4] (capture)
  static constexpr int mask_stage = sums + 4 * 128 * (CTA_K / 2);
  static constexpr int rowstate = mask_stage + kMaskStageBytes;  // float [5][128]: m, d[4] (capture)
  static constexpr int v_affine = rowstate + 5 * 128 * 4;  // float [2][128]: V scales, V centres
  static constexpr int bars = v_affine + 2 * 128 * 4;      // 8-byte mbarriers
  static constexpr int n_bars = 1 + 2 * kKStages + 2 * kVStages + 7 * 4 + 3;  // one spare
  static constexpr int tmem_slot = bars + n_bars * 8;
  static constexpr int gave_up = tmem_slot + 8;            // site of the first expired wait, or 0
  static constexpr int total = tmem_slot + 16;
  static constexpr size_t bytes = total + 1024;            // room to align the base to 1024
};
static_assert(SmemLayout<256, 128>::bytes <= 232448 && SmemLayout<128, 128>::bytes <= 232448 &&
                  SmemLayout<256, 64>::bytes <= 232448 && SmemLayout<128, 64>::bytes <= 232448 &&
                  SmemLayout<64, 64>::bytes <= 232448,
              "shared memory per CTA");

struct TileSeq {
  int n_iter;
  const int32_t* ids;
  bool key_list;  // ids come from a key-mask tile list: the list may stop before the last key tile
  int n_k;
  int first;      // without a list: the CTA visits tiles first .. first + n_iter - 1
  bool open_end;  // the range stops before the last key tile (a key-range part of a split CTA)
  __device__ __forceinline__ int tile(int it) const { return ids ? __ldg(ids + it) : first + it; }
  // The reference's generic last-visited-tile arithmetic applies on the last iteration, unless a
  // key-mask list ends on a tile that is not the final key tile (attention_int8.cuh:552-566) or the
  // CTA is a part of a split key range that does not hold the last tile.
  __device__ __forceinline__ bool last_rules(int it, int tile_id) const {
    return it == n_iter - 1 && !open_end && !(key_list && tile_id + 1 < n_k);
  }
};

template <int CTA_K>
__device__ __forceinline__ TileSeq tile_sequence(const AttentionArgs& a, int64_t bh, int bx,
                                                 int n_q, int n_k, bool capture, int part,
                                                 int parts) {
  TileSeq s;
  s.ids = nullptr;
  s.key_list = false;
  s.n_k = n_k;
  s.first = 0;
  s.open_end = false;
  if (a.row_offsets) {
    const int64_t r = bh * n_q + bx;
    const int start = __ldg(a.row_offsets + r);
    s.n_iter = __ldg(a.row_offsets + r + 1) - start;
    s.ids = a.block_indices + start;
  } else if (a.key_mask_tiles) {
    s.ids = a.key_mask_tiles + bh * (n_k + 1);
    s.n_iter = __ldg(s.ids + n_k);
    s.key_list = true;
  } else if (a.is_causal && !capture) {
    s.n_iter = (min(a.k_len, (bx + 1) * 128) + CTA_K - 1) / CTA_K;
  } else {
    s.first = n_k * part / parts;
    s.n_iter = n_k * (part + 1) / parts - s.first;
    s.open_end = part + 1 < parts;
  }
  return s;
}

struct Bars {
  uint32_t base;
  static constexpr int QFULL = 0, KFULL = 1, KEMPTY = KFULL + kKStages, VFULL = KEMPTY + kKStages,
                       VEMPTY = VFULL + kVStages, SFULL = VEMPTY + kVStages,
                       BUFFREE = SFULL + kBuffers, PFULL = BUFFREE + kBuffers, PFREE = PFULL + 4,
                       OFULL = PFREE + 4, STATFREE = OFULL + kBuffers, WFULL = STATFREE + 4,
                       PAIRS = WFULL + 4;  // two: the selection epilogue's bulk copies
  // Tensor memory is four accumulator buffers of 128 columns; tile it owns buffer it % 4 for its
  // whole life: Q.K^T writes the scores there (SFULL), the softmax group reads them, P.V then
  // overwrites the same columns with the tile's integer output (OFULL) and the correction group
  // hands the buffer back once it has it in registers (BUFFREE).  Three tiles can be in the
  // softmax stage while a fourth is in P.V / read-back, so no stage waits for another tile's
  // accumulator.  The probability tiles and the per-row statistics have four slots
  // (it % L::kSlots).
  __device__ __forceinline__ uint32_t operator()(int i) const { return base + 8u * i; }
};

// ---- softmax of one tile by the thread that owns the row -----------------------------------------
// Common case: every score of the tile is visible and it is not the last visited tile.  Pass 1
// takes the maxima on the raw integers (no conversion), pass 2 converts, scales, exponentiates and
// packs.  KIND selects the reference's arithmetic: kScoresInt fuses the scale into one FMA per
// score (unmasked, non-causal calls); kScoresScaled multiplies first and subtracts the maximum
// afterwards (causal calls, for their tiles below the diagonal) -- the positive scale keeps the
// maximum of the products equal to the product of the integer maximum.
// KEEPBITS (with kScoresScaled): a boolean per-query mask of the row arrives as one bit per key
// (bit i of keep[c] = key 32 c + i is visible).  Hidden scores enter the maxima as INT_MIN, which the
// -50000 floor of the pre-scaled arithmetic turns into the maximum a tile without a visible key
// has, and go into the exponent pass as -inf, so their codes are zero: the arithmetic of the
// general path on the same tile, without the trip through floats in tensor memory.
template <bool CAPTURE, int CTA_K, int KIND, bool KEEPBITS = false>
__device__ __forceinline__ void softmax_tile_int(uint32_t tmem_row, const float (&sc)[4],
                                                 unsigned char* p_row, int swz, float2* stat,
                                                 uint16_t* sums, PackMultipliers mul,
                                                 int max_floor = INT_MIN,
                                                 const uint32_t* keep = nullptr) {
  // (With kScoresInt the bits mark the keys that exist in a ragged last tile; the others go into
  // the exponent pass as -1e30, the value the general path gives them.)
  // Pass 1 lands two 32-column chunks per wait (nothing else is live yet, so 64 landing registers
  // are free); pass 2 walks the chunks backwards so that it starts on chunk 3, which is still in
  // registers, and every later chunk is fetched underneath the previous chunk's exponentials.
  uint32_t raw_a[32], raw[32];
  // max_floor: where the lane maxima start; the last visited tile starts them at -50000 (the
  // reference's generic arithmetic), every other tile below any score
  int imax[4] = {max_floor, max_floor, max_floor, max_floor};
#pragma unroll
  for (int h = 0; h < CTA_K / 64; ++h) {
    tmem_load32(tmem_row + 64 * h, raw_a);
    tmem_load32(tmem_row + 64 * h + 32, raw);
    tmem_load_wait();
    tmem_regs_ready<32>(raw_a);
    tmem_regs_ready<32>(raw);
    if constexpr (KEEPBITS) {
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        if (((keep[2 * h] >> i) & 1u) == 0u) raw_a[i] = 0x80000000u;
        if (((keep[2 * h + 1] >> i) & 1u) == 0u) raw[i] = 0x80000000u;
      }
    }
    // columns of K scale group g inside a chunk: 8k + 2g, 8k + 2g + 1 for k = 0..3
#pragma unroll
    for (int g = 0; g < 4; ++g) {
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        imax[g] = __vimax3_s32(imax[g], int(raw_a[8 * k + 2 * g]), int(raw_a[8 * k + 2 * g + 1]));
        imax[g] = __vimax3_s32(imax[g], int(raw[8 * k + 2 * g]), int(raw[8 * k + 2 * g + 1]));
      }
    }
  }
  float gm[4];
#pragma unroll
  for (int g = 0; g < 4; ++g)
    gm[g] = KIND == kScoresInt
                ? fmaf(static_cast<float>(imax[g]), sc[g], -kU8Offset)
                : fmaxf(static_cast<float>(imax[g]) * sc[g], -50000.0f) - kU8Offset;
  const float tile_m = fmaxf(fmaxf(gm[0], gm[1]), fmaxf(gm[2], gm[3]));
  const float neg_m = -tile_m;
  uint32_t numer = 0;
  // The chunk is converted to floats as soon as it lands, which frees the landing registers for
  // the next chunk's load to overlap the exponentials.
#pragma unroll kExpUnroll
  for (int c = CTA_K / 32 - 1; c >= 0; --c) {
    tmem_load_wait();
    tmem_regs_ready<32>(raw);
    float x[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) x[i] = static_cast<float>(int(raw[i]));
    if constexpr (KIND == kScoresScaled) {
#pragma unroll
      // one rounding for the product, a second one when the maximum is subtracted (the reference's
      // pre-scaled arithmetic); scalar multiplies with an explicit rounding mode on purpose: a packed
      // multiply followed by the packed add was observed to be merged into one fused operation
      for (int i = 0; i < 32; ++i) x[i] = __fmul_rn(x[i], sc[(i & 7) >> 1]);
    }
    if constexpr (KEEPBITS) {
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (((keep[c] >> i) & 1u) == 0u) x[i] = KIND == kScoresScaled ? -INFINITY : -1.0e30f;
    }
    if (c > 0) tmem_load32(tmem_row + 32 * (c - 1), raw);
    uint32_t P[8], s4[8];
    tile_exp_chunk<KIND, CAPTURE, 32, true>(x, sc, neg_m, P, numer, s4, mul);
    if constexpr (CAPTURE) {
#pragma unroll
      for (int i = 0; i < 8; i += 2)
        *reinterpret_cast<uint32_t*>(sums + 8 * c + i) = s4[i] | (s4[i + 1] << 16);
    }
    *reinterpret_cast<uint4*>(p_row + (((2 * c) ^ swz) << 4)) = make_uint4(P[0], P[1], P[2], P[3]);
    *reinterpret_cast<uint4*>(p_row + (((2 * c + 1) ^ swz) << 4)) =
        make_uint4(P[4], P[5], P[6], P[7]);
  }
  *stat = make_float2(tile_m, __uint_as_float(numer));
}

// The same block with 16-byte accesses, for masks whose keys are contiguous and whose rows start on
// 16-byte boundaries (checked by the caller): a row of the block is 32 * ESIZE bytes = LPR chunks of
// 16 bytes, so one warp-wide request covers 32 / LPR rows, and the block travels through the
// staging area as 16-byte chunks.  Chunk j of row r is stored at position j ^ f(r) of its row, f
// chosen per row width so that both the stores (lanes = chunks of a few rows) and the loads (lanes
// = rows, same chunk) touch every bank once per quarter warp.
// 32 mask entries held as packed words -> FP32 bit patterns: the additive bias, 0 for a kept
// boolean entry, NaN for a boolean false.
template <int ESIZE>
__device__ __forceinline__ void mask_words_to_bits(const AttentionArgs& a,
                                                   const uint32_t (&words)[8 * ESIZE],
                                                   uint32_t (&vals)[32]) {
  constexpr uint32_t kMasked = 0x7fc00000u;
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    if constexpr (ESIZE == 4) {
      vals[i] = words[i];
    } else if constexpr (ESIZE == 2) {
      const uint32_t half_bits = (words[i >> 1] >> (16 * (i & 1))) & 0xffffu;
      vals[i] = a.mask_dtype_code == 2
                    ? half_bits << 16
                    : __float_as_uint(__half2float(__ushort_as_half(static_cast<unsigned short>(half_bits))));
    } else {
      vals[i] = ((words[i >> 2] >> (8 * (i & 3))) & 0xffu) != 0 ? 0u : kMasked;
    }
  }
}

template <int ESIZE>
__device__ __forceinline__ void mask_block_rows_vec(const AttentionArgs& a, const char* block,
                                                    int64_t row_step_bytes, uint32_t* stage,
                                                    int lane, uint32_t (&vals)[32]) {
  constexpr int LPR = 2 * ESIZE;   // 16-byte chunks per row: 8 (FP32), 4 (FP16 / BF16), 2 (bool)
  constexpr int RPI = 32 / LPR;    // rows per warp-wide request
  auto fold = [](int r) { return LPR == 8 ? (r & 7) : LPR == 4 ? ((r >> 1) & 3) : ((r >> 2) & 1); };
  uint4* stage16 = reinterpret_cast<uint4*>(stage);
  const int j = lane % LPR, sub = lane / LPR;
#pragma unroll
  for (int i = 0; i < 32 / RPI; ++i) {
    const int r = i * RPI + sub;
    stage16[r * LPR + (j ^ fold(r))] =
        __ldg(reinterpret_cast<const uint4*>(block + r * row_step_bytes + 16 * j));
  }
  __syncwarp();
  uint32_t words[4 * LPR];
#pragma unroll
  for (int c = 0; c < LPR; ++c) {
    const uint4 v = stage16[lane * LPR + (c ^ fold(lane))];
    words[4 * c] = v.x;
    words[4 * c + 1] = v.y;
    words[4 * c + 2] = v.z;
    words[4 * c + 3] = v.w;
  }
  __syncwarp();
  mask_words_to_bits<ESIZE>(a, words, vals);
}

// A mask that is broadcast over the queries has one row per (batch, head): the 32 entries of a
// chunk are the same for every row of the CTA, so each thread reads them as 16-byte pieces (the
// same addresses in all lanes: one request per piece for the warp) instead of one entry at a time.
template <int ESIZE>
__device__ __forceinline__ void mask_shared_row_vec(const AttentionArgs& a, const char* entries,
                                                    uint32_t (&vals)[32]) {
  constexpr int LPR = 2 * ESIZE;
  uint32_t words[4 * LPR];
#pragma unroll
  for (int c = 0; c < LPR; ++c) {
    const uint4 v = __ldg(reinterpret_cast<const uint4*>(entries) + c);
    words[4 * c] = v.x;
    words[4 * c + 1] = v.y;
    words[4 * c + 2] = v.z;
    words[4 * c + 3] = v.w;
  }
  mask_words_to_bits<ESIZE>(a, words, vals);
}

// Mask values of a block of 32 query rows x 32 keys, fetched by the warp that owns the rows: for
// every row the 32 lanes read 32 consecutive keys (one coalesced request per row instead of one
// strided request per lane), the block is turned around through the warp's shared staging area
// (rows padded to 33 words: conflict-free both ways) and lane r leaves with row r's values as FP32
// bit patterns: the additive bias, 0 for a kept boolean entry, NaN for anything masked (boolean
// false, non-finite bias, rows or keys past the end).
__device__ __forceinline__ void mask_block_rows(const AttentionArgs& a, int batch, int head,
                                                int row0, int kv0, uint32_t* stage, int lane,
                                                uint32_t (&vals)[32]) {
  constexpr uint32_t kMasked = 0x7fc00000u;
  {
    // whole block inside the mask, contiguous keys, 16-byte aligned rows: vector form
    const int esize_v = a.mask_dtype_code == 3 ? 1 : a.mask_dtype_code == 0 ? 4 : 2;
    const char* block = static_cast<const char*>(a.mask) +
                        (int64_t(batch) * a.mask_stride_b + int64_t(head) * a.mask_stride_h +
                         int64_t(row0) * a.mask_stride_q + int64_t(kv0)) * esize_v;
    const int64_t row_step = a.mask_stride_q * esize_v;
    if (a.mask_stride_k == 1 && kv0 + 32 <= a.k_len && row0 + 32 <= a.q_len &&
        (reinterpret_cast<uintptr_t>(block) | uintptr_t(row_step)) % 16 == 0) {
      if (esize_v == 4) mask_block_rows_vec<4>(a, block, row_step, stage, lane, vals);
      else if (esize_v == 2) mask_block_rows_vec<2>(a, block, row_step, stage, lane, vals);
      else mask_block_rows_vec<1>(a, block, row_step, stage, lane, vals);
      return;
    }
  }
  const int kv = kv0 + lane;
  // rows of this block that exist, for a lane whose key exists (0 otherwise: nothing to load)
  const int rows = kv < a.k_len ? min(32, a.q_len - row0) : 0;
  const int esize = a.mask_dtype_code == 3 ? 1 : a.mask_dtype_code == 0 ? 4 : 2;
  const char* ptr = static_cast<const char*>(a.mask) +
                    (int64_t(batch) * a.mask_stride_b + int64_t(head) * a.mask_stride_h +
                     int64_t(row0) * a.mask_stride_q + int64_t(kv) * a.mask_stride_k) * esize;
  const int64_t step = a.mask_stride_q * esize;
  // one loop per element type, so that the body is a load, a conversion and a store
  auto fill = [&](auto convert) {
#pragma unroll 8
    for (int r = 0; r < 32; ++r) {
      stage[r * 33 + lane] = r < rows ? convert(ptr) : kMasked;
      ptr += step;
    }
  };
  switch (a.mask_dtype_code) {
    case 3:
      fill([](const char* q) { return *reinterpret_cast<const uint8_t*>(q) != 0 ? 0u : kMasked; });
      break;
    case 0:
      fill([](const char* q) { return *reinterpret_cast<const uint32_t*>(q); });
      break;
    case 1:
      fill([](const char* q) {
        return __float_as_uint(__half2float(*reinterpret_cast<const __half*>(q)));
      });
      break;
    default:
      fill([](const char* q) { return uint32_t(*reinterpret_cast<const uint16_t*>(q)) << 16; });
  }
  __syncwarp();
#pragma unroll
  for (int i = 0; i < 32; ++i) vals[i] = stage[lane * 33 + i];
  __syncwarp();
}

// 64 consecutive entries of one row of a boolean mask (16-byte aligned) as 64 bits: bit i of
// keep[c] = entry 32 c + i is non-zero.  Four 16-byte loads by the thread that owns the row (issued
// before the thread waits for the tile's scores, so that their latency passes during that wait);
// a word of four bytes, each made 0 / 1, times 0x01020408 leaves its four bits in the top nibble.
__device__ __forceinline__ void mask_row_load64(const unsigned char* entries, uint4 (&v)[4]) {
#pragma unroll
  for (int j = 0; j < 4; ++j) v[j] = __ldg(reinterpret_cast<const uint4*>(entries) + j);
}
__device__ __forceinline__ void mask_row_bits64(const uint4 (&v)[4], uint32_t (&keep)[2]) {
#pragma unroll
  for (int c = 0; c < 2; ++c) {
    uint32_t bits = 0;
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const uint32_t w[4] = {v[2 * c + j].x, v[2 * c + j].y, v[2 * c + j].z, v[2 * c + j].w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const uint32_t ones = __vcmpne4(w[i], 0u) & 0x01010101u;
        bits |= ((ones * 0x01020408u) >> 24) << (16 * j + 4 * i);
      }
    }
    keep[c] = bits;
  }
}

// A per-query mask is one long row per query: a CTA's tile touches 128 rows that lie far apart in
// memory and takes only CTA_K elements of each, which on its own makes every access open a new
// DRAM page.  Every kMaskRunKeys keys the warp that owns the rows therefore asks L2 for the next
// run of each of its rows in one piece (lane r = row r); the tile loads that follow hit L2.
constexpr int kMaskRunKeys = 512;

__device__ __forceinline__ void mask_prefetch_runs(const AttentionArgs& a, int batch, int head,
                                                   int row, int first_key) {
  if (row >= a.q_len || first_key >= a.k_len || a.mask_stride_k != 1) return;
  const int esize = a.mask_dtype_code == 3 ? 1 : a.mask_dtype_code == 0 ? 4 : 2;
  const int64_t off = int64_t(batch) * a.mask_stride_b + int64_t(head) * a.mask_stride_h +
                      int64_t(row) * a.mask_stride_q + first_key;
  const uintptr_t begin = (reinterpret_cast<uintptr_t>(a.mask) + off * esize) & ~uintptr_t(15);
  const uintptr_t row_end = reinterpret_cast<uintptr_t>(a.mask) +
                            (off - first_key + a.k_len) * esize;
  uintptr_t end = begin + kMaskRunKeys * esize + 16;
  if (end > row_end) end = row_end & ~uintptr_t(15);
  if (end > begin) l2_prefetch_run(reinterpret_cast<const void*>(begin), uint32_t(end - begin));
}

// Every other case (last visited tile, masks, causal diagonal, scale <= 0).  Pass 1 turns the raw
// integers into the scores the reference's generic path works on -- scaled, mask and causal rule
// applied, keys past the end removed -- takes their maxima and writes them back over the raw
// scores in tensor memory; pass 2 reads those floats, so masks are fetched once per tile.
// mask_stage: the warp's staging area (64-key-tile kernels), or nullptr.
// MASKED = false is the instantiation for causal diagonals and ragged last tiles of calls without
// a mask: none of the mask code is in it, which matters because every CTA of such a call runs it
// once or twice, cold.
template <bool CAPTURE, int CTA_K, bool MASKED, bool SHARED_ROW = false>
__device__ __forceinline__ void softmax_tile_general(const AttentionArgs& a, int batch, int head,
                                                     bool row_ok, uint32_t tmem_row,
                                                     const float (&sc)[4], unsigned char* p_row,
                                                     int swz, float2* stat, uint16_t* sums,
                                                     bool int_scores, bool last, int row, int c0,
                                                     uint32_t* mask_stage) {
  const bool causal = a.is_causal != 0;
  constexpr bool masked = MASKED;
  const int k_len = a.k_len;
  // per-query masks go through the staging area; masks broadcast over queries are read directly
  // (all lanes of a warp then ask for the same address)
  const bool staged = masked && mask_stage != nullptr && a.mask_stride_q != 0;
  const int lane = threadIdx.x & 31;
  if (staged && c0 % kMaskRunKeys == 0) mask_prefetch_runs(a, batch, head, row, c0 + kMaskRunKeys);
  TileMax tm;
  tile_max_init<kScoresScaled, true>(tm);  // maxima start at -50000 in all of these cases
#pragma unroll 1
  for (int c = 0; c < CTA_K / 32; ++c) {
    uint32_t raw[32];
    float x[32];
    tmem_load32(tmem_row + 32 * c, raw);
    // a mask broadcast over the queries, contiguous keys, chunk inside the key range and on a
    // 16-byte boundary: the chunk's entries as 16-byte pieces
    const char* shared_entries = nullptr;
    if (SHARED_ROW && masked && !staged && a.mask_stride_q == 0 && a.mask_stride_k == 1 &&
        c0 + 32 * c + 32 <= k_len) {
      const int esize = a.mask_dtype_code == 3 ? 1 : a.mask_dtype_code == 0 ? 4 : 2;
      const char* entries =
          static_cast<const char*>(a.mask) + (int64_t(batch) * a.mask_stride_b +
                                              int64_t(head) * a.mask_stride_h + c0 + 32 * c) * esize;
      if (reinterpret_cast<uintptr_t>(entries) % 16 == 0) shared_entries = entries;
    }
    if (staged || shared_entries != nullptr) {
      uint32_t bias_bits[32];
      if (staged) {
        mask_block_rows(a, batch, head, row - lane, c0 + 32 * c, mask_stage, lane, bias_bits);
      } else if (a.mask_dtype_code == 0) {
        mask_shared_row_vec<4>(a, shared_entries, bias_bits);
      } else if (a.mask_dtype_code == 3) {
        mask_shared_row_vec<1>(a, shared_entries, bias_bits);
      } else {
        mask_shared_row_vec<2>(a, shared_entries, bias_bits);
      }
      tmem_load_wait();
      tmem_regs_ready<32>(raw);
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        const float bias = __uint_as_float(bias_bits[i]);
        // score * scale and + bias * log2(e) are separate roundings, as in apply_mask
        float s = __fadd_rn(__fmul_rn(static_cast<float>(int(raw[i])), sc[(i & 7) >> 1]),
                            bias * kLog2e);
        if (!isfinite(bias)) s = -INFINITY;
        if (causal && c0 + 32 * c + i > row) s = -INFINITY;
        if (!staged && !row_ok) s = -INFINITY;  // the staged block marks rows past the end itself
        x[i] = s;
      }
    } else {
      tmem_load_wait();
      tmem_regs_ready<32>(raw);
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        const int kv = c0 + 32 * c + i;
        float s = static_cast<float>(int(raw[i]));
        if (int_scores) {
          if (last && kv >= k_len) s = -1.0e30f;
        } else {
          if (masked) s = apply_mask(a, batch, head, row, kv, row_ok, s, sc[(i & 7) >> 1]);
          else s = __fmul_rn(s, sc[(i & 7) >> 1]);
          if (causal && kv > row) s = -INFINITY;
          if (last && kv >= k_len) s = -INFINITY;
        }
        x[i] = s;
      }
    }
    tile_max_chunk(x, tm);
#pragma unroll
    for (int i = 0; i < 32; ++i) raw[i] = __float_as_uint(x[i]);
    tmem_store32(tmem_row + 32 * c, raw);
  }
  tmem_store_wait();
  const float tile_m = int_scores ? tile_max_finish<kScoresInt>(tm, sc)
                                  : tile_max_finish<kScoresScaled>(tm, sc);
  uint32_t numer = 0;
#pragma unroll 1
  for (int c = 0; c < CTA_K / 32; ++c) {
    uint32_t raw[32];
    float x[32];
    uint32_t P[8], s4[8];
    tmem_load32(tmem_row + 32 * c, raw);
    tmem_load_wait();
    tmem_regs_ready<32>(raw);
#pragma unroll
    for (int i = 0; i < 32; ++i) x[i] = __uint_as_float(raw[i]);
    const PackMultipliers mul{a.pack_by256, a.pack_by65536};
    if (int_scores) tile_exp_chunk<kScoresInt, CAPTURE, 32, true>(x, sc, -tile_m, P, numer, s4, mul);
    else tile_exp_chunk<kScoresScaled, CAPTURE, 32, true>(x, sc, -tile_m, P, numer, s4, mul);
    if constexpr (CAPTURE) {
#pragma unroll
      for (int i = 0; i < 8; i += 2)
        *reinterpret_cast<uint32_t*>(sums + 8 * c + i) = s4[i] | (s4[i + 1] << 16);
    }
    *reinterpret_cast<uint4*>(p_row + (((2 * c) ^ swz) << 4)) = make_uint4(P[0], P[1], P[2], P[3]);
    *reinterpret_cast<uint4*>(p_row + (((2 * c + 1) ^ swz) << 4)) =
        make_uint4(P[4], P[5], P[6], P[7]);
  }
  *stat = make_float2(tile_m, __uint_as_float(numer));
}

// BOOLROWS: the instantiation for dense calls with a boolean per-query mask whose rows can be read
// as 16-byte pieces (chosen on the host, launch_tc): their tiles take the bit form of the fast path.
// It is a kernel of its own so that the code of every other call stays exactly as it is -- the
// register allocation of the tile loop reacts to any path that is compiled into it.
template <int MODE, int CTA_K, int D, int VARIANT = 0>
__global__ __launch_bounds__(kThreads, 1) void attention_tc_kernel(
    const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
    const __grid_constant__ CUtensorMap map_v, const AttentionArgs a) {
  constexpr bool CAPTURE = MODE != kDense;  // exact per-tile statistics and denominators
  // Which softmax paths an instantiation holds (the host picks the instantiation, launch_tc):
  // 0 every path; 1 boolean per-query masks read as bits; 2 no mask, not causal, positive scale;
  // 3 causal without mask, positive scale; 4 any other per-query mask; 5 masks broadcast over the
  // queries (their entries are read as 16-byte pieces shared by all rows); 6 as 2 with a key length
  // that is a whole number of tiles (no ragged last tile: the integer fast path alone); 7 as 2 with
  // a ragged last tile, which takes the integer fast path with the existing keys marked by bits.
  constexpr bool BOOLROWS = VARIANT == 1, WHOLE = VARIANT == 6, RAGGED = VARIANT == 7,
                 PLAIN = VARIANT == 2 || WHOLE || RAGGED, CAUSAL = VARIANT == 3,
                 MASKED = VARIANT == 4, KEYMASK = VARIANT == 5;
  constexpr bool kHasInt = VARIANT == 0 || PLAIN, kHasScaled = VARIANT == 0 || CAUSAL,
                 kHasMasked = VARIANT == 0 || BOOLROWS || MASKED || KEYMASK,
                 kHasUnmasked = VARIANT == 0 || VARIANT == 2 || CAUSAL;
  using L = SmemLayout<D, CTA_K>;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t sbase = smem_u32(smem);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int wg = warp >> 2;
  const int n_k = (a.k_len + CTA_K - 1) / CTA_K, n_q = (a.q_len + 127) / 128;
  // Launch order is query block fastest, then (head, half), then batch.  With a split tail the grid
  // is one-dimensional: CTAs before tail_begin are whole (query block, head) units, the rest come
  // in groups of tail_splits parts of one unit each.
  int bx = blockIdx.x, by = blockIdx.y, batch = blockIdx.z, part = 0, parts = 1, tail_unit = -1;
  if (MODE == kDense && a.tail_splits > 1) {
    int unit = blockIdx.x;
    if (unit >= a.tail_begin) {
      tail_unit = (unit - a.tail_begin) / a.tail_splits;
      part = (unit - a.tail_begin) % a.tail_splits;
      parts = a.tail_splits;
      unit = a.tail_begin + tail_unit;
    }
    const int rows_y = a.q_heads * L::kHalves;
    bx = unit % n_q;
    by = (unit / n_q) % rows_y;
    batch = unit / (n_q * rows_y);
  }
  // Causal CTAs visit bx + 1 query blocks' worth of key tiles: the longest ones are launched first,
  // so that the short ones fill the end of the launch instead of the long ones stretching it.
  if (CAUSAL || (!PLAIN && a.is_causal)) bx = n_q - 1 - bx;
  const int head = by / L::kHalves, half = by % L::kHalves;
  const int kv_head = head / (a.q_heads / a.kv_heads);
  const int64_t bh = int64_t(batch) * a.q_heads + head;
  const int64_t kvh = int64_t(batch) * a.kv_heads + kv_head;
  const uint32_t gave_up = sbase + L::gave_up;  // set by the first wait of this CTA that expires
  Bars bar{sbase + L::bars};

  if (threadIdx.x == 0) {
    *reinterpret_cast<volatile uint32_t*>(smem + L::gave_up) = 0u;
    mbar_init(bar(Bars::QFULL), 1);
    for (int s = 0; s < kKStages; ++s) {
      mbar_init(bar(Bars::KFULL + s), 1);
      mbar_init(bar(Bars::KEMPTY + s), 1);
    }
    for (int s = 0; s < kVStages; ++s) {
      mbar_init(bar(Bars::VFULL + s), 1);
      mbar_init(bar(Bars::VEMPTY + s), 1);
    }
    for (int b = 0; b < kBuffers; ++b) {
      mbar_init(bar(Bars::SFULL + b), 1);
      mbar_init(bar(Bars::OFULL + b), 1);
      mbar_init(bar(Bars::BUFFREE + b), 128);
    }
    for (int i = 0; i < 4; ++i) {
      mbar_init(bar(Bars::STATFREE + i), 128);
      mbar_init(bar(Bars::PFULL + i), 128);
      mbar_init(bar(Bars::PFREE + i), 1);
      mbar_init(bar(Bars::WFULL + i), 128);
    }
    if constexpr (MODE == kSelect)
      for (int i = 0; i < 2; ++i) mbar_init(bar(Bars::PAIRS + i), 1);
    mbar_init_fence();
  }
  if (warp == 17) tmem_alloc(sbase + L::tmem_slot, 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(smem + L::tmem_slot);
  // everything above needs no result of the kernels before this one; everything below does
  chain_wait();

  const TileSeq seq = tile_sequence<CTA_K>(a, bh, bx, n_q, n_k, CAPTURE, part, parts);
  float2* stats = reinterpret_cast<float2*>(smem + L::stats);
  uint16_t* sums = reinterpret_cast<uint16_t*>(smem + L::sums);

  if (wg == 4) {
    regs_dec<kRegsIssue>();
    if (warp == 16 && lane == 0) {
      // ---------------------------------------------------------------- producer
      tma_prefetch_descriptor(&map_q);
      tma_prefetch_descriptor(&map_k);
      tma_prefetch_descriptor(&map_v);
      mbar_expect_tx(bar(Bars::QFULL), 128 * D);
#pragma unroll
      for (int panel = 0; panel < L::kPanels; ++panel)
        tma_load_3d(sbase + L::q + panel * kTile, &map_q, bar(Bars::QFULL), 128 * panel, bx * 128,
                    int(bh));
      bool ok = true;
      int k_issued = 0, v_issued = 0;
      // K runs two tiles ahead of V, matching the order in which the MMA warp consumes them.
      for (int step = 0; step < seq.n_iter + 2 && ok; ++step) {
        if (step < seq.n_iter) {
          const int s = step % L::kKSt, r = step / L::kKSt;
          ok = mbar_wait<true>(bar(Bars::KEMPTY + s), (r & 1) ^ 1, gave_up, 101);
          if (!ok) break;
          mbar_expect_tx(bar(Bars::KFULL + s), CTA_K * D);
#pragma unroll
          for (int panel = 0; panel < L::kPanels; ++panel)
            tma_load_3d(sbase + L::k + s * L::kKStage + panel * L::kKPanel, &map_k,
                        bar(Bars::KFULL + s), 128 * panel, seq.tile(step) * CTA_K, int(kvh));
          k_issued = step + 1;
        }
        const int it = step - 2;
        if (it >= 0) {
          const int s = it % L::kVSt, r = it / L::kVSt;
          ok = mbar_wait<true>(bar(Bars::VEMPTY + s), (r & 1) ^ 1, gave_up, 102);
          if (!ok) break;
          // V always arrives as the 128-key slab that holds the tile (64-key tiles use half of it):
          // rows stay 128 bytes wide, so one swizzle mode and one descriptor form serve both widths
          mbar_expect_tx(bar(Bars::VFULL + s), L::kOut * 128);
          tma_load_3d(sbase + L::v + s * kTile, &map_v, bar(Bars::VFULL + s),
                      (seq.tile(it) * CTA_K) & ~127, L::kOut * half, int(kvh));
          v_issued = it + 1;
        }
      }
      if (!ok) {
        // drain: every issued load must land before shared memory can be released
        mbar_drain(bar(Bars::QFULL), 0);
        for (int it = max(0, k_issued - L::kKSt); it < k_issued; ++it)
          mbar_drain(bar(Bars::KFULL + it % L::kKSt), (it / L::kKSt) & 1);
        for (int it = max(0, v_issued - L::kVSt); it < v_issued; ++it)
          mbar_drain(bar(Bars::VFULL + it % L::kVSt), (it / L::kVSt) & 1);
      }
    } else if (warp == 17 && lane == 0) {
      // ---------------------------------------------------------------- MMA issue: S = Q.K^T
      // Tile it goes to buffer it % 4 as soon as the correction group has read that buffer's
      // previous tile (it - 4) out.  Issuing the two GEMMs from two threads halves the per-tile
      // barrier round-trips on each.
      constexpr uint32_t idesc_qk = idesc_i8(true, true, CTA_K);
      bool ok = mbar_wait<true>(bar(Bars::QFULL), 0, gave_up, 201);
      for (int it = 0; it < seq.n_iter && ok; ++it) {
        const int b = it % kBuffers, u = it / kBuffers, s = it % L::kKSt, r = it / L::kKSt;
        ok = mbar_wait2<true>(bar(Bars::KFULL + s), r & 1, bar(Bars::BUFFREE + b), (u & 1) ^ 1,
                              gave_up, 202);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int panel = 0; panel < L::kPanels; ++panel) {
          const uint64_t desc_q = smem_desc_kmajor<L::kPanelBytes>(sbase + L::q + panel * kTile);
          const uint64_t desc_k = smem_desc_kmajor<L::kPanelBytes>(
              sbase + L::k + s * L::kKStage + panel * L::kKPanel);
#pragma unroll
          for (int kk = 0; kk < L::kPanelBytes / 32; ++kk)
            mma_i8(tmem + 128 * b, desc_q + 2 * kk, desc_k + 2 * kk, idesc_qk, (panel | kk) > 0);
        }
        mma_commit(bar(Bars::SFULL + b));
        mma_commit(bar(Bars::KEMPTY + s));
      }
    } else if (warp == 18 && lane == 0) {
      // ---------------------------------------------------------------- MMA issue: P.V
      constexpr uint32_t idesc_pv = idesc_i8(false, true, L::kOut);
      bool ok = true;
      for (int it = 0; it < seq.n_iter && ok; ++it) {
        const int s = it % L::kVSt, r = it / L::kVSt;
        const int slot = it % L::kSlots, j = it / L::kSlots;
        ok = mbar_wait2<true>(bar(Bars::PFULL + slot), j & 1, bar(Bars::VFULL + s), r & 1,
                              gave_up, 204);
        if (!ok) break;
        const int b = it % kBuffers;
        const uint32_t tmem_o = tmem + 128 * b;  // the tile's scores have all been read by now
        tc_fence_after();
        const uint64_t desc_p = smem_desc_k128(sbase + L::p + slot * kTile);
        const uint64_t desc_v = smem_desc_k128(sbase + L::v + s * kTile);
        // a 64-key tile is the first or second half (64 bytes per row) of its 128-key V slab
        const uint32_t v_k0 = CTA_K == 64 ? 4u * (seq.tile(it) & 1) : 0u;
#pragma unroll
        for (int kk = 0; kk < CTA_K / 32; ++kk)
          mma_i8(tmem_o, desc_p + 2 * kk, desc_v + v_k0 + 2 * kk, idesc_pv, kk > 0);
        mma_commit(bar(Bars::OFULL + b));
        mma_commit(bar(Bars::VEMPTY + s));
        mma_commit(bar(Bars::PFREE + slot));
      }
    }
  } else if (wg < kSoftmaxGroups) {
    // ------------------------------------------------------------------ softmax of tiles it = wg, wg+3, ...
    // every group must end up at its constant: a group left at the launch count while another one
    // grows would over-subscribe the pool (see the static_assert above)
    if constexpr (kRegsSoftmax > kRegsLaunch) regs_inc<kRegsSoftmax>();
    else if constexpr (kRegsSoftmax < kRegsLaunch) regs_dec<kRegsSoftmax>();
    const int b = wg;                      // first tile of this group
    const int row_in = threadIdx.x & 127;  // tensor-memory lane
    const int row = bx * 128 + row_in;
    const uint32_t tmem_lane = tmem + (uint32_t((warp & 3) * 32) << 16);
    const bool int_scores =
        PLAIN || (kHasInt && !a.is_causal && a.sm_scale > 0.0f && a.mask == nullptr);
    const bool causal_fast =
        CAUSAL || (kHasScaled && a.is_causal && a.sm_scale > 0.0f && a.mask == nullptr);
    const unsigned char* bool_row = nullptr;  // this row of a boolean per-query mask
    if constexpr (BOOLROWS)
      bool_row = static_cast<const unsigned char*>(a.mask) + int64_t(batch) * a.mask_stride_b +
                 int64_t(head) * a.mask_stride_h + int64_t(row) * a.mask_stride_q;
    const PackMultipliers pack_mul{a.pack_by256, a.pack_by65536};
    const bool row_ok = row < a.q_len;
    const float scale2 = a.sm_scale * kLog2e;
    const float q_scale =
        D == 256 ? __ldg(a.q_scale + bh * (n_q * 64) + (row / 16) * 8 + (row & 7))
                 : __ldg(a.q_scale + bh * (n_q * 32) + (row / 32) * 8 + (row & 7));
    const float* k_scale = a.k_scale + kvh * (n_k * 4);
    uint32_t* mask_stage = nullptr;  // this warp's staging area for per-query mask blocks
    if constexpr (L::kMaskStageBytes > 0)
      mask_stage = reinterpret_cast<uint32_t*>(smem + L::mask_stage) + warp * L::kMaskStageWords;
    bool ok = true;
    float* rowstate = reinterpret_cast<float*>(smem + L::rowstate);
    CaptureLayout cap;
    if constexpr (MODE == kCapture) cap = capture_layout(a, n_q, n_k);
    uint2* pairs = nullptr;
    if constexpr (MODE == kSelect) {
      // The CTA's (probability sum, tile maximum) pairs go to a slot of the scratch, [tile][row] so
      // that a warp's stores are one contiguous run.  A slot is claimed by compare-and-swap on its
      // flag, starting at this SM's number; there are at least as many slots as CTAs resident at
      // once, so the scan ends, and it is bounded like every other wait.  The first group claims
      // (its tile 0 comes before everybody else's statistics).
      if (b == 0 && half == 0) {
        if (row_in == 0) {
          int* flags = static_cast<int*>(a.select_scratch);
          unsigned int smid;
          asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
          int s = int(smid % unsigned(a.select_slots)), found = -1;
          for (int tries = 0; tries < 64 * a.select_slots && found < 0; ++tries) {
            if (atomicCAS(flags + s, 0, 1) == 0) found = s;
            else s = s + 1 == a.select_slots ? 0 : s + 1;
          }
          if (found < 0) {
            atomicCAS(&g_wait_status, 0u, 501u);
            asm volatile("st.volatile.shared::cta.u32 [%0], %1;" ::"r"(gave_up), "r"(501u)
                         : "memory");
          }
          *reinterpret_cast<volatile int*>(smem + L::tmem_slot + 12) = found;
        }
        asm volatile("bar.sync 2, 128;" ::: "memory");
      }
    }
    float ks_next[4] = {0.f, 0.f, 0.f, 0.f};
    if (kHasMasked && b == 0 && mask_stage != nullptr && a.mask != nullptr && a.mask_stride_q != 0 &&
        seq.ids == nullptr)
      mask_prefetch_runs(a, batch, head, row, 0);
    if (b < seq.n_iter) {
      const int first_tile = seq.tile(b);
#pragma unroll
      for (int g = 0; g < 4; ++g) ks_next[g] = __ldg(k_scale + first_tile * 4 + g);
    }
    for (int it = b; it < seq.n_iter && ok; it += kSoftmaxGroups) {
      const int sb = it % kBuffers, u = it / kBuffers;
      const uint32_t tmem_row = tmem_lane + 128 * sb;
      const int tile = seq.tile(it);
      const bool last = seq.last_rules(it, tile);
      float sc[4];
#pragma unroll
      for (int g = 0; g < 4; ++g) sc[g] = scale2 * (q_scale * ks_next[g]);
      if (it + kSoftmaxGroups < seq.n_iter) {  // next tile's K scales travel during this tile
        const int next_tile = seq.tile(it + kSoftmaxGroups);
#pragma unroll
        for (int g = 0; g < 4; ++g) ks_next[g] = __ldg(k_scale + next_tile * 4 + g);
      }
      // The P slot is free once the P.V that read it is done, the statistics slot once the
      // correction group has read the tile four back; S is ready when the MMA warp says so.
      const int slot = it % L::kSlots;
      float2* stat = stats + slot * 128 + row_in;
      uint16_t* my_sums = sums + (slot * 128 + row_in) * (CTA_K / 4);
      unsigned char* p_row = smem + L::p + slot * kTile + row_in * 128;
      uint4 mask_bytes[4] = {};
      if constexpr (BOOLROWS) {
        if (!last && row_ok) mask_row_load64(bool_row + tile * CTA_K, mask_bytes);
      }
      ok = mbar_wait3(bar(Bars::PFREE + slot), ((it / L::kSlots) & 1) ^ 1, bar(Bars::STATFREE + slot),
                      ((it / L::kSlots) & 1) ^ 1, bar(Bars::SFULL + sb), u & 1, gave_up, 301);
      if (!ok) break;
      tc_fence_after();
      // causal: tiles that end at or before the CTA's first query are fully visible
      const bool below_diagonal = causal_fast && (tile + 1) * CTA_K - 1 <= bx * 128;
      // A last tile without tail keys differs from the others only in where its maxima start;
      // with tail keys (their scores are zero-filled, not masked) it takes the general path.
      if (WHOLE || (kHasInt && int_scores && (!last || a.k_len % CTA_K == 0)))
        softmax_tile_int<CAPTURE, CTA_K, kScoresInt>(tmem_row, sc, p_row, row_in & 7, stat,
                                                     my_sums, pack_mul, last ? -50000 : INT_MIN);
      else if (RAGGED) {
        // last visited tile of a call without mask or causal rule: the keys that exist, as bits
        if constexpr (RAGGED) {
          uint32_t keep[CTA_K / 32];
#pragma unroll
          for (int c = 0; c < CTA_K / 32; ++c) {
            const int exist = a.k_len - (tile * CTA_K + 32 * c);
            keep[c] = exist >= 32 ? 0xffffffffu : exist <= 0 ? 0u : (1u << exist) - 1u;
          }
          softmax_tile_int<CAPTURE, CTA_K, kScoresInt, true>(tmem_row, sc, p_row, row_in & 7, stat,
                                                             my_sums, pack_mul, -50000, keep);
        }
      } else if (kHasScaled && below_diagonal && !last)
        softmax_tile_int<CAPTURE, CTA_K, kScoresScaled>(tmem_row, sc, p_row, row_in & 7, stat,
                                                        my_sums, pack_mul);
      else if (BOOLROWS && !last) {
        // boolean per-query mask, tile wholly inside the key range: the row's 64 entries as bits
        if constexpr (BOOLROWS) {
          if (tile * CTA_K % kMaskRunKeys == 0)
            mask_prefetch_runs(a, batch, head, row, tile * CTA_K + kMaskRunKeys);
          uint32_t keep[2];
          mask_row_bits64(mask_bytes, keep);  // rows past the end hold zeros: nothing visible
          softmax_tile_int<CAPTURE, CTA_K, kScoresScaled, true>(
              tmem_row, sc, p_row, row_in & 7, stat, my_sums, pack_mul, INT_MIN, keep);
        }
      } else if (kHasMasked && (!kHasUnmasked || a.mask != nullptr))
        softmax_tile_general<CAPTURE, CTA_K, true, KEYMASK>(a, batch, head, row_ok, tmem_row, sc,
                                                            p_row, row_in & 7, stat, my_sums,
                                                            int_scores, last, row, tile * CTA_K,
                                                            mask_stage);
      else if constexpr (kHasUnmasked)
        softmax_tile_general<CAPTURE, CTA_K, false>(a, batch, head, row_ok, tmem_row, sc, p_row,
                                                    row_in & 7, stat, my_sums, int_scores, last,
                                                    row, tile * CTA_K, mask_stage);
      // every score of the tile has been read (the loads were waited for) and the probabilities
      // are in shared memory: P.V may now overwrite the buffer
      tc_fence_before();
      fence_async_smem();
      mbar_arrive(bar(Bars::PFULL + slot));
      if constexpr (CAPTURE) {
        // With capture every tile needs the reference's exact running maximum and four denominator
        // partials per row (they decide block masses and tile sets bit for bit): a strictly
        // sequential chain over the tiles, but a short one.  It depends on the tile's probability
        // sums only, so the thread that produced them advances the row's state -- kept in shared
        // memory, handed from tile to tile: WFULL of tile it - 1 is the permission for tile it --
        // while P.V runs, leaves the tile's weights (w, o_scale) for the correction group in the
        // statistics slot, and writes the per-tile pair to the capture workspace or, for in-pass
        // selection, to the CTA's slot of the scratch.
        RowState st;
        if (it == 0) {
          row_state_init(st);
        } else {
          const int before = (it - 1) % L::kSlots;
          ok = mbar_wait(bar(Bars::WFULL + before), ((it - 1) / L::kSlots) & 1, gave_up, 303);
          if (!ok) break;
          st.m = rowstate[row_in];
#pragma unroll
          for (int i = 0; i < 4; ++i) st.d[i] = rowstate[128 * (1 + i) + row_in];
        }
        const float2 mine = *stat;  // (tile maximum, probability sum), written above
        const uint32_t numer = __float_as_uint(mine.y);
        const TileScales ts = tile_begin(st, mine.x);
        if (last) {
#pragma unroll
          for (int c = 0; c < CTA_K / 32; ++c) {
            uint16_t s4[8];
            *reinterpret_cast<uint4*>(s4) = *reinterpret_cast<const uint4*>(my_sums + 8 * c);
            denominator_chunk<true>(st, ts, c == 0, s4);
          }
        } else {
          // d[g] = fma(float(sum), w, d[g]) word by word in key order, as denominator_chunk<false>
          // does, with lanes (0, 1) and (2, 3) as packed pairs: a stored word holds the 16-bit sums
          // of two neighbouring lanes, a byte permute puts each under the exponent of 2^23, and
          // one packed subtract of 2^23 gives both exact float values
          const uint64_t w2 = pack_f32x2(ts.w, ts.w);
          const uint64_t unbias = pack_f32x2(-8388608.0f, -8388608.0f);
          uint64_t d01 = pack_f32x2(st.d[0], st.d[1]), d23 = pack_f32x2(st.d[2], st.d[3]);
#pragma unroll
          for (int c = 0; c < CTA_K / 32; ++c) {
            const uint4 words = *reinterpret_cast<const uint4*>(my_sums + 8 * c);
            const uint32_t pair[4] = {words.x, words.y, words.z, words.w};  // (g0,g1) (g2,g3) x 2
#pragma unroll
            for (int j = 0; j < 2; ++j) {
              const uint64_t f01 = add_f32x2(
                  (uint64_t(__byte_perm(pair[2 * j], 0x4B000000u, 0x7632)) << 32) |
                      __byte_perm(pair[2 * j], 0x4B000000u, 0x7610), unbias);
              const uint64_t f23 = add_f32x2(
                  (uint64_t(__byte_perm(pair[2 * j + 1], 0x4B000000u, 0x7632)) << 32) |
                      __byte_perm(pair[2 * j + 1], 0x4B000000u, 0x7610), unbias);
              d01 = fma_f32x2(f01, w2, d01);
              d23 = fma_f32x2(f23, w2, d23);
            }
          }
          unpack_f32x2(d01, st.d[0], st.d[1]);
          unpack_f32x2(d23, st.d[2], st.d[3]);
        }
        rowstate[row_in] = st.m;
#pragma unroll
        for (int i = 0; i < 4; ++i) rowstate[128 * (1 + i) + row_in] = st.d[i];
        *stat = make_float2(ts.w, ts.o_scale);
        if (half == 0) {
          if constexpr (MODE == kSelect) {
            if (pairs == nullptr) {
              const int claimed = *reinterpret_cast<volatile int*>(smem + L::tmem_slot + 12);
              if (claimed < 0) break;  // no slot: the claimer has raised the give-up word
              const size_t flag_bytes = (size_t(a.select_slots) * 4 + 255) / 256 * 256;
              pairs = reinterpret_cast<uint2*>(static_cast<char*>(a.select_scratch) + flag_bytes) +
                      size_t(claimed) * n_k * 128 + row_in;
            }
            pairs[size_t(it) * 128] = make_uint2(numer, __float_as_uint(ts.tile_m));
          } else if (row_ok) {
            const int64_t grow = bh * a.q_len + row;
            if (it == seq.n_iter - 1) {
              float* out = cap.last + grow * 2;
              out[0] = static_cast<float>(numer);
              out[1] = ts.tile_m;
            } else {
              uint32_t* out = cap.full + (grow * (n_k - 1) + it) * 2;
              out[0] = numer;
              out[1] = __float_as_uint(ts.tile_m);
            }
          }
        }
        mbar_arrive(bar(Bars::WFULL + slot));
      }
    }
  } else {
    // ------------------------------------------------------------------ correction + epilogue
    regs_inc<kRegsCorrection>();
    const int row_in = threadIdx.x & 127;
    const int row = bx * 128 + row_in;
    const bool row_ok = row < a.q_len;
    const uint32_t lane_base = uint32_t((warp & 3) * 32) << 16;
    const int64_t grow = bh * a.q_len + row;
    RowState st;
    row_state_init(st);
    constexpr int kOut = L::kOut;
    uint64_t O2[kOut / 2];
#pragma unroll
    for (int i = 0; i < kOut / 2; ++i) O2[i] = 0ull;
    bool ok = true;
    // The epilogue multiplies every output channel by its V scale and adds its V centre; the two
    // vectors are the same for all rows, so they are brought into shared memory now (their global
    // load latency passes during the first tiles instead of in front of every store).
    float* v_affine = reinterpret_cast<float*>(smem + L::v_affine);
    if (row_in < kOut) {
      v_affine[row_in] = __ldg(a.v_scale + kvh * D + kOut * half + row_in);
      v_affine[128 + row_in] = __ldg(a.v_center + kvh * D + kOut * half + row_in);
    }
    asm volatile("bar.sync 3, 128;" ::: "memory");
    // One iteration per tile and one barrier round trip per iteration: a finished accumulator
    // (OFULL) implies that the tile's probabilities and statistics were published before (P.V is
    // only issued after them), so the statistics need no wait of their own.  This group is the one
    // strictly sequential stage of the kernel and every barrier round trip costs a few hundred
    // cycles even when the phase is long complete, so its per-tile chain is: wait, statistics
    // (running maximum, denominator, weights), read-back and fold.  Without capture the statistics
    // are a single exponential: denominator and output row are both kept in units of a stale
    // maximum m_o that is only moved when the true maximum has run ahead of it by 2^8, so
    // d = d * f + sum * 2^(tile_m - m_o) and O = O * f + PV * 2^(tile_m - m_o) share weight and
    // (rare) rescale factor f, and their quotient needs no correction at the end.
    float m_o = -INFINITY;  // maximum the dense path's denominator and output rows are scaled to
    for (int it = 0; it < seq.n_iter && ok; ++it) {
      const int ob = it & (kBuffers - 1);
      const int slot = it % L::kSlots;
      const uint32_t tmem_o = tmem + 128 * ob;
      float o_scale = 1.0f, w = 0.0f;
      if constexpr (CAPTURE) {
        // the statistics warp has replaced the tile's (maximum, sum) by its weights
        ok = mbar_wait2(bar(Bars::OFULL + ob), (it / kBuffers) & 1, bar(Bars::WFULL + slot),
                        (it / L::kSlots) & 1, gave_up, 401);
        if (!ok) break;
        tc_fence_after();
        const float2 wf = stats[slot * 128 + row_in];
        w = wf.x;
        o_scale = wf.y;
        mbar_arrive(bar(Bars::STATFREE + slot));
      } else {
        ok = mbar_wait(bar(Bars::OFULL + ob), (it / kBuffers) & 1, gave_up, 401);
        if (!ok) break;
        tc_fence_after();
        const float2 stat = stats[slot * 128 + row_in];
        mbar_arrive(bar(Bars::STATFREE + slot));
        st.m = fmaxf(st.m, stat.x);
        if (st.m > m_o + 8.0f) {
          o_scale = ex2_approx(m_o - st.m);
          m_o = st.m;
        }
        w = ex2_approx(stat.x - m_o);
        st.d[0] = fmaf(static_cast<float>(__float_as_uint(stat.y)), w, st.d[0] * o_scale);
      }
      const bool rescale = __any_sync(0xffffffffu, o_scale != 1.0f);
      const uint64_t w2 = pack_f32x2(w, w), s2 = pack_f32x2(o_scale, o_scale);
      uint32_t acc[16];
      tmem_load16(tmem_o + lane_base, acc);
#pragma unroll
      for (int c = 0; c < kOut / 16; ++c) {
        tmem_load_wait();
        tmem_regs_ready<16>(acc);
        uint64_t f2[8];
#pragma unroll
        for (int i = 0; i < 8; ++i)
          f2[i] = pack_f32x2(static_cast<float>(int(acc[2 * i])),
                             static_cast<float>(int(acc[2 * i + 1])));
        if (c < kOut / 16 - 1) {
          tmem_load16(tmem_o + lane_base + 16 * (c + 1), acc);
        } else {
          tc_fence_before();
          mbar_arrive(bar(Bars::BUFFREE + ob));  // Q.K^T of tile it + 4 may take the buffer
        }
        if (rescale) {
#pragma unroll
          for (int i = 0; i < 8; ++i) O2[8 * c + i] = mul_f32x2(O2[8 * c + i], s2);
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) O2[8 * c + i] = fma_f32x2(f2[i], w2, O2[8 * c + i]);
      }
    }
    float O[kOut];
#pragma unroll
    for (int i = 0; i < kOut / 2; ++i) unpack_f32x2(O2[i], O[2 * i], O[2 * i + 1]);
    int claimed = -1;
    uint2* pairs = nullptr;
    if constexpr (CAPTURE) {
      // final (maximum, four denominator partials) of the row: the state the softmax threads
      // handed from tile to tile (the last tile's WFULL was waited for above)
      const float* rowstate = reinterpret_cast<const float*>(smem + L::rowstate);
      st.m = rowstate[row_in];
#pragma unroll
      for (int i = 0; i < 4; ++i) st.d[i] = rowstate[128 * (1 + i) + row_in];
      st.d[0] = row_denominator(st);
      if constexpr (MODE == kSelect) {
        if (half == 0) {
          claimed = *reinterpret_cast<volatile int*>(smem + L::tmem_slot + 12);
          const size_t flag_bytes = (size_t(a.select_slots) * 4 + 255) / 256 * 256;
          pairs = reinterpret_cast<uint2*>(static_cast<char*>(a.select_scratch) + flag_bytes) +
                  size_t(max(claimed, 0)) * n_k * 128 + row_in;
        }
      }
    }
    const float denom = st.d[0];
    if (MODE == kDense && parts > 1) {
      // part of a split key range: channel-major unnormalised rows (in units of 2^m_o), then m_o
      // and the denominator; NaN when a wait of this CTA expired, so the merged rows show it
      float* mine = a.tail_scratch + (size_t(tail_unit) * parts + part) * (130 * 128) + row_in;
      const float poison = ok ? 0.0f : __int_as_float(0x7fffffff);
#pragma unroll
      for (int ch = 0; ch < kOut; ++ch) mine[ch * 128] = O[ch] + poison;
      mine[128 * 128] = m_o;
      mine[129 * 128] = denom + poison;
    } else if (ok && row_ok) {
      if (MODE == kCapture && half == 0) {
        const CaptureLayout cap = capture_layout(a, n_q, n_k);
        cap.state[grow * 2] = st.m;
        cap.state[grow * 2 + 1] = denom;
      }
      // dense path: denominator and rows share the stale maximum's units, the quotient is exact
      const float inv = rcp_approx(denom);
      const bool zero = !PLAIN && (a.is_causal || a.mask != nullptr) && !(denom > 0.0f);
      const float* vs = v_affine;
      const float* vc = v_affine + 128;
      char* o_row = static_cast<char*>(a.o) + 2 * kOut * half +
                    2 * (batch * a.o_stride_b + head * a.o_stride_h + int64_t(row) * a.o_stride_n);
#pragma unroll
      for (int ch = 0; ch < kOut; ch += 8) {
        // eight channels' scales and centres as four 16-byte shared-memory loads (the same
        // addresses in every thread: one broadcast each)
        float scale8[8], centre8[8];
        *reinterpret_cast<float4*>(scale8) = *reinterpret_cast<const float4*>(vs + ch);
        *reinterpret_cast<float4*>(scale8 + 4) = *reinterpret_cast<const float4*>(vs + ch + 4);
        *reinterpret_cast<float4*>(centre8) = *reinterpret_cast<const float4*>(vc + ch);
        *reinterpret_cast<float4*>(centre8 + 4) = *reinterpret_cast<const float4*>(vc + ch + 4);
        uint32_t packed[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          float r0 = fmaf(O[ch + 2 * i] * inv, scale8[2 * i], centre8[2 * i]);
          float r1 = fmaf(O[ch + 2 * i + 1] * inv, scale8[2 * i + 1], centre8[2 * i + 1]);
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
      // the LSE wants the denominator's own reference point: the stale maximum without capture
      if (a.lse && half == 0) a.lse[grow] = row_lse(denom, CAPTURE ? st.m : m_o);
    } else if (row_ok) {
      // a wait of this CTA expired: mark the rows it owns, so that a failed launch cannot be taken
      // for a result (NaN in both 16-bit output formats, NaN LSE)
      char* o_row = static_cast<char*>(a.o) + 2 * kOut * half +
                    2 * (batch * a.o_stride_b + head * a.o_stride_h + int64_t(row) * a.o_stride_n);
#pragma unroll
      for (int ch = 0; ch < kOut; ch += 8)
        *reinterpret_cast<uint4*>(o_row + 2 * ch) =
            make_uint4(0x7fff7fffu, 0x7fff7fffu, 0x7fff7fffu, 0x7fff7fffu);
      if (a.lse && half == 0) a.lse[grow] = __int_as_float(0x7fffffff);
    }
    if constexpr (MODE == kSelect) {
      if (half == 0 && claimed >= 0) {
        // ---- block masses of this query block, then the retained-mass prefix ------------------
        // mass[t] = sum over the block's queries of numerator * 2^(tile_max - m_final) / d_final,
        // summed in the reference's tree (attention_int8.cuh:1067-1086: shift-down inside each
        // warp, then the four warp sums as (w0 + w2) + (w1 + w3)), because the masses feed an
        // exact selection.  The rings are idle by now: the capture sums' area is reused.
        const int n4 = (n_k + 3) & ~3;
        float* s_mass = reinterpret_cast<float*>(smem + L::sums);  // [n4], padded with -inf
        float* s_sorted = s_mass + n4;                             // [n_k] descending
        float* s_warp = s_sorted + n_k;                            // [4][n_k], then the ranks
        const int w = warp & 3;
        const bool live = ok && row_ok;
        // The pairs of 32 tiles are 32 KB in one piece of the scratch slot: they come back as bulk
        // copies into the idle K / V rings, two in flight, while the previous 32 tiles are reduced.
        // Sum over a warp's 32 rows: every lane leaves its row's 32 masses in a [tile][row] block
        // of the idle P ring (rows padded to 33 words), then lane l adds up tile l's column in the
        // order of the shift-down tree (x[i] += x[i + off] for off = 16, 8, 4, 2, 1: the value lane
        // 0 ends with after five shuffle steps) -- 31 independent additions per lane in place of
        // five dependent shuffles per tile.
        constexpr int kChunkTiles = 32;
        constexpr uint32_t kChunkBytes = kChunkTiles * 128 * 8;
        static_assert(L::p - L::k >= 2 * int(kChunkBytes) && L::k % 16 == 0,
                      "the K and V rings hold two chunks of pairs");
        static_assert(L::kSlots * kTile >= 4 * 32 * 33 * 4, "the P ring holds the four sum blocks");
        float* stage = reinterpret_cast<float*>(smem + L::p) + w * (32 * 33);
        const uint2* slot_pairs = pairs - row_in;
        const int n_chunks = (n_k + kChunkTiles - 1) / kChunkTiles;
        auto fetch = [&](int c) {
          const uint32_t bytes = uint32_t(min(kChunkTiles, n_k - c * kChunkTiles)) * (128u * 8u);
          const uint32_t full = bar(Bars::PAIRS + (c & 1));
          mbar_expect_tx(full, bytes);
          bulk_load(sbase + L::k + (c & 1) * kChunkBytes,
                    slot_pairs + size_t(c) * kChunkTiles * 128, bytes, full);
        };
        if (row_in == 0) {
          // the pairs were written through the generic proxy by the softmax threads, whose WFULL
          // arrivals this thread has waited for; the bulk copies read them through the async proxy
          fence_async_all();
          fetch(0);
          if (n_chunks > 1) fetch(1);
        }
        bool fetched = true;
        for (int c = 0; c < n_chunks; ++c) {
          const int t0 = c * kChunkTiles;
          // an expired wait raises the CTA's give-up word; the loop still runs to its end so that
          // the 128 threads meet at every barrier, and the copies in flight are drained below
          fetched &= mbar_wait(bar(Bars::PAIRS + (c & 1)), (c >> 1) & 1, gave_up, 501);
          const uint2* chunk =
              reinterpret_cast<const uint2*>(smem + L::k + (c & 1) * kChunkBytes) + row_in;
          // loads, arithmetic and stores as three separate sweeps: the 32 tiles are independent,
          // and a store between two loads of the same memory would keep them in program order
          uint2 pr[kChunkTiles];
#pragma unroll
          for (int j = 0; j < kChunkTiles; ++j) pr[j] = chunk[j * 128];
          float x[32];
#pragma unroll
          for (int j = 0; j < kChunkTiles; ++j) {
            x[j] = 0.0f;
            if (live && denom > 0.0f && t0 + j < n_k)
              x[j] = __uint2float_rn(pr[j].x) * ex2_approx(__uint_as_float(pr[j].y) - st.m) / denom;
          }
#pragma unroll
          for (int j = 0; j < kChunkTiles; ++j) stage[j * 33 + lane] = x[j];
          __syncwarp();
#pragma unroll
          for (int i = 0; i < 32; ++i) x[i] = stage[lane * 33 + i];
#pragma unroll
          for (int off = 16; off > 0; off >>= 1) {
#pragma unroll
            for (int i = 0; i < off; ++i) x[i] = __fadd_rn(x[i], x[i + off]);
          }
          if (t0 + lane < n_k) s_warp[w * n_k + t0 + lane] = x[0];
          asm volatile("bar.sync 1, 128;" ::: "memory");  // every row has read the chunk
          if (row_in == 0 && c + 2 < n_chunks) fetch(c + 2);
        }
        if (!fetched && row_in == 0) {
          // copies that were issued land in this CTA's shared memory: wait for them before leaving
          for (int c = max(n_chunks - 2, 0); c < n_chunks; ++c)
            mbar_drain(bar(Bars::PAIRS + (c & 1)), (c >> 1) & 1);
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        const int64_t block_row = bh * n_q + bx;
        for (int t = row_in; t < n4; t += 128) {
          float mass = -INFINITY;  // padding: never above and never equal to a mass
          if (t < n_k) {
            mass = __fadd_rn(__fadd_rn(s_warp[t], s_warp[2 * n_k + t]),
                             __fadd_rn(s_warp[n_k + t], s_warp[3 * n_k + t]));
            if (a.select_masses) a.select_masses[block_row * n_k + t] = mass;
          }
          s_mass[t] = mass;
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        // Descending order by counting: rank = tiles with a larger mass + earlier tiles with the
        // same mass.  Masses are non-negative, so their bit patterns order like signed integers
        // (the -inf padding is negative); "larger, or equal and earlier" is one comparison against
        // bits - 1 for the tiles before this one and against bits from this tile on.  The masses
        // are read four at a time (the same address in every lane: one broadcast), and a thread
        // ranks its tiles t and t + 128 from the same loads.
        int* s_rank = reinterpret_cast<int*>(s_warp);
        const int4* bits4 = reinterpret_cast<const int4*>(s_mass);
        for (int t = row_in; t < n_k; t += 256) {
          const int t2 = t + 128;
          const bool second = t2 < n_k;
          const int mine = __float_as_int(s_mass[t]);
          const int mine2 = second ? __float_as_int(s_mass[t2]) : 0x7f800000;
          int r0 = 0, r1 = 0, r2 = 0, r3 = 0, q0 = 0, q1 = 0, q2 = 0, q3 = 0;
#pragma unroll 4
          for (int u = 0; u < n4; u += 4) {
            const int4 other = bits4[u >> 2];
            r0 += other.x > mine - (u < t ? 1 : 0) ? 1 : 0;
            r1 += other.y > mine - (u + 1 < t ? 1 : 0) ? 1 : 0;
            r2 += other.z > mine - (u + 2 < t ? 1 : 0) ? 1 : 0;
            r3 += other.w > mine - (u + 3 < t ? 1 : 0) ? 1 : 0;
            q0 += other.x > mine2 - (u < t2 ? 1 : 0) ? 1 : 0;
            q1 += other.y > mine2 - (u + 1 < t2 ? 1 : 0) ? 1 : 0;
            q2 += other.z > mine2 - (u + 2 < t2 ? 1 : 0) ? 1 : 0;
            q3 += other.w > mine2 - (u + 3 < t2 ? 1 : 0) ? 1 : 0;
          }
          const int rank = (r0 + r1) + (r2 + r3);
          s_sorted[rank] = __int_as_float(mine);
          s_rank[t] = rank;
          if (second) {
            const int rank2 = (q0 + q1) + (q2 + q3);
            s_sorted[rank2] = __int_as_float(mine2);
            s_rank[t2] = rank2;
          }
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (w == 0) {
          const RetainedPrefix kept = retained_prefix(s_sorted, uint32_t(n_k), a.select_theta);
          const uint32_t words = bitmap_words(uint32_t(n_k));
          for (uint32_t wd = 0; wd < words; ++wd) {
            const int t = int(32 * wd) + lane;
            const uint32_t bits =
                __ballot_sync(0xffffffffu, t < n_k && uint32_t(s_rank[t]) < kept.count);
            if (lane == 0) a.select_bitmaps[block_row * words + wd] = bits;
          }
          if (lane == 0) {
            a.select_counts[block_row] = int32_t(kept.count);
            a.select_totals[block_row * 2] = kept.selected;
            a.select_totals[block_row * 2 + 1] = kept.total;
          }
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (row_in == 0) {
          __threadfence();
          atomicExch(static_cast<int*>(a.select_scratch) + claimed, 0);  // slot free again
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 17) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

// One warp waits on a barrier that nobody arrives at, with a caller-chosen limit: the bounded-wait
// machinery (expiry, site record, orderly return) exercised without any faulty launch.
__global__ void bounded_wait_self_test_kernel(uint64_t limit_ns) {
  __shared__ __align__(8) uint64_t barrier;
  __shared__ uint32_t gave_up_word;
  if (threadIdx.x == 0) {
    gave_up_word = 0u;
    mbar_init(smem_u32(&barrier), 1);
    mbar_init_fence();
  }
  __syncthreads();
  mbar_wait(smem_u32(&barrier), 0, smem_u32(&gave_up_word), kSelfTestSite, limit_ns);
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

// 3-D byte tensor {inner, rows, slabs} with a {box_inner, box_rows, 1} box; rows of 128 bytes use the
// 128-byte swizzle, rows of 64 bytes the 64-byte one (what the MMA descriptors expect).
bool make_map(CUtensorMap* map, const void* base, uint64_t inner, uint64_t rows, uint64_t slabs,
              uint32_t box_inner, uint32_t box_rows) {
  const cuuint64_t dims[3] = {inner, rows, slabs};
  const cuuint64_t strides[2] = {inner, inner * rows};
  const cuuint32_t box[3] = {box_inner, box_rows, 1};
  const cuuint32_t elem[3] = {1, 1, 1};
  return encode_fn()(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(base), dims, strides,
                     box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     box_inner == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B,
                     CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Combines the parts of the split CTAs (AttentionArgs::tail_*): per row the parts' maxima give the
// common unit, the rows and denominators are added in it, and the row is finished exactly as the
// attention kernel's epilogue finishes an unsplit one.  grid = (split units, groups of 16 output
// channels), 128 threads = rows; every load of a thread is independent of the others.
constexpr int kMergeChannels = 16;
__global__ __launch_bounds__(128) void tail_merge_kernel(const AttentionArgs a, int halves,
                                                         int k_out) {
  chain_wait();
  constexpr int kMaxParts = 4;
  const int n_q = (a.q_len + 127) / 128, rows_y = a.q_heads * halves, parts = a.tail_splits;
  const int unit = a.tail_begin + blockIdx.x, row_in = threadIdx.x, ch0 = blockIdx.y * kMergeChannels;
  const int bx = unit % n_q, by = (unit / n_q) % rows_y, batch = unit / (n_q * rows_y);
  const int head = by / halves, half = by % halves;
  const int row = bx * 128 + row_in;
  if (row >= a.q_len) return;
  const int kv_head = head / (a.q_heads / a.kv_heads);
  const int64_t kvh = int64_t(batch) * a.kv_heads + kv_head;
  const float* mine = a.tail_scratch + size_t(blockIdx.x) * parts * (130 * 128) + row_in;
  float part_m[kMaxParts], part_d[kMaxParts], x[kMaxParts][kMergeChannels];
#pragma unroll
  for (int p = 0; p < kMaxParts; ++p) {
    part_m[p] = -INFINITY;
    part_d[p] = 0.0f;
    if (p < parts) {
      part_m[p] = mine[(p * 130 + 128) * 128];
      part_d[p] = mine[(p * 130 + 129) * 128];
#pragma unroll
      for (int c = 0; c < kMergeChannels; ++c) x[p][c] = mine[(p * 130 + ch0 + c) * 128];
    }
  }
  float m = part_m[0];
#pragma unroll
  for (int p = 1; p < kMaxParts; ++p) m = fmaxf(m, part_m[p]);
  float w[kMaxParts], denom = 0.0f;
#pragma unroll
  for (int p = 0; p < kMaxParts; ++p) {
    w[p] = p < parts ? ex2_approx(part_m[p] - m) : 0.0f;
    denom = fmaf(part_d[p], w[p], denom);
  }
  const float inv = rcp_approx(denom);
  const float* vs = a.v_scale + kvh * a.head_dim + k_out * half + ch0;
  const float* vc = a.v_center + kvh * a.head_dim + k_out * half + ch0;
  char* o_row = static_cast<char*>(a.o) + 2 * (k_out * half + ch0) +
                2 * (batch * a.o_stride_b + head * a.o_stride_h + int64_t(row) * a.o_stride_n);
#pragma unroll
  for (int ch = 0; ch < kMergeChannels; ch += 8) {
    uint32_t packed[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float r[2];
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int c = ch + 2 * i + j;
        float acc = 0.0f;
#pragma unroll
        for (int p = 0; p < kMaxParts; ++p)
          if (p < parts) acc = fmaf(x[p][c], w[p], acc);
        r[j] = fmaf(acc * inv, __ldg(vs + c), __ldg(vc + c));
      }
      if (a.out_dtype_code == 1) {
        const __half2 h = __floats2half2_rn(r[0], r[1]);
        packed[i] = *reinterpret_cast<const uint32_t*>(&h);
      } else {
        const __nv_bfloat162 h = __floats2bfloat162_rn(r[0], r[1]);
        packed[i] = *reinterpret_cast<const uint32_t*>(&h);
      }
    }
    *reinterpret_cast<uint4*>(o_row + 2 * ch) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
  }
  if (a.lse && half == 0 && blockIdx.y == 0)
    a.lse[(int64_t(batch) * a.q_heads + head) * a.q_len + row] = row_lse(denom, m);
}

// How the last, partial wave of a dense unmasked launch is split (0 = not at all).  With C whole
// CTAs on S SMs the last wave holds R = C mod S of them and takes a whole CTA's time however few
// they are.  Cut into p key-range parts each (p = 2..4, at least eight key tiles per part) they are
// R * p parts that take ceil(R * p / S) rounds of 1 / p of a CTA's time; the p with the shortest
// last wave is taken if it saves at least a fifth of a CTA's time and at least 2048 keys' worth of
// tiles (about 16 us), several times what the parts' stores and the merge launch cost.
int split_parts(int ctas, int n_k, int cta_k, int sms) {
  if (sms <= 0 || ctas <= sms) return 0;
  const int rest = ctas % sms;
  if (rest == 0) return 0;
  int best = 0;
  double best_time = 0.8;  // of a whole CTA
  for (int parts = 2; parts <= 4 && n_k / parts >= 8; ++parts) {
    const double time = double((rest * parts + sms - 1) / sms) / parts;
    if (time < best_time - 1e-9) {
      best_time = time;
      best = parts;
    }
  }
  if (best == 0) return 0;
  return (1.0 - best_time) * n_k * cta_k >= 2048.0 ? best : 0;
}

int tail_split_factor(const AttentionArgs& a, int ctas, int n_k, int sms) {
  if (a.tail_scratch == nullptr || a.is_causal || a.mask || a.row_offsets || a.key_mask_tiles ||
      a.block_mass)
    return 0;
  const int parts = split_parts(ctas, n_k, a.cta_k, sms);
  // the scratch was sized by the same rule; a caller who sized it for another device gets whole CTAs
  if (parts > 0 && size_t(ctas % sms) * parts * kTailPartBytes > a.tail_scratch_bytes) return 0;
  return parts;
}

// Dense calls whose mask is boolean, per query, with contiguous keys and rows that start on 16-byte
// boundaries (base and every stride a multiple of 16 entries), a positive scale and neither causal
// rule nor tile lists: the kernel instantiation that reads such rows as bits (64-key tiles only,
// which per-query masks always have).
bool reads_mask_rows_as_bits(const AttentionArgs& a) {
  return a.cta_k == 64 && a.mask != nullptr && a.mask_dtype_code == 3 && a.mask_stride_k == 1 &&
         a.mask_stride_q != 0 && a.sm_scale > 0.0f && !a.is_causal && a.row_offsets == nullptr &&
         a.key_mask_tiles == nullptr && a.block_mass == nullptr && a.select_scratch == nullptr &&
         (reinterpret_cast<uintptr_t>(a.mask) | uintptr_t(a.mask_stride_b) |
          uintptr_t(a.mask_stride_h) | uintptr_t(a.mask_stride_q)) % 16 == 0;
}

template <int MODE, int CTA_K, int D, int VARIANT = 0>
int launch_tc(const AttentionArgs& a, const CUtensorMap& map_q, const CUtensorMap& map_k,
              const CUtensorMap& map_v, cudaStream_t stream) {
  auto kernel = attention_tc_kernel<MODE, CTA_K, D, VARIANT>;
  static thread_local int configured = -1;  // per instantiation, thread and device
  int device = -1;
  cudaGetDevice(&device);
  if (configured != device) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         int(SmemLayout<D, CTA_K>::bytes));
    if (e != cudaSuccess)
      return fail(RISA_B200_CUDA, "attention: cannot reserve %zu bytes of shared memory: %s",
                  SmemLayout<D, CTA_K>::bytes, cudaGetErrorString(e));
    // setmaxnreg hands out the registers the CTA is launched with; if the compiler ever gave this
    // kernel fewer than the roles ask for, the increase could never be granted (it blocks, beyond
    // the reach of the bounded waits), so such a build must not run
    cudaFuncAttributes attr;
    e = cudaFuncGetAttributes(&attr, kernel);
    if (e != cudaSuccess)
      return fail(RISA_B200_CUDA, "attention: cudaFuncGetAttributes: %s", cudaGetErrorString(e));
    constexpr int kPool = 128 * (kSoftmaxGroups * kRegsSoftmax + kRegsCorrection + kRegsIssue);
    if (attr.numRegs * kThreads < kPool)
      return fail(RISA_B200_CUDA,
                  "attention: kernel was compiled with %d registers per thread, the warp roles "
                  "need a pool of %d", attr.numRegs, kPool / kThreads);
    configured = device;
  }
  const dim3 grid((a.q_len + 127) / 128, a.q_heads * SmemLayout<D, CTA_K>::kHalves, a.batch);
  if constexpr (MODE == kDense) {
    static thread_local int sms = 0, sms_device = -1;
    if (sms_device != device) {
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
      sms_device = device;
    }
    const int ctas = int(grid.x * grid.y * grid.z), n_k = (a.k_len + CTA_K - 1) / CTA_K;
    const int parts = tail_split_factor(a, ctas, n_k, sms);
    if (parts > 0) {
      AttentionArgs split = a;
      const int rest = ctas % sms;
      split.tail_begin = ctas - rest;
      split.tail_splits = parts;
      launch_chained(kernel, dim3(split.tail_begin + rest * parts), dim3(kThreads),
                     SmemLayout<D, CTA_K>::bytes, stream, map_q, map_k, map_v, split);
      launch_chained(tail_merge_kernel, dim3(rest, SmemLayout<D, CTA_K>::kOut / kMergeChannels),
                     dim3(128), 0, stream, split,
                     SmemLayout<D, CTA_K>::kHalves, SmemLayout<D, CTA_K>::kOut);
      return check_launch("attention (tensor-core kernel, split tail)");
    }
  }
  AttentionArgs whole = a;
  whole.tail_splits = 0;
  launch_chained(kernel, grid, dim3(kThreads), SmemLayout<D, CTA_K>::bytes, stream, map_q, map_k, map_v,
                 whole);
  return check_launch("attention (tensor-core kernel)");
}

}  // namespace

// head_dim 128 and 256 with 64- or 128-key tiles and head_dim 64 with 64-key tiles (the only width
// the packed formats define for it); every mask form, causal, tile lists, capture.  The packed V row
// must hold at least one 128-key slab (the V box is always 128 keys wide) and TMA needs 16-byte
// aligned operand bases; anything else goes to the row-per-thread kernel.
bool attention_tc_supported(const AttentionArgs& a) {
  const int64_t padded = int64_t((a.k_len + a.cta_k - 1) / a.cta_k) * a.cta_k;
  const bool shape = ((a.head_dim == 128 || a.head_dim == 256) &&
                      (a.cta_k == 128 || a.cta_k == 64)) ||
                     (a.head_dim == 64 && a.cta_k == 64);
  auto aligned16 = [](const void* p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; };
  return shape && padded >= 128 && encode_fn() != nullptr && aligned16(a.q) && aligned16(a.k) &&
         aligned16(a.v) && aligned16(a.o) && a.o_stride_b % 8 == 0 &&
         a.o_stride_h % 8 == 0 && a.o_stride_n % 8 == 0;
}

int attention_tc(const AttentionArgs& a, cudaStream_t stream, bool every_path) {
  const int n_k = (a.k_len + a.cta_k - 1) / a.cta_k;
  const uint32_t d = uint32_t(a.head_dim);
  CUtensorMap map_q, map_k, map_v;
  const uint32_t panel = d < 128 ? d : 128;      // bytes per row of a Q / K box
  const uint32_t v_rows = d == 256 ? 128 : d;    // output channels (V rows) per CTA
  if (!make_map(&map_q, a.q, d, uint64_t(a.q_len), uint64_t(a.batch) * a.q_heads, panel, 128) ||
      !make_map(&map_k, a.k, d, uint64_t(a.k_len), uint64_t(a.batch) * a.kv_heads, panel,
                a.cta_k) ||
      !make_map(&map_v, a.v, uint64_t(n_k) * a.cta_k, d, uint64_t(a.batch) * a.kv_heads, 128,
                v_rows))
    return fail(RISA_B200_CUDA, "attention: tensor map creation failed");
  const int mode = a.select_scratch ? kSelect : a.block_mass ? kCapture : kDense;
  auto launch = [&](auto cta_k, auto head_dim) {
    constexpr int K = decltype(cta_k)::value, HD = decltype(head_dim)::value;
    // calls without mask or causal rule and with a positive scale: the instantiations that hold
    // nothing but the integer fast path and the ragged last tile
    // every_path: the instantiation that holds all paths, which the class-specific ones must
    // reproduce bit for bit (a diagnostic switch of the calling thread)
    if (every_path) {
      if (mode == kSelect) return launch_tc<kSelect, K, HD>(a, map_q, map_k, map_v, stream);
      if (mode == kCapture) return launch_tc<kCapture, K, HD>(a, map_q, map_k, map_v, stream);
      return launch_tc<kDense, K, HD>(a, map_q, map_k, map_v, stream);
    }
    const bool plain = a.mask == nullptr && !a.is_causal && a.sm_scale > 0.0f;
    if (mode == kSelect)
      return !plain ? launch_tc<kSelect, K, HD>(a, map_q, map_k, map_v, stream)
             : a.k_len % K == 0 ? launch_tc<kSelect, K, HD, 6>(a, map_q, map_k, map_v, stream)
                                : launch_tc<kSelect, K, HD, 2>(a, map_q, map_k, map_v, stream);
    if (mode == kCapture)
      return plain ? launch_tc<kCapture, K, HD, 2>(a, map_q, map_k, map_v, stream)
                   : launch_tc<kCapture, K, HD>(a, map_q, map_k, map_v, stream);
    if constexpr (K == 64) {
      if (reads_mask_rows_as_bits(a))
        return launch_tc<kDense, K, HD, 1>(a, map_q, map_k, map_v, stream);
    }
    if (plain) {
      if (a.k_len % K == 0) return launch_tc<kDense, K, HD, 6>(a, map_q, map_k, map_v, stream);
      // measured: the bit form of the ragged last tile gains at head_dim 128 (a 1000-key call
      // 45 -> 34 us, long calls 0.5-1.5 %) and loses 1-4 % at head_dim 64 and 256
      if constexpr (HD == 128) return launch_tc<kDense, K, HD, 7>(a, map_q, map_k, map_v, stream);
      return launch_tc<kDense, K, HD, 2>(a, map_q, map_k, map_v, stream);
    }
    if (a.mask != nullptr)
      return a.mask_stride_q == 0 ? launch_tc<kDense, K, HD, 5>(a, map_q, map_k, map_v, stream)
                                  : launch_tc<kDense, K, HD, 4>(a, map_q, map_k, map_v, stream);
    if (a.is_causal && a.sm_scale > 0.0f)
      return launch_tc<kDense, K, HD, 3>(a, map_q, map_k, map_v, stream);
    return launch_tc<kDense, K, HD>(a, map_q, map_k, map_v, stream);
  };
  using std::integral_constant;
  if (a.head_dim == 256)
    return a.cta_k == 64 ? launch(integral_constant<int, 64>{}, integral_constant<int, 256>{})
                         : launch(integral_constant<int, 128>{}, integral_constant<int, 256>{});
  if (a.head_dim == 64) return launch(integral_constant<int, 64>{}, integral_constant<int, 64>{});
  return a.cta_k == 64 ? launch(integral_constant<int, 64>{}, integral_constant<int, 128>{})
                       : launch(integral_constant<int, 128>{}, integral_constant<int, 128>{});
}

// Largest key-tile count whose masses, sorted copy and per-warp partials fit the shared-memory
// area the in-pass selection reuses (24 bytes per key tile).
int attention_tc_select_max_tiles(int cta_k) { return (256 * cta_k - 12) / 24; }

int attention_tc_split_parts(int ctas, int n_k, int cta_k, int sms) {
  return split_parts(ctas, n_k, cta_k, sms);
}

}  // namespace risa_b200

extern "C" int risa_b200_device_status(void) {
  unsigned int status = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&status, risa_b200::tc::g_wait_status, sizeof(status)) != cudaSuccess)
    return risa_b200::fail(RISA_B200_CUDA, "device status: %s",
                           cudaGetErrorString(cudaGetLastError()));
  if (status != 0) {
    cudaMemcpyToSymbol(risa_b200::tc::g_wait_status, &zero, sizeof(zero));
    return risa_b200::fail(RISA_B200_DEVICE,
                           "attention kernel gave up waiting at site %u (bounded wait expired)",
                           status);
  }
  return RISA_B200_OK;
}

extern "C" int risa_b200_bounded_wait_self_test(uint64_t limit_ns, void* stream) {
  if (limit_ns == 0 || limit_ns > 1000000000ull)
    return risa_b200::fail(RISA_B200_INVALID,
                           "bounded_wait_self_test: limit must be in (0, 1e9] nanoseconds");
  risa_b200::bounded_wait_self_test_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(
      limit_ns);
  return risa_b200::check_launch("bounded-wait self test");
}
