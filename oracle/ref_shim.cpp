// Test infrastructure, not product code.
//
// C wrappers around the reference project's extern "C" launchers
// (csrc/launchers.h:8-64).  Those launchers throw std::runtime_error through
// their C signatures and take risa::QuantInput structs by value; a ctypes
// caller can do neither, so each wrapper here catches the exception, stores
// its text, and returns a status.  Compiled only into oracle/_ref/librisa_ref.so
// by oracle/build_ref.sh; used by tests and by the benchmark's comparison legs
// as the bit-exact golden for codes, scales and tile sets.
#include "launchers.h"
#include <cstring>
#include <exception>
#include <string>

namespace {
thread_local std::string g_error;
template <typename F> int guarded(F&& f) {
  try {
    f();
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
      g_error = cudaGetErrorString(e);
      return 2;
    }
    return 0;
  } catch (const std::exception& ex) {
    g_error = ex.what();
    return 1;
  } catch (...) {
    g_error = "unknown exception";
    return 1;
  }
}
} // namespace

extern "C" {
const char* ref_last_error() { return g_error.c_str(); }

int ref_quantize_qk(const void* q, void* q_int8, void* q_scale, const void* k, void* k_int8,
                    void* k_scale, int batch, int hq, int lq, int hkv, int lk, int head_dim,
                    int blkq, int warpq, int blkk, int warpk, int64_t qb, int64_t qh, int64_t qn,
                    int64_t kb, int64_t kh, int64_t kn, int dtype, void* anchors, void* stream) {
  return guarded([&] {
    launch_quantize_qk(q, q_int8, q_scale, k, k_int8, k_scale, batch, hq, lq, hkv, lk, head_dim,
                       blkq, warpq, blkk, warpk, qb, qh, qn, kb, kh, kn, dtype, anchors,
                       static_cast<cudaStream_t>(stream));
  });
}

int ref_quantize_v(const void* v, void* out, void* scale, void* center, int batch, int heads,
                   int length, int head_dim, int padded, int64_t sb, int64_t sh, int64_t sn,
                   int dtype, int affine, void* stream) {
  return guarded([&] {
    launch_quantize_v(v, out, scale, center, batch, heads, length, head_dim, padded, sb, sh, sn,
                      dtype, affine != 0, static_cast<cudaStream_t>(stream));
  });
}

int ref_attention(const void* q, const void* k, const void* v, void* o, const void* q_scale,
                  const void* k_scale, const void* v_scale, const void* v_center, const void* mask,
                  int64_t msb, int64_t msh, int64_t msq, int64_t msk, int mask_dtype, int cta_k,
                  int batch, int lq, int lk, int hq, int hkv, int head_dim, int64_t q_b,
                  int64_t q_n, int64_t q_h, int64_t k_b, int64_t k_n, int64_t k_h, int64_t v_b,
                  int64_t v_h, int64_t v_d, int64_t o_b, int64_t o_n, int64_t o_h, float sm_scale,
                  int out_dtype, const void* row_offsets, const void* block_indices,
                  void* block_mass, int causal, void* lse, void* stream, const int32_t* key_tiles) {
  return guarded([&] {
    launch_attention(q, k, v, o, q_scale, k_scale, v_scale, v_center, mask, msb, msh, msq, msk,
                     mask_dtype, cta_k, batch, lq, lk, hq, hkv, head_dim, q_b, q_n, q_h, k_b, k_n,
                     k_h, v_b, v_h, v_d, o_b, o_n, o_h, sm_scale, out_dtype, row_offsets,
                     block_indices, block_mass, causal != 0, lse, static_cast<cudaStream_t>(stream),
                     key_tiles);
  });
}

int ref_select_retained_mass(const float* sorted_mass, const int64_t* order, int32_t* counts,
                             uint8_t* support, double* row_totals, int32_t* row_offsets,
                             int32_t* block_indices, double* summary, void* scan_ws,
                             size_t scan_bytes, int rows, int key_blocks, double theta,
                             void* stream) {
  return guarded([&] {
    launch_select_retained_mass(sorted_mass, order, counts, support, row_totals, row_offsets,
                                block_indices, summary, scan_ws, scan_bytes, rows, key_blocks,
                                theta, static_cast<cudaStream_t>(stream));
  });
}

size_t ref_selector_workspace_size(int rows) { return retained_mass_selector_workspace_size(rows); }

int ref_prepare_key_mask_tiles(const void* mask, int32_t* tiles, int batch, int hq, int lk,
                               int tile, int64_t sb, int64_t sh, int64_t sk, int dtype,
                               void* stream) {
  return guarded([&] {
    launch_prepare_key_mask_tiles(mask, tiles, batch, hq, lk, tile, sb, sh, sk, dtype,
                                  static_cast<cudaStream_t>(stream));
  });
}

int ref_correct_lse(const void* q, const void* k, const int* anchors, float* out, int batch,
                    int hq, int hk, int nq, int head_dim, int64_t qb, int64_t qh, int64_t qn,
                    int64_t kb, int64_t kh, int64_t kn, float scale, int dtype, void* stream) {
  return guarded([&] {
    launch_correct_lse(q, k, anchors, out, batch, hq, hk, nq, head_dim, qb, qh, qn, kb, kh, kn,
                       scale, dtype, static_cast<cudaStream_t>(stream));
  });
}
}
