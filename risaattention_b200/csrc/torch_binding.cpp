// PyTorch C++ extension over the C-ABI of librisa_b200.so: the native module the Python runtime
// calls.  It mirrors the reference project's nanobind module `_C` (csrc/bindings.cpp:642-673): same
// function names, argument order, keyword names and defaults, so the reference's own Python
// runtime can use it unchanged.  A tensor argument may be a torch.Tensor or a DLPack capsule (what
// the reference's runtime passes); scratch pointers may be tensors or raw integer addresses.  The
// module only unpacks shapes, strides and pointers and forwards them: every kernel, and every
// check on what the kernels can take, lives behind include/risa_b200.h.  A non-zero status becomes
// RuntimeError carrying risa_b200_last_error().  Every entry point makes the device of its first
// tensor current for the duration of the call, so tensors on a GPU other than the thread's current
// one are served on their own GPU (the library launches on the current device).
#include <torch/extension.h>

#include <ATen/DLConvertor.h>
#include <c10/core/DeviceGuard.h>

#include <climits>
#include <cstdint>
#include <initializer_list>
#include <optional>
#include <stdexcept>
#include <string>

#include "../../include/risa_b200.h"

namespace py = pybind11;

namespace {

void check(int status) {
  if (status != RISA_B200_OK) throw std::runtime_error(risa_b200_last_error());
}

// torch.Tensor passes through; a DLPack capsule is imported without a copy (and, as DLPack
// prescribes, can be imported only once).
at::Tensor tensor_of(const py::handle& object, const char* what) {
  if (THPVariable_Check(object.ptr())) return THPVariable_Unpack(object.ptr());
  if (PyCapsule_CheckExact(object.ptr())) {
    auto* managed =
        static_cast<DLManagedTensor*>(PyCapsule_GetPointer(object.ptr(), "dltensor"));
    if (managed == nullptr) {
      PyErr_Clear();
      throw std::runtime_error(std::string(what) +
                               ": DLPack capsule was already consumed or is not a tensor");
    }
    at::Tensor tensor = at::fromDLPack(managed);
    PyCapsule_SetName(object.ptr(), "used_dltensor");
    return tensor;
  }
  throw std::runtime_error(std::string(what) + ": expected a torch.Tensor or a DLPack capsule");
}

std::optional<at::Tensor> optional_tensor(const py::object& object, const char* what) {
  if (object.is_none()) return std::nullopt;
  return tensor_of(object, what);
}

// Device address from a tensor, a capsule, an integer address or None.
void* address_of(const py::object& object, const char* what) {
  if (object.is_none()) return nullptr;
  if (py::isinstance<py::int_>(object))
    return reinterpret_cast<void*>(object.cast<uintptr_t>());
  return tensor_of(object, what).data_ptr();
}

void* stream_of(uintptr_t stream_ptr) { return reinterpret_cast<void*>(stream_ptr); }

// True when `t` has this element type and exactly these sizes, densely packed in row-major order.
bool packed_as(const at::Tensor& t, at::ScalarType type, std::initializer_list<int64_t> sizes) {
  if (t.scalar_type() != type || t.dim() != int64_t(sizes.size())) return false;
  int64_t axis = 0;
  for (const int64_t size : sizes)
    if (t.size(axis++) != size) return false;
  return t.is_contiguous();
}

// Visible-tile lists hold, per (batch, query head), the ids of the key tiles with a visible key
// and, in the last slot, their count (csrc/bindings.cpp:52-68).
void require_key_mask_tiles(const at::Tensor& tiles, int64_t batch, int64_t q_heads,
                            int64_t key_length, int tile_size) {
  if (!tiles.is_cuda() ||
      !packed_as(tiles, at::kInt, {batch, q_heads, (key_length + tile_size - 1) / tile_size + 1}))
    throw std::runtime_error("key mask tiles must be contiguous CUDA int32 [B,Hq,tiles+1]");
}

int dtype_code(const at::Tensor& t) {
  switch (t.scalar_type()) {
    case at::kFloat: return 0;
    case at::kHalf: return 1;
    case at::kBFloat16: return 2;
    case at::kBool: return 3;
    default: return -1;
  }
}

void quantize_tensors(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v,
                      const at::Tensor& q_int8, const at::Tensor& q_scale,
                      const at::Tensor& k_int8, const at::Tensor& k_scale,
                      const at::Tensor& v_int8, const at::Tensor& v_scale,
                      const at::Tensor& v_center, int cta_k, int input_dtype_code,
                      bool use_midpoint_affine, uintptr_t stream_ptr, void* anchors,
                      void* kv_table, void* q_table, std::optional<at::Tensor> workspace) {
  const c10::DeviceGuard on_device(q.device());
  // shapes the kernels index by, checked in the order of the reference module
  // (csrc/bindings.cpp:196-246); what the kernels themselves can take is checked behind the C-ABI
  if (q.dim() != 4 || k.dim() != 4 || v.dim() != 4)
    throw std::runtime_error(
        "risa_sdpa_quantize: q, k, and v must be 4D [batch_size,num_heads,L,head_dim]");
  if (cta_k != 64 && cta_k != 128)
    throw std::runtime_error("risa_sdpa_quantize: cta_k must be 64 or 128");
  if (input_dtype_code < 0 || input_dtype_code > 2)
    throw std::runtime_error(
        "risa_sdpa_quantize: input_dtype_code must be 0 (fp32), 1 (fp16), or 2 (bf16)");
  if (anchors == nullptr)
    throw std::runtime_error("risa_sdpa_quantize: anchor_indices scratch is required");
  const int b = int(q.size(0)), hq = int(q.size(1)), lq = int(q.size(2)), d = int(q.size(3));
  const int hkv = int(k.size(1)), lk = int(k.size(2));
  const int64_t padded = int64_t(lk + cta_k - 1) / cta_k * cta_k;
  if (k.size(0) != b || v.size(0) != b || v.size(1) != hkv || v.size(2) != lk || k.size(3) != d ||
      v.size(3) != d)
    throw std::runtime_error("risa_sdpa_quantize: incompatible q, k, and v shapes");
  if (dtype_code(q) != input_dtype_code || dtype_code(k) != input_dtype_code ||
      dtype_code(v) != input_dtype_code)
    throw std::runtime_error("risa_sdpa_quantize: q, k, and v must have the element type "
                             "input_dtype_code names");
  if (!packed_as(q_int8, at::kChar, {b, hq, lq, d}) || !packed_as(k_int8, at::kChar, {b, hkv, lk, d}) ||
      !packed_as(v_int8, at::kChar, {int64_t(b) * hkv * d, padded}))
    throw std::runtime_error("risa_sdpa_quantize: incompatible INT8 output shapes");
  const int64_t q_blocks = (lq + 127) / 128, k_tiles = padded / cta_k;
  if (q_scale.numel() < int64_t(b) * hq * q_blocks * (d == 256 ? 64 : 32) ||
      k_scale.numel() < int64_t(b) * hkv * k_tiles * 4 || v_scale.numel() < int64_t(b) * hkv * d ||
      v_center.numel() < int64_t(b) * hkv * d || !q_scale.is_contiguous() ||
      !k_scale.is_contiguous() || !v_scale.is_contiguous() || !v_center.is_contiguous())
    throw std::runtime_error("risa_sdpa_quantize: scale and centre tensors must be contiguous "
                             "float32 with one entry per quantization group");
  if (!workspace.has_value()) {
    // scratch of the V quantiser, taken from the caching allocator on the current stream
    const size_t bytes = risa_b200_quantize_v_workspace_size(b, hkv, lk, d);
    workspace = at::empty({int64_t(bytes)}, q.options().dtype(at::kByte));
  }
  check(risa_b200_quantize_qkv(
      q.data_ptr(), q_int8.data_ptr(), q_scale.data_ptr<float>(), k.data_ptr(), k_int8.data_ptr(),
      k_scale.data_ptr<float>(), v.data_ptr(), v_int8.data_ptr(), v_scale.data_ptr<float>(),
      v_center.data_ptr<float>(), b, hq, lq, hkv, lk, d, cta_k, int(v_int8.size(1)), q.stride(0),
      q.stride(1), q.stride(2), k.stride(0), k.stride(1), k.stride(2), v.stride(0), v.stride(1),
      v.stride(2), input_dtype_code, use_midpoint_affine ? 1 : 0, static_cast<int32_t*>(anchors),
      static_cast<const int32_t*>(q_table), static_cast<const int32_t*>(kv_table),
      workspace->data_ptr(), size_t(workspace->numel()), stream_of(stream_ptr)));
}

void attend_tensors(const at::Tensor& q_int8, const at::Tensor& k_int8, const at::Tensor& v_int8,
                    const at::Tensor& o, const at::Tensor& q_scale, const at::Tensor& k_scale,
                    const at::Tensor& v_scale, const at::Tensor& v_center, int cta_k,
                    float sm_scale, int output_dtype_code, uintptr_t stream_ptr,
                    const std::optional<at::Tensor>& attn_mask,
                    const std::optional<at::Tensor>& row_offsets,
                    const std::optional<at::Tensor>& block_indices,
                    const std::optional<at::Tensor>& block_mass, bool is_causal,
                    const std::optional<at::Tensor>& lse,
                    const std::optional<at::Tensor>& key_mask_tiles) {
  const c10::DeviceGuard on_device(q_int8.device());
  // checked in the order of the reference module (csrc/bindings.cpp:290-432)
  if (q_int8.dim() != 4 || k_int8.dim() != 4 || v_int8.dim() != 2 || o.dim() != 4)
    throw std::runtime_error("risa_sdpa_prequantized: q/k/o must be 4D and packed v must be 2D");
  if (cta_k != 64 && cta_k != 128)
    throw std::runtime_error("risa_sdpa_prequantized: cta_k must be 64 or 128");
  if (output_dtype_code != 1 && output_dtype_code != 2)
    throw std::runtime_error(
        "risa_sdpa_prequantized: output_dtype_code must be 1 (fp16) or 2 (bf16)");
  const int64_t b = q_int8.size(0), hq = q_int8.size(1), lq = q_int8.size(2), d = q_int8.size(3);
  const int64_t hkv = k_int8.size(1), lk = k_int8.size(2);
  const int64_t padded = (lk + cta_k - 1) / cta_k * cta_k;
  if (cta_k == 128 && d == 64)
    throw std::runtime_error("risa_sdpa_prequantized: cta_k 128 requires head_dim 128 or 256");
  if (row_offsets.has_value() != block_indices.has_value())
    throw std::runtime_error(
        "risa_sdpa_prequantized: sparse row offsets and block indices must be provided together");
  if (block_mass.has_value() && row_offsets.has_value())
    throw std::runtime_error("risa_sdpa_prequantized: block mass requires dense attention");
  if (v_int8.size(0) != b * hkv * d || v_int8.size(1) != padded ||
      o.size(0) != b || o.size(1) != hq || o.size(2) != lq || o.size(3) != d ||
      k_int8.size(0) != b || k_int8.size(3) != d)
    throw std::runtime_error("risa_sdpa_prequantized: incompatible quantized tensor shapes");
  if (q_int8.scalar_type() != at::kChar || k_int8.scalar_type() != at::kChar ||
      v_int8.scalar_type() != at::kChar ||
      o.scalar_type() != (output_dtype_code == 1 ? at::kHalf : at::kBFloat16))
    throw std::runtime_error("risa_sdpa_prequantized: packed operands must be int8 and the "
                             "output of the type output_dtype_code names");
  const int64_t q_blocks = (lq + 127) / 128, k_tiles = padded / cta_k;
  if (q_scale.numel() < b * hq * q_blocks * (d == 256 ? 64 : 32) ||
      k_scale.numel() < b * hkv * k_tiles * 4 || v_scale.numel() < b * hkv * d ||
      v_center.numel() < b * hkv * d || !q_scale.is_contiguous() || !k_scale.is_contiguous() ||
      !v_scale.is_contiguous() || !v_center.is_contiguous())
    throw std::runtime_error("risa_sdpa_prequantized: scale and centre tensors must be "
                             "contiguous float32 with one entry per quantization group");
  const bool hnd = (lq <= 1 || o.stride(2) == d) && (hq <= 1 || o.stride(1) == lq * d);
  const bool nhd = (hq <= 1 || o.stride(1) == d) && (lq <= 1 || o.stride(2) == hq * d);
  if (!q_int8.is_contiguous() || !k_int8.is_contiguous() || !v_int8.is_contiguous() ||
      o.stride(3) != 1 || !(hnd || nhd))
    throw std::runtime_error("risa_sdpa_prequantized: quantized tensors must be contiguous and "
                             "output must use HND- or NHD-contiguous storage");
  if (lse.has_value() &&
      (lse->dim() != 3 || lse->size(0) != b || lse->size(1) != hq || lse->size(2) != lq ||
       lse->scalar_type() != at::kFloat || !lse->is_contiguous()))
    throw std::runtime_error(
        "risa_sdpa_prequantized: LSE must be contiguous float32 [batch_size,Hq,query_length]");
  int64_t ms[4] = {0, 0, 0, 0};
  int mask_code = -1;
  const void* mask_ptr = nullptr;
  if (attn_mask.has_value()) {
    const at::Tensor& m = *attn_mask;
    if (m.dim() != 4 || m.size(0) != b || m.size(1) != hq || m.size(2) != lq || m.size(3) != lk)
      throw std::runtime_error("risa_sdpa_prequantized: attention mask must be expanded to "
                               "[batch_size,query_heads,query_length,key_length]");
    mask_code = dtype_code(m);
    if (mask_code < 0)
      throw std::runtime_error("risa_sdpa_prequantized: attention mask must be bool, float16, "
                               "bfloat16, or float32");
    mask_ptr = m.data_ptr();
    for (int i = 0; i < 4; ++i) ms[i] = m.stride(i);
  }
  if (row_offsets.has_value()) {
    if (!packed_as(*row_offsets, at::kInt, {b * hq * q_blocks + 1}) ||
        block_indices->dim() != 1 || block_indices->scalar_type() != at::kInt)
      throw std::runtime_error("risa_sdpa_prequantized: sparse support must be contiguous int32 "
                               "CSR with batch_size*Hq*ceil(query_length/128)+1 row offsets");
    if (!block_indices->is_contiguous() || block_indices->numel() == 0)
      throw std::runtime_error(
          "risa_sdpa_prequantized: sparse CSR tensors must be non-empty and contiguous");
  }
  if (block_mass.has_value() &&
      !packed_as(*block_mass, at::kFloat,
                 {b * hq * q_blocks * k_tiles + b * hq * lq * (2 * k_tiles + 2)}))
    throw std::runtime_error("risa_sdpa_prequantized: block_mass workspace must contain "
                             "mass rows followed by captured tile statistics and softmax state");
  if (key_mask_tiles.has_value()) require_key_mask_tiles(*key_mask_tiles, b, hq, lk, cta_k);
  const int64_t o_b = b <= 1 ? hq * lq * d : o.stride(0);
  const int64_t o_n = lq <= 1 ? d : o.stride(2);
  const int64_t o_h = hq <= 1 ? lq * d : o.stride(1);
  auto i32 = [](const std::optional<at::Tensor>& t) {
    return t.has_value() ? static_cast<const int32_t*>(t->data_ptr()) : nullptr;
  };
  // room for the parts of a split last wave, only for the calls and shapes that take it
  std::optional<at::Tensor> scratch;
  if (mask_ptr == nullptr && !is_causal && !row_offsets.has_value() && !block_mass.has_value()) {
    const size_t bytes =
        risa_b200_attention_scratch_size(int(b), int(hq), int(lq), int(lk), int(d), cta_k);
    if (bytes > 0) scratch = at::empty({int64_t(bytes)}, q_int8.options().dtype(at::kByte));
  }
  check(risa_b200_attention_scratch(
      q_int8.data_ptr(), k_int8.data_ptr(), v_int8.data_ptr(), o.data_ptr(),
      q_scale.data_ptr<float>(), k_scale.data_ptr<float>(), v_scale.data_ptr<float>(),
      v_center.data_ptr<float>(), mask_ptr, ms[0], ms[1], ms[2], ms[3], mask_code, cta_k, int(b),
      int(lq), int(lk), int(hq), int(hkv), int(d), o_b, o_n, o_h, sm_scale, output_dtype_code,
      i32(row_offsets), i32(block_indices),
      block_mass.has_value() ? block_mass->data_ptr<float>() : nullptr, is_causal ? 1 : 0,
      lse.has_value() ? lse->data_ptr<float>() : nullptr, i32(key_mask_tiles),
      scratch.has_value() ? scratch->data_ptr() : nullptr,
      scratch.has_value() ? size_t(scratch->numel()) : 0, stream_of(stream_ptr)));
}

// ---- the reference module's entry points -------------------------------------------------------
void risa_sdpa_quantize(py::object q, py::object k, py::object v, py::object q_int8,
                        py::object q_scale, py::object k_int8, py::object k_scale,
                        py::object v_int8, py::object v_scale, py::object v_center, int cta_k,
                        int input_dtype_code, bool use_midpoint_affine, uintptr_t stream_ptr,
                        py::object anchor_indices_ptr, py::object permutation_ptr,
                        py::object q_permutation_ptr, py::object workspace) {
  quantize_tensors(tensor_of(q, "q"), tensor_of(k, "k"), tensor_of(v, "v"),
                   tensor_of(q_int8, "q_int8"), tensor_of(q_scale, "q_scale"),
                   tensor_of(k_int8, "k_int8"), tensor_of(k_scale, "k_scale"),
                   tensor_of(v_int8, "v_int8"), tensor_of(v_scale, "v_scale"),
                   tensor_of(v_center, "v_center"), cta_k, input_dtype_code, use_midpoint_affine,
                   stream_ptr, address_of(anchor_indices_ptr, "anchor_indices_ptr"),
                   address_of(permutation_ptr, "permutation_ptr"),
                   address_of(q_permutation_ptr, "q_permutation_ptr"),
                   optional_tensor(workspace, "workspace"));
}

void risa_sdpa_prequantized(py::object q_int8, py::object k_int8, py::object v_int8, py::object o,
                            py::object q_scale, py::object k_scale, py::object v_scale,
                            py::object v_center, int cta_k, float sm_scale, int output_dtype_code,
                            uintptr_t stream_ptr, py::object attn_mask,
                            py::object sparse_row_offsets, py::object sparse_block_indices,
                            py::object block_mass, bool is_causal, py::object lse,
                            py::object key_mask_tiles) {
  attend_tensors(tensor_of(q_int8, "q_int8"), tensor_of(k_int8, "k_int8"),
                 tensor_of(v_int8, "v_int8"), tensor_of(o, "o"), tensor_of(q_scale, "q_scale"),
                 tensor_of(k_scale, "k_scale"), tensor_of(v_scale, "v_scale"),
                 tensor_of(v_center, "v_center"), cta_k, sm_scale, output_dtype_code, stream_ptr,
                 optional_tensor(attn_mask, "attn_mask"),
                 optional_tensor(sparse_row_offsets, "sparse_row_offsets"),
                 optional_tensor(sparse_block_indices, "sparse_block_indices"),
                 optional_tensor(block_mass, "block_mass"), is_causal,
                 optional_tensor(lse, "lse"), optional_tensor(key_mask_tiles, "key_mask_tiles"));
}

void risa_sdpa(py::object q, py::object k, py::object v, py::object o, py::object q_int8,
               py::object q_scale, py::object k_int8, py::object k_scale, py::object v_int8,
               py::object v_scale, py::object v_center, float sm_scale, int input_dtype_code,
               int output_dtype_code, bool use_midpoint_affine, uintptr_t stream_ptr,
               py::object anchor_indices_ptr, py::object attn_mask, int cta_k, bool is_causal,
               py::object key_mask_tiles) {
  const at::Tensor tq = tensor_of(q, "q"), tk = tensor_of(k, "k"), tv = tensor_of(v, "v"),
                   to = tensor_of(o, "o");
  if (tq.dim() != 4 || tk.dim() != 4 || tv.dim() != 4 || to.dim() != 4)
    throw std::runtime_error("risa_sdpa: q, k, v, o must be 4D [batch_size,num_heads,L,head_dim]");
  if (input_dtype_code < 0 || input_dtype_code > 2)
    throw std::runtime_error("risa_sdpa: input_dtype_code must be 0 (fp32), 1 (fp16), or 2 (bf16)");
  void* anchors = address_of(anchor_indices_ptr, "anchor_indices_ptr");
  if (anchors == nullptr) throw std::runtime_error("risa_sdpa: anchor_indices scratch is required");
  const std::optional<at::Tensor> mask = optional_tensor(attn_mask, "attn_mask");
  if (cta_k == 0)  // csrc/bindings.cpp:549-551
    cta_k = (!mask.has_value() && tq.size(3) >= 128 && tk.size(2) > 1024) ? 128 : 64;
  const at::Tensor qi = tensor_of(q_int8, "q_int8"), qs = tensor_of(q_scale, "q_scale"),
                   ki = tensor_of(k_int8, "k_int8"), ks = tensor_of(k_scale, "k_scale"),
                   vi = tensor_of(v_int8, "v_int8"), vs = tensor_of(v_scale, "v_scale"),
                   vc = tensor_of(v_center, "v_center");
  quantize_tensors(tq, tk, tv, qi, qs, ki, ks, vi, vs, vc, cta_k, input_dtype_code,
                   use_midpoint_affine, stream_ptr, anchors, nullptr, nullptr, std::nullopt);
  attend_tensors(qi, ki, vi, to, qs, ks, vs, vc, cta_k, sm_scale, output_dtype_code, stream_ptr,
                 mask, std::nullopt, std::nullopt, std::nullopt, is_causal, std::nullopt,
                 optional_tensor(key_mask_tiles, "key_mask_tiles"));
}

size_t retained_mass_selector_workspace_size(int row_count) {
  return risa_b200_selector_workspace_size(row_count);
}

void select_retained_mass_csr(py::object sorted_mass, py::object descending_indices,
                              py::object counts, py::object support, py::object row_totals,
                              py::object row_offsets, py::object block_indices, py::object summary,
                              py::object scan_workspace, double theta, uintptr_t stream_ptr) {
  const at::Tensor mass = tensor_of(sorted_mass, "sorted_mass");
  const at::Tensor order = tensor_of(descending_indices, "descending_indices");
  const at::Tensor scan = tensor_of(scan_workspace, "scan_workspace");
  const c10::DeviceGuard on_device(mass.device());
  const at::Tensor count = tensor_of(counts, "counts"), kept = tensor_of(support, "support"),
                   totals = tensor_of(row_totals, "row_totals"),
                   offsets = tensor_of(row_offsets, "row_offsets"),
                   indices = tensor_of(block_indices, "block_indices"),
                   sums = tensor_of(summary, "summary");
  // every buffer the selector writes, checked as the reference module does
  // (csrc/bindings.cpp:95-140)
  if (mass.dim() != 2 || order.dim() != 2)
    throw std::runtime_error("select_retained_mass_csr: masses and indices must be 2D");
  const int64_t rows = mass.size(0), columns = mass.size(1);
  if (rows <= 0 || columns <= 0 || !packed_as(mass, at::kFloat, {rows, columns}) ||
      !packed_as(order, at::kLong, {rows, columns}) || !packed_as(count, at::kInt, {rows}) ||
      !packed_as(kept, at::kByte, {rows, columns}) || !packed_as(totals, at::kDouble, {rows, 2}) ||
      !packed_as(offsets, at::kInt, {rows + 1}) ||
      !packed_as(indices, at::kInt, {rows * columns}) || !packed_as(sums, at::kDouble, {3}) ||
      scan.dim() != 1 || scan.scalar_type() != at::kByte || !scan.is_contiguous())
    throw std::runtime_error("select_retained_mass_csr: invalid shape, dtype, or stride");
  if (rows > INT_MAX || columns > INT_MAX || rows > INT_MAX / columns)
    throw std::runtime_error("select_retained_mass_csr: matrix is too large");
  if (size_t(scan.numel()) < risa_b200_selector_workspace_size(int(rows)))
    throw std::runtime_error("select_retained_mass_csr: scan workspace is too small");
  check(risa_b200_select_retained_mass(
      mass.data_ptr<float>(), order.data_ptr<int64_t>(), count.data_ptr<int32_t>(),
      kept.data_ptr<uint8_t>(), totals.data_ptr<double>(), offsets.data_ptr<int32_t>(),
      indices.data_ptr<int32_t>(), sums.data_ptr<double>(),
      scan.numel() ? scan.data_ptr() : nullptr, size_t(scan.numel()), int(rows), int(columns),
      theta, stream_of(stream_ptr)));
}

void prepare_key_mask_tiles(py::object mask, py::object tiles, int tile_size,
                            uintptr_t stream_ptr) {
  const at::Tensor m = tensor_of(mask, "mask"), t = tensor_of(tiles, "tiles");
  const c10::DeviceGuard on_device(m.device());
  if (m.dim() != 4 || m.stride(2) != 0 || (tile_size != 64 && tile_size != 128))
    throw std::runtime_error("prepare_key_mask_tiles requires an expanded broadcast key mask");
  require_key_mask_tiles(t, m.size(0), m.size(1), m.size(3), tile_size);
  if (dtype_code(m) < 0 || !m.is_cuda() || m.device() != t.device())
    throw std::runtime_error(
        "prepare_key_mask_tiles requires matching CUDA devices and a supported mask dtype");
  check(risa_b200_prepare_key_mask_tiles(m.data_ptr(), static_cast<int32_t*>(t.data_ptr()),
                                         int(m.size(0)), int(m.size(1)), int(m.size(3)), tile_size,
                                         m.stride(0), m.stride(1), m.stride(3), dtype_code(m),
                                         stream_of(stream_ptr)));
}

void risa_lse_shift(py::object q, py::object k, py::object anchors, py::object out, float scale,
                    uintptr_t stream_ptr) {
  const at::Tensor tq = tensor_of(q, "q"), tk = tensor_of(k, "k");
  const c10::DeviceGuard on_device(tq.device());
  check(risa_b200_correct_lse(tq.data_ptr(), tk.data_ptr(),
                              static_cast<const int32_t*>(address_of(anchors, "anchors")),
                              tensor_of(out, "out").data_ptr<float>(), int(tq.size(0)),
                              int(tq.size(1)), int(tk.size(1)), int(tq.size(2)), int(tq.size(3)),
                              tq.stride(0), tq.stride(1), tq.stride(2), tk.stride(0), tk.stride(1),
                              tk.stride(2), scale, dtype_code(tq), stream_of(stream_ptr)));
}

// ---- additions of this library (declared in include/risa_b200.h) ------------------------------
size_t dense_scratch_size(int batch, int q_heads, int q_len, int kv_heads, int k_len, int head_dim,
                          int cta_k) {
  return risa_b200_dense_scratch_size(batch, q_heads, q_len, kv_heads, k_len, head_dim, cta_k);
}

void risa_dense_attention(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v,
                          const at::Tensor& o, const at::Tensor& scratch, int cta_k,
                          int input_dtype_code, bool use_midpoint_affine, float sm_scale,
                          int output_dtype_code, bool is_causal, uintptr_t stream_ptr) {
  const c10::DeviceGuard on_device(q.device());
  check(risa_b200_dense_attention(
      q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), scratch.data_ptr(),
      size_t(scratch.numel()), int(q.size(0)), int(q.size(1)), int(q.size(2)), int(k.size(1)),
      int(k.size(2)), int(q.size(3)), cta_k, q.stride(0), q.stride(1), q.stride(2), k.stride(0),
      k.stride(1), k.stride(2), v.stride(0), v.stride(1), v.stride(2), input_dtype_code,
      use_midpoint_affine ? 1 : 0, sm_scale, output_dtype_code, o.stride(0), o.stride(2),
      o.stride(1), is_causal ? 1 : 0, stream_of(stream_ptr)));
}

void risa_sdpa_select(const at::Tensor& q_int8, const at::Tensor& k_int8, const at::Tensor& v_int8,
                      const at::Tensor& o, const at::Tensor& q_scale, const at::Tensor& k_scale,
                      const at::Tensor& v_scale, const at::Tensor& v_center, int cta_k,
                      float sm_scale, int output_dtype_code, uintptr_t stream_ptr, double theta,
                      const at::Tensor& scratch, const at::Tensor& counts,
                      const at::Tensor& bitmaps, const at::Tensor& row_totals,
                      std::optional<at::Tensor> attn_mask, bool is_causal,
                      std::optional<at::Tensor> block_masses) {
  const c10::DeviceGuard on_device(q_int8.device());
  const int64_t b = q_int8.size(0), hq = q_int8.size(1), lq = q_int8.size(2), d = q_int8.size(3);
  const int64_t hkv = k_int8.size(1), lk = k_int8.size(2);
  int64_t ms[4] = {0, 0, 0, 0};
  int mask_code = -1;
  const void* mask_ptr = nullptr;
  if (attn_mask.has_value()) {
    mask_code = dtype_code(*attn_mask);
    mask_ptr = attn_mask->data_ptr();
    for (int i = 0; i < 4; ++i) ms[i] = attn_mask->stride(i);
  }
  const int64_t o_b = b <= 1 ? hq * lq * d : o.stride(0);
  const int64_t o_n = lq <= 1 ? d : o.stride(2);
  const int64_t o_h = hq <= 1 ? lq * d : o.stride(1);
  check(risa_b200_attention_select(
      q_int8.data_ptr(), k_int8.data_ptr(), v_int8.data_ptr(), o.data_ptr(),
      q_scale.data_ptr<float>(), k_scale.data_ptr<float>(), v_scale.data_ptr<float>(),
      v_center.data_ptr<float>(), mask_ptr, ms[0], ms[1], ms[2], ms[3], mask_code, cta_k, int(b),
      int(lq), int(lk), int(hq), int(hkv), int(d), o_b, o_n, o_h, sm_scale, output_dtype_code,
      is_causal ? 1 : 0, theta, scratch.data_ptr(), size_t(scratch.numel()) * scratch.element_size(),
      block_masses.has_value() ? block_masses->data_ptr<float>() : nullptr,
      static_cast<int32_t*>(counts.data_ptr()), static_cast<uint32_t*>(bitmaps.data_ptr()),
      row_totals.data_ptr<double>(), stream_of(stream_ptr)));
}

void pack_selected(const at::Tensor& counts, const at::Tensor& bitmaps,
                   const at::Tensor& row_totals, const at::Tensor& row_offsets,
                   const at::Tensor& block_indices, const at::Tensor& summary, int key_blocks,
                   uintptr_t stream_ptr) {
  const c10::DeviceGuard on_device(counts.device());
  check(risa_b200_pack_selected(
      static_cast<const int32_t*>(counts.data_ptr()),
      static_cast<const uint32_t*>(bitmaps.data_ptr()), row_totals.data_ptr<double>(),
      static_cast<int32_t*>(row_offsets.data_ptr()),
      static_cast<int32_t*>(block_indices.data_ptr()), summary.data_ptr<double>(),
      int(counts.numel()), key_blocks, stream_of(stream_ptr)));
}

size_t quantize_v_workspace_size(int batch, int kv_heads, int k_len, int head_dim) {
  return risa_b200_quantize_v_workspace_size(batch, kv_heads, k_len, head_dim);
}

// The nine device buffers of one quantisation call in the public packed layouts, allocated here in
// one foreign call (nine allocations from Python are a third of a short call's host time): Q codes,
// K codes, Q scales, K scales, packed V codes, V scales, V centres, anchor rows, V-quantiser
// scratch.  `q` and `k` are the padded inputs [B,H,L,D]; shapes as risa_sdpa_quantize expects them.
py::tuple allocate_packed(const at::Tensor& q, const at::Tensor& k, int cta_k) {
  if (q.dim() != 4 || k.dim() != 4 || (cta_k != 64 && cta_k != 128))
    throw std::runtime_error("allocate_packed: q and k must be 4D and cta_k 64 or 128");
  const c10::DeviceGuard on_device(q.device());
  const int64_t b = q.size(0), hq = q.size(1), lq = q.size(2), d = q.size(3);
  const int64_t hkv = k.size(1), lk = k.size(2);
  const int64_t padded = (lk + cta_k - 1) / cta_k * cta_k;
  const auto bytes = q.options().dtype(at::kChar);
  const auto floats = q.options().dtype(at::kFloat);
  at::Tensor v_scale = at::empty({b * hkv * d}, floats);
  return py::make_tuple(
      at::empty({b, hq, lq, d}, bytes), at::empty({b, hkv, lk, d}, bytes),
      at::empty({b, hq, (lq + 127) / 128 * (d == 256 ? 64 : 32)}, floats),
      at::empty({b, hkv, padded / cta_k * 4}, floats), at::empty({b * hkv * d, padded}, bytes),
      v_scale, at::empty_like(v_scale), at::empty({b, hkv}, q.options().dtype(at::kInt)),
      at::empty({int64_t(risa_b200_quantize_v_workspace_size(int(b), int(hkv), int(lk), int(d)))},
                q.options().dtype(at::kByte)));
}

}  // namespace

PYBIND11_MODULE(_C, m) {
  m.doc() = "B200-native RISA attention kernels (PyTorch C++ extension over librisa_b200.so)";
  m.attr("fused_gather_version") = 1;
  m.def("risa_lse_shift", &risa_lse_shift, py::arg("q"), py::arg("k"), py::arg("anchors"),
        py::arg("out"), py::arg("scale"), py::arg("stream_ptr"));
  m.def("risa_sdpa_quantize", &risa_sdpa_quantize, py::arg("q"), py::arg("k"), py::arg("v"),
        py::arg("q_int8"), py::arg("q_scale"), py::arg("k_int8"), py::arg("k_scale"),
        py::arg("v_int8"), py::arg("v_scale"), py::arg("v_center"), py::arg("cta_k"),
        py::arg("input_dtype_code"), py::arg("use_midpoint_affine"), py::arg("stream_ptr"),
        py::arg("anchor_indices_ptr"), py::arg("permutation_ptr") = 0, py::kw_only(),
        py::arg("q_permutation_ptr") = 0, py::arg("workspace") = py::none());
  m.def("prepare_key_mask_tiles", &prepare_key_mask_tiles, py::arg("mask"), py::arg("tiles"),
        py::arg("tile_size"), py::arg("stream_ptr"));
  m.def("risa_sdpa_prequantized", &risa_sdpa_prequantized, py::arg("q_int8"), py::arg("k_int8"),
        py::arg("v_int8"), py::arg("o"), py::arg("q_scale"), py::arg("k_scale"),
        py::arg("v_scale"), py::arg("v_center"), py::arg("cta_k"), py::arg("sm_scale"),
        py::arg("output_dtype_code"), py::arg("stream_ptr"), py::arg("attn_mask") = py::none(),
        py::arg("sparse_row_offsets") = py::none(), py::arg("sparse_block_indices") = py::none(),
        py::arg("block_mass") = py::none(), py::arg("is_causal") = false,
        py::arg("lse") = py::none(), py::arg("key_mask_tiles") = py::none());
  m.def("select_retained_mass_csr", &select_retained_mass_csr, py::arg("sorted_mass"),
        py::arg("descending_indices"), py::arg("counts"), py::arg("support"),
        py::arg("row_totals"), py::arg("row_offsets"), py::arg("block_indices"),
        py::arg("summary"), py::arg("scan_workspace"), py::arg("theta"), py::arg("stream_ptr"));
  m.def("retained_mass_selector_workspace_size", &retained_mass_selector_workspace_size,
        py::arg("row_count"));
  m.def("risa_sdpa", &risa_sdpa, py::arg("q"), py::arg("k"), py::arg("v"), py::arg("o"),
        py::arg("q_int8"), py::arg("q_scale"), py::arg("k_int8"), py::arg("k_scale"),
        py::arg("v_int8"), py::arg("v_scale"), py::arg("v_center"), py::arg("sm_scale"),
        py::arg("input_dtype_code"), py::arg("output_dtype_code"), py::arg("use_midpoint_affine"),
        py::arg("stream_ptr"), py::arg("anchor_indices_ptr"), py::arg("attn_mask") = py::none(),
        py::arg("cta_k") = 0, py::arg("is_causal") = false,
        py::arg("key_mask_tiles") = py::none());
  m.def("dense_scratch_size", &dense_scratch_size);
  m.def("risa_dense_attention", &risa_dense_attention);
  m.def("quantize_v_workspace_size", &quantize_v_workspace_size);
  m.def("allocate_packed", &allocate_packed, py::arg("q"), py::arg("k"), py::arg("cta_k"));
  m.def("select_scratch_size",
        [](int k_len, int cta_k) { return risa_b200_select_scratch_size(k_len, cta_k); });
  m.def("select_max_key_tiles", [](int cta_k) { return risa_b200_select_max_key_tiles(cta_k); });
  m.def("risa_sdpa_select", &risa_sdpa_select, py::arg("q_int8"), py::arg("k_int8"),
        py::arg("v_int8"), py::arg("o"), py::arg("q_scale"), py::arg("k_scale"),
        py::arg("v_scale"), py::arg("v_center"), py::arg("cta_k"), py::arg("sm_scale"),
        py::arg("output_dtype_code"), py::arg("stream_ptr"), py::arg("theta"), py::arg("scratch"),
        py::arg("counts"), py::arg("bitmaps"), py::arg("row_totals"),
        py::arg("attn_mask") = py::none(), py::arg("is_causal") = false,
        py::arg("block_masses") = py::none());
  m.def("pack_selected", &pack_selected);
  m.def("device_status", [] { check(risa_b200_device_status()); });
  m.def("set_attention_path", [](int path) { return risa_b200_set_attention_path(path); });
  m.def("bounded_wait_self_test", [](uint64_t limit_ns, uintptr_t stream_ptr) {
    check(risa_b200_bounded_wait_self_test(limit_ns, stream_of(stream_ptr)));
  });
  m.def("abi_version", [] { return risa_b200_abi_version(); });
}
