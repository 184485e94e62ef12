// Shared host/device helpers for the B200 RISA kernels.
#pragma once
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "../../include/risa_b200.h"

namespace risa_b200 {

// ---- host-side status plumbing -----------------------------------------------------------
char* error_buffer();  // thread-local, 512 bytes (defined in cabi.cu)

inline int fail(int code, const char* fmt, ...) {
  va_list args;
  va_start(args, fmt);
  vsnprintf(error_buffer(), 512, fmt, args);
  va_end(args);
  return code;
}

inline int check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(RISA_B200_CUDA, "%s: %s", what, cudaGetErrorString(e));
  return RISA_B200_OK;
}

#define RISA_REQUIRE(cond, ...)                                   \
  do {                                                            \
    if (!(cond)) return ::risa_b200::fail(RISA_B200_INVALID, __VA_ARGS__); \
  } while (0)

// ---- device helpers ----------------------------------------------------------------------
#ifdef __CUDACC__
template <typename T> struct Load4;
template <> struct Load4<float> {
  static __device__ __forceinline__ void load(const float* p, float* out) {
    const float4 raw = __ldg(reinterpret_cast<const float4*>(p));
    out[0] = raw.x; out[1] = raw.y; out[2] = raw.z; out[3] = raw.w;
  }
};
template <> struct Load4<__half> {
  static __device__ __forceinline__ void load(const __half* p, float* out) {
    const uint2 raw = __ldg(reinterpret_cast<const uint2*>(p));
    const __half2 a = *reinterpret_cast<const __half2*>(&raw.x);
    const __half2 b = *reinterpret_cast<const __half2*>(&raw.y);
    out[0] = __low2float(a); out[1] = __high2float(a);
    out[2] = __low2float(b); out[3] = __high2float(b);
  }
};
template <> struct Load4<__nv_bfloat16> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float* out) {
    const uint2 raw = __ldg(reinterpret_cast<const uint2*>(p));
    out[0] = __uint_as_float(raw.x << 16); out[1] = __uint_as_float(raw.x & 0xffff0000u);
    out[2] = __uint_as_float(raw.y << 16); out[3] = __uint_as_float(raw.y & 0xffff0000u);
  }
};

template <typename T> __device__ __forceinline__ float load_scalar(const T* p) {
  return static_cast<float>(__ldg(p));
}

// cvt.rni.sat.s8.f32: round to nearest even, saturate to [-128, 127].
__device__ __forceinline__ uint32_t to_s8(float x) {
  int32_t q;
  asm("cvt.rni.sat.s8.f32 %0, %1;" : "=r"(q) : "f"(x));
  return static_cast<uint32_t>(q) & 0xffu;
}
// Four codes in one word, a in the lowest byte.  Round to nearest even to a 32-bit integer, then the
// saturating pack (two values per instruction, the third operand supplies the upper half): the
// same bytes as four cvt.rni.sat.s8.f32 (both clamp to [-128, 127] after the same rounding; NaN
// gives 0 either way) with fewer than half the instructions.
__device__ __forceinline__ uint32_t pack4_s8(float a, float b, float c, float d) {
  int32_t ia, ib, ic, id;
  asm("cvt.rni.s32.f32 %0, %1;" : "=r"(ia) : "f"(a));
  asm("cvt.rni.s32.f32 %0, %1;" : "=r"(ib) : "f"(b));
  asm("cvt.rni.s32.f32 %0, %1;" : "=r"(ic) : "f"(c));
  asm("cvt.rni.s32.f32 %0, %1;" : "=r"(id) : "f"(d));
  uint32_t hi, w;
  asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(hi) : "r"(id), "r"(ic), "r"(0));
  asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(w) : "r"(ib), "r"(ia), "r"(hi));
  return w;
}
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float lg2_approx(float x) {
  float y;
  asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float rcp_approx(float x) {
  float y;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// ---- packed FP32 pairs --------------------------------------------------------------------------
// Two FP32 lanes in one 64-bit register: one instruction does both fused multiply-adds.
__device__ __forceinline__ uint64_t pack_f32x2(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack_f32x2(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma_f32x2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.ftz.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t add_f32x2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.ftz.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ uint64_t mul_f32x2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("mul.rn.ftz.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}

#endif


// ---- chained launches ---------------------------------------------------------------------------
// The kernels of one call form a chain in which each needs the results of the one before.  They are
// launched with programmatic stream serialisation: a kernel's CTAs may be placed on the SMs while
// the previous kernel drains, and wait at chain_wait() until that kernel has completed and its
// writes are visible; chain_release() lets the next kernel's CTAs be placed as soon as every CTA of
// this one has started.  Every kernel launched through launch_chained() must call chain_wait()
// before its first global memory access, which also keeps the chain ordered transitively.
#ifdef __CUDACC__
__device__ __forceinline__ void chain_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void chain_release() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
template <typename... Params, typename... Args>
inline cudaError_t launch_chained(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem,
                                  cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attribute;
  config.numAttrs = 1;
  return cudaLaunchKernelEx(&config, kernel, static_cast<Params>(args)...);
}
#endif

#define RISA_DISPATCH_FLOAT(code, T, ...)                 \
  do {                                                    \
    if ((code) == 0) { using T = float; __VA_ARGS__; }    \
    else if ((code) == 1) { using T = __half; __VA_ARGS__; } \
    else { using T = __nv_bfloat16; __VA_ARGS__; }        \
  } while (0)

}  // namespace risa_b200
