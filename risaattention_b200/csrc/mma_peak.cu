// Issue-loop microbenchmark of the INT8 tensor pipe: the denominator of the attention kernel's
// roofline when no measured INT8 figure is available from elsewhere.  One CTA per SM; one thread
// issues back-to-back tcgen05.mma kind::i8 128 x 256 x 32 instructions on operands that stay in
// shared memory, alternating between two tensor-memory accumulators, and waits (bounded) for the
// last one.  Operand values are whatever shared memory holds: integer MMAs have no slow inputs.
// Built into its own library (librisa_b200_probe.so): a measurement aid, not part of the product.
#include "../../include/risa_b200_probe.h"
#include "tc_ptx.cuh"

namespace risa_b200 {
namespace {

using namespace tc;

constexpr int kPeakThreads = 128;
constexpr int kPeakSmem = 16384 + 32768 + 1024 + 64;  // A 128 x 128 B, B 256 x 128 B, alignment, barrier

__global__ void __launch_bounds__(kPeakThreads, 1) mma_i8_issue_loop_kernel(int mma_count) {
  extern __shared__ unsigned char peak_smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(peak_smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t sbase = smem_u32(smem);
  const uint32_t bar = sbase + 16384 + 32768, slot = bar + 16, gave_up = bar + 32;
  const int warp = threadIdx.x >> 5;
  // defined operand bytes (any integers do)
  for (int i = threadIdx.x; i < (16384 + 32768) / 4; i += kPeakThreads)
    reinterpret_cast<uint32_t*>(smem)[i] = 0x01020304u * (i + 1);
  if (threadIdx.x == 0) {
    *reinterpret_cast<volatile uint32_t*>(smem + 16384 + 32768 + 32) = 0u;
    mbar_init(bar, 1);
    mbar_init_fence();
  }
  if (warp == 0) tmem_alloc(slot, 512);
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(smem + 16384 + 32768 + 16);
  if (threadIdx.x == 0) {
    constexpr uint32_t idesc = idesc_i8(true, true, 256);
    const uint64_t desc_a = smem_desc_k128(sbase), desc_b = smem_desc_k128(sbase + 16384);
#pragma unroll 1
    for (int i = 0; i < mma_count; ++i)
      mma_i8(tmem + 256 * ((i >> 2) & 1), desc_a + 2 * (i & 3), desc_b + 2 * (i & 3), idesc,
             (i & 3) != 0);
    mma_commit(bar);
    mbar_wait(bar, 0, gave_up, 901);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

}  // namespace
}  // namespace risa_b200

extern "C" int risa_b200_mma_i8_issue_loop(int mma_per_cta, int* ctas, double* ops_per_launch,
                                           void* stream) {
  using namespace risa_b200;
  if (mma_per_cta <= 0 || mma_per_cta > (1 << 20) || !ctas || !ops_per_launch)
    return int(cudaErrorInvalidValue);
  int device = 0, sms = 0;
  cudaError_t e = cudaGetDevice(&device);
  if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
  if (e != cudaSuccess) return int(e);
  static thread_local int configured = -1;
  if (configured != device) {
    e = cudaFuncSetAttribute(mma_i8_issue_loop_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             kPeakSmem);
    if (e != cudaSuccess) return int(e);
    configured = device;
  }
  mma_i8_issue_loop_kernel<<<sms, kPeakThreads, kPeakSmem, static_cast<cudaStream_t>(stream)>>>(
      mma_per_cta);
  *ctas = sms;
  *ops_per_launch = 2.0 * 128 * 256 * 32 * double(mma_per_cta) * sms;
  return int(cudaGetLastError());
}
