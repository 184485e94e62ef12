/*
 * Measurement probe shipped beside the library (librisa_b200_probe.so), not part of the product
 * ABI: the INT8 tensor-pipe ceiling the attention kernel's roofline fraction is read against.
 * No counterpart in the reference.
 */
#ifndef RISA_B200_PROBE_H
#define RISA_B200_PROBE_H
#ifdef __cplusplus
extern "C" {
#endif

/* Launches one CTA per SM that issues `mma_per_cta` back-to-back tcgen05.mma kind::i8 128x256x32
 * instructions on shared-memory operands (no global loads).  Timed by the caller (events on
 * `stream`), ops_per_launch / time is the INT8 tensor issue-loop throughput of this GPU at its
 * current clocks.  Writes the CTA count and the operation count (2*M*N*K per MMA) of one launch.
 * Returns 0 on success, a cudaError_t value otherwise. */
int risa_b200_mma_i8_issue_loop(int mma_per_cta, int* ctas, double* ops_per_launch, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* RISA_B200_PROBE_H */
