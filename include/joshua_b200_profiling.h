/* joshua_b200 - profiling aids, exported only by builds made with -DJQ_PROFILING
 * (python -m joshua_b200.build --profiling).  Release builds do not contain these entry
 * points, nor the measurement switches read from the environment (JQ_DEBUG_TC_SKIP,
 * JQ_NO_NARROW_K, JQ_MOE_BUCKET_TOKENS).  No counterpart in the reference. */
#ifndef JOSHUA_B200_PROFILING_H
#define JOSHUA_B200_PROFILING_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Profiling aid: with a device buffer of 512 uint64, CTA (0, 0) of the tile GEMM stores eight SM-cycle stamps
 * per K step for its first 64 steps (converter thread 0: stage free, stage handed over; issuing thread: top of
 * the step, accumulator half free, operands complete, MMAs issued, stage commit issued, end); NULL = off. */
int32_t jq_debug_gemm_trace(uint64_t* trace_dev);

/* Profiling aid: with a device buffer of 8 uint64 the last CTA of the decode router kernel stores the GPU
 * nanosecond timer at its phases (entered, logits stored, counted in, routed, jobs built); NULL = off. */
int32_t jq_debug_moe_trace(uint64_t* trace_dev);

#ifdef __cplusplus
}
#endif
#endif /* JOSHUA_B200_PROFILING_H */
