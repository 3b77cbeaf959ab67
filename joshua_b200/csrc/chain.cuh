// One operation of a persistent decode chain (gemv_mma.cu: gemv_chain_kernel).
#pragma once

#include "attention_fused.cuh"

namespace jq {

struct ChainOp {
    int32_t kind;    // 0 = quantized linear, 1 = attention
    int32_t swiglu;  // linear: tiles come in (gate, up) pairs and dst = silu(g) * u
    const uint8_t* w[2];
    uint64_t n, k;
    const float* x;         // [m, k] f32 input rows
    float* dst;             // [m, n]
    const float* norm_w;    // RMS-norm weights applied to x first, or NULL
    const float* residual;  // added to the product, or NULL (may be dst)
    float norm_eps, clamp;
    AttnArgs att;
};


// All linears of a chain share one block type and the batch m (1..8, activation planes of the widest input in
// shared memory).  ops_dev: the operations in device memory; max_k: the widest linear input; att_floats: the
// largest attention_fused_smem_floats of the chain's attention steps (0 = none); arrivals: a device u64 that
// starts at zero and is owned by this chain; trace: optional device buffer of 3 * n_ops u64 in which CTA 0
// leaves nanosecond timestamps (operation entered, activations split, last store done).
bool gemv_chain_supports(uint32_t type, uint64_t m, uint64_t max_k, uint32_t att_floats);
cudaError_t launch_gemv_chain(uint32_t type, uint32_t m, const ChainOp* ops_dev, uint32_t n_ops, uint64_t max_k,
                              uint32_t att_floats, unsigned long long* arrivals, int* error_flag, cudaStream_t s,
                              unsigned long long* trace = nullptr);

}  // namespace jq
