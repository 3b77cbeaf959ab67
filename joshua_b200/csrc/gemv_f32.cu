// Exact-decode float matmul over raw blocks: dst[m, n] = lhs[m, k] . W[n, k]^T.
//
// One warp per weight row.  Each lane decodes 8-value units (formats.cuh) to the
// same f32 weights the reference's fused kernels form in registers
// (src/kquant_dot.rs:268-483, src/iq2xxs.rs:331-391, src/mxfp4.rs:208-235),
// multiplies them into up to 8 activation rows at a time with f32 FMAs and the
// warp reduces with shuffles.  The weights are bit-identical to the reference's;
// only the summation order differs.  This is the any-shape path (any m, any k
// that is a block multiple, any alignment the format allows); the batch-1..8
// decode kernels in gemv_mma.cu are the fast path.
// HBM-bound for small m: algorithmic bytes = weight bytes + 4*m*(k + n).
#include "common.cuh"

namespace jq {

cudaError_t tables_gemv_f32() { return upload_tables(); }

namespace {

constexpr int MT = 8;             // activation rows per pass
constexpr int WARPS_PER_CTA = 8;  // rows per CTA

template <uint32_t TYPE, uint32_t ELEMS, uint32_t BYTES>
__global__ void __launch_bounds__(WARPS_PER_CTA * 32)
    matmul_f32_kernel(const uint8_t* __restrict__ w, uint64_t n, uint64_t k, const float* __restrict__ lhs, uint64_t m,
                      float* __restrict__ dst) {
    const uint32_t lane = threadIdx.x & 31;
    const uint64_t row = blockIdx.x * (uint64_t)WARPS_PER_CTA + (threadIdx.x >> 5);
    if (row >= n) return;
    const uint64_t row_bytes = k / ELEMS * BYTES;
    const uint8_t* wr = w + row * row_bytes;
    const uint32_t units = (uint32_t)(k / 8);
    constexpr uint32_t UPB = ELEMS / 8;
    for (uint64_t m0 = 0; m0 < m; m0 += MT) {
        const int mc = (int)(m - m0 < MT ? m - m0 : MT);
        float acc[MT];
#pragma unroll
        for (int i = 0; i < MT; ++i) acc[i] = 0.0f;
        for (uint32_t u = lane; u < units; u += 32) {
            float v[8];
            decode_unit<TYPE>(wr + (uint64_t)(u / UPB) * BYTES, u % UPB, v, false);
#pragma unroll
            for (int i = 0; i < MT; ++i) {
                if (i < mc) {
                    const float4* x = reinterpret_cast<const float4*>(lhs + (m0 + i) * k + (uint64_t)u * 8);
                    float4 a = __ldg(x), b = __ldg(x + 1);
                    float s = acc[i];
                    s = fmaf(a.x, v[0], s);
                    s = fmaf(a.y, v[1], s);
                    s = fmaf(a.z, v[2], s);
                    s = fmaf(a.w, v[3], s);
                    s = fmaf(b.x, v[4], s);
                    s = fmaf(b.y, v[5], s);
                    s = fmaf(b.z, v[6], s);
                    s = fmaf(b.w, v[7], s);
                    acc[i] = s;
                }
            }
        }
#pragma unroll
        for (int i = 0; i < MT; ++i) {
            float s = acc[i];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xFFFFFFFFu, s, o);
            if (lane == 0 && i < mc) dst[(m0 + i) * n + row] = s;
        }
    }
}

}  // namespace

cudaError_t launch_matmul_f32(uint32_t type, const uint8_t* w, uint64_t n, uint64_t k, const float* lhs, uint64_t m,
                              float* dst, cudaStream_t s) {
    if (n == 0 || m == 0) return cudaSuccess;
    unsigned g = (unsigned)((n + WARPS_PER_CTA - 1) / WARPS_PER_CTA);
    dim3 b(WARPS_PER_CTA * 32);
    switch (type) {
#define JQ_MM(T, E, B) \
    case T: matmul_f32_kernel<T, E, B><<<g, b, 0, s>>>(w, n, k, lhs, m, dst); break;
        JQ_FOR_EACH_TYPE(JQ_MM)
#undef JQ_MM
        default: return cudaErrorInvalidValue;
    }
    return cudaGetLastError();
}

}  // namespace jq
