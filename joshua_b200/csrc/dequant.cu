// Standalone block decode: raw GGUF blocks -> f32, one 8-value unit per thread.
//
// Serves QuantizedType::dequantize and QuantizedType::embedding of the
// reference's borrowed tensors (src/mmap_tensor.rs:140-174,379-440,452-513)
// and the raw decode of the streamed loader (src/quant_matmul.rs:36-103), and
// is what the bit-exactness check of the block decode runs against.
// HBM-bound: reads the block bytes once, writes 4 bytes per weight.
#include "common.cuh"

namespace jq {

cudaError_t tables_dequant() { return upload_tables(); }

namespace {

template <uint32_t TYPE, uint32_t ELEMS, uint32_t BYTES>
__global__ void __launch_bounds__(256) dequant_kernel(const uint8_t* __restrict__ w, uint64_t n_units,
                                                      float* __restrict__ out, bool two_step) {
    constexpr uint32_t UPB = ELEMS / 8;  // units per block
    for (uint64_t u = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; u < n_units;
         u += (uint64_t)gridDim.x * blockDim.x) {
        float v[8];
        decode_unit<TYPE>(w + (u / UPB) * BYTES, (uint32_t)(u % UPB), v, two_step);
        float4* o = reinterpret_cast<float4*>(out + u * 8);
        o[0] = make_float4(v[0], v[1], v[2], v[3]);
        o[1] = make_float4(v[4], v[5], v[6], v[7]);
    }
}

// out[i, :] = decode(row ids[i]); ids out of range raise the flag and leave the row untouched
// (the reference bails with "embedding id .. is out of range", src/mmap_tensor.rs:158-160).
template <uint32_t TYPE, uint32_t ELEMS, uint32_t BYTES>
__global__ void __launch_bounds__(256) embedding_kernel(const uint8_t* __restrict__ w, uint64_t rows, uint64_t hidden,
                                                        const uint32_t* __restrict__ ids, uint64_t n_ids,
                                                        float* __restrict__ out, int* bad_id) {
    constexpr uint32_t UPB = ELEMS / 8;
    const uint64_t units_per_row = hidden / 8;
    const uint64_t row_bytes = hidden / ELEMS * BYTES;
    const uint64_t total = n_ids * units_per_row;
    for (uint64_t t = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; t < total;
         t += (uint64_t)gridDim.x * blockDim.x) {
        uint64_t i = t / units_per_row, u = t % units_per_row;
        uint32_t id = ids[i];
        if (id >= rows) {
            if (u == 0) atomicExch(bad_id, 1);
            continue;
        }
        float v[8];
        decode_unit<TYPE>(w + id * row_bytes + (u / UPB) * BYTES, (uint32_t)(u % UPB), v, true);
        float4* o = reinterpret_cast<float4*>(out + i * hidden + u * 8);
        o[0] = make_float4(v[0], v[1], v[2], v[3]);
        o[1] = make_float4(v[4], v[5], v[6], v[7]);
    }
}

inline unsigned grid_for(uint64_t work) {
    uint64_t blocks = (work + 255) / 256;
    return (unsigned)(blocks < 148ull * 64 ? (blocks ? blocks : 1) : 148ull * 64);
}

}  // namespace

cudaError_t launch_dequant(uint32_t type, const uint8_t* w, uint64_t n_blocks, float* out, bool two_step,
                           cudaStream_t s) {
    Format f;
    if (!format_of(type, &f)) return cudaErrorInvalidValue;
    if (n_blocks == 0) return cudaSuccess;
    uint64_t n_units = n_blocks * (f.elems / 8);
    unsigned g = grid_for(n_units);
    switch (type) {
#define JQ_DEQ(T, E, B) \
    case T: dequant_kernel<T, E, B><<<g, 256, 0, s>>>(w, n_units, out, two_step); break;
        JQ_FOR_EACH_TYPE(JQ_DEQ)
#undef JQ_DEQ
    }
    return cudaGetLastError();
}

cudaError_t launch_embedding(uint32_t type, const uint8_t* w, uint64_t rows, uint64_t hidden, const uint32_t* ids,
                             uint64_t n_ids, float* out, int* bad_id, cudaStream_t s) {
    Format f;
    if (!format_of(type, &f)) return cudaErrorInvalidValue;
    if (n_ids == 0) return cudaSuccess;
    unsigned g = grid_for(n_ids * (hidden / 8));
#define JQ_EMB(T, E, B) \
    case T: embedding_kernel<T, E, B><<<g, 256, 0, s>>>(w, rows, hidden, ids, n_ids, out, bad_id); break;
    switch (type) { JQ_FOR_EACH_TYPE(JQ_EMB) }
#undef JQ_EMB
    return cudaGetLastError();
}

}  // namespace jq
