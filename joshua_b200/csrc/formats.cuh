// Block layouts of the five GGUF types on the path and their exact decode.
//
// Everything here works on 8-value "units": for every format, 8 consecutive
// weights of a row come from one small run of bytes with one scale (and one
// min), so a unit is the natural grain for a lane.  The decode reproduces the
// reference's arithmetic bit for bit:
//   Q8_0     w = fl(q * d)                                   src/kquant_dot.rs:286-302
//   Q2_K     w = fma(q, fl(d*(sc&15)), -fl(dmin*(sc>>4)))    src/kquant_dot.rs:345-384
//   Q4_K     w = fma(q, fl(d*sc), -fl(dmin*m))               src/kquant_dot.rs:426-465
//   IQ2_XXS  w = fl(fl(db*g)*s), db = fl(fl(d*fl(.5+s4))*.25) src/iq2xxs.rs:44-71
//   MXFP4    w = fl(2^(e-127) * E2M1[code]), e=255 -> 0      src/mxfp4.rs:67-94
// `two_step` selects the separately rounded k-quant form fl(fl(d1*q) - m1)
// that QuantizedType::dequantize / embedding return (src/mmap_tensor.rs:140-174).
#pragma once

#include <cuda_fp16.h>
#include <stdint.h>

#include "iq2xxs_grid_packed.h"

namespace jq {

enum : uint32_t { T_Q8_0 = 8, T_Q2_K = 10, T_Q4_K = 12, T_IQ2_XXS = 16, T_MXFP4 = 39 };

struct Format {
    uint32_t elems;  // weights per block
    uint32_t bytes;  // bytes per block
};

__host__ __device__ inline bool format_of(uint32_t type, Format* f) {
    switch (type) {
        case T_Q8_0: *f = {32, 34}; return true;
        case T_Q2_K: *f = {256, 84}; return true;
        case T_Q4_K: *f = {256, 144}; return true;
        case T_IQ2_XXS: *f = {256, 66}; return true;
        case T_MXFP4: *f = {32, 17}; return true;
        default: return false;
    }
}

#ifdef __CUDACC__

// IQ2_XXS codebook: entry i = 8 bytes (values 8 / 25 / 43).  One copy per
// translation unit (no relocatable device code is used); every unit that
// decodes IQ2_XXS exports a function that calls `upload_tables()` and the
// context runs them all, with its device current, when it is created.
static __device__ uint2 g_iq2xxs_grid[256];

static inline cudaError_t upload_tables() {
    static const uint8_t level[3] = {8, 25, 43};
    uint8_t host[256][8];
    for (int i = 0; i < 256; ++i) {
        unsigned c = JQ_IQ2XXS_GRID_PACKED[i];
        for (int j = 0; j < 8; ++j) {
            host[i][j] = level[c % 3];
            c /= 3;
        }
    }
    return cudaMemcpyToSymbol(g_iq2xxs_grid, host, sizeof(host));
}

__device__ __forceinline__ float f16_bits_to_f32(uint32_t h) {
    return __half2float(__ushort_as_half((unsigned short)h));
}
__device__ __forceinline__ uint32_t ld_u8(const uint8_t* p) { return __ldg(p); }
__device__ __forceinline__ uint32_t ld_u16(const uint8_t* p) {  // p 2-byte aligned
    return __ldg(reinterpret_cast<const unsigned short*>(p));
}
__device__ __forceinline__ uint32_t ld_u32(const uint8_t* p) {  // p 4-byte aligned
    return __ldg(reinterpret_cast<const uint32_t*>(p));
}
__device__ __forceinline__ uint32_t ld_u16_bytes(const uint8_t* p) { return ld_u8(p) | (ld_u8(p + 1) << 8); }

// The 8-bit sign pattern of a 7-bit IQ2_XXS sign index: bit 7 makes the
// population count even (the reference's KSIGNS table, src/iq2xxs.rs:441-449).
__device__ __forceinline__ uint32_t iq2_signs(uint32_t idx7) { return idx7 | ((__popc(idx7) & 1u) << 7); }

__device__ __forceinline__ float e2m1_value(uint32_t code) {
    // sign | 2-bit exponent (bias 1) | 1-bit mantissa; exponent 0 is subnormal
    uint32_t mag = code & 7u;
    uint32_t e = mag >> 1, f = mag & 1u;
    float v = e == 0 ? 0.5f * (float)f : (float)((2u + f) << (e - 1u)) * 0.5f;
    return (code & 8u) ? -v : v;
}

// Decode unit `u` (8 weights: columns 8u .. 8u+7) of a row that starts at
// `row`.  `row` must be aligned to 2 bytes for Q8_0 / IQ2_XXS, 4 for Q2_K /
// Q4_K; MXFP4 has no alignment.
template <uint32_t TYPE>
__device__ __forceinline__ void decode_unit(const uint8_t* row, uint32_t u, float w[8], bool two_step);

template <>
__device__ __forceinline__ void decode_unit<T_Q8_0>(const uint8_t* row, uint32_t u, float w[8], bool) {
    const uint8_t* blk = row + (size_t)(u >> 2) * 34;
    float d = f16_bits_to_f32(ld_u16(blk));
    const uint8_t* q = blk + 2 + 8 * (u & 3);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        uint32_t v = ld_u16(q + 2 * i);
        w[2 * i] = __fmul_rn((float)(int8_t)(v & 0xFF), d);
        w[2 * i + 1] = __fmul_rn((float)(int8_t)(v >> 8), d);
    }
}

template <>
__device__ __forceinline__ void decode_unit<T_Q2_K>(const uint8_t* row, uint32_t u, float w[8], bool two_step) {
    const uint8_t* blk = row + (size_t)(u >> 5) * 84;
    uint32_t v0 = (u & 31) * 8;  // first value inside the block
    uint32_t sg = v0 >> 7, r = v0 & 127;
    uint32_t sc = ld_u8(blk + sg * 8 + (r >> 4));
    uint32_t dd = ld_u32(blk + 80);
    float d1 = __fmul_rn(f16_bits_to_f32(dd & 0xFFFF), (float)(sc & 15));
    float m1 = __fmul_rn(f16_bits_to_f32(dd >> 16), (float)(sc >> 4));
    const uint8_t* q = blk + 16 + sg * 32 + (r & 31);
    uint32_t shift = 2 * (r >> 5);
    uint32_t lo = ld_u32(q), hi = ld_u32(q + 4);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        uint32_t word = i < 4 ? lo : hi;
        float qv = (float)((word >> (8 * (i & 3) + shift)) & 3u);
        w[i] = two_step ? __fsub_rn(__fmul_rn(d1, qv), m1) : __fmaf_rn(qv, d1, -m1);
    }
}

__device__ __forceinline__ void q4k_scale_min(const uint8_t* s, uint32_t j, uint32_t* sc, uint32_t* mn) {
    if (j < 4) {
        *sc = ld_u8(s + j) & 63;
        *mn = ld_u8(s + j + 4) & 63;
    } else {
        uint32_t a = ld_u8(s + j + 4), b = ld_u8(s + j - 4), c = ld_u8(s + j);
        *sc = (a & 0xF) | ((b >> 6) << 4);
        *mn = (a >> 4) | ((c >> 6) << 4);
    }
}

template <>
__device__ __forceinline__ void decode_unit<T_Q4_K>(const uint8_t* row, uint32_t u, float w[8], bool two_step) {
    const uint8_t* blk = row + (size_t)(u >> 5) * 144;
    uint32_t pair = (u & 31) >> 2;  // 32-value group
    uint32_t sc, mn;
    q4k_scale_min(blk + 4, pair, &sc, &mn);
    uint32_t dd = ld_u32(blk);
    float d1 = __fmul_rn(f16_bits_to_f32(dd & 0xFFFF), (float)sc);
    float m1 = __fmul_rn(f16_bits_to_f32(dd >> 16), (float)mn);
    const uint8_t* q = blk + 16 + 32 * (pair >> 1) + 8 * (u & 3);
    uint32_t shift = 4 * (pair & 1);
    uint32_t lo = ld_u32(q), hi = ld_u32(q + 4);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        uint32_t word = i < 4 ? lo : hi;
        float qv = (float)((word >> (8 * (i & 3) + shift)) & 15u);
        w[i] = two_step ? __fsub_rn(__fmul_rn(d1, qv), m1) : __fmaf_rn(qv, d1, -m1);
    }
}

template <>
__device__ __forceinline__ void decode_unit<T_IQ2_XXS>(const uint8_t* row, uint32_t u, float w[8], bool) {
    const uint8_t* blk = row + (size_t)(u >> 5) * 66;
    uint32_t ib32 = (u & 31) >> 2, l = u & 3;
    const uint8_t* p = blk + 2 + ib32 * 8;
    float d = f16_bits_to_f32(ld_u16(blk));
    uint32_t code = ld_u8(p + l);
    uint32_t hi = ld_u16(p + 4) | (ld_u16(p + 6) << 16);
    float db = __fmul_rn(__fmul_rn(d, __fadd_rn(0.5f, (float)(hi >> 28))), 0.25f);
    uint32_t signs = iq2_signs((hi >> (7 * l)) & 127u);
    uint2 g = g_iq2xxs_grid[code];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        uint32_t word = i < 4 ? g.x : g.y;
        float gv = (float)((word >> (8 * (i & 3))) & 0xFFu);
        float s = (signs >> i) & 1u ? -1.0f : 1.0f;
        w[i] = __fmul_rn(__fmul_rn(db, gv), s);
    }
}

template <>
__device__ __forceinline__ void decode_unit<T_MXFP4>(const uint8_t* row, uint32_t u, float w[8], bool) {
    const uint8_t* blk = row + (size_t)(u >> 2) * 17;
    uint32_t e = ld_u8(blk);
    uint32_t part = u & 3;  // values 8*part .. 8*part+7 of the block
    const uint8_t* q = blk + 1 + 8 * (part & 1);
    uint32_t shift = 4 * (part >> 1);  // split-half: high nibbles hold values 16..31
    float scale = __uint_as_float(e == 0 ? 0x00400000u : e << 23);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        uint32_t code = (ld_u8(q + i) >> shift) & 15u;
        w[i] = e == 0xFFu ? 0.0f : __fmul_rn(scale, e2m1_value(code));
    }
}

#endif  // __CUDACC__

}  // namespace jq
