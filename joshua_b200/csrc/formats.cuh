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

enum : uint32_t {
    T_Q4_0 = 2, T_Q4_1 = 3, T_Q5_0 = 6, T_Q5_1 = 7, T_Q8_0 = 8, T_Q8_1 = 9, T_Q2_K = 10, T_Q3_K = 11, T_Q4_K = 12,
    T_Q5_K = 13, T_Q6_K = 14, T_Q8_K = 15, T_IQ2_XXS = 16, T_MXFP4 = 39
};

// Every block type with a decoder here: X(type id, elements per block, bytes per block).  The first five are
// the types of the fused decode kernels; the rest take the exact-decode float path only, as in the reference
// (its generic path dequantises a row and dots it, src/quant_matmul.rs:228-249; block sizes src/gguf_ext.rs:483-512).
#define JQ_FOR_EACH_TYPE(X)                                                                                      \
    X(T_Q8_0, 32, 34) X(T_Q2_K, 256, 84) X(T_Q4_K, 256, 144) X(T_IQ2_XXS, 256, 66) X(T_MXFP4, 32, 17)            \
    X(T_Q4_0, 32, 18) X(T_Q4_1, 32, 20) X(T_Q5_0, 32, 22) X(T_Q5_1, 32, 24) X(T_Q8_1, 32, 36) X(T_Q3_K, 256, 110) \
    X(T_Q5_K, 256, 176) X(T_Q6_K, 256, 210) X(T_Q8_K, 256, 292)

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
        case T_Q4_0: *f = {32, 18}; return true;
        case T_Q4_1: *f = {32, 20}; return true;
        case T_Q5_0: *f = {32, 22}; return true;
        case T_Q5_1: *f = {32, 24}; return true;
        case T_Q8_1: *f = {32, 36}; return true;
        case T_Q3_K: *f = {256, 110}; return true;
        case T_Q5_K: *f = {256, 176}; return true;
        case T_Q6_K: *f = {256, 210}; return true;
        case T_Q8_K: *f = {256, 292}; return true;
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

// Where a decoder's block bytes live: global memory (read-only path) or this CTA's shared memory.
struct LdGlobal {
    static __device__ __forceinline__ uint32_t u8(const uint8_t* p) { return ld_u8(p); }
    static __device__ __forceinline__ uint32_t u16(const uint8_t* p) { return ld_u16(p); }
    static __device__ __forceinline__ uint32_t u32(const uint8_t* p) { return ld_u32(p); }
};
struct LdShared {
    static __device__ __forceinline__ uint32_t addr(const uint8_t* p) { return (uint32_t)__cvta_generic_to_shared(p); }
    static __device__ __forceinline__ uint32_t u8(const uint8_t* p) {
        uint32_t v;
        asm volatile("ld.shared.u8 %0, [%1];" : "=r"(v) : "r"(addr(p)));
        return v;
    }
    static __device__ __forceinline__ uint32_t u16(const uint8_t* p) {  // p 2-byte aligned
        uint32_t v;
        asm volatile("ld.shared.u16 %0, [%1];" : "=r"(v) : "r"(addr(p)));
        return v;
    }
    static __device__ __forceinline__ uint32_t u32(const uint8_t* p) {  // p 4-byte aligned
        uint32_t v;
        asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr(p)));
        return v;
    }
};

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
__device__ __forceinline__ void decode_unit_generic(const uint8_t* row, uint32_t u, float w[8], bool two_step);

template <class LD>
__device__ __forceinline__ void decode_q8_0(const uint8_t* row, uint32_t u, float w[8], bool) {
    const uint8_t* blk = row + (size_t)(u >> 2) * 34;
    float d = f16_bits_to_f32(LD::u16(blk));
    const uint8_t* q = blk + 2 + 8 * (u & 3);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        uint32_t v = LD::u16(q + 2 * i);
        w[2 * i] = __fmul_rn((float)(int8_t)(v & 0xFF), d);
        w[2 * i + 1] = __fmul_rn((float)(int8_t)(v >> 8), d);
    }
}

template <class LD>
__device__ __forceinline__ void decode_q2_k(const uint8_t* row, uint32_t u, float w[8], bool two_step) {
    const uint8_t* blk = row + (size_t)(u >> 5) * 84;
    uint32_t v0 = (u & 31) * 8;  // first value inside the block
    uint32_t sg = v0 >> 7, r = v0 & 127;
    uint32_t sc = LD::u8(blk + sg * 8 + (r >> 4));
    uint32_t dd = LD::u32(blk + 80);
    float d1 = __fmul_rn(f16_bits_to_f32(dd & 0xFFFF), (float)(sc & 15));
    float m1 = __fmul_rn(f16_bits_to_f32(dd >> 16), (float)(sc >> 4));
    const uint8_t* q = blk + 16 + sg * 32 + (r & 31);
    uint32_t shift = 2 * (r >> 5);
    uint32_t lo = LD::u32(q), hi = LD::u32(q + 4);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        uint32_t word = i < 4 ? lo : hi;
        float qv = (float)((word >> (8 * (i & 3) + shift)) & 3u);
        w[i] = two_step ? __fsub_rn(__fmul_rn(d1, qv), m1) : __fmaf_rn(qv, d1, -m1);
    }
}

template <class LD>
__device__ __forceinline__ void q4k_scale_min(const uint8_t* s, uint32_t j, uint32_t* sc, uint32_t* mn) {
    if (j < 4) {
        *sc = LD::u8(s + j) & 63;
        *mn = LD::u8(s + j + 4) & 63;
    } else {
        uint32_t a = LD::u8(s + j + 4), b = LD::u8(s + j - 4), c = LD::u8(s + j);
        *sc = (a & 0xF) | ((b >> 6) << 4);
        *mn = (a >> 4) | ((c >> 6) << 4);
    }
}

template <class LD>
__device__ __forceinline__ void decode_q4_k(const uint8_t* row, uint32_t u, float w[8], bool two_step) {
    const uint8_t* blk = row + (size_t)(u >> 5) * 144;
    uint32_t pair = (u & 31) >> 2;  // 32-value group
    uint32_t sc, mn;
    q4k_scale_min<LD>(blk + 4, pair, &sc, &mn);
    uint32_t dd = LD::u32(blk);
    float d1 = __fmul_rn(f16_bits_to_f32(dd & 0xFFFF), (float)sc);
    float m1 = __fmul_rn(f16_bits_to_f32(dd >> 16), (float)mn);
    const uint8_t* q = blk + 16 + 32 * (pair >> 1) + 8 * (u & 3);
    uint32_t shift = 4 * (pair & 1);
    uint32_t lo = LD::u32(q), hi = LD::u32(q + 4);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        uint32_t word = i < 4 ? lo : hi;
        float qv = (float)((word >> (8 * (i & 3) + shift)) & 15u);
        w[i] = two_step ? __fsub_rn(__fmul_rn(d1, qv), m1) : __fmaf_rn(qv, d1, -m1);
    }
}

template <class LD>
__device__ __forceinline__ void decode_iq2_xxs(const uint8_t* row, uint32_t u, float w[8], bool) {
    const uint8_t* blk = row + (size_t)(u >> 5) * 66;
    uint32_t ib32 = (u & 31) >> 2, l = u & 3;
    const uint8_t* p = blk + 2 + ib32 * 8;
    float d = f16_bits_to_f32(LD::u16(blk));
    uint32_t code = LD::u8(p + l);
    uint32_t hi = LD::u16(p + 4) | (LD::u16(p + 6) << 16);
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

template <class LD>
__device__ __forceinline__ void decode_mxfp4(const uint8_t* row, uint32_t u, float w[8], bool) {
    const uint8_t* blk = row + (size_t)(u >> 2) * 17;
    uint32_t e = LD::u8(blk);
    uint32_t part = u & 3;  // values 8*part .. 8*part+7 of the block
    const uint8_t* q = blk + 1 + 8 * (part & 1);
    uint32_t shift = 4 * (part >> 1);  // split-half: high nibbles hold values 16..31
    float scale = __uint_as_float(e == 0 ? 0x00400000u : e << 23);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        uint32_t code = (LD::u8(q + i) >> shift) & 15u;
        w[i] = e == 0xFFu ? 0.0f : __fmul_rn(scale, e2m1_value(code));
    }
}

// ── the other GGUF block types (exact path only) ──
// The reference decodes these with candle's `k_quants::*::to_float`, a port of ggml's `dequantize_row_*`; the
// layouts and the order of the float operations below are the published ggml ones.  All loads are single bytes:
// these blocks have no alignment beyond two.  `two_step` does not apply (one form each).
__device__ __forceinline__ float ld_f16(const uint8_t* p) { return f16_bits_to_f32(ld_u8(p) | (ld_u8(p + 1) << 8)); }

// 32-value blocks with split halves: value j < 16 is the low nibble of byte j, value j + 16 the high nibble.
template <>
__device__ __forceinline__ void decode_unit_generic<T_Q4_0>(const uint8_t* row, uint32_t u, float w[8], bool) {
    const uint8_t* blk = row + (size_t)(u >> 2) * 18;
    const float d = ld_f16(blk);
    const uint32_t part = u & 3, shift = 4 * (part >> 1);
    const uint8_t* q = blk + 2 + 8 * (part & 1);
#pragma unroll
    for (int i = 0; i < 8; ++i) w[i] = __fmul_rn((float)((int)((ld_u8(q + i) >> shift) & 15u) - 8), d);
}

template <>
__device__ __forceinline__ void decode_unit_generic<T_Q4_1>(const uint8_t* row, uint32_t u, float w[8], bool) {
    const uint8_t* blk = row + (size_t)(u >> 2) * 20;
    const float d = ld_f16(blk), m = ld_f16(blk + 2);
    const uint32_t part = u & 3, shift = 4 * (part >> 1);
    const uint8_t* q = blk + 4 + 8 * (part & 1);
#pragma unroll
    for (int i = 0; i < 8; ++i) w[i] = __fadd_rn(__fmul_rn((float)((ld_u8(q + i) >> shift) & 15u), d), m);
}

// fifth bit of value v of a Q5_0 / Q5_1 block from the 32-bit mask qh: bit v
__device__ __forceinline__ uint32_t q5_code(const uint8_t* qs, uint32_t qh, uint32_t v) {
    const uint32_t nib = v < 16 ? (ld_u8(qs + v) & 15u) : (ld_u8(qs + v - 16) >> 4);
    return nib | (((qh >> v) & 1u) << 4);
}

template <>
__device__ __forceinline__ void decode_unit_generic<T_Q5_0>(const uint8_t* row, uint32_t u, float w[8], bool) {
    const uint8_t* blk = row + (size_t)(u >> 2) * 22;
    const float d = ld_f16(blk);
    const uint32_t qh = ld_u8(blk + 2) | (ld_u8(blk + 3) << 8) | (ld_u8(blk + 4) << 16) | (ld_u8(blk + 5) << 24);
#pragma unroll
    for (int i = 0; i < 8; ++i) w[i] = __fmul_rn((float)((int)q5_code(blk + 6, qh, 8 * (u & 3) + i) - 16), d);
}

template <>
__device__ __forceinline__ void decode_unit_generic<T_Q5_1>(const uint8_t* row, uint32_t u, float w[8], bool) {
    const uint8_t* blk = row + (size_t)(u >> 2) * 24;
    const float d = ld_f16(blk), m = ld_f16(blk + 2);
    const uint32_t qh = ld_u8(blk + 4) | (ld_u8(blk + 5) << 8) | (ld_u8(blk + 6) << 16) | (ld_u8(blk + 7) << 24);
#pragma unroll
    for (int i = 0; i < 8; ++i) w[i] = __fadd_rn(__fmul_rn((float)q5_code(blk + 8, qh, 8 * (u & 3) + i), d), m);
}

template <>
__device__ __forceinline__ void decode_unit_generic<T_Q8_1>(const uint8_t* row, uint32_t u, float w[8], bool) {
    const uint8_t* blk = row + (size_t)(u >> 2) * 36;  // f16 d, f16 s (unused by the decode), 32 int8
    const float d = ld_f16(blk);
#pragma unroll
    for (int i = 0; i < 8; ++i) w[i] = __fmul_rn((float)(int8_t)ld_u8(blk + 4 + 8 * (u & 3) + i), d);
}

template <>
__device__ __forceinline__ void decode_unit_generic<T_Q8_K>(const uint8_t* row, uint32_t u, float w[8], bool) {
    const uint8_t* blk = row + (size_t)(u >> 5) * 292;  // f32 d, 256 int8, 16 int16 block sums (unused)
    const float d = __uint_as_float(ld_u8(blk) | (ld_u8(blk + 1) << 8) | (ld_u8(blk + 2) << 16) | (ld_u8(blk + 3) << 24));
#pragma unroll
    for (int i = 0; i < 8; ++i) w[i] = __fmul_rn(d, (float)(int8_t)ld_u8(blk + 4 + 8 * (u & 31) + i));
}

// Q3_K: hmask[32] | qs[64] | scales[12] | f16 d.  Value v: half = v / 128, j = (v % 128) / 32, l = v % 32; low two
// bits (qs[32 half + l] >> 2j) & 3, minus 4 unless bit (4 half + j) of hmask[l] is set; scale index v / 16.
__device__ __forceinline__ int q3k_scale(const uint8_t* s, uint32_t i) {  // six-bit scale i of 16, minus 32
    // low four bits: nibble (i / 8) of byte i % 8; high two bits: bit pair (i / 4) of byte 8 + i % 4
    const uint32_t lo = (ld_u8(s + (i & 7)) >> (4 * (i >> 3))) & 15u;
    const uint32_t hi = (ld_u8(s + 8 + (i & 3)) >> (2 * (i >> 2))) & 3u;
    return (int)(lo | (hi << 4)) - 32;
}

template <>
__device__ __forceinline__ void decode_unit_generic<T_Q3_K>(const uint8_t* row, uint32_t u, float w[8], bool) {
    const uint8_t* blk = row + (size_t)(u >> 5) * 110;
    const uint32_t v0 = (u & 31) * 8, half = v0 >> 7, j = (v0 & 127) >> 5, l0 = v0 & 31;
    const float dl = __fmul_rn(ld_f16(blk + 108), (float)q3k_scale(blk + 96, v0 >> 4));
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int two = (int)((ld_u8(blk + 32 + 32 * half + l0 + i) >> (2 * j)) & 3u);
        const int q = two - (((ld_u8(blk + l0 + i) >> (4 * half + j)) & 1u) ? 0 : 4);
        w[i] = __fmul_rn(dl, (float)q);
    }
}

// Q5_K: f16 d | f16 dmin | scales[12] | qh[32] | qs[128].  As Q4_K with a fifth bit: group g (32 values) takes
// bit g of qh[l].
template <>
__device__ __forceinline__ void decode_unit_generic<T_Q5_K>(const uint8_t* row, uint32_t u, float w[8], bool) {
    const uint8_t* blk = row + (size_t)(u >> 5) * 176;
    const uint32_t pair = (u & 31) >> 2, l0 = 8 * (u & 3);
    uint32_t sc, mn;
    q4k_scale_min<LdGlobal>(blk + 4, pair, &sc, &mn);
    const float d1 = __fmul_rn(ld_f16(blk), (float)sc), m1 = __fmul_rn(ld_f16(blk + 2), (float)mn);
    const uint8_t* q = blk + 48 + 32 * (pair >> 1) + l0;
    const uint32_t shift = 4 * (pair & 1);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const uint32_t code = ((ld_u8(q + i) >> shift) & 15u) + (((ld_u8(blk + 16 + l0 + i) >> pair) & 1u) << 4);
        w[i] = __fsub_rn(__fmul_rn(d1, (float)code), m1);
    }
}

// Q6_K: ql[128] | qh[64] | int8 scales[16] | f16 d.  Value v: half = v / 128, part = (v % 128) / 32, l = v % 32;
// low nibble from ql[64 half + 32 (part & 1) + l] (low for part < 2, high otherwise), two high bits
// (qh[32 half + l] >> 2 part) & 3, minus 32; scale index v / 16.
template <>
__device__ __forceinline__ void decode_unit_generic<T_Q6_K>(const uint8_t* row, uint32_t u, float w[8], bool) {
    const uint8_t* blk = row + (size_t)(u >> 5) * 210;
    const uint32_t v0 = (u & 31) * 8, half = v0 >> 7, part = (v0 & 127) >> 5, l0 = v0 & 31;
    const float ds = __fmul_rn(ld_f16(blk + 208), (float)(int8_t)ld_u8(blk + 192 + (v0 >> 4)));
    const uint8_t* ql = blk + 64 * half + 32 * (part & 1) + l0;
    const uint8_t* qh = blk + 128 + 32 * half + l0;
    const uint32_t nshift = 4 * (part >> 1);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const uint32_t code = ((ld_u8(ql + i) >> nshift) & 15u) | (((ld_u8(qh + i) >> (2 * part)) & 3u) << 4);
        w[i] = __fmul_rn(ds, (float)((int)code - 32));
    }
}

// One decoder per block type; LD says where the block bytes are read from.
template <uint32_t TYPE, class LD = LdGlobal>
__device__ __forceinline__ void decode_unit(const uint8_t* row, uint32_t u, float w[8], bool two_step) {
    if constexpr (TYPE == T_Q8_0) decode_q8_0<LD>(row, u, w, two_step);
    else if constexpr (TYPE == T_Q2_K) decode_q2_k<LD>(row, u, w, two_step);
    else if constexpr (TYPE == T_Q4_K) decode_q4_k<LD>(row, u, w, two_step);
    else if constexpr (TYPE == T_IQ2_XXS) decode_iq2_xxs<LD>(row, u, w, two_step);
    else if constexpr (TYPE == T_MXFP4) decode_mxfp4<LD>(row, u, w, two_step);
    else decode_unit_generic<TYPE>(row, u, w, two_step);
}

#endif  // __CUDACC__

}  // namespace jq
