// Decode-time matmul (batch 1..32) over raw GGUF blocks, HBM-bound.
//
// dst[m, n] = lhs[m, k] . W[n, k]^T with W left in its GGUF bytes.  The
// reference forms f32 weights in registers and FMAs them against f32
// activations (src/kquant_dot.rs:268-483, src/iq2xxs.rs:331-391,
// src/mxfp4.rs:208-235).  At HBM speed a B200 SM sees 40 to 90 weights per
// clock, which leaves one to three issue slots per weight, so the same
// arithmetic is regrouped around the integer codes that all five formats
// store:
//
//     sum_c x_c * (s_g * q_c - o_g)  =  s_g * sum_c x_c q_c  -  o_g * sum_c x_c     (per scale group g)
//
//   * q_c are the exact small integers of the format (Q8_0: int8; Q4_K: 0..15;
//     Q2_K: 0..3; IQ2_XXS: +-8/25/43; MXFP4: twice the E2M1 value, 0..+-12).
//   * each activation row is split, per 32-value group, into three int8 planes
//     x ~= (s/254^2) * (254^2*hi + 254*mid + lo), |error| <= max|x| * 6.1e-8, i.e.
//     to f32 precision (quantize_acts), so sum_c x_c q_c is three exact int32 dot
//     products computed by mma.sync.m16n8k32.s8 (m16n8k16 for the 16-value
//     groups of Q2_K);
//   * the f32 group scales s_g = d*sc, o_g = dmin*m and the f32 group sums of x
//     are applied once per group in the epilogue.
//
// One CTA owns 16 weight rows.  The rows' bytes for a K-chunk are pulled into
// shared memory by one cp.async.bulk per row (rows of a tile are adjacent in
// memory, so the tile is one contiguous HBM stream) behind an mbarrier, two
// stages deep; warps split the chunk's blocks, and partial sums meet in shared
// memory in a fixed order, so results do not depend on timing.
//
// MMA tile use: A = 16 weight rows x 32 codes.  B = 32 codes x 8 columns.  Two
// MMAs share each A fragment: the first takes the (hi, mid) planes of a batch
// row in a column pair, the second its lo plane in the even column of the same
// pair.  With MB batch rows per MMA (1, 2 or 4) only MB column pairs are live,
// so 4/MB consecutive groups are chained into one accumulator by giving each
// its own pair: after the chain, thread t of a quad holds the three dots of
// group (t / MB) and batch row (t % MB), and scales exactly that one.  Batches
// above 4 run NH passes over the same A fragments.
//
// Algorithmic bytes per launch: n*k/B*S (weights) + 4*m*(k + n).
#include <algorithm>

#include "common.cuh"

namespace jq {

cudaError_t tables_gemv_mma() { return upload_tables(); }

namespace {

constexpr int ROWS = 16;  // weight rows per CTA (one MMA M tile)

// ───────────────────────────── PTX helpers ────────────────────────────────

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
// Bounded wait: returns false when the phase has not completed after ~2^26 polls.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
    uint32_t addr = smem_u32(bar);
    for (uint32_t it = 0; it < (1u << 26); ++it) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done)
            : "r"(addr), "r"(parity)
            : "memory");
        if (done) return true;
    }
    return false;
}
// 1-D bulk copy global -> shared, completion counted on an mbarrier.  All of
// dst, src and bytes are multiples of 16.
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(dst)),
                 "l"(src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

__device__ __forceinline__ void mma_k32(int c[4], const uint32_t a[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_k16(int c[4], uint32_t a0, uint32_t a1, uint32_t b0) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%0,%1,%2,%3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                 : "r"(a0), "r"(a1), "r"(b0));
}

// prmt.b32, default mode: result byte i = byte (sel nibble i & 7) of {a, b}; if bit 3 of the nibble is
// set, the byte's most significant bit is replicated over the result byte instead.
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
    return r;
}

__device__ __forceinline__ uint32_t lds32(const uint8_t* p) { return *reinterpret_cast<const uint32_t*>(p); }
__device__ __forceinline__ uint2 lds64(const uint8_t* p) { return *reinterpret_cast<const uint2*>(p); }
__device__ __forceinline__ uint4 lds128(const uint8_t* p) { return *reinterpret_cast<const uint4*>(p); }
__device__ __forceinline__ uint32_t lds16(const uint8_t* p) { return *reinterpret_cast<const unsigned short*>(p); }
// 8 bytes starting at p (p 2-byte aligned with the given word misalignment in bytes: 0 or 2).
template <int MIS>
__device__ __forceinline__ uint2 lds64_mis(const uint8_t* p) {
    const uint8_t* q = p - MIS;
    if (MIS == 0) return make_uint2(lds32(q), lds32(q + 4));
    uint32_t w0 = lds32(q), w1 = lds32(q + 4), w2 = lds32(q + 8);
    return make_uint2(__funnelshift_r(w0, w1, 8 * MIS), __funnelshift_r(w1, w2, 8 * MIS));
}

// ─────────────────── activation planes (scratch in global memory) ─────────
//
// For batch row i and 32-value group G:
//   planes[(i*NG + G)*96 + 0..31]   hi plane, int8, in the format's lane order
//   planes[(i*NG + G)*96 + 32..63]  mid plane
//   planes[(i*NG + G)*96 + 64..95]  lo plane
//   meta[i*NG + G]                  float2 {s/254^2, sum of x over the group}
//   sum16[(i*NG + G)*2 + h]         sum of x over each 16-value half (Q2_K minima)
// Lane order: position 8t+j holds the element that lane t of a quad feeds to
// the MMA at byte j.  Identity for every format except MXFP4, whose packed
// nibbles give a lane the elements 4t..4t+3 and 16+4t..16+4t+3 interleaved.
struct ActPlanes {
    const int8_t* planes;
    const float2* meta;
    const float* sum16;
    uint32_t n_groups;  // k / 32
};

__device__ __forceinline__ uint32_t act_position(uint32_t type, uint32_t e) {
    if (type != T_MXFP4) return e;
    // element e -> (lane t, byte j): low-half elements 4t+r sit at even bytes 2r, high-half 16+4t+r at 2r+1
    uint32_t half = e >> 4, r = e & 15;
    return 8 * (r >> 2) + 2 * (r & 3) + half;
}

__global__ void __launch_bounds__(256) quantize_acts_kernel(const float* __restrict__ x, uint64_t m, uint64_t k,
                                                            uint32_t type, int8_t* __restrict__ planes,
                                                            float2* __restrict__ meta, float* __restrict__ sum16) {
    const uint32_t lane = threadIdx.x & 31;
    const uint64_t n_groups = k / 32;
    const uint64_t total = m * n_groups;
    for (uint64_t w = blockIdx.x * 8ull + (threadIdx.x >> 5); w < total; w += gridDim.x * 8ull) {
        float v = x[w * 32 + lane];
        float amax = fabsf(v);
        float sum = v;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
            if (o < 16) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, o);
        }
        // `sum` now holds the sum of this lane's 16-value half
        float other = __shfl_xor_sync(0xFFFFFFFFu, sum, 16);
        float s = amax * (1.0f / 127.0f);
        int hi = 0, mid = 0, lo = 0;
        const bool live = s > 0.0f && isfinite(s);
        if (live) {
            hi = max(-127, min(127, __float2int_rn(v / s)));
            float r1 = fmaf(-(float)hi, s, v);  // exact: |r1| <= s/2
            float s1 = s * (1.0f / 254.0f);
            mid = max(-127, min(127, __float2int_rn(r1 / s1)));
            float r2 = fmaf(-(float)mid, s1, r1);
            float s2 = s1 * (1.0f / 254.0f);
            lo = max(-127, min(127, __float2int_rn(r2 / s2)));
        }
        uint32_t pos = act_position(type, lane);
        planes[w * 96 + pos] = (int8_t)hi;
        planes[w * 96 + 32 + pos] = (int8_t)mid;
        planes[w * 96 + 64 + pos] = (int8_t)lo;
        if (lane == 0) {
            meta[w] = make_float2(live ? s * (1.0f / 254.0f) * (1.0f / 254.0f) : 0.0f, sum + other);
            sum16[w * 2] = sum;
            sum16[w * 2 + 1] = other;
        }
    }
}

// ───────────────────────── per-format block traits ────────────────────────
//
// A "unit" is what one warp processes at a time for its 16 rows: 8 groups of
// 32 values (256 columns) for every format.  UNIT_BYTES are contiguous in a
// row: one super-block for the K formats and IQ2_XXS, 8 blocks for Q8_0 and
// MXFP4.

template <uint32_t TYPE>
struct Traits;
template <>
struct Traits<T_Q4_K> {
    static constexpr uint32_t UNIT_BYTES = 144, CHUNK_UNITS = 16, ALIGN = 16;
};
template <>
struct Traits<T_Q8_0> {
    static constexpr uint32_t UNIT_BYTES = 272, CHUNK_UNITS = 8, ALIGN = 16;
};
template <>
struct Traits<T_Q2_K> {
    static constexpr uint32_t UNIT_BYTES = 84, CHUNK_UNITS = 24, ALIGN = 4;
};
template <>
struct Traits<T_IQ2_XXS> {
    static constexpr uint32_t UNIT_BYTES = 66, CHUNK_UNITS = 32, ALIGN = 2;
};
template <>
struct Traits<T_MXFP4> {
    static constexpr uint32_t UNIT_BYTES = 136, CHUNK_UNITS = 16, ALIGN = 8;
};

// Per-lane roles, fixed for the kernel's lifetime.
template <int MB, int NH>
struct Roles {
    static constexpr int CH = 4 / MB;  // groups chained into one accumulator
    int g, t;                          // MMA row group and quad lane
    int sup_p, sup_odd;                // as B supplier: chain position of column g, and whether g is odd
    int fin_p;                         // as finaliser: chain position of columns 2t, 2t+1
    uint32_t sup_row[NH], fin_row[NH]; // batch rows served in pass h, clamped to m-1 (clamped results are dropped)
    __device__ __forceinline__ Roles(int lane, uint64_t m) {
        g = lane >> 2;
        t = lane & 3;
        int pair = g >> 1;
        sup_odd = g & 1;
        sup_p = pair / MB;
        fin_p = t / MB;
#pragma unroll
        for (int h = 0; h < NH; ++h) {
            sup_row[h] = (uint32_t)min((uint64_t)(pair % MB + 4 * h), m - 1);
            fin_row[h] = (uint32_t)min((uint64_t)(t % MB + 4 * h), m - 1);
        }
    }
};

// Scale and offset of Q4_K pair j taken from the 16 header bytes
// (src/kquant_dot.rs:106-118); `hi_half` (j >= 4) is known at compile time.
__device__ __forceinline__ void q4k_pair(const uint4& h, bool hi_half, uint32_t jj, float* d1, float* m1) {
    float d = f16_bits_to_f32(h.x & 0xFFFF), dmin = f16_bits_to_f32(h.x >> 16);
    uint32_t sh = 8 * jj;  // jj = j & 3
    uint32_t sc, mn;
    if (!hi_half) {
        sc = (h.y >> sh) & 63;
        mn = (h.z >> sh) & 63;
    } else {
        uint32_t a = (h.w >> sh) & 0xFF;
        sc = (a & 0xF) | ((((h.y >> sh) & 0xFF) >> 6) << 4);
        mn = (a >> 4) | ((((h.z >> sh) & 0xFF) >> 6) << 4);
    }
    *d1 = __fmul_rn(d, (float)sc);
    *m1 = __fmul_rn(dmin, (float)mn);
}

// One unit (256 columns x 16 rows) of the warp's work.  u0 / u1 point at the
// unit's bytes for rows g and g+8 in shared memory; G0 is the unit's first
// 32-group index along k.  acc[h][0/1] accumulate rows g / g+8 for the lane's
// finaliser batch row fin_i + 4h.
template <uint32_t TYPE, int MB, int NH>
__device__ __forceinline__ void process_unit(const uint8_t* u0, const uint8_t* u1, uint32_t G0, const ActPlanes& act,
                                             const Roles<MB, NH>& ro, const uint2* s_grid, const uint2* s_mask,
                                             float acc[NH][2]) {
    constexpr int CH = Roles<MB, NH>::CH;
    int c[NH][4];   // (hi, mid) dots: c[0], c[1] row g; c[2], c[3] row g+8
    int cl[NH][4];  // lo dots: cl[0] row g, cl[2] row g+8 (odd columns are fed zeros)
    uint2 bsup[NH], bsupl[NH];

    // B fragment of the chain that starts at group Gc: the lane supplies column g for chain position sup_p.
    auto load_b = [&](uint32_t Gc) {
#pragma unroll
        for (int h = 0; h < NH; ++h) {
            uint64_t idx = ((uint64_t)ro.sup_row[h] * act.n_groups + (G0 + Gc + ro.sup_p)) * 96 + 8 * ro.t;
            bsup[h] = __ldg(reinterpret_cast<const uint2*>(act.planes + idx + 32 * ro.sup_odd));
            bsupl[h] = ro.sup_odd ? make_uint2(0u, 0u) : __ldg(reinterpret_cast<const uint2*>(act.planes + idx + 64));
        }
    };
    // Scale the finished chain that started at group Gc: s0 / s1 multiply the integer dots of rows g / g+8,
    // o0 / o1 multiply the group's sum of x.
    auto finish = [&](uint32_t Gc, float s0, float s1, float o0, float o1) {
#pragma unroll
        for (int h = 0; h < NH; ++h) {
            float2 mt = __ldg(act.meta + (uint64_t)ro.fin_row[h] * act.n_groups + (G0 + Gc + ro.fin_p));
            float i0 = fmaf((float)c[h][0], 64516.0f, (float)(c[h][1] * 254 + cl[h][0])) * mt.x;
            float i1 = fmaf((float)c[h][2], 64516.0f, (float)(c[h][3] * 254 + cl[h][2])) * mt.x;
            acc[h][0] = fmaf(s0, i0, fmaf(-o0, mt.y, acc[h][0]));
            acc[h][1] = fmaf(s1, i1, fmaf(-o1, mt.y, acc[h][1]));
        }
    };
    auto step = [&](int G, const uint32_t a[4]) {
        const int p = G % CH;
        if (p == 0) {
            load_b(G);
#pragma unroll
            for (int h = 0; h < NH; ++h)
                c[h][0] = c[h][1] = c[h][2] = c[h][3] = cl[h][0] = cl[h][1] = cl[h][2] = cl[h][3] = 0;
        }
#pragma unroll
        for (int h = 0; h < NH; ++h) {
            bool mine = ro.sup_p == p;
            mma_k32(c[h], a, mine ? bsup[h].x : 0u, mine ? bsup[h].y : 0u);
            mma_k32(cl[h], a, mine ? bsupl[h].x : 0u, mine ? bsupl[h].y : 0u);
        }
    };

    if constexpr (TYPE == T_Q4_K) {
        const uint4 h0 = lds128(u0), h1 = lds128(u1);
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) {
            uint2 q0 = lds64(u0 + 16 + 32 * cc + 8 * ro.t), q1 = lds64(u1 + 16 + 32 * cc + 8 * ro.t);
#pragma unroll
            for (int nib = 0; nib < 2; ++nib) {
                const int G = 2 * cc + nib;
                uint32_t a[4] = {(q0.x >> (4 * nib)) & 0x0F0F0F0Fu, (q1.x >> (4 * nib)) & 0x0F0F0F0Fu,
                                 (q0.y >> (4 * nib)) & 0x0F0F0F0Fu, (q1.y >> (4 * nib)) & 0x0F0F0F0Fu};
                step(G, a);
                if (G % CH == CH - 1) {
                    const int Gc = G - (CH - 1);
                    float d0, m0, d1, m1;
                    q4k_pair(h0, Gc >= 4, (Gc & 3) + ro.fin_p, &d0, &m0);
                    q4k_pair(h1, Gc >= 4, (Gc & 3) + ro.fin_p, &d1, &m1);
                    finish(Gc, d0, d1, m0, m1);
                }
            }
        }
    } else if constexpr (TYPE == T_Q8_0) {
#pragma unroll
        for (int G = 0; G < 8; ++G) {
            uint2 q0, q1;
            if (G % 2 == 0) {  // 34*G + 2 is 2 mod 4
                q0 = lds64_mis<2>(u0 + 34 * G + 2 + 8 * ro.t);
                q1 = lds64_mis<2>(u1 + 34 * G + 2 + 8 * ro.t);
            } else {
                q0 = lds64_mis<0>(u0 + 34 * G + 2 + 8 * ro.t);
                q1 = lds64_mis<0>(u1 + 34 * G + 2 + 8 * ro.t);
            }
            uint32_t a[4] = {q0.x, q1.x, q0.y, q1.y};
            step(G, a);
            if (G % CH == CH - 1) {
                const int Gc = G - (CH - 1);
                float d0 = f16_bits_to_f32(lds16(u0 + 34 * (Gc + ro.fin_p)));
                float d1 = f16_bits_to_f32(lds16(u1 + 34 * (Gc + ro.fin_p)));
                finish(Gc, d0, d1, 0.0f, 0.0f);
            }
        }
    } else if constexpr (TYPE == T_IQ2_XXS) {
        // The block is 2-byte aligned; its 8-byte groups start at +2, so whether they are word aligned depends
        // on the block's position.  Read three aligned words and shift.
        const float d0 = f16_bits_to_f32(lds16(u0)), d1 = f16_bits_to_f32(lds16(u1));
        const uint32_t s0 = 8 * (uint32_t)(reinterpret_cast<uintptr_t>(u0 + 2) & 3);
        const uint32_t s1 = 8 * (uint32_t)(reinterpret_cast<uintptr_t>(u1 + 2) & 3);
        const uint8_t* a0 = u0 + 2 - (s0 >> 3);
        const uint8_t* a1 = u1 + 2 - (s1 >> 3);
#pragma unroll
        for (int G = 0; G < 8; ++G) {
            // group bytes: 4 grid codes, then a word of 4 x 7 sign bits + 4-bit scale
            uint32_t x0 = lds32(a0 + 8 * G), x1 = lds32(a0 + 8 * G + 4), x2 = lds32(a0 + 8 * G + 8);
            uint32_t y0 = lds32(a1 + 8 * G), y1 = lds32(a1 + 8 * G + 4), y2 = lds32(a1 + 8 * G + 8);
            uint32_t lo0 = __funnelshift_r(x0, x1, s0), hi0 = __funnelshift_r(x1, x2, s0);
            uint32_t lo1 = __funnelshift_r(y0, y1, s1), hi1 = __funnelshift_r(y1, y2, s1);
            uint2 g0 = s_grid[(lo0 >> (8 * ro.t)) & 0xFF], g1 = s_grid[(lo1 >> (8 * ro.t)) & 0xFF];
            uint2 k0 = s_mask[(hi0 >> (7 * ro.t)) & 127], k1 = s_mask[(hi1 >> (7 * ro.t)) & 127];
            // negate the bytes under the mask: (v ^ 0xFF) + 1; grid bytes are never 0, so no carry leaves a byte
            uint32_t a[4] = {(g0.x ^ k0.x) + (k0.x & 0x01010101u), (g1.x ^ k1.x) + (k1.x & 0x01010101u),
                             (g0.y ^ k0.y) + (k0.y & 0x01010101u), (g1.y ^ k1.y) + (k1.y & 0x01010101u)};
            step(G, a);
            if (G % CH == CH - 1) {
                const int Gc = G - (CH - 1);
                // 4-bit scale of the finaliser's own group: top nibble of that group's last byte
                uint32_t b0 = u0[2 + 8 * (Gc + ro.fin_p) + 7] >> 4, b1 = u1[2 + 8 * (Gc + ro.fin_p) + 7] >> 4;
                float db0 = __fmul_rn(__fmul_rn(d0, __fadd_rn(0.5f, (float)b0)), 0.25f);
                float db1 = __fmul_rn(__fmul_rn(d1, __fadd_rn(0.5f, (float)b1)), 0.25f);
                finish(Gc, db0, db1, 0.0f, 0.0f);
            }
        }
    } else if constexpr (TYPE == T_MXFP4) {
        // codes -> twice the E2M1 value by byte-permute lookups; sign picks between a positive and a negated table
        const uint32_t P0 = 0x03020100u, P1 = 0x0C080604u, N0 = 0xFDFEFF00u, N1 = 0xF4F8FAFCu;
        auto decode4 = [&](uint32_t w, uint32_t w4, uint32_t sel, uint32_t sign_sel) {
            uint32_t pos = prmt(P0, P1, sel & 0xFFFFu), neg = prmt(N0, N1, sel & 0xFFFFu);
            uint32_t sm = prmt(w, w4, sign_sel);  // 0xFF where the nibble's sign bit is set
            return (pos & ~sm) | (neg & sm);
        };
#pragma unroll
        for (int G = 0; G < 8; ++G) {
            const int mis = (17 * G + 1) & 3;  // the unit is 4-byte aligned
            const uint8_t* p0 = u0 + 17 * G + 1 + 4 * ro.t - mis;
            const uint8_t* p1 = u1 + 17 * G + 1 + 4 * ro.t - mis;
            uint32_t w0 = lds32(p0), w1 = lds32(p1);
            if (mis) {
                w0 = __funnelshift_r(w0, lds32(p0 + 4), 8 * mis);
                w1 = __funnelshift_r(w1, lds32(p1 + 4), 8 * mis);
            }
            uint32_t m0 = w0 & 0x77777777u, m1 = w1 & 0x77777777u;
            uint32_t a[4] = {decode4(w0, w0 << 4, m0, 0x9D8Cu), decode4(w1, w1 << 4, m1, 0x9D8Cu),
                             decode4(w0, w0 << 4, m0 >> 16, 0xBFAEu), decode4(w1, w1 << 4, m1 >> 16, 0xBFAEu)};
            step(G, a);
            if (G % CH == CH - 1) {
                const int Gc = G - (CH - 1);
                uint32_t e0 = u0[17 * (Gc + ro.fin_p)], e1 = u1[17 * (Gc + ro.fin_p)];
                // codes are doubled, so the scale is 2^(e-128); e = 255 zeroes the block, e <= 1 is subnormal
                float sc0 = e0 == 255 ? 0.0f : __uint_as_float(e0 > 1 ? (e0 - 1) << 23 : (e0 == 1 ? 0x00400000u : 0x00200000u));
                float sc1 = e1 == 255 ? 0.0f : __uint_as_float(e1 > 1 ? (e1 - 1) << 23 : (e1 == 1 ? 0x00400000u : 0x00200000u));
                finish(Gc, sc0, sc1, 0.0f, 0.0f);
            }
        }
    } else if constexpr (TYPE == T_Q2_K) {
        // 16 groups of 16 values; word (sg, hf) of the 2-bit fields holds groups j = 2i + hf (shift 2i) of
        // super-group sg, which chain naturally.  m16n8k16: one A register per row, one B register.
        const uint32_t dd0 = lds32(u0 + 80), dd1 = lds32(u1 + 80);
        const float d0 = f16_bits_to_f32(dd0 & 0xFFFF), dm0 = f16_bits_to_f32(dd0 >> 16);
        const float d1 = f16_bits_to_f32(dd1 & 0xFFFF), dm1 = f16_bits_to_f32(dd1 >> 16);
#pragma unroll
        for (int sg = 0; sg < 2; ++sg) {
#pragma unroll
            for (int hf = 0; hf < 2; ++hf) {
                uint32_t q0 = lds32(u0 + 16 + 32 * sg + 16 * hf + 4 * ro.t);
                uint32_t q1 = lds32(u1 + 16 + 32 * sg + 16 * hf + 4 * ro.t);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int p = i % CH;
                    const int j = 2 * i + hf;                  // 16-group inside the super-group
                    const uint32_t G32 = 4 * sg + (j >> 1);    // its 32-group inside the unit (half = hf)
                    if (p == 0) {
#pragma unroll
                        for (int h = 0; h < NH; ++h) {
                            // chain positions are groups j = 2(i + sup_p) + hf -> 32-group 4sg + i + sup_p
                            uint64_t idx = ((uint64_t)ro.sup_row[h] * act.n_groups + (G0 + G32 + ro.sup_p)) * 96 +
                                           16 * hf + 4 * ro.t;
                            bsup[h].x = __ldg(reinterpret_cast<const uint32_t*>(act.planes + idx + 32 * ro.sup_odd));
                            bsupl[h].x = ro.sup_odd ? 0u : __ldg(reinterpret_cast<const uint32_t*>(act.planes + idx + 64));
                            c[h][0] = c[h][1] = c[h][2] = c[h][3] = cl[h][0] = cl[h][1] = cl[h][2] = cl[h][3] = 0;
                        }
                    }
                    uint32_t a0 = (q0 >> (2 * i)) & 0x03030303u, a1 = (q1 >> (2 * i)) & 0x03030303u;
#pragma unroll
                    for (int h = 0; h < NH; ++h) {
                        mma_k16(c[h], a0, a1, ro.sup_p == p ? bsup[h].x : 0u);
                        mma_k16(cl[h], a0, a1, ro.sup_p == p ? bsupl[h].x : 0u);
                    }
                    if (p == CH - 1) {
                        const int ic = i - (CH - 1);  // first group of the chain
                        const uint32_t jm = 2 * (ic + ro.fin_p) + hf;
                        uint32_t sc0 = u0[8 * sg + jm], sc1 = u1[8 * sg + jm];
                        float s0 = __fmul_rn(d0, (float)(sc0 & 15)), o0 = __fmul_rn(dm0, (float)(sc0 >> 4));
                        float s1 = __fmul_rn(d1, (float)(sc1 & 15)), o1 = __fmul_rn(dm1, (float)(sc1 >> 4));
                        const uint32_t Gm = G0 + 4 * sg + ic + ro.fin_p;
#pragma unroll
                        for (int h = 0; h < NH; ++h) {
                            uint64_t mi = (uint64_t)ro.fin_row[h] * act.n_groups + Gm;
                            float sa = __ldg(&act.meta[mi].x);
                            float sx = __ldg(act.sum16 + mi * 2 + hf);
                            float i0 = fmaf((float)c[h][0], 64516.0f, (float)(c[h][1] * 254 + cl[h][0])) * sa;
                            float i1 = fmaf((float)c[h][2], 64516.0f, (float)(c[h][3] * 254 + cl[h][2])) * sa;
                            acc[h][0] = fmaf(s0, i0, fmaf(-o0, sx, acc[h][0]));
                            acc[h][1] = fmaf(s1, i1, fmaf(-o1, sx, acc[h][1]));
                        }
                    }
                }
            }
        }
    }
}

// ────────────────────────────── the kernel ────────────────────────────────

template <uint32_t TYPE, int MB, int NH, int NWARP>
__global__ void __launch_bounds__(NWARP * 32)
    gemv_mma_kernel(const uint8_t* __restrict__ w, uint64_t n, uint64_t k, ActPlanes act, uint64_t m,
                    float* __restrict__ dst, uint32_t row_stride, int* __restrict__ error_flag) {
    using Tr = Traits<TYPE>;
    extern __shared__ __align__(128) uint8_t smem[];
    // layout: [2 stages][ROWS][row_stride] | grid table (IQ2_XXS) | reduction buffer | mbarriers
    const uint32_t stage_bytes = ROWS * row_stride;
    uint8_t* stages = smem;
    uint2* s_grid = reinterpret_cast<uint2*>(smem + 2 * stage_bytes);
    uint2* s_mask = s_grid + (TYPE == T_IQ2_XXS ? 256 : 0);
    float* s_red = reinterpret_cast<float*>(s_mask + (TYPE == T_IQ2_XXS ? 128 : 0));
    uint64_t* bars = reinterpret_cast<uint64_t*>(s_red + NWARP * ROWS * 4 * NH);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const Roles<MB, NH> ro(lane, m);
    const uint64_t row0 = (uint64_t)blockIdx.x * ROWS;
    const uint32_t units_per_row = (uint32_t)(k / 256);
    const uint64_t row_bytes = (uint64_t)units_per_row * Tr::UNIT_BYTES;
    const uint32_t n_chunks = (units_per_row + Tr::CHUNK_UNITS - 1) / Tr::CHUNK_UNITS;

    if (tid == 0) {
        mbar_init(&bars[0], ROWS);
        mbar_init(&bars[1], ROWS);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (TYPE == T_IQ2_XXS) {
        for (int i = tid; i < 256; i += NWARP * 32) s_grid[i] = g_iq2xxs_grid[i];
        for (int i = tid; i < 128; i += NWARP * 32) {
            uint32_t sg = iq2_signs(i);
            uint32_t lo = ((sg & 0xF) * 0x00204081u) & 0x01010101u, hi = ((sg >> 4) * 0x00204081u) & 0x01010101u;
            s_mask[i] = make_uint2(lo * 0xFFu, hi * 0xFFu);
        }
    }
    __syncthreads();

    // Row r of the tile, chunk c: copy the 16-byte aligned span that covers its bytes.
    auto issue = [&](uint32_t chunk) {
        if (warp == 0 && lane < ROWS) {
            uint64_t row = row0 + lane < n ? row0 + lane : n - 1;
            uint32_t u_lo = chunk * Tr::CHUNK_UNITS;
            uint32_t u_hi = min(units_per_row, u_lo + Tr::CHUNK_UNITS);
            uintptr_t beg = reinterpret_cast<uintptr_t>(w) + row * row_bytes + (uint64_t)u_lo * Tr::UNIT_BYTES;
            uintptr_t end = beg + (uint64_t)(u_hi - u_lo) * Tr::UNIT_BYTES;
            uintptr_t abeg = beg & ~(uintptr_t)15, aend = (end + 15) & ~(uintptr_t)15;
            uint32_t bytes = (uint32_t)(aend - abeg);
            uint64_t* bar = &bars[chunk & 1];
            mbar_arrive_expect_tx(bar, bytes);
            bulk_g2s(stages + (chunk & 1) * stage_bytes + lane * row_stride, reinterpret_cast<const void*>(abeg),
                     bytes, bar);
        }
    };

    float acc[NH][2];
#pragma unroll
    for (int h = 0; h < NH; ++h) acc[h][0] = acc[h][1] = 0.0f;

    issue(0);
    if (n_chunks > 1) issue(1);

    // byte offset of the row's first unit inside its aligned span
    auto row_shift = [&](int r) -> uint32_t {
        uint64_t row = row0 + r < n ? row0 + r : n - 1;
        return (uint32_t)((reinterpret_cast<uintptr_t>(w) + row * row_bytes) & 15);
    };
    // chunk starts are multiples of CHUNK_UNITS * UNIT_BYTES, a multiple of 16 for every format,
    // so the shift is the same for every chunk of a row
    const uint32_t sh0 = row_shift(ro.g), sh1 = row_shift(ro.g + 8);

    for (uint32_t chunk = 0; chunk < n_chunks; ++chunk) {
        bool ok = mbar_wait(&bars[chunk & 1], (chunk >> 1) & 1);
        if (!__syncthreads_and(ok)) {
            if (tid == 0) *reinterpret_cast<volatile int*>(error_flag) = 1;
            return;
        }
        const uint8_t* st = stages + (chunk & 1) * stage_bytes;
        const uint32_t u_lo = chunk * Tr::CHUNK_UNITS;
        const uint32_t cnt = min(units_per_row - u_lo, Tr::CHUNK_UNITS);
        for (uint32_t u = warp; u < cnt; u += NWARP) {
            const uint8_t* u0 = st + ro.g * row_stride + sh0 + u * Tr::UNIT_BYTES;
            const uint8_t* u1 = st + (ro.g + 8) * row_stride + sh1 + u * Tr::UNIT_BYTES;
            process_unit<TYPE, MB, NH>(u0, u1, (u_lo + u) * 8, act, ro, s_grid, s_mask, acc);
        }
        __syncthreads();  // every warp is done with this stage
        if (chunk + 2 < n_chunks) issue(chunk + 2);
    }

    // Sum the chain positions that share a batch row, then the warps, in a fixed order.
#pragma unroll
    for (int h = 0; h < NH; ++h)
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            float v = acc[h][r];
            if (MB == 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, 1);
            if (MB <= 2) v += __shfl_xor_sync(0xFFFFFFFFu, v, 2);
            acc[h][r] = v;
        }
    if (ro.t < MB) {
#pragma unroll
        for (int h = 0; h < NH; ++h) {
            s_red[((warp * NH + h) * 4 + ro.t) * ROWS + ro.g] = acc[h][0];
            s_red[((warp * NH + h) * 4 + ro.t) * ROWS + ro.g + 8] = acc[h][1];
        }
    }
    __syncthreads();
    for (int o = tid; o < NH * MB * ROWS; o += NWARP * 32) {
        int r = o % ROWS, bi = o / ROWS;  // bi = h * MB + i
        int h = bi / MB, i = bi % MB;
        uint64_t batch = (uint64_t)i + 4 * h;
        if (batch < m && row0 + r < n) {
            float v = 0.0f;
#pragma unroll
            for (int wv = 0; wv < NWARP; ++wv) v += s_red[((wv * NH + h) * 4 + i) * ROWS + r];
            dst[batch * n + row0 + r] = v;
        }
    }
}

template <uint32_t TYPE>
uint32_t row_stride_for(uint64_t k) {
    using Tr = Traits<TYPE>;
    uint32_t units = (uint32_t)std::min<uint64_t>(k / 256, Tr::CHUNK_UNITS);
    uint32_t span = units * Tr::UNIT_BYTES + 32;  // up to 15 bytes of lead-in and 15 of tail, rounded
    span = (span + 15) & ~15u;
    // stride = 8 words mod 32: rows g = 0..3 of a half-warp's 64-bit loads land in distinct bank octets
    uint32_t words = span / 4;
    uint32_t pad = (8 + 32 - words % 32) % 32;
    return (words + pad) * 4;
}

template <uint32_t TYPE, int MB, int NH>
cudaError_t launch_one(const uint8_t* w, uint64_t n, uint64_t k, const ActPlanes& act, uint64_t m, float* dst,
                       int* error_flag, cudaStream_t s) {
    constexpr int NWARP = 8;
    uint32_t stride = row_stride_for<TYPE>(k);
    size_t smem = 2 * (size_t)ROWS * stride + (TYPE == T_IQ2_XXS ? (256 + 128) * 8 : 0) +
                  (size_t)NWARP * ROWS * 4 * NH * 4 + 16;
    auto kern = gemv_mma_kernel<TYPE, MB, NH, NWARP>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    unsigned grid = (unsigned)((n + ROWS - 1) / ROWS);
    kern<<<grid, NWARP * 32, smem, s>>>(w, n, k, act, m, dst, stride, error_flag);
    return cudaGetLastError();
}

template <uint32_t TYPE>
cudaError_t launch_type(const uint8_t* w, uint64_t n, uint64_t k, const ActPlanes& act, uint64_t m, float* dst,
                        int* error_flag, cudaStream_t s) {
    if (m == 1) return launch_one<TYPE, 1, 1>(w, n, k, act, m, dst, error_flag, s);
    if (m == 2) return launch_one<TYPE, 2, 1>(w, n, k, act, m, dst, error_flag, s);
    if (m <= 4) return launch_one<TYPE, 4, 1>(w, n, k, act, m, dst, error_flag, s);
    if (m <= 8) return launch_one<TYPE, 4, 2>(w, n, k, act, m, dst, error_flag, s);
    if (m <= 16) return launch_one<TYPE, 4, 4>(w, n, k, act, m, dst, error_flag, s);
    return cudaErrorInvalidValue;
}

}  // namespace

size_t gemv_mma_scratch_bytes(uint64_t m, uint64_t k) {
    uint64_t groups = m * (k / 32);
    return (size_t)(groups * 96 + groups * 8 + groups * 8 + 256);
}

bool gemv_mma_supports(uint32_t type, const uint8_t* w, uint64_t n, uint64_t k, uint64_t m) {
    if (m == 0 || m > GEMV_MMA_MAX_M || n == 0 || k == 0 || k % 256 != 0) return false;
    uintptr_t a = reinterpret_cast<uintptr_t>(w);
    switch (type) {
        case T_Q4_K: return a % 16 == 0;
        case T_Q8_0: return a % 16 == 0;
        case T_Q2_K: return a % 4 == 0;
        case T_IQ2_XXS: return a % 2 == 0;
        case T_MXFP4: return a % 4 == 0 && (k / 32 * 17) % 4 == 0;
        default: return false;
    }
}

cudaError_t launch_gemv_mma(uint32_t type, const uint8_t* w, uint64_t n, uint64_t k, const float* lhs, uint64_t m,
                            float* dst, void* scratch, int* error_flag, cudaStream_t s) {
    uint64_t groups = m * (k / 32);
    ActPlanes act;
    int8_t* planes = static_cast<int8_t*>(scratch);
    float2* meta = reinterpret_cast<float2*>(planes + groups * 96);
    float* sum16 = reinterpret_cast<float*>(meta + groups);
    act.planes = planes;
    act.meta = meta;
    act.sum16 = sum16;
    act.n_groups = (uint32_t)(k / 32);
    unsigned qgrid = (unsigned)std::min<uint64_t>((groups + 7) / 8, 148 * 8);
    quantize_acts_kernel<<<qgrid, 256, 0, s>>>(lhs, m, k, type, planes, meta, sum16);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    switch (type) {
        case T_Q4_K: return launch_type<T_Q4_K>(w, n, k, act, m, dst, error_flag, s);
        case T_Q8_0: return launch_type<T_Q8_0>(w, n, k, act, m, dst, error_flag, s);
        case T_Q2_K: return launch_type<T_Q2_K>(w, n, k, act, m, dst, error_flag, s);
        case T_IQ2_XXS: return launch_type<T_IQ2_XXS>(w, n, k, act, m, dst, error_flag, s);
        case T_MXFP4: return launch_type<T_MXFP4>(w, n, k, act, m, dst, error_flag, s);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace jq
