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
//     x ~= (s/254^2) * (254^2*hi + 254*mid + lo) with one scale s per 256 values,
//     |error| <= max|x| * 6.1e-8, i.e. f32 precision (quantize_acts), so sum_c x_c q_c is three exact int32 dot
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
// MMA tile use: A = 16 weight rows x 32 codes, B = 32 codes x 8 columns.  The legacy integer MMA pipe is
// the scarce unit on this part (one m16n8k32 per 8 cycles per SM), so one MMA per group must do: the
// three planes of a batch row take three columns (a slot), an MMA carries two slots, and with one batch
// row 2 consecutive groups are chained into one accumulator by giving each its own slot.  Group scales
// that are small integers (Q4_K, Q2_K, IQ2_XXS) are multiplied in as integers and summed over the
// 256-value unit before one float conversion; f16 / power-of-two scales (Q8_0, MXFP4) are applied in
// float per group.  Batches above 2 run NH passes over the same A fragments.
//
// Algorithmic bytes per launch: n*k/B*S (weights) + 4*m*(k + n).
#include <algorithm>
#include <cstdlib>

#include "common.cuh"
#include "pipe.cuh"

namespace jq {

cudaError_t tables_gemv_mma() { return upload_tables(); }

namespace {

constexpr int ROWS = 16;  // weight rows per CTA (one MMA M tile)

// ───────────────────────────── PTX helpers ────────────────────────────────

__device__ __forceinline__ void mma_k32(int c[4], const uint32_t a[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// Same with an unsigned A operand (bytes 0..255).
__device__ __forceinline__ void mma_k32_u8(int c[4], const uint32_t a[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
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
//   meta[i*NG + G]                  float2 {s/254^2 of the group's 256-value unit, sum of x over the group}
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

// Splits the 256 values of one unit, 8 per lane (lane l holds values 8l .. 8l+7, group l / 4), into the three
// planes.  `planes` points at the unit's first group (8 x 96 bytes), `meta` / `sum16` at its first entries.
__device__ __forceinline__ void quantize_unit_values(const float (&v)[8], uint32_t lane, uint32_t type, int8_t* planes,
                                                     float2* meta, float* sum16) {
    float amax = 0.0f, sum = 0.0f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        amax = fmaxf(amax, fabsf(v[j]));
        sum += v[j];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
    float s16 = sum + __shfl_xor_sync(0xFFFFFFFFu, sum, 1);  // 16-value half: lanes 2h, 2h+1
    float s32 = s16 + __shfl_xor_sync(0xFFFFFFFFu, s16, 2);  // 32-value group: lanes 4G .. 4G+3
    const float s = amax * (1.0f / 127.0f);
    const bool live = s > 0.0f && isfinite(s);
    const float s1 = s * (1.0f / 254.0f), s2 = s1 * (1.0f / 254.0f);
    const float inv = live ? 1.0f / s : 0.0f;
    uint32_t pk[3][2] = {{0, 0}, {0, 0}, {0, 0}};
    int8_t* gp = planes + (lane >> 2) * 96;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        int q0 = 0, q1 = 0, q2 = 0;
        if (live) {
            q0 = max(-127, min(127, __float2int_rn(v[j] * inv)));
            float r1 = fmaf(-(float)q0, s, v[j]);
            q1 = max(-127, min(127, __float2int_rn(r1 * (inv * 254.0f))));
            float r2 = fmaf(-(float)q1, s1, r1);
            q2 = max(-127, min(127, __float2int_rn(r2 * (inv * 64516.0f))));
        }
        if (type == T_MXFP4) {
            uint32_t pos = act_position(type, 8 * (lane & 3) + j);
            gp[pos] = (int8_t)q0;
            gp[32 + pos] = (int8_t)q1;
            gp[64 + pos] = (int8_t)q2;
        } else {
            pk[0][j >> 2] |= (uint32_t)(q0 & 0xFF) << (8 * (j & 3));
            pk[1][j >> 2] |= (uint32_t)(q1 & 0xFF) << (8 * (j & 3));
            pk[2][j >> 2] |= (uint32_t)(q2 & 0xFF) << (8 * (j & 3));
        }
    }
    if (type != T_MXFP4) {
#pragma unroll
        for (int pl = 0; pl < 3; ++pl)
            *reinterpret_cast<uint2*>(gp + 32 * pl + 8 * (lane & 3)) = make_uint2(pk[pl][0], pk[pl][1]);
    }
    if ((lane & 3) == 0) meta[lane >> 2] = make_float2(live ? s2 : 0.0f, s32);
    if ((lane & 1) == 0) sum16[lane >> 1] = s16;
}


// The unit's values come from memory.  COHERENT: x may have been written by another CTA of this same launch
// (the persistent chain): read it from L2.  With `nw` (the unit's 256 RMS-norm weights) the values split are
// x * rs * nw, i.e. the normalised row.
template <bool COHERENT = false>
__device__ __forceinline__ void load_unit_values(const float* __restrict__ xu, uint32_t lane, float (&v)[8]) {
    const float4* src = reinterpret_cast<const float4*>(xu + lane * 8);
    float4 lo4 = COHERENT ? __ldcg(src) : __ldg(src), hi4 = COHERENT ? __ldcg(src + 1) : __ldg(src + 1);
    v[0] = lo4.x, v[1] = lo4.y, v[2] = lo4.z, v[3] = lo4.w, v[4] = hi4.x, v[5] = hi4.y, v[6] = hi4.z, v[7] = hi4.w;
}

template <bool COHERENT = false>
__device__ __forceinline__ void quantize_unit_warp(const float* __restrict__ xu, uint32_t lane, uint32_t type,
                                                   int8_t* planes, float2* meta, float* sum16,
                                                   const float* __restrict__ nw = nullptr, float rs = 1.0f) {
    float v[8];
    load_unit_values<COHERENT>(xu, lane, v);
    if (nw) {
        float g[8];
        load_unit_values<false>(nw, lane, g);
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = v[j] * rs * g[j];
    }
    quantize_unit_values(v, lane, type, planes, meta, sum16);
}

// The activation prologue of the matmul kernels: `rows` x k f32 values -> planes in shared memory, by NW warps
// (w = 0 .. NW-1) that meet on named barrier 1.  Loads are requested in batches before any is used, so the
// prologue costs about one trip to L2 instead of one per unit.  With `norm_w` every row is RMS-normalised
// first (1 / rms from the units' sums of squares, added in unit order).  s_tmp: NW * GEMV_MMA_MAX_M floats.
template <bool COHERENT, int NW>
__device__ __forceinline__ void split_activations(const float* __restrict__ x, uint32_t rows, uint32_t k,
                                                  const float* __restrict__ norm_w, float eps, uint32_t type,
                                                  uint8_t* s_act, int w, uint32_t lane, float* s_tmp) {
    const uint32_t units_per_row = k / 256, total = rows * units_per_row;
    const uint64_t groups = (uint64_t)rows * (k / 32);
    int8_t* planes = reinterpret_cast<int8_t*>(s_act);
    float2* meta = reinterpret_cast<float2*>(s_act + groups * 96);
    float* sum16 = reinterpret_cast<float*>(s_act + groups * 104);
    if (norm_w == nullptr) {
        for (uint32_t u0 = w; u0 < total; u0 += 4 * NW) {
            float v[4][8];
#pragma unroll
            for (int r = 0; r < 4; ++r)
                if (u0 + r * NW < total) load_unit_values<COHERENT>(x + (uint64_t)(u0 + r * NW) * 256, lane, v[r]);
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                const uint32_t u = u0 + r * NW;
                if (u < total) quantize_unit_values(v[r], lane, type, planes + (uint64_t)u * 768, meta + u * 8, sum16 + u * 16);
            }
        }
    } else if (total <= 2 * NW && total <= (uint32_t)NW * GEMV_MMA_MAX_M) {
        // at most two units per warp: values stay in registers between the sum of squares and the split
        float v[2][8], g[2][8];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const uint32_t u = w + r * NW;
            if (u < total) {
                load_unit_values<COHERENT>(x + (uint64_t)u * 256, lane, v[r]);
                load_unit_values<false>(norm_w + (u % units_per_row) * 256, lane, g[r]);
            }
        }
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const uint32_t u = w + r * NW;
            if (u < total) {
                float ss = 0.0f;
#pragma unroll
                for (int j = 0; j < 8; ++j) ss = fmaf(v[r][j], v[r][j], ss);
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xFFFFFFFFu, ss, o);
                if (lane == 0) s_tmp[u] = ss;
            }
        }
        asm volatile("bar.sync 1, %0;" ::"r"(NW * 32) : "memory");
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const uint32_t u = w + r * NW;
            if (u < total) {
                const uint32_t row = u / units_per_row;
                float tot = 0.0f;
                for (uint32_t q = 0; q < units_per_row; ++q) tot += s_tmp[row * units_per_row + q];
                const float rs = rsqrtf(tot / (float)k + eps);
#pragma unroll
                for (int j = 0; j < 8; ++j) v[r][j] = v[r][j] * rs * g[r][j];
                quantize_unit_values(v[r], lane, type, planes + (uint64_t)u * 768, meta + u * 8, sum16 + u * 16);
            }
        }
    } else {
        // wider inputs: two passes over x
        float* s_rs = s_tmp + (NW - 1) * GEMV_MMA_MAX_M;  // the last warp's slots double as the row scales
        for (uint32_t r = 0; r < rows; ++r) {
            const float4* xr = reinterpret_cast<const float4*>(x + (uint64_t)r * k);
            float ss = 0.0f;
            for (uint32_t i = w * 32 + lane; i < k / 4; i += NW * 32) {
                float4 q = COHERENT ? __ldcg(xr + i) : __ldg(xr + i);
                ss = fmaf(q.x, q.x, fmaf(q.y, q.y, fmaf(q.z, q.z, fmaf(q.w, q.w, ss))));
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xFFFFFFFFu, ss, o);
            float tot = 0.0f;
            // every warp's partial sum, in warp order, through shared memory (one row at a time)
            asm volatile("bar.sync 1, %0;" ::"r"(NW * 32) : "memory");
            if (lane == 0) s_tmp[w * GEMV_MMA_MAX_M] = ss;
            asm volatile("bar.sync 1, %0;" ::"r"(NW * 32) : "memory");
            for (int q = 0; q < NW; ++q) tot += s_tmp[q * GEMV_MMA_MAX_M];
            const float rs = rsqrtf(tot / (float)k + eps);
            for (uint32_t uc = w; uc < units_per_row; uc += NW) {
                const uint32_t u = r * units_per_row + uc;
                quantize_unit_warp<COHERENT>(x + (uint64_t)u * 256, lane, type, planes + (uint64_t)u * 768, meta + u * 8,
                                             sum16 + u * 16, norm_w + uc * 256, rs);
            }
        }
        (void)s_rs;
    }
    asm volatile("bar.sync 1, %0;" ::"r"(NW * 32) : "memory");
}

__global__ void __launch_bounds__(256) quantize_acts_kernel(const float* __restrict__ x, uint64_t m, uint64_t k,
                                                            uint32_t type, int8_t* __restrict__ planes,
                                                            float2* __restrict__ meta, float* __restrict__ sum16) {
    // one block per 256-value unit, one thread per value; warp = 32-value group
    __shared__ float s_max[8];
    pdl_trigger();
    pdl_wait();
    const uint32_t lane = threadIdx.x & 31, grp = threadIdx.x >> 5;
    const uint64_t total = m * (k / 256);
    for (uint64_t w = blockIdx.x; w < total; w += gridDim.x) {
        float v = x[w * 256 + threadIdx.x];
        float amax = fabsf(v), sum = v;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
            if (o < 16) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, o);
        }
        // `sum` holds the sum of the lane's 16-value half
        float other = __shfl_xor_sync(0xFFFFFFFFu, sum, 16);
        if (lane == 0) s_max[grp] = amax;
        __syncthreads();
        float umax = s_max[0];
#pragma unroll
        for (int i = 1; i < 8; ++i) umax = fmaxf(umax, s_max[i]);
        __syncthreads();
        const float s = umax * (1.0f / 127.0f);
        const bool live = s > 0.0f && isfinite(s);
        const float s1 = s * (1.0f / 254.0f), s2 = s1 * (1.0f / 254.0f);
        int q0 = 0, q1 = 0, q2 = 0;
        if (live) {
            // the rounded quotients need not be exact: each residual is formed exactly and handed down
            const float inv = 1.0f / s;
            q0 = max(-127, min(127, __float2int_rn(v * inv)));
            float r1 = fmaf(-(float)q0, s, v);
            q1 = max(-127, min(127, __float2int_rn(r1 * (inv * 254.0f))));
            float r2 = fmaf(-(float)q1, s1, r1);
            q2 = max(-127, min(127, __float2int_rn(r2 * (inv * 64516.0f))));
        }
        const uint64_t gbase = (w * 8 + grp) * 96;
        const uint32_t pos = act_position(type, lane);
        planes[gbase + pos] = (int8_t)q0;
        planes[gbase + 32 + pos] = (int8_t)q1;
        planes[gbase + 64 + pos] = (int8_t)q2;
        if (lane == 0) {
            meta[w * 8 + grp] = make_float2(live ? s2 : 0.0f, sum + other);
            sum16[(w * 8 + grp) * 2] = sum;
            sum16[(w * 8 + grp) * 2 + 1] = other;
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
    static constexpr uint32_t UNIT_BYTES = 144, CHUNK_UNITS = 16;
};
template <>
struct Traits<T_Q8_0> {
    static constexpr uint32_t UNIT_BYTES = 272, CHUNK_UNITS = 8;
};
template <>
struct Traits<T_Q2_K> {
    static constexpr uint32_t UNIT_BYTES = 84, CHUNK_UNITS = 24;
};
template <>
struct Traits<T_IQ2_XXS> {
    static constexpr uint32_t UNIT_BYTES = 66, CHUNK_UNITS = 32;
};
template <>
struct Traits<T_MXFP4> {
    static constexpr uint32_t UNIT_BYTES = 136, CHUNK_UNITS = 16;
};

// Activation data is read from shared memory when the kernel staged it there (ACT == 1) and from global
// memory through the read-only path otherwise.
template <int ACT, class T>
__device__ __forceinline__ T ld_act(const T* p) {
    if (ACT) return *p;
    return __ldg(p);
}

// Per-lane roles, fixed for the kernel's lifetime.
//
// One MMA has 8 activation columns.  A slot is three columns (hi, mid, lo planes of one batch row for one
// group); columns 0..2 are slot 0, 3..5 slot 1, 6..7 are fed zeros.  With MB batch rows per MMA (1 or 2),
// 2/MB consecutive groups are chained into one accumulator, slot = position * MB + batch row.
//   * supplier role: lane (g, t) feeds column g.
//   * holder role: lane t of a quad receives columns 2t and 2t+1 of rows g and g+8.  Scaling is linear in
//     every column, so each lane scales and accumulates its own two columns and the quad is summed once
//     per tile.
template <int MB, int NH>
struct Roles {
    static constexpr int CH = 2 / MB;  // groups chained into one accumulator
    static constexpr int NB = MB * NH; // batch slots of a tile
    int g, t;
    bool sup_live;                // column g carries data
    int sup_p, sup_plane, sup_i;  // chain position, plane and batch slot (within a pass) of column g
    int col_p[2], col_i[2];       // chain position and batch slot (within a pass) of held columns 2t, 2t+1
    float col_w[2];               // plane weight of the held columns: 254^2, 254, 1, or 0 for a dead column
    uint32_t brow[NB];            // activation row of batch slot b for the current tile (unused slots repeat the last)
    uint32_t col_row[NH][2];      // activation row behind held column j in pass h
    uint32_t sup_off[NH];         // byte offset of this lane's B bytes inside the planes for group 0 of pass h
    __device__ __forceinline__ explicit Roles(int lane) {
        g = lane >> 2;
        t = lane & 3;
        sup_live = g < 6;
        int slot = g / 3;
        sup_plane = g % 3;
        sup_p = slot / MB;
        sup_i = slot % MB;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            int col = 2 * t + j;
            int s = col / 3, pl = col % 3;
            col_p[j] = col < 6 ? s / MB : 0;
            col_i[j] = col < 6 ? s % MB : 0;
            col_w[j] = col >= 6 ? 0.0f : (pl == 0 ? 64516.0f : (pl == 1 ? 254.0f : 1.0f));
        }
    }
    // Point the roles at a tile's activation rows: slot b reads row `row0 + min(b, cnt-1)` of the
    // activation list (through `act_rows` when the rows are gathered).
    __device__ __forceinline__ void set_rows(uint32_t row0, uint32_t cnt, const uint32_t* act_rows, uint32_t n_groups) {
#pragma unroll
        for (int b = 0; b < NB; ++b) {
            uint32_t pos = row0 + min((uint32_t)b, cnt - 1);
            brow[b] = act_rows ? __ldg(act_rows + pos) : pos;
        }
        // register arrays must only be indexed by compile-time constants: pick with selects
#pragma unroll
        for (int h = 0; h < NH; ++h) {
            uint32_t srow = brow[h * MB];
#pragma unroll
            for (int i = 1; i < MB; ++i) srow = sup_i == i ? brow[h * MB + i] : srow;
            sup_off[h] = sup_live ? (uint32_t)(((uint64_t)srow * n_groups + sup_p) * 96 + 32 * sup_plane + 8 * t) : 0u;
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                uint32_t r = brow[h * MB];
#pragma unroll
                for (int i = 1; i < MB; ++i) r = col_i[j] == i ? brow[h * MB + i] : r;
                col_row[h][j] = r;
            }
        }
    }
};

// One unit (256 columns x 16 rows) of a warp's work.  u0 / u1 point at the unit's bytes for rows g and
// g+8 in shared memory; U is the unit's index along k (its first 32-group is 8U).
//   colacc[h][j][r]  running sum of held column j, row r (0: g, 1: g+8), pass h
//   minacc[b][r]     running sum of the minima terms of batch row b
template <uint32_t TYPE, int MB, int NH, int ACT>
__device__ __forceinline__ void process_unit(const uint8_t* u0, const uint8_t* u1, uint32_t U, const ActPlanes& act,
                                             const Roles<MB, NH>& ro, const uint2* s_grid, const uint2* s_mask,
                                             float colacc[NH][2][2], float minacc[MB * NH][2]) {
    constexpr int CH = Roles<MB, NH>::CH;
    constexpr bool INT_SCALE = TYPE == T_Q4_K || TYPE == T_Q2_K || TYPE == T_IQ2_XXS;
    const uint32_t G0 = 8 * U;
    int c[NH][4];           // MMA accumulators: c[0], c[1] = columns 2t, 2t+1 of row g; c[2], c[3] of row g+8
    int isum[NH][2][2];     // integer-scaled column sums over the unit (INT_SCALE formats)
    float fsum[NH][2][2];   // float-scaled column sums over the unit (other formats)
    uint2 bsup[NH];
#pragma unroll
    for (int h = 0; h < NH; ++h)
#pragma unroll
        for (int j = 0; j < 2; ++j) isum[h][j][0] = isum[h][j][1] = 0, fsum[h][j][0] = fsum[h][j][1] = 0.0f;

    // B fragment for the chain starting at group Gc (index inside the unit): this lane's column, 8 bytes
    // of its plane (4 bytes at byte offset `off16` for the 16-value groups of Q2_K).
    auto load_b = [&](uint32_t Gc, uint32_t off16, bool k16) {
#pragma unroll
        for (int h = 0; h < NH; ++h) {
            const int8_t* src = act.planes + ro.sup_off[h] + (uint64_t)(G0 + Gc) * 96;
            if (!ro.sup_live) {
                bsup[h] = make_uint2(0u, 0u);
            } else if (k16) {
                bsup[h].x = ld_act<ACT>(reinterpret_cast<const uint32_t*>(src + off16 - 4 * ro.t));
                bsup[h].y = 0u;
            } else {
                bsup[h] = ld_act<ACT>(reinterpret_cast<const uint2*>(src));
            }
        }
    };
    auto zero_c = [&]() {
#pragma unroll
        for (int h = 0; h < NH; ++h) c[h][0] = c[h][1] = c[h][2] = c[h][3] = 0;
    };
    auto mma_step = [&](int p, const uint32_t a[4], bool a_unsigned) {
#pragma unroll
        for (int h = 0; h < NH; ++h) {
            bool mine = ro.sup_p == p;
            if (a_unsigned)
                mma_k32_u8(c[h], a, mine ? bsup[h].x : 0u, mine ? bsup[h].y : 0u);
            else
                mma_k32(c[h], a, mine ? bsup[h].x : 0u, mine ? bsup[h].y : 0u);
        }
    };
    // After a chain: fold the accumulators into the unit sums.  sc[j][r] is the scale of the group that held
    // column j belongs to, for row r.
    auto fold_int = [&](const uint32_t sc[2][2]) {
#pragma unroll
        for (int h = 0; h < NH; ++h)
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                isum[h][j][0] += c[h][j] * (int)sc[j][0];
                isum[h][j][1] += c[h][2 + j] * (int)sc[j][1];
            }
    };
    auto fold_float = [&](const float sc[2][2]) {
#pragma unroll
        for (int h = 0; h < NH; ++h)
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                fsum[h][j][0] = fmaf((float)c[h][j], sc[j][0], fsum[h][j][0]);
                fsum[h][j][1] = fmaf((float)c[h][2 + j], sc[j][1], fsum[h][j][1]);
            }
    };
    // Unit end: unit sums -> running column sums.  f0 / f1: the unit's float factor for rows g / g+8.
    auto close_unit = [&](float f0, float f1) {
#pragma unroll
        for (int h = 0; h < NH; ++h)
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                // activation scale of the batch row this column belongs to (one per 256-value unit)
                uint32_t row = ro.col_row[h][j];
                float sa = ld_act<ACT>(&act.meta[(uint64_t)row * act.n_groups + G0].x) * ro.col_w[j];
                float v0 = INT_SCALE ? (float)isum[h][j][0] : fsum[h][j][0];
                float v1 = INT_SCALE ? (float)isum[h][j][1] : fsum[h][j][1];
                colacc[h][j][0] = fmaf(f0 * sa, v0, colacc[h][j][0]);
                colacc[h][j][1] = fmaf(f1 * sa, v1, colacc[h][j][1]);
            }
    };

    if constexpr (TYPE == T_Q4_K) {
        const uint4 h0 = lds128(u0), h1 = lds128(u1);
        // The 8 six-bit scales and 8 minima of a row as two words of 4 bytes each (src/kquant_dot.rs:106-118):
        // pairs 0..3 are the low 6 bits of bytes 0..3 / 4..7; pairs 4..7 take their low nibble from bytes
        // 8..11 (scale: low nibble, minimum: high nibble) and bits 4..5 from the top of bytes 0..3 / 4..7.
        const uint32_t sc0[2] = {h0.y & 0x3F3F3F3Fu, (h0.w & 0x0F0F0F0Fu) | ((h0.y >> 2) & 0x30303030u)};
        const uint32_t sc1[2] = {h1.y & 0x3F3F3F3Fu, (h1.w & 0x0F0F0F0Fu) | ((h1.y >> 2) & 0x30303030u)};
        const uint32_t mn0[2] = {h0.z & 0x3F3F3F3Fu, ((h0.w >> 4) & 0x0F0F0F0Fu) | ((h0.z >> 2) & 0x30303030u)};
        const uint32_t mn1[2] = {h1.z & 0x3F3F3F3Fu, ((h1.w >> 4) & 0x0F0F0F0Fu) | ((h1.z >> 2) & 0x30303030u)};
        // chunk cc = 64 values: low nibbles are group 2cc, high nibbles group 2cc+1.  High nibbles stay in
        // place (16*q as an unsigned byte).  With two groups per chain a held column always sees groups of
        // one parity, so the factor 16 sits in its column weight; otherwise even groups take 16*sc and the
        // unit factor carries 1/16.
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) {
            uint2 q0 = lds64(u0 + 16 + 32 * cc + 8 * ro.t), q1 = lds64(u1 + 16 + 32 * cc + 8 * ro.t);
#pragma unroll
            for (int nib = 0; nib < 2; ++nib) {
                const int G = 2 * cc + nib, p = G % CH;
                if (p == 0) {
                    load_b(G, 0, false);
                    zero_c();
                }
                const uint32_t mask = nib ? 0xF0F0F0F0u : 0x0F0F0F0Fu;
                uint32_t a[4] = {q0.x & mask, q1.x & mask, q0.y & mask, q1.y & mask};
                mma_step(p, a, true);
                if (p == CH - 1) {
                    uint32_t sc[2][2];
#pragma unroll
                    for (int j = 0; j < 2; ++j) {
                        // group of held column j: G - (CH-1) + col_p[j]; its byte inside the half-word
                        const int Gc = G - (CH - 1);
                        const uint32_t sh = 8 * ((Gc & 3) + ro.col_p[j]);
                        sc[j][0] = (sc0[Gc >> 2] >> sh) & 0xFF;
                        sc[j][1] = (sc1[Gc >> 2] >> sh) & 0xFF;
                        if (CH == 1 && (G & 1) == 0) sc[j][0] <<= 4, sc[j][1] <<= 4;
                    }
                    fold_int(sc);
                }
            }
        }
        // minima: lane t takes pairs 2t and 2t+1 of both rows
        const float dm0 = f16_bits_to_f32(h0.x >> 16), dm1 = f16_bits_to_f32(h1.x >> 16);
        const uint32_t mw0 = ro.t < 2 ? mn0[0] : mn0[1], mw1 = ro.t < 2 ? mn1[0] : mn1[1];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const uint32_t sh = 8 * (2 * (ro.t & 1) + e);
            float m0 = (float)((mw0 >> sh) & 0xFF) * dm0, m1 = (float)((mw1 >> sh) & 0xFF) * dm1;
#pragma unroll
            for (int b = 0; b < MB * NH; ++b) {
                float sx = ld_act<ACT>(&act.meta[(uint64_t)ro.brow[b] * act.n_groups + G0 + 2 * ro.t + e].y);
                minacc[b][0] = fmaf(m0, sx, minacc[b][0]);
                minacc[b][1] = fmaf(m1, sx, minacc[b][1]);
            }
        }
        const float fu = CH == 1 ? 0.0625f : 1.0f;
        close_unit(f16_bits_to_f32(h0.x & 0xFFFF) * fu, f16_bits_to_f32(h1.x & 0xFFFF) * fu);
    } else if constexpr (TYPE == T_Q8_0) {
#pragma unroll
        for (int G = 0; G < 8; ++G) {
            const int p = G % CH;
            if (p == 0) {
                load_b(G, 0, false);
                zero_c();
            }
            uint2 q0, q1;
            if (G % 2 == 0) {  // 34*G + 2 is 2 mod 4
                q0 = lds64_mis<2>(u0 + 34 * G + 2 + 8 * ro.t);
                q1 = lds64_mis<2>(u1 + 34 * G + 2 + 8 * ro.t);
            } else {
                q0 = lds64_mis<0>(u0 + 34 * G + 2 + 8 * ro.t);
                q1 = lds64_mis<0>(u1 + 34 * G + 2 + 8 * ro.t);
            }
            uint32_t a[4] = {q0.x, q1.x, q0.y, q1.y};
            mma_step(p, a, false);
            if (p == CH - 1) {
                float sc[2][2];
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    uint32_t Gj = G - (CH - 1) + ro.col_p[j];
                    sc[j][0] = f16_bits_to_f32(lds16(u0 + 34 * Gj));
                    sc[j][1] = f16_bits_to_f32(lds16(u1 + 34 * Gj));
                }
                fold_float(sc);
            }
        }
        close_unit(1.0f, 1.0f);
    } else if constexpr (TYPE == T_IQ2_XXS) {
        // The block is 2-byte aligned; its 8-byte groups start at +2, so whether they are word aligned depends
        // on the block's position.  Read three aligned words and shift.
        const uint32_t s0 = 8 * (uint32_t)(reinterpret_cast<uintptr_t>(u0 + 2) & 3);
        const uint32_t s1 = 8 * (uint32_t)(reinterpret_cast<uintptr_t>(u1 + 2) & 3);
        const uint8_t* a0 = u0 + 2 - (s0 >> 3);
        const uint8_t* a1 = u1 + 2 - (s1 >> 3);
#pragma unroll
        for (int G = 0; G < 8; ++G) {
            const int p = G % CH;
            if (p == 0) {
                load_b(G, 0, false);
                zero_c();
            }
            // group bytes: 4 grid codes, then a word of 4 x 7 sign bits + 4-bit scale
            uint32_t x0 = lds32(a0 + 8 * G), x1 = lds32(a0 + 8 * G + 4), x2 = lds32(a0 + 8 * G + 8);
            uint32_t y0 = lds32(a1 + 8 * G), y1 = lds32(a1 + 8 * G + 4), y2 = lds32(a1 + 8 * G + 8);
            uint32_t lo0 = __funnelshift_r(x0, x1, s0), hi0 = __funnelshift_r(x1, x2, s0);
            uint32_t lo1 = __funnelshift_r(y0, y1, s1), hi1 = __funnelshift_r(y1, y2, s1);
            uint2 g0 = s_grid[(lo0 >> (8 * ro.t)) & 0xFF], g1 = s_grid[(lo1 >> (8 * ro.t)) & 0xFF];
            // sign masks by arithmetic instead of a second table: the shared-memory pipe, not the ALU, is what
            // this format saturates (random 8-byte lookups conflict).  Seven stored sign bits, the eighth is
            // their parity; bit b of the byte -> 0xFF in byte b.
            auto sign_mask = [](uint32_t idx) {
                const uint32_t sg = idx | ((__popc(idx) & 1u) << 7);
                const uint32_t lo = ((sg & 0xFu) * 0x00204081u) & 0x01010101u;
                const uint32_t hi = ((sg >> 4) * 0x00204081u) & 0x01010101u;
                return make_uint2(lo * 0xFFu, hi * 0xFFu);
            };
            const uint2 k0 = sign_mask((hi0 >> (7 * ro.t)) & 127), k1 = sign_mask((hi1 >> (7 * ro.t)) & 127);
            // negate the bytes under the mask: (v ^ 0xFF) + 1; grid bytes are never 0, so no carry leaves a byte
            uint32_t a[4] = {(g0.x ^ k0.x) + (k0.x & 0x01010101u), (g1.x ^ k1.x) + (k1.x & 0x01010101u),
                             (g0.y ^ k0.y) + (k0.y & 0x01010101u), (g1.y ^ k1.y) + (k1.y & 0x01010101u)};
            mma_step(p, a, false);
            if (p == CH - 1) {
                // group scale (0.5 + s4) * 0.25 = (2*s4 + 1) / 8: the integer part here, 1/8 in the unit factor
                uint32_t sc[2][2];
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    uint32_t Gj = G - (CH - 1) + ro.col_p[j];
                    sc[j][0] = 2 * (u0[2 + 8 * Gj + 7] >> 4) + 1;
                    sc[j][1] = 2 * (u1[2 + 8 * Gj + 7] >> 4) + 1;
                }
                fold_int(sc);
            }
        }
        close_unit(f16_bits_to_f32(lds16(u0)) * 0.125f, f16_bits_to_f32(lds16(u1)) * 0.125f);
    } else if constexpr (TYPE == T_MXFP4) {
        // codes -> twice the E2M1 value by byte-permute lookups; sign picks between a positive and a negated table
        const uint32_t P0 = 0x03020100u, P1 = 0x0C080604u, N0 = 0xFDFEFF00u, N1 = 0xF4F8FAFCu;
        auto decode4 = [&](uint32_t w, uint32_t w4, uint32_t sel, uint32_t sign_sel) {
            uint32_t pos = prmt(P0, P1, sel & 0xFFFFu), neg = prmt(N0, N1, sel & 0xFFFFu);
            uint32_t sm = prmt(w, w4, sign_sel);  // 0xFF where the nibble's sign bit is set
            return (pos & ~sm) | (neg & sm);
        };
        // codes are doubled, so a block's scale is 2^(e-128); e = 255 zeroes the block, e <= 1 is subnormal
        auto block_scale = [&](uint32_t e) {
            return e == 255 ? 0.0f
                            : __uint_as_float(e > 1 ? (e - 1) << 23 : (e == 1 ? 0x00400000u : 0x00200000u));
        };
#pragma unroll
        for (int G = 0; G < 8; ++G) {
            const int p = G % CH;
            if (p == 0) {
                load_b(G, 0, false);
                zero_c();
            }
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
            mma_step(p, a, false);
            if (p == CH - 1) {
                float sc[2][2];
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    uint32_t Gj = G - (CH - 1) + ro.col_p[j];
                    sc[j][0] = block_scale(u0[17 * Gj]);
                    sc[j][1] = block_scale(u1[17 * Gj]);
                }
                fold_float(sc);
            }
        }
        close_unit(1.0f, 1.0f);
    } else if constexpr (TYPE == T_Q2_K) {
        // 16 groups of 16 values; word (sg, hf) of the 2-bit fields holds groups j = 2i + hf (shift 2i) of
        // super-group sg, which chain naturally.  m16n8k16: one A register per row, one B register.
        const uint32_t dd0 = lds32(u0 + 80), dd1 = lds32(u1 + 80);
#pragma unroll
        for (int sg = 0; sg < 2; ++sg) {
#pragma unroll
            for (int hf = 0; hf < 2; ++hf) {
                uint32_t q0 = lds32(u0 + 16 + 32 * sg + 16 * hf + 4 * ro.t);
                uint32_t q1 = lds32(u1 + 16 + 32 * sg + 16 * hf + 4 * ro.t);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int p = i % CH;
                    // 16-group j = 2i + hf of the super-group lives in 32-group 4sg + i (half hf) of the unit
                    if (p == 0) {
                        load_b(4 * sg + i, 16 * hf, true);
                        zero_c();
                    }
                    uint32_t a0 = (q0 >> (2 * i)) & 0x03030303u, a1 = (q1 >> (2 * i)) & 0x03030303u;
#pragma unroll
                    for (int h = 0; h < NH; ++h) mma_k16(c[h], a0, a1, ro.sup_p == p ? bsup[h].x : 0u);
                    if (p == CH - 1) {
                        uint32_t sc[2][2];
#pragma unroll
                        for (int j = 0; j < 2; ++j) {
                            uint32_t ij = i - (CH - 1) + ro.col_p[j];
                            sc[j][0] = u0[8 * sg + 2 * ij + hf] & 15;
                            sc[j][1] = u1[8 * sg + 2 * ij + hf] & 15;
                        }
                        fold_int(sc);
                    }
                }
            }
        }
        // minima: lane t takes 16-groups 4t .. 4t+3 of both rows
        const float dm0 = f16_bits_to_f32(dd0 >> 16), dm1 = f16_bits_to_f32(dd1 >> 16);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            uint32_t j16 = 4 * ro.t + e;  // 16-group of the unit; its 32-group is j16 / 2, half j16 & 1
            // scale byte of 16-group j16: super-group j16 / 8, group (j16 % 8) -> scales[j16]
            // value order inside a super-group is group-major, so 16-group j16 of the unit is scales[j16]
            float m0 = (float)(u0[j16] >> 4) * dm0, m1 = (float)(u1[j16] >> 4) * dm1;
#pragma unroll
            for (int b = 0; b < MB * NH; ++b) {
                float sx = ld_act<ACT>(act.sum16 + ((uint64_t)ro.brow[b] * act.n_groups + G0) * 2 + j16);
                minacc[b][0] = fmaf(m0, sx, minacc[b][0]);
                minacc[b][1] = fmaf(m1, sx, minacc[b][1]);
            }
        }
        close_unit(f16_bits_to_f32(dd0 & 0xFFFF), f16_bits_to_f32(dd1 & 0xFFFF));
    }
}

// ────────────────────────────── the kernel ────────────────────────────────
//
// Persistent: one CTA per SM walks row tiles blockIdx.x, blockIdx.x + gridDim.x, ...  Warp 0 produces
// (bulk copies into a ring of NS stages, each 16 rows x one K-chunk), warps 1..NCW consume (each takes
// every NCW-th unit of the chunk and keeps its partial sums in registers across the tile's chunks),
// warp NCW+1 reduces (adds the consumers' partial sums of a finished tile in a fixed order and stores
// dst) so that consumers move on to the next tile without waiting.  The activation planes of the whole
// product are copied to shared memory once per CTA when they fit.

struct SmemPlan {
    uint32_t row_stride;   // bytes between rows of a stage
    uint32_t n_stages;     // ring depth
    uint32_t act_bytes;    // activation region (0 = read activation planes from global memory)
    uint32_t total;        // dynamic shared memory of the launch
};

// Everything a launch needs.  A dense product is the single implicit job {expert 0, rows 0..m}.
struct GemvArgs {
    const uint8_t* w[2];        // weight bank; w[1] is the second bank of a SwiGLU pair (gate, up)
    uint64_t n;                 // rows of one expert's matrix (dense: all rows)
    uint64_t k;
    uint64_t expert_bytes;      // bytes between experts in a bank
    ActPlanes act;              // activation planes in global memory (ACT == 0)
    const float* x;             // f32 activation rows, split into planes inside the kernel (ACT == 1)
    uint32_t x_rows;            // rows of x to split (ACT == 1)
    uint32_t m;                 // dense: batch rows
    float* dst;                 // [activation list position, n]
    const MoeJob* jobs;         // grouped: device job list, else NULL
    const uint32_t* n_jobs;     // grouped: device count of jobs
    const uint32_t* act_rows;   // grouped: activation row of each list position (NULL = the position itself)
    float clamp;                // SwiGLU clamp (0 = off)
    int swiglu;                 // 1: tiles come in (gate, up) pairs and dst = silu(g) * u
    const float* norm_w;        // ACT == 1, dense: RMS-normalise every row of x with these k weights first
    float norm_eps;
    const float* residual;      // dense: dst = residual + product (may alias dst)
    SmemPlan plan;
    int* error_flag;
};

__device__ __forceinline__ float silu_f(float v) { return v / (1.0f + expf(-v)); }

// GROUPED == 0 is the dense product (one implicit job, one bank, plain store), 1 the dense SwiGLU pair
// (two banks, dst = silu(g) * u); the job list is compiled in only for GROUPED == 2.
template <uint32_t TYPE, int MB, int NH, int NCW, int ACT, int GROUPED>
__global__ void __launch_bounds__((NCW + 2) * 32, 1) gemv_mma_kernel(const __grid_constant__ GemvArgs ga) {
    using Tr = Traits<TYPE>;
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr int NB = MB * NH;                       // batch slots of a tile
    constexpr uint32_t RED_FLOATS = NCW * NB * ROWS;  // one reduction buffer
    const SmemPlan& plan = ga.plan;
    const uint32_t stage_bytes = ROWS * plan.row_stride;
    // layout: activation region | ring | tables (IQ2_XXS) | 2 reduction buffers | mbarriers
    uint8_t* s_act = smem;
    uint8_t* ring = smem + plan.act_bytes;
    uint2* s_grid = reinterpret_cast<uint2*>(ring + plan.n_stages * stage_bytes);
    uint2* s_mask = s_grid + (TYPE == T_IQ2_XXS ? 256 : 0);
    float* s_red = reinterpret_cast<float*>(s_mask + (TYPE == T_IQ2_XXS ? 128 : 0));
    uint64_t* full = reinterpret_cast<uint64_t*>(s_red + 2 * RED_FLOATS);
    uint64_t* empty = full + plan.n_stages;
    uint64_t* red_full = empty + plan.n_stages;
    uint64_t* red_empty = red_full + 2;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t NS = plan.n_stages;
    const uint64_t n = ga.n, k = ga.k;
    const uint32_t tiles_per_expert = (uint32_t)((n + ROWS - 1) / ROWS);
    const uint32_t units_per_row = (uint32_t)(k / 256);
    const uint64_t row_bytes = (uint64_t)units_per_row * Tr::UNIT_BYTES;
    const uint32_t n_chunks = (units_per_row + Tr::CHUNK_UNITS - 1) / Tr::CHUNK_UNITS;
    constexpr bool grouped = GROUPED == 2;
    const bool swiglu = GROUPED == 1 || (GROUPED == 2 && ga.swiglu);
    const uint32_t n_sub = swiglu ? 2 : 1;  // weight banks visited per tile
    const uint32_t n_groups = (uint32_t)(k / 32);

    if (tid == 0) {
        for (uint32_t s = 0; s < NS; ++s) {
            mbar_init(&full[s], ROWS);
            mbar_init(&empty[s], NCW);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&red_full[b], NCW);
            mbar_init(&red_empty[b], 1);
        }
        mbar_fence_init();
    }
    if (TYPE == T_IQ2_XXS) {
        for (int i = tid; i < 256; i += (NCW + 2) * 32) s_grid[i] = g_iq2xxs_grid[i];
        for (int i = tid; i < 128; i += (NCW + 2) * 32) {
            uint32_t sg = iq2_signs(i);
            uint32_t lo = ((sg & 0xF) * 0x00204081u) & 0x01010101u, hi = ((sg >> 4) * 0x00204081u) & 0x01010101u;
            s_mask[i] = make_uint2(lo * 0xFFu, hi * 0xFFu);
        }
    }
    __syncthreads();
    // From here on the three roles only meet through mbarriers.  Every wait is bounded; a role whose wait
    // runs out raises the error flag and leaves, and the roles that depend on it run out in turn.
    pdl_trigger();
    // A grouped launch learns its work from the kernel before it; a dense launch knows it already and may
    // prefetch weights at once.
    if (grouped || warp != 0) pdl_wait();
    if (ACT && warp != 0) {
        // Consumers and the reducer split the activations into planes in shared memory while the producer
        // fills the ring.
        __shared__ float s_tmp[(NCW + 1) * GEMV_MMA_MAX_M];
        split_activations<false, NCW + 1>(ga.x, ga.x_rows, (uint32_t)k, ga.norm_w, ga.norm_eps,
                                          TYPE, s_act, warp - 1, lane, s_tmp);
    }
    const uint32_t n_jobs = grouped ? __ldg(ga.n_jobs) : 1u;
    const uint32_t n_tiles = n_jobs * tiles_per_expert;
    // tile -> (job, row tile); the job gives the expert (weight offset) and the activation rows
    auto job_of = [&](uint32_t tile, uint32_t* rt) -> MoeJob {
        if (!grouped) {
            *rt = tile;
            return MoeJob{0u, 0u, ga.m};
        }
        uint32_t j = tile / tiles_per_expert;
        *rt = tile - j * tiles_per_expert;
        return ga.jobs[j];
    };
    // low four address bits of row `row` of expert `e` in bank `sub` (the offset of its bytes inside the
    // 16-byte aligned span that is copied)
    const uint32_t rb16 = (uint32_t)(row_bytes & 15), eb16 = (uint32_t)(ga.expert_bytes & 15);
    auto shift_of = [&](uint32_t sub, uint32_t e, uint32_t row) -> uint32_t {
        return ((uint32_t)(reinterpret_cast<uintptr_t>(ga.w[sub]) & 15) + e * eb16 + row * rb16) & 15;
    };

    if (warp == 0) {
        // ── producer ──
        if (lane < ROWS) {
            uint32_t job = 0;
            for (uint32_t tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
                uint32_t rt;
                const MoeJob jd = job_of(tile, &rt);
                uint64_t row = (uint64_t)rt * ROWS + lane < n ? (uint64_t)rt * ROWS + lane : n - 1;
                for (uint32_t sub = 0; sub < n_sub; ++sub) {
                    const uint8_t* wrow = ga.w[sub] + (uint64_t)jd.expert * ga.expert_bytes + row * row_bytes;
                    for (uint32_t chunk = 0; chunk < n_chunks; ++chunk, ++job) {
                        uint32_t s = job % NS, round = job / NS;
                        if (!mbar_wait(&empty[s], (round & 1) ^ 1)) {
                            *reinterpret_cast<volatile int*>(ga.error_flag) = 1;
                            return;
                        }
                        uint32_t u_lo = chunk * Tr::CHUNK_UNITS;
                        uint32_t u_hi = min(units_per_row, u_lo + Tr::CHUNK_UNITS);
                        uintptr_t beg = reinterpret_cast<uintptr_t>(wrow) + (uint64_t)u_lo * Tr::UNIT_BYTES;
                        uintptr_t end = beg + (uint64_t)(u_hi - u_lo) * Tr::UNIT_BYTES;
                        uintptr_t abeg = beg & ~(uintptr_t)15, aend = (end + 15) & ~(uintptr_t)15;
                        uint32_t bytes = (uint32_t)(aend - abeg);
                        mbar_arrive_expect_tx(&full[s], bytes);
                        bulk_g2s(ring + s * stage_bytes + lane * plan.row_stride,
                                 reinterpret_cast<const void*>(abeg), bytes, &full[s]);
                    }
                }
            }
        }
    } else if (warp <= NCW) {
        // ── consumers ──
        const int cw = warp - 1;
        Roles<MB, NH> ro(lane);
        if (TYPE == T_Q4_K && MB == 1) {
            // two groups per chain: held column j only ever sees odd (high-nibble, 16x) or even groups
#pragma unroll
            for (int j = 0; j < 2; ++j)
                if (ro.col_p[j] & 1) ro.col_w[j] *= 0.0625f;
        }
        ActPlanes a = ga.act;
        if (ACT) {
            const uint64_t groups = (uint64_t)ga.x_rows * n_groups;
            a.planes = reinterpret_cast<const int8_t*>(s_act);
            a.meta = reinterpret_cast<const float2*>(s_act + groups * 96);
            a.sum16 = reinterpret_cast<const float*>(s_act + groups * 104);
        }
        a.n_groups = n_groups;
        float colacc[NH][2][2], minacc[NB][2];
        uint32_t job = 0, red_it = 0;
        for (uint32_t tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
            uint32_t rt;
            const MoeJob jd = job_of(tile, &rt);
            if (grouped || tile == blockIdx.x) ro.set_rows(jd.row0, jd.cnt, ga.act_rows, n_groups);
            const uint64_t row0 = (uint64_t)rt * ROWS;
            for (uint32_t sub = 0; sub < n_sub; ++sub, ++red_it) {
#pragma unroll
                for (int h = 0; h < NH; ++h)
#pragma unroll
                    for (int j = 0; j < 2; ++j) colacc[h][j][0] = colacc[h][j][1] = 0.0f;
#pragma unroll
                for (int b = 0; b < NB; ++b) minacc[b][0] = minacc[b][1] = 0.0f;
                // byte offset of a row's first unit inside its 16-byte aligned span (the same for every
                // chunk: chunk starts are multiples of 16 bytes for every format)
                const uint32_t r0c = (uint32_t)min(row0 + ro.g, n - 1), r1c = (uint32_t)min(row0 + ro.g + 8, n - 1);
                const uint32_t sh0 = shift_of(sub, jd.expert, r0c), sh1 = shift_of(sub, jd.expert, r1c);
                for (uint32_t chunk = 0; chunk < n_chunks; ++chunk, ++job) {
                    uint32_t s = job % NS, round = job / NS;
                    if (!mbar_wait(&full[s], round & 1)) {
                        if (lane == 0) *reinterpret_cast<volatile int*>(ga.error_flag) = 1;
                        return;
                    }
                    const uint8_t* st = ring + s * stage_bytes;
                    const uint32_t u_lo = chunk * Tr::CHUNK_UNITS;
                    const uint32_t cnt = min(units_per_row - u_lo, Tr::CHUNK_UNITS);
                    for (uint32_t u = cw; u < cnt; u += NCW) {
                        const uint8_t* u0 = st + ro.g * plan.row_stride + sh0 + u * Tr::UNIT_BYTES;
                        const uint8_t* u1 = st + (ro.g + 8) * plan.row_stride + sh1 + u * Tr::UNIT_BYTES;
                        process_unit<TYPE, MB, NH, ACT>(u0, u1, u_lo + u, a, ro, s_grid, s_mask, colacc, minacc);
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&empty[s]);
                }
                // hand the partial sums to the reducer: per batch slot, the held columns that belong to it
                // minus its minima terms, summed over the quad
                const uint32_t rb = red_it & 1;
                if (!mbar_wait(&red_empty[rb], ((red_it >> 1) & 1) ^ 1)) {
                    if (lane == 0) *reinterpret_cast<volatile int*>(ga.error_flag) = 1;
                    return;
                }
                float* red = s_red + rb * RED_FLOATS;
#pragma unroll
                for (int b = 0; b < NB; ++b) {
                    const int h = b / MB, i = b % MB;
#pragma unroll
                    for (int r = 0; r < 2; ++r) {
                        float v = -minacc[b][r];
#pragma unroll
                        for (int j = 0; j < 2; ++j) v += ro.col_i[j] == i ? colacc[h][j][r] : 0.0f;
                        v += __shfl_xor_sync(0xFFFFFFFFu, v, 1);
                        v += __shfl_xor_sync(0xFFFFFFFFu, v, 2);
                        if (ro.t == 0) red[(cw * NB + b) * ROWS + ro.g + 8 * r] = v;
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&red_full[rb]);
            }
        }
    } else {
        // ── reducer ──
        constexpr int PER_LANE = (NB * ROWS + 31) / 32;
        float gate[PER_LANE];
        uint32_t red_it = 0;
        for (uint32_t tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
            uint32_t rt;
            const MoeJob jd = job_of(tile, &rt);
            const uint64_t row0 = (uint64_t)rt * ROWS;
            for (uint32_t sub = 0; sub < n_sub; ++sub, ++red_it) {
                const uint32_t rb = red_it & 1;
                if (!mbar_wait(&red_full[rb], (red_it >> 1) & 1)) {
                    if (lane == 0) *reinterpret_cast<volatile int*>(ga.error_flag) = 1;
                    return;
                }
                const float* red = s_red + rb * RED_FLOATS;
#pragma unroll
                for (int q = 0; q < PER_LANE; ++q) {
                    const int o = lane + 32 * q;
                    if (o < NB * ROWS) {
                        const int r = o % ROWS;
                        const uint32_t b = o / ROWS;
                        float v = 0.0f;
#pragma unroll
                        for (int cwv = 0; cwv < NCW; ++cwv) v += red[(cwv * NB + (int)b) * ROWS + r];
                        if (swiglu && sub == 0) {
                            gate[q] = v;
                        } else if (b < jd.cnt && row0 + r < n) {
                            if (swiglu) {
                                float gv = gate[q], uv = v;
                                if (ga.clamp > 0.0f) {
                                    gv = fminf(gv, ga.clamp);
                                    uv = fmaxf(-ga.clamp, fminf(uv, ga.clamp));
                                }
                                v = silu_f(gv) * uv;
                            }
                            const uint64_t o_idx = (uint64_t)(jd.row0 + b) * n + row0 + r;
                            if (GROUPED != 2 && ga.residual != nullptr) v += ga.residual[o_idx];
                            ga.dst[o_idx] = v;
                        }
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&red_empty[rb]);
            }
        }
    }
}

// ───────────────────────── narrow-K grouped variant ───────────────────────
//
// Expert matrices are small: with k = 768 a row is three units, so in the kernel above three consumer warps
// would work and thirteen would wait.  Here a ring stage holds T = NCW / units_per_row consecutive 16-row
// tiles of one job, whole rows at a time, and consumer warp c takes unit c % units_per_row of tile
// c / units_per_row, so (almost) every warp has a unit.  A stage is a complete product for its T tiles: the
// partial sums go to the reducer after every stage, which adds each tile's units_per_row partials in unit
// order.  Grouped (job list) launches only, 2 <= units_per_row <= 8.
template <uint32_t TYPE, int MB, int NH, int ACT>
__global__ void __launch_bounds__((16 + 2) * 32, 1) gemv_narrow_kernel(const __grid_constant__ GemvArgs ga) {
    using Tr = Traits<TYPE>;
    constexpr int NCW = 16;
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr int NB = MB * NH;
    constexpr uint32_t RED_FLOATS = NCW * NB * ROWS;
    const SmemPlan& plan = ga.plan;
    const uint64_t n = ga.n, k = ga.k;
    const uint32_t upr = (uint32_t)(k / 256);        // units per row = consumer warps per tile
    const uint32_t T = NCW / upr;                    // tiles per stage
    const uint32_t stage_bytes = T * ROWS * plan.row_stride;
    uint8_t* s_act = smem;
    uint8_t* ring = smem + plan.act_bytes;
    uint2* s_grid = reinterpret_cast<uint2*>(ring + plan.n_stages * stage_bytes);
    uint2* s_mask = s_grid + (TYPE == T_IQ2_XXS ? 256 : 0);
    float* s_red = reinterpret_cast<float*>(s_mask + (TYPE == T_IQ2_XXS ? 128 : 0));
    uint64_t* full = reinterpret_cast<uint64_t*>(s_red + 2 * RED_FLOATS);
    uint64_t* empty = full + plan.n_stages;
    uint64_t* red_full = empty + plan.n_stages;
    uint64_t* red_empty = red_full + 2;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t NS = plan.n_stages;
    const uint32_t tiles_per_expert = (uint32_t)((n + ROWS - 1) / ROWS);
    const uint32_t st_per_expert = (tiles_per_expert + T - 1) / T;
    const uint64_t row_bytes = (uint64_t)upr * Tr::UNIT_BYTES;
    const bool swiglu = ga.swiglu != 0;
    const uint32_t n_sub = swiglu ? 2 : 1;
    const uint32_t n_groups = (uint32_t)(k / 32);

    if (tid == 0) {
        for (uint32_t s = 0; s < NS; ++s) {
            mbar_init(&full[s], ROWS);
            mbar_init(&empty[s], NCW);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&red_full[b], NCW);
            mbar_init(&red_empty[b], 1);
        }
        mbar_fence_init();
    }
    if (TYPE == T_IQ2_XXS) {
        for (int i = tid; i < 256; i += (NCW + 2) * 32) s_grid[i] = g_iq2xxs_grid[i];
        for (int i = tid; i < 128; i += (NCW + 2) * 32) {
            uint32_t sg = iq2_signs(i);
            uint32_t lo = ((sg & 0xF) * 0x00204081u) & 0x01010101u, hi = ((sg >> 4) * 0x00204081u) & 0x01010101u;
            s_mask[i] = make_uint2(lo * 0xFFu, hi * 0xFFu);
        }
    }
    __syncthreads();
    pdl_trigger();
    pdl_wait();  // the job list comes from the kernel before this one
    if (ACT && warp != 0) {
        __shared__ float s_tmp[(NCW + 1) * GEMV_MMA_MAX_M];
        split_activations<false, NCW + 1>(ga.x, ga.x_rows, (uint32_t)k, ga.norm_w, ga.norm_eps, TYPE, s_act, warp - 1,
                                          lane, s_tmp);
    }
    const uint32_t n_st = __ldg(ga.n_jobs) * st_per_expert;
    const uint32_t rb16 = (uint32_t)(row_bytes & 15), eb16 = (uint32_t)(ga.expert_bytes & 15);
    auto shift_of = [&](uint32_t sub, uint32_t e, uint32_t row) -> uint32_t {
        return ((uint32_t)(reinterpret_cast<uintptr_t>(ga.w[sub]) & 15) + e * eb16 + row * rb16) & 15;
    };

    if (warp == 0) {
        // ── producer: lane l copies row l of each of the stage's tiles ──
        if (lane < ROWS) {
            uint32_t job = 0;
            for (uint32_t st = blockIdx.x; st < n_st; st += gridDim.x) {
                const uint32_t j = st / st_per_expert, rt0 = (st - j * st_per_expert) * T;
                const MoeJob jd = ga.jobs[j];
                const uint32_t nt = min(T, tiles_per_expert - rt0);
                for (uint32_t sub = 0; sub < n_sub; ++sub, ++job) {
                    const uint32_t s = job % NS, round = job / NS;
                    if (!mbar_wait(&empty[s], (round & 1) ^ 1)) {
                        *reinterpret_cast<volatile int*>(ga.error_flag) = 1;
                        return;
                    }
                    const uint8_t* wbase = ga.w[sub] + (uint64_t)jd.expert * ga.expert_bytes;
                    uint32_t total = 0;
                    for (uint32_t ti = 0; ti < nt; ++ti) {
                        uint64_t row = (uint64_t)(rt0 + ti) * ROWS + lane;
                        row = row < n ? row : n - 1;
                        uintptr_t beg = reinterpret_cast<uintptr_t>(wbase + row * row_bytes), end = beg + row_bytes;
                        total += (uint32_t)(((end + 15) & ~(uintptr_t)15) - (beg & ~(uintptr_t)15));
                    }
                    mbar_arrive_expect_tx(&full[s], total);
                    for (uint32_t ti = 0; ti < nt; ++ti) {
                        uint64_t row = (uint64_t)(rt0 + ti) * ROWS + lane;
                        row = row < n ? row : n - 1;
                        uintptr_t beg = reinterpret_cast<uintptr_t>(wbase + row * row_bytes), end = beg + row_bytes;
                        uintptr_t abeg = beg & ~(uintptr_t)15, aend = (end + 15) & ~(uintptr_t)15;
                        bulk_g2s(ring + s * stage_bytes + (ti * ROWS + lane) * plan.row_stride,
                                 reinterpret_cast<const void*>(abeg), (uint32_t)(aend - abeg), &full[s]);
                    }
                }
            }
        }
    } else if (warp <= NCW) {
        // ── consumers: warp c -> (tile c / upr of the stage, unit c % upr) ──
        const uint32_t cw = warp - 1, ti = cw / upr, u = cw - ti * upr;
        Roles<MB, NH> ro(lane);
        if (TYPE == T_Q4_K && MB == 1) {
#pragma unroll
            for (int j = 0; j < 2; ++j)
                if (ro.col_p[j] & 1) ro.col_w[j] *= 0.0625f;
        }
        ActPlanes a = ga.act;
        if (ACT) {
            const uint64_t groups = (uint64_t)ga.x_rows * n_groups;
            a.planes = reinterpret_cast<const int8_t*>(s_act);
            a.meta = reinterpret_cast<const float2*>(s_act + groups * 96);
            a.sum16 = reinterpret_cast<const float*>(s_act + groups * 104);
        }
        a.n_groups = n_groups;
        float colacc[NH][2][2], minacc[NB][2];
        uint32_t job = 0;
        for (uint32_t st = blockIdx.x; st < n_st; st += gridDim.x) {
            const uint32_t j = st / st_per_expert, rt0 = (st - j * st_per_expert) * T;
            const MoeJob jd = ga.jobs[j];
            const uint32_t nt = min(T, tiles_per_expert - rt0);
            const bool active = ti < nt;
            ro.set_rows(jd.row0, jd.cnt, ga.act_rows, n_groups);
            const uint64_t row0 = (uint64_t)(rt0 + ti) * ROWS;
            for (uint32_t sub = 0; sub < n_sub; ++sub, ++job) {
#pragma unroll
                for (int h = 0; h < NH; ++h)
#pragma unroll
                    for (int jj = 0; jj < 2; ++jj) colacc[h][jj][0] = colacc[h][jj][1] = 0.0f;
#pragma unroll
                for (int b = 0; b < NB; ++b) minacc[b][0] = minacc[b][1] = 0.0f;
                const uint32_t s = job % NS, round = job / NS;
                if (!mbar_wait(&full[s], round & 1)) {
                    if (lane == 0) *reinterpret_cast<volatile int*>(ga.error_flag) = 1;
                    return;
                }
                if (active) {
                    const uint32_t r0c = (uint32_t)min(row0 + ro.g, n - 1), r1c = (uint32_t)min(row0 + ro.g + 8, n - 1);
                    const uint32_t sh0 = shift_of(sub, jd.expert, r0c), sh1 = shift_of(sub, jd.expert, r1c);
                    const uint8_t* sp = ring + s * stage_bytes + ti * ROWS * plan.row_stride;
                    const uint8_t* u0 = sp + ro.g * plan.row_stride + sh0 + u * Tr::UNIT_BYTES;
                    const uint8_t* u1 = sp + (ro.g + 8) * plan.row_stride + sh1 + u * Tr::UNIT_BYTES;
                    process_unit<TYPE, MB, NH, ACT>(u0, u1, u, a, ro, s_grid, s_mask, colacc, minacc);
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&empty[s]);
                const uint32_t rb = job & 1;
                if (!mbar_wait(&red_empty[rb], ((job >> 1) & 1) ^ 1)) {
                    if (lane == 0) *reinterpret_cast<volatile int*>(ga.error_flag) = 1;
                    return;
                }
                float* red = s_red + rb * RED_FLOATS;
#pragma unroll
                for (int b = 0; b < NB; ++b) {
                    const int h = b / MB, i = b % MB;
#pragma unroll
                    for (int r = 0; r < 2; ++r) {
                        float v = -minacc[b][r];
#pragma unroll
                        for (int jj = 0; jj < 2; ++jj) v += ro.col_i[jj] == i ? colacc[h][jj][r] : 0.0f;
                        v += __shfl_xor_sync(0xFFFFFFFFu, v, 1);
                        v += __shfl_xor_sync(0xFFFFFFFFu, v, 2);
                        if (ro.t == 0) red[(cw * NB + b) * ROWS + ro.g + 8 * r] = active ? v : 0.0f;
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&red_full[rb]);
            }
        }
    } else {
        // ── reducer: per stage, each tile's partials in unit order ──
        constexpr int PER_LANE = (8 * NB * ROWS + 31) / 32;  // T <= 8
        float gate[PER_LANE];
        uint32_t job = 0;
        for (uint32_t st = blockIdx.x; st < n_st; st += gridDim.x) {
            const uint32_t j = st / st_per_expert, rt0 = (st - j * st_per_expert) * T;
            const MoeJob jd = ga.jobs[j];
            const uint32_t nt = min(T, tiles_per_expert - rt0);
            for (uint32_t sub = 0; sub < n_sub; ++sub, ++job) {
                const uint32_t rb = job & 1;
                if (!mbar_wait(&red_full[rb], (job >> 1) & 1)) {
                    if (lane == 0) *reinterpret_cast<volatile int*>(ga.error_flag) = 1;
                    return;
                }
                const float* red = s_red + rb * RED_FLOATS;
#pragma unroll
                for (int q = 0; q < PER_LANE; ++q) {
                    const uint32_t o = lane + 32 * q;
                    if (o < T * NB * ROWS) {
                        const uint32_t tt = o / (NB * ROWS), rem = o - tt * (NB * ROWS);
                        const uint32_t b = rem / ROWS, r = rem - b * ROWS;
                        float v = 0.0f;
                        for (uint32_t uu = 0; uu < upr; ++uu) v += red[((tt * upr + uu) * NB + b) * ROWS + r];
                        const uint64_t orow = (uint64_t)(rt0 + tt) * ROWS + r;
                        if (swiglu && sub == 0) {
                            gate[q] = v;
                        } else if (tt < nt && b < jd.cnt && orow < n) {
                            if (swiglu) {
                                float gv = gate[q], uv = v;
                                if (ga.clamp > 0.0f) {
                                    gv = fminf(gv, ga.clamp);
                                    uv = fmaxf(-ga.clamp, fminf(uv, ga.clamp));
                                }
                                v = silu_f(gv) * uv;
                            }
                            ga.dst[(uint64_t)(jd.row0 + b) * n + orow] = v;
                        }
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&red_empty[rb]);
            }
        }
    }
}

constexpr uint32_t SMEM_BUDGET = 220 * 1024;  // of the 227 KB a CTA may use
constexpr uint32_t ACT_SMEM_MAX = 96 * 1024;  // measured: 116 KB (8 rows of k = 4096 in shared memory, two ring stages left) is slower than planes in global memory with a deeper ring

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

template <uint32_t TYPE, int NCW, int NB>
SmemPlan plan_smem(uint64_t k, uint64_t act_rows_in_smem, uint64_t jobs_per_cta) {
    using Tr = Traits<TYPE>;
    SmemPlan p;
    p.row_stride = row_stride_for<TYPE>(k);
    uint32_t fixed = (TYPE == T_IQ2_XXS ? (256 + 128) * 8 : 0) + 2 * NCW * NB * ROWS * 4 + 8 * (2 * 8 + 4) + 128;
    p.act_bytes = (uint32_t)(act_rows_in_smem * (k / 32) * 112);
    uint32_t stage = ROWS * p.row_stride;
    uint32_t room = SMEM_BUDGET - fixed - p.act_bytes;
    uint32_t n_chunks = (uint32_t)((k / 256 + Tr::CHUNK_UNITS - 1) / Tr::CHUNK_UNITS);
    uint64_t jobs = std::max<uint64_t>(1, jobs_per_cta) * n_chunks;
    p.n_stages = (uint32_t)std::max<uint64_t>(1, std::min<uint64_t>({(uint64_t)8, (uint64_t)(room / stage), jobs}));
    p.total = p.act_bytes + p.n_stages * stage + fixed;
    return p;
}

template <uint32_t TYPE, int MB, int NH, int ACT, int GROUPED>
cudaError_t launch_variant(GemvArgs& ga, uint64_t max_tiles, cudaStream_t s) {
    constexpr int NCW = 16;
    const int g_num_sms = num_sms();
    unsigned grid = (unsigned)std::max<uint64_t>(1, std::min<uint64_t>(max_tiles, (uint64_t)g_num_sms));
    uint64_t per_cta = (max_tiles + grid - 1) / grid * (ga.swiglu ? 2 : 1);
    ga.plan = plan_smem<TYPE, NCW, MB * NH>(ga.k, ACT ? ga.x_rows : 0, per_cta);
    auto kern = gemv_mma_kernel<TYPE, MB, NH, NCW, ACT, GROUPED>;
    static bool configured[MAX_DEVICES] = {};  // per instantiation and device
    if (cudaError_t ce = set_max_smem_once(kern, (int)SMEM_BUDGET, configured); ce != cudaSuccess) return ce;
    cudaError_t e = launch_pdl(kern, grid, (NCW + 2) * 32, ga.plan.total, s, ga);
    return e != cudaSuccess ? e : cudaGetLastError();
}

// rows_per_job: the largest number of batch rows one tile carries (dense: m)
template <uint32_t TYPE, int ACT, int GROUPED>
cudaError_t launch_rows(GemvArgs& ga, uint32_t rows_per_job, uint64_t max_tiles, cudaStream_t s) {
    if (rows_per_job == 1) return launch_variant<TYPE, 1, 1, ACT, GROUPED>(ga, max_tiles, s);
    if (rows_per_job == 2) return launch_variant<TYPE, 2, 1, ACT, GROUPED>(ga, max_tiles, s);
    if (rows_per_job <= 4) return launch_variant<TYPE, 2, 2, ACT, GROUPED>(ga, max_tiles, s);
    if (rows_per_job <= 8) return launch_variant<TYPE, 2, 4, ACT, GROUPED>(ga, max_tiles, s);
    return cudaErrorInvalidValue;
}

template <int ACT, int GROUPED>
cudaError_t launch_typed(uint32_t type, GemvArgs& ga, uint32_t rows_per_job, uint64_t max_tiles, cudaStream_t s) {
    switch (type) {
        case T_Q4_K: return launch_rows<T_Q4_K, ACT, GROUPED>(ga, rows_per_job, max_tiles, s);
        case T_Q8_0: return launch_rows<T_Q8_0, ACT, GROUPED>(ga, rows_per_job, max_tiles, s);
        case T_Q2_K: return launch_rows<T_Q2_K, ACT, GROUPED>(ga, rows_per_job, max_tiles, s);
        case T_IQ2_XXS: return launch_rows<T_IQ2_XXS, ACT, GROUPED>(ga, rows_per_job, max_tiles, s);
        case T_MXFP4: return launch_rows<T_MXFP4, ACT, GROUPED>(ga, rows_per_job, max_tiles, s);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace

// Activation planes live in the kernel's shared memory when they fit; only larger products need scratch.
static bool acts_fit_in_smem(uint64_t rows, uint64_t k) { return rows * (k / 32) * 112 <= ACT_SMEM_MAX; }

size_t gemv_mma_scratch_bytes(uint64_t rows, uint64_t k) {
    if (acts_fit_in_smem(rows, k)) return 0;
    uint64_t groups = rows * (k / 32);
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

static ActPlanes planes_in(void* scratch, uint64_t rows, uint64_t k) {
    uint64_t groups = rows * (k / 32);
    ActPlanes act;
    int8_t* planes = static_cast<int8_t*>(scratch);
    act.planes = planes;
    act.meta = reinterpret_cast<float2*>(planes + groups * 96);
    act.sum16 = reinterpret_cast<float*>(planes + groups * 104);
    act.n_groups = (uint32_t)(k / 32);
    return act;
}

cudaError_t launch_quantize_acts(uint32_t type, const float* x, uint64_t rows, uint64_t k, void* scratch,
                                 cudaStream_t s) {
    ActPlanes act = planes_in(scratch, rows, k);
    unsigned qgrid = (unsigned)std::max<uint64_t>(1, std::min<uint64_t>(rows * (k / 256), 148 * 8));
    return launch_pdl(quantize_acts_kernel, qgrid, 256, 0, s, x, rows, k, type, const_cast<int8_t*>(act.planes),
                      const_cast<float2*>(act.meta), const_cast<float*>(act.sum16));
}

bool gemv_mma_fusable(uint64_t m, uint64_t k) { return m <= GEMV_MMA_MAX_M && acts_fit_in_smem(m, k); }

// dst = residual + rmsnorm(lhs; norm_w, eps) . W^T in one launch; norm_w and residual are optional.
cudaError_t launch_gemv_mma_fused(uint32_t type, const uint8_t* w, uint64_t n, uint64_t k, const float* lhs,
                                  uint64_t m, float* dst, const float* norm_w, float eps, const float* residual,
                                  int* error_flag, cudaStream_t s) {
    if (!gemv_mma_fusable(m, k)) return cudaErrorInvalidValue;
    GemvArgs ga = {};
    ga.w[0] = ga.w[1] = w;
    ga.n = n;
    ga.k = k;
    ga.x = lhs;
    ga.x_rows = (uint32_t)m;
    ga.m = (uint32_t)m;
    ga.dst = dst;
    ga.norm_w = norm_w;
    ga.norm_eps = eps;
    ga.residual = residual;
    ga.error_flag = error_flag;
    return launch_typed<1, 0>(type, ga, (uint32_t)m, (n + ROWS - 1) / ROWS, s);
}

cudaError_t launch_gemv_mma(uint32_t type, const uint8_t* w, uint64_t n, uint64_t k, const float* lhs, uint64_t m,
                            float* dst, void* scratch, int* error_flag, cudaStream_t s) {
    GemvArgs ga = {};
    ga.w[0] = ga.w[1] = w;
    ga.n = n;
    ga.k = k;
    ga.x = lhs;
    ga.x_rows = (uint32_t)m;
    ga.m = (uint32_t)m;
    ga.dst = dst;
    ga.error_flag = error_flag;
    uint64_t tiles = (n + ROWS - 1) / ROWS;
    if (acts_fit_in_smem(m, k)) return launch_typed<1, 0>(type, ga, (uint32_t)m, tiles, s);
    cudaError_t e = launch_quantize_acts(type, lhs, m, k, scratch, s);
    if (e != cudaSuccess) return e;
    ga.act = planes_in(scratch, m, k);
    return launch_typed<0, 0>(type, ga, (uint32_t)m, tiles, s);
}

// silu(clamp(gate x)) * clamp(up x) in one launch (activation planes in shared memory only)
cudaError_t launch_gemv_mma_swiglu(uint32_t type, const uint8_t* w_gate, const uint8_t* w_up, uint64_t n, uint64_t k,
                                   const float* lhs, uint64_t m, float* dst, float clamp, int* error_flag,
                                   cudaStream_t s, const float* norm_w, float eps) {
    if (!acts_fit_in_smem(m, k)) return cudaErrorInvalidValue;
    GemvArgs ga = {};
    ga.w[0] = w_gate;
    ga.w[1] = w_up;
    ga.n = n;
    ga.k = k;
    ga.x = lhs;
    ga.x_rows = (uint32_t)m;
    ga.m = (uint32_t)m;
    ga.dst = dst;
    ga.clamp = clamp;
    ga.swiglu = 1;
    ga.norm_w = norm_w;
    ga.norm_eps = eps;
    ga.error_flag = error_flag;
    return launch_typed<1, 1>(type, ga, (uint32_t)m, (n + ROWS - 1) / ROWS, s);
}

// ── the allocation-free variant ──────────────────────────────────────────────────────────────────────
//
// Same product as launch_gemv_mma on its scratch path (activation planes written to global memory by
// quantize_acts_kernel, then read by the matmul kernel), but the planes live in a fixed array that is part
// of the library image instead of a buffer from cudaMalloc.  Every GPU that loads the library carries these
// 4 MiB until the process exits.  All calls on a device share the array, and it keeps whatever the last
// call left there; nothing in it has to start at zero, because the first kernel of a call rewrites every
// byte the second one reads.  Two calls whose kernels overlap on the GPU (different streams, or the same
// call issued from two threads) would overwrite each other's planes.
static __device__ __align__(256) unsigned char g_static_planes[GEMV_STATIC_SCRATCH_BYTES];

// The array's name is only a handle on the host side; the device address has to be asked for, once per
// device and with that device current.
static void* g_static_planes_addr[64];

cudaError_t gemv_mma_static_setup(void** addr) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    if (g_static_planes_addr[dev] == nullptr) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_static_planes);
        if (e != cudaSuccess) return e;
        if (p == nullptr) return cudaErrorInvalidSymbol;
        g_static_planes_addr[dev] = p;
    }
    *addr = g_static_planes_addr[dev];
    return cudaSuccess;
}

size_t gemv_mma_static_bytes_needed(uint64_t m, uint64_t k) { return (size_t)(m * (k / 32) * 112 + 256); }

cudaError_t launch_gemv_mma_static(uint32_t type, const uint8_t* w, uint64_t n, uint64_t k, const float* lhs,
                                   uint64_t m, float* dst, int* error_flag, cudaStream_t s) {
    if (m == 0 || m > GEMV_MMA_MAX_M || k % 256 != 0 || gemv_mma_static_bytes_needed(m, k) > GEMV_STATIC_SCRATCH_BYTES)
        return cudaErrorInvalidValue;  // the planes would not fit the fixed array
    void* planes = nullptr;
    cudaError_t e = gemv_mma_static_setup(&planes);
    if (e != cudaSuccess) return e;
    e = launch_quantize_acts(type, lhs, m, k, planes, s);
    if (e != cudaSuccess) return e;
    GemvArgs ga = {};
    ga.w[0] = ga.w[1] = w;
    ga.n = n;
    ga.k = k;
    ga.x = lhs;
    ga.x_rows = (uint32_t)m;
    ga.m = (uint32_t)m;
    ga.dst = dst;
    ga.error_flag = error_flag;
    ga.act = planes_in(planes, m, k);
    return launch_typed<0, 0>(type, ga, (uint32_t)m, (n + ROWS - 1) / ROWS, s);
}

// ── narrow-K grouped launch ─────────────────────────────────────────────────────────────────────────
namespace {

template <uint32_t TYPE, int MB, int NH, int ACT>
cudaError_t launch_narrow_variant(GemvArgs& ga, uint32_t max_jobs, cudaStream_t s) {
    using Tr = Traits<TYPE>;
    constexpr int NCW = 16;
    const int g_num_sms = num_sms();
    const uint32_t upr = (uint32_t)(ga.k / 256), T = NCW / upr;
    const uint32_t tiles = (uint32_t)((ga.n + ROWS - 1) / ROWS), spe = (tiles + T - 1) / T;
    const uint64_t n_st = (uint64_t)max_jobs * spe;
    SmemPlan p;
    p.row_stride = row_stride_for<TYPE>(ga.k);
    const uint32_t fixed = (TYPE == T_IQ2_XXS ? (256 + 128) * 8 : 0) + 2 * NCW * MB * NH * ROWS * 4 + 8 * (2 * 8 + 4) + 128;
    p.act_bytes = ACT ? (uint32_t)((uint64_t)ga.x_rows * (ga.k / 32) * 112) : 0;
    const uint32_t stage = T * ROWS * p.row_stride;
    if (fixed + p.act_bytes + stage > SMEM_BUDGET) return cudaErrorInvalidValue;
    unsigned grid = (unsigned)std::max<uint64_t>(1, std::min<uint64_t>(n_st, (uint64_t)g_num_sms));
    const uint64_t per_cta = (n_st + grid - 1) / grid * (ga.swiglu ? 2 : 1);
    p.n_stages = (uint32_t)std::max<uint64_t>(1, std::min<uint64_t>({(uint64_t)8, (uint64_t)((SMEM_BUDGET - fixed - p.act_bytes) / stage), per_cta}));
    p.total = p.act_bytes + p.n_stages * stage + fixed;
    ga.plan = p;
    (void)sizeof(Tr);
    auto kern = gemv_narrow_kernel<TYPE, MB, NH, ACT>;
    static bool configured[MAX_DEVICES] = {};
    if (cudaError_t ce = set_max_smem_once(kern, (int)SMEM_BUDGET, configured); ce != cudaSuccess) return ce;
    cudaError_t e = launch_pdl(kern, grid, (NCW + 2) * 32, p.total, s, ga);
    return e != cudaSuccess ? e : cudaGetLastError();
}

template <uint32_t TYPE, int ACT>
cudaError_t launch_narrow_rows(GemvArgs& ga, uint32_t rows_per_job, uint32_t max_jobs, cudaStream_t s) {
    if (rows_per_job == 1) return launch_narrow_variant<TYPE, 1, 1, ACT>(ga, max_jobs, s);
    if (rows_per_job == 2) return launch_narrow_variant<TYPE, 2, 1, ACT>(ga, max_jobs, s);
    if (rows_per_job <= 4) return launch_narrow_variant<TYPE, 2, 2, ACT>(ga, max_jobs, s);
    if (rows_per_job <= 8) return launch_narrow_variant<TYPE, 2, 4, ACT>(ga, max_jobs, s);
    return cudaErrorInvalidValue;
}

template <int ACT>
cudaError_t launch_narrow_typed(uint32_t type, GemvArgs& ga, uint32_t rows_per_job, uint32_t max_jobs, cudaStream_t s) {
    switch (type) {
        case T_Q4_K: return launch_narrow_rows<T_Q4_K, ACT>(ga, rows_per_job, max_jobs, s);
        case T_Q8_0: return launch_narrow_rows<T_Q8_0, ACT>(ga, rows_per_job, max_jobs, s);
        case T_Q2_K: return launch_narrow_rows<T_Q2_K, ACT>(ga, rows_per_job, max_jobs, s);
        case T_IQ2_XXS: return launch_narrow_rows<T_IQ2_XXS, ACT>(ga, rows_per_job, max_jobs, s);
        case T_MXFP4: return launch_narrow_rows<T_MXFP4, ACT>(ga, rows_per_job, max_jobs, s);
        default: return cudaErrorInvalidValue;
    }
}

// units per row the narrow kernel takes: at least two tiles per stage, and one chunk per row
bool narrow_k(uint32_t type, uint64_t k) {
    const uint64_t upr = k / 256;
    uint32_t chunk = 8;
    switch (type) {
        case T_Q4_K: chunk = Traits<T_Q4_K>::CHUNK_UNITS; break;
        case T_Q8_0: chunk = Traits<T_Q8_0>::CHUNK_UNITS; break;
        case T_Q2_K: chunk = Traits<T_Q2_K>::CHUNK_UNITS; break;
        case T_IQ2_XXS: chunk = Traits<T_IQ2_XXS>::CHUNK_UNITS; break;
        case T_MXFP4: chunk = Traits<T_MXFP4>::CHUNK_UNITS; break;
    }
    return upr >= 2 && upr <= 8 && upr <= chunk;
}

}  // namespace

cudaError_t launch_gemv_grouped(const GroupedLaunch& g, cudaStream_t s) {
    GemvArgs ga = {};
    ga.w[0] = g.w0;
    ga.w[1] = g.w1 ? g.w1 : g.w0;
    ga.n = g.n;
    ga.k = g.k;
    ga.expert_bytes = g.expert_bytes;
    ga.x = g.x;
    ga.x_rows = g.x_rows;
    ga.dst = g.dst;
    ga.jobs = g.jobs;
    ga.n_jobs = g.n_jobs;
    ga.act_rows = g.act_rows;
    ga.clamp = g.clamp;
    ga.swiglu = g.w1 != nullptr;
    ga.error_flag = g.error_flag;
    ga.norm_w = g.planes == nullptr ? g.norm_w : nullptr;
    ga.norm_eps = g.norm_eps;
    uint64_t tiles = (uint64_t)g.max_jobs * ((g.n + ROWS - 1) / ROWS);
#ifdef JQ_PROFILING
    static const bool narrow_off = std::getenv("JQ_NO_NARROW_K") != nullptr;  // A/B switch for measurements
#else
    constexpr bool narrow_off = false;
#endif
    // measured on the Qwen3-MoE shape: +5..8 % at 8 and 16 tokens per step, -2 % at one (where a job is one row)
    const bool narrow = !narrow_off && g.rows_per_job > 1 && narrow_k(g.type, g.k);
    if (g.planes == nullptr)
        return narrow ? launch_narrow_typed<1>(g.type, ga, g.rows_per_job, g.max_jobs, s)
                      : launch_typed<1, 2>(g.type, ga, g.rows_per_job, tiles, s);
    ga.act = planes_in(g.planes, g.x_rows, g.k);
    return narrow ? launch_narrow_typed<0>(g.type, ga, g.rows_per_job, g.max_jobs, s)
                  : launch_typed<0, 2>(g.type, ga, g.rows_per_job, tiles, s);
}

}  // namespace jq
