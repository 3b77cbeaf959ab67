// Decode-time matmul for ONE activation row per weight matrix (batch 1, and routed-expert jobs of one row),
// HBM-bound: dst[n] = x[k] . W[n, k]^T with W left in its GGUF bytes.
//
// Same regrouping of the reference's arithmetic as the batched decode kernel (gemv_mma.cu; the reference forms
// f32 weights in registers and FMAs them against f32 activations, src/kquant_dot.rs:268-483):
//
//     sum_c x_c * (s_g * q_c - o_g)  =  s_g * sum_c x_c q_c  -  o_g * sum_c x_c        (per scale group g)
//
// with the exact integer codes q_c of the format and x split, per 256 values, into three int8 planes
// x ~= s2 * (254^2 hi + 254 mid + lo), |error| <= max|x| * 6.1e-8 (f32 precision: two planes are not enough, an
// output near zero in a sum of magnitude 100 must still be right to 1e-3).  With a single activation row the
// tensor-core tile of the batched kernel is mostly padding, so here the three dot products per group are dp4a
// (4 byte products per lane and instruction) and everything around them is kept short: about half the
// instructions per weight of the batched kernel, which leaves the kernel waiting on HBM, not on issue slots.
//
// Structure.  One CTA per SM owns a contiguous range of rows (n / gridDim.x of them, so the SMs finish together)
// and walks it in tiles of 8 rows.  Warp 0 streams the tiles' bytes into a ring of shared-memory stages with
// one cp.async.bulk per row behind mbarriers; 8 consumer warps take the units (256 columns) of a stage in
// turn - quad q of a warp works on row q, lane (q, c) on the 64 columns 64c .. 64c+63 of the unit - and keep
// one partial sum per lane; warp 9 adds the warps' partials in a fixed order and stores dst (with the SwiGLU,
// clamp and residual epilogues).  The activation planes of the row(s) are built in shared memory by the
// consumer warps while the producer already prefetches.
//
// A CTA needs about 100 KB of shared memory and 320 threads, so TWO fit on an SM: launched with programmatic
// stream serialization, the next matmul of a decode step becomes resident beside this one, fills its whole ring
// (for the small matrices of a step: all of its weights) while this one is still computing, and starts on it
// the moment its input exists.  HBM keeps streaming across kernel boundaries.
//
// Algorithmic bytes per launch: n*k/B*S (weights) + 4*(k + n).
#include <algorithm>

#include "common.cuh"
#include "pipe.cuh"

namespace jq {

namespace {

constexpr int NCW = 8;                        // consumer warps
constexpr int DP_THREADS = (NCW + 2) * 32;    // + producer + reducer
constexpr uint32_t TROWS = 8;                 // rows of a tile: one per quad of a consumer warp
constexpr uint32_t MAX_GROUPS = 8;            // tiles one ring stage may hold (inputs narrower than 8 units)
constexpr uint32_t DP_SMEM_BUDGET = 110 * 1024;  // two CTAs (of consecutive kernels) share an SM's 227 KB
constexpr uint32_t MAX_STAGES = 8;

// a (unsigned bytes) . b (signed bytes) + c
__device__ __forceinline__ int dp4a_us(uint32_t a, uint32_t b, int c) {
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ int dp4a_ss(uint32_t a, uint32_t b, int c) {
    int d;
    asm("dp4a.s32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

// ── activation planes in shared memory ──
// Per activation row (stride `xs` bytes): hi[k] | mid[k] | lo[k] int8, then sx[k/32] f32 (exact sum of x over
// each 32-value group), then s2[k/256] f32 (the unit's scale / 254^2; 0 for an all-zero or non-finite unit).
__host__ __device__ inline uint32_t x_stride(uint64_t k) { return (uint32_t)((3 * k + k / 8 + k / 64 + 15) & ~(uint64_t)15); }

struct XPlanes {
    const uint8_t* base;  // shared memory
    uint32_t k;
    __device__ __forceinline__ const uint8_t* plane(uint32_t row, uint32_t xs, int p) const { return base + row * xs + p * k; }
    __device__ __forceinline__ const float* sx(uint32_t row, uint32_t xs) const {
        return reinterpret_cast<const float*>(base + row * xs + 3 * k);
    }
    __device__ __forceinline__ const float* s2(uint32_t row, uint32_t xs) const {
        return reinterpret_cast<const float*>(base + row * xs + 3 * k + k / 8);
    }
};

// Splits the 256 values of unit `u` of one row, 8 per lane (lane l holds columns 8l .. 8l+7), into the planes.
__device__ __forceinline__ void quantize_unit3(const float (&v)[8], uint32_t lane, uint8_t* row_base, uint32_t k,
                                               uint32_t u) {
    float amax = 0.0f, sum = 0.0f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        amax = fmaxf(amax, fabsf(v[j]));
        sum += v[j];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
    sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 1);
    sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 2);  // the 32-value group: lanes 4G .. 4G+3
    const float s = amax * (1.0f / 127.0f);
    const bool live = s > 0.0f && isfinite(s);
    const float s1 = s * (1.0f / 254.0f);
    const float inv = live ? 1.0f / s : 0.0f;
    uint32_t pk[3][2] = {{0, 0}, {0, 0}, {0, 0}};
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        int q0 = 0, q1 = 0, q2 = 0;
        if (live) {
            // the rounded quotients need not be exact: each residual is formed exactly and handed down
            q0 = max(-127, min(127, __float2int_rn(v[j] * inv)));
            float r1 = fmaf(-(float)q0, s, v[j]);
            q1 = max(-127, min(127, __float2int_rn(r1 * (inv * 254.0f))));
            float r2 = fmaf(-(float)q1, s1, r1);
            q2 = max(-127, min(127, __float2int_rn(r2 * (inv * 64516.0f))));
        }
        pk[0][j >> 2] |= (uint32_t)(q0 & 0xFF) << (8 * (j & 3));
        pk[1][j >> 2] |= (uint32_t)(q1 & 0xFF) << (8 * (j & 3));
        pk[2][j >> 2] |= (uint32_t)(q2 & 0xFF) << (8 * (j & 3));
    }
#pragma unroll
    for (int p = 0; p < 3; ++p)
        *reinterpret_cast<uint2*>(row_base + (uint64_t)p * k + u * 256 + 8 * lane) = make_uint2(pk[p][0], pk[p][1]);
    if ((lane & 3) == 0) reinterpret_cast<float*>(row_base + 3 * (uint64_t)k)[u * 8 + (lane >> 2)] = sum;
    if (lane == 0) reinterpret_cast<float*>(row_base + 3 * (uint64_t)k + k / 8)[u] = live ? s1 * (1.0f / 254.0f) : 0.0f;
}

__device__ __forceinline__ void load8(const float* __restrict__ p, float (&v)[8]) {
    const float4 a = __ldg(reinterpret_cast<const float4*>(p)), b = __ldg(reinterpret_cast<const float4*>(p) + 1);
    v[0] = a.x, v[1] = a.y, v[2] = a.z, v[3] = a.w, v[4] = b.x, v[5] = b.y, v[6] = b.z, v[7] = b.w;
}

// `rows` x k f32 values -> planes in shared memory, by NW warps (w = 0 .. NW-1) that meet on named barrier 1.
// Loads are requested in batches before any is used.  With norm_w every row is RMS-normalised first (1 / rms from
// the units' sums of squares, added in unit order).  s_ss: rows * (k / 256) floats of shared scratch.
template <int NW>
__device__ __forceinline__ void build_planes(const float* __restrict__ x, uint32_t rows, uint32_t k,
                                             const float* __restrict__ norm_w, float eps, uint8_t* s_x, uint32_t xs,
                                             int w, uint32_t lane, float* s_ss) {
    const uint32_t upr = k / 256, total = rows * upr;
    if (norm_w == nullptr) {
        for (uint32_t u0 = w; u0 < total; u0 += 4 * NW) {
            float v[4][8];
#pragma unroll
            for (int r = 0; r < 4; ++r)
                if (u0 + r * NW < total) load8(x + (uint64_t)(u0 + r * NW) * 256 + lane * 8, v[r]);
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                const uint32_t u = u0 + r * NW;
                if (u < total) quantize_unit3(v[r], lane, s_x + (u / upr) * xs, k, u % upr);
            }
        }
    } else {
        // pass 1: sums of squares per unit; the first two units of a warp stay in registers for pass 2
        float keep[2][8], g[2][8];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const uint32_t u = w + r * NW;
            if (u < total) {
                load8(x + (uint64_t)u * 256 + lane * 8, keep[r]);
                load8(norm_w + (uint64_t)(u % upr) * 256 + lane * 8, g[r]);
            }
        }
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const uint32_t u = w + r * NW;
            if (u < total) {
                float ss = 0.0f;
#pragma unroll
                for (int j = 0; j < 8; ++j) ss = fmaf(keep[r][j], keep[r][j], ss);
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xFFFFFFFFu, ss, o);
                if (lane == 0) s_ss[u] = ss;
            }
        }
        for (uint32_t u = w + 2 * NW; u < total; u += NW) {
            float v[8];
            load8(x + (uint64_t)u * 256 + lane * 8, v);
            float ss = 0.0f;
#pragma unroll
            for (int j = 0; j < 8; ++j) ss = fmaf(v[j], v[j], ss);
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xFFFFFFFFu, ss, o);
            if (lane == 0) s_ss[u] = ss;
        }
        asm volatile("bar.sync 1, %0;" ::"r"(NW * 32) : "memory");
        auto row_scale = [&](uint32_t row) {
            float tot = 0.0f;
            for (uint32_t q = 0; q < upr; ++q) tot += s_ss[row * upr + q];  // unit order
            return rsqrtf(tot / (float)k + eps);
        };
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const uint32_t u = w + r * NW;
            if (u < total) {
                const float rs = row_scale(u / upr);
#pragma unroll
                for (int j = 0; j < 8; ++j) keep[r][j] = keep[r][j] * rs * g[r][j];
                quantize_unit3(keep[r], lane, s_x + (u / upr) * xs, k, u % upr);
            }
        }
        for (uint32_t u = w + 2 * NW; u < total; u += NW) {
            float v[8], gg[8];
            load8(x + (uint64_t)u * 256 + lane * 8, v);
            load8(norm_w + (uint64_t)(u % upr) * 256 + lane * 8, gg);
            const float rs = row_scale(u / upr);
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = v[j] * rs * gg[j];
            quantize_unit3(v, lane, s_x + (u / upr) * xs, k, u % upr);
        }
    }
    asm volatile("bar.sync 1, %0;" ::"r"(NW * 32) : "memory");
}

// ── per-format traits and the dot of one lane's 64 columns ──
template <uint32_t TYPE>
struct DpTraits;
template <>
struct DpTraits<T_Q4_K> {
    static constexpr uint32_t UNIT_BYTES = 144;
};
template <>
struct DpTraits<T_Q8_0> {
    static constexpr uint32_t UNIT_BYTES = 272;
};

// One lane's share of one (row, unit): columns 64c .. 64c+63 of the unit (32-value groups 2c and 2c+1).
//   up: the unit's bytes for this lane's row in shared memory;  xh / xm / xl: the three planes at the unit's
//   first column;  sx: the unit's 8 group sums;  s2: the unit's activation scale.  Returns the partial dot.
template <uint32_t TYPE>
__device__ __forceinline__ float lane_dot(const uint8_t* up, uint32_t c, const uint8_t* xh, const uint8_t* xm,
                                          const uint8_t* xl, const float* sx, float s2);

template <>
__device__ __forceinline__ float lane_dot<T_Q4_K>(const uint8_t* up, uint32_t c, const uint8_t* xh, const uint8_t* xm,
                                                  const uint8_t* xl, const float* sx, float s2) {
    const uint4 h = lds128(up);  // d | dmin, then the 12 packed scale bytes
    // six-bit scales and minima of groups 2c, 2c+1 (src/kquant_dot.rs:106-118): pairs 0..3 are the low 6 bits of
    // bytes 0..3 / 4..7, pairs 4..7 a nibble of bytes 8..11 plus the top two bits of bytes 0..3 / 4..7
    const uint32_t sh = 16 * (c & 1);
    const uint32_t a = h.y >> sh, b = h.z >> sh, e = h.w >> sh;
    const uint32_t sc2 = c < 2 ? (a & 0x3F3Fu) : ((e & 0x0F0Fu) | ((a >> 2) & 0x3030u));
    const uint32_t mn2 = c < 2 ? (b & 0x3F3Fu) : (((e >> 4) & 0x0F0Fu) | ((b >> 2) & 0x3030u));
    // 32 bytes of nibbles: low nibbles are group 2c, high nibbles group 2c+1 (kept in place: 16 * q)
    const uint4 q0 = lds128(up + 16 + 32 * c), q1 = lds128(up + 32 + 32 * c);
    const uint32_t q[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
    int dA[3] = {0, 0, 0}, dB[3] = {0, 0, 0};
    const uint8_t* xp[3] = {xh + 64 * c, xm + 64 * c, xl + 64 * c};
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        uint4 xa[3], xb[3];
#pragma unroll
        for (int p = 0; p < 3; ++p) {
            xa[p] = lds128(xp[p] + 16 * half);
            xb[p] = lds128(xp[p] + 32 + 16 * half);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t lo = q[4 * half + i] & 0x0F0F0F0Fu, hi = q[4 * half + i] & 0xF0F0F0F0u;
#pragma unroll
            for (int p = 0; p < 3; ++p) {
                const uint32_t wa = i == 0 ? xa[p].x : (i == 1 ? xa[p].y : (i == 2 ? xa[p].z : xa[p].w));
                const uint32_t wb = i == 0 ? xb[p].x : (i == 1 ? xb[p].y : (i == 2 ? xb[p].z : xb[p].w));
                dA[p] = dp4a_us(lo, wa, dA[p]);
                dB[p] = dp4a_us(hi, wb, dB[p]);
            }
        }
    }
    const int scA = (int)(sc2 & 0xFF), scB = (int)(sc2 >> 8);
    // |dA| <= 32*15*127; the high-nibble sums carry a factor 16 that divides out exactly
    const int t0 = scA * dA[0] + scB * (dB[0] >> 4);
    const int t1 = scA * dA[1] + scB * (dB[1] >> 4);
    const int t2 = scA * dA[2] + scB * (dB[2] >> 4);
    const float dot = fmaf((float)t0, 64516.0f, (float)(254 * t1 + t2));
    const float2 sg = *reinterpret_cast<const float2*>(sx + 2 * c);
    const float mins = fmaf((float)(mn2 & 0xFF), sg.x, (float)(mn2 >> 8) * sg.y);
    const float d = f16_bits_to_f32(h.x & 0xFFFF), dmin = f16_bits_to_f32(h.x >> 16);
    return fmaf(d * s2, dot, -(dmin * mins));
}

template <>
__device__ __forceinline__ float lane_dot<T_Q8_0>(const uint8_t* up, uint32_t c, const uint8_t* xh, const uint8_t* xm,
                                                  const uint8_t* xl, const float* sx, float s2) {
    // blocks 2c and 2c+1 of the unit: 68 bytes from offset 68c (a multiple of 4): [d q0..q31][d q0..q31].  The
    // first block's codes start two bytes into a word, the second block's are word aligned.
    const uint8_t* bp = up + 68 * c;
    uint32_t w[17];
#pragma unroll
    for (int i = 0; i < 17; ++i) w[i] = lds32(bp + 4 * i);
    const uint8_t* xp[3] = {xh + 64 * c, xm + 64 * c, xl + 64 * c};
    int dA[3] = {0, 0, 0}, dB[3] = {0, 0, 0};
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        uint4 xa[3], xb[3];
#pragma unroll
        for (int p = 0; p < 3; ++p) {
            xa[p] = lds128(xp[p] + 16 * half);
            xb[p] = lds128(xp[p] + 32 + 16 * half);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int j = 4 * half + i;
            const uint32_t qa = __funnelshift_r(w[j], w[j + 1], 16), qb = w[9 + j];
#pragma unroll
            for (int p = 0; p < 3; ++p) {
                const uint32_t wa = i == 0 ? xa[p].x : (i == 1 ? xa[p].y : (i == 2 ? xa[p].z : xa[p].w));
                const uint32_t wb = i == 0 ? xb[p].x : (i == 1 ? xb[p].y : (i == 2 ? xb[p].z : xb[p].w));
                dA[p] = dp4a_ss(qa, wa, dA[p]);
                dB[p] = dp4a_ss(qb, wb, dB[p]);
            }
        }
    }
    // |d| <= 32*128*127 = 520192: 254 * d + d' stays far inside int32
    const float fa = fmaf((float)dA[0], 64516.0f, (float)(254 * dA[1] + dA[2]));
    const float fb = fmaf((float)dB[0], 64516.0f, (float)(254 * dB[1] + dB[2]));
    const float da = f16_bits_to_f32(w[0] & 0xFFFF), db = f16_bits_to_f32(w[8] >> 16);
    (void)sx;
    return s2 * fmaf(da, fa, db * fb);
}

// ── launch description ──
struct DpPlan {
    uint32_t row_stride;   // bytes between rows of a stage
    uint32_t chunk_units;  // units of a row one stage holds
    uint32_t groups;       // 8-row tiles one stage holds (> 1 only when a row is a single short chunk)
    uint32_t n_stages;
    uint32_t x_bytes;      // activation region
    uint32_t total;        // dynamic shared memory
};

struct DpArgs {
    const uint8_t* w[2];     // weight bank; w[1]: second bank of a SwiGLU pair (gate, up)
    uint64_t n, k;           // rows of one matrix, columns
    uint64_t expert_bytes;   // grouped: bytes between experts of a bank
    const float* x;          // [x_rows, k]
    uint32_t x_rows;
    float* dst;              // dense: [n]; grouped: [list position, n]
    const MoeJob* jobs;      // grouped: one-row jobs (device); NULL = dense
    const uint32_t* n_jobs;  // grouped: device count
    const uint32_t* act_rows;  // grouped: activation row of a list position (NULL = the position itself)
    float clamp;
    int swiglu;
    const float* norm_w;
    float norm_eps;
    const float* residual;   // dense: dst = residual + product (may alias dst)
    DpPlan plan;
    int* error_flag;
};

__device__ __forceinline__ float silu_f(float v) { return v / (1.0f + expf(-v)); }

// The tiles of one ring stage: up to MAX_GROUPS 8-row tiles, each inside one job (matrix).
struct TileSet {
    uint32_t ng;
    uint32_t job[MAX_GROUPS], row0[MAX_GROUPS], rows[MAX_GROUPS];
};

// Cuts the next tile set off the CTA's range [v, v1) of virtual rows (virtual row = job * n + row).
__device__ __forceinline__ void next_tiles(uint64_t& v, uint64_t v1, uint64_t n, uint32_t groups, TileSet& ts) {
    ts.ng = 0;
#pragma unroll
    for (uint32_t g = 0; g < MAX_GROUPS; ++g) {
        if (g < groups && v < v1) {
            const uint32_t job = (uint32_t)(v / n);
            const uint64_t r = v - (uint64_t)job * n;
            const uint32_t rows = (uint32_t)min((uint64_t)TROWS, min(n - r, v1 - v));
            ts.job[g] = job, ts.row0[g] = (uint32_t)r, ts.rows[g] = rows;
            v += rows;
            ts.ng = g + 1;
        } else {
            ts.job[g] = 0, ts.row0[g] = 0, ts.rows[g] = 0;
        }
    }
}

template <uint32_t TYPE, bool GROUPED>
__global__ void __launch_bounds__(DP_THREADS, 2) gemv_dp4a_kernel(const __grid_constant__ DpArgs ga) {
    using Tr = DpTraits<TYPE>;
    extern __shared__ __align__(128) uint8_t smem[];
    const DpPlan& plan = ga.plan;
    // layout: activation planes | ring | 2 reduction buffers | unit sums of squares | mbarriers
    uint8_t* s_x = smem;
    uint8_t* ring = smem + plan.x_bytes;
    const uint32_t stage_bytes = plan.groups * TROWS * plan.row_stride;
    float* s_red = reinterpret_cast<float*>(ring + plan.n_stages * stage_bytes);
    constexpr uint32_t RED_FLOATS = NCW * TROWS;
    float* s_ss = s_red + 2 * RED_FLOATS;
    const uint32_t upr = (uint32_t)(ga.k / 256);
    uint64_t* full = reinterpret_cast<uint64_t*>(s_ss + ((ga.x_rows * upr + 1) & ~1u));
    uint64_t* empty = full + MAX_STAGES;
    uint64_t* red_full = empty + MAX_STAGES;
    uint64_t* red_empty = red_full + 2;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t NS = plan.n_stages;
    const uint64_t n = ga.n;
    const uint32_t k = (uint32_t)ga.k;
    const uint64_t row_bytes = (uint64_t)upr * Tr::UNIT_BYTES;
    const uint32_t n_chunks = (upr + plan.chunk_units - 1) / plan.chunk_units;
    const uint32_t n_sub = ga.swiglu ? 2 : 1;
    const uint32_t xs = x_stride(k);

    if (tid == 0) {
        for (uint32_t s = 0; s < NS; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], NCW);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&red_full[b], NCW);
            mbar_init(&red_empty[b], 1);
        }
        mbar_fence_init();
    }
    __syncthreads();
    // The next kernel of the stream may become resident beside this one and prefetch its weights.  From here on
    // the three roles only meet through mbarriers; every wait is bounded, a role whose wait runs out raises the
    // error flag and leaves, and the roles that depend on it run out in turn.
    pdl_trigger();
    // A grouped launch learns its work from the kernel before it; a dense launch knows it already and may
    // prefetch weights at once.  Everything else depends on the previous kernel's output.
    if (GROUPED || warp != 0) pdl_wait();
    if (warp != 0) build_planes<NCW + 1>(ga.x, ga.x_rows, k, ga.norm_w, ga.norm_eps, s_x, xs, warp - 1, lane, s_ss);

    // this CTA's range of virtual rows: equal shares, so that the SMs finish together
    const uint64_t n_virtual = (GROUPED ? (uint64_t)__ldg(ga.n_jobs) : 1ull) * n;
    uint64_t v = n_virtual * blockIdx.x / gridDim.x;
    const uint64_t v1 = n_virtual * (blockIdx.x + 1) / gridDim.x;
    const uint32_t rb16 = (uint32_t)(row_bytes & 15), eb16 = (uint32_t)(ga.expert_bytes & 15);
    auto expert_of = [&](uint32_t job) -> uint32_t { return GROUPED ? ga.jobs[job].expert : 0u; };
    // low four address bits of a row: the offset of its bytes inside the 16-byte aligned span that is copied
    auto shift_of = [&](uint32_t sub, uint32_t e, uint32_t row) -> uint32_t {
        return ((uint32_t)(reinterpret_cast<uintptr_t>(ga.w[sub]) & 15) + e * eb16 + row * rb16) & 15;
    };
    TileSet ts;

    if (warp == 0) {
        // ── producer: lane r copies row r of every tile of the stage ──
        uint32_t it = 0;
        while (v < v1) {
            next_tiles(v, v1, n, plan.groups, ts);
            for (uint32_t sub = 0; sub < n_sub; ++sub) {
                for (uint32_t chunk = 0; chunk < n_chunks; ++chunk, ++it) {
                    const uint32_t s = it % NS, round = it / NS;
                    if (!mbar_wait(&empty[s], (round & 1) ^ 1)) {
                        if (lane == 0) *reinterpret_cast<volatile int*>(ga.error_flag) = 1;
                        return;
                    }
                    const uint32_t u_lo = chunk * plan.chunk_units;
                    const uint32_t u_hi = min(upr, u_lo + plan.chunk_units);
                    uintptr_t abeg[MAX_GROUPS];
                    uint32_t bytes[MAX_GROUPS], total = 0;
#pragma unroll
                    for (uint32_t g = 0; g < MAX_GROUPS; ++g) {
                        bytes[g] = 0;
                        abeg[g] = 0;
                        if (g < ts.ng && lane < ts.rows[g]) {
                            const uint8_t* wrow = ga.w[sub] + (uint64_t)expert_of(ts.job[g]) * ga.expert_bytes +
                                                  (uint64_t)(ts.row0[g] + lane) * row_bytes;
                            const uintptr_t beg = reinterpret_cast<uintptr_t>(wrow) + (uint64_t)u_lo * Tr::UNIT_BYTES;
                            const uintptr_t end = beg + (uint64_t)(u_hi - u_lo) * Tr::UNIT_BYTES;
                            abeg[g] = beg & ~(uintptr_t)15;
                            bytes[g] = (uint32_t)(((end + 15) & ~(uintptr_t)15) - abeg[g]);
                        }
                        total += bytes[g];
                    }
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) total += __shfl_xor_sync(0xFFFFFFFFu, total, o);
                    if (lane == 0) mbar_arrive_expect_tx(&full[s], total);
                    __syncwarp();
#pragma unroll
                    for (uint32_t g = 0; g < MAX_GROUPS; ++g)
                        if (bytes[g])
                            bulk_g2s(ring + s * stage_bytes + (g * TROWS + lane) * plan.row_stride,
                                     reinterpret_cast<const void*>(abeg[g]), bytes[g], &full[s]);
                }
            }
        }
    } else if (warp <= NCW) {
        // ── consumers: quad q <-> row q of a tile, lane (q, c) <-> columns 64c .. 64c+63 of a unit ──
        const uint32_t cw = warp - 1, q = lane >> 2, c = lane & 3;
        const XPlanes xp{s_x, k};
        uint32_t it = 0, red_it = 0;
        while (v < v1) {
            next_tiles(v, v1, n, plan.groups, ts);
            for (uint32_t sub = 0; sub < n_sub; ++sub, ++red_it) {
                float acc = 0.0f;
                for (uint32_t chunk = 0; chunk < n_chunks; ++chunk, ++it) {
                    const uint32_t s = it % NS, round = it / NS;
                    if (!mbar_wait(&full[s], round & 1)) {
                        if (lane == 0) *reinterpret_cast<volatile int*>(ga.error_flag) = 1;
                        return;
                    }
                    const uint8_t* st = ring + s * stage_bytes;
                    const uint32_t u_lo = chunk * plan.chunk_units;
                    const uint32_t U = min(upr - u_lo, plan.chunk_units);
                    const uint32_t items = ts.ng * U;
                    for (uint32_t item = cw; item < items; item += NCW) {
                        const uint32_t g = item / U, u = item - g * U;
                        uint32_t xrow = 0;
                        if (GROUPED) {
                            const uint32_t pos = ga.jobs[ts.job[g]].row0;
                            xrow = ga.act_rows ? __ldg(ga.act_rows + pos) : pos;
                        }
                        const uint32_t row = min(ts.row0[g] + q, (uint32_t)n - 1);
                        const uint8_t* up = st + (g * TROWS + q) * plan.row_stride +
                                            shift_of(sub, expert_of(ts.job[g]), row) + u * Tr::UNIT_BYTES;
                        const uint32_t col = (u_lo + u) * 256;
                        acc += lane_dot<TYPE>(up, c, xp.plane(xrow, xs, 0) + col, xp.plane(xrow, xs, 1) + col,
                                              xp.plane(xrow, xs, 2) + col, xp.sx(xrow, xs) + (u_lo + u) * 8,
                                              xp.s2(xrow, xs)[u_lo + u]);
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&empty[s]);
                }
                // the quad's four column slices, then the partial goes to the reducer
                acc += __shfl_xor_sync(0xFFFFFFFFu, acc, 1);
                acc += __shfl_xor_sync(0xFFFFFFFFu, acc, 2);
                const uint32_t rb = red_it & 1;
                if (!mbar_wait(&red_empty[rb], ((red_it >> 1) & 1) ^ 1)) {
                    if (lane == 0) *reinterpret_cast<volatile int*>(ga.error_flag) = 1;
                    return;
                }
                if (c == 0) s_red[rb * RED_FLOATS + cw * TROWS + q] = acc;
                __syncwarp();
                if (lane == 0) mbar_arrive(&red_full[rb]);
            }
        }
    } else {
        // ── reducer: per tile, the warps' partials in warp order ──
        float gate[2] = {0.0f, 0.0f};
        uint32_t red_it = 0;
        while (v < v1) {
            next_tiles(v, v1, n, plan.groups, ts);
            // warps that worked on tile g: all of them for a single tile, otherwise `upr` consecutive ones
            const uint32_t wpt = plan.groups > 1 ? upr : NCW;
            for (uint32_t sub = 0; sub < n_sub; ++sub, ++red_it) {
                const uint32_t rb = red_it & 1;
                if (!mbar_wait(&red_full[rb], (red_it >> 1) & 1)) {
                    if (lane == 0) *reinterpret_cast<volatile int*>(ga.error_flag) = 1;
                    return;
                }
                const float* red = s_red + rb * RED_FLOATS;
#pragma unroll
                for (int o = 0; o < 2; ++o) {
                    const uint32_t idx = lane + 32 * o, g = idx / TROWS, r = idx % TROWS;
                    if (g < ts.ng) {
                        float val = 0.0f;
                        for (uint32_t w = 0; w < wpt; ++w) val += red[(g * (plan.groups > 1 ? upr : 0) + w) * TROWS + r];
                        if (ga.swiglu && sub == 0) {
                            gate[o] = val;
                        } else if (r < ts.rows[g]) {
                            if (ga.swiglu) {
                                float gv = gate[o], uv = val;
                                if (ga.clamp > 0.0f) {
                                    gv = fminf(gv, ga.clamp);
                                    uv = fmaxf(-ga.clamp, fminf(uv, ga.clamp));
                                }
                                val = silu_f(gv) * uv;
                            }
                            const uint64_t pos = GROUPED ? ga.jobs[ts.job[g]].row0 : 0u;
                            const uint64_t o_idx = pos * n + ts.row0[g] + r;
                            if (!GROUPED && ga.residual != nullptr) val += ga.residual[o_idx];
                            ga.dst[o_idx] = val;
                        }
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&red_empty[rb]);
            }
        }
    }
}

template <uint32_t TYPE>
uint32_t dp_row_stride(uint32_t units) {
    // up to 15 bytes of lead-in and tail around the copied span; stride = 16 (mod 128) bytes so that the eight
    // rows a warp's 16-byte loads touch land in distinct bank groups
    uint32_t span = (units * DpTraits<TYPE>::UNIT_BYTES + 32 + 15) & ~15u;
    return span + ((16 + 128 - span % 128) % 128);
}

template <uint32_t TYPE>
bool dp_plan(uint64_t k, uint32_t x_rows, DpPlan* p) {
    const uint32_t upr = (uint32_t)(k / 256);
    p->x_bytes = x_rows * x_stride(k);
    const uint32_t fixed = 2 * NCW * TROWS * 4 + ((x_rows * upr + 1) & ~1u) * 4 + 8 * (2 * MAX_STAGES + 4) + 128;
    if (p->x_bytes + fixed + 16 * 1024 > DP_SMEM_BUDGET) return false;
    const uint32_t room = DP_SMEM_BUDGET - p->x_bytes - fixed;
    if (upr < NCW) {
        // short rows: whole rows, several tiles per stage so that every consumer warp has a unit
        p->chunk_units = upr;
        p->groups = std::min<uint32_t>(MAX_GROUPS, NCW / upr);
    } else {
        p->groups = 1;
        p->chunk_units = std::min<uint32_t>(upr, 16);
        // a narrow ring still wants four stages or more: halve the stage
        if (room / (TROWS * dp_row_stride<TYPE>(p->chunk_units)) < 4 && p->chunk_units > 8) p->chunk_units = 8;
    }
    p->row_stride = dp_row_stride<TYPE>(p->chunk_units);
    const uint32_t stage = p->groups * TROWS * p->row_stride;
    p->n_stages = std::min<uint32_t>(MAX_STAGES, room / stage);
    if (p->n_stages < 2) return false;
    p->total = p->x_bytes + p->n_stages * stage + fixed;
    return true;
}

template <uint32_t TYPE, bool GROUPED>
cudaError_t dp_launch(DpArgs& ga, uint64_t max_virtual_rows, cudaStream_t s) {
    if (!dp_plan<TYPE>(ga.k, ga.x_rows, &ga.plan)) return cudaErrorInvalidValue;
    const uint64_t tiles = (max_virtual_rows + TROWS - 1) / TROWS;
    const unsigned grid = (unsigned)std::max<uint64_t>(1, std::min<uint64_t>(tiles, (uint64_t)num_sms()));
    auto kern = gemv_dp4a_kernel<TYPE, GROUPED>;
    static bool configured[MAX_DEVICES] = {};
    if (cudaError_t ce = set_max_smem_once(kern, (int)DP_SMEM_BUDGET, configured); ce != cudaSuccess) return ce;
    cudaError_t e = launch_pdl(kern, grid, DP_THREADS, ga.plan.total, s, ga);
    return e != cudaSuccess ? e : cudaGetLastError();
}

template <bool GROUPED>
cudaError_t dp_launch_typed(uint32_t type, DpArgs& ga, uint64_t max_virtual_rows, cudaStream_t s) {
    switch (type) {
        case T_Q4_K: return dp_launch<T_Q4_K, GROUPED>(ga, max_virtual_rows, s);
        case T_Q8_0: return dp_launch<T_Q8_0, GROUPED>(ga, max_virtual_rows, s);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace

bool gemv_dp4a_supports(uint32_t type, const uint8_t* w, uint64_t n, uint64_t k, uint32_t x_rows) {
    if (n == 0 || k == 0 || k % 256 != 0 || x_rows == 0 || n > 0xFFFFFFFFull) return false;
    const uintptr_t a = reinterpret_cast<uintptr_t>(w);
    DpPlan p;
    switch (type) {
        case T_Q4_K: return a % 16 == 0 && dp_plan<T_Q4_K>(k, x_rows, &p);
        case T_Q8_0: return a % 16 == 0 && dp_plan<T_Q8_0>(k, x_rows, &p);
        default: return false;
    }
}

cudaError_t launch_gemv_dp4a(uint32_t type, const uint8_t* w, const uint8_t* w_up, uint64_t n, uint64_t k,
                             const float* x, float* dst, const float* norm_w, float eps, const float* residual,
                             float clamp, int* error_flag, cudaStream_t s) {
    DpArgs ga = {};
    ga.w[0] = w;
    ga.w[1] = w_up ? w_up : w;
    ga.n = n;
    ga.k = k;
    ga.x = x;
    ga.x_rows = 1;
    ga.dst = dst;
    ga.clamp = clamp;
    ga.swiglu = w_up != nullptr;
    ga.norm_w = norm_w;
    ga.norm_eps = eps;
    ga.residual = residual;
    ga.error_flag = error_flag;
    return dp_launch_typed<false>(type, ga, n, s);
}

cudaError_t launch_gemv_dp4a_grouped(const GroupedLaunch& g, cudaStream_t s) {
    DpArgs ga = {};
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
    ga.norm_w = g.norm_w;
    ga.norm_eps = g.norm_eps;
    ga.error_flag = g.error_flag;
    return dp_launch_typed<true>(g.type, ga, (uint64_t)g.max_jobs * g.n, s);
}

}  // namespace jq
