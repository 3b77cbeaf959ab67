// Rope + KV-cache append + attention over the cache + merge for one new token per sequence, as a device
// function over 256 threads (the kernel that runs it is in decoder.cu).
//
// One item = (chunk of ATT_FUSED_CHUNK positions, kv head, sequence); it serves all G = nq / nkv query heads
// of its kv head, so a K or V row is read once per group.  The item that holds the newest position ropes k,
// stores k and v into the cache and uses them from shared memory.  Each item writes its un-normalised partial
// result with its own maximum and sum, then counts itself in; the last one of a (sequence, kv head) merges the
// chunks in chunk order and resets the counter.
//
// The function is written for latency, which is all a decode step sees of it: every global load that does
// not depend on another (the position, the qkv row, the chunk's K and V rows) is requested up front, the
// partials of the merge are requested before their weights are known, and the code is specialised on the
// head size and the group size so that it stays small.
#pragma once

#include <cstdint>
#include <cuda_runtime.h>

namespace jq {

constexpr uint32_t ATT_FUSED_CHUNK = 64;
constexpr uint32_t ATT_FUSED_THREADS = 256;
constexpr uint32_t ATT_MAX_GROUP = 8;   // query heads per kv head
constexpr uint32_t ATT_MAX_HD = 256;
constexpr uint32_t ATT_MERGE_BATCH = 16;  // partial rows a thread requests at a time in the merge

struct AttnArgs {
    const float* qkv;      // [B, (nq + 2 nkv) * hd], before the rotary embedding
    const int32_t* pos;    // [B]
    uint32_t batch, nq, nkv, hd, max_ctx, n_chunks;
    uint32_t gsplit;       // CTAs that share one kv head's query heads (1 or 2); an item serves nq / nkv / gsplit heads
    float theta;
    float* cache_k;        // [B, nkv, max_ctx, hd]
    float* cache_v;
    float* part;           // [B, nq, n_chunks, hd + 2]
    uint32_t* counters;    // [B * nkv * gsplit], zero between calls
    float* out;            // [B, nq * hd]
    unsigned long long* trace = nullptr;  // profiling aid: item (0, 0, 0) stores the GPU timer at its phases
    int32_t* bad_pos = nullptr;  // set to 1 when a position lies outside the cache (the item then does nothing)
    // per-head RMS norm of q and k before the rotary embedding (Qwen3: `attn_q_norm` / `attn_k_norm`, [hd] each,
    // src/quantized_qwen3_moe.rs:343-353); NULL = none
    const float* q_norm = nullptr;
    const float* k_norm = nullptr;
    float qk_eps = 0.0f;
};

// dynamic shared memory the item needs, in floats
__host__ __device__ inline uint32_t attention_fused_smem_floats(uint32_t nq, uint32_t nkv, uint32_t hd, uint32_t n_chunks) {
    const uint32_t G = nq / nkv, PG = ATT_FUSED_THREADS / hd > 0 ? ATT_FUSED_THREADS / hd : 1;
    return G * hd + 2 * hd + G * ATT_FUSED_CHUNK + 2 * G + PG * G * hd + G * n_chunks + G;
}

// head sizes and group sizes the specialised code exists for
__host__ __device__ inline bool attention_fused_shape_ok(uint32_t nq, uint32_t nkv, uint32_t hd) {
    if (nkv == 0 || nq % nkv) return false;
    const uint32_t G = nq / nkv;
    return (hd == 64 || hd == 128 || hd == 256) && (G == 1 || G == 2 || G == 4 || G == 8);
}

// Angular frequency of rotary pair i of a head of size hd: theta^(-2i/hd).
__device__ __forceinline__ float rope_freq(float theta, uint32_t i, uint32_t hd) {
    return exp2f(-2.0f * (float)i / (float)hd * log2f(theta));
}

__device__ __forceinline__ void att_trace(const AttnArgs& a, bool on, int slot) {
    if (on) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
        a.trace[slot] = t;
    }
}

// BAR == 0: the 256 threads are the whole CTA; otherwise they meet on named barrier BAR.
template <int BAR>
__device__ __forceinline__ void att_sync() {
    if (BAR == 0)
        __syncthreads();
    else
        asm volatile("bar.sync %0, %1;" ::"r"(BAR), "r"(ATT_FUSED_THREADS) : "memory");
}

// One (chunk, kv head, sequence) item.  tid = 0..255 inside the group of threads; s_f: the item's shared
// memory (attention_fused_smem_floats floats); s_last: one shared word.
template <int BAR, uint32_t HD, uint32_t G>
__device__ __forceinline__ void attention_fused_item_t(const AttnArgs& a, uint32_t chunk, uint32_t kvh, uint32_t sg,
                                                       uint32_t b, uint32_t tid, float* s_f, uint32_t* s_last) {
    constexpr uint32_t NW = ATT_FUSED_THREADS / 32;
    constexpr uint32_t PER_WARP = ATT_FUSED_CHUNK / NW;        // positions a warp scores: 8
    constexpr uint32_t PG = ATT_FUSED_THREADS / HD > 0 ? ATT_FUSED_THREADS / HD : 1;  // position groups of the V pass
    constexpr uint32_t VN = ATT_FUSED_CHUNK / PG;              // V rows per thread
    constexpr uint32_t HJ = HD / 32;                           // K elements per lane
    constexpr uint32_t HALF = HD / 2;
    constexpr uint32_t N_ROT = (G + 1) * HALF;                 // rotary pairs: the group's q heads and the new k
    constexpr uint32_t ROT_PER = (N_ROT + ATT_FUSED_THREADS - 1) / ATT_FUSED_THREADS;
    constexpr uint32_t OUT_PER = (G * HD + ATT_FUSED_THREADS - 1) / ATT_FUSED_THREADS;
    const uint32_t nq = a.nq, nkv = a.nkv, max_ctx = a.max_ctx, n_chunks = a.n_chunks;
    const uint32_t lane = tid & 31, warp = tid >> 5;
    const uint32_t hb = kvh * (nq / nkv) + sg * G;   // first query head of this item
    const uint32_t cix = (b * nkv + kvh) * a.gsplit + sg;  // its arrival counter
    const bool tr = a.trace != nullptr && chunk == 0 && kvh == 0 && sg == 0 && b == 0 && tid == 0;
    att_trace(a, tr, 0);
    float* sq = s_f;
    float* sk = sq + G * HD;
    float* sv = sk + HD;
    float* sc = sv + HD;
    float* smx = sc + G * ATT_FUSED_CHUNK;
    float* ssum = smx + G;
    float* spv = ssum + G;
    float* se = spv + PG * G * HD;
    float* sden = se + G * n_chunks;
    const uint32_t t0 = chunk * ATT_FUSED_CHUNK;
    const float* row = a.qkv + (uint64_t)b * (nq + 2 * nkv) * HD;
    float* Kc = a.cache_k + (((uint64_t)b * nkv + kvh) * max_ctx) * HD;
    float* Vc = a.cache_v + (((uint64_t)b * nkv + kvh) * max_ctx) * HD;

    // ── every independent load first: position, rotary inputs, the chunk's K rows and V rows ──
    const int32_t p_raw = __ldcg(a.pos + b);
    float ra[ROT_PER], rb[ROT_PER];
#pragma unroll
    for (uint32_t r = 0; r < ROT_PER; ++r) {
        const uint32_t idx = tid + r * ATT_FUSED_THREADS;
        if (idx < N_ROT) {
            const uint32_t g = idx / HALF, i = idx - g * HALF;
            const float* src = g < G ? row + (uint64_t)(hb + g) * HD : row + (uint64_t)(nq + kvh) * HD;
            ra[r] = __ldcg(src + i);  // qkv may have been written earlier in this same launch: read through L2
            rb[r] = __ldcg(src + i + HALF);
        }
    }
    const float vnew = tid < HD ? __ldcg(row + (uint64_t)(nq + nkv + kvh) * HD + tid) : 0.0f;
    // cache rows of the whole chunk are requested whether or not they are live yet (they lie inside the
    // allocation); rows at or beyond the newest position are ignored below
    float kreg[PER_WARP][HJ];
#pragma unroll
    for (uint32_t u = 0; u < PER_WARP; ++u) {
        const uint32_t t = t0 + warp + u * NW;
#pragma unroll
        for (uint32_t j = 0; j < HJ; ++j) kreg[u][j] = t < max_ctx ? Kc[(uint64_t)t * HD + lane + 32 * j] : 0.0f;
    }
    const bool v_thread = tid < PG * HD;
    const uint32_t vpg = tid / HD, vi = tid - vpg * HD;
    float vreg[VN];
#pragma unroll
    for (uint32_t u = 0; u < VN; ++u) {
        const uint32_t t = t0 + vpg + u * PG;
        vreg[u] = (v_thread && t < max_ctx) ? Vc[(uint64_t)t * HD + vi] : 0.0f;
    }

    // A position outside [0, max_ctx) has no cache row: store nothing, attend to nothing, say so.  Every item of
    // the sequence takes this exit, so the arrival counters stay at zero.
    if (p_raw < 0 || (uint32_t)p_raw >= max_ctx) {
        if (tid == 0 && a.bad_pos) atomicExch(a.bad_pos, 1);
        return;
    }
    if (a.q_norm != nullptr) {
        // per-head RMS norm: a head's HALF rotary pairs sit in HALF / 32 consecutive warps of one round, so its
        // sum of squares is those warps' partial sums, added in warp order
        __shared__ float s_nrm[ROT_PER][NW];
#pragma unroll
        for (uint32_t r = 0; r < ROT_PER; ++r) {
            const uint32_t idx = tid + r * ATT_FUSED_THREADS;
            float ss = idx < N_ROT ? fmaf(ra[r], ra[r], rb[r] * rb[r]) : 0.0f;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xFFFFFFFFu, ss, o);
            if (lane == 0) s_nrm[r][warp] = ss;
        }
        att_sync<BAR>();
        constexpr uint32_t WPH = HALF / 32;  // warps per head
#pragma unroll
        for (uint32_t r = 0; r < ROT_PER; ++r) {
            const uint32_t idx = tid + r * ATT_FUSED_THREADS;
            if (idx < N_ROT) {
                const uint32_t g = idx / HALF, i = idx - g * HALF, w0 = warp - warp % WPH;
                float ss = 0.0f;
#pragma unroll
                for (uint32_t w = 0; w < WPH; ++w) ss += s_nrm[r][w0 + w];
                const float sc = rsqrtf(ss / (float)HD + a.qk_eps);
                const float* nw = g < G ? a.q_norm : a.k_norm;
                ra[r] = ra[r] * sc * __ldg(nw + i);
                rb[r] = rb[r] * sc * __ldg(nw + i + HALF);
            }
        }
    }
    const uint32_t p = (uint32_t)p_raw, n_ctx = p + 1;
    const uint32_t active = (n_ctx + ATT_FUSED_CHUNK - 1) / ATT_FUSED_CHUNK;
    if (chunk >= active) return;
    const uint32_t cnt = min(ATT_FUSED_CHUNK, n_ctx - t0);
    const bool newest = chunk == active - 1;  // this chunk holds position p

    // rotate-half rotary embedding at position p of the group's q heads (and of the new k)
#pragma unroll
    for (uint32_t r = 0; r < ROT_PER; ++r) {
        const uint32_t idx = tid + r * ATT_FUSED_THREADS;
        if (idx < N_ROT) {
            const uint32_t g = idx / HALF, i = idx - g * HALF;
            float* dst = g < G ? sq + g * HD : sk;
            float sn, cs;
            sincosf((float)p * rope_freq(a.theta, i, HD), &sn, &cs);
            dst[i] = ra[r] * cs - rb[r] * sn;
            dst[i + HALF] = ra[r] * sn + rb[r] * cs;
        }
    }
    if (tid < HD) sv[tid] = vnew;
    att_sync<BAR>();
    if (newest && sg == 0 && tid < HD) {
        Kc[(uint64_t)p * HD + tid] = sk[tid];
        Vc[(uint64_t)p * HD + tid] = sv[tid];
    }
    att_trace(a, tr, 1);
    // scores: a warp takes positions warp, warp + 8, ...
    const float scale = rsqrtf((float)HD);
#pragma unroll
    for (uint32_t u = 0; u < PER_WARP; ++u) {
        const uint32_t t = warp + u * NW;
        if (t < cnt) {
            if (t0 + t == p) {
#pragma unroll
                for (uint32_t j = 0; j < HJ; ++j) kreg[u][j] = sk[lane + 32 * j];
            }
#pragma unroll
            for (uint32_t g = 0; g < G; ++g) {
                float acc = 0.0f;
#pragma unroll
                for (uint32_t j = 0; j < HJ; ++j) acc = fmaf(sq[g * HD + lane + 32 * j], kreg[u][j], acc);
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xFFFFFFFFu, acc, o);
                if (lane == 0) sc[g * ATT_FUSED_CHUNK + t] = acc * scale;
            }
        }
    }
    att_sync<BAR>();
    att_trace(a, tr, 2);
    // per head: maximum, exponentials, their sum (one warp per head; a lane holds positions lane, lane + 32)
    for (uint32_t g = warp; g < G; g += NW) {
        float v0 = lane < cnt ? sc[g * ATT_FUSED_CHUNK + lane] : -INFINITY;
        float v1 = lane + 32 < cnt ? sc[g * ATT_FUSED_CHUNK + lane + 32] : -INFINITY;
        float mx = fmaxf(v0, v1);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, o));
        const float e0 = lane < cnt ? expf(v0 - mx) : 0.0f, e1 = lane + 32 < cnt ? expf(v1 - mx) : 0.0f;
        sc[g * ATT_FUSED_CHUNK + lane] = e0;
        sc[g * ATT_FUSED_CHUNK + lane + 32] = e1;
        // sum in position order within each half, halves in order
        float s0 = e0, s1 = e1;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            s0 += __shfl_xor_sync(0xFFFFFFFFu, s0, o);
            s1 += __shfl_xor_sync(0xFFFFFFFFu, s1, o);
        }
        if (lane == 0) {
            smx[g] = mx;
            ssum[g] = s0 + s1;
        }
    }
    att_sync<BAR>();
    att_trace(a, tr, 3);
    // weighted V sum: thread = (position group, output dimension); a V element is read once for the group
    if (v_thread) {
        float acc[G];
#pragma unroll
        for (uint32_t g = 0; g < G; ++g) acc[g] = 0.0f;
#pragma unroll
        for (uint32_t u = 0; u < VN; ++u) {
            const uint32_t t = vpg + u * PG;
            if (t < cnt) {
                const float v = (t0 + t == p) ? sv[vi] : vreg[u];
#pragma unroll
                for (uint32_t g = 0; g < G; ++g) acc[g] = fmaf(sc[g * ATT_FUSED_CHUNK + t], v, acc[g]);
            }
        }
#pragma unroll
        for (uint32_t g = 0; g < G; ++g) spv[(vpg * G + g) * HD + vi] = acc[g];
    }
    att_sync<BAR>();
#pragma unroll
    for (uint32_t r = 0; r < OUT_PER; ++r) {
        const uint32_t idx = tid + r * ATT_FUSED_THREADS;
        if (idx < G * HD) {
            const uint32_t g = idx / HD, i = idx - g * HD;
            float v = 0.0f;
#pragma unroll
            for (uint32_t pg = 0; pg < PG; ++pg) v += spv[(pg * G + g) * HD + i];  // fixed order
            a.part[(((uint64_t)b * nq + hb + g) * n_chunks + chunk) * (HD + 2) + i] = v;
        }
    }
    if (tid < G) {
        float* dst = a.part + (((uint64_t)b * nq + hb + tid) * n_chunks + chunk) * (HD + 2);
        dst[HD] = smx[tid];
        dst[HD + 1] = ssum[tid];
    }
    att_trace(a, tr, 4);
    // count in; the last item of this (sequence, kv head) merges.  The barrier orders the threads' stores
    // before thread 0's fence and atomic (the grid-barrier pattern).
    att_sync<BAR>();
    if (tid == 0) {
        __threadfence();
        const uint32_t old = atomicAdd(&a.counters[cix], 1u);
        *s_last = old == active - 1 ? 1u : 0u;
        if (*s_last) {
            a.counters[cix] = 0;
            __threadfence();
        }
    }
    att_sync<BAR>();
    att_trace(a, tr, 5);
    if (!*s_last) return;
    // merge: the first batch of partial rows of every output element is requested before the weights exist
    float pv[OUT_PER][ATT_MERGE_BATCH];
#pragma unroll
    for (uint32_t r = 0; r < OUT_PER; ++r) {
        const uint32_t idx = tid + r * ATT_FUSED_THREADS;
        const uint32_t g = idx / HD, i = idx - g * HD;
        const float* src = a.part + (((uint64_t)b * nq + hb + g) * n_chunks) * (HD + 2) + i;
#pragma unroll
        for (uint32_t u = 0; u < ATT_MERGE_BATCH; ++u)
            pv[r][u] = (idx < G * HD && u < active) ? __ldcg(src + (uint64_t)u * (HD + 2)) : 0.0f;
    }
    // a warp per query head turns the chunks' (max, sum) into weights exp(m_c - max) and the denominator
    for (uint32_t g = warp; g < G; g += NW) {
        const float* src = a.part + (((uint64_t)b * nq + hb + g) * n_chunks) * (HD + 2);
        float mx = -INFINITY;
        for (uint32_t c = lane; c < active; c += 32) mx = fmaxf(mx, __ldcg(src + (uint64_t)c * (HD + 2) + HD));
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, o));
        float den = 0.0f;
        for (uint32_t c0 = 0; c0 < active; c0 += 32) {
            const uint32_t c = c0 + lane;
            float e = 0.0f, sm = 0.0f;
            if (c < active) {
                e = expf(__ldcg(src + (uint64_t)c * (HD + 2) + HD) - mx);
                sm = __ldcg(src + (uint64_t)c * (HD + 2) + HD + 1);
                se[g * n_chunks + c] = e;
            }
            const uint32_t lim = min(32u, active - c0);
            for (uint32_t cc = 0; cc < lim; ++cc)  // chunk order
                den = fmaf(__shfl_sync(0xFFFFFFFFu, e, cc), __shfl_sync(0xFFFFFFFFu, sm, cc), den);
        }
        if (lane == 0) sden[g] = den;
    }
    att_sync<BAR>();
#pragma unroll
    for (uint32_t r = 0; r < OUT_PER; ++r) {
        const uint32_t idx = tid + r * ATT_FUSED_THREADS;
        if (idx < G * HD) {
            const uint32_t g = idx / HD, i = idx - g * HD;
            const float* src = a.part + (((uint64_t)b * nq + hb + g) * n_chunks) * (HD + 2) + i;
            const float* wg = se + g * n_chunks;
            float acc = 0.0f;
#pragma unroll
            for (uint32_t u = 0; u < ATT_MERGE_BATCH; ++u)
                if (u < active) acc = fmaf(wg[u], pv[r][u], acc);
            for (uint32_t c0 = ATT_MERGE_BATCH; c0 < active; c0 += ATT_MERGE_BATCH) {
                float more[ATT_MERGE_BATCH];
#pragma unroll
                for (uint32_t u = 0; u < ATT_MERGE_BATCH; ++u)
                    more[u] = c0 + u < active ? __ldcg(src + (uint64_t)(c0 + u) * (HD + 2)) : 0.0f;
#pragma unroll
                for (uint32_t u = 0; u < ATT_MERGE_BATCH; ++u)
                    if (c0 + u < active) acc = fmaf(wg[c0 + u], more[u], acc);
            }
            a.out[((uint64_t)b * nq + hb + g) * HD + i] = acc / sden[g];
        }
    }
}

// Dispatch on the head size and the heads per item (attention_fused_shape_ok).
template <int BAR>
__device__ __forceinline__ void attention_fused_item(const AttnArgs& a, uint32_t chunk, uint32_t kvh, uint32_t sg,
                                                     uint32_t b, uint32_t tid, float* s_f, uint32_t* s_last) {
    const uint32_t G = a.nq / a.nkv / a.gsplit;
#define JQ_ATT_CASE(HDV, GV) \
    if (a.hd == HDV && G == GV) return attention_fused_item_t<BAR, HDV, GV>(a, chunk, kvh, sg, b, tid, s_f, s_last);
    JQ_ATT_CASE(128, 4)
    JQ_ATT_CASE(128, 8)
    JQ_ATT_CASE(128, 1)
    JQ_ATT_CASE(128, 2)
    JQ_ATT_CASE(64, 1)
    JQ_ATT_CASE(64, 2)
    JQ_ATT_CASE(64, 4)
    JQ_ATT_CASE(64, 8)
    JQ_ATT_CASE(256, 1)
    JQ_ATT_CASE(256, 2)
    JQ_ATT_CASE(256, 4)
    JQ_ATT_CASE(256, 8)
#undef JQ_ATT_CASE
}

}  // namespace jq
