// Element-wise and attention kernels of a decode step, so that a token never leaves the device between the
// quantized matmuls: RMS norm (optionally fused with the residual add), rotary embedding + KV-cache append,
// attention over the cache for one new token per sequence, SwiGLU, arg-max sampling.
//
// These are the callers on either side of the matmul path: the reference runs them as candle tensor ops
// in its loaders (RmsNorm / rope / softmax / cat of the KV cache, src/quantized_qwen3_moe.rs:297-386;
// greedy arg-max with the last maximal index winning ties, src/engine.rs:2371-2378).  All f32.
#include <algorithm>

#include "attention_fused.cuh"
#include "common.cuh"

namespace jq {

namespace {

__device__ __forceinline__ void pdl_wait_() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

__device__ __forceinline__ float block_sum(float v, float* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float t = 0.0f;
    for (int i = 0; i < nw; ++i) t += red[i];  // fixed order
    __syncthreads();
    return t;
}

// out[r, :] = rmsnorm(x[r, :] (+ res[r, :])) * w;  when res != NULL the sum is also written to sum_out
// (the new residual stream).  One CTA of 1024 threads per row; each thread keeps its float4 pieces in
// registers between the two passes (rows up to 16384 wide; wider rows re-read).
__global__ void __launch_bounds__(1024) rmsnorm_kernel(const float* __restrict__ x, const float* __restrict__ res,
                                                       const float* __restrict__ w, float eps, uint32_t h,
                                                       float* __restrict__ sum_out, float* __restrict__ out,
                                                       uint32_t x_stride) {
    __shared__ float red[32];
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    pdl_wait_();
    const uint64_t row = blockIdx.x;
    const uint32_t n4 = h / 4;
    const float4* x4 = reinterpret_cast<const float4*>(x + row * x_stride);  // rows of x may be wider than h
    const float4* r4 = res ? reinterpret_cast<const float4*>(res + row * h) : nullptr;
    float4* s4 = sum_out ? reinterpret_cast<float4*>(sum_out + row * h) : nullptr;
    float4 keep[4];
    float ss = 0.0f;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        uint32_t i = threadIdx.x + c * 1024;
        if (i < n4) {
            float4 v = x4[i];
            if (r4) {
                float4 r = r4[i];
                v.x += r.x, v.y += r.y, v.z += r.z, v.w += r.w;
            }
            if (s4) s4[i] = v;
            keep[c] = v;
            ss = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, fmaf(v.w, v.w, ss))));
        }
    }
    for (uint32_t i = threadIdx.x + 4096; i < n4; i += 1024) {  // rows wider than 16384
        float4 v = x4[i];
        if (r4) {
            float4 r = r4[i];
            v.x += r.x, v.y += r.y, v.z += r.z, v.w += r.w;
        }
        if (s4) s4[i] = v;
        ss = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, fmaf(v.w, v.w, ss))));
    }
    const float tot = block_sum(ss, red);
    const float scale = rsqrtf(tot / (float)h + eps);
    const float4* w4 = w ? reinterpret_cast<const float4*>(w) : nullptr;
    float4* o4 = reinterpret_cast<float4*>(out + row * h);
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        uint32_t i = threadIdx.x + c * 1024;
        if (i < n4) {
            float4 v = keep[c], g = w4 ? w4[i] : make_float4(1.f, 1.f, 1.f, 1.f);
            o4[i] = make_float4(v.x * scale * g.x, v.y * scale * g.y, v.z * scale * g.z, v.w * scale * g.w);
        }
    }
    for (uint32_t i = threadIdx.x + 4096; i < n4; i += 1024) {
        float4 v = x4[i];
        if (r4) {
            float4 r = r4[i];
            v.x += r.x, v.y += r.y, v.z += r.z, v.w += r.w;
        }
        float4 g = w4 ? w4[i] : make_float4(1.f, 1.f, 1.f, 1.f);
        o4[i] = make_float4(v.x * scale * g.x, v.y * scale * g.y, v.z * scale * g.z, v.w * scale * g.w);
    }
}

// Rotary embedding (rotate-half pairing: element i pairs with i + hd/2) of the q and k parts of a fused
// qkv row, then k and v are appended to the cache at position pos[b].
//   qkv [B, (nq + 2*nkv) * hd];  q_out [B, nq*hd];  cache_k / cache_v [B, nkv, max_ctx, hd]
__global__ void __launch_bounds__(128) rope_append_kernel(const float* __restrict__ qkv, const int32_t* __restrict__ pos,
                                                          uint32_t nq, uint32_t nkv, uint32_t hd, uint32_t max_ctx,
                                                          float theta, float* __restrict__ q_out,
                                                          float* __restrict__ cache_k, float* __restrict__ cache_v,
                                                          int32_t* __restrict__ bad_pos, uint32_t seq,
                                                          const float* __restrict__ q_norm,
                                                          const float* __restrict__ k_norm, float qk_eps) {
    __shared__ float red[4];
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    pdl_wait_();
    // decode (seq == 0): blockIdx.y is the sequence, its position pos[b].  Prefill (seq > 0): one sequence,
    // blockIdx.y is the token, its position pos[0] + token; the cache is sequence 0's.
    const uint32_t b = blockIdx.y, head = blockIdx.x;  // heads 0..nq-1: q; nq..nq+nkv-1: k; then v
    const int32_t p_raw = seq ? pos[0] + (int32_t)b : pos[b];
    const uint32_t cb = seq ? 0u : b;  // cache block
    if (p_raw < 0 || (uint32_t)p_raw >= max_ctx) {
        // the cache has no row for this position: nothing is stored, the flag says why
        if (threadIdx.x == 0 && bad_pos) atomicExch(bad_pos, 1);
        return;
    }
    const uint32_t p = (uint32_t)p_raw;
    const float* src = qkv + ((uint64_t)b * (nq + 2 * nkv) + head) * hd;
    const uint32_t half = hd / 2;
    if (head < nq + nkv) {
        float* dst = head < nq ? q_out + ((uint64_t)b * nq + head) * hd
                               : cache_k + (((uint64_t)cb * nkv + (head - nq)) * max_ctx + p) * hd;
        const float* nw = head < nq ? q_norm : k_norm;
        float sc = 1.0f;
        if (nw != nullptr) {  // per-head RMS norm in front of the rotary embedding
            float ss = 0.0f;
            for (uint32_t i = threadIdx.x; i < hd; i += blockDim.x) ss = fmaf(src[i], src[i], ss);
            sc = rsqrtf(block_sum(ss, red) / (float)hd + qk_eps);
        }
        for (uint32_t i = threadIdx.x; i < half; i += blockDim.x) {
            float freq = rope_freq(theta, i, hd);
            float s, c;
            sincosf((float)p * freq, &s, &c);
            float a = src[i], bb = src[i + half];
            if (nw != nullptr) a = a * sc * nw[i], bb = bb * sc * nw[i + half];
            dst[i] = a * c - bb * s;
            dst[i + half] = a * s + bb * c;
        }
    } else {
        float* dst = cache_v + (((uint64_t)cb * nkv + (head - nq - nkv)) * max_ctx + p) * hd;
        for (uint32_t i = threadIdx.x; i < hd; i += blockDim.x) dst[i] = src[i];
    }
}

// One new token per sequence: out[b, head, :] = softmax(q . K^T / sqrt(hd)) V over positions 0..pos[b].
// The positions are cut into chunks of ATT_CHUNK; one CTA per (q head, chunk, sequence) produces the
// chunk's un-normalised result with its own maximum and sum, and a second kernel merges the chunks in
// order.  Grouped-query: q head -> kv head = head / (nq / nkv).
constexpr uint32_t ATT_CHUNK = 64;

// part[b, head, chunk, 0..hd-1] = sum_t exp(s_t - m) V[t, :];  part[.., hd] = m;  part[.., hd+1] = sum_t exp(s_t - m)
__global__ void __launch_bounds__(128) attention_partial_kernel(const float* __restrict__ q, const float* __restrict__ cache_k,
                                                                const float* __restrict__ cache_v,
                                                                const int32_t* __restrict__ pos, uint32_t nq, uint32_t nkv,
                                                                uint32_t hd, uint32_t max_ctx, uint32_t n_chunks,
                                                                float* __restrict__ part, int32_t* __restrict__ bad_pos,
                                                                uint32_t dv, float scale) {
    // hd: width of q and K rows; dv: width of V rows and of the result (MLA: 192 / 128; otherwise the same)
    extern __shared__ float s_att[];  // hd (q) + ATT_CHUNK (scores)
    __shared__ float red[4];
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    pdl_wait_();
    const uint32_t head = blockIdx.x, chunk = blockIdx.y, b = blockIdx.z, kvh = head / (nq / nkv);
    const int32_t p_raw = pos[b];
    const bool in_cache = p_raw >= 0 && (uint32_t)p_raw < max_ctx;
    if (!in_cache && threadIdx.x == 0 && bad_pos) atomicExch(bad_pos, 1);
    const uint32_t n_ctx = in_cache ? (uint32_t)p_raw + 1 : 0u;  // a position outside the cache attends to nothing
    const uint32_t t0 = chunk * ATT_CHUNK;
    float* dst = part + (((uint64_t)b * nq + head) * n_chunks + chunk) * (dv + 2);
    if (t0 >= n_ctx) {
        if (threadIdx.x == 0) {
            dst[dv] = -INFINITY;
            dst[dv + 1] = 0.0f;
        }
        return;
    }
    const uint32_t cnt = min(ATT_CHUNK, n_ctx - t0);
    float* sq = s_att;
    float* sc = s_att + hd;
    const float* qr = q + ((uint64_t)b * nq + head) * hd;
    for (uint32_t i = threadIdx.x; i < hd; i += blockDim.x) sq[i] = qr[i];
    __syncthreads();
    const float* K = cache_k + (((uint64_t)b * nkv + kvh) * max_ctx + t0) * hd;
    const float* V = cache_v + (((uint64_t)b * nkv + kvh) * max_ctx + t0) * dv;
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    float mx = -INFINITY;
    for (uint32_t t = warp; t < cnt; t += nw) {
        const float* kr = K + (uint64_t)t * hd;
        float acc = 0.0f;
        for (uint32_t i = lane; i < hd; i += 32) acc = fmaf(sq[i], kr[i], acc);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xFFFFFFFFu, acc, o);
        acc *= scale;
        if (lane == 0) sc[t] = acc;
        mx = fmaxf(mx, acc);
    }
    if (lane == 0) red[warp] = mx;
    __syncthreads();
    mx = red[0];
    for (uint32_t i = 1; i < nw; ++i) mx = fmaxf(mx, red[i]);
    __syncthreads();
    float sum = 0.0f;
    for (uint32_t t = threadIdx.x; t < cnt; t += blockDim.x) {
        float e = expf(sc[t] - mx);
        sc[t] = e;
        sum += e;
    }
    sum = block_sum(sum, red);
    for (uint32_t i = threadIdx.x; i < dv; i += blockDim.x) {
        float acc = 0.0f;
        for (uint32_t t = 0; t < cnt; ++t) acc = fmaf(sc[t], V[(uint64_t)t * dv + i], acc);
        dst[i] = acc;
    }
    if (threadIdx.x == 0) {
        dst[dv] = mx;
        dst[dv + 1] = sum;
    }
}

__global__ void __launch_bounds__(128) attention_merge_kernel(const float* __restrict__ part, uint32_t hd, uint32_t n_chunks,
                                                              float* __restrict__ out) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    pdl_wait_();
    const uint64_t bh = blockIdx.x;  // (sequence, head)
    const float* src = part + bh * n_chunks * (hd + 2);
    float mx = -INFINITY;
    for (uint32_t c = 0; c < n_chunks; ++c) mx = fmaxf(mx, src[(uint64_t)c * (hd + 2) + hd]);
    float den = 0.0f;
    for (uint32_t c = 0; c < n_chunks; ++c) {
        float m = src[(uint64_t)c * (hd + 2) + hd];
        if (m != -INFINITY) den += expf(m - mx) * src[(uint64_t)c * (hd + 2) + hd + 1];
    }
    for (uint32_t i = threadIdx.x; i < hd; i += blockDim.x) {
        float acc = 0.0f;
        for (uint32_t c = 0; c < n_chunks; ++c) {
            float m = src[(uint64_t)c * (hd + 2) + hd];
            if (m != -INFINITY) acc = fmaf(expf(m - mx), src[(uint64_t)c * (hd + 2) + i], acc);
        }
        out[bh * hd + i] = acc / den;
    }
}

// Prefill: `seq` new tokens of ONE sequence at positions pos0 .. pos0 + seq - 1, causal over the cache (which
// already holds their k / v rows): out[s, head, :] = softmax(q_s . K[0 .. pos0 + s]^T / sqrt(hd)) V
// (src/quantized_qwen3_moe.rs:366-386 with the causal mask of :805-812).  One CTA per (64 queries, q head).
constexpr uint32_t PF_TQ = 64, PF_TK = 64, PF_THREADS = 256;

// 64 queries of one head against the keys they may see, 64 keys at a time, f32 throughout.  Threads form a 16 x 16
// grid: thread (ty, tx) holds the scores of queries 4ty .. 4ty+3 against keys tx, tx+16, tx+32, tx+48 of the tile
// (a 4 x 4 register tile, operands read from shared memory as float4 along the head dimension; rows are padded by
// four floats so that the eight lanes of a quarter warp hit distinct banks) and the outputs of the same four
// queries for dimensions 4tx .. 4tx+3 (+64).  Softmax is the running (max, sum) form; the probabilities go through
// shared memory key-major so that the P.V product reads them as one float4 per key.  K and V tiles share one
// buffer (85 KB of shared memory in all, two CTAs per SM).
template <uint32_t HD>
__global__ void __launch_bounds__(PF_THREADS, 2)
    attention_prefill_kernel(const float* __restrict__ q, const float* __restrict__ cache_k, const float* __restrict__ cache_v,
                             const int32_t* __restrict__ pos, uint32_t seq, uint32_t nq, uint32_t nkv, uint32_t max_ctx,
                             float* __restrict__ out, int32_t* __restrict__ bad_pos) {
    constexpr uint32_t LDQ = HD + 4, LDP = PF_TQ + 4, NV4 = HD / 64;  // row strides (floats), float4 of output per thread
    extern __shared__ __align__(16) float pf_smem[];
    float* sq = pf_smem;                  // [PF_TQ][LDQ] queries
    float* skv = sq + PF_TQ * LDQ;        // [PF_TK][LDQ] the key tile, then the value tile
    float* sp = skv + PF_TK * LDQ;        // [PF_TK][LDP] probabilities, key-major
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    pdl_wait_();
    const uint32_t head = blockIdx.y, kvh = head / (nq / nkv), s0 = blockIdx.x * PF_TQ;
    const uint32_t tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const int32_t p0 = pos[0];
    if (p0 < 0 || (uint64_t)p0 + seq > max_ctx) {
        if (tid == 0 && bad_pos) atomicExch(bad_pos, 1);
        return;
    }
    for (uint32_t i = tid; i < PF_TQ * (HD / 4); i += PF_THREADS) {
        const uint32_t r = i / (HD / 4), c4 = i % (HD / 4), sr = s0 + r;
        const float4 v = sr < seq ? *reinterpret_cast<const float4*>(q + ((uint64_t)sr * nq + head) * HD + 4 * c4)
                                  : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        *reinterpret_cast<float4*>(sq + r * LDQ + 4 * c4) = v;
    }
    const float* K = cache_k + (uint64_t)kvh * max_ctx * HD;
    const float* V = cache_v + (uint64_t)kvh * max_ctx * HD;
    const float scale = rsqrtf((float)HD);
    float o[4][4 * NV4], mx[4], sum[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        mx[i] = -INFINITY, sum[i] = 0.0f;
#pragma unroll
        for (uint32_t d = 0; d < 4 * NV4; ++d) o[i][d] = 0.0f;
    }
    const uint32_t last_q = min(seq, s0 + PF_TQ) - 1;   // newest query of the tile
    const uint32_t n_keys = (uint32_t)p0 + last_q + 1;  // keys the tile can see
    auto load_tile = [&](const float* src, uint32_t t0) {
        for (uint32_t i = tid; i < PF_TK * (HD / 4); i += PF_THREADS) {
            const uint32_t r = i / (HD / 4), c4 = i % (HD / 4), t = t0 + r;
            const float4 v = t < n_keys ? *reinterpret_cast<const float4*>(src + (uint64_t)t * HD + 4 * c4)
                                        : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            *reinterpret_cast<float4*>(skv + r * LDQ + 4 * c4) = v;
        }
    };
    for (uint32_t t0 = 0; t0 < n_keys; t0 += PF_TK) {
        __syncthreads();  // the previous tile's P.V product has read skv and sp
        load_tile(K, t0);
        __syncthreads();
        float sc[4][4];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) sc[i][j] = 0.0f;
#pragma unroll 4
        for (uint32_t c = 0; c < HD; c += 4) {
            float4 a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = *reinterpret_cast<const float4*>(sq + (4 * ty + i) * LDQ + c);
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = *reinterpret_cast<const float4*>(skv + (tx + 16 * j) * LDQ + c);
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    sc[i][j] = fmaf(a[i].w, b[j].w, fmaf(a[i].z, b[j].z, fmaf(a[i].y, b[j].y, fmaf(a[i].x, b[j].x, sc[i][j]))));
        }
        // causal mask, running softmax; a row's 64 scores sit in the 16 threads that share its ty
        float pr[4][4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t visible = (uint32_t)p0 + s0 + 4 * ty + i + 1;  // keys 0 .. p0 + s (rows past seq: never stored)
            float cm = -INFINITY;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                sc[i][j] = t0 + tx + 16 * j < visible ? sc[i][j] * scale : -INFINITY;
                cm = fmaxf(cm, sc[i][j]);
            }
#pragma unroll
            for (int off = 8; off > 0; off >>= 1) cm = fmaxf(cm, __shfl_xor_sync(0xFFFFFFFFu, cm, off));
            const float nm = fmaxf(mx[i], cm);       // finite from the first tile on: key 0 is visible to every query
            const float corr = expf(mx[i] - nm);     // 0 on the first tile (mx = -inf)
            float ps = 0.0f;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                pr[i][j] = expf(sc[i][j] - nm);      // 0 for masked keys
                ps += pr[i][j];
            }
#pragma unroll
            for (int off = 8; off > 0; off >>= 1) ps += __shfl_xor_sync(0xFFFFFFFFu, ps, off);
            sum[i] = sum[i] * corr + ps;
            mx[i] = nm;
#pragma unroll
            for (uint32_t d = 0; d < 4 * NV4; ++d) o[i][d] *= corr;
        }
#pragma unroll
        for (int j = 0; j < 4; ++j)
            *reinterpret_cast<float4*>(sp + (tx + 16 * j) * LDP + 4 * ty) = make_float4(pr[0][j], pr[1][j], pr[2][j], pr[3][j]);
        __syncthreads();  // every score has been formed from the key tile; the probabilities are in place
        load_tile(V, t0);
        __syncthreads();
#pragma unroll 4
        for (uint32_t kk = 0; kk < PF_TK; ++kk) {
            const float4 pv = *reinterpret_cast<const float4*>(sp + kk * LDP + 4 * ty);
            const float pq[4] = {pv.x, pv.y, pv.z, pv.w};
#pragma unroll
            for (uint32_t h = 0; h < NV4; ++h) {
                const float4 vv = *reinterpret_cast<const float4*>(skv + kk * LDQ + 4 * tx + 64 * h);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    o[i][4 * h + 0] = fmaf(pq[i], vv.x, o[i][4 * h + 0]);
                    o[i][4 * h + 1] = fmaf(pq[i], vv.y, o[i][4 * h + 1]);
                    o[i][4 * h + 2] = fmaf(pq[i], vv.z, o[i][4 * h + 2]);
                    o[i][4 * h + 3] = fmaf(pq[i], vv.w, o[i][4 * h + 3]);
                }
            }
        }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t sr = s0 + 4 * ty + i;
        if (sr < seq) {
            const float inv = 1.0f / sum[i];
#pragma unroll
            for (uint32_t h = 0; h < NV4; ++h)
                *reinterpret_cast<float4*>(out + ((uint64_t)sr * nq + head) * HD + 4 * tx + 64 * h) =
                    make_float4(o[i][4 * h] * inv, o[i][4 * h + 1] * inv, o[i][4 * h + 2] * inv, o[i][4 * h + 3] * inv);
        }
    }
}

// The same attention in ONE launch, straight from the fused qkv row (attention_fused.cuh): one CTA per
// (chunk, kv head, sequence).
__global__ void __launch_bounds__(ATT_FUSED_THREADS) attention_fused_kernel(AttnArgs a) {
    extern __shared__ float s_f[];
    __shared__ uint32_t s_last;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    pdl_wait_();
    attention_fused_item<0>(a, blockIdx.x, blockIdx.y / a.gsplit, blockIdx.y % a.gsplit, blockIdx.z, threadIdx.x, s_f,
                            &s_last);
}

// y = a + b
__global__ void __launch_bounds__(256) add_kernel(const float* __restrict__ a, const float* __restrict__ b, uint64_t n,
                                                  float* __restrict__ y) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    pdl_wait_();
    for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x)
        y[i] = a[i] + b[i];
}

// Greedy sampling: index of the maximum of each row; among equal maxima the LAST index wins, as
// `iter().enumerate().max_by(partial_cmp)` does (src/engine.rs:2371-2378).  Two stages: ARGMAX_SLICES CTAs
// per row reduce a slice each, then one CTA per row merges them and advances pos[b].
constexpr uint32_t ARGMAX_SLICES = 64;

__device__ __forceinline__ void argmax_merge(float& best, uint32_t& idx, float ob, uint32_t oi) {
    if (ob > best || (ob == best && oi > idx)) {
        best = ob;
        idx = oi;
    }
}

__device__ __forceinline__ void argmax_block(float& best, uint32_t& idx, float* sv, uint32_t* si) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        float ob = __shfl_xor_sync(0xFFFFFFFFu, best, o);
        uint32_t oi = __shfl_xor_sync(0xFFFFFFFFu, idx, o);
        argmax_merge(best, idx, ob, oi);
    }
    if (lane == 0) {
        sv[warp] = best;
        si[warp] = idx;
    }
    __syncthreads();
    if (threadIdx.x == 0)
        for (uint32_t w = 1; w < (blockDim.x >> 5); ++w) argmax_merge(best, idx, sv[w], si[w]);
}

// Repetition penalty of the reference's sampler (src/engine.rs:2349-2365): every OCCURRENCE of a token in the
// recent window divides its logit by `penalty` when positive and multiplies it otherwise, applied one
// occurrence after another.  The window (SAMPLE_WINDOW ids per row, src/engine.rs:1222-1232,1265-1269) is a ring:
// state[2b] = ids held, state[2b+1] = slot the next id goes to.  The slice's CTA writes the penalised values of
// its own tokens into the row, scans, and puts the originals back, so the logits the caller sees are unchanged
// as in the reference (which penalises a copy).
constexpr uint32_t SAMPLE_WINDOW = 64;

__global__ void __launch_bounds__(256) argmax_slices_kernel(float* __restrict__ logits, uint32_t vocab,
                                                            float* __restrict__ part_v, uint32_t* __restrict__ part_i,
                                                            float penalty, const int32_t* __restrict__ window,
                                                            const int32_t* __restrict__ win_state) {
    __shared__ float sv[8];
    __shared__ uint32_t si[8];
    __shared__ int32_t s_win[SAMPLE_WINDOW];
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    pdl_wait_();
    float* row = logits + (uint64_t)blockIdx.y * vocab;
    const uint32_t per = (vocab + ARGMAX_SLICES - 1) / ARGMAX_SLICES;
    const uint32_t lo = blockIdx.x * per, hi = min(vocab, lo + per);
    // penalties of this slice's tokens: the thread of a token's first occurrence applies all of them
    float original = 0.0f;
    int32_t mine = -1;
    const bool penalise = window != nullptr && penalty != 1.0f;
    if (penalise) {
        const uint32_t held = min((uint32_t)win_state[2 * blockIdx.y], SAMPLE_WINDOW);
        if (threadIdx.x < SAMPLE_WINDOW)
            s_win[threadIdx.x] = threadIdx.x < held ? window[(uint64_t)blockIdx.y * SAMPLE_WINDOW + threadIdx.x] : -1;
        __syncthreads();
        if (threadIdx.x < held) {
            const int32_t tok = s_win[threadIdx.x];
            bool first = tok >= (int32_t)lo && tok < (int32_t)hi;
            uint32_t occ = 0;
            for (uint32_t i = 0; i < held; ++i) {
                if (s_win[i] == tok) {
                    if (i < threadIdx.x) first = false;
                    ++occ;
                }
            }
            if (first) {
                mine = tok;
                original = row[tok];
                float v = original;
                for (uint32_t i = 0; i < occ; ++i) v = v > 0.0f ? v / penalty : v * penalty;
                row[tok] = v;
            }
        }
        __syncthreads();
    }
    float best = -INFINITY;
    uint32_t idx = 0;
    for (uint32_t i = lo + threadIdx.x; i < hi; i += blockDim.x) {
        float v = row[i];
        if (v >= best) {
            best = v;
            idx = i;
        }
    }
    argmax_block(best, idx, sv, si);  // contains a barrier: every thread's reads of the row are done after it
    if (mine >= 0) row[mine] = original;
    if (threadIdx.x == 0) {
        part_v[blockIdx.y * ARGMAX_SLICES + blockIdx.x] = best;
        part_i[blockIdx.y * ARGMAX_SLICES + blockIdx.x] = idx;
    }
}

__global__ void __launch_bounds__(64) argmax_final_kernel(const float* __restrict__ part_v, const uint32_t* __restrict__ part_i,
                                                          int32_t* __restrict__ token, int32_t* __restrict__ pos,
                                                          int32_t* __restrict__ window, int32_t* __restrict__ win_state) {
    __shared__ float sv[2];
    __shared__ uint32_t si[2];
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    pdl_wait_();
    float best = part_v[blockIdx.x * ARGMAX_SLICES + threadIdx.x];
    uint32_t idx = part_i[blockIdx.x * ARGMAX_SLICES + threadIdx.x];
    argmax_block(best, idx, sv, si);
    if (threadIdx.x == 0) {
        token[blockIdx.x] = (int32_t)idx;
        if (pos) pos[blockIdx.x] += 1;
        if (window) {
            // push the sampled id; once the window is full the oldest id is the one replaced
            int32_t held = win_state[2 * blockIdx.x], next = win_state[2 * blockIdx.x + 1];
            next = next < 0 || next >= (int32_t)SAMPLE_WINDOW ? 0 : next;
            window[(uint64_t)blockIdx.x * SAMPLE_WINDOW + next] = (int32_t)idx;
            win_state[2 * blockIdx.x] = min(held + 1, (int32_t)SAMPLE_WINDOW);
            win_state[2 * blockIdx.x + 1] = (next + 1) % (int32_t)SAMPLE_WINDOW;
        }
    }
}

unsigned blocks_for(uint64_t work, unsigned per_block) {
    uint64_t b = (work + per_block - 1) / per_block;
    return (unsigned)(b < 1 ? 1 : (b > 148ull * 16 ? 148ull * 16 : b));
}

}  // namespace

cudaError_t launch_rmsnorm(const float* x, const float* res, const float* w, float eps, uint64_t rows, uint32_t h,
                           float* sum_out, float* out, cudaStream_t s, uint32_t x_stride) {
    if (x_stride == 0) x_stride = h;
    if (h % 4 || x_stride % 4) return cudaErrorInvalidValue;
    cudaError_t le1__ = launch_pdl(rmsnorm_kernel, (unsigned)rows, 1024, 0, s, x, res, w, eps, h, sum_out, out, x_stride);
    if (le1__ != cudaSuccess) return le1__;
    return cudaGetLastError();
}

cudaError_t launch_rope_append(const float* qkv, const int32_t* pos, uint32_t batch, uint32_t nq, uint32_t nkv,
                               uint32_t hd, uint32_t max_ctx, float theta, float* q_out, float* cache_k, float* cache_v,
                               int32_t* bad_pos, cudaStream_t s, uint32_t seq, const float* q_norm, const float* k_norm,
                               float qk_eps) {
    cudaError_t le2__ = launch_pdl(rope_append_kernel, dim3(nq + 2 * nkv, seq ? seq : batch), 128, 0, s, qkv, pos, nq, nkv, hd, max_ctx, theta, q_out, cache_k,
                                                                 cache_v, bad_pos, seq, q_norm, k_norm, qk_eps);
    if (le2__ != cudaSuccess) return le2__;
    return cudaGetLastError();
}

size_t attention_scratch_bytes(uint32_t batch, uint32_t nq, uint32_t hd, uint32_t max_ctx) {
    uint32_t n_chunks = (max_ctx + ATT_CHUNK - 1) / ATT_CHUNK;
    return (size_t)batch * nq * n_chunks * (hd + 2) * 4;
}

// Multi-head latent attention (src/quantized_deepseek2.rs:422-504), the step between the projections and the
// attention proper for one new token per sequence: the rotary embedding (interleaved pairs 2i, 2i+1, angles
// pos * inv_freq[i], cos / sin scaled by `mscale`) of the last `rope` columns of every q head and of the shared key
// k_pe, then K[pos] = [k_nope of the head | k_pe] and V[pos] = v of the head appended to the per-head caches.
//   q [B, nh * (nope + rope)] in place;  comp [B, comp_stride], k_pe = comp[kv_lora ..];  kv [B, nh * (nope + vd)];
//   cache_k [B, nh, max_ctx, nope + rope];  cache_v [B, nh, max_ctx, vd].
__global__ void __launch_bounds__(128) mla_assemble_kernel(float* __restrict__ q, const float* __restrict__ comp,
                                                           const float* __restrict__ kv, const int32_t* __restrict__ pos,
                                                           uint32_t nh, uint32_t nope, uint32_t rope, uint32_t vd,
                                                           uint32_t kv_lora, uint32_t max_ctx,
                                                           const float* __restrict__ inv_freq, float mscale,
                                                           float* __restrict__ cache_k, float* __restrict__ cache_v,
                                                           int32_t* __restrict__ bad_pos) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    pdl_wait_();
    const uint32_t head = blockIdx.x, b = blockIdx.y, qd = nope + rope;
    const int32_t p_raw = pos[b];
    if (p_raw < 0 || (uint32_t)p_raw >= max_ctx) {
        if (threadIdx.x == 0 && bad_pos) atomicExch(bad_pos, 1);
        return;
    }
    const uint32_t p = (uint32_t)p_raw;
    float* qh = q + ((uint64_t)b * nh + head) * qd;
    const float* kpe = comp + (uint64_t)b * (kv_lora + rope) + kv_lora;
    const float* kvh = kv + ((uint64_t)b * nh + head) * (nope + vd);
    float* K = cache_k + (((uint64_t)b * nh + head) * max_ctx + p) * qd;
    float* V = cache_v + (((uint64_t)b * nh + head) * max_ctx + p) * vd;
    for (uint32_t i = threadIdx.x; i < rope / 2; i += blockDim.x) {
        float sn, cs;
        sincosf((float)p * inv_freq[i], &sn, &cs);
        sn *= mscale, cs *= mscale;
        const float a = qh[nope + 2 * i], bb = qh[nope + 2 * i + 1];
        qh[nope + 2 * i] = a * cs - bb * sn;
        qh[nope + 2 * i + 1] = a * sn + bb * cs;
        const float ka = kpe[2 * i], kb = kpe[2 * i + 1];
        K[nope + 2 * i] = ka * cs - kb * sn;
        K[nope + 2 * i + 1] = ka * sn + kb * cs;
    }
    for (uint32_t i = threadIdx.x; i < nope; i += blockDim.x) K[i] = kvh[i];
    for (uint32_t i = threadIdx.x; i < vd; i += blockDim.x) V[i] = kvh[nope + i];
}

cudaError_t launch_mla_assemble(float* q, const float* comp, const float* kv, const int32_t* pos, uint32_t batch,
                                uint32_t nh, uint32_t nope, uint32_t rope, uint32_t vd, uint32_t kv_lora, uint32_t max_ctx,
                                const float* inv_freq, float mscale, float* cache_k, float* cache_v, int32_t* bad_pos,
                                cudaStream_t s) {
    cudaError_t e = launch_pdl(mla_assemble_kernel, dim3(nh, batch), 128, 0, s, q, comp, kv, pos, nh, nope, rope, vd,
                               kv_lora, max_ctx, inv_freq, mscale, cache_k, cache_v, bad_pos);
    return e != cudaSuccess ? e : cudaGetLastError();
}

cudaError_t launch_attention_decode(const float* q, const float* cache_k, const float* cache_v, const int32_t* pos,
                                    uint32_t batch, uint32_t nq, uint32_t nkv, uint32_t hd, uint32_t max_ctx, float* out,
                                    float* scratch, int32_t* bad_pos, cudaStream_t s, uint32_t dv, float scale) {
    if (dv == 0) dv = hd;
    if (scale == 0.0f) scale = 1.0f / sqrtf((float)hd);
    uint32_t n_chunks = (max_ctx + ATT_CHUNK - 1) / ATT_CHUNK;
    size_t smem = (size_t)(hd + ATT_CHUNK) * 4;
    cudaError_t le3__ = launch_pdl(attention_partial_kernel, dim3(nq, n_chunks, batch), 128, smem, s, q, cache_k, cache_v, pos, nq, nkv, hd, max_ctx,
                                                                          n_chunks, scratch, bad_pos, dv, scale);
    if (le3__ != cudaSuccess) return le3__;
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    cudaError_t le4__ = launch_pdl(attention_merge_kernel, batch * nq, 128, 0, s, scratch, dv, n_chunks, out);
    if (le4__ != cudaSuccess) return le4__;
    return cudaGetLastError();
}

cudaError_t launch_attention_prefill(const float* q, const float* cache_k, const float* cache_v, const int32_t* pos,
                                     uint32_t seq, uint32_t nq, uint32_t nkv, uint32_t hd, uint32_t max_ctx, float* out,
                                     int32_t* bad_pos, cudaStream_t s) {
    const dim3 grid((seq + PF_TQ - 1) / PF_TQ, nq);
    const size_t smem = (size_t)((PF_TQ + PF_TK) * (hd + 4) + PF_TK * (PF_TQ + 4)) * 4;
    cudaError_t e;
    if (hd == 64) {
        static bool configured[MAX_DEVICES] = {};
        if (cudaError_t ce = set_max_smem_once(attention_prefill_kernel<64>, (int)smem, configured); ce != cudaSuccess) return ce;
        e = launch_pdl(attention_prefill_kernel<64>, grid, PF_THREADS, smem, s, q, cache_k, cache_v, pos, seq, nq, nkv, max_ctx, out, bad_pos);
    } else if (hd == 128) {
        static bool configured[MAX_DEVICES] = {};
        if (cudaError_t ce = set_max_smem_once(attention_prefill_kernel<128>, (int)smem, configured); ce != cudaSuccess) return ce;
        e = launch_pdl(attention_prefill_kernel<128>, grid, PF_THREADS, smem, s, q, cache_k, cache_v, pos, seq, nq, nkv, max_ctx, out, bad_pos);
    } else {
        return cudaErrorInvalidValue;
    }
    return e != cudaSuccess ? e : cudaGetLastError();
}

size_t attention_fused_scratch_bytes(uint32_t batch, uint32_t nq, uint32_t nkv, uint32_t hd, uint32_t max_ctx) {
    uint32_t n_chunks = (max_ctx + ATT_FUSED_CHUNK - 1) / ATT_FUSED_CHUNK;
    return (size_t)batch * nq * n_chunks * (hd + 2) * 4 + (size_t)batch * nkv * 2 * 4;  // partials + counters
}

// scratch: attention_fused_scratch_bytes bytes whose last batch * nkv words (the counters) are zero before
// the first call; the kernel leaves them zero.
cudaError_t launch_attention_fused(const float* qkv, const int32_t* pos, uint32_t batch, uint32_t nq, uint32_t nkv,
                                   uint32_t hd, uint32_t max_ctx, float theta, float* cache_k, float* cache_v,
                                   float* out, void* scratch, int32_t* bad_pos, cudaStream_t s, const float* q_norm,
                                   const float* k_norm, float qk_eps) {
    AttnArgs a;
    if (!attention_fused_args(qkv, pos, batch, nq, nkv, hd, max_ctx, theta, cache_k, cache_v, out, scratch, &a))
        return cudaErrorInvalidValue;
    a.bad_pos = bad_pos;
    a.q_norm = q_norm;
    a.k_norm = k_norm;
    a.qk_eps = qk_eps;
    size_t smem = (size_t)attention_fused_smem_floats(nq / a.gsplit, nkv, hd, a.n_chunks) * 4;
    cudaError_t e = launch_pdl(attention_fused_kernel, dim3(a.n_chunks, nkv * a.gsplit, batch), ATT_FUSED_THREADS, smem, s, a);
    if (e != cudaSuccess) return e;
    return cudaGetLastError();
}

bool attention_fused_args(const float* qkv, const int32_t* pos, uint32_t batch, uint32_t nq, uint32_t nkv, uint32_t hd,
                          uint32_t max_ctx, float theta, float* cache_k, float* cache_v, float* out, void* scratch,
                          AttnArgs* a) {
    if (!attention_fused_shape_ok(nq, nkv, hd)) return false;
    uint32_t n_chunks = (max_ctx + ATT_FUSED_CHUNK - 1) / ATT_FUSED_CHUNK;
    if ((size_t)attention_fused_smem_floats(nq, nkv, hd, n_chunks) * 4 > 48 * 1024) return false;
    float* part = static_cast<float*>(scratch);
    // eight query heads per kv head are shared by two CTAs: the K / V rows are read twice, the per-CTA chain
    // of work halves.  Not for four heads per kv head: measured on the Llama-8B shape the kernel alone gets
    // faster (11.0 -> 9.0 us) but the decode step slower (525 -> 500 tok/s), because twice the CTAs occupy every
    // SM and the next matmul's CTAs can no longer start early and prefetch their weights behind it.
    const uint32_t gsplit = nq / nkv == 8 ? 2u : 1u;
    *a = AttnArgs{qkv, pos, batch, nq, nkv, hd, max_ctx, n_chunks, gsplit, theta, cache_k, cache_v, part,
                  reinterpret_cast<uint32_t*>(part + (size_t)batch * nq * n_chunks * (hd + 2)), out};
    return true;
}

cudaError_t launch_add(const float* a, const float* b, uint64_t n, float* y, cudaStream_t s) {
    cudaError_t le5__ = launch_pdl(add_kernel, blocks_for(n, 256), 256, 0, s, a, b, n, y);
    if (le5__ != cudaSuccess) return le5__;
    return cudaGetLastError();
}

size_t argmax_scratch_bytes(uint32_t rows) { return (size_t)rows * ARGMAX_SLICES * 8; }

cudaError_t launch_argmax(const float* logits, uint32_t rows, uint32_t vocab, int32_t* token, int32_t* pos,
                          void* scratch, cudaStream_t s, float penalty, int32_t* window, int32_t* win_state) {
    float* pv = static_cast<float*>(scratch);
    uint32_t* pi = reinterpret_cast<uint32_t*>(pv + (size_t)rows * ARGMAX_SLICES);
    cudaError_t le6__ = launch_pdl(argmax_slices_kernel, dim3(ARGMAX_SLICES, rows), 256, 0, s, const_cast<float*>(logits), vocab, pv, pi,
                                   penalty, (const int32_t*)window, (const int32_t*)win_state);
    if (le6__ != cudaSuccess) return le6__;
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    cudaError_t le7__ = launch_pdl(argmax_final_kernel, rows, 64, 0, s, pv, pi, token, pos, window, win_state);
    if (le7__ != cudaSuccess) return le7__;
    return cudaGetLastError();
}

}  // namespace jq
