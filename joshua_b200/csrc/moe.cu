// Device-side MoE routing: router logits, gating + top-k, and the expert-sorted job list that feeds the
// grouped matmul, plus the weighted combine.  Replaces the host-side routing and bucketing of the
// reference's loaders, which read the ids and weights back to the host on every layer
// (src/quantized_qwen3_moe.rs:424-520, src/quantized_deepseek2.rs:522-671,
// src/quantized_deepseek4.rs:1354-1492, src/kimi_k3.rs:256-282).  Nothing here synchronises with the host.
#include "common.cuh"
#include "moe_jobs.cuh"

namespace jq {

namespace {

// logits[t, e] = sum_j x[t, j] * router[e, j], f32: one warp per (token, four consecutive experts), so that a token's
// row is read once for four dot products; each dot product sums its lane's strided pieces in column order and
// then across the lanes, the same order for every batch size.
__global__ void __launch_bounds__(256) moe_logits_kernel(const float* __restrict__ x, const float* __restrict__ router,
                                                         uint32_t T, uint32_t E, uint32_t h,
                                                         float* __restrict__ logits) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const uint32_t lane = threadIdx.x & 31, E4 = (E + 3) / 4;
    const uint64_t total = (uint64_t)T * E4;
    for (uint64_t p = blockIdx.x * 8ull + (threadIdx.x >> 5); p < total; p += gridDim.x * 8ull) {
        const uint32_t t = (uint32_t)(p / E4), e0 = (uint32_t)(p % E4) * 4;
        const float4* a = reinterpret_cast<const float4*>(x + (uint64_t)t * h);
        const float4* b[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) b[q] = reinterpret_cast<const float4*>(router + (uint64_t)min(e0 + q, E - 1) * h);
        float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        for (uint32_t j = lane; j < h / 4; j += 32) {
            const float4 u = __ldg(a + j);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const float4 v = __ldg(b[q] + j);
                acc[q] = fmaf(u.x, v.x, acc[q]);
                acc[q] = fmaf(u.y, v.y, acc[q]);
                acc[q] = fmaf(u.z, v.z, acc[q]);
                acc[q] = fmaf(u.w, v.w, acc[q]);
            }
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) {
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) acc[q] += __shfl_xor_sync(0xFFFFFFFFu, acc[q], o);
            if (lane == 0 && e0 + q < E) logits[(uint64_t)t * E + e0 + q] = acc[q];
        }
    }
}

// Warp-wide arg-max over values held one-per-slot in shared memory, ties to the lower index (the order a
// stable descending sort gives).  `taken` marks slots already chosen.
__device__ __forceinline__ uint32_t warp_argmax(const float* v, const uint8_t* taken, uint32_t n, uint32_t lane) {
    float best = -INFINITY;
    uint32_t idx = 0xFFFFFFFFu;
    for (uint32_t i = lane; i < n; i += 32) {
        float f = v[i];
        if (!taken[i] && (idx == 0xFFFFFFFFu || f > best)) {  // strictly greater keeps the lower index
            best = f;
            idx = i;
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        float ob = __shfl_xor_sync(0xFFFFFFFFu, best, o);
        uint32_t oi = __shfl_xor_sync(0xFFFFFFFFu, idx, o);
        bool take = oi != 0xFFFFFFFFu && (idx == 0xFFFFFFFFu || ob > best || (ob == best && oi < idx));
        if (take) {
            best = ob;
            idx = oi;
        }
    }
    return idx;
}


// Profiling aid (jq_debug_moe_trace): when set, the last CTA of the fused router kernel stores the GPU
// nanosecond timer at its phases.
__device__ unsigned long long* g_moe_trace = nullptr;
__device__ __forceinline__ unsigned long long moe_now() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

// Shared memory of the routing code for up to four warps (one token per warp at a time).
struct RouteSmem {
    float prob[4][MAX_EXPERTS];
    float sel[4][MAX_EXPERTS];
    uint8_t taken[4][MAX_EXPERTS];
    float group[4][64];
    uint8_t gtaken[4][64];
    uint32_t chosen[4][MAX_EXPERTS];  // the ids picked for the current token, in slot order
};

// One warp per token: scores, selection (bias, group limit), top-k, weights.  Warp `wq` of `nwq` (at most 4)
// takes tokens first + wq, first + wq + stride, ...
__device__ __forceinline__ void route_tokens(const float* __restrict__ logits, const MoeRouteParams& rp, uint32_t T,
                                             const float* __restrict__ bias, const uint32_t* __restrict__ forced_ids,
                                             uint32_t* __restrict__ ids, float* __restrict__ wts, RouteSmem& sm,
                                             uint32_t first, uint32_t stride, uint32_t wq, uint32_t lane) {
    const uint32_t E = rp.n_expert, K = rp.n_used;
    float* prob = sm.prob[wq];
    float* sel = sm.sel[wq];
    uint8_t* taken = sm.taken[wq];
    float (*s_group)[64] = sm.group;
    uint8_t (*s_gtaken)[64] = sm.gtaken;
    uint32_t* chosen = sm.chosen[wq];
    for (uint32_t t = first + wq; t < T; t += stride) {
        // one trip to memory for the token's logits (they were written by other CTAs: read through L2)
        for (uint32_t e = lane; e < E; e += 32) sel[e] = __ldcg(logits + (uint64_t)t * E + e);
        __syncwarp();
        const float* lg = sel;
        // scores
        if (rp.gating == MOE_GATE_SOFTMAX) {
            float mx = -INFINITY;
            for (uint32_t e = lane; e < E; e += 32) mx = fmaxf(mx, lg[e]);
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, o));
            float sum = 0.0f;
            for (uint32_t e = lane; e < E; e += 32) {
                float p = expf(lg[e] - mx);
                prob[e] = p;
                sum += p;
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, o);
            for (uint32_t e = lane; e < E; e += 32) prob[e] = prob[e] / sum;
        } else if (rp.gating == MOE_GATE_SIGMOID) {
            for (uint32_t e = lane; e < E; e += 32) prob[e] = 1.0f / (1.0f + expf(-lg[e]));
        } else {  // sqrt(softplus), softplus(x) = max(x, 0) + log(1 + exp(-|x|))
            for (uint32_t e = lane; e < E; e += 32) {
                float v = lg[e];
                prob[e] = sqrtf(fmaxf(v, 0.0f) + logf(expf(-fabsf(v)) + 1.0f));
            }
        }
        for (uint32_t e = lane; e < E; e += 32) {
            sel[e] = bias ? prob[e] + bias[e] : prob[e];
            taken[e] = 0;
        }
        __syncwarp();
        uint32_t* id = ids + (uint64_t)t * K;
        float* w = wts + (uint64_t)t * K;
        if (forced_ids) {
            // hash-routed layers: ids come from a token-id table, weights from the gate scores
            for (uint32_t s = lane; s < K; s += 32) {
                chosen[s] = forced_ids[(uint64_t)t * K + s];
                id[s] = chosen[s];
            }
        } else {
            if (rp.n_group > 1) {
                // group-limited selection: score groups by their two best members (sigmoid) or their best
                // member (softmax), keep the top `topk_group`, push everything else down by 1e30
                const uint32_t per = E / rp.n_group;
                for (uint32_t g = lane; g < rp.n_group; g += 32) {
                    const float* p = sel + g * per;
                    float b1 = -INFINITY, b2 = -INFINITY;
                    for (uint32_t i = 0; i < per; ++i) {
                        float f = p[i];
                        if (f > b1) {
                            b2 = b1;
                            b1 = f;
                        } else if (f > b2) {
                            b2 = f;
                        }
                    }
                    s_group[wq][g] = rp.gating == MOE_GATE_SIGMOID ? b1 + b2 : b1;
                    s_gtaken[wq][g] = 0;
                }
                __syncwarp();
                for (uint32_t r = 0; r < rp.topk_group; ++r) {
                    uint32_t g = warp_argmax(s_group[wq], s_gtaken[wq], rp.n_group, lane);
                    __syncwarp();
                    if (lane == 0) s_gtaken[wq][g] = 1;
                    __syncwarp();
                }
                for (uint32_t e = lane; e < E; e += 32) {
                    float mask = s_gtaken[wq][e / per] ? 1.0f : 0.0f;
                    sel[e] = sel[e] + (mask * 1e30f + -1e30f);
                }
                __syncwarp();
            }
            // top-k in registers: lane l holds sel[l + 32 i]; every round is a local scan, one warp-wide
            // maximum of the order-preserving integer image of the value, and one warp-wide minimum of the
            // candidates' indices (ties go to the lower index, the order a stable descending sort gives)
            constexpr int EPL = MAX_EXPERTS / 32;
            const int epl = (int)((E + 31) / 32);
            float val[EPL];
            uint32_t live = 0;
#pragma unroll
            for (int i = 0; i < EPL; ++i) {
                const uint32_t e = lane + 32 * i;
                val[i] = (i < epl && e < E) ? sel[e] : -INFINITY;
                if (i < epl && e < E) live |= 1u << i;
            }
            for (uint32_t s = 0; s < K; ++s) {
                float best = -INFINITY;
                int bi = -1;
#pragma unroll
                for (int i = 0; i < EPL; ++i) {
                    if (i >= epl) break;
                    if (((live >> i) & 1u) && (bi < 0 || val[i] > best)) {
                        best = val[i];
                        bi = i;
                    }
                }
                const uint32_t bits = __float_as_uint(best);
                const uint32_t key = bi < 0 ? 0u : (bits ^ ((bits >> 31) ? 0xFFFFFFFFu : 0x80000000u));
                const uint32_t mx = __reduce_max_sync(0xFFFFFFFFu, key);
                const uint32_t cand = (bi >= 0 && key == mx) ? lane + 32u * (uint32_t)bi : 0xFFFFFFFFu;
                const uint32_t e = __reduce_min_sync(0xFFFFFFFFu, cand);
                if (e != 0xFFFFFFFFu && (e & 31u) == lane) live &= ~(1u << (e >> 5));
                if (lane == 0) {
                    chosen[s] = e;
                    id[s] = e;
                }
            }
        }
        __syncwarp();
        // weights from the unbiased scores of the chosen experts: the sum runs in slot order, then every
        // weight is written once
        float sum = 0.0f;
        for (uint32_t s = 0; s < K; ++s) {
            const uint32_t e = chosen[s];
            sum += e < E ? prob[e] : 0.0f;
        }
        const float denom = rp.renorm_plus_eps ? sum + 1e-20f : fmaxf(sum, 6.1035156e-5f);
        for (uint32_t s = lane; s < K; s += 32) {
            const uint32_t e = chosen[s];
            float p = e < E ? prob[e] : 0.0f;
            if (rp.norm) p = p / denom;
            if (rp.scale != 0.0f && rp.scale != 1.0f) p = p * rp.scale;
            w[s] = p;
        }
        __syncwarp();
    }
}

// The same routing with a token's scores held in registers (lane l holds experts l, l + 32, ...: EPL of them),
// for layers without a group limit: no trips through shared memory between the steps, loops of the token's real
// width.  Same operations in the same order as route_tokens, hence the same ids and weights.
template <int EPL>
__device__ __forceinline__ void route_tokens_regs(const float* __restrict__ logits, const MoeRouteParams& rp, uint32_t T,
                                                  const float* __restrict__ bias, const uint32_t* __restrict__ forced_ids,
                                                  uint32_t* __restrict__ ids, float* __restrict__ wts, RouteSmem& sm,
                                                  uint32_t first, uint32_t stride, uint32_t wq, uint32_t lane) {
    const uint32_t E = rp.n_expert, K = rp.n_used;
    float* prob = sm.prob[wq];
    uint32_t* chosen = sm.chosen[wq];
    for (uint32_t t = first + wq; t < T; t += stride) {
        float lg[EPL], pv[EPL];
        bool in[EPL];
#pragma unroll
        for (int i = 0; i < EPL; ++i) {
            const uint32_t e = lane + 32 * i;
            in[i] = e < E;
            lg[i] = in[i] ? __ldcg(logits + (uint64_t)t * E + e) : -INFINITY;  // written by other CTAs: through L2
        }
        if (rp.gating == MOE_GATE_SOFTMAX) {
            float mx = -INFINITY;
#pragma unroll
            for (int i = 0; i < EPL; ++i)
                if (in[i]) mx = fmaxf(mx, lg[i]);
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, o));
            float sum = 0.0f;
#pragma unroll
            for (int i = 0; i < EPL; ++i) {
                pv[i] = in[i] ? expf(lg[i] - mx) : 0.0f;
                if (in[i]) sum += pv[i];
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, o);
#pragma unroll
            for (int i = 0; i < EPL; ++i) pv[i] = pv[i] / sum;
        } else if (rp.gating == MOE_GATE_SIGMOID) {
#pragma unroll
            for (int i = 0; i < EPL; ++i) pv[i] = 1.0f / (1.0f + expf(-lg[i]));
        } else {  // sqrt(softplus), softplus(x) = max(x, 0) + log(1 + exp(-|x|))
#pragma unroll
            for (int i = 0; i < EPL; ++i) pv[i] = sqrtf(fmaxf(lg[i], 0.0f) + logf(expf(-fabsf(lg[i])) + 1.0f));
        }
#pragma unroll
        for (int i = 0; i < EPL; ++i)
            if (in[i]) prob[lane + 32 * i] = pv[i];
        uint32_t* id = ids + (uint64_t)t * K;
        float* w = wts + (uint64_t)t * K;
        if (forced_ids) {
            // hash-routed layers: ids come from a token-id table, weights from the gate scores
            for (uint32_t s = lane; s < K; s += 32) {
                chosen[s] = forced_ids[(uint64_t)t * K + s];
                id[s] = chosen[s];
            }
        } else {
            // top-k: every round is a local scan, one warp-wide maximum of the order-preserving integer image of
            // the value, and one warp-wide minimum of the candidates' indices (ties go to the lower index)
            float val[EPL];
            uint32_t live = 0;
#pragma unroll
            for (int i = 0; i < EPL; ++i) {
                val[i] = in[i] ? (bias ? pv[i] + bias[lane + 32 * i] : pv[i]) : -INFINITY;
                if (in[i]) live |= 1u << i;
            }
            for (uint32_t s = 0; s < K; ++s) {
                float best = -INFINITY;
                int bi = -1;
#pragma unroll
                for (int i = 0; i < EPL; ++i) {
                    if (((live >> i) & 1u) && (bi < 0 || val[i] > best)) {
                        best = val[i];
                        bi = i;
                    }
                }
                const uint32_t bits = __float_as_uint(best);
                const uint32_t key = bi < 0 ? 0u : (bits ^ ((bits >> 31) ? 0xFFFFFFFFu : 0x80000000u));
                const uint32_t mx = __reduce_max_sync(0xFFFFFFFFu, key);
                const uint32_t cand = (bi >= 0 && key == mx) ? lane + 32u * (uint32_t)bi : 0xFFFFFFFFu;
                const uint32_t e = __reduce_min_sync(0xFFFFFFFFu, cand);
                if (e != 0xFFFFFFFFu && (e & 31u) == lane) live &= ~(1u << (e >> 5));
                if (lane == 0) {
                    chosen[s] = e;
                    id[s] = e;
                }
            }
        }
        __syncwarp();
        // weights from the unbiased scores of the chosen experts: the sum runs in slot order, then every
        // weight is written once
        float sum = 0.0f;
        for (uint32_t s = 0; s < K; ++s) {
            const uint32_t e = chosen[s];
            sum += e < E ? prob[e] : 0.0f;
        }
        const float denom = rp.renorm_plus_eps ? sum + 1e-20f : fmaxf(sum, 6.1035156e-5f);
        for (uint32_t s = lane; s < K; s += 32) {
            const uint32_t e = chosen[s];
            float p = e < E ? prob[e] : 0.0f;
            if (rp.norm) p = p / denom;
            if (rp.scale != 0.0f && rp.scale != 1.0f) p = p * rp.scale;
            w[s] = p;
        }
        __syncwarp();
    }
}

// Routing of tokens first + wq, ... by warp wq: the register form where it applies, else the general one.
__device__ __forceinline__ void route_dispatch(const float* __restrict__ logits, const MoeRouteParams& rp, uint32_t T,
                                               const float* __restrict__ bias, const uint32_t* __restrict__ forced_ids,
                                               uint32_t* __restrict__ ids, float* __restrict__ wts, RouteSmem& sm,
                                               uint32_t first, uint32_t stride, uint32_t wq, uint32_t lane) {
    if (rp.n_group <= 1 && rp.n_expert <= 128)
        route_tokens_regs<4>(logits, rp, T, bias, forced_ids, ids, wts, sm, first, stride, wq, lane);
    else if (rp.n_group <= 1 && rp.n_expert <= 256)
        route_tokens_regs<8>(logits, rp, T, bias, forced_ids, ids, wts, sm, first, stride, wq, lane);
    else
        route_tokens(logits, rp, T, bias, forced_ids, ids, wts, sm, first, stride, wq, lane);
}

__global__ void __launch_bounds__(128) moe_route_kernel(const float* __restrict__ logits, MoeRouteParams rp, uint32_t T,
                                                        const float* __restrict__ bias,
                                                        const uint32_t* __restrict__ forced_ids,
                                                        uint32_t* __restrict__ ids, float* __restrict__ wts) {
    __shared__ RouteSmem sm;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    route_dispatch(logits, rp, T, bias, forced_ids, ids, wts, sm, blockIdx.x * 4, gridDim.x * 4, threadIdx.x >> 5,
                   threadIdx.x & 31);
}

// The same lists for many pairs (prefill sizes).  The stable fill above lets every warp walk all pairs once per
// expert it owns; here the pairs are cut into JOB_SLICES contiguous slices, a warp counts its slice's pairs per
// expert, the slices' counts are prefixed per expert, and the warp walks its slice once more in order: a pair's
// position is its expert's offset + the pairs of earlier slices + its rank among the slice's earlier pairs of the
// same expert (`__match_any_sync` within a group of 32).  Same lists, P / JOB_SLICES steps per warp instead of
// P * E / warps.
constexpr uint32_t JOB_SLICES = 16;
struct JobsSliceSmem {
    uint32_t cnt[JOB_SLICES][MAX_EXPERTS];
};

__device__ __forceinline__ void build_jobs_sliced(const uint32_t* __restrict__ ids, uint32_t T, uint32_t K, uint32_t E,
                                                  uint32_t rows_per_job, uint32_t* __restrict__ list_token,
                                                  uint32_t* __restrict__ inv, MoeJob* __restrict__ jobs,
                                                  uint32_t* __restrict__ n_jobs, uint32_t* __restrict__ n_list,
                                                  int* __restrict__ bad_id, JobsSmem& js, JobsSliceSmem& ss, uint32_t tid,
                                                  uint32_t nthreads) {
    const uint32_t lane = tid & 31, warp = tid >> 5;
    const uint32_t P = T * K;
    const uint32_t slice = ((P + JOB_SLICES - 1) / JOB_SLICES + 31) & ~31u;  // pairs per slice, whole groups of 32
    for (uint32_t i = tid; i < JOB_SLICES * MAX_EXPERTS; i += nthreads) (&ss.cnt[0][0])[i] = 0;
    __syncthreads();
    if (warp < JOB_SLICES) {
        const uint32_t p_end = min(P, (warp + 1) * slice);
        for (uint32_t p = warp * slice + lane; p < p_end; p += 32) {
            const uint32_t e = ids[p];
            if (e < E) {
                atomicAdd(&ss.cnt[warp][e], 1u);
            } else {
                inv[p] = 0xFFFFFFFFu;
                *bad_id = 1;
            }
        }
    }
    __syncthreads();
    // per expert: the slices' counts become the count of earlier slices; the total goes to js.cnt
    for (uint32_t e = tid; e < E; e += nthreads) {
        uint32_t run = 0;
#pragma unroll
        for (uint32_t w = 0; w < JOB_SLICES; ++w) {
            const uint32_t c = ss.cnt[w][e];
            ss.cnt[w][e] = run;
            run += c;
        }
        js.cnt[e] = run;
    }
    __syncthreads();
    if (tid == 0) {
        uint32_t off = 0, job = 0;
        for (uint32_t e = 0; e < E; ++e) {
            js.off[e] = off;
            js.job[e] = job;
            off += js.cnt[e];
            job += (js.cnt[e] + rows_per_job - 1) / rows_per_job;
        }
        *n_jobs = job;
        *n_list = off;
    }
    __syncthreads();
    if (warp < JOB_SLICES) {
        const uint32_t p_end = min(P, (warp + 1) * slice);
        for (uint32_t p0 = warp * slice; p0 < p_end; p0 += 32) {  // warp-uniform bounds: every lane takes part
            const uint32_t p = p0 + lane;
            const uint32_t e = p < p_end ? ids[p] : 0xFFFFFFFFu;
            const bool valid = e < E;
            const uint32_t same = __match_any_sync(0xFFFFFFFFu, valid ? e : 0xFFFFFFFFu);
            uint32_t base = 0;
            if (valid) base = js.off[e] + ss.cnt[warp][e];
            __syncwarp();
            if (valid) {
                const uint32_t pos = base + __popc(same & ((1u << lane) - 1));
                list_token[pos] = p / K;
                inv[p] = pos;
                if ((same & ((1u << lane) - 1)) == 0) ss.cnt[warp][e] += __popc(same);  // the group's first lane of e
            }
            __syncwarp();
        }
    }
    for (uint32_t e = tid; e < E; e += nthreads) {
        const uint32_t cnt = js.cnt[e];
        for (uint32_t j = 0; j * rows_per_job < cnt; ++j) {
            MoeJob jd;
            jd.expert = e;
            jd.row0 = js.off[e] + j * rows_per_job;
            jd.cnt = min(rows_per_job, cnt - j * rows_per_job);
            jobs[js.job[e] + j] = jd;
        }
    }
}

__global__ void __launch_bounds__(1024) moe_jobs_kernel(const uint32_t* __restrict__ ids, uint32_t T, uint32_t K,
                                                        uint32_t E, uint32_t rows_per_job,
                                                        uint32_t* __restrict__ list_token, uint32_t* __restrict__ inv,
                                                        MoeJob* __restrict__ jobs, uint32_t* __restrict__ n_jobs,
                                                        uint32_t* __restrict__ n_list, int* __restrict__ bad_id) {
    __shared__ JobsSmem js;
    __shared__ JobsSliceSmem ss;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (T * K <= JOBS_SMALL_PAIRS) {
        __shared__ JobsSmallSmem jsm;
        build_jobs_small(ids, T, K, E, rows_per_job, list_token, inv, jobs, n_jobs, n_list, bad_id, js, jsm, threadIdx.x,
                         blockDim.x, [] { __syncthreads(); });
    } else if (T * K > 1024)
        build_jobs_sliced(ids, T, K, E, rows_per_job, list_token, inv, jobs, n_jobs, n_list, bad_id, js, ss, threadIdx.x,
                          blockDim.x);
    else
        build_jobs(ids, T, K, E, rows_per_job, list_token, inv, jobs, n_jobs, n_list, bad_id, js, threadIdx.x, blockDim.x,
                   [] { __syncthreads(); });
}

// Decode-sized batches (T <= 8): router logits, routing and the job list in ONE launch.  A CTA per (token,
// expert) dot product, spread over many CTAs so that the [E, h] router matrix streams at full speed; each CTA
// counts itself in when its logits are stored and the last one routes the tokens and builds the jobs.  With
// `norm_w` the tokens are RMS-normalised first (every CTA derives 1 / rms of its tokens itself), so the norm
// kernel in front of the layer disappears.
__global__ void __launch_bounds__(128) moe_route_fused_kernel(
    const float* __restrict__ x, const float* __restrict__ norm_w, float eps, const float* __restrict__ router,
    uint32_t T, uint32_t h, float* __restrict__ logits, MoeRouteParams rp, const float* __restrict__ bias,
    const uint32_t* __restrict__ forced_ids, uint32_t* __restrict__ ids, float* __restrict__ wts, int do_jobs,
    uint32_t rows_per_job, uint32_t* __restrict__ list_token, uint32_t* __restrict__ inv, MoeJob* __restrict__ jobs,
    uint32_t* __restrict__ n_jobs, uint32_t* __restrict__ n_list, int* __restrict__ bad_id,
    uint32_t* __restrict__ counter) {
    __shared__ RouteSmem sm;
    __shared__ JobsSmem js;
    __shared__ JobsSmallSmem jsm;
    __shared__ uint32_t s_last;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const uint32_t lane = threadIdx.x & 31, wq = threadIdx.x >> 5, E = rp.n_expert;
    __shared__ float s_acc[4], s_ss[4];
    unsigned long long* trace = g_moe_trace;
    unsigned long long t_start = 0, t_logits = 0, t_counted = 0;
    if (trace && threadIdx.x == 0) t_start = moe_now();
    {
        // one CTA per (token, expert) dot product; every thread requests all its pieces before using any
        const uint32_t pair = blockIdx.x, t = pair / E, e = pair - t * E;
        const float4* a = reinterpret_cast<const float4*>(x + (uint64_t)t * h);
        const float4* b = reinterpret_cast<const float4*>(router + (uint64_t)e * h);
        const float4* g = reinterpret_cast<const float4*>(norm_w);
        float acc = 0.0f, ss = 0.0f;
        for (uint32_t j0 = threadIdx.x; j0 < h / 4; j0 += 128 * 4) {
            float4 u[4], v[4], w[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const uint32_t j = j0 + q * 128;
                const bool in = j < h / 4;
                u[q] = in ? __ldg(a + j) : make_float4(0.f, 0.f, 0.f, 0.f);
                v[q] = in ? __ldg(b + j) : make_float4(0.f, 0.f, 0.f, 0.f);
                w[q] = (in && norm_w) ? __ldg(g + j) : make_float4(1.f, 1.f, 1.f, 1.f);
            }
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                ss = fmaf(u[q].x, u[q].x, fmaf(u[q].y, u[q].y, fmaf(u[q].z, u[q].z, fmaf(u[q].w, u[q].w, ss))));
                acc = fmaf(u[q].x * w[q].x, v[q].x, acc);
                acc = fmaf(u[q].y * w[q].y, v[q].y, acc);
                acc = fmaf(u[q].z * w[q].z, v[q].z, acc);
                acc = fmaf(u[q].w * w[q].w, v[q].w, acc);
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            acc += __shfl_xor_sync(0xFFFFFFFFu, acc, o);
            ss += __shfl_xor_sync(0xFFFFFFFFu, ss, o);
        }
        if (lane == 0) {
            s_acc[wq] = acc;
            s_ss[wq] = ss;
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            const float tot = (s_acc[0] + s_acc[1]) + (s_acc[2] + s_acc[3]);
            const float sq = (s_ss[0] + s_ss[1]) + (s_ss[2] + s_ss[3]);
            logits[pair] = norm_w ? tot * rsqrtf(sq / (float)h + eps) : tot;
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        if (trace) t_logits = moe_now();
        __threadfence();
        const uint32_t old = atomicAdd(counter, 1u);
        s_last = old == gridDim.x - 1 ? 1u : 0u;
        if (s_last) {
            *counter = 0;
            __threadfence();
        }
        if (trace) t_counted = moe_now();
    }
    __syncthreads();
    if (!s_last) return;
    route_dispatch(logits, rp, T, bias, forced_ids, ids, wts, sm, 0, 4, wq, lane);
    unsigned long long t_routed = 0;
    if (trace && threadIdx.x == 0) t_routed = moe_now();
    if (do_jobs) {
        __threadfence_block();
        __syncthreads();
        if (T * rp.n_used <= JOBS_SMALL_PAIRS)
            build_jobs_small(ids, T, rp.n_used, E, rows_per_job, list_token, inv, jobs, n_jobs, n_list, bad_id, js, jsm,
                             threadIdx.x, 128u, [] { __syncthreads(); });
        else
            build_jobs(ids, T, rp.n_used, E, rows_per_job, list_token, inv, jobs, n_jobs, n_list, bad_id, js, threadIdx.x,
                       128u, [] { __syncthreads(); });
    }
    if (trace && threadIdx.x == 0) {
        trace[0] = t_start, trace[1] = t_logits, trace[2] = t_counted, trace[3] = t_routed, trace[4] = moe_now();
    }
}

// y[t, :] = sum over slots (in slot order) of w[t, s] * out[inv[t*K + s], :]  (+ shared[t, :]) (+ residual[t, :],
// which may be y itself)
__global__ void __launch_bounds__(256) moe_combine_kernel(const float* __restrict__ out, const uint32_t* __restrict__ inv,
                                                          const float* __restrict__ wts, const float* __restrict__ shared,
                                                          const float* residual, uint32_t T, uint32_t K, uint32_t h,
                                                          float* y) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const uint64_t total = (uint64_t)T * (h / 4);
    for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < total;
         i += (uint64_t)gridDim.x * blockDim.x) {
        const uint32_t t = (uint32_t)(i / (h / 4)), c = (uint32_t)(i % (h / 4));
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        if (K <= 8) {
            // latency is all this kernel costs at decode sizes: all positions and weights are requested first, then
            // all rows, and only then summed in slot order (a loop that loads as it goes waits out 2 K round trips)
            uint32_t pos[8];
            float w[8];
            float4 v[8];
#pragma unroll
            for (uint32_t s = 0; s < 8; ++s) {
                pos[s] = s < K ? inv[(uint64_t)t * K + s] : 0xFFFFFFFFu;
                w[s] = s < K ? wts[(uint64_t)t * K + s] : 0.0f;
            }
#pragma unroll
            for (uint32_t s = 0; s < 8; ++s)
                v[s] = pos[s] != 0xFFFFFFFFu ? *reinterpret_cast<const float4*>(out + (uint64_t)pos[s] * h + 4 * c)
                                             : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (uint32_t s = 0; s < 8; ++s) {
                if (pos[s] == 0xFFFFFFFFu) continue;
                acc.x += v[s].x * w[s];
                acc.y += v[s].y * w[s];
                acc.z += v[s].z * w[s];
                acc.w += v[s].w * w[s];
            }
        } else {
            for (uint32_t s = 0; s < K; ++s) {
                uint32_t pos = inv[(uint64_t)t * K + s];
                if (pos == 0xFFFFFFFFu) continue;
                float w = wts[(uint64_t)t * K + s];
                float4 v = *reinterpret_cast<const float4*>(out + (uint64_t)pos * h + 4 * c);
                acc.x += v.x * w;
                acc.y += v.y * w;
                acc.z += v.z * w;
                acc.w += v.w * w;
            }
        }
        if (shared) {
            float4 v = *reinterpret_cast<const float4*>(shared + (uint64_t)t * h + 4 * c);
            acc.x += v.x;
            acc.y += v.y;
            acc.z += v.z;
            acc.w += v.w;
        }
        if (residual) {
            float4 v = *reinterpret_cast<const float4*>(residual + (uint64_t)t * h + 4 * c);
            acc.x += v.x;
            acc.y += v.y;
            acc.z += v.z;
            acc.w += v.w;
        }
        *reinterpret_cast<float4*>(y + (uint64_t)t * h + 4 * c) = acc;
    }
}

// out = silu(clamp(g)) * clamp(u), element-wise (the dense shared-expert path at batches the grouped kernel
// does not take)
__global__ void __launch_bounds__(256) swiglu_kernel(const float* __restrict__ g, const float* __restrict__ u,
                                                     uint64_t n, float clamp, float* __restrict__ out) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) {
        float gv = g[i], uv = u[i];
        if (clamp > 0.0f) {
            gv = fminf(gv, clamp);
            uv = fmaxf(-clamp, fminf(uv, clamp));
        }
        out[i] = gv / (1.0f + expf(-gv)) * uv;
    }
}

// xs[pos, :] = x[list_token[pos], :] for the expert-sorted list (pos < *n_list): the activation rows in bucket
// order, so that an expert's rows are contiguous for a tile GEMM.
__global__ void __launch_bounds__(256) moe_gather_kernel(const float* __restrict__ x, const uint32_t* __restrict__ list_token,
                                                         const uint32_t* __restrict__ n_list, uint32_t P, uint32_t h,
                                                         float* __restrict__ xs) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const uint32_t live = min(P, *n_list), h4 = h / 4;
    const uint64_t total = (uint64_t)live * h4;
    for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < total; i += (uint64_t)gridDim.x * blockDim.x) {
        const uint32_t pos = (uint32_t)(i / h4), c = (uint32_t)(i % h4);
        reinterpret_cast<float4*>(xs)[(uint64_t)pos * h4 + c] =
            __ldg(reinterpret_cast<const float4*>(x) + (uint64_t)list_token[pos] * h4 + c);
    }
}

// Work lists of the prefill form from the job list (jobs of one expert are consecutive and cover consecutive rows).
// An expert with at least `min_rows` rows goes to the tile GEMM: its rows are cut into tiles of 128, a last piece of
// at most 32 rows goes to the narrow list, anything else to the wide list.  The jobs of the other experts are copied
// to `small_jobs` for the grouped decode kernel.  counts = {narrow tiles, wide tiles, rows in the list, small jobs}.
// Which slot of a list an entry takes depends on timing; the products do not (every entry is computed on its own).
// One CTA.
__global__ void __launch_bounds__(1024) moe_tiles_kernel(const MoeJob* __restrict__ jobs, const uint32_t* __restrict__ n_jobs,
                                                         const uint32_t* __restrict__ n_list, uint32_t E, uint32_t min_rows,
                                                         GemmTile* __restrict__ narrow, GemmTile* __restrict__ wide,
                                                         MoeJob* __restrict__ small_jobs, uint32_t* __restrict__ counts) {
    __shared__ uint32_t s_row0[MAX_EXPERTS], s_cnt[MAX_EXPERTS], s_n[3];
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    for (uint32_t e = threadIdx.x; e < E; e += blockDim.x) s_row0[e] = 0xFFFFFFFFu, s_cnt[e] = 0;
    if (threadIdx.x < 3) s_n[threadIdx.x] = 0;
    __syncthreads();
    const uint32_t nj = *n_jobs;
    for (uint32_t j = threadIdx.x; j < nj; j += blockDim.x) {
        const MoeJob jb = jobs[j];
        if (jb.expert < E) {
            atomicMin(&s_row0[jb.expert], jb.row0);
            atomicAdd(&s_cnt[jb.expert], jb.cnt);
        }
    }
    __syncthreads();
    for (uint32_t e = threadIdx.x; e < E; e += blockDim.x) {
        const uint32_t cnt = s_cnt[e], row0 = s_row0[e];
        if (cnt < min_rows) continue;
        for (uint32_t r = 0; r < cnt; r += 128) {
            const uint32_t c = min(128u, cnt - r);
            GemmTile t = {e, row0 + r, c, 0};
            if (c <= 32)
                narrow[atomicAdd(&s_n[0], 1u)] = t;
            else
                wide[atomicAdd(&s_n[1], 1u)] = t;
        }
    }
    for (uint32_t j = threadIdx.x; j < nj; j += blockDim.x) {
        const MoeJob jb = jobs[j];
        if (jb.expert < E && s_cnt[jb.expert] < min_rows) small_jobs[atomicAdd(&s_n[2], 1u)] = jb;
    }
    __syncthreads();
    if (threadIdx.x == 0) counts[0] = s_n[0], counts[1] = s_n[1], counts[2] = *n_list, counts[3] = s_n[2];
}

// SwiGLU over the first *n_rows rows of [rows, inter] (rows of the expert-sorted list that exist).
__global__ void __launch_bounds__(256) swiglu_rows_kernel(const float* __restrict__ g, const float* __restrict__ u,
                                                          const uint32_t* __restrict__ n_rows, uint32_t max_rows, uint32_t inter,
                                                          float clamp, float* __restrict__ out) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const uint64_t n = (uint64_t)min(*n_rows, max_rows) * inter;
    for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) {
        float gv = g[i], uv = u[i];
        if (clamp > 0.0f) {
            gv = fminf(gv, clamp);
            uv = fmaxf(-clamp, fminf(uv, clamp));
        }
        out[i] = gv / (1.0f + expf(-gv)) * uv;
    }
}

unsigned blocks_for(uint64_t work, unsigned per_block) {
    uint64_t b = (work + per_block - 1) / per_block;
    return (unsigned)(b < 1 ? 1 : (b > 148ull * 16 ? 148ull * 16 : b));
}

}  // namespace

cudaError_t launch_moe_logits(const float* x, const float* router, uint32_t T, uint32_t E, uint32_t h, float* logits,
                              cudaStream_t s) {
    cudaError_t le1__ = launch_pdl(moe_logits_kernel, blocks_for((uint64_t)T * ((E + 3) / 4), 8), 256, 0, s, x, router, T, E, h, logits);
    if (le1__ != cudaSuccess) return le1__;
    return cudaGetLastError();
}

cudaError_t launch_moe_route(const float* logits, const MoeRouteParams& rp, uint32_t T, const float* bias,
                             const uint32_t* forced_ids, uint32_t* ids, float* wts, cudaStream_t s) {
    if (rp.n_expert > MAX_EXPERTS || rp.n_group > 64) return cudaErrorInvalidValue;
    cudaError_t le2__ = launch_pdl(moe_route_kernel, blocks_for(T, 4), 128, 0, s, logits, rp, T, bias, forced_ids, ids, wts);
    if (le2__ != cudaSuccess) return le2__;
    return cudaGetLastError();
}

cudaError_t launch_moe_jobs(const uint32_t* ids, uint32_t T, uint32_t K, uint32_t E, uint32_t rows_per_job,
                            uint32_t* list_token, uint32_t* inv, MoeJob* jobs, uint32_t* n_jobs, uint32_t* n_list,
                            int* bad_id, cudaStream_t s) {
    if (E > MAX_EXPERTS) return cudaErrorInvalidValue;
    cudaError_t le3__ = launch_pdl(moe_jobs_kernel, 1, 1024, 0, s, ids, T, K, E, rows_per_job, list_token, inv, jobs, n_jobs, n_list, bad_id);
    if (le3__ != cudaSuccess) return le3__;
    return cudaGetLastError();
}

cudaError_t launch_moe_gather(const float* x, const uint32_t* list_token, const uint32_t* n_list, uint32_t P, uint32_t h,
                              float* xs, cudaStream_t s) {
    cudaError_t e = launch_pdl(moe_gather_kernel, blocks_for((uint64_t)P * (h / 4), 256), 256, 0, s, x, list_token, n_list,
                               P, h, xs);
    if (e != cudaSuccess) return e;
    return cudaGetLastError();
}

cudaError_t launch_moe_tiles(const MoeJob* jobs, const uint32_t* n_jobs, const uint32_t* n_list, uint32_t E, uint32_t min_rows,
                             GemmTile* narrow, GemmTile* wide, MoeJob* small_jobs, uint32_t* counts, cudaStream_t s) {
    if (E > MAX_EXPERTS) return cudaErrorInvalidValue;
    cudaError_t e = launch_pdl(moe_tiles_kernel, 1, 1024, 0, s, jobs, n_jobs, n_list, E, min_rows, narrow, wide, small_jobs,
                               counts);
    return e != cudaSuccess ? e : cudaGetLastError();
}

cudaError_t launch_swiglu_rows(const float* g, const float* u, const uint32_t* n_rows, uint32_t max_rows, uint32_t inter,
                               float clamp, float* out, cudaStream_t s) {
    cudaError_t e = launch_pdl(swiglu_rows_kernel, blocks_for((uint64_t)max_rows * inter, 256), 256, 0, s, g, u, n_rows, max_rows,
                               inter, clamp, out);
    return e != cudaSuccess ? e : cudaGetLastError();
}

cudaError_t moe_set_trace(unsigned long long* dev_buf) {
    return cudaMemcpyToSymbol(g_moe_trace, &dev_buf, sizeof(dev_buf));
}

cudaError_t launch_moe_route_fused(const float* x, const float* norm_w, float eps, const float* router, uint32_t T,
                                   uint32_t h, float* logits, const MoeRouteParams& rp, const float* bias,
                                   const uint32_t* forced_ids, uint32_t* ids, float* wts, bool do_jobs,
                                   uint32_t rows_per_job, uint32_t* list_token, uint32_t* inv, MoeJob* jobs,
                                   uint32_t* n_jobs, uint32_t* n_list, int* bad_id, uint32_t* counter, cudaStream_t s) {
    if (rp.n_expert > MAX_EXPERTS || rp.n_group > 64 || h % 4) return cudaErrorInvalidValue;
    unsigned grid = T * rp.n_expert;
    cudaError_t e = launch_pdl(moe_route_fused_kernel, grid, 128, 0, s, x, norm_w, eps, router, T, h, logits, rp, bias,
                               forced_ids, ids, wts, do_jobs ? 1 : 0, rows_per_job, list_token, inv, jobs, n_jobs,
                               n_list, bad_id, counter);
    if (e != cudaSuccess) return e;
    return cudaGetLastError();
}

cudaError_t launch_moe_combine(const float* out, const uint32_t* inv, const float* wts, const float* shared, uint32_t T,
                               uint32_t K, uint32_t h, float* y, cudaStream_t s, const float* residual) {
    cudaError_t le4__ = launch_pdl(moe_combine_kernel, blocks_for((uint64_t)T * (h / 4), 256), 256, 0, s, out, inv, wts, shared, residual, T, K, h, y);
    if (le4__ != cudaSuccess) return le4__;
    return cudaGetLastError();
}

cudaError_t launch_swiglu(const float* g, const float* u, uint64_t n, float clamp, float* out, cudaStream_t s) {
    cudaError_t le5__ = launch_pdl(swiglu_kernel, blocks_for(n, 256), 256, 0, s, g, u, n, clamp, out);
    if (le5__ != cudaSuccess) return le5__;
    return cudaGetLastError();
}

}  // namespace jq
