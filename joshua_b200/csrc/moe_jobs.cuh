// The job list of the grouped expert matmuls, built by one CTA (the MoE layer's kernels in moe.cu).
#pragma once

#include <cstdint>

#include "common.cuh"

namespace jq {

constexpr uint32_t MAX_EXPERTS = 512;

// One CTA: expert histogram, offsets, the expert-sorted list of (token, slot) pairs (token-major inside an
// expert, like the reference's buckets), and the job list in chunks of `rows_per_job` positions.
//   list_token[pos]  token of list position pos (the activation row of the gate/up products)
//   inv[pair]        list position of pair = token * K + slot, or 0xFFFFFFFF if the id was out of range
// Out-of-range ids raise *bad_id (the caller turns it into an error or ignores it, per loader).
struct JobsSmem {
    uint32_t cnt[MAX_EXPERTS], off[MAX_EXPERTS], job[MAX_EXPERTS];
};

// Body of the job builder for the `nthreads` threads of one CTA (tid = 0 .. nthreads - 1, whole warps).
template <class Sync>
__device__ __forceinline__ void build_jobs(const uint32_t* __restrict__ ids, uint32_t T, uint32_t K, uint32_t E,
                                           uint32_t rows_per_job, uint32_t* __restrict__ list_token,
                                           uint32_t* __restrict__ inv, MoeJob* __restrict__ jobs,
                                           uint32_t* __restrict__ n_jobs, uint32_t* __restrict__ n_list,
                                           int* __restrict__ bad_id, JobsSmem& js, uint32_t tid, uint32_t nthreads,
                                           Sync cta_sync) {
    uint32_t* s_cnt = js.cnt;
    uint32_t* s_off = js.off;
    uint32_t* s_job = js.job;
    const uint32_t lane = tid & 31, warp = tid >> 5, nwarp = nthreads >> 5;
    const uint32_t P = T * K;
    for (uint32_t e = tid; e < E; e += nthreads) s_cnt[e] = 0;
    cta_sync();
    for (uint32_t p = tid; p < P; p += nthreads) {
        uint32_t e = ids[p];
        if (e < E)
            atomicAdd(&s_cnt[e], 1u);
        else {
            inv[p] = 0xFFFFFFFFu;
            *bad_id = 1;
        }
    }
    cta_sync();
    if (tid == 0) {
        uint32_t off = 0, job = 0;
        for (uint32_t e = 0; e < E; ++e) {
            s_off[e] = off;
            s_job[e] = job;
            off += s_cnt[e];
            job += (s_cnt[e] + rows_per_job - 1) / rows_per_job;
        }
        *n_jobs = job;
        *n_list = off;
    }
    cta_sync();
    // stable fill: a warp owns an expert and walks the pairs in order
    for (uint32_t e = warp; e < E; e += nwarp) {
        const uint32_t cnt = s_cnt[e];
        if (cnt == 0) continue;
        uint32_t base = s_off[e];
        for (uint32_t p0 = 0; p0 < P; p0 += 32) {
            uint32_t p = p0 + lane;
            bool hit = p < P && ids[p] == e;
            uint32_t ballot = __ballot_sync(0xFFFFFFFFu, hit);
            if (hit) {
                uint32_t pos = base + __popc(ballot & ((1u << lane) - 1));
                list_token[pos] = p / K;
                inv[p] = pos;
            }
            base += __popc(ballot);
        }
        for (uint32_t j = lane; j * rows_per_job < cnt; j += 32) {
            MoeJob jd;
            jd.expert = e;
            jd.row0 = s_off[e] + j * rows_per_job;
            jd.cnt = min(rows_per_job, cnt - j * rows_per_job);
            jobs[s_job[e] + j] = jd;
        }
    }
}

// The same lists for at most JOBS_SMALL_PAIRS pairs (decode batches of up to 32 tokens x 8), written for latency: one trip to memory for
// the ids, everything else out of shared memory, a parallel scan over the experts instead of one thread walking
// them.  Same lists as build_jobs.  `rows_per_job` is 1, 2, 4 or 8.
constexpr uint32_t JOBS_SMALL_PAIRS = 256;
struct JobsSmallSmem {
    uint32_t ids[JOBS_SMALL_PAIRS];
    uint32_t warp_rows[32], warp_jobs[32];
};

template <class Sync>
__device__ __forceinline__ void build_jobs_small(const uint32_t* __restrict__ ids, uint32_t T, uint32_t K, uint32_t E,
                                                 uint32_t rows_per_job, uint32_t* __restrict__ list_token,
                                                 uint32_t* __restrict__ inv, MoeJob* __restrict__ jobs,
                                                 uint32_t* __restrict__ n_jobs, uint32_t* __restrict__ n_list,
                                                 int* __restrict__ bad_id, JobsSmem& js, JobsSmallSmem& sm, uint32_t tid,
                                                 uint32_t nthreads, Sync cta_sync) {
    const uint32_t P = T * K, lane = tid & 31, warp = tid >> 5, nwarp = nthreads >> 5;
    const uint32_t shift = 31u - __clz(rows_per_job);
    if (tid < P) {
        const uint32_t e = ids[tid];
        sm.ids[tid] = e;
        if (e >= E) {
            inv[tid] = 0xFFFFFFFFu;
            *bad_id = 1;
        }
    }
    cta_sync();
    // thread t owns the experts [t * per, (t + 1) * per): counts, then an exclusive scan of rows and jobs
    const uint32_t per = (E + nthreads - 1) / nthreads;
    uint32_t rows = 0, njob = 0;
    for (uint32_t i = 0; i < per; ++i) {
        const uint32_t e = tid * per + i;
        if (e >= E) break;
        uint32_t c = 0;
        for (uint32_t p = 0; p < P; ++p) c += sm.ids[p] == e ? 1u : 0u;
        js.cnt[e] = c;
        rows += c;
        njob += (c + rows_per_job - 1) >> shift;
    }
    uint32_t sr = rows, sj = njob;  // inclusive scans over the warp
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
        const uint32_t ur = __shfl_up_sync(0xFFFFFFFFu, sr, off), uj = __shfl_up_sync(0xFFFFFFFFu, sj, off);
        if ((int)lane >= off) sr += ur, sj += uj;
    }
    if (lane == 31) sm.warp_rows[warp] = sr, sm.warp_jobs[warp] = sj;
    cta_sync();
    uint32_t base_r = 0, base_j = 0;
    for (uint32_t w = 0; w < warp; ++w) base_r += sm.warp_rows[w], base_j += sm.warp_jobs[w];
    uint32_t off_r = base_r + sr - rows, off_j = base_j + sj - njob;  // exclusive
    for (uint32_t i = 0; i < per; ++i) {
        const uint32_t e = tid * per + i;
        if (e >= E) break;
        const uint32_t c = js.cnt[e];
        js.off[e] = off_r;
        for (uint32_t j = 0; j * rows_per_job < c; ++j) {
            MoeJob jd;
            jd.expert = e;
            jd.row0 = off_r + j * rows_per_job;
            jd.cnt = min(rows_per_job, c - j * rows_per_job);
            jobs[off_j + j] = jd;
        }
        off_r += c;
        off_j += (c + rows_per_job - 1) >> shift;
    }
    if (tid == nthreads - 1) {
        *n_jobs = off_j;
        *n_list = off_r;
    }
    cta_sync();
    // a pair's position: its expert's offset + the earlier pairs of the same expert
    if (tid < P) {
        const uint32_t e = sm.ids[tid];
        if (e < E) {
            uint32_t rank = 0;
            for (uint32_t q = 0; q < tid; ++q) rank += sm.ids[q] == e ? 1u : 0u;
            const uint32_t pos = js.off[e] + rank;
            list_token[pos] = tid / K;
            inv[tid] = pos;
        }
    }
}

}  // namespace jq
