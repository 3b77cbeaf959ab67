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

}  // namespace jq
