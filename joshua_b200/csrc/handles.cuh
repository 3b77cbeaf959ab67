// Internal definitions shared by the translation units that implement the C ABI.
#pragma once

#include <cstdlib>
#include <map>
#include <mutex>
#include <new>
#include <string>
#include <vector>

#include "../../include/joshua_b200.h"
#include "common.cuh"

// error reporting (thread-local message behind jq_last_error)
int32_t jq_fail(int32_t code, const std::string& msg);
int32_t jq_fail_cuda(cudaError_t e, const char* what);
#define JQ_CUDA(call)                                         \
    do {                                                      \
        cudaError_t e__ = (call);                             \
        if (e__ != cudaSuccess) return jq_fail_cuda(e__, #call); \
    } while (0)

const char* jq_type_name(uint32_t t);

// A stream plus a grow-only device buffer, handed to one host-buffer call at a time.
struct Workspace {
    cudaStream_t stream = nullptr;
    uint8_t* dev = nullptr;
    size_t cap = 0;
    int* flag = nullptr;  // device error flag (embedding id range)

    cudaError_t reserve(size_t bytes) {
        if (bytes <= cap) return cudaSuccess;
        if (dev) cudaFree(dev);
        dev = nullptr;
        cap = 0;
        size_t want = (bytes + (1u << 20) - 1) & ~((size_t)(1u << 20) - 1);
        cudaError_t e = cudaMalloc(&dev, want);
        if (e == cudaSuccess) cap = want;
        return e;
    }
};

// Scratch of the decode kernels (activation planes), one per caller stream.
struct StreamScratch {
    void* dev = nullptr;
    size_t cap = 0;
};

struct jq_ctx {
    int device = 0;
    bool force_f32 = false;        // JQ_FORCE_F32_PATH=1: always take the exact-decode float kernels
    uint64_t sliced_max_m = 64;    // JQ_SLICED_MAX_M: largest batch run as 8-row slices of the decode kernel (0 = never)
    int* status_host = nullptr;    // pinned, device-visible: set to 1 by a kernel whose bounded wait gave up
    int* status_dev = nullptr;
    std::mutex mu;
    // MoE prefill path: the experts' matmuls are spread over these streams (created on first use, shared by all
    // layers of the context; `aux_mu` serialises the host-side fork / launch / join sequences that use them)
    std::mutex aux_mu;
    cudaStream_t aux[8] = {};
    cudaEvent_t fork_ev = nullptr, join_ev[8] = {};
    std::vector<Workspace*> idle;
    std::map<cudaStream_t, StreamScratch> scratch;

    // Scratch for `stream`, at least `bytes` large.  Growing it frees the old buffer (cudaFree
    // waits for the device), so warm a stream up at its largest shape before capturing it.
    cudaError_t scratch_for(cudaStream_t stream, size_t bytes, void** out) {
        std::lock_guard<std::mutex> g(mu);
        StreamScratch& sc = scratch[stream];
        if (bytes > sc.cap) {
            if (sc.dev) cudaFree(sc.dev);
            sc.dev = nullptr;
            sc.cap = 0;
            size_t want = (bytes + (1u << 20) - 1) & ~((size_t)(1u << 20) - 1);
            cudaError_t e = cudaMalloc(&sc.dev, want);
            if (e != cudaSuccess) return e;
            sc.cap = want;
        }
        *out = sc.dev;
        return cudaSuccess;
    }

    Workspace* acquire() {
        {
            std::lock_guard<std::mutex> g(mu);
            if (!idle.empty()) {
                Workspace* w = idle.back();
                idle.pop_back();
                return w;
            }
        }
        Workspace* w = new (std::nothrow) Workspace();
        if (!w) return nullptr;
        if (cudaStreamCreateWithFlags(&w->stream, cudaStreamNonBlocking) != cudaSuccess ||
            cudaMalloc(&w->flag, sizeof(int)) != cudaSuccess) {
            if (w->stream) cudaStreamDestroy(w->stream);
            delete w;
            return nullptr;
        }
        cudaMemsetAsync(w->flag, 0, sizeof(int), w->stream);
        return w;
    }
    void release(Workspace* w) {
        std::lock_guard<std::mutex> g(mu);
        idle.push_back(w);
    }
};

struct jq_weight {
    jq_ctx* ctx;
    uint32_t type;
    jq::Format fmt;
    const uint8_t* dev;
    uint64_t n_blocks;
    bool owns;
};

// Picks the kernel for a device-resident product (abi.cu).
int32_t jq_matmul_device(const jq_weight* w, uint64_t m, uint64_t k, uint64_t n, const float* lhs, float* dst,
                         cudaStream_t s);

// One MoE layer (moe_abi.cu); shared with the expert-parallel exchange (ep.cu).
struct jq_moe {
    jq_ctx* ctx;
    jq_moe_config cfg;
    jq::MoeRouteParams rp;
    float* router = nullptr;  // [E, h] f32, device
    float* bias = nullptr;    // [E] or NULL
    const jq_weight *gate, *up, *down, *sh_gate, *sh_up, *sh_down;
    uint64_t gate_expert_bytes, down_expert_bytes;
    // workspace, grown to the largest (tokens, pairs) seen
    uint64_t cap_tokens = 0, cap_pairs = 0;
    uint8_t* ws = nullptr;
    float *logits, *wts, *hidden, *out, *sh_hidden, *sh_out, *ones;
    uint32_t *ids, *list_token, *inv, *n_jobs, *n_list;
    jq::MoeJob* jobs;
    void *planes_x, *planes_h;
    // constants on the device: jobs {0, 0, c} for c = 1..8 (a dense product as a single job) and the count 1
    jq::MoeJob* dense_jobs = nullptr;
    uint32_t* one = nullptr;
    uint32_t* counter = nullptr;  // arrival counter of the fused router kernel (zero between calls)
    float* xn = nullptr;          // normalised tokens, for the paths that cannot fold the norm in
    float* bucket = nullptr;      // prefill path: gathered rows [P, hidden] + gate and up products [2][P, inter]
    uint64_t bucket_pairs = 0;
    uint64_t last_rows = 0, last_pairs = 0;  // shape of the job list the last decode-sized call left (replay entry)
    uint32_t last_rpj = 0;
    jq::GemmTile* tiles = nullptr;  // prefill path: narrow and wide tile lists, the small experts' job list, 4 counts
    uint64_t tiles_cap = 0;         // bytes allocated behind `tiles`
    int* bad_host = nullptr;  // pinned, device-visible: an expert id was out of range
    int* bad_dev = nullptr;
    std::mutex mu;
};

// Expert MLPs over n_rows rows with given local expert ids (an id out of range marks an unused row).
// `live_rows` is the caller's estimate of how many rows carry a valid id: from 12 per expert on, the rows run
// in buckets on the tile GEMM (which reads the job list back and so synchronises the stream).
int32_t jq_moe_experts_list(jq_moe* m, const float* x_dev, uint64_t n_rows, const uint32_t* expert_ids_dev,
                            uint64_t live_rows, cudaStream_t s);
// Rows per job for about `live_rows` rows with valid ids: one while two rows rarely share an expert (the decode
// kernel's one-row form), else as for a batch of tokens.
uint32_t jq_moe_rows_per_job(uint64_t live_rows, uint32_t n_expert);
